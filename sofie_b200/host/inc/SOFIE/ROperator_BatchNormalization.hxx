// Inference-mode BatchNormalization (reference:
// src/SOFIE_core/inc/SOFIE/ROperator_BatchNormalization.hxx:88-228). The reference broadcasts
// scale, bias, mean and var to the full activation shape at Initialize and runs scopy / saxpy /
// multiply / saxpy over it; here the per-channel vectors stay per-channel (C floats each), the
// variance is folded into the scale with the reference's roundings
// (scale * float(1. / sqrt(var + epsilon)), :163-168) and one kernel applies
// ((x - mean) * scale) + bias, with the optional fused Relu of :222-226. Reads NCHW or NHWC.
#ifndef SOFIE_ROPERATOR_BATCHNORMALIZATION
#define SOFIE_ROPERATOR_BATCHNORMALIZATION

#include <cmath>
#include <sstream>

#include "SOFIE/Emit.hxx"
#include "SOFIE/RModel.hxx"
#include "SOFIE/ROperator.hxx"

namespace SOFIE {

template <typename T>
class ROperator_BatchNormalization final : public ROperator {
private:
   float fepsilon = 1e-05;
   float fmomentum = 0.9;
   std::size_t ftraining_mode = 0;
   std::string fNX, fNScale, fNB, fNMean, fNVar, fNY, fNScaleDev;
   EActivationType fActivation = EActivationType::UNDEFINED;
   std::vector<size_t> fShapeX;
   ELayout fLayout = ELayout::NCHW;

public:
   ROperator_BatchNormalization() = delete;
   ROperator_BatchNormalization(float epsilon, float momentum, std::size_t training_mode, std::string nameX, std::string nameScale,
                                std::string nameB, std::string nameMean, std::string nameVar, std::string nameY,
                                EActivationType activation = EActivationType::UNDEFINED)
      : fepsilon(epsilon), fmomentum(momentum), ftraining_mode(training_mode), fNX(UTILITY::Clean_name(nameX)),
        fNScale(UTILITY::Clean_name(nameScale)), fNB(UTILITY::Clean_name(nameB)), fNMean(UTILITY::Clean_name(nameMean)),
        fNVar(UTILITY::Clean_name(nameVar)), fNY(UTILITY::Clean_name(nameY)), fActivation(activation)
   {
      fInputTensorNames = {fNX};
      fOutputTensorNames = {fNY};
   }
   EOpKind Kind() const override { return EOpKind::Eltwise; }
   bool AcceptsNHWC(const std::string &) const override { return true; }
   std::vector<ETensorType> TypeInference(std::vector<ETensorType> input) override { return {input[0]}; }
   std::vector<std::vector<size_t>> ShapeInference(std::vector<std::vector<size_t>> input) override { return {input[0]}; }
   // read by the model plan when it folds this operator into the convolution that feeds it
   const std::string &InputName() const { return fNX; }
   const std::string &OutputName() const { return fNY; }
   const std::string &ScaleName() const { return fNScale; }
   const std::string &BiasName() const { return fNB; }
   const std::string &MeanName() const { return fNMean; }
   const std::string &VarName() const { return fNVar; }
   float Epsilon() const { return fepsilon; }
   bool HasRelu() const { return fActivation == EActivationType::RELU; }

   void Initialize(RModel &model) override
   {
      for (const std::string *n : {&fNX, &fNScale, &fNB, &fNMean, &fNVar})
         if (!model.CheckIfTensorAlreadyExist(*n))
            throw std::runtime_error("SOFIE BatchNormalization op Input Tensor " + *n + " is not found in model");
      if (ftraining_mode) throw std::runtime_error("SOFIE BatchNormalization op: training mode is not supported");
      fShapeX = model.GetTensorShape(fNX);
      if (fShapeX.size() < 2 || fShapeX.size() > 4)
         throw std::runtime_error("SOFIE BatchNormalization Op input tensor " + fNX + " has wrong shape : " + ConvertShapeToString(fShapeX));
      for (const std::string *n : {&fNScale, &fNB, &fNMean, &fNVar}) {
         if (!model.IsInitializedTensor(*n)) throw std::runtime_error("SOFIE BatchNormalization op: " + *n + " must be a constant of the model");
         if (ConvertShapeToLength(model.GetTensorShape(*n)) != fShapeX[1])
            throw std::runtime_error("SOFIE BatchNormalization op: " + *n + " must hold one value per channel");
      }
      model.AddIntermediateTensor(fNY, model.GetTensorType(fNX), fShapeX);
   }
   void PlanDevice(RModel &model) override
   {
      fLayout = model.GetTensorLayout(model.ResolveAlias(fNX));
      model.SetTensorLayout(fNY, fLayout);
      const size_t C = fShapeX[1];
      const float *scale = model.GetInitializedTensor(fNScale).template data<float>();
      const float *var = model.GetInitializedTensor(fNVar).template data<float>();
      std::shared_ptr<void> buf(malloc(C * sizeof(float)), free);
      float *folded = static_cast<float *>(buf.get());
      for (size_t c = 0; c < C; c++) {
         float v = var[c] + fepsilon;
         float inv = 1. / std::sqrt((double)v);
         folded[c] = scale[c] * inv;
      }
      fNScaleDev = fNScale + "_bn_" + fNY;
      if (!model.IsInitializedTensor(fNScaleDev)) model.AddInitializedTensor(fNScaleDev, ETensorType::FLOAT, {C}, buf);
      model.UseOnDevice(fNScaleDev);
      model.UseOnDevice(fNB);
      model.UseOnDevice(fNMean);
   }
   std::string Generate(std::string OpName) override
   {
      OpName = "op_" + OpName;
      if (fShapeX.empty()) throw std::runtime_error("SOFIE Batch Normalization called to Generate without being initialized first");
      size_t hw = 1;
      for (size_t i = 2; i < fShapeX.size(); i++) hw *= fShapeX[i];
      std::stringstream out;
      out << "\n" << SP << "//---- BatchNorm " << OpName << (fActivation == EActivationType::RELU ? " + Relu" : "") << "\n";
      out << SP << "{\n";
      out << SP << SP << "const sofie_batchnorm_desc d = {" << fShapeX[0] << ", " << fShapeX[1] << ", " << hw << ", " << (int)fLayout << ", "
          << (fActivation == EActivationType::RELU ? 1 : 0) << "};\n";
      out << EMIT::Call(SP + SP, "sofie_cuda_batchnorm_f32(fStream, &d, " + EMIT::Dev(fNX) + ", " + EMIT::Dev(fNScaleDev) + ", " + EMIT::Dev(fNB) +
                                    ", " + EMIT::Dev(fNMean) + ", " + EMIT::Dev(fNY) + ")");
      out << SP << "}\n";
      return out.str();
   }
};

} // namespace SOFIE
#endif
