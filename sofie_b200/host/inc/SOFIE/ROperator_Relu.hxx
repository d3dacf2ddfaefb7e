// ONNX Relu: y = x > 0 ? x : 0 (reference: src/SOFIE_core/inc/SOFIE/ROperator_Relu.hxx:54-66).
// Normally the model plan folds it into the epilogue of the producing Gemm / Conv and this operator
// emits nothing; a stand-alone Relu is one call of sofie_cuda_relu_f32.
#ifndef SOFIE_ROPERATOR_RELU
#define SOFIE_ROPERATOR_RELU

#include <sstream>

#include "SOFIE/Emit.hxx"
#include "SOFIE/RModel.hxx"
#include "SOFIE/ROperator.hxx"

namespace SOFIE {

template <typename T>
class ROperator_Relu final : public ROperator {
private:
   std::string fNX, fNY;
   std::vector<size_t> fShape;

public:
   ROperator_Relu() {}
   ROperator_Relu(std::string nameX, std::string nameY) : fNX(UTILITY::Clean_name(nameX)), fNY(UTILITY::Clean_name(nameY))
   {
      fInputTensorNames = {fNX};
      fOutputTensorNames = {fNY};
   }
   EOpKind Kind() const override { return EOpKind::Relu; }
   bool AcceptsNHWC(const std::string &) const override { return true; }
   const std::string &InputName() const { return fNX; }
   const std::string &OutputName() const { return fNY; }

   std::vector<ETensorType> TypeInference(std::vector<ETensorType> input) override { return input; }
   std::vector<std::vector<size_t>> ShapeInference(std::vector<std::vector<size_t>> input) override { return input; }

   void Initialize(RModel &model) override
   {
      if (!model.CheckIfTensorAlreadyExist(fNX)) throw std::runtime_error("SOFIE Relu Op Input Tensor " + fNX + " is not found in model");
      fShape = model.GetTensorShape(fNX);
      model.AddIntermediateTensor(fNY, model.GetTensorType(fNX), fShape);
   }
   void PlanDevice(RModel &model) override
   {
      if (model.GetTensorType(fNX) != ETensorType::FLOAT)
         throw std::runtime_error("SOFIE Relu Op: a stand-alone Relu on a quantised tensor is not generated; it is fused into QLinear operators");
      model.SetTensorLayout(fNY, model.GetTensorLayout(model.ResolveAlias(fNX)));
   }
   // elementwise: any equal split of the elements is a valid launch
   bool CanSliceBatch(size_t parts) const override { return parts > 0 && !fShape.empty() && ConvertShapeToLength(fShape) % parts == 0; }
   std::string GenerateBatchSlice(std::string OpName, size_t parts) override { return GenerateCall(OpName, parts); }
   std::string Generate(std::string OpName) override { return GenerateCall(OpName, 1); }

private:
   std::string GenerateCall(std::string OpName, size_t parts)
   {
      OpName = "op_" + OpName;
      if (fShape.empty()) throw std::runtime_error("SOFIE Operator Relu called to Generate without being initialized first");
      std::stringstream out;
      const size_t n = ConvertShapeToLength(fShape);
      out << "\n" << SP << "//------ RELU " << OpName << (parts > 1 ? ", one slice of the batch" : "") << "\n";
      out << EMIT::Call(SP, "sofie_cuda_relu_f32(fStream, " + EMIT::DevSlice(fNX, n, parts) + ", " + EMIT::DevSlice(fNY, n, parts) + ", " +
                               std::to_string(n / parts) + ")");
      return out.str();
   }
};

} // namespace SOFIE
#endif
