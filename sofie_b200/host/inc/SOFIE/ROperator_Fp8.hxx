// FP8 (E4M3) GEMM chain on the CUDA path. The reference has no FP8 operator and ONNX defines no
// matrix product on FLOAT8E4M3FN tensors, so the chain is written with
//   QuantizeLinear (zero point of type FLOAT8E4M3FN)  float / bfloat16 -> E4M3, y = sat(rne(x / scale))
//   Fp8Gemm        (custom operator, registered like any RegisterOperator extension)
//                  Y = act((A_q . W_q^T) * a_scale * w_scale + bias), rounded to bfloat16; with
//                  out_scale > 0 the output is the E4M3 quantisation of that bfloat16 value for the
//                  next layer (what a following QuantizeLinear would compute), else bfloat16
//   Cast           bfloat16 <-> float
// W_q is an initialiser of type FLOAT8E4M3FN stored [N, K]; scales are static attributes, or -- "scales computed from
// amax" at run time -- come from
//   DynamicQuantizeE4M3 (custom operator)  X -> (Y = e4m3(x / scale), scale = max|x| / 448 as a one-element float tensor)
// whose second output is the fourth input of the Fp8Gemm that reads Y; such an Fp8Gemm writes bfloat16 (the next layer's
// scale is not known before the product is complete) and the next DynamicQuantizeE4M3 quantises it.
#ifndef SOFIE_ROPERATOR_FP8
#define SOFIE_ROPERATOR_FP8

#include <sstream>

#include "SOFIE/Emit.hxx"
#include "SOFIE/RModel.hxx"
#include "SOFIE/ROperator.hxx"

namespace SOFIE {

class ROperator_QuantizeE4M3 final : public ROperator {
   std::string fNX, fNScale, fNY;
   std::vector<size_t> fShape;
   float fScale = 1.f;
   ETensorType fInType = ETensorType::FLOAT;

public:
   ROperator_QuantizeE4M3(std::string nameX, std::string nameScale, std::string nameY)
      : fNX(UTILITY::Clean_name(nameX)), fNScale(UTILITY::Clean_name(nameScale)), fNY(UTILITY::Clean_name(nameY))
   {
      fInputTensorNames = {fNX};
      fOutputTensorNames = {fNY};
   }
   EOpKind Kind() const override { return EOpKind::Quantize; }
   std::vector<ETensorType> TypeInference(std::vector<ETensorType>) override { return {ETensorType::FLOAT8E4M3FN}; }
   std::vector<std::vector<size_t>> ShapeInference(std::vector<std::vector<size_t>> input) override { return {input[0]}; }
   void Initialize(RModel &model) override
   {
      if (!model.CheckIfTensorAlreadyExist(fNX)) throw std::runtime_error("SOFIE QuantizeLinear Op Input Tensor " + fNX + " is not found in model");
      fInType = model.GetTensorType(fNX);
      if (fInType != ETensorType::FLOAT && fInType != ETensorType::BFLOAT16)
         throw std::runtime_error("SOFIE QuantizeLinear Op to FLOAT8E4M3FN: input must be float or bfloat16");
      if (!model.IsInitializedTensor(fNScale)) throw std::runtime_error("SOFIE QuantizeLinear Op: scale " + fNScale + " must be a constant");
      const auto &t = model.GetInitializedTensor(fNScale);
      if (t.type() != ETensorType::FLOAT || t.length() != 1) throw std::runtime_error("SOFIE QuantizeLinear Op: scale must be one float");
      fScale = t.data<float>()[0];
      if (!(fScale > 0.f)) throw std::runtime_error("SOFIE QuantizeLinear Op: scale must be positive");
      model.SetNotWritableInitializedTensor(fNScale);
      fShape = model.GetTensorShape(fNX);
      model.AddIntermediateTensor(fNY, ETensorType::FLOAT8E4M3FN, fShape);
   }
   bool CanSliceBatch(size_t parts) const override { return parts > 0 && !fShape.empty() && fShape[0] % parts == 0; }
   std::string GenerateBatchSlice(std::string OpName, size_t parts) override { return GenerateCall(OpName, parts); }
   std::string Generate(std::string OpName) override { return GenerateCall(OpName, 1); }

private:
   std::string GenerateCall(std::string OpName, size_t parts)
   {
      std::stringstream out;
      const size_t n = ConvertShapeToLength(fShape);
      out << "\n" << SP << "//------ QuantizeLinear (E4M3) op_" << OpName << (parts > 1 ? ", one slice of the batch" : "") << "\n";
      out << EMIT::Call(SP, std::string(fInType == ETensorType::FLOAT ? "sofie_cuda_quantize_e4m3_f32" : "sofie_cuda_quantize_e4m3_bf16") +
                               "(fStream, " + EMIT::DevSlice(fNX, n, parts) + ", " + EMIT::DevSlice(fNY, n, parts) + ", " + std::to_string(n / parts) + ", " +
                               EMIT::FloatLit(fScale) + ")");
      return out.str();
   }
};

class ROperator_DynamicQuantizeE4M3 final : public ROperator {
   std::string fNX, fNY, fNScale;
   std::vector<size_t> fShape;
   ETensorType fInType = ETensorType::FLOAT;

public:
   ROperator_DynamicQuantizeE4M3(std::string nameX, std::string nameY, std::string nameScale)
      : fNX(UTILITY::Clean_name(nameX)), fNY(UTILITY::Clean_name(nameY)), fNScale(UTILITY::Clean_name(nameScale))
   {
      fInputTensorNames = {fNX};
      fOutputTensorNames = {fNY, fNScale};
   }
   EOpKind Kind() const override { return EOpKind::Quantize; }
   std::vector<ETensorType> TypeInference(std::vector<ETensorType>) override { return {ETensorType::FLOAT8E4M3FN, ETensorType::FLOAT}; }
   std::vector<std::vector<size_t>> ShapeInference(std::vector<std::vector<size_t>> input) override { return {input[0], {1}}; }
   void Initialize(RModel &model) override
   {
      if (!model.CheckIfTensorAlreadyExist(fNX)) throw std::runtime_error("SOFIE DynamicQuantizeE4M3 Op Input Tensor " + fNX + " is not found in model");
      fInType = model.GetTensorType(fNX);
      if (fInType != ETensorType::FLOAT && fInType != ETensorType::BFLOAT16)
         throw std::runtime_error("SOFIE DynamicQuantizeE4M3 Op: input must be float or bfloat16");
      fShape = model.GetTensorShape(fNX);
      model.AddIntermediateTensor(fNY, ETensorType::FLOAT8E4M3FN, fShape);
      model.AddIntermediateTensor(fNScale, ETensorType::FLOAT, std::vector<size_t>{1});
   }
   std::string Generate(std::string OpName) override
   {
      std::stringstream out;
      out << "\n" << SP << "//------ DynamicQuantizeE4M3 op_" << OpName << ": scale = max|x| / 448 on the device\n";
      out << EMIT::Call(SP, std::string(fInType == ETensorType::FLOAT ? "sofie_cuda_dynamic_quantize_e4m3_f32" : "sofie_cuda_dynamic_quantize_e4m3_bf16") +
                               "(fStream, " + EMIT::Dev(fNX) + ", " + EMIT::Dev(fNY) + ", " + std::to_string(ConvertShapeToLength(fShape)) + ", " +
                               EMIT::Dev(fNScale) + ")");
      return out.str();
   }
};

class ROperator_Cast final : public ROperator {
   std::string fNX, fNY;
   ETensorType fTo, fFrom = ETensorType::UNDEFINED;
   std::vector<size_t> fShape;

public:
   ROperator_Cast(ETensorType to, std::string nameX, std::string nameY) : fNX(UTILITY::Clean_name(nameX)), fNY(UTILITY::Clean_name(nameY)), fTo(to)
   {
      fInputTensorNames = {fNX};
      fOutputTensorNames = {fNY};
   }
   EOpKind Kind() const override { return EOpKind::Cast; }
   const std::string &InputName() const { return fNX; }
   const std::string &OutputName() const { return fNY; }
   bool IsBf16ToFloat() const { return fFrom == ETensorType::BFLOAT16 && fTo == ETensorType::FLOAT; }
   std::vector<ETensorType> TypeInference(std::vector<ETensorType>) override { return {fTo}; }
   std::vector<std::vector<size_t>> ShapeInference(std::vector<std::vector<size_t>> input) override { return {input[0]}; }
   void Initialize(RModel &model) override
   {
      if (!model.CheckIfTensorAlreadyExist(fNX)) throw std::runtime_error("SOFIE Cast Op Input Tensor " + fNX + " is not found in model");
      fFrom = model.GetTensorType(fNX);
      const bool ok = (fFrom == ETensorType::BFLOAT16 && fTo == ETensorType::FLOAT) || (fFrom == ETensorType::FLOAT && fTo == ETensorType::BFLOAT16);
      if (!ok) throw std::runtime_error("SOFIE Cast Op: only bfloat16 <-> float is generated for the device");
      fShape = model.GetTensorShape(fNX);
      model.AddIntermediateTensor(fNY, fTo, fShape);
   }
   void PlanDevice(RModel &model) override { model.SetTensorLayout(fNY, model.GetTensorLayout(model.ResolveAlias(fNX))); }
   std::string Generate(std::string OpName) override
   {
      std::stringstream out;
      out << "\n" << SP << "//------ Cast op_" << OpName << "\n";
      out << EMIT::Call(SP, std::string(fTo == ETensorType::FLOAT ? "sofie_cuda_cast_bf16_f32" : "sofie_cuda_cast_f32_bf16") + "(fStream, " +
                               EMIT::Dev(fNX) + ", " + EMIT::Dev(fNY) + ", " + std::to_string(ConvertShapeToLength(fShape)) + ")");
      return out.str();
   }
};

class ROperator_Fp8Gemm final : public ROperator {
   std::string fNA, fNW, fNB, fNY;
   float fAScale, fWScale, fOutScale;
   bool fRelu;
   std::vector<size_t> fShapeA, fShapeW;
   std::string fNYFloat; // set when a Cast to float behind this layer is written by the same launch
   std::string fNAScale; // run-time activation scale (second output of a DynamicQuantizeE4M3), empty for a static scale

public:
   ROperator_Fp8Gemm(float aScale, float wScale, float outScale, bool relu, std::string nameA, std::string nameW, std::string nameB,
                     std::string nameY, std::string nameAScale = "")
      : fNA(UTILITY::Clean_name(nameA)), fNW(UTILITY::Clean_name(nameW)), fNB(UTILITY::Clean_name(nameB)), fNY(UTILITY::Clean_name(nameY)),
        fAScale(aScale), fWScale(wScale), fOutScale(outScale), fRelu(relu), fNAScale(nameAScale.empty() ? "" : UTILITY::Clean_name(nameAScale))
   {
      fInputTensorNames = {fNA};
      if (!fNAScale.empty()) fInputTensorNames.push_back(fNAScale);
      fOutputTensorNames = {fNY};
   }
   EOpKind Kind() const override { return EOpKind::Fp8Gemm; }
   const std::string &OutputName() const { return fNY; }
   bool WritesBf16() const { return !(fOutScale > 0.f); }
   // a bfloat16 -> float Cast that is the only reader of this layer's output: the epilogue writes the float tensor
   void FuseCastToFloat(const std::string &castOutput)
   {
      fNYFloat = castOutput;
      fOutputTensorNames = {castOutput};
   }
   std::vector<ETensorType> TypeInference(std::vector<ETensorType>) override
   {
      return {fOutScale > 0.f ? ETensorType::FLOAT8E4M3FN : ETensorType::BFLOAT16};
   }
   std::vector<std::vector<size_t>> ShapeInference(std::vector<std::vector<size_t>> input) override { return {{input[0][0], input[1][0]}}; }
   void Initialize(RModel &model) override
   {
      if (!model.CheckIfTensorAlreadyExist(fNA)) throw std::runtime_error("SOFIE Fp8Gemm Op Input Tensor " + fNA + " is not found in model");
      if (model.GetTensorType(fNA) != ETensorType::FLOAT8E4M3FN) throw std::runtime_error("SOFIE Fp8Gemm Op: A must be FLOAT8E4M3FN");
      if (!model.IsInitializedTensor(fNW) || model.GetTensorType(fNW) != ETensorType::FLOAT8E4M3FN)
         throw std::runtime_error("SOFIE Fp8Gemm Op: W " + fNW + " must be a FLOAT8E4M3FN constant stored [N, K]");
      if (!fNB.empty() && (!model.IsInitializedTensor(fNB) || model.GetTensorType(fNB) != ETensorType::FLOAT))
         throw std::runtime_error("SOFIE Fp8Gemm Op: bias " + fNB + " must be a float constant");
      if (!(fAScale > 0.f) || !(fWScale > 0.f) || fOutScale < 0.f) throw std::runtime_error("SOFIE Fp8Gemm Op: scales must be positive");
      if (!fNAScale.empty()) {
         if (!model.CheckIfTensorAlreadyExist(fNAScale) || model.GetTensorType(fNAScale) != ETensorType::FLOAT || ConvertShapeToLength(model.GetTensorShape(fNAScale)) != 1)
            throw std::runtime_error("SOFIE Fp8Gemm Op: the run-time activation scale " + fNAScale + " must be a one-element float tensor");
         if (fOutScale > 0.f) throw std::runtime_error("SOFIE Fp8Gemm Op: with a run-time activation scale the output is bfloat16 (out_scale must be 0)");
      }
      fShapeA = model.GetTensorShape(fNA);
      fShapeW = model.GetTensorShape(fNW);
      if (fShapeA.size() != 2 || fShapeW.size() != 2 || fShapeA[1] != fShapeW[1])
         throw std::runtime_error("SOFIE Fp8Gemm Op: A [M, K] and W [N, K] do not match: " + ConvertShapeToString(fShapeA) + " " +
                                  ConvertShapeToString(fShapeW));
      if (!fNB.empty() && ConvertShapeToLength(model.GetTensorShape(fNB)) != fShapeW[0])
         throw std::runtime_error("SOFIE Fp8Gemm Op: bias must hold one value per output column");
      model.AddIntermediateTensor(fNY, fOutScale > 0.f ? ETensorType::FLOAT8E4M3FN : ETensorType::BFLOAT16, std::vector<size_t>{fShapeA[0], fShapeW[0]});
   }
   void PlanDevice(RModel &model) override
   {
      model.UseOnDevice(fNW);
      if (!fNB.empty()) model.UseOnDevice(fNB);
   }
   // rows are independent once the activation scale is a constant (a run-time scale is the maximum over ALL rows)
   bool CanSliceBatch(size_t parts) const override { return parts > 0 && fNAScale.empty() && !fShapeA.empty() && fShapeA[0] % parts == 0; }
   std::string GenerateBatchSlice(std::string OpName, size_t parts) override { return GenerateCall(OpName, parts); }
   std::string Generate(std::string OpName) override { return GenerateCall(OpName, 1); }

private:
   std::string GenerateCall(std::string OpName, size_t parts)
   {
      std::stringstream out;
      out << "\n" << SP << "//------ Fp8Gemm op_" << OpName << (fRelu ? " + Relu" : "")
          << (fOutScale > 0.f ? " -> E4M3" : (fNYFloat.empty() ? " -> bfloat16" : " -> bfloat16 -> float (Cast fused)"))
          << (parts > 1 ? ", one slice of the rows" : "") << "\n";
      out << SP << "{\n";
      out << SP << SP << "const sofie_fp8_gemm_desc d = {" << fShapeA[0] / parts << ", " << fShapeW[0] << ", " << fShapeA[1] << ", "
          << EMIT::FloatLit(fAScale) << ", " << EMIT::FloatLit(fWScale) << ", " << (fRelu ? 1 : 0) << ", " << EMIT::FloatLit(fOutScale) << "};\n";
      const std::string bias = fNB.empty() ? std::string("nullptr") : EMIT::Dev(fNB);
      const size_t lenA = fShapeA[0] * fShapeA[1], lenY = fShapeA[0] * fShapeW[0];
      if (!fNAScale.empty()) {
         // activation scale from device memory, written by the DynamicQuantizeE4M3 in front of this layer
         out << EMIT::Call(SP + SP, "sofie_cuda_gemm_e4m3_dynamic(fStream, &d, " + EMIT::Dev(fNA) + ", " + EMIT::Dev(fNAScale) + ", " + EMIT::Dev(fNW) + ", " + bias +
                                       ", " + (fNYFloat.empty() ? EMIT::Dev(fNY) : std::string("nullptr")) + ", " +
                                       (fNYFloat.empty() ? std::string("nullptr") : EMIT::Dev(fNYFloat)) + ")");
      } else if (!fNYFloat.empty()) {
         out << EMIT::Call(SP + SP, "sofie_cuda_gemm_e4m3_f32(fStream, &d, " + EMIT::DevSlice(fNA, lenA, parts) + ", " + EMIT::Dev(fNW) + ", " + bias + ", " +
                                       EMIT::DevSlice(fNYFloat, lenY, parts) + ")");
      } else {
         const std::string ybf = fOutScale > 0.f ? std::string("nullptr") : EMIT::DevSlice(fNY, lenY, parts);
         const std::string yq = fOutScale > 0.f ? EMIT::DevSlice(fNY, lenY, parts) : std::string("nullptr");
         out << EMIT::Call(SP + SP, "sofie_cuda_gemm_e4m3(fStream, &d, " + EMIT::DevSlice(fNA, lenA, parts) + ", " + EMIT::Dev(fNW) + ", " + bias + ", " + ybf + ", " + yq + ")");
      }
      out << SP << "}\n";
      return out.str();
   }
};

} // namespace SOFIE
#endif
