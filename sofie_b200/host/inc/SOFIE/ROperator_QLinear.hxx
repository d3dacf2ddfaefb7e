// Quantised operators of the CUDA path: QuantizeLinear, DequantizeLinear, QLinearMatMul, QLinearConv.
//
// The reference has none of them (src/SOFIE_parsers/src/RModelParser_ONNX.cxx:154-236 registers no
// quantised operator and :560-591 rejects int8 initialisers); they follow the ONNX operator
// definitions. Scales and zero points must be constant tensors. Arithmetic contract of the emitted
// calls: int32 accumulation, mult[n] = (a_scale * w_scale[n]) / y_scale in fp32,
// q = clamp(rne((float)acc * mult[n])) + y_zp; a following Relu is max(q, y_zp).
#ifndef SOFIE_ROPERATOR_QLINEAR
#define SOFIE_ROPERATOR_QLINEAR

#include <sstream>

#include "SOFIE/Emit.hxx"
#include "SOFIE/RModel.hxx"
#include "SOFIE/ROperator.hxx"
#include "SOFIE/ROperator_Conv.hxx"

namespace SOFIE {

namespace QUANT {
inline float ScalarFloat(RModel &model, const std::string &name, const char *what)
{
   if (!model.IsInitializedTensor(name)) throw std::runtime_error(std::string("SOFIE quantised op: ") + what + " " + name + " must be a constant");
   const auto &t = model.GetInitializedTensor(name);
   if (t.type() != ETensorType::FLOAT || t.length() != 1)
      throw std::runtime_error(std::string("SOFIE quantised op: ") + what + " " + name + " must be one float (per-tensor scale)");
   model.SetNotWritableInitializedTensor(name);
   return t.data<float>()[0];
}
inline int ScalarZeroPoint(RModel &model, const std::string &name, ETensorType expect, const char *what)
{
   if (name.empty()) return 0;
   if (!model.IsInitializedTensor(name)) throw std::runtime_error(std::string("SOFIE quantised op: ") + what + " " + name + " must be a constant");
   const auto &t = model.GetInitializedTensor(name);
   if (t.type() != expect) throw std::runtime_error(std::string("SOFIE quantised op: ") + what + " " + name + " has the wrong type");
   model.SetNotWritableInitializedTensor(name);
   int first = expect == ETensorType::UINT8 ? (int)t.data<uint8_t>()[0] : (int)t.data<int8_t>()[0];
   for (size_t i = 1; i < t.length(); i++) {
      int v = expect == ETensorType::UINT8 ? (int)t.data<uint8_t>()[i] : (int)t.data<int8_t>()[i];
      if (v != first) throw std::runtime_error(std::string("SOFIE quantised op: ") + what + " " + name + " must be uniform");
   }
   return first;
}
} // namespace QUANT

// ------------------------------------------------------------------------------------------------
class ROperator_QuantizeLinear final : public ROperator {
   std::string fNX, fNScale, fNZp, fNY;
   std::vector<size_t> fShape;
   float fScale = 1.f;
   int fZp = 0;

public:
   ROperator_QuantizeLinear(std::string nameX, std::string nameScale, std::string nameZp, std::string nameY)
      : fNX(UTILITY::Clean_name(nameX)), fNScale(UTILITY::Clean_name(nameScale)), fNZp(UTILITY::Clean_name(nameZp)),
        fNY(UTILITY::Clean_name(nameY))
   {
      fInputTensorNames = {fNX};
      fOutputTensorNames = {fNY};
   }
   EOpKind Kind() const override { return EOpKind::Quantize; }
   std::vector<ETensorType> TypeInference(std::vector<ETensorType>) override { return {ETensorType::UINT8}; }
   std::vector<std::vector<size_t>> ShapeInference(std::vector<std::vector<size_t>> input) override { return {input[0]}; }
   void Initialize(RModel &model) override
   {
      if (!model.CheckIfTensorAlreadyExist(fNX)) throw std::runtime_error("SOFIE QuantizeLinear Op Input Tensor " + fNX + " is not found in model");
      if (model.GetTensorType(fNX) != ETensorType::FLOAT) throw std::runtime_error("SOFIE QuantizeLinear Op: input must be float");
      fShape = model.GetTensorShape(fNX);
      fScale = QUANT::ScalarFloat(model, fNScale, "scale");
      fZp = QUANT::ScalarZeroPoint(model, fNZp, ETensorType::UINT8, "zero point");
      if (!(fScale > 0.f)) throw std::runtime_error("SOFIE QuantizeLinear Op: scale must be positive");
      model.AddIntermediateTensor(fNY, ETensorType::UINT8, fShape);
   }
   void PlanDevice(RModel &model) override { model.SetTensorLayout(fNY, model.GetTensorLayout(model.ResolveAlias(fNX))); }
   bool CanSliceBatch(size_t parts) const override { return parts > 0 && !fShape.empty() && fShape[0] % parts == 0; }
   std::string GenerateBatchSlice(std::string OpName, size_t parts) override { return GenerateCall(OpName, parts); }
   std::string Generate(std::string OpName) override { return GenerateCall(OpName, 1); }

private:
   std::string GenerateCall(std::string OpName, size_t parts)
   {
      std::stringstream out;
      const size_t n = ConvertShapeToLength(fShape);
      out << "\n" << SP << "//------ QuantizeLinear op_" << OpName << (parts > 1 ? ", one slice of the batch" : "") << "\n";
      out << EMIT::Call(SP, "sofie_cuda_quantize_u8(fStream, " + EMIT::DevSlice(fNX, n, parts) + ", " + EMIT::DevSlice(fNY, n, parts) + ", " +
                               std::to_string(n / parts) + ", " + EMIT::FloatLit(fScale) + ", " + std::to_string(fZp) + ")");
      return out.str();
   }
};

class ROperator_DequantizeLinear final : public ROperator {
   std::string fNX, fNScale, fNZp, fNY;
   std::vector<size_t> fShape;
   float fScale = 1.f;
   int fZp = 0;

public:
   ROperator_DequantizeLinear(std::string nameX, std::string nameScale, std::string nameZp, std::string nameY)
      : fNX(UTILITY::Clean_name(nameX)), fNScale(UTILITY::Clean_name(nameScale)), fNZp(UTILITY::Clean_name(nameZp)),
        fNY(UTILITY::Clean_name(nameY))
   {
      fInputTensorNames = {fNX};
      fOutputTensorNames = {fNY};
   }
   EOpKind Kind() const override { return EOpKind::Dequantize; }
   const std::string &OutputName() const { return fNY; }
   float Scale() const { return fScale; }
   int ZeroPoint() const { return fZp; }
   std::vector<ETensorType> TypeInference(std::vector<ETensorType>) override { return {ETensorType::FLOAT}; }
   std::vector<std::vector<size_t>> ShapeInference(std::vector<std::vector<size_t>> input) override { return {input[0]}; }
   void Initialize(RModel &model) override
   {
      if (!model.CheckIfTensorAlreadyExist(fNX)) throw std::runtime_error("SOFIE DequantizeLinear Op Input Tensor " + fNX + " is not found in model");
      if (model.GetTensorType(fNX) != ETensorType::UINT8) throw std::runtime_error("SOFIE DequantizeLinear Op: input must be uint8");
      fShape = model.GetTensorShape(fNX);
      fScale = QUANT::ScalarFloat(model, fNScale, "scale");
      fZp = QUANT::ScalarZeroPoint(model, fNZp, ETensorType::UINT8, "zero point");
      model.AddIntermediateTensor(fNY, ETensorType::FLOAT, fShape);
   }
   void PlanDevice(RModel &model) override
   {
      if (model.GetTensorLayout(model.ResolveAlias(fNX)) == ELayout::NHWC)
         throw std::runtime_error("SOFIE DequantizeLinear Op: NHWC input is not supported");
   }
   std::string Generate(std::string OpName) override
   {
      std::stringstream out;
      out << "\n" << SP << "//------ DequantizeLinear op_" << OpName << "\n";
      out << EMIT::Call(SP, "sofie_cuda_dequantize_u8(fStream, " + EMIT::Dev(fNX) + ", " + EMIT::Dev(fNY) + ", " +
                               std::to_string(ConvertShapeToLength(fShape)) + ", " + EMIT::FloatLit(fScale) + ", " + std::to_string(fZp) + ")");
      return out.str();
   }
};

// ------------------------------------------------------------------------------------------------
class ROperator_QLinearMatMul final : public ROperator {
   std::string fNA, fNAScale, fNAZp, fNB, fNBScale, fNBZp, fNYScale, fNYZp, fNY;
   std::string fNBdev, fNMult, fNCorr;
   std::string fNYFloat;       // output of a fused DequantizeLinear
   float fDequantScale = 0.f;
   std::vector<size_t> fShapeA, fShapeB, fShapeY;
   size_t fM = 0, fN = 0, fK = 0;
   float fAScale = 1.f, fYScale = 1.f;
   int fAZp = 0, fYZp = 0;
   bool fRelu = false;

public:
   ROperator_QLinearMatMul(std::string a, std::string aScale, std::string aZp, std::string b, std::string bScale, std::string bZp,
                           std::string yScale, std::string yZp, std::string y)
      : fNA(UTILITY::Clean_name(a)), fNAScale(UTILITY::Clean_name(aScale)), fNAZp(UTILITY::Clean_name(aZp)), fNB(UTILITY::Clean_name(b)),
        fNBScale(UTILITY::Clean_name(bScale)), fNBZp(UTILITY::Clean_name(bZp)), fNYScale(UTILITY::Clean_name(yScale)),
        fNYZp(UTILITY::Clean_name(yZp)), fNY(UTILITY::Clean_name(y))
   {
      fInputTensorNames = {fNA, fNB};
      fOutputTensorNames = {fNY};
   }
   EOpKind Kind() const override { return EOpKind::QLinearMatMul; }
   bool AcceptsNHWC(const std::string &input) const override { return input == fNA; }
   void FuseRelu(const std::string &reluOutput)
   {
      fRelu = true;
      fNY = reluOutput;
      fOutputTensorNames = {fNY};
   }
   const std::string &OutputName() const { return fNY; }
   int OutputZeroPoint() const { return fYZp; }
   // A DequantizeLinear with this product's zero point that is the only reader of its output: the product's own
   // launch writes the float tensor (the scale is the DequantizeLinear's, whatever the product's y_scale)
   void FuseDequantize(const std::string &floatOutput, float scale)
   {
      fNYFloat = floatOutput;
      fDequantScale = scale;
      fOutputTensorNames = {floatOutput};
   }
   std::vector<ETensorType> TypeInference(std::vector<ETensorType>) override { return {ETensorType::UINT8}; }
   std::vector<std::vector<size_t>> ShapeInference(std::vector<std::vector<size_t>> input) override
   {
      const auto &a = input[0], &b = input[1];
      if (a.size() < 2 || b.size() != 2) throw std::runtime_error("SOFIE QLinearMatMul Op: A needs rank >= 2 and B rank 2");
      if (a.back() != b[0]) throw std::runtime_error("SOFIE QLinearMatMul Op: inner dimensions differ");
      std::vector<size_t> y(a.begin(), a.end() - 1);
      y.push_back(b[1]);
      fK = b[0];
      fN = b[1];
      fM = ConvertShapeToLength(a) / fK;
      return {y};
   }
   void Initialize(RModel &model) override
   {
      if (!model.CheckIfTensorAlreadyExist(fNA)) throw std::runtime_error("SOFIE QLinearMatMul Op Input Tensor " + fNA + " is not found in model");
      if (!model.IsInitializedTensor(fNB)) throw std::runtime_error("SOFIE QLinearMatMul Op: B must be a constant int8 tensor");
      if (model.GetTensorType(fNA) != ETensorType::UINT8 || model.GetTensorType(fNB) != ETensorType::INT8)
         throw std::runtime_error("SOFIE QLinearMatMul Op: uint8 activations and int8 weights are generated");
      fShapeA = model.GetTensorShape(fNA);
      fShapeB = model.GetTensorShape(fNB);
      fShapeY = ShapeInference({fShapeA, fShapeB})[0];
      fAScale = QUANT::ScalarFloat(model, fNAScale, "a_scale");
      fYScale = QUANT::ScalarFloat(model, fNYScale, "y_scale");
      fAZp = QUANT::ScalarZeroPoint(model, fNAZp, ETensorType::UINT8, "a_zero_point");
      fYZp = QUANT::ScalarZeroPoint(model, fNYZp, ETensorType::UINT8, "y_zero_point");
      if (QUANT::ScalarZeroPoint(model, fNBZp, ETensorType::INT8, "b_zero_point") != 0)
         throw std::runtime_error("SOFIE QLinearMatMul Op: the weight zero point must be 0");
      const auto &s = model.GetInitializedTensor(fNBScale);
      if (s.type() != ETensorType::FLOAT || (s.length() != fN && s.length() != 1))
         throw std::runtime_error("SOFIE QLinearMatMul Op: b_scale must hold 1 or N floats");
      model.AddIntermediateTensor(fNY, ETensorType::UINT8, fShapeY);
   }
   void PlanDevice(RModel &model) override
   {
      // weight as [N,K], K axis in the device order of A
      const int8_t *src = model.GetInitializedTensor(fNB).data<int8_t>();
      std::vector<size_t> kperm(fK);
      for (size_t k = 0; k < fK; k++) kperm[k] = k;
      std::string owner = model.ResolveAlias(fNA);
      if (model.GetTensorLayout(owner) == ELayout::NHWC) {
         auto s4 = model.GetTensorShape(owner);
         if (s4.size() != 4 || s4[1] * s4[2] * s4[3] != fK) throw std::runtime_error("SOFIE QLinearMatMul Op: NHWC input does not flatten to K");
         size_t C = s4[1], H = s4[2], W = s4[3];
         for (size_t h = 0; h < H; h++)
            for (size_t x = 0; x < W; x++)
               for (size_t c = 0; c < C; c++) kperm[(h * W + x) * C + c] = (c * H + h) * W + x;
      }
      std::shared_ptr<void> buf(malloc(fN * fK + 1), free);
      int8_t *dst = static_cast<int8_t *>(buf.get());
      for (size_t n = 0; n < fN; n++)
         for (size_t k = 0; k < fK; k++) dst[n * fK + k] = src[kperm[k] * fN + n];
      fNBdev = fNB + "_nk_" + fNY;
      model.AddInitializedTensor(fNBdev, ETensorType::INT8, {fN, fK}, buf);
      model.UseOnDevice(fNBdev);
      // per-channel scales as N floats
      const auto &s = model.GetInitializedTensor(fNBScale);
      if (s.length() == 1) {
         std::shared_ptr<void> sb(malloc(fN * sizeof(float)), free);
         for (size_t n = 0; n < fN; n++) static_cast<float *>(sb.get())[n] = s.data<float>()[0];
         fNBScale = fNBScale + "_x" + std::to_string(fN);
         if (!model.IsInitializedTensor(fNBScale)) model.AddInitializedTensor(fNBScale, ETensorType::FLOAT, {fN}, sb);
      }
      model.UseOnDevice(fNBScale); // read on the host by the constructor; the upload is harmless
      fNMult = fNY + "_mult";
      fNCorr = fNY + "_corr";
      model.AddDeviceBuffer(fNMult, ETensorType::FLOAT, fN);
      model.AddDeviceBuffer(fNCorr, ETensorType::INT32, fN);
   }
   std::string GenerateInitCode() override
   {
      std::stringstream out;
      out << SP << "// requantisation table of " << fNY << ": mult[n] = (a_scale*w_scale[n])/y_scale, corr[n] = -a_zp*sum_k W[n][k]\n";
      out << EMIT::Call(SP, "sofie_cuda_qlinear_prepare(fStream, " + std::to_string(fN) + ", " + std::to_string(fK) + ", " +
                               EMIT::Host(fNBdev) + ".data(), 1, " + EMIT::FloatLit(fAScale) + ", " + std::to_string(fAZp) + ", " +
                               EMIT::Host(fNBScale) + ".data(), " + EMIT::FloatLit(fYScale) + ", nullptr, " + EMIT::Dev(fNMult) + ", " +
                               EMIT::Dev(fNCorr) + ")");
      return out.str();
   }
   // rows are independent: any equal split of the rows is a valid launch
   bool CanSliceBatch(size_t parts) const override { return parts > 0 && fM > 0 && fM % parts == 0; }
   std::string GenerateBatchSlice(std::string OpName, size_t parts) override { return GenerateCall(OpName, parts); }
   std::string Generate(std::string OpName) override { return GenerateCall(OpName, 1); }

private:
   std::string GenerateCall(std::string OpName, size_t parts)
   {
      std::stringstream out;
      const size_t m = fM / parts;
      out << "\n" << SP << "//--------- QLinearMatMul op_" << OpName << (fRelu ? " + Relu" : "") << ": [" << m << "," << fK << "] x [" << fK
          << "," << fN << "]" << (parts > 1 ? ", one slice of the rows" : "") << "\n";
      out << SP << "{\n";
      out << SP << SP << "const sofie_qgemm_desc d = {" << m << ", " << fN << ", " << fK << ", 1, " << fYZp << ", " << (fRelu ? 1 : 0) << "};\n";
      const std::string a = EMIT::DevSlice(fNA, fM * fK, parts);
      if (!fNYFloat.empty())
         out << EMIT::Call(SP + SP, "sofie_cuda_qlinear_matmul_f32(fStream, &d, " + a + ", " + EMIT::Dev(fNBdev) + ", " +
                                       EMIT::Dev(fNMult) + ", " + EMIT::Dev(fNCorr) + ", " + EMIT::FloatLit(fDequantScale) + ", " +
                                       EMIT::DevSlice(fNYFloat, fM * fN, parts) + ")  /* + DequantizeLinear */");
      else
         out << EMIT::Call(SP + SP, "sofie_cuda_qlinear_matmul(fStream, &d, " + a + ", " + EMIT::Dev(fNBdev) + ", " +
                                       EMIT::Dev(fNMult) + ", " + EMIT::Dev(fNCorr) + ", " + EMIT::DevSlice(fNY, fM * fN, parts) + ")");
      out << SP << "}\n";
      return out.str();
   }
};

// ------------------------------------------------------------------------------------------------
class ROperator_QLinearConv final : public ROperator {
   ConvAttributes fAttr;
   std::string fNX, fNXScale, fNXZp, fNW, fNWScale, fNWZp, fNYScale, fNYZp, fNB, fNY;
   std::string fNWdev, fNMult, fNCorr, fNOut;
   std::vector<size_t> fShapeX, fShapeW, fShapeY, fShapeOut;
   float fXScale = 1.f, fYScale = 1.f;
   int fXZp = 0, fYZp = 0;
   bool fRelu = false, fPacked = false;
   int fPool = 0;
   ELayout fLayoutX = ELayout::NCHW, fLayoutY = ELayout::NCHW;

public:
   ROperator_QLinearConv(std::string autopad, std::vector<size_t> dilations, size_t group, std::vector<size_t> kernelShape,
                         std::vector<size_t> pads, std::vector<size_t> strides, std::string x, std::string xScale, std::string xZp,
                         std::string w, std::string wScale, std::string wZp, std::string yScale, std::string yZp, std::string bias,
                         std::string y)
      : fNX(UTILITY::Clean_name(x)), fNXScale(UTILITY::Clean_name(xScale)), fNXZp(UTILITY::Clean_name(xZp)), fNW(UTILITY::Clean_name(w)),
        fNWScale(UTILITY::Clean_name(wScale)), fNWZp(UTILITY::Clean_name(wZp)), fNYScale(UTILITY::Clean_name(yScale)),
        fNYZp(UTILITY::Clean_name(yZp)), fNB(UTILITY::Clean_name(bias)), fNY(UTILITY::Clean_name(y))
   {
      fAttr.autopad = autopad;
      fAttr.dilations = dilations;
      fAttr.group = group;
      fAttr.kernel_shape = kernelShape;
      fAttr.pads = pads;
      fAttr.strides = strides;
      fInputTensorNames = {fNX, fNW};
      fOutputTensorNames = {fNY};
      fNOut = fNY;
   }
   EOpKind Kind() const override { return EOpKind::QLinearConv; }
   bool AcceptsNHWC(const std::string &input) const override { return input == fNX; }
   const std::string &OutputName() const { return fNOut; }
   void FuseRelu(const std::string &o)
   {
      fRelu = true;
      fNOut = o;
      fOutputTensorNames = {fNOut};
   }
   void FusePool2x2(const std::string &o)
   {
      fPool = 2;
      fNOut = o;
      fOutputTensorNames = {fNOut};
   }
   std::vector<ETensorType> TypeInference(std::vector<ETensorType>) override { return {ETensorType::UINT8}; }
   std::vector<std::vector<size_t>> ShapeInference(std::vector<std::vector<size_t>> input) override
   {
      fAttr.Resolve(input[0], input[1]);
      if (fAttr.volume) throw std::runtime_error("SOFIE QLinearConv Op: 3-D quantised convolutions are not generated");
      return {fAttr.OutputShape(input[0], input[1])};
   }
   void Initialize(RModel &model) override
   {
      if (!model.CheckIfTensorAlreadyExist(fNX)) throw std::runtime_error("SOFIE QLinearConv Op Input Tensor " + fNX + " is not found in model");
      if (!model.IsInitializedTensor(fNW)) throw std::runtime_error("SOFIE QLinearConv Op: weights must be a constant int8 tensor");
      if (model.GetTensorType(fNX) != ETensorType::UINT8 || model.GetTensorType(fNW) != ETensorType::INT8)
         throw std::runtime_error("SOFIE QLinearConv Op: uint8 activations and int8 weights are generated");
      fShapeX = model.GetTensorShape(fNX);
      fShapeW = model.GetTensorShape(fNW);
      fShapeY = ShapeInference({fShapeX, fShapeW})[0];
      if (fAttr.group != 1 || fAttr.dH != 1 || fAttr.dW != 1) throw std::runtime_error("SOFIE QLinearConv Op: group and dilation must be 1");
      fXScale = QUANT::ScalarFloat(model, fNXScale, "x_scale");
      fYScale = QUANT::ScalarFloat(model, fNYScale, "y_scale");
      fXZp = QUANT::ScalarZeroPoint(model, fNXZp, ETensorType::UINT8, "x_zero_point");
      fYZp = QUANT::ScalarZeroPoint(model, fNYZp, ETensorType::UINT8, "y_zero_point");
      if (QUANT::ScalarZeroPoint(model, fNWZp, ETensorType::INT8, "w_zero_point") != 0)
         throw std::runtime_error("SOFIE QLinearConv Op: the weight zero point must be 0");
      const auto &s = model.GetInitializedTensor(fNWScale);
      if (s.type() != ETensorType::FLOAT || (s.length() != fShapeW[0] && s.length() != 1))
         throw std::runtime_error("SOFIE QLinearConv Op: w_scale must hold 1 or Cout floats");
      if (!fNB.empty() && (!model.IsInitializedTensor(fNB) || model.GetTensorType(fNB) != ETensorType::INT32))
         throw std::runtime_error("SOFIE QLinearConv Op: bias must be a constant int32 tensor");
      model.AddIntermediateTensor(fNY, ETensorType::UINT8, fShapeY);
   }
   void PlanDevice(RModel &model) override
   {
      fLayoutX = model.GetTensorLayout(model.ResolveAlias(fNX));
      fShapeOut = model.GetTensorShape(fNOut);
      fLayoutY = model.CanStayNHWC(fNOut) ? ELayout::NHWC : ELayout::NCHW;
      model.SetTensorLayout(fNOut, fLayoutY);
      fPacked = fLayoutX == ELayout::NHWC;
      fNWdev = fNW;
      size_t Cout = fShapeW[0], C = fShapeW[1], kH = fShapeW[2], kW = fShapeW[3];
      if (fPacked) {
         const int8_t *src = model.GetInitializedTensor(fNW).data<int8_t>();
         std::shared_ptr<void> buf(malloc(Cout * C * kH * kW + 1), free);
         int8_t *dst = static_cast<int8_t *>(buf.get());
         for (size_t o = 0; o < Cout; o++)
            for (size_t c = 0; c < C; c++)
               for (size_t r = 0; r < kH; r++)
                  for (size_t s = 0; s < kW; s++) dst[((o * kH + r) * kW + s) * C + c] = src[((o * C + c) * kH + r) * kW + s];
         fNWdev = fNW + "_ohwi";
         if (!model.IsInitializedTensor(fNWdev)) model.AddInitializedTensor(fNWdev, ETensorType::INT8, {Cout, kH, kW, C}, buf);
      }
      model.UseOnDevice(fNWdev);
      const auto &s = model.GetInitializedTensor(fNWScale);
      if (s.length() == 1) {
         std::shared_ptr<void> sb(malloc(Cout * sizeof(float)), free);
         for (size_t n = 0; n < Cout; n++) static_cast<float *>(sb.get())[n] = s.data<float>()[0];
         fNWScale = fNWScale + "_x" + std::to_string(Cout);
         if (!model.IsInitializedTensor(fNWScale)) model.AddInitializedTensor(fNWScale, ETensorType::FLOAT, {Cout}, sb);
      }
      model.UseOnDevice(fNWScale);
      if (!fNB.empty()) model.UseOnDevice(fNB);
      fNMult = fNOut + "_mult";
      fNCorr = fNOut + "_bias";
      model.AddDeviceBuffer(fNMult, ETensorType::FLOAT, Cout);
      model.AddDeviceBuffer(fNCorr, ETensorType::INT32, Cout);
   }
   std::string GenerateInitCode() override
   {
      std::stringstream out;
      size_t rows = fShapeW[1] * fShapeW[2] * fShapeW[3];
      out << SP << "// requantisation table of " << fNOut << " (the zero point of the input is applied per tap inside the kernel)\n";
      out << EMIT::Call(SP, "sofie_cuda_qlinear_prepare(fStream, " + std::to_string(fShapeW[0]) + ", " + std::to_string(rows) + ", " +
                               EMIT::Host(fNWdev) + ".data(), 1, " + EMIT::FloatLit(fXScale) + ", 0, " + EMIT::Host(fNWScale) + ".data(), " +
                               EMIT::FloatLit(fYScale) + ", " + (fNB.empty() ? std::string("nullptr") : EMIT::Host(fNB) + ".data()") + ", " +
                               EMIT::Dev(fNMult) + ", " + EMIT::Dev(fNCorr) + ")");
      return out.str();
   }
   // the samples of a batch are independent: any equal split of the batch axis is a valid launch
   bool CanSliceBatch(size_t parts) const override { return parts > 0 && !fShapeX.empty() && fShapeX[0] % parts == 0; }
   std::string GenerateBatchSlice(std::string OpName, size_t parts) override { return GenerateCall(OpName, parts); }
   std::string Generate(std::string OpName) override { return GenerateCall(OpName, 1); }

private:
   std::string GenerateCall(std::string OpName, size_t parts)
   {
      std::stringstream out;
      out << "\n" << SP << "//----  operator QLinearConv op_" << OpName << (fRelu ? " + Relu" : "") << (fPool ? " + MaxPool2x2" : "") << " -> "
          << fNOut << " " << ConvertShapeToString(fShapeOut) << (fLayoutY == ELayout::NHWC ? " (NHWC)" : "")
          << (parts > 1 ? ", one slice of the batch" : "") << "\n";
      out << SP << "{\n";
      out << SP << SP << "const sofie_qconv2d_desc d = {" << fShapeX[0] / parts << ", " << fShapeX[1] << ", " << fShapeX[2] << ", " << fShapeX[3]
          << ", " << fShapeW[0] << ", " << fAttr.kH << ", " << fAttr.kW << ", " << fAttr.padH << ", " << fAttr.padW << ", " << fAttr.sH
          << ", " << fAttr.sW << ", " << (int)fLayoutX << ", " << (int)fLayoutY << ", " << (fPacked ? 1 : 0) << ", " << fXZp << ", "
          << fYZp << ", " << (fRelu ? 1 : 0) << ", " << fPool << "};\n";
      out << EMIT::Call(SP + SP, "sofie_cuda_qlinear_conv2d(fStream, &d, " + EMIT::DevSlice(fNX, ConvertShapeToLength(fShapeX), parts) + ", " +
                                    EMIT::Dev(fNWdev) + ", " + EMIT::Dev(fNMult) + ", " +
                                    (fNB.empty() ? std::string("nullptr") : EMIT::Dev(fNCorr)) + ", " +
                                    EMIT::DevSlice(fNOut, ConvertShapeToLength(fShapeOut), parts) + ")");
      out << SP << "}\n";
      return out.str();
   }
};

} // namespace SOFIE

#endif
