// ONNX Conv (1-D and 2-D), optional fused Relu and MaxPool 2x2.
//
// Constructor signatures as in the reference (src/SOFIE_core/inc/SOFIE/ROperator_Conv.hxx:52-92) and
// the same attribute rules: no `pads` attribute means pad 1 (:136-139), SAME_UPPER / SAME_LOWER give
// k/2 after the reference's averaging of asymmetric pads (:140-158, :387-410), output extent
// (in + pads - k_dilated) / stride + 1 (:178-199). The reference emits a weight repack, a per-image
// UTILITY::Im2col, sgemm_ and saxpy_ (:302-522); this emits ONE call of sofie_cuda_conv2d_f32 and
// registers no `_f` / `_xcol` scratch tensors. When the model plan fuses a following Relu and
// MaxPool(2x2, stride 2) the call's descriptor carries them and the output tensor is the pool's.
// A 1-D convolution [N,C,L] * [Cout,C/g,k] (reference: fDim == 1, :95-201) is the 2-D one on an image of height 1
// (kernel 1 x k, no padding in the added dimension): same call, same kernels. 3-D convolutions are outside the CUDA path.
#ifndef SOFIE_ROPERATOR_CONV
#define SOFIE_ROPERATOR_CONV

#include <cmath>
#include <sstream>

#include "SOFIE/Emit.hxx"
#include "SOFIE/RModel.hxx"
#include "SOFIE/ROperator.hxx"

namespace SOFIE {

// Attribute resolution shared by Conv and QLinearConv.
struct ConvAttributes {
   std::string autopad = "NOTSET";
   std::vector<size_t> dilations, kernel_shape, pads, strides;
   size_t group = 1;
   // resolved values
   size_t kH = 0, kW = 0, padH = 0, padW = 0, sH = 1, sW = 1, dH = 1, dW = 1;

   bool oneD = false; // rank-3 tensors: the single spatial axis is treated as the width of an image of height 1
   // rank-5 tensors [N, C, D, H, W] (reference: fDim == 3): kernel, averaged pads, strides and dilations of the three axes
   bool volume = false;
   size_t k3[3] = {0, 0, 0}, pad3[3] = {0, 0, 0}, s3[3] = {1, 1, 1}, d3[3] = {1, 1, 1};

   void Resolve(const std::vector<size_t> &shapeX, const std::vector<size_t> &shapeW)
   {
      oneD = shapeX.size() == 3 && shapeW.size() == 3;
      volume = shapeX.size() == 5 && shapeW.size() == 5;
      if (!oneD && !volume && (shapeX.size() != 4 || shapeW.size() != 4))
         throw std::runtime_error("SOFIE Conv Op: convolutions are generated for rank-3, rank-4 and rank-5 tensors");
      if (group == 0) group = shapeX[1] / shapeW[1];
      if (volume) {
         std::vector<size_t> p;
         for (size_t a = 0; a < 3; a++) {
            k3[a] = kernel_shape.empty() ? shapeW[2 + a] : kernel_shape.at(a);
            if (k3[a] != shapeW[2 + a]) throw std::runtime_error("SOFIE Conv Op: kernel_shape differs from the weight tensor");
            d3[a] = dilations.empty() ? 1 : dilations.at(a);
            s3[a] = strides.empty() ? 1 : strides.at(a);
         }
         if (autopad == "NOTSET") {
            p = pads.empty() ? std::vector<size_t>(6, 1) : pads; // the reference's default is 1, not 0
         } else if (autopad == "SAME_UPPER" || autopad == "SAME_LOWER") {
            p.assign(6, 0);
            for (size_t a = 0; a < 3; a++) {
               const size_t e = k3[a] + (d3[a] - 1) * (k3[a] - 1);
               p[a] = p[a + 3] = e / 2;
               if (e % 2 == 1) (autopad == "SAME_UPPER") ? p[a]++ : p[a + 3]++;
            }
         } else if (autopad == "VALID") {
            p.assign(6, 0);
         } else {
            throw std::runtime_error("SOFIE Conv Op invalid auto_pad " + autopad);
         }
         if (p.size() != 6) throw std::runtime_error("SOFIE Conv Op: pads of a 3-D convolution must have 6 values");
         // asymmetric padding is averaged, as for the 2-D operator
         for (size_t a = 0; a < 3; a++) pad3[a] = (p[a] == p[a + 3]) ? p[a] : (p[a] + p[a + 3]) / 2;
         pads = p;
         return;
      }
      if (oneD) {
         kH = 1;
         kW = kernel_shape.empty() ? shapeW[2] : kernel_shape[0];
         if (kW != shapeW[2]) throw std::runtime_error("SOFIE Conv Op: kernel_shape differs from the weight tensor");
         dH = sH = 1;
         dW = dilations.empty() ? 1 : dilations[0];
         sW = strides.empty() ? 1 : strides[0];
         const size_t eW = kW + (dW - 1) * (kW - 1);
         std::vector<size_t> p; // {begin, end} of the one spatial axis
         if (autopad == "NOTSET") {
            p = pads.empty() ? std::vector<size_t>{1, 1} : pads; // the reference's default is 1, not 0 (:136-139)
         } else if (autopad == "SAME_UPPER" || autopad == "SAME_LOWER") {
            p = {eW / 2, eW / 2};
            if (eW % 2 == 1) (autopad == "SAME_UPPER") ? p[0]++ : p[1]++;
         } else if (autopad == "VALID") {
            p = {0, 0};
         } else {
            throw std::runtime_error("SOFIE Conv Op invalid auto_pad " + autopad);
         }
         if (p.size() != 2) throw std::runtime_error("SOFIE Conv Op: pads of a 1-D convolution must have 2 values");
         padH = 0;
         padW = (p[0] == p[1]) ? p[0] : (p[0] + p[1]) / 2; // averaged like the 2-D case
         pads = {0, p[0], 0, p[1]};
         return;
      }
      kH = kernel_shape.empty() ? shapeW[2] : kernel_shape[0];
      kW = kernel_shape.empty() ? shapeW[3] : kernel_shape[1];
      if (kH != shapeW[2] || kW != shapeW[3]) throw std::runtime_error("SOFIE Conv Op: kernel_shape differs from the weight tensor");
      dH = dilations.empty() ? 1 : dilations[0];
      dW = dilations.size() < 2 ? dH : dilations[1];
      sH = strides.empty() ? 1 : strides[0];
      sW = strides.size() < 2 ? sH : strides[1];
      const size_t eH = kH + (dH - 1) * (kH - 1), eW = kW + (dW - 1) * (kW - 1);
      std::vector<size_t> p;
      if (autopad == "NOTSET") {
         p = pads.empty() ? std::vector<size_t>{1, 1, 1, 1} : pads; // the reference's default is 1, not 0
      } else if (autopad == "SAME_UPPER" || autopad == "SAME_LOWER") {
         p = {eH / 2, eW / 2, eH / 2, eW / 2};
         if (eH % 2 == 1) (autopad == "SAME_UPPER") ? p[0]++ : p[2]++;
         if (eW % 2 == 1) (autopad == "SAME_UPPER") ? p[1]++ : p[3]++;
      } else if (autopad == "VALID") {
         p = {0, 0, 0, 0};
      } else {
         throw std::runtime_error("SOFIE Conv Op invalid auto_pad " + autopad);
      }
      if (p.size() != 4) throw std::runtime_error("SOFIE Conv Op: pads must have 4 values");
      // asymmetric padding: the reference warns and averages; the same rule keeps results identical
      padH = (p[0] == p[2]) ? p[0] : (p[0] + p[2]) / 2;
      padW = (p[1] == p[3]) ? p[1] : (p[1] + p[3]) / 2;
      pads = p;
   }
   std::vector<size_t> OutputShape(const std::vector<size_t> &shapeX, const std::vector<size_t> &shapeW) const
   {
      const size_t eH = kH + (dH - 1) * (kH - 1), eW = kW + (dW - 1) * (kW - 1);
      if (oneD) return {shapeX[0], shapeW[0], (shapeX[2] + pads[1] + pads[3] - eW) / sW + 1};
      if (volume) {
         std::vector<size_t> y = {shapeX[0], shapeW[0]};
         for (size_t a = 0; a < 3; a++) y.push_back((shapeX[2 + a] + pads[a] + pads[a + 3] - (k3[a] + (d3[a] - 1) * (k3[a] - 1))) / s3[a] + 1);
         return y;
      }
      // the reference sizes the output from the un-averaged pads (ROperator_Conv.hxx:178-189)
      size_t oH = (shapeX[2] + pads[0] + pads[2] - eH) / sH + 1;
      size_t oW = (shapeX[3] + pads[1] + pads[3] - eW) / sW + 1;
      return {shapeX[0], shapeW[0], oH, oW};
   }
};

template <typename T>
class ROperator_Conv final : public ROperator {
private:
   ConvAttributes fAttr;
   std::string fNX, fNW, fNB, fNY;
   std::string fNWdev;          // weight tensor the emitted call reads (packed or original)
   std::string fNOut;           // tensor the call writes (the fused pool's output when fused)
   std::vector<size_t> fShapeX, fShapeW, fShapeB, fShapeY, fShapeOut;
   bool fFusedRelu = false;
   int fFusedPool = 0;
   ELayout fLayoutX = ELayout::NCHW, fLayoutY = ELayout::NCHW;
   bool fPacked = false;

public:
   ROperator_Conv() {}
   ROperator_Conv(std::string autopad, std::vector<size_t> dilations, size_t group, std::vector<size_t> kernelShape,
                  std::vector<size_t> pads, std::vector<size_t> strides, std::string nameX, std::string nameW,
                  std::string nameB, std::string nameY)
      : fNX(UTILITY::Clean_name(nameX)), fNW(UTILITY::Clean_name(nameW)), fNB(UTILITY::Clean_name(nameB)),
        fNY(UTILITY::Clean_name(nameY))
   {
      static_assert(std::is_same_v<T, float>, "SOFIE - Conv is generated for float tensors");
      fAttr.autopad = autopad;
      fAttr.dilations = dilations;
      fAttr.group = group;
      fAttr.kernel_shape = kernelShape;
      fAttr.pads = pads;
      fAttr.strides = strides;
      fInputTensorNames = {fNX, fNW};
      if (!fNB.empty()) fInputTensorNames.push_back(fNB);
      fOutputTensorNames = {fNY};
      fNOut = fNY;
   }
   ROperator_Conv(std::string autopad, std::vector<size_t> dilations, size_t group, std::vector<size_t> kernelShape,
                  std::vector<size_t> pads, std::vector<size_t> strides, std::string nameX, std::string nameW,
                  std::string nameY)
      : ROperator_Conv(autopad, dilations, group, kernelShape, pads, strides, nameX, nameW, "", nameY)
   {
   }

   EOpKind Kind() const override { return EOpKind::Conv; }
   bool AcceptsNHWC(const std::string &input) const override { return input == fNX && fAttr.group == 1 && !fAttr.volume; }
   // fusion interface used by the model plan
   const std::string &OutputName() const { return fNOut; }
   void FuseRelu(const std::string &reluOutput)
   {
      fFusedRelu = true;
      fNOut = reluOutput;
      fOutputTensorNames = {fNOut};
   }
   // Folds an inference BatchNormalization that reads this convolution's output into the weights:
   // w'[o] = w[o] * s[o], b'[o] = (b[o] - mean[o]) * s[o] + beta[o], s = gamma * float(1. / sqrt(var + eps)).
   void FoldBatchNorm(RModel &model, const std::string &scale, const std::string &beta, const std::string &mean, const std::string &var,
                      float epsilon, bool relu, const std::string &bnOutput)
   {
      const size_t Cout = fShapeW[0];
      size_t per = 1;
      for (size_t i = 1; i < fShapeW.size(); i++) per *= fShapeW[i];
      const float *w = model.GetInitializedTensor(fNW).template data<float>();
      const float *b = fNB.empty() ? nullptr : model.GetInitializedTensor(fNB).template data<float>();
      const float *g = model.GetInitializedTensor(scale).template data<float>();
      const float *be = model.GetInitializedTensor(beta).template data<float>();
      const float *mu = model.GetInitializedTensor(mean).template data<float>();
      const float *va = model.GetInitializedTensor(var).template data<float>();
      std::shared_ptr<void> wbuf(malloc(Cout * per * sizeof(float)), free), bbuf(malloc(Cout * sizeof(float)), free);
      float *w2 = static_cast<float *>(wbuf.get()), *b2 = static_cast<float *>(bbuf.get());
      for (size_t o = 0; o < Cout; o++) {
         float v = va[o] + epsilon;
         float inv = 1. / std::sqrt((double)v);
         float s = g[o] * inv;
         for (size_t i = 0; i < per; i++) w2[o * per + i] = w[o * per + i] * s;
         b2[o] = ((b ? b[o] : 0.f) - mu[o]) * s + be[o];
      }
      const std::string wname = fNW + "_bn_" + bnOutput, bname = bnOutput + "_bnbias";
      if (!model.IsInitializedTensor(wname)) model.AddInitializedTensor(wname, ETensorType::FLOAT, fShapeW, wbuf);
      if (!model.IsInitializedTensor(bname)) model.AddInitializedTensor(bname, ETensorType::FLOAT, {Cout}, bbuf);
      fNW = wname;
      fNB = bname;
      if (relu) fFusedRelu = true;
      fNOut = bnOutput;
      fOutputTensorNames = {fNOut};
   }
   void FusePool2x2(const std::string &poolOutput)
   {
      fFusedPool = 2;
      fNOut = poolOutput;
      fOutputTensorNames = {fNOut};
   }

   std::vector<ETensorType> TypeInference(std::vector<ETensorType> input) override { return {input[0]}; }
   std::vector<std::vector<size_t>> ShapeInference(std::vector<std::vector<size_t>> input) override
   {
      if (input.size() < 2 || input.size() > 3) throw std::runtime_error("SOFIE Conv Op Shape inference needs 2 or 3 input tensors");
      fAttr.Resolve(input[0], input[1]);
      return {fAttr.OutputShape(input[0], input[1])};
   }

   void Initialize(RModel &model) override
   {
      fUseSession = model.UseSession();
      if (!model.CheckIfTensorAlreadyExist(fNX)) throw std::runtime_error("SOFIE Conv op Input Tensor " + fNX + " is not found in model");
      if (!model.CheckIfTensorAlreadyExist(fNW)) throw std::runtime_error("SOFIE Conv op Input weight Tensor " + fNW + " is not found in model");
      if (!model.IsInitializedTensor(fNW)) throw std::runtime_error("SOFIE Conv op: weights must be a constant tensor");
      fShapeX = model.GetTensorShape(fNX);
      fShapeW = model.GetTensorShape(fNW);
      fShapeY = ShapeInference({fShapeX, fShapeW})[0];
      if (fShapeW[1] * fAttr.group != fShapeX[1]) throw std::runtime_error("SOFIE Conv op: channels of X and W do not match the group count");
      if (!fNB.empty()) {
         if (!model.IsInitializedTensor(fNB)) throw std::runtime_error("SOFIE Conv op Input Tensor " + fNB + " is not found in model");
         fShapeB = model.GetTensorShape(fNB);
         if (ConvertShapeToLength(fShapeB) != fShapeY[1])
            throw std::runtime_error("SOFIE Conv op: Bias Tensor has wrong shape: " + ConvertShapeToString(fShapeB));
      }
      model.AddIntermediateTensor(fNY, model.GetTensorType(fNX), fShapeY);
   }

   void PlanDevice(RModel &model) override
   {
      fLayoutX = model.GetTensorLayout(model.ResolveAlias(fNX));
      fShapeOut = model.GetTensorShape(fNOut);
      fLayoutY = (fAttr.group == 1 && !fAttr.volume && model.CanStayNHWC(fNOut)) ? ELayout::NHWC : ELayout::NCHW;
      if (fAttr.volume && (fLayoutX != ELayout::NCHW || fFusedPool))
         throw std::runtime_error("SOFIE Conv op: a 3-D convolution reads and writes the ONNX layout and fuses no pooling");
      model.SetTensorLayout(fNOut, fLayoutY);
      // NHWC input: weights packed [Cout][kH][kW][Cin], the operand layout of the tensor-core kernel
      fPacked = (fLayoutX == ELayout::NHWC && fAttr.group == 1);
      fNWdev = fNW;
      if (fPacked) {
         const float *src = model.GetInitializedTensor(fNW).data<float>();
         size_t Cout = fShapeW[0], C = fShapeW[1], kH = fShapeW[2], kW = fShapeW[3];
         std::shared_ptr<void> buf(malloc(Cout * C * kH * kW * sizeof(float)), free);
         float *dst = static_cast<float *>(buf.get());
         for (size_t o = 0; o < Cout; o++)
            for (size_t c = 0; c < C; c++)
               for (size_t r = 0; r < kH; r++)
                  for (size_t s = 0; s < kW; s++) dst[((o * kH + r) * kW + s) * C + c] = src[((o * C + c) * kH + r) * kW + s];
         fNWdev = fNW + "_ohwi";
         if (!model.IsInitializedTensor(fNWdev)) model.AddInitializedTensor(fNWdev, ETensorType::FLOAT, {Cout, kH, kW, C}, buf);
      }
      model.UseOnDevice(fNWdev);
      if (!fNB.empty()) model.UseOnDevice(fNB);
   }

   // the samples of a batch are independent: any equal split of the batch axis is a valid launch
   bool CanSliceBatch(size_t parts) const override { return parts > 0 && !fShapeX.empty() && fShapeX[0] % parts == 0 && fShapeX[0] >= parts; }
   std::string GenerateBatchSlice(std::string OpName, size_t parts) override { return GenerateCall(OpName, parts); }
   std::string Generate(std::string OpName) override { return GenerateCall(OpName, 1); }

private:
   // parts == 1: the whole batch; otherwise the launch for slice `part` (a variable of the emitted code)
   std::string GenerateCall(std::string OpName, size_t parts)
   {
      OpName = "op_" + OpName;
      if (fShapeX.empty() || fShapeW.empty() || fShapeY.empty())
         throw std::runtime_error("SOFIE Conv Op called to Generate without being initialized first");
      std::stringstream out;
      out << "\n" << SP << "//----  operator Conv " << OpName << (fFusedRelu ? " + Relu" : "") << (fFusedPool ? " + MaxPool2x2" : "")
          << " -> " << fNOut << " " << ConvertShapeToString(fShapeOut) << (fLayoutY == ELayout::NHWC ? " (NHWC)" : "");
      if (parts > 1) out << ", one of " << parts << " slices of the batch";
      out << "\n";
      out << SP << "{\n";
      std::string x = EMIT::Dev(fNX), y = EMIT::Dev(fNOut);
      if (parts > 1) {
         // the batch axis is outermost in NCHW and in NHWC: a slice is a contiguous range of both tensors
         x += " + (size_t)part * " + std::to_string(ConvertShapeToLength(fShapeX) / parts);
         y += " + (size_t)part * " + std::to_string(ConvertShapeToLength(fShapeOut) / parts);
      }
      if (fAttr.volume) {
         out << SP << SP << "const sofie_conv3d_desc d = {" << fShapeX[0] / parts << ", " << fShapeX[1] << ", " << fShapeX[2] << ", " << fShapeX[3]
             << ", " << fShapeX[4] << ", " << fShapeW[0] << ", " << fAttr.k3[0] << ", " << fAttr.k3[1] << ", " << fAttr.k3[2] << ", "
             << fAttr.pad3[0] << ", " << fAttr.pad3[1] << ", " << fAttr.pad3[2] << ", " << fAttr.s3[0] << ", " << fAttr.s3[1] << ", "
             << fAttr.s3[2] << ", " << fAttr.d3[0] << ", " << fAttr.d3[1] << ", " << fAttr.d3[2] << ", " << fAttr.group << ", "
             << (fFusedRelu ? 1 : 0) << "};\n";
         out << EMIT::Call(SP + SP, "sofie_cuda_conv3d_f32(fStream, &d, " + x + ", " + EMIT::Dev(fNWdev) + ", " +
                                       (fNB.empty() ? std::string("nullptr") : EMIT::Dev(fNB)) + ", " + y + ")");
         out << SP << "}\n";
         return out.str();
      }
      // a 1-D convolution runs as an image of height 1
      const size_t H = fAttr.oneD ? 1 : fShapeX[2], W = fAttr.oneD ? fShapeX[2] : fShapeX[3];
      out << SP << SP << "const sofie_conv2d_desc d = {" << fShapeX[0] / parts << ", " << fShapeX[1] << ", " << H << ", "
          << W << ", " << fShapeW[0] << ", " << fAttr.kH << ", " << fAttr.kW << ", " << fAttr.padH << ", " << fAttr.padW
          << ", " << fAttr.sH << ", " << fAttr.sW << ", " << fAttr.dH << ", " << fAttr.dW << ", " << fAttr.group << ", "
          << (int)fLayoutX << ", " << (int)fLayoutY << ", " << (fPacked ? 1 : 0) << ", " << (fFusedRelu ? 1 : 0) << ", "
          << fFusedPool << "};\n";
      out << EMIT::Call(SP + SP, "sofie_cuda_conv2d_f32(fStream, &d, " + x + ", " + EMIT::Dev(fNWdev) + ", " +
                                    (fNB.empty() ? std::string("nullptr") : EMIT::Dev(fNB)) + ", " + y + ")");
      out << SP << "}\n";
      return out.str();
   }
};

} // namespace SOFIE

#endif
