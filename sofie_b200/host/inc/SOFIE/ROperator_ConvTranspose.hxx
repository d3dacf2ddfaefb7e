// ONNX ConvTranspose, 1-D and 2-D, group 1.
//
// Constructor signature and attribute rules as in the reference
// (src/SOFIE_core/inc/SOFIE/ROperator_ConvTranspose.hxx:73-93, ROperator_ConvTranspose.icc:15-106):
// pads default to 0, output extent stride*(i-1) + dilated kernel + output_padding - pads (:83-90),
// an explicit output_shape and auto_pad other than NOTSET are refused (:53-80, :92-96), asymmetric
// pads are averaged (:332-356). The reference emits a filter-matrix copy, a per-image sgemm_,
// UTILITY::col2im and a saxpy_ of the broadcast bias (:364-474) and registers `_f` / `_xcol` scratch
// tensors; this emits ONE call of sofie_cuda_conv_transpose2d_f32 and no scratch. The reference's
// group > 1 branch reuses the whole filter matrix for every group and its 3-D branch throws
// (:411-430): both are refused here.
#ifndef SOFIE_ROPERATOR_CONVTRANSPOSE
#define SOFIE_ROPERATOR_CONVTRANSPOSE

#include <sstream>

#include "SOFIE/Emit.hxx"
#include "SOFIE/RModel.hxx"
#include "SOFIE/ROperator.hxx"
#include "sofie_cuda.h" // sofie_conv_transpose2d_gemm_scratch_bytes: host arithmetic only

namespace SOFIE {

template <typename T>
class ROperator_ConvTranspose final : public ROperator {
private:
   std::string fAttrAutopad;
   std::vector<size_t> fAttrDilations;
   size_t fAttrGroup;
   std::vector<size_t> fAttrKernelShape, fAttrOutputPadding, fAttrOutputShape, fAttrPads, fAttrStrides;
   std::string fNX, fNW, fNB, fNY;
   std::string fNProducts;   // arena slice of the product form (channel-last input, re-ordered filters, products), when it is used
   size_t fProductsBytes = 0;
   std::vector<size_t> fShapeX, fShapeW, fShapeB, fShapeY;
   size_t fDim = 0;
   // resolved 2-D values (a 1-D operator is the 2-D one with height 1)
   size_t fH = 1, fW = 1, fKH = 1, fKW = 1, fPadH = 0, fPadW = 0, fSH = 1, fSW = 1, fDH = 1, fDW = 1, fOPH = 0, fOPW = 0;

public:
   ROperator_ConvTranspose() {}
   ROperator_ConvTranspose(std::string autopad, std::vector<size_t> dilations, size_t group, std::vector<size_t> kernelShape,
                           std::vector<size_t> outputPadding, std::vector<size_t> outputShape, std::vector<size_t> pads,
                           std::vector<size_t> strides, std::string nameX, std::string nameW, std::string nameB, std::string nameY)
      : fAttrAutopad(autopad), fAttrDilations(dilations), fAttrGroup(group), fAttrKernelShape(kernelShape),
        fAttrOutputPadding(outputPadding), fAttrOutputShape(outputShape), fAttrPads(pads), fAttrStrides(strides),
        fNX(UTILITY::Clean_name(nameX)), fNW(UTILITY::Clean_name(nameW)), fNB(UTILITY::Clean_name(nameB)),
        fNY(UTILITY::Clean_name(nameY))
   {
      static_assert(std::is_same_v<T, float>, "SOFIE - ConvTranspose is generated for float tensors");
      fInputTensorNames = {fNX, fNW};
      if (!fNB.empty()) fInputTensorNames.push_back(fNB);
      fOutputTensorNames = {fNY};
   }

   EOpKind Kind() const override { return EOpKind::Other; }
   std::vector<ETensorType> TypeInference(std::vector<ETensorType> input) override { return {input[0]}; }
   std::vector<std::vector<size_t>> ShapeInference(std::vector<std::vector<size_t>> input) override
   {
      if (input.size() < 2) throw std::runtime_error("SOFIE ConvTranspose Op Shape inference needs 2 or 3 input tensors");
      const auto &x = input[0], &w = input[1];
      if (x.size() != w.size() || x.size() < 3 || x.size() > 4)
         throw std::runtime_error("SOFIE ConvTranspose Op: only 1-D and 2-D transposed convolutions are generated for the CUDA path");
      fDim = x.size() - 2;
      if (fAttrGroup == 0) fAttrGroup = 1;
      if (fAttrGroup != 1) throw std::runtime_error("SOFIE ConvTranspose Op: group > 1 is not supported");
      if (fAttrStrides.empty()) fAttrStrides.assign(fDim, 1);
      if (fAttrDilations.empty()) fAttrDilations.assign(fDim, 1);
      if (fAttrOutputPadding.empty()) fAttrOutputPadding.assign(fDim, 0);
      if (!fAttrOutputShape.empty()) throw std::runtime_error("ConvTranspose with output_shape explicitly set not yet supported.");
      if (fAttrPads.empty()) {
         if (fAttrAutopad != "NOTSET") throw std::runtime_error("ConvTranspose with padding SAME_UPPER or SAME_LOWER not supported");
         fAttrPads.assign(2 * fDim, 0);
      }
      if (fAttrStrides.size() != fDim || fAttrDilations.size() != fDim || fAttrOutputPadding.size() != fDim || fAttrPads.size() != 2 * fDim)
         throw std::runtime_error("SOFIE ConvTranspose Op: attribute lengths do not match the number of spatial axes");
      if (!fAttrKernelShape.empty())
         for (size_t i = 0; i < fDim; i++)
            if (fAttrKernelShape[i] != w[i + 2]) throw std::runtime_error("SOFIE ConvTranspose Op: kernel_shape differs from the weight tensor");
      if (w[0] != x[1]) throw std::runtime_error("SOFIE ConvTranspose Op: channels of X and W do not match");
      std::vector<size_t> out = {x[0], w[1] * fAttrGroup};
      for (size_t i = 0; i < fDim; i++) {
         const long o = (long)(fAttrStrides[i] * (x[i + 2] - 1) + fAttrDilations[i] * (w[i + 2] - 1) + 1 + fAttrOutputPadding[i]) -
                        (long)(fAttrPads[i] + fAttrPads[fDim + i]);
         if (o <= 0) throw std::runtime_error("SOFIE ConvTranspose Op: the pads leave no output");
         out.push_back((size_t)o);
      }
      return {out};
   }

   void Initialize(RModel &model) override
   {
      fUseSession = model.UseSession();
      if (!model.CheckIfTensorAlreadyExist(fNX))
         throw std::runtime_error("SOFIE Conv Transpose op Input Tensor " + fNX + " is not found in model");
      if (!model.CheckIfTensorAlreadyExist(fNW))
         throw std::runtime_error("SOFIE Conv Transpose op Input weight Tensor " + fNW + " is not found in model");
      if (!model.IsInitializedTensor(fNW)) throw std::runtime_error("SOFIE Conv Transpose op: weights must be a constant tensor");
      fShapeX = model.GetTensorShape(fNX);
      fShapeW = model.GetTensorShape(fNW);
      fShapeY = ShapeInference({fShapeX, fShapeW})[0];
      if (!fNB.empty()) {
         if (!model.IsInitializedTensor(fNB)) throw std::runtime_error("SOFIE ConvTrans op Input Tensor " + fNB + " is not found in model");
         fShapeB = model.GetTensorShape(fNB);
         if (ConvertShapeToLength(fShapeB) != fShapeY[1])
            throw std::runtime_error("SOFIE ConvTrans op: Bias Tensor has wrong shape: " + ConvertShapeToString(fShapeB));
      }
      // the last axis is the width; a 1-D operator has height 1
      const size_t a = fDim - 1;
      fW = fShapeX[2 + a], fKW = fShapeW[2 + a], fSW = fAttrStrides[a], fDW = fAttrDilations[a], fOPW = fAttrOutputPadding[a];
      fPadW = (fAttrPads[a] == fAttrPads[fDim + a]) ? fAttrPads[a] : (fAttrPads[a] + fAttrPads[fDim + a]) / 2;
      if (fDim == 2) {
         fH = fShapeX[2], fKH = fShapeW[2], fSH = fAttrStrides[0], fDH = fAttrDilations[0], fOPH = fAttrOutputPadding[0];
         fPadH = (fAttrPads[0] == fAttrPads[2]) ? fAttrPads[0] : (fAttrPads[0] + fAttrPads[2]) / 2;
      }
      model.AddIntermediateTensor(fNY, model.GetTensorType(fNX), fShapeY);
   }

   sofie_conv_transpose2d_desc Desc() const
   {
      sofie_conv_transpose2d_desc d = {};
      d.N = (int32_t)fShapeX[0], d.C = (int32_t)fShapeX[1], d.H = (int32_t)fH, d.W = (int32_t)fW, d.Cout = (int32_t)fShapeW[1];
      d.kH = (int32_t)fKH, d.kW = (int32_t)fKW, d.pad_h = (int32_t)fPadH, d.pad_w = (int32_t)fPadW, d.stride_h = (int32_t)fSH,
      d.stride_w = (int32_t)fSW, d.dil_h = (int32_t)fDH, d.dil_w = (int32_t)fDW, d.out_pad_h = (int32_t)fOPH, d.out_pad_w = (int32_t)fOPW;
      return d;
   }

   void PlanDevice(RModel &model) override
   {
      model.SetTensorLayout(fNY, ELayout::NCHW);
      model.UseOnDevice(fNW);
      if (!fNB.empty()) model.UseOnDevice(fNB);
      // With 16 or more input channels the operator is lowered as the reference lowers it -- a filter GEMM, here one for
      // all images and on the tensor cores, followed by the gather form of col2im -- and needs a slice of the arena for
      // the products (alive during this operator only). Not with a run-time batch: part of the slice (the re-ordered
      // filters) does not scale with the batch.
      const sofie_conv_transpose2d_desc d = Desc();
      fProductsBytes = model.RunTimeBatch() ? 0 : sofie_conv_transpose2d_gemm_scratch_bytes(&d);
      if (fProductsBytes) {
         fNProducts = fNY + "_products";
         model.AddIntermediateTensor(fNProducts, ETensorType::FLOAT, std::vector<size_t>{fProductsBytes / sizeof(float)});
         fOutputTensorNames = {fNY, fNProducts};
      }
   }

   std::string Generate(std::string OpName) override
   {
      OpName = "op_" + OpName;
      if (fShapeX.empty() || fShapeW.empty() || fShapeY.empty())
         throw std::runtime_error("SOFIE Conv Op called to Generate without being initialized first");
      std::stringstream out;
      out << "\n" << SP << "//----  operator ConvTranspose " << OpName << " -> " << fNY << " " << ConvertShapeToString(fShapeY) << "\n";
      out << SP << "{\n";
      out << SP << SP << "const sofie_conv_transpose2d_desc d = {" << fShapeX[0] << ", " << fShapeX[1] << ", " << fH << ", " << fW << ", "
          << fShapeW[1] << ", " << fKH << ", " << fKW << ", " << fPadH << ", " << fPadW << ", " << fSH << ", " << fSW << ", " << fDH << ", "
          << fDW << ", " << fOPH << ", " << fOPW << ", 0};\n";
      const std::string args = EMIT::Dev(fNX) + ", " + EMIT::Dev(fNW) + ", " + (fNB.empty() ? std::string("nullptr") : EMIT::Dev(fNB)) + ", " +
                               EMIT::Dev(fNY);
      if (fProductsBytes)
         out << EMIT::Call(SP + SP, "sofie_cuda_conv_transpose2d_f32_gemm(fStream, &d, " + args + ", " + EMIT::Dev(fNProducts) + ", " +
                                       std::to_string(fProductsBytes) + ")");
      else
         out << EMIT::Call(SP + SP, "sofie_cuda_conv_transpose2d_f32(fStream, &d, " + args + ")");
      out << SP << "}\n";
      return out.str();
   }
};

} // namespace SOFIE

#endif
