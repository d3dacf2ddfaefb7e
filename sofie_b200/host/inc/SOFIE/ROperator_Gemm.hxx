// ONNX Gemm and MatMul (MatMul = Gemm with alpha 1, beta 0), optional fused Relu.
//
// Same constructor signatures as the reference (src/SOFIE_core/inc/SOFIE/ROperator_Gemm.hxx:59-67).
// Where the reference emits "copy the pre-broadcast bias into Y; BLAS::sgemm_; Relu loop"
// (ROperator_Gemm.hxx:292-390), this emits one call of sofie_cuda_gemm_f32: bias broadcast and
// Relu happen in the GEMM epilogue and no broadcast copy of the bias exists. A constant B is
// re-laid at generation time as [N,K] (the tensor-core kernel's K-major operand); when A is the
// flattening of an NHWC activation, B's K axis is permuted to that order.
#ifndef SOFIE_ROPERATOR_GEMM
#define SOFIE_ROPERATOR_GEMM

#include <sstream>

#include "SOFIE/Emit.hxx"
#include "SOFIE/RModel.hxx"
#include "SOFIE/ROperator.hxx"

namespace SOFIE {

template <typename T>
class ROperator_Gemm final : public ROperator {
private:
   float fAttrAlpha = 1.0;
   float fAttrBeta = 1.0;
   int_t fAttrTransA = 0;
   int_t fAttrTransB = 0;
   std::string fNA, fNB, fNC, fNY;
   std::string fNBdev, fNCdev; // prepared copies used by the emitted call
   bool fPlainInput = true;     // false when A is the flattening of an NHWC activation (K axis permuted)
   std::vector<ROperator_Gemm<T> *> fChain; // the layers behind this one that its fused call covers
   std::string fNYChain;
   EActivationType fActivation = EActivationType::UNDEFINED;
   std::vector<size_t> fShapeA, fShapeB, fShapeC, fShapeY;
   size_t fM = 0, fN = 0, fK = 0;
   size_t fStack = 1; // matrices in a stacked MatMul (both operands carry the same leading dimensions)
   int fBiasKind = 0;
   int fEmitTransB = 0;

public:
   ROperator_Gemm() {}
   ROperator_Gemm(float alpha, float beta, int_t transA, int_t transB, std::string nameA, std::string nameB,
                  std::string nameY, EActivationType activation = EActivationType::UNDEFINED)
      : fAttrAlpha(alpha), fAttrBeta(beta), fAttrTransA(transA), fAttrTransB(transB), fNA(UTILITY::Clean_name(nameA)),
        fNB(UTILITY::Clean_name(nameB)), fNY(UTILITY::Clean_name(nameY)), fActivation(activation)
   {
      static_assert(std::is_same_v<T, float>, "SOFIE - Gemm is generated for float tensors");
      fInputTensorNames = {fNA, fNB};
      fOutputTensorNames = {fNY};
   }
   ROperator_Gemm(float alpha, float beta, int_t transA, int_t transB, std::string nameA, std::string nameB,
                  std::string nameC, std::string nameY, EActivationType activation = EActivationType::UNDEFINED)
      : fAttrAlpha(alpha), fAttrBeta(beta), fAttrTransA(transA), fAttrTransB(transB), fNA(UTILITY::Clean_name(nameA)),
        fNB(UTILITY::Clean_name(nameB)), fNC(UTILITY::Clean_name(nameC)), fNY(UTILITY::Clean_name(nameY)),
        fActivation(activation)
   {
      static_assert(std::is_same_v<T, float>, "SOFIE - Gemm is generated for float tensors");
      fInputTensorNames = {fNA, fNB, fNC};
      fOutputTensorNames = {fNY};
   }

   EOpKind Kind() const override { return EOpKind::Gemm; }
   bool AcceptsNHWC(const std::string &input) const override { return input == fNA && !fAttrTransA; }
   // ---- fused chain of small layers (sofie_cuda_mlp_f32): the head of a chain emits one call for all its layers ----
   const std::string &InputName() const { return fNA; }
   size_t WidthIn() const { return fK; }
   size_t WidthOut() const { return fN; }
   size_t Rows() const { return fM; }
   // Largest batch for the fused kernel: fp32 FMA out of shared memory beats one tensor-core GEMM launch per
   // layer only while those launches are latency bound (measured cross-over between 2048 and 4096 rows).
   static constexpr size_t kMlpFusedMaxRows = 2048;
   // valid after PlanDevice: a plain x W^T (+ b) (+ Relu) with constant weights on a row-major input
   bool MlpFusable() const
   {
      return fPlainInput && fNBdev != fNB && fAttrAlpha == 1.f && !fAttrTransA && (fBiasKind == 0 || (fBiasKind == 1 && fAttrBeta == 1.f)) &&
             fK <= 256 && fN <= 256 && fM <= kMlpFusedMaxRows && fShapeA.size() == 2 && fStack == 1;
   }
   void AbsorbChain(const std::vector<ROperator_Gemm<T> *> &tail)
   {
      fChain = tail;
      fNYChain = tail.back()->fNY;
      fOutputTensorNames = {fNYChain};
   }
   void SetActivation(EActivationType a) { fActivation = a; }
   void SetOutputName(const std::string &y) { fNY = y; fOutputTensorNames = {fNY}; }
   const std::string &OutputName() const { return fNY; }

   std::vector<ETensorType> TypeInference(std::vector<ETensorType> input) override { return {input[0]}; }

   std::vector<std::vector<size_t>> ShapeInference(std::vector<std::vector<size_t>> input) override
   {
      if (input.size() < 2 || input.size() > 3) throw std::runtime_error("SOFIE Gemm Op Shape Inference needs 2 or 3 input tensors");
      auto a = input[0], b = input[1];
      if (a.size() < 2 || b.size() < 2) throw std::runtime_error("SOFIE Gemm Op: A and B must have at least 2 dimensions");
      // B with leading dimensions of extent 1 only is a plain matrix
      while (b.size() > 2 && b[0] == 1) b.erase(b.begin());
      fStack = 1;
      if (b.size() > 2) {
         // a stack of matrices on both sides (ONNX MatMul): the leading dimensions must agree; product s multiplies
         // matrix s of A with matrix s of B
         if (a.size() != b.size() || !std::equal(a.begin(), a.end() - 2, b.begin()))
            throw std::runtime_error("SOFIE Gemm Op: stacked operands " + ConvertShapeToString(input[0]) + " and " + ConvertShapeToString(input[1]) +
                                     " need the same leading dimensions");
         if (fAttrTransA || fAttrTransB) throw std::runtime_error("SOFIE Gemm Op: transposed stacked operands are not supported");
         for (size_t i = 0; i + 2 < a.size(); i++) fStack *= a[i];
      }
      // leading dimensions of A fold into the row count when B is one matrix
      size_t rows = 1;
      if (fStack == 1)
         for (size_t i = 0; i + 2 < a.size(); i++) rows *= a[i];
      size_t am = a[a.size() - 2], ak = a[a.size() - 1];
      if (fAttrTransA) {
         if (a.size() != 2) throw std::runtime_error("SOFIE Gemm Op: transA with a stacked A is not supported");
         std::swap(am, ak);
      }
      size_t bk = fAttrTransB ? b[b.size() - 1] : b[b.size() - 2], bn = fAttrTransB ? b[b.size() - 2] : b[b.size() - 1];
      if (ak != bk) throw std::runtime_error("SOFIE Gemm Op: inner dimensions differ: " + std::to_string(ak) + " vs " + std::to_string(bk));
      std::vector<size_t> y(a.begin(), a.end() - 2);
      y.push_back(am);
      y.push_back(bn);
      fM = rows * am;
      fK = ak;
      fN = bn;
      return {y};
   }

   void Initialize(RModel &model) override
   {
      if (!model.CheckIfTensorAlreadyExist(fNA) || !model.CheckIfTensorAlreadyExist(fNB))
         throw std::runtime_error("SOFIE Gemm Op Input Tensor " + fNA + " or " + fNB + " is not found in model");
      if (!fNC.empty() && !model.CheckIfTensorAlreadyExist(fNC))
         throw std::runtime_error("SOFIE Gemm Op Input Tensor " + fNC + " is not found in model");
      fShapeA = model.GetTensorShape(fNA);
      if (fShapeA.size() == 1) fShapeA.insert(fShapeA.begin(), 1);
      fShapeB = model.GetTensorShape(fNB);
      if (fShapeB.size() == 1) fShapeB.push_back(1);
      fShapeY = ShapeInference({fShapeA, fShapeB})[0];
      if (fStack > 1 && !fNC.empty() && model.GetTensorShape(fNC).size() > 1 && ConvertShapeToLength(model.GetTensorShape(fNC)) != fN)
         throw std::runtime_error("SOFIE Gemm Op: a stacked product takes a bias per column only");
      if (!fNC.empty()) {
         if (!model.IsInitializedTensor(fNC)) throw std::runtime_error("SOFIE Gemm Op: bias " + fNC + " must be a constant tensor");
         fShapeC = model.GetTensorShape(fNC);
      } else if (fAttrBeta != 0 && false) {
         throw std::runtime_error("SOFIE Gemm Op: bias tensor is not present but beta is not zero");
      }
      model.AddIntermediateTensor(fNY, model.GetTensorType(fNA), fShapeY);
      if (model.Verbose()) std::cout << "Gemm (or MatMul)  ---> " << fNY << " shape " << ConvertShapeToString(fShapeY) << std::endl;
   }

   void PlanDevice(RModel &model) override
   {
      // ---- B: constant weights are stored [N,K]; activations are passed as they are ----
      fNBdev = fNB;
      fEmitTransB = (int)fAttrTransB;
      if (model.IsInitializedTensor(fNB)) {
         const auto &w = model.GetInitializedTensor(fNB);
         const float *src = w.data<float>();
         std::shared_ptr<void> buf(malloc(fStack * fN * fK * sizeof(float) + 1), free);
         float *dst = static_cast<float *>(buf.get());
         // K axis order of A on the device: (h,w,c) when A is the flattening of an NHWC activation
         std::vector<size_t> kperm(fK);
         for (size_t k = 0; k < fK; k++) kperm[k] = k;
         std::string owner = model.ResolveAlias(fNA);
         if (model.GetTensorLayout(owner) == ELayout::NHWC) {
            fPlainInput = false;
            auto s4 = model.GetTensorShape(owner); // logical N,C,H,W
            if (s4.size() != 4 || s4[1] * s4[2] * s4[3] != fK)
               throw std::runtime_error("SOFIE Gemm Op: NHWC input " + fNA + " does not flatten to K");
            size_t C = s4[1], H = s4[2], W = s4[3];
            for (size_t h = 0; h < H; h++)
               for (size_t x = 0; x < W; x++)
                  for (size_t c = 0; c < C; c++) kperm[(h * W + x) * C + c] = (c * H + h) * W + x;
         }
         for (size_t st = 0; st < fStack; st++)
            for (size_t n = 0; n < fN; n++)
               for (size_t k = 0; k < fK; k++) {
                  size_t ks = kperm[k];
                  dst[(st * fN + n) * fK + k] = fAttrTransB ? src[(st * fN + n) * fK + ks] : src[(st * fK + ks) * fN + n];
               }
         fNBdev = fNB + "_nk_" + fNY;
         model.AddInitializedTensor(fNBdev, ETensorType::FLOAT, {fStack * fN, fK}, buf);
         model.UseOnDevice(fNBdev);
         fEmitTransB = 1;
      } else if (model.GetTensorLayout(model.ResolveAlias(fNA)) == ELayout::NHWC) {
         throw std::runtime_error("SOFIE Gemm Op: NHWC activation times a non-constant B is not supported");
      }
      // ---- C: [N] or [1,N] broadcasts over rows in the epilogue, [M,N] is added elementwise,
      //         any other unidirectional broadcast is expanded to [N] or [M,N] here ----
      fBiasKind = 0;
      if (!fNC.empty()) {
         const auto &c = model.GetInitializedTensor(fNC);
         size_t len = c.length();
         fNCdev = fNC;
         if (len == fN && (fShapeC.size() == 1 || fShapeC.back() == fN)) {
            fBiasKind = 1;
         } else if (len == fM * fN) {
            fBiasKind = 2;
         } else if (len == 1) {
            std::shared_ptr<void> buf(malloc(fN * sizeof(float)), free);
            for (size_t n = 0; n < fN; n++) static_cast<float *>(buf.get())[n] = c.data<float>()[0];
            fNCdev = fNC + "_bcast_" + fNY;
            model.AddInitializedTensor(fNCdev, ETensorType::FLOAT, {fN}, buf);
            fBiasKind = 1;
         } else if (len == fM && fShapeC.size() == 2 && fShapeC[1] == 1) {
            std::shared_ptr<void> buf(malloc(fM * fN * sizeof(float)), free);
            for (size_t m = 0; m < fM; m++)
               for (size_t n = 0; n < fN; n++) static_cast<float *>(buf.get())[m * fN + n] = c.data<float>()[m];
            fNCdev = fNC + "_bcast_" + fNY;
            model.AddInitializedTensor(fNCdev, ETensorType::FLOAT, {fM, fN}, buf);
            fBiasKind = 2;
         } else {
            throw std::runtime_error("SOFIE Gemm Op: bias of shape " + ConvertShapeToString(fShapeC) + " does not broadcast to " +
                                     ConvertShapeToString(fShapeY));
         }
         model.UseOnDevice(fNCdev);
      }
   }

   // rows of A are independent: any equal split of the rows is a valid launch (not for a transposed A, a stack of products
   // or a bias with one value per row)
   bool CanSliceBatch(size_t parts) const override { return parts > 0 && fStack <= 1 && !fAttrTransA && fBiasKind != 2 && fM > 0 && fM % parts == 0; }
   std::string GenerateBatchSlice(std::string OpName, size_t parts) override { return GenerateCall(OpName, parts); }
   std::string Generate(std::string OpName) override { return GenerateCall(OpName, 1); }

private:
   std::string GenerateCall(std::string opName, size_t parts)
   {
      opName = "op_" + opName;
      const size_t M = fM / parts;
      if (fShapeA.empty() || fShapeB.empty() || fShapeY.empty())
         throw std::runtime_error("SOFIE Gemm Op called to Generate without being initialized first");
      std::stringstream out;
      if (!fChain.empty()) {
         // one launch for the whole chain: widths, Relu flags and the device pointers of every layer
         std::vector<const ROperator_Gemm<T> *> layers{this};
         layers.insert(layers.end(), fChain.begin(), fChain.end());
         out << "\n" << SP << "//--------- fused MLP " << opName << ": " << layers.size() << " Gemm layers, [" << M << "," << fK << "] -> ["
             << M << "," << layers.back()->fN << "]" << (parts > 1 ? ", one slice of the rows" : "") << "\n";
         out << SP << "{\n";
         std::string dims = std::to_string(fK), relu, nk, w, b;
         for (size_t l = 0; l < layers.size(); l++) {
            dims += ", " + std::to_string(layers[l]->fN);
            relu += (l ? ", " : "") + std::string(layers[l]->fActivation == EActivationType::RELU ? "1" : "0");
            nk += (l ? ", " : "") + std::string("1");
            w += (l ? ", " : "") + EMIT::Dev(layers[l]->fNBdev);
            b += (l ? ", " : "") + (layers[l]->fBiasKind ? EMIT::Dev(layers[l]->fNCdev) : std::string("nullptr"));
         }
         out << SP << SP << "const sofie_mlp_desc d = {" << M << ", " << layers.size() << ", {" << dims << "}, {" << relu << "}, {" << nk << "}};\n";
         out << SP << SP << "const float * const w[] = {" << w << "};\n";
         out << SP << SP << "const float * const b[] = {" << b << "};\n";
         out << EMIT::Call(SP + SP, "sofie_cuda_mlp_f32(fStream, &d, " + EMIT::DevSlice(fNA, fM * fK, parts) + ", w, b, " +
                                       EMIT::DevSlice(fNYChain, fM * layers.back()->fN, parts) + ")");
         out << SP << "}\n";
         return out.str();
      }
      if (fStack > 1) {
         out << "\n" << SP << "//--------- stacked MatMul " << opName << ": " << fStack << " x ([" << fM << "," << fK << "] x [" << fK << "," << fN << "])\n";
         out << SP << "{\n";
         out << SP << SP << "const sofie_gemm_f32_desc d = {" << fM << ", " << fN << ", " << fK << ", 0, " << fEmitTransB << ", "
             << EMIT::FloatLit(fAttrAlpha) << ", " << EMIT::FloatLit(fBiasKind ? fAttrBeta : 0.f) << ", " << fBiasKind << ", "
             << (fActivation == EActivationType::RELU ? 1 : 0) << "};\n";
         out << EMIT::Call(SP + SP, "sofie_cuda_gemm_f32_batched(fStream, &d, " + EMIT::Dev(fNA) + ", " + EMIT::Dev(fNBdev) + ", " +
                                       (fBiasKind ? EMIT::Dev(fNCdev) : std::string("nullptr")) + ", " + EMIT::Dev(fNY) + ", " +
                                       std::to_string(fStack) + ", " + std::to_string(fM * fK) + ", " + std::to_string(fN * fK) + ", " +
                                       std::to_string(fM * fN) + ")");
         out << SP << "}\n";
         return out.str();
      }
      out << "\n" << SP << "//--------- Gemm " << opName << ": [" << M << "," << fK << "] x [" << fK << "," << fN << "]"
          << (parts > 1 ? ", one slice of the rows" : "") << "\n";
      out << SP << "{\n";
      out << SP << SP << "const sofie_gemm_f32_desc d = {" << M << ", " << fN << ", " << fK << ", " << fAttrTransA << ", "
          << fEmitTransB << ", " << EMIT::FloatLit(fAttrAlpha) << ", " << EMIT::FloatLit(fBiasKind ? fAttrBeta : 0.f) << ", "
          << fBiasKind << ", " << (fActivation == EActivationType::RELU ? 1 : 0) << "};\n";
      out << EMIT::Call(SP + SP, "sofie_cuda_gemm_f32(fStream, &d, " + EMIT::DevSlice(fNA, fM * fK, parts) + ", " + EMIT::Dev(fNBdev) + ", " +
                                    (fBiasKind ? EMIT::Dev(fNCdev) : std::string("nullptr")) + ", " + EMIT::DevSlice(fNY, fM * fN, parts) + ")");
      out << SP << "}\n";
      return out.str();
   }

public:
   std::vector<std::string> GetBlasRoutines() override { return {}; }
};

} // namespace SOFIE

#endif
