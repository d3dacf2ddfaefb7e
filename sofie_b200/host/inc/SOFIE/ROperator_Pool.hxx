// ONNX MaxPool / AveragePool / GlobalAveragePool, 1-D, 2-D and 3-D.
// Constructor and attribute struct as in the reference (src/SOFIE_core/inc/SOFIE/ROperator_Pool.hxx:17-83).
// The reference emits scalar nested loops (:266-476); this emits one call of sofie_cuda_pool2d_f32
// (or sofie_cuda_maxpool2d_u8 on a quantised tensor), unless the model plan folded a 2x2 stride-2
// MaxPool into the preceding convolution. `pads` follow ONNX (h_begin, w_begin, h_end, w_end), the
// reading of the reference's shape inference (:172-189). A 3-D pooling of [N, C, D, H, W] (reference: fDim == 3)
// emits one call of sofie_cuda_pool3d_f32.
#ifndef SOFIE_ROPERATOR_POOL
#define SOFIE_ROPERATOR_POOL

#include <sstream>

#include "SOFIE/Emit.hxx"
#include "SOFIE/RModel.hxx"
#include "SOFIE/ROperator.hxx"

namespace SOFIE {

struct RAttributes_Pool {
   std::string auto_pad = "NOTSET";
   int ceil_mode = 0;
   int count_include_pad = 0;
   int storage_order = 0;
   std::vector<size_t> dilations;
   std::vector<size_t> kernel_shape;
   std::vector<size_t> pads;
   std::vector<size_t> strides;
};

enum PoolOpMode { InvalidPool, MaxPool, AveragePool, GlobalAveragePool };

template <typename T>
class ROperator_Pool final : public ROperator {
private:
   PoolOpMode fPoolMode = InvalidPool;
   RAttributes_Pool fAttr;
   std::string fNX, fNY;
   std::vector<size_t> fShapeX, fShapeY;
   std::vector<size_t> fShape4; // the input viewed as [N, C, H, W] (H = 1 for a 1-D pooling)
   size_t fKH = 0, fKW = 0, fSH = 1, fSW = 1;
   std::vector<size_t> fPads;
   bool fVolume = false;        // rank-5 input: 3-D pooling
   std::vector<size_t> fK3, fS3, fP3; // its window, strides and six pads
   ELayout fLayout = ELayout::NCHW;
   ETensorType fType = ETensorType::FLOAT;

public:
   ROperator_Pool() {}
   ROperator_Pool(PoolOpMode mode, RAttributes_Pool attr, std::string nameX, std::string nameY)
      : fPoolMode(mode), fAttr(attr), fNX(UTILITY::Clean_name(nameX)), fNY(UTILITY::Clean_name(nameY))
   {
      fInputTensorNames = {fNX};
      fOutputTensorNames = {fNY};
   }
   std::string Name() const
   {
      if (fPoolMode == AveragePool) return "AveragePool";
      if (fPoolMode == MaxPool) return "MaxPool";
      return "Invalid";
   }
   EOpKind Kind() const override { return EOpKind::Pool; }
   bool AcceptsNHWC(const std::string &) const override { return !fVolume; }
   const std::string &InputName() const { return fNX; }
   const std::string &OutputName() const { return fNY; }
   // 2x2 window, stride 2, no padding: the form a convolution epilogue can absorb
   bool IsMax2x2Stride2() const
   {
      return !fVolume && fPoolMode == MaxPool && fKH == 2 && fKW == 2 && fSH == 2 && fSW == 2 && fPads[0] + fPads[1] + fPads[2] + fPads[3] == 0;
   }

   std::vector<ETensorType> TypeInference(std::vector<ETensorType> input) override { return input; }
   std::vector<std::vector<size_t>> ShapeInference(std::vector<std::vector<size_t>> input) override
   {
      if (input.size() == 1 && input[0].size() == 5) return {ShapeInference3d(input[0])};
      if (input.size() != 1 || (input[0].size() != 4 && input[0].size() != 3))
         throw std::runtime_error("SOFIE " + Name() + " Op: pooling is generated for rank-3, rank-4 and rank-5 tensors");
      // a 1-D pooling of [N, C, W] is the 2-D one of [N, C, 1, W] with a window of height 1
      const bool oneD = input[0].size() == 3;
      std::vector<size_t> x = input[0];
      if (oneD) x.insert(x.begin() + 2, 1);
      auto lift = [&](std::vector<size_t> v, size_t fill) {
         if (oneD && v.size() == 1) v.insert(v.begin(), fill);
         return v;
      };
      std::vector<size_t> kernel = lift(fAttr.kernel_shape, 1), strides = lift(fAttr.strides, 1), pads = fAttr.pads;
      if (oneD && pads.size() == 2) pads = {0, pads[0], 0, pads[1]};
      fKH = kernel.empty() ? x[2] : kernel[0];
      fKW = kernel.size() < 2 ? (kernel.empty() ? x[3] : fKH) : kernel[1];
      fSH = strides.empty() ? 1 : strides[0];
      fSW = strides.size() < 2 ? fSH : strides[1];
      if (fAttr.auto_pad == "NOTSET") {
         fPads = pads.empty() ? std::vector<size_t>{0, 0, 0, 0} : pads;
      } else if (fAttr.auto_pad == "SAME_UPPER" || fAttr.auto_pad == "SAME_LOWER") {
         fPads = {fKH / 2, fKW / 2, fKH / 2, fKW / 2};
         if (fKH % 2 == 1) (fAttr.auto_pad == "SAME_UPPER") ? fPads[0]++ : fPads[2]++;
         if (fKW % 2 == 1) (fAttr.auto_pad == "SAME_UPPER") ? fPads[1]++ : fPads[3]++;
      } else if (fAttr.auto_pad == "VALID") {
         fPads = {0, 0, 0, 0};
      } else {
         throw std::runtime_error("SOFIE " + Name() + " Op invalid auto_pad value : " + fAttr.auto_pad);
      }
      if (fPads.size() != 4) throw std::runtime_error("SOFIE " + Name() + " Op: pads must have 4 values");
      fShape4 = x;
      size_t oH = (x[2] + fPads[0] + fPads[2] - fKH) / fSH + 1;
      size_t oW = (x[3] + fPads[1] + fPads[3] - fKW) / fSW + 1;
      if (oneD) return {{x[0], x[1], oW}};
      return {{x[0], x[1], oH, oW}};
   }

   // [N, C, D, H, W]: window, strides and pads per axis, output extent as the reference's shape inference (:172-197)
   std::vector<size_t> ShapeInference3d(const std::vector<size_t> &x)
   {
      fVolume = true;
      fK3 = fAttr.kernel_shape.empty() ? std::vector<size_t>{x[2], x[3], x[4]} : fAttr.kernel_shape;
      fS3 = fAttr.strides.empty() ? std::vector<size_t>{1, 1, 1} : fAttr.strides;
      if (fK3.size() != 3 || fS3.size() != 3) throw std::runtime_error("SOFIE " + Name() + " Op: a 3-D pooling needs 3 kernel and stride values");
      if (fAttr.auto_pad == "NOTSET") {
         fP3 = fAttr.pads.empty() ? std::vector<size_t>(6, 0) : fAttr.pads;
      } else if (fAttr.auto_pad == "SAME_UPPER" || fAttr.auto_pad == "SAME_LOWER") {
         fP3 = {fK3[0] / 2, fK3[1] / 2, fK3[2] / 2, fK3[0] / 2, fK3[1] / 2, fK3[2] / 2};
         for (size_t a = 0; a < 3; a++)
            if (fK3[a] % 2 == 1) (fAttr.auto_pad == "SAME_UPPER") ? fP3[a]++ : fP3[a + 3]++;
      } else if (fAttr.auto_pad == "VALID") {
         fP3 = std::vector<size_t>(6, 0);
      } else {
         throw std::runtime_error("SOFIE " + Name() + " Op invalid auto_pad value : " + fAttr.auto_pad);
      }
      if (fP3.size() != 6) throw std::runtime_error("SOFIE " + Name() + " Op: pads of a 3-D pooling must have 6 values");
      fPads = {0, 0, 0, 0};
      std::vector<size_t> y = {x[0], x[1]};
      for (size_t a = 0; a < 3; a++) y.push_back((x[2 + a] + fP3[a] + fP3[a + 3] - fK3[a]) / fS3[a] + 1);
      return y;
   }

   void Initialize(RModel &model) override
   {
      fUseSession = model.UseSession();
      if (!model.CheckIfTensorAlreadyExist(fNX)) throw std::runtime_error("SOFIE Pool op Input Tensor " + fNX + " is not found in model");
      fShapeX = model.GetTensorShape(fNX);
      if (fPoolMode == GlobalAveragePool) {
         fPoolMode = AveragePool;
         fAttr.kernel_shape.assign(fShapeX.begin() + 2, fShapeX.end());
         fAttr.auto_pad = "VALID";
         fAttr.pads.assign(2 * (fShapeX.size() - 2), 0);
         fAttr.strides.assign(fShapeX.size() - 2, 1);
      }
      fShapeY = ShapeInference({fShapeX})[0];
      fType = model.GetTensorType(fNX);
      model.AddIntermediateTensor(fNY, fType, fShapeY);
   }
   void PlanDevice(RModel &model) override
   {
      fLayout = model.GetTensorLayout(model.ResolveAlias(fNX));
      model.SetTensorLayout(fNY, fLayout);
      if (fVolume && (fType != ETensorType::FLOAT || fLayout != ELayout::NCHW))
         throw std::runtime_error("SOFIE Pool op: 3-D pooling is generated for float tensors in the ONNX layout");
      if (fType == ETensorType::UINT8 && (fPoolMode != MaxPool || fPads[0] + fPads[1] + fPads[2] + fPads[3] != 0))
         throw std::runtime_error("SOFIE Pool op: only un-padded MaxPool is generated for quantised tensors");
      if (fType != ETensorType::UINT8 && fType != ETensorType::FLOAT)
         throw std::runtime_error("SOFIE Pool op: unsupported tensor type");
   }
   // the samples of a batch are independent: any equal split of the batch axis is a valid launch (2-D and 1-D pooling)
   bool CanSliceBatch(size_t parts) const override { return parts > 0 && !fVolume && !fShapeX.empty() && fShapeX[0] % parts == 0; }
   std::string GenerateBatchSlice(std::string OpName, size_t parts) override { return GenerateCall(OpName, parts); }
   std::string Generate(std::string OpName) override { return GenerateCall(OpName, 1); }

private:
   std::string GenerateCall(std::string OpName, size_t parts)
   {
      OpName = "op_" + OpName;
      if (fShapeX.empty() || fShapeY.empty()) throw std::runtime_error("SOFIE Pool Op called to Generate without being initialized first");
      std::stringstream out;
      out << "\n" << SP << "//----  operator " << Name() << "  " << OpName << (parts > 1 ? ", one slice of the batch" : "") << "\n";
      const std::string x = EMIT::DevSlice(fNX, ConvertShapeToLength(fShapeX), parts), y = EMIT::DevSlice(fNY, ConvertShapeToLength(fShapeY), parts);
      if (fVolume) {
         out << SP << "{\n";
         out << SP << SP << "const sofie_pool3d_desc d = {" << (fPoolMode == MaxPool ? 0 : 1) << ", " << fShapeX[0] << ", " << fShapeX[1] << ", "
             << fShapeX[2] << ", " << fShapeX[3] << ", " << fShapeX[4] << ", " << fK3[0] << ", " << fK3[1] << ", " << fK3[2] << ", " << fS3[0]
             << ", " << fS3[1] << ", " << fS3[2] << ", {" << fP3[0] << ", " << fP3[1] << ", " << fP3[2] << ", " << fP3[3] << ", " << fP3[4]
             << ", " << fP3[5] << "}, " << fAttr.count_include_pad << "};\n";
         out << EMIT::Call(SP + SP, "sofie_cuda_pool3d_f32(fStream, &d, " + EMIT::Dev(fNX) + ", " + EMIT::Dev(fNY) + ")");
         out << SP << "}\n";
         return out.str();
      }
      if (fType == ETensorType::UINT8) {
         out << EMIT::Call(SP, "sofie_cuda_maxpool2d_u8(fStream, " + x + ", " + y + ", " +
                                  std::to_string(fShape4[0] / parts) + ", " + std::to_string(fShape4[1]) + ", " + std::to_string(fShape4[2]) +
                                  ", " + std::to_string(fShape4[3]) + ", " + std::to_string(fKH) + ", " + std::to_string(fKW) + ", " +
                                  std::to_string(fSH) + ", " + std::to_string(fSW) + ", " + std::to_string((int)fLayout) + ")");
         return out.str();
      }
      out << SP << "{\n";
      out << SP << SP << "const sofie_pool2d_desc d = {" << (fPoolMode == MaxPool ? 0 : 1) << ", " << fShape4[0] / parts << ", " << fShape4[1]
          << ", " << fShape4[2] << ", " << fShape4[3] << ", " << fKH << ", " << fKW << ", " << fSH << ", " << fSW << ", {" << fPads[0]
          << ", " << fPads[1] << ", " << fPads[2] << ", " << fPads[3] << "}, " << fAttr.count_include_pad << ", " << (int)fLayout << "};\n";
      out << EMIT::Call(SP + SP, "sofie_cuda_pool2d_f32(fStream, &d, " + x + ", " + y + ")");
      out << SP << "}\n";
      return out.str();
   }
};

} // namespace SOFIE
#endif
