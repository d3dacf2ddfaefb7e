// ONNX MaxPool / AveragePool / GlobalAveragePool, 2-D.
// Constructor and attribute struct as in the reference (src/SOFIE_core/inc/SOFIE/ROperator_Pool.hxx:17-83).
// The reference emits scalar nested loops (:266-476); this emits one call of sofie_cuda_pool2d_f32
// (or sofie_cuda_maxpool2d_u8 on a quantised tensor), unless the model plan folded a 2x2 stride-2
// MaxPool into the preceding convolution. `pads` follow ONNX (h_begin, w_begin, h_end, w_end), the
// reading of the reference's shape inference (:172-189).
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
   bool AcceptsNHWC(const std::string &) const override { return true; }
   const std::string &InputName() const { return fNX; }
   const std::string &OutputName() const { return fNY; }
   // 2x2 window, stride 2, no padding: the form a convolution epilogue can absorb
   bool IsMax2x2Stride2() const
   {
      return fPoolMode == MaxPool && fKH == 2 && fKW == 2 && fSH == 2 && fSW == 2 && fPads[0] + fPads[1] + fPads[2] + fPads[3] == 0;
   }

   std::vector<ETensorType> TypeInference(std::vector<ETensorType> input) override { return input; }
   std::vector<std::vector<size_t>> ShapeInference(std::vector<std::vector<size_t>> input) override
   {
      if (input.size() != 1 || (input[0].size() != 4 && input[0].size() != 3))
         throw std::runtime_error("SOFIE " + Name() + " Op: only 1-D and 2-D pooling (rank-3 and rank-4 tensors) is generated for the CUDA path");
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

   void Initialize(RModel &model) override
   {
      fUseSession = model.UseSession();
      if (!model.CheckIfTensorAlreadyExist(fNX)) throw std::runtime_error("SOFIE Pool op Input Tensor " + fNX + " is not found in model");
      fShapeX = model.GetTensorShape(fNX);
      if (fPoolMode == GlobalAveragePool) {
         fPoolMode = AveragePool;
         fAttr.kernel_shape = {fShapeX.at(2), fShapeX.at(3)};
         fAttr.auto_pad = "VALID";
         fAttr.pads = {0, 0, 0, 0};
         fAttr.strides = {1, 1};
      }
      fShapeY = ShapeInference({fShapeX})[0];
      fType = model.GetTensorType(fNX);
      model.AddIntermediateTensor(fNY, fType, fShapeY);
   }
   void PlanDevice(RModel &model) override
   {
      fLayout = model.GetTensorLayout(model.ResolveAlias(fNX));
      model.SetTensorLayout(fNY, fLayout);
      if (fType == ETensorType::UINT8 && (fPoolMode != MaxPool || fPads[0] + fPads[1] + fPads[2] + fPads[3] != 0))
         throw std::runtime_error("SOFIE Pool op: only un-padded MaxPool is generated for quantised tensors");
      if (fType != ETensorType::UINT8 && fType != ETensorType::FLOAT)
         throw std::runtime_error("SOFIE Pool op: unsupported tensor type");
   }
   std::string Generate(std::string OpName) override
   {
      OpName = "op_" + OpName;
      if (fShapeX.empty() || fShapeY.empty()) throw std::runtime_error("SOFIE Pool Op called to Generate without being initialized first");
      std::stringstream out;
      out << "\n" << SP << "//----  operator " << Name() << "  " << OpName << "\n";
      if (fType == ETensorType::UINT8) {
         out << EMIT::Call(SP, "sofie_cuda_maxpool2d_u8(fStream, " + EMIT::Dev(fNX) + ", " + EMIT::Dev(fNY) + ", " +
                                  std::to_string(fShape4[0]) + ", " + std::to_string(fShape4[1]) + ", " + std::to_string(fShape4[2]) +
                                  ", " + std::to_string(fShape4[3]) + ", " + std::to_string(fKH) + ", " + std::to_string(fKW) + ", " +
                                  std::to_string(fSH) + ", " + std::to_string(fSW) + ", " + std::to_string((int)fLayout) + ")");
         return out.str();
      }
      out << SP << "{\n";
      out << SP << SP << "const sofie_pool2d_desc d = {" << (fPoolMode == MaxPool ? 0 : 1) << ", " << fShape4[0] << ", " << fShape4[1]
          << ", " << fShape4[2] << ", " << fShape4[3] << ", " << fKH << ", " << fKW << ", " << fSH << ", " << fSW << ", {" << fPads[0]
          << ", " << fPads[1] << ", " << fPads[2] << ", " << fPads[3] << "}, " << fAttr.count_include_pad << ", " << (int)fLayout << "};\n";
      out << EMIT::Call(SP + SP, "sofie_cuda_pool2d_f32(fStream, &d, " + EMIT::Dev(fNX) + ", " + EMIT::Dev(fNY) + ")");
      out << SP << "}\n";
      return out.str();
   }
};

} // namespace SOFIE
#endif
