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
      if (input.size() != 1 || input[0].size() != 4)
         throw std::runtime_error("SOFIE " + Name() + " Op: only 2-D pooling of a rank-4 tensor is generated for the CUDA path");
      const auto &x = input[0];
      fKH = fAttr.kernel_shape.empty() ? x[2] : fAttr.kernel_shape[0];
      fKW = fAttr.kernel_shape.size() < 2 ? (fAttr.kernel_shape.empty() ? x[3] : fKH) : fAttr.kernel_shape[1];
      fSH = fAttr.strides.empty() ? 1 : fAttr.strides[0];
      fSW = fAttr.strides.size() < 2 ? fSH : fAttr.strides[1];
      if (fAttr.auto_pad == "NOTSET") {
         fPads = fAttr.pads.empty() ? std::vector<size_t>{0, 0, 0, 0} : fAttr.pads;
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
      size_t oH = (x[2] + fPads[0] + fPads[2] - fKH) / fSH + 1;
      size_t oW = (x[3] + fPads[1] + fPads[3] - fKW) / fSW + 1;
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
                                  std::to_string(fShapeX[0]) + ", " + std::to_string(fShapeX[1]) + ", " + std::to_string(fShapeX[2]) +
                                  ", " + std::to_string(fShapeX[3]) + ", " + std::to_string(fKH) + ", " + std::to_string(fKW) + ", " +
                                  std::to_string(fSH) + ", " + std::to_string(fSW) + ", " + std::to_string((int)fLayout) + ")");
         return out.str();
      }
      out << SP << "{\n";
      out << SP << SP << "const sofie_pool2d_desc d = {" << (fPoolMode == MaxPool ? 0 : 1) << ", " << fShapeX[0] << ", " << fShapeX[1]
          << ", " << fShapeX[2] << ", " << fShapeX[3] << ", " << fKH << ", " << fKW << ", " << fSH << ", " << fSW << ", {" << fPads[0]
          << ", " << fPads[1] << ", " << fPads[2] << ", " << fPads[3] << "}, " << fAttr.count_include_pad << ", " << (int)fLayout << "};\n";
      out << EMIT::Call(SP + SP, "sofie_cuda_pool2d_f32(fStream, &d, " + EMIT::Dev(fNX) + ", " + EMIT::Dev(fNY) + ")");
      out << SP << "}\n";
      return out.str();
   }
};

} // namespace SOFIE
#endif
