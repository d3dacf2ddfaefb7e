// ONNX Softmax along one axis (reference: src/SOFIE_core/inc/SOFIE/ROperator_Softmax.hxx:13-185, which
// emits per-line max / exp / normalise loops). Emits one call of sofie_cuda_softmax_f32 on the tensor
// viewed as [outer, axis, inner].
#ifndef SOFIE_ROPERATOR_SOFTMAX
#define SOFIE_ROPERATOR_SOFTMAX

#include <sstream>

#include "SOFIE/Emit.hxx"
#include "SOFIE/RModel.hxx"
#include "SOFIE/ROperator.hxx"

namespace SOFIE {

template <typename T>
class ROperator_Softmax final : public ROperator {
private:
   int64_t fAttrAxis = -1;
   std::string fNX, fNY;
   std::vector<size_t> fShape;

public:
   ROperator_Softmax() {}
   ROperator_Softmax(int64_t attr_axis, std::string nameX, std::string nameY)
      : fAttrAxis(attr_axis), fNX(UTILITY::Clean_name(nameX)), fNY(UTILITY::Clean_name(nameY))
   {
      fInputTensorNames = {fNX};
      fOutputTensorNames = {fNY};
   }
   EOpKind Kind() const override { return EOpKind::Softmax; }
   std::vector<ETensorType> TypeInference(std::vector<ETensorType> input) override { return input; }
   std::vector<std::vector<size_t>> ShapeInference(std::vector<std::vector<size_t>> input) override { return input; }
   void Initialize(RModel &model) override
   {
      if (!model.CheckIfTensorAlreadyExist(fNX)) throw std::runtime_error("SOFIE Softmax Op Input Tensor is not found in model");
      fShape = model.GetTensorShape(fNX);
      if (model.GetTensorType(fNX) != ETensorType::FLOAT) throw std::runtime_error("SOFIE Softmax Op: float tensors only");
      model.AddIntermediateTensor(fNY, model.GetTensorType(fNX), fShape);
   }
   // rows in front of the normalised axis are independent: a split of the leading dimension is a valid launch unless that
   // dimension is the axis itself
   bool CanSliceBatch(size_t parts) const override
   {
      if (parts == 0 || fShape.empty() || fShape[0] % parts != 0) return false;
      const int64_t axis = fAttrAxis < 0 ? fAttrAxis + (int64_t)fShape.size() : fAttrAxis;
      return axis > 0 && axis < (int64_t)fShape.size();
   }
   std::string GenerateBatchSlice(std::string OpName, size_t parts) override { return GenerateCall(OpName, parts); }
   std::string Generate(std::string OpName) override { return GenerateCall(OpName, 1); }

private:
   std::string GenerateCall(std::string OpName, size_t parts)
   {
      OpName = "op_" + OpName;
      if (fShape.empty()) throw std::runtime_error("SOFIE Operator Softmax called to Generate without being initialized first");
      size_t rank = fShape.size();
      int64_t axis = fAttrAxis < 0 ? fAttrAxis + (int64_t)rank : fAttrAxis;
      if (axis < 0 || axis >= (int64_t)rank) throw std::runtime_error("SOFIE Softmax Op: axis out of range");
      size_t outer = 1, inner = 1;
      for (int64_t i = 0; i < axis; i++) outer *= fShape[i];
      for (size_t i = axis + 1; i < rank; i++) inner *= fShape[i];
      if (fShape[axis] == 0) throw std::runtime_error("SOFIE - Softmax operator is along axis with zero elements");
      std::stringstream out;
      const size_t n = ConvertShapeToLength(fShape);
      out << "\n" << SP << "//------ SOFTMAX - " << rank << "  " << n << "  " << axis << (parts > 1 ? ", one slice of the batch" : "") << "\n";
      out << EMIT::Call(SP, "sofie_cuda_softmax_f32(fStream, " + EMIT::DevSlice(fNX, n, parts) + ", " + EMIT::DevSlice(fNY, n, parts) + ", " + std::to_string(outer / parts) +
                               ", " + std::to_string(fShape[axis]) + ", " + std::to_string(inner) + ")");
      return out.str();
   }
};

} // namespace SOFIE
#endif
