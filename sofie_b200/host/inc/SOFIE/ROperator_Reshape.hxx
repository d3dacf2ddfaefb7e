// ONNX Reshape / Flatten / Squeeze / Unsqueeze.
// Constructors as in the reference (src/SOFIE_core/inc/SOFIE/ROperator_Reshape.hxx:45-66). The
// reference emits a std::copy of the whole tensor (:221-246); on the device the output is an alias of
// the input's arena slice and no code is emitted. A flattened NHWC activation keeps its memory
// order; the matmul that consumes it has its constant weight permuted instead.
#ifndef SOFIE_ROPERATOR_RESHAPE
#define SOFIE_ROPERATOR_RESHAPE

#include <sstream>

#include "SOFIE/RModel.hxx"
#include "SOFIE/ROperator.hxx"

namespace SOFIE {

enum ReshapeOpMode { Reshape, Flatten, Squeeze, Unsqueeze };

class ROperator_Reshape final : public ROperator {
private:
   ReshapeOpMode fOpMode = Reshape;
   int fAllowZero = 0;
   int fAxis = 1;
   std::string fNData, fNShape, fNOutput;
   std::vector<size_t> fShapeInput, fShapeOutput;
   std::vector<int64_t> fAttrAxes;

public:
   std::string Name() const
   {
      if (fOpMode == Reshape) return "Reshape";
      if (fOpMode == Flatten) return "Flatten";
      if (fOpMode == Squeeze) return "Squeeze";
      return "Unsqueeze";
   }
   ROperator_Reshape() {}
   ROperator_Reshape(ReshapeOpMode opMode, int attr_value, std::string nameData, std::string nameShape, std::string nameOutput)
      : fOpMode(opMode), fNData(UTILITY::Clean_name(nameData)), fNShape(UTILITY::Clean_name(nameShape)),
        fNOutput(UTILITY::Clean_name(nameOutput))
   {
      if (opMode == Reshape) fAllowZero = attr_value;
      if (opMode == Flatten) fAxis = attr_value;
      fInputTensorNames = {fNData};
      if (!fNShape.empty()) fInputTensorNames.push_back(fNShape);
      fOutputTensorNames = {fNOutput};
   }
   ROperator_Reshape(ReshapeOpMode opMode, std::vector<int64_t> attrAxes, std::string nameData, std::string nameOutput)
      : fOpMode(opMode), fNData(UTILITY::Clean_name(nameData)), fNOutput(UTILITY::Clean_name(nameOutput)), fAttrAxes(attrAxes)
   {
      fInputTensorNames = {fNData};
      fOutputTensorNames = {fNOutput};
   }
   EOpKind Kind() const override { return EOpKind::Reshape; }
   // a Flatten at axis 1 of an NHWC tensor is fine as long as its consumers are matmuls with constant weights
   bool AcceptsNHWC(const std::string &) const override { return fOpMode == Flatten && fAxis == 1; }
   const std::string &OutputName() const { return fNOutput; }

   std::vector<ETensorType> TypeInference(std::vector<ETensorType> input) override { return {input[0]}; }

   std::vector<std::vector<size_t>> ShapeInference(std::vector<std::vector<size_t>> input) override
   {
      const auto &in = input[0];
      size_t len = ConvertShapeToLength(in);
      std::vector<size_t> out;
      if (fOpMode == Flatten) {
         int axis = fAxis < 0 ? fAxis + (int)in.size() : fAxis;
         size_t a = 1, b = 1;
         for (size_t i = 0; i < in.size(); i++) ((int)i < axis ? a : b) *= in[i];
         out = {a, b};
      } else if (fOpMode == Reshape) {
         if (input.size() != 2) throw std::runtime_error("SOFIE Reshape Op needs the target shape");
         out = input[1];
         size_t known = 1;
         int infer = -1;
         for (size_t i = 0; i < out.size(); i++) {
            if (out[i] == static_cast<size_t>(-1)) infer = (int)i;
            else {
               if (out[i] == 0 && !fAllowZero && i < in.size()) out[i] = in[i];
               known *= out[i];
            }
         }
         if (infer >= 0) out[infer] = known ? len / known : 0;
      } else if (fOpMode == Squeeze) {
         std::vector<int64_t> axes = fAttrAxes;
         if (input.size() == 2) axes.assign(input[1].begin(), input[1].end());
         for (size_t i = 0; i < in.size(); i++) {
            bool drop = axes.empty() ? in[i] == 1 : false;
            for (auto a : axes)
               if ((a < 0 ? a + (int64_t)in.size() : a) == (int64_t)i) drop = true;
            if (!drop) out.push_back(in[i]);
         }
      } else {
         std::vector<int64_t> axes = fAttrAxes;
         if (input.size() == 2) axes.assign(input[1].begin(), input[1].end());
         size_t rank = in.size() + axes.size();
         out.assign(rank, 0);
         for (auto a : axes) out[a < 0 ? a + (int64_t)rank : a] = 1;
         size_t j = 0;
         for (size_t i = 0; i < rank; i++)
            if (out[i] == 0) out[i] = in[j++];
      }
      if (ConvertShapeToLength(out) != len)
         throw std::runtime_error("SOFIE " + Name() + " Op : output shape " + ConvertShapeToString(out) + " does not hold " +
                                  std::to_string(len) + " elements");
      return {out};
   }

   void Initialize(RModel &model) override
   {
      if (!model.CheckIfTensorAlreadyExist(fNData)) throw std::runtime_error("SOFIE Reshape Op Input Tensor " + fNData + " is not found in model");
      fShapeInput = model.GetTensorShape(fNData);
      std::vector<std::vector<size_t>> in = {fShapeInput};
      if (!fNShape.empty()) {
         if (!model.IsInitializedTensor(fNShape)) throw std::runtime_error("SOFIE Reshape Op: shape tensor " + fNShape + " must be constant");
         const auto &t = model.GetInitializedTensor(fNShape);
         if (t.type() != ETensorType::INT64) throw std::runtime_error("SOFIE Reshape Op: shape tensor must be int64");
         std::vector<size_t> target(t.length());
         for (size_t i = 0; i < target.size(); i++) target[i] = static_cast<size_t>(t.data<int64_t>()[i]);
         in.push_back(target);
         model.SetNotWritableInitializedTensor(fNShape);
      }
      fShapeOutput = ShapeInference(in)[0];
      model.AddIntermediateTensor(fNOutput, model.GetTensorType(fNData), fShapeOutput);
   }
   void PlanDevice(RModel &model) override
   {
      std::string owner = model.ResolveAlias(fNData);
      if (model.GetTensorLayout(owner) == ELayout::NHWC && !(fOpMode == Flatten && fAxis == 1))
         throw std::runtime_error("SOFIE " + Name() + " Op: cannot reinterpret an NHWC tensor");
      model.AddAlias(fNOutput, owner);
   }
   // an alias: slice `part` of the output IS slice `part` of the input
   bool CanSliceBatch(size_t parts) const override { return parts > 0; }
   std::string GenerateBatchSlice(std::string OpName, size_t) override { return Generate(OpName); }
   std::string Generate(std::string OpName) override
   {
      if (fShapeInput.empty()) throw std::runtime_error("SOFIE Reshape Op called to Generate without being initialized first");
      return "\n" + SP + "//------ " + Name() + " op_" + OpName + ": " + fNOutput + " aliases " + fNData + " on the device\n";
   }
};

} // namespace SOFIE
#endif
