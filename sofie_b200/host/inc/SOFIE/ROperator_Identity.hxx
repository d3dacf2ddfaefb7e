// ONNX Identity. Constructor as in the reference (src/SOFIE_core/inc/SOFIE/ROperator_Identity.hxx:27-31), which emits
// a copy of the tensor; on the device the output is an alias of the input's memory and no kernel runs. An Identity
// of a constant (exporters write one per shared weight) never reaches this class: the parser registers its output
// as a second name of the same initialised tensor.
#ifndef SOFIE_ROPERATOR_IDENTITY
#define SOFIE_ROPERATOR_IDENTITY

#include "SOFIE/RModel.hxx"
#include "SOFIE/ROperator.hxx"

namespace SOFIE {

template <typename T>
class ROperator_Identity final : public ROperator {
private:
   std::string fNX, fNY;
   std::vector<size_t> fShape;

public:
   ROperator_Identity() {}
   ROperator_Identity(std::string nameX, std::string nameY) : fNX(UTILITY::Clean_name(nameX)), fNY(UTILITY::Clean_name(nameY))
   {
      fInputTensorNames = {fNX};
      fOutputTensorNames = {fNY};
   }
   EOpKind Kind() const override { return EOpKind::Eltwise; }
   bool AcceptsNHWC(const std::string &) const override { return true; }
   std::vector<ETensorType> TypeInference(std::vector<ETensorType> input) override { return input; }
   std::vector<std::vector<size_t>> ShapeInference(std::vector<std::vector<size_t>> input) override { return input; }

   void Initialize(RModel &model) override
   {
      if (!model.CheckIfTensorAlreadyExist(fNX)) throw std::runtime_error("SOFIE Identity Op Input Tensor " + fNX + " is not found in model");
      fShape = model.GetTensorShape(fNX);
      model.AddIntermediateTensor(fNY, model.GetTensorType(fNX), fShape);
   }
   void PlanDevice(RModel &model) override
   {
      std::string owner = model.ResolveAlias(fNX);
      model.SetTensorLayout(fNY, model.GetTensorLayout(owner));
      model.AddAlias(fNY, owner);
   }
   std::string Generate(std::string OpName) override
   {
      if (fShape.empty()) throw std::runtime_error("SOFIE Operator Identity called to Generate without being initialized first");
      return "\n" + SP + "//------ Identity op_" + OpName + ": " + fNY + " aliases " + fNX + " on the device\n";
   }
};

} // namespace SOFIE
#endif
