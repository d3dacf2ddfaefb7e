// Add / Sub / Mul / Div with multidirectional broadcasting (reference:
// src/SOFIE_core/inc/SOFIE/ROperator_BasicBinary.hxx:18-43 for the operators, :85-175 for the
// shape rules). The reference materialises broadcast copies of the operands; here the kernel reads
// the operands through strides that are 0 along broadcast dimensions, so nothing is copied.
// Operands are read in NCHW; a constant operand is uploaded once by the Session constructor.
#ifndef SOFIE_ROPERATOR_BASICBINARY
#define SOFIE_ROPERATOR_BASICBINARY

#include <sstream>

#include "SOFIE/Emit.hxx"
#include "SOFIE/RModel.hxx"
#include "SOFIE/ROperator.hxx"

namespace SOFIE {

enum EBasicBinaryOperator { Add, Sub, Mul, Div, Pow };

template <typename T, EBasicBinaryOperator Op>
class ROperator_BasicBinary final : public ROperator {
private:
   std::string fNA, fNB, fNY;
   std::vector<size_t> fShapeA, fShapeB, fShapeY;

   static const char *Name()
   {
      switch (Op) {
      case Add: return "Add";
      case Sub: return "Sub";
      case Mul: return "Mul";
      case Div: return "Div";
      default: return "Pow";
      }
   }
   // element strides of `shape` inside the rank-4 output, 0 where the operand is broadcast
   static std::vector<long long> Strides(const std::vector<size_t> &shape, const std::vector<size_t> &out)
   {
      std::vector<size_t> padded(out.size() - shape.size(), 1);
      padded.insert(padded.end(), shape.begin(), shape.end());
      std::vector<long long> st(4, 0);
      long long dense = 1;
      for (int i = (int)out.size() - 1; i >= 0; i--) {
         st[4 - out.size() + i] = padded[i] == 1 ? 0 : dense;
         dense *= (long long)padded[i];
      }
      return st;
   }

public:
   ROperator_BasicBinary() {}
   ROperator_BasicBinary(std::string nameA, std::string nameB, std::string nameY)
      : fNA(UTILITY::Clean_name(nameA)), fNB(UTILITY::Clean_name(nameB)), fNY(UTILITY::Clean_name(nameY))
   {
      fInputTensorNames = {fNA, fNB};
      fOutputTensorNames = {fNY};
   }
   std::vector<ETensorType> TypeInference(std::vector<ETensorType> input) override { return {input[0]}; }
   std::vector<std::vector<size_t>> ShapeInference(std::vector<std::vector<size_t>> input) override
   {
      return {UTILITY::MultidirectionalBroadcastShape(input[0], input[1])};
   }
   void Initialize(RModel &model) override
   {
      if (Op == Pow) throw std::runtime_error("SOFIE Binary Op Pow is not generated for the device");
      if (!model.CheckIfTensorAlreadyExist(fNA)) throw std::runtime_error(std::string("SOFIE Binary Op Input Tensor ") + fNA + " is not found in model");
      if (!model.CheckIfTensorAlreadyExist(fNB)) throw std::runtime_error(std::string("SOFIE Binary Op Input Tensor ") + fNB + " is not found in model");
      if (model.GetTensorType(fNA) != ETensorType::FLOAT || model.GetTensorType(fNB) != ETensorType::FLOAT)
         throw std::runtime_error(std::string("SOFIE Binary Op ") + Name() + ": only float tensors are supported");
      fShapeA = model.GetTensorShape(fNA);
      fShapeB = model.GetTensorShape(fNB);
      fShapeY = UTILITY::MultidirectionalBroadcastShape(fShapeA, fShapeB);
      fConstA = model.IsInitializedTensor(fNA);
      fConstB = model.IsInitializedTensor(fNB);
      if (fShapeY.size() > 4) throw std::runtime_error(std::string("SOFIE Binary Op ") + Name() + ": rank above 4 is not supported on the device");
      model.AddIntermediateTensor(fNY, ETensorType::FLOAT, fShapeY);
   }
   void PlanDevice(RModel &model) override
   {
      if (model.IsInitializedTensor(fNA)) model.UseOnDevice(fNA);
      if (model.IsInitializedTensor(fNB)) model.UseOnDevice(fNB);
      model.SetTensorLayout(fNY, ELayout::NCHW);
   }
   // elementwise over the output: an equal split of its leading dimension is a valid launch when every operand either has that
   // dimension too (its slice is read) or is a constant broadcast along it (read whole by every slice)
   bool CanSliceBatch(size_t parts) const override
   {
      if (parts == 0 || fShapeY.empty() || fShapeY[0] % parts != 0) return false;
      const size_t lead = 4 - fShapeY.size();
      const auto sa = Strides(fShapeA, fShapeY), sb = Strides(fShapeB, fShapeY);
      if (fShapeY[0] > 1 && ((sa[lead] == 0 && !fConstA) || (sb[lead] == 0 && !fConstB))) return false;
      return true;
   }
   std::string GenerateBatchSlice(std::string OpName, size_t parts) override { return GenerateCall(OpName, parts); }
   std::string Generate(std::string OpName) override { return GenerateCall(OpName, 1); }

private:
   bool fConstA = false, fConstB = false;
   std::string GenerateCall(std::string OpName, size_t parts)
   {
      OpName = "op_" + OpName;
      if (fShapeY.empty() && ConvertShapeToLength(fShapeY) != 1)
         throw std::runtime_error("SOFIE Binary Op called to Generate without being initialized first");
      std::vector<size_t> out4(4 - fShapeY.size(), 1);
      out4.insert(out4.end(), fShapeY.begin(), fShapeY.end());
      auto sa = Strides(fShapeA, fShapeY), sb = Strides(fShapeB, fShapeY);
      std::string a = EMIT::Dev(fNA), b = EMIT::Dev(fNB), y = EMIT::Dev(fNY);
      if (parts > 1) {
         const size_t lead = 4 - fShapeY.size(), rows = fShapeY[0] / parts;
         out4[lead] = rows;
         if (sa[lead]) a = "(" + a + " + (size_t)part * " + std::to_string((size_t)sa[lead] * rows) + ")";
         if (sb[lead]) b = "(" + b + " + (size_t)part * " + std::to_string((size_t)sb[lead] * rows) + ")";
         y = EMIT::DevSlice(fNY, ConvertShapeToLength(fShapeY), parts);
      }
      std::stringstream out;
      out << "\n" << SP << "//------ " << Name() << " " << OpName << " -> " << fNY << " " << ConvertShapeToString(fShapeY)
          << (parts > 1 ? ", one slice of the batch" : "") << "\n";
      out << SP << "{\n";
      out << SP << SP << "const sofie_binary_desc d = {" << (int)Op << ", {" << out4[0] << ", " << out4[1] << ", " << out4[2] << ", " << out4[3]
          << "}, {" << sa[0] << ", " << sa[1] << ", " << sa[2] << ", " << sa[3] << "}, {" << sb[0] << ", " << sb[1] << ", " << sb[2] << ", "
          << sb[3] << "}};\n";
      out << EMIT::Call(SP + SP, "sofie_cuda_binary_f32(fStream, &d, " + a + ", " + b + ", " + y + ")");
      out << SP << "}\n";
      return out.str();
   }
};

} // namespace SOFIE
#endif
