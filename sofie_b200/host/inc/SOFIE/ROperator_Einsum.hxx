// ONNX Einsum with two operands (no ellipsis, no label repeated within one operand).
//
// Constructor as in the reference (src/SOFIE_core/inc/SOFIE/ROperator_Einsum.hxx:40-60: equation, input names,
// output name). The reference emits nested loops over the output and the summation labels, or one sgemm_ per stack
// index when the equation is a (stacked) matrix product (:200-332). Here an equation of the form
// "<stack>ik,<stack>kj-><stack>ij" (either operand possibly transposed in its last two labels) becomes one call of
// sofie_cuda_gemm_f32_batched, i.e. the tensor-core GEMM per stack index; every other equation is ONE call of
// sofie_cuda_einsum_f32 with the labels' extents and strides worked out here. "ik,kj->ij" never gets here: the parser
// hands it to the GEMM operator.
#ifndef SOFIE_ROPERATOR_EINSUM
#define SOFIE_ROPERATOR_EINSUM

#include <algorithm>
#include <map>
#include <sstream>

#include "SOFIE/Emit.hxx"
#include "SOFIE/RModel.hxx"
#include "SOFIE/ROperator.hxx"

namespace SOFIE {

template <typename T>
class ROperator_Einsum final : public ROperator {
   std::string fEquation, fNA, fNB, fNY;
   std::string fLabelsA, fLabelsB, fLabelsOut;
   std::vector<size_t> fShapeA, fShapeB, fShapeY;
   std::vector<char> fLabels;            // output labels in output order, then the summed ones
   std::vector<size_t> fExtent, fStrideA, fStrideB;
   size_t fNOut = 0;
   // stacked matrix product form
   bool fIsMatMul = false;
   size_t fStack = 1, fM = 0, fN = 0, fK = 0;
   int fTransA = 0, fTransB = 0;

   // "<stack>ik,<stack>kj-><stack>ij": the same leading labels in the same order everywhere, then two labels each
   void DetectMatMul(const std::map<char, size_t> &size)
   {
      fIsMatMul = false;
      const size_t nb = fLabelsOut.size() < 2 ? std::string::npos : fLabelsOut.size() - 2;
      if (nb == std::string::npos || fLabelsA.size() != nb + 2 || fLabelsB.size() != nb + 2) return;
      if (fLabelsA.compare(0, nb, fLabelsOut, 0, nb) != 0 || fLabelsB.compare(0, nb, fLabelsOut, 0, nb) != 0) return;
      const std::string ra = fLabelsA.substr(nb), rb = fLabelsB.substr(nb), ro = fLabelsOut.substr(nb);
      const char i = ro[0], j = ro[1];
      if (ra.find(i) == std::string::npos || rb.find(j) == std::string::npos || ra.find(j) != std::string::npos || rb.find(i) != std::string::npos) return;
      const char ka = ra[0] == i ? ra[1] : ra[0], kb = rb[0] == j ? rb[1] : rb[0];
      if (ka != kb || ka == i || ka == j) return;
      fIsMatMul = true;
      fTransA = ra[0] == ka;   // A stored [k][i]
      fTransB = rb[0] == j;    // B stored [j][k]
      fM = size.at(i);
      fN = size.at(j);
      fK = size.at(ka);
      fStack = 1;
      for (size_t b = 0; b < nb; b++) fStack *= size.at(fLabelsOut[b]);
   }

   void ParseEquation()
   {
      std::string eq = fEquation;
      eq.erase(std::remove(eq.begin(), eq.end(), ' '), eq.end());
      if (eq.find('.') != std::string::npos) throw std::runtime_error("SOFIE Einsum Op: an ellipsis is not supported: " + fEquation);
      const size_t arrow = eq.find("->"), comma = eq.find(',');
      if (comma == std::string::npos || eq.find(',', comma + 1) != std::string::npos)
         throw std::runtime_error("SOFIE Einsum Op: exactly two operands are generated for the CUDA path: " + fEquation);
      const std::string lhs = arrow == std::string::npos ? eq : eq.substr(0, arrow);
      fLabelsA = lhs.substr(0, comma);
      fLabelsB = lhs.substr(comma + 1);
      if (arrow != std::string::npos) {
         fLabelsOut = eq.substr(arrow + 2);
      } else { // implicit form: the labels that appear once, in alphabetical order
         std::string all = fLabelsA + fLabelsB;
         for (char c : all)
            if (std::count(all.begin(), all.end(), c) == 1) fLabelsOut += c;
         std::sort(fLabelsOut.begin(), fLabelsOut.end());
      }
      auto unique = [](const std::string &l) { return std::all_of(l.begin(), l.end(), [&](char c) { return std::count(l.begin(), l.end(), c) == 1; }); };
      if (!unique(fLabelsA) || !unique(fLabelsB) || !unique(fLabelsOut))
         throw std::runtime_error("SOFIE Einsum Op: a label repeated within one operand is not supported: " + fEquation);
   }

public:
   ROperator_Einsum() {}
   ROperator_Einsum(const std::string &equation, const std::vector<std::string> &namesX, const std::string &nameY)
      : fEquation(equation), fNY(UTILITY::Clean_name(nameY))
   {
      static_assert(std::is_same_v<T, float>, "SOFIE - Einsum is generated for float tensors");
      if (namesX.size() != 2) throw std::runtime_error("SOFIE Einsum Op: exactly two operands are generated for the CUDA path");
      fNA = UTILITY::Clean_name(namesX[0]);
      fNB = UTILITY::Clean_name(namesX[1]);
      fInputTensorNames = {fNA, fNB};
      fOutputTensorNames = {fNY};
      ParseEquation();
   }
   EOpKind Kind() const override { return EOpKind::Other; }
   std::vector<ETensorType> TypeInference(std::vector<ETensorType> input) override { return {input[0]}; }
   std::vector<std::vector<size_t>> ShapeInference(std::vector<std::vector<size_t>> input) override
   {
      if (input.size() != 2 || input[0].size() != fLabelsA.size() || input[1].size() != fLabelsB.size())
         throw std::runtime_error("SOFIE Einsum Op: the equation " + fEquation + " does not match the ranks of its operands");
      std::map<char, size_t> size;
      auto take = [&](const std::string &labels, const std::vector<size_t> &shape) {
         for (size_t i = 0; i < labels.size(); i++) {
            auto it = size.find(labels[i]);
            if (it == size.end()) size[labels[i]] = shape[i];
            else if (it->second != shape[i]) throw std::runtime_error(std::string("SOFIE Einsum Op: label ") + labels[i] + " has two extents");
         }
      };
      take(fLabelsA, input[0]);
      take(fLabelsB, input[1]);
      fLabels.assign(fLabelsOut.begin(), fLabelsOut.end());
      for (char c : fLabelsOut)
         if (!size.count(c)) throw std::runtime_error(std::string("SOFIE Einsum Op: output label ") + c + " is in no operand");
      fNOut = fLabels.size();
      for (char c : fLabelsA + fLabelsB)
         if (std::find(fLabels.begin(), fLabels.end(), c) == fLabels.end()) fLabels.push_back(c);
      if (fLabels.size() > 8) throw std::runtime_error("SOFIE Einsum Op: at most 8 labels");
      auto strides = [&](const std::string &labels, const std::vector<size_t> &shape) {
         std::map<char, size_t> st;
         size_t dense = 1;
         for (size_t i = labels.size(); i-- > 0;) {
            st[labels[i]] = dense;
            dense *= shape[i];
         }
         std::vector<size_t> out;
         for (char c : fLabels) out.push_back(st.count(c) ? st[c] : 0);
         return out;
      };
      fExtent.clear();
      for (char c : fLabels) fExtent.push_back(size[c]);
      fStrideA = strides(fLabelsA, input[0]);
      fStrideB = strides(fLabelsB, input[1]);
      std::vector<size_t> y;
      for (char c : fLabelsOut) y.push_back(size[c]);
      if (y.empty()) y.push_back(1); // a scalar result is kept as one element
      DetectMatMul(size);
      return {y};
   }
   void Initialize(RModel &model) override
   {
      for (auto &n : {fNA, fNB})
         if (!model.CheckIfTensorAlreadyExist(n)) throw std::runtime_error("SOFIE Einsum Op Input Tensor " + n + " is not found in model");
      if (model.GetTensorType(fNA) != ETensorType::FLOAT || model.GetTensorType(fNB) != ETensorType::FLOAT)
         throw std::runtime_error("SOFIE Einsum Op: only float tensors are supported");
      fShapeA = model.GetTensorShape(fNA);
      fShapeB = model.GetTensorShape(fNB);
      fShapeY = ShapeInference({fShapeA, fShapeB})[0];
      model.AddIntermediateTensor(fNY, ETensorType::FLOAT, fShapeY);
   }
   void PlanDevice(RModel &model) override
   {
      for (auto &n : {fNA, fNB}) {
         if (model.IsInitializedTensor(n)) model.UseOnDevice(n);
         else if (model.GetTensorLayout(model.ResolveAlias(n)) == ELayout::NHWC)
            throw std::runtime_error("SOFIE Einsum Op: NHWC input is not supported");
      }
   }
   std::string Generate(std::string OpName) override
   {
      std::stringstream out;
      auto list = [](const std::vector<size_t> &v) {
         std::string s;
         for (size_t i = 0; i < 8; i++) s += (i ? ", " : "") + std::to_string(i < v.size() ? v[i] : 0);
         return s;
      };
      out << "\n" << SP << "//------ Einsum op_" << OpName << "  " << fEquation << " -> " << fNY << " " << ConvertShapeToString(fShapeY) << "\n";
      out << SP << "{\n";
      if (fIsMatMul) {
         // a (stacked) matrix product: the GEMM kernels, one product per stack index
         out << SP << SP << "const sofie_gemm_f32_desc d = {" << fM << ", " << fN << ", " << fK << ", " << fTransA << ", " << fTransB
             << ", 1.0f, 0.0f, 0, 0};\n";
         out << EMIT::Call(SP + SP, "sofie_cuda_gemm_f32_batched(fStream, &d, " + EMIT::Dev(fNA) + ", " + EMIT::Dev(fNB) + ", nullptr, " +
                                       EMIT::Dev(fNY) + ", " + std::to_string(fStack) + ", " + std::to_string(fM * fK) + ", " +
                                       std::to_string(fN * fK) + ", " + std::to_string(fM * fN) + ")");
         out << SP << "}\n";
         return out.str();
      }
      out << SP << SP << "const sofie_einsum_desc d = {" << fNOut << ", " << fLabels.size() - fNOut << ", {" << list(fExtent) << "}, {"
          << list(fStrideA) << "}, {" << list(fStrideB) << "}};\n";
      out << EMIT::Call(SP + SP, "sofie_cuda_einsum_f32(fStream, &d, " + EMIT::Dev(fNA) + ", " + EMIT::Dev(fNB) + ", " + EMIT::Dev(fNY) + ")");
      out << SP << "}\n";
      return out.str();
   }
};

} // namespace SOFIE
#endif
