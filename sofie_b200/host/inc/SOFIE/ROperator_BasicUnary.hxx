// Elementwise unary operators: the activations the reference has one class each for
// (ROperator_Sigmoid.hxx, ROperator_Tanh.hxx, ROperator_LeakyRelu.hxx, ROperator_Selu.hxx,
// ROperator_Elu.hxx, ROperator_Erf.hxx, ROperator_Swish.hxx) and its ROperator_BasicUnary<T, Op> family
// (Reciprocal, Sqrt, Neg, Exp, Log, Abs, Sin, Cos). Each emits one call of sofie_cuda_unary_f32; the formulas live in the library and follow
// the loops the reference emits (cited there).
#ifndef SOFIE_ROPERATOR_BASICUNARY
#define SOFIE_ROPERATOR_BASICUNARY

#include <sstream>

#include "SOFIE/Emit.hxx"
#include "SOFIE/RModel.hxx"
#include "SOFIE/ROperator.hxx"

namespace SOFIE {

enum class EBasicUnaryOperator { kReciprocal, kSqrt, kNeg, kExp, kLog, kAbs, kSin, kCos };

// Common body; `code` is the SOFIE_UNARY_* value of include/sofie_cuda.h.
class ROperator_UnaryDevice : public ROperator {
protected:
   std::string fNX, fNY, fOpLabel;
   int fCode = 0;
   float fAlpha = 0.f;
   std::vector<size_t> fShape;

   ROperator_UnaryDevice(std::string label, int code, float alpha, std::string nameX, std::string nameY)
      : fNX(UTILITY::Clean_name(nameX)), fNY(UTILITY::Clean_name(nameY)), fOpLabel(std::move(label)), fCode(code), fAlpha(alpha)
   {
      fInputTensorNames = {fNX};
      fOutputTensorNames = {fNY};
   }

public:
   EOpKind Kind() const override { return EOpKind::Eltwise; }
   bool AcceptsNHWC(const std::string &) const override { return true; } // elementwise: any layout
   std::vector<ETensorType> TypeInference(std::vector<ETensorType> input) override { return input; }
   std::vector<std::vector<size_t>> ShapeInference(std::vector<std::vector<size_t>> input) override { return input; }

   void Initialize(RModel &model) override
   {
      if (!model.CheckIfTensorAlreadyExist(fNX))
         throw std::runtime_error("SOFIE " + fOpLabel + " Op Input Tensor " + fNX + " is not found in model");
      if (model.GetTensorType(fNX) != ETensorType::FLOAT) throw std::runtime_error("SOFIE " + fOpLabel + " Op: only float tensors are supported");
      fShape = model.GetTensorShape(fNX);
      model.AddIntermediateTensor(fNY, model.GetTensorType(fNX), fShape);
   }
   void PlanDevice(RModel &model) override { model.SetTensorLayout(fNY, model.GetTensorLayout(model.ResolveAlias(fNX))); }
   // elementwise: any equal split of the elements is a valid launch
   bool CanSliceBatch(size_t parts) const override { return parts > 0 && !fShape.empty() && ConvertShapeToLength(fShape) % parts == 0; }
   std::string GenerateBatchSlice(std::string OpName, size_t parts) override { return GenerateCall(OpName, parts); }
   std::string Generate(std::string OpName) override { return GenerateCall(OpName, 1); }

private:
   std::string GenerateCall(std::string OpName, size_t parts)
   {
      OpName = "op_" + OpName;
      if (fShape.empty()) throw std::runtime_error("SOFIE Operator " + fOpLabel + " called to Generate without being initialized first");
      std::stringstream out;
      const size_t n = ConvertShapeToLength(fShape);
      out << "\n" << SP << "//------ " << fOpLabel << " " << OpName << (parts > 1 ? ", one slice of the batch" : "") << "\n";
      out << EMIT::Call(SP, "sofie_cuda_unary_f32(fStream, " + std::to_string(fCode) + ", " + EMIT::FloatLit(fAlpha) + ", " +
                               EMIT::DevSlice(fNX, n, parts) + ", " + EMIT::DevSlice(fNY, n, parts) + ", " + std::to_string(n / parts) + ")");
      return out.str();
   }
};

template <typename T>
class ROperator_Sigmoid final : public ROperator_UnaryDevice {
public:
   ROperator_Sigmoid(std::string nameX, std::string nameY) : ROperator_UnaryDevice("Sigmoid", 0, 0.f, nameX, nameY) {}
};
template <typename T>
class ROperator_Tanh final : public ROperator_UnaryDevice {
public:
   ROperator_Tanh(std::string nameX, std::string nameY) : ROperator_UnaryDevice("Tanh", 1, 0.f, nameX, nameY) {}
};
template <typename T>
class ROperator_LeakyRelu final : public ROperator_UnaryDevice {
public:
   ROperator_LeakyRelu(float alpha, std::string nameX, std::string nameY) : ROperator_UnaryDevice("LeakyRelu", 2, alpha, nameX, nameY) {}
};
template <typename T>
class ROperator_Selu final : public ROperator_UnaryDevice {
public:
   ROperator_Selu(std::string nameX, std::string nameY) : ROperator_UnaryDevice("Selu", 3, 0.f, nameX, nameY) {}
};
template <typename T>
class ROperator_Elu final : public ROperator_UnaryDevice {
public:
   ROperator_Elu(float alpha, std::string nameX, std::string nameY) : ROperator_UnaryDevice("Elu", 4, alpha, nameX, nameY) {}
};

// std::erf(x) (reference: ROperator_Erf.hxx:58) and x / (1 + exp(-x)) (reference: ROperator_Swish.hxx:59)
template <typename T>
class ROperator_Erf final : public ROperator_UnaryDevice {
public:
   ROperator_Erf(std::string nameX, std::string nameY) : ROperator_UnaryDevice("Erf", 11, 0.f, nameX, nameY) {}
};
template <typename T>
class ROperator_Swish final : public ROperator_UnaryDevice {
public:
   ROperator_Swish(std::string nameX, std::string nameY) : ROperator_UnaryDevice("Swish", 12, 0.f, nameX, nameY) {}
};

template <typename T, EBasicUnaryOperator Op>
class ROperator_BasicUnary final : public ROperator_UnaryDevice {
   static int Code()
   {
      switch (Op) {
      case EBasicUnaryOperator::kNeg: return 5;
      case EBasicUnaryOperator::kExp: return 6;
      case EBasicUnaryOperator::kLog: return 7;
      case EBasicUnaryOperator::kSqrt: return 8;
      case EBasicUnaryOperator::kReciprocal: return 9;
      case EBasicUnaryOperator::kCos: return 13;
      case EBasicUnaryOperator::kSin: return 14;
      default: return 10;
      }
   }
   static const char *Label()
   {
      switch (Op) {
      case EBasicUnaryOperator::kNeg: return "Neg";
      case EBasicUnaryOperator::kExp: return "Exp";
      case EBasicUnaryOperator::kLog: return "Log";
      case EBasicUnaryOperator::kSqrt: return "Sqrt";
      case EBasicUnaryOperator::kReciprocal: return "Reciprocal";
      case EBasicUnaryOperator::kCos: return "Cos";
      case EBasicUnaryOperator::kSin: return "Sin";
      default: return "Abs";
      }
   }

public:
   ROperator_BasicUnary(std::string nameX, std::string nameY) : ROperator_UnaryDevice(Label(), Code(), 0.f, nameX, nameY) {}
};

} // namespace SOFIE
#endif
