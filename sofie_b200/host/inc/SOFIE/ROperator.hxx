// Abstract operator of the code generator, CUDA edition.
//
// The virtual interface is the reference's (src/SOFIE_core/inc/SOFIE/ROperator.hxx:17-57):
// ShapeInference, TypeInference, Initialize, Generate, GenerateInitCode, GenerateDeclCode,
// GenerateSessionMembersCode, GetBlasRoutines, GetStdLibs, GetOpInputTensors / GetOpOutputTensors.
// Generate() returns the text of one or more calls into libSOFIE_cuda instead of CPU loops.
// Added for the device plan: Kind(), PlanDevice() (layout and weight-preparation decisions taken
// after every operator has been initialised) and IsFusedAway() (an operator whose work a
// neighbouring contraction's epilogue took over emits nothing).
#ifndef SOFIE_ROPERATOR
#define SOFIE_ROPERATOR

#include <string>
#include <string_view>
#include <vector>

#include "SOFIE/SOFIE_common.hxx"

namespace SOFIE {

class RModel;

enum class EOpKind { Other, Gemm, Conv, Relu, Pool, Reshape, Softmax, Cast, Quantize, Dequantize, QLinearMatMul, QLinearConv, Fp8Gemm, Eltwise };

class ROperator {
public:
   virtual std::vector<std::string> GetBlasRoutines() { return {}; } // kept for source compatibility; the CUDA path needs none
   virtual std::vector<std::string> GetStdLibs() { return {}; }
   virtual std::vector<std::vector<size_t>> ShapeInference(std::vector<std::vector<size_t>>) = 0;
   virtual std::vector<ETensorType> TypeInference(std::vector<ETensorType>) = 0;
   virtual void Initialize(RModel &) = 0;
   virtual std::string Generate(std::string OpName) = 0; // expects a unique OpName within one RModel
   virtual std::string GenerateInitCode() { return ""; }  // text for the Session constructor
   virtual std::string GenerateDeclCode() { return ""; }
   virtual std::string GenerateSessionMembersCode(std::string /*opName*/) { return ""; }
   virtual std::string Header() { return ""; }
   virtual ~ROperator() {}

   // ---- device plan ----
   virtual EOpKind Kind() const { return EOpKind::Other; }
   virtual void PlanDevice(RModel &) {}
   bool IsFusedAway() const { return fFusedAway; }
   void SetFusedAway() { fFusedAway = true; }
   // true when the operator can read a rank-4 input stored NHWC on the device
   virtual bool AcceptsNHWC(const std::string & /*input*/) const { return false; }

   // Pipelined input upload: an operator that treats the samples of a batch independently can be launched
   // on slice `part` of `parts` equal, contiguous slices of its batch-shaped inputs and outputs (`part` is a
   // variable of the emitted code), so that the model works on one slice while the next is still being copied.
   // Constant inputs (weights, tables) are read whole by every slice.
   virtual bool CanSliceBatch(size_t /*parts*/) const { return false; }
   virtual std::string GenerateBatchSlice(std::string /*OpName*/, size_t /*parts*/) { return ""; }

   const std::vector<std::string> &GetOpInputTensors() const { return fInputTensorNames; }
   const std::vector<std::string> &GetOpOutputTensors() const { return fOutputTensorNames; }

protected:
   const std::string SP = "   "; ///< indentation unit of the generated C++ code
   bool fUseSession = false;
   bool fIsOutputConstant = false;
   bool fFusedAway = false;
   std::vector<std::string> fInputTensorNames;
   std::vector<std::string> fOutputTensorNames;
};

} // namespace SOFIE

#endif
