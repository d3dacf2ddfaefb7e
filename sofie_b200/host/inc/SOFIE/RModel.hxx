// Graph IR and code-generation driver, CUDA edition.
//
// Public interface as in the reference (src/SOFIE_core/inc/SOFIE/RModel.hxx:59-200): tensor
// registries (AddInputTensorInfo, AddInitializedTensor, AddIntermediateTensor, ...), AddOperator,
// AddOutputTensorNameList, Initialize, Generate(Options, batchSize, pos, verbose), OutputGenerated,
// Print*. What Generate() emits differs: the Session owns a sofie_cuda_ctx (device arena, uploaded
// weights, stream, CUDA graph) and infer() is host->device copy, a captured sequence of
// libSOFIE_cuda launches, device->host copy -- with the reference's signature
//     struct Session { Session(std::string filename = "<name>.dat"); std::vector<float> infer(float* tensor_<in>); }
// (reference: src/SOFIE_core/src/RModel.cxx:744-910).
//
// Between Initialize() of the operators and code emission the model runs a device plan:
//   1. fusion   Conv -> Relu -> MaxPool(2x2, stride 2) and QLinearConv -> Relu -> MaxPool collapse
//               into the convolution's epilogue; Flatten/Reshape become aliases.
//   2. layout   rank-4 activations produced and consumed only by convolutions, pools, Relu and
//               Flatten->MatMul stay NHWC on the device; model inputs and outputs are NCHW.
//   3. weights  operators re-lay their weights at generation time (transpose to [N,K], OHWI
//               packing, column permutation after an NHWC Flatten); the weight file stores the
//               prepared tensors.
//   4. memory   liveness-based first-fit placement of every intermediate tensor in one arena
//               (the reference's pool planner: src/SOFIE_core/src/RModel.cxx:304-394).
#ifndef SOFIE_RMODEL
#define SOFIE_RMODEL

#include <map>
#include <memory>
#include <set>
#include <string>
#include <vector>

#include "SOFIE/RModel_Base.hxx"
#include "SOFIE/ROperator.hxx"
#include "SOFIE/SOFIE_common.hxx"

namespace SOFIE {

class RModel final : public RModel_Base {
private:
   bool fIsInitialized = false;
   int fVerbose = 0;
   int fBatchSize = -1;
   long fReadPos = 0;

   std::map<std::string, InputTensorInfo> fInputTensorInfos;   // inputs with parametric dimensions
   std::map<std::string, TensorInfo> fReadyInputTensorInfos;   // inputs with fully known shapes
   std::map<std::string, InitializedTensor> fInitializedTensors;
   std::map<std::string, TensorInfo> fIntermediateTensorInfos;
   std::map<std::string, std::string> fShapeParams;
   std::vector<std::string> fOutputTensorNames;
   std::vector<std::string> fInputTensorNames;
   std::vector<std::unique_ptr<ROperator>> fOperators;

   // ---- device plan ----
   std::map<std::string, ELayout> fLayouts;          // absent = NCHW / row-major
   std::map<std::string, std::string> fAliases;      // tensor -> tensor whose memory it shares
   std::map<std::string, size_t> fArenaOffsets;      // tensors that own arena memory
   size_t fArenaBytes = 0;
   bool fForcePipelinedUpload = false;
   bool fNeverPipelinedUpload = false;
   size_t fUploadParts = 4;                  // parts of a pipelined input upload (at most SOFIE_CUDA_MAX_PARTS)
   std::vector<size_t> fSlicedOps;           // operators launched once per uploaded part, in execution order
   // Run-time batch: Generate() without a batch size on a model whose inputs carry a batch parameter in their first
   // dimension keeps that parameter in the emitted Session (reference: RModel.cxx:680-713, 876-884). Shapes are then
   // inferred with the batch set to a large prime; a number of the emitted text that is a multiple of it scales with the
   // batch and is written as `k * fBatch`.
   bool fDynamicBatch = false;
   std::string fBatchParam;
   static constexpr size_t kBatchSentinel = 1000003;
   void MakeBatchSymbolic();
   std::vector<std::string> fSessionMembers;         // data members of the emitted Session, in declaration order
   std::set<std::string> fDeviceWeights;             // initialised tensors the emitted code uploads
   struct DeviceBuffer {
      ETensorType type;
      size_t length;
   };
   std::map<std::string, DeviceBuffer> fDeviceBuffers; // persistent buffers filled at Session construction

   const std::string SP = "   ";

public:
   RModel() = default;
   RModel(std::string name, std::string parsedtime) : RModel_Base(name, parsedtime) {}
   RModel(std::string function_name) : RModel_Base(function_name) {}
   RModel(RModel &&other) = default;
   RModel &operator=(RModel &&other) = default;
   RModel(const RModel &other) = delete;
   RModel &operator=(const RModel &other) = delete;
   ~RModel() = default;

   int Verbose() const { return fVerbose; }

   const std::vector<size_t> &GetTensorShape(std::string name) const;
   std::vector<Dim> GetDynamicTensorShape(std::string name) const;
   const ETensorType &GetTensorType(std::string name) const;

   bool CheckIfTensorAlreadyExist(std::string tensor_name);
   void AddInputTensorInfo(std::string input_name, ETensorType type, std::vector<Dim> shape);
   void AddInputTensorInfo(std::string input_name, ETensorType type, std::vector<size_t> shape);
   void AddOperator(std::unique_ptr<ROperator> op, int order_execution = -1);
   void AddOperatorReference(ROperator *op, int order_execution = -1)
   {
      std::unique_ptr<ROperator> tmp(op);
      AddOperator(std::move(tmp), order_execution);
   }
   void AddInitializedTensor(std::string tensor_name, ETensorType type, std::vector<std::size_t> shape,
                             std::shared_ptr<void> data);
   void AddConstantTensor(std::string tensor_name, ETensorType type, std::vector<std::size_t> shape,
                          std::shared_ptr<void> data);
   template <typename T>
   void AddInitializedTensor(const std::string &tensor_name, const std::vector<std::size_t> &shape, const T *raw_data)
   {
      size_t size = ConvertShapeToLength(shape);
      std::shared_ptr<void> data(malloc(size * sizeof(T) + 1), free);
      std::memcpy(data.get(), raw_data, size * sizeof(T));
      AddInitializedTensor(tensor_name, GetTemplatedType(T()), shape, data);
   }
   void SetNotWritableInitializedTensor(const std::string &tensor_name);
   bool IsInitializedTensor(const std::string &name) const;
   bool IsConstantTensor(const std::string &name) const;
   bool IsDynamicTensor(const std::string &) const { return false; } // shapes are fixed at Generate()
   bool IsDimInputTensor(const std::string &name) const;
   bool IsReadyInputTensor(const std::string &name) const;

   void AddIntermediateTensor(std::string tensor_name, ETensorType type, std::vector<Dim> dim_shape);
   void AddIntermediateTensor(std::string tensor_name, ETensorType type, std::vector<std::size_t> shape);
   void AddInputTensorName(std::string name);
   void AddOutputTensorNameList(std::vector<std::string> output_tensor_names);
   void UpdateOutputTensorList(std::vector<std::string> curr_output_tensor, std::vector<std::string> modify_output_tensor);
   void UpdateInitializedTensor(std::string tensor_name, ETensorType type, std::vector<std::size_t> shape,
                                std::shared_ptr<void> data);
   std::shared_ptr<void> GetInitializedTensorData(std::string tensor_name);

   void Initialize(int batchSize = -1, bool verbose = false);
   void Generate(std::underlying_type_t<Options> options, int batchSize = -1, long pos = 0, bool verbose = false);
   void Generate(Options options = Options::kDefault, int batchSize = -1, int pos = 0, bool verbose = false)
   {
      Generate(static_cast<std::underlying_type_t<Options>>(options), batchSize, pos, verbose);
   }
   std::string GenerateInferSignature(bool isdecl = true);

   const std::vector<std::string> &GetInputTensorNames() const { return fInputTensorNames; }
   const std::vector<std::string> &GetOutputTensorNames() const { return fOutputTensorNames; }

   long WriteInitializedTensorsToFile(std::string filename = "");
   void OutputGenerated(std::string filename = "", bool append = false);
   void PrintRequiredInputTensors();
   void PrintInitializedTensors();
   void PrintIntermediateTensors();
   void PrintOutputTensors();
   void PrintDynamicTensors() {}
   void HeadInitializedTensors(std::string name, int n_print = 50);
   bool UseSession() const { return fUseSession; }
   bool RunTimeBatch() const { return fDynamicBatch; } // the batch is a parameter of the emitted Session

   // ---- device plan interface used by the operators ----
   ELayout GetTensorLayout(const std::string &name) const;
   void SetTensorLayout(const std::string &name, ELayout layout) { fLayouts[name] = layout; }
   void AddAlias(const std::string &alias, const std::string &owner) { fAliases[alias] = owner; }
   std::string ResolveAlias(std::string name) const;
   // operators that read `name` (not fused away), in execution order
   std::vector<ROperator *> Consumers(const std::string &name) const;
   bool IsModelOutput(const std::string &name) const;
   // true when every consumer chain of a rank-4 tensor can read it in NHWC
   bool CanStayNHWC(const std::string &name, int depth = 0) const;
   // marks an initialised tensor as needed on the device (uploaded by the Session constructor)
   void UseOnDevice(const std::string &weight) { fDeviceWeights.insert(weight); }
   // a persistent device buffer that GenerateInitCode of an operator fills
   void AddDeviceBuffer(const std::string &name, ETensorType type, size_t length) { fDeviceBuffers[name] = {type, length}; }
   const InitializedTensor &GetInitializedTensor(const std::string &name) const;
   size_t ArenaBytes() const { return fArenaBytes; }

protected:
   void PlanDevice();
   void PlanSlices();
   void PlanArena();
   void GenerateSessionCode();
   void GenerateSessionMembers();
   void GenerateConstructor();
   void GenerateInfer();
   void GenerateWeightReader();
};

} // namespace SOFIE

#endif
