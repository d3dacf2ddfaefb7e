// RModel: tensor registries, device plan and emission of the Session.
// Public behaviour follows the reference (src/SOFIE_core/src/RModel.cxx); see RModel.hxx for what
// the emitted Session looks like on the CUDA path.
#include "SOFIE/RModel.hxx"

#include <algorithm>
#include <cctype>
#include <fstream>
#include <iomanip>
#include <iostream>
#include <limits>
#include <set>

#include "SOFIE/Emit.hxx"
#include "sofie_cuda.h" // sofie_mlp_smem_bytes: host arithmetic only, nothing of the library is linked
#include "SOFIE/ROperator_BatchNormalization.hxx"
#include "SOFIE/ROperator_Conv.hxx"
#include "SOFIE/ROperator_Fp8.hxx"
#include "SOFIE/ROperator_Gemm.hxx"
#include "SOFIE/ROperator_Pool.hxx"
#include "SOFIE/ROperator_QLinear.hxx"
#include "SOFIE/ROperator_Relu.hxx"
#include "SOFIE/ROperator_Reshape.hxx"

namespace SOFIE {

// ---------------------------------------------------------------------------------- registries
const std::vector<size_t> &RModel::GetTensorShape(std::string name) const
{
   auto f = fReadyInputTensorInfos.find(name);
   if (f != fReadyInputTensorInfos.end()) return f->second.shape;
   auto f2 = fInitializedTensors.find(name);
   if (f2 != fInitializedTensors.end()) return f2->second.shape();
   auto f3 = fIntermediateTensorInfos.find(name);
   if (f3 != fIntermediateTensorInfos.end()) return f3->second.shape;
   if (fInputTensorInfos.count(name))
      throw std::runtime_error("SOFIE tensor [" + name + "] is an input tensor with unspecified dimension parameter");
   throw std::runtime_error("SOFIE tensor [" + name + "] for which the shape is requested is not found");
}

std::vector<Dim> RModel::GetDynamicTensorShape(std::string name) const
{
   auto f = fInputTensorInfos.find(name);
   if (f != fInputTensorInfos.end()) return f->second.shape;
   return ConvertShapeToDim(GetTensorShape(name));
}

const ETensorType &RModel::GetTensorType(std::string name) const
{
   auto f = fReadyInputTensorInfos.find(name);
   if (f != fReadyInputTensorInfos.end()) return f->second.type;
   auto f2 = fInitializedTensors.find(name);
   if (f2 != fInitializedTensors.end()) return f2->second.type();
   auto f3 = fInputTensorInfos.find(name);
   if (f3 != fInputTensorInfos.end()) return f3->second.type;
   auto f4 = fIntermediateTensorInfos.find(name);
   if (f4 != fIntermediateTensorInfos.end()) return f4->second.type;
   throw std::runtime_error("SOFIE tensor [" + name + "] for which the type is requested is not found");
}

bool RModel::CheckIfTensorAlreadyExist(std::string name)
{
   return fReadyInputTensorInfos.count(name) || fInitializedTensors.count(name) || fIntermediateTensorInfos.count(name) ||
          fInputTensorInfos.count(name);
}

void RModel::AddInputTensorInfo(std::string input_name, ETensorType type, std::vector<Dim> shape)
{
   input_name = UTILITY::Clean_name(input_name);
   if (CheckIfTensorAlreadyExist(input_name))
      throw std::runtime_error("SOFIE input tensor with name " + input_name + " already exists \n");
   fInputTensorInfos[input_name] = InputTensorInfo{type, shape};
}

void RModel::AddInputTensorInfo(std::string input_name, ETensorType type, std::vector<size_t> shape)
{
   input_name = UTILITY::Clean_name(input_name);
   if (CheckIfTensorAlreadyExist(input_name))
      throw std::runtime_error("SOFIE input tensor with name " + input_name + " already exists \n");
   fReadyInputTensorInfos[input_name] = TensorInfo{type, shape};
}

void RModel::AddInputTensorName(std::string name) { fInputTensorNames.emplace_back(UTILITY::Clean_name(name)); }

void RModel::AddOperator(std::unique_ptr<ROperator> op, int order_execution)
{
   AddBlasRoutines(op->GetBlasRoutines());
   for (auto &lib : op->GetStdLibs()) AddNeededStdLib(lib);
   if (order_execution >= 0 && (size_t)order_execution <= fOperators.size())
      fOperators.insert(fOperators.begin() + order_execution, std::move(op));
   else
      fOperators.push_back(std::move(op));
}

void RModel::AddInitializedTensor(std::string tensor_name, ETensorType type, std::vector<std::size_t> shape,
                                  std::shared_ptr<void> data)
{
   tensor_name = UTILITY::Clean_name(tensor_name);
   if (CheckIfTensorAlreadyExist(tensor_name))
      throw std::runtime_error("SOFIE initialized tensor with name " + tensor_name + " already exists \n");
   fInitializedTensors[tensor_name] = InitializedTensor{type, shape, data};
}

void RModel::AddConstantTensor(std::string tensor_name, ETensorType type, std::vector<std::size_t> shape,
                               std::shared_ptr<void> data)
{
   tensor_name = UTILITY::Clean_name(tensor_name);
   if (CheckIfTensorAlreadyExist(tensor_name))
      throw std::runtime_error("SOFIE initialized tensor with name " + tensor_name + " already exists \n");
   fInitializedTensors[tensor_name] = InitializedTensor{type, shape, data, true};
}

void RModel::SetNotWritableInitializedTensor(const std::string &tensor_name)
{
   auto t = fInitializedTensors.find(tensor_name);
   if (t == fInitializedTensors.end()) throw std::runtime_error("SOFIE initialized tensor " + tensor_name + " not found");
   t->second.SetNotWritable();
}

bool RModel::IsInitializedTensor(const std::string &name) const { return fInitializedTensors.count(UTILITY::Clean_name(name)); }
bool RModel::IsConstantTensor(const std::string &name) const
{
   auto it = fInitializedTensors.find(UTILITY::Clean_name(name));
   return it != fInitializedTensors.end() && it->second.IsConstantTensor();
}
bool RModel::IsDimInputTensor(const std::string &name) const { return fInputTensorInfos.count(UTILITY::Clean_name(name)); }
bool RModel::IsReadyInputTensor(const std::string &name) const { return fReadyInputTensorInfos.count(UTILITY::Clean_name(name)); }

void RModel::AddIntermediateTensor(std::string tensor_name, ETensorType type, std::vector<Dim> dim_shape)
{
   auto int_shape = ConvertShapeToInt(dim_shape);
   if (int_shape.empty() && !dim_shape.empty())
      throw std::runtime_error("SOFIE intermediate tensor " + tensor_name + " has a parametric shape; shapes are fixed at Generate()");
   AddIntermediateTensor(tensor_name, type, int_shape);
}

void RModel::AddIntermediateTensor(std::string tensor_name, ETensorType type, std::vector<std::size_t> shape)
{
   tensor_name = UTILITY::Clean_name(tensor_name);
   if (CheckIfTensorAlreadyExist(tensor_name))
      throw std::runtime_error("SOFIE intermediate tensor with name " + tensor_name + " already exists \n");
   fIntermediateTensorInfos[tensor_name] = TensorInfo{type, shape};
}

void RModel::AddOutputTensorNameList(std::vector<std::string> names)
{
   fOutputTensorNames.clear();
   for (auto &n : names) fOutputTensorNames.emplace_back(UTILITY::Clean_name(n));
}

void RModel::UpdateOutputTensorList(std::vector<std::string> curr, std::vector<std::string> modify)
{
   for (size_t i = 0; i < curr.size(); ++i) {
      auto it = std::find(fOutputTensorNames.begin(), fOutputTensorNames.end(), UTILITY::Clean_name(curr[i]));
      if (it != fOutputTensorNames.end()) *it = UTILITY::Clean_name(modify[i]);
   }
}

void RModel::UpdateInitializedTensor(std::string tensor_name, ETensorType type, std::vector<std::size_t> shape,
                                     std::shared_ptr<void> data)
{
   tensor_name = UTILITY::Clean_name(tensor_name);
   if (!fInitializedTensors.count(tensor_name))
      throw std::runtime_error("SOFIE tensor " + tensor_name + " not found when trying to update it");
   fInitializedTensors[tensor_name] = InitializedTensor{type, shape, data};
}

std::shared_ptr<void> RModel::GetInitializedTensorData(std::string tensor_name)
{
   auto f = fInitializedTensors.find(tensor_name);
   if (f == fInitializedTensors.end())
      throw std::runtime_error("SOFIE tensor " + tensor_name + " not found when trying to get its data");
   return f->second.sharedptr();
}

const InitializedTensor &RModel::GetInitializedTensor(const std::string &name) const
{
   auto f = fInitializedTensors.find(name);
   if (f == fInitializedTensors.end()) throw std::runtime_error("SOFIE initialized tensor " + name + " not found");
   return f->second;
}

// ---------------------------------------------------------------------------------- device plan helpers
ELayout RModel::GetTensorLayout(const std::string &name) const
{
   auto it = fLayouts.find(name);
   return it == fLayouts.end() ? ELayout::NCHW : it->second;
}

std::string RModel::ResolveAlias(std::string name) const
{
   for (int depth = 0; depth < 64; depth++) {
      auto it = fAliases.find(name);
      if (it == fAliases.end()) return name;
      name = it->second;
   }
   throw std::runtime_error("SOFIE alias chain of tensor " + name + " does not end");
}

std::vector<ROperator *> RModel::Consumers(const std::string &name) const
{
   std::vector<ROperator *> out;
   for (auto &op : fOperators) {
      if (op->IsFusedAway()) continue;
      for (auto &in : op->GetOpInputTensors())
         if (in == name) {
            out.push_back(op.get());
            break;
         }
   }
   return out;
}

bool RModel::IsModelOutput(const std::string &name) const
{
   return std::find(fOutputTensorNames.begin(), fOutputTensorNames.end(), name) != fOutputTensorNames.end();
}

bool RModel::CanStayNHWC(const std::string &name, int depth) const
{
   if (depth > 16 || IsModelOutput(name)) return false;
   auto shape = GetTensorShape(name);
   if (shape.size() != 4) return false;
   auto consumers = Consumers(name);
   if (consumers.empty()) return false;
   for (ROperator *op : consumers) {
      if (!op->AcceptsNHWC(name)) return false;
      switch (op->Kind()) {
      case EOpKind::Conv:
      case EOpKind::QLinearConv: break;
      case EOpKind::Relu:
      case EOpKind::Pool:
      case EOpKind::Eltwise:
         if (!CanStayNHWC(op->GetOpOutputTensors()[0], depth + 1)) return false;
         break;
      case EOpKind::Reshape: {
         // Flatten: every reader of the flattened tensor must be a matmul with a constant weight
         const std::string &flat = op->GetOpOutputTensors()[0];
         if (IsModelOutput(flat)) return false;
         auto readers = Consumers(flat);
         if (readers.empty()) return false;
         for (ROperator *r : readers) {
            if ((r->Kind() != EOpKind::Gemm && r->Kind() != EOpKind::QLinearMatMul) || !r->AcceptsNHWC(flat)) return false;
            if (r->GetOpInputTensors().size() < 2 || !IsInitializedTensor(r->GetOpInputTensors()[1])) return false;
         }
         break;
      }
      default: return false;
      }
   }
   return true;
}

// ---------------------------------------------------------------------------------- Initialize
void RModel::Initialize(int batchSize, bool verbose)
{
   fVerbose = int(verbose);
   fBatchSize = batchSize;
   fIntermediateTensorInfos.clear();
   fLayouts.clear();
   fAliases.clear();
   fArenaOffsets.clear();
   fDeviceWeights.clear();
   fDeviceBuffers.clear();
   if (fIsInitialized) throw std::runtime_error("SOFIE: an RModel can be initialized (generated) only once");

   // shapes are fixed at generation time: parametric input dimensions take batchSize when given,
   // else their default value, else 1 (the reference substitutes batch parameters the same way,
   // src/SOFIE_core/src/RModel.cxx:399-440, and can leave others dynamic)
   // Without a batch size the parameter stays a run-time value when it is the first dimension of every parametric
   // input and the only parameter (what exporters write for a dynamic batch axis); any other parametric shape is
   // fixed to its default as before.
   fDynamicBatch = false;
   if (batchSize <= 0 && !fInputTensorInfos.empty()) {
      bool ok = true;
      std::string param;
      for (auto &input : fInputTensorInfos)
         for (size_t i = 0; i < input.second.shape.size(); i++) {
            const Dim &d = input.second.shape[i];
            if (!d.isParam) continue;
            if (i != 0 || (!param.empty() && param != d.param)) ok = false;
            param = d.param;
         }
      // every input must carry it: a fully specified input next to a batched one cannot be scaled
      if (ok && !param.empty() && fReadyInputTensorInfos.empty()) {
         fDynamicBatch = true;
         fBatchParam = param;
      }
   }
   for (auto &input : fInputTensorInfos) {
      std::vector<size_t> shape;
      for (auto &d : input.second.shape) {
         if (d.isParam) {
            size_t v = batchSize > 0 ? (size_t)batchSize : ((d.dim && d.dim != static_cast<size_t>(-1)) ? d.dim : 1);
            fShapeParams[d.param] = std::to_string(v);   // the constructor's default for the parameter
            shape.push_back(fDynamicBatch ? kBatchSentinel : v);
         } else {
            shape.push_back(d.dim);
         }
      }
      fReadyInputTensorInfos[input.first] = TensorInfo{input.second.type, shape};
      if (verbose) std::cout << "SOFIE: input " << input.first << " fixed to shape " << ConvertShapeToString(shape) << std::endl;
   }
   fInputTensorInfos.clear();
   if (fInputTensorNames.empty())
      for (auto &i : fReadyInputTensorInfos) fInputTensorNames.push_back(i.first);

   for (auto &op : fOperators) {
      if (verbose) std::cout << "Initializing operator " << typeid(*op).name() << std::endl;
      op->Initialize(*this);
   }
   PlanDevice();
   PlanSlices();
   PlanArena();
   fIsInitialized = true;
}

// Step 1-3 of the device plan: fusion, then layouts and weight preparation operator by operator.
void RModel::PlanDevice()
{
   auto single_consumer = [&](const std::string &t) -> ROperator * {
      if (IsModelOutput(t)) return nullptr;
      auto c = Consumers(t);
      return c.size() == 1 ? c[0] : nullptr;
   };
   for (auto &opp : fOperators) {
      ROperator *op = opp.get();
      if (op->IsFusedAway()) continue;
      if (op->Kind() == EOpKind::Conv || op->Kind() == EOpKind::QLinearConv) {
         auto *fconv = dynamic_cast<ROperator_Conv<float> *>(op);
         auto *qconv = dynamic_cast<ROperator_QLinearConv *>(op);
         std::string out = fconv ? fconv->OutputName() : qconv->OutputName();
         bool relu_done = false;
         if (fconv)
            if (ROperator *next = single_consumer(out))
               if (auto *bn = dynamic_cast<ROperator_BatchNormalization<float> *>(next)) {
                  // inference BatchNormalization behind a convolution: folded into its weights and bias
                  fconv->FoldBatchNorm(*this, bn->ScaleName(), bn->BiasName(), bn->MeanName(), bn->VarName(), bn->Epsilon(), bn->HasRelu(),
                                       bn->OutputName());
                  bn->SetFusedAway();
                  out = bn->OutputName();
                  relu_done = bn->HasRelu();
               }
         if (ROperator *next = relu_done ? nullptr : single_consumer(out)) {
            if (auto *relu = dynamic_cast<ROperator_Relu<float> *>(next)) {
               fconv ? fconv->FuseRelu(relu->OutputName()) : qconv->FuseRelu(relu->OutputName());
               relu->SetFusedAway();
               out = relu->OutputName();
            }
         }
         if (ROperator *next = single_consumer(out)) {
            auto *pool = dynamic_cast<ROperator_Pool<float> *>(next);
            if (pool && pool->IsMax2x2Stride2()) {
               fconv ? fconv->FusePool2x2(pool->OutputName()) : qconv->FusePool2x2(pool->OutputName());
               pool->SetFusedAway();
            }
         }
      } else if (op->Kind() == EOpKind::Gemm) {
         auto *gemm = dynamic_cast<ROperator_Gemm<float> *>(op);
         if (ROperator *next = gemm ? single_consumer(gemm->OutputName()) : nullptr)
            if (auto *relu = dynamic_cast<ROperator_Relu<float> *>(next)) {
               gemm->SetActivation(EActivationType::RELU);
               gemm->SetOutputName(relu->OutputName());
               relu->SetFusedAway();
            }
      } else if (op->Kind() == EOpKind::Fp8Gemm) {
         // the bfloat16 result of the last FP8 layer, read only by a Cast to float: one launch writes the float tensor
         auto *g = dynamic_cast<ROperator_Fp8Gemm *>(op);
         if (ROperator *next = (g && g->WritesBf16()) ? single_consumer(g->OutputName()) : nullptr)
            if (auto *cast = dynamic_cast<ROperator_Cast *>(next))
               if (cast->IsBf16ToFloat()) {
                  g->FuseCastToFloat(cast->OutputName());
                  cast->SetFusedAway();
               }
      } else if (op->Kind() == EOpKind::QLinearMatMul) {
         auto *qmm = dynamic_cast<ROperator_QLinearMatMul *>(op);
         if (ROperator *next = qmm ? single_consumer(qmm->OutputName()) : nullptr)
            if (auto *relu = dynamic_cast<ROperator_Relu<float> *>(next)) {
               qmm->FuseRelu(relu->OutputName());
               relu->SetFusedAway();
            }
         // the uint8 product read only by a DequantizeLinear with the same zero point: one launch writes the floats
         if (ROperator *next = qmm ? single_consumer(qmm->OutputName()) : nullptr)
            if (auto *dq = dynamic_cast<ROperator_DequantizeLinear *>(next))
               if (dq->ZeroPoint() == qmm->OutputZeroPoint()) {
                  qmm->FuseDequantize(dq->OutputName(), dq->Scale());
                  dq->SetFusedAway();
               }
      }
   }
   for (auto &op : fOperators)
      if (!op->IsFusedAway()) op->PlanDevice(*this);
   // Chains of small Gemm layers, each read only by the next: one fused launch (the layers keep their weights
   // in shared memory and the activations never leave the SM). Needs what PlanDevice prepared.
   for (auto &opp : fOperators) {
      auto *head = dynamic_cast<ROperator_Gemm<float> *>(opp.get());
      if (!head || head->IsFusedAway() || !head->MlpFusable()) continue;
      std::vector<ROperator_Gemm<float> *> tail;
      // the library's own arithmetic decides whether the layers' weights fit in shared memory
      sofie_mlp_desc d = {};
      d.layers = 1;
      d.dims[0] = static_cast<int32_t>(head->WidthIn());
      d.dims[1] = static_cast<int32_t>(head->WidthOut());
      ROperator_Gemm<float> *last = head;
      while (d.layers < SOFIE_MLP_MAX_LAYERS) {
         ROperator *next = single_consumer(last->OutputName());
         auto *g = dynamic_cast<ROperator_Gemm<float> *>(next);
         if (!g || g->IsFusedAway() || g->InputName() != last->OutputName() || !g->MlpFusable() || g->Rows() != head->Rows()) break;
         d.dims[d.layers + 1] = static_cast<int32_t>(g->WidthOut());
         d.layers++;
         if (sofie_mlp_smem_bytes(&d) > SOFIE_MLP_MAX_SMEM) break;
         tail.push_back(g);
         last = g;
      }
      if (tail.empty()) continue;
      head->AbsorbChain(tail);
      for (auto *g : tail) g->SetFusedAway();
   }
}

// Step 4: which operators run once per uploaded part of the input.
void RModel::PlanSlices()
{
   // Pipelined input upload: when the model has one large input and its leading operators treat the samples of a
   // batch independently, the input is copied in fUploadParts parts on the copy stream and those operators are
   // launched once per part as soon as the part has arrived (slice `part` of every tensor they read and write);
   // the operators behind the first one that cannot be sliced are the captured graph and run when all parts are done.
   // Every copy carries about 10 us of fixed cost on top of its bytes at ~55 GB/s, so splitting only pays when a part
   // is several megabytes: measured on B200, a 3 MB input in four parts is 12% slower end to end than in one piece.
   // What is left after the last copy is one part's share of the kernels: eight parts from 128 MB on, four below.
   fSlicedOps.clear();
   fUploadParts = 4;
   size_t head = fOperators.size();
   for (size_t i = 0; i < fOperators.size(); i++)
      if (!fOperators[i]->IsFusedAway()) {
         head = i;
         break;
      }
   if (head >= fOperators.size() || fInputTensorNames.size() != 1 || fNeverPipelinedUpload || fDynamicBatch) return;
   const std::string &in = fInputTensorNames[0];
   const size_t inBytes = ConvertShapeToLength(GetTensorShape(in)) * GetTypeSize(GetTensorType(in));
   if (inBytes < (fForcePipelinedUpload ? 0 : size_t(32) << 20)) return;
   auto prefix = [&](size_t parts) {
      std::vector<size_t> sliced;
      // every slice of a tensor starts on a 256-byte boundary, like the tensor itself
      auto slices = [&](const std::string &n) {
         return (ConvertShapeToLength(GetTensorShape(n)) * GetTypeSize(GetTensorType(n))) % (parts * 256) == 0;
      };
      if (!slices(in)) return sliced;
      std::set<std::string> parted{in}; // tensors that come into being slice by slice
      for (size_t i = head; i < fOperators.size(); i++) {
         auto &op = fOperators[i];
         if (op->IsFusedAway()) continue;
         bool ok = op->CanSliceBatch(parts);
         size_t batchInputs = 0;
         for (auto &n : op->GetOpInputTensors()) {
            if (IsInitializedTensor(n)) continue; // constants are read whole by every slice
            ok = ok && parted.count(n) != 0 && slices(n);
            batchInputs++;
         }
         ok = ok && batchInputs > 0;
         for (auto &w : op->GetOpOutputTensors()) ok = ok && slices(w);
         if (!ok) break;
         for (auto &w : op->GetOpOutputTensors()) parted.insert(w);
         sliced.push_back(i);
      }
      // the first sliced operator has to be the one that reads the input: otherwise nothing overlaps the copy
      if (!sliced.empty()) {
         bool readsInput = false;
         for (auto &n : fOperators[sliced[0]]->GetOpInputTensors()) readsInput = readsInput || n == in;
         if (!readsInput) sliced.clear();
      }
      return sliced;
   };
   fSlicedOps = prefix(4);
   if (inBytes >= (size_t(128) << 20)) {
      std::vector<size_t> eight = prefix(8);
      if (!eight.empty() && eight.size() >= fSlicedOps.size()) {
         fSlicedOps = eight;
         fUploadParts = 8;
      }
   }
}

// Step 5: liveness-based first-fit placement in one arena (256-byte aligned slices).
void RModel::PlanArena()
{
   struct Slot {
      std::string name;
      size_t bytes;
      int first, last;
      size_t offset;
   };
   const int nOps = (int)fOperators.size();
   std::vector<Slot> slots;
   auto bytes_of = [&](const std::string &n) {
      size_t b = ConvertShapeToLength(GetTensorShape(n)) * GetTypeSize(GetTensorType(n));
      if (fDynamicBatch) {
         // slices scale with the batch: the bytes of ONE sample are rounded to 256, so that every offset is a multiple of
         // 256 for every batch
         if (b % kBatchSentinel != 0)
            throw std::runtime_error("SOFIE: tensor " + n + " does not scale with the batch parameter " + fBatchParam +
                                     "; generate this model with a fixed batch size");
         return kBatchSentinel * ((std::max<size_t>(b / kBatchSentinel, 1) + 255) & ~size_t(255));
      }
      return (std::max<size_t>(b, 1) + 255) & ~size_t(255);
   };
   for (auto &in : fInputTensorNames) slots.push_back({in, bytes_of(in), -1, -1, 0});
   for (int i = 0; i < nOps; i++) {
      if (fOperators[i]->IsFusedAway()) continue;
      for (auto &out : fOperators[i]->GetOpOutputTensors())
         if (!fAliases.count(out)) slots.push_back({out, bytes_of(out), i, i, 0});
   }
   auto slot_of = [&](const std::string &n) -> Slot * {
      std::string owner = ResolveAlias(n);
      for (auto &s : slots)
         if (s.name == owner) return &s;
      return nullptr;
   };
   for (int i = 0; i < nOps; i++) {
      if (fOperators[i]->IsFusedAway()) continue;
      for (auto &in : fOperators[i]->GetOpInputTensors())
         if (Slot *s = slot_of(in)) s->last = std::max(s->last, i);
   }
   for (auto &o : fOutputTensorNames) {
      Slot *s = slot_of(o);
      if (!s) throw std::runtime_error("SOFIE: output tensor " + o + " is not produced by any operator");
      s->last = nOps;
   }
   // Operators launched per uploaded part run part after part: slice 1 of their first tensor is written after slice 0 of
   // their last one (and the input's later parts arrive meanwhile), so everything they touch is alive together.
   if (!fSlicedOps.empty()) {
      const int lo = (int)fSlicedOps.front(), hi = (int)fSlicedOps.back();
      auto together = [&](const std::string &n) {
         if (Slot *s = slot_of(n)) {
            s->first = std::min(s->first, lo);
            s->last = std::max(s->last, hi);
         }
      };
      for (auto &in : fInputTensorNames) together(in);
      for (size_t i : fSlicedOps)
         for (auto &out : fOperators[i]->GetOpOutputTensors()) together(out);
   }
   fArenaBytes = 0;
   for (size_t i = 0; i < slots.size(); i++) {
      // lowest offset that does not overlap an already placed slot alive at the same time
      size_t off = 0;
      bool moved = true;
      while (moved) {
         moved = false;
         for (size_t j = 0; j < i; j++) {
            const Slot &p = slots[j];
            bool time_overlap = !(p.last < slots[i].first || slots[i].last < p.first);
            bool space_overlap = off < p.offset + p.bytes && p.offset < off + slots[i].bytes;
            if (time_overlap && space_overlap) {
               off = p.offset + p.bytes;
               moved = true;
            }
         }
      }
      slots[i].offset = off;
      fArenaOffsets[slots[i].name] = off;
      fArenaBytes = std::max(fArenaBytes, off + slots[i].bytes);
   }
}

// ---------------------------------------------------------------------------------- Generate
std::string RModel::GenerateInferSignature(bool isdecl)
{
   std::string s;
   if (fDynamicBatch) s += std::string(isdecl ? "size_t " : "") + fBatchParam + ",";   // reference: RModel.cxx:688-702
   for (auto &name : fInputTensorNames) {
      if (isdecl) {
         std::string type = ConvertTypeToString(GetTensorType(name));
         if (type == "other") throw std::runtime_error("SOFIE: input tensor " + name + " is of a data type which is not yet supported.");
         s += type + "* ";
      }
      s += "tensor_" + name + ",";
   }
   if (!fInputTensorNames.empty()) s.pop_back();
   return s;
}

void RModel::Generate(std::underlying_type_t<Options> options, int batchSize, long pos, bool verbose)
{
   fVerbose = verbose;
   fBatchSize = batchSize;
   fReadPos = pos;
   auto has = [&](Options o) { return (static_cast<std::underlying_type_t<Options>>(o) & options) != 0; };
   if (has(Options::kNoSession))
      throw std::runtime_error("SOFIE: kNoSession is not available on the CUDA path: the Session owns the device context");
   if (has(Options::kRootBinaryWeightFile))
      throw std::runtime_error("SOFIE: ROOT binary weight files need ROOT I/O, which this build does not have");
   if (has(Options::kGNN) || has(Options::kGNNComponent))
      throw std::runtime_error("SOFIE: GNN models are outside the CUDA dense-contraction path");
   if (has(Options::kNoWeightFile)) {
      fUseWeightFile = false;
      fWeightFile = WeightFileType::None;
   } else if (has(Options::kBinaryWeightFile)) {
      fWeightFile = WeightFileType::Binary;
   }
   fForcePipelinedUpload = has(Options::kPipelinedUpload);
   fNeverPipelinedUpload = has(Options::kSingleUpload);
   Initialize(batchSize, verbose);
   std::string hgname;
   fGC.clear();
   GenerateHeaderInfo(hgname);
   GenerateSessionCode();
   if (fDynamicBatch) MakeBatchSymbolic();
   fGC += ("} //SOFIE_" + fName + "\n");
   fGC += "\n#endif  // " + hgname + "\n";
}

// Rewrites every integer literal of the emitted Session that is a non-zero multiple of the batch sentinel as
// `<multiple> * fBatch` (inside the braces of a descriptor, whose fields are 32-bit, with a cast). The sentinel is a
// prime above a million, so a number that does not scale with the batch is not a multiple of it.
void RModel::MakeBatchSymbolic()
{
   std::string out;
   out.reserve(fGC.size() + 1024);
   size_t line_start = 0;
   while (line_start < fGC.size()) {
      size_t line_end = fGC.find('\n', line_start);
      if (line_end == std::string::npos) line_end = fGC.size();
      const std::string line = fGC.substr(line_start, line_end - line_start);
      const bool in_desc = line.find("_desc ") != std::string::npos && line.find("= {") != std::string::npos;
      for (size_t i = 0; i < line.size();) {
         const char c = line[i];
         const bool starts_number = std::isdigit((unsigned char)c) && (i == 0 || !(std::isalnum((unsigned char)line[i - 1]) || line[i - 1] == '_' || line[i - 1] == '.'));
         if (!starts_number) {
            out += c;
            i++;
            continue;
         }
         size_t j = i;
         while (j < line.size() && std::isdigit((unsigned char)line[j])) j++;
         const bool plain = j == line.size() || !(std::isalnum((unsigned char)line[j]) || line[j] == '_' || line[j] == '.');
         const std::string digits = line.substr(i, j - i);
         unsigned long long v = 0;
         bool fits = digits.size() <= 18;
         if (fits) v = std::stoull(digits);
         if (plain && fits && v != 0 && v % kBatchSentinel == 0) {
            const std::string k = std::to_string(v / kBatchSentinel);
            out += in_desc ? "static_cast<int32_t>(" + k + " * fBatch)" : "(size_t(" + k + ") * fBatch)";
         } else {
            out += digits;
         }
         i = j;
      }
      if (line_end < fGC.size()) out += '\n';
      line_start = line_end + 1;
   }
   fGC.swap(out);
}

static std::string ByteCount(const std::vector<size_t> &shape, ETensorType t)
{
   return std::to_string(ConvertShapeToLength(shape) * GetTypeSize(t));
}

// results up to this size are written by the kernels straight into mapped host memory
static constexpr size_t kHostOutputMaxBytes = 64 * 1024;

void RModel::GenerateSessionMembers()
{
   fSessionMembers = {"fCtx", "fStream", "fGraphReady", "fUseGraph"};
   fGC += "sofie_cuda_ctx * fCtx = nullptr;   // device context: arena, uploaded weights, stream, captured graph\n";
   fGC += "void * fStream = nullptr;\n";
   fGC += "bool fGraphReady = false;\n";
   fGC += "bool fUseGraph = true;\n";
   if (fDynamicBatch) {
      fSessionMembers.push_back("fBatch");
      fSessionMembers.push_back("fMaxBatch");
      fGC += "size_t fBatch = 0;      // batch of the current / last infer(); the captured graph is the one of this batch\n";
      fGC += "size_t fMaxBatch = 0;   // the batch the Session was constructed for: the arena holds that many samples\n";
   }
   auto pointer = [this](ETensorType type, const std::string &name) {
      fGC += EMIT::CType(type) + " * " + EMIT::Dev(name) + " = nullptr;\n";
      fSessionMembers.push_back(EMIT::Dev(name));
   };
   fGC += "\n// device pointers: model inputs\n";
   for (auto &n : fInputTensorNames) pointer(GetTensorType(n), n);
   if (!fDeviceWeights.empty()) fGC += "// device pointers: weights uploaded by the constructor\n";
   for (auto &n : fDeviceWeights) pointer(GetTensorType(n), n);
   if (!fDeviceBuffers.empty()) fGC += "// device pointers: tables computed by the constructor\n";
   for (auto &b : fDeviceBuffers) pointer(b.second.type, b.first);
   fGC += "// device pointers: intermediate tensors, slices of one arena of " + std::to_string(fArenaBytes) + " bytes\n";
   for (auto &op : fOperators) {
      if (op->IsFusedAway()) continue;
      for (auto &out : op->GetOpOutputTensors()) pointer(GetTensorType(out), out);
   }
}

void RModel::GenerateWeightReader()
{
   if (fWeightFile == WeightFileType::Binary) {
      // one fread per tensor straight into the host copy; names, types and sizes are checked
      fGC += "   std::FILE * f = std::fopen(filename.c_str(), \"rb\");\n";
      fGC += "   if (!f) {\n";
      fGC += "      throw std::runtime_error(\"sofie failed to open file \" + filename + \" for input weights\");\n";
      fGC += "   }\n";
      fGC += "   struct Closer { std::FILE * f; ~Closer() { std::fclose(f); } } closer{f};\n";
      if (fReadPos > 0) fGC += "   std::fseek(f, " + std::to_string(fReadPos) + ", SEEK_SET);\n";
      fGC += "   char magic[8]; uint64_t count = 0;\n";
      fGC += "   if (std::fread(magic, 1, 8, f) != 8 || std::string(magic, 8) != \"SOFIEBW1\" || std::fread(&count, 8, 1, f) != 1 || count != " +
             std::to_string(fDeviceWeights.size()) + ") {\n";
      fGC += "      throw std::runtime_error(\"SOFIE: \" + filename + \" is not the binary weight file of this model\");\n";
      fGC += "   }\n";
      fGC += "   auto read_tensor = [&](const char * expected, uint32_t type, uint64_t length, void * dst, size_t bytes) {\n";
      fGC += "      uint32_t nlen = 0, t = 0; uint64_t len = 0, nbytes = 0; char name[512];\n";
      fGC += "      if (std::fread(&nlen, 4, 1, f) != 1 || nlen >= sizeof(name) || std::fread(name, 1, nlen, f) != nlen)\n";
      fGC += "         throw std::runtime_error(std::string(\"SOFIE failed to read the tensor name; expected name is \") + expected);\n";
      fGC += "      if (std::string(name, nlen) != expected)\n";
      fGC += "         throw std::runtime_error(std::string(\"SOFIE failed to read the correct tensor name; expected name is \") + expected + \" , read \" + std::string(name, nlen));\n";
      fGC += "      if (std::fread(&t, 4, 1, f) != 1 || std::fread(&len, 8, 1, f) != 1 || std::fread(&nbytes, 8, 1, f) != 1 || t != type || len != length || nbytes != bytes)\n";
      fGC += "         throw std::runtime_error(std::string(\"SOFIE failed to read the correct tensor size; expected size is \") + std::to_string(length) + \" for \" + expected);\n";
      fGC += "      if (std::fread(dst, 1, bytes, f) != bytes)\n";
      fGC += "         throw std::runtime_error(std::string(\"SOFIE failed to read the values for tensor \") + expected);\n";
      fGC += "      std::fseek(f, (long)((8 - (nlen + bytes) % 8) % 8), SEEK_CUR);\n";
      fGC += "   };\n";
      for (auto &n : fDeviceWeights) {
         const auto &t = fInitializedTensors.at(n);
         fGC += "   read_tensor(\"tensor_" + n + "\", " + std::to_string((int)t.type()) + ", " + std::to_string(t.length()) + ", " + EMIT::Host(n) +
                ".data(), " + std::to_string(t.length() * GetTypeSize(t.type())) + ");\n";
      }
      return;
   }
   // same text format as the reference writes and reads (src/SOFIE_core/src/RModel.cxx:970-1018,1121-1158):
   // "tensor_<name> <length>" followed by the values; integer tensors are written as integers
   fGC += "   std::ifstream f;\n";
   fGC += "   f.open(filename);\n";
   fGC += "   if (!f.is_open()) {\n";
   fGC += "      throw std::runtime_error(\"sofie failed to open file \" + filename + \" for input weights\");\n";
   fGC += "   }\n";
   if (fReadPos > 0) fGC += "   f.seekg(" + std::to_string(fReadPos) + ");\n";
   fGC += "   std::string tensor_name;\n";
   fGC += "   size_t length;\n";
   for (auto &n : fDeviceWeights) {
      const auto &t = fInitializedTensors.at(n);
      std::string tname = "tensor_" + n, len = std::to_string(t.length());
      fGC += "   f >> tensor_name >> length;\n";
      fGC += "   if (tensor_name != \"" + tname + "\" ) {\n";
      fGC += "      std::string err_msg = \"SOFIE failed to read the correct tensor name; expected name is " + tname + " , read \" + tensor_name;\n";
      fGC += "      throw std::runtime_error(err_msg);\n";
      fGC += "    }\n";
      fGC += "   if (length != " + len + ") {\n";
      fGC += "      std::string err_msg = \"SOFIE failed to read the correct tensor size; expected size is " + len + " , read \" + std::to_string(length) ;\n";
      fGC += "      throw std::runtime_error(err_msg);\n";
      fGC += "    }\n";
      if (t.type() == ETensorType::INT8 || t.type() == ETensorType::UINT8 || t.type() == ETensorType::FLOAT8E4M3FN)
         fGC += "   for (size_t i = 0; i < length; ++i) { int v; f >> v; " + EMIT::Host(n) + "[i] = static_cast<" + EMIT::CType(t.type()) + ">(v); }\n";
      else
         fGC += "   for (size_t i = 0; i < length; ++i)\n      f >> " + EMIT::Host(n) + "[i];\n";
      fGC += "   if (f.fail()) {\n";
      fGC += "      throw std::runtime_error(\"SOFIE failed to read the values for tensor " + tname + "\");\n";
      fGC += "   }\n";
   }
   fGC += "   f.close();\n";
}

void RModel::GenerateConstructor()
{
   if (fUseWeightFile) fGC += "Session(std::string filename =\"" + fName + (fWeightFile == WeightFileType::Binary ? ".bin" : ".dat") + "\"";
   else fGC += "Session(std::string = \"\"";
   for (auto &p : fShapeParams) fGC += ",\n        size_t " + p.first + " = " + p.second;
   fGC += ") {\n";
   if (fDynamicBatch) {
      fGC += "   if (" + fBatchParam + " == 0) throw std::runtime_error(\"SOFIE: a Session needs room for at least one sample\");\n";
      fGC += "   fBatch = fMaxBatch = " + fBatchParam + ";\n";
   } else {
      for (auto &p : fShapeParams)
         fGC += "   if (" + p.first + " != " + p.second + ") throw std::runtime_error(\"SOFIE: this Session was generated for " + p.first +
                " = " + p.second + "\");\n";
   }
   fGC += "   if (const char * g = std::getenv(\"SOFIE_CUDA_GRAPH\")) fUseGraph = (g[0] != '0');\n";
   fGC += "   Check(sofie_cuda_ctx_create(&fCtx, -1, " + std::to_string(fArenaBytes) + "), \"sofie_cuda_ctx_create\");\n";
   fGC += "   try {\n";
   fGC += "   Check(sofie_cuda_ctx_stream(fCtx, &fStream), \"sofie_cuda_ctx_stream\");\n";
   fGC += "   //--- arena slices of the inputs and intermediate tensors\n";
   for (auto &slot : fArenaOffsets) {
      const std::string &n = slot.first;
      // A small model output that no operator reads lives in mapped host memory: the last kernel writes it across
      // PCIe and infer() only waits for the stream instead of issuing a device-to-host copy.
      const size_t nbytes = ConvertShapeToLength(GetTensorShape(n)) * GetTypeSize(GetTensorType(n));
      bool aliased = false;
      for (auto &a : fAliases) aliased = aliased || a.first == n || ResolveAlias(a.first) == n;
      if (IsModelOutput(n) && Consumers(n).empty() && !aliased && nbytes > 0 && nbytes <= kHostOutputMaxBytes) {
         fGC += "   Check(sofie_cuda_ctx_host_output(fCtx, " + std::to_string(nbytes) + ", reinterpret_cast<void**>(&" + EMIT::Dev(n) +
                ")), \"sofie_cuda_ctx_host_output\");\n";
         continue;
      }
      fGC += "   Check(sofie_cuda_ctx_arena(fCtx, " + std::to_string(slot.second) + ", " + ByteCount(GetTensorShape(n), GetTensorType(n)) +
             ", reinterpret_cast<void**>(&" + EMIT::Dev(n) + ")), \"sofie_cuda_ctx_arena\");\n";
   }
   for (auto &a : fAliases)
      fGC += "   " + EMIT::Dev(a.first) + " = reinterpret_cast<" + EMIT::CType(GetTensorType(a.first)) + "*>(" + EMIT::Dev(ResolveAlias(a.first)) + ");\n";
   for (auto &b : fDeviceBuffers)
      fGC += "   Check(sofie_cuda_ctx_alloc(fCtx, " + std::to_string(b.second.length * GetTypeSize(b.second.type)) +
             ", reinterpret_cast<void**>(&" + EMIT::Dev(b.first) + ")), \"sofie_cuda_ctx_alloc\");\n";
   fGC += "   //--- weights: host copies live until the end of the constructor\n";
   for (auto &n : fDeviceWeights) {
      const auto &t = fInitializedTensors.at(n);
      std::string ct = EMIT::CType(t.type());
      if (fUseWeightFile) {
         fGC += "   std::vector<" + ct + "> " + EMIT::Host(n) + "(" + std::to_string(t.length()) + ");\n";
      } else {
         // kNoWeightFile: the values are written into the header
         std::stringstream vals;
         vals << std::setprecision(std::numeric_limits<float>::max_digits10);
         for (size_t i = 0; i < t.length(); i++) {
            if (i) vals << ", ";
            if (i % 16 == 15) vals << "\n      ";
            switch (t.type()) {
            case ETensorType::FLOAT: {
               float v = t.data<float>()[i];
               vals << EMIT::FloatLit(v);
               break;
            }
            case ETensorType::INT8: vals << (int)t.data<int8_t>()[i]; break;
            case ETensorType::UINT8: vals << (int)t.data<uint8_t>()[i]; break;
            case ETensorType::INT32: vals << t.data<int32_t>()[i]; break;
            case ETensorType::INT64: vals << t.data<int64_t>()[i]; break;
            default: throw std::runtime_error("SOFIE: tensor " + n + " has a type that cannot be written into the header");
            }
         }
         fGC += "   std::vector<" + ct + "> " + EMIT::Host(n) + " = {" + vals.str() + "};\n";
      }
   }
   if (fUseWeightFile && !fDeviceWeights.empty()) {
      fGC += "\n//--- reading weights from file\n";
      GenerateWeightReader();
      fGC += "\n";
   }
   for (auto &n : fDeviceWeights) {
      const auto &t = fInitializedTensors.at(n);
      fGC += "   Check(sofie_cuda_ctx_upload(fCtx, " + EMIT::Host(n) + ".data(), " + std::to_string(t.length() * GetTypeSize(t.type())) +
             ", reinterpret_cast<void**>(&" + EMIT::Dev(n) + ")), \"sofie_cuda_ctx_upload\");\n";
   }
   for (auto &op : fOperators)
      if (!op->IsFusedAway()) fGC += op->GenerateInitCode();
   fGC += "   Check(sofie_cuda_ctx_sync(fCtx), \"sofie_cuda_ctx_sync\");\n";
   fGC += "   } catch (...) {\n      sofie_cuda_ctx_destroy(fCtx);\n      fCtx = nullptr;\n      throw;\n   }\n";
   fGC += "}\n\n";
   fGC += "~Session() { sofie_cuda_ctx_destroy(fCtx); }\n";
   fGC += "Session(const Session &) = delete;\n";
   fGC += "Session & operator=(const Session &) = delete;\n";
   // movable, so that Sessions can live in a std::vector (one per slot, as SofieFunctor keeps them): the device
   // context and every pointer into it change hands, the source is left without a context
   fGC += "Session(Session && other) noexcept\n   : ";
   for (size_t i = 0; i < fSessionMembers.size(); i++)
      fGC += (i ? ", " : "") + fSessionMembers[i] + "(other." + fSessionMembers[i] + ")";
   fGC += "\n{\n   other.fCtx = nullptr;\n}\n\n";
}

void RModel::GenerateInfer()
{
   size_t nOut = fOutputTensorNames.size();
   if (nOut == 0) throw std::runtime_error("SOFIE: output size=0 are not supported");
   // the launches of one infer(), in execution order; captured into a CUDA graph on the first call
   const std::vector<size_t> &sliced = fSlicedOps; // the operators launched per uploaded part (PlanSlices)
   const bool pipelined = !sliced.empty();
   auto isSliced = [&](size_t i) { return std::find(sliced.begin(), sliced.end(), i) != sliced.end(); };
   size_t tailOps = 0;
   for (size_t i = 0; i < fOperators.size(); i++) tailOps += (!fOperators[i]->IsFusedAway() && !isSliced(i));
   if (pipelined) {
      fGC += "// the leading operators on one slice of the batch: launched as soon as that slice of the input has arrived\n";
      fGC += "void LaunchHead(int part) {\n";
      for (size_t i : sliced) fGC += fOperators[i]->GenerateBatchSlice(std::to_string(i), fUploadParts);
      fGC += "}\n\n";
   }
   fGC += pipelined ? "// all other kernel launches of one inference, on the context stream\n"
                    : "// all kernel launches of one inference, on the context stream\n";
   fGC += "void Launch() {\n";
   // a mark before every operator and one after the last: device timers when they are switched on, nothing otherwise
   size_t lastMark = 0;
   for (size_t i = 0; i < fOperators.size(); i++) {
      if (fOperators[i]->IsFusedAway() || isSliced(i)) continue;
      if (fVerbose) std::cout << "Generating code for operator .... " << i << std::endl;
      fGC += "   Check(sofie_cuda_ctx_mark(fCtx, " + std::to_string(i) + "), \"sofie_cuda_ctx_mark\");\n";
      fGC += fOperators[i]->Generate(std::to_string(i));
      lastMark = i + 1;
   }
   fGC += "   Check(sofie_cuda_ctx_mark(fCtx, " + std::to_string(lastMark) + "), \"sofie_cuda_ctx_mark\");\n";
   fGC += "}\n\n";

   ETensorType t0 = GetTensorType(fOutputTensorNames[0]);
   bool sameTypes = true;
   for (auto &o : fOutputTensorNames) sameTypes &= GetTensorType(o) == t0;
   std::string ret;
   if (nOut == 1) ret = "std::vector<" + ConvertTypeToString(t0) + ">";
   else if (sameTypes) ret = "std::vector<std::vector<" + ConvertTypeToString(t0) + ">>";
   else {
      ret = "std::tuple<";
      for (size_t i = 0; i < nOut; i++) ret += "std::vector<" + ConvertTypeToString(GetTensorType(fOutputTensorNames[i])) + ">" + (i + 1 < nOut ? "," : "");
      ret += ">";
   }
   // The kernels of one inference once the inputs are on the device (or, with the pipelined upload, while all but
   // the first operator's share of them is): replay of the captured graph, or the first, capturing, pass.
   fGC += "void Run() {\n";
   if (pipelined && tailOps == 0) {
      // every operator runs per slice: nothing is left to capture
      fGC += "}\n\n";
   } else {
   fGC += "   if (fGraphReady) {\n";
   fGC += "      Check(sofie_cuda_ctx_graph_launch(fCtx), \"sofie_cuda_ctx_graph_launch\");\n";
   fGC += "   } else {\n";
   fGC += "      Launch();\n";
   fGC += "      if (fUseGraph) {\n";
   fGC += "         Check(sofie_cuda_ctx_graph_begin(fCtx), \"sofie_cuda_ctx_graph_begin\");\n";
   fGC += "         try { Launch(); } catch (...) { sofie_cuda_ctx_graph_end(fCtx); throw; }\n";
   fGC += "         Check(sofie_cuda_ctx_graph_end(fCtx), \"sofie_cuda_ctx_graph_end\");\n";
   fGC += "         fGraphReady = true;\n";
   fGC += "      }\n";
   fGC += "   }\n";
   fGC += "}\n\n";
   }
   // Every kernel of one inference on the inputs of the previous infer() call, which are still on the device:
   // no copy in either direction and no wait (for callers that time or pipeline the device work themselves).
   fGC += "void RunResident() {\n";
   if (pipelined) fGC += "   for (int part = 0; part < " + std::to_string(fUploadParts) + "; part++) LaunchHead(part);\n";
   fGC += "   Run();\n";
   fGC += "}\n\n";
   fGC += ret + " infer(" + GenerateInferSignature() + "){\n";
   if (fDynamicBatch) {
      // any batch up to the one the Session was built for; the graph is captured again when the batch changes
      fGC += "   if (" + fBatchParam + " > fMaxBatch) throw std::runtime_error(\"SOFIE: infer() was called with " + fBatchParam +
             " = \" + std::to_string(" + fBatchParam + ") + \", the Session was constructed for at most \" + std::to_string(fMaxBatch));\n";
      fGC += "   if (" + fBatchParam + " == 0) return {};\n";
      fGC += "   if (" + fBatchParam + " != fBatch) { fBatch = " + fBatchParam + "; fGraphReady = false; }\n";
   }
   if (pipelined) {
      const std::string &n = fInputTensorNames[0];
      const size_t elems = ConvertShapeToLength(GetTensorShape(n)) / fUploadParts;
      const std::string parts = std::to_string(fUploadParts), slice = std::to_string(elems);
      // one loop: from pinned memory every call only enqueues (the copy of a part takes far longer than enqueueing the launches
      // behind it, so the copy stream never runs dry); from pageable memory the copy call returns when the part has been staged,
      // and the kernels of that part run while the host stages the next one
      fGC += "   for (int part = 0; part < " + parts + "; part++) {\n";
      fGC += "      Check(sofie_cuda_ctx_h2d_part(fCtx, " + EMIT::Dev(n) + " + (size_t)part * " + slice + ", tensor_" + n + " + (size_t)part * " + slice +
             ", " + std::to_string(elems * GetTypeSize(GetTensorType(n))) + ", part), \"sofie_cuda_ctx_h2d_part\");\n";
      fGC += "      Check(sofie_cuda_ctx_wait_part(fCtx, part), \"sofie_cuda_ctx_wait_part\");\n";
      fGC += "      LaunchHead(part);\n";
      fGC += "   }\n";
   } else {
      for (auto &n : fInputTensorNames)
         fGC += "   Check(sofie_cuda_ctx_h2d(fCtx, " + EMIT::Dev(n) + ", tensor_" + n + ", " + ByteCount(GetTensorShape(n), GetTensorType(n)) +
                "), \"sofie_cuda_ctx_h2d\");\n";
   }
   fGC += "   Run();\n";
   for (size_t i = 0; i < nOut; i++) {
      const std::string &o = fOutputTensorNames[i];
      std::string type = ConvertTypeToString(GetTensorType(o));
      // the result lands in the context's pinned buffer; the returned vector is built from it in one pass
      const std::string idx = std::to_string(i), len = std::to_string(ConvertShapeToLength(GetTensorShape(o)));
      fGC += "   void * host_ret_" + idx + " = nullptr;\n";
      fGC += "   Check(sofie_cuda_ctx_fetch(fCtx, " + EMIT::Dev(o) + ", " + ByteCount(GetTensorShape(o), GetTensorType(o)) + ", &host_ret_" + idx +
             "), \"sofie_cuda_ctx_fetch\");\n";
      fGC += "   std::vector<" + type + "> ret_" + idx + "(static_cast<const " + type + " *>(host_ret_" + idx + "), static_cast<const " + type +
             " *>(host_ret_" + idx + ") + " + len + ");\n";
   }
   if (nOut == 1) fGC += "   return ret_0;\n";
   else {
      fGC += "   return {";
      for (size_t i = 0; i < nOut; i++) fGC += "ret_" + std::to_string(i) + (i + 1 < nOut ? "," : "");
      fGC += "};\n";
   }
   fGC += "}\n";
}

void RModel::GenerateSessionCode()
{
   fGC += "struct Session {\n";
   GenerateSessionMembers();
   fGC += "\n";
   for (size_t id = 0; id < fOperators.size(); id++)
      if (!fOperators[id]->IsFusedAway()) fGC += fOperators[id]->GenerateSessionMembersCode(std::to_string(id));
   for (auto &op : fOperators)
      if (!op->IsFusedAway()) fGC += op->GenerateDeclCode();
   fGC += "\n";
   GenerateConstructor();
   GenerateInfer();
   fGC += "};   // end of Session\n";
}

// ---------------------------------------------------------------------------------- weight file, output
// Binary side file (Options::kBinaryWeightFile), little-endian:
//   "SOFIEBW1", uint64 tensor count, then per tensor: uint32 name length, the name ("tensor_<name>"),
//   uint32 ETensorType, uint64 element count, uint64 byte count, the raw values, zero padding to 8 bytes.
// A text file of C4's four 4096 x 4096 layers is 800 MB and takes minutes to parse; this form is
// read at the speed of the file system and stores int8 / FP8 tensors in one byte per value.
static long WriteBinaryWeights(const std::string &filename, const std::set<std::string> &names,
                               const std::map<std::string, InitializedTensor> &tensors, long readPos)
{
   std::ofstream f(filename, (readPos > 0 ? std::ios_base::app : std::ios_base::out) | std::ios_base::binary);
   if (!f.is_open()) throw std::runtime_error("sofie failed to open file " + filename + " for tensor weight data");
   auto put = [&](const void *p, size_t n) { f.write(static_cast<const char *>(p), (std::streamsize)n); };
   put("SOFIEBW1", 8);
   uint64_t count = names.size();
   put(&count, 8);
   for (auto &n : names) {
      const auto &t = tensors.at(n);
      std::string tname = "tensor_" + n;
      uint32_t nlen = (uint32_t)tname.size(), type = (uint32_t)t.type();
      uint64_t length = t.length(), bytes = length * GetTypeSize(t.type());
      put(&nlen, 4);
      put(tname.data(), nlen);
      put(&type, 4);
      put(&length, 8);
      put(&bytes, 8);
      put(t.data<char>(), bytes);
      static const char zeros[8] = {0};
      put(zeros, (8 - (nlen + bytes) % 8) % 8);
      if (f.fail()) throw std::runtime_error("sofie failed to write tensor data to file for " + n);
   }
   long pos = f.tellp();
   f.close();
   return pos;
}

long RModel::WriteInitializedTensorsToFile(std::string filename)
{
   if (fWeightFile == WeightFileType::Binary) {
      if (filename.empty()) filename = fName + ".bin";
      return WriteBinaryWeights(filename, fDeviceWeights, fInitializedTensors, fReadPos);
   }
   if (fWeightFile != WeightFileType::Text) return -1;
   if (filename.empty()) filename = fName + ".dat";
   std::ofstream f(filename, fReadPos > 0 ? std::ios_base::app : std::ios_base::out);
   if (!f.is_open()) throw std::runtime_error("sofie failed to open file " + filename + " for tensor weight data");
   // only the tensors the emitted constructor reads, in the order it reads them
   for (auto &n : fDeviceWeights) {
      const auto &t = fInitializedTensors.at(n);
      size_t length = t.length();
      f << "tensor_" << n << " " << length << "\n";
      switch (t.type()) {
      case ETensorType::FLOAT: {
         const float *data = t.data<float>();
         for (size_t i = 0; i < length; i++) {
            // as the reference does: max_digits10 digits, subnormals flushed to zero
            float v = data[i];
            if (v != 0.f && std::abs(v) < std::numeric_limits<float>::min()) v = 0.f;
            f << std::setprecision(std::numeric_limits<float>::max_digits10) << v << (i + 1 < length ? " " : "\n");
         }
         break;
      }
      case ETensorType::INT8:
         for (size_t i = 0; i < length; i++) f << (int)t.data<int8_t>()[i] << (i + 1 < length ? " " : "\n");
         break;
      case ETensorType::UINT8:
      case ETensorType::FLOAT8E4M3FN: // bit patterns
         for (size_t i = 0; i < length; i++) f << (int)t.data<uint8_t>()[i] << (i + 1 < length ? " " : "\n");
         break;
      case ETensorType::INT32:
         for (size_t i = 0; i < length; i++) f << t.data<int32_t>()[i] << (i + 1 < length ? " " : "\n");
         break;
      case ETensorType::INT64:
         for (size_t i = 0; i < length; i++) f << t.data<int64_t>()[i] << (i + 1 < length ? " " : "\n");
         break;
      default: throw std::runtime_error("sofie tensor " + n + " with type " + ConvertTypeToString(t.type()) + " cannot be written to a file");
      }
      if (f.fail()) throw std::runtime_error("sofie failed to write tensor data to file for " + n);
   }
   long pos = f.tellp();
   f.close();
   return pos;
}

void RModel::OutputGenerated(std::string filename, bool append)
{
   RModel_Base::OutputGenerated(filename, append);
   if (fUseWeightFile) {
      const std::string ext = fWeightFile == WeightFileType::Binary ? ".bin" : ".dat";
      if (!filename.empty()) {
         size_t pos = filename.find(".hxx");
         if (pos != std::string::npos) filename.replace(pos, 4, ext);
         else filename += ext;
      } else {
         filename = fName + ext;
      }
      WriteInitializedTensorsToFile(filename);
   }
}

void RModel::PrintRequiredInputTensors()
{
   std::cout << "Model requires following inputs:\n";
   for (auto &i : fInputTensorInfos)
      std::cout << "Parametrised Tensor name: " << i.first << "\ttype: " << ConvertTypeToString(i.second.type)
                << "\tshape: " << ConvertDynamicShapeToString(i.second.shape) << "\n";
   for (auto &i : fReadyInputTensorInfos)
      std::cout << "Fully Specified Tensor name: " << i.first << "\ttype: " << ConvertTypeToString(i.second.type)
                << "\tshape: " << ConvertShapeToString(i.second.shape) << "\n";
   std::cout << "\n";
}

void RModel::PrintInitializedTensors()
{
   std::cout << "Model initialized the following tensors:\n";
   for (auto &it : fInitializedTensors)
      std::cout << "Tensor name: \"" << it.first << "\"\ttype: " << ConvertTypeToString(it.second.type())
                << "\tshape: " << ConvertShapeToString(it.second.shape()) << (it.second.IsConstantTensor() ? " (Constant)" : "")
                << (!it.second.IsWeightTensor() ? " (Not Writable)" : "") << "\n";
   std::cout << "\n";
}

void RModel::PrintIntermediateTensors()
{
   std::cout << "Model specify the following intermediate tensors:\n";
   for (auto &it : fIntermediateTensorInfos)
      std::cout << "Tensor name: \"" << it.first << "\"\ttype: " << ConvertTypeToString(it.second.type)
                << "\tshape: " << ConvertShapeToString(it.second.shape)
                << (GetTensorLayout(it.first) == ELayout::NHWC ? " (NHWC on the device)" : "") << "\n";
   std::cout << "\n";
}

void RModel::PrintOutputTensors()
{
   std::cout << "Model specify the following output tensors:\n";
   for (auto &it : fOutputTensorNames)
      std::cout << "Tensor name: \"" << it << "\"\tshape: " << ConvertShapeToString(GetTensorShape(it)) << "\n";
   std::cout << "\n";
}

void RModel::HeadInitializedTensors(std::string name, int n_print)
{
   auto it = fInitializedTensors.find(name);
   if (it == fInitializedTensors.end()) {
      std::cout << "Tensor " << name << " not found in model's initialized tensor list" << std::endl;
      return;
   }
   std::cout << "Tensor name: " << it->first << "\ttype: " << ConvertTypeToString(it->second.type())
             << "\tshape: " << ConvertShapeToString(it->second.shape()) << "\n";
   size_t n = std::min<size_t>(it->second.length(), n_print);
   if (it->second.type() == ETensorType::FLOAT)
      for (size_t i = 0; i < n; i++) std::cout << it->second.data<float>()[i] << (i + 1 < n ? ", " : "\n");
}

} // namespace SOFIE
