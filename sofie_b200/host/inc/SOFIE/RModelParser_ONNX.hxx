// ONNX front end of the generator.
// Public interface as in the reference (src/SOFIE_parsers/inc/SOFIE/RModelParser_ONNX.hxx:27-88):
// Parse(filename, verbose) -> RModel, CheckModel, RegisterOperator, IsRegisteredOperator,
// GetRegisteredOperators, RegisterTensorType / GetTensorType. The model file is decoded by a built-in
// reader of the protobuf wire format (SOFIE/OnnxWire.hxx) instead of libprotobuf, and the float-only
// gates of the reference's operator parsers are widened to uint8 / int8 / int32 tensors, with
// QuantizeLinear, DequantizeLinear, QLinearMatMul and QLinearConv registered in addition.
#ifndef SOFIE_RMODELPARSER_ONNX
#define SOFIE_RMODELPARSER_ONNX

#include <functional>
#include <map>
#include <memory>
#include <unordered_map>

#include "SOFIE/OnnxWire.hxx"
#include "SOFIE/RModel.hxx"

namespace SOFIE {

class RModelParser_ONNX;

using ParserFuncSignature =
   std::function<std::unique_ptr<ROperator>(RModelParser_ONNX & /*parser*/, const onnx::NodeProto & /*nodeproto*/)>;
using ParserFuseFuncSignature = std::function<std::unique_ptr<ROperator>(
   RModelParser_ONNX & /*parser*/, const onnx::NodeProto & /*firstnode*/, const onnx::NodeProto & /*secondnode*/)>;

class RModelParser_ONNX {
public:
   struct OperatorsMapImpl {
      std::unordered_map<std::string, ParserFuncSignature> fOperatorsMap;
   };

private:
   bool fVerbose = false;
   std::unique_ptr<OperatorsMapImpl> fOperatorsMapImpl;
   std::unordered_map<std::string, ETensorType> fTensorTypeMap;
   std::vector<bool> fFusedOperators;

public:
   void RegisterOperator(const std::string &name, ParserFuncSignature func);
   bool IsRegisteredOperator(const std::string &name);
   std::vector<std::string> GetRegisteredOperators();
   void RegisterTensorType(const std::string &name, ETensorType type);
   bool IsRegisteredTensorType(const std::string &name);
   bool Verbose() const { return fVerbose; }
   ETensorType GetTensorType(const std::string &name);

   // Parse the index'th node (in execution order) of the graph; may fuse it with its only child.
   std::unique_ptr<ROperator> ParseOperator(const size_t index, const onnx::GraphProto &graphproto,
                                            const std::vector<size_t> &nodes, const std::vector<int> &children);
   void CheckGraph(const onnx::GraphProto &g, int &level, std::map<std::string, int> &missingOperators);
   void ParseONNXGraph(RModel &model, const onnx::GraphProto &g, std::string name = "");
   std::unique_ptr<onnx::ModelProto> LoadModel(std::string filename);

   RModelParser_ONNX() noexcept;
   RModel Parse(std::string filename, bool verbose = false);
   bool CheckModel(std::string filename, bool verbose = false);
   ~RModelParser_ONNX();
};

} // namespace SOFIE

#endif
