// Protobuf-free decoder of the ONNX wire format: just enough of ModelProto / GraphProto / NodeProto /
// TensorProto / AttributeProto / ValueInfoProto for the operators of the dense-contraction path.
// The structs live in namespace onnx and carry protobuf-style accessors (op_type(), input(i),
// attribute(i).ints(j), ...) so that operator parsers read like the ones written against the
// protobuf-generated classes. Field numbers follow the ONNX schema the reference vendors
// (src/SOFIE_parsers/onnx_proto3).
#ifndef SOFIE_ONNX_WIRE
#define SOFIE_ONNX_WIRE

#include <cstdint>
#include <string>
#include <vector>

namespace onnx {

class TensorProto {
public:
   enum DataType { UNDEFINED = 0, FLOAT = 1, UINT8 = 2, INT8 = 3, UINT16 = 4, INT16 = 5, INT32 = 6, INT64 = 7, STRING = 8, BOOL = 9,
                   FLOAT16 = 10, DOUBLE = 11, UINT32 = 12, UINT64 = 13, BFLOAT16 = 16, FLOAT8E4M3FN = 17 };
   std::vector<int64_t> fDims;
   int fDataType = 0;
   std::string fName, fRawData;
   std::vector<float> fFloatData;
   std::vector<int32_t> fInt32Data;
   std::vector<int64_t> fInt64Data;
   std::vector<double> fDoubleData;
   int dims_size() const { return (int)fDims.size(); }
   int64_t dims(int i) const { return fDims[i]; }
   int data_type() const { return fDataType; }
   const std::string &name() const { return fName; }
   const std::string &raw_data() const { return fRawData; }
   bool has_raw_data() const { return !fRawData.empty(); }
   int float_data_size() const { return (int)fFloatData.size(); }
   float float_data(int i) const { return fFloatData[i]; }
   int int32_data_size() const { return (int)fInt32Data.size(); }
   int32_t int32_data(int i) const { return fInt32Data[i]; }
   int int64_data_size() const { return (int)fInt64Data.size(); }
   int64_t int64_data(int i) const { return fInt64Data[i]; }
};

class AttributeProto {
public:
   std::string fName, fS;
   float fF = 0.f;
   int64_t fI = 0;
   int fType = 0;
   std::vector<int64_t> fInts;
   std::vector<float> fFloats;
   TensorProto fT;
   const std::string &name() const { return fName; }
   float f() const { return fF; }
   int64_t i() const { return fI; }
   const std::string &s() const { return fS; }
   const TensorProto &t() const { return fT; }
   int ints_size() const { return (int)fInts.size(); }
   int64_t ints(int i) const { return fInts[i]; }
   const std::vector<int64_t> &ints() const { return fInts; }
   int floats_size() const { return (int)fFloats.size(); }
   float floats(int i) const { return fFloats[i]; }
};

class NodeProto {
public:
   std::vector<std::string> fInput, fOutput;
   std::string fName, fOpType;
   std::vector<AttributeProto> fAttribute;
   int input_size() const { return (int)fInput.size(); }
   const std::string &input(int i) const { return fInput[i]; }
   int output_size() const { return (int)fOutput.size(); }
   const std::string &output(int i) const { return fOutput[i]; }
   const std::string &name() const { return fName; }
   const std::string &op_type() const { return fOpType; }
   int attribute_size() const { return (int)fAttribute.size(); }
   const AttributeProto &attribute(int i) const { return fAttribute[i]; }
   const AttributeProto *find_attribute(const std::string &name) const
   {
      for (auto &a : fAttribute)
         if (a.fName == name) return &a;
      return nullptr;
   }
};

class ValueInfoProto {
public:
   struct Dimension {
      bool fHasValue = false;
      int64_t fValue = 0;
      std::string fParam;
   };
   std::string fName;
   int fElemType = 0;
   bool fHasShape = false;
   std::vector<Dimension> fDims;
   const std::string &name() const { return fName; }
};

class GraphProto {
public:
   std::vector<NodeProto> fNode;
   std::string fName;
   std::vector<TensorProto> fInitializer;
   std::vector<ValueInfoProto> fInput, fOutput;
   int node_size() const { return (int)fNode.size(); }
   const NodeProto &node(int i) const { return fNode[i]; }
   int initializer_size() const { return (int)fInitializer.size(); }
   const TensorProto &initializer(int i) const { return fInitializer[i]; }
   int input_size() const { return (int)fInput.size(); }
   const ValueInfoProto &input(int i) const { return fInput[i]; }
   int output_size() const { return (int)fOutput.size(); }
   const ValueInfoProto &output(int i) const { return fOutput[i]; }
};

class ModelProto {
public:
   int64_t fIrVersion = 0;
   std::string fProducerName;
   GraphProto fGraph;
   bool fHasGraph = false;
   const GraphProto &graph() const { return fGraph; }
   // Decodes a serialized ModelProto; throws std::runtime_error on malformed input.
   void ParseFromString(const std::string &bytes);
};

} // namespace onnx

#endif
