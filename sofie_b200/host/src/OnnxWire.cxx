// Decoder of the protobuf wire format for the ONNX messages declared in SOFIE/OnnxWire.hxx.
// Wire types: 0 varint, 1 64-bit, 2 length-delimited, 5 32-bit. Repeated scalars may arrive packed
// (one length-delimited blob) or one by one; both forms are accepted.
#include "SOFIE/OnnxWire.hxx"

#include <cstring>
#include <stdexcept>

namespace onnx {
namespace {

struct Reader {
   const unsigned char *p, *end;
   Reader(const char *data, size_t n) : p(reinterpret_cast<const unsigned char *>(data)), end(p + n) {}
   bool done() const { return p >= end; }
   uint64_t varint()
   {
      uint64_t v = 0;
      for (int shift = 0; shift < 70; shift += 7) {
         if (p >= end) throw std::runtime_error("ONNX decode: truncated varint");
         unsigned char b = *p++;
         v |= (uint64_t)(b & 0x7F) << shift;
         if (!(b & 0x80)) return v;
      }
      throw std::runtime_error("ONNX decode: varint too long");
   }
   Reader bytes()
   {
      uint64_t n = varint();
      if (n > (uint64_t)(end - p)) throw std::runtime_error("ONNX decode: length-delimited field runs past the buffer");
      Reader r(reinterpret_cast<const char *>(p), (size_t)n);
      p += n;
      return r;
   }
   std::string str()
   {
      Reader r = bytes();
      return std::string(reinterpret_cast<const char *>(r.p), r.end - r.p);
   }
   template <typename T> T fixed()
   {
      if ((size_t)(end - p) < sizeof(T)) throw std::runtime_error("ONNX decode: truncated fixed-width field");
      T v;
      std::memcpy(&v, p, sizeof(T));
      p += sizeof(T);
      return v;
   }
   void skip(int wire)
   {
      switch (wire) {
      case 0: varint(); break;
      case 1: fixed<uint64_t>(); break;
      case 2: bytes(); break;
      case 5: fixed<uint32_t>(); break;
      default: throw std::runtime_error("ONNX decode: unsupported wire type " + std::to_string(wire));
      }
   }
};

template <typename T> void repeated_varint(Reader &r, int wire, std::vector<T> &out)
{
   if (wire == 2) {
      Reader b = r.bytes();
      while (!b.done()) out.push_back((T)(int64_t)b.varint());
   } else {
      out.push_back((T)(int64_t)r.varint());
   }
}
void repeated_float(Reader &r, int wire, std::vector<float> &out)
{
   if (wire == 2) {
      Reader b = r.bytes();
      while (!b.done()) out.push_back(b.fixed<float>());
   } else {
      out.push_back(r.fixed<float>());
   }
}

void decode_tensor(Reader r, TensorProto &t)
{
   while (!r.done()) {
      uint64_t key = r.varint();
      int field = (int)(key >> 3), wire = (int)(key & 7);
      switch (field) {
      case 1: repeated_varint(r, wire, t.fDims); break;
      case 2: t.fDataType = (int)r.varint(); break;
      case 4: repeated_float(r, wire, t.fFloatData); break;
      case 5: repeated_varint(r, wire, t.fInt32Data); break;
      case 7: repeated_varint(r, wire, t.fInt64Data); break;
      case 8: t.fName = r.str(); break;
      case 9: t.fRawData = r.str(); break;
      case 10:
         if (wire == 2) {
            Reader b = r.bytes();
            while (!b.done()) t.fDoubleData.push_back(b.fixed<double>());
         } else {
            t.fDoubleData.push_back(r.fixed<double>());
         }
         break;
      default: r.skip(wire);
      }
   }
}

void decode_attribute(Reader r, AttributeProto &a)
{
   while (!r.done()) {
      uint64_t key = r.varint();
      int field = (int)(key >> 3), wire = (int)(key & 7);
      switch (field) {
      case 1: a.fName = r.str(); break;
      case 2: a.fF = r.fixed<float>(); break;
      case 3: a.fI = (int64_t)r.varint(); break;
      case 4: a.fS = r.str(); break;
      case 5: decode_tensor(r.bytes(), a.fT); break;
      case 7: repeated_float(r, wire, a.fFloats); break;
      case 8: repeated_varint(r, wire, a.fInts); break;
      case 20: a.fType = (int)r.varint(); break;
      default: r.skip(wire);
      }
   }
}

void decode_node(Reader r, NodeProto &n)
{
   while (!r.done()) {
      uint64_t key = r.varint();
      int field = (int)(key >> 3), wire = (int)(key & 7);
      switch (field) {
      case 1: n.fInput.push_back(r.str()); break;
      case 2: n.fOutput.push_back(r.str()); break;
      case 3: n.fName = r.str(); break;
      case 4: n.fOpType = r.str(); break;
      case 5: n.fAttribute.emplace_back(); decode_attribute(r.bytes(), n.fAttribute.back()); break;
      default: r.skip(wire);
      }
   }
}

void decode_value_info(Reader r, ValueInfoProto &v)
{
   while (!r.done()) {
      uint64_t key = r.varint();
      int field = (int)(key >> 3), wire = (int)(key & 7);
      if (field == 1) v.fName = r.str();
      else if (field == 2) { // TypeProto
         Reader type = r.bytes();
         while (!type.done()) {
            uint64_t k2 = type.varint();
            if ((k2 >> 3) == 1 && (k2 & 7) == 2) { // tensor_type
               Reader tt = type.bytes();
               while (!tt.done()) {
                  uint64_t k3 = tt.varint();
                  int f3 = (int)(k3 >> 3), w3 = (int)(k3 & 7);
                  if (f3 == 1) v.fElemType = (int)tt.varint();
                  else if (f3 == 2) { // TensorShapeProto
                     v.fHasShape = true;
                     Reader shape = tt.bytes();
                     while (!shape.done()) {
                        uint64_t k4 = shape.varint();
                        if ((k4 >> 3) == 1 && (k4 & 7) == 2) {
                           Reader dim = shape.bytes();
                           ValueInfoProto::Dimension d;
                           while (!dim.done()) {
                              uint64_t k5 = dim.varint();
                              int f5 = (int)(k5 >> 3), w5 = (int)(k5 & 7);
                              if (f5 == 1) { d.fHasValue = true; d.fValue = (int64_t)dim.varint(); }
                              else if (f5 == 2) d.fParam = dim.str();
                              else dim.skip(w5);
                           }
                           v.fDims.push_back(d);
                        } else shape.skip((int)(k4 & 7));
                     }
                  } else tt.skip(w3);
               }
            } else type.skip((int)(k2 & 7));
         }
      } else r.skip(wire);
   }
}

void decode_graph(Reader r, GraphProto &g)
{
   while (!r.done()) {
      uint64_t key = r.varint();
      int field = (int)(key >> 3), wire = (int)(key & 7);
      switch (field) {
      case 1: g.fNode.emplace_back(); decode_node(r.bytes(), g.fNode.back()); break;
      case 2: g.fName = r.str(); break;
      case 5: g.fInitializer.emplace_back(); decode_tensor(r.bytes(), g.fInitializer.back()); break;
      case 11: g.fInput.emplace_back(); decode_value_info(r.bytes(), g.fInput.back()); break;
      case 12: g.fOutput.emplace_back(); decode_value_info(r.bytes(), g.fOutput.back()); break;
      default: r.skip(wire);
      }
   }
}

} // namespace

void ModelProto::ParseFromString(const std::string &bytes)
{
   Reader r(bytes.data(), bytes.size());
   while (!r.done()) {
      uint64_t key = r.varint();
      int field = (int)(key >> 3), wire = (int)(key & 7);
      if (field == 1 && wire == 0) fIrVersion = (int64_t)r.varint();
      else if (field == 2 && wire == 2) fProducerName = r.str();
      else if (field == 7 && wire == 2) {
         decode_graph(r.bytes(), fGraph);
         fHasGraph = true;
      } else r.skip(wire);
   }
   if (!fHasGraph) throw std::runtime_error("ONNX decode: the file holds no graph");
}

} // namespace onnx
