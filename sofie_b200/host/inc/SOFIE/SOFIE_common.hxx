// Common types of the SOFIE code generator, CUDA edition.
//
// Public names follow the reference (src/SOFIE_core/inc/SOFIE/SOFIE_common.hxx:29-149,272-300):
// ETensorType, EActivationType, Dim, InitializedTensor, ConvertShapeTo*, UTILITY::Clean_name.
// Nothing here depends on ROOT; the header compiles with a plain C++17 compiler because the code
// the generator emits includes it too. The reference's run-time helpers that the emitted CPU code
// needed (Im2col, UnidirectionalBroadcast) have no counterpart: the emitted code calls libSOFIE_cuda.
#ifndef SOFIE_SOFIE_COMMON
#define SOFIE_SOFIE_COMMON

#include <cstddef>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace SOFIE {

// Values are the ONNX TensorProto.DataType codes (the reference spells UINT8 "UNINT8"; both names
// are kept). FLOAT8E4M3FN is newer than the schema the reference vendors.
enum class ETensorType {
   UNDEFINED = 0, FLOAT = 1, UINT8 = 2, UNINT8 = 2, INT8 = 3, UINT16 = 4, INT16 = 5, INT32 = 6, INT64 = 7, STRING = 8,
   BOOL = 9, FLOAT16 = 10, DOUBLE = 11, UINT32 = 12, UINT64 = 13, COMPLEX64 = 14, COMPLEX28 = 15, BFLOAT16 = 16,
   FLOAT8E4M3FN = 17
};

enum class EActivationType { UNDEFINED = 0, RELU = 1, SOFTMAX = 2, SIGMOID = 3, LEAKYRELU = 4, TANH = 5, ELU = 6 };

// Memory layout of a rank-4 activation on the device. The reference knows NCHW only; between
// fused convolutions the CUDA path keeps NHWC, which is what the tensor-core kernels consume.
enum class ELayout { NCHW = 0, NHWC = 1 };

typedef std::int64_t int_t;

constexpr size_t GetTypeSize(ETensorType type)
{
   switch (type) {
   case ETensorType::FLOAT: return 4;
   case ETensorType::DOUBLE: return 8;
   case ETensorType::UINT8: return 1;
   case ETensorType::INT8: return 1;
   case ETensorType::FLOAT8E4M3FN: return 1;
   case ETensorType::UINT16: return 2;
   case ETensorType::INT16: return 2;
   case ETensorType::FLOAT16: return 2;
   case ETensorType::BFLOAT16: return 2;
   case ETensorType::INT32: return 4;
   case ETensorType::UINT32: return 4;
   case ETensorType::INT64: return 8;
   case ETensorType::UINT64: return 8;
   case ETensorType::BOOL: return 1;
   default: return 0;
   }
}

std::string ConvertTypeToString(ETensorType type);
ETensorType ConvertStringToType(std::string type);

struct Dim {
   bool isParam = false;
   size_t dim = 0;
   std::string param;
   Dim() {}
   Dim(const std::string &p, size_t d = 0) : isParam(true), dim(d), param(p) {}
   Dim(size_t d) : dim(d) {}
   std::string GetVal() const { return isParam ? param : std::to_string(dim); }
};

struct InputTensorInfo {
   ETensorType type;
   std::vector<Dim> shape;
};
struct TensorInfo {
   ETensorType type;
   std::vector<size_t> shape;
};
struct DynamicTensorInfo {
   ETensorType type;
   std::vector<Dim> shape;
};

template <typename T> ETensorType GetTemplatedType(T) { return ETensorType::UNDEFINED; }
template <> inline ETensorType GetTemplatedType(float) { return ETensorType::FLOAT; }
template <> inline ETensorType GetTemplatedType(double) { return ETensorType::DOUBLE; }
template <> inline ETensorType GetTemplatedType(uint8_t) { return ETensorType::UINT8; }
template <> inline ETensorType GetTemplatedType(int8_t) { return ETensorType::INT8; }
template <> inline ETensorType GetTemplatedType(int32_t) { return ETensorType::INT32; }
template <> inline ETensorType GetTemplatedType(int64_t) { return ETensorType::INT64; }

std::size_t ConvertShapeToLength(const std::vector<size_t> &shape);
std::string ConvertShapeToString(const std::vector<size_t> &shape);
std::string ConvertDynamicShapeToString(const std::vector<Dim> &shape);
std::string ConvertDynamicShapeToLength(const std::vector<Dim> &shape);
std::vector<Dim> ConvertShapeToDim(const std::vector<size_t> &shape);
std::vector<size_t> ConvertShapeToInt(const std::vector<Dim> &shape); // empty when a dimension is parametric

// A weight: type, shape and a shared host buffer (reference: SOFIE_common.hxx:152-270).
class InitializedTensor {
public:
   InitializedTensor() = default;
   InitializedTensor(ETensorType type, const std::vector<size_t> &shape, std::shared_ptr<void> data, bool isConstant = false)
      : fConstant(isConstant), fType(type), fShape(shape), fData(std::move(data))
   {
   }
   ETensorType const &type() const { return fType; }
   std::vector<size_t> const &shape() const { return fShape; }
   std::shared_ptr<void> const &sharedptr() const { return fData; }
   bool IsConstantTensor() const { return fConstant; }
   bool IsWeightTensor() const { return !fConstant && !fIsNotWritable; }
   void SetNotWritable() { fIsNotWritable = true; }
   template <class T = void> T const *data() const { return static_cast<T const *>(fData.get()); }
   size_t length() const { return ConvertShapeToLength(fShape); }

private:
   bool fConstant = false;
   bool fIsNotWritable = false;
   ETensorType fType = ETensorType::UNDEFINED;
   std::vector<size_t> fShape;
   std::shared_ptr<void> fData;
};

namespace UTILITY {
// Shape of A op B under numpy-style (multidirectional) broadcasting; throws when the shapes do not
// broadcast (reference: UTILITY::MultidirectionalBroadcastShape, src/SOFIE_core/src/SOFIE_common.cxx).
inline std::vector<size_t> MultidirectionalBroadcastShape(std::vector<size_t> a, std::vector<size_t> b)
{
   if (a.size() < b.size()) a.insert(a.begin(), b.size() - a.size(), 1);
   if (b.size() < a.size()) b.insert(b.begin(), a.size() - b.size(), 1);
   std::vector<size_t> out(a.size());
   for (size_t i = 0; i < a.size(); i++) {
      if (a[i] != b[i] && a[i] != 1 && b[i] != 1)
         throw std::runtime_error("SOFIE - Error multidirectional broadcasting shapes " + ConvertShapeToString(a) + " and " +
                                  ConvertShapeToString(b));
      out[i] = a[i] == 1 ? b[i] : a[i];
   }
   return out;
}

// Makes a tensor name usable as a C++ identifier (reference: src/SOFIE_core/src/SOFIE_common.cxx:394-400).
std::string Clean_name(std::string input_tensor_name);
bool AreSameShape(const std::vector<size_t> &a, const std::vector<size_t> &b);
} // namespace UTILITY

} // namespace SOFIE

#endif
