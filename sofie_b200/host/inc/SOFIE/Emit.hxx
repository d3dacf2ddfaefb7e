// Small helpers shared by the operators when they write C++ text for the generated Session.
// Naming convention of the emitted code:
//   tensor_<name>   host pointer passed to infer(), exactly as in the reference's signature
//   dev_<name>      device pointer (arena slice, uploaded weight or persistent buffer), Session member
//   host_<name>     host copy of a weight, alive during the Session constructor only
#ifndef SOFIE_EMIT
#define SOFIE_EMIT

#include <iomanip>
#include <limits>
#include <sstream>
#include <string>

#include "SOFIE/SOFIE_common.hxx"

namespace SOFIE {
namespace EMIT {

inline std::string Dev(const std::string &name) { return "dev_" + name; }
inline std::string Host(const std::string &name) { return "host_" + name; }
// slice `part` (a variable of the emitted code) of `parts` equal, contiguous slices of a tensor of `elems` elements
inline std::string DevSlice(const std::string &name, size_t elems, size_t parts)
{
   return parts > 1 ? "(" + Dev(name) + " + (size_t)part * " + std::to_string(elems / parts) + ")" : Dev(name);
}

inline std::string CType(ETensorType t)
{
   switch (t) {
   case ETensorType::FLOAT: return "float";
   case ETensorType::DOUBLE: return "double";
   case ETensorType::UINT8: return "uint8_t";
   case ETensorType::INT8: return "int8_t";
   case ETensorType::FLOAT8E4M3FN: return "uint8_t";
   case ETensorType::BFLOAT16: return "uint16_t";
   case ETensorType::INT32: return "int32_t";
   case ETensorType::INT64: return "int64_t";
   case ETensorType::BOOL: return "bool";
   default: throw std::runtime_error("SOFIE: tensor type " + ConvertTypeToString(t) + " has no device representation");
   }
}

// A float literal that reads back to exactly the same value.
inline std::string FloatLit(float v)
{
   std::ostringstream s;
   s << std::setprecision(std::numeric_limits<float>::max_digits10) << v;
   std::string t = s.str();
   if (t.find_first_of(".eEn") == std::string::npos) t += ".0";
   if (t.find("inf") != std::string::npos || t.find("nan") != std::string::npos)
      throw std::runtime_error("SOFIE: non-finite attribute value cannot be emitted");
   return t + "f";
}

// "SOFIE_CUDA_CHECK(<call>);" -- the emitted header defines the macro-free helper Check().
inline std::string Call(const std::string &indent, const std::string &call)
{
   return indent + "Check(" + call + ", \"" + call.substr(0, call.find('(')) + "\");\n";
}

} // namespace EMIT
} // namespace SOFIE

#endif
