// Shape / type utilities of the generator (reference: src/SOFIE_core/src/SOFIE_common.cxx:1-130,394-400).
#include "SOFIE/SOFIE_common.hxx"

#include <algorithm>
#include <cctype>

namespace SOFIE {

std::string ConvertTypeToString(ETensorType type)
{
   switch (type) {
   case ETensorType::FLOAT: return "float";
   case ETensorType::INT8: return "int8_t";
   case ETensorType::INT16: return "int16_t";
   case ETensorType::INT32: return "int32_t";
   case ETensorType::INT64: return "int64_t";
   case ETensorType::UINT8: return "uint8_t";
   case ETensorType::UINT16: return "uint16_t";
   case ETensorType::UINT32: return "uint32_t";
   case ETensorType::UINT64: return "uint64_t";
   case ETensorType::DOUBLE: return "double";
   case ETensorType::BOOL: return "bool";
   case ETensorType::BFLOAT16: return "uint16_t";
   case ETensorType::FLOAT8E4M3FN: return "uint8_t";
   default: return "other";
   }
}

ETensorType ConvertStringToType(std::string type)
{
   if (type == "float32" || type == "float" || type == "Float") return ETensorType::FLOAT;
   if (type == "int64" || type == "int64_t") return ETensorType::INT64;
   if (type == "int32" || type == "int32_t") return ETensorType::INT32;
   if (type == "uint8" || type == "uint8_t") return ETensorType::UINT8;
   if (type == "int8" || type == "int8_t") return ETensorType::INT8;
   if (type == "double" || type == "float64") return ETensorType::DOUBLE;
   if (type == "bool") return ETensorType::BOOL;
   return ETensorType::UNDEFINED;
}

std::size_t ConvertShapeToLength(const std::vector<size_t> &shape)
{
   std::size_t n = 1;
   for (auto d : shape) n *= d;
   return n;
}

std::string ConvertShapeToString(const std::vector<size_t> &shape)
{
   std::stringstream out;
   out << "{ ";
   for (size_t i = 0; i < shape.size(); i++) out << shape[i] << (i + 1 < shape.size() ? " , " : "");
   out << " }";
   return out.str();
}

std::string ConvertDynamicShapeToString(const std::vector<Dim> &shape)
{
   std::stringstream out;
   out << "{ ";
   for (size_t i = 0; i < shape.size(); i++) out << shape[i].GetVal() << (i + 1 < shape.size() ? " , " : "");
   out << " }";
   return out.str();
}

std::string ConvertDynamicShapeToLength(const std::vector<Dim> &shape)
{
   size_t fixed = 1;
   std::string params;
   for (auto &d : shape) {
      if (d.isParam) params += (params.empty() ? "" : " * ") + d.param;
      else fixed *= d.dim;
   }
   if (params.empty()) return std::to_string(fixed);
   return fixed == 1 ? params : std::to_string(fixed) + " * " + params;
}

std::vector<Dim> ConvertShapeToDim(const std::vector<size_t> &shape)
{
   std::vector<Dim> out;
   for (auto d : shape) out.emplace_back(d);
   return out;
}

std::vector<size_t> ConvertShapeToInt(const std::vector<Dim> &shape)
{
   std::vector<size_t> out;
   for (auto &d : shape) {
      if (d.isParam) return {};
      out.push_back(d.dim);
   }
   return out;
}

std::string UTILITY::Clean_name(std::string name)
{
   std::replace(name.begin(), name.end(), '-', '_');
   name.erase(std::remove_if(name.begin(), name.end(), [](unsigned char c) { return !std::isalnum(c) && c != '_'; }), name.end());
   return name;
}

bool UTILITY::AreSameShape(const std::vector<size_t> &a, const std::vector<size_t> &b) { return a == b; }

} // namespace SOFIE
