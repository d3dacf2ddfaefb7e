// Header prologue and file output of a generated model
// (reference: src/SOFIE_core/src/RModel_Base.cxx:9-78).
#include "SOFIE/RModel_Base.hxx"

#include <algorithm>
#include <cctype>
#include <fstream>

namespace SOFIE {

std::underlying_type_t<Options> operator|(Options opA, Options opB)
{
   return static_cast<std::underlying_type_t<Options>>(opA) | static_cast<std::underlying_type_t<Options>>(opB);
}
std::underlying_type_t<Options> operator|(std::underlying_type_t<Options> opA, Options opB)
{
   return opA | static_cast<std::underlying_type_t<Options>>(opB);
}

RModel_Base::RModel_Base(std::string name, std::string parsedtime) : fFileName(name), fParseTime(parsedtime)
{
   fName = fFileName.substr(0, fFileName.rfind("."));
   auto slash = fName.find_last_of("/\\");
   if (slash != std::string::npos) fName = fName.substr(slash + 1);
   fName = UTILITY::Clean_name(fName);
}

void RModel_Base::GenerateHeaderInfo(std::string &hgname)
{
   std::string when = fParseTime;
   while (!when.empty() && (when.back() == '\n' || when.back() == ' ')) when.pop_back();
   fGC += "//Code generated automatically by SOFIE (CUDA path, libSOFIE_cuda) for Inference of Model file [" + fFileName + "] at [" + when + "] \n";
   hgname = fName;
   std::transform(hgname.begin(), hgname.end(), hgname.begin(), [](unsigned char c) { return std::toupper(c); });
   hgname = "SOFIE_" + hgname;
   fGC += "\n#ifndef " + hgname + "\n#define " + hgname + "\n\n";
   for (auto &lib : fNeededStdLib) fGC += "#include <" + lib + ">\n";
   for (auto &h : fCustomOpHeaders) fGC += "#include \"" + h + "\"\n";
   fGC += "#include <cstdint>\n#include <cstdlib>\n";
   if (fUseWeightFile) fGC += "#include <fstream>\n";
   // the C ABI of the device library takes the place of the reference's in-header BLAS prototypes
   fGC += "#include \"sofie_cuda.h\"\n";
   fGC += "\nnamespace SOFIE_" + fName + "{\n";
   fGC += "// a non-zero status of libSOFIE_cuda becomes the exception the reference's Session throws\n";
   fGC += "inline void Check(int status, const char * what) {\n";
   fGC += "   if (status != 0) throw std::runtime_error(std::string(\"SOFIE CUDA: \") + what + \" failed: \" + sofie_cuda_last_error() + \" (\" + sofie_cuda_strerror(status) + \")\");\n";
   fGC += "}\n";
}

void RModel_Base::OutputGenerated(std::string filename, bool append)
{
   if (filename.empty()) {
      filename = fName + ".hxx";
      append = false;
   }
   std::ofstream f;
   if (append) f.open(filename, std::ios_base::app);
   else f.open(filename);
   if (!f.is_open()) throw std::runtime_error("sofie failed to open file for output generated inference code");
   f << fGC;
   f.close();
}

} // namespace SOFIE
