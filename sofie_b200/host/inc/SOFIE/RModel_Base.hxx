// Options, header emission and file output shared by the model classes.
// Public names follow the reference (src/SOFIE_core/inc/SOFIE/RModel_Base.hxx:21-90): Options and its
// operator|, WeightFileType, RModel_Base::{GenerateHeaderInfo, PrintGenerated, ReturnGenerated,
// OutputGenerated, SetFilename, GetFilename, GetName, AddNeededStdLib, AddBlasRoutines}.
#ifndef SOFIE_RMODEL_BASE
#define SOFIE_RMODEL_BASE

#include <iostream>
#include <set>
#include <string>
#include <type_traits>
#include <vector>

#include "SOFIE/SOFIE_common.hxx"

namespace SOFIE {

enum class Options {
   kDefault = 0x0,
   kNoSession = 0x1,            // not available on the CUDA path: the Session owns the device context
   kNoWeightFile = 0x2,         // weights are written into the generated header
   kRootBinaryWeightFile = 0x4, // needs ROOT I/O: not available
   kGNN = 0x8,
   kGNNComponent = 0x10,
   kBinaryWeightFile = 0x40,    // addition: weights in a raw little-endian side file <name>.bin read with one fread per tensor
   kPipelinedUpload = 0x80,     // addition: upload the input in parts under the first convolution whatever its size (default: from 32 MB)
   kSingleUpload = 0x100,       // addition: never upload the input in parts (every operator is then part of Launch() and of the graph)
};

enum class WeightFileType { None, RootBinary, Text, Binary };

std::underlying_type_t<Options> operator|(Options opA, Options opB);
std::underlying_type_t<Options> operator|(std::underlying_type_t<Options> opA, Options opB);

class RModel_Base {
protected:
   std::string fFileName;  // name of the model file the RModel came from
   std::string fParseTime; // UTC time of parsing
   WeightFileType fWeightFile = WeightFileType::Text;
   std::set<std::string> fNeededBlasRoutines; // unused by the CUDA path, kept for source compatibility
   const std::set<std::string> fAllowedStdLib = {"vector", "algorithm", "cmath", "memory", "span", "string", "stdexcept"};
   std::set<std::string> fNeededStdLib = {"vector", "string", "stdexcept"};
   std::set<std::string> fCustomOpHeaders;
   std::string fName = "UnnamedModel";
   std::string fGC; // generated code
   bool fUseWeightFile = true;
   bool fUseSession = true;

public:
   RModel_Base() = default;
   RModel_Base(std::string name, std::string parsedtime);
   RModel_Base(std::string function_name) : fName(function_name) {}

   void AddBlasRoutines(std::vector<std::string> routines)
   {
      for (auto &r : routines) fNeededBlasRoutines.insert(r);
   }
   void AddNeededStdLib(std::string libname)
   {
      if (fAllowedStdLib.count(libname)) fNeededStdLib.insert(libname);
   }
   void AddNeededCustomHeader(std::string filename) { fCustomOpHeaders.insert(filename); }
   // Writes the prologue of the generated header: guards, includes, namespace SOFIE_<name> and, in
   // place of the reference's block of BLAS prototypes (RModel_Base.cxx:40-58), the include of
   // sofie_cuda.h plus the status-to-exception helper.
   void GenerateHeaderInfo(std::string &hgname);
   void PrintGenerated() { std::cout << fGC; }
   std::string ReturnGenerated() { return fGC; }
   void OutputGenerated(std::string filename = "", bool append = false);
   void SetFilename(std::string filename) { fName = filename; }
   std::string GetFilename() { return fName; }
   const std::string &GetName() const { return fName; }
};

} // namespace SOFIE

#endif
