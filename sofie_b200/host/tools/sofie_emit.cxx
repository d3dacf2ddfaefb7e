// sofie_emit <model.onnx> <output.hxx> [batch] [--binary] [--pipelined-upload | --single-upload]
// The reference's usage pattern (src/SOFIE_core/README.md:26-57, test/EmitFromONNX.cxx.in:13-22):
// Parse -> Generate -> OutputGenerated, which writes the header and, next to it, the weight file.
#include <cstdlib>
#include <iostream>
#include <string>

#include "SOFIE/RModelParser_ONNX.hxx"

int main(int argc, char **argv)
{
   if (argc < 3) {
      std::cerr << "usage: " << argv[0] << " <model.onnx> <output.hxx> [batch size for parametric inputs] [--binary] [--pipelined-upload | --single-upload]\n";
      return 2;
   }
   try {
      SOFIE::RModelParser_ONNX parser;
      SOFIE::RModel model = parser.Parse(argv[1]);
      auto options = static_cast<std::underlying_type_t<SOFIE::Options>>(SOFIE::Options::kDefault);
      int batch = -1;
      for (int i = 3; i < argc; i++) {
         if (std::string(argv[i]) == "--binary") options = options | SOFIE::Options::kBinaryWeightFile;
         else if (std::string(argv[i]) == "--pipelined-upload") options = options | SOFIE::Options::kPipelinedUpload;
         else if (std::string(argv[i]) == "--single-upload") options = options | SOFIE::Options::kSingleUpload;
         else batch = std::atoi(argv[i]);
      }
      model.Generate(options, batch);
      model.OutputGenerated(argv[2]);
   } catch (const std::exception &e) {
      std::cerr << "sofie_emit: " << e.what() << "\n";
      return 1;
   }
   return 0;
}
