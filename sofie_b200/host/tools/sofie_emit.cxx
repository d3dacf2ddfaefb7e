// sofie_emit <model.onnx> <output.hxx> [batch]
// The reference's usage pattern (src/SOFIE_core/README.md:26-57, test/EmitFromONNX.cxx.in:13-22):
// Parse -> Generate -> OutputGenerated, which writes the header and, next to it, the weight file.
#include <cstdlib>
#include <iostream>

#include "SOFIE/RModelParser_ONNX.hxx"

int main(int argc, char **argv)
{
   if (argc < 3) {
      std::cerr << "usage: " << argv[0] << " <model.onnx> <output.hxx> [batch size for parametric inputs]\n";
      return 2;
   }
   try {
      SOFIE::RModelParser_ONNX parser;
      SOFIE::RModel model = parser.Parse(argv[1]);
      model.Generate(SOFIE::Options::kDefault, argc > 3 ? std::atoi(argv[3]) : -1);
      model.OutputGenerated(argv[2]);
   } catch (const std::exception &e) {
      std::cerr << "sofie_emit: " << e.what() << "\n";
      return 1;
   }
   return 0;
}
