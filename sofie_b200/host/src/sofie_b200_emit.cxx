// sofie_b200_emit: ONNX file -> Session header for the B200 target (+ weight file), the counterpart
// of the reference's emitter programs (tests/templates/EmitFromONNX_GPU_ALPAKA.cxx.in:9-17).
//
//   sofie_b200_emit <model.onnx> <out.hxx> [--batch N] [--external-stream] [--custom-memory]
//                   [--profile] [--debug] [--no-weight-file] [--safetensors] [--check]
//
// Prints a one-line JSON report of what generation decided (fusions, arena size) on stdout.
#include <cstring>
#include <iostream>

#include "SOFIE_B200/RModelParser_ONNX.hxx"

using namespace SOFIE_B200;

int main(int argc, char **argv)
{
   if (argc < 3) {
      std::cerr << "usage: sofie_b200_emit <model.onnx> <out.hxx> [--batch N] [--external-stream] [--custom-memory] [--profile] [--debug] "
                   "[--no-weight-file] [--safetensors] [--check]\n";
      return 2;
   }
   std::underlying_type_t<Options> opts = 0;
   int batch = -1;
   bool checkOnly = false;
   for (int i = 3; i < argc; ++i) {
      if (!std::strcmp(argv[i], "--batch") && i + 1 < argc) batch = std::atoi(argv[++i]);
      else if (!std::strcmp(argv[i], "--external-stream")) opts = opts | Options::kExternalStream;
      else if (!std::strcmp(argv[i], "--custom-memory")) opts = opts | Options::kCustomMemory;
      else if (!std::strcmp(argv[i], "--profile")) opts = opts | Options::kProfile;
      else if (!std::strcmp(argv[i], "--debug")) opts = opts | Options::kDebug;
      else if (!std::strcmp(argv[i], "--no-weight-file")) opts = opts | Options::kNoWeightFile;
      else if (!std::strcmp(argv[i], "--safetensors")) opts = opts | Options::kSafetensorsWeightFile;
      else if (!std::strcmp(argv[i], "--check")) checkOnly = true;
      else { std::cerr << "unknown option " << argv[i] << "\n"; return 2; }
   }
   try {
      RModelParser_ONNX parser;
      if (checkOnly) return parser.CheckModel(argv[1], true) ? 0 : 1;
      RModel model = parser.Parse(argv[1]);
      model.GenerateGPU_B200(opts, batch);
      model.OutputGenerated(argv[2]);
      std::cout << "{\"model\": \"" << model.GetName() << "\", \"operators\": " << model.GetNumberOfOperators() << ", \"fusions\": [";
      for (size_t i = 0; i < model.GetFusionLog().size(); ++i) std::cout << (i ? ", " : "") << "\"" << model.GetFusionLog()[i] << "\"";
      std::cout << "]";
      // a size of a model with a symbolic dimension N is a * N + b: reported as "<key>_per_unit": a, "<key>": b
      const bool symbolic = !model.GetSymbolicDimension().empty();
      if (symbolic) std::cout << ", \"symbolic_dimension\": \"" << model.GetSymbolicDimension() << "\"";
      auto size = [&](const char *key, unsigned long long v) {
         SymbolicValue sv;
         if (symbolic && DecodeSymbolic(v, sv)) std::cout << ", \"" << key << "_per_unit\": " << sv.a << ", \"" << key << "\": " << sv.b;
         else std::cout << ", \"" << key << "\": " << v;
      };
      size("arena_bytes", (unsigned long long)model.GetArenaBytes());
      size("pool_bytes", (unsigned long long)model.GetIntermediateMemoryPoolSize());
      size("unplanned_pool_bytes", (unsigned long long)model.GetUnplannedIntermediateBytes());
      std::cout << ", \"regions\": " << model.GetArenaRegions().size() << "}\n";
   } catch (const std::exception &e) {
      std::cerr << e.what() << "\n";
      return 1;
   }
   return 0;
}
