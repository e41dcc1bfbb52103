// Test infrastructure: drives the UNMODIFIED reference generator (linked from oracle/_ref) to emit
// the CPU inference code it produces for the pinned models, i.e. the code whose results this
// repository's kernels must reproduce.
//
//   ref_emit <onnx dir> <list file>
//
// For every line "<Name>" of the list file it parses <onnx dir>/<Name>.onnx with the reference's
// ONNX parser and calls RModel::Generate() + OutputGenerated(), which writes <Name>.hxx and the
// text weight file <Name>.dat into the current directory (core/src/RModel.cxx:1744-1828,2242).
// It also builds the benchmark MLP (fp32, 64 -> 256 -> 256 -> 10, Relu after the first two Gemms)
// through the reference's C++ model API, the way the reference's own generators do
// (tests/models/LowRankModelGenerator.cxx:36-51), and finally writes ref_<Name>.cxx per model:
// a C entry point `ref_run` around the emitted Session, built into its own shared library.
#include "SOFIE/RModel.hxx"
#include "SOFIE/RModelParser_ONNX.hxx"
#include "SOFIE/operators/ROperator_Gemm.hxx"

#include <cmath>
#include <fstream>
#include <iostream>
#include <memory>
#include <random>
#include <string>
#include <vector>

using namespace SOFIE;

// Xavier-uniform weights from a fixed seed; biases zero.
static std::vector<float> xavier(std::mt19937_64 &rng, size_t fan_in, size_t fan_out)
{
   const double a = std::sqrt(6.0 / double(fan_in + fan_out));
   std::uniform_real_distribution<double> dist(-a, a);
   std::vector<float> w(fan_in * fan_out);
   for (auto &v : w) v = float(dist(rng));
   return w;
}

static void emit_mlp(const std::string &name, size_t batch)
{
   std::mt19937_64 rng(20240607ull);
   const size_t dims[4] = {64, 256, 256, 10};
   RModel model(name, "now");
   model.AddInputTensorInfo("X", ETensorType::FLOAT, std::vector<Dim>{Dim(batch), Dim(dims[0])});
   model.AddInputTensorName("X");
   std::string in = "X";
   for (int l = 0; l < 3; ++l) {
      auto w = xavier(rng, dims[l], dims[l + 1]);
      std::vector<float> b(dims[l + 1], 0.f);
      const std::string wn = "W" + std::to_string(l), bn = "B" + std::to_string(l);
      const std::string out = l == 2 ? "Y" : "H" + std::to_string(l);
      model.AddInitializedTensor(wn, ETensorType::FLOAT, std::vector<std::size_t>{dims[l], dims[l + 1]}, w.data());
      model.AddInitializedTensor(bn, ETensorType::FLOAT, std::vector<std::size_t>{dims[l + 1]}, b.data());
      const auto act = l < 2 ? EActivationType::RELU : EActivationType::UNDEFINED;
      model.AddOperator(std::make_unique<ROperator_Gemm<float>>(1.0, 1.0, 0, 0, in, wn, bn, out, act));
      in = out;
   }
   model.AddOutputTensorNameList({"Y"});
   model.Generate();
   model.OutputGenerated(name + ".hxx");
}

int main(int argc, char **argv)
{
   if (argc < 3) {
      std::cerr << "usage: ref_emit <onnx dir> <list file>\n";
      return 2;
   }
   const std::string dir = argv[1];
   std::ifstream list(argv[2]);
   std::vector<std::string> names;
   std::vector<size_t> ninputs;
   for (std::string n; std::getline(list, n);) {
      if (n.empty() || n[0] == '#') continue;
      names.push_back(n);
   }
   for (const auto &n : names) {
      RModelParser_ONNX parser;
      RModel model = parser.Parse(dir + "/" + n + ".onnx");
      model.Generate();
      model.OutputGenerated(n + ".hxx");
      ninputs.push_back(model.GetInputTensorNames().size());
   }
   emit_mlp("MLP_C1", 1024);
   names.push_back("MLP_C1");
   ninputs.push_back(1);

   // One translation unit per model: the emitted headers paste their helper functions on demand,
   // so two of them cannot share a translation unit (nor, safely, a shared library).
   for (size_t m = 0; m < names.size(); ++m) {
      const auto &n = names[m];
      std::ofstream tu("ref_" + n + ".cxx");
      tu << "#include \"" << n << ".hxx\"\n#include <cstring>\n#include <string>\n"
         << "static std::string g_err;\n"
         << "extern \"C\" const char *ref_last_error(void) { return g_err.c_str(); }\n"
         << "extern \"C\" int ref_ninputs(void) { return " << ninputs[m] << "; }\n"
         << "extern \"C\" long ref_run(const float *const *x, const char *dir, float *out, long cap) {\n"
         << "   try {\n"
         << "      SOFIE_" << n << "::Session s(std::string(dir) + \"/" << n << ".dat\");\n"
         << "      std::vector<float> y = s.infer(";
      for (size_t i = 0; i < ninputs[m]; ++i) tu << (i ? ", " : "") << "x[" << i << "]";
      tu << ");\n"
         << "      const long n = long(y.size());\n"
         << "      std::memcpy(out, y.data(), sizeof(float) * size_t(n < cap ? n : cap));\n"
         << "      return n;\n"
         << "   } catch (const std::exception &e) { g_err = e.what(); return -3; }\n"
         << "}\n";
   }
   return 0;
}
