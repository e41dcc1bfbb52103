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
// (tests/models/LowRankModelGenerator.cxx:36-51), and finally writes ref_models_gen.inc: one
// wrapper per model so that ref_models.cxx can expose them through one C function.
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
   for (std::string n; std::getline(list, n);) {
      if (n.empty() || n[0] == '#') continue;
      names.push_back(n);
   }
   for (const auto &n : names) {
      RModelParser_ONNX parser;
      RModel model = parser.Parse(dir + "/" + n + ".onnx");
      model.Generate();
      model.OutputGenerated(n + ".hxx");
   }
   emit_mlp("MLP_C1", 1024);
   names.push_back("MLP_C1");

   std::ofstream inc("ref_models_gen.inc");
   for (const auto &n : names) inc << "#include \"" << n << ".hxx\"\n";
   for (const auto &n : names)
      inc << "static std::vector<float> run_" << n << "(const float *x, const std::string &dir) {\n"
          << "   SOFIE_" << n << "::Session s(dir + \"/" << n << ".dat\");\n"
          << "   return s.infer(const_cast<float *>(x));\n}\n";
   inc << "static const RefModel kModels[] = {\n";
   for (const auto &n : names) inc << "   {\"" << n << "\", run_" << n << "},\n";
   inc << "};\n";
   return 0;
}
