// Test infrastructure: drives the UNMODIFIED reference generator (linked from oracle/_ref) to emit
// the CPU inference code it produces for the pinned models, i.e. the code whose results this
// repository's kernels must reproduce.
//
//   ref_emit <onnx dir> <list file>
//
// For every line "<Name>" of the list file it parses <onnx dir>/<Name>.onnx with the reference's
// ONNX parser and calls RModel::Generate() + OutputGenerated(), which writes <Name>.hxx and the
// text weight file <Name>.dat into the current directory (core/src/RModel.cxx:1744-1828,2242).
// It also builds, through the reference's C++ model API the way the reference's own generators do
// (tests/models/LowRankModelGenerator.cxx:36-51):
//   MLP_C1        the benchmark MLP (fp32, 64 -> 256 -> 256 -> 10, Relu after the first two Gemms)
//   ConvNet_C4r   the conv-net configuration (8 x Conv3x3 -> BatchNormalization+Relu, GlobalAveragePool, Gemm 512 -> 1000)
//                 on 2 images of 32 x 32: the parity model;  ConvNet_C4t: the same network on 4 images of 224 x 224,
//                 the sample the CPU baseline is timed on
//   Encoder_C5r   the transformer-encoder configuration in fp32 on the DEQUANTISED int8 weights, 2 layers, 2 sequences of
//                 128 tokens (LayerNormalization, Gemm, ScaledDotProductAttention, Gelu, Add): the parity model;
//                 Encoder_C5t: 6 layers, 2 sequences, the CPU baseline's sample
//   MatMul_C2, Gemm_C3   fp32 products of two INPUT matrices (4096^3; 8192^3 + bias + Gelu): what the reference can run for
//                 the int8 / FP8 configurations, on dequantised operands (the timed "reference" arm of those workloads)
// Weights come from the counter-based generator of sofie_b200/synth.py, restated below, so the GPU side draws the very
// same values.  Models marked for it write their weights as a safetensors file (binary) instead of text.
// Finally it writes ref_<Name>.cxx per model: C entry points around the emitted Session (ref_run: construct, infer
// once, destroy; ref_open / ref_infer / ref_close: a Session kept alive for timing), built into its own shared library.
#include "SOFIE/RModel.hxx"
#include "SOFIE/RModelParser_ONNX.hxx"
#include "SOFIE/operators/ROperator_BasicBinary.hxx"
#include "SOFIE/operators/ROperator_BatchNormalization.hxx"
#include "SOFIE/operators/ROperator_Conv.hxx"
#include "SOFIE/operators/ROperator_Gelu.hxx"
#include "SOFIE/operators/ROperator_Gemm.hxx"
#include "SOFIE/operators/ROperator_LayerNormalization.hxx"
#include "SOFIE/operators/ROperator_Pool.hxx"
#include "SOFIE/operators/ROperator_Reshape.hxx"
#include "SOFIE/operators/ROperator_SDPA.hxx"

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

// ---- sofie_b200/synth.py in C++: splitmix64 by counter, uniforms on [0,1), Irwin-Hall normals ---------------------------
struct Synth {
   uint64_t seed, k = 0;
   explicit Synth(uint64_t s) : seed(s) {}
   double uniform()
   {
      ++k;
      uint64_t z = seed + k * 0x9E3779B97F4A7C15ull;
      z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
      z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
      z ^= z >> 31;
      return double(z >> 11) * (1.0 / 9007199254740992.0);
   }
   double normal()
   {
      double a = uniform();
      for (int j = 1; j < 12; ++j) a = a + uniform();
      return a - 6.0;
   }
};
static uint64_t tensor_seed(uint64_t base, uint64_t index) { return base * 1000003ull + index * 7919ull + 12345ull; }
static std::vector<float> normal_f32(uint64_t seed, size_t n, double std_)
{
   Synth g(seed);
   std::vector<float> v(n);
   for (auto &x : v) x = float(g.normal() * std_);
   return v;
}
static std::vector<float> uniform_f32(uint64_t seed, size_t n, double lo, double hi)
{
   Synth g(seed);
   std::vector<float> v(n);
   for (auto &x : v) x = float(lo + (hi - lo) * g.uniform());
   return v;
}

static void add_f32(RModel &m, const std::string &name, std::vector<size_t> shape, std::vector<float> &data)
{
   m.AddInitializedTensor(name, ETensorType::FLOAT, shape, data.data());
}
static void add_i64(RModel &m, const std::string &name, std::vector<int64_t> data)
{
   m.AddInitializedTensor(name, ETensorType::INT64, std::vector<size_t>{data.size()}, data.data());
}

// The conv-net configuration (sofie_b200/convnet.py: raw_parameters) as the reference's operators.
static void emit_convnet(const std::string &name, size_t batch, size_t img, uint64_t seed)
{
   const size_t ch[9] = {3, 64, 64, 128, 128, 256, 256, 512, 512};
   const size_t strides[8] = {1, 2, 1, 2, 1, 2, 1, 2};
   RModel model(name, "now");
   model.AddInputTensorInfo("X", ETensorType::FLOAT, std::vector<Dim>{Dim(batch), Dim(3), Dim(img), Dim(img)});
   model.AddInputTensorName("X");
   std::string in = "X";
   for (size_t i = 0; i < 8; ++i) {
      const size_t cin = ch[i], cout = ch[i + 1];
      const std::string t = std::to_string(i);
      auto w = normal_f32(tensor_seed(seed, 10 * i + 0), cout * cin * 9, std::sqrt(2.0 / double(cin * 9)));
      auto gamma = uniform_f32(tensor_seed(seed, 10 * i + 1), cout, 0.5, 1.5);
      auto beta = normal_f32(tensor_seed(seed, 10 * i + 2), cout, 0.1);
      auto mean = normal_f32(tensor_seed(seed, 10 * i + 3), cout, 0.1);
      auto var = uniform_f32(tensor_seed(seed, 10 * i + 4), cout, 0.5, 1.5);
      add_f32(model, "w" + t, {cout, cin, 3, 3}, w);
      add_f32(model, "gamma" + t, {cout}, gamma);
      add_f32(model, "beta" + t, {cout}, beta);
      add_f32(model, "mean" + t, {cout}, mean);
      add_f32(model, "var" + t, {cout}, var);
      model.AddOperator(std::make_unique<ROperator_Conv<float>>("NOTSET", std::vector<size_t>{1, 1}, 1, std::vector<size_t>{3, 3},
                                                                std::vector<size_t>{1, 1, 1, 1}, std::vector<size_t>{strides[i], strides[i]},
                                                                in, "w" + t, "c" + t));
      model.AddOperator(std::make_unique<ROperator_BatchNormalization<float>>(1e-5f, 0.9f, 0, "c" + t, "gamma" + t, "beta" + t, "mean" + t,
                                                                              "var" + t, "r" + t, EActivationType::RELU));
      in = "r" + t;
   }
   RAttributes_Pool attr;
   model.AddOperator(std::make_unique<ROperator_Pool<float>>(GlobalAveragePool, attr, in, "pool"));
   model.AddOperator(std::make_unique<ROperator_Reshape>(Flatten, 1, "pool", "", "flat"));
   auto fcw = normal_f32(tensor_seed(seed, 100), 512 * 1000, std::sqrt(2.0 / 512.0));
   std::vector<float> fcb(1000, 0.f);
   add_f32(model, "fcw", {512, 1000}, fcw);
   add_f32(model, "fcb", {1000}, fcb);
   model.AddOperator(std::make_unique<ROperator_Gemm<float>>(1.0, 1.0, 0, 0, "flat", "fcw", "fcb", "Y"));
   model.AddOutputTensorNameList({"Y"});
   model.Generate(static_cast<std::underlying_type_t<Options>>(Options::kSafetensorsWeightFile));
   model.OutputGenerated(name + ".hxx");
}

// int8 per-output-channel weight of the encoder configuration (sofie_b200/encoder.py: qlinear), dequantised: float(q) * scale
static std::vector<float> dequantised_linear(uint64_t seed, size_t n_out, size_t n_in)
{
   auto w = normal_f32(seed, n_out * n_in, 0.02);
   for (size_t o = 0; o < n_out; ++o) {
      float amax = 0.f;
      for (size_t i = 0; i < n_in; ++i) amax = std::max(amax, std::fabs(w[o * n_in + i]));
      const float scale = amax / 127.0f;
      for (size_t i = 0; i < n_in; ++i) {
         float q = std::nearbyintf(w[o * n_in + i] / scale);
         q = std::min(127.f, std::max(-127.f, q));
         w[o * n_in + i] = q * scale;
      }
   }
   return w;
}

// The transformer-encoder configuration in fp32: pre-LayerNorm layers, heads of 64, FFN with Gelu, tokens as rows [batch*seq, d].
static void emit_encoder(const std::string &name, size_t batch, size_t layers, uint64_t seed)
{
   const size_t seq = 128, d = 512, heads = 8, ffn = 2048, m = batch * seq;
   RModel model(name, "now");
   model.AddInputTensorInfo("X", ETensorType::FLOAT, std::vector<Dim>{Dim(m), Dim(d)});
   model.AddInputTensorName("X");
   add_i64(model, "shape_bsd", {int64_t(batch), int64_t(seq), int64_t(d)});
   add_i64(model, "shape_md", {int64_t(m), int64_t(d)});
   std::vector<float> ones(d, 1.f), zeros(d, 0.f);
   add_f32(model, "ln_gamma", {d}, ones);
   add_f32(model, "ln_beta", {d}, zeros);
   std::string x = "X";
   for (size_t l = 0; l < layers; ++l) {
      const std::string t = "_" + std::to_string(l);
      auto ts = [&](size_t j) { return tensor_seed(seed, 10 * l + j); };
      auto wqkv = dequantised_linear(ts(0), 3 * d, d);
      auto bqkv = normal_f32(ts(1), 3 * d, 0.02);
      auto wo = dequantised_linear(ts(2), d, d);
      auto bo = normal_f32(ts(3), d, 0.02);
      auto w1 = dequantised_linear(ts(4), ffn, d);
      auto b1 = normal_f32(ts(5), ffn, 0.02);
      auto w2 = dequantised_linear(ts(6), d, ffn);
      auto b2 = normal_f32(ts(7), d, 0.02);
      const char *part[3] = {"q", "k", "v"};
      model.AddOperator(std::make_unique<ROperator_LayerNormalization<float>>(-1, 1e-5f, 1, x, "ln_gamma", "ln_beta", "h1" + t, "", ""));
      for (int p = 0; p < 3; ++p) {   // Q, K, V: the three row blocks of the packed projection
         std::vector<float> wp(wqkv.begin() + p * d * d, wqkv.begin() + (p + 1) * d * d), bp(bqkv.begin() + p * d, bqkv.begin() + (p + 1) * d);
         const std::string n = part[p] + t;
         add_f32(model, "w" + n, {d, d}, wp);
         add_f32(model, "b" + n, {d}, bp);
         model.AddOperator(std::make_unique<ROperator_Gemm<float>>(1.0, 1.0, 0, 1, "h1" + t, "w" + n, "b" + n, n));
         model.AddOperator(std::make_unique<ROperator_Reshape>(Reshape, 0, n, "shape_bsd", n + "3"));
      }
      model.AddOperator(std::make_unique<ROperator_SDPA<float>>("q" + t + "3", "k" + t + "3", "v" + t + "3", "att" + t + "3", "", 0.0f, heads));
      model.AddOperator(std::make_unique<ROperator_Reshape>(Reshape, 0, "att" + t + "3", "shape_md", "att" + t));
      add_f32(model, "wo" + t, {d, d}, wo);
      add_f32(model, "bo" + t, {d}, bo);
      model.AddOperator(std::make_unique<ROperator_Gemm<float>>(1.0, 1.0, 0, 1, "att" + t, "wo" + t, "bo" + t, "proj" + t));
      model.AddOperator(std::make_unique<ROperator_BasicBinary<float, EBasicBinaryOperator::Add>>("proj" + t, x, "x1" + t));
      model.AddOperator(std::make_unique<ROperator_LayerNormalization<float>>(-1, 1e-5f, 1, "x1" + t, "ln_gamma", "ln_beta", "h2" + t, "", ""));
      add_f32(model, "w1" + t, {ffn, d}, w1);
      add_f32(model, "b1" + t, {ffn}, b1);
      model.AddOperator(std::make_unique<ROperator_Gemm<float>>(1.0, 1.0, 0, 1, "h2" + t, "w1" + t, "b1" + t, "f" + t));
      model.AddOperator(std::make_unique<ROperator_Gelu>("f" + t, "g" + t));
      add_f32(model, "w2" + t, {d, ffn}, w2);
      add_f32(model, "b2" + t, {d}, b2);
      model.AddOperator(std::make_unique<ROperator_Gemm<float>>(1.0, 1.0, 0, 1, "g" + t, "w2" + t, "b2" + t, "ff" + t));
      const std::string out = l + 1 == layers ? "Y" : "x2" + t;
      model.AddOperator(std::make_unique<ROperator_BasicBinary<float, EBasicBinaryOperator::Add>>("ff" + t, "x1" + t, out));
      x = out;
   }
   model.AddOutputTensorNameList({"Y"});
   model.Generate(static_cast<std::underlying_type_t<Options>>(Options::kSafetensorsWeightFile));
   model.OutputGenerated(name + ".hxx");
}

// Y = A x B (+ bias, Gelu) with both matrices as INPUTS: no weight file, the operands are the caller's.
static void emit_product(const std::string &name, size_t n, bool bias_gelu)
{
   RModel model(name, "now");
   for (const char *in : {"A", "B"}) {
      model.AddInputTensorInfo(in, ETensorType::FLOAT, std::vector<Dim>{Dim(n), Dim(n)});
      model.AddInputTensorName(in);
   }
   if (!bias_gelu) {
      model.AddOperator(std::make_unique<ROperator_Gemm<float>>(1.0, 0.0, 0, 0, "A", "B", "Y"));
   } else {
      model.AddInputTensorInfo("C", ETensorType::FLOAT, std::vector<Dim>{Dim(n)});
      model.AddInputTensorName("C");
      model.AddOperator(std::make_unique<ROperator_Gemm<float>>(1.0, 1.0, 0, 0, "A", "B", "C", "P"));
      model.AddOperator(std::make_unique<ROperator_Gelu>("P", "Y"));
   }
   model.AddOutputTensorNameList({"Y"});
   model.Generate();
   model.OutputGenerated(name + ".hxx");
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
   std::vector<std::string> weights;   // extension of each model's weight file
   weights.assign(names.size(), ".dat");
   auto built = [&](const std::string &n, size_t nin, const std::string &ext) { names.push_back(n); ninputs.push_back(nin); weights.push_back(ext); };
   emit_mlp("MLP_C1", 1024);
   built("MLP_C1", 1, ".dat");
   emit_convnet("ConvNet_C4r", 2, 32, 11);
   built("ConvNet_C4r", 1, ".safetensors");
   emit_convnet("ConvNet_C4t", 4, 224, 11);
   built("ConvNet_C4t", 1, ".safetensors");
   emit_encoder("Encoder_C5r", 2, 2, 7);
   built("Encoder_C5r", 1, ".safetensors");
   emit_encoder("Encoder_C5t", 2, 6, 7);
   built("Encoder_C5t", 1, ".safetensors");
   emit_product("MatMul_C2", 4096, false);
   built("MatMul_C2", 2, ".dat");
   emit_product("Gemm_C3", 8192, true);
   built("Gemm_C3", 3, ".dat");

   // One translation unit per model: the emitted headers paste their helper functions on demand,
   // so two of them cannot share a translation unit (nor, safely, a shared library).
   for (size_t m = 0; m < names.size(); ++m) {
      const auto &n = names[m];
      std::string args;
      for (size_t i = 0; i < ninputs[m]; ++i) args += std::string(i ? ", " : "") + "x[" + std::to_string(i) + "]";
      std::ofstream tu("ref_" + n + ".cxx");
      tu << "#include \"" << n << ".hxx\"\n#include <cstring>\n#include <string>\n"
         << "using Session = SOFIE_" << n << "::Session;\n"
         << "static std::string g_err;\n"
         << "extern \"C\" const char *ref_last_error(void) { return g_err.c_str(); }\n"
         << "extern \"C\" int ref_ninputs(void) { return " << ninputs[m] << "; }\n"
         << "extern \"C\" void *ref_open(const char *dir) {\n"
         << "   try { return new Session(std::string(dir) + \"/" << n << weights[m] << "\"); }\n"
         << "   catch (const std::exception &e) { g_err = e.what(); return nullptr; }\n"
         << "}\n"
         << "extern \"C\" void ref_close(void *s) { delete static_cast<Session *>(s); }\n"
         << "extern \"C\" long ref_infer(void *s, const float *const *x, float *out, long cap) {\n"
         << "   try {\n"
         << "      std::vector<float> y = static_cast<Session *>(s)->infer(" << args << ");\n"
         << "      const long n = long(y.size());\n"
         << "      if (out) std::memcpy(out, y.data(), sizeof(float) * size_t(n < cap ? n : cap));\n"
         << "      return n;\n"
         << "   } catch (const std::exception &e) { g_err = e.what(); return -3; }\n"
         << "}\n"
         << "extern \"C\" long ref_run(const float *const *x, const char *dir, float *out, long cap) {\n"
         << "   void *s = ref_open(dir);\n"
         << "   if (!s) return -3;\n"
         << "   const long n = ref_infer(s, x, out, cap);\n"
         << "   ref_close(s);\n"
         << "   return n;\n"
         << "}\n";
   }
   return 0;
}
