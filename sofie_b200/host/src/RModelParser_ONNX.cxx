// ONNX wire reader and node -> operator translation (see SOFIE_B200/RModelParser_ONNX.hxx).
#include "SOFIE_B200/RModelParser_ONNX.hxx"

#include <cstring>
#include <fstream>
#include <functional>
#include <iostream>
#include <set>

#include "SOFIE_B200/operators/OperatorList.hxx"

namespace SOFIE_B200 {
namespace onnx_wire {

namespace {

// One protobuf message: a cursor over [p, end)
struct Reader {
   const uint8_t *p, *end;
   bool Done() const { return p >= end; }
   uint64_t Varint()
   {
      uint64_t v = 0;
      int shift = 0;
      while (p < end) {
         const uint8_t b = *p++;
         v |= uint64_t(b & 0x7f) << shift;
         if (!(b & 0x80)) return v;
         shift += 7;
         if (shift > 63) break;
      }
      throw std::runtime_error("SOFIE_B200 ONNX reader: truncated varint");
   }
   // reads a key; returns field number, sets wire type
   int Key(int &wt)
   {
      const uint64_t k = Varint();
      wt = int(k & 7);
      return int(k >> 3);
   }
   Reader Sub()
   {
      const uint64_t n = Varint();
      if (n > uint64_t(end - p)) throw std::runtime_error("SOFIE_B200 ONNX reader: length-delimited field overruns the message");
      Reader r{p, p + n};
      p += n;
      return r;
   }
   std::string Str()
   {
      Reader r = Sub();
      return std::string(reinterpret_cast<const char *>(r.p), size_t(r.end - r.p));
   }
   void Skip(int wt)
   {
      switch (wt) {
      case 0: Varint(); break;
      case 1: p += 8; break;
      case 2: Sub(); break;
      case 5: p += 4; break;
      default: throw std::runtime_error("SOFIE_B200 ONNX reader: unsupported wire type " + std::to_string(wt));
      }
      if (p > end) throw std::runtime_error("SOFIE_B200 ONNX reader: field overruns the message");
   }
   float F32()
   {
      float f;
      if (end - p < 4) throw std::runtime_error("SOFIE_B200 ONNX reader: truncated fixed32");
      std::memcpy(&f, p, 4);
      p += 4;
      return f;
   }
};

void PackedInts(Reader &r, int wt, std::vector<int64_t> &out)
{
   if (wt == 0) { out.push_back(int64_t(r.Varint())); return; }
   Reader s = r.Sub();
   while (!s.Done()) out.push_back(int64_t(s.Varint()));
}
void PackedFloats(Reader &r, int wt, std::vector<float> &out)
{
   if (wt == 5) { out.push_back(r.F32()); return; }
   Reader s = r.Sub();
   while (!s.Done()) out.push_back(s.F32());
}

size_t ElemSize(int dt)
{
   switch (dt) {
   case 1: case 6: case 12: return 4;
   case 7: case 11: case 13: return 8;
   case 2: case 3: case 9: case 17: return 1;
   case 4: case 5: case 10: case 16: return 2;
   default: return 0;
   }
}

Tensor ParseTensor(Reader r)
{
   Tensor t;
   std::vector<int64_t> dims, i32, i64;
   std::vector<float> f32;
   std::string raw;
   bool hasRaw = false;
   while (!r.Done()) {
      int wt;
      switch (r.Key(wt)) {
      case 1: PackedInts(r, wt, dims); break;
      case 2: t.data_type = int(r.Varint()); break;
      case 4: PackedFloats(r, wt, f32); break;
      case 5: PackedInts(r, wt, i32); break;
      case 7: PackedInts(r, wt, i64); break;
      case 8: t.name = r.Str(); break;
      case 9: raw = r.Str(); hasRaw = true; break;
      case 13: case 14: throw std::runtime_error("SOFIE_B200 ONNX reader: tensors with external data are not supported");
      default: r.Skip(wt);
      }
   }
   for (auto d : dims) t.dims.push_back(size_t(d));
   const size_t len = ConvertShapeToLength(t.dims), es = ElemSize(t.data_type);
   if (es == 0) throw std::runtime_error("SOFIE_B200 ONNX reader: tensor " + t.name + " has unsupported data type " + std::to_string(t.data_type));
   std::shared_ptr<void> buf(malloc(len * es + 8), free);
   if (hasRaw) {
      if (raw.size() != len * es) throw std::runtime_error("SOFIE_B200 ONNX reader: raw_data of tensor " + t.name + " has the wrong size");
      std::memcpy(buf.get(), raw.data(), raw.size());
   } else if (t.data_type == 1) {
      if (f32.size() != len) throw std::runtime_error("SOFIE_B200 ONNX reader: float_data of tensor " + t.name + " has the wrong size");
      std::memcpy(buf.get(), f32.data(), len * 4);
   } else if (t.data_type == 7) {
      if (i64.size() != len) throw std::runtime_error("SOFIE_B200 ONNX reader: int64_data of tensor " + t.name + " has the wrong size");
      std::memcpy(buf.get(), i64.data(), len * 8);
   } else {
      // int32_data carries int32 and every narrower integer type, one value per element
      if (i32.size() != len) throw std::runtime_error("SOFIE_B200 ONNX reader: int32_data of tensor " + t.name + " has the wrong size");
      for (size_t i = 0; i < len; ++i) {
         const int32_t v = int32_t(i32[i]);
         if (es == 4) static_cast<int32_t *>(buf.get())[i] = v;
         else if (es == 2) static_cast<uint16_t *>(buf.get())[i] = uint16_t(v);
         else static_cast<uint8_t *>(buf.get())[i] = uint8_t(v);
      }
   }
   t.data = buf;
   return t;
}

Attribute ParseAttribute(Reader r)
{
   Attribute a;
   while (!r.Done()) {
      int wt;
      switch (r.Key(wt)) {
      case 1: a.name = r.Str(); break;
      case 2: a.f = r.F32(); a.hasF = true; break;
      case 3: a.i = int64_t(r.Varint()); a.hasI = true; break;
      case 4: a.s = r.Str(); a.hasS = true; break;
      case 7: PackedFloats(r, wt, a.floats); break;
      case 8: PackedInts(r, wt, a.ints); break;
      default: r.Skip(wt);
      }
   }
   return a;
}

Node ParseNode(Reader r)
{
   Node n;
   while (!r.Done()) {
      int wt;
      switch (r.Key(wt)) {
      case 1: n.input.push_back(r.Str()); break;
      case 2: n.output.push_back(r.Str()); break;
      case 3: n.name = r.Str(); break;
      case 4: n.op_type = r.Str(); break;
      case 5: { Attribute a = ParseAttribute(r.Sub()); n.attr[a.name] = a; break; }
      default: r.Skip(wt);
      }
   }
   return n;
}

ValueInfo ParseValueInfo(Reader r)
{
   ValueInfo v;
   while (!r.Done()) {
      int wt;
      const int f = r.Key(wt);
      if (f == 1) v.name = r.Str();
      else if (f == 2) {  // TypeProto
         Reader t = r.Sub();
         while (!t.Done()) {
            int wt2;
            if (t.Key(wt2) != 1) { t.Skip(wt2); continue; }  // tensor_type
            Reader tt = t.Sub();
            while (!tt.Done()) {
               int wt3;
               const int f3 = tt.Key(wt3);
               if (f3 == 1) v.elem_type = int(tt.Varint());
               else if (f3 == 2) {  // TensorShapeProto
                  Reader sh = tt.Sub();
                  while (!sh.Done()) {
                     int wt4;
                     if (sh.Key(wt4) != 1) { sh.Skip(wt4); continue; }
                     Reader d = sh.Sub();
                     Dim dim;
                     while (!d.Done()) {
                        int wt5;
                        const int f5 = d.Key(wt5);
                        if (f5 == 1) dim = Dim(size_t(d.Varint()));
                        else if (f5 == 2) dim = Dim(d.Str(), 0);
                        else d.Skip(wt5);
                     }
                     v.shape.push_back(dim);
                  }
               } else tt.Skip(wt3);
            }
         }
      } else r.Skip(wt);
   }
   return v;
}

}  // namespace

Graph LoadModel(const std::string &filename)
{
   std::ifstream f(filename, std::ios::binary);
   if (!f.is_open()) throw std::runtime_error("SOFIE_B200 ONNX parser: cannot open " + filename);
   std::vector<uint8_t> buf((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
   Reader model{buf.data(), buf.data() + buf.size()};
   Graph g;
   bool found = false;
   while (!model.Done()) {
      int wt;
      if (model.Key(wt) != 7) { model.Skip(wt); continue; }  // ModelProto.graph
      Reader gr = model.Sub();
      found = true;
      while (!gr.Done()) {
         int wt2;
         switch (gr.Key(wt2)) {
         case 1: g.node.push_back(ParseNode(gr.Sub())); break;
         case 5: g.initializer.push_back(ParseTensor(gr.Sub())); break;
         case 11: g.input.push_back(ParseValueInfo(gr.Sub())); break;
         case 12: g.output.push_back(ParseValueInfo(gr.Sub())); break;
         default: gr.Skip(wt2);
         }
      }
   }
   if (!found) throw std::runtime_error("SOFIE_B200 ONNX parser: " + filename + " has no graph");
   return g;
}

}  // namespace onnx_wire

// ---------------------------------------------------------------------------------------------------
namespace {

using onnx_wire::Attribute;
using onnx_wire::Graph;
using onnx_wire::Node;

std::vector<size_t> Ints(const Node &n, const char *name)
{
   auto it = n.attr.find(name);
   if (it == n.attr.end()) return {};
   return std::vector<size_t>(it->second.ints.begin(), it->second.ints.end());
}
int64_t Int(const Node &n, const char *name, int64_t def)
{
   auto it = n.attr.find(name);
   return it == n.attr.end() ? def : it->second.i;
}
float Float(const Node &n, const char *name, float def)
{
   auto it = n.attr.find(name);
   return it == n.attr.end() ? def : it->second.f;
}
std::string Str(const Node &n, const char *name, const std::string &def)
{
   auto it = n.attr.find(name);
   return it == n.attr.end() ? def : it->second.s;
}
std::string In(const Node &n, size_t i) { return i < n.input.size() ? n.input[i] : std::string(); }

using Maker = std::function<std::unique_ptr<ROperator>(const Node &)>;

const std::map<std::string, Maker> &Makers()
{
   static const std::map<std::string, Maker> m = {
      {"Gemm", [](const Node &n) -> std::unique_ptr<ROperator> {
          const float alpha = Float(n, "alpha", 1.f), beta = Float(n, "beta", 1.f);
          const int64_t ta = Int(n, "transA", 0), tb = Int(n, "transB", 0);
          if (n.input.size() > 2 && !n.input[2].empty())
             return std::make_unique<ROperator_Gemm<float>>(alpha, beta, ta, tb, n.input[0], n.input[1], n.input[2], n.output[0]);
          return std::make_unique<ROperator_Gemm<float>>(alpha, beta, ta, tb, n.input[0], n.input[1], n.output[0]);
       }},
      {"MatMul", [](const Node &n) -> std::unique_ptr<ROperator> {
          return std::make_unique<ROperator_Gemm<float>>(1.f, 0.f, 0, 0, n.input[0], n.input[1], n.output[0]);
       }},
      {"Conv", [](const Node &n) -> std::unique_ptr<ROperator> {
          return std::make_unique<ROperator_Conv<float>>(Str(n, "auto_pad", "NOTSET"), Ints(n, "dilations"), size_t(Int(n, "group", 0)),
                                                         Ints(n, "kernel_shape"), Ints(n, "pads"), Ints(n, "strides"), n.input[0], n.input[1],
                                                         In(n, 2), n.output[0]);
       }},
      {"Relu", [](const Node &n) -> std::unique_ptr<ROperator> { return std::make_unique<ROperator_Relu<float>>(n.input[0], n.output[0]); }},
      {"LeakyRelu", [](const Node &n) -> std::unique_ptr<ROperator> {
          return std::make_unique<ROperator_LeakyRelu<float>>(Float(n, "alpha", 0.01f), n.input[0], n.output[0]);
       }},
      {"Sigmoid", [](const Node &n) -> std::unique_ptr<ROperator> { return std::make_unique<ROperator_Sigmoid<float>>(n.input[0], n.output[0]); }},
      {"Gelu", [](const Node &n) -> std::unique_ptr<ROperator> {
          return std::make_unique<ROperator_Gelu>(n.input[0], n.output[0], Str(n, "approximate", "none"));
       }},
      {"BatchNormalization", [](const Node &n) -> std::unique_ptr<ROperator> {
          return std::make_unique<ROperator_BatchNormalization<float>>(Float(n, "epsilon", 1e-5f), Float(n, "momentum", 0.9f),
                                                                       size_t(Int(n, "training_mode", 0)), n.input[0], n.input[1], n.input[2],
                                                                       n.input[3], n.input[4], n.output[0]);
       }},
      {"LayerNormalization", [](const Node &n) -> std::unique_ptr<ROperator> {
          // defaults of parsers/src/ParseLayerNormalization.cxx:17-19
          return std::make_unique<ROperator_LayerNormalization<float>>(int(Int(n, "axis", -1)), Float(n, "epsilon", 1e-5f),
                                                                       size_t(Int(n, "stash_type", 1)), n.input[0], In(n, 1), In(n, 2), n.output[0],
                                                                       n.output.size() > 1 ? n.output[1] : "", n.output.size() > 2 ? n.output[2] : "");
       }},
      {"Softmax", [](const Node &n) -> std::unique_ptr<ROperator> { return std::make_unique<ROperator_Softmax>(Int(n, "axis", -1), n.input[0], n.output[0]); }},
      {"LogSoftmax", [](const Node &n) -> std::unique_ptr<ROperator> { return std::make_unique<ROperator_Softmax>(Int(n, "axis", -1), n.input[0], n.output[0], true); }},
      {"ScaledDotProductAttention", [](const Node &n) -> std::unique_ptr<ROperator> {
          // inputs and attributes of parsers/src/ParseSDPA.cxx:10-29
          if (n.input.size() < 3) throw std::runtime_error("SOFIE ParseSDPA: need at least 3 inputs (query, key, value)");
          return std::make_unique<ROperator_SDPA<float>>(n.input[0], n.input[1], n.input[2], n.output[0], In(n, 3), Float(n, "scale", 0.f),
                                                         size_t(Int(n, "num_heads", 0)));
       }},
      {"Split", [](const Node &n) -> std::unique_ptr<ROperator> {
          return std::make_unique<ROperator_Split>(Int(n, "axis", 0), n.input[0], In(n, 1), n.output);
       }},
      {"Transpose", [](const Node &n) -> std::unique_ptr<ROperator> {
          auto p = Ints(n, "perm");
          return std::make_unique<ROperator_Transpose>(std::vector<int64_t>(p.begin(), p.end()), n.input[0], n.output[0]);
       }},
      {"Add", [](const Node &n) -> std::unique_ptr<ROperator> { return std::make_unique<ROperator_BasicBinary<float, EBasicBinaryOperator::Add>>(n.input[0], n.input[1], n.output[0]); }},
      {"Sub", [](const Node &n) -> std::unique_ptr<ROperator> { return std::make_unique<ROperator_BasicBinary<float, EBasicBinaryOperator::Sub>>(n.input[0], n.input[1], n.output[0]); }},
      {"Mul", [](const Node &n) -> std::unique_ptr<ROperator> { return std::make_unique<ROperator_BasicBinary<float, EBasicBinaryOperator::Mul>>(n.input[0], n.input[1], n.output[0]); }},
      {"Div", [](const Node &n) -> std::unique_ptr<ROperator> { return std::make_unique<ROperator_BasicBinary<float, EBasicBinaryOperator::Div>>(n.input[0], n.input[1], n.output[0]); }},
      {"GlobalAveragePool", [](const Node &n) -> std::unique_ptr<ROperator> { return std::make_unique<ROperator_Pool<float>>(GlobalAveragePool, n.input[0], n.output[0]); }},
      {"Flatten", [](const Node &n) -> std::unique_ptr<ROperator> { return std::make_unique<ROperator_Reshape>(Flatten, int(Int(n, "axis", 1)), n.input[0], "", n.output[0]); }},
      {"Reshape", [](const Node &n) -> std::unique_ptr<ROperator> { return std::make_unique<ROperator_Reshape>(Reshape, int(Int(n, "allowzero", 0)), n.input[0], In(n, 1), n.output[0]); }},
      {"Squeeze", [](const Node &n) -> std::unique_ptr<ROperator> { return std::make_unique<ROperator_Reshape>(Squeeze, 0, n.input[0], In(n, 1), n.output[0]); }},
      {"Unsqueeze", [](const Node &n) -> std::unique_ptr<ROperator> { return std::make_unique<ROperator_Reshape>(Unsqueeze, 0, n.input[0], In(n, 1), n.output[0]); }},
      {"QLinearMatMul", [](const Node &n) -> std::unique_ptr<ROperator> {
          return std::make_unique<ROperator_QLinearMatMul>(n.input[0], n.input[1], n.input[2], n.input[3], n.input[4], n.input[5], n.input[6], In(n, 7), n.output[0]);
       }},
      {"QLinearConv", [](const Node &n) -> std::unique_ptr<ROperator> {
          return std::make_unique<ROperator_QLinearConv>(Str(n, "auto_pad", "NOTSET"), Ints(n, "dilations"), size_t(Int(n, "group", 0)), Ints(n, "kernel_shape"),
                                                         Ints(n, "pads"), Ints(n, "strides"), n.input[0], n.input[1], n.input[2], n.input[3], n.input[4],
                                                         n.input[5], n.input[6], In(n, 7), In(n, 8), n.output[0]);
       }},
      {"ScaledGemm", [](const Node &n) -> std::unique_ptr<ROperator> {
          // FP8 e4m3 product with per-row / per-column fp32 scales and a bias (no counterpart among the reference's operators):
          // inputs A, B, row_scale, col_scale, bias (the last three optional); attributes transB, to (ONNX type of Y, default BFLOAT16)
          return std::make_unique<ROperator_ScaledGemm>(int(Int(n, "transB", 0)), n.input[0], n.input[1], In(n, 2), In(n, 3), In(n, 4), n.output[0],
                                                        static_cast<ETensorType>(Int(n, "to", 16)));
       }},
      {"QuantizeLinear", [](const Node &n) -> std::unique_ptr<ROperator> {
          return std::make_unique<ROperator_QuantizeLinear>(false, Int(n, "axis", 1), n.input[0], n.input[1], In(n, 2), n.output[0]);
       }},
      {"DequantizeLinear", [](const Node &n) -> std::unique_ptr<ROperator> {
          return std::make_unique<ROperator_QuantizeLinear>(true, Int(n, "axis", 1), n.input[0], n.input[1], In(n, 2), n.output[0]);
       }},
   };
   return m;
}

ETensorType TypeOf(int onnxType)
{
   if (onnxType < 0 || onnxType > 17) throw std::runtime_error("SOFIE_B200 ONNX parser: data type " + std::to_string(onnxType) + " not supported");
   return static_cast<ETensorType>(onnxType);
}

}  // namespace

std::vector<std::string> RModelParser_ONNX::GetRegisteredOperators()
{
   std::vector<std::string> v;
   for (auto &kv : Makers()) v.push_back(kv.first);
   v.push_back("Identity");
   return v;
}

bool RModelParser_ONNX::CheckModel(std::string filename, bool verbose)
{
   Graph g = onnx_wire::LoadModel(filename);
   std::set<std::string> missing;
   for (auto &n : g.node)
      if (!Makers().count(n.op_type) && n.op_type != "Identity") missing.insert(n.op_type);
   if (verbose || !missing.empty())
      for (auto &m : missing) std::cout << "operator " << m << " is not supported" << std::endl;
   return missing.empty();
}

RModel RModelParser_ONNX::Parse(std::string filename, bool verbose)
{
   Graph g = onnx_wire::LoadModel(filename);
   RModel model(filename, "");
   std::set<std::string> initNames;
   for (auto &t : g.initializer) {
      model.AddInitializedTensor(t.name, TypeOf(t.data_type), t.dims, t.data);
      initNames.insert(t.name);
   }
   for (auto &v : g.input) {
      if (initNames.count(v.name)) continue;
      model.AddInputTensorInfo(v.name, TypeOf(v.elem_type), v.shape);
      model.AddInputTensorName(v.name);
   }
   std::set<std::string> graphOutputs;
   for (auto &v : g.output) graphOutputs.insert(v.name);

   // children of every node output, for the pair fusions (RModelParser_ONNX.cxx:1656-1673)
   std::map<std::string, std::vector<size_t>> consumers;
   for (size_t i = 0; i < g.node.size(); ++i)
      for (auto &in : g.node[i].input) consumers[in].push_back(i);

   std::map<std::string, std::string> rename;           // Identity outputs and absorbed Transposes
   std::map<std::string, bool> transposed;              // tensor is a last-two-axes transpose of rename[tensor]
   std::map<size_t, size_t> fuseInto;                   // consumer node index -> producer node index (MatMul+Add, Conv+Add)
   struct Dequantised { std::string weight, scale; int64_t axis; };
   std::map<std::string, Dequantised> dequantised;     // DequantizeLinear outputs folded into the contractions that read them
   auto resolve = [&](std::string n) {
      for (auto it = rename.find(n); it != rename.end(); it = rename.find(n)) n = it->second;
      return n;
   };

   for (size_t i = 0; i < g.node.size(); ++i) {
      Node n = g.node[i];
      if (n.output.empty()) continue;
      if (verbose) std::cout << "\tCreating operator " << n.op_type << std::endl;
      const std::vector<size_t> &ch = consumers[n.output[0]];
      const bool single = ch.size() == 1 && !graphOutputs.count(n.output[0]);

      if (n.op_type == "Identity") { rename[n.output[0]] = n.input[0]; continue; }
      if (n.op_type == "DequantizeLinear" && initNames.count(resolve(n.input[0])) && n.input.size() >= 2 && initNames.count(resolve(n.input[1])) &&
          (n.input.size() < 3 || n.input[2].empty() || initNames.count(resolve(n.input[2])))) {
         // DequantizeLinear of a weight that only feeds contractions as their B operand: folded into those contractions
         bool onlyB = !ch.empty() && !graphOutputs.count(n.output[0]);
         for (auto c : ch) {
            const Node &u = g.node[c];
            onlyB = onlyB && (u.op_type == "MatMul" || u.op_type == "Gemm") && u.input.size() >= 2 && u.input[1] == n.output[0] && u.input[0] != n.output[0];
         }
         if (onlyB && model.GetTensorType(resolve(n.input[0])) == ETensorType::INT8) {
            if (n.input.size() >= 3 && !n.input[2].empty()) {
               auto zp = model.GetTensorData<int8_t>(resolve(n.input[2]));
               for (auto z : zp) if (z != 0) throw std::runtime_error("SOFIE DequantizeLinear of a weight: only symmetric quantisation (zero point 0) is folded");
            }
            dequantised[n.output[0]] = {resolve(n.input[0]), resolve(n.input[1]), Int(n, "axis", 1)};
            continue;
         }
      }
      if (n.op_type == "Transpose") {
         // only a transpose of the last two axes feeding MatMul nodes is absorbed (RModelParser_ONNX.cxx:1186-1197)
         auto perm = Ints(n, "perm");
         bool lastTwo = perm.size() >= 2;
         for (size_t k = 0; lastTwo && k + 2 < perm.size(); ++k) lastTwo = perm[k] == k;
         if (lastTwo) lastTwo = perm[perm.size() - 2] == perm.size() - 1 && perm[perm.size() - 1] == perm.size() - 2;
         bool allMatMul = !ch.empty() && !graphOutputs.count(n.output[0]);
         for (auto c : ch) allMatMul = allMatMul && g.node[c].op_type == "MatMul";
         if (lastTwo && allMatMul) {
            rename[n.output[0]] = n.input[0];
            transposed[n.output[0]] = true;
            continue;
         }
         // any other Transpose is an operator of its own (ROperator_Transpose)
      }
      // a fused consumer was already emitted together with its producer
      if (fuseInto.count(i)) continue;

      std::vector<bool> tflag;
      for (auto &in : n.input) {
         tflag.push_back(transposed.count(in) != 0);
         in = resolve(in);
      }
      if (!Makers().count(n.op_type)) {
         std::cout << "operator " << n.op_type << " is not supported" << std::endl;
         throw std::runtime_error("SOFIE Operator type " + n.op_type + " is not yet supported");
      }

      if (n.op_type == "MatMul") {
         const bool ta = tflag[0], tb = tflag[1];
         // MatMul followed only by an Add: Gemm with C (ParseFuseMatMulAdd.cxx:23-40), placed where the MatMul stands
         // if the other operand of the Add already exists, else the pair is left to the fusion pass
         if (single && g.node[ch[0]].op_type == "Add" && g.node[ch[0]].input.size() == 2) {
            const Node &add = g.node[ch[0]];
            const std::string other = resolve(add.input[0] == n.output[0] ? add.input[1] : add.input[0]);
            if (other != n.output[0] && model.CheckIfTensorAlreadyExist(other) && model.IsInitializedTensor(other)) {
               auto op = std::make_unique<ROperator_Gemm<float>>(1.f, 1.f, ta, tb, n.input[0], n.input[1], other, add.output[0]);
               if (auto dq = dequantised.find(n.input[1]); dq != dequantised.end()) op->SetDequantisedWeight(dq->second.weight, dq->second.scale, dq->second.axis);
               model.AddOperator(std::move(op));
               fuseInto[ch[0]] = i;
               continue;
            }
         }
         auto op = std::make_unique<ROperator_Gemm<float>>(1.f, 0.f, ta, tb, n.input[0], n.input[1], n.output[0]);
         if (auto dq = dequantised.find(n.input[1]); dq != dequantised.end()) op->SetDequantisedWeight(dq->second.weight, dq->second.scale, dq->second.axis);
         model.AddOperator(std::move(op));
         continue;
      }
      if (n.op_type == "Gemm" && n.input.size() >= 2 && dequantised.count(n.input[1])) {
         const auto &dq = dequantised.at(n.input[1]);
         auto made = Makers().at("Gemm")(n);
         static_cast<ROperator_Gemm<float> *>(made.get())->SetDequantisedWeight(dq.weight, dq.scale, dq.axis);
         model.AddOperator(std::move(made));
         continue;
      }
      if (n.op_type == "Conv" && n.input.size() == 2 && single && g.node[ch[0]].op_type == "Add") {
         // Conv followed only by an Add of a per-channel constant: the Add is the bias (ParseFuseConvAdd.cxx:57-61)
         const Node &add = g.node[ch[0]];
         const std::string other = resolve(add.input[0] == n.output[0] ? add.input[1] : add.input[0]);
         if (initNames.count(other)) {
            const auto &bs = model.GetTensorShape(other);
            const auto &ws = model.GetTensorShape(n.input[1]);
            size_t nonOne = 0, pos = 0;
            for (size_t k = 0; k < bs.size(); ++k)
               if (bs[k] != 1) { ++nonOne; pos = k; }
            // [1,K,1,1] or [K,1,1]: the only non-unit dimension sits where the channel axis of the output is
            const bool perChannel = ConvertShapeToLength(bs) == ws[0] && nonOne <= 1 && bs.size() + 1 >= ws.size() && pos == bs.size() - (ws.size() - 1);
            if (perChannel) {
               Node fused = n;
               fused.input.push_back(other);
               fused.output[0] = add.output[0];
               model.AddOperator(Makers().at("Conv")(fused));
               fuseInto[ch[0]] = i;
               continue;
            }
         }
      }
      model.AddOperator(Makers().at(n.op_type)(n));
   }
   std::vector<std::string> outs;
   for (auto &v : g.output) outs.push_back(resolve(v.name));
   model.AddOutputTensorNameList(outs);
   return model;
}

}  // namespace SOFIE_B200
