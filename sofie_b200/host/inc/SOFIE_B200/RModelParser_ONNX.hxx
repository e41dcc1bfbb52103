// ONNX front-end of the B200 generator for the hot-path node types.
//
// Same entry points as the reference parser (parsers/inc/SOFIE/RModelParser_ONNX.hxx:60-123):
// Parse(filename) returns an RModel, CheckModel(filename) lists the node types that have no
// operator.  The file is decoded with a small protobuf wire reader, as the reference does
// (parsers/src/onnx.hxx:19-120), so no protobuf library is needed.  Node types covered: Gemm,
// MatMul, Conv, Relu, LeakyRelu, Sigmoid, Gelu, BatchNormalization, LayerNormalization, Softmax,
// LogSoftmax, Add / Sub / Mul / Div, GlobalAveragePool, Flatten, Reshape, Squeeze, Unsqueeze,
// Identity, and the quantised nodes the reference lacks: QLinearMatMul, QLinearConv,
// QuantizeLinear, DequantizeLinear.  The parser-level pair fusions of the reference are applied:
// MatMul + Add -> Gemm with C, Conv + Add(bias) -> Conv with bias, and a last-two-axes Transpose
// feeding a MatMul becomes its trans flag (parsers/src/RModelParser_ONNX.cxx:1182-1219);
// Gemm + Relu and BatchNormalization + Relu are folded later by RModel's fusion pass.
#pragma once
#include <map>
#include <string>
#include <vector>

#include "SOFIE_B200/RModel.hxx"

namespace SOFIE_B200 {

namespace onnx_wire {

struct Attribute {
   std::string name;
   float f = 0;
   int64_t i = 0;
   std::string s;
   std::vector<float> floats;
   std::vector<int64_t> ints;
   bool hasF = false, hasI = false, hasS = false;
};

struct Node {
   std::string op_type, name;
   std::vector<std::string> input, output;
   std::map<std::string, Attribute> attr;
};

struct Tensor {
   std::string name;
   int data_type = 1;
   std::vector<size_t> dims;
   std::shared_ptr<void> data;  // GetTypeSize(type) * length bytes
};

struct ValueInfo {
   std::string name;
   int elem_type = 1;
   std::vector<Dim> shape;
};

struct Graph {
   std::vector<Node> node;
   std::vector<Tensor> initializer;
   std::vector<ValueInfo> input, output;
};

Graph LoadModel(const std::string &filename);

}  // namespace onnx_wire

class RModelParser_ONNX {
public:
   RModel Parse(std::string filename, bool verbose = false);
   // true if every node of the model has a B200 operator; prints the unsupported ones otherwise
   bool CheckModel(std::string filename, bool verbose = false);
   // node types this parser creates operators for
   static std::vector<std::string> GetRegisteredOperators();
};

}  // namespace SOFIE_B200
