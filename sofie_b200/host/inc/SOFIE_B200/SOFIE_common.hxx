// Types shared by the B200 code generator: tensor element types, dimensions, generation options.
// Names, enumerator values and meanings follow the reference generator so that model-building
// code written against it reads the same here (core/inc/SOFIE/utils/SOFIE_common.hxx:29-60,
// core/inc/SOFIE/RModel_Base.hxx:19-54).
#pragma once
#include <cstddef>
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <vector>

namespace SOFIE_B200 {

// ONNX TensorProto.DataType numbering (the reference stops at BFLOAT16; FLOAT8E4M3FN is ONNX 17)
enum class ETensorType {
   UNDEFINED = 0, FLOAT = 1, UINT8 = 2, INT8 = 3, UINT16 = 4, INT16 = 5, INT32 = 6, INT64 = 7, STRING = 8, BOOL = 9,
   FLOAT16 = 10, DOUBLE = 11, UINT32 = 12, UINT64 = 13, COMPLEX64 = 14, COMPLEX28 = 15, BFLOAT16 = 16, FLOAT8E4M3FN = 17
};

enum class EActivationType { UNDEFINED = 0, RELU = 1, SOFTMAX = 2, SIGMOID = 3, LEAKYRELU = 4, TANH = 5, ELU = 6, GELU = 7, GELU_TANH = 8 };

enum class Options {
   kDefault = 0x0,
   kNoSession = 0x1,
   kNoWeightFile = 0x2,
   kGNN = 0x8,
   kGNNComponent = 0x10,
   kProfile = 0x20,
   kLowRankFactorize = 0x40,
   kKernelOnly = 0x80,
   kSafetensorsWeightFile = 0x100,
   kStridedInput = 0x200,
   kExternalStream = 0x400,
   kCustomMemory = 0x800,
   kDebug = 0x1000,
};

inline std::underlying_type_t<Options> operator|(Options a, Options b)
{
   return static_cast<std::underlying_type_t<Options>>(a) | static_cast<std::underlying_type_t<Options>>(b);
}
inline std::underlying_type_t<Options> operator|(std::underlying_type_t<Options> a, Options b)
{
   return a | static_cast<std::underlying_type_t<Options>>(b);
}

// A dimension: a number, or a named parameter that Generate*() replaces by the batch size when
// it is called input_size, batch_size or bs (core/src/RModel.cxx:676-685).
struct Dim {
   bool isParam = false;
   size_t dim = 0;
   std::string param;
   Dim() = default;
   Dim(size_t d) : dim(d) {}
   Dim(const std::string &p, size_t d = 0) : isParam(true), dim(d), param(p) {}
   std::string GetVal() const { return isParam ? param : std::to_string(dim); }
};

// One symbolic dimension (the reference's dynamic models take it as a Session constructor argument,
// tests/alpaka/TestAlpakaLinear.cxx:121-203) travels through shape inference as the number kSymbolicBase.  The base
// is far above any static size and a multiple of every alignment, so each size, stride or offset the generator derives
// from it is a * kSymbolicBase + b with small a and b, and reads back as "a * n + b" when the Session is emitted.
constexpr size_t kSymbolicBase = size_t(1) << 36;
struct SymbolicValue {
   long long a = 0, b = 0;   // a * n + b
};
// false when v is static (below half the base); throws when v is not linear in the symbol (a product of two symbolic
// sizes, a division that does not go through)
inline bool DecodeSymbolic(unsigned long long v, SymbolicValue &out)
{
   if (v < kSymbolicBase / 2) return false;
   const unsigned long long a = (v + kSymbolicBase / 2) / kSymbolicBase;
   const long long b = (long long)(v - a * kSymbolicBase);
   if (a >= (1ull << 26) || b >= (1ll << 32) || b <= -(1ll << 32))
      throw std::runtime_error("SOFIE_B200: a size is not linear in the symbolic dimension (value " + std::to_string(v) + ")");
   out.a = (long long)a;
   out.b = b;
   return true;
}

inline size_t GetTypeSize(ETensorType t)
{
   switch (t) {
   case ETensorType::FLOAT: case ETensorType::INT32: case ETensorType::UINT32: return 4;
   case ETensorType::DOUBLE: case ETensorType::INT64: case ETensorType::UINT64: return 8;
   case ETensorType::UINT8: case ETensorType::INT8: case ETensorType::BOOL: case ETensorType::FLOAT8E4M3FN: return 1;
   case ETensorType::UINT16: case ETensorType::INT16: case ETensorType::FLOAT16: case ETensorType::BFLOAT16: return 2;
   default: return 0;
   }
}

// C++ type used for a tensor of this element type in emitted code (bf16 / fp8 travel as raw bits)
inline std::string ConvertTypeToString(ETensorType t)
{
   switch (t) {
   case ETensorType::FLOAT: return "float";
   case ETensorType::INT8: return "int8_t";
   case ETensorType::UINT8: return "uint8_t";
   case ETensorType::INT32: return "int32_t";
   case ETensorType::INT64: return "int64_t";
   case ETensorType::BFLOAT16: return "uint16_t";
   case ETensorType::FLOAT8E4M3FN: return "uint8_t";
   case ETensorType::DOUBLE: return "double";
   case ETensorType::BOOL: return "uint8_t";
   default: return "other";
   }
}

// sofie_b200_dtype enumerator name for emitted calls; empty if the runtime has no such type
inline std::string ConvertTypeToRuntimeEnum(ETensorType t)
{
   switch (t) {
   case ETensorType::FLOAT: return "SOFIE_B200_F32";
   case ETensorType::BFLOAT16: return "SOFIE_B200_BF16";
   case ETensorType::INT8: return "SOFIE_B200_I8";
   case ETensorType::FLOAT8E4M3FN: return "SOFIE_B200_F8E4M3";
   case ETensorType::INT32: return "SOFIE_B200_I32";
   case ETensorType::UINT8: return "SOFIE_B200_U8";
   default: return "";
   }
}

inline size_t ConvertShapeToLength(const std::vector<size_t> &shape)
{
   size_t n = 1;
   for (auto d : shape) n *= d;
   return n;
}

inline std::string ConvertShapeToString(const std::vector<size_t> &shape)
{
   std::string s = "{";
   for (size_t i = 0; i < shape.size(); ++i) s += (i ? ", " : " ") + std::to_string(shape[i]);
   return s + " }";
}

namespace UTILITY {
// identifier-safe tensor name (the reference's Clean_name: every non-alphanumeric becomes '_')
inline std::string Clean_name(std::string name)
{
   for (auto &c : name)
      if (!std::isalnum(static_cast<unsigned char>(c))) c = '_';
   return name;
}
}  // namespace UTILITY

struct InitializedTensor {
   ETensorType type = ETensorType::UNDEFINED;
   std::vector<size_t> shape;
   std::shared_ptr<void> data;  // host copy, GetTypeSize(type) * length bytes
   bool constant = false;       // consumed at generation time only: not written to the weight file
};

struct TensorInfo {
   ETensorType type = ETensorType::UNDEFINED;
   std::vector<size_t> shape;
};

}  // namespace SOFIE_B200
