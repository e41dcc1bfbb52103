// Elementwise, normalisation, pooling and aliasing operators for the B200 target: the operators
// the fusion pass may leave standing, each emitted as one call into libsofie_b200.
//
//   ROperator_Relu / LeakyRelu / Sigmoid / Gelu   core/inc/SOFIE/operators/ROperator_Relu.hxx:25-114,
//                                                 ROperator_LeakyRelu.hxx, ROperator_Sigmoid.hxx, ROperator_Gelu.hxx:23-123
//   ROperator_BasicBinary<T, Op>                  ROperator_BasicBinary.hxx:124,380,520-636
//   ROperator_BatchNormalization<T>               ROperator_BatchNormalization.hxx:43-110 (scale/sqrt(var+eps) folded at generation)
//   ROperator_LayerNormalization<T>               ROperator_LayerNormalization.hxx:54-56,186-324
//   ROperator_Softmax                             ROperator_Softmax.hxx:27,58-200 (last axis)
//   ROperator_Pool<T> (GlobalAveragePool)         ROperator_Pool.hxx:16-27,225-237
//   ROperator_Reshape (Reshape/Flatten/Squeeze/Unsqueeze) ROperator_Reshape.hxx:51-65,343-354: a zero-copy alias
#pragma once
#include <cmath>

#include "SOFIE_B200/operators/ROperator_Gemm.hxx"

namespace SOFIE_B200 {

// ---- unary activations --------------------------------------------------------------------------
class ROperator_Unary : public ROperator_B200 {
protected:
   std::string fNX, fNY, fOpLabel;
   EActivationType fAct;
   float fAlpha = 0.f;
   std::vector<size_t> fShape;
   ETensorType fType = ETensorType::FLOAT;

public:
   ROperator_Unary(std::string label, EActivationType act, float alpha, std::string nameX, std::string nameY)
      : fNX(UTILITY::Clean_name(nameX)), fNY(UTILITY::Clean_name(nameY)), fOpLabel(std::move(label)), fAct(act), fAlpha(alpha)
   {
      fInputTensorNames = {fNX};
      fOutputTensorNames = {fNY};
   }
   EActivationType Activation() const { return fAct; }
   float GetAlpha() const { return fAlpha; }
   bool SupportsSymbolicDim() const override { return true; }   // one element count
   void Initialize(RModel &model) override
   {
      if (!model.CheckIfTensorAlreadyExist(fNX))
         throw std::runtime_error("SOFIE " + fOpLabel + " Op Input Tensor " + fNX + " is not found in model");
      fShape = model.GetTensorShape(fNX);
      fType = model.GetTensorType(fNX);
      // an integer Relu only exists folded into the quantised contraction before it (checked at emission)
      const bool intRelu = fAct == EActivationType::RELU && (fType == ETensorType::INT8 || fType == ETensorType::UINT8);
      if (fType != ETensorType::FLOAT && fType != ETensorType::BFLOAT16 && !intRelu)
         throw std::runtime_error("SOFIE " + fOpLabel + " Op: FLOAT or BFLOAT16 input expected");
      model.AddIntermediateTensor(fNY, fType, fShape);
   }
   std::string Generate_GPU_B200(std::string opName) override
   {
      opName = "op_" + opName;
      if (fShape.empty()) throw std::runtime_error("SOFIE " + fOpLabel + " operator called to Generate without being initialized first");
      if (fType != ETensorType::FLOAT && fType != ETensorType::BFLOAT16)
         throw std::runtime_error("SOFIE " + fOpLabel + " Op: an integer Relu must directly follow a quantised contraction with output zero point 0 (it is folded into it)");
      std::stringstream out;
      out << "\n      //------ " << fOpLabel << " " << opName << "\n";
      out << "      Check(sofie_b200_unary_enqueue(ctx, tensor_" << fNX << ", tensor_" << fNY << ", " << ConvertTypeToRuntimeEnum(fType) << ", "
          << ConvertShapeToLength(fShape) << ", " << ActivationEnum(fAct) << ", " << FloatLit(fAlpha) << "), \"" << fOpLabel << " " << opName << "\");\n";
      return out.str();
   }
};

template <typename T>
class ROperator_Relu final : public ROperator_Unary {
public:
   ROperator_Relu(std::string nameX, std::string nameY) : ROperator_Unary("Relu", EActivationType::RELU, 0.f, nameX, nameY) {}
};
template <typename T>
class ROperator_LeakyRelu final : public ROperator_Unary {
public:
   ROperator_LeakyRelu(float alpha, std::string nameX, std::string nameY) : ROperator_Unary("LeakyRelu", EActivationType::LEAKYRELU, alpha, nameX, nameY) {}
};
template <typename T>
class ROperator_Sigmoid final : public ROperator_Unary {
public:
   ROperator_Sigmoid(std::string nameX, std::string nameY) : ROperator_Unary("Sigmoid", EActivationType::SIGMOID, 0.f, nameX, nameY) {}
};
class ROperator_Gelu final : public ROperator_Unary {
public:
   ROperator_Gelu(std::string nameX, std::string nameY, std::string approximate = "none")
      : ROperator_Unary("Gelu", approximate == "tanh" ? EActivationType::GELU_TANH : EActivationType::GELU, 0.f, nameX, nameY)
   {
      if (approximate != "none" && approximate != "tanh")
         throw std::runtime_error("SOFIE Gelu Op: approximate must be \"none\" or \"tanh\"");
   }
};

// ---- binary with trailing broadcast ---------------------------------------------------------------
enum class EBasicBinaryOperator { Add = 0, Sub = 1, Mul = 2, Div = 3 };

template <typename T, EBasicBinaryOperator Op>
class ROperator_BasicBinary final : public ROperator_B200 {
   std::string fNA, fNB, fNY;
   std::vector<size_t> fShapeA, fShapeB;
   ETensorType fType = ETensorType::FLOAT;
   bool fSwap = false;

public:
   ROperator_BasicBinary(std::string nameA, std::string nameB, std::string nameY)
      : fNA(UTILITY::Clean_name(nameA)), fNB(UTILITY::Clean_name(nameB)), fNY(UTILITY::Clean_name(nameY))
   {
      fInputTensorNames = {fNA, fNB};
      fOutputTensorNames = {fNY};
   }
   static constexpr EBasicBinaryOperator Kind() { return Op; }
   bool SupportsSymbolicDim() const override { return true; }   // two element counts; the broadcast rule compares trailing dimensions only
   const std::string &NameA() const { return fNA; }
   const std::string &NameB() const { return fNB; }
   void Initialize(RModel &model) override
   {
      for (auto &n : {fNA, fNB})
         if (!model.CheckIfTensorAlreadyExist(n)) throw std::runtime_error("SOFIE Binary Op Input Tensor " + n + " is not found in model");
      fShapeA = model.GetTensorShape(fNA);
      fShapeB = model.GetTensorShape(fNB);
      fType = model.GetTensorType(fNA);
      if (model.GetTensorType(fNB) != fType || (fType != ETensorType::FLOAT && fType != ETensorType::BFLOAT16))
         throw std::runtime_error("SOFIE Binary Op: both inputs must be FLOAT or both BFLOAT16");
      // supported broadcast: the shorter operand equals the trailing dimensions of the longer one
      auto trailing = [](const std::vector<size_t> &big, std::vector<size_t> small) {
         while (!small.empty() && small.front() == 1) small.erase(small.begin());
         if (small.size() > big.size()) return false;
         return std::equal(small.rbegin(), small.rend(), big.rbegin());
      };
      if (trailing(fShapeA, fShapeB)) fSwap = false;
      else if (trailing(fShapeB, fShapeA) && (Op == EBasicBinaryOperator::Add || Op == EBasicBinaryOperator::Mul)) fSwap = true;
      else
         throw std::runtime_error("SOFIE Binary Op: only trailing-dimension broadcasting is on the B200 path, got " +
                                  ConvertShapeToString(fShapeA) + " and " + ConvertShapeToString(fShapeB));
      model.AddIntermediateTensor(fNY, fType, fSwap ? fShapeB : fShapeA);
   }
   std::string Generate_GPU_B200(std::string opName) override
   {
      opName = "op_" + opName;
      const std::string &a = fSwap ? fNB : fNA, &b = fSwap ? fNA : fNB;
      const size_t n = ConvertShapeToLength(fSwap ? fShapeB : fShapeA), nb = ConvertShapeToLength(fSwap ? fShapeA : fShapeB);
      std::stringstream out;
      out << "\n      //------ BasicBinary " << opName << "\n";
      out << "      Check(sofie_b200_binary_enqueue(ctx, tensor_" << a << ", tensor_" << b << ", tensor_" << fNY << ", "
          << ConvertTypeToRuntimeEnum(fType) << ", " << n << ", " << nb << ", " << int(Op) << ", SOFIE_B200_ACT_NONE), \"Binary " << opName << "\");\n";
      return out.str();
   }
};

// ---- BatchNormalization (inference) ------------------------------------------------------------------
template <typename T>
class ROperator_BatchNormalization final : public ROperator_B200 {
   float fEpsilon = 1e-05, fMomentum = 0.9;
   std::size_t fTrainingMode = 0;
   std::string fNX, fNScale, fNB, fNMean, fNVar, fNY, fNFused;
   std::vector<size_t> fShapeX;
   EActivationType fActivation;

public:
   ROperator_BatchNormalization(float epsilon, float momentum, std::size_t training_mode, std::string nameX, std::string nameScale,
                                std::string nameB, std::string nameMean, std::string nameVar, std::string nameY,
                                EActivationType activation = EActivationType::UNDEFINED)
      : fEpsilon(epsilon), fMomentum(momentum), fTrainingMode(training_mode), fNX(UTILITY::Clean_name(nameX)),
        fNScale(UTILITY::Clean_name(nameScale)), fNB(UTILITY::Clean_name(nameB)), fNMean(UTILITY::Clean_name(nameMean)),
        fNVar(UTILITY::Clean_name(nameVar)), fNY(UTILITY::Clean_name(nameY)), fActivation(activation)
   {
      fInputTensorNames = {fNX};
      fOutputTensorNames = {fNY};
   }
   const std::string &NameX() const { return fNX; }
   const std::string &NameY() const { return fNY; }
   EActivationType GetActivationType() const override { return fActivation; }

   bool SupportsSymbolicDim() const override { return true; }   // the leading dimension is the batch count of the call
   void Initialize(RModel &model) override
   {
      for (auto &n : {fNX, fNScale, fNB, fNMean, fNVar})
         if (!model.CheckIfTensorAlreadyExist(n)) throw std::runtime_error("SOFIE BatchNormalization op Input Tensor " + n + " fnx is not found in model");
      for (auto &n : {fNScale, fNB, fNMean, fNVar})
         if (!model.IsInitializedTensor(n)) throw std::runtime_error("SOFIE BatchNormalization op: " + n + " must be an initialized tensor");
      fShapeX = model.GetTensorShape(fNX);
      if (fShapeX.size() < 2 || fShapeX.size() > 4)
         throw std::runtime_error("SOFIE BatchNormalization Op input tensor " + fNX + " fnx has wrong shape : " + ConvertShapeToString(fShapeX));
      if (fTrainingMode) throw std::runtime_error("SOFIE BatchNormalization Op: training mode is not supported");
      const size_t ch = fShapeX[1];
      auto scale = model.GetTensorData<float>(fNScale), var = model.GetTensorData<float>(fNVar);
      if (scale.size() != ch || var.size() != ch || ConvertShapeToLength(model.GetTensorShape(fNB)) != ch ||
          ConvertShapeToLength(model.GetTensorShape(fNMean)) != ch)
         throw std::runtime_error("SOFIE BatchNormalization Op: parameter tensors must have one value per channel");
      // scale / sqrt(var + eps), in fp32 at generation time (ROperator_BatchNormalization.hxx:100-109)
      std::vector<float> fused(ch);
      for (size_t c = 0; c < ch; ++c) fused[c] = scale[c] / std::sqrt(var[c] + fEpsilon);
      fNFused = fNY + "_fused_scale";
      model.AddInitializedTensor(fNFused, ETensorType::FLOAT, {ch}, fused);
      fInputTensorNames = {fNX, fNFused, fNB, fNMean};
      model.AddIntermediateTensor(fNY, ETensorType::FLOAT, fShapeX);
   }
   // y = x*s + t with s = fused scale and t = B - mean*s: what a producing Conv / Gemm folds
   void MakeScaleShift(RModel &model, std::string &scaleName, std::string &shiftName) const
   {
      auto s = model.GetTensorData<float>(fNFused), b = model.GetTensorData<float>(fNB), m = model.GetTensorData<float>(fNMean);
      std::vector<float> t(s.size());
      for (size_t c = 0; c < s.size(); ++c) t[c] = b[c] - m[c] * s[c];
      scaleName = fNFused;
      shiftName = fNY + "_fused_shift";
      if (!model.CheckIfTensorAlreadyExist(shiftName)) model.AddInitializedTensor(shiftName, ETensorType::FLOAT, {s.size()}, t);
   }
   bool FuseActivation(EActivationType act, float, const std::string &newOutput) override
   {
      if (act != EActivationType::RELU || fActivation != EActivationType::UNDEFINED) return false;  // parser-level BN+Relu (ParseFuseBatchnormRelu.cxx:31-37)
      fActivation = act;
      fNY = newOutput; fOutputTensorNames = {fNY};
      return true;
   }
   bool HasFusableEpilogue() const override { return true; }
   std::string Generate_GPU_B200(std::string opName) override
   {
      opName = "op_" + opName;
      size_t inner = 1;
      for (size_t i = 2; i < fShapeX.size(); ++i) inner *= fShapeX[i];
      std::stringstream out;
      out << "\n      //------ BatchNormalization " << opName << "\n";
      out << "      Check(sofie_b200_batchnorm_enqueue(ctx, tensor_" << fNX << ", tensor_" << fNY << ", " << fShapeX[0] << ", " << fShapeX[1] << ", "
          << inner << ", tensor_" << fNFused << ", tensor_" << fNB << ", tensor_" << fNMean << ", " << ActivationEnum(fActivation)
          << "), \"BatchNormalization " << opName << "\");\n";
      return out.str();
   }
};

// ---- LayerNormalization ---------------------------------------------------------------------------------
template <typename T>
class ROperator_LayerNormalization final : public ROperator_B200 {
   int fAttrAxis;
   float fAttrEpsilon;
   size_t fAttrStashType;
   std::string fNX, fNScale, fNB, fNY, fNMean, fNInvStdDev;
   std::vector<size_t> fShapeX;
   size_t fRows = 0, fCols = 0;
   ETensorType fType = ETensorType::FLOAT;

public:
   ROperator_LayerNormalization(int axis, float epsilon, size_t stashType, const std::string &nameX, const std::string &nameScale,
                                const std::string &nameB, const std::string &nameY, const std::string &nameMean = "",
                                const std::string &nameInvStdDev = "")
      : fAttrAxis(axis), fAttrEpsilon(epsilon), fAttrStashType(stashType), fNX(UTILITY::Clean_name(nameX)),
        fNScale(UTILITY::Clean_name(nameScale)), fNB(UTILITY::Clean_name(nameB)), fNY(UTILITY::Clean_name(nameY)),
        fNMean(UTILITY::Clean_name(nameMean)), fNInvStdDev(UTILITY::Clean_name(nameInvStdDev))
   {
      fInputTensorNames = {fNX};
      if (!fNScale.empty()) fInputTensorNames.push_back(fNScale);
      if (!fNB.empty()) fInputTensorNames.push_back(fNB);
      fOutputTensorNames = {fNY};
      if (!fNMean.empty()) fOutputTensorNames.push_back(fNMean);
      if (!fNInvStdDev.empty()) fOutputTensorNames.push_back(fNInvStdDev);
   }
   bool fAxisIsInner = false;
   bool SupportsSymbolicDim() const override { return fAxisIsInner; }   // the leading dimension only counts rows
   void Initialize(RModel &model) override
   {
      if (!model.CheckIfTensorAlreadyExist(fNX)) throw std::runtime_error("SOFIE LayerNormalization Op Input Tensor " + fNX + " is not found in model");
      fShapeX = model.GetTensorShape(fNX);
      fType = model.GetTensorType(fNX);
      if (fType != ETensorType::FLOAT && fType != ETensorType::BFLOAT16)
         throw std::runtime_error("SOFIE LayerNormalization Op: FLOAT or BFLOAT16 input expected");
      const int rank = int(fShapeX.size());
      const int axis = fAttrAxis < 0 ? fAttrAxis + rank : fAttrAxis;
      if (axis < 0 || axis >= rank) throw std::runtime_error("SOFIE LayerNormalization Op: axis out of range");
      fRows = 1; fCols = 1;
      fAxisIsInner = axis > 0;
      for (int i = 0; i < axis; ++i) fRows *= fShapeX[i];
      for (int i = axis; i < rank; ++i) fCols *= fShapeX[i];
      for (auto &n : {fNScale, fNB})
         if (!n.empty()) {
            if (!model.CheckIfTensorAlreadyExist(n)) throw std::runtime_error("SOFIE LayerNormalization Op Input Tensor " + n + " is not found in model");
            if (ConvertShapeToLength(model.GetTensorShape(n)) != fCols || model.GetTensorType(n) != ETensorType::FLOAT)
               throw std::runtime_error("SOFIE LayerNormalization Op: scale and bias must be FLOAT tensors over the normalised dimensions");
         }
      model.AddIntermediateTensor(fNY, fType, fShapeX);
      std::vector<size_t> red(fShapeX.begin(), fShapeX.begin() + axis);
      red.resize(rank, 1);
      if (!fNMean.empty()) model.AddIntermediateTensor(fNMean, ETensorType::FLOAT, red);
      if (!fNInvStdDev.empty()) model.AddIntermediateTensor(fNInvStdDev, ETensorType::FLOAT, red);
   }
   std::string Generate_GPU_B200(std::string opName) override
   {
      opName = "op_" + opName;
      auto ptr = [](const std::string &n) { return n.empty() ? std::string("nullptr") : "tensor_" + n; };
      std::stringstream out;
      out << "\n      //------ LayerNormalization " << opName << " rows " << fRows << " cols " << fCols << "\n";
      out << "      Check(sofie_b200_layernorm_enqueue(ctx, tensor_" << fNX << ", tensor_" << fNY << ", " << ConvertTypeToRuntimeEnum(fType) << ", "
          << ConvertTypeToRuntimeEnum(fType) << ", " << fRows << ", " << fCols << ", " << ptr(fNScale) << ", " << ptr(fNB) << ", "
          << FloatLit(fAttrEpsilon) << ", " << ptr(fNMean) << ", " << ptr(fNInvStdDev) << "), \"LayerNormalization " << opName << "\");\n";
      return out.str();
   }
};

// ---- Softmax ------------------------------------------------------------------------------------------------
class ROperator_Softmax final : public ROperator_B200 {
   int64_t fAttrAxis;
   std::string fNX, fNY;
   std::vector<size_t> fShape;
   bool fLogSoftmax;
   size_t fAxis = 0;
   ETensorType fType = ETensorType::FLOAT;

public:
   ROperator_Softmax(int64_t attr_axis, std::string nameX, std::string nameY, bool logSoftmax = false)
      : fAttrAxis(attr_axis), fNX(UTILITY::Clean_name(nameX)), fNY(UTILITY::Clean_name(nameY)), fLogSoftmax(logSoftmax)
   {
      fInputTensorNames = {fNX};
      fOutputTensorNames = {fNY};
   }
   bool SupportsSymbolicDim() const override { return fAxis > 0; }   // the leading dimension only counts rows (or outer slices)
   void Initialize(RModel &model) override
   {
      if (!model.CheckIfTensorAlreadyExist(fNX)) throw std::runtime_error("SOFIE Softmax Op Input Tensor is not found in model");
      fShape = model.GetTensorShape(fNX);
      fType = model.GetTensorType(fNX);
      const int64_t rank = int64_t(fShape.size());
      const int64_t axis = fAttrAxis < 0 ? fAttrAxis + rank : fAttrAxis;
      if (axis < 0 || axis >= rank) throw std::runtime_error("SOFIE Softmax Op: axis " + std::to_string(fAttrAxis) + " out of range");
      fAxis = size_t(axis);
      model.AddIntermediateTensor(fNY, fType, fShape);
   }
   std::string Generate_GPU_B200(std::string opName) override
   {
      opName = "op_" + opName;
      const size_t cols = fShape.back(), rows = ConvertShapeToLength(fShape) / (cols ? cols : 1);
      std::stringstream out;
      out << "\n      //------ " << (fLogSoftmax ? "LogSoftmax " : "Softmax ") << opName << "\n";
      if (fAxis + 1 != fShape.size()) {   // any other axis: [outer, n, inner] (ROperator_Softmax.hxx:120-200)
         size_t outer = 1, inner = 1;
         for (size_t i = 0; i < fAxis; ++i) outer *= fShape[i];
         for (size_t i = fAxis + 1; i < fShape.size(); ++i) inner *= fShape[i];
         out << "      Check(sofie_b200_softmax_axis_enqueue(ctx, tensor_" << fNX << ", tensor_" << fNY << ", " << ConvertTypeToRuntimeEnum(fType) << ", "
             << outer << ", " << fShape[fAxis] << ", " << inner << ", " << (fLogSoftmax ? 1 : 0) << "), \"Softmax " << opName << "\");\n";
         return out.str();
      }
      out << "      Check(sofie_b200_softmax_enqueue(ctx, tensor_" << fNX << ", tensor_" << fNY << ", " << ConvertTypeToRuntimeEnum(fType) << ", "
          << ConvertTypeToRuntimeEnum(fType) << ", " << rows << ", " << cols << ", " << (fLogSoftmax ? 1 : 0) << "), \"Softmax " << opName << "\");\n";
      return out.str();
   }
};

// ---- GlobalAveragePool ------------------------------------------------------------------------------------------
enum PoolOpMode { InvalidPool, MaxPool, AveragePool, GlobalAveragePool };

template <typename T>
class ROperator_Pool final : public ROperator_B200 {
   PoolOpMode fPoolMode;
   std::string fNX, fNY;
   std::vector<size_t> fShapeX;
   bool fChannelsLast = false;   // the input is stored [N, H, W, C] (set by the layout pass behind a channels-last convolution)
   ETensorType fTypeX = ETensorType::FLOAT;

public:
   ROperator_Pool(PoolOpMode mode, std::string nameX, std::string nameY)
      : fPoolMode(mode), fNX(UTILITY::Clean_name(nameX)), fNY(UTILITY::Clean_name(nameY))
   {
      fInputTensorNames = {fNX};
      fOutputTensorNames = {fNY};
   }
   void Initialize(RModel &model) override
   {
      if (fPoolMode != GlobalAveragePool) throw std::runtime_error("SOFIE Pool Op: only GlobalAveragePool is on the B200 path");
      if (!model.CheckIfTensorAlreadyExist(fNX)) throw std::runtime_error("SOFIE Pool op Input Tensor " + fNX + " is not found in model");
      fShapeX = model.GetTensorShape(fNX);
      fTypeX = model.GetTensorType(fNX);
      if (fShapeX.size() < 3 || fTypeX != ETensorType::FLOAT) throw std::runtime_error("SOFIE Pool Op: FLOAT NC... input expected");
      std::vector<size_t> y(fShapeX.size(), 1);
      y[0] = fShapeX[0]; y[1] = fShapeX[1];
      model.AddIntermediateTensor(fNY, ETensorType::FLOAT, y);
   }
   const std::string &NameX() const { return fNX; }
   void SetChannelsLast(bool on) { fChannelsLast = on; }
   const std::string &NameY() const { return fNY; }
   // read the quantised tensor a per-tensor DequantizeLinear was applied to (the scale moves to the consumer of the pool)
   void ReadQuantised(const std::string &name, ETensorType type) { fNX = name; fTypeX = type; fInputTensorNames = {fNX}; }
   std::string Generate_GPU_B200(std::string opName) override
   {
      opName = "op_" + opName;
      size_t inner = 1;
      for (size_t i = 2; i < fShapeX.size(); ++i) inner *= fShapeX[i];
      std::stringstream out;
      out << "\n      //------ GlobalAveragePool " << opName << (fChannelsLast ? " (channels-last input)" : "") << "\n";
      if (fChannelsLast) {
         out << "      Check(sofie_b200_global_avgpool_nhwc_enqueue(ctx, tensor_" << fNX << ", tensor_" << fNY << ", " << ConvertTypeToRuntimeEnum(fTypeX) << ", " << fShapeX[0] << ", "
             << inner << ", " << fShapeX[1] << "), \"GlobalAveragePool " << opName << "\");\n";
         return out.str();
      }
      out << "      Check(sofie_b200_global_avgpool_enqueue(ctx, tensor_" << fNX << ", tensor_" << fNY << ", " << ConvertTypeToRuntimeEnum(fTypeX) << ", " << fShapeX[0] * fShapeX[1]
          << ", " << inner << "), \"GlobalAveragePool " << opName << "\");\n";
      return out.str();
   }
};

// ---- Reshape family: a zero-copy alias ----------------------------------------------------------------------------
enum ReshapeOpMode { Reshape, Flatten, Squeeze, Unsqueeze };

class ROperator_Reshape final : public ROperator_B200 {
   ReshapeOpMode fOpMode;
   int fAttr;  // allowzero (Reshape) or axis (Flatten)
   std::string fNData, fNShape, fNOutput;
   std::vector<int64_t> fAxes;

public:
   ROperator_Reshape(ReshapeOpMode opMode, int attr_value, std::string nameData, std::string nameShape, std::string nameOutput)
      : fOpMode(opMode), fAttr(attr_value), fNData(UTILITY::Clean_name(nameData)), fNShape(UTILITY::Clean_name(nameShape)),
        fNOutput(UTILITY::Clean_name(nameOutput))
   {
      fInputTensorNames = {fNData};
      fOutputTensorNames = {fNOutput};
   }
   bool IsAlias() const override { return true; }
   bool SupportsSymbolicDim() const override { return true; }   // emits nothing; RModel checks where the dimension ends up
   void Initialize(RModel &model) override
   {
      if (!model.CheckIfTensorAlreadyExist(fNData)) throw std::runtime_error("SOFIE Reshape Op Input Tensor " + fNData + " is not found in model");
      const auto in = model.GetTensorShape(fNData);
      const size_t len = ConvertShapeToLength(in);
      std::vector<size_t> out;
      if (fOpMode == Flatten) {
         const int rank = int(in.size()), axis = fAttr < 0 ? fAttr + rank : fAttr;
         size_t a = 1, b = 1;
         for (int i = 0; i < rank; ++i) (i < axis ? a : b) *= in[i];
         out = {a, b};
      } else {
         if (fNShape.empty() || !model.IsInitializedTensor(fNShape))
            throw std::runtime_error("SOFIE Reshape Op: the shape / axes operand must be an initialized INT64 tensor on the B200 path");
         auto v = model.GetTensorData<int64_t>(fNShape);
         if (fOpMode == Reshape) {
            size_t known = 1; int infer = -1;
            for (size_t i = 0; i < v.size(); ++i) {
               if (v[i] == -1) { infer = int(i); out.push_back(1); }
               else if (v[i] == 0 && !fAttr) { out.push_back(in.at(i)); known *= in[i]; }
               else { out.push_back(size_t(v[i])); known *= size_t(v[i]); }
            }
            if (infer >= 0) out[infer] = known ? len / known : 0;
         } else if (fOpMode == Squeeze) {
            std::set<int64_t> ax;
            for (auto a : v) ax.insert(a < 0 ? a + int64_t(in.size()) : a);
            for (size_t i = 0; i < in.size(); ++i)
               if (!ax.count(int64_t(i))) out.push_back(in[i]);
         } else {
            out = in;
            std::vector<int64_t> ax(v.begin(), v.end());
            for (auto &a : ax) if (a < 0) a += int64_t(in.size() + v.size());
            std::sort(ax.begin(), ax.end());
            for (auto a : ax) out.insert(out.begin() + a, 1);
         }
      }
      if (ConvertShapeToLength(out) != len)
         throw std::runtime_error("SOFIE Reshape Op : Invalid  shapes : " + ConvertShapeToString(in) + ConvertShapeToString(out));
      model.AddIntermediateTensor(fNOutput, model.GetTensorType(fNData), out);
      model.AddAliasTensor(fNOutput, fNData);
   }
   std::string Generate_GPU_B200(std::string) override { return ""; }  // nothing to run: the output aliases the input
};

}  // namespace SOFIE_B200
