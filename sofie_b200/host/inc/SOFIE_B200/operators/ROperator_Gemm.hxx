// Gemm and MatMul for the B200 target.
//
// Constructor and semantics are the reference's ROperator_Gemm (core/inc/SOFIE/operators/
// ROperator_Gemm.hxx:61-84): Y = alpha * op(A) * op(B) + beta * C, MatMul = (1, 0, tA, tB, A, B, Y),
// stacked MatMul over leading dimensions (shape rules :86-155), C broadcast to Y unidirectionally
// (:270-301), constant folding when every input is an initializer (:317-373).  Where the reference
// emits blas.gemm / gemmrelu / matmul / gemmStridedBatched plus GemmBiasAddKernel (:743-1140), this
// operator emits one sofie_b200_gemm_plan per contraction and one enqueue with a fused epilogue.
// Difference kept on purpose: a beta other than 1 multiplies C as ONNX defines it (the reference's
// bias-broadcast branch drops it, :580).
#pragma once
#include <cstring>
#include <iomanip>
#include <sstream>

#include "SOFIE_B200/RModel.hxx"

namespace SOFIE_B200 {

inline std::string FloatLit(float v)
{
   if (v != v) return "std::numeric_limits<float>::quiet_NaN()";
   if (v > 3.4e38f) return "std::numeric_limits<float>::infinity()";
   if (v < -3.4e38f) return "-std::numeric_limits<float>::infinity()";
   std::ostringstream o;
   o << std::setprecision(9) << v;
   std::string s = o.str();
   if (s.find_first_of(".e") == std::string::npos) s += ".0";
   return s + "f";
}

// What a contraction can fold into its epilogue; shared by Gemm, Conv and the quantised operators.
struct EpilogueState {
   EActivationType act = EActivationType::UNDEFINED;
   float actAlpha = 0.f;
   std::string colScale;   // initialized F32 [N] tensor, or empty
   std::string bias;       // initialized / intermediate tensor, or empty
   std::string biasMode = "SOFIE_B200_BIAS_NONE";
   std::string residual;   // tensor added before the activation, or empty
   float alpha = 1.f, beta = 1.f;
   float outScale = 1.f;
   int outZeroPoint = 0;

   // members and constructor text for `sofie_b200_epilogue ep_<op>`
   std::string InitCode(const std::string &ep) const
   {
      std::stringstream out;
      out << "      " << ep << ".alpha = " << FloatLit(alpha) << "; " << ep << ".beta = " << FloatLit(beta) << "; " << ep
          << ".out_scale = " << FloatLit(outScale) << "; " << ep << ".out_zero_point = " << outZeroPoint << ";\n";
      if (!bias.empty()) out << "      " << ep << ".bias_mode = " << biasMode << ";\n";
      if (act != EActivationType::UNDEFINED)
         out << "      " << ep << ".act = " << ActivationEnum(act) << "; " << ep << ".act_alpha = " << FloatLit(actAlpha) << ";\n";
      return out.str();
   }
   // text for the inference body: tensor pointers are bound at every call, because a scale, bias or
   // residual may be a graph input whose address the caller chooses per call
   std::string BindCode(const std::string &ep) const
   {
      std::stringstream out;
      if (!colScale.empty()) out << "      " << ep << ".col_scale = tensor_" << colScale << ";\n";
      if (!bias.empty()) out << "      " << ep << ".bias = tensor_" << bias << ";\n";
      return out.str();
   }
};

template <typename T>
class ROperator_Gemm final : public ROperator_B200 {
   static_assert(std::is_same<T, float>::value, "ROperator_Gemm<T>: T is float, as in the reference; other element types come from the tensors");

private:
   float fAttrAlpha = 1.0, fAttrBeta = 1.0;
   int_fast64_t fAttrTransA = 0, fAttrTransB = 0;
   std::string fNA, fNB, fNC, fNY;
   EpilogueState fEpi;
   std::vector<size_t> fShapeA, fShapeB, fShapeC, fShapeY;
   bool fBIsWeight = false;   // B is an initialized tensor (a weight)
   std::string fNQuantB, fNQuantScale;   // see SetDequantisedWeight
   int64_t fQuantAxis = 0;
   ETensorType fType = ETensorType::FLOAT, fTypeY = ETensorType::FLOAT;
   size_t fM = 0, fN = 0, fK = 0, fBatch = 1;
   int64_t fStrideA = 0, fStrideB = 0;
   bool fIsOutputConstant = false;
   bool fPrecise = true;

public:
   ROperator_Gemm() {}
   ROperator_Gemm(float alpha, float beta, int_fast64_t transA, int_fast64_t transB, std::string nameA, std::string nameB,
                  std::string nameY, EActivationType activation = EActivationType::UNDEFINED)
      : fAttrAlpha(alpha), fAttrBeta(beta), fAttrTransA(transA), fAttrTransB(transB), fNA(UTILITY::Clean_name(nameA)),
        fNB(UTILITY::Clean_name(nameB)), fNY(UTILITY::Clean_name(nameY))
   {
      fEpi.act = activation;
      fInputTensorNames = {fNA, fNB};
      fOutputTensorNames = {fNY};
   }
   ROperator_Gemm(float alpha, float beta, int_fast64_t transA, int_fast64_t transB, std::string nameA, std::string nameB,
                  std::string nameC, std::string nameY, EActivationType activation = EActivationType::UNDEFINED)
      : fAttrAlpha(alpha), fAttrBeta(beta), fAttrTransA(transA), fAttrTransB(transB), fNA(UTILITY::Clean_name(nameA)),
        fNB(UTILITY::Clean_name(nameB)), fNC(UTILITY::Clean_name(nameC)), fNY(UTILITY::Clean_name(nameY))
   {
      fEpi.act = activation;
      fInputTensorNames = {fNA, fNB, fNC};
      fOutputTensorNames = {fNY};
   }

   bool HasBias() const { return !fNC.empty(); }
   // B is DequantizeLinear(quantised INT8 initializer, per-output-channel scale): the weight-only quantised linear layer.
   // With BFLOAT16 activations the int8 values become a BFLOAT16 initializer (exact: |q| <= 127) and the scale the column
   // scale of the epilogue, so the dequantisation costs nothing at run time; with FLOAT activations the weight is folded
   // to q * scale at generation (what the reference computes on dequantised weights).
   void SetDequantisedWeight(const std::string &quantised, const std::string &scale, int64_t axis)
   {
      fNQuantB = UTILITY::Clean_name(quantised); fNQuantScale = UTILITY::Clean_name(scale); fQuantAxis = axis;
   }
   EActivationType GetActivationType() const override { return fEpi.act; }
   // single-pass TF32 instead of the fp32-accurate path (off by default: parity bar is 1e-5)
   void SetPrecise(bool p) { fPrecise = p; }
   const EpilogueState &GetEpilogue() const { return fEpi; }
   const std::string &NameA() const { return fNA; }
   // A was rescaled by a constant that is applied here instead (a per-tensor dequantisation moved behind a pooling)
   void ScaleAlpha(float s) { fAttrAlpha *= s; fEpi.alpha *= s; }

   void Initialize(RModel &model) override
   {
      if (!model.CheckIfTensorAlreadyExist(fNA))
         throw std::runtime_error("SOFIE Gemm Op Input Tensor " + fNA + " is not found in model");
      if (!fNQuantB.empty()) FoldDequantisedWeight(model);
      if (!model.CheckIfTensorAlreadyExist(fNB))
         throw std::runtime_error("SOFIE Gemm Op Input Tensor " + fNB + " is not found in model");
      if (!fNC.empty() && !model.CheckIfTensorAlreadyExist(fNC))
         throw std::runtime_error("SOFIE Gemm Op Input Tensor " + fNC + " is not found in model");
      fShapeA = model.GetTensorShape(fNA);
      fShapeB = model.GetTensorShape(fNB);
      fBIsWeight = model.IsInitializedTensor(fNB);
      fType = model.GetTensorType(fNA);
      if (model.GetTensorType(fNB) != fType)
         throw std::runtime_error("SOFIE Gemm Op: A and B have different element types");
      if (fType != ETensorType::FLOAT && fType != ETensorType::BFLOAT16)
         throw std::runtime_error("SOFIE Gemm Op: element type not supported (FLOAT and BFLOAT16; quantised types have their own operators)");
      fTypeY = fType;
      // rank-1 operands: prepend / append a 1, removed from Y afterwards (ROperator_Gemm.hxx:176-205)
      bool prependOne = false, appendOne = false;
      if (fShapeA.size() == 1) { fShapeA.insert(fShapeA.begin(), 1); prependOne = true; }
      if (fShapeB.size() == 1) { fShapeB.push_back(1); appendOne = true; }
      if (fShapeA.size() < 2 || fShapeB.size() < 2)
         throw std::runtime_error("SOFIE Gemm Op: scalar operands are not supported");
      const size_t ra = fShapeA.size(), rb = fShapeB.size();
      const size_t am = fShapeA[ra - 2], ak = fShapeA[ra - 1], bk = fShapeB[rb - 2], bn = fShapeB[rb - 1];
      fM = fAttrTransA ? ak : am;
      fK = fAttrTransA ? am : ak;
      const size_t kb = fAttrTransB ? bn : bk;
      fN = fAttrTransB ? bk : bn;
      if (kb != fK)
         throw std::runtime_error("SOFIE Gemm Op : invalid input shapes A " + ConvertShapeToString(fShapeA) + " B " +
                                  ConvertShapeToString(fShapeB));
      // stacked MatMul: leading dimensions of A and B broadcast (ROperator_Gemm.hxx:86-155)
      std::vector<size_t> batchA(fShapeA.begin(), fShapeA.end() - 2), batchB(fShapeB.begin(), fShapeB.end() - 2);
      const size_t nbA = ConvertShapeToLength(batchA), nbB = ConvertShapeToLength(batchB);
      std::vector<size_t> batchY = nbA >= nbB ? batchA : batchB;
      if (nbB == 1) {
         // a shared weight: the stack of A collapses into rows (ROperator_Gemm.hxx:854-859)
         if (!fAttrTransA) { fM *= nbA; fBatch = 1; }
         else { fBatch = nbA; fStrideA = int64_t(am * ak); fStrideB = 0; }
      } else if (nbA == 1) {
         fBatch = nbB; fStrideA = 0; fStrideB = int64_t(bk * bn);
      } else {
         if (batchA != batchB)
            throw std::runtime_error("SOFIE Gemm Op: stacked operands need equal leading dimensions, A " + ConvertShapeToString(fShapeA) +
                                     " B " + ConvertShapeToString(fShapeB));
         fBatch = nbA; fStrideA = int64_t(am * ak); fStrideB = int64_t(bk * bn);
      }
      fShapeY = batchY;
      if (!prependOne) fShapeY.push_back(fAttrTransA ? ak : am);
      if (!appendOne) fShapeY.push_back(fN);
      if (fShapeY.empty()) fShapeY.push_back(1);

      // C must broadcast unidirectionally to the [M,N] result (ROperator_Gemm.hxx:270-301)
      if (!fNC.empty()) {
         fShapeC = model.GetTensorShape(fNC);
         const size_t rowsY = fBatch == 1 ? fM : fM, lenC = ConvertShapeToLength(fShapeC);
         std::vector<size_t> c = fShapeC;
         while (c.size() > 2 && c.front() == 1) c.erase(c.begin());
         if (lenC == 1) fEpi.biasMode = "SOFIE_B200_BIAS_SCALAR_F32";
         else if ((c.size() == 1 && c[0] == fN) || (c.size() == 2 && c[0] == 1 && c[1] == fN)) fEpi.biasMode = "SOFIE_B200_BIAS_COL_F32";
         else if (c.size() == 2 && c[0] == rowsY && c[1] == 1 && fBatch == 1) fEpi.biasMode = "SOFIE_B200_BIAS_ROW_F32";
         else if (c.size() == 2 && c[0] == rowsY && c[1] == fN && fBatch == 1) fEpi.biasMode = "SOFIE_B200_BIAS_FULL_F32";
         else
            throw std::runtime_error("SOFIE Gemm Op - bias tensor of shape " + ConvertShapeToString(fShapeC) +
                                     " cannot be uni-directional broadcasted to " + ConvertShapeToString(fShapeY));
         if (model.GetTensorType(fNC) != ETensorType::FLOAT)
            throw std::runtime_error("SOFIE Gemm Op: the bias tensor must be FLOAT");
         fEpi.bias = fNC;
         fEpi.beta = fAttrBeta;
         if (fEpi.biasMode != "SOFIE_B200_BIAS_FULL_F32" && fAttrBeta != 1.f) {
            // fold beta into a copy of C at generation time when C is a weight
            if (!model.IsInitializedTensor(fNC))
               throw std::runtime_error("SOFIE Gemm Op: beta != 1 needs an initialized or full-shape C");
            auto cv = model.GetTensorData<float>(fNC);
            for (auto &v : cv) v *= fAttrBeta;
            fEpi.bias = fNC + "_beta";
            model.AddInitializedTensor(fEpi.bias, ETensorType::FLOAT, fShapeC, cv);
            fEpi.beta = 1.f;
         }
      }
      fEpi.alpha = fAttrAlpha;

      // every input an initializer: fold now (ROperator_Gemm.hxx:317-373)
      if (fType == ETensorType::FLOAT && model.IsInitializedTensor(fNA) && model.IsInitializedTensor(fNB) &&
          (fNC.empty() || model.IsInitializedTensor(fNC)) && fBatch == 1 && fEpi.act == EActivationType::UNDEFINED) {
         auto a = model.GetTensorData<float>(fNA), b = model.GetTensorData<float>(fNB);
         std::vector<float> cvals;
         if (!fNC.empty()) cvals = model.GetTensorData<float>(fEpi.bias);
         std::vector<float> y(fM * fN);
         for (size_t i = 0; i < fM; ++i)
            for (size_t j = 0; j < fN; ++j) {
               double acc = 0;
               for (size_t k = 0; k < fK; ++k)
                  acc += double(fAttrTransA ? a[k * fM + i] : a[i * fK + k]) * double(fAttrTransB ? b[j * fK + k] : b[k * fN + j]);
               float v = fAttrAlpha * float(acc);
               if (!fNC.empty()) {
                  float cv = fEpi.biasMode == "SOFIE_B200_BIAS_SCALAR_F32" ? cvals[0]
                             : fEpi.biasMode == "SOFIE_B200_BIAS_COL_F32" ? cvals[j]
                             : fEpi.biasMode == "SOFIE_B200_BIAS_ROW_F32" ? cvals[i] : fEpi.beta * cvals[i * fN + j];
                  v += cv;
               }
               y[i * fN + j] = v;
            }
         model.AddInitializedTensor(fNY, ETensorType::FLOAT, fShapeY, y);
         fIsOutputConstant = true;
         return;
      }
      model.AddIntermediateTensor(fNY, fTypeY, fShapeY);
   }

   void FoldDequantisedWeight(RModel &model)
   {
      if (!model.IsInitializedTensor(fNQuantB) || model.GetTensorType(fNQuantB) != ETensorType::INT8 || !model.IsInitializedTensor(fNQuantScale))
         throw std::runtime_error("SOFIE Gemm Op: a dequantised weight needs an initialized INT8 tensor and an initialized scale");
      const auto shape = model.GetTensorShape(fNQuantB);
      if (shape.size() != 2) throw std::runtime_error("SOFIE Gemm Op: a dequantised weight must have rank 2");
      const auto q = model.GetTensorData<int8_t>(fNQuantB);
      const auto sc = model.GetTensorData<float>(fNQuantScale);
      const size_t nAxis = fAttrTransB ? 0 : 1, n = shape[nAxis];
      const int64_t axis = fQuantAxis < 0 ? fQuantAxis + 2 : fQuantAxis;
      if (sc.size() != 1 && (sc.size() != n || size_t(axis) != nAxis))
         throw std::runtime_error("SOFIE Gemm Op: the scale of a dequantised weight must be a scalar or run along the output channels");
      auto scaleOf = [&](size_t r, size_t c) { return sc.size() == 1 ? sc[0] : sc[nAxis == 0 ? r : c]; };
      if (model.GetTensorType(fNA) == ETensorType::BFLOAT16) {
         std::vector<uint16_t> w(q.size());
         for (size_t i = 0; i < q.size(); ++i) {
            const float f = float(q[i]);
            uint32_t u;
            std::memcpy(&u, &f, 4);
            w[i] = uint16_t(u >> 16);   // integers up to 127 fit the 8 significand bits exactly
         }
         model.AddInitializedTensor(fNB, ETensorType::BFLOAT16, shape, w);
         if (sc.size() == 1) fAttrAlpha *= sc[0];
         else { fEpi.colScale = fNQuantScale; fInputTensorNames.push_back(fNQuantScale); }
      } else {
         std::vector<float> w(q.size());
         for (size_t r = 0; r < shape[0]; ++r)
            for (size_t c = 0; c < shape[1]; ++c) w[r * shape[1] + c] = float(q[r * shape[1] + c]) * scaleOf(r, c);
         model.AddInitializedTensor(fNB, ETensorType::FLOAT, shape, w);
      }
   }

   // ---- fusion hooks ------------------------------------------------------------------------
   bool HasFusableEpilogue() const override { return !fIsOutputConstant; }
   bool FuseActivation(EActivationType act, float alpha, const std::string &newOutput) override
   {
      if (fEpi.act != EActivationType::UNDEFINED || fIsOutputConstant) return false;
      fEpi.act = act;
      fEpi.actAlpha = alpha;
      fNY = newOutput;
      fOutputTensorNames = {fNY};
      return true;
   }
   bool FuseScaleShift(RModel &model, const std::string &scale, const std::string &shift, const std::string &newOutput) override
   {
      // y*s[c] + t[c] on top of acc*alpha + bias[c]: new column scale s, new bias bias*s + t
      if (fEpi.act != EActivationType::UNDEFINED || !fEpi.residual.empty() || fIsOutputConstant) return false;
      // BatchNormalization's channel axis is dimension 1: the columns of a rank-2 product, but the ROWS of a stacked one
      if (fShapeY.size() != 2) return false;
      if (!fEpi.bias.empty() && (fEpi.biasMode != "SOFIE_B200_BIAS_COL_F32" || !model.IsInitializedTensor(fEpi.bias))) return false;
      auto s = model.GetTensorData<float>(scale), t = model.GetTensorData<float>(shift);
      if (s.size() != fN || t.size() != fN) return false;
      std::vector<float> nb(fN);
      if (!fEpi.bias.empty()) {
         auto b = model.GetTensorData<float>(fEpi.bias);
         for (size_t j = 0; j < fN; ++j) nb[j] = b[j] * s[j] + t[j];
      } else {
         nb = t;
      }
      if (!fEpi.colScale.empty()) {
         auto cs = model.GetTensorData<float>(fEpi.colScale);
         for (size_t j = 0; j < fN; ++j) s[j] *= cs[j];
      }
      fEpi.colScale = newOutput + "_fold_scale";
      fEpi.bias = newOutput + "_fold_bias";
      fEpi.biasMode = "SOFIE_B200_BIAS_COL_F32";
      model.AddInitializedTensor(fEpi.colScale, ETensorType::FLOAT, {fN}, s);
      model.AddInitializedTensor(fEpi.bias, ETensorType::FLOAT, {fN}, nb);
      fInputTensorNames = {fNA, fNB, fEpi.colScale, fEpi.bias};
      fNY = newOutput;
      fOutputTensorNames = {fNY};
      return true;
   }
   bool FuseResidual(RModel &model, const std::string &residual, const std::string &newOutput) override
   {
      if (fEpi.act != EActivationType::UNDEFINED || !fEpi.residual.empty() || fIsOutputConstant) return false;
      if (model.GetTensorShape(residual) != fShapeY) return false;
      const ETensorType rt = model.GetTensorType(residual);
      if (rt != ETensorType::FLOAT && rt != ETensorType::BFLOAT16) return false;
      fEpi.residual = residual;
      fResidualType = rt;
      fInputTensorNames.push_back(residual);
      fNY = newOutput;
      fOutputTensorNames = {fNY};
      return true;
   }

   // ---- emission ------------------------------------------------------------------------------
   std::string GenerateSessionMembersCode_GPU_B200(std::string opName) override
   {
      if (fIsOutputConstant) return "";
      opName = "op_" + opName;
      return "   sofie_b200_gemm_plan *plan_" + opName + " = nullptr;\n   sofie_b200_epilogue ep_" + opName + "{};\n";
   }

   std::string GenerateInitCode_GPU_B200(std::string opName) override
   {
      if (fIsOutputConstant) return "";
      opName = "op_" + opName;
      const size_t lda = fAttrTransA ? (fStrideA && fBatch > 1 ? fShapeA[fShapeA.size() - 1] : fM) : fK;
      std::stringstream out;
      out << "      {  // Gemm " << opName << ": " << ConvertShapeToString(fShapeA) << " x " << ConvertShapeToString(fShapeB) << "\n";
      out << "      sofie_b200_gemm_desc d{};\n";
      out << "      d.M = " << fM << "; d.N = " << fN << "; d.K = " << fK << "; d.batch = " << fBatch << ";\n";
      out << "      d.trans_a = " << (fAttrTransA ? 1 : 0) << "; d.trans_b = " << (fAttrTransB ? 1 : 0) << ";\n";
      out << "      d.ab_dtype = " << ConvertTypeToRuntimeEnum(fType) << "; d.y_dtype = " << ConvertTypeToRuntimeEnum(fTypeY) << ";\n";
      out << "      d.lda = " << (fAttrTransA ? fShapeA.back() : fK) << "; d.ldb = " << fShapeB.back() << "; d.ldy = " << fN << ";\n";
      out << "      d.stride_a = " << fStrideA << "; d.stride_b = " << fStrideB << "; d.stride_y = " << (fBatch > 1 ? fM * fN : 0)
          << "; d.stride_r = " << (fBatch > 1 ? fM * fN : 0) << ";\n";
      out << "      d.precise = " << (fPrecise ? 1 : 0) << ";\n";
      if (fBIsWeight) out << "      d.flags = SOFIE_B200_GEMM_B_CONSTANT;  // B is an initializer: the plan may keep its own layout of it\n";
      out << "      Check(sofie_b200_gemm_plan_create(ctx, &d, &plan_" << opName << "), \"Gemm " << opName << ": plan\");\n";
      out << fEpi.InitCode("ep_" + opName);
      if (fEpi.biasMode == "SOFIE_B200_BIAS_FULL_F32") out << "      ep_" << opName << ".ldc = " << fN << ";\n";
      out << "      }\n";
      (void)lda;
      return out.str();
   }

   // the leading dimension only reaches M (rows of a shared weight) or the batch count, both plain descriptor fields
   bool SupportsSymbolicDim() const override { return !fIsOutputConstant; }
   std::string Generate_GPU_B200(std::string opName) override
   {
      if (fIsOutputConstant) return "";
      opName = "op_" + opName;
      if (fShapeA.empty() || fShapeB.empty() || fShapeY.empty())
         throw std::runtime_error("SOFIE Gemm Op called to Generate without being initialized first");
      std::stringstream out;
      out << "\n      //--------- Gemm " << opName << " " << ConvertShapeToString(fShapeA) << " * " << ConvertShapeToString(fShapeB) << " -> "
          << ConvertShapeToString(fShapeY) << "\n";
      if (!fEpi.residual.empty())
         out << "      ep_" << opName << ".residual = tensor_" << fEpi.residual << "; ep_" << opName << ".residual_dtype = "
             << ConvertTypeToRuntimeEnum(fResidualType) << "; ep_" << opName << ".ldr = " << fN << ";\n";
      out << fEpi.BindCode("ep_" + opName);
      out << "      Check(sofie_b200_gemm_enqueue(plan_" << opName << ", tensor_" << fNA << ", tensor_" << fNB << ", tensor_" << fNY
          << ", &ep_" << opName << "), \"Gemm " << opName << "\");\n";
      return out.str();
   }

   std::string GenerateDestroyCode_GPU_B200(std::string opName) override
   {
      if (fIsOutputConstant) return "";
      return "      sofie_b200_gemm_plan_destroy(plan_op_" + opName + ");\n";
   }

private:
   ETensorType fResidualType = ETensorType::FLOAT;
};

}  // namespace SOFIE_B200
