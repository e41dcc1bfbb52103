// Quantised and low-precision contractions for the B200 target: QLinearMatMul, QLinearConv,
// QuantizeLinear, DequantizeLinear (ONNX operator definitions) and ScaledGemm (FP8 e4m3 operands
// with per-row / per-column fp32 scales).  The reference has none of them: its parser throws
// "Operator type ... is not yet supported" for these node types
// (parsers/src/RModelParser_ONNX.cxx:1221-1225) and ROperator_Gemm static_asserts float
// (core/inc/SOFIE/operators/ROperator_Gemm.hxx:67-68).  They implement the same ROperator
// interface so that the parser and RModel treat them like any other operator.
//
// Requantisation is fixed once, here, at generation time: the multiplier
// M = a_scale * b_scale / y_scale is computed in fp32 on the host (per output channel when b_scale
// is a vector) and the kernels evaluate sat(rint(float(acc) * M) + y_zp), round half to even.
// A non-zero activation zero point is folded into an int32 bias, -a_zp * sum_k B[k,n]; weights
// must be symmetric (zero point 0), which is what the tensor-core path multiplies.
#pragma once
#include "SOFIE_B200/operators/ROperator_Conv.hxx"

namespace SOFIE_B200 {

namespace quant_detail {
inline float ScalarF(RModel &m, const std::string &n, const char *what)
{
   if (!m.IsInitializedTensor(n)) throw std::runtime_error(std::string("SOFIE quantised Op: ") + what + " " + n + " must be an initialized tensor");
   auto v = m.GetTensorData<float>(n);
   if (v.size() != 1) throw std::runtime_error(std::string("SOFIE quantised Op: ") + what + " " + n + " must be a scalar");
   return v[0];
}
inline int ZeroPoint(RModel &m, const std::string &n)
{
   if (n.empty()) return 0;
   if (!m.IsInitializedTensor(n)) throw std::runtime_error("SOFIE quantised Op: zero point " + n + " must be an initialized tensor");
   const auto t = m.GetTensorType(n);
   if (ConvertShapeToLength(m.GetTensorShape(n)) != 1) {
      // a per-channel zero point vector is accepted only if it is all zeros
      if (t == ETensorType::INT8) { for (auto v : m.GetTensorData<int8_t>(n)) if (v) throw std::runtime_error("SOFIE quantised Op: per-channel zero points must be 0"); }
      else if (t == ETensorType::UINT8) { for (auto v : m.GetTensorData<uint8_t>(n)) if (v) throw std::runtime_error("SOFIE quantised Op: per-channel zero points must be 0"); }
      return 0;
   }
   if (t == ETensorType::INT8) return m.GetTensorData<int8_t>(n)[0];
   if (t == ETensorType::UINT8) return m.GetTensorData<uint8_t>(n)[0];
   if (t == ETensorType::INT32) return m.GetTensorData<int32_t>(n)[0];
   throw std::runtime_error("SOFIE quantised Op: zero point " + n + " has an unsupported type");
}
}  // namespace quant_detail

// ---- QLinearMatMul ---------------------------------------------------------------------------------
class ROperator_QLinearMatMul final : public ROperator_B200 {
   bool fBIsWeight = false;
   std::string fNA, fNAScale, fNAZp, fNB, fNBScale, fNBZp, fNYScale, fNYZp, fNY;
   std::vector<size_t> fShapeA, fShapeB, fShapeY;
   size_t fM = 0, fN = 0, fK = 0;
   EpilogueState fEpi;
   ETensorType fTypeY = ETensorType::INT8;
   std::string fNMult, fNBiasI32;

public:
   ROperator_QLinearMatMul(std::string a, std::string aScale, std::string aZp, std::string b, std::string bScale, std::string bZp,
                           std::string yScale, std::string yZp, std::string y)
      : fNA(UTILITY::Clean_name(a)), fNAScale(UTILITY::Clean_name(aScale)), fNAZp(UTILITY::Clean_name(aZp)), fNB(UTILITY::Clean_name(b)),
        fNBScale(UTILITY::Clean_name(bScale)), fNBZp(UTILITY::Clean_name(bZp)), fNYScale(UTILITY::Clean_name(yScale)),
        fNYZp(UTILITY::Clean_name(yZp)), fNY(UTILITY::Clean_name(y))
   {
      fInputTensorNames = {fNA, fNB};
      fOutputTensorNames = {fNY};
   }
   const EpilogueState &GetEpilogue() const { return fEpi; }

   void Initialize(RModel &model) override
   {
      for (auto &n : {fNA, fNB})
         if (!model.CheckIfTensorAlreadyExist(n)) throw std::runtime_error("SOFIE QLinearMatMul Op Input Tensor " + n + " is not found in model");
      if (model.GetTensorType(fNA) != ETensorType::INT8 || model.GetTensorType(fNB) != ETensorType::INT8)
         throw std::runtime_error("SOFIE QLinearMatMul Op: INT8 operands expected");
      fShapeA = model.GetTensorShape(fNA);
      fShapeB = model.GetTensorShape(fNB);
      if (fShapeB.size() != 2 || fShapeA.size() < 2 || fShapeA.back() != fShapeB[0])
         throw std::runtime_error("SOFIE QLinearMatMul Op : invalid input shapes A " + ConvertShapeToString(fShapeA) + " B " + ConvertShapeToString(fShapeB));
      fK = fShapeB[0]; fN = fShapeB[1];
      fBIsWeight = model.IsInitializedTensor(fNB);
      fM = ConvertShapeToLength(fShapeA) / fK;
      fShapeY = fShapeA;
      fShapeY.back() = fN;
      const float aS = quant_detail::ScalarF(model, fNAScale, "a_scale"), yS = quant_detail::ScalarF(model, fNYScale, "y_scale");
      if (!model.IsInitializedTensor(fNBScale)) throw std::runtime_error("SOFIE QLinearMatMul Op: b_scale must be an initialized tensor");
      auto bS = model.GetTensorData<float>(fNBScale);
      if (quant_detail::ZeroPoint(model, fNBZp) != 0) throw std::runtime_error("SOFIE QLinearMatMul Op: b_zero_point must be 0 (symmetric weights)");
      const int aZp = quant_detail::ZeroPoint(model, fNAZp);
      fEpi.outZeroPoint = quant_detail::ZeroPoint(model, fNYZp);
      fTypeY = fNYZp.empty() ? ETensorType::INT8 : model.GetTensorType(fNYZp);
      if (fTypeY != ETensorType::INT8 && fTypeY != ETensorType::UINT8) throw std::runtime_error("SOFIE QLinearMatMul Op: y must be INT8 or UINT8");
      if (bS.size() == 1) {
         fEpi.alpha = aS * bS[0] / yS;  // fp32, evaluated left to right
      } else {
         if (bS.size() != fN) throw std::runtime_error("SOFIE QLinearMatMul Op: b_scale must be a scalar or have one value per column");
         std::vector<float> mult(fN);
         for (size_t j = 0; j < fN; ++j) mult[j] = aS * bS[j] / yS;
         fNMult = fNY + "_requant_mult";
         model.AddInitializedTensor(fNMult, ETensorType::FLOAT, {fN}, mult);
         fEpi.colScale = fNMult;
         fInputTensorNames.push_back(fNMult);
      }
      if (aZp != 0) {
         if (!model.IsInitializedTensor(fNB)) throw std::runtime_error("SOFIE QLinearMatMul Op: a non-zero a_zero_point needs an initialized B");
         auto b = model.GetTensorData<int8_t>(fNB);
         std::vector<int32_t> corr(fN, 0);
         for (size_t k = 0; k < fK; ++k)
            for (size_t j = 0; j < fN; ++j) corr[j] -= int32_t(aZp) * int32_t(b[k * fN + j]);
         fNBiasI32 = fNY + "_zp_bias";
         model.AddInitializedTensor(fNBiasI32, ETensorType::INT32, {fN}, corr);
         fEpi.bias = fNBiasI32;
         fEpi.biasMode = "SOFIE_B200_BIAS_COL_I32";
         fInputTensorNames.push_back(fNBiasI32);
      }
      model.AddIntermediateTensor(fNY, fTypeY, fShapeY);
   }
   std::string GenerateSessionMembersCode_GPU_B200(std::string opName) override
   {
      return "   sofie_b200_gemm_plan *plan_op_" + opName + " = nullptr;\n   sofie_b200_epilogue ep_op_" + opName + "{};\n";
   }
   std::string GenerateInitCode_GPU_B200(std::string opName) override
   {
      opName = "op_" + opName;
      std::stringstream out;
      out << "      {  // QLinearMatMul " << opName << "\n      sofie_b200_gemm_desc d{};\n";
      out << "      d.M = " << fM << "; d.N = " << fN << "; d.K = " << fK << "; d.batch = 1;\n";
      out << "      d.ab_dtype = SOFIE_B200_I8; d.y_dtype = " << ConvertTypeToRuntimeEnum(fTypeY) << ";\n";
      if (fBIsWeight) out << "      d.flags = SOFIE_B200_GEMM_B_CONSTANT;  // B is an initializer: the plan keeps it K-major\n";
      out << "      Check(sofie_b200_gemm_plan_create(ctx, &d, &plan_" << opName << "), \"QLinearMatMul " << opName << ": plan\");\n";
      out << fEpi.InitCode("ep_" + opName) << "      }\n";
      return out.str();
   }
   std::string Generate_GPU_B200(std::string opName) override
   {
      opName = "op_" + opName;
      std::stringstream out;
      out << "\n      //--------- QLinearMatMul " << opName << " " << ConvertShapeToString(fShapeA) << " * " << ConvertShapeToString(fShapeB) << "\n";
      out << fEpi.BindCode("ep_" + opName);
      out << "      Check(sofie_b200_gemm_enqueue(plan_" << opName << ", tensor_" << fNA << ", tensor_" << fNB << ", tensor_" << fNY << ", &ep_"
          << opName << "), \"QLinearMatMul " << opName << "\");\n";
      return out.str();
   }
   std::string GenerateDestroyCode_GPU_B200(std::string opName) override { return "      sofie_b200_gemm_plan_destroy(plan_op_" + opName + ");\n"; }
};

// ---- QLinearConv --------------------------------------------------------------------------------------
class ROperator_QLinearConv final : public ROperator_B200, public ConvLayoutHooks {
   std::string fAttrAutopad;
   std::vector<size_t> fAttrDilations, fAttrKernelShape, fAttrPads, fAttrStrides;
   size_t fAttrGroup;
   std::string fNX, fNXScale, fNXZp, fNW, fNWScale, fNWZp, fNYScale, fNYZp, fNB, fNY;
   std::vector<size_t> fShapeX, fShapeW, fShapeY;
   ConvGeometry fGeo;
   EpilogueState fEpi;
   ETensorType fTypeY = ETensorType::INT8;
   int fXZp = 0;

public:
   ROperator_QLinearConv(std::string autopad, std::vector<size_t> dilations, size_t group, std::vector<size_t> kernelShape,
                         std::vector<size_t> pads, std::vector<size_t> strides, std::string x, std::string xScale, std::string xZp,
                         std::string w, std::string wScale, std::string wZp, std::string yScale, std::string yZp, std::string bias,
                         std::string y)
      : fAttrAutopad(autopad), fAttrDilations(dilations), fAttrKernelShape(kernelShape), fAttrPads(pads), fAttrStrides(strides),
        fAttrGroup(group), fNX(UTILITY::Clean_name(x)), fNXScale(UTILITY::Clean_name(xScale)), fNXZp(UTILITY::Clean_name(xZp)),
        fNW(UTILITY::Clean_name(w)), fNWScale(UTILITY::Clean_name(wScale)), fNWZp(UTILITY::Clean_name(wZp)),
        fNYScale(UTILITY::Clean_name(yScale)), fNYZp(UTILITY::Clean_name(yZp)), fNB(UTILITY::Clean_name(bias)), fNY(UTILITY::Clean_name(y))
   {
      fInputTensorNames = {fNX, fNW};
      fOutputTensorNames = {fNY};
   }
   const ConvGeometry &GetGeometry() const { return fGeo; }
   EActivationType GetActivationType() const override { return fEpi.act; }
   bool HasFusableEpilogue() const override { return true; }
   bool FuseActivation(EActivationType act, float alpha, const std::string &newOutput) override
   {
      // Relu on the quantised output equals clamping the float value at 0 before rounding only when the output zero
      // point is 0: rint(max(v, 0)) + zp differs from max(rint(v) + zp, 0) otherwise
      if (fEpi.act != EActivationType::UNDEFINED || act != EActivationType::RELU || fEpi.outZeroPoint != 0) return false;
      fEpi.act = act; fEpi.actAlpha = alpha;
      fNY = newOutput; fOutputTensorNames = {fNY};
      return true;
   }

   void Initialize(RModel &model) override
   {
      for (auto &n : {fNX, fNW})
         if (!model.CheckIfTensorAlreadyExist(n)) throw std::runtime_error("SOFIE QLinearConv Op Input Tensor " + n + " is not found in model");
      if (model.GetTensorType(fNX) != ETensorType::INT8 || model.GetTensorType(fNW) != ETensorType::INT8)
         throw std::runtime_error("SOFIE QLinearConv Op: INT8 input and weights expected");
      if (!model.IsInitializedTensor(fNW)) throw std::runtime_error("SOFIE QLinearConv Op: weights must be initialized");
      fShapeX = model.GetTensorShape(fNX);
      fShapeW = model.GetTensorShape(fNW);
      if (fShapeX.size() != 4) throw std::runtime_error("SOFIE QLinearConv Op: NCHW input expected");
      fGeo = ConvShapeInference(fShapeX, fShapeW, fAttrAutopad, fAttrDilations, fAttrGroup, fAttrKernelShape, fAttrPads, fAttrStrides);
      fShapeY = {fGeo.N, fGeo.K, fGeo.Ho, fGeo.Wo};
      const float xS = quant_detail::ScalarF(model, fNXScale, "x_scale"), yS = quant_detail::ScalarF(model, fNYScale, "y_scale");
      auto wS = model.GetTensorData<float>(fNWScale);
      if (wS.size() != 1 && wS.size() != fGeo.K) throw std::runtime_error("SOFIE QLinearConv Op: w_scale must be a scalar or per output channel");
      if (quant_detail::ZeroPoint(model, fNWZp) != 0) throw std::runtime_error("SOFIE QLinearConv Op: w_zero_point must be 0 (symmetric weights)");
      fXZp = quant_detail::ZeroPoint(model, fNXZp);
      fEpi.outZeroPoint = quant_detail::ZeroPoint(model, fNYZp);
      fTypeY = fNYZp.empty() ? ETensorType::INT8 : model.GetTensorType(fNYZp);
      std::vector<float> mult(fGeo.K);
      for (size_t k = 0; k < fGeo.K; ++k) mult[k] = xS * wS[wS.size() == 1 ? 0 : k] / yS;
      fEpi.colScale = fNY + "_requant_mult";
      model.AddInitializedTensor(fEpi.colScale, ETensorType::FLOAT, {fGeo.K}, mult);
      fInputTensorNames.push_back(fEpi.colScale);
      // int32 bias at scale x_scale*w_scale[c]; a non-zero x zero point adds -x_zp * sum(w[c,:,:,:])
      std::vector<int32_t> bias(fGeo.K, 0);
      bool haveBias = false;
      if (!fNB.empty()) {
         if (!model.IsInitializedTensor(fNB) || model.GetTensorType(fNB) != ETensorType::INT32)
            throw std::runtime_error("SOFIE QLinearConv Op: the bias must be an initialized INT32 tensor");
         bias = model.GetTensorData<int32_t>(fNB);
         haveBias = true;
      }
      if (fXZp != 0) {
         auto w = model.GetTensorData<int8_t>(fNW);
         const size_t per = w.size() / fGeo.K;
         for (size_t k = 0; k < fGeo.K; ++k) {
            int32_t s = 0;
            for (size_t i = 0; i < per; ++i) s += w[k * per + i];
            bias[k] -= int32_t(fXZp) * s;
         }
         haveBias = true;
      }
      if (haveBias) {
         fEpi.bias = fNY + "_bias_i32";
         fEpi.biasMode = "SOFIE_B200_BIAS_COL_I32";
         model.AddInitializedTensor(fEpi.bias, ETensorType::INT32, {fGeo.K}, bias);
         fInputTensorNames.push_back(fEpi.bias);
      }
      model.AddIntermediateTensor(fNY, fTypeY, fShapeY);
   }
   // ---- layout pass
   const ConvGeometry &Geometry() const override { return fGeo; }
   bool IsInt8() const override { return true; }
   int InputZeroPoint() const override { return fXZp; }
   bool HasResidual() const override { return !fEpi.residual.empty(); }
   const std::string &LayoutInput() const override { return fNX; }
   const std::string &LayoutOutput() const override { return fNY; }
   void SetLayouts(int x, int y) override { fXLayout = x; fYLayout = y; }
   size_t Workspace() const { return ConvWorkspaceBytes(fGeo, 1, 1, fXLayout, fYLayout, fXZp); }

   std::vector<DeviceScratch> GetDeviceScratch_GPU_B200() const override
   {
      return Workspace() ? std::vector<DeviceScratch>{{fNY + "_xcol", Workspace()}} : std::vector<DeviceScratch>{};
   }
   std::string GenerateSessionMembersCode_GPU_B200(std::string opName) override
   {
      return "   sofie_b200_conv_plan *plan_op_" + opName + " = nullptr;\n   sofie_b200_epilogue ep_op_" + opName + "{};\n";
   }
   std::string GenerateInitCode_GPU_B200(std::string opName) override
   {
      opName = "op_" + opName;
      std::stringstream out;
      out << "      {  // QLinearConv " << opName << "\n" << ConvDescCode(fGeo, "SOFIE_B200_I8", ConvertTypeToRuntimeEnum(fTypeY), fXZp, fXLayout, fYLayout);
      out << "      Check(sofie_b200_conv_plan_create(ctx, &d, tensor_" << fNW << ", &plan_" << opName << "), \"QLinearConv " << opName << ": plan\");\n";
      out << "      if (sofie_b200_conv_workspace_bytes(plan_" << opName << ") > " << Workspace() << "LL)\n"
          << "         throw std::runtime_error(\"QLinearConv " << opName << ": the library wants more scratch than the arena reserves\");\n";
      out << fEpi.InitCode("ep_" + opName) << "      }\n";
      return out.str();
   }
   std::string Generate_GPU_B200(std::string opName) override
   {
      opName = "op_" + opName;
      std::stringstream out;
      out << "\n      //--------- QLinearConv " << opName << " " << ConvertShapeToString(fShapeX) << " -> " << ConvertShapeToString(fShapeY) << "\n";
      out << fEpi.BindCode("ep_" + opName);
      out << "      Check(sofie_b200_conv_enqueue(plan_" << opName << ", tensor_" << fNX << ", tensor_" << fNY << ", "
          << (Workspace() ? "tensor_" + fNY + "_xcol" : std::string("nullptr")) << ", &ep_" << opName << "), \"QLinearConv " << opName << "\");\n";
      return out.str();
   }
   std::string GenerateDestroyCode_GPU_B200(std::string opName) override { return "      sofie_b200_conv_plan_destroy(plan_op_" + opName + ");\n"; }
};

// ---- QuantizeLinear / DequantizeLinear --------------------------------------------------------------------
class ROperator_QuantizeLinear final : public ROperator_B200 {
   std::string fNX, fNScale, fNZp, fNY;
   int64_t fAxis;
   bool fDequantize;
   std::vector<size_t> fShape;
   ETensorType fQType = ETensorType::INT8;
   size_t fChannels = 1, fInner = 1;

public:
   // dequantize = false: QuantizeLinear(x, y_scale, y_zero_point); true: DequantizeLinear(x, x_scale, x_zero_point)
   ROperator_QuantizeLinear(bool dequantize, int64_t axis, std::string x, std::string scale, std::string zp, std::string y)
      : fNX(UTILITY::Clean_name(x)), fNScale(UTILITY::Clean_name(scale)), fNZp(UTILITY::Clean_name(zp)), fNY(UTILITY::Clean_name(y)),
        fAxis(axis), fDequantize(dequantize)
   {
      fInputTensorNames = {fNX, fNScale};
      if (!fNZp.empty()) fInputTensorNames.push_back(fNZp);
      fOutputTensorNames = {fNY};
   }
   bool IsDequantize() const { return fDequantize; }
   bool IsPerTensor() const { return fChannels == 1; }
   const std::string &NameY() const { return fNY; }
   const std::string &NameX() const { return fNX; }
   const std::string &NameScale() const { return fNScale; }
   const std::string &NameZp() const { return fNZp; }
   void Initialize(RModel &model) override
   {
      for (auto &n : {fNX, fNScale})
         if (!model.CheckIfTensorAlreadyExist(n)) throw std::runtime_error("SOFIE QuantizeLinear Op Input Tensor " + n + " is not found in model");
      fShape = model.GetTensorShape(fNX);
      const size_t ns = ConvertShapeToLength(model.GetTensorShape(fNScale));
      if (ns != 1) {
         const int64_t rank = int64_t(fShape.size()), ax = fAxis < 0 ? fAxis + rank : fAxis;
         if (ax < 0 || ax >= rank || fShape[ax] != ns) throw std::runtime_error("SOFIE QuantizeLinear Op: the scale does not match the axis dimension");
         fChannels = ns;
         for (int64_t i = ax + 1; i < rank; ++i) fInner *= fShape[i];
      }
      if (!fNZp.empty()) {
         if (model.GetTensorType(fNZp) != ETensorType::INT8 && model.GetTensorType(fNZp) != ETensorType::UINT8)
            throw std::runtime_error("SOFIE QuantizeLinear Op: zero point must be INT8 or UINT8");
         if (!model.IsInitializedTensor(fNZp)) throw std::runtime_error("SOFIE QuantizeLinear Op: zero point must be initialized");
      }
      if (fDequantize) {
         fQType = model.GetTensorType(fNX);
         model.AddIntermediateTensor(fNY, ETensorType::FLOAT, fShape);
      } else {
         if (model.GetTensorType(fNX) != ETensorType::FLOAT) throw std::runtime_error("SOFIE QuantizeLinear Op: FLOAT input expected");
         fQType = fNZp.empty() ? ETensorType::UINT8 : model.GetTensorType(fNZp);
         model.AddIntermediateTensor(fNY, fQType, fShape);
      }
      // the kernels take the zero point as int32 [channels]
      if (!fNZp.empty()) {
         std::vector<int32_t> z;
         if (model.GetTensorType(fNZp) == ETensorType::INT8) for (auto v : model.GetTensorData<int8_t>(fNZp)) z.push_back(v);
         else for (auto v : model.GetTensorData<uint8_t>(fNZp)) z.push_back(v);
         if (z.size() == 1 && fChannels > 1) z.assign(fChannels, z[0]);
         model.AddInitializedTensor(fNY + "_zp_i32", ETensorType::INT32, {z.size()}, z);
         fInputTensorNames = {fNX, fNScale, fNY + "_zp_i32"};
      }
   }
   std::string Generate_GPU_B200(std::string opName) override
   {
      opName = "op_" + opName;
      const std::string zp = fNZp.empty() ? "nullptr" : "tensor_" + fNY + "_zp_i32";
      std::stringstream out;
      out << "\n      //------ " << (fDequantize ? "DequantizeLinear " : "QuantizeLinear ") << opName << "\n";
      out << "      Check(sofie_b200_" << (fDequantize ? "dequantize" : "quantize") << "_enqueue(ctx, tensor_" << fNX << ", tensor_" << fNY << ", "
          << ConvertTypeToRuntimeEnum(fQType) << ", " << ConvertShapeToLength(fShape) << ", tensor_" << fNScale << ", " << zp << ", " << fChannels
          << ", " << fInner << "), \"QuantizeLinear " << opName << "\");\n";
      return out.str();
   }
};

// ---- ScaledGemm: FP8 e4m3 x e4m3 -> fp32, per-row / per-column scales, bias, activation -------------------------
class ROperator_ScaledGemm final : public ROperator_B200 {
   bool fBIsWeight = false;
   std::string fNA, fNB, fNRowScale, fNColScale, fNBias, fNY;
   int fTransB;
   EpilogueState fEpi;
   ETensorType fTypeY;
   std::vector<size_t> fShapeA, fShapeB;
   size_t fM = 0, fN = 0, fK = 0;

public:
   ROperator_ScaledGemm(int transB, std::string a, std::string b, std::string rowScale, std::string colScale, std::string bias, std::string y,
                        ETensorType yType = ETensorType::BFLOAT16, EActivationType act = EActivationType::UNDEFINED)
      : fNA(UTILITY::Clean_name(a)), fNB(UTILITY::Clean_name(b)), fNRowScale(UTILITY::Clean_name(rowScale)),
        fNColScale(UTILITY::Clean_name(colScale)), fNBias(UTILITY::Clean_name(bias)), fNY(UTILITY::Clean_name(y)), fTransB(transB), fTypeY(yType)
   {
      fEpi.act = act;
      fInputTensorNames = {fNA, fNB};
      for (auto &n : {fNRowScale, fNColScale, fNBias})
         if (!n.empty()) fInputTensorNames.push_back(n);
      fOutputTensorNames = {fNY};
   }
   EActivationType GetActivationType() const override { return fEpi.act; }
   bool HasFusableEpilogue() const override { return true; }
   bool FuseActivation(EActivationType act, float alpha, const std::string &newOutput) override
   {
      if (fEpi.act != EActivationType::UNDEFINED) return false;
      fEpi.act = act; fEpi.actAlpha = alpha;
      fNY = newOutput; fOutputTensorNames = {fNY};
      return true;
   }
   void Initialize(RModel &model) override
   {
      for (auto &n : fInputTensorNames)
         if (!model.CheckIfTensorAlreadyExist(n)) throw std::runtime_error("SOFIE ScaledGemm Op Input Tensor " + n + " is not found in model");
      if (model.GetTensorType(fNA) != ETensorType::FLOAT8E4M3FN || model.GetTensorType(fNB) != ETensorType::FLOAT8E4M3FN)
         throw std::runtime_error("SOFIE ScaledGemm Op: FLOAT8E4M3FN operands expected");
      fShapeA = model.GetTensorShape(fNA);
      fShapeB = model.GetTensorShape(fNB);
      if (fShapeA.size() != 2 || fShapeB.size() != 2) throw std::runtime_error("SOFIE ScaledGemm Op: rank-2 operands expected");
      fM = fShapeA[0]; fK = fShapeA[1];
      fN = fTransB ? fShapeB[0] : fShapeB[1];
      fBIsWeight = model.IsInitializedTensor(fNB);
      if ((fTransB ? fShapeB[1] : fShapeB[0]) != fK) throw std::runtime_error("SOFIE ScaledGemm Op : invalid input shapes");
      if (!fNColScale.empty()) fEpi.colScale = fNColScale;
      if (!fNBias.empty()) { fEpi.bias = fNBias; fEpi.biasMode = "SOFIE_B200_BIAS_COL_F32"; }
      model.AddIntermediateTensor(fNY, fTypeY, {fM, fN});
   }
   std::string GenerateSessionMembersCode_GPU_B200(std::string opName) override
   {
      return "   sofie_b200_gemm_plan *plan_op_" + opName + " = nullptr;\n   sofie_b200_epilogue ep_op_" + opName + "{};\n";
   }
   std::string GenerateInitCode_GPU_B200(std::string opName) override
   {
      opName = "op_" + opName;
      std::stringstream out;
      out << "      {  // ScaledGemm " << opName << "\n      sofie_b200_gemm_desc d{};\n";
      out << "      d.M = " << fM << "; d.N = " << fN << "; d.K = " << fK << "; d.batch = 1; d.trans_b = " << fTransB << ";\n";
      out << "      d.ab_dtype = SOFIE_B200_F8E4M3; d.y_dtype = " << ConvertTypeToRuntimeEnum(fTypeY) << ";\n";
      if (fBIsWeight) out << "      d.flags = SOFIE_B200_GEMM_B_CONSTANT;  // B is an initializer: the plan keeps it K-major\n";
      out << "      Check(sofie_b200_gemm_plan_create(ctx, &d, &plan_" << opName << "), \"ScaledGemm " << opName << ": plan\");\n";
      out << fEpi.InitCode("ep_" + opName);
      out << "      }\n";
      return out.str();
   }
   std::string Generate_GPU_B200(std::string opName) override
   {
      opName = "op_" + opName;
      std::stringstream out;
      out << "\n      //--------- ScaledGemm " << opName << "\n";
      if (!fNRowScale.empty()) out << "      ep_" << opName << ".row_scale = tensor_" << fNRowScale << ";\n";
      out << fEpi.BindCode("ep_" + opName);
      out << "      Check(sofie_b200_gemm_enqueue(plan_" << opName << ", tensor_" << fNA << ", tensor_" << fNB << ", tensor_" << fNY << ", &ep_"
          << opName << "), \"ScaledGemm " << opName << "\");\n";
      return out.str();
   }
   std::string GenerateDestroyCode_GPU_B200(std::string opName) override { return "      sofie_b200_gemm_plan_destroy(plan_op_" + opName + ");\n"; }
};

}  // namespace SOFIE_B200
