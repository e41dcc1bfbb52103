// Conv for the B200 target.
//
// Constructor, attribute defaults and shape inference follow the reference's ROperator_Conv
// (core/inc/SOFIE/operators/ROperator_Conv.hxx:83-120 constructor, :123-262 DoShapeInference):
// group 0 means "infer from the weights", dilated kernel extents, SAME_UPPER / SAME_LOWER, and
// the reference's own default of pads = 1 when auto_pad is NOTSET and no pads are given.
// Where the reference emits a host loop of per-image im2col + blas.matmul (:985-1103), this
// operator emits one sofie_b200_conv_plan (weights re-laid once) and one enqueue over the batch.
// 1-D and 2-D convolutions (a 1-D one is a 2-D one of height 1).  A 3-D convolution is emitted as three calls: the depth
// taps are unfolded into channels (X [N,C,D,H,W] -> [N*Do, C*T, H, W]; the weights [K,C,T,R,S] are already [K, C*T, R, S] in
// memory), the 2-D convolution runs over the N*Do slices, and the result [N*Do, K, Ho, Wo] is transposed to [N,K,Do,Ho,Wo].
#pragma once
#include "SOFIE_B200/operators/ROperator_Gemm.hxx"

namespace SOFIE_B200 {

struct ConvGeometry {
   size_t N = 0, C = 0, H = 1, W = 1, K = 0, R = 1, S = 1, Ho = 1, Wo = 1, group = 1;
   size_t pads[4] = {0, 0, 0, 0};  // top, left, bottom, right
   size_t strides[2] = {1, 1}, dil[2] = {1, 1};
   // A 3-D convolution lowered to 2-D: N and C above are then N*Do and C*T of the 2-D convolution that runs; these are the
   // extents of the original tensors and the depth taps.
   size_t N3 = 0, C3 = 0, D = 1, T = 1, Do = 1, padFront = 0, padBack = 0, strideD = 1, dilD = 1;
   bool Is3D() const { return N3 != 0; }
};

// Shape rules of ROperator_Conv.hxx:123-262 for rank-3 and rank-4 inputs.
inline ConvGeometry ConvShapeInference(const std::vector<size_t> &x, const std::vector<size_t> &w, std::string autopad,
                                       std::vector<size_t> dilations, size_t group, std::vector<size_t> kernel,
                                       std::vector<size_t> pads, std::vector<size_t> strides)
{
   const size_t dim = x.size() - 2;
   if (dim < 1 || dim > 3) throw std::runtime_error("SOFIE Conv Op Shape inference - invalid inputs ");
   if (w.size() - 2 != dim) throw std::runtime_error("SOFIE Conv Op Shape inference - invalid weights ");
   if (dim == 3) {
      // depth first (ROperator_Conv.hxx:123-262 treats the three spatial ranks alike), then the 2-D rules on the slices
      const size_t T = kernel.empty() ? w[2] : kernel[0];
      if (dilations.empty()) dilations = {1, 1, 1};
      if (strides.empty()) strides = {1, 1, 1};
      dilations.resize(3, 1); strides.resize(3, 1);
      const size_t et = T + (dilations[0] - 1) * (T - 1);
      size_t front = 0, back = 0;
      std::vector<size_t> pads2;
      if (autopad == "NOTSET") {
         if (pads.empty()) pads = {1, 1, 1, 1, 1, 1};   // the reference's default
         if (pads.size() != 6) throw std::runtime_error("SOFIE Conv Op Shape inference - invalid pads for a 3-D convolution");
         front = pads[0]; back = pads[3];
         pads2 = {pads[1], pads[2], pads[4], pads[5]};
      } else if (autopad == "SAME_UPPER" || autopad == "SAME_LOWER") {
         const size_t out = (x[2] + strides[0] - 1) / strides[0];
         const long total = std::max(0L, long((out - 1) * strides[0] + et) - long(x[2]));
         front = autopad == "SAME_UPPER" ? total / 2 : total - total / 2;
         back = size_t(total) - front;
      } else if (autopad != "VALID") {
         throw std::runtime_error("SOFIE Conv Op invalid fAutopad");
      }
      if (x[2] + front + back < et) throw std::runtime_error("SOFIE Conv Op -  invalid values");
      const size_t Do = (x[2] + front + back - et) / strides[0] + 1;
      const size_t grp = group == 0 ? x[1] / w[1] : group;
      ConvGeometry g = ConvShapeInference({x[0] * Do, x[1] * T, x[3], x[4]}, {w[0], w[1] * T, w[3], w[4]}, autopad, {dilations[1], dilations[2]}, grp,
                                          kernel.empty() ? std::vector<size_t>{} : std::vector<size_t>{kernel[1], kernel[2]}, pads2, {strides[1], strides[2]});
      g.N3 = x[0]; g.C3 = x[1]; g.D = x[2]; g.T = T; g.Do = Do; g.padFront = front; g.padBack = back; g.strideD = strides[0]; g.dilD = dilations[0];
      return g;
   }
   ConvGeometry g;
   g.N = x[0]; g.C = x[1]; g.K = w[0];
   g.group = group == 0 ? x[1] / w[1] : group;
   const bool d1 = dim == 1;
   g.H = d1 ? 1 : x[2];
   g.W = d1 ? x[2] : x[3];
   const size_t k1 = kernel.empty() ? w[2] : kernel[0];
   const size_t k2 = d1 ? 1 : (kernel.empty() ? w[3] : kernel[1]);
   g.R = d1 ? 1 : k1;
   g.S = d1 ? k1 : k2;
   if (dilations.empty()) dilations = {1, 1};
   dilations.resize(2, 1);
   if (strides.empty()) strides = {1, 1};
   strides.resize(2, 1);
   g.dil[0] = d1 ? 1 : dilations[0]; g.dil[1] = d1 ? dilations[0] : dilations[1];
   g.strides[0] = d1 ? 1 : strides[0]; g.strides[1] = d1 ? strides[0] : strides[1];
   const size_t er = g.R + (g.dil[0] - 1) * (g.R - 1), es = g.S + (g.dil[1] - 1) * (g.S - 1);
   if (autopad == "NOTSET") {
      if (pads.empty()) pads = d1 ? std::vector<size_t>{1, 1} : std::vector<size_t>{1, 1, 1, 1};  // the reference's default
      if (d1) { g.pads[1] = pads[0]; g.pads[3] = pads[1]; }
      else { g.pads[0] = pads[0]; g.pads[1] = pads[1]; g.pads[2] = pads[2]; g.pads[3] = pads[3]; }
   } else if (autopad == "SAME_UPPER" || autopad == "SAME_LOWER") {
      // total = max(0, (ceil(in/stride)-1)*stride + kernel - in); UPPER puts the odd element at the end
      const size_t in[2] = {g.H, g.W}, ek[2] = {er, es};
      for (int d = d1 ? 1 : 0; d < 2; ++d) {
         const size_t out = (in[d] + g.strides[d] - 1) / g.strides[d];
         const long total = std::max(0L, long((out - 1) * g.strides[d] + ek[d]) - long(in[d]));
         const size_t lo = autopad == "SAME_UPPER" ? total / 2 : total - total / 2;
         g.pads[d] = lo;
         g.pads[d + 2] = size_t(total) - lo;
      }
   } else if (autopad != "VALID") {
      throw std::runtime_error("SOFIE Conv Op invalid fAutopad");
   }
   if (g.H + g.pads[0] + g.pads[2] < er || g.W + g.pads[1] + g.pads[3] < es)
      throw std::runtime_error("SOFIE Conv Op -  invalid values");
   g.Ho = (g.H + g.pads[0] + g.pads[2] - er) / g.strides[0] + 1;
   g.Wo = (g.W + g.pads[1] + g.pads[3] - es) / g.strides[1] + 1;
   return g;
}

// Layout of a convolution's tensors (sofie_b200_conv_desc::x_layout / y_layout): 0 NCHW, 1 channels-last, 2 channels-last TF32
// pairs.  The reference keeps every tensor NCHW; the layout pass of RModel sets these for conv -> conv chains.
class ConvLayoutHooks {
public:
   virtual ~ConvLayoutHooks() = default;
   virtual const ConvGeometry &Geometry() const = 0;
   virtual bool IsInt8() const = 0;
   virtual int InputZeroPoint() const { return 0; }
   virtual bool HasResidual() const = 0;
   virtual const std::string &LayoutInput() const = 0;
   virtual const std::string &LayoutOutput() const = 0;
   virtual void SetLayouts(int xLayout, int yLayout) = 0;
   int fXLayout = 0, fYLayout = 0;
};

inline std::string ConvDescCode(const ConvGeometry &g, const std::string &xEnum, const std::string &yEnum, int xZeroPoint, int xLayout = 0, int yLayout = 0)
{
   std::stringstream out;
   out << "      sofie_b200_conv_desc d{};\n";
   out << "      d.N = " << g.N << "; d.C = " << g.C << "; d.H = " << g.H << "; d.W = " << g.W << "; d.K = " << g.K << "; d.R = " << g.R
       << "; d.S = " << g.S << ";\n";
   out << "      d.pad_top = " << g.pads[0] << "; d.pad_left = " << g.pads[1] << "; d.pad_bottom = " << g.pads[2] << "; d.pad_right = " << g.pads[3] << ";\n";
   out << "      d.stride_h = " << g.strides[0] << "; d.stride_w = " << g.strides[1] << "; d.dil_h = " << g.dil[0] << "; d.dil_w = " << g.dil[1]
       << "; d.groups = " << g.group << ";\n";
   out << "      d.x_dtype = " << xEnum << "; d.y_dtype = " << yEnum << "; d.x_zero_point = " << xZeroPoint << "; d.precise = 1;\n";
   if (xLayout || yLayout) out << "      d.x_layout = " << xLayout << "; d.y_layout = " << yLayout << ";\n";
   return out.str();
}

// The library's plan selection restated (sofie_b200_conv_plan_kernel): the forms that need no workspace.
inline bool ConvNeedsNoWorkspace(const ConvGeometry &g, size_t elemSize, size_t outElemSize, int xLayout, int yLayout, int xZeroPoint)
{
   // the 3-channel 3x3 first layer on the CUDA cores, while its filters and staging fit its shared memory -- except the int8
   // layer with a channels-last output and at least 16384 output pixels, which unfolds to [pixels][32] for the tensor cores
   const bool stem = elemSize == 1 && yLayout == 1 && g.K % 16 == 0 && g.N * g.Ho * g.Wo >= 16384;
   if (g.group == 1 && g.C == 3 && g.R == 3 && g.S == 3 && xLayout == 0 && g.K <= 256 && !stem) {
      const size_t wsm = g.K * ((elemSize == 4 ? 28 * 4 : 8 * 4) + 16);
      const size_t stage = yLayout == 0 ? 0 : (yLayout == 2 ? 4 * 32 * (32 * 8 + 16) : 4 * 32 * (g.K * outElemSize + 16));
      if (wsm + stage <= 160 * 1024) return true;
   }
   if (xLayout == 2) return true;   // TF32 pairs read in place
   const bool hasPad = g.pads[0] || g.pads[1] || g.pads[2] || g.pads[3];
   // implicit convolution: channels-last int8, a pixel a whole number of 64-byte blocks, padding that reads as zero
   return xLayout == 1 && yLayout == 1 && g.group == 1 && elemSize == 1 && (g.C * elemSize) % 64 == 0 && (xZeroPoint == 0 || !hasPad);
}

inline size_t ConvWorkspaceBytes(const ConvGeometry &g, size_t elemSize, size_t outElemSize = 0, int xLayout = 0, int yLayout = 0, int xZeroPoint = 0)
{
   if (ConvNeedsNoWorkspace(g, elemSize, outElemSize ? outElemSize : elemSize, xLayout, yLayout, xZeroPoint)) return 0;
   // [groups][N][Ho*Wo][kpad] with kpad = C/groups*R*S rounded up to 16 bytes (sofie_b200_conv_workspace_bytes)
   const size_t kdim = g.C / g.group * g.R * g.S, vec = 16 / elemSize;
   size_t kpad = (kdim + vec - 1) / vec * vec;
   // a large fp32 convolution runs as 3xTF32 and unfolds into hi | lo segments of K rounded up to 32 (SOFIE_B200_SPLIT_MIN_FLOPS of sofie_b200.h)
   const bool split = elemSize == sizeof(float) && 2.0 * double(g.K / g.group) * double(g.Ho * g.Wo) * double(kpad) * double(g.N) >= 4e8;
   if (split) kpad = (kdim + 31) / 32 * 32 * 2;
   size_t bytes = g.group * g.N * g.Ho * g.Wo * kpad * elemSize;
   // when the channels per group are whole 16-byte vectors the library unfolds from a channels-last copy of the input kept behind it
   if ((g.C / g.group) % vec == 0 && xLayout == 0) bytes = (bytes + 255) / 256 * 256 + g.N * g.C * g.H * g.W * elemSize;
   return bytes;
}

template <typename T>
class ROperator_Conv final : public ROperator_B200, public ConvLayoutHooks {
   static_assert(std::is_same<T, float>::value, "ROperator_Conv<T>: T is float, as in the reference");

private:
   std::string fAttrAutopad;
   std::vector<size_t> fAttrDilations, fAttrKernelShape, fAttrPads, fAttrStrides;
   size_t fAttrGroup;
   std::string fNX, fNW, fNB, fNY;
   std::vector<size_t> fShapeX, fShapeW, fShapeY;
   ConvGeometry fGeo;
   EpilogueState fEpi;
   ETensorType fResidualType = ETensorType::FLOAT;

public:
   ROperator_Conv(std::string autopad, std::vector<size_t> dilations, size_t group, std::vector<size_t> kernelShape,
                  std::vector<size_t> pads, std::vector<size_t> strides, std::string nameX, std::string nameW, std::string nameB,
                  std::string nameY)
      : fAttrAutopad(autopad), fAttrDilations(dilations), fAttrKernelShape(kernelShape), fAttrPads(pads), fAttrStrides(strides),
        fAttrGroup(group), fNX(UTILITY::Clean_name(nameX)), fNW(UTILITY::Clean_name(nameW)), fNB(UTILITY::Clean_name(nameB)),
        fNY(UTILITY::Clean_name(nameY))
   {
      fInputTensorNames = {fNX, fNW};
      if (!fNB.empty()) fInputTensorNames.push_back(fNB);
      fOutputTensorNames = {fNY};
   }
   ROperator_Conv(std::string autopad, std::vector<size_t> dilations, size_t group, std::vector<size_t> kernelShape,
                  std::vector<size_t> pads, std::vector<size_t> strides, std::string nameX, std::string nameW, std::string nameY)
      : ROperator_Conv(autopad, dilations, group, kernelShape, pads, strides, nameX, nameW, "", nameY) {}

   const ConvGeometry &GetGeometry() const { return fGeo; }
   const EpilogueState &GetEpilogue() const { return fEpi; }
   EActivationType GetActivationType() const override { return fEpi.act; }

   void Initialize(RModel &model) override
   {
      if (!model.CheckIfTensorAlreadyExist(fNX)) throw std::runtime_error("SOFIE Conv op Input Tensor " + fNX + " is not found in model");
      if (!model.CheckIfTensorAlreadyExist(fNW)) throw std::runtime_error("SOFIE Conv op Input weight Tensor " + fNW + " is not found in model");
      fShapeX = model.GetTensorShape(fNX);
      fShapeW = model.GetTensorShape(fNW);
      if (fShapeX.size() < 3 || fShapeX.size() > 5)
         throw std::runtime_error("SOFIE Conv Op input data tensor" + fNX + " is not of 3,4 or 5 dimensions");
      if (model.GetTensorType(fNX) != ETensorType::FLOAT)
         throw std::runtime_error("SOFIE Conv Op: FLOAT input expected (int8 convolutions use QLinearConv)");
      if (!model.IsInitializedTensor(fNW))
         throw std::runtime_error("SOFIE Conv Op: the B200 path re-lays the weights at Session construction and needs them initialized");
      fGeo = ConvShapeInference(fShapeX, fShapeW, fAttrAutopad, fAttrDilations, fAttrGroup, fAttrKernelShape, fAttrPads, fAttrStrides);
      if (fShapeW[1] * fGeo.group != (fGeo.Is3D() ? fGeo.C3 : fGeo.C))
         throw std::runtime_error("SOFIE Conv Op: weight channels x group does not match the input channels");
      fShapeY = fShapeX.size() == 3 ? std::vector<size_t>{fGeo.N, fGeo.K, fGeo.Wo} : std::vector<size_t>{fGeo.N, fGeo.K, fGeo.Ho, fGeo.Wo};
      if (fGeo.Is3D()) fShapeY = {fGeo.N3, fGeo.K, fGeo.Do, fGeo.Ho, fGeo.Wo};
      if (!fNB.empty()) {
         if (!model.CheckIfTensorAlreadyExist(fNB)) throw std::runtime_error("SOFIE Conv op Input Tensor " + fNB + " is not found in model");
         if (ConvertShapeToLength(model.GetTensorShape(fNB)) != fGeo.K)
            throw std::runtime_error("SOFIE Conv op: Bias Tensor has not the right length (output channels)");
         fEpi.bias = fNB;
         fEpi.biasMode = "SOFIE_B200_BIAS_COL_F32";
      }
      model.AddIntermediateTensor(fNY, ETensorType::FLOAT, fShapeY);
   }

   bool HasFusableEpilogue() const override { return true; }
   bool FuseActivation(EActivationType act, float alpha, const std::string &newOutput) override
   {
      if (fEpi.act != EActivationType::UNDEFINED) return false;
      fEpi.act = act; fEpi.actAlpha = alpha;
      fNY = newOutput; fOutputTensorNames = {fNY};
      return true;
   }
   bool FuseScaleShift(RModel &model, const std::string &scale, const std::string &shift, const std::string &newOutput) override
   {
      if (fEpi.act != EActivationType::UNDEFINED || !fEpi.residual.empty()) return false;
      if (!fEpi.bias.empty() && !model.IsInitializedTensor(fEpi.bias)) return false;
      auto s = model.GetTensorData<float>(scale), t = model.GetTensorData<float>(shift);
      if (s.size() != fGeo.K || t.size() != fGeo.K) return false;
      std::vector<float> nb(fGeo.K);
      if (!fEpi.bias.empty()) {
         auto b = model.GetTensorData<float>(fEpi.bias);
         for (size_t j = 0; j < fGeo.K; ++j) nb[j] = b[j] * s[j] + t[j];
      } else nb = t;
      if (!fEpi.colScale.empty()) {
         auto cs = model.GetTensorData<float>(fEpi.colScale);
         for (size_t j = 0; j < fGeo.K; ++j) s[j] *= cs[j];
      }
      fEpi.colScale = newOutput + "_fold_scale";
      fEpi.bias = newOutput + "_fold_bias";
      fEpi.biasMode = "SOFIE_B200_BIAS_COL_F32";
      model.AddInitializedTensor(fEpi.colScale, ETensorType::FLOAT, {fGeo.K}, s);
      model.AddInitializedTensor(fEpi.bias, ETensorType::FLOAT, {fGeo.K}, nb);
      fInputTensorNames = {fNX, fNW, fEpi.colScale, fEpi.bias};
      fNY = newOutput; fOutputTensorNames = {fNY};
      return true;
   }
   bool FuseResidual(RModel &model, const std::string &residual, const std::string &newOutput) override
   {
      if (fEpi.act != EActivationType::UNDEFINED || !fEpi.residual.empty()) return false;
      if (fGeo.Is3D()) return false;   // the 2-D convolution of a lowered 3-D one writes [N*Do, K, Ho, Wo], not the residual's layout
      if (model.GetTensorShape(residual) != fShapeY || model.GetTensorType(residual) != ETensorType::FLOAT) return false;
      fEpi.residual = residual;
      fInputTensorNames.push_back(residual);
      fNY = newOutput; fOutputTensorNames = {fNY};
      return true;
   }

   // ---- layout pass
   const ConvGeometry &Geometry() const override { return fGeo; }
   bool IsInt8() const override { return false; }
   bool HasResidual() const override { return !fEpi.residual.empty(); }
   const std::string &LayoutInput() const override { return fNX; }
   const std::string &LayoutOutput() const override { return fNY; }
   void SetLayouts(int x, int y) override { fXLayout = x; fYLayout = y; }
   size_t Workspace() const { return ConvWorkspaceBytes(fGeo, sizeof(float), sizeof(float), fXLayout, fYLayout, 0); }

   std::vector<DeviceScratch> GetDeviceScratch_GPU_B200() const override
   {
      std::vector<DeviceScratch> s;
      if (Workspace()) s.push_back({fNY + "_xcol", Workspace()});
      if (fGeo.Is3D()) {
         s.push_back({fNY + "_slices", fGeo.N * fGeo.C * fGeo.H * fGeo.W * sizeof(float)});        // X with the depth taps as channels
         s.push_back({fNY + "_planes", fGeo.N * fGeo.K * fGeo.Ho * fGeo.Wo * sizeof(float)});     // [N*Do, K, Ho, Wo]
      }
      return s;
   }

   std::string GenerateSessionMembersCode_GPU_B200(std::string opName) override
   {
      opName = "op_" + opName;
      return "   sofie_b200_conv_plan *plan_" + opName + " = nullptr;\n   sofie_b200_epilogue ep_" + opName + "{};\n";
   }
   std::string GenerateInitCode_GPU_B200(std::string opName) override
   {
      opName = "op_" + opName;
      std::stringstream out;
      out << "      {  // Conv " << opName << ": " << ConvertShapeToString(fShapeX) << " * " << ConvertShapeToString(fShapeW) << "\n";
      out << ConvDescCode(fGeo, "SOFIE_B200_F32", "SOFIE_B200_F32", 0, fXLayout, fYLayout);
      out << "      Check(sofie_b200_conv_plan_create(ctx, &d, tensor_" << fNW << ", &plan_" << opName << "), \"Conv " << opName << ": plan\");\n";
      out << "      if (sofie_b200_conv_workspace_bytes(plan_" << opName << ") > " << Workspace() << "LL)\n"
          << "         throw std::runtime_error(\"Conv " << opName << ": the library wants more scratch than the arena reserves\");\n";
      out << fEpi.InitCode("ep_" + opName);
      out << "      }\n";
      return out.str();
   }
   std::string Generate_GPU_B200(std::string opName) override
   {
      opName = "op_" + opName;
      if (fShapeX.empty() || fShapeW.empty() || fShapeY.empty())
         throw std::runtime_error("SOFIE Conv Op called to Generate without being initialized first");
      std::stringstream out;
      out << "\n      //--------- Conv " << opName << " " << ConvertShapeToString(fShapeX) << " -> " << ConvertShapeToString(fShapeY) << "\n";
      if (!fEpi.residual.empty())
         out << "      ep_" << opName << ".residual = tensor_" << fEpi.residual << "; ep_" << opName << ".residual_dtype = "
             << ConvertTypeToRuntimeEnum(fResidualType) << ";\n";
      out << fEpi.BindCode("ep_" + opName);
      const std::string ws = Workspace() ? "tensor_" + fNY + "_xcol" : std::string("nullptr");
      if (fGeo.Is3D()) {
         out << "      Check(sofie_b200_depth_unfold_enqueue(ctx, tensor_" << fNX << ", tensor_" << fNY << "_slices, SOFIE_B200_F32, " << fGeo.N3 << ", " << fGeo.C3
             << ", " << fGeo.D << ", " << fGeo.H * fGeo.W << ", " << fGeo.T << ", " << fGeo.Do << ", " << fGeo.strideD << ", " << fGeo.padFront << ", " << fGeo.dilD
             << "), \"Conv " << opName << ": depth taps\");\n";
         out << "      Check(sofie_b200_conv_enqueue(plan_" << opName << ", tensor_" << fNY << "_slices, tensor_" << fNY << "_planes, " << ws << ", &ep_" << opName
             << "), \"Conv " << opName << "\");\n";
         out << "      {\n         const int64_t shape[4] = {" << fGeo.N3 << ", " << fGeo.Do << ", " << fGeo.K << ", " << fGeo.Ho * fGeo.Wo << "};\n"
             << "         const int32_t perm[4] = {0, 2, 1, 3};\n"
             << "         Check(sofie_b200_transpose_enqueue(ctx, tensor_" << fNY << "_planes, tensor_" << fNY << ", SOFIE_B200_F32, 4, shape, perm), \"Conv " << opName
             << ": depth to its place\");\n      }\n";
         return out.str();
      }
      out << "      Check(sofie_b200_conv_enqueue(plan_" << opName << ", tensor_" << fNX << ", tensor_" << fNY << ", " << ws << ", &ep_" << opName << "), \"Conv "
          << opName << "\");\n";
      return out.str();
   }
   std::string GenerateDestroyCode_GPU_B200(std::string opName) override { return "      sofie_b200_conv_plan_destroy(plan_op_" + opName + ");\n"; }
};

}  // namespace SOFIE_B200
