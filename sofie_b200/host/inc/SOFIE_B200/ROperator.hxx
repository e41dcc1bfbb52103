// Operator plug-in interface of the B200 code generator.
//
// ROperator keeps the reference's contract (core/inc/SOFIE/operators/ROperator.hxx:111-134):
// Initialize(RModel&) does shape inference and registers the outputs, Generate(opName) returns the
// text the Session's inference body gets for this operator.  The reference's second interface,
// ROperator_ALPAKA (core/inc/SOFIE/operators/ROperator_ALPAKA.hxx:20-135), emits alpaka kernels and
// sofieBLAS calls; its sibling here, ROperator_B200, emits calls into libsofie_b200 instead:
//
//   Generate_GPU_ALPAKA(opName)            ->  Generate_GPU_B200(opName)             enqueue call(s)
//   GenerateInitCode_GPU_ALPAKA()          ->  GenerateInitCode_GPU_B200(opName)     plan creation at Session init
//   GetBlasConfigs()                       ->  (part of GenerateInitCode_GPU_B200: one plan per contraction)
//   GetDeviceScratch_GPU_ALPAKA()          ->  GetDeviceScratch_GPU_B200()           scratch regions in the arena
//   GenerateSessionMembersCode(opName)     ->  GenerateSessionMembersCode_GPU_B200(opName)
//   fusion hooks (SetActivation, UpdateFusableTensorName) -> FuseActivation / FuseScaleShift / FuseResidual
//
// An operator that cannot run through the library throws std::runtime_error at generation, the
// reference's convention ("has no alpaka implementation", core/src/RModel_ALPAKA.cxx:957-965).
#pragma once
#include <string>
#include <string_view>
#include <vector>

#include "SOFIE_B200/SOFIE_common.hxx"

namespace SOFIE_B200 {

class RModel;

class ROperator {
public:
   virtual ~ROperator() = default;
   virtual void Initialize(RModel &) = 0;
   // CPU emission is the reference generator's job; this generator has no CPU path by design.
   virtual std::string Generate(std::string opName)
   {
      throw std::runtime_error("SOFIE_B200 operator " + opName + ": CPU code emission is not part of this generator (no CPU fallback)");
   }
   virtual std::string GenerateInitCode() { return ""; }
   virtual std::string GenerateDeclCode() { return ""; }
   virtual std::string GenerateSessionMembersCode(std::string /*opName*/) { return ""; }

   const std::vector<std::string> &GetOpInputTensors() const { return fInputTensorNames; }
   const std::vector<std::string> &GetOpOutputTensors() const { return fOutputTensorNames; }
   std::string fName = "UnnamedOperator";
   const std::string &Name() const { return fName; }

protected:
   std::vector<std::string> fInputTensorNames;
   std::vector<std::string> fOutputTensorNames;
};

class ROperator_B200 : public ROperator {
public:
   struct DeviceScratch {
      std::string name;   // becomes the Session member tensor_<name> (char*)
      size_t bytes;
   };
   // text for the Session's _infer_impl: records work on the stream, never synchronises
   virtual std::string Generate_GPU_B200(std::string opName) = 0;
   // text for the Session constructor, after weights are on the device and the arena is placed
   virtual std::string GenerateInitCode_GPU_B200(std::string /*opName*/) { return ""; }
   // text for the Session destructor
   virtual std::string GenerateDestroyCode_GPU_B200(std::string /*opName*/) { return ""; }
   virtual std::string GenerateSessionMembersCode_GPU_B200(std::string /*opName*/) { return ""; }
   virtual std::vector<DeviceScratch> GetDeviceScratch_GPU_B200() const { return {}; }

   // ---- epilogue fusion (decided by RModel's fusion pass) -----------------------------------
   // true if a following elementwise operator can be folded into this operator's epilogue
   virtual bool HasFusableEpilogue() const { return false; }
   virtual EActivationType GetActivationType() const { return EActivationType::UNDEFINED; }
   // fold act(output) and rename the output (reference: SetActivation + UpdateFusableTensorName,
   // core/inc/SOFIE/operators/ROperator_Gemm.hxx:1155-1163)
   virtual bool FuseActivation(EActivationType, float /*alpha*/, const std::string & /*newOutput*/) { return false; }
   // fold y*scale[c] + shift[c] per output channel (an inference BatchNormalization that follows)
   virtual bool FuseScaleShift(RModel &, const std::string & /*scaleTensor*/, const std::string & /*shiftTensor*/,
                               const std::string & /*newOutput*/) { return false; }
   // fold y + residual (a following Add with a tensor of the output's shape)
   virtual bool FuseResidual(RModel &, const std::string & /*residualTensor*/, const std::string & /*newOutput*/) { return false; }
   // a zero-copy alias (Reshape / Flatten): output shares the input's storage
   virtual bool IsAlias() const { return false; }
   // true if every number the operator emits is linear in a symbolic leading dimension and none of its generation-time
   // decisions looks at it (see kSymbolicBase)
   virtual bool SupportsSymbolicDim() const { return false; }
};

// emitted-code spelling of a sofie_b200_act
inline std::string ActivationEnum(EActivationType a)
{
   switch (a) {
   case EActivationType::RELU: return "SOFIE_B200_ACT_RELU";
   case EActivationType::LEAKYRELU: return "SOFIE_B200_ACT_LEAKY_RELU";
   case EActivationType::SIGMOID: return "SOFIE_B200_ACT_SIGMOID";
   case EActivationType::GELU: return "SOFIE_B200_ACT_GELU_ERF";
   case EActivationType::GELU_TANH: return "SOFIE_B200_ACT_GELU_TANH";
   default: return "SOFIE_B200_ACT_NONE";
   }
}

}  // namespace SOFIE_B200
