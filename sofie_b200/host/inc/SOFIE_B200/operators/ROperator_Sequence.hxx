// Sequence operators of the B200 target: ScaledDotProductAttention and Transpose.
//
// ROperator_SDPA keeps the reference operator's constructor and shape rules
// (core/inc/SOFIE/operators/ROperator_SDPA.hxx:38-57, 81-139): rank-4 Q, K, V are [B, H, S, D], rank-3 ones are the folded
// form [B, S, H*D] and need num_heads; the optional mask is additive, [B, H, S, S]; scale 0 means 1/sqrt(D).  Instead of
// the reference's kernel text (:203-330) it emits one sofie_b200_sdpa plan, which the library runs as the fused
// tcgen05 attention kernel (bf16, folded, heads of 64, sequences up to 128) or as the batched contraction / Softmax /
// contraction chain.  ROperator_Transpose (ROperator_Transpose.hxx:32-36) emits sofie_b200_transpose_enqueue.
#pragma once
#include <sstream>

#include "SOFIE_B200/RModel.hxx"
#include "SOFIE_B200/ROperator.hxx"

namespace SOFIE_B200 {

template <typename T>
class ROperator_SDPA final : public ROperator_B200 {
   std::string fNQ, fNK, fNV, fNMask, fNY;
   float fScale;
   size_t fNumHeads;
   bool fFolded = false, fHasMask = false;
   size_t fB = 0, fH = 0, fS = 0, fD = 0, fDv = 0;
   size_t fLdq = 0, fLdk = 0, fLdv = 0;   // folded: row pitches when Q, K, V are column blocks of a wider tensor (set by the fusion pass)
   std::string fQBase, fKBase, fVBase;    // tensors the pointers are taken from (with a column offset) when they are column blocks
   size_t fQOff = 0, fKOff = 0, fVOff = 0;
   ETensorType fType = ETensorType::FLOAT;
   std::vector<size_t> fShapeY;

public:
   ROperator_SDPA(const std::string &nameQ, const std::string &nameK, const std::string &nameV, const std::string &nameY,
                  const std::string &nameMask = "", float scale = 0.0f, size_t numHeads = 0)
      : fNQ(UTILITY::Clean_name(nameQ)), fNK(UTILITY::Clean_name(nameK)), fNV(UTILITY::Clean_name(nameV)), fNMask(UTILITY::Clean_name(nameMask)),
        fNY(UTILITY::Clean_name(nameY)), fScale(scale), fNumHeads(numHeads)
   {
      fInputTensorNames = {fNQ, fNK, fNV};
      if (!fNMask.empty()) fInputTensorNames.push_back(fNMask);
      fOutputTensorNames = {fNY};
   }

   void Initialize(RModel &model) override
   {
      if (!model.CheckIfTensorAlreadyExist(fNQ)) throw std::runtime_error("SOFIE SDPA: query tensor " + fNQ + " not found");
      if (!model.CheckIfTensorAlreadyExist(fNK)) throw std::runtime_error("SOFIE SDPA: key tensor " + fNK + " not found");
      if (!model.CheckIfTensorAlreadyExist(fNV)) throw std::runtime_error("SOFIE SDPA: value tensor " + fNV + " not found");
      const auto q = model.GetTensorShape(fNQ), k = model.GetTensorShape(fNK), v = model.GetTensorShape(fNV);
      fType = model.GetTensorType(fNQ);
      if (fType != ETensorType::FLOAT && fType != ETensorType::BFLOAT16) throw std::runtime_error("SOFIE SDPA: FLOAT or BFLOAT16 tensors expected");
      if (model.GetTensorType(fNK) != fType || model.GetTensorType(fNV) != fType) throw std::runtime_error("SOFIE SDPA: Q, K and V must have one type");
      if (q.size() == 4) {
         fFolded = false;
         fB = q[0]; fH = q[1]; fS = q[2]; fD = q[3]; fDv = v.at(3);
         fShapeY = {q[0], q[1], q[2], v[3]};
      } else if (q.size() == 3) {
         if (fNumHeads == 0)
            throw std::runtime_error("SOFIE SDPA: rank-3 [B, S, H*D] query requires num_heads to be specified (it cannot be inferred from the tensor shape)");
         fFolded = true;
         fB = q[0]; fS = q[1]; fH = fNumHeads; fD = q[2] / fNumHeads; fDv = v.at(2) / fNumHeads;
         fShapeY = {q[0], q[1], v[2]};
      } else {
         throw std::runtime_error("SOFIE SDPA: query must be rank-4 [B, H, S, D] or rank-3 [B, S, H*D] with num_heads specified");
      }
      if (k != q || v.size() != q.size()) throw std::runtime_error("SOFIE SDPA: K must have the shape of Q and V its rank");
      fHasMask = !fNMask.empty() && model.CheckIfTensorAlreadyExist(fNMask);
      if (fHasMask) {
         if (model.GetTensorType(fNMask) != ETensorType::FLOAT || fType != ETensorType::FLOAT)
            throw std::runtime_error("SOFIE SDPA: the additive mask is supported for FLOAT tensors");
         if (model.GetTensorShape(fNMask) != std::vector<size_t>{fB, fH, fS, fS}) throw std::runtime_error("SOFIE SDPA: mask must be [B, H, S, S]");
      }
      model.AddIntermediateTensor(fNY, fType, fShapeY);
   }

   // Q, K, V as column blocks [off, off + H*D) of rows of `ld` elements of tensor `base` (a Split of a packed projection)
   bool IsFolded() const { return fFolded; }
   void ReadFromColumnBlock(int which, const std::string &base, size_t off, size_t ld)
   {
      std::string &b = which == 0 ? fQBase : which == 1 ? fKBase : fVBase;
      (which == 0 ? fQOff : which == 1 ? fKOff : fVOff) = off;
      (which == 0 ? fLdq : which == 1 ? fLdk : fLdv) = ld;
      b = base;
      fInputTensorNames[which] = base;
   }

   size_t ElemSize() const { return fType == ETensorType::FLOAT ? 4 : 2; }
   bool Fused() const
   {
      const size_t es = ElemSize();
      auto ok = [&](size_t ld) { return (ld * es) % 16 == 0; };
      return fType == ETensorType::BFLOAT16 && fFolded && !fHasMask && fD == 64 && fDv == 64 && fS <= 128 && ok(fLdq ? fLdq : fH * fD) &&
             ok(fLdk ? fLdk : fH * fD) && ok(fLdv ? fLdv : fH * fDv);
   }
   size_t WorkspaceBytes() const
   {
      if (Fused() || fB * fS == 0) return 0;
      const size_t es = ElemSize(), bh = fB * fH;
      auto region = [&](size_t elems) { return (elems * es + 255) / 256 * 256; };
      size_t bytes = region(bh * fS * fS);
      if (fFolded) bytes += 2 * region(bh * fS * fD) + 2 * region(bh * fS * fDv);
      return bytes;
   }
   std::vector<DeviceScratch> GetDeviceScratch_GPU_B200() const override
   {
      const size_t b = WorkspaceBytes();
      return b ? std::vector<DeviceScratch>{{fNY + "_sdpa", b}} : std::vector<DeviceScratch>{};
   }
   std::string GenerateSessionMembersCode_GPU_B200(std::string opName) override { return "   sofie_b200_sdpa_plan *plan_op_" + opName + " = nullptr;\n"; }
   std::string GenerateInitCode_GPU_B200(std::string opName) override
   {
      opName = "op_" + opName;
      std::stringstream out;
      out << "      {  // SDPA " << opName << ": batch " << fB << ", heads " << fH << ", seq " << fS << ", head sizes " << fD << " / " << fDv
          << (fFolded ? ", folded" : "") << "\n";
      out << "      sofie_b200_sdpa_desc d{};\n";
      out << "      d.batch = " << fB << "; d.heads = " << fH << "; d.seq = " << fS << "; d.head_dim = " << fD << "; d.v_head_dim = " << fDv << ";\n";
      out << "      d.dtype = " << ConvertTypeToRuntimeEnum(fType) << "; d.folded = " << (fFolded ? 1 : 0) << "; d.has_mask = " << (fHasMask ? 1 : 0)
          << "; d.scale = float(" << std::setprecision(9) << fScale << ");\n";
      out << "      d.ldq = " << fLdq << "; d.ldk = " << fLdk << "; d.ldv = " << fLdv << ";\n";
      out << "      Check(sofie_b200_sdpa_plan_create(ctx, &d, &plan_" << opName << "), \"SDPA " << opName << ": plan\");\n";
      out << "      if (sofie_b200_sdpa_workspace_bytes(plan_" << opName << ") > " << WorkspaceBytes() << "LL)\n"
          << "         throw std::runtime_error(\"SDPA " << opName << ": the library wants more scratch than the arena reserves\");\n";
      out << "      }\n";
      return out.str();
   }
   std::string Generate_GPU_B200(std::string opName) override
   {
      opName = "op_" + opName;
      auto ptr = [&](const std::string &own, const std::string &base, size_t off) {
         return base.empty() ? "tensor_" + own : "(tensor_" + base + " + " + std::to_string(off) + ")";
      };
      std::stringstream out;
      out << "\n      //------ SDPA " << opName << "\n";
      out << "      Check(sofie_b200_sdpa_enqueue(plan_" << opName << ", " << ptr(fNQ, fQBase, fQOff) << ", " << ptr(fNK, fKBase, fKOff) << ", "
          << ptr(fNV, fVBase, fVOff) << ", " << (fHasMask ? "tensor_" + fNMask : std::string("nullptr")) << ", tensor_" << fNY << ", "
          << (WorkspaceBytes() ? "tensor_" + fNY + "_sdpa" : std::string("nullptr")) << "), \"SDPA " << opName << "\");\n";
      return out.str();
   }
   std::string GenerateDestroyCode_GPU_B200(std::string opName) override { return "      sofie_b200_sdpa_plan_destroy(plan_op_" + opName + ");\n"; }
};

// Split along one axis (the reference's ROperator_Split, core/inc/SOFIE/operators/ROperator_Split.hxx): the input viewed as
// [outer, along * inner] and each output as a block of columns of it, copied with one strided device-to-device copy.  When
// the outputs only feed a folded SDPA the fusion pass lets the attention kernel read the blocks in place and drops the copies.
class ROperator_Split final : public ROperator_B200 {
   int64_t fAxis;
   std::string fNX, fNSplit;
   std::vector<std::string> fNYs;
   std::vector<size_t> fShapeX, fLens, fStarts;
   size_t fOuter = 1, fInner = 1;
   ETensorType fType = ETensorType::FLOAT;

public:
   ROperator_Split(int64_t axis, std::string nameX, std::string nameSplit, const std::vector<std::string> &namesY)
      : fAxis(axis), fNX(UTILITY::Clean_name(nameX)), fNSplit(UTILITY::Clean_name(nameSplit))
   {
      for (auto &n : namesY) fNYs.push_back(UTILITY::Clean_name(n));
      fInputTensorNames = {fNX};
      fOutputTensorNames = fNYs;
   }
   void Initialize(RModel &model) override
   {
      if (!model.CheckIfTensorAlreadyExist(fNX)) throw std::runtime_error("SOFIE Split Op Input Tensor is not found in model");
      fShapeX = model.GetTensorShape(fNX);
      fType = model.GetTensorType(fNX);
      const int64_t rank = int64_t(fShapeX.size());
      const int64_t axis = fAxis < 0 ? fAxis + rank : fAxis;
      if (axis < 0 || axis >= rank) throw std::runtime_error("SOFIE Split Op: axis out of range");
      fAxis = axis;
      const size_t along = fShapeX[size_t(axis)], parts = fNYs.size();
      if (!fNSplit.empty()) {
         if (!model.IsInitializedTensor(fNSplit)) throw std::runtime_error("SOFIE Split Op: the split sizes must be an initialized INT64 tensor");
         for (auto v : model.GetTensorData<int64_t>(fNSplit)) fLens.push_back(size_t(v));
         if (fLens.size() != parts) throw std::runtime_error("SOFIE Split Op: one split size per output expected");
      } else {
         if (parts == 0 || along % parts) throw std::runtime_error("SOFIE Split Op: the axis does not divide evenly among the outputs");
         fLens.assign(parts, along / parts);
      }
      size_t start = 0;
      for (size_t k = 0; k < parts; ++k) { fStarts.push_back(start); start += fLens[k]; }
      if (start != along) throw std::runtime_error("SOFIE Split Op: the split sizes do not add up to the axis length");
      fOuter = fInner = 1;
      for (int64_t i = 0; i < axis; ++i) fOuter *= fShapeX[size_t(i)];
      for (int64_t i = axis + 1; i < rank; ++i) fInner *= fShapeX[size_t(i)];
      for (size_t k = 0; k < parts; ++k) {
         auto shp = fShapeX;
         shp[size_t(axis)] = fLens[k];
         model.AddIntermediateTensor(fNYs[k], fType, shp);
      }
   }
   // for the fusion pass: output k as a block of columns of the input seen as a matrix of `RowPitch` columns
   const std::string &Input() const { return fNX; }
   int OutputIndex(const std::string &name) const
   {
      for (size_t k = 0; k < fNYs.size(); ++k) if (fNYs[k] == name) return int(k);
      return -1;
   }
   bool SplitsLastAxis() const { return fInner == 1; }
   size_t RowPitch() const { return fShapeX.empty() ? 0 : fShapeX.back(); }
   size_t ColumnStart(int k) const { return fStarts[size_t(k)]; }
   std::string Generate_GPU_B200(std::string opName) override
   {
      opName = "op_" + opName;
      const size_t es = GetTypeSize(fType), pitch = fShapeX[size_t(fAxis)] * fInner * es;
      std::stringstream out;
      out << "\n      //------ Split " << opName << " " << ConvertShapeToString(fShapeX) << " along axis " << fAxis << "\n";
      for (size_t k = 0; k < fNYs.size(); ++k) {
         const size_t width = fLens[k] * fInner * es;
         if (width == 0 || fOuter == 0) continue;
         out << "      CheckCuda(cudaMemcpy2DAsync(tensor_" << fNYs[k] << ", " << width << ", reinterpret_cast<const char *>(tensor_" << fNX << ") + "
             << fStarts[k] * fInner * es << ", " << pitch << ", " << width << ", " << fOuter << ", cudaMemcpyDeviceToDevice, stream), \"Split " << opName << "\");\n";
      }
      return out.str();
   }
};

class ROperator_Transpose final : public ROperator_B200 {
   std::vector<int64_t> fAttrPerm;
   std::string fNData, fNOutput;
   std::vector<size_t> fShapeData, fShapeOutput;
   ETensorType fType = ETensorType::FLOAT;

public:
   ROperator_Transpose(std::vector<int64_t> attr_perm, std::string nameData, std::string nameOutput)
      : fAttrPerm(std::move(attr_perm)), fNData(UTILITY::Clean_name(nameData)), fNOutput(UTILITY::Clean_name(nameOutput))
   {
      fInputTensorNames = {fNData};
      fOutputTensorNames = {fNOutput};
   }
   void Initialize(RModel &model) override
   {
      if (!model.CheckIfTensorAlreadyExist(fNData)) throw std::runtime_error("SOFIE Tranpose Op Input Tensor is not found in model");
      fShapeData = model.GetTensorShape(fNData);
      fType = model.GetTensorType(fNData);
      const size_t rank = fShapeData.size();
      if (fAttrPerm.empty()) {   // default: reverse the axes (ROperator_Transpose.hxx:68-72)
         fAttrPerm.resize(rank);
         for (size_t i = 0; i < rank; ++i) fAttrPerm[i] = int64_t(rank - 1 - i);
      }
      if (fAttrPerm.size() != rank) throw std::runtime_error("SOFIE Tranpose Op - Invalid axes attributes");
      if (rank < 1 || rank > 4) throw std::runtime_error("SOFIE Transpose Op: ranks 1 to 4 are on the B200 path, got " + std::to_string(rank));
      fShapeOutput.resize(rank);
      for (size_t i = 0; i < rank; ++i) {
         if (fAttrPerm[i] < 0 || size_t(fAttrPerm[i]) >= rank) throw std::runtime_error("SOFIE Tranpose Op - Invalid axes attributes");
         fShapeOutput[i] = fShapeData[size_t(fAttrPerm[i])];
      }
      model.AddIntermediateTensor(fNOutput, fType, fShapeOutput);
   }
   std::string Generate_GPU_B200(std::string opName) override
   {
      opName = "op_" + opName;
      std::stringstream out;
      out << "\n      //------ Transpose " << opName << " " << ConvertShapeToString(fShapeData) << " -> " << ConvertShapeToString(fShapeOutput) << "\n";
      out << "      { const int64_t shape[] = {";
      for (size_t i = 0; i < fShapeData.size(); ++i) out << (i ? ", " : "") << fShapeData[i];
      out << "}; const int32_t perm[] = {";
      for (size_t i = 0; i < fAttrPerm.size(); ++i) out << (i ? ", " : "") << fAttrPerm[i];
      out << "};\n        Check(sofie_b200_transpose_enqueue(ctx, tensor_" << fNData << ", tensor_" << fNOutput << ", " << ConvertTypeToRuntimeEnum(fType) << ", "
          << fShapeData.size() << ", shape, perm), \"Transpose " << opName << "\"); }\n";
      return out.str();
   }
};

}  // namespace SOFIE_B200
