// RModel: model IR, operator initialisation, epilogue fusion, arena planning and emission of the
// Session header for the B200 target (see SOFIE_B200/RModel.hxx).
#include "SOFIE_B200/RModel.hxx"

#include <fstream>
#include <iomanip>
#include <iostream>
#include <limits>
#include <sstream>

#include "SOFIE_B200/operators/OperatorList.hxx"

namespace SOFIE_B200 {

RModel::RModel(std::string name, std::string parsedtime) : fName(std::move(name)), fParseTime(std::move(parsedtime))
{
   // a file name may be given: keep the stem, as the reference does for "model.onnx"
   auto slash = fName.find_last_of("/\\");
   if (slash != std::string::npos) fName = fName.substr(slash + 1);
   auto dot = fName.find_last_of('.');
   if (dot != std::string::npos) fName = fName.substr(0, dot);
   fName = UTILITY::Clean_name(fName);
}

// ---------------------------------------------------------------------------------------------------
// model building
// ---------------------------------------------------------------------------------------------------
void RModel::AddInputTensorInfo(std::string input_name, ETensorType type, std::vector<Dim> shape)
{
   input_name = UTILITY::Clean_name(input_name);
   if (CheckIfTensorAlreadyExist(input_name))
      throw std::runtime_error("SOFIE: input tensor with name " + input_name + " already exists \n");
   fInputDimShapes[input_name] = shape;
   std::vector<size_t> s;
   for (auto &d : shape) s.push_back(d.dim);
   fInputTensorInfos[input_name] = TensorInfo{type, s};
}

void RModel::AddInputTensorInfo(std::string input_name, ETensorType type, std::vector<size_t> shape)
{
   std::vector<Dim> d(shape.begin(), shape.end());
   AddInputTensorInfo(std::move(input_name), type, std::move(d));
}

void RModel::AddInputTensorName(std::string name) { fInputTensorNames.emplace_back(UTILITY::Clean_name(name)); }

void RModel::AddInitializedTensor(std::string tensor_name, ETensorType type, std::vector<std::size_t> shape, std::shared_ptr<void> data)
{
   tensor_name = UTILITY::Clean_name(tensor_name);
   if (CheckIfTensorAlreadyExist(tensor_name))
      throw std::runtime_error("SOFIE: initialized tensor with name " + tensor_name + " already exists \n");
   fInitializedTensors[tensor_name] = InitializedTensor{type, std::move(shape), std::move(data), false};
   fInitializedOrder.push_back(tensor_name);
}

void RModel::AddInitializedTensor(const std::string &tensor_name, ETensorType type, const std::vector<std::size_t> &shape, void *raw_data)
{
   const size_t bytes = ConvertShapeToLength(shape) * GetTypeSize(type);
   std::shared_ptr<void> p(malloc(bytes + 1), free);
   std::memcpy(p.get(), raw_data, bytes);
   AddInitializedTensor(tensor_name, type, shape, p);
}

void RModel::AddConstantTensor(std::string tensor_name, ETensorType type, std::vector<std::size_t> shape, std::shared_ptr<void> data)
{
   AddInitializedTensor(tensor_name, type, std::move(shape), std::move(data));
   fInitializedTensors[UTILITY::Clean_name(tensor_name)].constant = true;
}

void RModel::AddIntermediateTensor(std::string tensor_name, ETensorType type, std::vector<std::size_t> shape)
{
   tensor_name = UTILITY::Clean_name(tensor_name);
   if (CheckIfTensorAlreadyExist(tensor_name))
      throw std::runtime_error("SOFIE: intermediate tensor with name " + tensor_name + " already exists \n");
   fIntermediateTensorInfos[tensor_name] = TensorInfo{type, std::move(shape)};
}

bool RModel::AddAliasTensor(const std::string &tensor_name, const std::string &orig_tensor_name)
{
   const std::string a = UTILITY::Clean_name(tensor_name), o = UTILITY::Clean_name(orig_tensor_name);
   if (!CheckIfTensorAlreadyExist(o)) return false;
   fAliasTensors[a] = ResolveAliasTensor(o);
   return true;
}

std::string RModel::ResolveAliasTensor(const std::string &name) const
{
   std::string n = name;
   for (auto it = fAliasTensors.find(n); it != fAliasTensors.end(); it = fAliasTensors.find(n)) n = it->second;
   return n;
}

void RModel::AddOperator(std::unique_ptr<ROperator> op, int order_execution)
{
   if (order_execution >= 0 && size_t(order_execution) <= fOperators.size()) fOperators.insert(fOperators.begin() + order_execution, std::move(op));
   else fOperators.push_back(std::move(op));
}

void RModel::AddOutputTensorNameList(std::vector<std::string> names)
{
   fOutputTensorNames.clear();
   for (auto &n : names) fOutputTensorNames.emplace_back(UTILITY::Clean_name(n));
}

void RModel::UpdateOutputTensorList(std::vector<std::string> curr, std::vector<std::string> mod)
{
   for (size_t i = 0; i < curr.size(); ++i)
      for (auto &o : fOutputTensorNames)
         if (o == UTILITY::Clean_name(curr[i])) o = UTILITY::Clean_name(mod[i]);
}

// ---------------------------------------------------------------------------------------------------
// queries
// ---------------------------------------------------------------------------------------------------
bool RModel::CheckIfTensorAlreadyExist(std::string n) const
{
   n = UTILITY::Clean_name(n);
   return fInputTensorInfos.count(n) || fInitializedTensors.count(n) || fIntermediateTensorInfos.count(n);
}
bool RModel::IsInitializedTensor(const std::string &name) const { return fInitializedTensors.count(UTILITY::Clean_name(name)) != 0; }
bool RModel::IsConstantTensor(const std::string &name) const
{
   auto it = fInitializedTensors.find(UTILITY::Clean_name(name));
   return it != fInitializedTensors.end() && it->second.constant;
}
bool RModel::IsInputTensor(const std::string &name) const { return fInputTensorInfos.count(UTILITY::Clean_name(name)) != 0; }
bool RModel::IsOutputTensor(const std::string &name) const
{
   const std::string n = UTILITY::Clean_name(name);
   return std::find(fOutputTensorNames.begin(), fOutputTensorNames.end(), n) != fOutputTensorNames.end();
}

const std::vector<size_t> &RModel::GetTensorShape(const std::string &name) const
{
   const std::string n = UTILITY::Clean_name(name);
   if (auto it = fInitializedTensors.find(n); it != fInitializedTensors.end()) return it->second.shape;
   if (auto it = fInputTensorInfos.find(n); it != fInputTensorInfos.end()) return it->second.shape;
   if (auto it = fIntermediateTensorInfos.find(n); it != fIntermediateTensorInfos.end()) return it->second.shape;
   throw std::runtime_error("SOFIE tensor [" + n + "] for which the shape is requested is not found");
}

ETensorType RModel::GetTensorType(const std::string &name) const
{
   const std::string n = UTILITY::Clean_name(name);
   if (auto it = fInitializedTensors.find(n); it != fInitializedTensors.end()) return it->second.type;
   if (auto it = fInputTensorInfos.find(n); it != fInputTensorInfos.end()) return it->second.type;
   if (auto it = fIntermediateTensorInfos.find(n); it != fIntermediateTensorInfos.end()) return it->second.type;
   throw std::runtime_error("SOFIE tensor [" + n + "] for which the type is requested is not found");
}

std::shared_ptr<void> RModel::GetInitializedTensorData(const std::string &name) const
{
   auto it = fInitializedTensors.find(UTILITY::Clean_name(name));
   if (it == fInitializedTensors.end()) throw std::runtime_error("SOFIE tensor [" + name + "] for which the data is requested is not found");
   return it->second.data;
}

// ---------------------------------------------------------------------------------------------------
// initialisation: shapes, then epilogue fusion
// ---------------------------------------------------------------------------------------------------
void RModel::Initialize(int batchSize, bool verbose)
{
   if (fIsInitialized) return;
   fBatchSize = batchSize;
   for (auto &[name, dims] : fInputDimShapes) {
      std::vector<size_t> s;
      for (auto &d : dims) {
         if (!d.isParam) { s.push_back(d.dim); continue; }
         // input_size, batch_size, bs take the batch size (core/src/RModel.cxx:676-685)
         if ((d.param == "input_size" || d.param == "batch_size" || d.param == "bs") && batchSize > 0) s.push_back(size_t(batchSize));
         else if (d.dim > 0) s.push_back(d.dim);
         else {
            // a dynamic dimension: the Session constructor takes its value (tests/alpaka/TestAlpakaLinear.cxx:121-203).
            // One symbol per model, and only as the leading dimension of an input.
            if (!fSymbol.empty() && fSymbol != d.param)
               throw std::runtime_error("SOFIE_B200: input " + name + " has the symbolic dimension " + d.param + " beside " + fSymbol +
                                        "; the B200 target carries one symbolic dimension per model");
            if (&d != &dims.front())
               throw std::runtime_error("SOFIE_B200: input " + name + " has the symbolic dimension " + d.param +
                                        " in an inner position; only a leading (batch) dimension may be symbolic");
            fSymbol = d.param;
            s.push_back(kSymbolicBase);
         }
      }
      fInputTensorInfos[name].shape = s;
   }
   for (auto &n : fInputTensorNames)
      if (!fInputTensorInfos.count(n)) throw std::runtime_error("SOFIE: input tensor " + n + " has no type and shape information");
   size_t i = 0;
   for (auto &op : fOperators) {
      if (verbose) std::cout << "[SOFIE_B200 generator] initializing operator " << i << " " << typeid(*op).name() << std::endl;
      op->Initialize(*this);
      ++i;
   }
   for (auto &o : fOutputTensorNames)
      if (!CheckIfTensorAlreadyExist(o)) throw std::runtime_error("SOFIE: output tensor " + o + " is not produced by any operator");
   fIsInitialized = true;
}

namespace {
ROperator_B200 *AsB200(ROperator *op) { return dynamic_cast<ROperator_B200 *>(op); }
}  // namespace

bool RModel::CheckGPUOperators() const
{
   for (auto &op : fOperators)
      if (!dynamic_cast<ROperator_B200 *>(op.get())) return false;
   return true;
}

// Which epilogues fold into which contraction.  Legality is the reference's: the producer's output
// has exactly one consumer and is not a graph output (core/src/RModel_Fusion_ALPAKA.cxx:376-415).
// The reference folds only Relu / LeakyRelu into Gemm (and needs a bias for Relu, a limit of its BLAS
// epilogues); here any activation, a following inference BatchNormalization (as column scale + shift)
// and a residual Add fold into Gemm / Conv / the quantised contractions, in that order of appearance.
void RModel::FuseOperators()
{
   auto consumers = [&](const std::string &t) {
      size_t n = 0;
      for (size_t k = 0; k < fOperators.size(); ++k) {
         if (fSkippedOperators.count(k)) continue;
         for (auto &in : fOperators[k]->GetOpInputTensors())
            if (in == t) ++n;
      }
      return n;
   };
   for (size_t i = 0; i < fOperators.size(); ++i) {
      if (fSkippedOperators.count(i)) continue;
      auto *prod = AsB200(fOperators[i].get());
      if (!prod || !prod->HasFusableEpilogue()) continue;
      for (size_t j = i + 1; j < fOperators.size(); ++j) {
         if (fSkippedOperators.count(j)) continue;
         if (prod->GetOpOutputTensors().size() != 1) break;
         const std::string out = prod->GetOpOutputTensors()[0];
         if (consumers(out) != 1 || IsOutputTensor(out)) break;
         ROperator *next = fOperators[j].get();
         const auto &nin = next->GetOpInputTensors();
         if (std::find(nin.begin(), nin.end(), out) == nin.end()) break;  // only the operator that follows directly
         bool fused = false;
         std::string what;
         if (auto *u = dynamic_cast<ROperator_Unary *>(next)) {
            fused = prod->FuseActivation(u->Activation(), u->GetAlpha(), u->GetOpOutputTensors()[0]);
            what = "activation";
         } else if (auto *bn = dynamic_cast<ROperator_BatchNormalization<float> *>(next)) {
            const bool isContraction = !dynamic_cast<ROperator_BatchNormalization<float> *>(fOperators[i].get());
            if (isContraction && bn->NameX() == out) {
               std::string s, t;
               bn->MakeScaleShift(*this, s, t);
               fused = prod->FuseScaleShift(*this, s, t, bn->NameY());
               if (fused && bn->GetActivationType() == EActivationType::RELU) prod->FuseActivation(EActivationType::RELU, 0.f, bn->NameY());
               what = "BatchNormalization as column scale + shift";
            }
         } else if (auto *add = dynamic_cast<ROperator_BasicBinary<float, EBasicBinaryOperator::Add> *>(next)) {
            const std::string other = add->NameA() == out ? add->NameB() : add->NameA();
            if (other != out) {
               fused = prod->FuseResidual(*this, other, add->GetOpOutputTensors()[0]);
               what = "residual Add";
            }
         }
         if (!fused) break;
         fIntermediateTensorInfos.erase(out);
         fSkippedOperators.insert(j);
         fFusionLog.push_back("op_" + std::to_string(i) + " <- op_" + std::to_string(j) + " (" + what + ")");
      }
   }
}

// A folded SDPA whose Q, K or V is (a reshaped view of) an output of a Split along the last axis reads that block of
// columns of the Split's input in place; operators whose outputs nobody reads any more (the Split, the Reshapes) are dropped.
void RModel::FuseAttentionInputs()
{
   std::map<std::string, size_t> producer;
   for (size_t k = 0; k < fOperators.size(); ++k)
      if (!fSkippedOperators.count(k))
         for (auto &o : fOperators[k]->GetOpOutputTensors()) producer[o] = k;
   for (size_t k = 0; k < fOperators.size(); ++k) {
      if (fSkippedOperators.count(k)) continue;
      auto *sdpa = dynamic_cast<ROperator_SDPA<float> *>(fOperators[k].get());
      if (!sdpa || !sdpa->IsFolded()) continue;
      for (int which = 0; which < 3; ++which) {
         const std::string in = ResolveAliasTensor(sdpa->GetOpInputTensors()[size_t(which)]);
         auto it = producer.find(in);
         if (it == producer.end()) continue;
         auto *split = dynamic_cast<ROperator_Split *>(fOperators[it->second].get());
         if (!split || !split->SplitsLastAxis()) continue;
         const int idx = split->OutputIndex(in);
         if (idx < 0) continue;
         sdpa->ReadFromColumnBlock(which, split->Input(), split->ColumnStart(idx), split->RowPitch());
         fFusionLog.push_back("op_" + std::to_string(k) + " reads " + in + " in place from " + split->Input());
      }
   }
   // dead operators: no output is read by a live operator or is a graph output
   for (bool changed = true; changed;) {
      changed = false;
      std::set<std::string> read;
      for (size_t k = 0; k < fOperators.size(); ++k)
         if (!fSkippedOperators.count(k))
            for (auto &in : fOperators[k]->GetOpInputTensors()) { read.insert(in); read.insert(ResolveAliasTensor(in)); }
      for (auto &o : fOutputTensorNames) { read.insert(o); read.insert(ResolveAliasTensor(o)); }
      for (size_t k = 0; k < fOperators.size(); ++k) {
         if (fSkippedOperators.count(k)) continue;
         if (!dynamic_cast<ROperator_Split *>(fOperators[k].get()) && !(AsB200(fOperators[k].get()) && AsB200(fOperators[k].get())->IsAlias())) continue;
         bool used = false;
         for (auto &o : fOperators[k]->GetOpOutputTensors()) used = used || read.count(o);
         if (!used) { fSkippedOperators.insert(k); changed = true; }
      }
   }
}

// DequantizeLinear (per tensor, zero point 0) -> GlobalAveragePool -> [Flatten / Reshape] -> Gemm: the pool averages the
// quantised values themselves and the scale becomes part of the Gemm's alpha (a mean is linear), which saves the pass
// that would write the dequantised tensor.
void RModel::FuseDequantizePool()
{
   auto soleReader = [&](const std::string &t) -> long {
      long found = -1;
      if (IsOutputTensor(t)) return -1;
      for (size_t k = 0; k < fOperators.size(); ++k) {
         if (fSkippedOperators.count(k)) continue;
         for (auto &in : fOperators[k]->GetOpInputTensors())
            if (in == t) { if (found >= 0) return -1; found = long(k); }
      }
      return found;
   };
   for (size_t k = 0; k < fOperators.size(); ++k) {
      if (fSkippedOperators.count(k)) continue;
      auto *dq = dynamic_cast<ROperator_QuantizeLinear *>(fOperators[k].get());
      if (!dq || !dq->IsDequantize() || !dq->IsPerTensor() || GetTensorType(dq->NameX()) != ETensorType::INT8) continue;
      if (!dq->NameZp().empty())
         if (auto zp = GetTensorData<int8_t>(dq->NameZp()); !zp.empty() && zp[0] != 0) continue;
      if (!IsInitializedTensor(dq->NameScale())) continue;
      const long pk = soleReader(dq->NameY());
      auto *pool = pk >= 0 ? dynamic_cast<ROperator_Pool<float> *>(fOperators[size_t(pk)].get()) : nullptr;
      if (!pool) continue;
      std::string t = pool->NameY();
      long gk = soleReader(t);
      while (gk >= 0 && AsB200(fOperators[size_t(gk)].get()) && AsB200(fOperators[size_t(gk)].get())->IsAlias()) {
         t = fOperators[size_t(gk)]->GetOpOutputTensors()[0];
         gk = soleReader(t);
      }
      auto *gemm = gk >= 0 ? dynamic_cast<ROperator_Gemm<float> *>(fOperators[size_t(gk)].get()) : nullptr;
      if (!gemm || ResolveAliasTensor(gemm->NameA()) != ResolveAliasTensor(t)) continue;
      pool->ReadQuantised(dq->NameX(), ETensorType::INT8);
      gemm->ScaleAlpha(GetTensorData<float>(dq->NameScale())[0]);
      fSkippedOperators.insert(k);
      fFusionLog.push_back("op_" + std::to_string(pk) + " pools the quantised tensor; op_" + std::to_string(gk) + " applies the scale of op_" + std::to_string(k));
   }
}

// Layout pass.  The reference keeps every tensor NCHW.  Here a convolution whose result is read by exactly one other
// convolution hands it over channels-last (int8: plain; fp32: as TF32 pairs, which the 3xTF32 contraction reads in
// place), so that the inner layers of a conv -> conv chain run as implicit convolutions without an unfolded copy, and a
// GlobalAveragePool behind the chain reads the channels-last tensor directly.  The ends of a chain stay NCHW.
void RModel::AssignConvLayouts()
{
   std::map<std::string, std::vector<size_t>> readers;
   for (size_t k = 0; k < fOperators.size(); ++k)
      if (!fSkippedOperators.count(k))
         for (auto &in : fOperators[k]->GetOpInputTensors()) readers[in].push_back(k);
   std::map<std::string, size_t> convOf;   // tensor -> convolution that writes it
   for (size_t k = 0; k < fOperators.size(); ++k)
      if (!fSkippedOperators.count(k))
         if (auto *c = dynamic_cast<ConvLayoutHooks *>(fOperators[k].get())) convOf[c->LayoutOutput()] = k;
   auto sole = [&](const std::string &t) -> ROperator * {
      auto it = readers.find(t);
      if (it == readers.end() || it->second.size() != 1 || IsOutputTensor(t)) return nullptr;
      return fOperators[it->second[0]].get();
   };
   for (size_t k = 0; k < fOperators.size(); ++k) {
      if (fSkippedOperators.count(k)) continue;
      auto *c = dynamic_cast<ConvLayoutHooks *>(fOperators[k].get());
      if (!c) continue;
      const ConvGeometry &g = c->Geometry();
      if (g.Is3D()) continue;   // a lowered 3-D convolution keeps the reference's layout on both sides
      int y = 0;
      if (!c->HasResidual()) {
         ROperator *next = sole(c->LayoutOutput());
         // a per-tensor DequantizeLinear is elementwise: it passes the layout through to what follows it
         std::string t = c->LayoutOutput();
         while (auto *dq = dynamic_cast<ROperator_QuantizeLinear *>(next)) {
            if (!dq->IsDequantize() || !dq->IsPerTensor() || dq->NameX() != t) { next = nullptr; break; }
            t = dq->NameY();
            next = sole(t);
         }
         if (auto *n = dynamic_cast<ConvLayoutHooks *>(next); n && t == c->LayoutOutput() && n->LayoutInput() == t && n->IsInt8() == c->IsInt8()) {
            const ConvGeometry &ng = n->Geometry();
            if (c->IsInt8()) {
               if ((ng.C / ng.group) % 16 == 0) y = 1;
            } else {
               const bool canWritePairs = c->fXLayout == 2 || ConvNeedsNoWorkspace(g, 4, 4, c->fXLayout, 2, 0);
               if (g.group == 1 && ng.group == 1 && ng.C % 32 == 0 && g.K % 4 == 0 && canWritePairs) y = 2;
               else if ((ng.C / ng.group) % 4 == 0) y = 1;
            }
            if (y) n->SetLayouts(y, n->fYLayout);
         } else if (auto *pool = dynamic_cast<ROperator_Pool<float> *>(next); pool && pool->NameX() == t) {
            y = 1;
            pool->SetChannelsLast(true);
         }
      }
      int x = c->fXLayout;
      if (x == 2 && y == 0) {
         // a tensor of TF32 pairs can only feed a convolution with a channels-last result: take the plain channels-last
         // tensor from the producer instead
         x = 1;
         if (auto it = convOf.find(c->LayoutInput()); it != convOf.end()) {
            auto *p = dynamic_cast<ConvLayoutHooks *>(fOperators[it->second].get());
            p->SetLayouts(p->fXLayout, 1);
            fStorageFactor.erase(c->LayoutInput());
         }
      }
      c->SetLayouts(x, y);
      if (y == 2) fStorageFactor[c->LayoutOutput()] = 2;
      if (x || y) fFusionLog.push_back("op_" + std::to_string(k) + " layouts x " + std::to_string(x) + " y " + std::to_string(y));
   }
}

// ---------------------------------------------------------------------------------------------------
// arena
// ---------------------------------------------------------------------------------------------------
void RModel::PlanArena()
{
   fRegions.clear();
   const int64_t nOps = int64_t(fOperators.size());
   std::set<std::string> usedWeights;
   std::map<std::string, std::pair<int64_t, int64_t>> life;  // pooled tensors: [begin, end)
   auto root = [&](const std::string &n) { return ResolveAliasTensor(n); };
   std::set<std::string> outputRoots;
   for (auto &o : fOutputTensorNames) outputRoots.insert(root(o));
   for (int64_t k = 0; k < nOps; ++k) {
      if (fSkippedOperators.count(size_t(k))) continue;
      for (auto &in : fOperators[k]->GetOpInputTensors()) {
         const std::string r = root(in);
         if (IsInitializedTensor(r)) { if (!IsConstantTensor(r)) usedWeights.insert(r); continue; }
         if (auto it = life.find(r); it != life.end()) it->second.second = std::max(it->second.second, k + 1);
      }
      for (auto &o : fOperators[k]->GetOpOutputTensors()) {
         const std::string r = root(o);
         if (IsInitializedTensor(r) || IsInputTensor(r) || outputRoots.count(r)) continue;
         if (!life.count(r)) life[r] = {k, k + 1};
      }
   }
   // graph outputs that are weights or folded constants still need device storage
   for (auto &r : outputRoots)
      if (IsInitializedTensor(r)) usedWeights.insert(r);

   // With a symbolic dimension every size is a * n + b (kSymbolicBase stands for n): both parts are aligned, and the pooled
   // tensors all count as alive for the whole inference -- a block freed by a tensor of a * n bytes cannot be promised to
   // one of b bytes for every n -- so every offset is a sum of aligned sizes, linear in n.
   const int64_t symBase = fSymbol.empty() ? 0 : int64_t(kSymbolicBase);
   auto AlignUp = [symBase](int64_t v) { return AlignUpSymbolic(v, symBase); };
   int64_t off = 0;
   auto place = [&](const std::string &name, int64_t bytes, const char *kind) {
      fRegions.push_back({name, off, bytes, 0, nOps + 1, kind});
      off += AlignUp(bytes);
   };
   for (auto &n : fInitializedOrder)
      if (usedWeights.count(n)) {
         auto &t = fInitializedTensors.at(n);
         place(n, int64_t(ConvertShapeToLength(t.shape) * GetTypeSize(t.type)), "weight");
      }
   fWeightBytes = off;
   for (auto &n : fInputTensorNames) {
      auto &t = fInputTensorInfos.at(n);
      place(n, int64_t(ConvertShapeToLength(t.shape) * GetTypeSize(t.type)), "input");
   }
   for (auto &r : outputRoots)
      if (!IsInitializedTensor(r) && !IsInputTensor(r)) {
         auto &t = fIntermediateTensorInfos.at(r);
         place(r, int64_t(ConvertShapeToLength(t.shape) * GetTypeSize(t.type)), "output");
      }
   // pooled: intermediates by lifetime, operator scratch for the one step that uses it
   std::vector<TensorLifeInfo> lives;
   std::vector<ArenaRegion> pooled;
   fUnplannedBytes = 0;
   for (auto &[n, be] : life) {
      auto &t = fIntermediateTensorInfos.at(n);
      const size_t factor = fStorageFactor.count(n) ? fStorageFactor.at(n) : 1;   // a tensor of TF32 pairs holds two values per element
      const int64_t bytes = int64_t(ConvertShapeToLength(t.shape) * GetTypeSize(t.type) * factor);
      if (symBase) lives.push_back({0, nOps + 1, AlignUp(bytes)});
      else lives.push_back({be.first, be.second, bytes});
      pooled.push_back({n, 0, bytes, be.first, be.second, "intermediate"});
      fUnplannedBytes += AlignUp(bytes);
   }
   for (int64_t k = 0; k < nOps; ++k) {
      if (fSkippedOperators.count(size_t(k))) continue;
      if (auto *b = AsB200(fOperators[k].get()))
         for (auto &s : b->GetDeviceScratch_GPU_B200()) {
            if (symBase) lives.push_back({0, nOps + 1, AlignUp(int64_t(s.bytes))});
            else lives.push_back({k, k + 1, int64_t(s.bytes)});
            pooled.push_back({s.name, 0, int64_t(s.bytes), k, k + 1, "scratch"});
            fUnplannedBytes += AlignUp(int64_t(s.bytes));
         }
   }
   MemoryResult res = OrganizeMemory(lives);
   for (size_t i = 0; i < pooled.size(); ++i) {
      pooled[i].offset = off + res.offsets[i];
      fRegions.push_back(pooled[i]);
   }
   fPoolBytes = res.total_bytes;
   fPoolFreeBytes = size_t(res.total_free_bytes);
   fPoolLargestFree = size_t(res.largest_free_block);
   fArenaBytes = off + res.total_bytes;
}

// ---------------------------------------------------------------------------------------------------
// emission
// ---------------------------------------------------------------------------------------------------
void RModel::Generate(std::underlying_type_t<Options>, int, bool)
{
   throw std::runtime_error("SOFIE_B200::RModel::Generate: the CPU target belongs to the reference generator; use GenerateGPU_B200 "
                            "(this generator has no CPU path)");
}

void RModel::GenerateGPU_B200(std::underlying_type_t<Options> options, int batchSize, bool verbose)
{
   fOptions = options;
   const auto unsupported = Options::kGNN | Options::kGNNComponent | Options::kLowRankFactorize | Options::kStridedInput | Options::kNoSession |
                            Options::kKernelOnly;
   if (options & unsupported)
      throw std::runtime_error("SOFIE_B200::GenerateGPU_B200: an option outside the B200 target was requested (GNN, low-rank, strided input, "
                               "no-session and kernel-only generation are not part of it)");
   Initialize(batchSize, verbose);
   for (size_t i = 0; i < fOperators.size(); ++i)
      if (!AsB200(fOperators[i].get()))
         throw std::runtime_error("SOFIE_B200: operator " + std::to_string(i) + " has no B200 implementation");
   if (!fSymbol.empty())
      for (auto &[name, info] : fIntermediateTensorInfos)   // the dimension may only lead: a Reshape or a transposing operator that moves it inward is refused
         for (size_t i = 1; i < info.shape.size(); ++i)
            if (info.shape[i] >= kSymbolicBase / 2)
               throw std::runtime_error("SOFIE_B200: tensor " + name + " carries the symbolic dimension " + fSymbol + " in an inner position " +
                                        ConvertShapeToString(info.shape) + "; only a leading dimension may be symbolic");
   if (!fSymbol.empty())
      for (size_t i = 0; i < fOperators.size(); ++i)
         if (!AsB200(fOperators[i].get())->SupportsSymbolicDim())
            throw std::runtime_error("SOFIE_B200: operator " + std::to_string(i) + " (output " + (fOperators[i]->GetOpOutputTensors().empty() ? std::string("-") : fOperators[i]->GetOpOutputTensors()[0]) +
                                     ") needs static shapes; the model has the symbolic dimension " +
                                     fSymbol + " (pass a batch size for input_size / batch_size / bs, or fix the dimension in the model)");
   FuseOperators();
   FuseAttentionInputs();
   FuseDequantizePool();
   AssignConvLayouts();
   PlanArena();
   fGC = GenerateSessionCode_GPU_B200();
}

std::string SafetensorsDType(ETensorType type);

namespace {

std::string PtrType(ETensorType t) { return ConvertTypeToString(t) + " *"; }

template <class T>
void WriteValues(std::ostream &o, const void *data, size_t n, bool asInt)
{
   const T *p = static_cast<const T *>(data);
   for (size_t i = 0; i < n; ++i) {
      if (asInt) o << long(p[i]);
      else o << p[i];
      o << (i + 1 < n ? " " : "");
   }
}

void WriteTensorText(std::ostream &o, const InitializedTensor &t)
{
   const size_t n = ConvertShapeToLength(t.shape);
   switch (t.type) {
   case ETensorType::FLOAT: {
      // max_digits10 digits, subnormals flushed to zero: the reference's text format (core/src/RModel.cxx:1936-1951)
      o << std::setprecision(std::numeric_limits<float>::max_digits10);
      const float *p = static_cast<const float *>(t.data.get());
      for (size_t i = 0; i < n; ++i) {
         float v = p[i];
         if (v != 0.f && std::abs(v) < std::numeric_limits<float>::min()) v = 0.f;
         o << v << (i + 1 < n ? " " : "");
      }
      break;
   }
   case ETensorType::INT8: WriteValues<int8_t>(o, t.data.get(), n, true); break;
   case ETensorType::UINT8: case ETensorType::FLOAT8E4M3FN: case ETensorType::BOOL: WriteValues<uint8_t>(o, t.data.get(), n, true); break;
   case ETensorType::BFLOAT16: WriteValues<uint16_t>(o, t.data.get(), n, true); break;
   case ETensorType::INT32: WriteValues<int32_t>(o, t.data.get(), n, true); break;
   case ETensorType::INT64: WriteValues<int64_t>(o, t.data.get(), n, true); break;
   default: throw std::runtime_error("SOFIE_B200: tensor type cannot be written to the weight file");
   }
}

}  // namespace

namespace {

// Rewrites every integer literal that carries the symbolic dimension (see kSymbolicBase) as "a * <member> + b".  A literal is
// a run of digits that is not part of an identifier, a floating-point or a suffixed number.  A line that defined a
// compile-time constant from such a literal becomes a const member initialised from the dimension.
std::string SymbolizeCode(const std::string &code, const std::string &member)
{
   auto isWord = [](char c) { return std::isalnum(static_cast<unsigned char>(c)) || c == '_' || c == '.'; };
   std::string out;
   out.reserve(code.size() + code.size() / 8);
   size_t lineStart = 0;
   bool lineSymbolic = false;
   auto endLine = [&]() {
      if (lineSymbolic) {
         const size_t p = out.find("static constexpr", lineStart);
         if (p != std::string::npos) out.replace(p, 16, "const");
      }
      lineStart = out.size();
      lineSymbolic = false;
   };
   static const std::string kWeights = "static const ";   // (Options::kNoWeightFile: the embedded weight values are data, not sizes)
   for (size_t i = 0; i < code.size();) {
      if (out.size() == lineStart && code.compare(i, kWeights.size(), kWeights) == 0 && code.find(" fWeights_", i) < code.find('\n', i)) {
         const size_t e = code.find('\n', i);
         out.append(code, i, e == std::string::npos ? std::string::npos : e - i);
         i = e == std::string::npos ? code.size() : e;
         continue;
      }
      const char c = code[i];
      if (std::isdigit(static_cast<unsigned char>(c)) && (i == 0 || !isWord(code[i - 1]))) {
         size_t j = i;
         while (j < code.size() && std::isdigit(static_cast<unsigned char>(code[j]))) ++j;
         const std::string tok = code.substr(i, j - i);
         SymbolicValue sv;
         if ((j == code.size() || !isWord(code[j])) && tok.size() >= 11 && tok.size() <= 19 && DecodeSymbolic(std::stoull(tok), sv)) {
            out += "(size_t(" + std::to_string(sv.a) + ") * " + member;
            if (sv.b > 0) out += " + " + std::to_string(sv.b);
            if (sv.b < 0) out += " - " + std::to_string(-sv.b);
            out += ")";
            lineSymbolic = true;
         } else {
            out += tok;
         }
         i = j;
         continue;
      }
      out += c;
      ++i;
      if (c == '\n') endLine();
   }
   endLine();
   return out;
}

}  // namespace

std::string RModel::GenerateSessionCode_GPU_B200()
{
   const bool dynamic = !fSymbol.empty();
   const std::string symMember = "fDim_" + fSymbol;
   const bool extStream = fOptions & static_cast<std::underlying_type_t<Options>>(Options::kExternalStream);
   const bool customMem = fOptions & static_cast<std::underlying_type_t<Options>>(Options::kCustomMemory);
   const bool profile = fOptions & static_cast<std::underlying_type_t<Options>>(Options::kProfile);
   const bool debug = fOptions & static_cast<std::underlying_type_t<Options>>(Options::kDebug);
   const bool noWeightFile = fOptions & static_cast<std::underlying_type_t<Options>>(Options::kNoWeightFile);
   const bool safetensors = !noWeightFile && (fOptions & static_cast<std::underlying_type_t<Options>>(Options::kSafetensorsWeightFile));

   std::map<std::string, const ArenaRegion *> region;
   for (auto &r : fRegions) region[r.name] = &r;
   auto typeOf = [&](const std::string &n) { return GetTensorType(n); };

   std::stringstream o;
   std::string guard = fName;
   for (auto &c : guard) c = char(std::toupper(static_cast<unsigned char>(c)));
   o << "// Code generated automatically by SOFIE_B200 (B200 / sm_100a target) from the model " << fName << "\n";
   o << "// Link with libsofie_b200 and the CUDA runtime.\n";
   o << "#ifndef SOFIE_B200_" << guard << "\n#define SOFIE_B200_" << guard << "\n\n";
   o << "#include <cuda_runtime.h>\n#include <cstdint>\n#include <cstdio>\n#include <fstream>\n#include <iterator>\n#include <limits>\n#include <span>\n#include <stdexcept>\n#include <string>\n#include <vector>\n";
   o << "#include \"sofie_b200.h\"\n\nnamespace SOFIE_" << fName << " {\n\n";
   if (customMem) {
      o << "// One block for weights, inputs, outputs and the pooled intermediates: alloc is called once by the\n"
           "// constructor, dealloc once by the destructor (Options::kCustomMemory).\n"
           "struct MemoryProvider {\n   void *(*alloc)(size_t bytes, void *user);\n   void (*dealloc)(void *block, void *user);\n   void *user;\n};\n\n";
   }
   if (noWeightFile) {
      for (auto &r : fRegions) {
         if (r.kind != "weight") continue;
         auto &t = fInitializedTensors.at(r.name);
         o << "static const " << ConvertTypeToString(t.type) << " fWeights_" << r.name << "[] = {";
         std::stringstream vals;
         WriteTensorText(vals, t);
         std::string v = vals.str();
         for (auto &c : v) if (c == ' ') c = ',';
         o << v << "};\n";
      }
      o << "\n";
   }
   o << "struct Session {\n";
   if (dynamic)
      o << "   // the model's symbolic dimension " << fSymbol << ": fixed by the constructor, every size below follows from it\n   const size_t " << symMember << ";\n";
   o << "   static constexpr size_t kArenaBytes = " << fArenaBytes << ";\n";
   o << "   static constexpr size_t kWeightBytes = " << fWeightBytes << ";\n";
   o << "   static constexpr size_t kPoolBytes = " << fPoolBytes << ";        // pooled intermediates + scratch, planned by lifetime\n";
   o << "   static constexpr size_t kUnplannedPoolBytes = " << fUnplannedBytes << ";  // the same tensors without reuse\n";
   o << "   cudaStream_t stream = nullptr;\n   bool fOwnStream = false;\n   sofie_b200_ctx *ctx = nullptr;\n   char *fArena = nullptr;\n";
   if (customMem) o << "   MemoryProvider fProvider{};\n";
   o << "\n   // tensors: pointers into the arena\n";
   for (auto &r : fRegions) {
      const std::string t = r.kind == "scratch" ? std::string("char *") : PtrType(typeOf(r.name));
      const std::string member = r.kind == "input" ? "fInputStage_" + r.name : "tensor_" + r.name;
      o << "   " << t << member << " = nullptr;  // " << r.kind << ", offset " << r.offset << ", " << r.bytes << " bytes";
      if (r.kind == "intermediate" || r.kind == "scratch") o << ", alive on steps [" << r.begin << "," << r.end << ")";
      o << "\n";
   }
   o << "\n   // per-operator state\n";
   for (size_t i = 0; i < fOperators.size(); ++i)
      if (!fSkippedOperators.count(i)) o << AsB200(fOperators[i].get())->GenerateSessionMembersCode_GPU_B200(std::to_string(i));
   if (profile) {
      o << "   std::vector<cudaEvent_t> fProfEvents;\n   std::vector<double> fProfTotalMs;\n   size_t fProfCalls = 0;\n";
   }
   const size_t nIn = fInputTensorNames.size();
   o << "\n   // CUDA graphs of the inference body, one per set of input pointers seen (the two staging sets of infer_host_many);\n"
        "   // the first call runs eagerly (plans finish their one-time work), the next one is captured, later ones replay\n";
   o << "   struct CapturedGraph { cudaGraphExec_t exec = nullptr; const void *in[" << (nIn ? nIn : 1) << "] = {}; size_t age = 0; };\n";
   o << "   CapturedGraph fGraphs[2];\n   bool fUseCudaGraph = " << (profile ? "false" : "true") << ";\n   size_t fCalls = 0;\n";
   if (!customMem) {
      o << "   // second staging set, output parking buffers, copy streams and events of infer_host_many (created on first use)\n";
      o << "   char *fQueueMem = nullptr;\n   cudaStream_t fCopyIn = nullptr, fCopyOut = nullptr;\n"
           "   cudaEvent_t fEvReady[2] = {}, fEvConsumed[2] = {}, fEvParked[2] = {}, fEvLeft[2] = {};\n";
   }

   o << R"(
   static void Check(int rc, const char *what)
   {
      if (rc != 0) throw std::runtime_error(std::string("SOFIE_B200 ") + what + ": " + sofie_b200_status_string(rc) + ": " + sofie_b200_last_error());
   }
   static void CheckCuda(cudaError_t e, const char *what)
   {
      if (e != cudaSuccess) throw std::runtime_error(std::string("SOFIE_B200 ") + what + ": " + cudaGetErrorString(e));
   }
   template <class T>
   static void ReadTensorFromStream(std::istream &is, std::vector<T> &target, const std::string &expectedName, size_t expectedLength)
   {
      std::string name;
      size_t length = 0;
      is >> name >> length;
      if (name != expectedName)
         throw std::runtime_error("sofie failed to read the correct tensor name; expected name is " + expectedName + " , read " + name);
      if (length != expectedLength)
         throw std::runtime_error("sofie failed to read the correct tensor size; expected size is " + std::to_string(expectedLength) + " , read " + std::to_string(length));
      target.resize(length);
      for (size_t i = 0; i < length; ++i) {
         if constexpr (sizeof(T) == 1) { int v; is >> v; target[i] = T(v); }
         else if constexpr (std::is_floating_point<T>::value) {
            std::string tok; is >> tok;
            target[i] = tok == "inf" ? std::numeric_limits<T>::infinity() : tok == "-inf" ? -std::numeric_limits<T>::infinity()
                        : tok == "nan" ? std::numeric_limits<T>::quiet_NaN() : T(std::stod(tok));
         } else is >> target[i];
      }
      if (is.fail()) throw std::runtime_error("sofie failed to read the values for tensor " + expectedName);
   }
)";
   if (safetensors) {
      o << R"(
   // safetensors: 8-byte little-endian header size, a JSON header {"name": {"dtype": "..", "shape": [..], "data_offsets": [b, e]}, ..},
   // then the raw little-endian payload.  Finds one tensor and checks its type and size; returns a pointer into the blob.
   static const char *FindSafetensor(const std::string &blob, const std::string &name, const std::string &dtype, size_t bytes)
   {
      if (blob.size() < 8) throw std::runtime_error("sofie: truncated safetensors blob: missing JSON header size");
      unsigned long long hs = 0;
      for (int i = 0; i < 8; ++i) hs |= (unsigned long long)(static_cast<unsigned char>(blob[i])) << (8 * i);
      if (hs > blob.size() - 8) throw std::runtime_error("sofie: truncated JSON header in safetensors blob");
      const std::string header = blob.substr(8, hs);
      const size_t at = header.find("\"" + name + "\":");
      if (at == std::string::npos) throw std::runtime_error("sofie: tensor " + name + " not found in safetensors blob");
      const size_t close = header.find('}', at);
      const std::string entry = header.substr(at, close == std::string::npos ? std::string::npos : close - at);
      const size_t dt = entry.find("\"dtype\":\"");
      if (dt == std::string::npos) throw std::runtime_error("sofie: tensor " + name + " has no dtype in safetensors blob");
      const std::string found = entry.substr(dt + 9, entry.find('"', dt + 9) - (dt + 9));
      if (found != dtype) throw std::runtime_error("sofie: tensor " + name + " in safetensors blob has dtype " + found + " , expected " + dtype);
      const size_t off = entry.find("\"data_offsets\":[");
      if (off == std::string::npos) throw std::runtime_error("sofie: tensor " + name + " has no data_offsets in safetensors blob");
      unsigned long long b = 0, e = 0;
      if (std::sscanf(entry.c_str() + off + 16, "%llu,%llu", &b, &e) != 2 || e < b || 8 + hs + e > blob.size())
         throw std::runtime_error("sofie: bad data_offsets for tensor " + name + " in safetensors blob");
      if (e - b != bytes)
         throw std::runtime_error("sofie: tensor " + name + " in safetensors blob has " + std::to_string(e - b) + " bytes , expected " + std::to_string(bytes));
      return blob.data() + 8 + hs + b;
   }
)";
   }

   // ---- InitSession
   o << "\n   void InitSession(const std::string &filename)\n   {\n";
   o << "      int device = 0;\n      CheckCuda(cudaGetDevice(&device), \"cudaGetDevice\");\n";
   o << "      Check(sofie_b200_ctx_create(&ctx, device, stream), \"ctx_create\");\n";
   if (customMem) {
      o << "      if (!fProvider.alloc || !fProvider.dealloc) throw std::runtime_error(\"SOFIE_B200 MemoryProvider needs alloc and dealloc\");\n";
      o << "      fArena = static_cast<char *>(fProvider.alloc(kArenaBytes, fProvider.user));\n";
      o << "      if (!fArena) throw std::runtime_error(\"SOFIE_B200 MemoryProvider::alloc returned null\");\n";
      o << "      if (reinterpret_cast<uintptr_t>(fArena) % 256) throw std::runtime_error(\"SOFIE_B200 MemoryProvider block is not 256-byte aligned\");\n";
   } else {
      o << "      CheckCuda(cudaMalloc(reinterpret_cast<void **>(&fArena), kArenaBytes ? kArenaBytes : 256), \"arena allocation\");\n";
   }
   for (auto &r : fRegions) {
      const std::string t = r.kind == "scratch" ? std::string("char *") : PtrType(typeOf(r.name));
      const std::string member = r.kind == "input" ? "fInputStage_" + r.name : "tensor_" + r.name;
      o << "      " << member << " = reinterpret_cast<" << t << ">(fArena + " << r.offset << ");\n";
   }
   if (debug) o << "      ValidateMemory();\n";
   bool anyWeight = false;
   for (auto &r : fRegions) anyWeight |= r.kind == "weight";
   if (anyWeight) {
      if (safetensors) {
         o << "      std::ifstream f(filename, std::ios::binary);\n      if (!f.is_open()) throw std::runtime_error(\"sofie failed to open file \" + filename + \" for input weights\");\n";
         o << "      const std::string blob((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());\n";
      } else if (!noWeightFile) {
         o << "      std::ifstream f(filename);\n      if (!f.is_open()) throw std::runtime_error(\"sofie failed to open file \" + filename + \" for input weights\");\n";
      } else {
         o << "      (void)filename;\n";
      }
      for (auto &r : fRegions) {
         if (r.kind != "weight") continue;
         auto &t = fInitializedTensors.at(r.name);
         const std::string ct = ConvertTypeToString(t.type);
         const size_t len = ConvertShapeToLength(t.shape);
         if (safetensors) {
            o << "      CheckCuda(cudaMemcpyAsync(tensor_" << r.name << ", FindSafetensor(blob, \"tensor_" << r.name << "\", \"" << SafetensorsDType(t.type)
              << "\", " << r.bytes << "), " << r.bytes << ", cudaMemcpyHostToDevice, stream), \"weight upload\");\n";
            (void)len;
         } else if (!noWeightFile) {
            o << "      { std::vector<" << ct << "> h; ReadTensorFromStream(f, h, \"tensor_" << r.name << "\", " << len << ");\n";
            o << "        CheckCuda(cudaMemcpyAsync(tensor_" << r.name << ", h.data(), " << r.bytes
              << ", cudaMemcpyHostToDevice, stream), \"weight upload\"); CheckCuda(cudaStreamSynchronize(stream), \"weight upload\"); }\n";
         } else {
            o << "      CheckCuda(cudaMemcpyAsync(tensor_" << r.name << ", fWeights_" << r.name << ", " << r.bytes
              << ", cudaMemcpyHostToDevice, stream), \"weight upload\");\n";
         }
      }
      o << "      CheckCuda(cudaStreamSynchronize(stream), \"weight upload\");\n";
   } else {
      o << "      (void)filename;\n";
   }
   for (size_t i = 0; i < fOperators.size(); ++i)
      if (!fSkippedOperators.count(i)) o << AsB200(fOperators[i].get())->GenerateInitCode_GPU_B200(std::to_string(i));
   if (profile) {
      o << "      fProfEvents.resize(" << fOperators.size() + 1 << ");\n      for (auto &e : fProfEvents) CheckCuda(cudaEventCreate(&e), \"event\");\n";
      o << "      fProfTotalMs.assign(" << fOperators.size() << ", 0.0);\n";
   }
   o << "      Check(sofie_b200_ctx_sync(ctx), \"Session initialisation\");\n";
   o << "   }\n\n";

   // ---- constructors / destructor
   const std::string defFile = noWeightFile ? "\"\"" : "\"" + fName + (safetensors ? ".safetensors\"" : ".dat\"");
   const std::string prov = customMem ? "MemoryProvider provider, " : "";
   const std::string provInit = customMem ? "fProvider = provider; " : "";
   // with a symbolic dimension the constructor takes its value after the file name (Session(filename, N) in the reference's tests)
   const std::string fileParam = dynamic ? std::string("std::string filename, size_t ") + fSymbol + "_value" : "std::string filename = " + defFile;
   const std::string memInit = dynamic ? ") : " + symMember + "(" + fSymbol + "_value" : "";
   o << "   Session(" << prov << fileParam << memInit << ")\n   {\n      " << provInit
     << "CheckCuda(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking), \"stream\");\n      fOwnStream = true;\n      InitSession(filename);\n   }\n";
   if (extStream) {
      o << "   // the stream is borrowed: it must outlive the Session and is never destroyed here\n";
      o << "   Session(" << prov << "cudaStream_t externalStream, " << fileParam << memInit << ")\n   {\n      " << provInit
        << "stream = externalStream;\n      InitSession(filename);\n   }\n";
   }
   o << "   Session(const Session &) = delete;\n   Session &operator=(const Session &) = delete;\n";
   o << "   ~Session()\n   {\n      if (stream || ctx) cudaStreamSynchronize(stream);\n";
   for (size_t i = 0; i < fOperators.size(); ++i)
      if (!fSkippedOperators.count(i)) o << AsB200(fOperators[i].get())->GenerateDestroyCode_GPU_B200(std::to_string(i));
   if (profile) o << "      for (auto &e : fProfEvents) cudaEventDestroy(e);\n";
   o << "      for (auto &g : fGraphs) if (g.exec) cudaGraphExecDestroy(g.exec);\n";
   if (!customMem) {
      o << "      if (fCopyIn) { cudaStreamSynchronize(fCopyIn); cudaStreamSynchronize(fCopyOut); cudaStreamDestroy(fCopyIn); cudaStreamDestroy(fCopyOut);\n"
           "         for (int i = 0; i < 2; ++i) { cudaEventDestroy(fEvReady[i]); cudaEventDestroy(fEvConsumed[i]); cudaEventDestroy(fEvParked[i]); cudaEventDestroy(fEvLeft[i]); } }\n"
           "      if (fQueueMem) cudaFree(fQueueMem);\n";
   }
   o << "      if (ctx) sofie_b200_ctx_destroy(ctx);\n";
   if (customMem) o << "      if (fArena) fProvider.dealloc(fArena, fProvider.user);\n";
   else o << "      if (fArena) cudaFree(fArena);\n";
   o << "      if (fOwnStream && stream) cudaStreamDestroy(stream);\n   }\n\n";

   // ---- _infer_impl
   std::string params, args, hostParams;
   for (size_t i = 0; i < fInputTensorNames.size(); ++i) {
      const auto &n = fInputTensorNames[i];
      const std::string ct = ConvertTypeToString(typeOf(n));
      params += (i ? ", " : "") + std::string("const ") + ct + " *tensor_" + n;
      hostParams += (i ? ", " : "") + std::string("const ") + ct + " *host_" + n;
      args += (i ? ", " : "") + std::string("tensor_") + n;
   }
   o << "   // records the whole inference on the stream; device pointers in, nothing is synchronised\n";
   o << "   void _infer_impl(" << params << ")\n   {\n";
   for (size_t i = 0; i < fOperators.size(); ++i) {
      if (fSkippedOperators.count(i)) continue;
      auto *op = AsB200(fOperators[i].get());
      if (profile) o << "      CheckCuda(cudaEventRecord(fProfEvents[" << i << "], stream), \"event\");\n";
      if (op->IsAlias()) {
         const std::string out = op->GetOpOutputTensors()[0], r = ResolveAliasTensor(out);
         o << "      " << PtrType(typeOf(out)) << "tensor_" << out << " = const_cast<" << PtrType(typeOf(out)) << ">(tensor_" << r << ");  // alias\n";
      }
      o << op->Generate_GPU_B200(std::to_string(i));
   }
   if (profile) o << "      CheckCuda(cudaEventRecord(fProfEvents[" << fOperators.size() << "], stream), \"event\");\n";
   o << "   }\n\n";

   // ---- infer surface
   auto outMember = [&](const std::string &n) {
      const std::string r = ResolveAliasTensor(n);
      return IsInputTensor(r) ? std::string() : "tensor_" + r;
   };
   const std::string out0 = fOutputTensorNames.empty() ? "" : fOutputTensorNames[0];
   const std::string outT = out0.empty() ? "void" : ConvertTypeToString(typeOf(out0));
   o << "   // device pointers in; the returned device pointer is owned by the Session and overwritten by the next call\n";
   {
      std::string same, remember, inArr;
      for (size_t i = 0; i < nIn; ++i) {
         same += " && g.in[" + std::to_string(i) + "] == tensor_" + fInputTensorNames[i];
         remember += " slot->in[" + std::to_string(i) + "] = tensor_" + fInputTensorNames[i] + ";";
      }
      o << "   // " << (profile ? "with SetUseCudaGraph(true) " : "after the first call ") << "the body is replayed from a CUDA graph (one launch instead of one per operator); a stream that is\n"
           "   // already being captured by the caller just records the operators into the caller's graph\n";
      o << "   void SetUseCudaGraph(bool on) { fUseCudaGraph = on; }\n";
      o << "   void Enqueue(" << params << ")\n   {\n";
      o << "      const size_t call = fCalls++;\n";
      o << "      cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;\n";
      o << "      if (!fUseCudaGraph || call == 0 || cudaStreamIsCapturing(stream, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) { _infer_impl(" << args << "); return; }\n";
      o << "      CapturedGraph *slot = &fGraphs[0];\n";
      o << "      for (auto &g : fGraphs) {\n";
      o << "         if (g.exec" << same << ") { g.age = call; CheckCuda(cudaGraphLaunch(g.exec, stream), \"graph launch\"); return; }\n";
      o << "         if (!g.exec || g.age < slot->age) slot = &g;\n";
      o << "      }\n";
      o << "      if (fGraphs[0].exec == nullptr) slot = &fGraphs[0]; else if (fGraphs[1].exec == nullptr) slot = &fGraphs[1];\n";
      o << "      if (slot->exec) { cudaGraphExecDestroy(slot->exec); slot->exec = nullptr; }\n";
      o << "      CheckCuda(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal), \"graph capture\");\n";
      o << "      cudaGraph_t graph = nullptr;\n";
      o << "      try { _infer_impl(" << args << "); } catch (...) { cudaStreamEndCapture(stream, &graph); if (graph) cudaGraphDestroy(graph); throw; }\n";
      o << "      CheckCuda(cudaStreamEndCapture(stream, &graph), \"graph capture\");\n";
      o << "      const cudaError_t ie = cudaGraphInstantiate(&slot->exec, graph, 0);\n";
      o << "      cudaGraphDestroy(graph);\n";
      o << "      CheckCuda(ie, \"graph instantiation\");\n";
      o << "     " << remember << " slot->age = call;\n";
      o << "      CheckCuda(cudaGraphLaunch(slot->exec, stream), \"graph launch\");\n";
      o << "   }\n";
   }
   o << "   " << outT << " *infer_nosync(" << params << ")\n   {\n      Enqueue(" << args << ");\n      return " << outMember(out0) << ";\n   }\n";
   o << "   " << outT << " *infer(" << params << ")\n   {\n      " << outT << " *r = infer_nosync(" << args << ");\n"
     << "      Check(sofie_b200_ctx_sync(ctx), \"infer\");\n";
   if (profile) {
      o << "      for (size_t i = 0; i + 1 < fProfEvents.size(); ++i) { float ms = 0; if (cudaEventElapsedTime(&ms, fProfEvents[i], fProfEvents[i + 1]) == cudaSuccess) fProfTotalMs[i] += ms; }\n      ++fProfCalls;\n";
   }
   o << "      return r;\n   }\n";
   if (dynamic) {
      // the reference's dynamic form repeats the dimension in front of the inputs (session.infer(N, input))
      o << "   // the dimension again, as the reference's dynamic Sessions take it: it must be the one the Session was built for\n";
      o << "   " << outT << " *infer(size_t " << fSymbol << "_value, " << params << ")\n   {\n";
      o << "      if (" << fSymbol << "_value != " << symMember << ") throw std::runtime_error(\"SOFIE_B200 Session::infer: the Session was built for another value of " << fSymbol << "\");\n";
      o << "      return infer(" << args << ");\n   }\n";
      o << "   size_t GetSymbolicDimension() const { return " << symMember << "; }\n";
   }
   // the reference's span form (RModel_ALPAKA.cxx:814-838): views of the inputs in, results copied into the caller's output views
   o << "   // runs the model on device pointers to the inputs, copies every output into the caller's device buffers and waits\n";
   o << "   void infer(std::span<const void *const> inputs, std::span<void *const> outputs)\n   {\n";
   o << "      if (inputs.size() != " << nIn << " || outputs.size() != " << fOutputTensorNames.size() << ") throw std::runtime_error(\"SOFIE_B200 Session::infer: expected " << nIn
     << " input and " << fOutputTensorNames.size() << " output views\");\n";
   {
      std::string spanArgs;
      for (size_t i = 0; i < nIn; ++i)
         spanArgs += (i ? ", " : "") + std::string("static_cast<const ") + ConvertTypeToString(typeOf(fInputTensorNames[i])) + " *>(inputs[" + std::to_string(i) + "])";
      o << "      Enqueue(" << spanArgs << ");\n";
   }
   for (size_t i = 0; i < fOutputTensorNames.size(); ++i) {
      const std::string &n = fOutputTensorNames[i];
      const std::string src = outMember(n).empty() ? "tensor_" + ResolveAliasTensor(n) : outMember(n);
      o << "      CheckCuda(cudaMemcpyAsync(outputs[" << i << "], " << src << ", " << ConvertShapeToLength(GetTensorShape(n)) * GetTypeSize(typeOf(n))
        << ", cudaMemcpyDeviceToDevice, stream), \"output copy\");\n";
   }
   o << "      Check(sofie_b200_ctx_sync(ctx), \"infer\");\n   }\n";
   o << "   // output i of the graph (device pointer), valid after infer()\n   const void *output(size_t i) const\n   {\n      switch (i) {\n";
   for (size_t i = 0; i < fOutputTensorNames.size(); ++i) o << "      case " << i << ": return " << outMember(fOutputTensorNames[i]) << ";\n";
   o << "      default: throw std::runtime_error(\"SOFIE_B200 Session::output: index out of range\");\n      }\n   }\n";
   o << "   // host pointers in, host vector out: copies in, runs, copies the first output back\n";
   o << "   std::vector<" << outT << "> infer_host(" << hostParams << ")\n   {\n";
   for (auto &n : fInputTensorNames) {
      o << "      CheckCuda(cudaMemcpyAsync(fInputStage_" << n << ", host_" << n << ", " << region.at(n)->bytes
        << ", cudaMemcpyHostToDevice, stream), \"input upload\");\n";
   }
   std::string stageArgs;
   for (size_t i = 0; i < fInputTensorNames.size(); ++i) stageArgs += (i ? ", " : "") + std::string("fInputStage_") + fInputTensorNames[i];
   const size_t outLen = out0.empty() ? 0 : ConvertShapeToLength(GetTensorShape(out0));
   o << "      " << outT << " *d = infer_nosync(" << stageArgs << ");\n";
   o << "      std::vector<" << outT << "> h(" << outLen << ");\n";
   o << "      CheckCuda(cudaMemcpyAsync(h.data(), d, " << outLen << " * sizeof(" << outT << "), cudaMemcpyDeviceToHost, stream), \"output download\");\n";
   o << "      Check(sofie_b200_ctx_sync(ctx), \"infer_host\");\n      return h;\n   }\n";
   if (!customMem && !out0.empty()) {
      // a queue of inferences from host memory
      size_t inBytes = 0;
      std::vector<size_t> inOff;
      const int64_t symBase = dynamic ? int64_t(kSymbolicBase) : 0;   // (sizes linear in the symbolic dimension: both parts aligned)
      for (auto &n : fInputTensorNames) { inOff.push_back(inBytes); inBytes += size_t(AlignUpSymbolic(int64_t(region.at(n)->bytes), symBase)); }
      const size_t outBytes = outLen * GetTypeSize(typeOf(out0)), outPad = size_t(AlignUpSymbolic(int64_t(outBytes), symBase));
      std::string manyParams, stage0, stage1;
      for (size_t i = 0; i < fInputTensorNames.size(); ++i) {
         const auto &n = fInputTensorNames[i];
         const std::string ct = ConvertTypeToString(typeOf(n));
         manyParams += "const " + ct + " *const *hosts_" + n + ", ";
         stage0 += (i ? ", " : "") + std::string("fInputStage_") + n;
         stage1 += (i ? ", " : "") + std::string("reinterpret_cast<const ") + ct + " *>(fQueueMem + " + std::to_string(inOff[i]) + ")";
      }
      o << "   // A queue of `count` inferences from host memory (pinned memory lets the copies run beside the kernels): input i + 1 is\n"
           "   // copied to the second staging set while inference i runs, and output i leaves through a parking buffer while inference\n"
           "   // i + 1 runs.  host_out[i] receives the first output of inference i; returns when all of them are written.\n";
      o << "   void infer_host_many(size_t count, " << manyParams << outT << " *const *host_out)\n   {\n";
      o << "      if (!fCopyIn) {\n";
      o << "         CheckCuda(cudaMalloc(reinterpret_cast<void **>(&fQueueMem), " << inBytes + 2 * outPad << "), \"queue buffers\");\n";
      o << "         CheckCuda(cudaStreamCreateWithFlags(&fCopyIn, cudaStreamNonBlocking), \"stream\");\n";
      o << "         CheckCuda(cudaStreamCreateWithFlags(&fCopyOut, cudaStreamNonBlocking), \"stream\");\n";
      o << "         for (int i = 0; i < 2; ++i) for (cudaEvent_t *e : {&fEvReady[i], &fEvConsumed[i], &fEvParked[i], &fEvLeft[i]}) CheckCuda(cudaEventCreateWithFlags(e, cudaEventDisableTiming), \"event\");\n";
      o << "      }\n";
      o << "      CheckCuda(cudaStreamSynchronize(stream), \"queue start\");\n";
      o << "      for (size_t i = 0; i < count; ++i) {\n";
      o << "         const int s = int(i & 1);\n";
      o << "         if (i >= 2) CheckCuda(cudaStreamWaitEvent(fCopyIn, fEvConsumed[s], 0), \"queue\");\n";
      for (size_t i = 0; i < fInputTensorNames.size(); ++i) {
         const auto &n = fInputTensorNames[i];
         o << "         CheckCuda(cudaMemcpyAsync(s ? static_cast<void *>(fQueueMem + " << inOff[i] << ") : static_cast<void *>(fInputStage_" << n << "), hosts_" << n
           << "[i], " << region.at(n)->bytes << ", cudaMemcpyHostToDevice, fCopyIn), \"input upload\");\n";
      }
      o << "         CheckCuda(cudaEventRecord(fEvReady[s], fCopyIn), \"queue\");\n";
      o << "         CheckCuda(cudaStreamWaitEvent(stream, fEvReady[s], 0), \"queue\");\n";
      o << "         " << outT << " *d = s ? infer_nosync(" << stage1 << ") : infer_nosync(" << stage0 << ");\n";
      o << "         CheckCuda(cudaEventRecord(fEvConsumed[s], stream), \"queue\");\n";
      o << "         char *park = fQueueMem + " << inBytes << " + size_t(s) * " << outPad << ";\n";
      o << "         if (i >= 2) CheckCuda(cudaStreamWaitEvent(stream, fEvLeft[s], 0), \"queue\");\n";
      o << "         CheckCuda(cudaMemcpyAsync(park, d, " << outBytes << ", cudaMemcpyDeviceToDevice, stream), \"output parking\");\n";
      o << "         CheckCuda(cudaEventRecord(fEvParked[s], stream), \"queue\");\n";
      o << "         CheckCuda(cudaStreamWaitEvent(fCopyOut, fEvParked[s], 0), \"queue\");\n";
      o << "         CheckCuda(cudaMemcpyAsync(host_out[i], park, " << outBytes << ", cudaMemcpyDeviceToHost, fCopyOut), \"output download\");\n";
      o << "         CheckCuda(cudaEventRecord(fEvLeft[s], fCopyOut), \"queue\");\n";
      o << "      }\n";
      o << "      CheckCuda(cudaStreamSynchronize(fCopyOut), \"queue end\");\n";
      o << "      Check(sofie_b200_ctx_sync(ctx), \"infer_host_many\");\n";
      o << "   }\n";
   }
   o << "   // zeroes the pooled intermediates (the reference's resetState)\n";
   o << "   void resetState()\n   {\n      CheckCuda(cudaMemsetAsync(fArena + (kArenaBytes - kPoolBytes), 0, kPoolBytes, stream), \"resetState\");\n   }\n";
   o << "   size_t GetIntermediateMemoryPoolSize() const { return kPoolBytes; }\n";
   o << "   // free space inside the pool when its footprint last grew, as the reference reports it (RModel_ALPAKA.cxx:1262-1269)\n";
   o << "   size_t GetTotalFreeMemory() const { return " << fPoolFreeBytes << "; }\n";
   o << "   size_t GetLargestFreeBlock() const { return " << fPoolLargestFree << "; }\n";
   o << "   double GetFragmentation() const { return GetTotalFreeMemory() == 0 ? 0.0 : 1.0 - double(GetLargestFreeBlock()) / double(GetTotalFreeMemory()); }\n";
   o << "   size_t GetArenaSize() const { return kArenaBytes; }\n";
   o << "   long long GetLaunchCount() const { return sofie_b200_ctx_launch_count(ctx); }\n";
   if (profile) {
      o << "   double GetOpAvgTime(size_t op) const { return fProfCalls ? fProfTotalMs.at(op) / double(fProfCalls) : 0.0; }\n";
      o << "   void PrintProfilingResults() const\n   {\n      for (size_t i = 0; i < fProfTotalMs.size(); ++i) if (fProfTotalMs[i] > 0) std::printf(\"op_%zu : %.4f ms\\n\", i, GetOpAvgTime(i));\n   }\n";
   }
   if (debug) {
      o << "   // alignment and overlap-while-alive check of the arena regions (the reference's ValidateMemory)\n";
      o << "   void ValidateMemory() const\n   {\n      struct R { const char *name; size_t off, bytes; long b, e; };\n      " << (dynamic ? "" : "static ") << "const R regions[] = {\n";
      for (auto &r : fRegions) o << "         {\"" << r.name << "\", " << r.offset << ", " << r.bytes << ", " << r.begin << ", " << r.end << "},\n";
      o << "      };\n      const size_t n = sizeof(regions) / sizeof(regions[0]);\n"
           "      for (size_t i = 0; i < n; ++i) {\n"
           "         if (regions[i].off % 256) throw std::runtime_error(std::string(\"SOFIE_B200 arena region not 256-byte aligned: \") + regions[i].name);\n"
           "         if (regions[i].off + regions[i].bytes > kArenaBytes) throw std::runtime_error(std::string(\"SOFIE_B200 arena region out of bounds: \") + regions[i].name);\n"
           "         for (size_t j = 0; j < i; ++j) {\n"
           "            const bool alive = regions[i].b < regions[j].e && regions[j].b < regions[i].e;\n"
           "            const bool overlap = regions[i].off < regions[j].off + regions[j].bytes && regions[j].off < regions[i].off + regions[i].bytes;\n"
           "            if (alive && overlap && regions[i].bytes && regions[j].bytes)\n"
           "               throw std::runtime_error(std::string(\"SOFIE_B200 arena regions overlap while alive: \") + regions[i].name + \" / \" + regions[j].name);\n"
           "         }\n      }\n"
           "      std::printf(\"[SOFIE debug] arena %zu bytes, %zu regions validated\\n\", size_t(kArenaBytes), n);\n   }\n";
   }
   o << "};\n\n}  // namespace SOFIE_" << fName << "\n\n#endif  // SOFIE_B200_" << guard << "\n";
   return dynamic ? SymbolizeCode(o.str(), symMember) : o.str();
}

// safetensors type names: the reference's F32 / F64 / I64 (core/src/RModel.cxx:51-59) plus the low-precision types of this target
std::string SafetensorsDType(ETensorType type)
{
   switch (type) {
   case ETensorType::FLOAT: return "F32";
   case ETensorType::DOUBLE: return "F64";
   case ETensorType::INT64: return "I64";
   case ETensorType::INT32: return "I32";
   case ETensorType::INT8: return "I8";
   case ETensorType::UINT8: return "U8";
   case ETensorType::BOOL: return "BOOL";
   case ETensorType::BFLOAT16: return "BF16";
   case ETensorType::FLOAT8E4M3FN: return "F8_E4M3";
   default: throw std::runtime_error("sofie tensor with type " + ConvertTypeToString(type) + " cannot be written to a safetensors file");
   }
}

// Layout of the reference's writer (core/src/RModel.cxx:1967-2010): names sorted, header size as 8 little-endian bytes, JSON
// header, payload in the same order with no padding.
void RModel::WriteSafetensorsFile(const std::string &filename) const
{
   const std::uint16_t one = 1;
   if (!*reinterpret_cast<const std::uint8_t *>(&one)) throw std::runtime_error("sofie: safetensors weights can only be written on a little-endian host");
   std::vector<std::string> names;
   for (auto &r : fRegions)
      if (r.kind == "weight") names.push_back(r.name);
   std::sort(names.begin(), names.end());
   std::string header = "{";
   std::uint64_t offset = 0;
   for (size_t i = 0; i < names.size(); ++i) {
      const auto &t = fInitializedTensors.at(names[i]);
      const std::uint64_t nbytes = ConvertShapeToLength(t.shape) * GetTypeSize(t.type);
      header += std::string(i ? "," : "") + "\"tensor_" + names[i] + "\":{\"dtype\":\"" + SafetensorsDType(t.type) + "\",\"shape\":[";
      for (size_t d = 0; d < t.shape.size(); ++d) header += (d ? "," : "") + std::to_string(t.shape[d]);
      header += "],\"data_offsets\":[" + std::to_string(offset) + "," + std::to_string(offset + nbytes) + "]}";
      offset += nbytes;
   }
   header += "}";
   std::ofstream f(filename, std::ios::binary);
   if (!f.is_open()) throw std::runtime_error("sofie-b200 failed to open file " + filename + " for tensor weight data");
   const std::uint64_t hs = header.size();
   char sz[8];
   for (int i = 0; i < 8; ++i) sz[i] = static_cast<char>((hs >> (8 * i)) & 0xff);
   f.write(sz, 8);
   f.write(header.data(), std::streamsize(header.size()));
   for (auto &n : names) {
      const auto &t = fInitializedTensors.at(n);
      f.write(static_cast<const char *>(t.data.get()), std::streamsize(ConvertShapeToLength(t.shape) * GetTypeSize(t.type)));
   }
   if (f.fail()) throw std::runtime_error("sofie failed to write safetensors payload");
}

void RModel::WriteWeightFile(const std::string &filename) const
{
   std::ofstream f(filename);
   if (!f.is_open()) throw std::runtime_error("sofie-b200 failed to open file " + filename + " for tensor weight data");
   for (auto &r : fRegions) {
      if (r.kind != "weight") continue;
      auto &t = fInitializedTensors.at(r.name);
      f << "tensor_" << r.name << " " << ConvertShapeToLength(t.shape) << "\n";
      WriteTensorText(f, t);
      f << "\n";
   }
   if (f.fail()) throw std::runtime_error("sofie-b200 failed to write tensor weight data to " + filename);
}

void RModel::OutputGenerated(std::string filename, bool append)
{
   if (fGC.empty()) throw std::runtime_error("SOFIE_B200::OutputGenerated: nothing generated yet; call GenerateGPU_B200 first");
   if (filename.empty()) filename = fName + ".hxx";
   std::ofstream f(filename, append ? std::ios::app : std::ios::out);
   if (!f.is_open()) throw std::runtime_error("sofie-b200 failed to open file " + filename + " for output");
   f << fGC;
   f.close();
   if (!(fOptions & static_cast<std::underlying_type_t<Options>>(Options::kNoWeightFile))) {
      std::string dat = filename;
      auto dot = dat.find_last_of('.');
      if (dot != std::string::npos) dat = dat.substr(0, dot);
      // the Session's default weight file name is <model>.dat, next to the header
      auto slash = dat.find_last_of("/\\");
      const std::string dir = slash == std::string::npos ? "" : dat.substr(0, slash + 1);
      if (fOptions & static_cast<std::underlying_type_t<Options>>(Options::kSafetensorsWeightFile)) WriteSafetensorsFile(dir + fName + ".safetensors");
      else WriteWeightFile(dir + fName + ".dat");
   }
}

void RModel::PrintGenerated() const { std::cout << fGC; }

}  // namespace SOFIE_B200
