// Model IR and generation driver of the B200 target.
//
// The model-building API is the reference's (core/inc/SOFIE/RModel.hxx:104-215): AddInputTensorInfo,
// AddInitializedTensor, AddOperator, AddOutputTensorNameList, Initialize, OutputGenerated.  Where
// the reference has Generate() (CPU) and GenerateGPU_ALPAKA() (core/src/RModel_ALPAKA.cxx:1595-1693),
// this driver has GenerateGPU_B200(): it emits a header with the same Session / infer() /
// infer_nosync() surface whose body is a sequence of calls into libsofie_b200 (include/sofie_b200.h),
// with all weights, intermediates and scratch placed in one lifetime-planned device arena.
// A symbolic dimension named input_size, batch_size or bs takes the batch size given to GenerateGPU_B200
// (core/src/RModel.cxx:676-685).  One other symbolic leading dimension per model stays open until the Session is constructed
// (Session(file, N), infer(N, inputs...), tests/alpaka/TestAlpakaLinear.cxx:121-203): it travels through shape inference as
// kSymbolicBase and every emitted size is rewritten as a * N + b (operators declare SupportsSymbolicDim).
#pragma once
#include <cstring>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <unordered_map>
#include <vector>

#include "SOFIE_B200/MemoryPlanner.hxx"
#include "SOFIE_B200/ROperator.hxx"

namespace SOFIE_B200 {

class RModel {
public:
   RModel() = default;
   RModel(std::string name, std::string parsedtime);
   RModel(RModel &&) = default;
   RModel &operator=(RModel &&) = default;

   // ---- model building ------------------------------------------------------------------
   void AddInputTensorInfo(std::string input_name, ETensorType type, std::vector<Dim> shape);
   void AddInputTensorInfo(std::string input_name, ETensorType type, std::vector<size_t> shape);
   void AddInputTensorName(std::string name);
   void AddInitializedTensor(std::string tensor_name, ETensorType type, std::vector<std::size_t> shape, std::shared_ptr<void> data);
   void AddInitializedTensor(const std::string &tensor_name, ETensorType type, const std::vector<std::size_t> &shape, void *raw_data);
   // a tensor consumed at generation time only (shape operands, folded parameters)
   void AddConstantTensor(std::string tensor_name, ETensorType type, std::vector<std::size_t> shape, std::shared_ptr<void> data);
   template <class T>
   void AddInitializedTensor(const std::string &name, ETensorType type, const std::vector<size_t> &shape, const std::vector<T> &values)
   {
      std::shared_ptr<void> p(malloc(values.size() * sizeof(T) + 1), free);
      std::memcpy(p.get(), values.data(), values.size() * sizeof(T));
      AddInitializedTensor(name, type, shape, p);
   }
   void AddIntermediateTensor(std::string tensor_name, ETensorType type, std::vector<std::size_t> shape);
   bool AddAliasTensor(const std::string &tensor_name, const std::string &orig_tensor_name);
   void AddOperator(std::unique_ptr<ROperator> op, int order_execution = -1);
   void AddOutputTensorNameList(std::vector<std::string> output_tensor_names);
   void UpdateOutputTensorList(std::vector<std::string> curr_output_tensor, std::vector<std::string> modify_output_tensor);

   // ---- queries (used by operators during Initialize) ---------------------------------------
   bool CheckIfTensorAlreadyExist(std::string tensor_name) const;
   bool IsInitializedTensor(const std::string &name) const;
   bool IsConstantTensor(const std::string &name) const;
   bool IsInputTensor(const std::string &name) const;
   bool IsOutputTensor(const std::string &name) const;
   bool IsAliasTensor(const std::string &name) const { return fAliasTensors.count(name) != 0; }
   std::string ResolveAliasTensor(const std::string &name) const;
   const std::vector<size_t> &GetTensorShape(const std::string &name) const;
   ETensorType GetTensorType(const std::string &name) const;
   std::shared_ptr<void> GetInitializedTensorData(const std::string &name) const;
   template <class T>
   std::vector<T> GetTensorData(const std::string &name) const
   {
      const auto &t = fInitializedTensors.at(UTILITY::Clean_name(name));
      const T *p = static_cast<const T *>(t.data.get());
      return std::vector<T>(p, p + ConvertShapeToLength(t.shape));
   }
   const std::vector<std::string> &GetInputTensorNames() const { return fInputTensorNames; }
   const std::vector<std::string> &GetOutputTensorNames() const { return fOutputTensorNames; }
   const std::string &GetName() const { return fName; }
   size_t GetNumberOfOperators() const { return fOperators.size(); }

   // ---- generation -----------------------------------------------------------------------
   void Initialize(int batchSize = -1, bool verbose = false);
   // The CPU target belongs to the reference generator; kept so that calling code compiles, throws.
   void Generate(std::underlying_type_t<Options> options = 0, int batchSize = -1, bool verbose = false);
   void Generate(Options options, int batchSize = -1, bool verbose = false) { Generate(static_cast<std::underlying_type_t<Options>>(options), batchSize, verbose); }
   void GenerateGPU_B200(std::underlying_type_t<Options> options, int batchSize = -1, bool verbose = false);
   void GenerateGPU_B200(Options options = Options::kDefault, int batchSize = -1, bool verbose = false)
   {
      GenerateGPU_B200(static_cast<std::underlying_type_t<Options>>(options), batchSize, verbose);
   }
   // true if every operator of the model has a B200 implementation (reference: CheckGPUOperators)
   bool CheckGPUOperators() const;
   void OutputGenerated(std::string filename = "", bool append = false);
   const std::string &ReturnGenerated() const { return fGC; }
   void PrintGenerated() const;
   void SetFilename(std::string filename) { fName = std::move(filename); }

   // ---- what generation decided (for tests and reports) -----------------------------------------
   struct ArenaRegion {
      std::string name;
      int64_t offset, bytes;
      int64_t begin, end;  // lifetime in operator steps; weights and outputs span the whole inference
      std::string kind;    // weight | input | intermediate | scratch | output
   };
   const std::vector<ArenaRegion> &GetArenaRegions() const { return fRegions; }
   int64_t GetArenaBytes() const { return fArenaBytes; }   // with a symbolic dimension: a * kSymbolicBase + b (DecodeSymbolic)
   // name of the model's symbolic dimension after Initialize / GenerateGPU_B200; empty when every shape is static
   const std::string &GetSymbolicDimension() const { return fSymbol; }
   int64_t GetIntermediateMemoryPoolSize() const { return fPoolBytes; }
   int64_t GetUnplannedIntermediateBytes() const { return fUnplannedBytes; }  // sum of pooled tensors without reuse
   const std::vector<std::string> &GetFusionLog() const { return fFusionLog; }

private:
   void FuseOperators();
   void FuseAttentionInputs();
   void AssignConvLayouts();
   void FuseDequantizePool();
   void PlanArena();
   std::string GenerateSessionCode_GPU_B200();
   void WriteWeightFile(const std::string &filename) const;
   void WriteSafetensorsFile(const std::string &filename) const;

   std::string fName = "model";
   std::string fParseTime;
   std::map<std::string, TensorInfo> fInputTensorInfos;  // graph inputs (static after Initialize)
   std::map<std::string, std::vector<Dim>> fInputDimShapes;
   std::vector<std::string> fInputTensorNames;
   std::map<std::string, InitializedTensor> fInitializedTensors;
   std::vector<std::string> fInitializedOrder;
   std::map<std::string, TensorInfo> fIntermediateTensorInfos;
   std::map<std::string, std::string> fAliasTensors;  // alias -> tensor whose storage it shares
   std::vector<std::string> fOutputTensorNames;
   std::vector<std::unique_ptr<ROperator>> fOperators;
   std::set<size_t> fSkippedOperators;
   std::map<std::string, size_t> fStorageFactor;   // bytes per element multiplier of tensors in a wider storage layout  // folded into a producer by the fusion pass

   std::underlying_type_t<Options> fOptions = 0;
   bool fIsInitialized = false;
   int fBatchSize = -1;
   std::string fSymbol;   // name of the model's symbolic dimension (empty: all shapes are static); see kSymbolicBase
   std::string fGC;  // generated code
   std::vector<ArenaRegion> fRegions;
   int64_t fArenaBytes = 0, fPoolBytes = 0, fUnplannedBytes = 0, fWeightBytes = 0;
   size_t fPoolFreeBytes = 0, fPoolLargestFree = 0;   // free space inside the pool when its footprint last grew
   std::vector<std::string> fFusionLog;
};

}  // namespace SOFIE_B200
