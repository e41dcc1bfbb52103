// sofie_b200_plan_arena: the C entry point over the arena planner the code generator also uses
// (sofie_b200/host/inc/SOFIE_B200/MemoryPlanner.hxx).  Host-only code; it lives in the runtime
// library because an emitted Session may re-plan its pool at construction, next to the
// plan-creation calls (the reference's Session calls OrganizeMemory there,
// core/src/RModel_ALPAKA.cxx:285-544).
#include "../host/inc/SOFIE_B200/MemoryPlanner.hxx"
#include "common.cuh"

extern "C" int sofie_b200_plan_arena(const sofie_b200_tensor_life *lives, int64_t n, int64_t *offsets,
                                     int64_t *total_bytes) {
  using sb200::fail;
  if (n < 0 || (n > 0 && (!lives || !offsets)) || !total_bytes)
    return fail(SOFIE_B200_ERR_INVALID, "plan_arena: NULL argument");
  std::vector<SOFIE_B200::TensorLifeInfo> v((size_t)n);
  for (int64_t i = 0; i < n; ++i) v[i] = {lives[i].begin, lives[i].end, lives[i].size};
  try {
    SOFIE_B200::MemoryResult r = SOFIE_B200::OrganizeMemory(v);
    for (int64_t i = 0; i < n; ++i) offsets[i] = r.offsets[i];
    *total_bytes = r.total_bytes;
  } catch (const std::exception &e) {
    return fail(SOFIE_B200_ERR_INVALID, "plan_arena: %s", e.what());
  }
  return 0;
}
