// FP32 tile GEMM. Placeholder translation unit until the 3xTF32 tcgen05 kernel lands:
// the entry points exist and report PARALIA_ERR_UNSUPPORTED.
#include "sgemm_tile.cuh"

#include "exec.hpp"
#include "runtime.hpp"

namespace paralia {

cudaError_t sgemm_tile_configure() { return cudaSuccess; }

int exec_tile_sgemm(int, void*, char, char, int64_t, int64_t, int64_t, float, const float*, int64_t,
                    const float*, int64_t, float, float*, int64_t) {
  return fail(PARALIA_ERR_UNSUPPORTED, "SGEMM tile kernel is not built yet");
}

int exec_sgemm(char, char, int64_t, int64_t, int64_t, float, const float*, int64_t, int,
               const float*, int64_t, int, float, float*, int64_t, int, const paralia_ctl*,
               paralia_report*) {
  return fail(PARALIA_ERR_UNSUPPORTED, "SGEMM is not built yet");
}

}  // namespace paralia
