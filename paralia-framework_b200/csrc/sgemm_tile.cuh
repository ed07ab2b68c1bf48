// Host-visible interface of the FP32 tile GEMM (3xTF32 on the tcgen05 tensor path).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace paralia {

// Opt the kernels into their dynamic shared memory size; once per device.
cudaError_t sgemm_tile_configure();

}  // namespace paralia
