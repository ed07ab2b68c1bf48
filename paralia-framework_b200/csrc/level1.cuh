// Launchers of the level-1 tile kernels and the input-fill kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace paralia {

// Number of thread blocks (= number of per-block partial sums) used for a vector of n
// elements. Depends on n only.
int l1_grid_blocks(int64_t n);

// y <- alpha*x + y on the current device; *launches (optional) is incremented per kernel.
cudaError_t launch_daxpy(int64_t n, double alpha, const double* x, int64_t incx, double* y,
                         int64_t incy, cudaStream_t stream, int* launches);

// *result_dev <- sum x_i*y_i. `partials` must hold l1_grid_blocks(n) doubles.
cudaError_t launch_ddot(int64_t n, const double* x, int64_t incx, const double* y, int64_t incy,
                        double* partials, double* result_dev, cudaStream_t stream,
                        int* launches);

// Drops the cached device addresses of the allocation-free dot product's static scratch.
void ddot_noalloc_forget_addresses();

cudaError_t launch_fill_f64(double* p, int64_t n, uint64_t seed, int dist, cudaStream_t stream);
cudaError_t launch_fill_f32(float* p, int64_t n, uint64_t seed, int dist, cudaStream_t stream);

}  // namespace paralia
