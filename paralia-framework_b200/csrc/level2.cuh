// Launcher of the FP64 matrix-vector tile kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace paralia {

// Number of column slices (= partial vectors of `rows` doubles) the op = N kernel uses for
// a rows x cols tile. Depends on the shape only.
int gemv_n_slices(int rows, int cols);

// y <- alpha*op(A)*x + beta*y for one column-major rows x cols tile on the current device.
// x has rows (op = T) or cols (op = N) elements with increment incx; y has rows (op = N) or
// cols (op = T) elements with increment incy. `partial` (op = N only) holds
// gemv_n_slices()*rows doubles.
cudaError_t launch_dgemv_tile(bool trans, int rows, int cols, double alpha, const double* A,
                              int64_t lda, const double* x, int64_t incx, double beta, double* y,
                              int64_t incy, double* partial, cudaStream_t stream, int* launches);

}  // namespace paralia
