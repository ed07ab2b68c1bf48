// FP64 matrix-vector tile kernels: y <- alpha*op(A)*x + beta*y on one column-major tile.
//
// They stand where the reference reaches cublasDgemv through its backend for
// PARALiADgemv (Library_scheduler/src/Functions/dgemv.cpp:288). Both are HBM-bound:
// every element of A (8 bytes) is read once and used for one multiply-add.
//
//  op = N: threads run along the rows (the contiguous direction), two rows per thread as
//          one 128-bit load; the columns of the tile are cut into slices (grid.y) so that
//          enough loads are in flight; each slice leaves a partial vector, and a second
//          kernel adds the slices in slice order and applies alpha/beta. Fixed order, so
//          the result is bit-reproducible.
//  op = T: one warp per column; lanes stride down the column with 128-bit loads, a
//          xor-shuffle tree adds the lanes. alpha/beta applied by lane 0.
#include "level2.cuh"

namespace paralia {
namespace {

constexpr int GV_THREADS = 256;
constexpr int GV_XCHUNK = 512;   // x values staged in shared memory at a time

// partial[slice][m] = sum over the slice's columns of A[m, n] * x[n]
__global__ void __launch_bounds__(GV_THREADS)
dgemv_n_partial_kernel(int rows, int cols, const double* __restrict__ A, int64_t lda,
                       const double* __restrict__ x, int64_t incx, int cols_per_slice,
                       double* __restrict__ partial, int vec_ok) {
  __shared__ double xs[GV_XCHUNK];
  const int m = (blockIdx.x * GV_THREADS + threadIdx.x) * 2;
  const int n_begin = blockIdx.y * cols_per_slice;
  const int n_end = min(cols, n_begin + cols_per_slice);
  double acc0 = 0.0, acc1 = 0.0;
  for (int n0 = n_begin; n0 < n_end; n0 += GV_XCHUNK) {
    const int cnt = min(GV_XCHUNK, n_end - n0);
    __syncthreads();
    for (int i = threadIdx.x; i < cnt; i += GV_THREADS) xs[i] = x[(int64_t)(n0 + i) * incx];
    __syncthreads();
    if (m + 1 < rows && vec_ok) {
      const double* col = A + m + (int64_t)n0 * lda;
#pragma unroll 8
      for (int i = 0; i < cnt; ++i) {
        const double2 a = *reinterpret_cast<const double2*>(col + (int64_t)i * lda);
        acc0 = fma(a.x, xs[i], acc0);
        acc1 = fma(a.y, xs[i], acc1);
      }
    } else if (m < rows) {
      const double* col = A + m + (int64_t)n0 * lda;
      const bool two = m + 1 < rows;
#pragma unroll 4
      for (int i = 0; i < cnt; ++i) {
        acc0 = fma(col[(int64_t)i * lda], xs[i], acc0);
        if (two) acc1 = fma(col[(int64_t)i * lda + 1], xs[i], acc1);
      }
    }
  }
  if (m < rows) partial[(int64_t)blockIdx.y * rows + m] = acc0;
  if (m + 1 < rows) partial[(int64_t)blockIdx.y * rows + m + 1] = acc1;
}

// y[m] = alpha * (partial[0][m] + partial[1][m] + ...) + beta * y[m]
__global__ void __launch_bounds__(GV_THREADS)
dgemv_n_combine_kernel(int rows, int slices, const double* __restrict__ partial, double alpha,
                       double beta, double* __restrict__ y, int64_t incy) {
  const int m = blockIdx.x * GV_THREADS + threadIdx.x;
  if (m >= rows) return;
  double s = 0.0;
  for (int k = 0; k < slices; ++k) s += partial[(int64_t)k * rows + m];
  double v = alpha * s;
  if (beta != 0.0) v = fma(beta, y[(int64_t)m * incy], v);
  y[(int64_t)m * incy] = v;
}

// y[n] = alpha * dot(A[:, n], x) + beta * y[n], one warp per column
__global__ void __launch_bounds__(GV_THREADS)
dgemv_t_kernel(int rows, int cols, const double* __restrict__ A, int64_t lda,
               const double* __restrict__ x, int64_t incx, double alpha, double beta,
               double* __restrict__ y, int64_t incy, int vec_ok) {
  const int lane = threadIdx.x & 31;
  const int n = blockIdx.x * (GV_THREADS / 32) + (threadIdx.x >> 5);
  if (n >= cols) return;
  const double* col = A + (int64_t)n * lda;
  double acc[4] = {0.0, 0.0, 0.0, 0.0};
  if (vec_ok) {
    const int pairs = rows / 2;
    int i = lane;
    for (; i + 96 < pairs; i += 128) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const double2 a = *reinterpret_cast<const double2*>(col + 2 * (i + 32 * u));
        const double2 b = *reinterpret_cast<const double2*>(x + 2 * (i + 32 * u));
        acc[u] = fma(a.x, b.x, acc[u]);
        acc[u] = fma(a.y, b.y, acc[u]);
      }
    }
    for (; i < pairs; i += 32) {
      const double2 a = *reinterpret_cast<const double2*>(col + 2 * i);
      const double2 b = *reinterpret_cast<const double2*>(x + 2 * i);
      acc[0] = fma(a.x, b.x, acc[0]);
      acc[0] = fma(a.y, b.y, acc[0]);
    }
    if ((rows & 1) && lane == 0) acc[1] = fma(col[rows - 1], x[rows - 1], acc[1]);
  } else {
    for (int i = lane; i < rows; i += 32) acc[0] = fma(col[i], x[(int64_t)i * incx], acc[0]);
  }
  double s = (acc[0] + acc[1]) + (acc[2] + acc[3]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) {
    double v = alpha * s;
    if (beta != 0.0) v = fma(beta, y[(int64_t)n * incy], v);
    y[(int64_t)n * incy] = v;
  }
}

}  // namespace

int gemv_n_slices(int rows, int cols) {
  // enough blocks for ~4 per SM, at least 64 columns per slice; depends on the shape only
  const int row_blocks = (rows + GV_THREADS * 2 - 1) / (GV_THREADS * 2);
  int slices = (148 * 4 + row_blocks - 1) / row_blocks;
  const int max_slices = (cols + 63) / 64;
  if (slices > max_slices) slices = max_slices;
  if (slices < 1) slices = 1;
  return slices;
}

cudaError_t launch_dgemv_tile(bool trans, int rows, int cols, double alpha, const double* A,
                              int64_t lda, const double* x, int64_t incx, double beta, double* y,
                              int64_t incy, double* partial, cudaStream_t stream, int* launches) {
  // a transposed tile without rows still scales y by beta (every dot product is empty)
  if (cols <= 0 || rows < 0 || (rows == 0 && !trans)) return cudaSuccess;
  const bool a_ok = (reinterpret_cast<uintptr_t>(A) & 15) == 0 && (lda & 1) == 0;
  if (!trans) {
    const int slices = gemv_n_slices(rows, cols);
    const int cps = (cols + slices - 1) / slices;
    dim3 grid((rows + GV_THREADS * 2 - 1) / (GV_THREADS * 2), slices);
    dgemv_n_partial_kernel<<<grid, GV_THREADS, 0, stream>>>(rows, cols, A, lda, x, incx, cps, partial,
                                                            a_ok ? 1 : 0);
    dgemv_n_combine_kernel<<<(rows + GV_THREADS - 1) / GV_THREADS, GV_THREADS, 0, stream>>>(
        rows, slices, partial, alpha, beta, y, incy);
    if (launches) *launches += 2;
  } else {
    const bool x_ok = (reinterpret_cast<uintptr_t>(x) & 15) == 0 && incx == 1;
    const int warps = GV_THREADS / 32;
    dgemv_t_kernel<<<(cols + warps - 1) / warps, GV_THREADS, 0, stream>>>(
        rows, cols, A, lda, x, incx, alpha, beta, y, incy, (a_ok && x_ok) ? 1 : 0);
    if (launches) *launches += 1;
  }
  return cudaGetLastError();
}

}  // namespace paralia
