// Level-1 tile kernels (FP64 axpy and dot) and the input-fill kernels.
//
// These stand where the reference reaches cublasDaxpy / cublasDdot through
// backend_run_operation(params, "Daxpy" | "Ddot", queue)
// (Library_scheduler/src/Functions/daxpy.cpp:53-69, ddot.cpp:54-70).
// Both are HBM-bound: 24 bytes per element for axpy (read x, read y, write y) and 16 for
// dot. Unit-stride operands on 16-byte boundaries move as 128-bit accesses, four in
// flight per thread; anything else takes the strided scalar path.
#include "level1.cuh"

#include <mutex>

#include "../../include/paralia_c.h"
#include "paralia_rng.h"
#include "runtime.hpp"

namespace paralia {
namespace {

constexpr int L1_THREADS = 512;
constexpr int L1_UNROLL = 4;

__global__ void __launch_bounds__(L1_THREADS)
daxpy_vec_kernel(int64_t n2, double alpha, const double2* __restrict__ x, double2* __restrict__ y) {
  const int64_t stride = (int64_t)gridDim.x * L1_THREADS;
  int64_t i = (int64_t)blockIdx.x * L1_THREADS + threadIdx.x;
  for (; i + (L1_UNROLL - 1) * stride < n2; i += L1_UNROLL * stride) {
    double2 xv[L1_UNROLL], yv[L1_UNROLL];
#pragma unroll
    for (int u = 0; u < L1_UNROLL; ++u) xv[u] = x[i + u * stride];
#pragma unroll
    for (int u = 0; u < L1_UNROLL; ++u) yv[u] = y[i + u * stride];
#pragma unroll
    for (int u = 0; u < L1_UNROLL; ++u) {
      yv[u].x = fma(alpha, xv[u].x, yv[u].x);
      yv[u].y = fma(alpha, xv[u].y, yv[u].y);
      y[i + u * stride] = yv[u];
    }
  }
  for (; i < n2; i += stride) {
    double2 xv = x[i], yv = y[i];
    yv.x = fma(alpha, xv.x, yv.x);
    yv.y = fma(alpha, xv.y, yv.y);
    y[i] = yv;
  }
}

__global__ void __launch_bounds__(L1_THREADS)
daxpy_strided_kernel(int64_t n, double alpha, const double* __restrict__ x, int64_t incx,
                     double* __restrict__ y, int64_t incy) {
  const int64_t stride = (int64_t)gridDim.x * L1_THREADS;
  for (int64_t i = (int64_t)blockIdx.x * L1_THREADS + threadIdx.x; i < n; i += stride)
    y[i * incy] = fma(alpha, x[i * incx], y[i * incy]);
}

// Sum of the 512 per-thread values of a block in a fixed order: xor-shuffle tree inside
// each warp, then the 16 warp sums in warp order by thread 0.
__device__ __forceinline__ double block_sum(double v, double* warp_sums) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = v;
  __syncthreads();
  double s = 0.0;
  if (threadIdx.x == 0) {
#pragma unroll
    for (int w = 0; w < L1_THREADS / 32; ++w) s += warp_sums[w];
  }
  return s;
}

__global__ void __launch_bounds__(L1_THREADS)
ddot_vec_kernel(int64_t n2, const double2* __restrict__ x, const double2* __restrict__ y,
                double* __restrict__ partials) {
  __shared__ double warp_sums[L1_THREADS / 32];
  const int64_t stride = (int64_t)gridDim.x * L1_THREADS;
  int64_t i = (int64_t)blockIdx.x * L1_THREADS + threadIdx.x;
  double acc[L1_UNROLL];
#pragma unroll
  for (int u = 0; u < L1_UNROLL; ++u) acc[u] = 0.0;
  for (; i + (L1_UNROLL - 1) * stride < n2; i += L1_UNROLL * stride) {
    double2 xv[L1_UNROLL], yv[L1_UNROLL];
#pragma unroll
    for (int u = 0; u < L1_UNROLL; ++u) xv[u] = x[i + u * stride];
#pragma unroll
    for (int u = 0; u < L1_UNROLL; ++u) yv[u] = y[i + u * stride];
#pragma unroll
    for (int u = 0; u < L1_UNROLL; ++u) {
      acc[u] = fma(xv[u].x, yv[u].x, acc[u]);
      acc[u] = fma(xv[u].y, yv[u].y, acc[u]);
    }
  }
  for (; i < n2; i += stride) {
    const double2 xv = x[i], yv = y[i];
    acc[0] = fma(xv.x, yv.x, acc[0]);
    acc[0] = fma(xv.y, yv.y, acc[0]);
  }
  const double v = (acc[0] + acc[1]) + (acc[2] + acc[3]);
  const double s = block_sum(v, warp_sums);
  if (threadIdx.x == 0) partials[blockIdx.x] = s;
}

__global__ void __launch_bounds__(L1_THREADS)
ddot_strided_kernel(int64_t n, const double* __restrict__ x, int64_t incx,
                    const double* __restrict__ y, int64_t incy, double* __restrict__ partials) {
  __shared__ double warp_sums[L1_THREADS / 32];
  const int64_t stride = (int64_t)gridDim.x * L1_THREADS;
  double acc = 0.0;
  for (int64_t i = (int64_t)blockIdx.x * L1_THREADS + threadIdx.x; i < n; i += stride)
    acc = fma(x[i * incx], y[i * incy], acc);
  const double s = block_sum(acc, warp_sums);
  if (threadIdx.x == 0) partials[blockIdx.x] = s;
}

// One block adds the per-block partials (and an optional odd tail element) in a fixed
// order and writes the tile's dot product.
__global__ void __launch_bounds__(L1_THREADS)
ddot_final_kernel(int nparts, const double* __restrict__ partials, const double* tail_x,
                  const double* tail_y, double* __restrict__ result) {
  __shared__ double warp_sums[L1_THREADS / 32];
  double acc = 0.0;
  for (int i = threadIdx.x; i < nparts; i += L1_THREADS) acc += partials[i];
  double s = block_sum(acc, warp_sums);
  if (threadIdx.x == 0) {
    if (tail_x) s = fma(*tail_x, *tail_y, s);
    *result = s;
  }
}

template <typename T, int DIST>
__global__ void fill_kernel(T* p, int64_t n, uint64_t seed) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    if (DIST == 0) {
      if (sizeof(T) == 8) p[i] = (T)paralia_uniform_f64(seed, (uint64_t)i);
      else p[i] = (T)paralia_uniform_f32(seed, (uint64_t)i);
    } else {
      p[i] = (T)paralia_normal_f64(seed, (uint64_t)i);
    }
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

int l1_grid_blocks(int64_t n) {
  // Fixed function of n only, so a given n always reduces in the same order.
  int64_t want = (n / 2 + (int64_t)L1_THREADS * L1_UNROLL - 1) / ((int64_t)L1_THREADS * L1_UNROLL);
  if (want < 1) want = 1;
  const int64_t cap = 148 * 4;  // four resident 512-thread blocks on each of 148 SMs
  return (int)(want < cap ? want : cap);
}

cudaError_t launch_daxpy(int64_t n, double alpha, const double* x, int64_t incx, double* y,
                         int64_t incy, cudaStream_t stream, int* launches) {
  if (n <= 0) return cudaSuccess;
  const int blocks = l1_grid_blocks(n);
  if (incx == 1 && incy == 1 && aligned16(x) && aligned16(y)) {
    const int64_t n2 = n / 2;
    if (n2 > 0) {
      daxpy_vec_kernel<<<blocks, L1_THREADS, 0, stream>>>(
          n2, alpha, reinterpret_cast<const double2*>(x), reinterpret_cast<double2*>(y));
      if (launches) ++*launches;
    }
    if (n & 1) {
      daxpy_strided_kernel<<<1, L1_THREADS, 0, stream>>>(1, alpha, x + n - 1, 1, y + n - 1, 1);
      if (launches) ++*launches;
    }
  } else {
    daxpy_strided_kernel<<<blocks, L1_THREADS, 0, stream>>>(n, alpha, x, incx, y, incy);
    if (launches) ++*launches;
  }
  return cudaGetLastError();
}

cudaError_t launch_ddot(int64_t n, const double* x, int64_t incx, const double* y, int64_t incy,
                        double* partials, double* result_dev, cudaStream_t stream,
                        int* launches) {
  const int blocks = l1_grid_blocks(n > 0 ? n : 1);
  if (n <= 0) {
    ddot_final_kernel<<<1, L1_THREADS, 0, stream>>>(0, partials, nullptr, nullptr, result_dev);
    if (launches) ++*launches;
    return cudaGetLastError();
  }
  if (incx == 1 && incy == 1 && aligned16(x) && aligned16(y)) {
    const int64_t n2 = n / 2;
    ddot_vec_kernel<<<blocks, L1_THREADS, 0, stream>>>(
        n2, reinterpret_cast<const double2*>(x), reinterpret_cast<const double2*>(y), partials);
    const bool odd = (n & 1) != 0;
    ddot_final_kernel<<<1, L1_THREADS, 0, stream>>>(blocks, partials, odd ? x + n - 1 : nullptr,
                                                    odd ? y + n - 1 : nullptr, result_dev);
    if (launches) *launches += 2;
  } else {
    ddot_strided_kernel<<<blocks, L1_THREADS, 0, stream>>>(n, x, incx, y, incy, partials);
    ddot_final_kernel<<<1, L1_THREADS, 0, stream>>>(blocks, partials, nullptr, nullptr,
                                                    result_dev);
    if (launches) *launches += 2;
  }
  return cudaGetLastError();
}

cudaError_t launch_fill_f64(double* p, int64_t n, uint64_t seed, int dist, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  const int blocks = 148 * 8;
  if (dist == 0) fill_kernel<double, 0><<<blocks, 256, 0, stream>>>(p, n, seed);
  else fill_kernel<double, 1><<<blocks, 256, 0, stream>>>(p, n, seed);
  return cudaGetLastError();
}

cudaError_t launch_fill_f32(float* p, int64_t n, uint64_t seed, int dist, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  const int blocks = 148 * 8;
  if (dist == 0) fill_kernel<float, 0><<<blocks, 256, 0, stream>>>(p, n, seed);
  else fill_kernel<float, 1><<<blocks, 256, 0, stream>>>(p, n, seed);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------
// Dot product for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need a dot
// product: code running between the warm-up and the steady state of a latency-critical
// loop where an allocation would synchronise the whole device, plugins that are handed a
// fixed memory budget by their host application, and code that runs while another
// library owns the allocator. PARALiA_tile_ddot asks such a caller for a scratch buffer;
// this variant needs none: the per-block partial sums live in the file-scope device
// array below, which every GPU that loads the library holds until the process exits
// (8 KB per GPU).
namespace {

constexpr int NOALLOC_SCRATCH_DOUBLES = 1024;
static __device__ __align__(256) double g_ddot_noalloc_scratch[NOALLOC_SCRATCH_DOUBLES];

// Device address of the array on each GPU. In host code the array's name is only a
// handle for the runtime, not an address a kernel could use, so the address is looked up
// once per device with that device current.
std::mutex g_noalloc_mutex;
double* g_noalloc_ptr[PARALIA_MAX_UNITS] = {};

}  // namespace

// Forget the looked-up addresses (library shutdown: after a device reset the next call must
// ask the runtime again instead of using an address of a context that is gone).
void ddot_noalloc_forget_addresses() {
  std::lock_guard<std::mutex> lk(g_noalloc_mutex);
  for (double*& p : g_noalloc_ptr) p = nullptr;
}

}  // namespace paralia

extern "C" int64_t PARALiA_tile_ddot_noalloc_max_n(void) { return (int64_t)1 << 31; }

extern "C" int PARALiA_tile_ddot_noalloc(int dev, void* stream, int64_t N, const double* x,
                                         int64_t incx, const double* y, int64_t incy,
                                         double* result_dev) {
  using namespace paralia;
  if (N < 0 || incx <= 0 || incy <= 0) return fail(PARALIA_ERR_INVALID_ARG, "bad N or increment");
  if (!result_dev || (N > 0 && (!x || !y)))
    return fail(PARALIA_ERR_INVALID_ARG, "NULL vector or result pointer");
  if (N > PARALiA_tile_ddot_noalloc_max_n())
    return fail(PARALIA_ERR_INVALID_ARG,
                "N = %lld exceeds the %lld elements the allocation-free dot product supports",
                (long long)N, (long long)PARALiA_tile_ddot_noalloc_max_n());
  if (l1_grid_blocks(N > 0 ? N : 1) > NOALLOC_SCRATCH_DOUBLES)
    return fail(PARALIA_ERR_INVALID_ARG, "N = %lld needs more partial sums than the static scratch holds",
                (long long)N);
  if (dev < 0 || dev >= PARALIA_MAX_UNITS) return fail(PARALIA_ERR_INVALID_ARG, "GPU id %d out of range", dev);
  int count = 0;
  PL_CUDA(cudaGetDeviceCount(&count));
  if (dev >= count) return fail(PARALIA_ERR_INVALID_ARG, "GPU id %d out of range", dev);
  DeviceGuard guard;   // cudaGetDevice / cudaSetDevice only
  PL_CUDA(cudaSetDevice(dev));
  double* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_noalloc_mutex);
    if (!g_noalloc_ptr[dev]) {
      void* p = nullptr;
      PL_CUDA(cudaGetSymbolAddress(&p, g_ddot_noalloc_scratch));
      g_noalloc_ptr[dev] = static_cast<double*>(p);
    }
    scratch = g_noalloc_ptr[dev];
  }
  // Every partial the final kernel reads is written by the first kernel of the same
  // call, so nothing in the array has to be cleared between calls.
  PL_CUDA(launch_ddot(N, x, incx, y, incy, scratch, result_dev, static_cast<cudaStream_t>(stream),
                      nullptr));
  return PARALIA_OK;
}
