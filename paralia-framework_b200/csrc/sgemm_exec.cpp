// Per-tile FP32 GEMM entry point on device-resident data: pack both operands (stream-
// ordered scratch), run the 3xTF32 kernel. What the reference reaches through
// backend_run_operation(params, "Sgemm", queue) (Library_scheduler/src/Functions/
// sgemm.cpp:85-139).
#include <algorithm>
#include <cstring>

#include "exec.hpp"
#include "runtime.hpp"
#include "sgemm_tile.cuh"

namespace paralia {

int sm_count_of(int dev) {
  static int cached[PARALIA_MAX_UNITS] = {};
  if (dev < 0 || dev >= PARALIA_MAX_UNITS) return 148;
  if (!cached[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = 148;
    }
    cached[dev] = n;
  }
  return cached[dev];
}

int exec_tile_sgemm(int dev, void* stream, char TransA, char TransB, int64_t M, int64_t N,
                    int64_t K, float alpha, const float* A, int64_t ldA, const float* B,
                    int64_t ldB, float beta, float* C, int64_t ldC) {
  auto is_t = [](char t) { return t == 'T' || t == 't' || t == 'C' || t == 'c'; };
  auto ok_t = [&](char t) { return is_t(t) || t == 'N' || t == 'n'; };
  if (!ok_t(TransA) || !ok_t(TransB)) return fail(PARALIA_ERR_INVALID_ARG, "transpose flag is not N or T");
  if (M < 0 || N < 0 || K < 0 || M > INT32_MAX || N > INT32_MAX || K > INT32_MAX)
    return fail(PARALIA_ERR_INVALID_ARG, "dimension out of range");
  if (M == 0 || N == 0) return PARALIA_OK;
  const bool ta = is_t(TransA), tb = is_t(TransB);
  const int64_t a_rows = ta ? K : M, b_rows = tb ? N : K;
  if (ldA < std::max<int64_t>(1, a_rows) || ldB < std::max<int64_t>(1, b_rows) ||
      ldC < std::max<int64_t>(1, M))
    return fail(PARALIA_ERR_INVALID_ARG, "leading dimension smaller than the stored row count");
  Runtime& rt = Runtime::get();
  PL_TRY(rt.init());
  DeviceGuard guard;
  PL_TRY(rt.ensure_device(dev));
  PL_CUDA(cudaSetDevice(dev));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  SgemmArgs args;
  memset(&args, 0, sizeof(args));
  args.C = C;
  args.ldc = ldC;
  args.alpha = alpha;
  args.beta_c = beta;
  args.M = (int32_t)M;
  args.N = (int32_t)N;
  args.status = rt.dev(dev).status_dev;
  void *pa = nullptr, *pb = nullptr;
  if (K > 0) {
    // A stored M x K (k runs across columns) unless transposed; B stored K x N (k
    // contiguous) unless transposed.
    PL_CUDA(cudaMallocAsync(&pa, sgemm_packed_bytes(M, K, SG_BM), s));
    PL_CUDA(cudaMallocAsync(&pb, sgemm_packed_bytes(N, K, SG_BN), s));
    PL_CUDA(launch_sgemm_pack(A, ldA, ta, (int)M, (int)K, SG_BM, pa, s));
    PL_CUDA(launch_sgemm_pack(B, ldB, !tb, (int)N, (int)K, SG_BN, pb, s));
    args.nparts = 1;
    args.parts[0].a_packed = pa;
    args.parts[0].b_packed = pb;
    args.parts[0].klen = (int32_t)K;
  }
  PL_CUDA(launch_sgemm_tile(args, sm_count_of(dev), s));
  if (pa) PL_CUDA(cudaFreeAsync(pa, s));
  if (pb) PL_CUDA(cudaFreeAsync(pb, s));
  return PARALIA_OK;
}

}  // namespace paralia
