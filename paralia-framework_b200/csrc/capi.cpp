// extern "C" layer of libparalia.so: every symbol declared in include/paralia_c.h.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <string>
#include <vector>

#include "autotune.hpp"
#include "dgemm_tile.cuh"
#include "exec.hpp"
#include "group.hpp"
#include "level1.cuh"
#include "level2.cuh"
#include "paralia_rng.h"
#include "plan.hpp"
#include "runtime.hpp"
#include "sgemm_tile.cuh"

using namespace paralia;

namespace {

int norm_t(char t) { return (t == 'T' || t == 't' || t == 'C' || t == 'c') ? 1 : 0; }
bool valid_t(char t) {
  return t == 'N' || t == 'n' || t == 'T' || t == 't' || t == 'C' || t == 'c';
}

int setup_device(int dev) {
  Runtime& rt = Runtime::get();
  PL_TRY(rt.init());
  PL_TRY(rt.ensure_device(dev));
  PL_CUDA(cudaSetDevice(dev));
  return PARALIA_OK;
}

template <typename F>
void parallel_fill(int64_t n, F f) {
  unsigned hw = std::thread::hardware_concurrency();
  int nt = (int)std::min<int64_t>(hw ? hw : 1, std::max<int64_t>(1, n / (1 << 16)));
  if (nt <= 1) { f(0, n); return; }
  std::vector<std::thread> th;
  const int64_t chunk = (n + nt - 1) / nt;
  for (int t = 0; t < nt; ++t) {
    const int64_t lo = t * chunk, hi = std::min<int64_t>(n, lo + chunk);
    if (lo >= hi) break;
    th.emplace_back([=] { f(lo, hi); });
  }
  for (auto& t : th) t.join();
}

}  // namespace

extern "C" {

int PARALiA_init(void) { return Runtime::get().init(); }
int PARALiA_finalize(void) { return Runtime::get().finalize(); }
int PARALiA_device_count(void) {
  Runtime& rt = Runtime::get();
  if (rt.init() != PARALIA_OK) return 0;
  return rt.device_count();
}
const char* PARALiA_last_error(void) { return last_error_cstr(); }

int PARALiA_dev_cache_free(int loc) {
  Runtime& rt = Runtime::get();
  PL_TRY(rt.init());
  std::lock_guard<std::mutex> lk(rt.call_mutex());
  DeviceGuard guard;
  if (loc == -1) return PARALIA_OK;  // the host keeps no cache in this build
  return rt.free_slab(loc);
}

int PARALiA_dgemm(char TransA, char TransB, int64_t M, int64_t N, int64_t K, double alpha,
                  const double* A, int64_t ldA, int locA, const double* B, int64_t ldB, int locB,
                  double beta, double* C, int64_t ldC, int locC, const paralia_ctl* ctl,
                  paralia_report* out) {
  return exec_dgemm(TransA, TransB, M, N, K, alpha, A, ldA, locA, B, ldB, locB, beta, C, ldC, locC,
                    ctl, out);
}

int PARALiA_sgemm(char TransA, char TransB, int64_t M, int64_t N, int64_t K, float alpha,
                  const float* A, int64_t ldA, int locA, const float* B, int64_t ldB, int locB,
                  float beta, float* C, int64_t ldC, int locC, const paralia_ctl* ctl,
                  paralia_report* out) {
  return exec_sgemm(TransA, TransB, M, N, K, alpha, A, ldA, locA, B, ldB, locB, beta, C, ldC, locC,
                    ctl, out);
}

int PARALiA_dgemv(char TransA, int64_t M, int64_t N, double alpha, const double* A, int64_t ldA,
                  int locA, const double* x, int64_t incx, int locx, double beta, double* y,
                  int64_t incy, int locy, const paralia_ctl* ctl, paralia_report* out) {
  return exec_dgemv(TransA, M, N, alpha, A, ldA, locA, x, incx, locx, beta, y, incy, locy, ctl, out);
}

int PARALiA_daxpy(int64_t N, double alpha, const double* x, int64_t incx, int locx, double* y,
                  int64_t incy, int locy, const paralia_ctl* ctl, paralia_report* out) {
  return exec_daxpy(N, alpha, x, incx, locx, y, incy, locy, ctl, out);
}

int PARALiA_ddot(int64_t N, const double* x, int64_t incx, int locx, const double* y, int64_t incy,
                 int locy, double* result, const paralia_ctl* ctl, paralia_report* out) {
  return exec_ddot(N, x, incx, locx, y, incy, locy, result, ctl, out);
}

int PARALiA_ddot_tiles(int64_t N, const double* x, int64_t incx, int locx, const double* y,
                       int64_t incy, int locy, double* tile_sums, int64_t capacity, int64_t* count,
                       const paralia_ctl* ctl, paralia_report* out) {
  return exec_ddot_tiles(N, x, incx, locx, y, incy, locy, tile_sums, capacity, count, ctl, out);
}

int PARALiA_group_init(const char* name, int rank, int world, int dev) {
  return Group::init(name, rank, world, dev);
}
int PARALiA_group_finalize(void) { return Group::finalize(); }

int PARALiA_group_dgemm(char TransA, char TransB, int64_t Mloc, int64_t Nloc, int64_t K,
                        double alpha, const double* A, int64_t ldA, int locA, const double* B,
                        int64_t ldB, int locB, double beta, double* C, int64_t ldC, int locC,
                        const paralia_ctl* ctl, paralia_report* out) {
  return exec_group_dgemm(TransA, TransB, Mloc, Nloc, K, alpha, A, ldA, locA, B, ldB, locB, beta,
                          C, ldC, locC, ctl, out);
}

// ------------------------------ per-tile kernels ------------------------------

// `lone`: the launch has the GPU to itself (a caller's per-tile call); the calibration
// benchmark passes 0 when it keeps several launches in flight, as the executor does.
static int tile_dgemm_launch(int dev, void* stream, char TransA, char TransB, int64_t M, int64_t N,
                             int64_t K, double alpha, const double* A, int64_t ldA, const double* B,
                             int64_t ldB, double beta, double* C, int64_t ldC, int lone) {
  if (!valid_t(TransA) || !valid_t(TransB))
    return fail(PARALIA_ERR_INVALID_ARG, "transpose flag is not N or T");
  if (M < 0 || N < 0 || K < 0 || M > INT32_MAX || N > INT32_MAX || K > INT32_MAX)
    return fail(PARALIA_ERR_INVALID_ARG, "dimension out of range");
  if (M == 0 || N == 0) return PARALIA_OK;
  const int ta = norm_t(TransA), tb = norm_t(TransB);
  const int64_t a_rows = ta ? K : M, a_cols = ta ? M : K, b_rows = tb ? N : K, b_cols = tb ? K : N;
  if (ldA < std::max<int64_t>(1, a_rows) || ldB < std::max<int64_t>(1, b_rows) ||
      ldC < std::max<int64_t>(1, M))
    return fail(PARALIA_ERR_INVALID_ARG, "leading dimension smaller than the stored row count");
  DeviceGuard guard;
  PL_TRY(setup_device(dev));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool tma = K > 0 && tma_addressable(A, ldA, 8) && tma_addressable(B, ldB, 8);
  if (!tma) {
    PL_CUDA(launch_dgemm_generic(ta ? 'T' : 'N', tb ? 'T' : 'N', (int)M, (int)N, (int)K, alpha, A,
                                 ldA, B, ldB, beta, C, ldC, s));
    return PARALIA_OK;
  }
  CUtensorMap mapA, mapB;
  PL_TRY(make_tensor_map(&mapA, A, 8, a_rows, a_cols, 1, ldA * 8, (uint64_t)ldA * a_cols * 8, 16,
                         ta ? DG_KC_BOX_ROWS : 16));
  PL_TRY(make_tensor_map(&mapB, B, 8, b_rows, b_cols, 1, ldB * 8, (uint64_t)ldB * b_cols * 8, 16,
                         tb ? 16 : DG_KC_BOX_ROWS));
  DgemmArgs args;
  memset(&args, 0, sizeof(args));
  args.C = C;
  args.ldc = ldC;
  args.alpha = alpha;
  args.beta_c = beta;
  args.M = (int32_t)M;
  args.N = (int32_t)N;
  args.vec_ok = tma_addressable(C, ldC, 8) ? 1 : 0;
  args.status = Runtime::get().dev(dev).status_dev;
  args.nparts = 1;
  args.parts[0].klen = (int32_t)K;
  args.lone = lone;
  PL_CUDA(launch_dgemm_tile(mapA, mapB, args, ta != 0, tb == 0, s));
  return PARALIA_OK;
}

int PARALiA_tile_dgemm(int dev, void* stream, char TransA, char TransB, int64_t M, int64_t N,
                       int64_t K, double alpha, const double* A, int64_t ldA, const double* B,
                       int64_t ldB, double beta, double* C, int64_t ldC) {
  // a per-tile call: nothing of this library runs beside it
  return tile_dgemm_launch(dev, stream, TransA, TransB, M, N, K, alpha, A, ldA, B, ldB, beta, C, ldC, 1);
}

int PARALiA_tile_status(int dev) {
  Runtime& rt = Runtime::get();
  PL_TRY(rt.init());
  if (dev < 0 || dev >= rt.device_count()) return fail(PARALIA_ERR_INVALID_ARG, "GPU id %d out of range", dev);
  DeviceGuard guard;
  return rt.check_status(dev);
}

int PARALiA_tile_sgemm(int dev, void* stream, char TransA, char TransB, int64_t M, int64_t N,
                       int64_t K, float alpha, const float* A, int64_t ldA, const float* B,
                       int64_t ldB, float beta, float* C, int64_t ldC) {
  return exec_tile_sgemm(dev, stream, TransA, TransB, M, N, K, alpha, A, ldA, B, ldB, beta, C, ldC);
}

int PARALiA_tile_daxpy(int dev, void* stream, int64_t N, double alpha, const double* x,
                       int64_t incx, double* y, int64_t incy) {
  if (N < 0 || incx <= 0 || incy <= 0) return fail(PARALIA_ERR_INVALID_ARG, "bad N or increment");
  DeviceGuard guard;
  PL_TRY(setup_device(dev));
  PL_CUDA(launch_daxpy(N, alpha, x, incx, y, incy, static_cast<cudaStream_t>(stream), nullptr));
  return PARALIA_OK;
}

int64_t PARALiA_tile_ddot_scratch_bytes(int64_t N) {
  return (int64_t)l1_grid_blocks(N > 0 ? N : 1) * (int64_t)sizeof(double);
}

int PARALiA_tile_ddot(int dev, void* stream, int64_t N, const double* x, int64_t incx,
                      const double* y, int64_t incy, double* partials, double* result_dev) {
  if (N < 0 || incx <= 0 || incy <= 0) return fail(PARALIA_ERR_INVALID_ARG, "bad N or increment");
  if (!partials || !result_dev) return fail(PARALIA_ERR_INVALID_ARG, "NULL scratch or result");
  DeviceGuard guard;
  PL_TRY(setup_device(dev));
  PL_CUDA(launch_ddot(N, x, incx, y, incy, partials, result_dev, static_cast<cudaStream_t>(stream),
                      nullptr));
  return PARALIA_OK;
}

int64_t PARALiA_tile_dgemv_scratch_bytes(char TransA, int64_t M, int64_t N) {
  if (!valid_t(TransA) || M <= 0 || N <= 0 || M > INT32_MAX || N > INT32_MAX) return 0;
  if (norm_t(TransA)) return 0;
  return (int64_t)gemv_n_slices((int)M, (int)N) * M * (int64_t)sizeof(double);
}

int PARALiA_tile_dgemv(int dev, void* stream, char TransA, int64_t M, int64_t N, double alpha,
                       const double* A, int64_t ldA, const double* x, int64_t incx, double beta,
                       double* y, int64_t incy, double* scratch) {
  if (!valid_t(TransA)) return fail(PARALIA_ERR_INVALID_ARG, "transpose flag is not N or T");
  if (M < 0 || N < 0 || M > INT32_MAX || N > INT32_MAX)
    return fail(PARALIA_ERR_INVALID_ARG, "dimension out of range");
  if (incx <= 0 || incy <= 0) return fail(PARALIA_ERR_UNSUPPORTED, "non-positive increments are not supported");
  if (ldA < std::max<int64_t>(1, M))
    return fail(PARALIA_ERR_INVALID_ARG, "leading dimension smaller than the row count");
  const bool trans = norm_t(TransA) != 0;
  const int64_t out_len = trans ? N : M, in_len = trans ? M : N;
  if (out_len == 0) return PARALIA_OK;
  if (in_len == 0) return fail(PARALIA_ERR_UNSUPPORTED, "empty product: scale y with PARALiA_tile_daxpy");
  if (!A || !x || !y) return fail(PARALIA_ERR_INVALID_ARG, "NULL operand");
  if (!trans && !scratch) return fail(PARALIA_ERR_INVALID_ARG, "op = N needs scratch");
  DeviceGuard guard;
  PL_TRY(setup_device(dev));
  PL_CUDA(launch_dgemv_tile(trans, (int)M, (int)N, alpha, A, ldA, x, incx, beta, y, incy, scratch,
                            static_cast<cudaStream_t>(stream), nullptr));
  return PARALIA_OK;
}

// ------------------------------ memory and inputs ------------------------------

int PARALiA_malloc(void** ptr, int64_t bytes, int loc) {
  if (!ptr || bytes < 0) return fail(PARALIA_ERR_INVALID_ARG, "bad malloc arguments");
  *ptr = nullptr;
  if (bytes == 0) return PARALIA_OK;
  Runtime& rt = Runtime::get();
  PL_TRY(rt.init());
  DeviceGuard guard;
  if (loc == -1) {
    cudaError_t e = cudaHostAlloc(ptr, (size_t)bytes, cudaHostAllocPortable);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(PARALIA_ERR_OUT_OF_MEMORY, "pinned host allocation of %lld bytes failed: %s",
                  (long long)bytes, cudaGetErrorString(e));
    }
    return PARALIA_OK;
  }
  if (loc < 0 || loc >= rt.device_count())
    return fail(PARALIA_ERR_INVALID_ARG, "location id %d is not valid", loc);
  PL_CUDA(cudaSetDevice(loc));
  cudaError_t e = cudaMalloc(ptr, (size_t)bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(PARALIA_ERR_OUT_OF_MEMORY, "GPU %d allocation of %lld bytes failed: %s", loc,
                (long long)bytes, cudaGetErrorString(e));
  }
  return PARALIA_OK;
}

int PARALiA_free(void* ptr, int loc) {
  if (!ptr) return PARALIA_OK;
  DeviceGuard guard;
  if (loc == -1) PL_CUDA(cudaFreeHost(ptr));
  else {
    PL_CUDA(cudaSetDevice(loc));
    PL_CUDA(cudaFree(ptr));
  }
  return PARALIA_OK;
}

int PARALiA_memcpy(void* dst, int loc_dst, const void* src, int loc_src, int64_t bytes) {
  (void)loc_dst;
  (void)loc_src;
  if (bytes < 0) return fail(PARALIA_ERR_INVALID_ARG, "negative byte count");
  if (bytes == 0) return PARALIA_OK;
  PL_TRY(Runtime::get().init());
  PL_CUDA(cudaMemcpy(dst, src, (size_t)bytes, cudaMemcpyDefault));
  return PARALIA_OK;
}

int PARALiA_fill_f64(double* ptr, int64_t n, uint64_t seed, int dist, int loc) {
  if (n < 0 || (dist != 0 && dist != 1)) return fail(PARALIA_ERR_INVALID_ARG, "bad fill arguments");
  if (n == 0) return PARALIA_OK;
  if (loc == -1) {
    if (dist == 0)
      parallel_fill(n, [=](int64_t lo, int64_t hi) {
        for (int64_t i = lo; i < hi; ++i) ptr[i] = paralia_uniform_f64(seed, (uint64_t)i);
      });
    else
      parallel_fill(n, [=](int64_t lo, int64_t hi) {
        for (int64_t i = lo; i < hi; ++i) ptr[i] = paralia_normal_f64(seed, (uint64_t)i);
      });
    return PARALIA_OK;
  }
  DeviceGuard guard;
  PL_TRY(setup_device(loc));
  PL_CUDA(launch_fill_f64(ptr, n, seed, dist, nullptr));
  PL_CUDA(cudaDeviceSynchronize());
  return PARALIA_OK;
}

int PARALiA_fill_f32(float* ptr, int64_t n, uint64_t seed, int dist, int loc) {
  if (n < 0 || (dist != 0 && dist != 1)) return fail(PARALIA_ERR_INVALID_ARG, "bad fill arguments");
  if (n == 0) return PARALIA_OK;
  if (loc == -1) {
    if (dist == 0)
      parallel_fill(n, [=](int64_t lo, int64_t hi) {
        for (int64_t i = lo; i < hi; ++i) ptr[i] = paralia_uniform_f32(seed, (uint64_t)i);
      });
    else
      parallel_fill(n, [=](int64_t lo, int64_t hi) {
        for (int64_t i = lo; i < hi; ++i) ptr[i] = (float)paralia_normal_f64(seed, (uint64_t)i);
      });
    return PARALIA_OK;
  }
  DeviceGuard guard;
  PL_TRY(setup_device(loc));
  PL_CUDA(launch_fill_f32(ptr, n, seed, dist, nullptr));
  PL_CUDA(cudaDeviceSynchronize());
  return PARALIA_OK;
}

// ------------------------------ autotuner ------------------------------

int PARALiA_autotune_gemm(int elem_size, char TransA, char TransB, int64_t M, int64_t N, int64_t K,
                          int locA, int locB, int locC, const paralia_ctl* ctl,
                          paralia_report* out) {
  if (elem_size != 4 && elem_size != 8)
    return fail(PARALIA_ERR_INVALID_ARG, "element size must be 4 or 8");
  if (!valid_t(TransA) || !valid_t(TransB))
    return fail(PARALIA_ERR_INVALID_ARG, "transpose flag is not N or T");
  int ngpu = 0;
  if (!(ctl && ctl->active_unit_num > 0)) {
    Runtime& rt = Runtime::get();
    PL_TRY(rt.init());
    ngpu = rt.device_count();
  } else {
    // a fixed unit list needs no GPU: size the default link table from the list
    for (int i = 0; i < ctl->active_unit_num && i < PARALIA_MAX_UNITS; ++i)
      ngpu = std::max(ngpu, ctl->active_unit_id_list[i] + 1);
    ngpu = std::max(ngpu, std::max(locA, std::max(locB, locC)) + 1);
  }
  if (model_db().link.empty() || (int)model_db().link.size() < ngpu + 1)
    reset_database_defaults(ngpu);
  GemmModelInput in;
  in.esz = elem_size;
  in.ta = norm_t(TransA) ? 'T' : 'N';
  in.tb = norm_t(TransB) ? 'T' : 'N';
  in.M = M; in.N = N; in.K = K;
  in.locA = locA; in.locB = locB; in.locC = locC;
  in.func = elem_size == 8 ? "Dgemm" : "Sgemm";
  in.beta_nonzero = !(ctl && (ctl->flags & PARALIA_FLAG_BETA_ZERO));
  return autotune_gemm(in, ngpu, ctl, out);
}

int PARALiA_tile_slowdowns(int64_t M, int64_t N, int64_t K, int64_t T, int active_units,
                           double* slowdowns) {
  if (M <= 0 || N <= 0 || K <= 0 || T <= 0 || active_units <= 0 || !slowdowns)
    return fail(PARALIA_ERR_INVALID_ARG, "bad tile_slowdowns arguments");
  tile_slowdowns(M, N, K, T, active_units, tune_constants(), slowdowns);
  return PARALIA_OK;
}

int PARALiA_distribute_2d(int units, int Mt, int Nt, int Kt, int32_t* sk_unit, int32_t* d1,
                          int32_t* d2) {
  if (units <= 0 || Mt <= 0 || Nt <= 0 || Kt <= 0 || !sk_unit)
    return fail(PARALIA_ERR_INVALID_ARG, "bad distribute_2d arguments");
  std::vector<std::vector<int>> lists;
  int g1 = 1, g2 = 1;
  const int active = distribute_subkernels_2d(units, Mt, Nt, Kt, &lists, &g1, &g2);
  if (active < 0) return fail(PARALIA_ERR_INVALID_ARG, "distribution failed");
  for (int i = 0; i < Mt * Nt * Kt; ++i) sk_unit[i] = -1;
  for (int u = 0; u < active; ++u)
    for (int sk : lists[u]) sk_unit[sk] = u;
  if (d1) *d1 = g1;
  if (d2) *d2 = g2;
  return PARALIA_OK;
}

int PARALiA_plan_gemm(int64_t M, int64_t N, int64_t K, int64_t T, int units, int bounded_cache,
                      int32_t* items, int64_t capacity, int64_t* count, int32_t* d1, int32_t* d2) {
  if (M <= 0 || N <= 0 || K < 0 || T <= 0 || units <= 0 || !count || capacity < 0)
    return fail(PARALIA_ERR_INVALID_ARG, "bad plan_gemm arguments");
  const int64_t Mt = (M + T - 1) / T, Nt = (N + T - 1) / T, Kt = K > 0 ? (K + T - 1) / T : 0;
  if (Mt * Nt * std::max<int64_t>(Kt, 1) > INT32_MAX)
    return fail(PARALIA_ERR_INVALID_ARG, "too many subkernels");
  const int kt_for_ids = (int)std::max<int64_t>(Kt, 1);
  std::vector<std::vector<int>> lists, ctiles;
  std::vector<int> owner;
  int g1 = 1, g2 = 1;
  const int active = distribute_subkernels_2d(units, (int)Mt, (int)Nt, kt_for_ids, &lists, &g1, &g2);
  if (active <= 0) return fail(PARALIA_ERR_INVALID_ARG, "distribution failed");
  lists.resize(active);
  if (!plan_unit_ctiles(lists, kt_for_ids, (int)(Mt * Nt), &ctiles, &owner))
    return fail(PARALIA_ERR_UNSUPPORTED, "distribution split one C tile across units");
  std::vector<std::vector<LaunchItem>> per_unit(active);
  // band sizes as the executor derives them for FP64 operands that all live in host memory
  // (the streaming case), from the calibration database that is loaded now
  if (model_db().link.empty()) reset_database_defaults(std::max(units, 1));
  GemmModelInput mi;
  mi.esz = 8; mi.ta = 'N'; mi.tb = 'N';
  mi.M = M; mi.N = N; mi.K = std::max<int64_t>(K, 1);
  mi.locA = mi.locB = mi.locC = -1;
  mi.beta_nonzero = true;
  mi.func = "Dgemm";
  for (int u = 0; u < active; ++u) {
    int row_len = 0;
    for (int ct : ctiles[u]) {
      if (ct / Nt != ctiles[u][0] / Nt) break;
      ++row_len;
    }
    int a_sh = 0, b_sh = 0;   // units that own tiles of this unit's first tile row / column
    if (!ctiles[u].empty()) {
      std::vector<char> in_row(active, 0), in_col(active, 0);
      for (int64_t ct = 0; ct < Mt * Nt; ++ct) {
        if (ct / Nt == ctiles[u][0] / Nt) in_row[owner[ct]] = 1;
        if (ct % Nt == ctiles[u][0] % Nt) in_col[owner[ct]] = 1;
      }
      for (int v = 0; v < active; ++v) { a_sh += in_row[v]; b_sh += in_col[v]; }
    }
    const BandHints hints = band_hints(mi, T, u, active, std::max(a_sh, 1), std::max(b_sh, 1), row_len);
    std::vector<int> bands;
    plan_band_sizes((int)ctiles[u].size(), (int)Kt, bounded_cache != 0, hints, &bands);
    plan_launch_order(bands, (int)Kt, bounded_cache != 0, DG_MAX_PARTS, &per_unit[u]);
  }
  // the executor walks the units round-robin, one launch per turn
  int64_t n = 0;
  std::vector<size_t> cursor(active, 0);
  for (bool left = true; left;) {
    left = false;
    for (int u = 0; u < active; ++u) {
      if (cursor[u] >= per_unit[u].size()) continue;
      const LaunchItem it = per_unit[u][cursor[u]++];
      if (items && n < capacity) {
        const int ct = ctiles[u][it.order_idx];
        int32_t* o = items + 5 * n;
        o[0] = u; o[1] = (int32_t)(ct / Nt); o[2] = (int32_t)(ct % Nt); o[3] = it.ki0; o[4] = it.ki1;
      }
      ++n;
      if (cursor[u] < per_unit[u].size()) left = true;
    }
  }
  *count = n;
  if (d1) *d1 = g1;
  if (d2) *d2 = g2;
  return PARALIA_OK;
}

int PARALiA_load_database(const char* dir) {
  if (model_db().link.empty()) {
    int n = 8;
    Runtime& rt = Runtime::get();
    if (rt.init() == PARALIA_OK) n = rt.device_count();
    reset_database_defaults(n);
  }
  return load_database(dir);
}

// Failure-detection self test: a kernel waits (bounded) for a signal that never comes.
// Returns PARALIA_ERR_TIMEOUT when the give-up path worked, i.e. the kernel ended by
// itself and reported through the device status word; the context stays usable.
int PARALiA_selftest_bounded_wait(int dev, double budget_ms) {
  if (!(budget_ms > 0.0) || budget_ms > 1000.0)
    return fail(PARALIA_ERR_INVALID_ARG, "budget must be in (0, 1000] ms");
  DeviceGuard guard;
  PL_TRY(setup_device(dev));
  int khz = 0;
  PL_CUDA(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev));
  const long long clocks = (long long)(budget_ms * (double)khz);
  PL_CUDA(launch_bounded_wait_selftest(Runtime::get().dev(dev).status_dev, clocks, nullptr));
  PL_CUDA(cudaDeviceSynchronize());
  return Runtime::get().check_status(dev);
}

// The host join of the whole-problem routines waits for a GPU's end event with a deadline. A
// kernel whose only wait runs out by itself after kernel_ms is queued and the join is given
// deadline_ms < kernel_ms: it must come back with PARALIA_ERR_TIMEOUT instead of blocking.
// The kernel then ends on its own, the status word is cleared and the context stays usable.
int PARALiA_selftest_join_deadline(int dev, double kernel_ms, double deadline_ms) {
  if (!(kernel_ms > 0.0) || kernel_ms > 1000.0 || !(deadline_ms > 0.0))
    return fail(PARALIA_ERR_INVALID_ARG, "kernel_ms must be in (0, 1000], deadline_ms positive");
  DeviceGuard guard;
  PL_TRY(setup_device(dev));
  DeviceCtx& dc = Runtime::get().dev(dev);
  int khz = 0;
  PL_CUDA(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev));
  const long long clocks = (long long)(kernel_ms * (double)khz);
  PL_CUDA(launch_bounded_wait_selftest(dc.status_dev, clocks, dc.exec[0]));
  PL_CUDA(cudaEventRecord(dc.t_end, dc.exec[0]));
  const int rc = wait_event_with_deadline(dc.t_end, deadline_ms, dev);
  std::string msg = rc != PARALIA_OK ? PARALiA_last_error() : "";
  PL_CUDA(cudaStreamSynchronize(dc.exec[0]));   // the kernel gives up by itself
  Runtime::get().check_status(dev);             // reads and clears the kernel's time-out word
  if (rc != PARALIA_OK) return fail(rc, "%s", msg.c_str());
  return PARALIA_OK;
}

int PARALiA_selftest_group_rendezvous(const char* name, int rank, int world, int rounds,
                                      int fail_rank, int fail_round, int fail_mode,
                                      double* waited_ms) {
  if (rounds < 0 || fail_mode < 0 || fail_mode > 2)
    return fail(PARALIA_ERR_INVALID_ARG, "bad self-test arguments");
  return Group::selftest_rendezvous(name, rank, world, rounds, fail_mode ? fail_rank : -1, fail_round,
                                    fail_mode, waited_ms);
}

int PARALiA_group_sgemm(char TransA, char TransB, int64_t Mloc, int64_t Nloc, int64_t K,
                        float alpha, const float* A, int64_t ldA, int locA, const float* B,
                        int64_t ldB, int locB, float beta, float* C, int64_t ldC, int locC,
                        const paralia_ctl* ctl, paralia_report* out) {
  return exec_group_sgemm(TransA, TransB, Mloc, Nloc, K, alpha, A, ldA, locA, B, ldB, locB, beta,
                          C, ldC, locC, ctl, out);
}

// ------------------------------ calibration ------------------------------

int PARALiA_bench_dmma_peak(int dev, int shape, int iters, double* tflops) {
  if (!tflops || iters <= 0) return fail(PARALIA_ERR_INVALID_ARG, "bad bench arguments");
  DeviceGuard guard;
  PL_TRY(setup_device(dev));
  int sms = 0;
  PL_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int blocks = sms * 2;  // 2 x 256 threads per SM: four warps per scheduler
  double* sink = nullptr;
  PL_CUDA(cudaMalloc(&sink, sizeof(double)));
  cudaEvent_t e0, e1;
  PL_CUDA(cudaEventCreate(&e0));
  PL_CUDA(cudaEventCreate(&e1));
  PL_CUDA(launch_dmma_peak(shape, iters / 4 + 1, blocks, sink, nullptr));  // warm-up
  PL_CUDA(cudaEventRecord(e0, nullptr));
  PL_CUDA(launch_dmma_peak(shape, iters, blocks, sink, nullptr));
  PL_CUDA(cudaEventRecord(e1, nullptr));
  PL_CUDA(cudaEventSynchronize(e1));
  float ms = 0.f;
  PL_CUDA(cudaEventElapsedTime(&ms, e0, e1));
  double flop_per_mma = 0;
  switch (shape) {
    case 884: flop_per_mma = 2.0 * 8 * 8 * 4; break;
    case 1684: flop_per_mma = 2.0 * 16 * 8 * 4; break;
    case 1688: flop_per_mma = 2.0 * 16 * 8 * 8; break;
    case 16816: flop_per_mma = 2.0 * 16 * 8 * 16; break;
  }
  const double total = flop_per_mma * 8.0 /*chains*/ * (double)iters * 8.0 /*warps*/ * blocks;
  *tflops = total / (ms * 1e-3) / 1e12;
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(sink);
  return PARALIA_OK;
}

int PARALiA_bench_tile_dgemm(int dev, char TransA, char TransB, int64_t T, int reps,
                             double* mean_s) {
  return PARALiA_bench_tile_dgemm_chain(dev, TransA, TransB, T, 1, reps, mean_s);
}

int PARALiA_bench_tile_dgemm_chain(int dev, char TransA, char TransB, int64_t T, int chain,
                                   int reps, double* mean_s) {
  // The tile time the model needs is the one the executor sees: tiles of different C
  // accumulators run on several exec streams at once, so the partial last wave of one tile
  // is filled by the next. `reps` tiles are therefore spread round-robin over up to four
  // streams (one C per stream) and the mean is total time / reps; reps = 1 times one tile
  // alone, as the reference's microbenchmark does (dgemm_microbench.cu:125-187).
  // A launch of the executor usually covers a chain of k tiles of one C tile (four after the
  // first): `chain` makes each timed launch T x T x (chain*T) and the result is the time
  // per k tile, i.e. per T x T x T subkernel, inside such a launch.
  if (!mean_s || reps <= 0 || T <= 0 || chain <= 0 || chain > 16)
    return fail(PARALIA_ERR_INVALID_ARG, "bad bench arguments");
  const int64_t Kc = T * chain;
  DeviceGuard guard;
  PL_TRY(setup_device(dev));
  DeviceCtx& dc = Runtime::get().dev(dev);
  const int S = std::min(reps, 4);
  const size_t n = (size_t)T * T;
  double *A = nullptr, *B = nullptr, *C = nullptr;
  PL_CUDA(cudaMalloc(&A, n * 8 * chain));
  PL_CUDA(cudaMalloc(&B, n * 8 * chain));
  PL_CUDA(cudaMalloc(&C, n * 8 * S));
  PL_CUDA(launch_fill_f64(A, n * chain, 42, 0, nullptr));
  PL_CUDA(launch_fill_f64(B, n * chain, 43, 0, nullptr));
  PL_CUDA(launch_fill_f64(C, n * S, 44, 0, nullptr));
  PL_CUDA(cudaDeviceSynchronize());
  cudaEvent_t e0, e1, join[4] = {nullptr, nullptr, nullptr, nullptr};
  PL_CUDA(cudaEventCreate(&e0));
  PL_CUDA(cudaEventCreate(&e1));
  for (int s = 1; s < S; ++s) PL_CUDA(cudaEventCreateWithFlags(&join[s], cudaEventDisableTiming));
  int rc = PARALIA_OK;
  const int64_t lda = norm_t(TransA) ? Kc : T, ldb = norm_t(TransB) ? T : Kc;
  for (int i = 0; i < 2 && rc == PARALIA_OK; ++i)
    rc = tile_dgemm_launch(dev, dc.exec[0], TransA, TransB, T, T, Kc, 1.0, A, lda, B, ldb, 0.5, C, T,
                           reps == 1);
  if (rc == PARALIA_OK) {
    PL_CUDA(cudaSetDevice(dev));
    PL_CUDA(cudaDeviceSynchronize());
    PL_CUDA(cudaEventRecord(e0, dc.exec[0]));
    for (int s = 1; s < S; ++s) PL_CUDA(cudaStreamWaitEvent(dc.exec[s], e0, 0));
    for (int i = 0; i < reps && rc == PARALIA_OK; ++i)
      rc = tile_dgemm_launch(dev, dc.exec[i % S], TransA, TransB, T, T, Kc, 1.0, A, lda, B, ldb, 0.5,
                             C + (size_t)(i % S) * n, T, reps == 1);
    PL_CUDA(cudaSetDevice(dev));
    for (int s = 1; s < S; ++s) {
      PL_CUDA(cudaEventRecord(join[s], dc.exec[s]));
      PL_CUDA(cudaStreamWaitEvent(dc.exec[0], join[s], 0));
    }
    PL_CUDA(cudaEventRecord(e1, dc.exec[0]));
    PL_CUDA(cudaEventSynchronize(e1));
    float ms = 0.f;
    PL_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    *mean_s = ms * 1e-3 / reps / chain;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  for (int s = 1; s < S; ++s) cudaEventDestroy(join[s]);
  cudaFree(A);
  cudaFree(B);
  cudaFree(C);
  if (rc == PARALIA_OK) rc = Runtime::get().check_status(dev);
  return rc;
}

int PARALiA_bench_tile_sgemm(int dev, int64_t T, int reps, double* mean_s) {
  if (!mean_s || reps <= 0 || T <= 0 || T > 32768) return fail(PARALIA_ERR_INVALID_ARG, "bad bench arguments");
  DeviceGuard guard;
  PL_TRY(setup_device(dev));
  const size_t n = (size_t)T * T;
  float *A = nullptr, *B = nullptr, *C = nullptr;
  void *pa = nullptr, *pb = nullptr;
  PL_CUDA(cudaMalloc(&A, n * 4));
  PL_CUDA(cudaMalloc(&B, n * 4));
  PL_CUDA(cudaMalloc(&C, n * 4));
  PL_CUDA(cudaMalloc(&pa, sgemm_packed_bytes(T, T, SG_BM)));
  PL_CUDA(cudaMalloc(&pb, sgemm_packed_bytes(T, T, SG_BN)));
  PL_CUDA(launch_fill_f32(A, n, 42, 1, nullptr));
  PL_CUDA(launch_fill_f32(B, n, 43, 1, nullptr));
  PL_CUDA(cudaMemset(C, 0, n * 4));
  PL_CUDA(launch_sgemm_pack(A, T, false, (int)T, (int)T, SG_BM, pa, nullptr));
  PL_CUDA(launch_sgemm_pack(B, T, true, (int)T, (int)T, SG_BN, pb, nullptr));
  SgemmArgs args;
  memset(&args, 0, sizeof(args));
  args.C = C; args.ldc = T; args.alpha = 1.0f; args.beta_c = 0.5f;
  args.M = (int32_t)T; args.N = (int32_t)T;
  args.status = Runtime::get().dev(dev).status_dev;
  args.nparts = 1;
  args.parts[0].a_packed = pa; args.parts[0].b_packed = pb; args.parts[0].klen = (int32_t)T;
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaEvent_t e0, e1;
  PL_CUDA(cudaEventCreate(&e0));
  PL_CUDA(cudaEventCreate(&e1));
  for (int i = 0; i < 2; ++i) PL_CUDA(launch_sgemm_tile(args, sms, nullptr));
  PL_CUDA(cudaEventRecord(e0, nullptr));
  for (int i = 0; i < reps; ++i) PL_CUDA(launch_sgemm_tile(args, sms, nullptr));
  PL_CUDA(cudaEventRecord(e1, nullptr));
  PL_CUDA(cudaEventSynchronize(e1));
  float ms = 0.f;
  PL_CUDA(cudaEventElapsedTime(&ms, e0, e1));
  *mean_s = ms * 1e-3 / reps;
  cudaEventDestroy(e0); cudaEventDestroy(e1);
  cudaFree(A); cudaFree(B); cudaFree(C); cudaFree(pa); cudaFree(pb);
  return Runtime::get().check_status(dev);
}

int PARALiA_bench_link(int dst_loc, int src_loc, int64_t dim, int reps, double* mean_s) {
  if (!mean_s || reps <= 0 || dim <= 0) return fail(PARALIA_ERR_INVALID_ARG, "bad bench arguments");
  Runtime& rt = Runtime::get();
  PL_TRY(rt.init());
  if (dst_loc == src_loc) return fail(PARALIA_ERR_INVALID_ARG, "source and destination are the same");
  DeviceGuard guard;
  // A dim x dim tile cut out of a (dim+64)-row matrix: the strided 2-D copy the scheduler issues.
  const int64_t ld = dim + 64;
  const int64_t bytes = ld * dim * 8;
  void *src = nullptr, *dst = nullptr;
  PL_TRY(PARALiA_malloc(&src, bytes, src_loc));
  int rc = PARALiA_malloc(&dst, bytes, dst_loc);
  if (rc != PARALIA_OK) { PARALiA_free(src, src_loc); return rc; }
  const int drive = dst_loc >= 0 ? dst_loc : src_loc;
  rc = rt.ensure_device(drive);
  if (rc == PARALIA_OK && dst_loc >= 0 && src_loc >= 0) rc = rt.ensure_device(src_loc);  // peer access
  if (rc == PARALIA_OK) {
    cudaSetDevice(drive);
    cudaStream_t s = dst_loc >= 0 ? (src_loc >= 0 ? rt.dev(drive).p2p : rt.dev(drive).h2d)
                                  : rt.dev(drive).d2h;
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    cudaMemcpy2DAsync(dst, ld * 8, src, ld * 8, dim * 8, dim, cudaMemcpyDefault, s);  // warm-up
    cudaEventRecord(e0, s);
    for (int i = 0; i < reps; ++i)
      cudaMemcpy2DAsync(dst, ld * 8, src, ld * 8, dim * 8, dim, cudaMemcpyDefault, s);
    cudaEventRecord(e1, s);
    cudaError_t e = cudaEventSynchronize(e1);
    float ms = 0.f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
    if (e != cudaSuccess) rc = fail(PARALIA_ERR_CUDA, "link benchmark failed: %s", cudaGetErrorString(e));
    else *mean_s = ms * 1e-3 / reps;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
  }
  PARALiA_free(src, src_loc);
  PARALiA_free(dst, dst_loc);
  return rc;
}

// Time a dim x dim tile copy on link (dst <- src) alone and while `background` copies of
// the same size keep link (odst <- osrc) busy: the reference's link-sharing measurement
// (Database_builder/CuCuBLAS/src/transfer_link_microbench.cu:186-218).
int PARALiA_bench_link_overlap(int dst_loc, int src_loc, int odst_loc, int osrc_loc, int64_t dim,
                               int reps, double* t_alone, double* t_shared) {
  if (!t_alone || !t_shared || reps <= 0 || dim <= 0)
    return fail(PARALIA_ERR_INVALID_ARG, "bad bench arguments");
  if (dst_loc == src_loc || odst_loc == osrc_loc)
    return fail(PARALIA_ERR_INVALID_ARG, "source and destination are the same");
  Runtime& rt = Runtime::get();
  PL_TRY(rt.init());
  DeviceGuard guard;
  const int64_t bytes = dim * dim * 8;
  void *s1 = nullptr, *d1 = nullptr, *s2 = nullptr, *d2 = nullptr;
  int rc = PARALiA_malloc(&s1, bytes, src_loc);
  if (rc == PARALIA_OK) rc = PARALiA_malloc(&d1, bytes, dst_loc);
  if (rc == PARALIA_OK) rc = PARALiA_malloc(&s2, bytes, osrc_loc);
  if (rc == PARALIA_OK) rc = PARALiA_malloc(&d2, bytes, odst_loc);
  const int drv1 = dst_loc >= 0 ? dst_loc : src_loc, drv2 = odst_loc >= 0 ? odst_loc : osrc_loc;
  for (int l : {dst_loc, src_loc, odst_loc, osrc_loc})
    if (rc == PARALIA_OK && l >= 0) rc = rt.ensure_device(l);
  if (rc == PARALIA_OK) {
    auto pick = [&](int dst, int src, int drv) {
      DeviceCtx& c = rt.dev(drv);
      return dst >= 0 ? (src >= 0 ? c.p2p : c.h2d) : c.d2h;
    };
    cudaStream_t q1 = pick(dst_loc, src_loc, drv1), q2 = pick(odst_loc, osrc_loc, drv2);
    if (q1 == q2) q2 = rt.dev(drv2).exec[0];
    cudaEvent_t e0, e1;
    cudaSetDevice(drv1);
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    auto timed = [&](bool with_bg, double* out) {
      cudaSetDevice(drv1);
      cudaMemcpyAsync(d1, s1, bytes, cudaMemcpyDefault, q1);   // warm-up
      cudaStreamSynchronize(q1);
      if (with_bg) {
        cudaSetDevice(drv2);
        for (int i = 0; i < 10 * reps; ++i) cudaMemcpyAsync(d2, s2, bytes, cudaMemcpyDefault, q2);
      }
      cudaSetDevice(drv1);
      cudaEventRecord(e0, q1);
      for (int i = 0; i < reps; ++i) cudaMemcpyAsync(d1, s1, bytes, cudaMemcpyDefault, q1);
      cudaEventRecord(e1, q1);
      cudaEventSynchronize(e1);
      float ms = 0.f;
      cudaEventElapsedTime(&ms, e0, e1);
      *out = ms * 1e-3 / reps;
      cudaSetDevice(drv2);
      cudaStreamSynchronize(q2);
    };
    timed(false, t_alone);
    timed(true, t_shared);
    cudaSetDevice(drv1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (cudaGetLastError() != cudaSuccess) rc = fail(PARALIA_ERR_CUDA, "link overlap benchmark failed");
  }
  if (s1) PARALiA_free(s1, src_loc);
  if (d1) PARALiA_free(d1, dst_loc);
  if (s2) PARALiA_free(s2, osrc_loc);
  if (d2) PARALiA_free(d2, odst_loc);
  return rc;
}

}  // extern "C"
