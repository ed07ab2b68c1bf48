// Calibration microbenchmarks of the level-1 kernels and of the shared host link, and the
// model introspection entry points that go with them.
//
// Reference: Database_builder/CuCuBLAS/src/daxpy_microbench.cu:26-231 and
// ddot_microbench.cu:26-228 (time one device-resident vector tile per length),
// dgemv_microbench.cu:127-190 (one square matrix-vector tile per edge),
// transfer_link_microbench.cu:186-218 (a link while another link is busy). The aggregate
// measurement has no counterpart there: it times all host links of n GPUs at once, which is
// what shows the cap of this class of host (root complex / host memory) that pairwise
// probes cannot see.
#include <algorithm>
#include <cstring>
#include <vector>

#include "autotune.hpp"
#include "level1.cuh"
#include "level2.cuh"
#include "runtime.hpp"
#include "sgemm_tile.cuh"

namespace paralia {
namespace {

int bench_level1(bool is_dot, int dev, int64_t N, int reps, double* mean_s) {
  if (!mean_s || reps <= 0 || N <= 0) return fail(PARALIA_ERR_INVALID_ARG, "bad bench arguments");
  Runtime& rt = Runtime::get();
  PL_TRY(rt.init());
  DeviceGuard guard;
  PL_TRY(rt.ensure_device(dev));
  PL_CUDA(cudaSetDevice(dev));
  DeviceCtx& dc = rt.dev(dev);
  cudaStream_t s = dc.exec[0];
  // Tiles arrive in a ring of slots in the executor; rotate through enough distinct slots
  // that a tile is not served from L2 just because the previous repetition left it there.
  const size_t bytes = (size_t)N * 8;
  const int slots = (int)std::max<size_t>(2, std::min<size_t>(16, ((size_t)192 << 20) / bytes + 1));
  double *x = nullptr, *y = nullptr, *partials = nullptr, *result = nullptr;
  PL_CUDA(cudaMalloc(&x, bytes * slots));
  cudaError_t e = cudaMalloc(&y, bytes * slots);
  if (e == cudaSuccess) e = cudaMalloc(&partials, sizeof(double) * (size_t)l1_grid_blocks(N));
  if (e == cudaSuccess) e = cudaMalloc(&result, sizeof(double));
  int rc = PARALIA_OK;
  if (e != cudaSuccess) rc = fail(PARALIA_ERR_OUT_OF_MEMORY, "bench buffers: %s", cudaGetErrorString(e));
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if (rc == PARALIA_OK) {
    launch_fill_f64(x, N * slots, 42, 0, s);
    launch_fill_f64(y, N * slots, 43, 0, s);
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    auto one = [&](int i) {
      double* xs = x + (size_t)(i % slots) * N;
      double* ys = y + (size_t)(i % slots) * N;
      return is_dot ? launch_ddot(N, xs, 1, ys, 1, partials, result, s, nullptr)
                    : launch_daxpy(N, -0.5, xs, 1, ys, 1, s, nullptr);
    };
    for (int i = 0; i < 2 && e == cudaSuccess; ++i) e = one(i);
    cudaEventRecord(e0, s);
    for (int i = 0; i < reps && e == cudaSuccess; ++i) e = one(i + 2);
    cudaEventRecord(e1, s);
    if (e == cudaSuccess) e = cudaEventSynchronize(e1);
    float ms = 0.f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
    if (e != cudaSuccess) rc = fail(PARALIA_ERR_CUDA, "level-1 benchmark failed: %s", cudaGetErrorString(e));
    else *mean_s = ms * 1e-3 / reps;
  }
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  cudaFree(x);
  cudaFree(y);
  cudaFree(partials);
  cudaFree(result);
  cudaGetLastError();
  return rc;
}

// One square T x T matrix-vector tile on device-resident operands, as the reference's
// Database_builder/CuCuBLAS/src/dgemv_microbench.cu:127-190 times cublasDgemv.
int bench_level2(bool trans, int dev, int64_t T, int reps, double* mean_s) {
  if (!mean_s || reps <= 0 || T <= 0 || T > (1 << 17))
    return fail(PARALIA_ERR_INVALID_ARG, "bad bench arguments");
  Runtime& rt = Runtime::get();
  PL_TRY(rt.init());
  DeviceGuard guard;
  PL_TRY(rt.ensure_device(dev));
  PL_CUDA(cudaSetDevice(dev));
  DeviceCtx& dc = rt.dev(dev);
  cudaStream_t s = dc.exec[0];
  // rotate through enough copies of the matrix that a tile is never served from L2
  const size_t bytes = (size_t)T * T * 8;
  const int slots = (int)std::max<size_t>(2, std::min<size_t>(16, ((size_t)192 << 20) / bytes + 1));
  const int slices = trans ? 0 : gemv_n_slices((int)T, (int)T);
  double *a = nullptr, *x = nullptr, *y = nullptr, *partial = nullptr;
  cudaError_t e = cudaMalloc(&a, bytes * slots);
  if (e == cudaSuccess) e = cudaMalloc(&x, (size_t)T * 8);
  if (e == cudaSuccess) e = cudaMalloc(&y, (size_t)T * 8);
  if (e == cudaSuccess && slices > 0) e = cudaMalloc(&partial, (size_t)slices * T * 8);
  int rc = PARALIA_OK;
  if (e != cudaSuccess) rc = fail(PARALIA_ERR_OUT_OF_MEMORY, "bench buffers: %s", cudaGetErrorString(e));
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if (rc == PARALIA_OK) {
    launch_fill_f64(a, (int64_t)T * T * slots, 42, 0, s);
    launch_fill_f64(x, T, 43, 0, s);
    launch_fill_f64(y, T, 44, 0, s);
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    int launches = 0;
    auto one = [&](int i) {
      return launch_dgemv_tile(trans, (int)T, (int)T, 1.0, a + (size_t)(i % slots) * T * T, T, x, 1,
                               0.5, y, 1, partial, s, &launches);
    };
    for (int i = 0; i < 2 && e == cudaSuccess; ++i) e = one(i);
    cudaEventRecord(e0, s);
    for (int i = 0; i < reps && e == cudaSuccess; ++i) e = one(i + 2);
    cudaEventRecord(e1, s);
    if (e == cudaSuccess) e = cudaEventSynchronize(e1);
    float ms = 0.f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
    if (e != cudaSuccess) rc = fail(PARALIA_ERR_CUDA, "level-2 benchmark failed: %s", cudaGetErrorString(e));
    else *mean_s = ms * 1e-3 / reps;
  }
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  cudaFree(a);
  cudaFree(x);
  cudaFree(y);
  cudaFree(partial);
  cudaGetLastError();
  return rc;
}

}  // namespace
}  // namespace paralia

using namespace paralia;

extern "C" {

int PARALiA_bench_tile_dgemv(int dev, char TransA, int64_t T, int reps, double* mean_s) {
  if (TransA != 'N' && TransA != 'T') return fail(PARALIA_ERR_INVALID_ARG, "TransA must be N or T");
  return bench_level2(TransA == 'T', dev, T, reps, mean_s);
}

int PARALiA_bench_tile_daxpy(int dev, int64_t N, int reps, double* mean_s) {
  return bench_level1(false, dev, N, reps, mean_s);
}

int PARALiA_bench_tile_ddot(int dev, int64_t N, int reps, double* mean_s) {
  return bench_level1(true, dev, N, reps, mean_s);
}

static int bench_tf32_peak(int dev, int stages, bool random_operands, double* tflops) {
  if (!tflops || stages <= 0) return fail(PARALIA_ERR_INVALID_ARG, "bad bench arguments");
  Runtime& rt = Runtime::get();
  PL_TRY(rt.init());
  DeviceGuard guard;
  PL_TRY(rt.ensure_device(dev));
  PL_CUDA(cudaSetDevice(dev));
  DeviceCtx& dc = rt.dev(dev);
  int sms = 0;
  PL_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  cudaEvent_t e0, e1;
  PL_CUDA(cudaEventCreate(&e0));
  PL_CUDA(cudaEventCreate(&e1));
  cudaStream_t s = dc.exec[0];
  cudaError_t e = launch_tf32_peak(std::min(stages, 2000), sms, random_operands, dc.status_dev, s);   // warm-up
  if (e == cudaSuccess) e = cudaEventRecord(e0, s);
  if (e == cudaSuccess) e = launch_tf32_peak(stages, sms, random_operands, dc.status_dev, s);
  if (e == cudaSuccess) e = cudaEventRecord(e1, s);
  if (e == cudaSuccess) e = cudaEventSynchronize(e1);
  float ms = 0.f;
  if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (e != cudaSuccess) return fail(PARALIA_ERR_CUDA, "TF32 peak loop failed: %s", cudaGetErrorString(e));
  PL_TRY(rt.check_status(dev));
  *tflops = SG_PEAK_FLOP_PER_STAGE * (double)stages * sms / (ms * 1e-3) / 1e12;
  return PARALIA_OK;
}

int PARALiA_bench_tf32_peak(int dev, int stages, double* tflops) {
  return bench_tf32_peak(dev, stages, false, tflops);
}

int PARALiA_bench_tf32_peak_random(int dev, int stages, double* tflops) {
  return bench_tf32_peak(dev, stages, true, tflops);
}

int PARALiA_bench_host_aggregate(int ngpu, int mode, int64_t bytes, int reps, double* gbs) {
  if (!gbs || ngpu <= 0 || mode < 0 || mode > 2 || bytes <= 0 || reps <= 0)
    return fail(PARALIA_ERR_INVALID_ARG, "bad bench arguments");
  Runtime& rt = Runtime::get();
  PL_TRY(rt.init());
  if (ngpu > rt.device_count())
    return fail(PARALIA_ERR_INVALID_ARG, "%d GPUs asked for, %d present", ngpu, rt.device_count());
  DeviceGuard guard;
  const bool in = mode == 0 || mode == 2, out = mode == 1 || mode == 2;
  struct Leg { void *h_in = nullptr, *d_in = nullptr, *h_out = nullptr, *d_out = nullptr; };
  std::vector<Leg> legs(ngpu);
  int rc = PARALIA_OK;
  for (int g = 0; g < ngpu && rc == PARALIA_OK; ++g) {
    rc = rt.ensure_device(g);
    if (rc != PARALIA_OK) break;
    cudaSetDevice(g);
    cudaError_t e = cudaSuccess;
    if (in) {
      e = cudaMallocHost(&legs[g].h_in, (size_t)bytes);
      if (e == cudaSuccess) e = cudaMalloc(&legs[g].d_in, (size_t)bytes);
      if (e == cudaSuccess) memset(legs[g].h_in, 1, (size_t)bytes);
    }
    if (out && e == cudaSuccess) {
      e = cudaMallocHost(&legs[g].h_out, (size_t)bytes);
      if (e == cudaSuccess) e = cudaMalloc(&legs[g].d_out, (size_t)bytes);
      if (e == cudaSuccess) memset(legs[g].h_out, 1, (size_t)bytes);
    }
    if (e != cudaSuccess) rc = fail(PARALIA_ERR_OUT_OF_MEMORY, "bench buffers: %s", cudaGetErrorString(e));
  }
  if (rc == PARALIA_OK) {
    auto issue = [&](int n) {
      for (int i = 0; i < n; ++i)
        for (int g = 0; g < ngpu; ++g) {
          cudaSetDevice(g);
          DeviceCtx& dc = rt.dev(g);
          if (in) cudaMemcpyAsync(legs[g].d_in, legs[g].h_in, (size_t)bytes, cudaMemcpyHostToDevice, dc.h2d);
          if (out) cudaMemcpyAsync(legs[g].h_out, legs[g].d_out, (size_t)bytes, cudaMemcpyDeviceToHost, dc.d2h);
        }
    };
    auto sync_all = [&]() {
      cudaError_t e = cudaSuccess;
      for (int g = 0; g < ngpu; ++g) {
        cudaSetDevice(g);
        cudaError_t e1 = cudaStreamSynchronize(rt.dev(g).h2d);
        cudaError_t e2 = cudaStreamSynchronize(rt.dev(g).d2h);
        if (e == cudaSuccess) e = e1 != cudaSuccess ? e1 : e2;
      }
      return e;
    };
    issue(1);   // warm-up
    cudaError_t e = sync_all();
    const double t0 = wall_ms();
    issue(reps);
    if (e == cudaSuccess) e = sync_all();
    const double dt = (wall_ms() - t0) * 1e-3;
    if (e != cudaSuccess) rc = fail(PARALIA_ERR_CUDA, "host aggregate benchmark failed: %s", cudaGetErrorString(e));
    else *gbs = (double)bytes * reps * ngpu / dt / 1e9;   // per direction
  }
  for (int g = 0; g < ngpu; ++g) {
    cudaSetDevice(g);
    if (legs[g].h_in) cudaFreeHost(legs[g].h_in);
    if (legs[g].h_out) cudaFreeHost(legs[g].h_out);
    if (legs[g].d_in) cudaFree(legs[g].d_in);
    if (legs[g].d_out) cudaFree(legs[g].d_out);
  }
  cudaGetLastError();
  return rc;
}

int PARALiA_autotune_vec(int is_dot, int64_t N, int locx, int locy, const paralia_ctl* ctl,
                         paralia_report* out) {
  int ngpu = 0;
  if (!(ctl && ctl->active_unit_num > 0)) {
    Runtime& rt = Runtime::get();
    PL_TRY(rt.init());
    ngpu = rt.device_count();
  } else {
    for (int i = 0; i < ctl->active_unit_num && i < PARALIA_MAX_UNITS; ++i)
      ngpu = std::max(ngpu, ctl->active_unit_id_list[i] + 1);
    ngpu = std::max(ngpu, std::max(locx, locy) + 1);
  }
  if (model_db().link.empty() || (int)model_db().link.size() < ngpu + 1) reset_database_defaults(ngpu);
  VecModelInput in;
  in.func = is_dot ? "Ddot" : "Daxpy";
  in.N = N;
  in.locx = locx;
  in.locy = locy;
  return autotune_vec(in, ngpu, ctl, out);
}

int PARALiA_model_host_link(int dev, int to_gpu, int64_t bytes, int n_active, int both_directions,
                            const int32_t* active_devs, int n_devs, double* seconds,
                            int32_t* defer_writebacks_out) {
  if (!seconds || bytes < 0 || n_active <= 0 || dev < 0)
    return fail(PARALIA_ERR_INVALID_ARG, "bad model arguments");
  if (model_db().link.empty() || (int)model_db().link.size() < dev + 2)
    reset_database_defaults(std::max(dev + 1, n_active));
  std::vector<int> devs;
  for (int i = 0; active_devs && i < n_devs; ++i) devs.push_back(active_devs[i]);
  *seconds = host_link_time_shared(dev, to_gpu != 0, (double)bytes, n_active, both_directions != 0,
                                   active_devs ? &devs : nullptr);
  if (defer_writebacks_out) *defer_writebacks_out = defer_writebacks(n_active) ? 1 : 0;
  return PARALIA_OK;
}

}  // extern "C"
