// Multi-GPU tiled DAXPY and DDOT.
//
// Stands where the reference has PARALiADaxpy (Library_scheduler/src/Functions/
// daxpy.cpp:200-469) and PARALiADdot (ddot.cpp:201-469): the vector is cut into 1-D
// tiles of T elements, one subkernel per tile (daxpy.cpp:35-78, ddot.cpp:35-78), tiles
// stream host -> GPU -> host through a small ring of cache blocks, and for the dot
// product every tile leaves one partial that the host adds into *result in tile order
// (ddot.cpp:431). Each GPU owns one contiguous run of tiles.
#include <algorithm>
#include <cstring>
#include <vector>

#include "level1.cuh"
#include "autotune.hpp"
#include "runtime.hpp"

namespace paralia {
namespace {

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

struct VecDesc {
  const double* ptr = nullptr;
  int64_t inc = 1;
  int loc = -1;
  HostPin pin;   // page-lock taken by this call, if any
};

int resolve_vec(VecDesc* v, int loc_in, int64_t n, int ngpu, double* pin_ms) {
  const size_t bytes = n > 0 ? (size_t)(1 + (n - 1) * std::llabs(v->inc)) * sizeof(double) : 0;
  return resolve_operand_location(v->ptr, loc_in, bytes, ngpu, &v->loc, &v->pin, pin_ms);
}

void unpin(VecDesc* v) { v->pin.release(); }

constexpr int RING = 4;  // cache blocks per vector and GPU

struct L1Unit {
  int dev;
  int64_t tile_lo, tile_hi;      // global tile range [lo, hi)
  cudaEvent_t x_free[RING] = {}, y_free[RING] = {};  // slot may be overwritten after this
  cudaEvent_t tail = nullptr;
};

// Bring `len` elements starting at element `start` of a strided vector into contiguous
// device memory `dst` on the current GPU.
int fetch_vec(double* dst, const VecDesc& v, int64_t start, int64_t len, cudaStream_t s,
              paralia_report* rep, int dev) {
  const double* src = v.ptr + start * v.inc;
  if (v.inc == 1)
    PL_CUDA(cudaMemcpyAsync(dst, src, len * sizeof(double), cudaMemcpyDefault, s));
  else
    PL_CUDA(cudaMemcpy2DAsync(dst, sizeof(double), src, v.inc * sizeof(double), sizeof(double), len,
                              cudaMemcpyDefault, s));
  if (v.loc == -1) rep->h2d_bytes += len * 8;
  else if (v.loc == dev) rep->d2d_bytes += len * 8;
  else rep->p2p_bytes += len * 8;
  return PARALIA_OK;
}

// is_dot == false: y <- alpha*x + y;  is_dot == true: *result += x . y
int run_level1(bool is_dot, int64_t N, double alpha, const double* x, int64_t incx, int locx,
               double* y, int64_t incy, int locy, double* result, const paralia_ctl* ctl,
               paralia_report* out, double* tile_sums = nullptr, int64_t tile_capacity = 0,
               int64_t* tile_count = nullptr) {
  const double t_call0 = wall_ms();
  paralia_report local_rep;
  paralia_report* rep = out ? out : &local_rep;
  memset(rep, 0, sizeof(*rep));
  if (N < 0) return fail(PARALIA_ERR_INVALID_ARG, "negative vector length");
  if (is_dot && !result && !tile_count) return fail(PARALIA_ERR_INVALID_ARG, "NULL result pointer");
  if (tile_count) *tile_count = 0;
  if (N == 0) return PARALIA_OK;
  if (!x || !y) return fail(PARALIA_ERR_INVALID_ARG, "NULL vector");
  if (incx <= 0 || incy <= 0)
    return fail(PARALIA_ERR_UNSUPPORTED, "non-positive increments are not supported");

  Runtime& rt = Runtime::get();
  PL_TRY(rt.init());
  std::lock_guard<std::mutex> call_lock(rt.call_mutex());
  DeviceGuard guard;
  const int ngpu = rt.device_count();

  VecDesc vx, vy;
  vx.ptr = x; vx.inc = incx;
  vy.ptr = y; vy.inc = incy;
  double pin_ms = 0.0;
  int rc = resolve_vec(&vx, locx, N, ngpu, &pin_ms);
  if (rc == PARALIA_OK) rc = resolve_vec(&vy, locy, N, ngpu, &pin_ms);
  const bool keep_pinned = ctl && (ctl->flags & PARALIA_FLAG_KEEP_PINNED);
  auto cleanup = [&]() { if (!keep_pinned) { unpin(&vx); unpin(&vy); } };
  if (rc != PARALIA_OK) { cleanup(); return rc; }
  rep->pin_ms = pin_ms;

  // ---- units and tile length from the model (ModelLvl1.cpp:19-144 with the measured
  // Daxpy / Ddot tile tables and the shared host-link model): a vector that already sits on
  // a GPU ends up processed there, host vectors are spread over as many GPUs as the host
  // links reward; the caller's control values override either choice.
  const double t_plan0 = wall_ms();
  VecModelInput vin;
  vin.func = is_dot ? "Ddot" : "Daxpy";
  vin.N = N;
  vin.locx = vx.loc;
  vin.locy = vy.loc;
  paralia_report tuned;
  rc = autotune_vec(vin, ngpu, ctl, &tuned);
  if (rc != PARALIA_OK) { cleanup(); return rc; }
  std::vector<int> devs(tuned.active_unit_id_list, tuned.active_unit_id_list + tuned.active_unit_num);
  int U = (int)devs.size();
  int64_t T = tuned.T;
  rep->pred_t = tuned.pred_t;
  if (T > N) T = N;
  const int64_t Nt = ceil_div(N, T);
  if (Nt < U) U = (int)Nt;
  devs.resize(U);
  rep->T = T;
  rep->active_unit_num = U;
  rep->subkernel_num = Nt;
  rep->grid_d1 = U; rep->grid_d2 = 1;

  std::vector<L1Unit> units(U);
  const int64_t base = Nt / U, extra = Nt % U;
  int64_t lo = 0;
  for (int ui = 0; ui < U; ++ui) {
    units[ui].dev = devs[ui];
    units[ui].tile_lo = lo;
    lo += base + (ui < extra ? 1 : 0);
    units[ui].tile_hi = lo;
    rep->active_unit_id_list[ui] = devs[ui];
    rep->active_unit_score[ui] = 1.0 / U;
    rep->subkernels_per_unit[ui] = (int)(units[ui].tile_hi - units[ui].tile_lo);
  }

  double alloc_ms = 0.0;
  const size_t blk = (size_t)T * sizeof(double);
  for (int ui = 0; ui < U && rc == PARALIA_OK; ++ui) {
    L1Unit& u = units[ui];
    rc = rt.ensure_device(u.dev);
    if (rc != PARALIA_OK) break;
    rt.release_events(u.dev);
    const bool x_here = vx.loc == u.dev && vx.inc == 1;
    const bool y_here = vy.loc == u.dev && vy.inc == 1;
    size_t need = 0;
    if (!x_here) need += RING * blk;
    if (!y_here) need += RING * blk;
    if (need) rc = rt.ensure_slab(u.dev, need, &alloc_ms);
    if (rc == PARALIA_OK && is_dot)
      rc = rt.ensure_dot_scratch(u.dev, (size_t)RING * l1_grid_blocks(T),
                                 (size_t)(u.tile_hi - u.tile_lo));
  }
  if (rc != PARALIA_OK) { cleanup(); return rc; }
  rep->alloc_ms = alloc_ms;
  rep->plan_ms = wall_ms() - t_plan0 - alloc_ms;

  {
    std::vector<int> op_devs = {vx.loc, vy.loc}, unit_devs;
    for (const L1Unit& u : units) { op_devs.push_back(u.dev); unit_devs.push_back(u.dev); }
    rc = rt.order_after_caller(op_devs, unit_devs);
    if (rc != PARALIA_OK) { cleanup(); return rc; }
  }
  // ---- enqueue, round-robin over the GPUs one tile at a time
  for (int ui = 0; ui < U; ++ui) {
    DeviceCtx& dc = rt.dev(units[ui].dev);
    cudaSetDevice(units[ui].dev);
    cudaEventRecord(dc.t_begin, dc.h2d);
    cudaStreamWaitEvent(dc.exec[0], dc.t_begin, 0);
    cudaStreamWaitEvent(dc.d2h, dc.t_begin, 0);
    cudaStreamWaitEvent(dc.p2p, dc.t_begin, 0);
  }
  int64_t max_tiles = 0;
  for (auto& u : units) max_tiles = std::max(max_tiles, u.tile_hi - u.tile_lo);
  auto enqueue_tile = [&](int ui, int64_t j) -> int {
    L1Unit& u = units[ui];
    DeviceCtx& dc = rt.dev(u.dev);
    PL_CUDA(cudaSetDevice(u.dev));
    const int64_t tile = u.tile_lo + j;
    const int64_t start = tile * T, len = std::min(T, N - start);
    const int slot = (int)(j % RING);
    const bool x_here = vx.loc == u.dev && vx.inc == 1;
    const bool y_here = vy.loc == u.dev && vy.inc == 1;
    char* slab = static_cast<char*>(dc.slab);
    double* xs = x_here ? const_cast<double*>(vx.ptr) + start
                        : reinterpret_cast<double*>(slab + (size_t)slot * blk);
    double* ys = y_here ? const_cast<double*>(vy.ptr) + start
                        : reinterpret_cast<double*>(slab + (size_t)((x_here ? 0 : RING) + slot) * blk);
    cudaStream_t es = dc.exec[0];
    if (!x_here) {
      cudaStream_t cs = vx.loc == -1 ? dc.h2d : dc.p2p;
      if (u.x_free[slot]) PL_CUDA(cudaStreamWaitEvent(cs, u.x_free[slot], 0));
      PL_TRY(fetch_vec(xs, vx, start, len, cs, rep, u.dev));
      cudaEvent_t ev; PL_TRY(rt.get_event(u.dev, &ev));
      PL_CUDA(cudaEventRecord(ev, cs));
      PL_CUDA(cudaStreamWaitEvent(es, ev, 0));
    }
    if (!y_here) {
      cudaStream_t cs = vy.loc == -1 ? dc.h2d : dc.p2p;
      if (u.y_free[slot]) PL_CUDA(cudaStreamWaitEvent(cs, u.y_free[slot], 0));
      PL_TRY(fetch_vec(ys, vy, start, len, cs, rep, u.dev));
      cudaEvent_t ev; PL_TRY(rt.get_event(u.dev, &ev));
      PL_CUDA(cudaEventRecord(ev, cs));
      PL_CUDA(cudaStreamWaitEvent(es, ev, 0));
    }
    int launches = 0;
    if (is_dot) {
      double* partials = dc.dot_partials + (size_t)slot * l1_grid_blocks(T);
      PL_CUDA(launch_ddot(len, xs, 1 * (x_here ? vx.inc : 1), ys, 1 * (y_here ? vy.inc : 1),
                          partials, dc.dot_results + j, es, &launches));
    } else {
      PL_CUDA(launch_daxpy(len, alpha, xs, x_here ? vx.inc : 1, ys, y_here ? vy.inc : 1, es,
                           &launches));
    }
    rep->kernel_launches += launches;
    cudaEvent_t kdone; PL_TRY(rt.get_event(u.dev, &kdone));
    PL_CUDA(cudaEventRecord(kdone, es));
    u.x_free[slot] = kdone;
    u.tail = kdone;
    if (!is_dot && !y_here) {
      // write the updated tile back to where y lives
      PL_CUDA(cudaStreamWaitEvent(dc.d2h, kdone, 0));
      double* dst = const_cast<double*>(vy.ptr) + start * vy.inc;
      if (vy.inc == 1)
        PL_CUDA(cudaMemcpyAsync(dst, ys, len * sizeof(double), cudaMemcpyDefault, dc.d2h));
      else
        PL_CUDA(cudaMemcpy2DAsync(dst, vy.inc * sizeof(double), ys, sizeof(double), sizeof(double),
                                  len, cudaMemcpyDefault, dc.d2h));
      if (vy.loc == -1) rep->d2h_bytes += len * 8; else rep->p2p_bytes += len * 8;
      cudaEvent_t wb; PL_TRY(rt.get_event(u.dev, &wb));
      PL_CUDA(cudaEventRecord(wb, dc.d2h));
      u.y_free[slot] = wb;
    } else {
      u.y_free[slot] = kdone;
    }
    return PARALIA_OK;
  };
  for (int64_t j = 0; j < max_tiles && rc == PARALIA_OK; ++j)
    for (int ui = 0; ui < U && rc == PARALIA_OK; ++ui)
      if (j < units[ui].tile_hi - units[ui].tile_lo) rc = enqueue_tile(ui, j);

  // ---- join
  for (int ui = 0; ui < U; ++ui) {
    L1Unit& u = units[ui];
    DeviceCtx& dc = rt.dev(u.dev);
    cudaSetDevice(u.dev);
    if (rc == PARALIA_OK) {
      if (u.tail) cudaStreamWaitEvent(dc.d2h, u.tail, 0);
      if (is_dot) {
        const size_t n = (size_t)(u.tile_hi - u.tile_lo);
        cudaMemcpyAsync(dc.dot_results_host, dc.dot_results, n * sizeof(double),
                        cudaMemcpyDeviceToHost, dc.d2h);
        rep->d2h_bytes += n * 8;
      }
      cudaEventRecord(dc.t_end, dc.d2h);
    }
  }
  double dev_ms = 0.0;
  for (int ui = 0; ui < U; ++ui) {
    L1Unit& u = units[ui];
    DeviceCtx& dc = rt.dev(u.dev);
    cudaSetDevice(u.dev);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess && rc == PARALIA_OK)
      rc = fail(PARALIA_ERR_CUDA, "GPU %d failed while running the plan: %s", u.dev,
                cudaGetErrorString(e));
    if (rc == PARALIA_OK) {
      float ms = 0.f;
      if (cudaEventElapsedTime(&ms, dc.t_begin, dc.t_end) == cudaSuccess)
        dev_ms = std::max(dev_ms, (double)ms);
    }
  }
  if (rc == PARALIA_OK && is_dot) {
    // Partials are added into *result in tile order; *result is not zeroed first
    // (ddot.cpp:431).
    double acc = result ? *result : 0.0;
    int64_t t = 0;
    for (int ui = 0; ui < U; ++ui) {
      const DeviceCtx& dc = rt.dev(units[ui].dev);
      const int64_t n = units[ui].tile_hi - units[ui].tile_lo;
      for (int64_t j = 0; j < n; ++j, ++t) {
        acc += dc.dot_results_host[j];
        if (tile_sums && t < tile_capacity) tile_sums[t] = dc.dot_results_host[j];
      }
    }
    if (result) *result = acc;
    if (tile_count) *tile_count = t;
  }
  cleanup();
  rep->device_ms = dev_ms;
  rep->host_ms = wall_ms() - t_call0;
  return rc;
}

}  // namespace

int exec_daxpy(int64_t N, double alpha, const double* x, int64_t incx, int locx, double* y,
               int64_t incy, int locy, const paralia_ctl* ctl, paralia_report* out) {
  return run_level1(false, N, alpha, x, incx, locx, y, incy, locy, nullptr, ctl, out);
}

int exec_ddot(int64_t N, const double* x, int64_t incx, int locx, const double* y, int64_t incy,
              int locy, double* result, const paralia_ctl* ctl, paralia_report* out) {
  return run_level1(true, N, 0.0, x, incx, locx, const_cast<double*>(y), incy, locy, result, ctl,
                    out);
}

int exec_ddot_tiles(int64_t N, const double* x, int64_t incx, int locx, const double* y,
                    int64_t incy, int locy, double* tile_sums, int64_t capacity, int64_t* count,
                    const paralia_ctl* ctl, paralia_report* out) {
  if (!count || capacity < 0 || (capacity > 0 && !tile_sums))
    return fail(PARALIA_ERR_INVALID_ARG, "bad tile-sum buffer");
  return run_level1(true, N, 0.0, x, incx, locx, const_cast<double*>(y), incy, locy, nullptr, ctl,
                    out, tile_sums, capacity, count);
}

}  // namespace paralia
