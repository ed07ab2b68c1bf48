// Multi-GPU tiled DGEMV: y <- alpha*op(A)*x + beta*y.
//
// Stands where the reference has PARALiADgemv (Library_scheduler/src/Functions/
// dgemv.cpp:288; Library_scheduler/include/PARALiA.hpp:48-53). The output vector is cut
// into one contiguous run per GPU (rows of A for op = N, columns for op = T); each GPU
// streams its panel of A in column tiles through a two-slot ring (host link or NVLink),
// keeps x and its run of y on the device, and writes its run of y back at the end. A is
// read exactly once, so the routine is bound by the link A crosses (or by HBM when A
// already lives on the GPU). The order of every sum is fixed: bit-reproducible.
#include <algorithm>
#include <cstring>
#include <vector>

#include "exec.hpp"
#include "level2.cuh"
#include "runtime.hpp"

namespace paralia {
namespace {

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline size_t align_up(size_t a, size_t b) { return (a + b - 1) / b * b; }

struct GvUnit {
  int dev;
  int64_t o_lo, o_hi;          // run of the output vector
  double *x_dev, *y_dev, *partial;
  char* ring[2];
  int64_t y_inc;               // increment of y as the kernels see it
  cudaEvent_t slot_free[2] = {nullptr, nullptr};
  cudaEvent_t tail = nullptr;
};

}  // namespace

int exec_dgemv(char TransA, int64_t M, int64_t N, double alpha, const double* A, int64_t ldA,
               int locA, const double* x, int64_t incx, int locx, double beta, double* y,
               int64_t incy, int locy, const paralia_ctl* ctl, paralia_report* out) {
  const double t_call0 = wall_ms();
  paralia_report local_rep;
  paralia_report* rep = out ? out : &local_rep;
  memset(rep, 0, sizeof(*rep));
  bool trans;
  switch (TransA) {
    case 'N': case 'n': trans = false; break;
    case 'T': case 't': case 'C': case 'c': trans = true; break;
    default: return fail(PARALIA_ERR_INVALID_ARG, "transpose flag '%c' is not N or T", TransA);
  }
  if (M < 0 || N < 0 || M > INT32_MAX || N > INT32_MAX)
    return fail(PARALIA_ERR_INVALID_ARG, "dimension out of range");
  if (ldA < std::max<int64_t>(1, M))
    return fail(PARALIA_ERR_INVALID_ARG, "leading dimension smaller than the row count");
  if (incx <= 0 || incy <= 0)
    return fail(PARALIA_ERR_UNSUPPORTED, "non-positive increments are not supported");
  const int64_t out_len = trans ? N : M, in_len = trans ? M : N;
  if (out_len == 0) return PARALIA_OK;
  if (!y || (in_len > 0 && (!A || !x))) return fail(PARALIA_ERR_INVALID_ARG, "NULL operand");
  if (in_len == 0 && !(trans && M == 0)) {
    // Nothing to multiply: y <- beta*y (y <- 0 for beta == 0, without reading y, as BLAS
    // defines it). Run as the transposed product of a matrix with no rows: every column's
    // dot product is empty and the kernel's epilogue applies beta in one rounding. A and x
    // are never read; y's own pointer stands in for them. (That call falls through here.)
    return exec_dgemv('T', 0, out_len, alpha, y, 1, locy, y, 1, locy, beta, y, incy, locy, ctl, out);
  }

  Runtime& rt = Runtime::get();
  PL_TRY(rt.init());
  std::lock_guard<std::mutex> call_lock(rt.call_mutex());
  DeviceGuard guard;
  const int ngpu = rt.device_count();

  HostPin pins[3];
  double pin_ms = 0.0;
  int lA = -1, lx = -1, ly = -1;
  int rc = resolve_operand_location(A, locA, (M > 0 && N > 0) ? (size_t)(ldA * (N - 1) + M) * 8 : 0, ngpu, &lA, &pins[0], &pin_ms);
  if (rc == PARALIA_OK) rc = resolve_operand_location(x, locx, (size_t)(1 + (in_len - 1) * incx) * 8, ngpu, &lx, &pins[1], &pin_ms);
  if (rc == PARALIA_OK) rc = resolve_operand_location(y, locy, (size_t)(1 + (out_len - 1) * incy) * 8, ngpu, &ly, &pins[2], &pin_ms);
  const bool keep_pinned = ctl && (ctl->flags & PARALIA_FLAG_KEEP_PINNED);
  auto cleanup = [&]() { if (!keep_pinned) for (auto& p : pins) p.release(); };
  if (rc != PARALIA_OK) { cleanup(); return rc; }
  rep->pin_ms = pin_ms;

  // ---- units and their runs of the output vector
  const double t_plan0 = wall_ms();
  std::vector<int> devs;
  if (ctl && ctl->active_unit_num > 0) {
    for (int i = 0; i < ctl->active_unit_num && i < PARALIA_MAX_UNITS; ++i) {
      const int d = ctl->active_unit_id_list[i];
      if (d < 0 || d >= ngpu) { cleanup(); return fail(PARALIA_ERR_INVALID_ARG, "unit id %d is not a GPU", d); }
      devs.push_back(d);
    }
  } else if (lA >= 0) devs.push_back(lA);
  else for (int d = 0; d < ngpu; ++d) devs.push_back(d);
  int U = (int)std::min<int64_t>((int64_t)devs.size(), ceil_div(out_len, 2));
  devs.resize(U);
  std::vector<GvUnit> units(U);
  const int64_t pairs = ceil_div(out_len, 2), base = pairs / U, extra = pairs % U;
  int64_t lo = 0;
  int64_t max_run = 0;
  for (int ui = 0; ui < U; ++ui) {
    units[ui].dev = devs[ui];
    units[ui].o_lo = std::min(out_len, lo * 2);
    lo += base + (ui < extra ? 1 : 0);
    units[ui].o_hi = std::min(out_len, lo * 2);
    max_run = std::max(max_run, units[ui].o_hi - units[ui].o_lo);
  }
  // columns per tile: about 64 MiB of A per tile, a multiple of 64 columns; a panel that
  // already lives on its (only) GPU is not staged at all and runs as one tile
  const int64_t panel_rows = trans ? M : max_run;
  int64_t Tc = (ctl && ctl->T > 0) ? ctl->T : 0;
  if (Tc <= 0 && U == 1 && lA == devs[0]) {
    Tc = ceil_div(trans ? max_run : N, 64) * 64;
  } else if (Tc <= 0) {
    Tc = (64ll << 20) / std::max<int64_t>(8, panel_rows * 8);
    Tc = std::max<int64_t>(64, Tc / 64 * 64);
  }
  rep->T = Tc;
  rep->active_unit_num = U;
  rep->grid_d1 = U; rep->grid_d2 = 1;

  double alloc_ms = 0.0;
  for (int ui = 0; ui < U && rc == PARALIA_OK; ++ui) {
    GvUnit& u = units[ui];
    rep->active_unit_id_list[ui] = u.dev;
    rep->active_unit_score[ui] = 1.0 / U;
    rc = rt.ensure_device(u.dev);
    if (rc != PARALIA_OK) break;
    rt.release_events(u.dev);
    const int64_t run = u.o_hi - u.o_lo;
    const int64_t rows = trans ? M : run;                 // rows of this unit's panel of A
    const int64_t cols_total = trans ? run : N;           // columns it walks through
    const int64_t ntiles = ceil_div(cols_total, Tc);
    rep->subkernels_per_unit[ui] = (int)ntiles;
    rep->subkernel_num += ntiles;
    const bool x_here = lx == u.dev && incx == 1;
    const bool y_here = ly == u.dev;
    const bool a_here = lA == u.dev;
    const int64_t ld_ring = rows + (rows & 1);
    size_t off = 0, x_off = 0, y_off = 0, p_off = 0, r_off[2] = {0, 0};
    if (!x_here) { x_off = off; off = align_up(off + (size_t)in_len * 8, 256); }
    if (!y_here) { y_off = off; off = align_up(off + (size_t)run * 8, 256); }
    if (!trans) {
      p_off = off;
      off = align_up(off + (size_t)gemv_n_slices((int)rows, (int)std::min(Tc, cols_total)) * rows * 8, 256);
    }
    if (!a_here)
      for (int s = 0; s < 2; ++s) { r_off[s] = off; off = align_up(off + (size_t)ld_ring * Tc * 8, 256); }
    if (off > 0) rc = rt.ensure_slab(u.dev, off, &alloc_ms);
    if (rc != PARALIA_OK) break;
    char* slab = static_cast<char*>(rt.dev(u.dev).slab);
    u.x_dev = x_here ? const_cast<double*>(x) : reinterpret_cast<double*>(slab + x_off);
    u.y_dev = y_here ? y + u.o_lo * incy : reinterpret_cast<double*>(slab + y_off);
    u.y_inc = y_here ? incy : 1;
    u.partial = trans ? nullptr : reinterpret_cast<double*>(slab + p_off);
    u.ring[0] = a_here ? nullptr : slab + r_off[0];
    u.ring[1] = a_here ? nullptr : slab + r_off[1];
  }
  if (rc != PARALIA_OK) { cleanup(); return rc; }
  rep->alloc_ms = alloc_ms;
  rep->plan_ms = wall_ms() - t_plan0 - alloc_ms;

  {
    std::vector<int> op_devs = {lA, lx, ly}, unit_devs;
    for (const GvUnit& u : units) { op_devs.push_back(u.dev); unit_devs.push_back(u.dev); }
    rc = rt.order_after_caller(op_devs, unit_devs);
    if (rc != PARALIA_OK) { cleanup(); return rc; }
  }
  // ---- enqueue: per GPU x, its run of y, then the column tiles of its panel
  auto enqueue_unit = [&](int ui) -> int {
    GvUnit& u = units[ui];
    DeviceCtx& dc = rt.dev(u.dev);
    PL_CUDA(cudaSetDevice(u.dev));
    PL_CUDA(cudaEventRecord(dc.t_begin, dc.h2d));
    cudaStream_t es = dc.exec[0];
    PL_CUDA(cudaStreamWaitEvent(es, dc.t_begin, 0));
    PL_CUDA(cudaStreamWaitEvent(dc.p2p, dc.t_begin, 0));
    PL_CUDA(cudaStreamWaitEvent(dc.d2h, dc.t_begin, 0));
    const int64_t run = u.o_hi - u.o_lo;
    const int64_t rows = trans ? M : run;
    const int64_t cols_total = trans ? run : N;
    const int64_t ld_ring = rows + (rows & 1);
    const bool x_here = lx == u.dev && incx == 1;
    const bool y_here = ly == u.dev;
    const bool a_here = lA == u.dev;
    auto count = [&](int loc, int64_t bytes) {
      if (loc == -1) rep->h2d_bytes += bytes;
      else if (loc == u.dev) rep->d2d_bytes += bytes;
      else rep->p2p_bytes += bytes;
    };
    if (!x_here && in_len > 0) {
      cudaStream_t cs = lx == -1 ? dc.h2d : dc.p2p;
      if (incx == 1) PL_CUDA(cudaMemcpyAsync(u.x_dev, x, in_len * 8, cudaMemcpyDefault, cs));
      else PL_CUDA(cudaMemcpy2DAsync(u.x_dev, 8, x, incx * 8, 8, in_len, cudaMemcpyDefault, cs));
      count(lx, in_len * 8);
      cudaEvent_t ev; PL_TRY(rt.get_event(u.dev, &ev));
      PL_CUDA(cudaEventRecord(ev, cs));
      PL_CUDA(cudaStreamWaitEvent(es, ev, 0));
    }
    if (!y_here && beta != 0.0) {
      cudaStream_t cs = ly == -1 ? dc.h2d : dc.p2p;
      const double* src = y + u.o_lo * incy;
      if (incy == 1) PL_CUDA(cudaMemcpyAsync(u.y_dev, src, run * 8, cudaMemcpyDefault, cs));
      else PL_CUDA(cudaMemcpy2DAsync(u.y_dev, 8, src, incy * 8, 8, run, cudaMemcpyDefault, cs));
      count(ly, run * 8);
      cudaEvent_t ev; PL_TRY(rt.get_event(u.dev, &ev));
      PL_CUDA(cudaEventRecord(ev, cs));
      PL_CUDA(cudaStreamWaitEvent(es, ev, 0));
    }
    const int64_t ntiles = ceil_div(cols_total, Tc);
    for (int64_t j = 0; j < ntiles; ++j) {
      const int64_t c0 = j * Tc, cn = std::min(Tc, cols_total - c0);
      // first element of the tile in the user's A
      const double* a_src = trans ? A + (u.o_lo + c0) * ldA : A + u.o_lo + c0 * ldA;
      const double* a_tile = a_src;
      int64_t lda_tile = ldA;
      if (!a_here && rows > 0) {
        const int slot = (int)(j & 1);
        cudaStream_t cs = lA == -1 ? dc.h2d : dc.p2p;
        if (u.slot_free[slot]) PL_CUDA(cudaStreamWaitEvent(cs, u.slot_free[slot], 0));
        PL_CUDA(cudaMemcpy2DAsync(u.ring[slot], ld_ring * 8, a_src, ldA * 8, rows * 8, cn,
                                  cudaMemcpyDefault, cs));
        count(lA, rows * cn * 8);
        cudaEvent_t ev; PL_TRY(rt.get_event(u.dev, &ev));
        PL_CUDA(cudaEventRecord(ev, cs));
        PL_CUDA(cudaStreamWaitEvent(es, ev, 0));
        a_tile = reinterpret_cast<const double*>(u.ring[slot]);
        lda_tile = ld_ring;
      }
      int launches = 0;
      if (!trans) {
        // this tile adds its columns' contribution to the whole run of y
        PL_CUDA(launch_dgemv_tile(false, (int)rows, (int)cn, alpha, a_tile, lda_tile, u.x_dev + c0, 1,
                                  j == 0 ? beta : 1.0, u.y_dev, u.y_inc, u.partial, es, &launches));
      } else {
        // this tile finishes y[c0 .. c0+cn) of the run
        PL_CUDA(launch_dgemv_tile(true, (int)rows, (int)cn, alpha, a_tile, lda_tile, u.x_dev, 1, beta,
                                  u.y_dev + c0 * u.y_inc, u.y_inc, nullptr, es, &launches));
      }
      rep->kernel_launches += launches;
      cudaEvent_t kdone; PL_TRY(rt.get_event(u.dev, &kdone));
      PL_CUDA(cudaEventRecord(kdone, es));
      u.slot_free[j & 1] = kdone;
      u.tail = kdone;
    }
    if (u.tail) PL_CUDA(cudaStreamWaitEvent(dc.d2h, u.tail, 0));
    if (!y_here) {
      double* dst = y + u.o_lo * incy;
      if (incy == 1) PL_CUDA(cudaMemcpyAsync(dst, u.y_dev, run * 8, cudaMemcpyDefault, dc.d2h));
      else PL_CUDA(cudaMemcpy2DAsync(dst, incy * 8, u.y_dev, 8, 8, run, cudaMemcpyDefault, dc.d2h));
      if (ly == -1) rep->d2h_bytes += run * 8; else rep->p2p_bytes += run * 8;
    }
    PL_CUDA(cudaEventRecord(dc.t_end, dc.d2h));
    return PARALIA_OK;
  };
  for (int ui = 0; ui < U && rc == PARALIA_OK; ++ui) rc = enqueue_unit(ui);

  double dev_ms = 0.0;
  for (int ui = 0; ui < U; ++ui) {
    DeviceCtx& dc = rt.dev(units[ui].dev);
    cudaSetDevice(units[ui].dev);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess && rc == PARALIA_OK)
      rc = fail(PARALIA_ERR_CUDA, "GPU %d failed while running the plan: %s", units[ui].dev,
                cudaGetErrorString(e));
    if (rc == PARALIA_OK) {
      float ms = 0.f;
      if (cudaEventElapsedTime(&ms, dc.t_begin, dc.t_end) == cudaSuccess)
        dev_ms = std::max(dev_ms, (double)ms);
    }
  }
  cleanup();
  rep->device_ms = dev_ms;
  rep->host_ms = wall_ms() - t_call0;
  return rc;
}

}  // namespace paralia
