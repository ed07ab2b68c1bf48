// Multi-GPU tiled GEMM: static plan, per-GPU tile cache, stream/event overlap engine.
//
// This file stands where the reference has PARALiADgemm / PARALiASgemm
// (Library_scheduler/src/Functions/dgemm.cpp:318-694, sgemm.cpp:296-...) together with
// the subkernel scheduler underneath them (Library_scheduler/src/Subkernel.cpp:90-247,
// 384-449). What is kept: square T x T tiles, one subkernel per (mi, ni, ki) with id
// mi*Nt*Kt + ni*Kt + ki (dgemm.cpp:157-161), every subkernel of a C tile on the GPU that
// owns the tile (2D block distribution), beta applied lazily after the last k
// (ALGO_WR_LAZY, dgemm.cpp:173-179,273-279), a tile cached on a peer fetched from the
// peer instead of the host, C tiles written back as they finish.
//
// What is different by design: the order of everything is fixed before the first copy is
// enqueued (no ETA-driven selection, no rand() tie break, no polling manager thread), so
// a given problem always runs the same arithmetic in the same order on every GPU.
// One host thread walks the GPUs round-robin and enqueues, per subkernel, the tile
// fetches it still needs and its kernel; dependencies are CUDA events only.
#include <algorithm>
#include <cstdlib>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <type_traits>
#include <vector>

#include "autotune.hpp"
#include "dgemm_tile.cuh"
#include "plan.hpp"
#include "runtime.hpp"
#include "sgemm_tile.cuh"
#include "exec.hpp"
#include "group.hpp"

namespace paralia {

int sm_count_of(int dev);   // sgemm_exec.cpp

namespace {

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline size_t matrix_span_bytes(int64_t ld, int64_t rows, int64_t cols, int esz) {
  return (rows <= 0 || cols <= 0) ? 0 : (size_t)(ld * (cols - 1) + rows) * esz;
}
inline int64_t round_up(int64_t a, int64_t b) { return ceil_div(a, b) * b; }

// Which unit pulls a host-resident A tile (mi, ki) or B tile (ki, ni) over its host link
// and forwards it to the other consumers. `cons` are the consumers of the tile row / column
// in grid order, `first` the first tile row / column with the same consumers, `lead` the
// grid row (A) or grid column + 1 (B) of that set. The rotation by (local index + k) spreads
// a unit's fetches over k; the lead term makes the tiles that the very first launches need
// (local index 0, k 0) come over different host links on a device grid of 2 x 2 and more.
inline int rotating_home(int n_cons, int lead, int64_t local, int64_t ki) {
  return (int)(((int64_t)lead + local + ki) % n_cons);
}

struct OperandDesc {
  const void* ptr = nullptr;
  int64_t ld = 0;
  int loc = -1;          // -1 host, >=0 GPU
  bool trans = false;    // stored transposed w.r.t. its role in the GEMM
  int64_t rows = 0, cols = 0;  // stored extent
  HostPin pin;   // page-lock taken by this call, if any
};

// Where one tile of an operand can be read on one GPU.
struct Resident {
  bool present = false;   // fetch enqueued (or native)
  bool native = false;    // read in place from the user's matrix
  int block = -1;         // tile-cache block otherwise
  cudaEvent_t ready = nullptr;
};

struct UnitState {
  int dev = -1;
  std::vector<int> ctiles;             // C tiles (mi*Nt+ni) in processing order
  std::vector<Resident> a, b, c, csrc; // indexed by tile id of each operand
  int next_block = 0;
  int nblocks = 0;
  // Bounded cache (only when the slab cannot hold every tile the unit touches): what each
  // block holds, who may still be reading it, and blocks handed back after a write-back.
  struct BlockInfo {
    int kind = 0;            // 0 free, 1 A tile, 2 B tile, 3 C accumulator / original C
    int64_t tid = -1;
    uint64_t last_seq = 0;   // launch number that last used it
    cudaEvent_t readers[MAX_EXEC_STREAMS] = {};
    cudaEvent_t freed = nullptr;
  };
  std::vector<BlockInfo> blocks;
  std::vector<int> free_blocks;
  uint64_t seq = 0;          // launches enqueued so far
  CUtensorMap map_slab_kc, map_slab_mn;   // tile cache seen k-contiguous / row-contiguous
  CUtensorMap map_a_native, map_b_native; // user matrices on this GPU
  bool a_native_ok = false, b_native_ok = false, c_native = false;
  // Launches of this unit in enqueue order: (index into ctiles, first k tile, end k tile).
  using Item = LaunchItem;
  std::vector<Item> items;
  size_t cursor = 0;                   // next item to enqueue
  std::vector<cudaEvent_t> exec_tail;  // last event per exec stream
  bool first_exec_marked = false;      // the call's first kernel start has been recorded
  cudaEvent_t h2d_tail = nullptr, p2p_tail = nullptr, pack_tail = nullptr;
};

template <typename T>
struct GemmCall {
  char ta, tb;
  int64_t M, N, K;
  T alpha, beta;
  OperandDesc A, B, C;
  int64_t Tt = 0, TL = 0;   // tile edge, padded edge of a cache block
  int64_t Mt = 0, Nt = 0, Kt = 0;
  int exec_streams = 4;
  bool peer_fetch = true;
  // one-process-per-GPU group (null in the default in-process mode)
  Group* grp = nullptr;
  bool share_a = false, share_b = false;   // tiles shared inside the grid row / column
  int nA = 0, nB = 0;                       // fixed block ranges of A and B tiles in group mode
  bool prefetch_phase = false;              // enqueueing only this rank's home tiles
  bool evict = false;                       // the slab is smaller than the working set
  int64_t evictions = 0;
  // Write-backs held until the unit's host->GPU stream has drained (see run_gemm).
  bool defer_wb = false;
  struct PendingWb { int ui; int ct; cudaEvent_t done; char* dst; int64_t dst_ld; const char* src; int64_t rows, cols; };
  std::vector<PendingWb> pending_wb;
  std::vector<UnitState> units;
  std::vector<int> ctile_owner;             // C tile -> unit index
  std::vector<std::vector<int>> a_consumers; // per tile-row mi: units that read A(mi,*)
  std::vector<std::vector<int>> b_consumers; // per tile-col ni: units that read B(*,ni)
  std::vector<int> a_first, b_first;          // first tile row / column with the same consumers
  int grid_d1 = 1, grid_d2 = 1;

  // In-process mode: index into a_consumers[mi] / b_consumers[ni] of the tile's home unit.
  int home_index(bool is_a, int64_t i0, int64_t i1) const {
    if (is_a) {
      const std::vector<int>& cons = a_consumers[i0];
      return rotating_home((int)cons.size(), cons[0] / std::max(grid_d2, 1), i0 - a_first[i0], i1);
    }
    const std::vector<int>& cons = b_consumers[i1];
    return rotating_home((int)cons.size(), cons[0] % std::max(grid_d2, 1) + 1, i1 - b_first[i1], i0);
  }
  // Group mode: rank that is the home of a shared tile of this rank's own panels.
  int group_home(bool is_a, int64_t i0, int64_t i1) const {
    int d1, d2;
    grp->grid(&d1, &d2);
    const int me = grp->rank(), gr = me / d2, gc = me % d2;
    if (is_a) return gr * d2 + rotating_home(d2, gr, i0, i1);
    return rotating_home(d1, gc + 1, i1, i0) * d2 + gc;
  }
  paralia_report* rep = nullptr;
  static constexpr int esz = (int)sizeof(T);

  int64_t mrows(int64_t mi) const { return std::min(Tt, M - mi * Tt); }
  int64_t ncols(int64_t ni) const { return std::min(Tt, N - ni * Tt); }
  int64_t klen(int64_t ki) const { return std::min(Tt, K - ki * Tt); }
  // A cache block holds one FP64 tile, or one packed FP32 operand tile (hi and lo planes,
  // rows padded to the MMA's N) -- which is also large enough for an FP32 C tile.
  size_t block_bytes() const {
    if (std::is_same<T, float>::value)
      return (size_t)2 * round_up(Tt, SG_BN) * round_up(Tt, SG_BK) * 4;
    return (size_t)TL * TL * esz;
  }
  char* block_ptr(const UnitState& u, int blk) const {
    return static_cast<char*>(Runtime::get().dev(u.dev).slab) + (size_t)blk * block_bytes();
  }
};

int norm_trans(char t, bool* out) {
  switch (t) {
    case 'N': case 'n': *out = false; return PARALIA_OK;
    case 'T': case 't': case 'C': case 'c': *out = true; return PARALIA_OK;
    default: return fail(PARALIA_ERR_INVALID_ARG, "transpose flag '%c' is not N or T", t);
  }
}

// Resolve where an operand lives and make host memory DMA-able.
int resolve_operand(OperandDesc* op, int loc_in, size_t bytes, int ngpu, double* pin_ms) {
  return resolve_operand_location(op->ptr, loc_in, bytes, ngpu, &op->loc, &op->pin, pin_ms);
}

void unpin(OperandDesc* op) { op->pin.release(); }

template <typename T>
struct TileGeom {
  const char* src;    // first element in the user's matrix
  int64_t nr, nc;     // stored rows x cols of the tile
  bool k_is_row;      // k runs along stored rows (contiguous) rather than columns
};

template <typename T>
TileGeom<T> geom_a(const GemmCall<T>& g, int64_t mi, int64_t ki) {
  TileGeom<T> t;
  if (!g.A.trans) {
    t.src = (const char*)g.A.ptr + (mi * g.Tt + ki * g.Tt * g.A.ld) * g.esz;
    t.nr = g.mrows(mi); t.nc = g.klen(ki); t.k_is_row = false;
  } else {
    t.src = (const char*)g.A.ptr + (ki * g.Tt + mi * g.Tt * g.A.ld) * g.esz;
    t.nr = g.klen(ki); t.nc = g.mrows(mi); t.k_is_row = true;
  }
  return t;
}
template <typename T>
TileGeom<T> geom_b(const GemmCall<T>& g, int64_t ki, int64_t ni) {
  TileGeom<T> t;
  if (!g.B.trans) {
    t.src = (const char*)g.B.ptr + (ki * g.Tt + ni * g.Tt * g.B.ld) * g.esz;
    t.nr = g.klen(ki); t.nc = g.ncols(ni); t.k_is_row = true;
  } else {
    t.src = (const char*)g.B.ptr + (ni * g.Tt + ki * g.Tt * g.B.ld) * g.esz;
    t.nr = g.ncols(ni); t.nc = g.klen(ki); t.k_is_row = false;
  }
  return t;
}

// Hand out a cache block for tile `tid` of `kind` (1 A, 2 B, 3 C). While fresh blocks
// remain they are used in order. In bounded-cache mode a block returned after a write-back
// is reused next, else the least recently used A/B tile that the current launch does not
// need is evicted (the reference recycles blocks of a clamped slab the same way,
// dgemm.cpp:80-94; its policy lives in the backend that is not part of the checkout).
// Every stream that may fill the block waits for the kernels and copies still using it.
template <typename T>
int take_block(GemmCall<T>& g, UnitState& u, int* blk, int kind = 0, int64_t tid = -1,
               cudaStream_t extra_writer = nullptr) {
  if (u.next_block < u.nblocks) {
    *blk = u.next_block++;
    if (g.evict) {
      UnitState::BlockInfo& bi = u.blocks[*blk];
      bi.kind = kind; bi.tid = tid; bi.last_seq = u.seq;
    }
    return PARALIA_OK;
  }
  if (!g.evict)
    return fail(PARALIA_ERR_OUT_OF_MEMORY, "GPU %d: tile cache of %d blocks exhausted", u.dev,
                u.nblocks);
  int pick = -1;
  if (!u.free_blocks.empty()) {
    pick = u.free_blocks.back();
    u.free_blocks.pop_back();
  } else {
    uint64_t oldest = UINT64_MAX;
    for (int b = 0; b < u.nblocks; ++b) {
      const UnitState::BlockInfo& bi = u.blocks[b];
      if ((bi.kind == 1 || bi.kind == 2) && bi.last_seq < u.seq && bi.last_seq < oldest) {
        oldest = bi.last_seq;
        pick = b;
      }
    }
    if (pick < 0)
      return fail(PARALIA_ERR_OUT_OF_MEMORY,
                  "GPU %d: a tile cache of %d blocks is too small for one launch", u.dev, u.nblocks);
    UnitState::BlockInfo& v = u.blocks[pick];
    Resident& r = v.kind == 1 ? u.a[v.tid] : u.b[v.tid];
    r.present = false;
    r.block = -1;
    g.evictions += 1;
  }
  UnitState::BlockInfo& bi = u.blocks[pick];
  DeviceCtx& dc = Runtime::get().dev(u.dev);
  PL_CUDA(cudaSetDevice(u.dev));
  cudaStream_t writers[4] = {dc.h2d, dc.p2p, dc.pack, extra_writer};
  for (cudaStream_t w : writers) {
    if (!w) continue;
    for (int i = 0; i < MAX_EXEC_STREAMS; ++i)
      if (bi.readers[i]) PL_CUDA(cudaStreamWaitEvent(w, bi.readers[i], 0));
    if (bi.freed) PL_CUDA(cudaStreamWaitEvent(w, bi.freed, 0));
  }
  bi = UnitState::BlockInfo();
  bi.kind = kind; bi.tid = tid; bi.last_seq = u.seq;
  *blk = pick;
  return PARALIA_OK;
}

// Zero the k padding of a cache block so that the last 16-deep pipeline stage of an edge
// tile multiplies zeros, then copy the tile in. `stream` belongs to GPU u.dev.
template <typename T>
int copy_tile_in(GemmCall<T>& g, UnitState& u, int blk, const char* src, int64_t src_ld,
                 const TileGeom<T>& t, cudaStream_t stream, int64_t* byte_counter) {
  char* dst = g.block_ptr(u, blk);
  const int64_t kext = t.k_is_row ? t.nr : t.nc;
  const int64_t kpad = round_up(kext, DG_BK) - kext;
  if (kpad > 0) {
    if (t.k_is_row)
      PL_CUDA(cudaMemset2DAsync(dst + kext * g.esz, g.TL * g.esz, 0, kpad * g.esz, t.nc, stream));
    else
      PL_CUDA(cudaMemsetAsync(dst + kext * g.TL * g.esz, 0, kpad * g.TL * g.esz, stream));
  }
  PL_CUDA(cudaMemcpy2DAsync(dst, g.TL * g.esz, src, src_ld * g.esz, t.nr * g.esz, t.nc,
                            cudaMemcpyDefault, stream));
  if (byte_counter) *byte_counter += t.nr * t.nc * g.esz;
  return PARALIA_OK;
}

// ---- FP32 operands --------------------------------------------------------------------
// An FP32 tile is never read in place: the tensor-core kernel wants it split into TF32
// hi/lo planes in its shared-memory order (sgemm_tile.cuh). A tile therefore goes
//   user memory on a reachable GPU --pack kernel--> cache block, or
//   host (or unreachable GPU) --copy--> staging slot --pack kernel--> cache block,
// and a tile that another GPU has already packed is copied from that GPU's block.
template <typename T>
int pack_into_block(GemmCall<T>& g, UnitState& u, Resident& r, const OperandDesc& op,
                    const TileGeom<T>& t, int rows, int klen, int rb, cudaEvent_t also_record) {
  Runtime& rt = Runtime::get();
  DeviceCtx& dc = rt.dev(u.dev);
  void* dst = g.block_ptr(u, r.block);
  const bool reachable = op.loc >= 0 && (op.loc == u.dev || rt.peer_ok(u.dev, op.loc));
  if (reachable) {
    PL_CUDA(launch_sgemm_pack((const float*)t.src, op.ld, t.k_is_row, rows, klen, rb, dst, dc.pack));
    if (op.loc == u.dev) g.rep->d2d_bytes += (int64_t)rows * klen * 4;
    else g.rep->p2p_bytes += (int64_t)rows * klen * 4;
  } else {
    const int slot = dc.stage_next;
    dc.stage_next = (dc.stage_next + 1) % DeviceCtx::STAGE_SLOTS;
    char* stage = static_cast<char*>(dc.stage) + (size_t)slot * dc.stage_slot_bytes;
    cudaStream_t cs = op.loc == -1 ? dc.h2d : dc.p2p;
    if (dc.stage_used[slot]) PL_CUDA(cudaStreamWaitEvent(cs, dc.stage_free[slot], 0));
    PL_CUDA(cudaMemcpy2DAsync(stage, t.nr * 4, t.src, op.ld * 4, t.nr * 4, t.nc, cudaMemcpyDefault, cs));
    cudaEvent_t landed;
    PL_TRY(rt.get_event(u.dev, &landed));
    PL_CUDA(cudaEventRecord(landed, cs));
    if (op.loc == -1) { g.rep->h2d_bytes += t.nr * t.nc * 4; u.h2d_tail = landed; }
    else { g.rep->p2p_bytes += t.nr * t.nc * 4; u.p2p_tail = landed; }
    PL_CUDA(cudaStreamWaitEvent(dc.pack, landed, 0));
    PL_CUDA(launch_sgemm_pack((const float*)stage, t.nr, t.k_is_row, rows, klen, rb, dst, dc.pack));
    PL_CUDA(cudaEventRecord(dc.stage_free[slot], dc.pack));
    dc.stage_used[slot] = true;
  }
  g.rep->kernel_launches += 1;
  PL_CUDA(cudaEventRecord(r.ready, dc.pack));
  if (also_record) PL_CUDA(cudaEventRecord(also_record, dc.pack));
  u.pack_tail = r.ready;
  return PARALIA_OK;
}

template <typename T>
int ensure_input(GemmCall<T>& g, int ui, bool is_a, int64_t i0, int64_t i1);

template <typename T>
int ensure_input_f32(GemmCall<T>& g, int ui, bool is_a, int64_t i0, int64_t i1) {
  Runtime& rt = Runtime::get();
  UnitState& u = g.units[ui];
  const OperandDesc& op = is_a ? g.A : g.B;
  const int64_t tid = is_a ? i0 * g.Kt + i1 : i0 * g.Nt + i1;
  Resident& r = is_a ? u.a[tid] : u.b[tid];
  if (r.present) return PARALIA_OK;
  const TileGeom<T> t = is_a ? geom_a(g, i0, i1) : geom_b(g, i0, i1);
  const int rows = (int)(is_a ? g.mrows(i0) : g.ncols(i1));
  const int klen = (int)(is_a ? g.klen(i1) : g.klen(i0));
  const int rb = is_a ? SG_BM : SG_BN;
  const size_t packed = sgemm_packed_bytes(rows, klen, rb);
  PL_CUDA(cudaSetDevice(u.dev));
  DeviceCtx& dc = rt.dev(u.dev);
  if (g.grp && op.loc == -1 && (is_a ? g.share_a : g.share_b)) {
    const int me = g.grp->rank();
    const int slot = is_a ? (int)tid : g.nA + (int)tid;
    const int home = g.group_home(is_a, i0, i1);
    if (home == me) {
      r.block = slot;
      PL_TRY(rt.get_event(u.dev, &r.ready));
      PL_TRY(pack_into_block(g, u, r, op, t, rows, klen, rb, g.grp->own_event(slot)));
      r.present = true;
      return PARALIA_OK;
    }
    if (g.prefetch_phase) return PARALIA_OK;
    r.block = slot;
    PL_TRY(rt.get_event(u.dev, &r.ready));
    cudaEvent_t landed;
    PL_TRY(g.grp->peer_event(home, slot, &landed));
    PL_CUDA(cudaStreamWaitEvent(dc.p2p, landed, 0));
    const int peer_slot = is_a ? (int)tid : g.grp->info(home).nA + (int)tid;
    PL_CUDA(cudaMemcpyAsync(g.block_ptr(u, r.block),
                            g.grp->peer_slab(home) + (size_t)peer_slot * g.block_bytes(), packed,
                            cudaMemcpyDefault, dc.p2p));
    g.rep->p2p_bytes += (int64_t)packed;
    PL_CUDA(cudaEventRecord(r.ready, dc.p2p));
    u.p2p_tail = r.ready;
    r.present = true;
    return PARALIA_OK;
  }
  if (g.grp) r.block = is_a ? (int)tid : g.nA + (int)tid;
  else PL_TRY(take_block(g, u, &r.block, is_a ? 1 : 2, tid));
  PL_TRY(rt.get_event(u.dev, &r.ready));
  int home = ui;
  if (op.loc == -1 && !g.grp) {
    const std::vector<int>& cons = is_a ? g.a_consumers[i0] : g.b_consumers[i1];
    if (g.peer_fetch && cons.size() > 1) home = cons[g.home_index(is_a, i0, i1)];
    if (home != ui && !rt.peer_ok(u.dev, g.units[home].dev)) home = ui;
  }
  if (home == ui) {
    PL_TRY(pack_into_block(g, u, r, op, t, rows, klen, rb, nullptr));
  } else {
    // packed once on the home GPU, copied from its cache block over NVLink
    PL_TRY(ensure_input(g, home, is_a, i0, i1));
    PL_CUDA(cudaSetDevice(u.dev));
    UnitState& h = g.units[home];
    const Resident& hr = is_a ? h.a[tid] : h.b[tid];
    PL_CUDA(cudaStreamWaitEvent(dc.p2p, hr.ready, 0));
    PL_CUDA(cudaMemcpyAsync(g.block_ptr(u, r.block), g.block_ptr(h, hr.block), packed,
                            cudaMemcpyDefault, dc.p2p));
    g.rep->p2p_bytes += (int64_t)packed;
    PL_CUDA(cudaEventRecord(r.ready, dc.p2p));
    u.p2p_tail = r.ready;
  }
  r.present = true;
  return PARALIA_OK;
}

// Make a tile of A or B readable on unit `ui`; enqueue whatever copies that takes.
template <typename T>
int ensure_input(GemmCall<T>& g, int ui, bool is_a, int64_t i0, int64_t i1) {
  if (std::is_same<T, float>::value) return ensure_input_f32(g, ui, is_a, i0, i1);
  Runtime& rt = Runtime::get();
  UnitState& u = g.units[ui];
  const OperandDesc& op = is_a ? g.A : g.B;
  const int64_t tid = is_a ? i0 * g.Kt + i1 : i0 * g.Nt + i1;
  Resident& r = is_a ? u.a[tid] : u.b[tid];
  if (r.present) return PARALIA_OK;
  const TileGeom<T> t = is_a ? geom_a(g, i0, i1) : geom_b(g, i0, i1);
  if (op.loc == u.dev && (is_a ? u.a_native_ok : u.b_native_ok)) {
    r.present = true;
    r.native = true;
    return PARALIA_OK;
  }
  PL_CUDA(cudaSetDevice(u.dev));
  DeviceCtx& dc = rt.dev(u.dev);
  if (g.grp && op.loc == -1 && (is_a ? g.share_a : g.share_b)) {
    // Group mode: the tile is shared between the processes of this rank's grid row (A) or
    // column (B). Blocks and event slots are fixed functions of the tile so that every
    // process knows where a peer keeps it.
    const int me = g.grp->rank();
    const int slot = is_a ? (int)tid : g.nA + (int)tid;
    const int home = g.group_home(is_a, i0, i1);
    if (home == me) {
      r.block = slot;
      PL_TRY(rt.get_event(u.dev, &r.ready));
      PL_TRY(copy_tile_in(g, u, r.block, t.src, op.ld, t, dc.h2d, &g.rep->h2d_bytes));
      PL_CUDA(cudaEventRecord(r.ready, dc.h2d));
      PL_CUDA(cudaEventRecord(g.grp->own_event(slot), dc.h2d));
      u.h2d_tail = r.ready;
      r.present = true;
      return PARALIA_OK;
    }
    if (g.prefetch_phase) return PARALIA_OK;   // a peer's tile: fetched after the hand-shake
    r.block = slot;
    PL_TRY(rt.get_event(u.dev, &r.ready));
    cudaEvent_t landed;
    PL_TRY(g.grp->peer_event(home, slot, &landed));
    PL_CUDA(cudaStreamWaitEvent(dc.p2p, landed, 0));
    const int peer_slot = is_a ? (int)tid : g.grp->info(home).nA + (int)tid;
    TileGeom<T> tp = t;
    if (t.k_is_row) tp.nr = round_up(t.nr, DG_BK); else tp.nc = round_up(t.nc, DG_BK);
    PL_CUDA(cudaMemcpy2DAsync(g.block_ptr(u, r.block), g.TL * g.esz,
                              g.grp->peer_slab(home) + (size_t)peer_slot * g.block_bytes(),
                              g.TL * g.esz, tp.nr * g.esz, tp.nc, cudaMemcpyDefault, dc.p2p));
    g.rep->p2p_bytes += t.nr * t.nc * g.esz;
    PL_CUDA(cudaEventRecord(r.ready, dc.p2p));
    u.p2p_tail = r.ready;
    r.present = true;
    return PARALIA_OK;
  }
  if (g.grp) r.block = is_a ? (int)tid : g.nA + (int)tid;   // fixed slots in group mode
  else PL_TRY(take_block(g, u, &r.block, is_a ? 1 : 2, tid));
  PL_TRY(rt.get_event(u.dev, &r.ready));
  if (op.loc == -1) {
    // Host-resident tile: one consumer (its "home") pulls it over its host link, the
    // others take it from the home's cache over NVLink.
    const std::vector<int>& cons = is_a ? g.a_consumers[i0] : g.b_consumers[i1];
    int home = ui;
    if (g.peer_fetch && cons.size() > 1) home = cons[g.home_index(is_a, i0, i1)];
    if (home != ui && !rt.peer_ok(u.dev, g.units[home].dev)) home = ui;
    if (home == ui) {
      PL_TRY(copy_tile_in(g, u, r.block, t.src, op.ld, t, dc.h2d, &g.rep->h2d_bytes));
      PL_CUDA(cudaEventRecord(r.ready, dc.h2d));
      u.h2d_tail = r.ready;
    } else {
      PL_TRY(ensure_input(g, home, is_a, i0, i1));
      PL_CUDA(cudaSetDevice(u.dev));
      UnitState& h = g.units[home];
      const Resident& hr = is_a ? h.a[tid] : h.b[tid];
      PL_CUDA(cudaStreamWaitEvent(dc.p2p, hr.ready, 0));
      // The home's block already carries the zero padding: copy the padded extent.
      TileGeom<T> tp = t;
      if (t.k_is_row) tp.nr = round_up(t.nr, DG_BK); else tp.nc = round_up(t.nc, DG_BK);
      PL_CUDA(cudaMemcpy2DAsync(g.block_ptr(u, r.block), g.TL * g.esz, g.block_ptr(h, hr.block),
                                g.TL * g.esz, tp.nr * g.esz, tp.nc, cudaMemcpyDefault, dc.p2p));
      g.rep->p2p_bytes += t.nr * t.nc * g.esz;
      PL_CUDA(cudaEventRecord(r.ready, dc.p2p));
      u.p2p_tail = r.ready;
    }
  } else {
    // Operand lives on a GPU (another one, or this one at an address TMA cannot use).
    PL_TRY(copy_tile_in(g, u, r.block, t.src, op.ld, t, dc.p2p,
                        op.loc == u.dev ? &g.rep->d2d_bytes : &g.rep->p2p_bytes));
    PL_CUDA(cudaEventRecord(r.ready, dc.p2p));
    u.p2p_tail = r.ready;
  }
  r.present = true;
  return PARALIA_OK;
}

// Original C tile of a staged (non-native) C tile, needed by the last k only: fetched
// into its own block behind the inputs of the tile's first k.
template <typename T>
int ensure_csrc(GemmCall<T>& g, int ui, int ct) {
  Runtime& rt = Runtime::get();
  UnitState& u = g.units[ui];
  Resident& rs = u.csrc[ct];
  if (rs.present || u.c_native || g.beta == (T)0) return PARALIA_OK;
  DeviceCtx& dc = rt.dev(u.dev);
  const int64_t mi = ct / g.Nt, ni = ct % g.Nt;
  PL_CUDA(cudaSetDevice(u.dev));
  PL_TRY(take_block(g, u, &rs.block, 3, ct));
  PL_TRY(rt.get_event(u.dev, &rs.ready));
  const char* src = (const char*)g.C.ptr + (mi * g.Tt + ni * g.Tt * g.C.ld) * g.esz;
  const int64_t nr = g.mrows(mi), nc = g.ncols(ni);
  cudaStream_t cs = g.C.loc == -1 ? dc.h2d : dc.p2p;
  PL_CUDA(cudaMemcpy2DAsync(g.block_ptr(u, rs.block), g.TL * g.esz, src, g.C.ld * g.esz,
                            nr * g.esz, nc, cudaMemcpyDefault, cs));
  if (g.C.loc == -1) g.rep->h2d_bytes += nr * nc * g.esz;
  else g.rep->p2p_bytes += nr * nc * g.esz;
  PL_CUDA(cudaEventRecord(rs.ready, cs));
  if (g.C.loc == -1) u.h2d_tail = rs.ready; else u.p2p_tail = rs.ready;
  rs.present = true;
  return PARALIA_OK;
}

// Copy a finished C tile from its cache block to where C lives, after its last kernel.
template <typename T>
int issue_writeback(GemmCall<T>& g, const typename GemmCall<T>::PendingWb& wb) {
  UnitState& u = g.units[wb.ui];
  DeviceCtx& dc = Runtime::get().dev(u.dev);
  PL_CUDA(cudaSetDevice(u.dev));
  PL_CUDA(cudaStreamWaitEvent(dc.d2h, wb.done, 0));
  PL_CUDA(cudaMemcpy2DAsync(wb.dst, wb.dst_ld * g.esz, wb.src, g.TL * g.esz,
                            (size_t)wb.rows * g.esz, wb.cols, cudaMemcpyDefault, dc.d2h));
  if (g.C.loc == -1) g.rep->d2h_bytes += wb.rows * wb.cols * g.esz;
  else g.rep->p2p_bytes += wb.rows * wb.cols * g.esz;
  if (g.evict) {
    // the accumulator and original-C blocks of this tile can be reused once it is home
    cudaEvent_t home;
    PL_TRY(Runtime::get().get_event(u.dev, &home));
    PL_CUDA(cudaEventRecord(home, dc.d2h));
    const int ct = wb.ct;
    for (Resident* r : {&u.c[ct], &u.csrc[ct]})
      if (r->block >= 0) {
        u.blocks[r->block] = UnitState::BlockInfo();
        u.blocks[r->block].freed = home;
        u.free_blocks.push_back(r->block);
        r->block = -1;
      }
  }
  return PARALIA_OK;
}

template <typename T> struct TileKernel;
template <> struct TileKernel<double> { using Args = DgemmArgs; };
template <> struct TileKernel<float> { using Args = SgemmArgs; };

// Enqueue subkernels [ki0, ki1) of C tile `ct` on unit ui as one launch.
template <typename T>
int enqueue_subkernels(GemmCall<T>& g, int ui, int order_idx, int ct, int ki0, int ki1, int band) {
  constexpr bool IS_F64 = std::is_same<T, double>::value;
  Runtime& rt = Runtime::get();
  UnitState& u = g.units[ui];
  DeviceCtx& dc = rt.dev(u.dev);
  const int64_t mi = ct / g.Nt, ni = ct % g.Nt;
  const int sidx = order_idx % g.exec_streams;
  cudaStream_t es = dc.exec[sidx];
  PL_CUDA(cudaSetDevice(u.dev));
  ++u.seq;   // tiles taken from here on belong to this launch and cannot be evicted by it

  typename TileKernel<T>::Args args;
  memset(&args, 0, sizeof(args));
  args.nparts = 0;
  bool a_native = false, b_native = false;
  for (int ki = ki0; ki < ki1; ++ki) {
    if (g.evict) {
      // a tile that is already cached must survive the fetch of its partner
      Resident& pa = u.a[mi * g.Kt + ki];
      Resident& pb = u.b[ki * g.Nt + ni];
      if (pa.present && pa.block >= 0) u.blocks[pa.block].last_seq = u.seq;
      if (pb.present && pb.block >= 0) u.blocks[pb.block].last_seq = u.seq;
    }
    PL_TRY(ensure_input(g, ui, true, mi, ki));
    PL_TRY(ensure_input(g, ui, false, ki, ni));
    PL_CUDA(cudaSetDevice(u.dev));
    const Resident& ra = u.a[mi * g.Kt + ki];
    const Resident& rb = u.b[ki * g.Nt + ni];
    auto& p = args.parts[args.nparts++];
    p.klen = (int32_t)g.klen(ki);
    a_native = ra.native;
    b_native = rb.native;
    if (!ra.native) PL_CUDA(cudaStreamWaitEvent(es, ra.ready, 0));
    if (!rb.native) PL_CUDA(cudaStreamWaitEvent(es, rb.ready, 0));
    if constexpr (IS_F64) {
      if (ra.native) { p.a_m = (int32_t)(mi * g.Tt); p.a_k = (int32_t)(ki * g.Tt); p.a_z = 0; }
      else { p.a_m = 0; p.a_k = 0; p.a_z = ra.block; }
      if (rb.native) { p.b_k = (int32_t)(ki * g.Tt); p.b_n = (int32_t)(ni * g.Tt); p.b_z = 0; }
      else { p.b_k = 0; p.b_n = 0; p.b_z = rb.block; }
    } else {
      p.a_packed = g.block_ptr(u, ra.block);
      p.b_packed = g.block_ptr(u, rb.block);
    }
  }

  const bool first = (ki0 == 0), last = (ki1 == g.Kt);
  Resident& rc = u.c[ct];
  if (!rc.present) {
    rc.present = true;
    if (u.c_native) rc.native = true;
    else PL_TRY(take_block(g, u, &rc.block, 3, ct, es));
  }
  args.M = (int32_t)g.mrows(mi);
  args.N = (int32_t)g.ncols(ni);
  // launches of a band of one or two C tiles have the GPU nearly to themselves
  if constexpr (IS_F64) args.lone = band <= 2 ? 1 : 0;
  args.alpha = g.alpha;
  args.status = dc.status_dev;
  args.Csrc = nullptr;
  args.beta_src = 0;
  if (rc.native) {
    // C lives on this GPU: update it in place, beta on the first k only
    // (the reference switches such tiles to plain WR, dgemm.cpp:262-263).
    args.C = (T*)g.C.ptr + mi * g.Tt + ni * g.Tt * g.C.ld;
    args.ldc = g.C.ld;
    args.beta_c = first ? g.beta : (T)1;
    if constexpr (IS_F64) args.vec_ok = tma_addressable(g.C.ptr, g.C.ld, g.esz) ? 1 : 0;
  } else {
    args.C = (T*)g.block_ptr(u, rc.block);
    args.ldc = g.TL;
    args.beta_c = first ? (T)0 : (T)1;   // WR_LAZY: accumulate from zero (dgemm.cpp:273-279)
    if constexpr (IS_F64) args.vec_ok = 1;
    if (g.beta != (T)0) {
      Resident& rs = u.csrc[ct];
      if (csrc_due(g, ki1)) PL_TRY(ensure_csrc(g, ui, ct));
      if (last) {
        PL_CUDA(cudaStreamWaitEvent(es, rs.ready, 0));
        args.Csrc = (const T*)g.block_ptr(u, rs.block);
        args.ldcsrc = g.TL;
        args.beta_src = g.beta;
      }
    }
  }
  if (!u.first_exec_marked) {
    // lands when everything the first launch waits for has arrived
    PL_CUDA(cudaEventRecord(dc.t_first_exec, es));
    u.first_exec_marked = true;
  }
  if constexpr (IS_F64) {
    const bool a_kc = g.A.trans, b_kc = !g.B.trans;
    const CUtensorMap& mapA = a_native ? u.map_a_native : (a_kc ? u.map_slab_kc : u.map_slab_mn);
    const CUtensorMap& mapB = b_native ? u.map_b_native : (b_kc ? u.map_slab_kc : u.map_slab_mn);
    PL_CUDA(launch_dgemm_tile(mapA, mapB, args, a_kc, b_kc, es));
  } else {
    (void)a_native; (void)b_native;
    PL_CUDA(launch_sgemm_tile(args, sm_count_of(u.dev), es));
  }
  g.rep->kernel_launches += 1;

  cudaEvent_t done;
  PL_TRY(rt.get_event(u.dev, &done));
  PL_CUDA(cudaEventRecord(done, es));
  u.exec_tail[sidx] = done;
  if (g.evict) {
    for (int ki = ki0; ki < ki1; ++ki) {
      const Resident* rr[2] = {&u.a[mi * g.Kt + ki], &u.b[ki * g.Nt + ni]};
      for (const Resident* r : rr)
        if (!r->native && r->block >= 0) {
          u.blocks[r->block].readers[sidx] = done;
          u.blocks[r->block].last_seq = u.seq;
        }
    }
  }
  if (last && !rc.native) {
    // Write the finished tile back to where C lives (reference: WBTileMap, dgemm.cpp:583).
    char* dst = (char*)g.C.ptr + (mi * g.Tt + ni * g.Tt * g.C.ld) * g.esz;
    typename GemmCall<T>::PendingWb wb{ui, ct, done, dst, g.C.ld, g.block_ptr(u, rc.block),
                                      (int64_t)args.M, (int64_t)args.N};
    if (g.defer_wb && g.C.loc == -1) g.pending_wb.push_back(wb);
    else PL_TRY(issue_writeback(g, wb));
  }
  return PARALIA_OK;
}

// The k split of a C tile (plan_kchain_len) is a function of the k tile alone, so the
// arithmetic of a C tile -- and therefore every bit of the result -- is the same whichever
// GPU runs the tile, however many GPUs take part and wherever A and B live. (A C tile that
// lives on the executing GPU is updated in place with beta applied by the first launch
// instead of the last, which rounds differently from a staged tile.)

// The original C tile is needed only by the last launch of its C tile: it is fetched when
// the launch before that one is enqueued (or with the only launch), so that it rides the
// host link behind the A/B tiles that are needed sooner.
template <typename T>
bool csrc_due(const GemmCall<T>& g, int ki1) {
  return ki1 >= (int)g.Kt - 4;
}

// Order of a unit's launches. C tiles are taken in bands (consecutive tiles of the unit's
// distribution order); inside a band all tiles advance through k together: the first k tile
// of every C tile of the band, then the next chain of k tiles of every C tile, and so on.
// A fetched A or B tile is thus used by a whole band row or column of launches straight
// away, which matters while the host link is the bottleneck at start-up; finished bands
// write back while the next band computes. The k split of each C tile is untouched, so
// the arithmetic -- and every bit of the result -- is the same as in tile-major order.
template <typename T>
void build_items(const GemmCall<T>& g, UnitState& u, const GemmModelInput& model_in) {
  // tiles of the unit's first tile row: the unit's list is row-major over its block
  int row_len = 0;
  for (int ct : u.ctiles) {
    if (ct / g.Nt != u.ctiles[0] / g.Nt) break;
    ++row_len;
  }
  int a_sharers = 1, b_sharers = 1, pulling = (int)g.units.size();
  if (g.grp) {
    int d1, d2;
    g.grp->grid(&d1, &d2);
    a_sharers = g.share_a ? d2 : 1;
    b_sharers = g.share_b ? d1 : 1;
    pulling = g.grp->world();
  } else if (g.peer_fetch && !u.ctiles.empty()) {
    a_sharers = (int)g.a_consumers[u.ctiles[0] / g.Nt].size();
    b_sharers = (int)g.b_consumers[u.ctiles[0] % g.Nt].size();
  }
  const BandHints hints = band_hints(model_in, g.Tt, u.dev, pulling, a_sharers, b_sharers, row_len);
  std::vector<int> bands;
  plan_band_sizes((int)u.ctiles.size(), (int)g.Kt, g.evict, hints, &bands);
  // FP32 launches take one k tile each: the tcgen05 kernel streams its packed operand strips
  // through L2 with all CTAs of a launch in step, and they drift apart over longer k loops
  // (measured on a device-resident 40960^3: one k tile per launch 224 TFLOP/s, two 210,
  // four 189). PARALIA_KCHAIN still overrides.
  const int max_chain = std::is_same<T, float>::value && plan_kchain_forced() == 0 ? 1 : DG_MAX_PARTS;
  plan_launch_order(bands, (int)g.Kt, g.evict, max_chain, &u.items);
  u.cursor = 0;
}

template <typename T>
int run_gemm(char TransA, char TransB, int64_t M, int64_t N, int64_t K, T alpha, const T* A,
             int64_t ldA, int locA, const T* B, int64_t ldB, int locB, T beta, T* C, int64_t ldC,
             int locC, const paralia_ctl* ctl, paralia_report* out, const char* func,
             Group* grp = nullptr) {
  const double t_call0 = wall_ms();
  paralia_report local_rep;
  paralia_report* rep = out ? out : &local_rep;
  memset(rep, 0, sizeof(*rep));

  GemmCall<T> g;
  g.rep = rep;
  PL_TRY(norm_trans(TransA, &g.A.trans));
  PL_TRY(norm_trans(TransB, &g.B.trans));
  g.ta = g.A.trans ? 'T' : 'N';
  g.tb = g.B.trans ? 'T' : 'N';
  if (M < 0 || N < 0 || K < 0) return fail(PARALIA_ERR_INVALID_ARG, "negative dimension");
  g.M = M; g.N = N; g.K = K; g.alpha = alpha; g.beta = beta;
  g.A.ptr = A; g.A.ld = ldA; g.A.rows = g.A.trans ? K : M; g.A.cols = g.A.trans ? M : K;
  g.B.ptr = B; g.B.ld = ldB; g.B.rows = g.B.trans ? N : K; g.B.cols = g.B.trans ? K : N;
  g.C.ptr = C; g.C.ld = ldC; g.C.rows = M; g.C.cols = N;
  if (ldA < std::max<int64_t>(1, g.A.rows) || ldB < std::max<int64_t>(1, g.B.rows) ||
      ldC < std::max<int64_t>(1, M))
    return fail(PARALIA_ERR_INVALID_ARG, "leading dimension smaller than the stored row count");
  if (M == 0 || N == 0) return PARALIA_OK;
  if ((!A && K > 0) || (!B && K > 0) || !C) return fail(PARALIA_ERR_INVALID_ARG, "NULL operand");
  if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX)
    return fail(PARALIA_ERR_INVALID_ARG, "dimension exceeds 2^31-1");

  Runtime& rt = Runtime::get();
  PL_TRY(rt.init());
  std::lock_guard<std::mutex> call_lock(rt.call_mutex());
  DeviceGuard dev_guard;
  const int ngpu = rt.device_count();

  double pin_ms = 0.0;
  int rc = PARALIA_OK;
  // a column-major matrix spans ld*(cols-1) + rows elements, not ld*cols
  const size_t spanA = K > 0 ? matrix_span_bytes(g.A.ld, g.A.rows, g.A.cols, g.esz) : 0;
  const size_t spanB = K > 0 ? matrix_span_bytes(g.B.ld, g.B.rows, g.B.cols, g.esz) : 0;
  const size_t spanC = matrix_span_bytes(g.C.ld, M, N, g.esz);
  if (K > 0) {
    rc = resolve_operand_location(g.A.ptr, locA, spanA, ngpu, &g.A.loc, nullptr, nullptr);
    if (rc == PARALIA_OK) rc = resolve_operand_location(g.B.ptr, locB, spanB, ngpu, &g.B.loc, nullptr, nullptr);
  } else {
    g.A.loc = g.B.loc = -1;
  }
  if (rc == PARALIA_OK) rc = resolve_operand_location(g.C.ptr, locC, spanC, ngpu, &g.C.loc, nullptr, nullptr);
  if (rc == PARALIA_OK) {
    // host operands are page-locked together: views of one parent matrix overlap
    HostRange hr[3] = {{g.A.loc == -1 && K > 0 ? g.A.ptr : nullptr, spanA},
                       {g.B.loc == -1 && K > 0 ? g.B.ptr : nullptr, spanB},
                       {g.C.loc == -1 ? g.C.ptr : nullptr, spanC}};
    HostPin pins[3];
    rc = pin_host_ranges(hr, 3, pins, &pin_ms);
    g.A.pin = pins[0]; g.B.pin = pins[1]; g.C.pin = pins[2];
  }
  const bool keep_pinned = ctl && (ctl->flags & PARALIA_FLAG_KEEP_PINNED);
  auto cleanup_pins = [&]() {
    if (!keep_pinned) { unpin(&g.A); unpin(&g.B); unpin(&g.C); }
  };
  if (rc != PARALIA_OK) { cleanup_pins(); return rc; }
  rep->pin_ms = pin_ms;

  // ------------------------------ plan ------------------------------
  const double t_plan0 = wall_ms();
  GemmModelInput mi_in;
  mi_in.esz = g.esz; mi_in.ta = g.ta; mi_in.tb = g.tb;
  mi_in.M = M; mi_in.N = N; mi_in.K = std::max<int64_t>(K, 1);
  mi_in.locA = g.A.loc; mi_in.locB = g.B.loc; mi_in.locC = g.C.loc;
  mi_in.beta_nonzero = beta != (T)0;
  mi_in.func = func;
  paralia_ctl eff_ctl;
  memset(&eff_ctl, 0, sizeof(eff_ctl));
  if (ctl) eff_ctl = *ctl;
  if (eff_ctl.T > 0) {
    // Tiles that are not the whole problem must be a multiple of the 16-deep pipeline stage.
    const int64_t maxdim = std::max(M, std::max(N, mi_in.K));
    if (eff_ctl.T < maxdim && (eff_ctl.T % DG_BK)) eff_ctl.T = std::max<int64_t>(DG_BK, eff_ctl.T - eff_ctl.T % DG_BK);
  }
  if (grp) {
    // one process, one GPU: the rank's own block of the problem runs on the group's GPU
    eff_ctl.active_unit_num = 1;
    eff_ctl.active_unit_id_list[0] = grp->dev();
    g.grp = grp;
  }
  // Problem-metadata reuse (reference: PMD_cache keyed by transposes, dimensions and
  // operand locations, dgemm.cpp:342-380): a signature seen before skips the autotuner.
  struct CachedPlan { paralia_report tuned; };
  static std::map<std::string, CachedPlan> plan_cache;   // guarded by the call mutex
  char sig[256];
  snprintf(sig, sizeof(sig), "%s|%c%c|%lld,%lld,%lld|%d,%d,%d|T%lld|u%d:", func, g.ta, g.tb,
           (long long)M, (long long)N, (long long)K, g.A.loc, g.B.loc, g.C.loc,
           (long long)eff_ctl.T, eff_ctl.active_unit_num);
  std::string key(sig);
  for (int i = 0; i < eff_ctl.active_unit_num && i < PARALIA_MAX_UNITS; ++i)
    key += std::to_string(eff_ctl.active_unit_id_list[i]) + ",";
  key += model_db().from_disk ? model_db().dir : std::string("defaults");
  paralia_report tuned;
  bool reused = false;
  auto hit = plan_cache.find(key);
  if (hit != plan_cache.end() && !(eff_ctl.flags & PARALIA_FLAG_NO_METADATA_REUSE)) {
    tuned = hit->second.tuned;
    reused = true;
  } else {
    if (grp && grp->world() > 1 && eff_ctl.T <= 0) {
      // The tile edge of a group call is chosen for the whole problem on all ranks' GPUs (this
      // rank's block times the device grid), not for one GPU working alone on its block: the
      // ranks share the host link, so the fill, drain and link terms are those of the group.
      // Every rank has a block of the same shape and so arrives at the same T.
      int gd1, gd2;
      grp->grid(&gd1, &gd2);
      GemmModelInput whole = mi_in;
      whole.M = M * gd1;
      whole.N = N * gd2;
      whole.enqueue_threads = grp->world();   // every rank enqueues its own block
      paralia_ctl all = eff_ctl;
      all.active_unit_num = std::min(grp->world(), PARALIA_MAX_UNITS);
      for (int i = 0; i < all.active_unit_num; ++i) all.active_unit_id_list[i] = i;
      paralia_report whole_rep;
      rc = autotune_gemm(whole, all.active_unit_num, &all, &whole_rep);
      if (rc != PARALIA_OK) { cleanup_pins(); return rc; }
      eff_ctl.T = whole_rep.T;
      rc = autotune_gemm(mi_in, ngpu, &eff_ctl, &tuned);
      tuned.pred_t = whole_rep.pred_t;
    } else {
      rc = autotune_gemm(mi_in, ngpu, &eff_ctl, &tuned);
    }
    if (rc != PARALIA_OK) { cleanup_pins(); return rc; }
    if (plan_cache.size() >= 100) plan_cache.clear();   // reference: PROBLEM_MD_CACHE = 100
    plan_cache[key] = CachedPlan{tuned};
  }
  g.Tt = tuned.T;
  if (g.Tt % DG_BK && g.Tt < std::max(M, std::max(N, mi_in.K)))
    g.Tt = std::max<int64_t>(DG_BK, g.Tt - g.Tt % DG_BK);
  g.TL = round_up(g.Tt, DG_BK);
  g.Mt = ceil_div(M, g.Tt); g.Nt = ceil_div(N, g.Tt); g.Kt = K > 0 ? ceil_div(K, g.Tt) : 0;
  g.exec_streams = eff_ctl.exec_streams > 0 ? std::min(eff_ctl.exec_streams, MAX_EXEC_STREAMS) : 4;
  g.peer_fetch = !(eff_ctl.flags & PARALIA_FLAG_NO_PEER_FETCH);

  std::vector<std::vector<int>> lists;
  int d1 = 1, d2 = 1;
  const int kt_for_ids = (int)std::max<int64_t>(g.Kt, 1);
  int active = distribute_subkernels_2d(tuned.active_unit_num, (int)g.Mt, (int)g.Nt, kt_for_ids,
                                        &lists, &d1, &d2);
  if (active <= 0) { cleanup_pins(); return fail(PARALIA_ERR_INVALID_ARG, "subkernel distribution failed"); }
  *rep = tuned;
  rep->T = g.Tt;
  rep->active_unit_num = active;
  rep->grid_d1 = d1; rep->grid_d2 = d2;
  rep->subkernel_num = g.Mt * g.Nt * kt_for_ids;
  rep->pin_ms = pin_ms;
  rep->metadata_reused = reused ? 1 : 0;
  rep->cache_limit = eff_ctl.cache_limit;

  g.units.assign(active, UnitState());
  g.a_consumers.assign(g.Mt, std::vector<int>());
  g.b_consumers.assign(g.Nt, std::vector<int>());
  {
    lists.resize(active);
    std::vector<std::vector<int>> unit_ctiles;
    if (!plan_unit_ctiles(lists, kt_for_ids, (int)(g.Mt * g.Nt), &unit_ctiles, &g.ctile_owner)) {
      cleanup_pins();
      return fail(PARALIA_ERR_UNSUPPORTED, "distribution split one C tile across units");
    }
    for (int ui = 0; ui < active; ++ui) {
      UnitState& u = g.units[ui];
      u.dev = tuned.active_unit_id_list[ui];
      rep->subkernels_per_unit[ui] = (int)lists[ui].size();
      rep->active_unit_score[ui] = 1.0 / active;
      u.ctiles = unit_ctiles[ui];
    }
  }
  for (int64_t ct = 0; ct < g.Mt * g.Nt; ++ct) {
    const int ui = g.ctile_owner[ct];
    auto add = [](std::vector<int>& v, int x) {
      if (std::find(v.begin(), v.end(), x) == v.end()) v.push_back(x);
    };
    add(g.a_consumers[ct / g.Nt], ui);
    add(g.b_consumers[ct % g.Nt], ui);
  }
  g.grid_d1 = d1; g.grid_d2 = d2;
  g.a_first.assign(g.Mt, 0);
  g.b_first.assign(g.Nt, 0);
  for (int64_t mi = 1; mi < g.Mt; ++mi)
    g.a_first[mi] = g.a_consumers[mi] == g.a_consumers[mi - 1] ? g.a_first[mi - 1] : (int)mi;
  for (int64_t ni = 1; ni < g.Nt; ++ni)
    g.b_first[ni] = g.b_consumers[ni] == g.b_consumers[ni - 1] ? g.b_first[ni - 1] : (int)ni;

  // ------------------------------ resources ------------------------------
  double alloc_ms = 0.0;
  auto fail_out = [&](int code) { cleanup_pins(); return code; };
  for (int ui = 0; ui < active; ++ui) {
    UnitState& u = g.units[ui];
    rc = rt.ensure_device(u.dev);
    if (rc != PARALIA_OK) return fail_out(rc);
    rt.release_events(u.dev);
    u.a.assign(g.Mt * std::max<int64_t>(g.Kt, 1), Resident());
    u.b.assign(std::max<int64_t>(g.Kt, 1) * g.Nt, Resident());
    u.c.assign(g.Mt * g.Nt, Resident());
    u.csrc.assign(g.Mt * g.Nt, Resident());
    u.exec_tail.assign(g.exec_streams, nullptr);
    // FP32 tiles are always packed into cache blocks, never read in place
    const bool in_place_ok = std::is_same<T, double>::value;
    u.a_native_ok = in_place_ok && g.A.loc == u.dev && tma_addressable(g.A.ptr, g.A.ld, g.esz);
    u.b_native_ok = in_place_ok && g.B.loc == u.dev && tma_addressable(g.B.ptr, g.B.ld, g.esz);
    u.c_native = g.C.loc == u.dev;
    // Blocks this unit needs if nothing is ever evicted: the A tile rows and B tile
    // columns of its C tiles, plus accumulator (and original-C) blocks
    // (reference sizing: 1 + At + Bt + 2*Ct, dgemm.cpp:80-87).
    std::vector<char> rows(g.Mt, 0), cols(g.Nt, 0);
    for (int ct : u.ctiles) { rows[ct / g.Nt] = 1; cols[ct % g.Nt] = 1; }
    int64_t need = 0;
    if (!u.a_native_ok) for (int64_t r = 0; r < g.Mt; ++r) if (rows[r]) need += g.Kt;
    if (!u.b_native_ok) for (int64_t c = 0; c < g.Nt; ++c) if (cols[c]) need += g.Kt;
    // (a home GPU is always a consumer of the tiles it forwards, so it needs no extra blocks)
    if (!u.c_native) need += (int64_t)u.ctiles.size() * ((beta != (T)0) ? 2 : 1);
    // The slab is clamped by the caller's cache_limit and by what the GPU has left
    // (reference: min(cache_limit, free - 30 % of total), dgemm.cpp:53-54,80-87; here 90 %
    // of free memory plus the slab already held). A clamped slab recycles its blocks.
    int64_t cap = need;
    if (eff_ctl.cache_limit > 0) cap = std::min<int64_t>(cap, eff_ctl.cache_limit / (int64_t)g.block_bytes());
    // (a slab that already holds the working set needs no look at the free memory; the query
    // costs about a millisecond per GPU)
    if ((size_t)need * g.block_bytes() > rt.dev(u.dev).slab_bytes) {
      size_t free_b = 0, total_b = 0;
      if (cudaSetDevice(u.dev) == cudaSuccess && cudaMemGetInfo(&free_b, &total_b) == cudaSuccess) {
        const double avail = 0.9 * ((double)free_b + (double)rt.dev(u.dev).slab_bytes);
        cap = std::min<int64_t>(cap, (int64_t)(avail / (double)g.block_bytes()));
      } else {
        cudaGetLastError();
      }
    }
    if (cap < need) {
      const int64_t min_blocks = (u.c_native ? 0 : (beta != (T)0 ? 2 : 1)) +
                                 (u.a_native_ok ? 0 : 1) + (u.b_native_ok ? 0 : 1);
      if (grp)
        return fail_out(fail(PARALIA_ERR_OUT_OF_MEMORY,
                             "GPU %d: the tile cache (%lld of %lld blocks) is too small; process "
                             "groups need the whole working set cached",
                             u.dev, (long long)cap, (long long)need));
      if (cap < min_blocks)
        return fail_out(fail(PARALIA_ERR_OUT_OF_MEMORY,
                             "GPU %d needs at least %lld cache blocks of %zu bytes but only %lld fit "
                             "(cache_limit %lld)",
                             u.dev, (long long)min_blocks, g.block_bytes(), (long long)cap,
                             (long long)eff_ctl.cache_limit));
      g.evict = true;
      g.peer_fetch = false;   // every GPU fetches for itself: a block may be recycled at any time
    }
    u.nblocks = (int)cap;
    u.blocks.assign((size_t)cap, UnitState::BlockInfo());
    u.free_blocks.clear();
    size_t bytes = (size_t)cap * g.block_bytes();
    if (grp) {
      // collective: agree on sharing, exchange slab handles (group.hpp)
      g.nA = u.a_native_ok ? 0 : (int)(g.Mt * g.Kt);
      g.nB = u.b_native_ok ? 0 : (int)(g.Kt * g.Nt);
      u.next_block = g.nA + g.nB;
      GroupCallInfo info;
      memset(&info, 0, sizeof(info));
      info.Mloc = M; info.Nloc = N; info.K = K; info.T = g.Tt; info.TL = g.TL;
      info.ta = g.A.trans; info.tb = g.B.trans; info.esz = g.esz;
      info.a_host = g.A.loc == -1 && K > 0; info.b_host = g.B.loc == -1 && K > 0;
      info.nA = g.nA; info.nB = g.nB;
      info.want_share = g.peer_fetch ? 1 : 0;
      rc = grp->begin_call(info, bytes, &alloc_ms, &g.share_a, &g.share_b);
      if (rc != PARALIA_OK) return fail_out(rc);
    }
    if (bytes > 0) {
      rc = rt.ensure_slab(u.dev, bytes, &alloc_ms);
      if (rc != PARALIA_OK) return fail_out(rc);
      DeviceCtx& dc = rt.dev(u.dev);
      if (std::is_same<T, double>::value) {
        const uint64_t nb = dc.slab_bytes / g.block_bytes();
        rc = make_tensor_map(&u.map_slab_kc, dc.slab, g.esz, g.TL, g.TL, nb, g.TL * g.esz,
                             g.block_bytes(), 16, DG_KC_BOX_ROWS);
        if (rc == PARALIA_OK)
          rc = make_tensor_map(&u.map_slab_mn, dc.slab, g.esz, g.TL, g.TL, nb, g.TL * g.esz,
                               g.block_bytes(), 16, 16);
        if (rc != PARALIA_OK) return fail_out(rc);
      }
    }
    if (std::is_same<T, float>::value && K > 0) {
      rc = rt.ensure_stage(u.dev, (size_t)g.Tt * g.Tt * g.esz);
      if (rc != PARALIA_OK) return fail_out(rc);
    }
    if (u.a_native_ok && K > 0) {
      rc = make_tensor_map(&u.map_a_native, g.A.ptr, g.esz, g.A.rows, g.A.cols, 1, g.A.ld * g.esz,
                           (uint64_t)g.A.ld * g.A.cols * g.esz, 16, g.A.trans ? DG_KC_BOX_ROWS : 16);
      if (rc != PARALIA_OK) return fail_out(rc);
    }
    if (u.b_native_ok && K > 0) {
      rc = make_tensor_map(&u.map_b_native, g.B.ptr, g.esz, g.B.rows, g.B.cols, 1, g.B.ld * g.esz,
                           (uint64_t)g.B.ld * g.B.cols * g.esz, 16, g.B.trans ? 16 : DG_KC_BOX_ROWS);
      if (rc != PARALIA_OK) return fail_out(rc);
    }
  }
  rep->alloc_ms = alloc_ms;
  rep->plan_ms = wall_ms() - t_plan0 - alloc_ms;

  // ------------------------------ enqueue ------------------------------
  {
    // operands the caller produced on the default stream of a GPU are ready before we read
    std::vector<int> op_devs = {g.A.loc, g.B.loc, g.C.loc}, unit_devs;
    for (int ui = 0; ui < active; ++ui) {
      op_devs.push_back(g.units[ui].dev);
      unit_devs.push_back(g.units[ui].dev);
    }
    const int orc = rt.order_after_caller(op_devs, unit_devs);
    if (orc != PARALIA_OK) return fail_out(orc);
  }
  for (int ui = 0; ui < active; ++ui) {
    UnitState& u = g.units[ui];
    DeviceCtx& dc = rt.dev(u.dev);
    if (cudaSetDevice(u.dev) != cudaSuccess || cudaEventRecord(dc.t_begin, dc.h2d) != cudaSuccess)
      return fail_out(fail(PARALIA_ERR_CUDA, "cannot record the start event on GPU %d", u.dev));
    // Nothing of this call may start before the start event.
    for (int s = 0; s < g.exec_streams; ++s) cudaStreamWaitEvent(dc.exec[s], dc.t_begin, 0);
    cudaStreamWaitEvent(dc.p2p, dc.t_begin, 0);
    cudaStreamWaitEvent(dc.pack, dc.t_begin, 0);
    cudaStreamWaitEvent(dc.d2h, dc.t_begin, 0);
  }
  for (int ui = 0; ui < active; ++ui) build_items(g, g.units[ui], mi_in);
  // With four or more GPUs pulling from the host at once, this class of host delivers far
  // less in both directions together than in one direction alone (measured on an
  // 8 x B200 box: 185 GB/s host->GPU alone, 63 + 63 GB/s with GPU->host traffic running),
  // so C tiles are written back only after the unit's input stream has drained; with
  // fewer GPUs the two directions overlap well and tiles go back as they finish. The
  // decision is read off the calibration database's host aggregate table.
  {
    const char* e = getenv("PARALIA_DEFER_WB");
    g.defer_wb = e ? atoi(e) != 0 : defer_writebacks(grp ? grp->world() : active);
    if (g.evict) g.defer_wb = false;   // blocks are needed back as soon as a tile is home
  }
  if (grp) {
    // Group mode, phase 1: enqueue the host fetches of the tiles this rank is the home of
    // (in the order its own kernels will want them) and record their inter-process
    // events; after the barrier every rank may wait on any peer's events.
    if ((g.share_a || g.share_b) && g.Kt > 0) {
      g.prefetch_phase = true;
      UnitState& u = g.units[0];
      for (size_t it = 0; it < u.items.size() && rc == PARALIA_OK; ++it) {
        const UnitState::Item item = u.items[it];
        const int ct = u.ctiles[item.order_idx];
        const int64_t mi = ct / g.Nt, ni = ct % g.Nt;
        for (int64_t ki = item.ki0; ki < item.ki1 && rc == PARALIA_OK; ++ki) {
          rc = ensure_input(g, 0, true, mi, ki);
          if (rc == PARALIA_OK) rc = ensure_input(g, 0, false, ki, ni);
        }
        // keep the host link's queue in the order of use (same rule as the launch path)
        if (rc == PARALIA_OK && csrc_due(g, item.ki1)) rc = ensure_csrc(g, 0, ct);
      }
      g.prefetch_phase = false;
    }
    const int brc = grp->barrier();
    if (rc == PARALIA_OK) rc = brc;
  }
  // Round-robin over the GPUs, one launch per turn (the reference's fire loop walks the
  // devices the same way, dgemm.cpp:516-544).
  bool work_left = rc == PARALIA_OK;
  while (work_left) {
    work_left = false;
    for (int ui = 0; ui < active; ++ui) {
      UnitState& u = g.units[ui];
      if (u.cursor >= u.items.size()) continue;
      const UnitState::Item item = u.items[u.cursor++];
      rc = enqueue_subkernels<T>(g, ui, item.order_idx, u.ctiles[item.order_idx], item.ki0,
                                 item.ki1, item.band);
      if (rc != PARALIA_OK) break;
      if (u.cursor < u.items.size()) work_left = true;
    }
    if (rc != PARALIA_OK) break;
  }
  if (rc == PARALIA_OK && !g.pending_wb.empty()) {
    for (int ui = 0; ui < active; ++ui) {
      UnitState& u = g.units[ui];
      if (u.h2d_tail) {
        cudaSetDevice(u.dev);
        cudaStreamWaitEvent(rt.dev(u.dev).d2h, u.h2d_tail, 0);
      }
    }
    for (const auto& wb : g.pending_wb) {
      rc = issue_writeback(g, wb);
      if (rc != PARALIA_OK) break;
    }
  }
  // ------------------------------ join ------------------------------
  double dev_ms = 0.0;
  for (int ui = 0; ui < active; ++ui) {
    UnitState& u = g.units[ui];
    DeviceCtx& dc = rt.dev(u.dev);
    cudaSetDevice(u.dev);
    if (rc == PARALIA_OK) {
      for (int s = 0; s < g.exec_streams; ++s)
        if (u.exec_tail[s]) cudaEventRecord(dc.t_exec_end[s], dc.exec[s]);
      cudaEventRecord(dc.t_h2d_end, dc.h2d);
      for (int s = 0; s < g.exec_streams; ++s)
        if (u.exec_tail[s]) cudaStreamWaitEvent(dc.d2h, u.exec_tail[s], 0);
      if (u.h2d_tail) cudaStreamWaitEvent(dc.d2h, u.h2d_tail, 0);
      if (u.p2p_tail) cudaStreamWaitEvent(dc.d2h, u.p2p_tail, 0);
      if (u.pack_tail) cudaStreamWaitEvent(dc.d2h, u.pack_tail, 0);
      cudaEventRecord(dc.t_end, dc.d2h);
    }
  }
  for (int ui = 0; ui < active; ++ui) {
    UnitState& u = g.units[ui];
    DeviceCtx& dc = rt.dev(u.dev);
    cudaSetDevice(u.dev);
    // the end event of a unit follows everything the unit enqueued; the wait is bounded
    // (a copy that never completes must not hang the caller)
    if (rc == PARALIA_OK) rc = wait_event_with_deadline(dc.t_end, join_deadline_ms(rep->pred_t), u.dev);
    else cudaDeviceSynchronize();
    if (rc == PARALIA_OK) {
      float ms = 0.f;
      if (cudaEventElapsedTime(&ms, dc.t_begin, dc.t_end) == cudaSuccess)
        dev_ms = std::max(dev_ms, (double)ms);
      if (u.first_exec_marked && cudaEventElapsedTime(&ms, dc.t_begin, dc.t_first_exec) == cudaSuccess)
        rep->fill_ms = std::max(rep->fill_ms, (double)ms);
      for (int s = 0; s < g.exec_streams; ++s)
        if (u.exec_tail[s] && cudaEventElapsedTime(&ms, dc.t_begin, dc.t_exec_end[s]) == cudaSuccess)
          rep->exec_end_ms = std::max(rep->exec_end_ms, (double)ms);
      if (cudaEventElapsedTime(&ms, dc.t_begin, dc.t_h2d_end) == cudaSuccess)
        rep->h2d_end_ms = std::max(rep->h2d_end_ms, (double)ms);
      cudaGetLastError();
    }
  }
  if (rc == PARALIA_OK)
    for (int ui = 0; ui < active && rc == PARALIA_OK; ++ui) rc = rt.check_status(g.units[ui].dev);
  if (grp) {
    // no rank may start overwriting its slab while a peer still copies out of it
    const int brc = grp->barrier();
    if (rc == PARALIA_OK) rc = brc;
  }
  cleanup_pins();
  rep->device_ms = dev_ms;
  rep->host_ms = wall_ms() - t_call0;
  return rc;
}

// A collective call of one rank: whatever makes this rank leave the call early (a bad
// argument, an allocation that fails, a CUDA error) is published to the group, so that the
// peers -- which are inside, or about to enter, the call's hand-shakes -- return an error at
// once instead of waiting out a time-out.
template <typename Fn>
int group_call(Group* grp, int64_t Mloc, int64_t Nloc, Fn&& run) {
  if (grp->poisoned()) return grp->barrier();   // reports why the group was abandoned
  int rc;
  if (Mloc <= 0 || Nloc <= 0)
    rc = fail(PARALIA_ERR_INVALID_ARG, "a rank's block of C is empty (%lld x %lld)", (long long)Mloc,
              (long long)Nloc);
  else
    rc = run();
  if (rc != PARALIA_OK && rc != PARALIA_ERR_GROUP_FAILED) grp->poison(last_error_cstr());
  return rc;
}

}  // namespace

int exec_dgemm(char ta, char tb, int64_t M, int64_t N, int64_t K, double alpha, const double* A,
               int64_t ldA, int locA, const double* B, int64_t ldB, int locB, double beta,
               double* C, int64_t ldC, int locC, const paralia_ctl* ctl, paralia_report* out) {
  return run_gemm<double>(ta, tb, M, N, K, alpha, A, ldA, locA, B, ldB, locB, beta, C, ldC, locC,
                          ctl, out, "Dgemm");
}

int exec_sgemm(char ta, char tb, int64_t M, int64_t N, int64_t K, float alpha, const float* A,
               int64_t ldA, int locA, const float* B, int64_t ldB, int locB, float beta, float* C,
               int64_t ldC, int locC, const paralia_ctl* ctl, paralia_report* out) {
  return run_gemm<float>(ta, tb, M, N, K, alpha, A, ldA, locA, B, ldB, locB, beta, C, ldC, locC,
                         ctl, out, "Sgemm");
}

int exec_group_dgemm(char ta, char tb, int64_t M, int64_t N, int64_t K, double alpha,
                     const double* A, int64_t ldA, int locA, const double* B, int64_t ldB,
                     int locB, double beta, double* C, int64_t ldC, int locC,
                     const paralia_ctl* ctl, paralia_report* out) {
  Group* grp = Group::current();
  if (!grp) return fail(PARALIA_ERR_INVALID_ARG, "PARALiA_group_init has not been called");
  return group_call(grp, M, N, [&]() {
    return run_gemm<double>(ta, tb, M, N, K, alpha, A, ldA, locA, B, ldB, locB, beta, C, ldC, locC,
                          ctl, out, "Dgemm", grp);
  });
}

int exec_group_sgemm(char ta, char tb, int64_t M, int64_t N, int64_t K, float alpha, const float* A,
                     int64_t ldA, int locA, const float* B, int64_t ldB, int locB, float beta,
                     float* C, int64_t ldC, int locC, const paralia_ctl* ctl, paralia_report* out) {
  Group* grp = Group::current();
  if (!grp) return fail(PARALIA_ERR_INVALID_ARG, "PARALiA_group_init has not been called");
  return group_call(grp, M, N, [&]() {
    return run_gemm<float>(ta, tb, M, N, K, alpha, A, ldA, locA, B, ldB, locB, beta, C, ldC, locC,
                          ctl, out, "Sgemm", grp);
  });
}

}  // namespace paralia
