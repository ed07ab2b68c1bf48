// Host-visible description of one launch of the FP64 tile GEMM kernel.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace paralia {

// CTA tile and pipeline shape of the DMMA kernel.
constexpr int DG_BM = 128;      // rows of C per CTA
constexpr int DG_BN = 128;      // columns of C per CTA
constexpr int DG_BK = 16;       // k per pipeline stage (16 doubles = one 128-byte swizzle row)
constexpr int DG_STAGES = 6;    // 6 x 32 KB of operand tiles in flight
constexpr int DG_CONSUMER_WARPS = 8;
// Three CTA shapes of the same kernel (same stages, same arithmetic, same result bits):
//   DG_MODE_WARP   one extra warp is the TMA producer (288 threads; three warps share one
//                  scheduler's registers, so a thread gets at most 168);
//   DG_MODE_FOLD   no producer warp: lane 0 of consumer warp 0 issues the loads between its
//                  own MMAs (256 threads, up to 255 registers per thread);
//   DG_MODE_GROUP  a whole producer warpgroup that hands most of its registers to the
//                  consumers with setmaxnreg (384 threads, consumers run with 232).
// Which one is fastest depends on the storage order of the operands (how many TMA boxes a
// stage takes and how the fragment loads are addressed); launch_dgemm_tile picks by
// measurement, see dgemm_mode_for().
enum : int { DG_MODE_WARP = 0, DG_MODE_FOLD = 1, DG_MODE_GROUP = 2 };
constexpr int dg_threads(int mode) {
  return (DG_CONSUMER_WARPS + (mode == DG_MODE_FOLD ? 0 : (mode == DG_MODE_GROUP ? 4 : 1))) * 32;
}
constexpr int DG_FOLD_LAG = 2;  // fold: a stage is refilled this many iterations after its use
constexpr int DG_STAGE_BYTES = (DG_BM + DG_BN) * DG_BK * 8;
constexpr int DG_SMEM_BYTES = DG_STAGES * DG_STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
constexpr int DG_MAX_PARTS = 64;
constexpr int DG_PANEL = 12;    // tile columns per panel of the CTA tile numbering

// One slice of the K loop: where the A and B tiles of that slice start inside the
// tensors their TMA maps describe. (row, k, z) for A and (k, col, z) for B are logical
// GEMM coordinates; z selects a block of the tile cache (0 for a user matrix).
struct DgemmKPart {
  int32_t a_m, a_k, a_z;
  int32_t b_k, b_n, b_z;
  int32_t klen;
};

struct DgemmArgs {
  double* C;            // accumulator / output tile, column-major
  const double* Csrc;   // optional second source added as beta_src*Csrc (may be null)
  int64_t ldc, ldcsrc;
  double alpha, beta_c, beta_src;
  int32_t M, N;         // extent of the C tile
  int32_t nparts;
  int32_t vec_ok;       // C and Csrc allow 16-byte accesses
  int* status;          // device word that receives a KERR_* code on a timed-out wait
  int32_t lone;         // the launch is expected to have the GPU to itself: its last partial
                        // round of CTA tiles is cut into quarter items
  // Work items of the launch, filled in by launch_dgemm_tile (dgemm_tile_schedule):
  // items [0, full_items) are 128 x 128 CTA tiles, the next quarter_items are 64 x 64
  // quarters of the CTA tiles that follow; tiles_m / tiles_n = CTA tiles per column / row of C.
  int32_t tiles_m, tiles_n, full_items, quarter_items;
  DgemmKPart parts[DG_MAX_PARTS];
};

// The work list of a launch over an M x N C tile on a GPU with `sms` SMs: how many CTA tiles
// are whole items and how many quarter items follow. The grid is their sum.
void dgemm_tile_schedule(int M, int N, int sms, bool lone, int* tiles_m, int* full_items,
                         int* quarter_items);

// Rows per TMA box of an operand stored with k contiguous (box = 16 k x 128 rows); an
// operand stored row-contiguous uses boxes of 16 rows x 16 k.
constexpr int DG_KC_BOX_ROWS = 128;

// Launch on `stream`. a_kcontig: A is stored with k contiguous (TransA == 'T' for a
// column-major A); b_kcontig: B is stored with k contiguous (TransB == 'N').
cudaError_t launch_dgemm_tile(const CUtensorMap& mapA, const CUtensorMap& mapB,
                              const DgemmArgs& args, bool a_kcontig, bool b_kcontig,
                              cudaStream_t stream);

// Plain-load version for operands TMA cannot address (odd leading dimension or a base
// that is not 16-byte aligned). Same arithmetic, far slower; used only by the direct
// per-tile entry point.
cudaError_t launch_dgemm_generic(char ta, char tb, int M, int N, int K, double alpha,
                                 const double* A, int64_t lda, const double* B, int64_t ldb,
                                 double beta, double* C, int64_t ldc, cudaStream_t stream);

// Opt the kernels into their dynamic shared memory size; once per device.
cudaError_t dgemm_tile_configure();

// One warp waits on an mbarrier that never completes, for at most budget_clocks, then
// writes a KERR_* code to *status: exercises the give-up path of every bounded wait.
cudaError_t launch_bounded_wait_selftest(int* status, long long budget_clocks, cudaStream_t stream);

// Register-only DMMA throughput loop. shape in {884, 1684, 1688, 16816}.
cudaError_t launch_dmma_peak(int shape, int iters, int blocks, double* sink, cudaStream_t stream);

}  // namespace paralia
