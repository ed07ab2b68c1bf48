// Host-visible interface of the FP32 tile GEMM: 3xTF32 on the tcgen05 tensor path.
//
// Every FP32 operand tile is first "packed": split into a TF32-exact high part and a
// TF32-exact low part (x = hi + lo + O(2^-22 |x|)) and laid out in the order the tensor
// core reads shared memory, so that the GEMM kernel can move it with plain bulk copies.
// The GEMM kernel then accumulates lo*hi + hi*lo + hi*hi in FP32 in tensor memory.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace paralia {

constexpr int SG_BM = 128;       // rows of C per CTA tile (one MMA M)
constexpr int SG_BN = 256;       // columns of C per CTA tile (one MMA N)
constexpr int SG_BK = 16;        // k per pipeline stage (two K=8 TF32 MMAs)
constexpr int SG_STAGES = 4;
constexpr int SG_THREADS = 192;  // warp 0 copies, warp 1 issues MMAs, warps 2-5 epilogue
constexpr int SG_A_CHUNK = SG_BM * SG_BK * 4 * 2;   // hi + lo plane of an A stage: 16 KB
constexpr int SG_B_CHUNK = SG_BN * SG_BK * 4 * 2;   // hi + lo plane of a B stage: 32 KB
constexpr int SG_STAGE_BYTES = SG_A_CHUNK + SG_B_CHUNK;
constexpr int SG_SMEM_BYTES = SG_STAGES * SG_STAGE_BYTES + 1024;
constexpr int SG_MAX_PARTS = 64;
constexpr int SG_PANEL = 8;      // column strips per panel of the CTA tile numbering

// Bytes of the packed form of a tile with `rows` rows and `klen` k values, for an operand
// packed in blocks of `rb` rows (SG_BM for A, SG_BN for B).
inline size_t sgemm_packed_bytes(int64_t rows, int64_t klen, int rb) {
  const int64_t rblocks = (rows + rb - 1) / rb, kblocks = (klen + SG_BK - 1) / SG_BK;
  return (size_t)rblocks * kblocks * rb * SG_BK * 4 * 2;
}

// Pack a rows x klen operand tile. Element (r, k) is read from src[k + r*ld] when
// k_contig, else from src[r + k*ld]. Output chunk (row block, k block) is contiguous:
// [hi plane][lo plane], each plane in core-matrix order [k/4][row/8][row%8][k%4].
cudaError_t launch_sgemm_pack(const float* src, int64_t ld, bool k_contig, int rows, int klen,
                              int rb, void* packed, cudaStream_t stream);

struct SgemmKPart {
  const void* a_packed;   // A tile packed with SG_BM-row blocks
  const void* b_packed;   // B tile packed with SG_BN-row blocks
  int32_t klen;
  int32_t pad;
};

struct SgemmArgs {
  float* C;
  const float* Csrc;
  int64_t ldc, ldcsrc;
  float alpha, beta_c, beta_src;
  int32_t M, N;
  int32_t nparts;
  int* status;
  // Work items, filled in by launch_sgemm_tile (sgemm_tile_schedule): whole CTA tiles, then
  // halves of the CTA tiles that follow.
  int32_t whole_items, half_items;
  SgemmKPart parts[SG_MAX_PARTS];
};

// The static work list of a launch over an M x N C tile on a GPU with `sms` SMs.
void sgemm_tile_schedule(int M, int N, int sms, int* whole_items, int* half_items, int* grid);

cudaError_t launch_sgemm_tile(const SgemmArgs& args, int sm_count, cudaStream_t stream);

// Tensor-pipe throughput loop of the GEMM kernel's MMA shape on shared-memory-resident
// operands: every block issues `stages` x 6 tcgen05.mma.kind::tf32 of 128 x 256 x 8
// (2 * 128 * 256 * 8 flop each). `status` receives a KERR_* code if a wait gives up.
// `random_operands`: fill the stage with TF32-exact uniform(-1, 1) values instead of ones, so
// that the figure includes what the board's power limit does to a real product.
cudaError_t launch_tf32_peak(int stages, int blocks, bool random_operands, int* status,
                             cudaStream_t stream);
constexpr double SG_PEAK_FLOP_PER_STAGE = 6.0 * 2.0 * SG_BM * SG_BN * 8;

// Opt the kernels into their dynamic shared memory size; once per device.
cudaError_t sgemm_tile_configure();

}  // namespace paralia
