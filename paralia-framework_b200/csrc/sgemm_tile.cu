// FP32 tile GEMM for sm_100a as a 3xTF32 split on the tcgen05 tensor path:
//   C_tile = alpha * sum_parts op(A_p) op(B_p) + beta_c*C_tile (+ beta_src*Csrc).
//
// It stands where the reference calls cublasSgemm through backend_run_operation
// (Library_scheduler/src/Functions/sgemm.cpp:85-139). Each FP32 value x is written as
// hi + lo with hi = x rounded to the nearest TF32 number and lo = (x - hi) rounded to the
// nearest TF32 number; both are exact TF32 values and |x - hi - lo| <= 2^-22 |x|. The
// kernel accumulates lo*hi + hi*lo + hi*hi in FP32, which keeps the normwise error of the
// product far inside the 4*K*eps32 budget that a plain FP32 GEMM is allowed.
//
// Pack kernel: splits an operand tile and writes it in the order tcgen05.mma reads shared
// memory for a K-major operand without swizzle: 8 x 16-byte "core matrices"
// (8 rows x 4 k), core matrices of one k group stored row block after row block, so that
//   leading byte offset (next core matrix along k)  = rows_per_block * 16
//   stride  byte offset (next 8 rows)                = 128.
// A (row block, 16-k block) chunk -- hi plane then lo plane -- is one contiguous piece of
// memory, so the GEMM kernel's producer moves a whole pipeline stage with two
// cp.async.bulk copies and needs neither tensor maps nor a transposing variant: every
// storage order of A and B is handled by the pack kernel.
//
// GEMM kernel, one persistent CTA per SM, 192 threads:
//   warp 0   producer: bulk copies of A and B chunks into a 4-stage ring (mbarrier tx);
//   warp 1   allocates tensor memory (512 columns = two 128 x 256 FP32 accumulators),
//            one lane issues tcgen05.mma.kind::tf32 (M=128, N=256, K=8), six per stage,
//            and commits to the stage's "empty" barrier / the accumulator's "full" barrier;
//   warps 2-5 epilogue: tcgen05.ld of the finished accumulator, alpha/beta, coalesced
//            stores to column-major C, while warp 1 already fills the other accumulator.
// Every wait is bounded; on a timeout the CTA records an error word, stops issuing work,
// frees its tensor memory and exits.
#include "sgemm_tile.cuh"

#include <algorithm>

#include "sm100_prims.cuh"

namespace paralia {
using namespace prims;

namespace {

// ------------------------------------------------------------------ pack
// Nearest TF32 number (ties away from zero), returned as an FP32 value whose low 13
// mantissa bits are zero. Rounding to nearest keeps the split error unbiased, so it grows
// with sqrt(K) instead of K.
__device__ __forceinline__ float tf32_round(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r & 0xFFFFE000u);
}

// One thread per (row, group of 4 k): reads four values, writes one 16-byte row of a core
// matrix into the hi plane and one into the lo plane.
__global__ void __launch_bounds__(256)
sgemm_pack_kernel(const float* __restrict__ src, int64_t ld, int k_contig, int rows, int klen,
                  int rb, int rblocks, int kblocks, float* __restrict__ packed) {
  const int64_t total = (int64_t)rblocks * kblocks * rb * (SG_BK / 4);
  const int plane = rb * SG_BK;   // floats per plane
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    // decode so that consecutive threads walk rows first: coalesced 16-byte stores, and
    // coalesced 4-byte loads when rows are contiguous in the source
    const int r_in = (int)(idx % rb);
    int64_t rest = idx / rb;
    const int kc = (int)(rest % (SG_BK / 4));
    rest /= (SG_BK / 4);
    const int kb = (int)(rest % kblocks);
    const int rblk = (int)(rest / kblocks);
    const int row = rblk * rb + r_in;
    const int k0 = kb * SG_BK + kc * 4;
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + j;
      float x = 0.0f;
      if (row < rows && k < klen) x = k_contig ? src[k + (int64_t)row * ld] : src[row + (int64_t)k * ld];
      v[j] = x;
    }
    float4 hi, lo;
    hi.x = tf32_round(v[0]); lo.x = tf32_round(v[0] - hi.x);
    hi.y = tf32_round(v[1]); lo.y = tf32_round(v[1] - hi.y);
    hi.z = tf32_round(v[2]); lo.z = tf32_round(v[2] - hi.z);
    hi.w = tf32_round(v[3]); lo.w = tf32_round(v[3] - hi.w);
    float* chunk = packed + ((int64_t)rblk * kblocks + kb) * (2 * plane);
    const int off = kc * (rb * 4) + (r_in >> 3) * 32 + (r_in & 7) * 4;   // floats
    *reinterpret_cast<float4*>(chunk + off) = hi;
    *reinterpret_cast<float4*>(chunk + plane + off) = lo;
  }
}

// ------------------------------------------------------------------ tcgen05 helpers
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes),
        "r"(smem_u32(bar))
      : "memory");
}

// Shared-memory operand descriptor: K-major, no swizzle.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes,
                                              uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;   // descriptor version of this architecture
  return d;                 // base offset 0, layout type 0 = no swizzle
}

// Instruction descriptor: D = F32, A = B = TF32, both K-major, M = 128, N = 256.
constexpr uint32_t SG_IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(SG_BN >> 3) << 17) |
                              ((uint32_t)(SG_BM >> 4) << 24);

// The same with N = 128, for the half items.
constexpr uint32_t SG_IDESC_HALF = (1u << 4) | (2u << 7) | (2u << 10) |
                                   ((uint32_t)((SG_BN / 2) >> 3) << 17) | ((uint32_t)(SG_BM >> 4) << 24);

__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ------------------------------------------------------------------ work items
// One work item of a persistent CTA: a 128 x 256 CTA tile, or one 128 x 128 half of it.
struct SgItem {
  int mt, nt;     // CTA tile coordinates (128-row strip, 256-column strip)
  int half;       // -1: the whole tile; 0 / 1: its left / right 128 columns
};

// Items [0, whole) are whole CTA tiles, the rest are halves of the tiles that follow. CTA
// tiles are numbered in panels of SG_PANEL column strips, inside a panel along the columns
// first: the 148 CTAs of a round then share about 18 A strips and 8 B strips instead of all
// A strips and 5 B strips, which cuts what a round pulls through L2.
__device__ __forceinline__ SgItem sg_decode(const SgemmArgs& args, int item, int mtiles, int ntiles) {
  SgItem w;
  int tile;
  if (item < args.whole_items) {
    tile = item;
    w.half = -1;
  } else {
    const int h = item - args.whole_items;
    tile = args.whole_items + (h >> 1);
    w.half = h & 1;
  }
  const int per_panel = mtiles * SG_PANEL;
  const int panel = tile / per_panel;
  const int width = min(SG_PANEL, ntiles - panel * SG_PANEL);
  const int r = tile - panel * per_panel;
  w.mt = r / width;
  w.nt = panel * SG_PANEL + r % width;
  return w;
}

// ------------------------------------------------------------------ GEMM kernel
struct SgSmem {
  uint64_t full[SG_STAGES];
  uint64_t empty[SG_STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(SG_THREADS, 1)
sgemm_tile_kernel(const __grid_constant__ SgemmArgs args) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  SgSmem* ctl = reinterpret_cast<SgSmem*>(smem + SG_STAGES * SG_STAGE_BYTES);
  volatile int* abort_flag = &ctl->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mtiles = (args.M + SG_BM - 1) / SG_BM, ntiles = (args.N + SG_BN - 1) / SG_BN;
  const int items = args.whole_items + args.half_items;

  if (threadIdx.x == 0) {
    for (int s = 0; s < SG_STAGES; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&ctl->acc_full[b], 1);
      mbar_init(&ctl->acc_empty[b], 4);   // one arrival per epilogue warp
    }
    ctl->abort_flag = 0;
    ctl->tmem_base = 0;
    mbar_fence_init();
  }
  __syncthreads();
  if (warp == 1) {
    // the whole tensor memory of the SM: two 256-column accumulators
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&ctl->tmem_base)), "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  // k blocks of every part (same for all tiles of the launch)
  int stages_per_tile = 0;
  for (int p = 0; p < args.nparts; ++p) stages_per_tile += (args.parts[p].klen + SG_BK - 1) / SG_BK;

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
        const SgItem w = sg_decode(args, item, mtiles, ntiles);
        const int mt = w.mt, nt = w.nt;
        for (int p = 0; p < args.nparts && ok; ++p) {
          const SgemmKPart part = args.parts[p];
          const int kblocks = (part.klen + SG_BK - 1) / SG_BK;
          const unsigned char* a = static_cast<const unsigned char*>(part.a_packed) +
                                   (size_t)mt * kblocks * SG_A_CHUNK;
          const unsigned char* b = static_cast<const unsigned char*>(part.b_packed) +
                                   (size_t)nt * kblocks * SG_B_CHUNK;
          for (int kb = 0; kb < kblocks; ++kb, ++it) {
            const int s = it % SG_STAGES;
            if (it >= SG_STAGES &&
                !mbar_wait_bounded(&ctl->empty[s], (uint32_t)(((it / SG_STAGES) - 1) & 1),
                                   abort_flag)) {
              if (!*abort_flag) { *abort_flag = 1; atomicExch(args.status, KERR_EMPTY_WAIT_TIMEOUT); }
              ok = false;
              break;
            }
            unsigned char* st = smem + s * SG_STAGE_BYTES;
            if (w.half < 0) {
              mbar_expect_tx(&ctl->full[s], SG_STAGE_BYTES);
              bulk_load(st, a + (size_t)kb * SG_A_CHUNK, SG_A_CHUNK, &ctl->full[s]);
              bulk_load(st + SG_A_CHUNK, b + (size_t)kb * SG_B_CHUNK, SG_B_CHUNK, &ctl->full[s]);
            } else {
              // Half of the B strip: in each plane the 256 rows of one group of 4 k values
              // are contiguous (4 KB), so the 128 rows of a half are eight 2 KB pieces (four
              // k groups x hi / lo plane). They go to the places they have in a whole stage.
              mbar_expect_tx(&ctl->full[s], SG_A_CHUNK + SG_B_CHUNK / 2);
              bulk_load(st, a + (size_t)kb * SG_A_CHUNK, SG_A_CHUNK, &ctl->full[s]);
              const unsigned char* bsrc = b + (size_t)kb * SG_B_CHUNK + (size_t)w.half * (SG_BN / 2) * 16;
              unsigned char* bdst = st + SG_A_CHUNK + (size_t)w.half * (SG_BN / 2) * 16;
#pragma unroll
              for (int piece = 0; piece < 2 * (SG_BK / 4); ++piece)
                bulk_load(bdst + piece * (SG_BN * 16), bsrc + piece * (SG_BN * 16), (SG_BN / 2) * 16,
                          &ctl->full[s]);
            }
          }
        }
      }
      if (!ok || *abort_flag) {
        // let the copies already issued land before shared memory is released
        const int first = it > SG_STAGES ? it - SG_STAGES : 0;
        for (int j = first; j < it; ++j) {
          int zero = 0;
          if (!mbar_wait_bounded(&ctl->full[j % SG_STAGES], (uint32_t)((j / SG_STAGES) & 1), &zero))
            atomicExch(args.status, KERR_DRAIN_TIMEOUT);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      int it = 0, local_tile = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < items && ok; item += gridDim.x, ++local_tile) {
        const SgItem w = sg_decode(args, item, mtiles, ntiles);
        const uint32_t idesc = w.half < 0 ? SG_IDESC : SG_IDESC_HALF;
        const uint32_t b_half = w.half > 0 ? (uint32_t)((SG_BN / 2) * 16) : 0u;
        const int buf = local_tile & 1;
        if (local_tile >= 2 &&
            !mbar_wait_bounded(&ctl->acc_empty[buf], (uint32_t)(((local_tile >> 1) - 1) & 1),
                               abort_flag)) {
          if (!*abort_flag) { *abort_flag = 1; atomicExch(args.status, KERR_TMEM_WAIT_TIMEOUT); }
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d = tmem_base + (uint32_t)(buf * SG_BN);
        for (int ks = 0; ks < stages_per_tile; ++ks, ++it) {
          const int s = it % SG_STAGES;
          if (!mbar_wait_bounded(&ctl->full[s], (uint32_t)((it / SG_STAGES) & 1), abort_flag)) {
            if (!*abort_flag) { *abort_flag = 1; atomicExch(args.status, KERR_FULL_WAIT_TIMEOUT); }
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * SG_STAGE_BYTES);
          const uint32_t a_hi = sa, a_lo = sa + SG_A_CHUNK / 2;
          const uint32_t b_hi = sa + SG_A_CHUNK + b_half, b_lo = b_hi + SG_B_CHUNK / 2;
          constexpr uint32_t LBO_A = SG_BM * 16, LBO_B = SG_BN * 16, SBO = 128;
#pragma unroll
          for (int j = 0; j < SG_BK / 8; ++j) {
            // K = 8 covers two core matrices along k
            const uint64_t dah = smem_desc(a_hi + j * 2 * LBO_A, LBO_A, SBO);
            const uint64_t dal = smem_desc(a_lo + j * 2 * LBO_A, LBO_A, SBO);
            const uint64_t dbh = smem_desc(b_hi + j * 2 * LBO_B, LBO_B, SBO);
            const uint64_t dbl = smem_desc(b_lo + j * 2 * LBO_B, LBO_B, SBO);
            mma_tf32(d, dal, dbh, idesc, (ks > 0 || j > 0) ? 1u : 0u);   // small terms first
            mma_tf32(d, dah, dbl, idesc, 1u);
            mma_tf32(d, dah, dbh, idesc, 1u);
          }
          mma_commit(&ctl->empty[s]);   // the stage is free once these MMAs have read it
        }
        if (ok) mma_commit(&ctl->acc_full[buf]);
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int quad = warp & 3;   // tensor-memory lanes 32*quad .. 32*quad+31
    const float alpha = args.alpha, beta_c = args.beta_c, beta_src = args.beta_src;
    const bool use_c = beta_c != 0.0f;
    const bool use_src = args.Csrc != nullptr && beta_src != 0.0f;
    int local_tile = 0;
    bool ok = true;
    const bool zero_acc = stages_per_tile == 0;   // K == 0: the accumulator was never written
    for (int item = blockIdx.x; item < items && ok; item += gridDim.x, ++local_tile) {
      const int buf = local_tile & 1;
      const SgItem w = sg_decode(args, item, mtiles, ntiles);
      const int mt = w.mt, nt = w.nt;
      // a half item's accumulator holds 128 columns, those of its half of the tile
      const int n_base = nt * SG_BN + (w.half > 0 ? SG_BN / 2 : 0);
      const int col_blocks = (w.half < 0 ? SG_BN : SG_BN / 2) / 32;
      if (!mbar_wait_bounded(&ctl->acc_full[buf], (uint32_t)((local_tile >> 1) & 1), abort_flag)) {
        if (!*abort_flag) { *abort_flag = 1; atomicExch(args.status, KERR_TMEM_WAIT_TIMEOUT); }
        ok = false;
        break;
      }
      tc_fence_after();
      const int m = mt * SG_BM + quad * 32 + lane;
#pragma unroll 1
      for (int cb = 0; cb < col_blocks; ++cb) {
        uint32_t r[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) +
                               (uint32_t)(buf * SG_BN + cb * 32);
        tmem_ld32(taddr, r);
        if (m < args.M) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int n = n_base + cb * 32 + j;
            if (n < args.N) {
              float v = zero_acc ? 0.0f : alpha * __uint_as_float(r[j]);
              float* cp = args.C + m + (int64_t)n * args.ldc;
              if (use_c) v = fmaf(beta_c, *cp, v);
              if (use_src) v = fmaf(beta_src, args.Csrc[m + (int64_t)n * args.ldcsrc], v);
              *cp = v;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->acc_empty[buf]);
    }
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u)
                 : "memory");
  }
}

// ------------------------------------------------------------------ TF32 peak loop
// The MMA issue loop of the GEMM kernel without any global traffic: the operands of one
// pipeline stage sit in shared memory for the whole run and `stages` times the six
// tcgen05.mma of a stage (lo*hi, hi*lo, hi*hi for two K = 8 steps) are issued into the two
// tensor-memory accumulators, committing to a ring of four barriers exactly like the GEMM
// kernel does. What it measures is the rate the tensor pipe sustains for this instruction
// shape (M = 128, N = 256, K = 8, operands read from shared memory through no-swizzle
// K-major descriptors): the roofline of the 3xTF32 kernel is a third of it.
__global__ void __launch_bounds__(64, 1) tf32_peak_kernel(int stages, int random_operands, int* status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  __shared__ uint64_t done[SG_STAGES];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < SG_STAGE_BYTES / 4; i += blockDim.x)
  {
    // constant operands measure the issue rate of the tensor pipe; operands drawn from
    // uniform(-1, 1) (TF32-exact) toggle the datapath like a real product does, which is what
    // the board's power limit sees
    float v = 1.0f;
    if (random_operands) {
      uint32_t h = (uint32_t)i * 2654435761u ^ (blockIdx.x * 40503u + 0x9E3779B9u);
      h ^= h >> 16; h *= 0x7feb352du; h ^= h >> 15; h *= 0x846ca68bu; h ^= h >> 16;
      v = tf32_round((float)(h >> 8) * (2.0f / 16777216.0f) - 1.0f);
    }
    reinterpret_cast<float*>(smem)[i] = v;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < SG_STAGES; ++s) mbar_init(&done[s], 1);
    abort_flag = 0;
    tmem_slot = 0;
    mbar_fence_init();
  }
  // the tensor core reads shared memory through the async proxy
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_slot)), "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  if (warp == 1 && lane == 0) {
    const uint32_t sa = smem_u32(smem);
    const uint32_t a_hi = sa, a_lo = sa + SG_A_CHUNK / 2;
    const uint32_t b_hi = sa + SG_A_CHUNK, b_lo = b_hi + SG_B_CHUNK / 2;
    constexpr uint32_t LBO_A = SG_BM * 16, LBO_B = SG_BN * 16, SBO = 128;
    bool ok = true;
    for (int it = 0; it < stages && ok; ++it) {
      const int s = it % SG_STAGES;
      if (it >= SG_STAGES &&
          !mbar_wait_bounded(&done[s], (uint32_t)(((it / SG_STAGES) - 1) & 1), &abort_flag)) {
        atomicExch(status, KERR_TMEM_WAIT_TIMEOUT);
        ok = false;
        break;
      }
      // a new accumulator every 256 stages, as a 4096-deep tile would
      const uint32_t d = tmem_base + (uint32_t)(((it >> 8) & 1) * SG_BN);
#pragma unroll
      for (int j = 0; j < SG_BK / 8; ++j) {
        const uint64_t dah = smem_desc(a_hi + j * 2 * LBO_A, LBO_A, SBO);
        const uint64_t dal = smem_desc(a_lo + j * 2 * LBO_A, LBO_A, SBO);
        const uint64_t dbh = smem_desc(b_hi + j * 2 * LBO_B, LBO_B, SBO);
        const uint64_t dbl = smem_desc(b_lo + j * 2 * LBO_B, LBO_B, SBO);
        mma_tf32(d, dal, dbh, SG_IDESC, ((it & 255) > 0 || j > 0) ? 1u : 0u);
        mma_tf32(d, dah, dbl, SG_IDESC, 1u);
        mma_tf32(d, dah, dbh, SG_IDESC, 1u);
      }
      mma_commit(&done[s]);
    }
    // everything issued has to finish before tensor memory is handed back
    const int first = stages > SG_STAGES ? stages - SG_STAGES : 0;
    for (int j = first; j < stages && ok; ++j) {
      int zero = 0;
      if (!mbar_wait_bounded(&done[j % SG_STAGES], (uint32_t)((j / SG_STAGES) & 1), &zero)) {
        atomicExch(status, KERR_TMEM_WAIT_TIMEOUT);
        ok = false;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u)
                 : "memory");
  }
}

}  // namespace

cudaError_t launch_tf32_peak(int stages, int blocks, bool random_operands, int* status,
                             cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(tf32_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SG_STAGE_BYTES + 256);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  tf32_peak_kernel<<<blocks, 64, SG_STAGE_BYTES + 256, stream>>>(stages, random_operands ? 1 : 0,
                                                                 status);
  return cudaGetLastError();
}

cudaError_t sgemm_tile_configure() {
  return cudaFuncSetAttribute(sgemm_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              SG_SMEM_BYTES);
}

cudaError_t launch_sgemm_pack(const float* src, int64_t ld, bool k_contig, int rows, int klen,
                              int rb, void* packed, cudaStream_t stream) {
  const int rblocks = (rows + rb - 1) / rb, kblocks = (klen + SG_BK - 1) / SG_BK;
  const int64_t total = (int64_t)rblocks * kblocks * rb * (SG_BK / 4);
  if (total == 0) return cudaSuccess;
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  sgemm_pack_kernel<<<(int)blocks, 256, 0, stream>>>(src, ld, k_contig ? 1 : 0, rows, klen, rb,
                                                     rblocks, kblocks,
                                                     static_cast<float*>(packed));
  return cudaGetLastError();
}

void sgemm_tile_schedule(int M, int N, int sms, int* whole_items, int* half_items, int* grid) {
  const int tiles = ((M + SG_BM - 1) / SG_BM) * ((N + SG_BN - 1) / SG_BN);
  const int G = sms > 0 ? sms : 1;
  int whole = (tiles / G) * G;
  const int rest = tiles - whole;
  int halves = 0;
  // What is left after the last whole round of the grid is cut into halves when those fit
  // into one more round: that round then takes half the time of a whole-tile round.
  if (rest > 0 && 2 * rest <= G) halves = 2 * rest;
  else whole += rest;
  *whole_items = whole;
  *half_items = halves;
  const int items = whole + halves;
  *grid = items < G ? items : G;
}

cudaError_t launch_sgemm_tile(const SgemmArgs& args_in, int sm_count, cudaStream_t stream) {
  SgemmArgs args = args_in;
  int grid = 0;
  sgemm_tile_schedule(args.M, args.N, sm_count, &args.whole_items, &args.half_items, &grid);
  if (grid == 0) return cudaSuccess;
  sgemm_tile_kernel<<<grid, SG_THREADS, SG_SMEM_BYTES, stream>>>(args);
  return cudaGetLastError();
}

}  // namespace paralia
