/*
 * paralia_c.h -- C ABI of libparalia.so (B200 / sm_100a build).
 *
 * Plain pointers and sizes only; no C++ or framework types cross this boundary.
 * Every entry point returns a status code (PARALIA_OK == 0) instead of terminating
 * the process, which is what the reference does on error
 * (Library_scheduler/src/Functions/dgemm.cpp:42,92,399,450).
 *
 * Location ids follow the reference's convention
 * (Benchmarking/CuCuBLAS/src/PARALia/dgemm_runner.cpp:55-57, Subkernel.cpp:46):
 *   -1      pinned (or pinnable) host memory
 *   0..G-1  memory of GPU <id>
 *   PARALIA_LOC_AUTO  ask the CUDA runtime where the pointer lives, which is what the
 *                     reference always does (CoCoGetPtrLoc, dgemm.cpp:356-363).
 *
 * All matrices are column-major, exactly as in BLAS / the reference.
 */
#ifndef PARALIA_C_H
#define PARALIA_C_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PARALIA_MAX_UNITS 16
#define PARALIA_LOC_HOST (-1)
#define PARALIA_LOC_AUTO (-100)

/* status codes */
enum {
  PARALIA_OK = 0,
  PARALIA_ERR_INVALID_ARG = 1,
  PARALIA_ERR_OUT_OF_MEMORY = 2,
  PARALIA_ERR_CUDA = 3,
  PARALIA_ERR_TIMEOUT = 4,
  PARALIA_ERR_NO_PEER_ACCESS = 5,
  PARALIA_ERR_DB_MISSING = 6,
  PARALIA_ERR_NO_DEVICE = 7,
  PARALIA_ERR_UNSUPPORTED = 8,
  PARALIA_ERR_GROUP_FAILED = 9   /* another rank of the process group failed or went missing */
};

/*
 * Caller-fixed control values: the C form of the "predefined" autotune controller that
 * the reference passes to its ...Controled entry points
 * (Library_scheduler/src/Functions/dgemm.cpp:697-705, fields Autotuner.hpp:121-149;
 * CLI meaning Benchmarking/CuCuBLAS/src/testing.cpp:280-308).
 * A field <= 0 (or a NULL ctl) means "let the autotuner choose".
 */
typedef struct paralia_ctl {
  int64_t T;                                   /* tile edge in elements                */
  int32_t active_unit_num;                     /* number of GPUs to use                */
  int32_t active_unit_id_list[PARALIA_MAX_UNITS]; /* their ids, grid order (r*D2+c)    */
  int64_t cache_limit;                         /* bytes of tile cache per GPU          */
  int32_t exec_streams;                        /* compute streams per GPU (default 4;
                                                  reference MAX_BACKEND_L=8,
                                                  CMakeLists.txt:69)                   */
  int32_t flags;                               /* PARALIA_FLAG_* below                 */
} paralia_ctl;

#define PARALIA_FLAG_NO_PEER_FETCH 1  /* every GPU fetches host tiles itself            */
#define PARALIA_FLAG_KEEP_PINNED   2  /* leave host operands registered after the call  */
#define PARALIA_FLAG_NO_METADATA_REUSE 4 /* rebuild the plan even for a known signature */
#define PARALIA_FLAG_BETA_ZERO 8      /* PARALiA_autotune_gemm only (it takes no beta): model
                                         the call with beta == 0, i.e. C is not fetched  */

/*
 * What a call did: the POD form of the ATC object the reference returns
 * (dgemm.cpp:689-693; fields read by callers: dgemm_runner.cpp:26-33,140,147).
 */
typedef struct paralia_report {
  int64_t T;
  int32_t active_unit_num;
  int32_t active_unit_id_list[PARALIA_MAX_UNITS];
  double  active_unit_score[PARALIA_MAX_UNITS];
  int64_t cache_limit;
  int64_t subkernel_num;
  int32_t subkernels_per_unit[PARALIA_MAX_UNITS];
  double  pred_t;            /* model-predicted seconds                         */
  double  pred_J;            /* always 0: energy modelling is not built         */
  double  T_slowdowns[6];    /* aggregate, imbalance, remainder, small, sknum, big
                                (Autotuner.cpp:562-603)                          */
  /* measured */
  double  device_ms;         /* first enqueue -> last write-back, CUDA events,
                                max over the GPUs used                           */
  double  host_ms;           /* wall clock of the whole call                    */
  double  plan_ms;           /* autotune + plan construction                    */
  double  pin_ms;            /* host registration inside the call               */
  double  alloc_ms;          /* tile-cache slab (re)allocation                  */
  int64_t h2d_bytes, d2h_bytes, p2p_bytes, d2d_bytes;
  int64_t kernel_launches;   /* launches of this library's own kernels          */
  int32_t metadata_reused;   /* 1 if the plan came from the signature cache     */
  int32_t grid_d1, grid_d2;  /* device grid D1_parts x D2_parts                 */
  /* phases of device_ms (GEMM routines; 0 elsewhere), each the max over the GPUs used,
   * measured from the call's start event:                                      */
  double  fill_ms;           /* until the first tile kernel starts              */
  double  exec_end_ms;       /* until the last tile kernel ends                 */
  double  h2d_end_ms;        /* until the last host -> GPU copy ends            */
} paralia_report;

/* ---- environment variables -------------------------------------------------------
 * Read once, at first use. None of them is needed for normal operation.
 *   PARALIA_DB               directory of the calibration database (lookup tables and link
 *                            models, reference DEPLOYDB); default: the tables shipped beside
 *                            the library.
 *   PARALIA_KCHAIN=<n>       k tiles per launch (default: 1 for the first launch of a C tile,
 *                            then 4). CHANGES RESULT BITS: the k split decides where partial
 *                            sums are rounded; results are bit-reproducible only for a fixed
 *                            value. For experiments.
 *   PARALIA_BAND=<n>, PARALIA_BAND_PLAN=<a,b,...>  force the band sizes of the launch order.
 *                            Launch order only: no result bit changes.
 *   PARALIA_DEFER_WB=<0|1>   force write-backs to overlap with (0) or follow (1) the input
 *                            stream of a GPU; default: decided from the database. Order only.
 *   PARALIA_GROUP_TIMEOUT_MS hand-shake time-out of process groups (default 60000).
 *   PARALIA_JOIN_TIMEOUT_MS  deadline of the host join of a whole-problem call (default: the
 *                            larger of 120000 and fifty times the predicted duration).
 */

/* ---- library life cycle ---------------------------------------------------------- */
/* Discover GPUs, enable peer access between every pair (reference: CoCoEnableLinks,
 * dgemm.cpp:423). Idempotent; every other entry point calls it on first use. */
int PARALiA_init(void);
/* Free every slab, stream, event and cached plan. */
int PARALiA_finalize(void);
/* Number of GPUs the library sees (reference: compile-time LOC_NUM-1). */
int PARALiA_device_count(void);
/* Text of the last error on the calling thread. */
const char* PARALiA_last_error(void);
/* Replaces PARALiADevCacheFree (Library_scheduler/src/Subkernel.cpp:488-495):
 * frees the tile-cache slab of one location and drops it from cached plans. */
int PARALiA_dev_cache_free(int loc);

/* ---- the four routines of the hot path -------------------------------------------- */
/* Stream semantics of the whole-problem routines below: they run on the library's own
 * (non-blocking) streams and are blocking calls, so everything they wrote is visible when
 * they return. On entry they wait for work the caller already queued on the legacy default
 * stream of every GPU that holds an operand or takes part (a kernel or copy that produced an
 * operand there); work queued on other streams has to be synchronised by the caller. The
 * PARALiA_tile_* entry points further down run on the stream the caller passes. */
/* Replaces PARALiADgemm / PARALiADgemmControled (PARALiA.hpp:33-38,
 * dgemm.cpp:318-705): C <- alpha*op(A)*op(B) + beta*C, FP64. Blocking: returns after C
 * is completely written (dgemm.cpp:596-597). */
int PARALiA_dgemm(char TransA, char TransB, int64_t M, int64_t N, int64_t K,
                  double alpha, const double* A, int64_t ldA, int locA,
                  const double* B, int64_t ldB, int locB,
                  double beta, double* C, int64_t ldC, int locC,
                  const paralia_ctl* ctl, paralia_report* out);

/* Replaces PARALiASgemm / PARALiASgemmControled (PARALiA.hpp:41-46,
 * Library_scheduler/src/Functions/sgemm.cpp:296-...): FP32 via a 3xTF32 split. */
int PARALiA_sgemm(char TransA, char TransB, int64_t M, int64_t N, int64_t K,
                  float alpha, const float* A, int64_t ldA, int locA,
                  const float* B, int64_t ldB, int locB,
                  float beta, float* C, int64_t ldC, int locC,
                  const paralia_ctl* ctl, paralia_report* out);

/* Replaces PARALiADgemv / PARALiADgemvControled (PARALiA.hpp:48-53,
 * Library_scheduler/src/Functions/dgemv.cpp:288): y <- alpha*op(A)*x + beta*y, A is M x N
 * column-major. ctl->T, if set, is the number of columns of A per tile. */
int PARALiA_dgemv(char TransA, int64_t M, int64_t N, double alpha,
                  const double* A, int64_t ldA, int locA,
                  const double* x, int64_t incx, int locx,
                  double beta, double* y, int64_t incy, int locy,
                  const paralia_ctl* ctl, paralia_report* out);

/* Replaces PARALiADaxpy / PARALiADaxpyControled (PARALiA.hpp:56-61,
 * Library_scheduler/src/Functions/daxpy.cpp:200-469): y <- alpha*x + y. */
int PARALiA_daxpy(int64_t N, double alpha, const double* x, int64_t incx, int locx,
                  double* y, int64_t incy, int locy,
                  const paralia_ctl* ctl, paralia_report* out);

/* Replaces PARALiADdot / PARALiADdotControled (PARALiA.hpp:64-69,
 * Library_scheduler/src/Functions/ddot.cpp:201-469): *result += sum_i x_i*y_i.
 * As in the reference the partial sums are ADDED to *result, which the caller zeroes
 * (ddot.cpp:431, Benchmarking/CuCuBLAS/src/PARALia/ddot_runner.cpp:45). The sum order
 * is fixed (tile order, then a fixed tree inside a tile), so results are bit-reproducible. */
int PARALiA_ddot(int64_t N, const double* x, int64_t incx, int locx,
                 const double* y, int64_t incy, int locy, double* result,
                 const paralia_ctl* ctl, paralia_report* out);

/* The same dot product, but the per-tile sums are returned in tile order instead of being
 * added up: tile_sums[i] = sum over tile i (tile length = out->T, ctl->T if given), *count =
 * number of tiles (at most `capacity` are written; pass capacity 0 to ask for the count).
 * Adding them in order to a start value gives PARALiA_ddot's result bit for bit. This is
 * what lets several processes, each holding a run of whole tiles of the vectors, combine
 * their parts in the one global tile order (reference: the host-side sum, ddot.cpp:431). */
int PARALiA_ddot_tiles(int64_t N, const double* x, int64_t incx, int locx,
                       const double* y, int64_t incy, int locy,
                       double* tile_sums, int64_t capacity, int64_t* count,
                       const paralia_ctl* ctl, paralia_report* out);

/* ---- one process per GPU ------------------------------------------------------------
 * The reference drives all GPUs from one process. Under a launcher that starts one
 * process per GPU, the processes form a group: rank = r*D2 + c of the D1 x D2 device grid
 * (the grid rule of Autotuner/src/Subkernel_distributions.cpp:325-336) owns the C block
 * of grid cell (r, c), as the in-process distribution would give it to that GPU (:399).
 * PARALiA_group_dgemm is collective: every rank passes ITS row panel of op(A)
 * (Mloc x K), ITS column panel of op(B) (K x Nloc) and ITS block of C (Mloc x Nloc).
 * Host-resident A/B tiles then cross the host link once per grid row / column and reach
 * the other ranks GPU -> GPU through CUDA IPC -- the cross-process form of "a tile cached
 * on a peer is fetched from the peer". `name` must be the same, unique string on all
 * ranks (it names a small POSIX shared-memory segment used for the hand-shakes).
 * No counterpart in the reference (which has no multi-process mode). */
int PARALiA_group_init(const char* name, int rank, int world, int dev);
int PARALiA_group_finalize(void);
int PARALiA_group_dgemm(char TransA, char TransB, int64_t Mloc, int64_t Nloc, int64_t K,
                        double alpha, const double* A_panel, int64_t ldA, int locA,
                        const double* B_panel, int64_t ldB, int locB,
                        double beta, double* C_block, int64_t ldC, int locC,
                        const paralia_ctl* ctl, paralia_report* out);

int PARALiA_group_sgemm(char TransA, char TransB, int64_t Mloc, int64_t Nloc, int64_t K,
                        float alpha, const float* A_panel, int64_t ldA, int locA,
                        const float* B_panel, int64_t ldB, int locB,
                        float beta, float* C_block, int64_t ldC, int locC,
                        const paralia_ctl* ctl, paralia_report* out);

/* Failure-detection self test (no counterpart in the reference, which has no failure
 * detection): launches a kernel whose only wait can never be satisfied, with a clock
 * budget of budget_ms. Returns PARALIA_ERR_TIMEOUT when the wait gave up, the kernel ended
 * by itself and the error word reached the host -- the path every device-side wait of this
 * library takes instead of hanging the GPU. The CUDA context stays usable afterwards. */
int PARALiA_selftest_bounded_wait(int dev, double budget_ms);

/* Same idea for the host side of a whole-problem call: the call joins its GPUs by waiting
 * for their end events with a deadline (PARALIA_JOIN_TIMEOUT_MS, default the larger of two
 * minutes and fifty times the predicted duration). The self test queues a kernel that ends by
 * itself after kernel_ms and joins with deadline_ms; with deadline_ms < kernel_ms it returns
 * PARALIA_ERR_TIMEOUT. Nothing hangs and the context stays usable. */
int PARALiA_selftest_join_deadline(int dev, double kernel_ms, double deadline_ms);
/* The hand-shake layer of process groups alone, without CUDA: `rounds` barriers between
 * `world` processes over the shared segment `name`. fail_mode 0: nobody fails. 1: rank
 * fail_rank reports an error of its own at round fail_round (what a collective call does when
 * its arguments are bad or an allocation fails): the others return PARALIA_ERR_GROUP_FAILED
 * at once. 2: that rank silently stops arriving: the others time out after
 * PARALIA_GROUP_TIMEOUT_MS (default 60000), the first to do so abandons the group and the
 * rest follow at once. *waited_ms (may be NULL) = time spent in the failing barrier. */
int PARALiA_selftest_group_rendezvous(const char* name, int rank, int world, int rounds,
                                      int fail_rank, int fail_round, int fail_mode,
                                      double* waited_ms);

/* ---- per-tile kernels on device-resident data ---------------------------------------
 * What the reference reaches through backend_run_operation(params, "Dgemm"|"Sgemm"|
 * "Daxpy"|"Ddot", queue) (Library_scheduler/src/Subkernel.cpp:168,228; parameter blocks
 * dgemm.cpp:181-197, daxpy.cpp:62-69, ddot.cpp:62-70) and the microbenchmarks time
 * (Database_builder/CuCuBLAS/src/dgemm_microbench.cu:141-142). All pointers are device
 * pointers on GPU `dev`; `stream` is a cudaStream_t (NULL = the legacy default stream).
 * Asynchronous: the caller synchronises the stream. */
/* The tile kernels bound every wait inside them; a wait that runs out makes the kernel stop
 * and leave a code in a per-GPU status word. The asynchronous tile entry points cannot
 * report that themselves: after synchronising the stream, PARALiA_tile_status(dev) reads and
 * clears the word (it synchronises the GPU) and returns PARALIA_ERR_TIMEOUT if a tile kernel
 * gave up since the last check. The whole-problem routines do this check on their own. */
int PARALiA_tile_status(int dev);
int PARALiA_tile_dgemm(int dev, void* stream, char TransA, char TransB,
                       int64_t M, int64_t N, int64_t K, double alpha,
                       const double* A, int64_t ldA, const double* B, int64_t ldB,
                       double beta, double* C, int64_t ldC);
int PARALiA_tile_sgemm(int dev, void* stream, char TransA, char TransB,
                       int64_t M, int64_t N, int64_t K, float alpha,
                       const float* A, int64_t ldA, const float* B, int64_t ldB,
                       float beta, float* C, int64_t ldC);
int PARALiA_tile_daxpy(int dev, void* stream, int64_t N, double alpha,
                       const double* x, int64_t incx, double* y, int64_t incy);
/* `partials` is device scratch of PARALiA_tile_ddot_scratch_bytes(N) bytes; the result
 * (one double) is written to device memory at `result_dev`. */
int64_t PARALiA_tile_ddot_scratch_bytes(int64_t N);
int PARALiA_tile_ddot(int dev, void* stream, int64_t N,
                      const double* x, int64_t incx, const double* y, int64_t incy,
                      double* partials, double* result_dev);

/* Per-tile FP64 matrix-vector product y <- alpha*op(A)*x + beta*y on the caller's stream:
 * the compute call behind the reference's DGEMV subkernels (backend_run_operation with
 * "Dgemv", Library_scheduler/src/Subkernel.cpp:168,228, set up in
 * Library_scheduler/src/Functions/dgemv.cpp). A is M x N column-major on GPU `dev`.
 * `scratch` is device memory of PARALiA_tile_dgemv_scratch_bytes(TransA, M, N) bytes
 * (op = N keeps partial vectors there; op = T needs none and accepts NULL). */
int64_t PARALiA_tile_dgemv_scratch_bytes(char TransA, int64_t M, int64_t N);
int PARALiA_tile_dgemv(int dev, void* stream, char TransA, int64_t M, int64_t N, double alpha,
                       const double* A, int64_t ldA, const double* x, int64_t incx,
                       double beta, double* y, int64_t incy, double* scratch);

/* Dot product that allocates nothing. It has no counterpart in the reference.
 * For callers that cannot call cudaMalloc where they need the result (inside a
 * latency-critical loop where an allocation would stall the device, inside a host
 * application that hands its plugins a fixed memory budget, or while another library
 * owns the allocator) and therefore cannot provide the scratch PARALiA_tile_ddot asks
 * for: the per-block partial sums go to a fixed array in the library's own device image
 * (8 KB, held by every GPU that loads the library until the process exits).
 *  - N may be at most PARALiA_tile_ddot_noalloc_max_n() (2^31 elements); larger N is
 *    rejected with PARALIA_ERR_INVALID_ARG.
 *  - The first call on each GPU looks up the array's device address; make that first
 *    call before starting any stream capture.
 *  - All calls on one GPU share the array: two calls whose kernels can overlap on the GPU
 *    (different streams, no ordering between them) race. Calls on one stream are safe.
 *  - x, y and result_dev are device pointers on GPU `dev`; the call is asynchronous. */
int64_t PARALiA_tile_ddot_noalloc_max_n(void);
int PARALiA_tile_ddot_noalloc(int dev, void* stream, int64_t N,
                              const double* x, int64_t incx, const double* y, int64_t incy,
                              double* result_dev);

/* ---- memory and input helpers (reference: CoCoMalloc/CoCoFree/CoCoVecInit/CoCoMemcpy,
 * used at dgemm_runner.cpp:55-69,77) ------------------------------------------------- */
int PARALiA_malloc(void** ptr, int64_t bytes, int loc);   /* loc -1: pinned host     */
int PARALiA_free(void* ptr, int loc);
int PARALiA_memcpy(void* dst, int loc_dst, const void* src, int loc_src, int64_t bytes);
/* Counter-based generators: element i of a buffer depends only on (seed, i), so the
 * same bits come out on the host and on any GPU. dist: 0 = uniform[-1,1), 1 = normal(0,1). */
int PARALiA_fill_f64(double* ptr, int64_t n, uint64_t seed, int dist, int loc);
int PARALiA_fill_f32(float* ptr, int64_t n, uint64_t seed, int dist, int loc);

/* ---- autotuner / plan introspection ---------------------------------------------------
 * Runs only the model (reference: ATC::autotune_problem, Autotuner.cpp:279-560; the
 * autotune-only CLI Benchmarking/CuCuBLAS/src/PARALia/dgemm_predictor.cpp:16-93).
 * Needs no GPU when ctl fixes active_unit_num. */
int PARALiA_autotune_gemm(int elem_size, char TransA, char TransB,
                          int64_t M, int64_t N, int64_t K, int locA, int locB, int locC,
                          const paralia_ctl* ctl, paralia_report* out);
/* Level-1 counterpart (ModelLvl1.cpp:19-144 with Autotuner.cpp:279-560): unit set, tile
 * length and predicted seconds of DAXPY (is_dot == 0) or DDOT on vectors of N doubles at
 * locx / locy, from the measured Daxpy / Ddot tile tables and the shared host-link model. */
int PARALiA_autotune_vec(int is_dot, int64_t N, int locx, int locy, const paralia_ctl* ctl,
                         paralia_report* out);
/* The shared host-link model (Autotuner/src/CoModel.cpp:120-140 t_com_predict_shared,
 * LinkMap.cpp:121-269 update_link_shared_weights, restated for one NVSwitch box): seconds to
 * move `bytes` over the host link of GPU `dev` (to_gpu != 0: host -> GPU) while n_active
 * GPUs use their host links in the same direction and, if both_directions != 0, the other
 * direction is busy too. active_devs (may be NULL) names those GPUs, for the pairwise
 * "Slowdown" factors of the link files; the aggregate table caps the result.
 * *defer_writebacks (may be NULL) receives 1 if, with n_active GPUs, the executor holds C
 * write-backs until a GPU's input stream has drained. */
int PARALiA_model_host_link(int dev, int to_gpu, int64_t bytes, int n_active, int both_directions,
                            const int32_t* active_devs, int n_devs, double* seconds,
                            int32_t* defer_writebacks);
/* Tile-size score of one candidate T (Autotuner.cpp:571-603); slowdowns[6]. */
int PARALiA_tile_slowdowns(int64_t M, int64_t N, int64_t K, int64_t T, int active_units,
                           double* slowdowns);
/* Subkernel -> unit assignment of the 2D block distribution
 * (Autotuner/src/Subkernel_distributions.cpp:315-485). sk_unit[sk_id] receives the
 * index (into the active unit list) that owns subkernel sk_id = mi*Nt*Kt + ni*Kt + ki;
 * d1/d2 receive the device grid. */
int PARALiA_distribute_2d(int units, int Mt, int Nt, int Kt, int32_t* sk_unit,
                          int32_t* d1, int32_t* d2);
/* The launch plan of a tiled GEMM with `units` GPUs and tile edge T, in the order the
 * launches are enqueued (round-robin over the units, one launch per turn): for launch i,
 * items[5*i .. 5*i+4] = unit index, C tile row mi, C tile column ni, first k tile, end k
 * tile. Pure host arithmetic, a function of (M, N, K, T, units, bounded_cache) alone --
 * this is what makes the tile order, and with it the result bits, reproducible. It stands
 * where the reference chooses the next subkernel at run time (SubkernelSelect,
 * Library_scheduler/src/Subkernel.cpp:384-449, fire loop
 * Library_scheduler/src/Functions/dgemm.cpp:516-544). bounded_cache != 0 gives the order
 * used when the tile cache cannot hold a unit's working set. *count receives the number
 * of launches; at most `capacity` of them are written (items may be NULL to ask for the
 * count only). */
int PARALiA_plan_gemm(int64_t M, int64_t N, int64_t K, int64_t T, int units, int bounded_cache,
                      int32_t* items, int64_t capacity, int64_t* count, int32_t* d1, int32_t* d2);
/* Load / replace the calibration database directory (lookup tables + link models). */
int PARALiA_load_database(const char* dir);

/* ---- calibration microbenchmarks (reference: Database_builder/CuCuBLAS/src/
 * dgemm_microbench.cu, transfer_link_microbench.cu) ------------------------------------ */
/* Register-only FP64 tensor-core loop; returns sustained TFLOP/s of GPU `dev`.
 * shape: 884, 1684, 1688 or 16816 (mma.sync m/n/k). */
int PARALiA_bench_dmma_peak(int dev, int shape, int iters, double* tflops);
/* The issue loop of the FP32 kernel's tensor-core instruction (tcgen05.mma.kind::tf32,
 * M = 128, N = 256, K = 8, operands resident in shared memory, no global traffic) on every SM
 * of GPU `dev`: `stages` x 6 MMAs per SM. Returns the dense TF32 TFLOP/s sustained over the
 * run; the 3xTF32 kernel's roofline is a third of it. A few thousand stages give the burst
 * figure, a few hundred thousand (about a second) the figure under the power cap. */
int PARALiA_bench_tf32_peak(int dev, int stages, double* tflops);
/* The same loop on operands drawn from uniform(-1, 1) instead of ones: the rate a real
 * product can be issued at once the datapath toggles and the board's power limit applies. */
int PARALiA_bench_tf32_peak_random(int dev, int stages, double* tflops);
/* Time `reps` launches of the tile DGEMM on square T; returns mean seconds. */
int PARALiA_bench_tile_dgemm(int dev, char TransA, char TransB, int64_t T, int reps,
                             double* mean_s);
/* The same with launches of T x T x (chain*T), the shape the executor launches when it
 * chains k tiles of one C tile (spread over up to four streams as the executor does); returns
 * mean seconds per k tile. chain = 4 is what the shipped tile tables hold. */
int PARALiA_bench_tile_dgemm_chain(int dev, char TransA, char TransB, int64_t T, int chain,
                                   int reps, double* mean_s);
/* Same for the FP32 kernel: operands are packed once, only the GEMM kernel is timed. */
int PARALiA_bench_tile_sgemm(int dev, int64_t T, int reps, double* mean_s);
/* Level-1 tile kernels on device-resident vectors of N doubles (reference:
 * Database_builder/CuCuBLAS/src/daxpy_microbench.cu:26-231, ddot_microbench.cu:26-228);
 * mean seconds per tile. */
int PARALiA_bench_tile_daxpy(int dev, int64_t N, int reps, double* mean_s);
int PARALiA_bench_tile_ddot(int dev, int64_t N, int reps, double* mean_s);
/* One square T x T DGEMV tile (TransA 'N' or 'T') on device-resident operands (reference:
 * Database_builder/CuCuBLAS/src/dgemv_microbench.cu:127-190); mean seconds per tile. */
int PARALiA_bench_tile_dgemv(int dev, char TransA, int64_t T, int reps, double* mean_s);
/* All host links of GPUs 0..ngpu-1 at once, `reps` pinned copies of `bytes` each per GPU
 * and direction. mode 0: host -> GPU only, 1: GPU -> host only, 2: both directions together.
 * *gbs receives the aggregate GB/s per direction. No counterpart in the reference. */
int PARALiA_bench_host_aggregate(int ngpu, int mode, int64_t bytes, int reps, double* gbs);
/* Time a strided 2-D tile copy dim x dim doubles src_loc -> dst_loc; mean seconds. */
int PARALiA_bench_link(int dst_loc, int src_loc, int64_t dim, int reps, double* mean_s);

/* The same copy alone and while ten times as many copies keep link (odst <- osrc) busy
 * (reference: transfer_link_microbench.cu:186-218); slowdown = t_shared / t_alone. */
int PARALiA_bench_link_overlap(int dst_loc, int src_loc, int odst_loc, int osrc_loc, int64_t dim,
                               int reps, double* t_alone, double* t_shared);

#ifdef __cplusplus
}
#endif
#endif /* PARALIA_C_H */
