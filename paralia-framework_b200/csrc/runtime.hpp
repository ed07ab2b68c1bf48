// Process-wide runtime of libparalia: per-GPU streams, tile-cache slabs, status words,
// TMA descriptor helper, pointer-location and pinning helpers.
//
// It rebuilds, for one NVSwitch box, what the reference keeps in process-global arrays
// (exec_queue / recv_queues / wb_queues / current_SAB, Library_scheduler/src/
// Subkernel.cpp:18-22,249-306) and in its backend library (CommandQueue, Event, Buffer),
// whose source is not part of the reference checkout.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/paralia_c.h"

namespace paralia {

// Record an error message for PARALiA_last_error() and return `code`.
int fail(int code, const char* fmt, ...);
const char* last_error_cstr();

#define PL_CUDA(expr)                                                                  \
  do {                                                                                 \
    cudaError_t e__ = (expr);                                                          \
    if (e__ != cudaSuccess)                                                            \
      return ::paralia::fail(PARALIA_ERR_CUDA, "%s:%d: %s -> %s", __FILE__, __LINE__,  \
                             #expr, cudaGetErrorString(e__));                          \
  } while (0)

#define PL_TRY(expr)              \
  do {                            \
    int rc__ = (expr);            \
    if (rc__ != PARALIA_OK) return rc__; \
  } while (0)

constexpr int MAX_EXEC_STREAMS = 8;

struct DeviceCtx {
  int dev = -1;
  bool ready = false;
  cudaStream_t h2d = nullptr;   // host -> this GPU tile fetches
  cudaStream_t d2h = nullptr;   // this GPU -> host (or owner GPU) write-backs
  cudaStream_t p2p = nullptr;   // peer GPU -> this GPU tile fetches
  cudaStream_t exec[MAX_EXEC_STREAMS] = {};
  cudaStream_t pack = nullptr;  // FP32 operand packing (hi/lo split) kernels
  // Ring of raw-tile staging buffers between a host/peer copy and its pack kernel.
  static constexpr int STAGE_SLOTS = 4;
  void* stage = nullptr;
  size_t stage_slot_bytes = 0;
  cudaEvent_t stage_free[STAGE_SLOTS] = {};   // slot may be overwritten after this
  bool stage_used[STAGE_SLOTS] = {};
  int stage_next = 0;
  cudaEvent_t t_begin = nullptr, t_end = nullptr;  // timing events
  // Phases of a call: start of the first kernel, end of the last kernel per compute stream,
  // end of the host -> GPU stream.
  cudaEvent_t t_first_exec = nullptr, t_h2d_end = nullptr;
  cudaEvent_t t_exec_end[MAX_EXEC_STREAMS] = {};
  cudaEvent_t caller_ready = nullptr;  // marks the caller's default-stream work at call entry
  // Tile cache: one allocation cut into equal blocks (reference: Buffer / CBlock,
  // sized by ManageCachesDgemm, Library_scheduler/src/Functions/dgemm.cpp:23-121).
  void* slab = nullptr;
  size_t slab_bytes = 0;
  uint64_t slab_gen = 0;   // bumped whenever the slab is (re)allocated or freed
  // Device word the kernels write a KERR_* code into when a bounded wait gives up.
  int* status_dev = nullptr;
  // Scratch for dot products: per-block partials and per-tile results.
  double* dot_partials = nullptr;
  size_t dot_partials_n = 0;
  double* dot_results = nullptr;   // device
  double* dot_results_host = nullptr;  // pinned host mirror
  size_t dot_results_n = 0;
  std::vector<cudaEvent_t> event_pool;
  size_t events_used = 0;
};

class Runtime {
 public:
  static Runtime& get();
  int init();       // idempotent
  int finalize();
  int device_count() const { return ndev_; }
  DeviceCtx& dev(int d) { return devs_[d]; }
  bool peer_ok(int a, int b) const { return a == b || peer_[a][b]; }
  // Make sure streams/status words of GPU d exist.
  int ensure_device(int d);
  // Grow (never shrink) the slab of GPU d to at least `bytes`.
  int ensure_slab(int d, size_t bytes, double* alloc_ms);
  int free_slab(int d);
  int ensure_dot_scratch(int d, size_t partials_n, size_t results_n);
  // Staging ring of GPU d with slots of at least `slot_bytes`.
  int ensure_stage(int d, size_t slot_bytes);
  // Borrow an event (timing disabled) from GPU d's pool; valid until release_events(d).
  int get_event(int d, cudaEvent_t* ev);
  void release_events(int d) { devs_[d].events_used = 0; }
  // Read and clear GPU d's kernel status word (synchronises the device).
  int check_status(int d);
  // Order a call after what the caller already queued on the legacy default stream of the
  // GPUs in `devs` (a fill, a copy or a kernel that produces an operand): the library's
  // streams are non-blocking and would not see that work otherwise. The h2d stream of every
  // GPU in `units` waits; the call's start event is recorded on that stream afterwards.
  // Work on other streams of the caller has to be synchronised by the caller.
  int order_after_caller(const std::vector<int>& devs, const std::vector<int>& units);
  std::mutex& call_mutex() { return call_mutex_; }

 private:
  bool inited_ = false;
  int ndev_ = 0;
  std::vector<DeviceCtx> devs_;
  bool peer_[PARALIA_MAX_UNITS][PARALIA_MAX_UNITS] = {};
  std::mutex call_mutex_;
  std::mutex init_mutex_;
  std::mutex device_mutex_;
};

// RAII: remember the caller's current device and restore it on scope exit (the reference
// saves it at dgemm.cpp:336 but restores it only on one branch, dgemm.cpp:667).
struct DeviceGuard {
  int prev = -1;
  DeviceGuard() { if (cudaGetDevice(&prev) != cudaSuccess) prev = -1; }
  ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

// Where does a pointer live? Returns -1 for host memory (pinned or pageable; *pinned
// tells which), 0..G-1 for device memory. Reference: CoCoGetPtrLoc.
int pointer_location(const void* p, bool* pinned);

// The page-lock a call took on a pageable host operand (the reference pins host operands
// in place for the call, Decom2D::prepareAsync at dgemm.cpp:413-416, and unpins them at
// teardown, dgemm.cpp:669-678).
struct HostPin {
  const void* ptr = nullptr;
  bool registered = false;
  void release();
};

// Page-lock host ranges that are not page-locked yet; overlapping ranges are registered as
// one. pins[i] (n entries) receive the registrations, to be released by the caller.
struct HostRange {
  const void* ptr;
  size_t bytes;
};
int pin_host_ranges(const HostRange* ranges, int n, HostPin* pins, double* pin_ms);

// Check the location a caller declared for an operand (PARALIA_LOC_AUTO = ask the driver)
// against where the pointer really lives, and page-lock `bytes` of it if it is pageable
// host memory and `pin` is not null (callers with several host operands pass null and pin
// them together with pin_host_ranges). *loc_out receives -1 (host) or the GPU id.
int resolve_operand_location(const void* ptr, int loc_in, size_t bytes, int ngpu, int* loc_out,
                             HostPin* pin, double* pin_ms);

// 3-D tiled TMA descriptor over {d0 (contiguous), d1, d2} elements of `esz` bytes with
// 128-byte swizzle and zero fill outside the tensor.
int make_tensor_map(CUtensorMap* map, const void* base, int esz, uint64_t d0, uint64_t d1,
                    uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0,
                    uint32_t box1);

// True if TMA can address a matrix at `base` with leading dimension ld (elements of esz bytes).
inline bool tma_addressable(const void* base, int64_t ld, int esz) {
  return (reinterpret_cast<uintptr_t>(base) & 15) == 0 && ((ld * esz) & 15) == 0;
}

double wall_ms();

// Wait on the host for `ev` (recorded on GPU `dev`) with a deadline: PARALIA_ERR_TIMEOUT when
// it has not completed after deadline_ms, PARALIA_ERR_CUDA when the GPU reports an error.
int wait_event_with_deadline(cudaEvent_t ev, double deadline_ms, int dev);
// Deadline of a whole-problem call: PARALIA_JOIN_TIMEOUT_MS if set, else the larger of two
// minutes and fifty times the predicted duration.
double join_deadline_ms(double predicted_s);

}  // namespace paralia
