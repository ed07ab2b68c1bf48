#include <algorithm>
#include "runtime.hpp"

#include <dlfcn.h>
#include <unistd.h>

#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "autotune.hpp"
#include "dgemm_tile.cuh"
#include "level1.cuh"
#include "sgemm_tile.cuh"

namespace paralia {

static thread_local char g_err[1024] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
const char* last_error_cstr() { return g_err; }

double wall_ms() {
  using namespace std::chrono;
  return duration<double, std::milli>(steady_clock::now().time_since_epoch()).count();
}

Runtime& Runtime::get() {
  static Runtime rt;
  return rt;
}

int Runtime::init() {
  std::lock_guard<std::mutex> lk(init_mutex_);
  if (inited_) return PARALIA_OK;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n <= 0) {
    cudaGetLastError();
    return fail(PARALIA_ERR_NO_DEVICE, "no CUDA device visible (%s)",
                e == cudaSuccess ? "count is 0" : cudaGetErrorString(e));
  }
  if (n > PARALIA_MAX_UNITS) n = PARALIA_MAX_UNITS;
  DeviceGuard guard;
  ndev_ = n;
  devs_.assign(n, DeviceCtx());
  for (int d = 0; d < n; ++d) devs_[d].dev = d;
  inited_ = true;
  // Calibration database named by the environment (reference: compile-time DEPLOYDB).
  // Otherwise the tables shipped beside the library (<dir of libparalia.so>/../db_b200).
  if (const char* db = getenv("PARALIA_DB")) {
    reset_database_defaults(ndev_);
    if (load_database(db) != PARALIA_OK) fprintf(stderr, "libparalia: %s\n", last_error_cstr());
  } else {
    Dl_info info;
    if (dladdr(reinterpret_cast<const void*>(&wall_ms), &info) && info.dli_fname) {
      std::string path(info.dli_fname);
      const size_t cut = path.rfind('/');
      if (cut != std::string::npos) {
        const std::string db = path.substr(0, cut) + "/../db_b200";
        FILE* probe = fopen((db + "/Processed/Dgemm_lookup-table_dev-0.log").c_str(), "r");
        if (probe) {
          fclose(probe);
          reset_database_defaults(ndev_);
          if (load_database(db.c_str()) != PARALIA_OK) reset_database_defaults(ndev_);
        }
      }
    }
  }
  return PARALIA_OK;
}

int wait_event_with_deadline(cudaEvent_t ev, double deadline_ms, int dev) {
  const double t0 = wall_ms();
  for (unsigned spins = 0;; ++spins) {
    const cudaError_t e = cudaEventQuery(ev);
    if (e == cudaSuccess) return PARALIA_OK;
    if (e != cudaErrorNotReady)
      return fail(PARALIA_ERR_CUDA, "GPU %d failed while running the plan: %s", dev, cudaGetErrorString(e));
    if (wall_ms() - t0 > deadline_ms)
      return fail(PARALIA_ERR_TIMEOUT, "GPU %d: the work of this call did not finish within its "
                  "deadline of %.0f ms", dev, deadline_ms);
    if (spins > 2000) usleep(50);   // the first milliseconds are polled without sleeping
  }
}

double join_deadline_ms(double predicted_s) {
  static const double forced = [] {
    const char* e = getenv("PARALIA_JOIN_TIMEOUT_MS");
    return e ? atof(e) : 0.0;
  }();
  if (forced > 0.0) return forced;
  return std::max(120000.0, 50.0 * 1e3 * std::max(predicted_s, 0.0));
}

void HostPin::release() {
  if (registered) cudaHostUnregister(const_cast<void*>(ptr));
  registered = false;
}

int resolve_operand_location(const void* ptr, int loc_in, size_t bytes, int ngpu, int* loc_out,
                             HostPin* pin, double* pin_ms) {
  bool pinned = false;
  const int actual = pointer_location(ptr, &pinned);
  const int loc = loc_in == PARALIA_LOC_AUTO ? actual : loc_in;
  if (loc < -1 || loc >= ngpu)
    return fail(PARALIA_ERR_INVALID_ARG, "location id %d is neither -1 nor a GPU of this box", loc);
  if (loc >= 0 && actual != loc)
    return fail(PARALIA_ERR_INVALID_ARG, "operand declared on GPU %d but the pointer lives on %d",
                loc, actual);
  if (loc == -1 && actual >= 0)
    return fail(PARALIA_ERR_INVALID_ARG, "operand declared on the host but the pointer is on GPU %d",
                actual);
  *loc_out = loc;
  if (loc == -1 && bytes > 0 && pin) {
    HostRange r{ptr, bytes};
    return pin_host_ranges(&r, 1, pin, pin_ms);
  }
  return PARALIA_OK;
}

// Page-lock the host ranges that are not page-locked yet. Ranges that overlap (operands that
// are interleaved views of one parent matrix: their address ranges interleave column by
// column) are registered as one range: CUDA neither registers a range that overlaps a
// registered one nor copies asynchronously from a half-registered range. pins[i] receives
// the registration made on behalf of range i (several ranges may share one; it is recorded
// with the first of them).
int pin_host_ranges(const HostRange* ranges, int n, HostPin* pins, double* pin_ms) {
  struct Need { uintptr_t lo, hi; int first; };
  std::vector<Need> need;
  for (int i = 0; i < n; ++i) {
    if (!ranges[i].ptr || ranges[i].bytes == 0) continue;
    const char* base = static_cast<const char*>(ranges[i].ptr);
    bool head = false, tail = false;
    if (pointer_location(base, &head) >= 0) continue;   // not host memory: nothing to pin
    pointer_location(base + ranges[i].bytes - 1, &tail);
    if (head && tail) continue;                          // page-locked already
    need.push_back({reinterpret_cast<uintptr_t>(base),
                    reinterpret_cast<uintptr_t>(base) + ranges[i].bytes, i});
  }
  std::sort(need.begin(), need.end(), [](const Need& a, const Need& b) { return a.lo < b.lo; });
  std::vector<Need> merged;
  for (const Need& r : need) {
    if (!merged.empty() && r.lo < merged.back().hi) {
      merged.back().hi = std::max(merged.back().hi, r.hi);
      merged.back().first = std::min(merged.back().first, r.first);
    } else {
      merged.push_back(r);
    }
  }
  const double t0 = wall_ms();
  for (const Need& r : merged) {
    cudaError_t e = cudaHostRegister(reinterpret_cast<void*>(r.lo), r.hi - r.lo, cudaHostRegisterPortable);
    if (e != cudaSuccess) {
      cudaGetLastError();
      for (int i = 0; i < n; ++i) pins[i].release();
      return fail(PARALIA_ERR_CUDA, "cannot page-lock a host operand of %zu bytes: %s",
                  (size_t)(r.hi - r.lo), cudaGetErrorString(e));
    }
    pins[r.first].ptr = reinterpret_cast<const void*>(r.lo);
    pins[r.first].registered = true;
  }
  if (pin_ms && !merged.empty()) *pin_ms += wall_ms() - t0;
  return PARALIA_OK;
}

int Runtime::order_after_caller(const std::vector<int>& devs, const std::vector<int>& units) {
  std::vector<int> marked;
  for (int d : devs) {
    if (d < 0 || d >= ndev_) continue;   // host operands have no stream to join
    if (std::find(marked.begin(), marked.end(), d) != marked.end()) continue;
    PL_TRY(ensure_device(d));
    PL_CUDA(cudaSetDevice(d));
    PL_CUDA(cudaEventRecord(devs_[d].caller_ready, cudaStreamLegacy));
    marked.push_back(d);
  }
  for (int u : units) {
    PL_TRY(ensure_device(u));
    PL_CUDA(cudaSetDevice(u));
    for (int d : marked) PL_CUDA(cudaStreamWaitEvent(devs_[u].h2d, devs_[d].caller_ready, 0));
  }
  return PARALIA_OK;
}

int Runtime::ensure_device(int d) {
  if (d < 0 || d >= ndev_) return fail(PARALIA_ERR_INVALID_ARG, "GPU id %d out of range", d);
  DeviceCtx& c = devs_[d];
  // the per-tile entry points may be called from several threads: one of them sets a GPU up
  std::lock_guard<std::mutex> lk(device_mutex_);
  if (c.ready) return PARALIA_OK;
  PL_CUDA(cudaSetDevice(d));
  PL_CUDA(cudaStreamCreateWithFlags(&c.h2d, cudaStreamNonBlocking));
  PL_CUDA(cudaStreamCreateWithFlags(&c.d2h, cudaStreamNonBlocking));
  PL_CUDA(cudaStreamCreateWithFlags(&c.p2p, cudaStreamNonBlocking));
  for (int i = 0; i < MAX_EXEC_STREAMS; ++i)
    PL_CUDA(cudaStreamCreateWithFlags(&c.exec[i], cudaStreamNonBlocking));
  PL_CUDA(cudaStreamCreateWithFlags(&c.pack, cudaStreamNonBlocking));
  for (int i = 0; i < DeviceCtx::STAGE_SLOTS; ++i)
    PL_CUDA(cudaEventCreateWithFlags(&c.stage_free[i], cudaEventDisableTiming));
  PL_CUDA(cudaEventCreate(&c.t_begin));
  PL_CUDA(cudaEventCreate(&c.t_end));
  PL_CUDA(cudaEventCreate(&c.t_first_exec));
  PL_CUDA(cudaEventCreate(&c.t_h2d_end));
  for (int i = 0; i < MAX_EXEC_STREAMS; ++i) PL_CUDA(cudaEventCreate(&c.t_exec_end[i]));
  PL_CUDA(cudaEventCreateWithFlags(&c.caller_ready, cudaEventDisableTiming));
  PL_CUDA(cudaMalloc(&c.status_dev, sizeof(int)));
  PL_CUDA(cudaMemset(c.status_dev, 0, sizeof(int)));
  PL_CUDA(dgemm_tile_configure());
  PL_CUDA(sgemm_tile_configure());
  {
    // keep stream-ordered scratch (per-tile SGEMM packing) cached between calls
    cudaMemPool_t pool;
    if (cudaDeviceGetDefaultMemPool(&pool, d) == cudaSuccess) {
      uint64_t keep = UINT64_MAX;
      cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    }
    cudaGetLastError();
  }
  // Peer access between this GPU and every GPU already in use (reference: CoCoEnableLinks
  // for every location, dgemm.cpp:423). Done pairwise as GPUs come into use, so a process
  // that drives a single GPU never creates a context on the others. On an NVSwitch box
  // every pair is reachable at the same bandwidth.
  for (int o = 0; o < ndev_; ++o) {
    if (o == d || !devs_[o].ready) continue;
    for (int dir = 0; dir < 2; ++dir) {
      const int a = dir ? o : d, b = dir ? d : o;
      int can = 0;
      PL_CUDA(cudaSetDevice(a));
      PL_CUDA(cudaDeviceCanAccessPeer(&can, a, b));
      if (!can) continue;
      cudaError_t pe = cudaDeviceEnablePeerAccess(b, 0);
      if (pe == cudaErrorPeerAccessAlreadyEnabled) pe = cudaSuccess;
      cudaGetLastError();
      peer_[a][b] = (pe == cudaSuccess);
    }
  }
  PL_CUDA(cudaSetDevice(d));
  c.ready = true;
  return PARALIA_OK;
}

int Runtime::ensure_slab(int d, size_t bytes, double* alloc_ms) {
  DeviceCtx& c = devs_[d];
  if (c.slab_bytes >= bytes) return PARALIA_OK;
  const double t0 = wall_ms();
  PL_CUDA(cudaSetDevice(d));
  if (c.slab) {
    PL_CUDA(cudaDeviceSynchronize());
    PL_CUDA(cudaFree(c.slab));
    c.slab = nullptr;
    c.slab_bytes = 0;
  }
  cudaError_t e = cudaMalloc(&c.slab, bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    c.slab = nullptr;
    return fail(PARALIA_ERR_OUT_OF_MEMORY, "GPU %d: cannot allocate a %zu-byte tile cache (%s)", d,
                bytes, cudaGetErrorString(e));
  }
  c.slab_bytes = bytes;
  ++c.slab_gen;
  if (alloc_ms) *alloc_ms += wall_ms() - t0;
  return PARALIA_OK;
}

int Runtime::free_slab(int d) {
  if (d < 0 || d >= ndev_) return fail(PARALIA_ERR_INVALID_ARG, "GPU id %d out of range", d);
  DeviceCtx& c = devs_[d];
  if (!c.slab) return PARALIA_OK;
  PL_CUDA(cudaSetDevice(d));
  PL_CUDA(cudaDeviceSynchronize());
  PL_CUDA(cudaFree(c.slab));
  c.slab = nullptr;
  c.slab_bytes = 0;
  ++c.slab_gen;
  return PARALIA_OK;
}

int Runtime::ensure_dot_scratch(int d, size_t partials_n, size_t results_n) {
  DeviceCtx& c = devs_[d];
  PL_CUDA(cudaSetDevice(d));
  if (c.dot_partials_n < partials_n) {
    if (c.dot_partials) PL_CUDA(cudaFree(c.dot_partials));
    PL_CUDA(cudaMalloc(&c.dot_partials, partials_n * sizeof(double)));
    c.dot_partials_n = partials_n;
  }
  if (c.dot_results_n < results_n) {
    if (c.dot_results) PL_CUDA(cudaFree(c.dot_results));
    if (c.dot_results_host) PL_CUDA(cudaFreeHost(c.dot_results_host));
    PL_CUDA(cudaMalloc(&c.dot_results, results_n * sizeof(double)));
    PL_CUDA(cudaMallocHost(&c.dot_results_host, results_n * sizeof(double)));
    c.dot_results_n = results_n;
  }
  return PARALIA_OK;
}

int Runtime::ensure_stage(int d, size_t slot_bytes) {
  DeviceCtx& c = devs_[d];
  if (c.stage_slot_bytes >= slot_bytes) return PARALIA_OK;
  PL_CUDA(cudaSetDevice(d));
  if (c.stage) {
    PL_CUDA(cudaDeviceSynchronize());
    PL_CUDA(cudaFree(c.stage));
    c.stage = nullptr;
    c.stage_slot_bytes = 0;
  }
  cudaError_t e = cudaMalloc(&c.stage, slot_bytes * DeviceCtx::STAGE_SLOTS);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(PARALIA_ERR_OUT_OF_MEMORY, "GPU %d: cannot allocate the staging ring (%s)", d,
                cudaGetErrorString(e));
  }
  c.stage_slot_bytes = slot_bytes;
  for (int i = 0; i < DeviceCtx::STAGE_SLOTS; ++i) c.stage_used[i] = false;
  c.stage_next = 0;
  return PARALIA_OK;
}

int Runtime::get_event(int d, cudaEvent_t* ev) {
  DeviceCtx& c = devs_[d];
  if (c.events_used == c.event_pool.size()) {
    PL_CUDA(cudaSetDevice(d));
    cudaEvent_t e;
    PL_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    c.event_pool.push_back(e);
  }
  *ev = c.event_pool[c.events_used++];
  return PARALIA_OK;
}

int Runtime::check_status(int d) {
  DeviceCtx& c = devs_[d];
  if (!c.ready) return PARALIA_OK;
  int word = 0;
  PL_CUDA(cudaSetDevice(d));
  PL_CUDA(cudaMemcpy(&word, c.status_dev, sizeof(int), cudaMemcpyDeviceToHost));
  if (word != 0) {
    PL_CUDA(cudaMemset(c.status_dev, 0, sizeof(int)));
    return fail(PARALIA_ERR_TIMEOUT, "GPU %d: a kernel gave up on a bounded wait (code %d)", d,
                word);
  }
  return PARALIA_OK;
}

int Runtime::finalize() {
  std::lock_guard<std::mutex> lk(init_mutex_);
  if (!inited_) return PARALIA_OK;
  DeviceGuard guard;
  for (int d = 0; d < ndev_; ++d) {
    DeviceCtx& c = devs_[d];
    if (cudaSetDevice(d) != cudaSuccess) continue;
    cudaDeviceSynchronize();
    if (c.slab) cudaFree(c.slab);
    if (c.stage) cudaFree(c.stage);
    if (c.status_dev) cudaFree(c.status_dev);
    if (c.dot_partials) cudaFree(c.dot_partials);
    if (c.dot_results) cudaFree(c.dot_results);
    if (c.dot_results_host) cudaFreeHost(c.dot_results_host);
    for (cudaEvent_t e : c.event_pool) cudaEventDestroy(e);
    if (c.ready) {
      cudaStreamDestroy(c.h2d);
      cudaStreamDestroy(c.d2h);
      cudaStreamDestroy(c.p2p);
      cudaStreamDestroy(c.pack);
      for (int i = 0; i < DeviceCtx::STAGE_SLOTS; ++i) cudaEventDestroy(c.stage_free[i]);
      for (int i = 0; i < MAX_EXEC_STREAMS; ++i) cudaStreamDestroy(c.exec[i]);
      cudaEventDestroy(c.t_begin);
      if (c.caller_ready) cudaEventDestroy(c.caller_ready);
      cudaEventDestroy(c.t_end);
      if (c.t_first_exec) cudaEventDestroy(c.t_first_exec);
      if (c.t_h2d_end) cudaEventDestroy(c.t_h2d_end);
      for (int i = 0; i < MAX_EXEC_STREAMS; ++i)
        if (c.t_exec_end[i]) cudaEventDestroy(c.t_exec_end[i]);
    }
  }
  ddot_noalloc_forget_addresses();
  devs_.clear();
  ndev_ = 0;
  inited_ = false;
  cudaGetLastError();
  return PARALIA_OK;
}

int pointer_location(const void* p, bool* pinned) {
  cudaPointerAttributes at;
  memset(&at, 0, sizeof(at));
  cudaError_t e = cudaPointerGetAttributes(&at, p);
  if (pinned) *pinned = false;
  if (e != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  if (at.type == cudaMemoryTypeDevice) return at.device;
  if (at.type == cudaMemoryTypeManaged) return at.device;
  if (at.type == cudaMemoryTypeHost) {
    if (pinned) *pinned = true;
    return -1;
  }
  return -1;  // unregistered host memory
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    else
      cudaGetLastError();
  });
  return fn;
}

int make_tensor_map(CUtensorMap* map, const void* base, int esz, uint64_t d0, uint64_t d1,
                    uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0,
                    uint32_t box1) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(PARALIA_ERR_CUDA, "driver entry point cuTensorMapEncodeTiled not found");
  const cuuint64_t dims[3] = {d0, d1, d2};
  const cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  const cuuint32_t box[3] = {box0, box1, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt =
      esz == 8 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT64 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = fn(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(PARALIA_ERR_CUDA,
                "cuTensorMapEncodeTiled failed (%d): base=%p dims=%llu,%llu,%llu strides=%llu,%llu "
                "box=%u,%u",
                (int)r, base, (unsigned long long)d0, (unsigned long long)d1,
                (unsigned long long)d2, (unsigned long long)stride1_bytes,
                (unsigned long long)stride2_bytes, box0, box1);
  return PARALIA_OK;
}

}  // namespace paralia
