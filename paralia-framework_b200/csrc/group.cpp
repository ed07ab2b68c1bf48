#include "group.hpp"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>

#include "autotune.hpp"
#include "runtime.hpp"

namespace paralia {

namespace {
constexpr uint32_t SHM_MAGIC = 0x50414c47u;  // "PALG"
// How long a rank waits for the others at a hand-shake before it reports a missing rank.
static double barrier_timeout_ms() {
  static const double v = [] {
    const char* e = getenv("PARALIA_GROUP_TIMEOUT_MS");
    const double t = e ? atof(e) : 0.0;
    return t > 0.0 ? t : 60000.0;
  }();
  return v;
}
#define BARRIER_TIMEOUT_MS (barrier_timeout_ms())
Group* g_group = nullptr;
}  // namespace

struct Group::Shm {
  std::atomic<uint32_t> magic;
  std::atomic<uint32_t> arrived;
  std::atomic<uint32_t> generation;
  std::atomic<uint32_t> attached;
  // Set by the first rank that gives up on, or fails inside, a collective: from then on
  // every hand-shake of every rank fails at once with the recorded reason, so that one
  // rank's error never costs the others a time-out and an off-by-one arrival counter can
  // never let a later barrier pass with a rank missing.
  std::atomic<uint32_t> poisoned;
  int32_t poison_rank;
  char poison_msg[160];
  int32_t world;
  struct Rank {
    cudaIpcMemHandle_t slab_handle;
    uint64_t slab_gen;        // 0 = no slab exported
    uint64_t slab_bytes;
    int32_t will_realloc;
    int32_t failed;
    int32_t share_a_ok, share_b_ok;   // this rank's own verdict for the current call
    GroupCallInfo call;
    cudaIpcEventHandle_t ev[GROUP_MAX_EVENTS];
  } ranks[GROUP_MAX_RANKS];
};

Group* Group::current() { return g_group; }

const GroupCallInfo& Group::info(int peer) const { return shm_->ranks[peer].call; }

// Map the group's shared segment (rank 0 creates it) and wait until it is initialised.
// No CUDA involved. On success *out is a Group with rank, world, grid and shm_ set.
int Group::attach(const char* name, int rank, int world, Group** out) {
  if (!name || world < 1 || world > GROUP_MAX_RANKS || rank < 0 || rank >= world)
    return fail(PARALIA_ERR_INVALID_ARG, "bad group arguments (rank %d of %d)", rank, world);
  Group* g = new (std::nothrow) Group();
  if (!g) return fail(PARALIA_ERR_OUT_OF_MEMORY, "out of host memory");
  g->rank_ = rank;
  g->world_ = world;
  device_grid(world, &g->d1_, &g->d2_);
  snprintf(g->shm_name_, sizeof(g->shm_name_), "/paralia_%s", name);
  g->shm_bytes_ = sizeof(Shm);
  int fd = -1;
  const double t0 = wall_ms();
  if (rank == 0) {
    shm_unlink(g->shm_name_);
    fd = shm_open(g->shm_name_, O_CREAT | O_EXCL | O_RDWR, 0600);
    if (fd < 0 || ftruncate(fd, (off_t)g->shm_bytes_) != 0) {
      if (fd >= 0) close(fd);
      const int rc = fail(PARALIA_ERR_CUDA, "cannot create the shared segment %s", g->shm_name_);
      delete g;
      return rc;
    }
  } else {
    while ((fd = shm_open(g->shm_name_, O_RDWR, 0600)) < 0) {
      if (wall_ms() - t0 > BARRIER_TIMEOUT_MS) {
        delete g;
        return fail(PARALIA_ERR_TIMEOUT, "rank 0 never created the shared segment");
      }
      usleep(1000);
    }
    struct stat st;
    while (fstat(fd, &st) == 0 && (size_t)st.st_size < g->shm_bytes_) {
      if (wall_ms() - t0 > BARRIER_TIMEOUT_MS) {
        close(fd);
        delete g;
        return fail(PARALIA_ERR_TIMEOUT, "the shared segment never reached its size");
      }
      usleep(1000);
    }
  }
  void* p = mmap(nullptr, g->shm_bytes_, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) {
    delete g;
    return fail(PARALIA_ERR_CUDA, "cannot map the shared segment");
  }
  g->shm_ = static_cast<Shm*>(p);
  if (rank == 0) {
    memset(p, 0, g->shm_bytes_);
    g->shm_->world = world;
    g->shm_->magic.store(SHM_MAGIC, std::memory_order_release);
  } else {
    while (g->shm_->magic.load(std::memory_order_acquire) != SHM_MAGIC) {
      if (wall_ms() - t0 > BARRIER_TIMEOUT_MS) {
        munmap(p, g->shm_bytes_);
        delete g;
        return fail(PARALIA_ERR_TIMEOUT, "rank 0 never initialised the shared segment");
      }
      usleep(200);
    }
  }
  *out = g;
  return PARALIA_OK;
}

void Group::detach(Group* g) {
  if (g->shm_) munmap(g->shm_, g->shm_bytes_);
  delete g;
}

int Group::init(const char* name, int rank, int world, int dev) {
  if (g_group) return fail(PARALIA_ERR_INVALID_ARG, "a group is already initialised in this process");
  if (!name || world < 1 || world > GROUP_MAX_RANKS || rank < 0 || rank >= world)
    return fail(PARALIA_ERR_INVALID_ARG, "bad group arguments (rank %d of %d)", rank, world);
  Runtime& rt = Runtime::get();
  PL_TRY(rt.init());
  DeviceGuard guard;
  PL_TRY(rt.ensure_device(dev));
  Group* g = nullptr;
  PL_TRY(attach(name, rank, world, &g));
  g->dev_ = dev;
  // Inter-process events, one per shareable tile slot, exported once.
  cudaError_t ce = cudaSetDevice(dev);
  for (int i = 0; i < GROUP_MAX_EVENTS && ce == cudaSuccess; ++i) {
    ce = cudaEventCreateWithFlags(&g->own_ev_[i], cudaEventDisableTiming | cudaEventInterprocess);
    if (ce == cudaSuccess) ce = cudaIpcGetEventHandle(&g->shm_->ranks[rank].ev[i], g->own_ev_[i]);
  }
  if (ce != cudaSuccess) g->poison("a rank could not create its inter-process events");
  g->shm_->attached.fetch_add(1);
  g_group = g;
  int rc = g->barrier();
  if (ce != cudaSuccess && rc == PARALIA_OK)
    rc = fail(PARALIA_ERR_CUDA, "inter-process events: %s", cudaGetErrorString(ce));
  if (rank == 0) shm_unlink(g->shm_name_);  // every rank has it mapped (or never will)
  if (rc != PARALIA_OK) {
    // a rank never arrived: leave no half-built group behind
    for (int i = 0; i < GROUP_MAX_EVENTS; ++i)
      if (g->own_ev_[i]) cudaEventDestroy(g->own_ev_[i]);
    cudaGetLastError();
    detach(g);
    g_group = nullptr;
    return rc;
  }
  return PARALIA_OK;
}

// The hand-shake layer alone, without CUDA: `rounds` barriers between `world` processes.
// The rank named by fail_rank leaves at round fail_round: fail_mode 1 = it reports an error
// of its own (as a collective call does when its arguments are bad), fail_mode 2 = it just
// stops arriving. *waited_ms receives how long this rank spent in the barrier that failed.
int Group::selftest_rendezvous(const char* name, int rank, int world, int rounds, int fail_rank,
                               int fail_round, int fail_mode, double* waited_ms) {
  Group* g = nullptr;
  PL_TRY(attach(name, rank, world, &g));
  int rc = PARALIA_OK;
  if (waited_ms) *waited_ms = 0.0;
  for (int r = 0; r < rounds && rc == PARALIA_OK; ++r) {
    if (rank == fail_rank && r == fail_round) {
      if (fail_mode == 1) {
        rc = fail(PARALIA_ERR_INVALID_ARG, "injected failure of rank %d at round %d", rank, r);
        g->poison(last_error_cstr());
      } else {
        rc = fail(PARALIA_ERR_UNSUPPORTED, "rank %d stops arriving at round %d", rank, r);
      }
      break;
    }
    const double t0 = wall_ms();
    rc = g->barrier();
    if (rc != PARALIA_OK && waited_ms) *waited_ms = wall_ms() - t0;
  }
  if (rank == 0) shm_unlink(g->shm_name_);
  // a rank that leaves early keeps the segment mapped by its peers alive; nothing to wait for
  detach(g);
  return rc;
}

int Group::finalize() {
  Group* g = g_group;
  if (!g) return PARALIA_OK;
  DeviceGuard guard;
  cudaSetDevice(g->dev_);
  cudaDeviceSynchronize();
  // In an abandoned group the two hand-shakes below fail at once; the peers have been told
  // (every collective of theirs fails with the reason) and enqueue nothing that reads this
  // rank's slab any more, and the slab itself stays allocated until PARALiA_dev_cache_free.
  g->barrier();   // nobody is still reading a peer's slab
  for (int p = 0; p < g->world_; ++p) {
    if (g->peer_slab_[p]) cudaIpcCloseMemHandle(g->peer_slab_[p]);
    for (int i = 0; i < GROUP_MAX_EVENTS; ++i)
      if (g->peer_ev_[p][i]) cudaEventDestroy(g->peer_ev_[p][i]);
  }
  g->barrier();   // every importer has closed its mappings before slabs may be freed
  for (int i = 0; i < GROUP_MAX_EVENTS; ++i)
    if (g->own_ev_[i]) cudaEventDestroy(g->own_ev_[i]);
  cudaGetLastError();
  detach(g);
  g_group = nullptr;
  return PARALIA_OK;
}

void Group::poison(const char* why) {
  if (!shm_) return;
  uint32_t expected = 0;
  if (shm_->poisoned.compare_exchange_strong(expected, 1u, std::memory_order_acq_rel)) {
    shm_->poison_rank = rank_;
    snprintf(shm_->poison_msg, sizeof(shm_->poison_msg), "%s", why ? why : "unspecified error");
    shm_->poisoned.store(2u, std::memory_order_release);   // message complete
  }
}

bool Group::poisoned() const {
  return shm_ && shm_->poisoned.load(std::memory_order_acquire) != 0;
}

int Group::poisoned_error() const {
  // give the poisoning rank a moment to finish writing its reason
  for (int i = 0; i < 1000 && shm_->poisoned.load(std::memory_order_acquire) == 1u; ++i) usleep(10);
  char msg[160];
  snprintf(msg, sizeof(msg), "%s", shm_->poison_msg);
  msg[sizeof(msg) - 1] = 0;
  return fail(PARALIA_ERR_GROUP_FAILED, "rank %d: the process group was abandoned by rank %d (%s)",
              rank_, (int)shm_->poison_rank, msg);
}

int Group::barrier() {
  if (world_ == 1) return PARALIA_OK;
  if (poisoned()) return poisoned_error();
  const uint32_t gen = shm_->generation.load(std::memory_order_acquire);
  if (shm_->arrived.fetch_add(1, std::memory_order_acq_rel) + 1 == (uint32_t)world_) {
    shm_->arrived.store(0, std::memory_order_relaxed);
    shm_->generation.store(gen + 1, std::memory_order_release);
    return PARALIA_OK;
  }
  const double t0 = wall_ms();
  uint32_t spins = 0;
  while (shm_->generation.load(std::memory_order_acquire) == gen) {
    if ((++spins & 255u) == 0) {
      if (poisoned()) {
        shm_->arrived.fetch_sub(1, std::memory_order_acq_rel);
        return poisoned_error();
      }
      if ((spins & 1023u) == 0) {
        if (wall_ms() - t0 > BARRIER_TIMEOUT_MS) {
          // take the arrival back and abandon the group: nobody may pass a later
          // hand-shake on a counter that is one too high
          char why[96];
          snprintf(why, sizeof(why), "a hand-shake timed out after %.0f ms: a rank is missing",
                   BARRIER_TIMEOUT_MS);
          poison(why);
          shm_->arrived.fetch_sub(1, std::memory_order_acq_rel);
          return fail(PARALIA_ERR_TIMEOUT, "rank %d: a group barrier timed out (a rank is missing)",
                      rank_);
        }
        usleep(20);
      }
    }
  }
  return PARALIA_OK;
}

int Group::peer_event(int peer, int slot, cudaEvent_t* ev) {
  if (peer < 0 || peer >= world_ || slot < 0 || slot >= GROUP_MAX_EVENTS)
    return fail(PARALIA_ERR_INVALID_ARG, "bad peer event (%d, %d)", peer, slot);
  if (!peer_ev_[peer][slot])
    PL_CUDA(cudaIpcOpenEventHandle(&peer_ev_[peer][slot], shm_->ranks[peer].ev[slot]));
  *ev = peer_ev_[peer][slot];
  return PARALIA_OK;
}

int Group::open_peer_slabs() {
  for (int p = 0; p < world_; ++p) {
    if (p == rank_) continue;
    const Shm::Rank& r = shm_->ranks[p];
    if (r.slab_gen == peer_gen_[p]) continue;
    if (peer_slab_[p]) {   // normally closed already in begin_call
      PL_CUDA(cudaIpcCloseMemHandle(peer_slab_[p]));
      peer_slab_[p] = nullptr;
    }
    if (r.slab_gen != 0) {
      // A slab that cannot be mapped only switches sharing with that rank off.
      cudaError_t e = cudaIpcOpenMemHandle(&peer_slab_[p], r.slab_handle,
                                           cudaIpcMemLazyEnablePeerAccess);
      if (e != cudaSuccess) {
        cudaGetLastError();
        peer_slab_[p] = nullptr;
      }
    }
    peer_gen_[p] = r.slab_gen;
  }
  return PARALIA_OK;
}

int Group::begin_call(const GroupCallInfo& mine, size_t slab_bytes, double* alloc_ms,
                      bool* share_a, bool* share_b) {
  Runtime& rt = Runtime::get();
  DeviceCtx& dc = rt.dev(dev_);
  Shm::Rank& me = shm_->ranks[rank_];
  PL_CUDA(cudaSetDevice(dev_));
  // 1. say whether the slab is about to be replaced, so importers unmap it first
  me.call = mine;
  me.will_realloc = dc.slab_bytes < slab_bytes ? 1 : 0;
  PL_TRY(barrier());
  for (int p = 0; p < world_; ++p)
    if (p != rank_ && shm_->ranks[p].will_realloc && peer_slab_[p]) {
      PL_CUDA(cudaIpcCloseMemHandle(peer_slab_[p]));
      peer_slab_[p] = nullptr;
      peer_gen_[p] = 0;
    }
  PL_TRY(barrier());
  // 2. (re)allocate and export
  int rc = rt.ensure_slab(dev_, slab_bytes, alloc_ms);
  me.failed = rc != PARALIA_OK;
  if (rc == PARALIA_OK && dc.slab && dc.slab_gen != my_gen_) {
    cudaError_t e = cudaIpcGetMemHandle(&me.slab_handle, dc.slab);
    if (e != cudaSuccess) {
      cudaGetLastError();
      me.failed = 1;
      rc = fail(PARALIA_ERR_CUDA, "cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
    } else {
      my_gen_ = dc.slab_gen;
      // generations of different ranks never collide with "0 = nothing exported"
      me.slab_gen = my_gen_ + 1;
      me.slab_bytes = dc.slab_bytes;
    }
  }
  int rcb = barrier();
  if (rc != PARALIA_OK) return rc;
  PL_TRY(rcb);
  for (int p = 0; p < world_; ++p)
    if (shm_->ranks[p].failed)
      return fail(PARALIA_ERR_OUT_OF_MEMORY, "rank %d could not set up its tile cache", p);
  PL_TRY(open_peer_slabs());
  // 3. sharing is on for an operand only if every rank of the grid row (A) / column (B)
  //    runs the same tiling of the same panel
  const int r = rank_ / d2_, c = rank_ % d2_;
  bool sa = mine.a_host && mine.want_share && d2_ > 1 && mine.nA + mine.nB <= GROUP_MAX_EVENTS;
  bool sb = mine.b_host && mine.want_share && d1_ > 1 && mine.nA + mine.nB <= GROUP_MAX_EVENTS;
  for (int cc = 0; cc < d2_ && sa; ++cc) {
    const GroupCallInfo& o = shm_->ranks[r * d2_ + cc].call;
    sa = o.a_host && o.want_share && o.T == mine.T && o.TL == mine.TL && o.Mloc == mine.Mloc &&
         o.K == mine.K && o.ta == mine.ta && o.esz == mine.esz && o.nA == mine.nA &&
         o.nA + o.nB <= GROUP_MAX_EVENTS &&
         (r * d2_ + cc == rank_ || peer_slab_[r * d2_ + cc] != nullptr);
  }
  for (int rr = 0; rr < d1_ && sb; ++rr) {
    const GroupCallInfo& o = shm_->ranks[rr * d2_ + c].call;
    sb = o.b_host && o.want_share && o.T == mine.T && o.TL == mine.TL && o.Nloc == mine.Nloc &&
         o.K == mine.K && o.tb == mine.tb && o.esz == mine.esz && o.nB == mine.nB &&
         o.nA + o.nB <= GROUP_MAX_EVENTS &&
         (rr * d2_ + c == rank_ || peer_slab_[rr * d2_ + c] != nullptr);
  }
  // 4. the verdict must be the same on every rank of the row / column: a rank that
  //    shares waits for events that a rank that does not share would never record
  me.share_a_ok = sa;
  me.share_b_ok = sb;
  PL_TRY(barrier());
  for (int cc = 0; cc < d2_; ++cc) sa = sa && shm_->ranks[r * d2_ + cc].share_a_ok;
  for (int rr = 0; rr < d1_; ++rr) sb = sb && shm_->ranks[rr * d2_ + c].share_b_ok;
  *share_a = sa;
  *share_b = sb;
  return PARALIA_OK;
}

}  // namespace paralia
