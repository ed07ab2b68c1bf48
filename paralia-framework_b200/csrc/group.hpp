// One-process-per-GPU groups.
//
// The reference (and this library's default mode) drives every GPU of the box from one
// process, so a tile fetched from the host by one GPU can be handed to another GPU with a
// plain peer copy. When a launcher starts one process per GPU instead, the processes of a
// group get the same effect through CUDA IPC: each rank exports its tile-cache slab and a
// pool of inter-process events once; during a call the rank that is the "home" of a
// host-resident tile copies it over its host link and records the tile's event, the other
// ranks that need the tile wait on that event and copy it GPU -> GPU out of the home's
// slab. Hand-shakes between the processes (three cheap barriers per call) go through a
// small POSIX shared-memory segment; no other transport is needed.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/paralia_c.h"

namespace paralia {

constexpr int GROUP_MAX_RANKS = 16;
constexpr int GROUP_MAX_EVENTS = 1024;   // shareable tiles per rank and call

// What a rank tells the others about the call it is in.
struct GroupCallInfo {
  int64_t Mloc, Nloc, K, T, TL;
  int32_t ta, tb, esz;
  int32_t a_host, b_host;   // operand is host-resident (and may therefore be shared)
  int32_t nA, nB;           // A tiles occupy blocks [0,nA), B tiles [nA, nA+nB)
  int32_t want_share;       // caller did not disable peer fetches
};

class Group {
 public:
  static Group* current();   // null when no group is initialised
  static int init(const char* name, int rank, int world, int dev);
  static int finalize();
  // The hand-shake layer alone (no CUDA): see group.cpp.
  static int selftest_rendezvous(const char* name, int rank, int world, int rounds, int fail_rank,
                                 int fail_round, int fail_mode, double* waited_ms);

  int rank() const { return rank_; }
  int world() const { return world_; }
  int dev() const { return dev_; }
  void grid(int* d1, int* d2) const { *d1 = d1_; *d2 = d2_; }

  // Collective. Bounded wait: PARALIA_ERR_TIMEOUT when a rank does not arrive; the rank that
  // times out abandons ("poisons") the group, after which every hand-shake of every rank
  // fails at once with PARALIA_ERR_GROUP_FAILED and the reason.
  int barrier();
  // Abandon the group because this rank failed where its peers expect it in a collective.
  void poison(const char* why);
  bool poisoned() const;

  // Collective start of a call: agree on sharing, (re)allocate the slab of `bytes` with
  // every importer's mapping closed first, exchange slab handles. On return *share_a /
  // *share_b say whether A / B tiles are shared inside this rank's grid row / column.
  int begin_call(const GroupCallInfo& mine, size_t slab_bytes, double* alloc_ms, bool* share_a,
                 bool* share_b);

  // Event this rank records when its home tile `slot` has landed in its slab.
  cudaEvent_t own_event(int slot) { return own_ev_[slot]; }
  // The same event of another rank (opened on first use), and that rank's slab.
  int peer_event(int peer, int slot, cudaEvent_t* ev);
  char* peer_slab(int peer) { return static_cast<char*>(peer_slab_[peer]); }
  const GroupCallInfo& info(int peer) const;

 private:
  Group() = default;
  static int attach(const char* name, int rank, int world, Group** out);
  static void detach(Group* g);
  int open_peer_slabs();
  int poisoned_error() const;
  struct Shm;
  Shm* shm_ = nullptr;
  size_t shm_bytes_ = 0;
  char shm_name_[128] = {0};
  int rank_ = 0, world_ = 1, dev_ = 0, d1_ = 1, d2_ = 1;
  cudaEvent_t own_ev_[GROUP_MAX_EVENTS] = {};
  cudaEvent_t peer_ev_[GROUP_MAX_RANKS][GROUP_MAX_EVENTS] = {};
  void* peer_slab_[GROUP_MAX_RANKS] = {};
  uint64_t peer_gen_[GROUP_MAX_RANKS] = {};
  uint64_t my_gen_ = 0;
};

}  // namespace paralia
