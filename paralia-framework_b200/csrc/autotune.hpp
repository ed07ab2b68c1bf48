// Model-driven choice of tile size, device set and subkernel distribution.
//
// Keeps the form of the reference's autotuner (Autotuner/src/Autotuner.cpp:279-818,
// Subkernel_distributions.cpp:315-485, ModelLvl3.cpp:75-237, ModelLvl1.cpp:19-144,
// CoModel.cpp:108-140, LinkMap.cpp:121-269, GPUexec_lookup.cpp:103-129,250-359): measured
// tile-time tables, a linear model per link, slowdown factors between links that share
// hardware, per-unit time = max(exec, receive, send, peer traffic). What is specific to one
// 8 x B200 NVSwitch box: only the host links contend (every GPU pair has its own full-rate
// path through the switch), the contention is measured as an aggregate over the number of
// GPUs pulling at once, and the tile edge is the arg-min of the predicted time over the
// measured tile sizes instead of a score with hand-set constants.
#pragma once
#include <stdint.h>
#include <map>
#include <string>
#include <vector>

#include "../../include/paralia_c.h"
#include "plan.hpp"

namespace paralia {

// Compile-time -D switches of the reference (CMakeLists.txt:157-165,
// Autotuner/CMakeLists.txt:10-24) as one run-time record. They feed tile_slowdowns(), the
// reference's tile score, which is still reported but no longer picks the tile.
struct TuneConstants {
  int64_t tile_min = 2048;
  double tile_min_slowdown = 0.2;
  int64_t tile_max = 4096;
  double tile_max_slowdown = 0.1;
  int64_t max_desired_sk_dev = 512;
  double max_desired_sk_dev_slowdown = 0.1;
  double minimum_unit_contribution = 0.05;
  // Tile edges this build considers: multiples of tile_step (TMA rows are 16 elements
  // wide; CTA tiles are 128 wide), or the whole smallest dimension.
  int64_t tile_step = 128;
  // Host side of a call, measured on an 8 x B200 box with one thread driving all GPUs
  // (70-problem placement sweep): a fixed part (set-up, start and end events, the join) and a
  // part per enqueued operation (a tile kernel launch with its event waits, or a tile copy
  // with its event record). The executor enqueues just in time, so this time adds to the
  // device time instead of hiding under it; it is what makes small tiles expensive on
  // millisecond-sized problems.
  double call_fixed_s = 0.5e-3;
  double enqueue_op_s = 2.8e-6;
};

// t = ti + tb*bytes (CoModel.cpp:108-117) plus how much slower the link gets while
// another link is busy (the "Slowdown([src]->[dst]): ratio" lines, CoModel.cpp:32-55).
struct LinkSlowdown {
  int dst, src;     // location ids of the other link (-1 host)
  double ratio;     // t_shared / t_alone, clamped to [1, 2] as the reference does
};
struct LinkModel {
  double ti = 0.0;   // seconds
  double tb = 0.0;   // seconds per byte
  std::vector<LinkSlowdown> slow;
};

// Aggregate host-link bandwidth (GB/s, summed over the GPUs) against the number of GPUs
// that copy at the same time: host -> GPU alone, GPU -> host alone, and per direction when
// both directions run together. The pairwise slowdowns cannot express a cap that only
// shows with many GPUs (root complex, host memory), this table does.
struct HostAggregate {
  std::map<int, double> h2d, d2h, bidir;
  bool empty() const { return h2d.empty() && d2h.empty() && bidir.empty(); }
};

// One routine's measured tile time on a GPU: (T -> seconds) per transpose pair
// (GPUexec_lookup.cpp:41-101); level-1 routines use the key "--" and T = vector length
// (GPUexec_lookup.cpp:250-359).
struct ExecTable {
  std::map<std::string, std::map<int64_t, double>> by_trans;  // key "NN","NT","TN","TT","--"
  bool empty() const { return by_trans.empty(); }
};

struct ModelDB {
  // index 0 = host (-1), 1.. = GPU 0..; [dst][src]
  std::vector<std::vector<LinkModel>> link;
  std::map<std::string, ExecTable> exec;  // "Dgemm", "Sgemm", "Daxpy", "Ddot"
  HostAggregate host;
  bool from_disk = false;
  std::string dir;
};

// The library's current database (defaults describing a B200 box until
// load_database() replaces them).
ModelDB& model_db();
TuneConstants& tune_constants();
int load_database(const char* dir);
void reset_database_defaults(int ngpu);

// The reference's tile-size score, lower is better (Autotuner.cpp:571-603). sl[0] aggregate,
// sl[1] imbalance, sl[2] remainder, sl[3] small tile, sl[4] subkernel count, sl[5] big tile.
void tile_slowdowns(int64_t D1, int64_t D2, int64_t D3, int64_t T, int units,
                    const TuneConstants& c, double sl[6]);

// The reference's tile choice: argmin of sl[0], scanning from min(D1,D2,D3) downwards, first
// strict minimum wins (Autotuner.cpp:605-655). step = 1 is its exhaustive scan. Kept as the
// fallback when no tile table is loaded, and for comparison.
int64_t optimize_tile(int64_t D1, int64_t D2, int64_t D3, int units, const TuneConstants& c,
                      int64_t step, double sl[6]);

// Most-square factorisation units = d1*d2 by the reference's rule
// (Subkernel_distributions.cpp:325-336).
void device_grid(int units, int* d1, int* d2);

// Subkernel lists per unit for a Mt x Nt x Kt grid, equal scores: the owner map of
// Subkernel_distributions.cpp:315-485 (with its round-robin cases :10-76, :143-220).
// Returns the number of units that received work (fewer than `units` when there are fewer
// C tiles than units), or -1 where the reference's rule runs out of room.
int distribute_subkernels_2d(int units, int Mt, int Nt, int Kt,
                             std::vector<std::vector<int>>* lists, int* d1, int* d2);

struct GemmModelInput {
  int esz;
  char ta, tb;
  int64_t M, N, K;
  int locA, locB, locC;   // -1 host, >=0 GPU
  bool beta_nonzero = true;
  const char* func;       // "Dgemm" / "Sgemm"
  int enqueue_threads = 1;   // host threads that enqueue (one per rank in a process group)
};

struct UnitPrediction {
  double t_exec, t_recv, t_send, t_extra, t_fill, t_drain, t_total;
};

// Operations the host enqueues for a problem cut into Mt x Nt x Kt tiles on a d1 x d2 device
// grid: tile kernel launches (the k chains of plan.hpp) and tile copies (every consumer of an
// A or B tile gets its own copy unless the tile already lives on it; C tiles in and out).
int64_t count_enqueue_ops(const GemmModelInput& in, int64_t Mt, int64_t Nt, int64_t Kt, int d1,
                          int d2, int n_active);

// Seconds one tile GEMM of edge T takes on a GPU (lookup with cubic extrapolation,
// GPUexec_lookup.cpp:103-129).
double predict_tile_exec(const char* func, char ta, char tb, int64_t T);
// Seconds one level-1 tile of n elements takes ("Daxpy", "Ddot"); -1 without a table.
double predict_vec_exec(const char* func, int64_t n);

// Seconds to move `bytes` over the host link of GPU `dev` (to_gpu: host -> GPU) while
// `n_active` GPUs use their host links in that direction at the same time and, if
// `both_directions`, the opposite direction is busy too (LinkMap.cpp:121-269 and
// CoModel.cpp:120-140 restated for this box).
double host_link_time_shared(int dev, bool to_gpu, double bytes, int n_active,
                             bool both_directions, const std::vector<int>* active_devs = nullptr);

// True when write-backs are held until a unit's input stream has drained: with this many
// GPUs on the host link the two directions together deliver less than one after the other.
bool defer_writebacks(int n_units);

// Whole-problem prediction for `units` GPUs with tile T
// (ModelLvl3.cpp:75-237 combined as in Autotuner.cpp:709-716,739,766).
double predict_gemm(const GemmModelInput& in, int64_t T, const std::vector<int>& units,
                    const double sl[6], std::vector<UnitPrediction>* per_unit);

// Tile edge with the smallest predicted time among the measured tile sizes (and the
// smallest dimension itself); the reference's score (sl) of the winner is returned too.
int64_t optimize_tile_model(const GemmModelInput& in, const std::vector<int>& units,
                            const TuneConstants& c, double sl[6], double* pred);

// Band hints of one unit (plan.hpp) from the model: `a_sharers` / `b_sharers` = how many
// units share the host fetches of the unit's A tile rows / B tile columns, `n_units` = how
// many pull from the host at once.
BandHints band_hints(const GemmModelInput& in, int64_t T, int dev, int n_units, int a_sharers,
                     int b_sharers, int row_len);

// Full autotune: device set (prefix sets of 1,2,...,G GPUs unless ctl fixes it), T,
// distribution; fills the report's model fields.
int autotune_gemm(const GemmModelInput& in, int ngpu, const paralia_ctl* ctl,
                  paralia_report* rep);

// Level-1 (ModelLvl1.cpp:19-144, Autotuner.cpp:279-560 for one-dimensional problems):
// unit set and tile length of y <- alpha*x + y ("Daxpy") or x.y ("Ddot") on vectors of N
// doubles at locx / locy. Fills T, the unit list and pred_t.
struct VecModelInput {
  const char* func;   // "Daxpy" / "Ddot"
  int64_t N;
  int locx, locy;
};
double predict_vec(const VecModelInput& in, int64_t T, const std::vector<int>& units);
int autotune_vec(const VecModelInput& in, int ngpu, const paralia_ctl* ctl, paralia_report* rep);

}  // namespace paralia
