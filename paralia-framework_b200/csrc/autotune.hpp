// Model-driven choice of tile size, device set and subkernel distribution.
//
// Keeps the form of the reference's autotuner (Autotuner/src/Autotuner.cpp:279-818,
// Subkernel_distributions.cpp:315-485, ModelLvl3.cpp:75-237, CoModel.cpp:108-140,
// GPUexec_lookup.cpp:103-129) with its constants as run-time values and the link map
// reduced to what one NVSwitch box has: a host link per GPU and uniform GPU-GPU links.
#pragma once
#include <stdint.h>
#include <map>
#include <string>
#include <vector>

#include "../../include/paralia_c.h"

namespace paralia {

// Compile-time -D switches of the reference (CMakeLists.txt:157-165,
// Autotuner/CMakeLists.txt:10-24) as one run-time record.
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
};

// t = ti + tb*bytes (CoModel.cpp:108-117).
struct LinkModel {
  double ti = 0.0;   // seconds
  double tb = 0.0;   // seconds per byte
};

// One routine's measured tile time on a GPU: (T -> seconds) per transpose pair
// (GPUexec_lookup.cpp:41-101).
struct ExecTable {
  std::map<std::string, std::map<int64_t, double>> by_trans;  // key "NN","NT","TN","TT"
  bool empty() const { return by_trans.empty(); }
};

struct ModelDB {
  // index 0 = host (-1), 1.. = GPU 0..; [dst][src]
  std::vector<std::vector<LinkModel>> link;
  std::map<std::string, ExecTable> exec;  // "Dgemm", "Sgemm", "Daxpy", "Ddot"
  bool from_disk = false;
  std::string dir;
};

// The library's current database (defaults describing a B200 box until
// load_database() replaces them).
ModelDB& model_db();
TuneConstants& tune_constants();
int load_database(const char* dir);
void reset_database_defaults(int ngpu);

// Tile-size score, lower is better (Autotuner.cpp:571-603). sl[0] aggregate,
// sl[1] imbalance, sl[2] remainder, sl[3] small tile, sl[4] subkernel count, sl[5] big tile.
void tile_slowdowns(int64_t D1, int64_t D2, int64_t D3, int64_t T, int units,
                    const TuneConstants& c, double sl[6]);

// T = argmin of sl[0], scanning from min(D1,D2,D3) downwards, first strict minimum wins
// (Autotuner.cpp:605-655). step = 1 reproduces the reference's exhaustive scan.
int64_t optimize_tile(int64_t D1, int64_t D2, int64_t D3, int units, const TuneConstants& c,
                      int64_t step, double sl[6]);

// Most-square factorisation units = d1*d2 by the reference's rule
// (Subkernel_distributions.cpp:325-336).
void device_grid(int units, int* d1, int* d2);

// Subkernel lists per unit for a Mt x Nt x Kt grid, equal scores
// (Subkernel_distributions.cpp:315-485 with its round-robin fallbacks :10-76, :143-220).
// Returns the number of units that received work (the reference lowers active_unit_num
// when there are fewer C tiles than units).
int distribute_subkernels_2d(int units, int Mt, int Nt, int Kt,
                             std::vector<std::vector<int>>* lists, int* d1, int* d2);

struct GemmModelInput {
  int esz;
  char ta, tb;
  int64_t M, N, K;
  int locA, locB, locC;   // -1 host, >=0 GPU
  bool beta_nonzero = true;
  const char* func;       // "Dgemm" / "Sgemm"
};

struct UnitPrediction {
  double t_exec, t_recv, t_send, t_extra, t_total;
};

// Seconds one tile GEMM of edge T takes on a GPU (lookup with cubic extrapolation,
// GPUexec_lookup.cpp:103-129).
double predict_tile_exec(const char* func, char ta, char tb, int64_t T);

// Whole-problem prediction for `units` GPUs with tile T
// (ModelLvl3.cpp:75-237 combined as in Autotuner.cpp:709-716,739,766).
double predict_gemm(const GemmModelInput& in, int64_t T, const std::vector<int>& units,
                    const double sl[6], std::vector<UnitPrediction>* per_unit);

// Full autotune: device set (prefix sets of 1,2,4,... GPUs unless ctl fixes it), T,
// distribution; fills the report's model fields.
int autotune_gemm(const GemmModelInput& in, int ngpu, const paralia_ctl* ctl,
                  paralia_report* rep);

}  // namespace paralia
