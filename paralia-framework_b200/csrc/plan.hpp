// The static launch plan of a tiled GEMM: pure host arithmetic, no CUDA.
//
// The reference decides at run time which subkernel fires next (SubkernelSelect,
// Library_scheduler/src/Subkernel.cpp:384-449, with a random tie-break) from the fire loop
// at Library_scheduler/src/Functions/dgemm.cpp:516-544. Here the order is a function of
// (tile counts, unit count, cache mode) alone, so that a rerun enqueues the same launches
// in the same order and the result bits are reproducible.
#pragma once
#include <vector>

namespace paralia {

// One launch of a unit: C tile `order_idx` (index into the unit's C tile list) advanced
// over the k tiles [ki0, ki1).
struct LaunchItem {
  int order_idx, ki0, ki1;
};

// How many consecutive k tiles the launch starting at k tile ki0 covers. A function of
// ki0 and the cache mode only (never of the tile, the unit or the GPU count): the first
// launch of a C tile takes one k tile, so that a streamed problem starts as soon as one
// A/B pair has landed; later launches take four. A bounded cache keeps one A and one B
// tile per launch alive. PARALIA_KCHAIN overrides the length (experiments: it changes
// the rounding).
int plan_kchain_len(bool bounded_cache, int ki0, int max_parts);

// Order of a unit's launches over its n_ctiles C tiles and Kt k tiles. C tiles are taken in
// bands (consecutive tiles of the unit's distribution order; about four bands per unit,
// 4 to 16 tiles each, PARALIA_BAND overrides); inside a band all tiles advance through k
// together. With a bounded cache the order is tile-major (bands of one).
void plan_launch_order(int n_ctiles, int Kt, bool bounded_cache, int max_parts,
                       std::vector<LaunchItem>* items);

// C tiles (mi*Nt+ni) of every unit in processing order = order of first appearance in the
// unit's subkernel list (ids mi*Nt*Kt + ni*Kt + ki). owner[ct] receives the unit index.
// Returns false if one C tile appears in the lists of two units.
bool plan_unit_ctiles(const std::vector<std::vector<int>>& sk_lists, int kt_for_ids, int n_ctiles,
                      std::vector<std::vector<int>>* ctiles, std::vector<int>* owner);

}  // namespace paralia
