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
  int band;   // number of C tiles in the band the launch belongs to
};

// Value of PARALIA_KCHAIN (0 = not set).
int plan_kchain_forced();

// How many consecutive k tiles the launch starting at k tile ki0 covers. A function of
// ki0 and the cache mode only (never of the tile, the unit or the GPU count): the first
// launch of a C tile takes one k tile, so that a streamed problem starts as soon as one
// A/B pair has landed; later launches take four. A bounded cache keeps one A and one B
// tile per launch alive. PARALIA_KCHAIN overrides the length (experiments: it changes
// the rounding).
int plan_kchain_len(bool bounded_cache, int ki0, int max_parts);
// What the band sizes of a unit are derived from. The rho values are times relative to one
// tile product (one launch of one k tile) on the unit: what it costs the unit's own host
// link to bring in one more tile row of A (rho_a), one more tile column of B (rho_b) per k
// step, and the original of one C tile (rho_c). A value of 0 means that operand does not
// cross the unit's host link.
struct BandHints {
  int row_len = 0;      // C tiles per tile row of the unit's block (0: treat the list as one row)
  double rho_a = 0.0, rho_b = 0.0, rho_c = 0.0;
  int last_band = 2;    // tiles in the very last band (what is left to write back after the
                        // last launch); 1 when one tile alone fills the GPU
};

// Sizes of the bands a unit's n_ctiles C tiles (in the unit's distribution order) are cut
// into. Inside a band all tiles advance through k together.
//  * The first band is the smallest whole number of tile rows whose launches per k step take
//    longer than fetching what they need (rows*rho_a + cols*rho_b + tiles*rho_c/Kt), so that
//    the unit is not input-bound while every later tile still has to arrive.
//  * The last bands shrink (..., 4, 2[, 1]): all tiles of a band finish together, and what
//    the last band writes back after the last launch is pure drain time.
//  * What lies between is cut into equal bands of at most eight tiles.
// With a bounded cache every band is one tile (tile-major order). PARALIA_BAND=<n> forces
// uniform bands of n tiles, PARALIA_BAND_PLAN=<a,b,c,...> forces the list (the last entry
// repeats); both are for experiments and do not change any result bit.
void plan_band_sizes(int n_ctiles, int Kt, bool bounded_cache, const BandHints& hints,
                     std::vector<int>* bands);

// Order of a unit's launches over its C tiles and Kt k tiles, band after band (the sizes
// must add up to the number of C tiles): inside a band the first k tile of every C tile,
// then the next chain of k tiles of every C tile, and so on.
void plan_launch_order(const std::vector<int>& bands, int Kt, bool bounded_cache, int max_parts,
                       std::vector<LaunchItem>* items);

// C tiles (mi*Nt+ni) of every unit in processing order = order of first appearance in the
// unit's subkernel list (ids mi*Nt*Kt + ni*Kt + ki). owner[ct] receives the unit index.
// Returns false if one C tile appears in the lists of two units.
bool plan_unit_ctiles(const std::vector<std::vector<int>>& sk_lists, int kt_for_ids, int n_ctiles,
                      std::vector<std::vector<int>>* ctiles, std::vector<int>* owner);

}  // namespace paralia
