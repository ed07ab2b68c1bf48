#include "autotune.hpp"

#include <algorithm>
#include <cfloat>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "runtime.hpp"

namespace paralia {

static ModelDB g_db;
static TuneConstants g_consts;

ModelDB& model_db() { return g_db; }
TuneConstants& tune_constants() { return g_consts; }

// ---------------------------------------------------------------------------------------
// Database: defaults, readers
// ---------------------------------------------------------------------------------------

// Defaults for one 8 x B200 NVSwitch box, used until a measured database is loaded:
// host link ~55 GB/s per GPU and direction when alone, GPU-GPU ~700 GB/s through NVSwitch,
// ~10 us of launch/copy latency, DMMA tile kernel ~33 TFLOP/s, level-1 kernels at ~6.3 TB/s.
// The host aggregate figures were measured on a box of this kind (pinned 1 GiB copies).
void reset_database_defaults(int ngpu) {
  g_db = ModelDB();
  const int L = ngpu + 1;
  g_db.link.assign(L, std::vector<LinkModel>(L));
  for (int d = 0; d < L; ++d)
    for (int s = 0; s < L; ++s) {
      LinkModel& m = g_db.link[d][s];
      if (d == s) { m.ti = 0; m.tb = 0; }
      else if (d == 0 || s == 0) { m.ti = 12e-6; m.tb = 1.0 / 55e9; }
      else { m.ti = 10e-6; m.tb = 1.0 / 700e9; }
    }
  g_db.host.h2d = {{1, 55.0}, {2, 111.0}, {4, 115.0}, {8, 185.0}};
  g_db.host.d2h = {{1, 55.0}, {2, 111.0}, {4, 115.0}, {8, 185.0}};
  g_db.host.bidir = {{1, 47.0}, {2, 52.0}, {4, 51.0}, {8, 63.0}};
  const char* tr[4] = {"NN", "NT", "TN", "TT"};
  ExecTable dg, sg;
  for (int i = 0; i < 4; ++i)
    for (int64_t T = 256; T <= 8192; T *= 2) {
      const double flops = 2.0 * (double)T * T * T;
      // efficiency ramps with T: launch latency + wave quantisation on 148 SMs
      const double tiles = std::ceil(T / 128.0) * std::ceil(T / 128.0);
      const double waves = std::ceil(tiles / 148.0);
      const double eff = tiles / (waves * 148.0);
      dg.by_trans[tr[i]][T] = 8e-6 + flops / (33e12 * eff);
      sg.by_trans[tr[i]][T] = 8e-6 + flops / (250e12 * eff);
    }
  g_db.exec["Dgemm"] = dg;
  g_db.exec["Sgemm"] = sg;
  ExecTable ax, dt;
  for (int64_t n = 1 << 12; n <= (1 << 26); n *= 2) {
    ax.by_trans["--"][n] = 4e-6 + 24.0 * n / 6.3e12;
    dt.by_trans["--"][n] = 7e-6 + 16.0 * n / 6.2e12;
  }
  g_db.exec["Daxpy"] = ax;
  g_db.exec["Ddot"] = dt;
}

// "Intercept: <ti>\nCoefficient: <tb>\n" followed by "Slowdown([src]->[dst]): <ratio>" lines
// (written by the link post-processing step, read by Autotuner/src/CoModel.cpp:26-55).
// A ratio below 1 is noise and one above 2 means more than an even split, which the
// reference resets to 2; ratios within 5 % of 1 are dropped.
static bool read_link_file(const std::string& path, LinkModel* m) {
  FILE* fp = fopen(path.c_str(), "r");
  if (!fp) return false;
  double ti = 0, tb = 0;
  const int items = fscanf(fp, "Intercept: %le\nCoefficient: %le\n", &ti, &tb);
  if (items != 2) {
    fclose(fp);
    return false;
  }
  m->ti = ti;
  m->tb = tb;
  m->slow.clear();
  int src = 0, dst = 0;
  double ratio = 0;
  while (fscanf(fp, " Slowdown([%d]->[%d]): %le", &src, &dst, &ratio) == 3) {
    if (ratio > 2.0) ratio = 2.0;
    if (ratio < 1.05) continue;
    m->slow.push_back({dst, src, ratio});
  }
  fclose(fp);
  return true;
}

// Rows: TransA,TransB,T,T,T,mean_t,W,J,err,samples,bench_t (GPUexec_lookup.cpp:79-81).
static bool read_exec_file(const std::string& path, ExecTable* t) {
  FILE* fp = fopen(path.c_str(), "r");
  if (!fp) return false;
  char line[512];
  while (fgets(line, sizeof(line), fp)) {
    char ta, tb;
    long t1, t2, t3;
    double mean_t;
    if (sscanf(line, " %c,%c,%ld,%ld,%ld,%le", &ta, &tb, &t1, &t2, &t3, &mean_t) == 6) {
      std::string key;
      key += ta;
      key += tb;
      t->by_trans[key][t1] = mean_t;
    }
  }
  fclose(fp);
  return !t->empty();
}

// Rows: N,mean_t,W,J,err,samples,bench_t (GPUexec_lookup.cpp:318-323).
static bool read_vec_file(const std::string& path, ExecTable* t) {
  FILE* fp = fopen(path.c_str(), "r");
  if (!fp) return false;
  char line[512];
  while (fgets(line, sizeof(line), fp)) {
    long n;
    double mean_t;
    if (sscanf(line, " %ld,%le", &n, &mean_t) == 2 && n > 0 && mean_t > 0) t->by_trans["--"][n] = mean_t;
  }
  fclose(fp);
  return !t->empty();
}

// Lines "<H2D|D2H|BIDIR> <gpus> <aggregate GB/s>".
static bool read_host_aggregate(const std::string& path, HostAggregate* h) {
  FILE* fp = fopen(path.c_str(), "r");
  if (!fp) return false;
  char kind[32];
  int n;
  double gbs;
  HostAggregate out;
  while (fscanf(fp, " %31s %d %le", kind, &n, &gbs) == 3) {
    if (n <= 0 || !(gbs > 0)) continue;
    if (!strcmp(kind, "H2D")) out.h2d[n] = gbs;
    else if (!strcmp(kind, "D2H")) out.d2h[n] = gbs;
    else if (!strcmp(kind, "BIDIR")) out.bidir[n] = gbs;
  }
  fclose(fp);
  if (out.empty()) return false;
  *h = out;
  return true;
}

int load_database(const char* dir) {
  if (!dir) return fail(PARALIA_ERR_INVALID_ARG, "database directory is NULL");
  const int L = (int)g_db.link.size();
  if (L == 0) return fail(PARALIA_ERR_DB_MISSING, "model database not initialised");
  int found = 0;
  // a database is self-contained: what its files do not define is the default, never a
  // left-over of the database loaded before
  ModelDB db;
  {
    const ModelDB saved = g_db;
    reset_database_defaults(L - 1);
    db = g_db;
    g_db = saved;
  }
  std::vector<std::vector<char>> have(L, std::vector<char>(L, 0));
  for (int d = 0; d < L; ++d)
    for (int s = 0; s < L; ++s) {
      if (d == s) continue;
      char name[512];
      snprintf(name, sizeof(name), "%s/Processed/Link-Stats_loc_dest-%d_loc_src-%d.log", dir, d - 1,
               s - 1);
      if (read_link_file(name, &db.link[d][s])) {
        ++found;
        have[d][s] = 1;
      }
    }
  // The GPUs of the box are identical and sit behind one switch: a link that was not
  // measured takes the model of the measured link of the same kind (host<->GPU 0 for
  // every host link, GPU 1<-GPU 0 for every GPU pair), without its slowdown entries.
  for (int d = 0; d < L; ++d)
    for (int s = 0; s < L; ++s) {
      if (d == s || have[d][s]) continue;
      const LinkModel* from = nullptr;
      if (s == 0 && d >= 1 && have[1][0]) from = &db.link[1][0];
      else if (d == 0 && s >= 1 && have[0][1]) from = &db.link[0][1];
      else if (d >= 1 && s >= 1 && L > 2 && have[2][1]) from = &db.link[2][1];
      if (from) {
        db.link[d][s].ti = from->ti;
        db.link[d][s].tb = from->tb;
        db.link[d][s].slow.clear();
      }
    }
  char name[512];
  for (const char* f : {"Dgemm", "Sgemm"}) {
    // one table per device in the reference; identical GPUs share device 0's table here
    snprintf(name, sizeof(name), "%s/Processed/%s_lookup-table_dev-0.log", dir, f);
    ExecTable t;
    if (read_exec_file(name, &t)) {
      db.exec[f] = t;
      ++found;
    }
  }
  for (const char* f : {"Daxpy", "Ddot"}) {
    snprintf(name, sizeof(name), "%s/Processed/%s_lookup-table_dev-0.log", dir, f);
    ExecTable t;
    if (read_vec_file(name, &t)) {
      db.exec[f] = t;
      ++found;
    }
  }
  snprintf(name, sizeof(name), "%s/Processed/Host-Link-Aggregate.log", dir);
  if (read_host_aggregate(name, &db.host)) ++found;
  if (!found)
    return fail(PARALIA_ERR_DB_MISSING, "no model files found under %s/Processed", dir);
  db.from_disk = true;
  db.dir = dir;
  g_db = db;
  return PARALIA_OK;
}

// ---------------------------------------------------------------------------------------
// The reference's tile score (reported; the fallback tile choice without a tile table)
// ---------------------------------------------------------------------------------------

void tile_slowdowns(int64_t D1, int64_t D2, int64_t D3, int64_t T, int units,
                    const TuneConstants& c, double sl[6]) {
  for (int i = 0; i < 6; ++i) sl[i] = 0.0;
  const int64_t Mt = D1 / T + ((D1 % T) ? 1 : 0);
  const int64_t Nt = D2 / T + ((D2 % T) ? 1 : 0);
  const int64_t Kt = D3 / T + ((D3 % T) ? 1 : 0);
  const int64_t sk = Mt * Nt * Kt;
  // Condition 1: C tiles ("buckets") that do not divide evenly among the units.
  const int64_t buckets = sk / Kt;
  sl[1] = (buckets / units) ? 1.0 * (buckets % units) / (buckets / units) * units
                            : 1.0 * buckets / units;
  // Condition 2: remainder tiles.
  if (D1 % T) sl[2] += 1.0 / (D1 / T);
  if (D2 % T) sl[2] += 1.0 / (D2 / T);
  if (D3 % T) sl[2] += 1.0 / (D3 / T);
  // Condition 3: tile smaller than the kernel likes.
  if (T < c.tile_min) sl[3] += 1.0 * c.tile_min / T * c.tile_min_slowdown;
  // Condition 4: too few / too many subkernels per unit.
  const int64_t dev_sks = (int64_t)((1.0 * sk) / units);
  sl[4] += 2.0 / dev_sks;
  if (dev_sks > c.max_desired_sk_dev)
    sl[4] += (1.0 * dev_sks / c.max_desired_sk_dev) * c.max_desired_sk_dev_slowdown;
  // Condition 5: tile larger than useful (integer division as in the reference).
  if (T > c.tile_max) sl[5] += (double)(T / c.tile_max) * c.tile_max_slowdown;
  sl[0] = sl[1] + sl[2] + sl[3] + sl[4] + sl[5];
}

int64_t optimize_tile(int64_t D1, int64_t D2, int64_t D3, int units, const TuneConstants& c,
                      int64_t step, double sl_out[6]) {
  const int64_t max_T = std::min(D1, std::min(D2, D3));
  int64_t best_T = -1;
  double best[6], cur[6];
  for (int i = 0; i < 6; ++i) best[i] = DBL_MAX;
  if (step < 1) step = 1;
  for (int64_t T = max_T; T > 0; --T) {
    if (T != max_T && (T % step) != 0) continue;
    tile_slowdowns(D1, D2, D3, T, units, c, cur);
    if (cur[0] < best[0]) {
      for (int i = 0; i < 6; ++i) best[i] = cur[i];
      best_T = T;
    }
  }
  for (int i = 0; i < 6; ++i) sl_out[i] = best[i];
  return best_T;
}

// ---------------------------------------------------------------------------------------
// Device grid and C tile ownership
// ---------------------------------------------------------------------------------------

void device_grid(int units, int* d1_out, int* d2_out) {
  // the first divisor found scanning down from floor(sqrt(units)) + 1 becomes D1
  int d1 = units, d2 = 1;
  for (int g = (int)std::sqrt((double)units) + 1; g > 0; --g)
    if (units % g == 0) {
      d1 = g;
      d2 = units / g;
      break;
    }
  *d1_out = d1;
  *d2_out = d2;
}

// Owner of every C tile, as a map. Three regimes:
//  * a single column of C tiles with one k tile, or fewer tile rows / columns than the device
//    grid has: the tiles are dealt out cyclically, tile t to unit t mod units;
//  * otherwise the part of the tile grid that divides evenly by D1 x D2 is cut into D1 x D2
//    equal blocks, block (r, c) to unit r*D2 + c. Each unit has a quota of
//    int((1/units) * tiles) tiles, evaluated in double precision exactly like that; where
//    the product lands one below the true quotient the block's last tiles spill to the
//    next unit with room, and where nobody has room the rule fails;
//  * the leftover strips (right, bottom, corner, in that order) are dealt out cyclically,
//    one C tile at a time, starting again from unit 0.
// A unit's list holds the subkernel ids mi*Nt*Kt + ni*Kt + ki of its tiles in the order the
// tiles were assigned.
int distribute_subkernels_2d(int units, int Mt, int Nt, int Kt,
                             std::vector<std::vector<int>>* lists, int* d1_out, int* d2_out) {
  int d1, d2;
  device_grid(units, &d1, &d2);
  if (d1_out) *d1_out = d1;
  if (d2_out) *d2_out = d2;
  const int n_ct = Mt * Nt;
  auto give = [&](int unit, int mi, int ni) {
    std::vector<int>& l = (*lists)[unit];
    const int base = (mi * Nt + ni) * Kt;
    for (int k = 0; k < Kt; ++k) l.push_back(base + k);
  };
  if ((Nt == 1 && Kt == 1) || Mt < d1 || Nt < d2) {
    const int active = std::min(units, n_ct);
    lists->assign(active, std::vector<int>());
    for (int t = 0; t < n_ct; ++t) give(t % units, t / Nt, t % Nt);
    return active;
  }
  const int rows_per = Mt / d1, cols_per = Nt / d2;
  const int Mdiv = rows_per * d1, Ndiv = cols_per * d2;
  const double score = 1.0 / units;
  std::vector<int> quota(units, (int)(score * Mdiv * Ndiv)), filled(units, 0);
  if (Mdiv == Mt && Ndiv == Nt) {
    // no strips to absorb a shortfall: top the quotas up to the exact block size
    int missing = n_ct - units * quota[0];
    for (int d = 0; d < units && missing > 0; ++d)
      if (quota[d] < n_ct / units) {
        ++quota[d];
        --missing;
      }
  }
  lists->assign(units, std::vector<int>());
  for (int mi = 0; mi < Mdiv; ++mi)
    for (int ni = 0; ni < Ndiv; ++ni) {
      int unit = (mi / rows_per) * d2 + ni / cols_per;
      int tries = units;
      while (filled[unit] == quota[unit]) {
        if (tries-- == 0) return -1;
        unit = (unit + 1) % units;
      }
      ++filled[unit];
      give(unit, mi, ni);
    }
  int next = 0;
  auto deal = [&](int m0, int m1, int n0, int n1) {
    for (int mi = m0; mi < m1; ++mi)
      for (int ni = n0; ni < n1; ++ni) {
        give(next, mi, ni);
        next = (next + 1) % units;
      }
  };
  deal(0, Mdiv, Ndiv, Nt);
  deal(Mdiv, Mt, 0, Ndiv);
  deal(Mdiv, Mt, Ndiv, Nt);
  return units;
}

// ---------------------------------------------------------------------------------------
// Lookups: tile times, links
// ---------------------------------------------------------------------------------------

static const std::map<int64_t, double>* exec_curve(const char* func, char ta, char tb) {
  auto it = g_db.exec.find(func);
  if (it == g_db.exec.end()) return nullptr;
  std::string key;
  key += (ta == 'T' ? 'T' : 'N');
  key += (tb == 'T' ? 'T' : 'N');
  auto jt = it->second.by_trans.find(key);
  if (jt == it->second.by_trans.end() || jt->second.empty()) return nullptr;
  return &jt->second;
}

double predict_tile_exec(const char* func, char ta, char tb, int64_t T) {
  const std::map<int64_t, double>* curve = exec_curve(func, ta, tb);
  if (!curve) return -1.0;
  auto hit = curve->find(T);
  if (hit != curve->end()) return hit->second;
  // nearest measured T, scaled with T^3 (GPUexec_lookup.cpp:118-128)
  int64_t nearest = curve->begin()->first;
  for (const auto& kv : *curve)
    if (std::llabs(kv.first - T) < std::llabs(nearest - T)) nearest = kv.first;
  const double t = curve->at(nearest);
  return t * std::pow((double)T, 3) / std::pow((double)nearest, 3);
}

double predict_vec_exec(const char* func, int64_t n) {
  auto it = g_db.exec.find(func);
  if (it == g_db.exec.end()) return -1.0;
  auto jt = it->second.by_trans.find("--");
  if (jt == it->second.by_trans.end() || jt->second.empty()) return -1.0;
  const std::map<int64_t, double>& curve = jt->second;
  auto hi = curve.lower_bound(n);
  if (hi != curve.end() && hi->first == n) return hi->second;
  if (hi == curve.begin()) return hi->second;   // shorter than anything measured: latency floor
  if (hi == curve.end()) {
    // longer than anything measured: bandwidth-bound, time grows linearly
    auto last = std::prev(hi);
    return last->second * (double)n / (double)last->first;
  }
  auto lo = std::prev(hi);
  const double f = (double)(n - lo->first) / (double)(hi->first - lo->first);
  return lo->second + f * (hi->second - lo->second);
}

static const LinkModel* link_model(int dst_loc, int src_loc) {
  const int L = (int)g_db.link.size();
  int d = dst_loc + 1, s = src_loc + 1;
  if (d >= L) d = L - 1;
  if (s >= L) s = L - 1;
  if (d < 0 || s < 0 || L == 0) return nullptr;
  return &g_db.link[d][s];
}

static double link_time(int dst_loc, int src_loc, double bytes) {
  if (bytes <= 0 || dst_loc == src_loc) return 0.0;
  const LinkModel* m = link_model(dst_loc, src_loc);
  return m ? m->ti + m->tb * bytes : 0.0;
}

// Aggregate GB/s for n GPUs: the measured point, else a straight line between its measured
// neighbours; beyond the largest measured count the aggregate is taken as saturated.
static double aggregate_at(const std::map<int, double>& table, int n) {
  if (table.empty() || n <= 0) return 0.0;
  auto hi = table.lower_bound(n);
  if (hi != table.end() && hi->first == n) return hi->second;
  if (hi == table.begin()) return hi->second * n / hi->first;
  if (hi == table.end()) return std::prev(hi)->second;
  auto lo = std::prev(hi);
  const double f = (double)(n - lo->first) / (double)(hi->first - lo->first);
  return lo->second + f * (hi->second - lo->second);
}

double host_link_time_shared(int dev, bool to_gpu, double bytes, int n_active,
                             bool both_directions, const std::vector<int>* active_devs) {
  if (bytes <= 0) return 0.0;
  const LinkModel* m = to_gpu ? link_model(dev, -1) : link_model(-1, dev);
  if (!m || m->tb <= 0) return 0.0;
  // pairwise: the worst slowdown any concurrently busy host link imposes on this one
  // (GPU <-> GPU entries are ignored: every pair has its own path through the switch)
  double factor = 1.0;
  for (const LinkSlowdown& s : m->slow) {
    bool x_to_gpu;
    int other;
    if (s.src == -1 && s.dst >= 0) { x_to_gpu = true; other = s.dst; }
    else if (s.dst == -1 && s.src >= 0) { x_to_gpu = false; other = s.src; }
    else continue;
    const bool same_dir = x_to_gpu == to_gpu;
    if (!same_dir && !both_directions) continue;
    if (other == dev) {
      if (same_dir) continue;   // the link itself
    } else if (!active_devs ||
               std::find(active_devs->begin(), active_devs->end(), other) == active_devs->end()) {
      continue;
    }
    factor = std::max(factor, s.ratio);
  }
  double bw = 1.0 / (m->tb * factor);
  // aggregate: all active GPUs together cannot exceed what the host delivers
  const std::map<int, double>& table = both_directions ? g_db.host.bidir
                                                       : (to_gpu ? g_db.host.h2d : g_db.host.d2h);
  const int n = std::max(n_active, 1);
  const double agg = aggregate_at(table, n);
  if (agg > 0) bw = std::min(bw, agg * 1e9 / n);
  return m->ti + bytes / bw;
}

bool defer_writebacks(int n_units) {
  const double one = aggregate_at(g_db.host.h2d, n_units);
  const double both = aggregate_at(g_db.host.bidir, n_units);
  if (one <= 0 || both <= 0) return n_units >= 4;
  // both directions together (2 x per-direction) against one direction after the other
  return 2.0 * both < 0.92 * one;
}

// ---------------------------------------------------------------------------------------
// GEMM model
// ---------------------------------------------------------------------------------------

static inline int64_t cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Seconds to bring `bytes` into GPU `dev` from another GPU (every pair is alike).
static double peer_time(int dev, double bytes) { return link_time(dev, dev == 0 ? 1 : 0, bytes); }

// Tiles in the last band of a unit: one when a single tile's CTAs keep the GPU full for
// several waves (148 SMs, 128 x 128 CTA tiles), else two.
static int last_band_tiles(int64_t T) {
  const int64_t ctas = cdiv(T, 128) * cdiv(T, 128);
  return ctas >= 4 * 148 ? 1 : 2;
}

// Seconds of tile products for a block of mloc x nloc elements of C over all of K with
// tile edge T. Full tiles run at the measured rate of T; the remainder strips (where T does
// not divide the block) are narrower launches and run at the rate measured for their own
// narrow edge, rounded up to whole 128-wide CTA tiles.
static double block_exec_time(const GemmModelInput& in, int64_t T, double mloc, double nloc) {
  auto per_volume = [&](double edge) {
    const int64_t e = std::max<int64_t>(16, (int64_t)edge);
    const double t = predict_tile_exec(in.func, in.ta, in.tb, e);
    return t > 0 ? t / ((double)e * e * e) : 0.0;
  };
  auto cta = [](double x) { return std::ceil(x / 128.0) * 128.0; };
  const double fm = std::floor(mloc / T), rm = mloc - fm * T;
  const double fn = std::floor(nloc / T), rn = nloc - fn * T;
  const double K = (double)in.K;
  double t = fm * fn * (double)T * T * K * per_volume((double)std::min<int64_t>(T, in.K));
  if (rm > 0) t += fn * cta(rm) * T * K * per_volume(std::min(rm, (double)T));
  if (rn > 0) t += fm * cta(rn) * T * K * per_volume(std::min(rn, (double)T));
  if (rm > 0 && rn > 0) t += cta(rm) * cta(rn) * K * per_volume(std::min(rm, rn));
  return t;
}

int64_t count_enqueue_ops(const GemmModelInput& in, int64_t Mt, int64_t Nt, int64_t Kt, int d1,
                          int d2, int n_active) {
  // launches per C tile: the first covers one k tile, the rest chains of four
  const int64_t per_ctile = Kt <= 0 ? 1 : 1 + (Kt - 1 + 3) / 4;
  int64_t ops = Mt * Nt * per_ctile;
  const int64_t kt = std::max<int64_t>(Kt, 0);
  const int a_cons = n_active > 1 ? d2 : 1, b_cons = n_active > 1 ? d1 : 1;
  // a tile on a GPU is read in place by that GPU (FP64) or packed from where it lies (FP32)
  ops += Mt * kt * a_cons - (in.locA >= 0 ? Mt * kt / std::max(d1, 1) : 0);
  ops += kt * Nt * b_cons - (in.locB >= 0 ? kt * Nt / std::max(d2, 1) : 0);
  const int64_t c_moves = (in.beta_nonzero ? 2 : 1) * Mt * Nt;
  ops += in.locC >= 0 ? c_moves - c_moves / std::max(n_active, 1) : c_moves;
  return ops;
}

double predict_gemm(const GemmModelInput& in, int64_t T, const std::vector<int>& units,
                    const double sl[6], std::vector<UnitPrediction>* per_unit) {
  (void)sl;   // the reference's score is reported, not applied: its terms are modelled here
  const int U = (int)units.size();
  int d1, d2;
  device_grid(U, &d1, &d2);
  const int64_t Tb = std::min<int64_t>(T, std::min(in.M, std::min(in.N, in.K)));
  const int64_t Mt = cdiv(in.M, T), Nt = cdiv(in.N, T);
  const bool regular = Mt >= d1 && Nt >= d2;
  // the largest block a unit owns, in elements
  double Mloc, Nloc;
  if (regular) {
    Mloc = (double)std::min<int64_t>(in.M, cdiv(Mt, d1) * T);
    Nloc = (double)std::min<int64_t>(in.N, cdiv(Nt, d2) * T);
  } else {
    const int64_t tiles_u = cdiv(Mt * Nt, std::min<int64_t>(U, Mt * Nt));
    Mloc = (double)std::min<int64_t>(in.M, T);
    Nloc = (double)std::min<int64_t>(in.N, tiles_u * T);
  }
  const int n_active = (int)std::min<int64_t>(U, Mt * Nt);
  const double t_tile = predict_tile_exec(in.func, in.ta, in.tb, Tb);
  const double exec_block = block_exec_time(in, T, Mloc, Nloc);
  const double esz = in.esz;
  const double tile_bytes = (double)Tb * Tb * esz;
  const double inC = in.beta_nonzero ? 1.0 : 0.0;
  const bool defer = defer_writebacks(n_active);
  const int a_sharers = regular && n_active > 1 ? d2 : 1;
  const int b_sharers = regular && n_active > 1 ? d1 : 1;
  double worst = 0.0;
  if (per_unit) per_unit->clear();
  for (int u = 0; u < n_active; ++u) {
    const int dev = units[u];
    UnitPrediction p{};
    p.t_exec = exec_block;
    const double panelA = Mloc * in.K * esz, panelB = in.K * Nloc * esz, blockC = Mloc * Nloc * esz;
    // what crosses this unit's host link: its share of the host-resident panels (each tile
    // is fetched by one unit of the grid row / column and forwarded), its C block both ways
    double host_in = 0.0, host_out = 0.0, peer_in = 0.0, src_out = 0.0;
    if (in.locA == -1) { host_in += panelA / a_sharers; peer_in += panelA * (1.0 - 1.0 / a_sharers); }
    else if (in.locA != dev) { peer_in += panelA; }
    if (in.locB == -1) { host_in += panelB / b_sharers; peer_in += panelB * (1.0 - 1.0 / b_sharers); }
    else if (in.locB != dev) { peer_in += panelB; }
    if (in.locC == -1) { host_in += blockC * inC; host_out += blockC; }
    else if (in.locC != dev) { peer_in += blockC * inC; }
    // an operand that lives on one GPU leaves it once per unit that reads it; two operands
    // on the same GPU leave through the same links
    const double outA = in.locA >= 0 ? panelA * (n_active - (in.locA == dev ? 1 : 0)) : 0.0;
    const double outB = in.locB >= 0 ? panelB * (n_active - (in.locB == dev ? 1 : 0)) : 0.0;
    src_out = (in.locA >= 0 && in.locA == in.locB) ? outA + outB : std::max(outA, outB);
    const bool both = !defer && host_in > 0 && host_out > 0;
    p.t_recv = host_link_time_shared(dev, true, host_in, n_active, both, &units);
    p.t_send = host_link_time_shared(dev, false, host_out, n_active, both, &units);
    if (in.locC >= 0 && in.locC != dev) p.t_send += link_time(in.locC, dev, blockC);
    p.t_extra = std::max(peer_time(dev, peer_in), peer_time(dev, src_out));
    // fill: what must land before the first tile product. With a device grid of at least
    // 2 x 2 the first A and B tiles of every unit come over different host links at the
    // same time; with fewer units one link brings both.
    const int host_first = (in.locA == -1 ? 1 : 0) + (in.locB == -1 ? 1 : 0);
    const int serial_first = (d1 >= 2 && d2 >= 2) ? std::min(host_first, 1) : host_first;
    p.t_fill = host_link_time_shared(dev, true, tile_bytes * serial_first, n_active, false, &units);
    if (peer_in > 0) p.t_fill += peer_time(dev, tile_bytes);
    // drain: the last band's C tiles leave after the last launch
    const int lb = last_band_tiles(Tb);
    if (in.locC == -1) p.t_drain = host_link_time_shared(dev, false, tile_bytes * lb, n_active, false, &units);
    else if (in.locC != dev) p.t_drain = link_time(in.locC, dev, tile_bytes * lb);
    const double t_host = defer ? p.t_recv + p.t_send : std::max(p.t_recv, p.t_send);
    const double tail_compute = std::min(p.t_exec, 4.0 * std::max(t_tile, 0.0));
    double t = p.t_fill + p.t_exec + p.t_drain;                      // compute-bound pipeline
    t = std::max(t, p.t_recv + tail_compute + p.t_drain);           // input-bound
    t = std::max(t, t_host + (defer ? 0.0 : p.t_fill));             // host-link-bound
    t = std::max(t, p.t_extra + tail_compute + p.t_drain);          // NVLink-bound
    p.t_total = t;
    worst = std::max(worst, p.t_total);
    if (per_unit) per_unit->push_back(p);
  }
  // the host side of the call
  const int64_t Kt = in.K > 0 ? cdiv(in.K, T) : 0;
  const double ops = (double)count_enqueue_ops(in, Mt, Nt, Kt, d1, d2, n_active);
  const TuneConstants& c = g_consts;
  return worst + c.call_fixed_s + c.enqueue_op_s * ops / std::max(in.enqueue_threads, 1);
}

int64_t optimize_tile_model(const GemmModelInput& in, const std::vector<int>& units,
                            const TuneConstants& c, double sl[6], double* pred) {
  const int U = (int)units.size();
  const int64_t min_dim = std::min(in.M, std::min(in.N, in.K));
  const std::map<int64_t, double>* curve = exec_curve(in.func, in.ta, in.tb);
  std::vector<int64_t> cands;
  if (curve)
    for (const auto& kv : *curve)
      if (kv.first <= min_dim && kv.first % 16 == 0) cands.push_back(kv.first);
  // plus a plain ladder of tile edges (the lookup interpolates between measured sizes), so
  // that a sparse or missing table does not restrict the choice
  for (int64_t T = 256; T <= std::min<int64_t>(min_dim, 8192); T += 256)
    if (std::find(cands.begin(), cands.end(), T) == cands.end()) cands.push_back(T);
  // the smallest dimension as one tile edge (a tile that is not the whole problem has to be
  // a multiple of the 16-deep pipeline stage)
  if (cands.empty() || (min_dim % 16 == 0 && min_dim <= 8192 &&
                        std::find(cands.begin(), cands.end(), min_dim) == cands.end()))
    cands.push_back(min_dim);
  int64_t best_T = -1;
  double best = DBL_MAX;
  // larger tiles first: on a tie the larger tile (fewer launches) wins
  std::sort(cands.begin(), cands.end());
  for (size_t i = cands.size(); i-- > 0;) {
    const int64_t T = cands[i];
    const double t = predict_gemm(in, T, units, nullptr, nullptr);
    if (t < best * (1.0 - 1e-9)) {
      best = t;
      best_T = T;
    }
  }
  tile_slowdowns(in.M, in.N, in.K, best_T, U, c, sl);
  if (pred) *pred = best;
  return best_T;
}

BandHints band_hints(const GemmModelInput& in, int64_t T, int dev, int n_units, int a_sharers,
                     int b_sharers, int row_len) {
  BandHints h;
  h.row_len = row_len;
  const int64_t Tb = std::min<int64_t>(T, std::min(in.M, std::min(in.N, std::max<int64_t>(in.K, 1))));
  h.last_band = last_band_tiles(Tb);
  const double t_tile = predict_tile_exec(in.func, in.ta, in.tb, Tb);
  if (!(t_tile > 0)) return h;
  const double tile_bytes = (double)Tb * Tb * in.esz;
  const double t_host = host_link_time_shared(dev, true, tile_bytes, n_units, false) / t_tile;
  auto rho = [&](int loc, int sharers) {
    if (loc == -1) return t_host / std::max(sharers, 1);
    if (loc != dev) return link_time(dev, loc, tile_bytes) / t_tile;
    return 0.0;
  };
  h.rho_a = rho(in.locA, a_sharers);
  h.rho_b = rho(in.locB, b_sharers);
  h.rho_c = in.beta_nonzero ? rho(in.locC, 1) : 0.0;
  return h;
}

int autotune_gemm(const GemmModelInput& in, int ngpu, const paralia_ctl* ctl,
                  paralia_report* rep) {
  if (in.M <= 0 || in.N <= 0 || in.K <= 0)
    return fail(PARALIA_ERR_INVALID_ARG, "autotune: non-positive dimension");
  if (g_db.link.empty()) reset_database_defaults(ngpu > 0 ? ngpu : 1);
  const TuneConstants& c = g_consts;
  std::vector<std::vector<int>> candidates;
  if (ctl && ctl->active_unit_num > 0) {
    if (ctl->active_unit_num > PARALIA_MAX_UNITS)
      return fail(PARALIA_ERR_INVALID_ARG, "active_unit_num %d too large", ctl->active_unit_num);
    std::vector<int> u(ctl->active_unit_id_list, ctl->active_unit_id_list + ctl->active_unit_num);
    for (size_t i = 0; i < u.size(); ++i) {
      if (ngpu > 0 && (u[i] < 0 || u[i] >= ngpu))
        return fail(PARALIA_ERR_INVALID_ARG, "unit id %d is not a GPU of this box", u[i]);
      for (size_t j = 0; j < i; ++j)
        if (u[j] == u[i]) return fail(PARALIA_ERR_INVALID_ARG, "unit id %d listed twice", u[i]);
    }
    candidates.push_back(u);
  } else {
    if (ngpu <= 0) return fail(PARALIA_ERR_NO_DEVICE, "autotune: no GPU and no fixed unit list");
    // Identical GPUs behind one switch: only the count matters, so the 2^LOC_NUM subset
    // scan of the reference (Autotuner.cpp:318-478) collapses to prefix sets.
    for (int n = 1; n <= ngpu; ++n) {
      std::vector<int> u(n);
      for (int i = 0; i < n; ++i) u[i] = i;
      candidates.push_back(u);
    }
  }
  double best_score = DBL_MAX;
  size_t best_card = 0;
  bool have = false;
  struct Choice { std::vector<int> units; int64_t T; double sl[6]; double pred; } best{};
  for (const auto& u : candidates) {
    Choice ch;
    ch.units = u;
    if (ctl && ctl->T > 0) {
      ch.T = ctl->T;
      tile_slowdowns(in.M, in.N, in.K, ch.T, (int)u.size(), c, ch.sl);
      ch.pred = predict_gemm(in, ch.T, u, ch.sl, nullptr);
    } else {
      ch.T = optimize_tile_model(in, u, c, ch.sl, &ch.pred);
    }
    // 5% per extra unit hysteresis (Autotuner.cpp:388-396)
    bool take = false;
    if (!have) take = true;
    else {
      const double adj = ch.pred * (1.0 + ((double)u.size() - (double)best_card) *
                                              c.minimum_unit_contribution);
      take = adj < best_score;
    }
    if (take) {
      best = ch;
      best_score = ch.pred;
      best_card = u.size();
      have = true;
    }
  }
  if (!have) return fail(PARALIA_ERR_INVALID_ARG, "autotune: no candidate configuration");
  if (rep) {
    memset(rep, 0, sizeof(*rep));
    rep->T = best.T;
    const int64_t Mt = cdiv(in.M, best.T), Nt = cdiv(in.N, best.T), Kt = cdiv(in.K, best.T);
    std::vector<std::vector<int>> lists;
    int d1 = 1, d2 = 1;
    int active = distribute_subkernels_2d((int)best.units.size(), (int)Mt, (int)Nt, (int)Kt,
                                          &lists, &d1, &d2);
    if (active < 0) return fail(PARALIA_ERR_INVALID_ARG, "autotune: distribution failed");
    rep->active_unit_num = active;
    for (int i = 0; i < active; ++i) {
      rep->active_unit_id_list[i] = best.units[i];
      rep->active_unit_score[i] = 1.0 / active;
      rep->subkernels_per_unit[i] = (int)lists[i].size();
    }
    rep->subkernel_num = Mt * Nt * Kt;
    rep->pred_t = best.pred;
    rep->pred_J = 0.0;
    for (int i = 0; i < 6; ++i) rep->T_slowdowns[i] = best.sl[i];
    rep->cache_limit = ctl ? ctl->cache_limit : 0;
    rep->grid_d1 = d1;
    rep->grid_d2 = d2;
  }
  return PARALIA_OK;
}

// ---------------------------------------------------------------------------------------
// Level-1 model
// ---------------------------------------------------------------------------------------

// One unit streams its contiguous run of tiles: fetch tile j+1 while tile j computes and
// tile j-1 goes back. Time = the slowest stage over the run plus what the overlap cannot
// hide: the first tile in, the last tile's kernel, the last tile out.
double predict_vec(const VecModelInput& in, int64_t T, const std::vector<int>& units) {
  const int U = (int)units.size();
  if (U <= 0 || T <= 0) return DBL_MAX;
  const bool axpy = !strcmp(in.func, "Daxpy");
  const int64_t Nt = cdiv(in.N, T);
  const int n_active = (int)std::min<int64_t>(U, Nt);
  const double tiles_u = (double)cdiv(Nt, n_active);
  const double t_tile = std::max(predict_vec_exec(in.func, std::min(T, in.N)), 0.0);
  const double tile_bytes = 8.0 * std::min(T, in.N);
  const bool any_host_in = in.locx == -1 || in.locy == -1;
  const bool host_out = axpy && in.locy == -1;
  const bool both = any_host_in && host_out;   // level-1 write-backs are never deferred
  double worst = 0.0;
  for (int u = 0; u < n_active; ++u) {
    const int dev = units[u];
    double in_tile = 0.0, out_tile = 0.0, peer_tile = 0.0;
    for (int loc : {in.locx, in.locy}) {
      if (loc == -1) in_tile += host_link_time_shared(dev, true, tile_bytes, n_active, both, &units);
      else if (loc != dev) peer_tile += link_time(dev, loc, tile_bytes);
    }
    if (axpy) {
      if (in.locy == -1) out_tile = host_link_time_shared(dev, false, tile_bytes, n_active, both, &units);
      else if (in.locy != dev) out_tile = link_time(in.locy, dev, tile_bytes);
    }
    const double stage = std::max(std::max(t_tile, in_tile), std::max(out_tile, peer_tile));
    const double t = tiles_u * stage + (in_tile + peer_tile) + t_tile + out_tile - stage;
    worst = std::max(worst, t);
  }
  return worst;
}

int autotune_vec(const VecModelInput& in, int ngpu, const paralia_ctl* ctl, paralia_report* rep) {
  if (in.N <= 0) return fail(PARALIA_ERR_INVALID_ARG, "autotune: non-positive length");
  if (g_db.link.empty()) reset_database_defaults(ngpu > 0 ? ngpu : 1);
  const TuneConstants& c = g_consts;
  std::vector<std::vector<int>> candidates;
  if (ctl && ctl->active_unit_num > 0) {
    std::vector<int> u;
    for (int i = 0; i < ctl->active_unit_num && i < PARALIA_MAX_UNITS; ++i) {
      const int d = ctl->active_unit_id_list[i];
      if (ngpu > 0 && (d < 0 || d >= ngpu))
        return fail(PARALIA_ERR_INVALID_ARG, "unit id %d is not a GPU", d);
      u.push_back(d);
    }
    candidates.push_back(u);
  } else {
    if (ngpu <= 0) return fail(PARALIA_ERR_NO_DEVICE, "autotune: no GPU and no fixed unit list");
    // the GPU that already holds a vector, alone; then prefix sets
    for (int loc : {in.locy, in.locx})
      if (loc >= 0 && loc < ngpu) candidates.push_back({loc});
    for (int n = 1; n <= ngpu; ++n) {
      std::vector<int> u(n);
      for (int i = 0; i < n; ++i) u[i] = i;
      candidates.push_back(u);
    }
  }
  // tile lengths: the measured ones between 2^16 and 2^25 elements (0.5 .. 256 MiB), or
  // the caller's
  std::vector<int64_t> tiles;
  if (ctl && ctl->T > 0) tiles.push_back(ctl->T);
  else {
    auto it = g_db.exec.find(in.func);
    if (it != g_db.exec.end()) {
      auto jt = it->second.by_trans.find("--");
      if (jt != it->second.by_trans.end())
        for (const auto& kv : jt->second)
          if (kv.first >= (1 << 16) && kv.first <= (1 << 25) && kv.first % 1024 == 0) tiles.push_back(kv.first);
    }
    if (tiles.empty()) for (int64_t t = 1 << 16; t <= (1 << 25); t *= 2) tiles.push_back(t);
  }
  double best_score = DBL_MAX, best_pred = 0;
  size_t best_card = 0;
  int64_t best_T = 0;
  std::vector<int> best_units;
  bool have = false;
  for (const auto& u : candidates) {
    int64_t uT = 0;
    double ut = DBL_MAX;
    for (size_t i = tiles.size(); i-- > 0;) {   // larger first: ties go to fewer tiles
      const int64_t T = std::min(tiles[i], in.N);
      const double t = predict_vec(in, T, u);
      if (t < ut * (1.0 - 1e-9)) { ut = t; uT = T; }
    }
    bool take = !have;
    if (have) {
      const double adj = ut * (1.0 + ((double)u.size() - (double)best_card) * c.minimum_unit_contribution);
      take = adj < best_score;
    }
    if (take) {
      best_score = ut; best_pred = ut; best_card = u.size(); best_T = uT; best_units = u; have = true;
    }
  }
  if (!have) return fail(PARALIA_ERR_INVALID_ARG, "autotune: no candidate configuration");
  if (rep) {
    memset(rep, 0, sizeof(*rep));
    rep->T = best_T;
    const int64_t Nt = cdiv(in.N, best_T);
    const int active = (int)std::min<int64_t>((int64_t)best_units.size(), Nt);
    rep->active_unit_num = active;
    for (int i = 0; i < active; ++i) {
      rep->active_unit_id_list[i] = best_units[i];
      rep->active_unit_score[i] = 1.0 / active;
    }
    rep->subkernel_num = Nt;
    rep->pred_t = best_pred;
    rep->grid_d1 = active;
    rep->grid_d2 = 1;
  }
  return PARALIA_OK;
}

}  // namespace paralia
