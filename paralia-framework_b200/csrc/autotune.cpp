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

// Defaults for one 8xB200 NVSwitch box, used until a measured database is loaded:
// host link ~52 GB/s per GPU and direction (PCIe Gen5 x16), GPU-GPU ~700 GB/s through
// NVSwitch, ~10 us of launch/copy latency, DMMA tile kernel ~33 TFLOP/s.
void reset_database_defaults(int ngpu) {
  g_db = ModelDB();
  const int L = ngpu + 1;
  g_db.link.assign(L, std::vector<LinkModel>(L));
  for (int d = 0; d < L; ++d)
    for (int s = 0; s < L; ++s) {
      LinkModel& m = g_db.link[d][s];
      if (d == s) { m.ti = 0; m.tb = 0; }
      else if (d == 0 || s == 0) { m.ti = 12e-6; m.tb = 1.0 / 52e9; }
      else { m.ti = 10e-6; m.tb = 1.0 / 700e9; }
    }
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
}

static bool read_link_file(const std::string& path, LinkModel* m) {
  FILE* fp = fopen(path.c_str(), "r");
  if (!fp) return false;
  double ti = 0, tb = 0;
  // Format written by the link post-processing step: "Intercept: <ti>\nCoefficient: <tb>\n"
  // followed by Slowdown lines (Autotuner/src/CoModel.cpp:26-38).
  int items = fscanf(fp, "Intercept: %le\nCoefficient: %le\n", &ti, &tb);
  fclose(fp);
  if (items != 2) return false;
  m->ti = ti;
  m->tb = tb;
  return true;
}

static bool read_exec_file(const std::string& path, ExecTable* t) {
  FILE* fp = fopen(path.c_str(), "r");
  if (!fp) return false;
  char line[512];
  // Rows: TransA,TransB,T,T,T,mean_t,W,J,err,samples,bench_t
  // (Autotuner/src/GPUexec_lookup.cpp:79-81).
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

int load_database(const char* dir) {
  if (!dir) return fail(PARALIA_ERR_INVALID_ARG, "database directory is NULL");
  const int L = (int)g_db.link.size();
  if (L == 0) return fail(PARALIA_ERR_DB_MISSING, "model database not initialised");
  int found = 0;
  ModelDB db = g_db;
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
  // every host link, GPU 1<-GPU 0 for every GPU pair).
  for (int d = 0; d < L; ++d)
    for (int s = 0; s < L; ++s) {
      if (d == s || have[d][s]) continue;
      if (s == 0 && d >= 1 && have[1][0]) db.link[d][s] = db.link[1][0];
      else if (d == 0 && s >= 1 && have[0][1]) db.link[d][s] = db.link[0][1];
      else if (d >= 1 && s >= 1 && L > 2 && have[2][1]) db.link[d][s] = db.link[2][1];
    }
  const char* funcs[2] = {"Dgemm", "Sgemm"};
  for (const char* f : funcs) {
    char name[512];
    // one table per device in the reference; identical GPUs share device 0's table here
    snprintf(name, sizeof(name), "%s/Processed/%s_lookup-table_dev-0.log", dir, f);
    ExecTable t;
    if (read_exec_file(name, &t)) {
      db.exec[f] = t;
      ++found;
    }
  }
  if (!found)
    return fail(PARALIA_ERR_DB_MISSING, "no model files found under %s/Processed", dir);
  db.from_disk = true;
  db.dir = dir;
  g_db = db;
  return PARALIA_OK;
}

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

void device_grid(int units, int* d1_out, int* d2_out) {
  int d1 = (int)std::sqrt((double)units);
  int d2 = d1;
  if (d1 == 0) {
    d2 = units;
    d1 = 1;
  } else {
    int g;
    for (g = d1 + 1; g > 0; --g)
      if (units % g == 0) break;
    if (g == 0) {
      d1 = units;
      d2 = 1;
    } else {
      d1 = g;
      d2 = units / g;
    }
  }
  *d1_out = d1;
  *d2_out = d2;
}

// Plain round robin over subkernel ids (Subkernel_distributions.cpp:10-76), equal scores.
static int distribute_round_robin(int units, int sk_num, std::vector<std::vector<int>>* lists) {
  if (sk_num < units) {
    lists->assign(sk_num, std::vector<int>());
    for (int d = 0; d < sk_num; ++d) (*lists)[d].push_back(d);
    return sk_num;
  }
  std::vector<int> num(units);
  int rem = sk_num;
  for (int d = 0; d < units; ++d) {
    num[d] = (int)(1.0 * (1.0 / units) * sk_num);
    rem -= num[d];
  }
  while (rem != 0)
    for (int d = 0; d < units; ++d) {
      if (rem != 0) {
        num[d] += 1;
        --rem;
      } else break;
    }
  lists->assign(units, std::vector<int>());
  int total = 0;
  while (total < sk_num)
    for (int d = 0; d < units; ++d) {
      if (total == sk_num) break;
      if ((int)(*lists)[d].size() == num[d]) continue;
      (*lists)[d].push_back(total++);
    }
  return units;
}

// Round robin in chunks of one C tile's k-chain (Subkernel_distributions.cpp:143-220).
static int distribute_round_robin_chunk(int units, int sk_num, int chunk,
                                        std::vector<std::vector<int>>* lists) {
  const int buckets = sk_num / chunk;
  if (buckets <= units) {
    lists->assign(buckets, std::vector<int>());
    for (int d = 0; d < buckets; ++d)
      for (int i = 0; i < chunk; ++i) (*lists)[d].push_back(d * chunk + i);
    return buckets;
  }
  std::vector<int> num(units);
  int accounted = 0;
  for (int d = 0; d < units; ++d) {
    num[d] = chunk * (int)(1.0 * (1.0 / units) * buckets);
    accounted += num[d];
  }
  lists->assign(units, std::vector<int>());
  int sk = 0, devidx = 0;
  for (int b = 0; b < buckets; ++b) {
    for (int i = 0; i < chunk; ++i) {
      int full_circle = units;
      while ((int)(*lists)[devidx].size() == num[devidx] && sk < accounted) {
        if (!full_circle) return -1;
        devidx = (devidx == units - 1) ? 0 : devidx + 1;
        --full_circle;
      }
      (*lists)[devidx].push_back(sk);
      if (sk >= accounted) num[devidx]++;
      ++sk;
    }
    devidx = (devidx == units - 1) ? 0 : devidx + 1;
  }
  return units;
}

int distribute_subkernels_2d(int units, int Mt, int Nt, int Kt,
                             std::vector<std::vector<int>>* lists, int* d1_out, int* d2_out) {
  const int sk_num = Mt * Nt * Kt;
  int d1, d2;
  device_grid(units, &d1, &d2);
  if (d1_out) *d1_out = d1;
  if (d2_out) *d2_out = d2;
  if (Nt == Kt && Nt == 1) return distribute_round_robin(units, sk_num, lists);
  if (Mt < d1 || Nt < d2) return distribute_round_robin_chunk(units, sk_num, Kt, lists);
  const int Mt_div = Mt / d1 * d1, Nt_div = Nt / d2 * d2;
  const int Mt_mod = Mt % d1, Nt_mod = Nt % d2;
  if (Mt * Nt < units) {
    // Cannot be reached after the check above (Mt >= d1 and Nt >= d2 imply
    // Mt*Nt >= units); kept so that the branch structure matches the reference.
    lists->assign(Mt * Nt, std::vector<int>());
    for (int d = 0; d < Mt * Nt; ++d)
      for (int k = 0; k < Kt; ++k) (*lists)[d].push_back(d * Kt + k);
    return Mt * Nt;
  }
  std::vector<int> num(units);
  int accounted = 0;
  const double score = 1.0 / units;
  for (int d = 0; d < units; ++d) {
    num[d] = Kt * (int)(score * Mt_div * Nt_div);
    accounted += num[d];
  }
  if (!Mt_mod && !Nt_mod && accounted < sk_num) {
    // int(score*buckets) can land one below the exact quotient in floating point.
    const int buckets = Mt_div * Nt_div;
    int buckets_rem = (sk_num - accounted) / Kt;
    const int intended = buckets / units;
    for (int d = 0; d < units; ++d)
      if (num[d] / Kt < intended && buckets_rem) {
        num[d] += Kt;
        --buckets_rem;
      }
  }
  lists->assign(units, std::vector<int>());
  int devidx = 0;
  for (int i1 = 0; i1 < Mt_div; ++i1)
    for (int i2 = 0; i2 < Nt_div; ++i2)
      for (int i3 = 0; i3 < Kt; ++i3) {
        const int sk = i1 * Nt * Kt + i2 * Kt + i3;
        devidx = i1 / (Mt / d1) * d2 + i2 / (Nt / d2);
        int full_circle = units;
        while ((int)(*lists)[devidx].size() == num[devidx]) {
          if (!full_circle) return -1;
          devidx = (devidx == units - 1) ? 0 : devidx + 1;
          --full_circle;
        }
        (*lists)[devidx].push_back(sk);
      }
  devidx = 0;
  for (int i1 = 0; i1 < Mt_div; ++i1)
    for (int i2 = Nt_div; i2 < Nt_div + Nt_mod; ++i2) {
      for (int i3 = 0; i3 < Kt; ++i3) (*lists)[devidx].push_back(i1 * Nt * Kt + i2 * Kt + i3);
      devidx = (devidx == units - 1) ? 0 : devidx + 1;
    }
  for (int i1 = Mt_div; i1 < Mt_div + Mt_mod; ++i1)
    for (int i2 = 0; i2 < Nt_div; ++i2) {
      for (int i3 = 0; i3 < Kt; ++i3) (*lists)[devidx].push_back(i1 * Nt * Kt + i2 * Kt + i3);
      devidx = (devidx == units - 1) ? 0 : devidx + 1;
    }
  for (int i1 = Mt_div; i1 < Mt_div + Mt_mod; ++i1)
    for (int i2 = Nt_div; i2 < Nt_div + Nt_mod; ++i2) {
      for (int i3 = 0; i3 < Kt; ++i3) (*lists)[devidx].push_back(i1 * Nt * Kt + i2 * Kt + i3);
      devidx = (devidx == units - 1) ? 0 : devidx + 1;
    }
  return units;
}

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

static double link_time(int dst_loc, int src_loc, double bytes) {
  if (bytes <= 0 || dst_loc == src_loc) return 0.0;
  const int L = (int)g_db.link.size();
  int d = dst_loc + 1, s = src_loc + 1;
  if (d >= L) d = L - 1;
  if (s >= L) s = L - 1;
  if (d < 0 || s < 0 || L == 0) return 0.0;
  const LinkModel& m = g_db.link[d][s];
  return m.ti + m.tb * bytes;
}

double predict_gemm(const GemmModelInput& in, int64_t T, const std::vector<int>& units,
                    const double sl[6], std::vector<UnitPrediction>* per_unit) {
  const int U = (int)units.size();
  int d1, d2;
  device_grid(U, &d1, &d2);
  const double share = 1.0 / U;
  const double szA = (double)in.M * in.K * in.esz, szB = (double)in.K * in.N * in.esz,
               szC = (double)in.M * in.N * in.esz;
  // exec: tile count times the tile time at the largest measured T that fits
  // (ModelLvl3.cpp:84-90)
  const int64_t Tb = std::min<int64_t>(T, std::min(in.M, std::min(in.N, in.K)));
  const double t_tile = predict_tile_exec(in.func, in.ta, in.tb, Tb);
  const double tiles = ((double)in.M / Tb) * ((double)in.N / Tb) * ((double)in.K / Tb);
  double worst = 0.0;
  if (per_unit) per_unit->clear();
  // Host-resident operands cross each host link once and are then forwarded between GPUs,
  // so the host term of a unit is its share of every host operand.
  for (int u = 0; u < U; ++u) {
    const int dev = units[u];
    UnitPrediction p{};
    p.t_exec = t_tile > 0 ? tiles * t_tile * share : 0.0;
    double recv = 0.0, send = 0.0, extra = 0.0;
    const double inC = in.beta_nonzero ? 1.0 : 0.0;
    if (in.locA != dev) recv += link_time(dev, in.locA, szA * share);
    if (in.locB != dev) recv += link_time(dev, in.locB, szB * share);
    if (in.locC != dev) {
      recv += link_time(dev, in.locC, szC * share * inC);
      send += link_time(in.locC, dev, szC * share);
    }
    // Peer traffic of the 2D grid: the rest of the A row panel from the d2-1 row mates
    // and of the B column panel from the d1-1 column mates (ModelLvl3.cpp:193-200).
    const int mate = units[(u + 1) % U];
    if (U > 1) {
      if (in.locA != dev) extra += link_time(dev, mate, szA * share * (d2 - 1));
      if (in.locB != dev) extra += link_time(dev, mate, szB * share * (d1 - 1));
    }
    p.t_recv = recv;
    p.t_send = send;
    p.t_extra = extra;
    p.t_total = std::max(std::max(p.t_exec, p.t_recv), std::max(p.t_send, p.t_extra));
    p.t_total *= (1.0 + (sl ? sl[0] : 0.0));
    // What the overlap cannot hide: the first A and B (and C) tiles have to arrive before
    // the first tile product starts, and the last C tile leaves after the last one ends.
    // (The reference folds this into its tile-size slowdown constants; with measured links
    // it is cheaper to state it.)
    const double tile_bytes = (double)Tb * Tb * in.esz;
    double fill = 0.0;
    if (in.locA != dev) fill += link_time(dev, in.locA, tile_bytes);
    if (in.locB != dev) fill += link_time(dev, in.locB, tile_bytes);
    if (in.locC != dev) fill += link_time(dev, in.locC, tile_bytes * inC) + link_time(in.locC, dev, tile_bytes);
    p.t_total += fill;
    worst = std::max(worst, p.t_total);
    if (per_unit) per_unit->push_back(p);
  }
  return worst;
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
    } else {
      ch.T = optimize_tile(in.M, in.N, in.K, (int)u.size(), c, c.tile_step, ch.sl);
    }
    ch.pred = predict_gemm(in, ch.T, u, ch.sl, nullptr);
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
    const int64_t Mt = (in.M + best.T - 1) / best.T, Nt = (in.N + best.T - 1) / best.T,
                  Kt = (in.K + best.T - 1) / best.T;
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

}  // namespace paralia
