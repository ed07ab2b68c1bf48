#include "plan.hpp"

#include <algorithm>
#include <cstdlib>

namespace paralia {

int plan_kchain_forced() {
  static const int forced = [] {
    const char* e = getenv("PARALIA_KCHAIN");
    return e ? atoi(e) : 0;
  }();
  return forced;
}

int plan_kchain_len(bool bounded_cache, int ki0, int max_parts) {
  const int forced = plan_kchain_forced();
  int len = bounded_cache ? 1 : (forced > 0 ? forced : (ki0 == 0 ? 1 : 4));
  len = std::min(len, max_parts);
  return std::max(len, 1);
}

static std::vector<int> env_int_list(const char* name) {
  std::vector<int> out;
  const char* e = getenv(name);
  if (!e) return out;
  for (const char* p = e; *p;) {
    char* end = nullptr;
    const long v = strtol(p, &end, 10);
    if (end == p) break;
    if (v > 0) out.push_back((int)v);
    p = (*end == ',') ? end + 1 : end;
    if (*end && *end != ',') break;
  }
  return out;
}

void plan_band_sizes(int n_ctiles, int Kt, bool bounded_cache, const BandHints& h,
                     std::vector<int>* bands) {
  static const std::vector<int> forced_plan = env_int_list("PARALIA_BAND_PLAN");
  static const int forced_band = [] {
    const char* e = getenv("PARALIA_BAND");
    return e ? atoi(e) : 0;
  }();
  const int n = n_ctiles;
  bands->clear();
  if (n <= 0) return;
  if (bounded_cache) {
    bands->assign(n, 1);
    return;
  }
  if (!forced_plan.empty() || forced_band > 0) {
    for (int left = n, i = 0; left > 0; ++i) {
      int b = forced_band > 0 ? forced_band
                              : forced_plan[std::min<size_t>(i, forced_plan.size() - 1)];
      b = std::min(b, left);
      bands->push_back(b);
      left -= b;
    }
    return;
  }
  const int w = h.row_len > 0 ? std::min(h.row_len, n) : n;
  const int kt = std::max(Kt, 1);
  // first band: whole tile rows until a k step computes longer than it fetches (10 % margin);
  // a unit that stays input-bound whatever the band takes about half its tiles
  int first = -1;
  for (int rows = 1; rows * w < n; ++rows) {
    const int b = rows * w;
    const double need = rows * h.rho_a + w * h.rho_b + b * h.rho_c / kt;
    if ((double)b >= 1.1 * need && b >= std::min(n, 4)) {
      first = b;
      break;
    }
  }
  if (first < 0) first = n <= 4 ? n : std::max(w, (n / 2 / w) * w);
  first = std::min(first, n);
  // shrinking tail, built from the end: last_band, then doubling up to four tiles
  std::vector<int> tail;
  int left = n - first;
  for (int sz = std::max(1, h.last_band); left >= sz && sz <= 4; sz *= 2) {
    tail.push_back(sz);
    left -= sz;
  }
  bands->push_back(first);
  if (left > 0) {
    const int chunks = (left + 7) / 8;
    for (int c = 0; c < chunks; ++c) bands->push_back(left / chunks + (c < left % chunks ? 1 : 0));
  }
  for (size_t i = tail.size(); i-- > 0;) bands->push_back(tail[i]);
}

void plan_launch_order(const std::vector<int>& bands, int Kt, bool bounded_cache, int max_parts,
                       std::vector<LaunchItem>* items) {
  const int kt = std::max(Kt, 1);
  items->clear();
  int b0 = 0;
  for (int band : bands) {
    const int b1 = b0 + band;
    if (Kt == 0) {   // no product: one launch per tile scales C by beta
      for (int oi = b0; oi < b1; ++oi) items->push_back({oi, 0, 0, band});
      b0 = b1;
      continue;
    }
    for (int ki0 = 0; ki0 < kt;) {
      const int ki1 = std::min(kt, ki0 + plan_kchain_len(bounded_cache, ki0, max_parts));
      for (int oi = b0; oi < b1; ++oi) items->push_back({oi, ki0, ki1, band});
      ki0 = ki1;
    }
    b0 = b1;
  }
}

bool plan_unit_ctiles(const std::vector<std::vector<int>>& sk_lists, int kt_for_ids, int n_ctiles,
                      std::vector<std::vector<int>>* ctiles, std::vector<int>* owner) {
  ctiles->assign(sk_lists.size(), std::vector<int>());
  owner->assign(n_ctiles, -1);
  for (size_t ui = 0; ui < sk_lists.size(); ++ui) {
    for (int sk : sk_lists[ui]) {
      const int ct = sk / kt_for_ids;
      if ((*owner)[ct] == -1) {
        (*owner)[ct] = (int)ui;
        (*ctiles)[ui].push_back(ct);
      } else if ((*owner)[ct] != (int)ui) {
        return false;
      }
    }
  }
  return true;
}

}  // namespace paralia
