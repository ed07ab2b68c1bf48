#include "plan.hpp"

#include <algorithm>
#include <cstdlib>

namespace paralia {

int plan_kchain_len(bool bounded_cache, int ki0, int max_parts) {
  static const int forced = [] {
    const char* e = getenv("PARALIA_KCHAIN");
    return e ? atoi(e) : 0;
  }();
  int len = bounded_cache ? 1 : (forced > 0 ? forced : (ki0 == 0 ? 1 : 4));
  len = std::min(len, max_parts);
  return std::max(len, 1);
}

void plan_launch_order(int n_ctiles, int Kt, bool bounded_cache, int max_parts,
                       std::vector<LaunchItem>* items) {
  static const int band_env = [] {
    const char* e = getenv("PARALIA_BAND");
    return e ? atoi(e) : 0;
  }();
  const int n = n_ctiles;
  const int kt = std::max(Kt, 1);
  int band = band_env > 0 ? band_env : std::min(16, std::max(4, (n + 3) / 4));
  if (bounded_cache) band = 1;
  items->clear();
  for (int b0 = 0; b0 < n; b0 += band) {
    const int b1 = std::min(n, b0 + band);
    if (Kt == 0) {   // no product: one launch per tile scales C by beta
      for (int oi = b0; oi < b1; ++oi) items->push_back({oi, 0, 0});
      continue;
    }
    for (int ki0 = 0; ki0 < kt;) {
      const int ki1 = std::min(kt, ki0 + plan_kchain_len(bounded_cache, ki0, max_parts));
      for (int oi = b0; oi < b1; ++oi) items->push_back({oi, ki0, ki1});
      ki0 = ki1;
    }
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
