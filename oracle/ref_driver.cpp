// Driver around the reference's own subkernel distribution, compiled from its source
// where it lies (see Makefile, target _ref). Prints, for a list of
// (units, Mt, Nt, Kt) cases, the unit index that owns every subkernel id.
// TEST INFRASTRUCTURE ONLY: used to pin the oracle's and the library's restatements.
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "Subkernel_distributions.hpp"

int main(int argc, char** argv) {
  if (argc != 5) {
    fprintf(stderr, "usage: %s units Mt Nt Kt\n", argv[0]);
    return 2;
  }
  const int units = atoi(argv[1]), Mt = atoi(argv[2]), Nt = atoi(argv[3]), Kt = atoi(argv[4]);
  const int sk = Mt * Nt * Kt;
  // The controller is filled by hand: its constructor lives in a source file that needs
  // the absent backend.
  ATC_p a = (ATC_p)calloc(1, sizeof(ATC));
  a->active_unit_num = units;
  a->subkernel_num = sk;
  a->active_unit_id_list = (int*)malloc(units * sizeof(int));
  a->active_unit_score = (double*)malloc(units * sizeof(double));
  a->Subkernels_per_unit_num = (int*)calloc(units, sizeof(int));
  a->Subkernels_per_unit_list = (int**)malloc(units * sizeof(int*));
  a->linkmap = new LinkMap();
  for (int d = 0; d < units; ++d) {
    a->active_unit_id_list[d] = d;
    a->active_unit_score[d] = 1.0 / units;
    a->Subkernels_per_unit_list[d] = (int*)malloc(sk * sizeof(int));
    for (int i = 0; i < sk; ++i) a->Subkernels_per_unit_list[d][i] = -1;
  }
  CoCoDistributeSubkernels2DBlockCyclic(a, Mt, Nt, Kt);
  int* owner = (int*)malloc(sk * sizeof(int));
  for (int i = 0; i < sk; ++i) owner[i] = -1;
  for (int d = 0; d < a->active_unit_num; ++d)
    for (int j = 0; j < a->Subkernels_per_unit_num[d]; ++j) {
      const int id = a->Subkernels_per_unit_list[d][j];
      if (id >= 0 && id < sk) owner[id] = d;
    }
  printf("%d", a->active_unit_num);
  for (int i = 0; i < sk; ++i) printf(" %d", owner[i]);
  printf("\n");
  return 0;
}
