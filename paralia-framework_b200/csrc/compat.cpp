// C++ wrappers with the reference's names (include/PARALiA.hpp) over the C ABI.
#include "../../include/PARALiA.hpp"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

ATC::ATC() {
  active_unit_id_list = (int*)malloc(PARALIA_MAX_UNITS * sizeof(int));
  active_unit_score = (double*)malloc(PARALIA_MAX_UNITS * sizeof(double));
  Subkernels_per_unit_num = (int*)malloc(PARALIA_MAX_UNITS * sizeof(int));
  reset();
}
ATC::~ATC() {
  free(active_unit_id_list);
  free(active_unit_score);
  free(Subkernels_per_unit_num);
}
ATC::ATC(const ATC& other) : ATC() { mimic_ATC(const_cast<ATC*>(&other)); }
ATC& ATC::operator=(const ATC& other) {
  if (this != &other) mimic_ATC(const_cast<ATC*>(&other));
  return *this;
}

// Untuned state, as the reference's ATC::reset leaves it.
void ATC::reset() {
  T = -1;
  T_aggregate_sl = T_imbalance_sl = T_remainder_sl = T_small_sl = T_sknum_sl = T_big_sl = 0.0;
  active_unit_num = -1;
  split_homogeneously = 0;
  pred_t = pred_J = -1.0;
  subkernel_num = -1;
  cache_limit = 0;
  for (int i = 0; i < PARALIA_MAX_UNITS; ++i) {
    active_unit_id_list[i] = -42;
    active_unit_score[i] = 0.0;
    Subkernels_per_unit_num[i] = 0;
  }
  memset(&report, 0, sizeof(report));
}

void ATC::mimic_ATC(ATC* o) {
  T = o->T;
  T_aggregate_sl = o->T_aggregate_sl; T_imbalance_sl = o->T_imbalance_sl;
  T_remainder_sl = o->T_remainder_sl; T_small_sl = o->T_small_sl;
  T_sknum_sl = o->T_sknum_sl; T_big_sl = o->T_big_sl;
  active_unit_num = o->active_unit_num;
  split_homogeneously = o->split_homogeneously;
  pred_t = o->pred_t; pred_J = o->pred_J;
  subkernel_num = o->subkernel_num;
  cache_limit = o->cache_limit;
  for (int i = 0; i < PARALIA_MAX_UNITS; ++i) {
    active_unit_id_list[i] = o->active_unit_id_list[i];
    active_unit_score[i] = o->active_unit_score[i];
    Subkernels_per_unit_num[i] = o->Subkernels_per_unit_num[i];
  }
  report = o->report;
}

static std::string list_str(const int* v, int n) {
  std::string s = "[ ";
  for (int i = 0; i < n; ++i) s += std::to_string(v[i]) + " ";
  return s + "]";
}

void ATC::print() {
  const int n = active_unit_num > 0 ? active_unit_num : 0;
  std::string scores = "[ ";
  for (int i = 0; i < n; ++i) scores += std::to_string(active_unit_score[i]) + " ";
  scores += "]";
  fprintf(stderr,
          "Autotune controller:\n->T = %ld\n->active_unit_num = %d\n->active_unit_id_list = %s\n"
          "->active_unit_score = %s\n->pred_t = %lf\n->subkernel_num = %ld\n"
          "->Subkernels_per_unit_num = %s\n\n",
          T, active_unit_num, list_str(active_unit_id_list, n).c_str(), scores.c_str(), pred_t,
          subkernel_num, list_str(Subkernels_per_unit_num, n).c_str());
}

// "T,ndev,devmask,cache_limit": the first four columns of the reference's run logs
// (Autotuner/src/Autotuner.cpp:839-846; devmask has a decimal 1 at position id).
const char* ATC::print_csv() {
  char* out = (char*)malloc(256);
  long mask = 0;
  if (active_unit_num > 0)
    for (int i = 0; i < active_unit_num; ++i)
      if (active_unit_id_list[i] >= 0) mask += (long)std::pow(10.0, active_unit_id_list[i]);
  snprintf(out, 256, "%ld,%d,%ld,%lld", T, active_unit_num, mask, cache_limit);
  return out;
}

static const paralia_ctl* to_ctl(ATC_p p, paralia_ctl* c) {
  if (!p) return nullptr;
  memset(c, 0, sizeof(*c));
  c->T = p->T > 0 ? p->T : 0;
  c->cache_limit = p->cache_limit > 0 ? p->cache_limit : 0;
  if (p->active_unit_num > 0) {
    c->active_unit_num = p->active_unit_num;
    for (int i = 0; i < p->active_unit_num && i < PARALIA_MAX_UNITS; ++i)
      c->active_unit_id_list[i] = p->active_unit_id_list[i];
  }
  return c;
}

static ATC_p from_report(int rc, const paralia_report& r, const char* who) {
  if (rc != PARALIA_OK) {
    fprintf(stderr, "%s: error %d: %s\n", who, rc, PARALiA_last_error());
    return nullptr;
  }
  ATC_p a = new ATC();
  a->T = (long)r.T;
  a->active_unit_num = r.active_unit_num;
  for (int i = 0; i < r.active_unit_num && i < PARALIA_MAX_UNITS; ++i) {
    a->active_unit_id_list[i] = r.active_unit_id_list[i];
    a->active_unit_score[i] = r.active_unit_score[i];
    a->Subkernels_per_unit_num[i] = r.subkernels_per_unit[i];
  }
  a->cache_limit = r.cache_limit;
  a->pred_t = r.pred_t;
  a->pred_J = r.pred_J;
  a->subkernel_num = (long)r.subkernel_num;
  a->T_aggregate_sl = r.T_slowdowns[0]; a->T_imbalance_sl = r.T_slowdowns[1];
  a->T_remainder_sl = r.T_slowdowns[2]; a->T_small_sl = r.T_slowdowns[3];
  a->T_sknum_sl = r.T_slowdowns[4]; a->T_big_sl = r.T_slowdowns[5];
  a->report = r;
  return a;
}

ATC_p PARALiADgemmControled(char TransA, char TransB, long int M, long int N, long int K,
                            double alpha, double* A, long int ldA, double* B, long int ldB,
                            double beta, double* C, long int ldC, ATC_p predef) {
  paralia_ctl c;
  paralia_report r;
  int rc = PARALiA_dgemm(TransA, TransB, M, N, K, alpha, A, ldA, PARALIA_LOC_AUTO, B, ldB,
                         PARALIA_LOC_AUTO, beta, C, ldC, PARALIA_LOC_AUTO, to_ctl(predef, &c), &r);
  return from_report(rc, r, "PARALiADgemm");
}
ATC_p PARALiADgemm(char TransA, char TransB, long int M, long int N, long int K, double alpha,
                   double* A, long int ldA, double* B, long int ldB, double beta, double* C,
                   long int ldC) {
  return PARALiADgemmControled(TransA, TransB, M, N, K, alpha, A, ldA, B, ldB, beta, C, ldC, NULL);
}

ATC_p PARALiASgemmControled(char TransA, char TransB, long int M, long int N, long int K,
                            float alpha, float* A, long int ldA, float* B, long int ldB,
                            float beta, float* C, long int ldC, ATC_p predef) {
  paralia_ctl c;
  paralia_report r;
  int rc = PARALiA_sgemm(TransA, TransB, M, N, K, alpha, A, ldA, PARALIA_LOC_AUTO, B, ldB,
                         PARALIA_LOC_AUTO, beta, C, ldC, PARALIA_LOC_AUTO, to_ctl(predef, &c), &r);
  return from_report(rc, r, "PARALiASgemm");
}
ATC_p PARALiASgemm(char TransA, char TransB, long int M, long int N, long int K, float alpha,
                   float* A, long int ldA, float* B, long int ldB, float beta, float* C,
                   long int ldC) {
  return PARALiASgemmControled(TransA, TransB, M, N, K, alpha, A, ldA, B, ldB, beta, C, ldC, NULL);
}

ATC_p PARALiADgemvControled(char TransA, long int M, long int N, double alpha, double* A,
                            long int ldA, double* x, long int incx, double beta, double* y,
                            long int incy, ATC_p predef) {
  paralia_ctl c;
  paralia_report r;
  int rc = PARALiA_dgemv(TransA, M, N, alpha, A, ldA, PARALIA_LOC_AUTO, x, incx, PARALIA_LOC_AUTO,
                         beta, y, incy, PARALIA_LOC_AUTO, to_ctl(predef, &c), &r);
  return from_report(rc, r, "PARALiADgemv");
}
ATC_p PARALiADgemv(char TransA, long int M, long int N, double alpha, double* A, long int ldA,
                   double* x, long int incx, double beta, double* y, long int incy) {
  return PARALiADgemvControled(TransA, M, N, alpha, A, ldA, x, incx, beta, y, incy, NULL);
}

ATC_p PARALiADaxpyControled(long int N, double alpha, double* x, long int incx, double* y,
                            long int incy, ATC_p predef) {
  paralia_ctl c;
  paralia_report r;
  int rc = PARALiA_daxpy(N, alpha, x, incx, PARALIA_LOC_AUTO, y, incy, PARALIA_LOC_AUTO,
                         to_ctl(predef, &c), &r);
  return from_report(rc, r, "PARALiADaxpy");
}
ATC_p PARALiADaxpy(long int N, double alpha, double* x, long int incx, double* y, long int incy) {
  return PARALiADaxpyControled(N, alpha, x, incx, y, incy, NULL);
}

ATC_p PARALiADdotControled(long int N, double* x, long int incx, double* y, long int incy,
                           double* result, ATC_p predef) {
  paralia_ctl c;
  paralia_report r;
  int rc = PARALiA_ddot(N, x, incx, PARALIA_LOC_AUTO, y, incy, PARALIA_LOC_AUTO, result,
                        to_ctl(predef, &c), &r);
  return from_report(rc, r, "PARALiADdot");
}
ATC_p PARALiADdot(long int N, double* x, long int incx, double* y, long int incy, double* result) {
  return PARALiADdotControled(N, x, incx, y, incy, result, NULL);
}

void PARALiADevCacheFree(short dev_id) {
  if (PARALiA_dev_cache_free(dev_id) != PARALIA_OK)
    fprintf(stderr, "PARALiADevCacheFree: %s\n", PARALiA_last_error());
}
