// C++ entry points with the names and argument lists of the reference's public header
// (Library_scheduler/include/PARALiA.hpp:33-72), so that callers written against it
// (e.g. Benchmarking/CuCuBLAS/src/PARALia/dgemm_runner.cpp:80-137) recompile unchanged.
// Each one forwards to the C ABI in paralia_c.h with PARALIA_LOC_AUTO, i.e. the location
// of every operand is inferred from its pointer as the reference does
// (CoCoGetPtrLoc, dgemm.cpp:356-363).
//
// ATC is a self-contained stand-in for the reference's autotune controller
// (Autotuner/include/Autotuner.hpp:121-174) that exposes the fields callers read or set:
// T, active_unit_num, active_unit_id_list, active_unit_score, cache_limit, pred_t, pred_J,
// subkernel_num, Subkernels_per_unit_num, print(), print_csv().
//
// Error behaviour: like the reference these wrappers do not return a status; on failure
// they print the library's message to stderr and return NULL.
#ifndef PARALiA_H
#define PARALiA_H

#include "paralia_c.h"

typedef class ATC {
 public:
  long int T;
  double T_aggregate_sl, T_imbalance_sl, T_remainder_sl, T_small_sl, T_sknum_sl, T_big_sl;
  int active_unit_num;
  int* active_unit_id_list;
  double* active_unit_score;
  short split_homogeneously;
  double pred_t;
  double pred_J;
  long int subkernel_num;
  int* Subkernels_per_unit_num;
  long long cache_limit;
  paralia_report report;   // everything the call measured (not in the reference)

  ATC();
  ~ATC();
  ATC(const ATC& other);
  ATC& operator=(const ATC& other);
  void reset();
  void mimic_ATC(class ATC* other_ATC);
  void print();
  const char* print_csv();
}* ATC_p;

ATC_p PARALiADgemm(char TransA, char TransB, long int M, long int N, long int K, double alpha,
                   double* A, long int ldA, double* B, long int ldB, double beta, double* C,
                   long int ldC);
ATC_p PARALiADgemmControled(char TransA, char TransB, long int M, long int N, long int K,
                            double alpha, double* A, long int ldA, double* B, long int ldB,
                            double beta, double* C, long int ldC, ATC_p predef_control_values);
ATC_p PARALiASgemm(char TransA, char TransB, long int M, long int N, long int K, float alpha,
                   float* A, long int ldA, float* B, long int ldB, float beta, float* C,
                   long int ldC);
ATC_p PARALiASgemmControled(char TransA, char TransB, long int M, long int N, long int K,
                            float alpha, float* A, long int ldA, float* B, long int ldB,
                            float beta, float* C, long int ldC, ATC_p predef_control_values);
ATC_p PARALiADgemv(char TransA, long int M, long int N, double alpha, double* A, long int ldA,
                   double* x, long int incx, double beta, double* y, long int incy);
ATC_p PARALiADgemvControled(char TransA, long int M, long int N, double alpha, double* A,
                            long int ldA, double* x, long int incx, double beta, double* y,
                            long int incy, ATC_p predef_control_values);
ATC_p PARALiADaxpy(long int N, double alpha, double* x, long int incx, double* y, long int incy);
ATC_p PARALiADaxpyControled(long int N, double alpha, double* x, long int incx, double* y,
                            long int incy, ATC_p predef_control_values);
ATC_p PARALiADdot(long int N, double* x, long int incx, double* y, long int incy, double* result);
ATC_p PARALiADdotControled(long int N, double* x, long int incx, double* y, long int incy,
                           double* result, ATC_p predef_control_values);
void PARALiADevCacheFree(short dev_id);

#endif
