// Entry points of the routine executors, called by the extern "C" layer.
#pragma once
#include <stdint.h>

#include "../../include/paralia_c.h"

namespace paralia {

int exec_dgemm(char ta, char tb, int64_t M, int64_t N, int64_t K, double alpha, const double* A,
               int64_t ldA, int locA, const double* B, int64_t ldB, int locB, double beta,
               double* C, int64_t ldC, int locC, const paralia_ctl* ctl, paralia_report* out);

// Collective over the ranks of the process group (group.hpp): every rank passes its own
// row panel of A, column panel of B and block of C.
int exec_group_dgemm(char ta, char tb, int64_t M, int64_t N, int64_t K, double alpha,
                     const double* A, int64_t ldA, int locA, const double* B, int64_t ldB,
                     int locB, double beta, double* C, int64_t ldC, int locC,
                     const paralia_ctl* ctl, paralia_report* out);

int exec_group_sgemm(char ta, char tb, int64_t M, int64_t N, int64_t K, float alpha, const float* A,
                     int64_t ldA, int locA, const float* B, int64_t ldB, int locB, float beta,
                     float* C, int64_t ldC, int locC, const paralia_ctl* ctl, paralia_report* out);

int exec_sgemm(char ta, char tb, int64_t M, int64_t N, int64_t K, float alpha, const float* A,
               int64_t ldA, int locA, const float* B, int64_t ldB, int locB, float beta, float* C,
               int64_t ldC, int locC, const paralia_ctl* ctl, paralia_report* out);

int exec_tile_sgemm(int dev, void* stream, char ta, char tb, int64_t M, int64_t N, int64_t K,
                    float alpha, const float* A, int64_t ldA, const float* B, int64_t ldB,
                    float beta, float* C, int64_t ldC);

int exec_dgemv(char TransA, int64_t M, int64_t N, double alpha, const double* A, int64_t ldA,
               int locA, const double* x, int64_t incx, int locx, double beta, double* y,
               int64_t incy, int locy, const paralia_ctl* ctl, paralia_report* out);

int exec_daxpy(int64_t N, double alpha, const double* x, int64_t incx, int locx, double* y,
               int64_t incy, int locy, const paralia_ctl* ctl, paralia_report* out);

int exec_ddot(int64_t N, const double* x, int64_t incx, int locx, const double* y, int64_t incy,
              int locy, double* result, const paralia_ctl* ctl, paralia_report* out);

// The per-tile sums of a DDOT in tile order instead of their total (for callers that combine
// tiles computed by several processes in one global order).
int exec_ddot_tiles(int64_t N, const double* x, int64_t incx, int locx, const double* y,
                    int64_t incy, int locy, double* tile_sums, int64_t capacity, int64_t* count,
                    const paralia_ctl* ctl, paralia_report* out);

}  // namespace paralia
