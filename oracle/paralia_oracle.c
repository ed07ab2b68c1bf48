/*
 * CPU oracle for the tiled BLAS hot path -- TEST INFRASTRUCTURE ONLY.
 *
 * Nothing in the shipped library links, loads or calls this file; it is used by the
 * tests, by the smoke check and by the CPU-baseline leg of the benchmark to check the
 * CUDA path.
 *
 * It restates, in plain C, the arithmetic the reference performs for one call:
 *   - GEMM: the problem is cut into T x T tiles; C tile (mi,ni) receives, for
 *     ki = 0..Kt-1 in order, acc = alpha*op(A(mi,ki))*op(B(ki,ni)) + b*acc with b = 0 for
 *     the first ki and 1 afterwards (Library_scheduler/src/Functions/dgemm.cpp:273-279),
 *     and after the last ki the original tile is combined as C = acc + beta*C
 *     (WR_LAZY with reduce_mult = beta, dgemm.cpp:173-179). Subkernel ids are
 *     mi*Nt*Kt + ni*Kt + ki (dgemm.cpp:157-161).
 *   - DAXPY: y_t = alpha*x_t + y_t per 1-D tile (daxpy.cpp:53-69).
 *   - DDOT: one partial per tile, added to *result in tile order without zeroing it
 *     (ddot.cpp:62-70,431).
 *   - tile-size score (Autotuner/src/Autotuner.cpp:571-603), tile choice (:605-655), and
 *     the 2D block distribution with its fallbacks
 *     (Autotuner/src/Subkernel_distributions.cpp:10-76,143-220,315-485).
 *
 * Pinning. The reference holds no golden vectors or known-answer tests for this path
 * (its testers compare against cuBLASXt / OpenBLAS at run time), and its own
 * implementation cannot be built because its backend submodule is absent, so absolute
 * parity is UNPINNED. What is pinned: (1) this file agrees with OpenBLAS cblas_dgemm /
 * sgemm / daxpy / ddot -- the routines the reference itself uses as its CPU comparator
 * (Benchmarking/CuCuBLAS/src/cuBLASXt/cuBLASXtWrappers.cpp:15-28) -- on seeded inputs,
 * and (2) the distribution restated here agrees with the reference's own
 * Subkernel_distributions.cpp compiled from its source (see Makefile, target _ref).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ---- input generator: element i depends on (seed, i) only ------------------------- */
static uint64_t mix64(uint64_t seed, uint64_t idx) {
  uint64_t z = seed + (idx + 1) * 0x9E3779B97F4A7C15ULL;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  return z ^ (z >> 31);
}
void oracle_fill_uniform_f64(double* p, int64_t n, uint64_t seed) {
  for (int64_t i = 0; i < n; ++i)
    p[i] = (double)(mix64(seed, (uint64_t)i) >> 11) * (1.0 / 4503599627370496.0) - 1.0;
}
void oracle_fill_uniform_f32(float* p, int64_t n, uint64_t seed) {
  for (int64_t i = 0; i < n; ++i)
    p[i] = (float)(mix64(seed, (uint64_t)i) >> 40) * (1.0f / 8388608.0f) - 1.0f;
}
void oracle_fill_normal_f64(double* p, int64_t n, uint64_t seed) {
  for (int64_t i = 0; i < n; ++i) {
    const uint64_t a = mix64(seed, 2 * (uint64_t)i);
    const uint64_t b = mix64(seed ^ 0xD1B54A32D192ED03ULL, 2 * (uint64_t)i + 1);
    const double u1 = ((double)(a >> 11) + 1.0) * (1.0 / 9007199254740992.0);
    const double u2 = (double)(b >> 11) * (1.0 / 9007199254740992.0);
    p[i] = sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925286766559 * u2);
  }
}

static int64_t imin(int64_t a, int64_t b) { return a < b ? a : b; }

/* op(A)(m,k), op(B)(k,n) for column-major storage */
#define A_AT(m, k) (ta ? A[(int64_t)(k) + (int64_t)(m) * lda] : A[(int64_t)(m) + (int64_t)(k) * lda])
#define B_AT(k, n) (tb ? B[(int64_t)(n) + (int64_t)(k) * ldb] : B[(int64_t)(k) + (int64_t)(n) * ldb])

/* ---- tiled DGEMM (dgemm.cpp:123-205, 273-279) -------------------------------------- */
int oracle_dgemm_tiled(int ta, int tb, int64_t M, int64_t N, int64_t K, double alpha,
                       const double* A, int64_t lda, const double* B, int64_t ldb, double beta,
                       double* C, int64_t ldc, int64_t T) {
  if (T <= 0 || M < 0 || N < 0 || K < 0) return 1;
  const int64_t Mt = (M + T - 1) / T, Nt = (N + T - 1) / T, Kt = (K + T - 1) / T;
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int64_t mi = 0; mi < Mt; ++mi)
    for (int64_t ni = 0; ni < Nt; ++ni) {
      const int64_t m0 = mi * T, n0 = ni * T, mr = imin(T, M - m0), nc = imin(T, N - n0);
      double* acc = (double*)calloc((size_t)mr * nc, sizeof(double));
      double* col = (double*)malloc((size_t)mr * sizeof(double));
      for (int64_t ki = 0; ki < Kt; ++ki) {
        const int64_t k0 = ki * T, kl = imin(T, K - k0);
        const double b = ki == 0 ? 0.0 : 1.0;
        for (int64_t j = 0; j < nc; ++j) {
          for (int64_t i = 0; i < mr; ++i) col[i] = 0.0;
          for (int64_t k = 0; k < kl; ++k) {
            const double bv = B_AT(k0 + k, n0 + j);
            if (!ta) {
              const double* ac = A + (m0) + (k0 + k) * lda;
              for (int64_t i = 0; i < mr; ++i) col[i] += ac[i] * bv;
            } else {
              for (int64_t i = 0; i < mr; ++i) col[i] += A_AT(m0 + i, k0 + k) * bv;
            }
          }
          for (int64_t i = 0; i < mr; ++i) acc[i + j * mr] = alpha * col[i] + b * acc[i + j * mr];
        }
      }
      for (int64_t j = 0; j < nc; ++j)
        for (int64_t i = 0; i < mr; ++i) {
          double* c = &C[(m0 + i) + (n0 + j) * ldc];
          /* beta == 0 must not propagate NaN/Inf from C, as in BLAS */
          *c = (beta == 0.0) ? acc[i + j * mr] : acc[i + j * mr] + beta * (*c);
        }
      free(acc);
      free(col);
    }
  return 0;
}

/* ---- tiled SGEMM, FP32 arithmetic (sgemm.cpp:85-139) -------------------------------- */
#undef A_AT
#undef B_AT
#define A_AT(m, k) (ta ? A[(int64_t)(k) + (int64_t)(m) * lda] : A[(int64_t)(m) + (int64_t)(k) * lda])
#define B_AT(k, n) (tb ? B[(int64_t)(n) + (int64_t)(k) * ldb] : B[(int64_t)(k) + (int64_t)(n) * ldb])
int oracle_sgemm_tiled(int ta, int tb, int64_t M, int64_t N, int64_t K, float alpha,
                       const float* A, int64_t lda, const float* B, int64_t ldb, float beta,
                       float* C, int64_t ldc, int64_t T) {
  if (T <= 0 || M < 0 || N < 0 || K < 0) return 1;
  const int64_t Mt = (M + T - 1) / T, Nt = (N + T - 1) / T, Kt = (K + T - 1) / T;
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int64_t mi = 0; mi < Mt; ++mi)
    for (int64_t ni = 0; ni < Nt; ++ni) {
      const int64_t m0 = mi * T, n0 = ni * T, mr = imin(T, M - m0), nc = imin(T, N - n0);
      float* acc = (float*)calloc((size_t)mr * nc, sizeof(float));
      float* col = (float*)malloc((size_t)mr * sizeof(float));
      for (int64_t ki = 0; ki < Kt; ++ki) {
        const int64_t k0 = ki * T, kl = imin(T, K - k0);
        const float b = ki == 0 ? 0.0f : 1.0f;
        for (int64_t j = 0; j < nc; ++j) {
          for (int64_t i = 0; i < mr; ++i) col[i] = 0.0f;
          for (int64_t k = 0; k < kl; ++k) {
            const float bv = B_AT(k0 + k, n0 + j);
            for (int64_t i = 0; i < mr; ++i) col[i] += A_AT(m0 + i, k0 + k) * bv;
          }
          for (int64_t i = 0; i < mr; ++i) acc[i + j * mr] = alpha * col[i] + b * acc[i + j * mr];
        }
      }
      for (int64_t j = 0; j < nc; ++j)
        for (int64_t i = 0; i < mr; ++i) {
          float* c = &C[(m0 + i) + (n0 + j) * ldc];
          *c = (beta == 0.0f) ? acc[i + j * mr] : acc[i + j * mr] + beta * (*c);
        }
      free(acc);
      free(col);
    }
  return 0;
}

/* ---- DAXPY per tile (daxpy.cpp:53-69). One fused multiply-add per element, which is
 * what a GPU axpy computes; the result is therefore bit-comparable. ------------------- */
int oracle_daxpy_tiled(int64_t N, double alpha, const double* x, int64_t incx, double* y,
                       int64_t incy, int64_t T) {
  if (T <= 0 || N < 0) return 1;
  const int64_t Nt = (N + T - 1) / T;
  for (int64_t t = 0; t < Nt; ++t) {
    const int64_t lo = t * T, hi = imin(N, lo + T);
    for (int64_t i = lo; i < hi; ++i) y[i * incy] = fma(alpha, x[i * incx], y[i * incy]);
  }
  return 0;
}

/* ---- DDOT: a partial per tile, added to *result in tile order (ddot.cpp:431).
 * Inside a tile the sum is taken in long double so that the oracle is at least as
 * accurate as any summation order the GPU uses. -------------------------------------- */
int oracle_ddot_tiled(int64_t N, const double* x, int64_t incx, const double* y, int64_t incy,
                      int64_t T, double* result, double* abs_sum) {
  if (T <= 0 || N < 0) return 1;
  const int64_t Nt = (N + T - 1) / T;
  long double mag = 0.0L;
  for (int64_t t = 0; t < Nt; ++t) {
    const int64_t lo = t * T, hi = imin(N, lo + T);
    long double part = 0.0L;
    for (int64_t i = lo; i < hi; ++i) {
      const long double p = (long double)x[i * incx] * (long double)y[i * incy];
      part += p;
      mag += fabsl(p);
    }
    *result += (double)part;
  }
  if (abs_sum) *abs_sum = (double)mag;
  return 0;
}

/* ---- tile-size score (Autotuner.cpp:571-603) with the reference's constants
 * (CMakeLists.txt:157-165) --------------------------------------------------------- */
void oracle_tile_slowdowns(int64_t D1, int64_t D2, int64_t D3, int64_t T, int units, double* sl) {
  const int64_t TILE_MIN = 2048, TILE_MAX = 4096, MAX_SK = 512;
  const double TILE_MIN_SL = 0.2, TILE_MAX_SL = 0.1, MAX_SK_SL = 0.1;
  for (int i = 0; i < 6; ++i) sl[i] = 0.0;
  const int64_t sk = (D1 / T + ((D1 % T) ? 1 : 0)) * (D2 / T + ((D2 % T) ? 1 : 0)) *
                     (D3 / T + ((D3 % T) ? 1 : 0));
  const int64_t buckets = sk / (D3 / T + ((D3 % T) ? 1 : 0));
  sl[1] = (buckets / units) ? 1.0 * (buckets % units) / (buckets / units) * units
                            : 1.0 * buckets / units;
  if (D1 % T) sl[2] += 1.0 / (D1 / T);
  if (D2 % T) sl[2] += 1.0 / (D2 / T);
  if (D3 % T) sl[2] += 1.0 / (D3 / T);
  if (T < TILE_MIN) sl[3] += 1.0 * TILE_MIN / T * TILE_MIN_SL;
  const long dev_sks = (long)((1.0 * sk) / units);
  sl[4] += 2.0 / dev_sks;
  if (dev_sks > MAX_SK) sl[4] += (1.0 * dev_sks / MAX_SK) * MAX_SK_SL;
  if (T > TILE_MAX) sl[5] += T / TILE_MAX * TILE_MAX_SL;
  sl[0] = sl[1] + sl[2] + sl[3] + sl[4] + sl[5];
}

/* T scanned from min(D1,D2,D3) down to 1, first strict minimum wins (Autotuner.cpp:605-655);
 * step > 1 keeps only multiples of step (and the largest T). */
int64_t oracle_optimize_tile(int64_t D1, int64_t D2, int64_t D3, int units, int64_t step,
                             double* sl_out) {
  const int64_t maxT = imin(D1, imin(D2, D3));
  double best[6], cur[6];
  int64_t bestT = -1;
  for (int i = 0; i < 6; ++i) best[i] = 1e300;
  for (int64_t T = maxT; T > 0; --T) {
    if (step > 1 && T != maxT && (T % step)) continue;
    oracle_tile_slowdowns(D1, D2, D3, T, units, cur);
    if (cur[0] < best[0]) {
      memcpy(best, cur, sizeof(best));
      bestT = T;
    }
  }
  if (sl_out) memcpy(sl_out, best, sizeof(best));
  return bestT;
}

/* ---- 2D block distribution with equal unit scores
 * (Subkernel_distributions.cpp:315-485; fallbacks :10-76 and :143-220).
 * owner[sk] = index of the unit that runs subkernel sk. Returns the number of units
 * that received work, or -1 where the reference would abort. ------------------------ */
static void grid_of(int units, int* d1o, int* d2o) {
  int d1 = (int)sqrt((double)units), d2 = d1;
  if (d1 == 0) { d2 = units; d1 = 1; }
  else {
    int g;
    for (g = d1 + 1; g > 0; --g) if (units % g == 0) break;
    if (g == 0) { d1 = units; d2 = 1; } else { d1 = g; d2 = units / g; }
  }
  *d1o = d1; *d2o = d2;
}

int oracle_distribute_2d(int units, int Mt, int Nt, int Kt, int32_t* owner, int32_t* d1_out,
                         int32_t* d2_out) {
  const int sk_num = Mt * Nt * Kt;
  int d1, d2;
  grid_of(units, &d1, &d2);
  if (d1_out) *d1_out = d1;
  if (d2_out) *d2_out = d2;
  for (int i = 0; i < sk_num; ++i) owner[i] = -1;
  int* cnt = (int*)calloc((size_t)units, sizeof(int));
  int* num = (int*)calloc((size_t)units, sizeof(int));
  int active = units;
  const double score = 1.0 / units;
  if (Nt == 1 && Kt == 1) { /* round robin */
    if (sk_num < units) {
      for (int d = 0; d < sk_num; ++d) owner[d] = d;
      active = sk_num;
    } else {
      int rem = sk_num;
      for (int d = 0; d < units; ++d) { num[d] = (int)(1.0 * score * sk_num); rem -= num[d]; }
      while (rem != 0)
        for (int d = 0; d < units; ++d) { if (rem != 0) { num[d]++; rem--; } else break; }
      int total = 0;
      while (total < sk_num)
        for (int d = 0; d < units; ++d) {
          if (total == sk_num) break;
          if (cnt[d] == num[d]) continue;
          owner[total++] = d; cnt[d]++;
        }
    }
  } else if (Mt < d1 || Nt < d2) { /* round robin in chunks of Kt */
    const int buckets = sk_num / Kt;
    if (buckets <= units) {
      for (int d = 0; d < buckets; ++d) for (int i = 0; i < Kt; ++i) owner[d * Kt + i] = d;
      active = buckets;
    } else {
      int accounted = 0;
      for (int d = 0; d < units; ++d) { num[d] = Kt * (int)(1.0 * score * buckets); accounted += num[d]; }
      int sk = 0, dev = 0;
      for (int b = 0; b < buckets; ++b) {
        for (int i = 0; i < Kt; ++i) {
          int circle = units;
          while (cnt[dev] == num[dev] && sk < accounted) {
            if (!circle) { free(cnt); free(num); return -1; }
            dev = (dev == units - 1) ? 0 : dev + 1; circle--;
          }
          owner[sk] = dev;
          if (sk >= accounted) num[dev]++;
          cnt[dev]++; sk++;
        }
        dev = (dev == units - 1) ? 0 : dev + 1;
      }
    }
  } else {
    const int Md = Mt / d1 * d1, Nd = Nt / d2 * d2, Mm = Mt % d1, Nm = Nt % d2;
    int accounted = 0;
    for (int d = 0; d < units; ++d) { num[d] = Kt * (int)(score * Md * Nd); accounted += num[d]; }
    if (!Mm && !Nm && accounted < sk_num) {
      int rem = (sk_num - accounted) / Kt;
      const int intended = Md * Nd / units;
      for (int d = 0; d < units; ++d)
        if (num[d] / Kt < intended && rem) { num[d] += Kt; rem--; }
    }
    int dev = 0;
    for (int i1 = 0; i1 < Md; ++i1)
      for (int i2 = 0; i2 < Nd; ++i2)
        for (int i3 = 0; i3 < Kt; ++i3) {
          const int sk = i1 * Nt * Kt + i2 * Kt + i3;
          dev = i1 / (Mt / d1) * d2 + i2 / (Nt / d2);
          int circle = units;
          while (cnt[dev] == num[dev]) {
            if (!circle) { free(cnt); free(num); return -1; }
            dev = (dev == units - 1) ? 0 : dev + 1; circle--;
          }
          owner[sk] = dev; cnt[dev]++;
        }
    dev = 0;
    for (int i1 = 0; i1 < Md; ++i1)
      for (int i2 = Nd; i2 < Nd + Nm; ++i2) {
        for (int i3 = 0; i3 < Kt; ++i3) owner[i1 * Nt * Kt + i2 * Kt + i3] = dev;
        dev = (dev == units - 1) ? 0 : dev + 1;
      }
    for (int i1 = Md; i1 < Md + Mm; ++i1)
      for (int i2 = 0; i2 < Nd; ++i2) {
        for (int i3 = 0; i3 < Kt; ++i3) owner[i1 * Nt * Kt + i2 * Kt + i3] = dev;
        dev = (dev == units - 1) ? 0 : dev + 1;
      }
    for (int i1 = Md; i1 < Md + Mm; ++i1)
      for (int i2 = Nd; i2 < Nd + Nm; ++i2) {
        for (int i3 = 0; i3 < Kt; ++i3) owner[i1 * Nt * Kt + i2 * Kt + i3] = dev;
        dev = (dev == units - 1) ? 0 : dev + 1;
      }
  }
  free(cnt);
  free(num);
  return active;
}

/* ---- DGEMV: y <- alpha*op(A)*x + beta*y, A is M x N column-major
 * (Library_scheduler/include/PARALiA.hpp:48-53, Library_scheduler/src/Functions/dgemv.cpp:288).
 * Sums are taken in long double so that the oracle is at least as accurate as any
 * summation order of the GPU path. */
int oracle_dgemv(int trans, int64_t M, int64_t N, double alpha, const double* A, int64_t lda,
                 const double* x, int64_t incx, double beta, double* y, int64_t incy) {
  if (M < 0 || N < 0) return 1;
  const int64_t out_len = trans ? N : M, in_len = trans ? M : N;
  for (int64_t o = 0; o < out_len; ++o) {
    long double s = 0.0L;
    for (int64_t i = 0; i < in_len; ++i) {
      const double a = trans ? A[i + o * lda] : A[o + i * lda];
      s += (long double)a * (long double)x[i * incx];
    }
    double* yo = &y[o * incy];
    *yo = (beta == 0.0) ? (double)(alpha * s) : (double)(alpha * s + (long double)beta * (*yo));
  }
  return 0;
}
