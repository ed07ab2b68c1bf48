// A caller written against the reference's public C++ header (the names and argument
// lists of Library_scheduler/include/PARALiA.hpp:33-72), the way its runners use it
// (Benchmarking/CuCuBLAS/src/PARALia/dgemm_runner.cpp:80-151): plain host pointers, no
// location arguments, an optional predefined controller, results read from the returned
// controller. It checks every routine against naive loops on small problems and prints one
// line per routine; exit status 0 means all of them agreed.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "PARALiA.hpp"

namespace {

double next_uniform(unsigned long long* state) {   // splitmix64 -> [-1, 1)
  unsigned long long z = (*state += 0x9E3779B97F4A7C15ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return (double)(z >> 11) * (2.0 / 9007199254740992.0) - 1.0;
}

template <typename T>
std::vector<T> random_vec(size_t n, unsigned long long seed) {
  std::vector<T> v(n);
  for (size_t i = 0; i < n; ++i) v[i] = (T)next_uniform(&seed);
  return v;
}

template <typename T>
double rel_err(const std::vector<T>& got, const std::vector<double>& want) {
  double num = 0.0, den = 0.0;
  for (size_t i = 0; i < got.size(); ++i) {
    const double d = (double)got[i] - want[i];
    num += d * d;
    den += want[i] * want[i];
  }
  return den > 0.0 ? std::sqrt(num / den) : std::sqrt(num);
}

// C <- alpha*op(A)*op(B) + beta*C in FP64, column-major
template <typename T>
std::vector<double> naive_gemm(char ta, char tb, long M, long N, long K, double alpha,
                               const std::vector<T>& A, long ldA, const std::vector<T>& B, long ldB,
                               double beta, const std::vector<T>& C, long ldC) {
  std::vector<double> out((size_t)ldC * N);
  for (long j = 0; j < N; ++j)
    for (long i = 0; i < M; ++i) {
      double s = 0.0;
      for (long k = 0; k < K; ++k) {
        const double a = ta == 'N' ? A[i + k * ldA] : A[k + i * ldA];
        const double b = tb == 'N' ? B[k + j * ldB] : B[j + k * ldB];
        s += a * b;
      }
      out[i + j * ldC] = alpha * s + beta * (double)C[i + j * ldC];
    }
  return out;
}

int failures = 0;

void report(const char* what, double err, double bound, ATC_p ctl) {
  const bool ok = ctl != NULL && err <= bound;
  std::printf("%-28s err %.3e (bound %.3e) T=%ld units=%d %s\n", what, err, bound,
              ctl ? ctl->T : -1L, ctl ? ctl->active_unit_num : -1, ok ? "ok" : "FAILED");
  if (!ok) ++failures;
  delete ctl;   // the caller owns the returned controller (dgemm.cpp:691-693)
}

}  // namespace

int main() {
  const long M = 300, N = 260, K = 280;
  const double eps64 = std::ldexp(1.0, -52), eps32 = std::ldexp(1.0, -23);

  {  // DGEMM, autotuned, then with a predefined controller (T and unit list given)
    std::vector<double> A = random_vec<double>(M * K, 42), B = random_vec<double>(K * N, 43),
                        C = random_vec<double>(M * N, 44);
    std::vector<double> want = naive_gemm('N', 'N', M, N, K, 1.23, A, M, B, K, 0.9876, C, M);
    std::vector<double> C1 = C;
    ATC_p r = PARALiADgemm('N', 'N', M, N, K, 1.23, A.data(), M, B.data(), K, 0.9876, C1.data(), M);
    report("PARALiADgemm NN", rel_err(C1, want), 8 * K * eps64, r);

    ATC predef;
    predef.T = 128;
    predef.active_unit_num = 1;
    predef.active_unit_id_list[0] = 0;
    std::vector<double> At = random_vec<double>(K * M, 45);   // stored K x M, used transposed
    std::vector<double> want_t = naive_gemm('T', 'N', M, N, K, -0.5, At, K, B, K, 0.0, C, M);
    std::vector<double> C2 = C;
    r = PARALiADgemmControled('T', 'N', M, N, K, -0.5, At.data(), K, B.data(), K, 0.0, C2.data(), M,
                              &predef);
    const bool kept = r && r->T == 128 && r->active_unit_num == 1;
    report("PARALiADgemmControled TN", kept ? rel_err(C2, want_t) : 1.0, 8 * K * eps64, r);
  }
  {  // SGEMM against the FP64 product of the FP32 inputs
    std::vector<float> A = random_vec<float>(M * K, 52), B = random_vec<float>(N * K, 53),
                       C = random_vec<float>(M * N, 54);
    std::vector<double> want = naive_gemm('N', 'T', M, N, K, 1.0, A, M, B, N, 0.5, C, M);
    ATC_p r = PARALiASgemm('N', 'T', M, N, K, 1.0f, A.data(), M, B.data(), N, 0.5f, C.data(), M);
    report("PARALiASgemm NT", rel_err(C, want), 4 * K * eps32, r);
  }
  {  // DGEMV, both transposes
    std::vector<double> A = random_vec<double>(M * N, 62), x = random_vec<double>(N, 63),
                        y = random_vec<double>(M, 64);
    std::vector<double> want(M), want_t(N);
    for (long i = 0; i < M; ++i) {
      double s = 0.0;
      for (long j = 0; j < N; ++j) s += A[i + j * M] * x[j];
      want[i] = 1.5 * s - 0.25 * y[i];
    }
    std::vector<double> y1 = y;
    ATC_p r = PARALiADgemv('N', M, N, 1.5, A.data(), M, x.data(), 1, -0.25, y1.data(), 1);
    report("PARALiADgemv N", rel_err(y1, want), 8 * N * eps64, r);
    for (long j = 0; j < N; ++j) {
      double s = 0.0;
      for (long i = 0; i < M; ++i) s += A[i + j * M] * y[i];
      want_t[j] = 1.5 * s - 0.25 * x[j];
    }
    std::vector<double> x1 = x;
    r = PARALiADgemv('T', M, N, 1.5, A.data(), M, y.data(), 1, -0.25, x1.data(), 1);
    report("PARALiADgemv T", rel_err(x1, want_t), 8 * M * eps64, r);
  }
  {  // DAXPY (exact: one fused multiply-add per element) and DDOT (*result += x.y)
    const long n = 100003;
    std::vector<double> x = random_vec<double>(n, 72), y = random_vec<double>(n, 73);
    std::vector<double> want(n);
    double dot = 0.0, mag = 0.0;
    for (long i = 0; i < n; ++i) {
      want[i] = std::fma(-0.5, x[i], y[i]);
      dot += x[i] * y[i];
      mag += std::fabs(x[i] * y[i]);
    }
    double result = 2.0;
    ATC_p r = PARALiADdot(n, x.data(), 1, y.data(), 1, &result);
    report("PARALiADdot", std::fabs(result - (2.0 + dot)), n * eps64 * mag, r);
    r = PARALiADaxpy(n, -0.5, x.data(), 1, y.data(), 1);
    report("PARALiADaxpy", rel_err(y, want), 0.0, r);
  }
  for (short d = 0; d < (short)PARALiA_device_count(); ++d) PARALiADevCacheFree(d);   // as the reference's runner does
  std::printf("%s\n", failures ? "MISMATCH" : "ALL OK");
  return failures ? 1 : 0;
}
