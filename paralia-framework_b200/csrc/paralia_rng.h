// Counter-based input generator shared by host and device code: element i of a buffer is
// a pure function of (seed, i), so a buffer filled on the host and one filled on a GPU
// hold the same bits. It takes the place of the reference's CoCoVecInit(ptr, n, seed, loc)
// (Benchmarking/CuCuBLAS/src/PARALia/dgemm_runner.cpp:64-66), whose generator lives in
// the backend that is not part of the reference checkout.
#pragma once
#include <stdint.h>
#include <math.h>

#if defined(__CUDACC__)
#define PARALIA_HD __host__ __device__ __forceinline__
#else
#define PARALIA_HD static inline
#endif

// splitmix64 finaliser over seed + golden-ratio stride: passes through every 64-bit state.
PARALIA_HD uint64_t paralia_mix64(uint64_t seed, uint64_t idx) {
  uint64_t z = seed + (idx + 1) * 0x9E3779B97F4A7C15ULL;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  return z ^ (z >> 31);
}

// uniform on [-1, 1): 53 random bits scaled by 2^-52, minus one. Every step is exact in
// binary64, so host and device agree bit for bit.
PARALIA_HD double paralia_uniform_f64(uint64_t seed, uint64_t idx) {
  return (double)(paralia_mix64(seed, idx) >> 11) * (1.0 / 4503599627370496.0) - 1.0;
}

// uniform on [-1, 1) with 24 random bits, exact in binary32.
PARALIA_HD float paralia_uniform_f32(uint64_t seed, uint64_t idx) {
  return (float)(paralia_mix64(seed, idx) >> 40) * (1.0f / 8388608.0f) - 1.0f;
}

// normal(0,1) by Box-Muller in binary64 from two independent uniforms on (0,1].
// log/cos are library functions, so host and device may differ in the last place; a
// buffer is always produced by one side and copied, never generated twice.
PARALIA_HD double paralia_normal_f64(uint64_t seed, uint64_t idx) {
  const uint64_t a = paralia_mix64(seed, 2 * idx);
  const uint64_t b = paralia_mix64(seed ^ 0xD1B54A32D192ED03ULL, 2 * idx + 1);
  const double u1 = ((double)(a >> 11) + 1.0) * (1.0 / 9007199254740992.0);  // (0,1]
  const double u2 = (double)(b >> 11) * (1.0 / 9007199254740992.0);          // [0,1)
  return sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925286766559 * u2);
}
