// Shared helpers of the C-ABI library: status codes, error text, launch checks.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/cuda_mace_b200.h"

namespace cmace {

// thread-local message returned by cmace_last_error()
char *error_buffer();

inline int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

inline int check_launch(const char *what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(CMACE_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return CMACE_OK;
}

// l of each of the 16 (l, m) components
__host__ __device__ constexpr int l_of_lm(int lm) { return lm == 0 ? 0 : (lm < 4 ? 1 : (lm < 9 ? 2 : 3)); }

template <typename T, int VEC>
struct Vec;  // VEC scalars moved with one load/store
template <>
struct Vec<float, 4> { using type = float4; };
template <>
struct Vec<float, 2> { using type = float2; };
template <>
struct Vec<float, 1> { using type = float; };
template <>
struct Vec<double, 2> { using type = double2; };
template <>
struct Vec<double, 1> { using type = double; };

// Vector load/store of VEC consecutive scalars; p must be VEC*sizeof(T) aligned.
template <typename T, int VEC>
__device__ __forceinline__ void load_vec(T (&dst)[VEC], const T *p) {
  using V = typename Vec<T, VEC>::type;
  V v = __ldg(reinterpret_cast<const V *>(p));
  const T *s = reinterpret_cast<const T *>(&v);
#pragma unroll
  for (int i = 0; i < VEC; i++) dst[i] = s[i];
}
// streaming variant for data read exactly once (evict-first)
template <typename T, int VEC>
__device__ __forceinline__ void load_vec_stream(T (&dst)[VEC], const T *p) {
  using V = typename Vec<T, VEC>::type;
  V v = __ldcs(reinterpret_cast<const V *>(p));
  const T *s = reinterpret_cast<const T *>(&v);
#pragma unroll
  for (int i = 0; i < VEC; i++) dst[i] = s[i];
}
template <typename T, int VEC>
__device__ __forceinline__ void store_vec(T *p, const T (&src)[VEC]) {
  using V = typename Vec<T, VEC>::type;
  V v;
  T *d = reinterpret_cast<T *>(&v);
#pragma unroll
  for (int i = 0; i < VEC; i++) d[i] = src[i];
  *reinterpret_cast<V *>(p) = v;
}
template <typename T, int VEC>
__device__ __forceinline__ void store_vec_stream(T *p, const T (&src)[VEC]) {
  using V = typename Vec<T, VEC>::type;
  V v;
  T *d = reinterpret_cast<T *>(&v);
#pragma unroll
  for (int i = 0; i < VEC; i++) d[i] = src[i];
  __stcs(reinterpret_cast<V *>(p), v);
}

// ---- two floats in one 64-bit register, handled by one instruction (fma / mul / add / sub .f32x2) --------------
// The kernels that use these are bound by instruction issue, not by the FMA pipe.
__device__ __forceinline__ unsigned long long pack2(float a, float b) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float &a, float &b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ unsigned long long mul2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ unsigned long long sub2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

// channels handled per lane: the widest 16-byte-or-narrower vector that tiles C in 32-lane chunks
template <typename T>
inline int pick_vec(int channels);
template <>
inline int pick_vec<float>(int c) { return c % 128 == 0 ? 4 : (c % 64 == 0 ? 2 : 1); }
template <>
inline int pick_vec<double>(int c) { return c % 64 == 0 ? 2 : 1; }

}  // namespace cmace
