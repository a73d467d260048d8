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

// channels handled per lane: the widest 16-byte-or-narrower vector that tiles C in 32-lane chunks
template <typename T>
inline int pick_vec(int channels);
template <>
inline int pick_vec<float>(int c) { return c % 128 == 0 ? 4 : (c % 64 == 0 ? 2 : 1); }
template <>
inline int pick_vec<double>(int c) { return c % 64 == 0 ? 2 : 1; }

}  // namespace cmace
