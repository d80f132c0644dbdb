// Four consecutive elements of a row at a time: 16-byte accesses for fp32, 8-byte for the 16-bit types.  The caller
// guarantees the alignment (element index a multiple of 4 from a pointer aligned to 4 elements).
#pragma once
#include "common.cuh"

template <typename T>
__device__ __forceinline__ void row_load4(const T* p, float (&v)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int c = 0; c < 4; ++c) v[c] = to_f32(e[c]);
}
template <>
__device__ __forceinline__ void row_load4<float>(const float* p, float (&v)[4]) {
  const float4 raw = *reinterpret_cast<const float4*>(p);
  v[0] = raw.x; v[1] = raw.y; v[2] = raw.z; v[3] = raw.w;
}
template <typename T>
__device__ __forceinline__ void row_store4(T* p, const float (&v)[4]) {
  uint2 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int c = 0; c < 4; ++c) e[c] = from_f32<T>(v[c]);
  *reinterpret_cast<uint2*>(p) = raw;
}
template <>
__device__ __forceinline__ void row_store4<float>(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
// true when `p` (nullable) is aligned for 4-element accesses of T
template <typename T>
static inline bool row_aligned4(const void* p) { return p == nullptr || (uintptr_t)p % (4 * sizeof(T)) == 0; }
