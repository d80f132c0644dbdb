// Rotary positions with per-pair frequencies given as a table (frequency-interpolated variants compute the table on
// the host), and the per-token preparation of attention layers that norm each head on its own:
//   * rope_table_freqs         cos_sin[t] = [mag * cos(pos[t] * f_i), i < rot_dims / 2 | mag * sin(pos[t] * f_i)],
//                              frequencies and angles in fp64 (an fp32 angle of a thousand radians is already off by
//                              6e-5), the table in fp32; once per step
//   * head_norm_rope_prepare   per token of a fused [q | k | v] projection row: every q head and every k head is
//                              RMS-normed over its own head_dim entries with ONE weight [head_dim] shared by the heads
//                              (nullable = no norm), then its first rot_dims entries are rotated (pairing 0: entries
//                              2i and 2i+1; pairing 1: entries i and i + rot_dims / 2); q is updated in place, k and v
//                              go to pool row kv_rows[t] = [k heads | v heads].
// Statistics and the rotation are fp32; one rounding to T at the end.
#include "common.cuh"
#include "rowvec.cuh"

namespace {

__global__ void rope_table_freqs_kernel(float* __restrict__ out, const int* __restrict__ pos,
                                        const double* __restrict__ freqs, int64_t total, int half, float mag) {
  pdl_prologue();
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = idx / half;
    const int i = (int)(idx - t * half);
    const double a = (double)pos[t] * freqs[i];
    double sn, cs;
    sincos(a, &sn, &cs);
    out[t * 2 * half + i] = (float)(cs * (double)mag);
    out[t * 2 * half + half + i] = (float)(sn * (double)mag);
  }
}

constexpr int kPrepWarps = 4;

// One CTA per token, one warp per head at a time.  A head is staged (normed, fp32) in the warp's shared-memory row so
// that either pairing finds its partner there.
template <typename T>
__global__ void __launch_bounds__(kPrepWarps * 32) head_norm_rope_prepare_kernel(
    T* __restrict__ qkv, int64_t qkv_stride, T* __restrict__ pool, int64_t pool_stride, const int* __restrict__ kv_rows,
    const float* __restrict__ cos_sin, const T* __restrict__ q_w, const T* __restrict__ k_w, int H, int G, int D,
    int Dv, int rot_dims, int pairing, float eps) {
  pdl_prologue();
  extern __shared__ float stage[];                 // [kPrepWarps][D]
  const int64_t t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* row = stage + warp * D;
  T* src = qkv + t * qkv_stride;
  T* dst_pool = pool + (int64_t)kv_rows[t] * pool_stride;
  const int half = rot_dims / 2;
  const float* cs = cos_sin ? cos_sin + t * rot_dims : nullptr;
  for (int h = warp; h < H + G; h += kPrepWarps) {
    const bool is_q = h < H;
    const T* in = src + (int64_t)h * D;            // q heads, then k heads, are consecutive in the row
    const T* w = is_q ? q_w : k_w;
    T* out = is_q ? src + (int64_t)h * D : dst_pool + (int64_t)(h - H) * D;
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) { const float v = to_f32(in[d]); row[d] = v; ss = fmaf(v, v, ss); }
    float rstd = 1.f;
    if (w) rstd = 1.0f / sqrtf(warp_reduce_sum(ss) / (float)D + eps);
    __syncwarp();
    if (w)
      for (int d = lane; d < D; d += 32) row[d] = row[d] * rstd * to_f32(w[d]);
    __syncwarp();
    for (int d = lane; d < D; d += 32) {
      float v = row[d];
      if (d < rot_dims && cs) {
        int i, partner;
        bool first;
        if (pairing == 0) { i = d >> 1; first = (d & 1) == 0; partner = first ? d + 1 : d - 1; }
        else { first = d < half; i = first ? d : d - half; partner = first ? d + half : d - half; }
        const float c = cs[i], s = cs[half + i], o = row[partner];
        v = first ? v * c - o * s : v * c + o * s;
      }
      out[d] = from_f32<T>(v);
    }
    __syncwarp();                                  // the row is reused by the warp's next head
  }
  const T* vin = src + (int64_t)(H + G) * D;
  T* vout = dst_pool + (int64_t)G * D;
  for (int i = threadIdx.x; i < G * Dv; i += blockDim.x) vout[i] = vin[i];
}

// The same for the neighbour pairing with 4 elements per access: head_dim a multiple of 4 and at most C * 128, every
// row and head start aligned to 4 elements.  A lane's 4 elements hold two whole pairs, so the head never leaves the
// registers: one read and one write per element.
constexpr int kVecWarps = 8;

template <typename T, int C>
__global__ void __launch_bounds__(kVecWarps * 32) head_norm_rope_prepare_vec_kernel(
    T* __restrict__ qkv, int64_t qkv_stride, T* __restrict__ pool, int64_t pool_stride, const int* __restrict__ kv_rows,
    const float* __restrict__ cos_sin, const T* __restrict__ q_w, const T* __restrict__ k_w, int H, int G, int D,
    int Dv, int rot_dims, float eps) {
  pdl_prologue();
  const int64_t t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  T* src = qkv + t * qkv_stride;
  T* dst_pool = pool + (int64_t)kv_rows[t] * pool_stride;
  const int half = rot_dims / 2;
  const float* cs = cos_sin ? cos_sin + t * rot_dims : nullptr;
  for (int h = warp; h < H + G; h += kVecWarps) {
    const bool is_q = h < H;
    const T* in = src + (int64_t)h * D;
    const T* w = is_q ? q_w : k_w;
    T* out = is_q ? src + (int64_t)h * D : dst_pool + (int64_t)(h - H) * D;
    float v[C][4];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < C; ++c) {
      const int d = (c * 32 + lane) * 4;
      v[c][0] = v[c][1] = v[c][2] = v[c][3] = 0.f;
      if (d < D) row_load4(in + d, v[c]);
#pragma unroll
      for (int e = 0; e < 4; ++e) ss = fmaf(v[c][e], v[c][e], ss);
    }
    float rstd = 1.f;
    if (w) rstd = 1.0f / sqrtf(warp_reduce_sum(ss) / (float)D + eps);
#pragma unroll
    for (int c = 0; c < C; ++c) {
      const int d = (c * 32 + lane) * 4;
      if (d >= D) continue;
      if (w) {
        float g[4];
        row_load4(w + d, g);
#pragma unroll
        for (int e = 0; e < 4; ++e) v[c][e] = v[c][e] * rstd * g[e];
      }
#pragma unroll
      for (int pr = 0; pr < 2; ++pr) {
        const int dd = d + 2 * pr;
        if (cs && dd < rot_dims) {
          const float co = cs[dd >> 1], si = cs[half + (dd >> 1)];
          const float a = v[c][2 * pr], b = v[c][2 * pr + 1];
          v[c][2 * pr] = a * co - b * si;
          v[c][2 * pr + 1] = b * co + a * si;
        }
      }
      row_store4(out + d, v[c]);
    }
  }
  const T* vin = src + (int64_t)(H + G) * D;
  T* vout = dst_pool + (int64_t)G * D;
  if ((G * Dv) % 4 == 0) {
    for (int i = threadIdx.x * 4; i < G * Dv; i += blockDim.x * 4) {
      float x[4];
      row_load4(vin + i, x);
      row_store4(vout + i, x);
    }
  } else {
    for (int i = threadIdx.x; i < G * Dv; i += blockDim.x) vout[i] = vin[i];
  }
}

}  // namespace

extern "C" int b2l_rope_table_freqs(void* cos_sin_f32, const void* pos_i32, const void* freqs_f64, int64_t tokens,
                                    int rot_dims, float magnitude, void* stream) {
  B2L_REQUIRE(cos_sin_f32 && pos_i32 && freqs_f64, "rope_table_freqs: null pointer");
  B2L_REQUIRE(rot_dims > 0 && rot_dims % 2 == 0, "rope_table_freqs: %d rotated entries", rot_dims);
  if (tokens <= 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t total = tokens * (rot_dims / 2);
  const unsigned grid = (unsigned)(cdiv64(total, 256) < 148 * 16 ? cdiv64(total, 256) : 148 * 16);
  b2l_launch(rope_table_freqs_kernel, dim3(grid), dim3(256), (size_t)0, st, (float*)cos_sin_f32, (const int*)pos_i32,
             (const double*)freqs_f64, total, rot_dims / 2, magnitude);
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

extern "C" int b2l_head_norm_rope_prepare(void* qkv, int64_t qkv_row_stride, void* kv_pool, int64_t kv_row_stride,
                                          const void* kv_rows_i32, const void* cos_sin_f32, const void* q_norm_weight,
                                          const void* k_norm_weight, int64_t tokens, int heads, int kv_heads,
                                          int head_dim, int v_head_dim, int rot_dims, int pairing, float eps, int dtype,
                                          void* stream) {
  B2L_REQUIRE(qkv && kv_pool && kv_rows_i32, "head_norm_rope_prepare: null pointer");
  B2L_REQUIRE(heads > 0 && kv_heads > 0 && head_dim > 0 && v_head_dim > 0, "head_norm_rope_prepare: bad shape");
  B2L_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= head_dim && (rot_dims == 0 || cos_sin_f32),
              "head_norm_rope_prepare: %d rotated entries of %d", rot_dims, head_dim);
  B2L_REQUIRE(pairing == 0 || pairing == 1, "head_norm_rope_prepare: pairing %d", pairing);
  if (tokens <= 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t smem = (size_t)kPrepWarps * head_dim * sizeof(float);
  B2L_REQUIRE(smem <= 48 * 1024, "head_norm_rope_prepare: head_dim %d too large", head_dim);
#define B2L_PREP_VEC(CV)                                                                                            \
  b2l_launch(head_norm_rope_prepare_vec_kernel<T, CV>, dim3((unsigned)tokens), dim3(kVecWarps * 32), (size_t)0, st, \
             (T*)qkv, qkv_row_stride, (T*)kv_pool, kv_row_stride, (const int*)kv_rows_i32,                          \
             (const float*)cos_sin_f32, (const T*)q_norm_weight, (const T*)k_norm_weight, heads, kv_heads, head_dim, \
             v_head_dim, rot_dims, eps)
  B2L_DISPATCH_FLOAT(dtype, "head_norm_rope_prepare", {
    const bool vec = pairing == 0 && head_dim % 4 == 0 && head_dim <= 256 && qkv_row_stride % 4 == 0 &&
                     kv_row_stride % 4 == 0 && row_aligned4<T>(qkv) && row_aligned4<T>(kv_pool) &&
                     row_aligned4<T>(q_norm_weight) && row_aligned4<T>(k_norm_weight) &&
                     ((kv_heads * v_head_dim) % 4 != 0 || ((int64_t)(heads + kv_heads) * head_dim) % 4 == 0);
    if (vec && head_dim <= 128) { B2L_PREP_VEC(1); B2L_LAUNCH_CHECK(); return B2L_OK; }
    if (vec) { B2L_PREP_VEC(2); B2L_LAUNCH_CHECK(); return B2L_OK; }
    b2l_launch(head_norm_rope_prepare_kernel<T>, dim3((unsigned)tokens), dim3(kPrepWarps * 32), smem, st, (T*)qkv,
               qkv_row_stride, (T*)kv_pool, kv_row_stride, (const int*)kv_rows_i32, (const float*)cos_sin_f32,
               (const T*)q_norm_weight, (const T*)k_norm_weight, heads, kv_heads, head_dim, v_head_dim, rot_dims,
               pairing, eps);
  });
#undef B2L_PREP_VEC
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}
