// Kernels around an fp32 residual stream (layer-list models: the residual sum stays in 32 bits while the
// projections run in the activation dtype T):
//   * embed_positions      r = scale * embed[token] + position_table[pos]               (+ copy in T for the next GEMM)
//   * post_norm_residual   r += norm(y) * (offset + w) * layer_scale                    (norm on the SUBLAYER OUTPUT)
//                          and, fused, the NEXT sublayer's input norm: act = norm'(r) * w'   (pre+post-norm designs)
//   * rmsnorm_from_f32     o = norm(r) * (offset + w), selected rows                    (input norm / final norm)
//   * relu_squared, gelu   o = max(x, 0)^2;  o = gelu(x), exact (erf) or tanh form
//   * softcap_to_f32       o = cap * tanh(s x / cap) as fp32 (cap <= 0: s x)            (logits)
// norm = x / sqrt(mean(x^2) + eps) (kind 0, RMS) or (x - mean) / sqrt(mean((x - mean)^2) + eps) (kind 1, layer norm
// without bias; the variance is taken from the deviations in a pass of its own).
// `offset` = 1 for weights stored around zero, 0 for plain weights.  All statistics in fp32.
#include "common.cuh"

namespace {

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_reduce_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_reduce_sum(t);
  __syncthreads();
  return t;
}

template <typename T>
__global__ void embed_positions_kernel(float* __restrict__ r, T* __restrict__ act, const int* __restrict__ tokens,
                                       const int* __restrict__ pos, const T* __restrict__ embed,
                                       const T* __restrict__ ptab, int64_t n, int64_t vocab, int64_t max_pos,
                                       float scale) {
  pdl_prologue();
  const int64_t t = blockIdx.x;
  int64_t tok = tokens[t], p = pos[t];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);        // ids are validated on the host; never read outside
  const bool has_pos = ptab != nullptr;
  p = p < 0 ? 0 : (p >= max_pos ? max_pos - 1 : p);
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
    float v = to_f32(embed[tok * n + i]) * scale;
    if (has_pos) v += to_f32(ptab[p * n + i]);
    r[t * n + i] = v;
    if (act) act[t * n + i] = from_f32<T>(v);
  }
}

// (mean, 1 / sqrt(var + eps)) of row `x` under norm kind `kind`; every thread walks the same elements in every pass
template <typename X>
__device__ __forceinline__ void row_stats(const X* x, int64_t n, int kind, float eps, float* red, float& mean, float& rstd) {
  mean = 0.f;
  if (kind == 1) {
    float s = 0.f;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) s += to_f32(x[i]);
    mean = block_sum(s, red) / (float)n;
  }
  float ss = 0.f;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) { const float v = to_f32(x[i]) - mean; ss = fmaf(v, v, ss); }
  rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)n + eps);
}

template <typename T>
__global__ void post_norm_residual_kernel(float* __restrict__ r, T* __restrict__ act, const T* __restrict__ y,
                                          const T* __restrict__ w, const T* __restrict__ ls, const T* __restrict__ wn,
                                          int64_t n, int64_t ys, float eps, float offset, int kind, int next_kind) {
  pdl_prologue();
  __shared__ float red[32];
  const int64_t t = blockIdx.x;
  const T* yr = y + t * ys;
  float* rr = r + t * n;
  float mean, rstd;
  row_stats(yr, n, kind, eps, red, mean, rstd);
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
    float d = (to_f32(yr[i]) - mean) * rstd * (offset + to_f32(w[i]));
    if (ls) d *= to_f32(ls[i]);
    const float v = rr[i] + d;
    rr[i] = v;
    if (act && !wn) act[t * n + i] = from_f32<T>(v);
  }
  if (act && wn) {                       // the next sublayer's input norm of the row this thread block just wrote
    row_stats(rr, n, next_kind, eps, red, mean, rstd);
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x)
      act[t * n + i] = from_f32<T>((rr[i] - mean) * rstd * (offset + to_f32(wn[i])));
  }
}

// Register-resident version for rows of up to NV * 1024 elements (n a multiple of 4, 16-byte aligned rows): every
// thread keeps its float4 slices of y and of the residual row in registers, so each is read once, and the four
// statistics (mean and deviation sums of y, then of the updated row) are block reductions over registers.  Same
// arithmetic as the kernel above.
template <int N> struct RawVec;
template <> struct RawVec<4> { using type = uint2; };       // four 16-bit elements
template <> struct RawVec<8> { using type = uint2; };
template <> struct RawVec<16> { using type = uint4; };      // four 32-bit elements

template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&v)[4]) {
  using R = typename RawVec<4 * sizeof(T)>::type;
  const R raw = *reinterpret_cast<const R*>(p);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int c = 0; c < 4; ++c) v[c] = to_f32(e[c]);
}
template <typename T>
__device__ __forceinline__ void store4(T* p, const float (&v)[4]) {
  using R = typename RawVec<4 * sizeof(T)>::type;
  R raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int c = 0; c < 4; ++c) e[c] = from_f32<T>(v[c]);
  *reinterpret_cast<R*>(p) = raw;
}

template <int NV>
__device__ __forceinline__ void reg_stats(const float (&v)[NV][4], int64_t n, int kind, float eps, float* red,
                                          float& mean, float& rstd) {
  mean = 0.f;
  if (kind == 1) {
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j)
      if ((int64_t)(j * 256 + threadIdx.x) * 4 < n) s += (v[j][0] + v[j][1]) + (v[j][2] + v[j][3]);
    mean = block_sum(s, red) / (float)n;
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < NV; ++j)
    if ((int64_t)(j * 256 + threadIdx.x) * 4 < n) {
#pragma unroll
      for (int c = 0; c < 4; ++c) { const float d = v[j][c] - mean; ss = fmaf(d, d, ss); }
    }
  rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)n + eps);
}

template <typename T, int NV>
__global__ void __launch_bounds__(256) post_norm_residual_reg_kernel(float* __restrict__ r, T* __restrict__ act,
                                                                     const T* __restrict__ y, const T* __restrict__ w,
                                                                     const T* __restrict__ ls, const T* __restrict__ wn,
                                                                     int64_t n, int64_t ys, float eps, float offset,
                                                                     int kind, int next_kind) {
  pdl_prologue();
  __shared__ float red[32];
  const int64_t t = blockIdx.x;
  const T* yr = y + t * ys;
  float* rr = r + t * n;
  float yv[NV][4], rv[NV][4];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int64_t i = (int64_t)(j * 256 + threadIdx.x) * 4;
    if (i < n) { load4(yr + i, yv[j]); load4(rr + i, rv[j]); }
  }
  float mean, rstd;
  reg_stats<NV>(yv, n, kind, eps, red, mean, rstd);
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int64_t i = (int64_t)(j * 256 + threadIdx.x) * 4;
    if (i >= n) continue;
    float wv[4], lv[4] = {1.f, 1.f, 1.f, 1.f};
    load4(w + i, wv);
    if (ls) load4(ls + i, lv);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      float d = (yv[j][c] - mean) * rstd * (offset + wv[c]);
      if (ls) d *= lv[c];
      rv[j][c] += d;
    }
    store4(rr + i, rv[j]);
    if (act && !wn) store4(act + t * n + i, rv[j]);
  }
  if (act && wn) {
    reg_stats<NV>(rv, n, next_kind, eps, red, mean, rstd);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int64_t i = (int64_t)(j * 256 + threadIdx.x) * 4;
      if (i >= n) continue;
      float wv[4], o[4];
      load4(wn + i, wv);
#pragma unroll
      for (int c = 0; c < 4; ++c) o[c] = (rv[j][c] - mean) * rstd * (offset + wv[c]);
      store4(act + t * n + i, o);
    }
  }
}

template <typename T>
__global__ void rmsnorm_from_f32_kernel(T* __restrict__ o, const float* __restrict__ r, const int* __restrict__ rows,
                                        const T* __restrict__ w, int64_t n, float eps, float offset, int kind) {
  pdl_prologue();
  __shared__ float red[32];
  const int64_t src = rows ? rows[blockIdx.x] : blockIdx.x;
  const float* x = r + src * n;
  float mean, rstd;
  row_stats(x, n, kind, eps, red, mean, rstd);
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x)
    o[(int64_t)blockIdx.x * n + i] = from_f32<T>((x[i] - mean) * rstd * (offset + to_f32(w[i])));
}

__device__ __forceinline__ float gelu_f(float v, int tanh_form) {
  return tanh_form ? 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)))
                   : 0.5f * v * (1.0f + erff(v * 0.7071067811865476f));
}

// 16-byte accesses over the aligned body (`vec` = 1), scalars over the tail or everything
template <typename T>
__global__ void gelu_kernel(T* __restrict__ o, const T* __restrict__ x, int64_t total, int tanh_form, int vec) {
  pdl_prologue();
  constexpr int VEC = 16 / (int)sizeof(T);
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, step = (int64_t)gridDim.x * blockDim.x;
  const int64_t chunks = vec ? total / VEC : 0;
  for (int64_t c = tid; c < chunks; c += step) {
    const uint4 raw = ldg_stream_128(x + c * VEC);
    const T* e = reinterpret_cast<const T*>(&raw);
    uint4 res;
    T* r = reinterpret_cast<T*>(&res);
#pragma unroll
    for (int j = 0; j < VEC; ++j) r[j] = from_f32<T>(gelu_f(to_f32(e[j]), tanh_form));
    stg_128(o + c * VEC, res);
  }
  for (int64_t i = chunks * VEC + tid; i < total; i += step) o[i] = from_f32<T>(gelu_f(to_f32(x[i]), tanh_form));
}

template <typename T>
__global__ void softcap_to_f32_kernel(float* __restrict__ o, const T* __restrict__ x, int64_t total, float cap,
                                      float scale) {
  pdl_prologue();
  const float inv = cap > 0.f ? 1.0f / cap : 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = to_f32(x[i]) * scale;
    o[i] = cap > 0.f ? cap * tanhf(v * inv) : v;
  }
}

template <typename T>
__global__ void relu_squared_kernel(T* __restrict__ o, const T* __restrict__ x, int64_t total) {
  pdl_prologue();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = fmaxf(to_f32(x[i]), 0.f);
    o[i] = from_f32<T>(v * v);
  }
}

template <typename T>
void launch_post_norm(float* r, T* act, const T* y, const T* w, const T* ls, const T* wn, int64_t rows, int64_t n,
                      int64_t ys, float eps, float offset, int kind, int next_kind, cudaStream_t st) {
  constexpr uintptr_t A = 4 * sizeof(T);
  auto al = [](const void* p, uintptr_t a) { return p == nullptr || (uintptr_t)p % a == 0; };
  const bool fast = n % 4 == 0 && n <= 8 * 1024 && ys % 4 == 0 && al(r, 16) && al(act, A) && al(y, A) && al(w, A) &&
                    al(ls, A) && al(wn, A);
  const dim3 grid((unsigned)rows), block(256);
  if (fast && n <= 1024)
    b2l_launch(post_norm_residual_reg_kernel<T, 1>, grid, block, (size_t)0, st, r, act, y, w, ls, wn, n, ys, eps, offset, kind, next_kind);
  else if (fast && n <= 2048)
    b2l_launch(post_norm_residual_reg_kernel<T, 2>, grid, block, (size_t)0, st, r, act, y, w, ls, wn, n, ys, eps, offset, kind, next_kind);
  else if (fast && n <= 4096)
    b2l_launch(post_norm_residual_reg_kernel<T, 4>, grid, block, (size_t)0, st, r, act, y, w, ls, wn, n, ys, eps, offset, kind, next_kind);
  else if (fast)
    b2l_launch(post_norm_residual_reg_kernel<T, 8>, grid, block, (size_t)0, st, r, act, y, w, ls, wn, n, ys, eps, offset, kind, next_kind);
  else
    b2l_launch(post_norm_residual_kernel<T>, grid, block, (size_t)0, st, r, act, y, w, ls, wn, n, ys, eps, offset, kind, next_kind);
}

}  // namespace

extern "C" int b2l_embed_positions(void* residual_f32, void* act, const void* tokens_i32, const void* pos_i32,
                                   const void* embed, const void* pos_table, int64_t rows, int64_t n, int64_t vocab,
                                   int64_t max_pos, float scale, int dtype, void* stream) {
  B2L_REQUIRE(residual_f32 && tokens_i32 && pos_i32 && embed, "embed_positions: null pointer");
  B2L_REQUIRE(rows >= 0 && n > 0 && vocab > 0, "embed_positions: bad shape");
  if (rows == 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  B2L_DISPATCH_FLOAT(dtype, "embed_positions", {
    b2l_launch(embed_positions_kernel<T>, dim3((unsigned)rows), dim3(256), (size_t)0, st, (float*)residual_f32, (T*)act,
               (const int*)tokens_i32, (const int*)pos_i32, (const T*)embed, (const T*)pos_table, n, vocab, max_pos, scale);
  });
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

extern "C" int b2l_post_norm_residual(void* residual_f32, void* act, const void* y, const void* weight,
                                      const void* layer_scale, const void* next_weight, int64_t rows, int64_t n,
                                      int64_t y_row_stride, float eps, float weight_offset, int norm_kind,
                                      int next_norm_kind, int dtype, void* stream) {
  B2L_REQUIRE((norm_kind == 0 || norm_kind == 1) && (next_norm_kind == 0 || next_norm_kind == 1),
              "post_norm_residual: norm kind %d / %d", norm_kind, next_norm_kind);
  B2L_REQUIRE(residual_f32 && y && weight, "post_norm_residual: null pointer");
  B2L_REQUIRE(rows >= 0 && n > 0, "post_norm_residual: bad shape");
  if (rows == 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  B2L_DISPATCH_FLOAT(dtype, "post_norm_residual", {
    launch_post_norm<T>((float*)residual_f32, (T*)act, (const T*)y, (const T*)weight, (const T*)layer_scale,
                        (const T*)next_weight, rows, n, y_row_stride, eps, weight_offset, norm_kind, next_norm_kind, st);
  });
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

extern "C" int b2l_rmsnorm_from_f32(void* out, const void* residual_f32, const void* rows_i32, const void* weight,
                                    int64_t rows, int64_t n, float eps, float weight_offset, int norm_kind, int dtype,
                                    void* stream) {
  B2L_REQUIRE(out && residual_f32 && weight, "rmsnorm_from_f32: null pointer");
  B2L_REQUIRE(norm_kind == 0 || norm_kind == 1, "rmsnorm_from_f32: norm kind %d", norm_kind);
  B2L_REQUIRE(rows >= 0 && n > 0, "rmsnorm_from_f32: bad shape");
  if (rows == 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  B2L_DISPATCH_FLOAT(dtype, "rmsnorm_from_f32", {
    b2l_launch(rmsnorm_from_f32_kernel<T>, dim3((unsigned)rows), dim3(256), (size_t)0, st, (T*)out,
               (const float*)residual_f32, (const int*)rows_i32, (const T*)weight, n, eps, weight_offset, norm_kind);
  });
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

extern "C" int b2l_relu_squared(void* out, const void* x, int64_t total, int dtype, void* stream) {
  B2L_REQUIRE(out && x, "relu_squared: null pointer");
  if (total <= 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned grid = (unsigned)(cdiv64(total, 256) < 148 * 16 ? cdiv64(total, 256) : 148 * 16);
  B2L_DISPATCH_FLOAT(dtype, "relu_squared", {
    b2l_launch(relu_squared_kernel<T>, dim3(grid), dim3(256), (size_t)0, st, (T*)out, (const T*)x, total);
  });
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

extern "C" int b2l_gelu(void* out, const void* x, int64_t total, int tanh_form, int dtype, void* stream) {
  B2L_REQUIRE(out && x, "gelu: null pointer");
  if (total <= 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int vec = ((uintptr_t)out % 16 == 0 && (uintptr_t)x % 16 == 0) ? 1 : 0;
  const int64_t work = vec ? cdiv64(total, 4) : total;
  const unsigned grid = (unsigned)(cdiv64(work, 256) < 148 * 16 ? cdiv64(work, 256) : 148 * 16);
  B2L_DISPATCH_FLOAT(dtype, "gelu", {
    b2l_launch(gelu_kernel<T>, dim3(grid), dim3(256), (size_t)0, st, (T*)out, (const T*)x, total, tanh_form, vec);
  });
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

extern "C" int b2l_softcap_to_f32(void* out_f32, const void* x, int64_t total, float cap, float scale, int dtype,
                                  void* stream) {
  B2L_REQUIRE(out_f32 && x, "softcap_to_f32: null pointer");
  if (total <= 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned grid = (unsigned)(cdiv64(total, 256) < 148 * 16 ? cdiv64(total, 256) : 148 * 16);
  B2L_DISPATCH_FLOAT(dtype, "softcap_to_f32", {
    b2l_launch(softcap_to_f32_kernel<T>, dim3(grid), dim3(256), (size_t)0, st, (float*)out_f32, (const T*)x, total, cap,
               scale);
  });
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}
