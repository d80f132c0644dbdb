// Kernels for layer-list models whose layers are PARALLEL blocks around an fp32 residual stream that keeps every
// layer's result (a depth-weighted average feeds the next layer):
//   * embed_rmsnorm         X_0[t] = unit_rms(scale * embed[token]) * (offset + w)                        (fp32)
//   * depth_mix_norms       x = sum_j c_j X_j over the kept results (or x = X_last when c == NULL), written as the next
//                           level of the stack, and, from the same statistic, the two input norms of a parallel block:
//                           h1 = unit_rms(x) * (offset + w1), h2 = unit_rms(x) * (offset + w2)            (in T)
//   * branch_sum_residual   x += s * a' + s_b * b' + c, where a' = unit_rms(a) * wa when wa is given, else a (b' likewise;
//                           b and c optional): a mixer with one or two normed branches plus a feed-forward output
//                           joining the residual in one pass; optional copy of the new x in T for the next GEMM
//   * gelu_mul_gather       o[t, d] = gelu_tanh(z[t, d]) * table[token[t], col0 + d]       (per-layer token input)
// unit_rms(v) = v / sqrt(mean(v^2) + eps).  All statistics, sums and the stack itself are fp32.
#include "common.cuh"
#include "rowvec.cuh"

namespace {

__device__ __forceinline__ float block_sum_ps(float v, float* red) {
  v = warp_reduce_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_reduce_sum(t);
  __syncthreads();
  return t;
}

__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void embed_rmsnorm_kernel(float* __restrict__ r, const int* __restrict__ tokens, const T* __restrict__ embed,
                                     const T* __restrict__ w, int64_t n, int64_t vocab, float eps, float offset,
                                     float scale, int vec) {
  pdl_prologue();
  __shared__ float red[32];
  const int64_t t = blockIdx.x;
  int64_t tok = tokens[t];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);        // ids are validated on the host; never read outside
  const T* e = embed + tok * n;
  float ss = 0.f;
  if (vec) {                                   // 4 elements per access; the second pass finds the row in L1
    for (int64_t i = (int64_t)threadIdx.x * 4; i < n; i += (int64_t)blockDim.x * 4) {
      float v[4];
      row_load4(e + i, v);
#pragma unroll
      for (int c = 0; c < 4; ++c) { v[c] *= scale; ss = fmaf(v[c], v[c], ss); }
    }
    const float rstd = 1.0f / sqrtf(block_sum_ps(ss, red) / (float)n + eps);
    for (int64_t i = (int64_t)threadIdx.x * 4; i < n; i += (int64_t)blockDim.x * 4) {
      float v[4], g[4] = {0.f, 0.f, 0.f, 0.f};
      row_load4(e + i, v);
      if (w) row_load4(w + i, g);
#pragma unroll
      for (int c = 0; c < 4; ++c) v[c] = v[c] * scale * rstd * (w ? offset + g[c] : 1.0f);
      row_store4(r + t * n + i, v);
    }
    return;
  }
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) { const float v = to_f32(e[i]) * scale; ss = fmaf(v, v, ss); }
  const float rstd = 1.0f / sqrtf(block_sum_ps(ss, red) / (float)n + eps);
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x)
    r[t * n + i] = to_f32(e[i]) * scale * rstd * (w ? offset + to_f32(w[i]) : 1.0f);
}

// One CTA per token.  NV > 0: the row fits NV float4 per thread (n % 4 == 0, n <= NV * 1024), the mixed row stays in
// registers between the sum and the norms; NV == 0: any n, the row is re-read from x_out.
template <typename T, int NV>
__global__ void __launch_bounds__(256) depth_mix_norms_kernel(float* __restrict__ x_out, T* __restrict__ h1,
                                                              T* __restrict__ h2, const float* __restrict__ stack,
                                                              int64_t level_stride, const T* __restrict__ coef,
                                                              int count, const T* __restrict__ w1,
                                                              const T* __restrict__ w2, int64_t n, float eps,
                                                              float offset) {
  pdl_prologue();
  __shared__ float red[32];
  __shared__ float cs[64];
  const int64_t t = blockIdx.x;
  const bool mixes = coef != nullptr;
  if (mixes) {
    for (int j = threadIdx.x; j < count && j < 64; j += blockDim.x) cs[j] = to_f32(coef[j]);
    __syncthreads();
  }
  const float* base = stack + t * n;
  if (NV > 0) {
    float v[NV > 0 ? NV : 1][4];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int64_t i = (int64_t)(k * 256 + threadIdx.x) * 4;
      v[k][0] = v[k][1] = v[k][2] = v[k][3] = 0.f;
      if (i < n) {
        if (mixes) {
          for (int j = 0; j < count; ++j) {
            const float4 s4 = *reinterpret_cast<const float4*>(base + j * level_stride + i);
            const float c = j < 64 ? cs[j] : to_f32(coef[j]);
            v[k][0] = fmaf(c, s4.x, v[k][0]); v[k][1] = fmaf(c, s4.y, v[k][1]);
            v[k][2] = fmaf(c, s4.z, v[k][2]); v[k][3] = fmaf(c, s4.w, v[k][3]);
          }
        } else {
          const float4 s4 = *reinterpret_cast<const float4*>(base + (count - 1) * level_stride + i);
          v[k][0] = s4.x; v[k][1] = s4.y; v[k][2] = s4.z; v[k][3] = s4.w;
        }
        if (x_out) *reinterpret_cast<float4*>(x_out + t * n + i) = make_float4(v[k][0], v[k][1], v[k][2], v[k][3]);
#pragma unroll
        for (int c = 0; c < 4; ++c) ss = fmaf(v[k][c], v[k][c], ss);
      }
    }
    if (!h1 && !h2) return;
    const float rstd = 1.0f / sqrtf(block_sum_ps(ss, red) / (float)n + eps);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int64_t i = (int64_t)(k * 256 + threadIdx.x) * 4;
      if (i >= n) continue;
      float g[4], o[4];
      if (h1) {
        row_load4(w1 + i, g);
#pragma unroll
        for (int c = 0; c < 4; ++c) o[c] = v[k][c] * rstd * (offset + g[c]);
        row_store4(h1 + t * n + i, o);
      }
      if (h2) {
        row_load4(w2 + i, g);
#pragma unroll
        for (int c = 0; c < 4; ++c) o[c] = v[k][c] * rstd * (offset + g[c]);
        row_store4(h2 + t * n + i, o);
      }
    }
  } else {
    float ss = 0.f;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
      float v = 0.f;
      if (mixes) {
        for (int j = 0; j < count; ++j) v = fmaf(j < 64 ? cs[j] : to_f32(coef[j]), base[j * level_stride + i], v);
      } else {
        v = base[(count - 1) * level_stride + i];
      }
      x_out[t * n + i] = v;
      ss = fmaf(v, v, ss);
    }
    if (!h1 && !h2) return;
    const float rstd = 1.0f / sqrtf(block_sum_ps(ss, red) / (float)n + eps);
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
      const float u = x_out[t * n + i] * rstd;                 // this thread's own store
      if (h1) h1[t * n + i] = from_f32<T>(u * (offset + to_f32(w1[i])));
      if (h2) h2[t * n + i] = from_f32<T>(u * (offset + to_f32(w2[i])));
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) branch_sum_residual_kernel(float* __restrict__ r, T* __restrict__ act,
                                                                  const T* __restrict__ a, int64_t as,
                                                                  const T* __restrict__ wa, const T* __restrict__ b,
                                                                  int64_t bs, const T* __restrict__ wb,
                                                                  const T* __restrict__ c, int64_t cs,
                                                                  const T* __restrict__ wn, int64_t n, float eps,
                                                                  float scale, float scale_b, int vec) {
  pdl_prologue();
  __shared__ float red[32];
  const int64_t t = blockIdx.x;
  const T* ar = a + t * as;
  const T* br = b ? b + t * bs : nullptr;
  const T* cr = c ? c + t * cs : nullptr;
  float ra = 1.f, rb = 1.f;
  if (vec) {
    // 4 elements per access: statistics first (the branches are read again from L1 in the second pass)
    if (wa || (br && wb)) {
      float sa = 0.f, sb = 0.f;
      for (int64_t i = (int64_t)threadIdx.x * 4; i < n; i += (int64_t)blockDim.x * 4) {
        float v[4];
        if (wa) {
          row_load4(ar + i, v);
#pragma unroll
          for (int k = 0; k < 4; ++k) sa = fmaf(v[k], v[k], sa);
        }
        if (br && wb) {
          row_load4(br + i, v);
#pragma unroll
          for (int k = 0; k < 4; ++k) sb = fmaf(v[k], v[k], sb);
        }
      }
      if (wa) ra = 1.0f / sqrtf(block_sum_ps(sa, red) / (float)n + eps);
      if (br && wb) rb = 1.0f / sqrtf(block_sum_ps(sb, red) / (float)n + eps);
    }
    float sn = 0.f;
    for (int64_t i = (int64_t)threadIdx.x * 4; i < n; i += (int64_t)blockDim.x * 4) {
      float m[4], g[4], x[4];
      row_load4(ar + i, m);
      if (wa) {
        row_load4(wa + i, g);
#pragma unroll
        for (int k = 0; k < 4; ++k) m[k] = m[k] * ra * g[k];
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) m[k] *= scale;
      if (br) {
        row_load4(br + i, x);
        if (wb) {
          row_load4(wb + i, g);
#pragma unroll
          for (int k = 0; k < 4; ++k) m[k] = fmaf(x[k] * rb * g[k], scale_b, m[k]);
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k) m[k] = fmaf(x[k], scale_b, m[k]);
        }
      }
      if (cr) {
        row_load4(cr + i, x);
#pragma unroll
        for (int k = 0; k < 4; ++k) m[k] += x[k];
      }
      row_load4(r + t * n + i, x);
#pragma unroll
      for (int k = 0; k < 4; ++k) { m[k] += x[k]; sn = fmaf(m[k], m[k], sn); }
      row_store4(r + t * n + i, m);
      if (act && !wn) row_store4(act + t * n + i, m);
    }
    if (act && wn) {                         // the next block's input norm of the new residual (own stores re-read)
      const float rn = 1.0f / sqrtf(block_sum_ps(sn, red) / (float)n + eps);
      for (int64_t i = (int64_t)threadIdx.x * 4; i < n; i += (int64_t)blockDim.x * 4) {
        float m[4], g[4];
        row_load4(r + t * n + i, m);
        row_load4(wn + i, g);
#pragma unroll
        for (int k = 0; k < 4; ++k) m[k] = m[k] * rn * g[k];
        row_store4(act + t * n + i, m);
      }
    }
    return;
  }
  if (wa) {
    float ss = 0.f;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) { const float v = to_f32(ar[i]); ss = fmaf(v, v, ss); }
    ra = 1.0f / sqrtf(block_sum_ps(ss, red) / (float)n + eps);
  }
  if (br && wb) {
    float ss = 0.f;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) { const float v = to_f32(br[i]); ss = fmaf(v, v, ss); }
    rb = 1.0f / sqrtf(block_sum_ps(ss, red) / (float)n + eps);
  }
  float sn = 0.f;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
    float m = to_f32(ar[i]) * ra;
    if (wa) m *= to_f32(wa[i]);
    m *= scale;
    if (br) {
      float m2 = to_f32(br[i]) * rb;
      if (wb) m2 *= to_f32(wb[i]);
      m = fmaf(m2, scale_b, m);
    }
    if (cr) m += to_f32(cr[i]);
    const float v = r[t * n + i] + m;
    r[t * n + i] = v;
    sn = fmaf(v, v, sn);
    if (act && !wn) act[t * n + i] = from_f32<T>(v);
  }
  if (act && wn) {
    const float rn = 1.0f / sqrtf(block_sum_ps(sn, red) / (float)n + eps);
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x)
      act[t * n + i] = from_f32<T>(r[t * n + i] * rn * to_f32(wn[i]));
  }
}

template <typename T>
__global__ void gelu_mul_gather_kernel(T* __restrict__ o, const T* __restrict__ z, int64_t zs,
                                       const int* __restrict__ tokens, const T* __restrict__ table, int64_t table_stride,
                                       int64_t vocab, int col0, int dim, int64_t total) {
  pdl_prologue();
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = idx / dim;
    const int d = (int)(idx - t * dim);
    int64_t tok = tokens[t];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    o[idx] = from_f32<T>(gelu_tanh_f(to_f32(z[t * zs + d])) * to_f32(table[tok * table_stride + col0 + d]));
  }
}

}  // namespace

extern "C" int b2l_embed_rmsnorm(void* residual_f32, const void* tokens_i32, const void* embed, const void* weight,
                                 int64_t rows, int64_t n, int64_t vocab, float eps, float weight_offset, float scale,
                                 int dtype, void* stream) {
  B2L_REQUIRE(residual_f32 && tokens_i32 && embed, "embed_rmsnorm: null pointer");
  B2L_REQUIRE(rows >= 0 && n > 0 && vocab > 0, "embed_rmsnorm: bad shape");
  if (rows == 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  B2L_DISPATCH_FLOAT(dtype, "embed_rmsnorm", {
    b2l_launch(embed_rmsnorm_kernel<T>, dim3((unsigned)rows), dim3(256), (size_t)0, st, (float*)residual_f32,
               (const int*)tokens_i32, (const T*)embed, (const T*)weight, n, vocab, eps, weight_offset, scale,
               (int)(n % 4 == 0 && row_aligned4<T>(embed) && row_aligned4<T>(weight) && (uintptr_t)residual_f32 % 16 == 0));
  });
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

extern "C" int b2l_depth_mix_norms(void* x_out_f32, void* h1, void* h2, const void* stack_f32, int64_t level_stride,
                                   const void* coef, int count, const void* w1, const void* w2, int64_t rows, int64_t n,
                                   float eps, float weight_offset, int dtype, void* stream) {
  B2L_REQUIRE(stack_f32 && count >= 1, "depth_mix_norms: null pointer or no level");
  B2L_REQUIRE((!h1 || w1) && (!h2 || w2), "depth_mix_norms: a norm output without its weight");
  B2L_REQUIRE(rows >= 0 && n > 0, "depth_mix_norms: bad shape");
  if (rows == 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  bool fast = n % 4 == 0 && n <= 8192 && level_stride % 4 == 0 && (uintptr_t)stack_f32 % 16 == 0 &&
              (x_out_f32 == nullptr || (uintptr_t)x_out_f32 % 16 == 0);
  B2L_DISPATCH_FLOAT(dtype, "depth_mix_norms", {
    fast = fast && row_aligned4<T>(h1) && row_aligned4<T>(h2) && row_aligned4<T>(w1) && row_aligned4<T>(w2);
  });
  B2L_REQUIRE(fast || x_out_f32, "depth_mix_norms: rows of %lld elements need the mixed output buffer", (long long)n);
#define B2L_DMN(NVV)                                                                                                \
  b2l_launch(depth_mix_norms_kernel<T, NVV>, dim3((unsigned)rows), dim3(256), (size_t)0, st, (float*)x_out_f32,    \
             (T*)h1, (T*)h2, (const float*)stack_f32, level_stride, (const T*)coef, count, (const T*)w1,           \
             (const T*)w2, n, eps, weight_offset)
  B2L_DISPATCH_FLOAT(dtype, "depth_mix_norms", {
    if (fast && n <= 1024) B2L_DMN(1);
    else if (fast && n <= 2048) B2L_DMN(2);
    else if (fast && n <= 4096) B2L_DMN(4);
    else if (fast) B2L_DMN(8);
    else B2L_DMN(0);
  });
#undef B2L_DMN
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

extern "C" int b2l_branch_sum_residual(void* residual_f32, void* act, const void* a, int64_t a_row_stride,
                                       const void* a_weight, const void* b, int64_t b_row_stride, const void* b_weight,
                                       const void* c, int64_t c_row_stride, const void* next_weight, int64_t rows,
                                       int64_t n, float eps, float scale, float scale_b, int dtype, void* stream) {
  B2L_REQUIRE(residual_f32 && a, "branch_sum_residual: null pointer");
  B2L_REQUIRE(rows >= 0 && n > 0, "branch_sum_residual: bad shape");
  if (rows == 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  B2L_DISPATCH_FLOAT(dtype, "branch_sum_residual", {
    b2l_launch(branch_sum_residual_kernel<T>, dim3((unsigned)rows), dim3(256), (size_t)0, st, (float*)residual_f32,
               (T*)act, (const T*)a, a_row_stride, (const T*)a_weight, (const T*)b, b_row_stride, (const T*)b_weight,
               (const T*)c, c_row_stride, (const T*)next_weight, n, eps, scale, scale_b,
               (int)(n % 4 == 0 && row_aligned4<T>(next_weight) && a_row_stride % 4 == 0 && b_row_stride % 4 == 0 && c_row_stride % 4 == 0 &&
                     row_aligned4<T>(a) && row_aligned4<T>(b) && row_aligned4<T>(c) && row_aligned4<T>(a_weight) &&
                     row_aligned4<T>(b_weight) && row_aligned4<T>(act) && (uintptr_t)residual_f32 % 16 == 0));
  });
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

extern "C" int b2l_gelu_mul_gather(void* out, const void* z, int64_t z_row_stride, const void* tokens_i32,
                                   const void* table, int64_t table_row_stride, int64_t vocab, int col0, int dim,
                                   int64_t rows, int dtype, void* stream) {
  B2L_REQUIRE(out && z && tokens_i32 && table, "gelu_mul_gather: null pointer");
  B2L_REQUIRE(rows >= 0 && dim > 0 && col0 >= 0 && col0 + dim <= table_row_stride, "gelu_mul_gather: bad shape");
  if (rows == 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t total = rows * dim;
  const unsigned grid = (unsigned)(cdiv64(total, 256) < 148 * 16 ? cdiv64(total, 256) : 148 * 16);
  B2L_DISPATCH_FLOAT(dtype, "gelu_mul_gather", {
    b2l_launch(gelu_mul_gather_kernel<T>, dim3(grid), dim3(256), (size_t)0, st, (T*)out, (const T*)z, z_row_stride,
               (const int*)tokens_i32, (const T*)table, table_row_stride, vocab, col0, dim, total);
  });
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}
