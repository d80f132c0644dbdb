// Element-wise gated linear recurrences over a RAGGED batch (sequence s owns tokens [seq_start[s], seq_start[s+1]),
// has seq_ctx[s] earlier tokens whose effect lives in state slot seq_slot[s]):
//
//     S_t = a_t * S_(t-1) + b_t          o_t = S_t * g_t          per channel, S in fp32, one value per channel and slot
//
//   mode 0, minimal GRU:        z = sigmoid(p0);  candidate = p1 + 1/2 (p1 >= 0) | sigmoid(p1) (p1 < 0)
//                               a = 1 - z;  b = z * candidate;  g = silu(p2)
//   mode 1, real-gated LRU:     r = sigmoid(p1 + bias_r);  i = sigmoid(p2 + bias_i);  a = exp(-c * r * softplus(lam))
//                               b = sqrt(1 - a^2) * i * p0;  g = gelu_tanh(p3)
//
// p0 .. p3 are column views of projection outputs in T (row strides given); gates, decays and the state are fp32.
// The recurrence is associative, so a CTA = (32 channels, sequence) cuts its tokens into segments of kSeg: each of
// its kWarps warps loads one segment (kSeg independent loads per input in flight; 16 warps of 8 tokens at no more
// than 64 registers, so that two CTAs share an SM: occupancy, not arithmetic, bounds the kernel), reduces it to the pair
// (A = prod a, B = its end state from zero), the pairs are chained through shared memory from the CTA's running
// state, and each warp then replays its segment from registers with the right start value.  A single new token takes
// the same path with one live warp.  A sequence with seq_ctx == 0 starts from zero: slots need no clearing.
//
//   norm_sigmoid_gate   o = unit_rms(y) * w * sigmoid(z)   (y fp32 rows, z a column view in T; the gate acts AFTER
//                       the norm, unlike gated_group_norm)
#include "common.cuh"
#include "rowvec.cuh"

namespace {

constexpr int kSeg = 8;
constexpr int kWarps = 16;

__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_gr(float v) { return v > 20.f ? v : log1pf(expf(v)); }
__device__ __forceinline__ float gelu_tanh_gr(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// Gate arithmetic in two grades: true fp32 library functions when the activations are fp32 (the exact mode), and
// ex2.approx-based forms (relative error ~2^-22, far below the rounding of the 16-bit projections that feed the gates)
// when they are 16-bit: the library forms cost ~200 dependent instructions per token and channel, which bound the
// kernel at the occupancy its registers allow.
constexpr float kLog2eG = 1.4426950408889634f;
template <bool FAST> __device__ __forceinline__ float sigm(float v) {
  return FAST ? __fdividef(1.0f, 1.0f + fast_exp2(-v * kLog2eG)) : sigmoid_f(v);
}
template <bool FAST> __device__ __forceinline__ float gelu_t(float z) {
  if (!FAST) return gelu_tanh_gr(z);
  const float u = 0.7978845608028654f * (z + 0.044715f * z * z * z);
  const float th = 1.0f - __fdividef(2.0f, fast_exp2(u * (2.0f * kLog2eG)) + 1.0f);
  return 0.5f * z * (1.0f + th);
}

struct ScanArgs {
  const void* p[4];
  int64_t ps[4];
  const void* bias_r; const void* bias_i; const void* lam;
  float* state;
  void* out; int64_t out_stride;
  const int* seq_start; const int* seq_ctx; const int* seq_slot;
  int width;
  float decay_scale;           // c of mode 1
};

template <typename T, int MODE>
__global__ void __launch_bounds__(kWarps * 32, 2) gated_scan_kernel(ScanArgs k) {
  pdl_prologue();
  __shared__ float sA[kWarps][32], sB[kWarps][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  const bool live = c < k.width;
  constexpr bool FAST = sizeof(T) == 2;
  const int s = blockIdx.y;
  const int start = k.seq_start[s], len = k.seq_start[s + 1] - start, ctx = k.seq_ctx[s];
  if (len <= 0) return;
  const int64_t slot = k.seq_slot[s];
  float carry = (ctx > 0 && live) ? k.state[slot * k.width + c] : 0.f;
  const T* p0 = (const T*)k.p[0];
  const T* p1 = (const T*)k.p[1];
  const T* p2 = (const T*)k.p[2];
  const T* p3 = (const T*)k.p[3];
  float br = 0.f, bi = 0.f, rate = 0.f;
  if (MODE == 1 && live) {
    br = to_f32(((const T*)k.bias_r)[c]);
    bi = to_f32(((const T*)k.bias_i)[c]);
    rate = -k.decay_scale * softplus_gr(to_f32(((const T*)k.lam)[c]));
  }
  for (int base = 0; base < len; base += kWarps * kSeg) {
    const int t0 = base + warp * kSeg;
    const int cnt = max(0, min(kSeg, len - t0));
    float a[kSeg], b[kSeg], g[kSeg];
    // every load of the segment is issued before the first gate is evaluated
    float v0[kSeg], v1[kSeg], v2[kSeg], v3[kSeg];
#pragma unroll
    for (int j = 0; j < kSeg; ++j) {
      v0[j] = v1[j] = v2[j] = v3[j] = 0.f;
      if (j < cnt && live) {
        const int64_t row = start + t0 + j;
        v0[j] = to_f32(p0[row * k.ps[0] + c]);
        v1[j] = to_f32(p1[row * k.ps[1] + c]);
        v2[j] = to_f32(p2[row * k.ps[2] + c]);
        if (MODE == 1) v3[j] = to_f32(p3[row * k.ps[3] + c]);
      }
    }
    float A = 1.f, B = 0.f;
#pragma unroll
    for (int j = 0; j < kSeg; ++j) {
      if (j < cnt && live) {
        if (MODE == 0) {
          const float z = sigm<FAST>(v0[j]);
          const float cand = v1[j] >= 0.f ? v1[j] + 0.5f : sigm<FAST>(v1[j]);
          a[j] = 1.0f - z;
          b[j] = z * cand;
          g[j] = v2[j] * sigm<FAST>(v2[j]);
        } else {
          const float r = sigm<FAST>(v1[j] + br), i = sigm<FAST>(v2[j] + bi);
          const float la = rate * r;                       // log a <= 0
          if (FAST) {
            a[j] = fast_exp2(la * kLog2eG);
            b[j] = sqrtf(fmaxf(1.0f - a[j] * a[j], 0.f)) * i * v0[j];
          } else {
            a[j] = expf(la);
            b[j] = sqrtf(fmaxf(-expm1f(2.0f * la), 0.f)) * i * v0[j];    // sqrt(1 - a^2) without cancellation
          }
          g[j] = gelu_t<FAST>(v3[j]);
        }
        B = fmaf(a[j], B, b[j]);
        A *= a[j];
      } else {
        a[j] = 1.f; b[j] = 0.f; g[j] = 0.f;
      }
    }
    sA[warp][lane] = A;
    sB[warp][lane] = B;
    __syncthreads();
    float S = carry;
    for (int w = 0; w < warp; ++w) S = fmaf(sA[w][lane], S, sB[w][lane]);
    float next = S;
    for (int w = warp; w < kWarps; ++w) next = fmaf(sA[w][lane], next, sB[w][lane]);
    T* o = (T*)k.out;
#pragma unroll
    for (int j = 0; j < kSeg; ++j) {
      if (j < cnt && live) {
        S = fmaf(a[j], S, b[j]);
        o[(int64_t)(start + t0 + j) * k.out_stride + c] = from_f32<T>(S * g[j]);
      }
    }
    carry = next;
    __syncthreads();                                       // the pairs are overwritten by the next round
  }
  if (warp == 0 && live) k.state[slot * k.width + c] = carry;
}

template <typename T>
__global__ void __launch_bounds__(256) norm_sigmoid_gate_kernel(T* __restrict__ o, const float* __restrict__ y,
                                                                const T* __restrict__ z, int64_t zs,
                                                                const T* __restrict__ w, int n, float eps, int vec) {
  pdl_prologue();
  __shared__ float red[32];
  const int64_t t = blockIdx.x;
  const float* yr = y + t * n;
  float ss = 0.f;
  if (vec) {
    for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(yr + i);
      ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
    }
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss = fmaf(yr[i], yr[i], ss);
  }
  ss = warp_reduce_sum(ss);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float tot = lane < nw ? red[lane] : 0.f;
  tot = warp_reduce_sum(tot);
  const float rstd = 1.0f / sqrtf(tot / (float)n + eps);
  if (vec) {                                   // the row is read again from L1
    for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4) {
      float v[4], g[4], q[4];
      row_load4(yr + i, v);
      row_load4(w + i, g);
      row_load4(z + t * zs + i, q);
#pragma unroll
      for (int c = 0; c < 4; ++c) v[c] = v[c] * rstd * g[c] * sigmoid_f(q[c]);
      row_store4(o + t * (int64_t)n + i, v);
    }
    return;
  }
  for (int i = threadIdx.x; i < n; i += blockDim.x)
    o[t * n + i] = from_f32<T>(yr[i] * rstd * to_f32(w[i]) * sigmoid_f(to_f32(z[t * zs + i])));
}

}  // namespace

/* mode 0 (minimal GRU): p0 = update-gate, p1 = candidate, p2 = output-gate pre-activations; p3, biases, lam unused.
 * mode 1 (real-gated LRU): p0 = recurrence input, p1 / p2 = recurrence- / input-gate pre-activations (their biases in
 * bias_r / bias_i), p3 = the gelu branch's pre-activation, lam [width], decay_scale = c.
 * state_f32 [slots, width]; out [tokens, width] in dtype with its row stride. */
extern "C" int b2l_gated_scan(void* out, int64_t out_row_stride, void* state_f32, const void* p0, int64_t p0_row_stride,
                              const void* p1, int64_t p1_row_stride, const void* p2, int64_t p2_row_stride,
                              const void* p3, int64_t p3_row_stride, const void* bias_r, const void* bias_i,
                              const void* lam, float decay_scale, const void* seq_start, const void* seq_ctx,
                              const void* seq_slot, int64_t num_seqs, int width, int mode, int dtype, void* stream) {
  B2L_REQUIRE(out && state_f32 && p0 && p1 && p2 && seq_start && seq_ctx && seq_slot, "gated_scan: null pointer");
  B2L_REQUIRE(mode == 0 || mode == 1, "gated_scan: mode %d", mode);
  B2L_REQUIRE(mode == 0 || (p3 && bias_r && bias_i && lam), "gated_scan: the gated LRU needs p3, both biases and lam");
  B2L_REQUIRE(width > 0, "gated_scan: bad width %d", width);
  if (num_seqs <= 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  ScanArgs k;
  k.p[0] = p0; k.p[1] = p1; k.p[2] = p2; k.p[3] = p3;
  k.ps[0] = p0_row_stride; k.ps[1] = p1_row_stride; k.ps[2] = p2_row_stride; k.ps[3] = p3_row_stride;
  k.bias_r = bias_r; k.bias_i = bias_i; k.lam = lam; k.state = (float*)state_f32; k.out = out;
  k.out_stride = out_row_stride; k.seq_start = (const int*)seq_start; k.seq_ctx = (const int*)seq_ctx;
  k.seq_slot = (const int*)seq_slot; k.width = width; k.decay_scale = decay_scale;
  const dim3 grid((unsigned)cdiv64(width, 32), (unsigned)num_seqs), block(kWarps * 32);
  B2L_DISPATCH_FLOAT(dtype, "gated_scan", {
    if (mode == 0) b2l_launch(gated_scan_kernel<T, 0>, grid, block, (size_t)0, st, k);
    else b2l_launch(gated_scan_kernel<T, 1>, grid, block, (size_t)0, st, k);
  });
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

extern "C" int b2l_norm_sigmoid_gate(void* out, const void* y_f32, const void* z, int64_t z_row_stride,
                                     const void* weight, int64_t rows, int n, float eps, int dtype, void* stream) {
  B2L_REQUIRE(out && y_f32 && z && weight, "norm_sigmoid_gate: null pointer");
  B2L_REQUIRE(n > 0, "norm_sigmoid_gate: bad shape");
  if (rows <= 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int threads = n >= 1024 ? 256 : (n >= 256 ? 128 : 64);
  B2L_DISPATCH_FLOAT(dtype, "norm_sigmoid_gate", {
    b2l_launch(norm_sigmoid_gate_kernel<T>, dim3((unsigned)rows), dim3(threads), (size_t)0, st, (T*)out,
               (const float*)y_f32, (const T*)z, z_row_stride, (const T*)weight, n, eps,
               (int)(n % 4 == 0 && z_row_stride % 4 == 0 && (uintptr_t)y_f32 % 16 == 0 && row_aligned4<T>(z) &&
                     row_aligned4<T>(weight) && row_aligned4<T>(out)));
  });
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}
