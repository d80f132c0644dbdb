// Selective state-space mixer (Mamba-2 form: scalar decay per head, state S[N, P] per head) over a RAGGED batch:
// sequence s owns tokens [seq_start[s], seq_start[s+1]) of the flat batch, has seq_ctx[s] earlier tokens whose
// effect lives in state slot seq_slot[s], and may bring any number of new tokens (1 = a decode step).
//
//   causal_conv_silu      (`activation` 1; 0 = the plain convolution) out[t, c] = silu(bias[c] + sum_j w[c, K-1-j] * in[t-j, c]); inputs before the step come from
//                         the slot's conv tail (the last K-1 inputs), inputs before the sequence are zero
//   conv_tail_update      the slot's conv tail after the step (in place)
//   ssm_scan              dt = softplus(dt_raw + dt_bias); S <- exp(-exp(A_log) dt) S + dt B x^T; y = S^T C + D x
//                         S in fp32 registers for the whole step, read from / written to the slot once
//                         (slot layout [head, n, p]).  With `fixed_decay` (fp32 per head) the same kernel runs a
//                         decayed linear attention: S <- decay_h S + B x^T, y = S^T C (dt = 1, no skip term), and
//                         `silu_inputs` applies SiLU to x, B and C as they are staged (fp32)
//   gated_group_norm      o = unit_rms_g(y * silu(z)) * w   in `groups` equal parts of the row
// A sequence with seq_ctx == 0 starts from zero: its slot is never read, so slots need no clearing when reused.
#include "common.cuh"

namespace {

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// ---- seq lookup for a flat token: binary search in seq_start -------------------------------------------------------
__device__ __forceinline__ int find_seq(const int* __restrict__ seq_start, int nseq, int tok) {
  int lo = 0, hi = nseq - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (seq_start[mid] <= tok) lo = mid; else hi = mid - 1;
  }
  return lo;
}

template <typename T>
__global__ void causal_conv_silu_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t in_stride,
                                        const T* __restrict__ w, const T* __restrict__ bias,
                                        const T* __restrict__ tail, const int* __restrict__ seq_start,
                                        const int* __restrict__ seq_ctx, const int* __restrict__ seq_slot, int nseq,
                                        int channels, int taps, int act) {
  pdl_prologue();
  const int tok = blockIdx.y;
  const int s = find_seq(seq_start, nseq, tok);
  const int local = tok - seq_start[s], ctx = seq_ctx[s];
  const int64_t slot = seq_slot[s];
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  float acc = to_f32(bias[c]);
  for (int j = 0; j < taps; ++j) {                 // j tokens back
    const int i = local - j;
    float v = 0.f;
    if (i >= 0) v = to_f32(in[(int64_t)(tok - j) * in_stride + c]);
    else if (ctx + i >= 0) v = to_f32(tail[(slot * (taps - 1) + (taps - 1 + i)) * channels + c]);
    acc = fmaf(to_f32(w[(int64_t)c * taps + (taps - 1 - j)]), v, acc);
  }
  out[(int64_t)tok * channels + c] = from_f32<T>(act ? silu_f(acc) : acc);
}

// The same with 16-byte accesses: one thread = VEC consecutive channels (channels, the input row stride and the
// column window's start all multiples of VEC elements).
template <typename T, int TAPS>     // TAPS > 0: tap count known at compile time, weights held in registers
__global__ void causal_conv_silu_vec_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t in_stride,
                                            const T* __restrict__ w, const T* __restrict__ bias,
                                            const T* __restrict__ tail, const int* __restrict__ seq_start,
                                            const int* __restrict__ seq_ctx, const int* __restrict__ seq_slot,
                                            int nseq, int channels, int taps, int act) {
  pdl_prologue();
  constexpr int VEC = 16 / (int)sizeof(T);
  const int tok = blockIdx.y;
  const int s = find_seq(seq_start, nseq, tok);
  const int local = tok - seq_start[s], ctx = seq_ctx[s];
  const int64_t slot = seq_slot[s];
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * VEC;
  if (c >= channels) return;
  float acc[VEC];
  {
    const uint4 raw = ldg_128(bias + c);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int k = 0; k < VEC; ++k) acc[k] = to_f32(e[k]);
  }
  if (TAPS > 0) {
    // the VEC channels' taps are VEC * TAPS consecutive elements = TAPS 16-byte vectors
    float wf[VEC * (TAPS > 0 ? TAPS : 1)];
#pragma unroll
    for (int v = 0; v < TAPS; ++v) {
      const uint4 raw = ldg_128(w + (int64_t)c * TAPS + v * VEC);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int k = 0; k < VEC; ++k) wf[v * VEC + k] = to_f32(e[k]);
    }
#pragma unroll
    for (int j = 0; j < TAPS; ++j) {
      const int i = local - j;
      uint4 raw = make_uint4(0u, 0u, 0u, 0u);
      if (i >= 0) raw = ldg_128(in + (int64_t)(tok - j) * in_stride + c);
      else if (ctx + i >= 0) raw = ldg_128(tail + (slot * (TAPS - 1) + (TAPS - 1 + i)) * channels + c);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int k = 0; k < VEC; ++k) acc[k] = fmaf(wf[k * TAPS + (TAPS - 1 - j)], to_f32(e[k]), acc[k]);
    }
  } else {
    for (int j = 0; j < taps; ++j) {
      const int i = local - j;
      uint4 raw = make_uint4(0u, 0u, 0u, 0u);
      if (i >= 0) raw = ldg_128(in + (int64_t)(tok - j) * in_stride + c);
      else if (ctx + i >= 0) raw = ldg_128(tail + (slot * (taps - 1) + (taps - 1 + i)) * channels + c);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int k = 0; k < VEC; ++k) acc[k] = fmaf(to_f32(w[(int64_t)(c + k) * taps + (taps - 1 - j)]), to_f32(e[k]), acc[k]);
    }
  }
  uint4 res;
  T* e = reinterpret_cast<T*>(&res);
#pragma unroll
  for (int k = 0; k < VEC; ++k) e[k] = from_f32<T>(act ? silu_f(acc[k]) : acc[k]);
  *reinterpret_cast<uint4*>(out + (int64_t)tok * channels + c) = res;
}

template <typename T>
__global__ void conv_tail_update_kernel(T* __restrict__ tail, const T* __restrict__ in, int64_t in_stride,
                                        const int* __restrict__ seq_start, const int* __restrict__ seq_ctx,
                                        const int* __restrict__ seq_slot, int channels, int taps) {
  pdl_prologue();
  const int s = blockIdx.y;
  const int start = seq_start[s], len = seq_start[s + 1] - start, ctx = seq_ctx[s];
  const int64_t slot = seq_slot[s];
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels || len <= 0) return;
  const int keep = taps - 1;
  T* mine = tail + slot * keep * channels;
  // entry j holds the input at absolute index ctx + len - keep + j; ascending j only reads entries > j of the old tail
  for (int j = 0; j < keep; ++j) {
    const int a = ctx + len - keep + j;
    T v = from_f32<T>(0.f);
    if (a >= ctx) v = in[(int64_t)(start + a - ctx) * in_stride + c];
    else if (a >= 0) v = mine[(int64_t)(j + len) * channels + c];
    mine[(int64_t)j * channels + c] = v;
  }
}

// Scan: one CTA = (tile of 32 * ctiles columns p, head, sequence).  Lane = column, so y_t[p] = sum_n S[n, p] C_t[n]
// needs no cross-lane reduction; a compute warp keeps NPT state rows of its 32 columns in registers, and when N > NPT
// the rows are cut into `nslices` warps whose partial sums meet in shared memory once per chunk of kChunk tokens
// (fixed slice order: deterministic).  The scan of one sequence is serial, so latency decides: kLoadWarps extra warps
// stage the NEXT chunk's B_t, C_t, x_t (as fp32) and dt / decay into the other half of a double buffer while the
// compute warps run the current one; the compute warps read them as broadcast float4, and with CPL = 2 every value
// read serves two columns per lane (shared-memory bandwidth, not the FMA pipe, bounds the token loop).
// State layout: [slot, head, n, p] (p contiguous = coalesced per n).
constexpr int kChunk = 16;
constexpr int kLoadWarps = 4;
constexpr int kVecBatch = 4;

template <typename T, int NPT, int CPL>
__global__ void __launch_bounds__(512) ssm_scan_kernel(
    float* __restrict__ y, float* __restrict__ state, const T* __restrict__ xbc, int64_t xbc_stride,
    const T* __restrict__ dt_raw, int64_t dt_stride, const T* __restrict__ dt_bias, const T* __restrict__ a_log,
    const T* __restrict__ d_skip, const int* __restrict__ seq_start, const int* __restrict__ seq_ctx,
    const int* __restrict__ seq_slot, int heads, int groups, int N, int P, int ctiles, int nslices,
    const float* __restrict__ fixed_decay, int silu_inputs) {
  pdl_prologue();
  extern __shared__ __align__(16) float sm[];
  const int Np = nslices * NPT, cols = ctiles * 32 * CPL;
  const int stage_floats = 2 * kChunk * Np + kChunk * cols + 2 * kChunk;
  float* sYbase = sm + 2 * stage_floats;       // [2][nslices][kChunk][cols], nslices > 1 only
  const int s = blockIdx.z, h = blockIdx.y, col0 = blockIdx.x * cols;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int cwarps = ctiles * nslices;
  const bool computes = warp < cwarps;
  const int ct = warp / nslices, sl = warp - ct * nslices;
  const int wcol = ct * 32 * CPL + lane;                   // this lane's first column inside the CTA's tile
  const int col = col0 + wcol, n0 = sl * NPT;              // its columns: col + 32 j, j < CPL
  const int start = seq_start[s], len = seq_start[s + 1] - start, ctx = seq_ctx[s];
  if (len <= 0) return;
  const int64_t slot = seq_slot[s];
  const int g = h / (heads / groups), inner = heads * P;
  const bool fixed = fixed_decay != nullptr;
  const float neg_a = fixed ? 0.f : -expf(to_f32(a_log[h])), bias = fixed ? 0.f : to_f32(dt_bias[h]);
  const float dsk = fixed ? 0.f : to_f32(d_skip[h]), fdec = fixed ? fixed_decay[h] : 0.f;
  auto act_in = [&](float v) { return silu_inputs ? silu_f(v) : v; };
  const int boff = inner + g * N, coff = inner + groups * N + g * N;
  const int nchunks = (len + kChunk - 1) / kChunk;

  constexpr int VEC = 16 / (int)sizeof(T);
  // whole 16-byte vectors line up when every column offset and the row stride are multiples of VEC elements
  const bool vec_ok = (N % VEC == 0) && (P % VEC == 0) && (xbc_stride % VEC == 0) && (((uintptr_t)xbc % 16) == 0);
  // stage chunk k into half k & 1 with `nth` threads numbered `t0`
  auto stage = [&](int k, int t0, int nth) {
    float* sB = sm + (k & 1) * stage_floats;
    float* sC = sB + kChunk * Np;
    float* sX = sC + kChunk * Np;
    float* sDt = sX + kChunk * cols;
    const int c0 = k * kChunk, tc = min(kChunk, len - c0);
    const T* rows = xbc + (int64_t)(start + c0) * xbc_stride;
    if (vec_ok) {
      // 16-byte loads, kVecBatch of them in flight per thread before the first shared-memory store
      const int nv = Np / VEC, per_op = tc * nv;
      for (int base = t0; base < 2 * per_op; base += nth * kVecBatch) {
        uint4 raw[kVecBatch];
#pragma unroll
        for (int u = 0; u < kVecBatch; ++u) {
          const int idx = base + u * nth;
          raw[u] = make_uint4(0u, 0u, 0u, 0u);
          if (idx < 2 * per_op) {
            const int op = idx >= per_op, rem = idx - op * per_op, t = rem / nv, n = (rem - t * nv) * VEC;
            if (n < N) raw[u] = ldg_128(rows + (int64_t)t * xbc_stride + (op ? coff : boff) + n);
          }
        }
#pragma unroll
        for (int u = 0; u < kVecBatch; ++u) {
          const int idx = base + u * nth;
          if (idx < 2 * per_op) {
            const int op = idx >= per_op, rem = idx - op * per_op, t = rem / nv, n = (rem - t * nv) * VEC;
            float* dst = (op ? sC : sB) + t * Np + n;
            const T* e = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
            for (int c = 0; c < VEC; ++c) dst[c] = act_in(to_f32(e[c]));
          }
        }
      }
      const int xv = cols / VEC;
      for (int base = t0; base < tc * xv; base += nth * kVecBatch) {
        uint4 raw[kVecBatch];
#pragma unroll
        for (int u = 0; u < kVecBatch; ++u) {
          const int idx = base + u * nth;
          raw[u] = make_uint4(0u, 0u, 0u, 0u);
          if (idx < tc * xv) {
            const int t = idx / xv, c = (idx - t * xv) * VEC;
            if (col0 + c < P) raw[u] = ldg_128(rows + (int64_t)t * xbc_stride + h * P + col0 + c);
          }
        }
#pragma unroll
        for (int u = 0; u < kVecBatch; ++u) {
          const int idx = base + u * nth;
          if (idx < tc * xv) {
            const int t = idx / xv, c = (idx - t * xv) * VEC;
            const T* e = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
            for (int k2 = 0; k2 < VEC; ++k2) sX[t * cols + c + k2] = act_in(to_f32(e[k2]));
          }
        }
      }
    } else {
#pragma unroll 8
      for (int i = t0; i < tc * Np; i += nth) {
        const int t = i / Np, n = i - t * Np;
        const T* r = rows + (int64_t)t * xbc_stride;
        const float bv = n < N ? act_in(to_f32(r[boff + n])) : 0.f;
        const float cv = n < N ? act_in(to_f32(r[coff + n])) : 0.f;
        sB[i] = bv;
        sC[i] = cv;
      }
#pragma unroll 8
      for (int i = t0; i < tc * cols; i += nth) {
        const int t = i / cols, c = i - t * cols;
        sX[i] = (col0 + c < P) ? act_in(to_f32(rows[(int64_t)t * xbc_stride + h * P + col0 + c])) : 0.f;
      }
    }
    if (t0 < tc) {
      const float dtv = fixed ? 1.0f : softplus_f(to_f32(dt_raw[(int64_t)(start + c0 + t0) * dt_stride + h]) + bias);
      sDt[t0] = dtv;
      sDt[kChunk + t0] = fixed ? fdec : expf(neg_a * dtv);
    }
  };
  // y of chunk k from the slices' partial sums (nslices > 1)
  auto reduce = [&](int k, int t0, int nth) {
    const float* sX = sm + (k & 1) * stage_floats + 2 * kChunk * Np;
    const float* sY = sYbase + (k & 1) * nslices * kChunk * cols;
    const int c0 = k * kChunk, tc = min(kChunk, len - c0);
    for (int i = t0; i < tc * cols; i += nth) {
      const int t = i / cols, c = i - t * cols;
      if (col0 + c >= P) continue;
      float v = 0.f;
      for (int q = 0; q < nslices; ++q) v += sY[(q * kChunk + t) * cols + c];
      y[(int64_t)(start + c0 + t) * inner + h * P + col0 + c] = fmaf(dsk, sX[i], v);
    }
  };

  float* st = state + ((slot * heads + h) * (int64_t)N) * P;            // [N, P]
  float2 S[CPL][NPT / 2];                                               // rows n0 + 2i, n0 + 2i + 1 of column j
  if (computes) {
#pragma unroll
    for (int j = 0; j < CPL; ++j)
#pragma unroll
      for (int i = 0; i < NPT / 2; ++i) {
        const bool live = ctx > 0 && col + 32 * j < P;
        S[j][i].x = (live && n0 + 2 * i < N) ? st[(int64_t)(n0 + 2 * i) * P + col + 32 * j] : 0.f;
        S[j][i].y = (live && n0 + 2 * i + 1 < N) ? st[(int64_t)(n0 + 2 * i + 1) * P + col + 32 * j] : 0.f;
      }
  }
  stage(0, tid, blockDim.x);
  __syncthreads();
  for (int k = 0; k < nchunks; ++k) {
    if (computes) {
      const float* sB = sm + (k & 1) * stage_floats;
      const float* sC = sB + kChunk * Np;
      const float* sX = sC + kChunk * Np;
      const float* sDt = sX + kChunk * cols;
      float* sY = sYbase + (k & 1) * nslices * kChunk * cols;
      const int c0 = k * kChunk, tc = min(kChunk, len - c0);
      for (int t = 0; t < tc; ++t) {
        const float dtv = sDt[t], dec = sDt[kChunk + t];
        float xv[CPL];
        float2 dx2[CPL], acc0[CPL], acc1[CPL];
#pragma unroll
        for (int j = 0; j < CPL; ++j) {
          xv[j] = sX[t * cols + wcol + 32 * j];
          dx2[j] = make_float2(dtv * xv[j], dtv * xv[j]);
          acc0[j] = acc1[j] = make_float2(0.f, 0.f);
        }
        const float4* b4 = reinterpret_cast<const float4*>(sB + t * Np + n0);
        const float4* c4 = reinterpret_cast<const float4*>(sC + t * Np + n0);
        // packed fp32 (two state rows per instruction): S <- dec * S + dx * b;  acc += S * c
        // every B / C value read from shared memory serves CPL columns
        const float2 dec2 = make_float2(dec, dec);
#pragma unroll
        for (int i = 0; i < NPT / 4; ++i) {
          const float4 b = b4[i], c = c4[i];
#pragma unroll
          for (int j = 0; j < CPL; ++j) {
            S[j][2 * i] = __ffma2_rn(dec2, S[j][2 * i], __fmul2_rn(dx2[j], make_float2(b.x, b.y)));
            acc0[j] = __ffma2_rn(S[j][2 * i], make_float2(c.x, c.y), acc0[j]);
            S[j][2 * i + 1] = __ffma2_rn(dec2, S[j][2 * i + 1], __fmul2_rn(dx2[j], make_float2(b.z, b.w)));
            acc1[j] = __ffma2_rn(S[j][2 * i + 1], make_float2(c.z, c.w), acc1[j]);
          }
        }
#pragma unroll
        for (int j = 0; j < CPL; ++j) {
          const float acc = (acc0[j].x + acc0[j].y) + (acc1[j].x + acc1[j].y);
          if (nslices == 1) {
            if (col + 32 * j < P) y[(int64_t)(start + c0 + t) * inner + h * P + col + 32 * j] = fmaf(dsk, xv[j], acc);
          } else {
            sY[(sl * kChunk + t) * cols + wcol + 32 * j] = acc;
          }
        }
      }
    } else {
      const int t0 = tid - cwarps * 32, nth = kLoadWarps * 32;
      if (nslices > 1 && k > 0) {
        reduce(k - 1, t0, nth);                 // reads the half that chunk k + 1 is about to overwrite
        asm volatile("bar.sync 1, %0;" ::"n"(kLoadWarps * 32) : "memory");
      }
      if (k + 1 < nchunks) stage(k + 1, t0, nth);
    }
    __syncthreads();
  }
  if (nslices > 1) reduce(nchunks - 1, tid, blockDim.x);
  if (computes) {
#pragma unroll
    for (int j = 0; j < CPL; ++j)
#pragma unroll
      for (int i = 0; i < NPT / 2; ++i) {
        if (n0 + 2 * i < N && col + 32 * j < P) st[(int64_t)(n0 + 2 * i) * P + col + 32 * j] = S[j][i].x;
        if (n0 + 2 * i + 1 < N && col + 32 * j < P) st[(int64_t)(n0 + 2 * i + 1) * P + col + 32 * j] = S[j][i].y;
      }
  }
}

// One CTA per (group, token).  VPT > 0: the gated values of the group fit in VPT registers per thread, so y and z are
// read once; VPT == 0: any group size, the gate is recomputed in the second pass.
template <typename T, int VPT>
__global__ void gated_group_norm_kernel(T* __restrict__ o, const float* __restrict__ y, const T* __restrict__ z,
                                        int64_t z_stride, const T* __restrict__ w, int inner, int groups, float eps) {
  pdl_prologue();
  __shared__ float red[32];
  const int64_t t = blockIdx.y;
  const int gs = inner / groups, base = blockIdx.x * gs;
  float ss = 0.f;
  float keep[VPT > 0 ? VPT : 1];
  if (VPT > 0) {
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      keep[k] = i < gs ? y[t * inner + base + i] * silu_f(to_f32(z[t * z_stride + base + i])) : 0.f;
      ss = fmaf(keep[k], keep[k], ss);
    }
  } else {
    for (int i = threadIdx.x; i < gs; i += blockDim.x) {
      const float v = y[t * inner + base + i] * silu_f(to_f32(z[t * z_stride + base + i]));
      ss = fmaf(v, v, ss);
    }
  }
  ss = warp_reduce_sum(ss);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float tot = lane < nw ? red[lane] : 0.f;
  tot = warp_reduce_sum(tot);
  const float rr = 1.0f / sqrtf(tot / (float)gs + eps);
  if (VPT > 0) {
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      if (i < gs) o[t * inner + base + i] = from_f32<T>(keep[k] * rr * to_f32(w[base + i]));
    }
  } else {
    for (int i = threadIdx.x; i < gs; i += blockDim.x) {
      const float v = y[t * inner + base + i] * silu_f(to_f32(z[t * z_stride + base + i]));
      o[t * inner + base + i] = from_f32<T>(v * rr * to_f32(w[base + i]));
    }
  }
}

// 16-byte version: one thread = VPV vectors of VEC consecutive columns, kept in registers between the two passes.
template <typename T, int VPV>
__global__ void gated_group_norm_vec_kernel(T* __restrict__ o, const float* __restrict__ y, const T* __restrict__ z,
                                            int64_t z_stride, const T* __restrict__ w, int inner, int groups,
                                            float eps) {
  pdl_prologue();
  constexpr int VEC = 16 / (int)sizeof(T);
  __shared__ float red[32];
  const int64_t t = blockIdx.y;
  const int gs = inner / groups, base = blockIdx.x * gs, nvec = gs / VEC;
  float keep[VPV][VEC];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VPV; ++k) {
    const int v = threadIdx.x + k * blockDim.x;
    if (v < nvec) {
      const int i = base + v * VEC;
      const uint4 zr = ldg_128(z + t * z_stride + i);
      const T* ze = reinterpret_cast<const T*>(&zr);
#pragma unroll
      for (int q = 0; q < VEC / 4; ++q) {
        const float4 yv = *reinterpret_cast<const float4*>(y + t * inner + i + 4 * q);
        keep[k][4 * q + 0] = yv.x * silu_f(to_f32(ze[4 * q + 0]));
        keep[k][4 * q + 1] = yv.y * silu_f(to_f32(ze[4 * q + 1]));
        keep[k][4 * q + 2] = yv.z * silu_f(to_f32(ze[4 * q + 2]));
        keep[k][4 * q + 3] = yv.w * silu_f(to_f32(ze[4 * q + 3]));
      }
#pragma unroll
      for (int c = 0; c < VEC; ++c) ss = fmaf(keep[k][c], keep[k][c], ss);
    }
  }
  ss = warp_reduce_sum(ss);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float tot = lane < nw ? red[lane] : 0.f;
  tot = warp_reduce_sum(tot);
  const float rr = 1.0f / sqrtf(tot / (float)gs + eps);
#pragma unroll
  for (int k = 0; k < VPV; ++k) {
    const int v = threadIdx.x + k * blockDim.x;
    if (v < nvec) {
      const int i = base + v * VEC;
      const uint4 wr = ldg_128(w + i);
      const T* we = reinterpret_cast<const T*>(&wr);
      uint4 res;
      T* re = reinterpret_cast<T*>(&res);
#pragma unroll
      for (int c = 0; c < VEC; ++c) re[c] = from_f32<T>(keep[k][c] * rr * to_f32(we[c]));
      *reinterpret_cast<uint4*>(o + t * inner + i) = res;
    }
  }
}

}  // namespace

extern "C" int b2l_causal_conv_silu(void* out, const void* in, int64_t in_row_stride, const void* weight,
                                    const void* bias, void* tail, const void* seq_start, const void* seq_ctx,
                                    const void* seq_slot, int64_t num_seqs, int64_t tokens, int channels, int taps,
                                    int activation, int dtype, void* stream) {
  B2L_REQUIRE(out && in && weight && bias && (tail || taps == 1) && seq_start && seq_ctx && seq_slot, "causal_conv_silu: null pointer");
  B2L_REQUIRE(channels > 0 && taps >= 1 && num_seqs >= 0 && tokens >= 0, "causal_conv_silu: bad shape");
  if (tokens == 0 || num_seqs == 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const dim3 block(128), grid((unsigned)cdiv64(channels, 128), (unsigned)tokens);
  const dim3 grid2((unsigned)cdiv64(channels, 128), (unsigned)num_seqs);
#define B2L_CONV(TP)                                                                                                 \
  b2l_launch(causal_conv_silu_vec_kernel<T, TP>, dim3((unsigned)cdiv64(channels / VEC, 128), (unsigned)tokens), block, \
             (size_t)0, st, (T*)out, (const T*)in, in_row_stride, (const T*)weight, (const T*)bias, (const T*)tail,  \
             (const int*)seq_start, (const int*)seq_ctx, (const int*)seq_slot, (int)num_seqs, channels, taps,        \
             activation)
  B2L_DISPATCH_FLOAT(dtype, "causal_conv_silu", {
    constexpr int VEC = 16 / (int)sizeof(T);
    const bool vec = channels % VEC == 0 && in_row_stride % VEC == 0 && (uintptr_t)in % 16 == 0 &&
                     (uintptr_t)out % 16 == 0 && (uintptr_t)bias % 16 == 0 && (uintptr_t)tail % 16 == 0;
    const bool wvec = (uintptr_t)weight % 16 == 0;
    if (vec && wvec && taps == 4) B2L_CONV(4);
    else if (vec && wvec && taps == 3) B2L_CONV(3);
    else if (vec && wvec && taps == 2) B2L_CONV(2);
    else if (vec) B2L_CONV(0);
    else
      b2l_launch(causal_conv_silu_kernel<T>, grid, block, (size_t)0, st, (T*)out, (const T*)in, in_row_stride,
                 (const T*)weight, (const T*)bias, (const T*)tail, (const int*)seq_start, (const int*)seq_ctx,
                 (const int*)seq_slot, (int)num_seqs, channels, taps, activation);
    b2l_count_launch();
    if (taps > 1)
      b2l_launch(conv_tail_update_kernel<T>, grid2, block, (size_t)0, st, (T*)tail, (const T*)in, in_row_stride,
                 (const int*)seq_start, (const int*)seq_ctx, (const int*)seq_slot, channels, taps);
  });
#undef B2L_CONV
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

extern "C" int b2l_ssm_scan(void* y_f32, void* state_f32, const void* xbc, int64_t xbc_row_stride, const void* dt_raw,
                            int64_t dt_row_stride, const void* dt_bias, const void* a_log, const void* d_skip,
                            const void* seq_start, const void* seq_ctx, const void* seq_slot, int64_t num_seqs,
                            int heads, int groups, int state_size, int head_dim, const void* fixed_decay_f32,
                            int silu_inputs, int dtype, void* stream) {
  B2L_REQUIRE(y_f32 && state_f32 && xbc && seq_start && seq_ctx && seq_slot, "ssm_scan: null pointer");
  B2L_REQUIRE(fixed_decay_f32 || (dt_raw && dt_bias && a_log && d_skip), "ssm_scan: null pointer");
  B2L_REQUIRE(heads > 0 && groups > 0 && heads % groups == 0 && state_size > 0 && head_dim > 0,
              "ssm_scan: bad geometry heads=%d groups=%d state=%d head_dim=%d", heads, groups, state_size, head_dim);
  B2L_REQUIRE(state_size <= 768, "ssm_scan: state size %d > 768", state_size);
  if (num_seqs <= 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  // two columns per lane when the head is wider than a warp and the state rows still fit 12 compute warps
  // (a state of up to 64 rows fits one warp's registers at one column per lane: no slices, no partial sums)
  const int cpl = (head_dim > 32 && state_size > 64 && state_size <= 384) ? 2 : 1;
  const int npt = state_size <= 16 ? 16 : ((state_size <= 32 || cpl == 2) ? 32 : 64);
  const int nslices = (state_size + npt - 1) / npt;
  int ctiles = (head_dim + 32 * cpl - 1) / (32 * cpl);
  const int room = 8 / nslices > 1 ? 8 / nslices : 1;      // compute warps <= 12 with the 4 loaders: <= 512 threads
  if (ctiles > room) ctiles = room;
  // the token loop of a CTA is serial, so the grid is all the parallelism there is: with sliced states (several
  // compute warps per column tile) narrower column tiles until two CTAs per SM are there to be had; B and C are then
  // staged once per tile, which the loader warps absorb.  (Unsliced states lose: one compute warp per four loaders.)
  while (cpl == 2 && ctiles > 1 && cdiv64(head_dim, (int64_t)ctiles * 32 * cpl) * heads * num_seqs < 2 * 148) --ctiles;
  const int cols = ctiles * 32 * cpl, np = nslices * npt;
  const size_t smem = (size_t)(2 * (2 * kChunk * np + kChunk * cols + 2 * kChunk) +
                               (nslices > 1 ? 2 * nslices * kChunk * cols : 0)) * sizeof(float);
  B2L_REQUIRE((int64_t)smem <= b2l_max_smem_optin(), "ssm_scan: state size %d needs %lld bytes of shared memory",
              state_size, (long long)smem);
  const dim3 block((ctiles * nslices + kLoadWarps) * 32), grid((unsigned)cdiv64(head_dim, cols), (unsigned)heads,
                                                               (unsigned)num_seqs);
#define B2L_SCAN(NPTV, CPLV)                                                                                         \
  do {                                                                                                               \
    static int cache[64] = {0};                                                                                      \
    B2L_CUDA_CHECK(b2l_ensure_dynamic_smem(ssm_scan_kernel<T, NPTV, CPLV>, (int)smem, cache));                       \
    b2l_launch(ssm_scan_kernel<T, NPTV, CPLV>, grid, block, smem, st, (float*)y_f32, (float*)state_f32,              \
               (const T*)xbc, xbc_row_stride, (const T*)dt_raw, dt_row_stride, (const T*)dt_bias, (const T*)a_log,   \
               (const T*)d_skip, (const int*)seq_start, (const int*)seq_ctx, (const int*)seq_slot, heads, groups,    \
               state_size, head_dim, ctiles, nslices, (const float*)fixed_decay_f32, silu_inputs);                   \
  } while (0)
  B2L_DISPATCH_FLOAT(dtype, "ssm_scan", {
    if (cpl == 2) {
      if (npt == 16) B2L_SCAN(16, 2);
      else B2L_SCAN(32, 2);
    } else {
      if (npt == 16) B2L_SCAN(16, 1);
      else if (npt == 32) B2L_SCAN(32, 1);
      else B2L_SCAN(64, 1);
    }
  });
#undef B2L_SCAN
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

extern "C" int b2l_gated_group_norm(void* out, const void* y_f32, const void* z, int64_t z_row_stride,
                                    const void* weight, int64_t rows, int inner, int groups, float eps, int dtype,
                                    void* stream) {
  B2L_REQUIRE(out && y_f32 && z && weight, "gated_group_norm: null pointer");
  B2L_REQUIRE(inner > 0 && groups > 0 && inner % groups == 0, "gated_group_norm: %d columns in %d groups", inner, groups);
  if (rows <= 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int gs = inner / groups;
  const int threads = gs >= 1024 ? 256 : (gs >= 256 ? 128 : (gs >= 64 ? 64 : 32));
  const int vpt = (gs + threads - 1) / threads;
  {
    int rc = 1;
    B2L_DISPATCH_FLOAT(dtype, "gated_group_norm", {
      constexpr int VEC = 16 / (int)sizeof(T);
      const bool vec = gs % VEC == 0 && z_row_stride % VEC == 0 && (uintptr_t)z % 16 == 0 && (uintptr_t)y_f32 % 16 == 0 &&
                       (uintptr_t)out % 16 == 0 && (uintptr_t)weight % 16 == 0;
      const int nvec = gs / VEC;
      int vth = ((nvec + 31) / 32) * 32;
      if (vth > 256) vth = 256;
      const int vpv = vec ? (nvec + vth - 1) / vth : 99;
      if (vpv <= 4) {
        const dim3 g2((unsigned)groups, (unsigned)rows), b2((unsigned)vth);
        if (vpv <= 1)
          b2l_launch(gated_group_norm_vec_kernel<T, 1>, g2, b2, (size_t)0, st, (T*)out, (const float*)y_f32, (const T*)z,
                     z_row_stride, (const T*)weight, inner, groups, eps);
        else if (vpv <= 2)
          b2l_launch(gated_group_norm_vec_kernel<T, 2>, g2, b2, (size_t)0, st, (T*)out, (const float*)y_f32, (const T*)z,
                     z_row_stride, (const T*)weight, inner, groups, eps);
        else
          b2l_launch(gated_group_norm_vec_kernel<T, 4>, g2, b2, (size_t)0, st, (T*)out, (const float*)y_f32, (const T*)z,
                     z_row_stride, (const T*)weight, inner, groups, eps);
        rc = 0;
      }
    });
    if (rc == 0) {
      B2L_LAUNCH_CHECK();
      return B2L_OK;
    }
  }
#define B2L_GGN(V)                                                                                                  \
  b2l_launch(gated_group_norm_kernel<T, V>, dim3((unsigned)groups, (unsigned)rows), dim3(threads), (size_t)0, st,  \
             (T*)out, (const float*)y_f32, (const T*)z, z_row_stride, (const T*)weight, inner, groups, eps)
  B2L_DISPATCH_FLOAT(dtype, "gated_group_norm", {
    if (vpt <= 1) B2L_GGN(1);
    else if (vpt <= 2) B2L_GGN(2);
    else if (vpt <= 4) B2L_GGN(4);
    else if (vpt <= 8) B2L_GGN(8);
    else B2L_GGN(0);
  });
#undef B2L_GGN
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}
