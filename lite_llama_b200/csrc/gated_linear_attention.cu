// Linear attention with data-dependent gates over RAGGED steps: per head an fp32 memory S [D x V] kept per request
// slot, advanced token by token, read out by the query.  Two recurrences share one kernel:
//
//   forget-gate (mode 0)   f = l + (1 - l) * sigmoid(z)         per key channel d, lower bound l in [0, 1)
//                          S[d, :] <- f[d] S[d, :] + (1 - f[d]) v;   o = S^T silu(q)
//                          (the forget gate also decides what is written: there is no separate key)
//   gated delta rule (1)   q, k unit vectors (x / sqrt(sum x^2 + unit_eps)), q times q_scale;
//                          beta = sigmoid(b), g = exp(-exp(A_log) * softplus(a + dt_bias))       per head
//                          S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//                          (the read-out sees the current token's write)
//
// 4 to 16 neighbouring lanes share one value column of one head and hold at most 16 of its D memory entries each in
// registers, so a contraction over D (S^T k, S^T q) is a sum inside a thread plus a few shuffles, nothing spills
// (87 to 128 registers with the prefetched rows: two CTAs of 8 warps per SM), and several times the threads work on a
// head than with one thread per value column.  The delta rule's two
// contractions both read the memory before the token's write (S'^T q = g S^T q + u (k . q)), so they run side by side.
// A CTA = (256 / lanes value columns, head, sequence) stages 16 tokens at a time in one of two buffers: the token's
// gates, unit norms and scalars are evaluated in fp32 by the warps in parallel and left in shared memory with the
// round's v columns; the next round's rows are fetched into registers before the current round's 16 updates run back
// to back.  A sequence without cached tokens starts from zero and never
// reads its slot; every sequence writes its slot at the end of the step.
//
//   head_norm_gate   out[t, h, :] = unit_rms(y[t, h, :]) * w * (silu(gate[t, h, :]) or 1): the per-head output norm
//                    (weight [V] shared by the heads) with an optional SiLU gate AFTER the norm
//   head_mix         out[t, h, :] = sum_g M[h, g] * wide[t, g, kv(h), :]: attention weights mixed ACROSS heads after
//                    the softmax, done on per-head outputs -- head g's weights were applied to every kv head's values
//                    (sum_j (sum_g M[h,g] p_g(j)) v(j) = sum_g M[h,g] (sum_j p_g(j) v(j)))
//   swiglu_scaled    out[r, :] = silu(s_r * gate) * (s_r * up) * sigmoid(z_r): a gated activation whose INPUT carries
//                    a per-row fp32 factor (an expert weight on the expert's input: W (s x) = s (W x)) and whose output
//                    a per-row logistic gate (both optional)
#include "common.cuh"
#include "rowvec.cuh"

namespace {

__device__ __forceinline__ float gla_sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float gla_silu(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float gla_softplus(float v) { return v > 20.f ? v : log1pf(expf(v)); }

constexpr int kTok = 16;                  // tokens staged per round

struct GlaArgs {
  float* y; float* state;
  const void* q; int64_t q_stride;        // [tokens, QH * D]
  const void* k; int64_t k_stride;        // mode 1: keys [tokens, QH * D]; mode 0: forget-gate logits [tokens, H * D]
  const void* v; int64_t v_stride;        // [tokens, H * V]
  const void* p0; int64_t p0_stride;      // mode 1: write-strength logits [tokens, H]
  const void* p1; int64_t p1_stride;      // mode 1: decay logits [tokens, H]
  const void* c0;                         // mode 1: dt_bias [H];  mode 0: lower bounds [H * D]
  const void* c1;                         // mode 1: A_log [H]
  const int* seq_start; const int* seq_ctx; const int* seq_slot;
  int H, QH, D, V;
  float q_scale, unit_eps;
};

constexpr int kScanThreads = 256;
// lanes that share one value column (neighbouring lanes): each holds at most 16 memory rows, so nothing spills and a
// head's update is spread over 4 to 16 times the threads of one-thread-per-column
constexpr int scan_parts(int dp) { return dp <= 64 ? 4 : dp / 16; }

template <typename T, int DP, int MODE, int C>
__global__ void __launch_bounds__(kScanThreads, 2) gated_linear_scan_kernel(GlaArgs a) {
  pdl_prologue();
  constexpr int PARTS = scan_parts(DP);
  constexpr int R4 = DP / (4 * PARTS);              // float4 groups of memory rows per thread
  // C value columns per thread: a staged k / q entry read from shared memory feeds C memories
  constexpr int COLS = kScanThreads / PARTS * C;
  constexpr int TOK = DP > 128 ? 8 : kTok;          // tokens per round
  constexpr int NW = kScanThreads / 32;
  constexpr int TPW = TOK / NW;                     // tokens a warp prepares per round
  constexpr int NI = (DP + 31) / 32;
  constexpr int NA = C == 1 ? 4 : 2;                // partial sums of a contraction inside a thread (chains of D / (PARTS NA) products)
  constexpr int NV = (TOK * COLS + kScanThreads - 1) / kScanThreads;   // v entries a thread fetches per round
  // two rounds of staged tokens: the next round's rows are fetched into registers before the current round's updates
  // run, and prepared (gates, unit norms) into the other buffer after them, so their latency hides behind the updates
  __shared__ __align__(16) float qs[2][TOK * DP];
  __shared__ __align__(16) float ks[2][TOK * DP];   // mode 1: unit keys; mode 0: forget gates
  __shared__ float vs[2][TOK * COLS];
  __shared__ float sc[2][TOK * 4];                  // mode 1: (g, beta, k . q) per token
  const int D = a.D, V = a.V, H = a.H;
  const int h = blockIdx.y, s = blockIdx.z;
  const int qh = h / (H / a.QH);
  const int part = threadIdx.x & (PARTS - 1), lcol = threadIdx.x / PARTS * C;
  const int col = blockIdx.x * COLS + lcol;          // the thread's first column
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int start = a.seq_start[s], len = a.seq_start[s + 1] - start, ctx = a.seq_ctx[s];
  const int64_t slot = a.seq_slot[s];
  float* sp = a.state + ((slot * H + h) * (int64_t)D) * V;
  // thread (col, part) holds rows d = 4 PARTS i + 4 part + e (i < R4, e < 4): the parts of a column read neighbouring
  // float4 of a staged vector, so a warp's reads fall in different banks
  float S[C][R4 * 4];
#pragma unroll
  for (int c = 0; c < C; ++c)
#pragma unroll
    for (int i = 0; i < R4; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int d = 4 * PARTS * i + 4 * part + e;
        S[c][4 * i + e] = (ctx > 0 && col + c < V && d < D) ? sp[(int64_t)d * V + col + c] : 0.f;
      }
  const T* qp = (const T*)a.q;
  const T* kp = (const T*)a.k;
  const T* vp = (const T*)a.v;
  float neg_a = 0.f, dtb = 0.f;
  if (MODE == 1) { neg_a = -expf(to_f32(((const T*)a.c1)[h])); dtb = to_f32(((const T*)a.c0)[h]); }
  float rq[TPW][NI], rk[TPW][NI], rs0[TPW], rs1[TPW], rv[NV];

  auto fetch = [&](int t0) {                         // raw rows of round t0 -> registers (loads stay in flight)
    const int nt = min(TOK, len - t0);
#pragma unroll
    for (int j = 0; j < TPW; ++j) {
      const int t = warp + NW * j;
      const int64_t row = start + t0 + t;
      const int hq = MODE == 1 ? qh : h;
#pragma unroll
      for (int i = 0; i < NI; ++i) {
        const int d = lane + 32 * i;
        const bool in = t < nt && d < D;
        rq[j][i] = in ? to_f32(qp[row * a.q_stride + hq * D + d]) : 0.f;
        rk[j][i] = in ? to_f32(kp[row * a.k_stride + hq * D + d]) : 0.f;
      }
      rs0[j] = rs1[j] = 0.f;
      if (MODE == 1 && t < nt && lane == 0) {
        rs0[j] = to_f32(((const T*)a.p0)[row * a.p0_stride + h]);
        rs1[j] = to_f32(((const T*)a.p1)[row * a.p1_stride + h]);
      }
    }
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = threadIdx.x + kScanThreads * j;
      const int t = i / COLS, c = blockIdx.x * COLS + (i - t * COLS);
      rv[j] = (t < nt && c < V) ? to_f32(vp[(int64_t)(start + t0 + t) * a.v_stride + h * V + c]) : 0.f;
    }
  };
  auto stage = [&](int buf) {                        // registers -> gates / unit vectors in shared memory
#pragma unroll
    for (int j = 0; j < TPW; ++j) {
      const int t = warp + NW * j;
      if (MODE == 1) {
        float sq = 0.f, sk = 0.f, qk = 0.f;
#pragma unroll
        for (int i = 0; i < NI; ++i) {
          sq = fmaf(rq[j][i], rq[j][i], sq); sk = fmaf(rk[j][i], rk[j][i], sk); qk = fmaf(rq[j][i], rk[j][i], qk);
        }
        const float nq = a.q_scale / sqrtf(warp_reduce_sum(sq) + a.unit_eps);
        const float nk = 1.0f / sqrtf(warp_reduce_sum(sk) + a.unit_eps);
        qk = warp_reduce_sum(qk) * nq * nk;
#pragma unroll
        for (int i = 0; i < NI; ++i) {
          const int d = lane + 32 * i;
          if (d < DP) { qs[buf][t * DP + d] = rq[j][i] * nq; ks[buf][t * DP + d] = rk[j][i] * nk; }
        }
        if (lane == 0) {
          sc[buf][4 * t] = expf(neg_a * gla_softplus(rs1[j] + dtb));
          sc[buf][4 * t + 1] = gla_sigmoid(rs0[j]);
          sc[buf][4 * t + 2] = qk;
        }
      } else {
#pragma unroll
        for (int i = 0; i < NI; ++i) {
          const int d = lane + 32 * i;
          // rows beyond D: nothing written (f = 1 keeps the zero), nothing read (q = 0)
          const float lo = d < D ? to_f32(((const T*)a.c0)[h * D + d]) : 0.f;
          const float f = d < D ? lo + (1.0f - lo) * gla_sigmoid(rk[j][i]) : 1.f;
          if (d < DP) { qs[buf][t * DP + d] = d < D ? gla_silu(rq[j][i]) : 0.f; ks[buf][t * DP + d] = f; }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int i = threadIdx.x + kScanThreads * j;
      if (i < TOK * COLS) vs[buf][i] = rv[j];
    }
  };
  auto column_sum = [&](float x) {                   // over the lanes of one column
#pragma unroll
    for (int m = 1; m < PARTS; m <<= 1) x += __shfl_xor_sync(0xffffffffu, x, m);
    return x;
  };

  if (len > 0) { fetch(0); stage(0); }
  __syncthreads();
  int buf = 0;
  for (int t0 = 0; t0 < len; t0 += TOK, buf ^= 1) {
    const int nt = min(TOK, len - t0);
    const bool more = t0 + TOK < len;
    if (more) fetch(t0 + TOK);
#pragma unroll 2
    for (int t = 0; t < nt; ++t) {
      const float4* q4 = reinterpret_cast<const float4*>(qs[buf] + t * DP) + part;
      const float4* k4 = reinterpret_cast<const float4*>(ks[buf] + t * DP) + part;
      float x[C], o[C];
#pragma unroll
      for (int c = 0; c < C; ++c) x[c] = vs[buf][t * COLS + lcol + c];
      if (MODE == 1) {
        // both contractions read the memory BEFORE the token's write, so they run side by side:
        //   S' = g S + k u^T,  u = beta (v - g S^T k);   S'^T q = g S^T q + u (k . q)
        const float g = sc[buf][4 * t], beta = sc[buf][4 * t + 1], kq = sc[buf][4 * t + 2];
        float4 kk[R4];
        float dk[C][NA], dq[C][NA];
#pragma unroll
        for (int c = 0; c < C; ++c)
#pragma unroll
          for (int e = 0; e < NA; ++e) dk[c][e] = dq[c][e] = 0.f;
#pragma unroll
        for (int i = 0; i < R4; ++i) {
          kk[i] = k4[PARTS * i];
          const float4 qq = q4[PARTS * i];
#pragma unroll
          for (int c = 0; c < C; ++c) {
            dk[c][0] = fmaf(S[c][4 * i], kk[i].x, dk[c][0]); dk[c][1] = fmaf(S[c][4 * i + 1], kk[i].y, dk[c][1]);
            dk[c][2 % NA] = fmaf(S[c][4 * i + 2], kk[i].z, dk[c][2 % NA]); dk[c][3 % NA] = fmaf(S[c][4 * i + 3], kk[i].w, dk[c][3 % NA]);
            dq[c][0] = fmaf(S[c][4 * i], qq.x, dq[c][0]); dq[c][1] = fmaf(S[c][4 * i + 1], qq.y, dq[c][1]);
            dq[c][2 % NA] = fmaf(S[c][4 * i + 2], qq.z, dq[c][2 % NA]); dq[c][3 % NA] = fmaf(S[c][4 * i + 3], qq.w, dq[c][3 % NA]);
          }
        }
#pragma unroll
        for (int c = 0; c < C; ++c) {
          const float dot = column_sum(NA == 4 ? (dk[c][0] + dk[c][1]) + (dk[c][2 % NA] + dk[c][3 % NA]) : dk[c][0] + dk[c][1]);
          const float rd = column_sum(NA == 4 ? (dq[c][0] + dq[c][1]) + (dq[c][2 % NA] + dq[c][3 % NA]) : dq[c][0] + dq[c][1]);
          const float u = beta * (x[c] - g * dot);
          o[c] = fmaf(g, rd, u * kq);
#pragma unroll
          for (int i = 0; i < R4; ++i) {
            S[c][4 * i] = fmaf(g, S[c][4 * i], kk[i].x * u); S[c][4 * i + 1] = fmaf(g, S[c][4 * i + 1], kk[i].y * u);
            S[c][4 * i + 2] = fmaf(g, S[c][4 * i + 2], kk[i].z * u); S[c][4 * i + 3] = fmaf(g, S[c][4 * i + 3], kk[i].w * u);
          }
        }
      } else {
        float oa[C][NA];
#pragma unroll
        for (int c = 0; c < C; ++c)
#pragma unroll
          for (int e = 0; e < NA; ++e) oa[c][e] = 0.f;
#pragma unroll
        for (int i = 0; i < R4; ++i) {                // f S + (1 - f) x = x + f (S - x)
          const float4 ff = k4[PARTS * i], qq = q4[PARTS * i];
#pragma unroll
          for (int c = 0; c < C; ++c) {
            S[c][4 * i] = fmaf(ff.x, S[c][4 * i] - x[c], x[c]); S[c][4 * i + 1] = fmaf(ff.y, S[c][4 * i + 1] - x[c], x[c]);
            S[c][4 * i + 2] = fmaf(ff.z, S[c][4 * i + 2] - x[c], x[c]); S[c][4 * i + 3] = fmaf(ff.w, S[c][4 * i + 3] - x[c], x[c]);
            oa[c][0] = fmaf(S[c][4 * i], qq.x, oa[c][0]); oa[c][1] = fmaf(S[c][4 * i + 1], qq.y, oa[c][1]);
            oa[c][2 % NA] = fmaf(S[c][4 * i + 2], qq.z, oa[c][2 % NA]); oa[c][3 % NA] = fmaf(S[c][4 * i + 3], qq.w, oa[c][3 % NA]);
          }
        }
#pragma unroll
        for (int c = 0; c < C; ++c)
          o[c] = column_sum(NA == 4 ? (oa[c][0] + oa[c][1]) + (oa[c][2 % NA] + oa[c][3 % NA]) : oa[c][0] + oa[c][1]);
      }
      if (part == 0) {
#pragma unroll
        for (int c = 0; c < C; ++c)
          if (col + c < V) a.y[(int64_t)(start + t0 + t) * H * V + h * V + col + c] = o[c];
      }
    }
    if (more) stage(buf ^ 1);
    __syncthreads();
  }
#pragma unroll
  for (int c = 0; c < C; ++c)
#pragma unroll
    for (int i = 0; i < R4; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int d = 4 * PARTS * i + 4 * part + e;
        if (col + c < V && d < D) sp[(int64_t)d * V + col + c] = S[c][4 * i + e];
      }
}

template <typename T>
__global__ void __launch_bounds__(128) head_norm_gate_kernel(T* __restrict__ out, const float* __restrict__ y,
                                                             const T* __restrict__ gate, int64_t gs,
                                                             const T* __restrict__ w, int heads, int V, float eps,
                                                             int vec) {
  pdl_prologue();
  const int64_t t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int h = warp; h < heads; h += nw) {
    const float* yr = y + (t * heads + h) * (int64_t)V;
    float ss = 0.f;
    if (vec) {                                       // 4 elements per access
      for (int i = lane * 4; i < V; i += 128) {
        float v[4];
        row_load4(yr + i, v);
#pragma unroll
        for (int c = 0; c < 4; ++c) ss = fmaf(v[c], v[c], ss);
      }
      const float rstd = 1.0f / sqrtf(warp_reduce_sum(ss) / (float)V + eps);
      for (int i = lane * 4; i < V; i += 128) {
        float v[4], g[4];
        row_load4(yr + i, v);
        row_load4(w + i, g);
#pragma unroll
        for (int c = 0; c < 4; ++c) v[c] = v[c] * rstd * g[c];
        if (gate) {
          row_load4(gate + t * gs + (int64_t)h * V + i, g);
#pragma unroll
          for (int c = 0; c < 4; ++c) v[c] *= gla_silu(g[c]);
        }
        row_store4(out + (t * heads + h) * (int64_t)V + i, v);
      }
      continue;
    }
    for (int i = lane; i < V; i += 32) { const float v = yr[i]; ss = fmaf(v, v, ss); }
    const float rstd = 1.0f / sqrtf(warp_reduce_sum(ss) / (float)V + eps);
    for (int i = lane; i < V; i += 32) {
      float v = yr[i] * rstd * to_f32(w[i]);
      if (gate) v *= gla_silu(to_f32(gate[t * gs + (int64_t)h * V + i]));
      out[(t * heads + h) * (int64_t)V + i] = from_f32<T>(v);
    }
  }
}

template <typename T>
__global__ void head_mix_kernel(T* __restrict__ out, const T* __restrict__ wide, int64_t wide_stride,
                                const T* __restrict__ mix, int heads, int kv_heads, int per_call, int Dv,
                                int64_t total) {
  pdl_prologue();
  const int per = heads / kv_heads;
  const int64_t call_stride = (int64_t)heads * per_call * Dv;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int i = (int)(idx % Dv);
    const int h = (int)((idx / Dv) % heads);
    const int64_t t = idx / ((int64_t)Dv * heads);
    const int c = h / per;
    const T* src = wide + t * wide_stride + (c / per_call) * call_stride + (int64_t)(c % per_call) * Dv + i;
    float acc = 0.f;
    for (int g = 0; g < heads; ++g) acc = fmaf(to_f32(mix[h * heads + g]), to_f32(src[(int64_t)g * per_call * Dv]), acc);
    out[idx] = from_f32<T>(acc);
  }
}

// the same with 4 value columns per thread (vdim and the row stride multiples of 4, aligned pointers)
template <typename T>
__global__ void head_mix_vec_kernel(T* __restrict__ out, const T* __restrict__ wide, int64_t wide_stride,
                                    const T* __restrict__ mix, int heads, int kv_heads, int per_call, int Dv,
                                    int64_t total4) {
  pdl_prologue();
  const int per = heads / kv_heads, q4 = Dv / 4;
  const int64_t call_stride = (int64_t)heads * per_call * Dv;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total4; idx += (int64_t)gridDim.x * blockDim.x) {
    const int i = (int)(idx % q4) * 4;
    const int h = (int)((idx / q4) % heads);
    const int64_t t = idx / ((int64_t)q4 * heads);
    const int c = h / per;
    const T* src = wide + t * wide_stride + (c / per_call) * call_stride + (int64_t)(c % per_call) * Dv + i;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int g = 0; g < heads; ++g) {
      float v[4];
      row_load4(src + (int64_t)g * per_call * Dv, v);
      const float m = to_f32(mix[h * heads + g]);
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[e] = fmaf(m, v[e], acc[e]);
    }
    row_store4(out + (t * heads + h) * (int64_t)Dv + i, acc);
  }
}

// the same with one thread per (token, kv head, 4 value columns) forming ALL the PER output heads of that kv head: a
// wide element is loaded once instead of once per output head; every output is the same g-ascending sum as above
template <typename T, int PER>
__global__ void head_mix_group_kernel(T* __restrict__ out, const T* __restrict__ wide, int64_t wide_stride,
                                      const T* __restrict__ mix, int heads, int kv_heads, int per_call, int Dv,
                                      int64_t total4) {
  pdl_prologue();
  const int q4 = Dv / 4;
  const int64_t call_stride = (int64_t)heads * per_call * Dv, g_stride = (int64_t)per_call * Dv;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total4; idx += (int64_t)gridDim.x * blockDim.x) {
    const int i = (int)(idx % q4) * 4;
    const int c = (int)((idx / q4) % kv_heads);
    const int64_t t = idx / ((int64_t)q4 * kv_heads);
    const T* src = wide + t * wide_stride + (c / per_call) * call_stride + (int64_t)(c % per_call) * Dv + i;
    const T* mrow = mix + (int64_t)c * PER * heads;
    float acc[PER][4];
#pragma unroll
    for (int r = 0; r < PER; ++r)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[r][e] = 0.f;
#pragma unroll 4
    for (int g = 0; g < heads; ++g) {
      float v[4];
      row_load4(src + g * g_stride, v);
#pragma unroll
      for (int r = 0; r < PER; ++r) {
        const float m = to_f32(mrow[r * heads + g]);
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[r][e] = fmaf(m, v[e], acc[r][e]);
      }
    }
#pragma unroll
    for (int r = 0; r < PER; ++r) row_store4(out + (t * heads + c * PER + r) * (int64_t)Dv + i, acc[r]);
  }
}

template <typename T>
__global__ void swiglu_scaled_vec_kernel(T* __restrict__ out, int64_t os, const T* __restrict__ gate, int64_t gs,
                                         const T* __restrict__ up, int64_t us, const float* __restrict__ in_scale,
                                         const T* __restrict__ z, int64_t zs, int64_t n4, int64_t total4) {
  pdl_prologue();
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total4; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / n4, i = (idx - r * n4) * 4;
    const float s = in_scale ? in_scale[r] : 1.0f;
    const float zo = z ? gla_sigmoid(to_f32(z[r * zs])) : 1.0f;
    float g[4], u[4];
    row_load4(gate + r * gs + i, g);
    row_load4(up + r * us + i, u);
#pragma unroll
    for (int e = 0; e < 4; ++e) g[e] = gla_silu(s * g[e]) * (s * u[e]) * zo;
    row_store4(out + r * os + i, g);
  }
}

template <typename T>
__global__ void swiglu_scaled_kernel(T* __restrict__ out, int64_t os, const T* __restrict__ gate, int64_t gs,
                                     const T* __restrict__ up, int64_t us, const float* __restrict__ in_scale,
                                     const T* __restrict__ z, int64_t zs, int64_t n, int64_t total) {
  pdl_prologue();
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / n, i = idx - r * n;
    const float s = in_scale ? in_scale[r] : 1.0f;
    const float g = s * to_f32(gate[r * gs + i]), u = s * to_f32(up[r * us + i]);
    const float zo = z ? gla_sigmoid(to_f32(z[r * zs])) : 1.0f;
    out[r * os + i] = from_f32<T>(gla_silu(g) * u * zo);
  }
}

template <typename T, int MODE>
int launch_scan(const GlaArgs& a, int64_t num_seqs, cudaStream_t st) {
  // two columns per thread halve the shared-memory reads per update; one column per thread gives twice the CTAs, which
  // matters more while the grid does not fill the SMs
  const auto ctas = [&](int dp, int c) {
    const int cols = kScanThreads / scan_parts(dp) * c;
    return (int64_t)((a.V + cols - 1) / cols) * a.H * num_seqs;
  };
#define B2L_GLA_C(DPV, CV)                                                                               \
  do {                                                                                                   \
    constexpr int cols = kScanThreads / scan_parts(DPV) * CV;                                            \
    const dim3 grid((unsigned)((a.V + cols - 1) / cols), (unsigned)a.H, (unsigned)num_seqs);             \
    b2l_launch(gated_linear_scan_kernel<T, DPV, MODE, CV>, grid, dim3(kScanThreads), (size_t)0, st, a);  \
  } while (0)
#define B2L_GLA(DPV)                                                                                     \
  do {                                                                                                   \
    if (ctas(DPV, 2) >= b2l_num_sms()) B2L_GLA_C(DPV, 2);                                               \
    else B2L_GLA_C(DPV, 1);                                                                              \
  } while (0)
  if (a.D <= 16) B2L_GLA(16);
  else if (a.D <= 32) B2L_GLA(32);
  else if (a.D <= 64) B2L_GLA(64);
  else if (a.D <= 128) B2L_GLA(128);
  else B2L_GLA(256);
#undef B2L_GLA_C
#undef B2L_GLA
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

}  // namespace

/* mode 0: forget-gate linear attention (q [tokens, heads*dim] pre-activation, k = forget-gate logits [tokens, heads*dim],
 * c0 = lower bounds [heads*dim]); mode 1: gated delta rule (q, k [tokens, qk_heads*dim] after their activation, p0 =
 * write-strength logits, p1 = decay logits [tokens, heads], c0 = dt_bias, c1 = A_log [heads]).  v [tokens, heads*vdim];
 * y_f32 [tokens, heads*vdim]; state_f32 [slots, heads, dim, vdim] advanced in place. */
extern "C" int b2l_gated_linear_scan(void* y_f32, void* state_f32, const void* q, int64_t q_row_stride, const void* k,
                                     int64_t k_row_stride, const void* v, int64_t v_row_stride, const void* p0,
                                     int64_t p0_row_stride, const void* p1, int64_t p1_row_stride, const void* c0,
                                     const void* c1, const void* seq_start, const void* seq_ctx, const void* seq_slot,
                                     int64_t num_seqs, int heads, int qk_heads, int dim, int vdim, float q_scale,
                                     float unit_eps, int mode, int dtype, void* stream) {
  B2L_REQUIRE(y_f32 && state_f32 && q && k && v && c0 && seq_start && seq_ctx && seq_slot, "gated_linear_scan: null pointer");
  B2L_REQUIRE(mode == 0 || (p0 && p1 && c1), "gated_linear_scan: the delta rule needs its gates");
  B2L_REQUIRE(heads > 0 && qk_heads > 0 && heads % qk_heads == 0 && dim > 0 && dim <= 256 && vdim > 0,
              "gated_linear_scan: %d heads, %d q/k heads, sizes %d x %d", heads, qk_heads, dim, vdim);
  B2L_REQUIRE(mode == 1 || qk_heads == heads, "gated_linear_scan: the forget-gate form has one query head per head");
  if (num_seqs <= 0) return B2L_OK;
  GlaArgs a;
  a.y = (float*)y_f32; a.state = (float*)state_f32;
  a.q = q; a.q_stride = q_row_stride; a.k = k; a.k_stride = k_row_stride; a.v = v; a.v_stride = v_row_stride;
  a.p0 = p0; a.p0_stride = p0_row_stride; a.p1 = p1; a.p1_stride = p1_row_stride; a.c0 = c0; a.c1 = c1;
  a.seq_start = (const int*)seq_start; a.seq_ctx = (const int*)seq_ctx; a.seq_slot = (const int*)seq_slot;
  a.H = heads; a.QH = qk_heads; a.D = dim; a.V = vdim; a.q_scale = q_scale; a.unit_eps = unit_eps;
  cudaStream_t st = (cudaStream_t)stream;
  int rc = B2L_OK;
  B2L_DISPATCH_FLOAT(dtype, "gated_linear_scan", {
    rc = mode == 0 ? launch_scan<T, 0>(a, num_seqs, st) : launch_scan<T, 1>(a, num_seqs, st);
  });
  return rc;
}

extern "C" int b2l_head_norm_gate(void* out, const void* y_f32, const void* gate, int64_t gate_row_stride,
                                  const void* weight, int64_t rows, int heads, int vdim, float eps, int dtype,
                                  void* stream) {
  B2L_REQUIRE(out && y_f32 && weight, "head_norm_gate: null pointer");
  B2L_REQUIRE(heads > 0 && vdim > 0, "head_norm_gate: bad shape");
  if (rows <= 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int threads = heads >= 4 ? 128 : heads * 32;
  B2L_DISPATCH_FLOAT(dtype, "head_norm_gate", {
    b2l_launch(head_norm_gate_kernel<T>, dim3((unsigned)rows), dim3(threads), (size_t)0, st, (T*)out, (const float*)y_f32,
               (const T*)gate, gate_row_stride, (const T*)weight, heads, vdim, eps,
               (int)(vdim % 4 == 0 && gate_row_stride % 4 == 0 && row_aligned4<T>(out) && row_aligned4<T>(gate) &&
                     row_aligned4<T>(weight) && (uintptr_t)y_f32 % 16 == 0));
  });
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

/* wide [rows, calls, heads, per_call, vdim] (row stride given): query head g's softmax weights applied to the values of
 * kv head c lie at call c / per_call, head g, part c % per_call.  out[t, h, :] = sum_g mix[h, g] * wide[t, g, kv(h), :]. */
extern "C" int b2l_head_mix(void* out, const void* wide, int64_t wide_row_stride, const void* mix, int64_t rows,
                            int heads, int kv_heads, int per_call, int vdim, int dtype, void* stream) {
  B2L_REQUIRE(out && wide && mix, "head_mix: null pointer");
  B2L_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && per_call > 0 && kv_heads % per_call == 0 && vdim > 0,
              "head_mix: bad shape");
  if (rows <= 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t total = rows * heads * vdim;
#define B2L_MIX_GROUP(P)                                                                                       \
  b2l_launch(head_mix_group_kernel<T, P>, dim3(grid), dim3(256), (size_t)0, st, (T*)out, (const T*)wide,        \
             wide_row_stride, (const T*)mix, heads, kv_heads, per_call, vdim, items)
  B2L_DISPATCH_FLOAT(dtype, "head_mix", {
    if (vdim % 4 == 0 && wide_row_stride % 4 == 0 && row_aligned4<T>(out) && row_aligned4<T>(wide)) {
      const int per = heads / kv_heads;
      const int64_t items = (per == 2 || per == 4 || per == 8) ? total / 4 / per : total / 4;
      const unsigned grid = (unsigned)(cdiv64(items, 256) < 148 * 16 ? cdiv64(items, 256) : 148 * 16);
      if (per == 2) B2L_MIX_GROUP(2);
      else if (per == 4) B2L_MIX_GROUP(4);
      else if (per == 8) B2L_MIX_GROUP(8);
      else
        b2l_launch(head_mix_vec_kernel<T>, dim3(grid), dim3(256), (size_t)0, st, (T*)out, (const T*)wide, wide_row_stride,
                   (const T*)mix, heads, kv_heads, per_call, vdim, total / 4);
    } else {
      const unsigned grid = (unsigned)(cdiv64(total, 256) < 148 * 16 ? cdiv64(total, 256) : 148 * 16);
      b2l_launch(head_mix_kernel<T>, dim3(grid), dim3(256), (size_t)0, st, (T*)out, (const T*)wide, wide_row_stride,
                 (const T*)mix, heads, kv_heads, per_call, vdim, total);
    }
  });
#undef B2L_MIX_GROUP
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

extern "C" int b2l_swiglu_scaled(void* out, int64_t out_row_stride, const void* gate, int64_t gate_row_stride,
                                 const void* up, int64_t up_row_stride, const void* in_scale_f32, const void* z,
                                 int64_t z_row_stride, int64_t rows, int64_t n, int dtype, void* stream) {
  B2L_REQUIRE(out && gate && up, "swiglu_scaled: null pointer");
  B2L_REQUIRE(n > 0, "swiglu_scaled: bad shape");
  if (rows <= 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t total = rows * n;
  B2L_DISPATCH_FLOAT(dtype, "swiglu_scaled", {
    if (n % 4 == 0 && out_row_stride % 4 == 0 && gate_row_stride % 4 == 0 && up_row_stride % 4 == 0 &&
        row_aligned4<T>(out) && row_aligned4<T>(gate) && row_aligned4<T>(up)) {
      const unsigned grid = (unsigned)(cdiv64(total / 4, 256) < 148 * 32 ? cdiv64(total / 4, 256) : 148 * 32);
      b2l_launch(swiglu_scaled_vec_kernel<T>, dim3(grid), dim3(256), (size_t)0, st, (T*)out, out_row_stride,
                 (const T*)gate, gate_row_stride, (const T*)up, up_row_stride, (const float*)in_scale_f32, (const T*)z,
                 z_row_stride, n / 4, total / 4);
    } else {
      const unsigned grid = (unsigned)(cdiv64(total, 256) < 148 * 16 ? cdiv64(total, 256) : 148 * 16);
      b2l_launch(swiglu_scaled_kernel<T>, dim3(grid), dim3(256), (size_t)0, st, (T*)out, out_row_stride, (const T*)gate,
                 gate_row_stride, (const T*)up, up_row_stride, (const float*)in_scale_f32, (const T*)z, z_row_stride, n,
                 total);
    }
  });
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}
