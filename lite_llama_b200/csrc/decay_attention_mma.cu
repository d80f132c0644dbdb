// Decayed linear attention over prompt portions on the tensor cores (16-bit activations): per head a memory S [N, P]
// (fp32, one per request slot, the layout of the scan in ssm_scan.cu) and
//     S_t = d S_(t-1) + k_t v_t^T,   y_t = S_t^T q_t,     q, k, v = SiLU of the projection columns.
// The scan walks a sequence token by token; here a CTA = (head, sequence) walks it in CHUNKS of 64 tokens, and a chunk
// is four products on mma.sync m16n8k16 tiles:
//     A = Q K^T                       scores of the chunk against itself (fp32 accumulators)
//     W[i, j] = d^(i-j) A[i, j]       j <= i, else 0 (fp32)
//     Y = W V + diag(d^(i+1)) Q S     inside the chunk + what the memory carried in
//     S <- d^n S + K^T (diag(d^(n-1-j)) V)     n = tokens of the chunk
// Every fp32 factor that enters a product (W, S, the scaled V) goes in as the sum of two 16-bit halves (hi + lo, two
// mma each), so nothing but SiLU(q), SiLU(k), SiLU(v) themselves is rounded to 16 bits; the memory and all sums stay
// fp32.  Rows of x: [v: H*P | k: H*N | q: H*N] (the scan's [x | B | C] with one group per head).
// N, P in {32, 64, 128}; 16-byte aligned rows.  Other shapes, fp32 activations and single tokens take the scan.
// The value columns of a head may be cut over several CTAs (blockIdx.z; each repeats the scores and owns its columns
// of V, S and y): the walk over a sequence is serial, so columns are the only parallelism beyond heads x sequences.
#include "common.cuh"

namespace {

constexpr int kC = 64;          // tokens per chunk
constexpr int kDaWarps = 4;

__device__ __forceinline__ float silu_da(float v) { return v / (1.0f + __expf(-v)); }

// (a, b) as two packed 16-bit pairs whose sum is (a, b) to ~16 mantissa bits
template <typename T>
__device__ __forceinline__ void split2(float a, float b, uint32_t& hi, uint32_t& lo) {
  const T ha = from_f32<T>(a), hb = from_f32<T>(b);
  hi = pack2<T>(to_f32(ha), to_f32(hb));
  lo = pack2<T>(a - to_f32(ha), b - to_f32(hb));
}

struct DaArgs {
  float* y; float* state; const void* x; int64_t x_stride;
  const float* decay; const int* seq_start; const int* seq_ctx; const int* seq_slot;
  int H, Pfull;                // Pfull: value columns of a head (a CTA serves P of them, from blockIdx.z * P)
};

template <typename T, int N, int P>
__global__ void __launch_bounds__(kDaWarps * 32) decay_attention_mma_kernel(DaArgs a) {
  pdl_prologue();
  extern __shared__ __align__(16) uint8_t da_smem[];
  constexpr int QP = (N + 8) * 2, VP = (P + 8) * 2;           // row pitches in bytes (16-bit tiles)
  constexpr int SP = P + 4;                                    // fp32 memory pitch in floats
  uint8_t* sQ = da_smem;                                       // [kC][N + 8]
  uint8_t* sK = sQ + kC * QP;
  uint8_t* sV = sK + kC * QP;                                  // [kC][P + 8]  SiLU(v)
  uint8_t* sVh = sV + kC * VP;                                 // scaled by d^(n-1-j): high halves
  uint8_t* sVl = sVh + kC * VP;                                // low halves
  float* sS = reinterpret_cast<float*>(sVl + kC * VP);         // [N][SP]
  float* dpw = sS + N * SP;                                    // d^e, e = 0 .. kC
  const int h = blockIdx.x, s = blockIdx.y, H = a.H, Pf = a.Pfull, p0 = blockIdx.z * P;
  const int start = a.seq_start[s], len = a.seq_start[s + 1] - start, ctx = a.seq_ctx[s];
  if (len <= 0) return;
  const int64_t slot = a.seq_slot[s];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gq = lane >> 2, tq = lane & 3;
  const float d = a.decay[h];
  float* st = a.state + ((slot * H + h) * (int64_t)N) * Pf + p0;
  for (int e = tid; e <= kC; e += blockDim.x)
    dpw[e] = e == 0 ? 1.0f : (d <= 0.f ? 0.f : exp2f((float)e * log2f(d)));
  for (int i = tid; i < N * P; i += blockDim.x) {
    const int n = i / P, p = i - n * P;
    sS[n * SP + p] = ctx > 0 ? st[n * Pf + p] : 0.f;
  }
  const T* x = (const T*)a.x;
  const int inner = H * Pf;
  const int64_t voff = (int64_t)h * Pf + p0, koff = (int64_t)inner + (int64_t)h * N, qoff = (int64_t)inner + (int64_t)H * N + (int64_t)h * N;
  bool carried = ctx > 0;                                      // the memory is non-zero
  // A chunk's rows travel global -> registers -> (SiLU, scaling, halves) -> shared memory; the loads of the NEXT chunk
  // are issued before the products of the current one and land while they run.
  constexpr int QV = kC * (N / 8) / (kDaWarps * 32), VV = kC * (P / 8) / (kDaWarps * 32);
  uint4 pq[QV], pk[QV], pv[VV];
  auto fetch = [&](int c0) {
    const int cnt = min(kC, len - c0);
#pragma unroll
    for (int u = 0; u < QV; ++u) {
      const int i = tid + u * (kDaWarps * 32), j = i / (N / 8), c = (i - j * (N / 8)) * 8;
      pq[u] = pk[u] = make_uint4(0u, 0u, 0u, 0u);
      if (j < cnt) {
        const T* row = x + (int64_t)(start + c0 + j) * a.x_stride;
        pq[u] = ldg_128(row + qoff + c);
        pk[u] = ldg_128(row + koff + c);
      }
    }
#pragma unroll
    for (int u = 0; u < VV; ++u) {
      const int i = tid + u * (kDaWarps * 32), j = i / (P / 8), c = (i - j * (P / 8)) * 8;
      pv[u] = make_uint4(0u, 0u, 0u, 0u);
      if (j < cnt) pv[u] = ldg_128(x + (int64_t)(start + c0 + j) * a.x_stride + voff + c);
    }
  };
  // SiLU in fp32, one rounding to T; rows past the end are zero (SiLU(0) = 0)
  auto commit = [&](int cnt) {
#pragma unroll
    for (int u = 0; u < QV; ++u) {
      const int i = tid + u * (kDaWarps * 32), j = i / (N / 8), c = (i - j * (N / 8)) * 8;
      uint4 rq, rk;
      const T* eq = reinterpret_cast<const T*>(&pq[u]);
      const T* ek = reinterpret_cast<const T*>(&pk[u]);
      T* oq = reinterpret_cast<T*>(&rq);
      T* ok = reinterpret_cast<T*>(&rk);
#pragma unroll
      for (int e = 0; e < 8; ++e) { oq[e] = from_f32<T>(silu_da(to_f32(eq[e]))); ok[e] = from_f32<T>(silu_da(to_f32(ek[e]))); }
      *reinterpret_cast<uint4*>(sQ + j * QP + c * 2) = rq;
      *reinterpret_cast<uint4*>(sK + j * QP + c * 2) = rk;
    }
#pragma unroll
    for (int u = 0; u < VV; ++u) {
      const int i = tid + u * (kDaWarps * 32), j = i / (P / 8), c = (i - j * (P / 8)) * 8;
      uint4 rv, rh, rl;
      const T* ev = reinterpret_cast<const T*>(&pv[u]);
      T* ov = reinterpret_cast<T*>(&rv);
      T* oh = reinterpret_cast<T*>(&rh);
      T* ol = reinterpret_cast<T*>(&rl);
      const float w = j < cnt ? dpw[cnt - 1 - j] : 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        ov[e] = from_f32<T>(silu_da(to_f32(ev[e])));
        const float sv = to_f32(ov[e]) * w;                    // the rounded value is THE v of this path
        oh[e] = from_f32<T>(sv);
        ol[e] = from_f32<T>(sv - to_f32(oh[e]));
      }
      *reinterpret_cast<uint4*>(sV + j * VP + c * 2) = rv;
      *reinterpret_cast<uint4*>(sVh + j * VP + c * 2) = rh;
      *reinterpret_cast<uint4*>(sVl + j * VP + c * 2) = rl;
    }
  };
  fetch(0);
  for (int c0 = 0; c0 < len; c0 += kC) {
    const int cnt = min(kC, len - c0);
    __syncthreads();                                           // dpw / sS ready; the previous chunk's tiles are free
    commit(cnt);
    if (c0 + kC < len) fetch(c0 + kC);
    __syncthreads();
    // ---- outputs of the warp's 16 tokens
    const int r0 = warp * 16 + gq, r1 = r0 + 8;                 // rows of the chunk
    if (warp * 16 < cnt) {
      uint32_t qf[N / 16][4];
#pragma unroll
      for (int kk = 0; kk < N / 16; ++kk)
        ldmatrix_x4(qf[kk], smem_u32(sQ + (warp * 16 + (lane & 15)) * QP + (kk * 16 + (lane >> 4) * 8) * 2));
      float o[P / 8][4];
#pragma unroll
      for (int i = 0; i < P / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
      if (carried) {                                           // diag(d^(i+1)) Q S, the memory as hi + lo
#pragma unroll
        for (int kk = 0; kk < N / 16; ++kk) {
          const float* s0 = sS + (kk * 16 + 2 * tq) * SP + gq;
#pragma unroll
          for (int nt = 0; nt < P / 8; ++nt) {
            uint32_t h0, l0, h1, l1;
            split2<T>(s0[nt * 8], s0[SP + nt * 8], h0, l0);
            split2<T>(s0[8 * SP + nt * 8], s0[9 * SP + nt * 8], h1, l1);
            mma_m16n8k16<T>(o[nt], qf[kk], h0, h1);
            mma_m16n8k16<T>(o[nt], qf[kk], l0, l1);
          }
        }
        const float w0 = dpw[min(r0, kC - 1) + 1], w1 = dpw[min(r1, kC - 1) + 1];
#pragma unroll
        for (int i = 0; i < P / 8; ++i) { o[i][0] *= w0; o[i][1] *= w0; o[i][2] *= w1; o[i][3] *= w1; }
      }
      // scores of the warp's rows against the keys up to its last row, decay mask in fp32
      const int kt_end = warp + 1;                             // 16-key tiles that hold a visible key
      {
        const int mj = lane >> 3, r = lane & 7;
        const uint32_t ka = smem_u32(sK) + ((mj >> 1) * 8 + r) * QP + (mj & 1) * 16;
        const uint32_t va = smem_u32(sV) + ((mj & 1) * 8 + r) * VP + (mj >> 1) * 16;
        for (int kt = 0; kt < kt_end; ++kt) {
          float sc[2][4];
          sc[0][0] = sc[0][1] = sc[0][2] = sc[0][3] = sc[1][0] = sc[1][1] = sc[1][2] = sc[1][3] = 0.f;
#pragma unroll
          for (int kk = 0; kk < N / 16; ++kk) {
            uint32_t bf[4];
            ldmatrix_x4(bf, ka + kt * 16 * QP + kk * 32);
            mma_m16n8k16<T>(sc[0], qf[kk], bf[0], bf[1]);
            mma_m16n8k16<T>(sc[1], qf[kk], bf[2], bf[3]);
          }
#pragma unroll
          for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int key = kt * 16 + j * 8 + 2 * tq + (e & 1), row = (e >> 1) ? r1 : r0;
              sc[j][e] = (key <= row && key < cnt) ? sc[j][e] * dpw[row - key] : 0.f;
            }
          uint32_t ph[4], pl[4];
          split2<T>(sc[0][0], sc[0][1], ph[0], pl[0]);
          split2<T>(sc[0][2], sc[0][3], ph[1], pl[1]);
          split2<T>(sc[1][0], sc[1][1], ph[2], pl[2]);
          split2<T>(sc[1][2], sc[1][3], ph[3], pl[3]);
#pragma unroll
          for (int dn = 0; dn < P / 16; ++dn) {
            uint32_t bf[4];
            ldmatrix_x4_trans(bf, va + kt * 16 * VP + dn * 32);
            mma_m16n8k16<T>(o[2 * dn], ph, bf[0], bf[1]);
            mma_m16n8k16<T>(o[2 * dn + 1], ph, bf[2], bf[3]);
            mma_m16n8k16<T>(o[2 * dn], pl, bf[0], bf[1]);
            mma_m16n8k16<T>(o[2 * dn + 1], pl, bf[2], bf[3]);
          }
        }
      }
      float* y0 = a.y + (int64_t)(start + c0 + r0) * inner + h * Pf + p0;
      float* y1 = a.y + (int64_t)(start + c0 + r1) * inner + h * Pf + p0;
#pragma unroll
      for (int i = 0; i < P / 8; ++i) {
        const int c = i * 8 + 2 * tq;
        if (r0 < cnt) *reinterpret_cast<float2*>(y0 + c) = make_float2(o[i][0], o[i][1]);
        if (r1 < cnt) *reinterpret_cast<float2*>(y1 + c) = make_float2(o[i][2], o[i][3]);
      }
    }
    __syncthreads();                                           // every warp is done with the old memory
    // ---- memory update: rows [16 mt, 16 mt + 16) of S per warp, 32 columns at a time
    const float dc = dpw[cnt];
    for (int mt = warp; mt < N / 16; mt += kDaWarps) {
      const int mj = lane >> 3, r = lane & 7;
      const uint32_t ka = smem_u32(sK) + ((mj >> 1) * 8 + r) * QP + (mt * 16 + (mj & 1) * 8) * 2;
      const uint32_t vh = smem_u32(sVh) + ((mj & 1) * 8 + r) * VP + (mj >> 1) * 16;
      const uint32_t vl = smem_u32(sVl) + ((mj & 1) * 8 + r) * VP + (mj >> 1) * 16;
      uint32_t af[kC / 16][4];
#pragma unroll
      for (int kk = 0; kk < kC / 16; ++kk) ldmatrix_x4_trans(af[kk], ka + kk * 16 * QP);
#pragma unroll
      for (int ng = 0; ng < P / 32; ++ng) {
        float acc[4][4];
        float* s0 = sS + (mt * 16 + gq) * SP + ng * 32 + 2 * tq;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          acc[nt][0] = dc * s0[nt * 8]; acc[nt][1] = dc * s0[nt * 8 + 1];
          acc[nt][2] = dc * s0[8 * SP + nt * 8]; acc[nt][3] = dc * s0[8 * SP + nt * 8 + 1];
        }
#pragma unroll
        for (int kk = 0; kk < kC / 16; ++kk) {
          if (kk * 16 >= cnt) break;
#pragma unroll
          for (int pr = 0; pr < 2; ++pr) {
            uint32_t bh[4], bl[4];
            ldmatrix_x4_trans(bh, vh + kk * 16 * VP + (ng * 32 + pr * 16) * 2);
            ldmatrix_x4_trans(bl, vl + kk * 16 * VP + (ng * 32 + pr * 16) * 2);
            mma_m16n8k16<T>(acc[2 * pr], af[kk], bh[0], bh[1]);
            mma_m16n8k16<T>(acc[2 * pr + 1], af[kk], bh[2], bh[3]);
            mma_m16n8k16<T>(acc[2 * pr], af[kk], bl[0], bl[1]);
            mma_m16n8k16<T>(acc[2 * pr + 1], af[kk], bl[2], bl[3]);
          }
        }
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          s0[nt * 8] = acc[nt][0]; s0[nt * 8 + 1] = acc[nt][1];
          s0[8 * SP + nt * 8] = acc[nt][2]; s0[8 * SP + nt * 8 + 1] = acc[nt][3];
        }
      }
    }
    carried = true;
  }
  __syncthreads();
  for (int i = tid; i < N * P; i += blockDim.x) {
    const int n = i / P, p = i - n * P;
    st[n * Pf + p] = sS[n * SP + p];
  }
}

template <typename T, int N, int P>
int launch_da(const DaArgs& a, int64_t num_seqs, cudaStream_t st) {
  const size_t smem = (size_t)kC * (2 * (N + 8) + 3 * (P + 8)) * 2 + (size_t)N * (P + 4) * 4 + (kC + 1) * 4;
  static int cache[64] = {0};
  B2L_CUDA_CHECK(b2l_ensure_dynamic_smem(decay_attention_mma_kernel<T, N, P>, (int)smem, cache));
  b2l_launch(decay_attention_mma_kernel<T, N, P>, dim3((unsigned)a.H, (unsigned)num_seqs, (unsigned)(a.Pfull / P)),
             dim3(kDaWarps * 32), smem, st, a);
  return B2L_OK;
}

template <typename T, int N>
int dispatch_da_p(const DaArgs& a, int P, int64_t num_seqs, cudaStream_t st) {
  if (P == 32) return launch_da<T, N, 32>(a, num_seqs, st);
  if (P == 64) return launch_da<T, N, 64>(a, num_seqs, st);
  return launch_da<T, N, 128>(a, num_seqs, st);
}

bool da_size_ok(int v) { return v == 32 || v == 64 || v == 128; }

}  // namespace

/* 1 when b2l_decay_attention_mma takes this geometry: 16-bit dtype, state_size and head_dim in {32, 64, 128}, x rows
 * 16-byte aligned. */
extern "C" int b2l_decay_attention_mma_ok(const void* x, int64_t x_row_stride, int state_size, int head_dim, int dtype) {
  return (dtype == B2L_F16 || dtype == B2L_BF16) && da_size_ok(state_size) && da_size_ok(head_dim) &&
         x_row_stride % 8 == 0 && (uintptr_t)x % 16 == 0;
}

/* y_f32 [tokens, heads * head_dim] and state_f32 [slots, heads, state_size, head_dim] as b2l_ssm_scan with fixed
 * decays and SiLU inputs computes them; x rows = [v: heads*head_dim | k: heads*state_size | q: heads*state_size]. */
extern "C" int b2l_decay_attention_mma(void* y_f32, void* state_f32, const void* x, int64_t x_row_stride,
                                       const void* decay_f32, const void* seq_start, const void* seq_ctx,
                                       const void* seq_slot, int64_t num_seqs, int heads, int state_size, int head_dim,
                                       int dtype, void* stream) {
  B2L_REQUIRE(y_f32 && state_f32 && x && decay_f32 && seq_start && seq_ctx && seq_slot, "decay_attention_mma: null pointer");
  B2L_REQUIRE(heads > 0 && b2l_decay_attention_mma_ok(x, x_row_stride, state_size, head_dim, dtype),
              "decay_attention_mma: geometry heads=%d state=%d head_dim=%d dtype=%d is served by the scan", heads,
              state_size, head_dim, dtype);
  if (num_seqs <= 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  DaArgs a;
  a.y = (float*)y_f32; a.state = (float*)state_f32; a.x = x; a.x_stride = x_row_stride; a.decay = (const float*)decay_f32;
  a.seq_start = (const int*)seq_start; a.seq_ctx = (const int*)seq_ctx; a.seq_slot = (const int*)seq_slot; a.H = heads;
  a.Pfull = head_dim;
  // value columns per CTA: halved once when heads x sequences leave SMs without two CTAs (a second halving repeats
  // the scores and the q / k staging four times and loses: 301 us against 253 us unsplit at 16 heads x 8 sequences)
  int cols = head_dim;
  if (cols > 32 && (int64_t)heads * num_seqs < 2 * 148) cols /= 2;
  int rc = B2L_OK;
#define B2L_DA(TT)                                                                     \
  do {                                                                                 \
    if (state_size == 32) rc = dispatch_da_p<TT, 32>(a, cols, num_seqs, st);           \
    else if (state_size == 64) rc = dispatch_da_p<TT, 64>(a, cols, num_seqs, st);      \
    else rc = dispatch_da_p<TT, 128>(a, cols, num_seqs, st);                           \
  } while (0)
  if (dtype == B2L_F16) B2L_DA(__half); else B2L_DA(__nv_bfloat16);
#undef B2L_DA
  if (rc != B2L_OK) return rc;
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}
