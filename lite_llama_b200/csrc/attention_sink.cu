// Attention over the token-granular KV pool for RAGGED steps, with the score shaping of the sink / soft-cap family:
//   score = softcap * tanh(q.k * scale / softcap)   (softcap <= 0: plain q.k * scale)
//   p_j   = exp(score_j) / (sum_i exp(score_i) + exp(sink_h))      (sink == NULL: ordinary softmax)
// K and V rows may have different head sizes (D, Dv): a pool row is [G*D keys | G*Dv values]; the values may instead
// start at any column `v_col0` of the row (v_col0 = 0: the values ARE the leading Dv columns of the keys, which is
// how a latent cache [latent | rotated key part] is read by queries that were multiplied into the latent space).
// A sliding window (`window` > 0) limits token p to the keys p - window + 1 .. p; a block-diagonal mask (`block` > 0)
// to the keys of its own run of `block` positions, floor(p / block) * block .. p (runs are counted from position 0).
//
//   attn_prepare   per token: whole-row RMS norm of q and of k (one statistic over ALL heads, plain weight),
//                  position-dependent query gain, value mixing with an earlier layer's values, K|V cache write
//   sink_attention sequence s brings q_len new tokens after ctx cached ones; token i sees cache positions 0..ctx+i
//                  (its own K/V is already in the pool).  One launch covers a list of sequences:
//                  * tiled mode, 16-bit T: CTA = (64 tokens, query head, sequence) on mma.sync tensor-core tiles
//                  * tiled mode, fp32 T (or head sizes the tensor-core tiles do not take): CTA = (token tile, kv head,
//                    sequence) on the CUDA cores; the rows of a CTA (tokens x the kv head's query heads) share every
//                    K/V tile that is staged in shared memory
//                  * split mode (one new token per sequence: decode): CTA = (key range, kv head, sequence), fp32
//                    partial (max, sum, acc) per range, merged with the sink by sink_attention_merge.  With more than 4
//                    query heads per kv head (a latent cache: ALL heads share one row) and 16-bit T the partials come
//                    from the tensor-core kernel with the HEADS as the rows of its tile: a cached row is read once
//                    per key range and scored against every head by mma
// Softmax statistics, scores and the output accumulator are fp32 whatever T is.
#include "common.cuh"

namespace {

constexpr int kRows = 16;      // query rows per CTA
constexpr int kWarps = 4;
constexpr int kRowsPerWarp = kRows / kWarps;
constexpr int kKeys = 32;      // keys per tile: one per lane

struct AttnArgs {
  const void* q; int64_t q_stride;
  const void* kv; int64_t kv_stride;
  const int* table; int64_t table_stride;
  const int* seq_start; const int* seq_ctx; const int* seq_slot; const int* seq_list;
  const void* sink;
  void* out; int64_t out_stride;
  float* part;
  int H, G, D, Dv, PH, BQ, nsplit, chunk;
  int window, v_col0;          // window <= 0: every earlier key is visible; v_col0: first value column of a pool row
  int v_hstride;               // columns between the values of neighbouring kv heads (Dv; 0: every kv head reads the
                               // same Dv value columns, e.g. ALL value heads side by side as one wide head)
  int block;                   // > 0 (and no window): block-diagonal mask, see first_visible
  int v_blocks;                // split mode: one launch covers v_blocks blocks of Dv value columns (block c starts c * Dv
                               // columns after v_col0), each as H more heads: results [v_blocks][H][Dv] per token
  int head_rows;               // tensor-core kernel, one new token per sequence: the tile's rows are the query HEADS of
                               // one kv head (not tokens), blockIdx.x is a key range, results go to `part`
  float scale, softcap;
};

// first key position the token at `pos` sees (may be negative under a window: callers clamp where they index);
// non-decreasing in pos for every mask kind, which the tile-level bounds below rely on
__device__ __forceinline__ int first_visible(const AttnArgs& a, int pos) {
  return a.window > 0 ? pos - a.window + 1 : (a.block > 0 ? pos - pos % a.block : 0);
}

// ---- tiled mode on the CUDA cores (fp32 activations, or head sizes the tensor-core tiles do not take) ------------
template <typename T, int DVJ>
__global__ void __launch_bounds__(kWarps * 32) sink_attention_kernel(AttnArgs a) {
  pdl_prologue();
  extern __shared__ float smem[];
  const int D = a.D, Dv = a.Dv, per = a.H / a.G;
  float* qs = smem;                              // [kRows][D]
  float* ks = qs + kRows * D;                    // [kKeys][D + 1]
  float* vs = ks + kKeys * (D + 1);              // [kKeys][Dv]
  const int z = blockIdx.z, s = a.seq_list ? a.seq_list[z] : z;
  const int start = a.seq_start[s], qlen = a.seq_start[s + 1] - start, ctx = a.seq_ctx[s];
  const int64_t slot = a.seq_slot[s];
  const int hchunks = (per + a.PH - 1) / a.PH;
  const int g = blockIdx.y / hchunks, h_first = g * per + (blockIdx.y % hchunks) * a.PH;
  const int h_count = min(a.PH, g * per + per - h_first);
  const int t0 = blockIdx.x * a.BQ;
  if (t0 >= qlen) return;
  const int t_count = min(a.BQ, qlen - t0);
  const int key_hi = ctx + t0 + t_count;                // exclusive
  const int key_lo = max(0, first_visible(a, ctx + t0));                      // first key the tile's first token sees
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const T* q = (const T*)a.q;
  const T* kv = (const T*)a.kv;
  // rows: r = tl * PH + hl
  for (int i = tid; i < kRows * D; i += blockDim.x) {
    const int r = i / D, d = i - r * D, tl = r / a.PH, hl = r - tl * a.PH;
    float v = 0.f;
    if (tl < t_count && hl < h_count) v = to_f32(q[(int64_t)(start + t0 + tl) * a.q_stride + (h_first + hl) * D + d]);
    qs[i] = v;
  }
  float m[kRowsPerWarp], l[kRowsPerWarp], acc[kRowsPerWarp][DVJ];
  int row_pos[kRowsPerWarp];                      // last visible key position of the row, -1 = unused row
#pragma unroll
  for (int i = 0; i < kRowsPerWarp; ++i) {
    const int r = warp * kRowsPerWarp + i, tl = r / a.PH, hl = r - tl * a.PH;
    m[i] = -INFINITY; l[i] = 0.f;
    row_pos[i] = (tl < t_count && hl < h_count) ? ctx + t0 + tl : -1;
#pragma unroll
    for (int j = 0; j < DVJ; ++j) acc[i][j] = 0.f;
  }
  const int* trow = a.table + slot * a.table_stride;
  const float inv_cap = a.softcap > 0.f ? 1.0f / a.softcap : 0.f;
  for (int k0 = key_lo; k0 < key_hi; k0 += kKeys) {
    __syncthreads();
    const int nk = min(kKeys, key_hi - k0);
    for (int i = tid; i < kKeys * D; i += blockDim.x) {
      const int j = i / D, d = i - j * D;
      ks[j * (D + 1) + d] = j < nk ? to_f32(kv[(int64_t)trow[k0 + j] * a.kv_stride + g * D + d]) : 0.f;
    }
    for (int i = tid; i < kKeys * Dv; i += blockDim.x) {
      const int j = i / Dv, d = i - j * Dv;
      vs[i] = j < nk ? to_f32(kv[(int64_t)trow[k0 + j] * a.kv_stride + a.v_col0 + g * a.v_hstride + d]) : 0.f;
    }
    __syncthreads();
    float sc[kRowsPerWarp];
#pragma unroll
    for (int i = 0; i < kRowsPerWarp; ++i) sc[i] = 0.f;
    const float* kr = ks + lane * (D + 1);
    const float* qr = qs + warp * kRowsPerWarp * D;
    for (int d = 0; d < D; ++d) {
      const float kvv = kr[d];
#pragma unroll
      for (int i = 0; i < kRowsPerWarp; ++i) sc[i] = fmaf(qr[i * D + d], kvv, sc[i]);
    }
#pragma unroll
    for (int i = 0; i < kRowsPerWarp; ++i) {
      if (row_pos[i] < k0) continue;              // warp-uniform: nothing visible in this tile (or unused row)
      const int row_lo = first_visible(a, row_pos[i]);
      if (row_lo >= k0 + nk) continue;            // warp-uniform: the row's window starts after this tile
      float sv = sc[i] * a.scale;
      if (a.softcap > 0.f) sv = a.softcap * tanhf(sv * inv_cap);
      const bool ok = lane < nk && k0 + lane <= row_pos[i] && k0 + lane >= row_lo;
      sv = ok ? sv : -INFINITY;
      const float mt = warp_reduce_max(sv);
      const float mn = fmaxf(m[i], mt);
      const float corr = expf(m[i] - mn);          // exp(-inf) = 0 on the first tile
      const float p = ok ? expf(sv - mn) : 0.f;
      l[i] = l[i] * corr + warp_reduce_sum(p);
      m[i] = mn;
#pragma unroll
      for (int j = 0; j < DVJ; ++j) acc[i][j] *= corr;
      for (int kk = 0; kk < nk; ++kk) {
        const float pk = __shfl_sync(0xffffffffu, p, kk);
#pragma unroll
        for (int j = 0; j < DVJ; ++j) {
          const int d = lane + 32 * j;
          if (d < Dv) acc[i][j] = fmaf(pk, vs[kk * Dv + d], acc[i][j]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kRowsPerWarp; ++i) {
    if (row_pos[i] < 0) continue;
    const int r = warp * kRowsPerWarp + i, tl = r / a.PH, hl = r - tl * a.PH, h = h_first + hl;
    {
      float mf = m[i], den = l[i], num = 1.f;
      if (a.sink) {
        const float sk = to_f32(((const T*)a.sink)[h]);
        mf = fmaxf(m[i], sk);
        num = expf(m[i] - mf);
        den = l[i] * num + expf(sk - mf);
      }
      const float inv = num / den;
      T* o = (T*)a.out + (int64_t)(start + t0 + tl) * a.out_stride + h * Dv;
#pragma unroll
      for (int j = 0; j < DVJ; ++j) {
        const int d = lane + 32 * j;
        if (d < Dv) o[d] = from_f32<T>(acc[i][j] * inv);
      }
    }
  }
}

// ---- tiled mode on the tensor cores (16-bit T) ------------------------------------------------------------------
// CTA = 64 new tokens of one (sequence, query head); 4 warps x 16 query rows (FlashAttention-2 schedule, the same
// fragment handling as flash_attention_nopad.cu).  64-key K and V tiles are gathered through the request table with
// 16-byte asynchronous copies into a two-stage padded shared-memory ring (head sizes are padded to DP / DVP columns
// of zeros; the next tile's copies fly while the current one is multiplied), S = Q K^T and
// O += P V run on mma.sync m16n8k16 with fp32 accumulators, the soft cap is applied to the fp32 scores, the online
// softmax works in the log2 domain, the sink joins the denominator once at the end.  Keys 0 .. ctx + t (cached prefix
// + the portion itself) are visible to token t.  Needs D, Dv multiples of 8 and <= 128, 16-byte aligned pool rows.
constexpr int kTileM = 64, kTileN = 64;
constexpr float kLog2e = 1.4426950408889634f;

// tanh(x) = 1 - 2 / (exp(2x) + 1) on ex2.approx + a fast reciprocal: absolute error ~1e-7, far below the rounding of
// the 16-bit q and k that feed the score (the fp32 path keeps tanhf)
__device__ __forceinline__ float tanh_fast(float x) {
  const float e = fast_exp2(x * (2.0f * kLog2e));
  return 1.0f - __fdividef(2.0f, e + 1.0f);
}

// 16-byte asynchronous global -> shared copies (the gathered rows have no tensor-map shape, so no TMA tile)
__device__ __forceinline__ void cp_async_16(uint32_t saddr, const void* g) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(saddr), "l"(g) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <typename T, int DP, int DVP>
__global__ void __launch_bounds__(128) sink_attention_mma_kernel(AttnArgs a) {
  pdl_prologue();
  extern __shared__ __align__(16) uint8_t smem_raw[];
  constexpr int KP = (DP + 8) * 2, VP = (DVP + 8) * 2;          // row pitches in bytes
  constexpr int kStage = kTileN * (KP + VP);                    // one K tile + one V tile; two stages
  const int D = a.D, Dv = a.Dv, per = a.H / a.G;
  const int z = blockIdx.z, s = a.seq_list ? a.seq_list[z] : z;
  const int start = a.seq_start[s], qlen = a.seq_start[s + 1] - start, ctx = a.seq_ctx[s];
  const bool hr = a.head_rows != 0;
  const int t0 = hr ? 0 : blockIdx.x * kTileM;
  if (!hr && t0 >= qlen) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gq = lane >> 2, tq = lane & 3;
  const int r0 = warp * 16 + gq, r1 = r0 + 8;                    // rows of the tile
  // token rows: row r = token t0 + r of head blockIdx.y.  head rows: row r = head h_base + r of the ONE new token,
  // blockIdx.y = (kv head, 64-head chunk of its query heads), blockIdx.x = key range
  const int hchunks = (per + kTileM - 1) / kTileM;
  const int g = hr ? blockIdx.y / hchunks : blockIdx.y / per;
  const int h_base = hr ? g * per + (blockIdx.y % hchunks) * kTileM : blockIdx.y;
  const int t_count = hr ? min(kTileM, g * per + per - h_base) : min(kTileM, qlen - t0);       // live rows
  const int h = h_base;
  const int64_t slot = a.seq_slot[s];
  const int win_lo = max(0, first_visible(a, ctx));                            // head rows: the token's first visible key
  const int range_lo = hr ? win_lo + blockIdx.x * a.chunk : 0;
  const int key_hi = hr ? min(range_lo + a.chunk, ctx + 1) : ctx + t0 + t_count;               // exclusive
  const bool ok0 = r0 < t_count, ok1 = r1 < t_count;
  const int pos0 = hr ? key_hi - 1 : ctx + t0 + r0, pos1 = hr ? key_hi - 1 : ctx + t0 + r1;     // last visible key of each row
  const int lo0 = hr ? range_lo : first_visible(a, pos0);                                       // first one
  const int lo1 = hr ? range_lo : first_visible(a, pos1);
  // first key tile: the one that holds the first key of the tile's first row (tiles stay aligned to kTileN)
  const int k_first = hr ? range_lo / kTileN * kTileN : max(0, first_visible(a, ctx + t0)) / kTileN * kTileN;
  const int warp_first = hr ? range_lo : first_visible(a, ctx + t0 + warp * 16);                    // first key of the warp's rows
  const T* q = (const T*)a.q;
  const T* kv = (const T*)a.kv;
  uint32_t qf[DP / 16][4];
  {
    const T* q0 = hr ? q + (int64_t)start * a.q_stride + (h_base + (ok0 ? r0 : 0)) * D
                     : q + (int64_t)(start + t0 + (ok0 ? r0 : 0)) * a.q_stride + h * D;
    const T* q1 = hr ? q + (int64_t)start * a.q_stride + (h_base + (ok1 ? r1 : 0)) * D
                     : q + (int64_t)(start + t0 + (ok1 ? r1 : 0)) * a.q_stride + h * D;
#pragma unroll
    for (int kk = 0; kk < DP / 16; ++kk) {
      const int c = kk * 16 + 2 * tq;
      qf[kk][0] = (ok0 && c < D) ? *reinterpret_cast<const uint32_t*>(q0 + c) : 0u;
      qf[kk][1] = (ok1 && c < D) ? *reinterpret_cast<const uint32_t*>(q1 + c) : 0u;
      qf[kk][2] = (ok0 && c + 8 < D) ? *reinterpret_cast<const uint32_t*>(q0 + c + 8) : 0u;
      qf[kk][3] = (ok1 && c + 8 < D) ? *reinterpret_cast<const uint32_t*>(q1 + c + 8) : 0u;
    }
  }
  float o[DVP / 8][4];
#pragma unroll
  for (int i = 0; i < DVP / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  // last key any row of the warp sees; a warp without live rows (head rows: fewer than 16 * warp heads) sees none
  const int warp_last = hr ? (warp * 16 < t_count ? key_hi - 1 : -1) : ctx + t0 + warp * 16 + 15;
  const int* trow = a.table + slot * a.table_stride;
  const float cap = a.softcap, inv_cap = cap > 0.f ? 1.0f / cap : 0.f;
  // tile k0 -> stage `st`: asynchronous 16-byte copies of the rows the table names; rows / columns past the end are
  // zero-filled with plain stores (disjoint addresses)
  auto issue = [&](int k0, int st) {
    uint8_t* kdst = smem_raw + st * kStage;
    uint8_t* vdst = kdst + kTileN * KP;
    // the pool rows of this thread's copies first (independent loads), then the copies
    constexpr int JK = kTileN * (DP / 8) / 128, JV = kTileN * (DVP / 8) / 128;
    int rk[JK], rv[JV];
#pragma unroll
    for (int j = 0; j < JK; ++j) {
      const int r = (tid + 128 * j) / (DP / 8);
      rk[j] = k0 + r < key_hi ? trow[k0 + r] : -1;
    }
#pragma unroll
    for (int j = 0; j < JV; ++j) {
      const int r = (tid + 128 * j) / (DVP / 8);
      rv[j] = k0 + r < key_hi ? trow[k0 + r] : -1;
    }
#pragma unroll
    for (int j = 0; j < JK; ++j) {
      const int i = tid + 128 * j, r = i / (DP / 8), c = (i - r * (DP / 8)) * 8;
      if (rk[j] >= 0 && c < D)
        cp_async_16(smem_u32(kdst + r * KP + c * 2), kv + (int64_t)rk[j] * a.kv_stride + g * D + c);
      else
        *reinterpret_cast<uint4*>(kdst + r * KP + c * 2) = make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int j = 0; j < JV; ++j) {
      const int i = tid + 128 * j, r = i / (DVP / 8), c = (i - r * (DVP / 8)) * 8;
      if (rv[j] >= 0 && c < Dv)
        cp_async_16(smem_u32(vdst + r * VP + c * 2), kv + (int64_t)rv[j] * a.kv_stride + a.v_col0 + g * a.v_hstride + c);
      else
        *reinterpret_cast<uint4*>(vdst + r * VP + c * 2) = make_uint4(0u, 0u, 0u, 0u);
    }
    cp_async_commit();
  };
  if (k_first < key_hi) issue(k_first, 0);
  for (int k0 = k_first, it = 0; k0 < key_hi; k0 += kTileN, ++it) {
    const bool more = k0 + kTileN < key_hi;
    if (more) issue(k0 + kTileN, (it + 1) & 1);                  // the next tile flies while this one is used
    if (more) cp_async_wait<1>(); else cp_async_wait<0>();
    __syncthreads();                                             // tile `it` is complete and visible to every warp
    const uint32_t ks = smem_u32(smem_raw + (it & 1) * kStage), vs = ks + kTileN * KP;
    // the barrier at the END of the body keeps stage it & 1 intact until every warp is done with it
    if (k0 > warp_last || k0 + kTileN <= warp_first) { __syncthreads(); continue; }
    float sc[kTileN / 8][4];
#pragma unroll
    for (int j = 0; j < kTileN / 8; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
    {
      const int mj = lane >> 3, r = lane & 7;
      const uint32_t a0 = ks + ((mj >> 1) * 8 + r) * KP + (mj & 1) * 16;
#pragma unroll
      for (int kk = 0; kk < DP / 16; ++kk) {
#pragma unroll
        for (int jp = 0; jp < kTileN / 16; ++jp) {
          uint32_t bf[4];
          ldmatrix_x4(bf, a0 + jp * 16 * KP + kk * 32);
          mma_m16n8k16<T>(sc[2 * jp], qf[kk], bf[0], bf[1]);
          mma_m16n8k16<T>(sc[2 * jp + 1], qf[kk], bf[2], bf[3]);
        }
      }
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < kTileN / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = k0 + j * 8 + 2 * tq + (e & 1);
        const int lim = (e >> 1) ? pos1 : pos0, first = (e >> 1) ? lo1 : lo0;
        float v = sc[j][e] * a.scale;
        if (cap > 0.f) v = cap * tanh_fast(v * inv_cap);
        v = (key <= lim && key >= first) ? v * kLog2e : -INFINITY;
        sc[j][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
    float alpha[2], base[2];
#pragma unroll
    for (int r2 = 0; r2 < 2; ++r2) {
      mx[r2] = fmaxf(mx[r2], __shfl_xor_sync(0xffffffffu, mx[r2], 1));
      mx[r2] = fmaxf(mx[r2], __shfl_xor_sync(0xffffffffu, mx[r2], 2));
      const float mnew = fmaxf(m_run[r2], mx[r2]);
      base[r2] = mnew == -INFINITY ? 0.f : mnew;
      alpha[r2] = fast_exp2(m_run[r2] - base[r2]);
      m_run[r2] = mnew;
    }
    float ps[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < kTileN / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pv = fast_exp2(sc[j][e] - base[e >> 1]);
        sc[j][e] = pv;
        ps[e >> 1] += pv;
      }
    }
    l_run[0] = l_run[0] * alpha[0] + ps[0];
    l_run[1] = l_run[1] * alpha[1] + ps[1];
#pragma unroll
    for (int i = 0; i < DVP / 8; ++i) {
      o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
      o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
    }
    {
      const int mj = lane >> 3, r = lane & 7;
      const uint32_t a0 = vs + ((mj & 1) * 8 + r) * VP + (mj >> 1) * 16;
#pragma unroll
      for (int kt = 0; kt < kTileN / 16; ++kt) {
        uint32_t pf[4];
        pf[0] = pack2<T>(sc[2 * kt][0], sc[2 * kt][1]);
        pf[1] = pack2<T>(sc[2 * kt][2], sc[2 * kt][3]);
        pf[2] = pack2<T>(sc[2 * kt + 1][0], sc[2 * kt + 1][1]);
        pf[3] = pack2<T>(sc[2 * kt + 1][2], sc[2 * kt + 1][3]);
#pragma unroll
        for (int dn = 0; dn < DVP / 16; ++dn) {
          uint32_t bf[4];
          ldmatrix_x4_trans(bf, a0 + kt * 16 * VP + dn * 32);
          mma_m16n8k16<T>(o[2 * dn], pf, bf[0], bf[1]);
          mma_m16n8k16<T>(o[2 * dn + 1], pf, bf[2], bf[3]);
        }
      }
    }
    __syncthreads();
  }
  if (hr) {
    // one fp32 partial (max, sum, unnormalised values) per (head, key range) in the layout sink_attention_merge reads;
    // the maximum goes back from the log2 domain to natural units
#pragma unroll
    for (int r2 = 0; r2 < 2; ++r2) {
      l_run[r2] += __shfl_xor_sync(0xffffffffu, l_run[r2], 1);
      l_run[r2] += __shfl_xor_sync(0xffffffffu, l_run[r2], 2);
      const int r = r2 ? r1 : r0;
      if (r >= t_count) continue;
      float* dst = a.part + (((int64_t)z * a.H + h_base + r) * a.nsplit + blockIdx.x) * (Dv + 2);
      if (tq == 0) { dst[0] = m_run[r2] * 0.6931471805599453f; dst[1] = l_run[r2]; }
#pragma unroll
      for (int i = 0; i < DVP / 8; ++i) {
        const int c = i * 8 + 2 * tq;
        if (c < Dv) { dst[2 + c] = o[i][2 * r2]; dst[3 + c] = o[i][2 * r2 + 1]; }
      }
    }
    return;
  }
  float inv[2];
#pragma unroll
  for (int r2 = 0; r2 < 2; ++r2) {
    l_run[r2] += __shfl_xor_sync(0xffffffffu, l_run[r2], 1);
    l_run[r2] += __shfl_xor_sync(0xffffffffu, l_run[r2], 2);
    float num = 1.f, den = l_run[r2];
    if (a.sink) {
      const float sk = to_f32(((const T*)a.sink)[h]) * kLog2e;
      const float mf = fmaxf(m_run[r2], sk);
      num = fast_exp2(m_run[r2] - mf);
      den = l_run[r2] * num + fast_exp2(sk - mf);
    }
    inv[r2] = num / den;
  }
  T* ob = (T*)a.out + h * Dv;
  if (ok0) {
    T* orow = ob + (int64_t)(start + t0 + r0) * a.out_stride;
#pragma unroll
    for (int i = 0; i < DVP / 8; ++i)
      if (i * 8 + 2 * tq < Dv) *reinterpret_cast<uint32_t*>(orow + i * 8 + 2 * tq) = pack2<T>(o[i][0] * inv[0], o[i][1] * inv[0]);
  }
  if (ok1) {
    T* orow = ob + (int64_t)(start + t0 + r1) * a.out_stride;
#pragma unroll
    for (int i = 0; i < DVP / 8; ++i)
      if (i * 8 + 2 * tq < Dv) *reinterpret_cast<uint32_t*>(orow + i * 8 + 2 * tq) = pack2<T>(o[i][2] * inv[1], o[i][3] * inv[1]);
  }
}

template <typename T, int DP, int DVP>
int launch_attention_mma(const AttnArgs& a, int max_q_len, int64_t num_seqs, cudaStream_t st) {
  constexpr int smem = 2 * kTileN * ((DP + 8) * 2 + (DVP + 8) * 2);      // two stages
  static int cache[64] = {0};
  B2L_CUDA_CHECK(b2l_ensure_dynamic_smem(sink_attention_mma_kernel<T, DP, DVP>, smem, cache));
  const int per = a.H / a.G;
  const dim3 grid = a.head_rows ? dim3((unsigned)a.nsplit, (unsigned)(a.G * ((per + kTileM - 1) / kTileM)), (unsigned)num_seqs)
                                : dim3((unsigned)((max_q_len + kTileM - 1) / kTileM), (unsigned)a.H, (unsigned)num_seqs);
  b2l_launch(sink_attention_mma_kernel<T, DP, DVP>, grid, dim3(128), (size_t)smem, st, a);
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

template <typename T>
int dispatch_attention_mma(const AttnArgs& a, int max_q_len, int64_t num_seqs, cudaStream_t st) {
  const int dp = a.D <= 32 ? 32 : (a.D <= 64 ? 64 : 128), dvp = a.Dv <= 32 ? 32 : (a.Dv <= 64 ? 64 : 128);
#define B2L_MMA(P, V) if (dp == P && dvp == V) return launch_attention_mma<T, P, V>(a, max_q_len, num_seqs, st)
  B2L_MMA(32, 32); B2L_MMA(32, 64); B2L_MMA(32, 128);
  B2L_MMA(64, 32); B2L_MMA(64, 64); B2L_MMA(64, 128);
  B2L_MMA(128, 32); B2L_MMA(128, 64); B2L_MMA(128, 128);
#undef B2L_MMA
  B2L_UNSUPPORTED("sink_attention: head sizes %d / %d", a.D, a.Dv);
}

// the tensor-core tiled kernel takes 16-bit activations, head sizes in 8-element steps up to 128, and pool / q rows
// whose 16-byte vectors are aligned
inline bool mma_path_ok(const AttnArgs& a, int dtype) {
  if (dtype != B2L_F16 && dtype != B2L_BF16) return false;
  if (a.D % 8 || a.Dv % 8 || a.D > 128 || a.Dv > 128) return false;
  if (a.kv_stride % 8 || a.v_col0 % 8 || a.v_hstride % 8 || a.q_stride % 2 || a.out_stride % 2) return false;
  if (((uintptr_t)a.kv % 16) || ((uintptr_t)a.q % 4) || ((uintptr_t)a.out % 4)) return false;
  return true;
}

// ---- split mode (decode): one new token per sequence ---------------------------------------------------------------
// CTA = (key range, kv head x chunk of <= 4 of its query heads, sequence).  Each of the 4 warps walks its own quarter
// of the range 32 keys at a time: the 32 K rows and V rows are copied raw (T) into the warp's private shared-memory
// stage with 16-byte loads, lane j scores key j against all the CTA's query heads (so K is read once per kv head, not
// once per query head), and the value sum runs with lanes over the value columns.  The warps' (max, sum, acc) meet in
// shared memory, the CTA writes one fp32 partial per (head, range), sink_attention_merge adds the sink.
constexpr int kSplitRows = 4;
constexpr int kStageBatch = 8;

template <typename T, int DVJ>
__global__ void __launch_bounds__(128) sink_attention_split_kernel(AttnArgs a) {
  pdl_prologue();
  extern __shared__ __align__(16) uint8_t smem_raw[];
  const int D = a.D, Dv = a.Dv, per = a.H / a.G;
  constexpr int VEC = 16 / (int)sizeof(T);
  const int Dp = (D + VEC - 1) / VEC * VEC + VEC, Dvp = (Dv + VEC - 1) / VEC * VEC;       // stage pitches (elements)
  float* qs = reinterpret_cast<float*>(smem_raw);                        // [kSplitRows][D]
  float* mrg = qs + kSplitRows * ((D + 3) / 4 * 4);                      // [4 warps][kSplitRows][2 + Dv]
  T* stage = reinterpret_cast<T*>(mrg + 4 * kSplitRows * (2 + Dv) + ((4 - (4 * kSplitRows * (2 + Dv)) % 4) % 4));
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  T* ks = stage + (size_t)warp * 32 * (Dp + Dvp);
  T* vs = ks + 32 * Dp;
  const int z = blockIdx.z, s = a.seq_list ? a.seq_list[z] : z;
  const int start = a.seq_start[s], ctx = a.seq_ctx[s];
  const int64_t slot = a.seq_slot[s];
  const int hchunks = (per + kSplitRows - 1) / kSplitRows;
  const int vb = blockIdx.y / (a.G * hchunks), by = blockIdx.y - vb * (a.G * hchunks);
  const int g = by / hchunks, h_first = g * per + (by % hchunks) * kSplitRows;
  const int h_count = min(kSplitRows, g * per + per - h_first);
  const int v_col = a.v_col0 + vb * Dv + g * a.v_hstride;                    // first value column of this CTA
  const int win_lo = max(0, first_visible(a, ctx));                          // the new token's first visible key
  const int key_lo = win_lo + blockIdx.x * a.chunk, key_hi = min(key_lo + a.chunk, ctx + 1);
  const T* q = (const T*)a.q;
  const T* kv = (const T*)a.kv;
  const int Dq = (D + 3) / 4 * 4;
  for (int i = tid; i < kSplitRows * Dq; i += 128) {
    const int r = i / Dq, d = i - r * Dq;
    qs[i] = (r < h_count && d < D) ? to_f32(q[(int64_t)start * a.q_stride + (h_first + r) * D + d]) : 0.f;
  }
  __syncthreads();
  float m[kSplitRows], l[kSplitRows], acc[kSplitRows][DVJ];
#pragma unroll
  for (int r = 0; r < kSplitRows; ++r) {
    m[r] = -INFINITY; l[r] = 0.f;
#pragma unroll
    for (int j = 0; j < DVJ; ++j) acc[r][j] = 0.f;
  }
  const int* trow = a.table + slot * a.table_stride;
  const float inv_cap = a.softcap > 0.f ? 1.0f / a.softcap : 0.f;
  const bool vec_ok = (D % VEC == 0) && (Dv % VEC == 0) && (a.kv_stride % VEC == 0) && (a.v_col0 % VEC == 0) &&
                      (a.v_hstride % VEC == 0) && (((uintptr_t)a.kv % 16) == 0);
  for (int k0 = key_lo + warp * 32; k0 < key_hi; k0 += 128) {
    const int nk = min(32, key_hi - k0);
    __syncwarp();
    if (vec_ok) {
      // lane j fetches key j's pool row once; the 16-byte copies run in batches of kStageBatch loads per lane that
      // are all in flight before the first shared-memory store
      const int my_row = lane < nk ? trow[k0 + lane] : 0;
      auto stage_rows = [&](T* dst, int pitch, int col0, int vecs) {
        for (int base = 0; base < nk * vecs; base += 32 * kStageBatch) {
          uint4 raw[kStageBatch];
#pragma unroll
          for (int u = 0; u < kStageBatch; ++u) {
            const int idx = base + u * 32 + lane, j = min(idx / vecs, 31), c = (idx - (idx / vecs) * vecs) * VEC;
            const int row = __shfl_sync(0xffffffffu, my_row, j);
            raw[u] = make_uint4(0u, 0u, 0u, 0u);
            if (idx < nk * vecs) raw[u] = ldg_128(kv + (int64_t)row * a.kv_stride + col0 + c);
          }
#pragma unroll
          for (int u = 0; u < kStageBatch; ++u) {
            const int idx = base + u * 32 + lane, j = idx / vecs, c = (idx - j * vecs) * VEC;
            if (idx < nk * vecs) *reinterpret_cast<uint4*>(dst + j * pitch + c) = raw[u];
          }
        }
      };
      stage_rows(ks, Dp, g * D, D / VEC);
      stage_rows(vs, Dvp, v_col, Dv / VEC);
    } else {
      for (int i = lane; i < nk * D; i += 32) {
        const int j = i / D, d = i - j * D;
        ks[j * Dp + d] = kv[(int64_t)trow[k0 + j] * a.kv_stride + g * D + d];
      }
      for (int i = lane; i < nk * Dv; i += 32) {
        const int j = i / Dv, d = i - j * Dv;
        vs[j * Dvp + d] = kv[(int64_t)trow[k0 + j] * a.kv_stride + v_col + d];
      }
    }
    __syncwarp();
    float sc[kSplitRows];
#pragma unroll
    for (int r = 0; r < kSplitRows; ++r) sc[r] = 0.f;
    if (lane < nk) {
      const T* kr = ks + lane * Dp;
      if (vec_ok) {                                // 16-byte reads: a quarter warp covers all banks at this pitch
        for (int d = 0; d < D; d += VEC) {
          const uint4 raw = *reinterpret_cast<const uint4*>(kr + d);
          const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
          for (int c = 0; c < VEC; ++c) {
            const float kvv = to_f32(e[c]);
#pragma unroll
            for (int r = 0; r < kSplitRows; ++r) sc[r] = fmaf(qs[r * Dq + d + c], kvv, sc[r]);
          }
        }
      } else {
        for (int d = 0; d < D; ++d) {
          const float kvv = to_f32(kr[d]);
#pragma unroll
          for (int r = 0; r < kSplitRows; ++r) sc[r] = fmaf(qs[r * Dq + d], kvv, sc[r]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kSplitRows; ++r) {
      if (r >= h_count) continue;
      float sv = sc[r] * a.scale;
      if (a.softcap > 0.f) sv = a.softcap * tanhf(sv * inv_cap);
      const bool ok = lane < nk;
      sv = ok ? sv : -INFINITY;
      const float mn = fmaxf(m[r], warp_reduce_max(sv));
      const float corr = expf(m[r] - mn);
      const float p = ok ? expf(sv - mn) : 0.f;
      l[r] = l[r] * corr + warp_reduce_sum(p);
      m[r] = mn;
#pragma unroll
      for (int j = 0; j < DVJ; ++j) acc[r][j] *= corr;
      sc[r] = p;
    }
    for (int kk = 0; kk < nk; ++kk) {
      float vv[DVJ];
#pragma unroll
      for (int j = 0; j < DVJ; ++j) {
        const int d = lane + 32 * j;
        vv[j] = d < Dv ? to_f32(vs[kk * Dvp + d]) : 0.f;
      }
#pragma unroll
      for (int r = 0; r < kSplitRows; ++r) {
        const float pk = __shfl_sync(0xffffffffu, sc[r], kk);
#pragma unroll
        for (int j = 0; j < DVJ; ++j) acc[r][j] = fmaf(pk, vv[j], acc[r][j]);
      }
    }
  }
  // the four warps' partials meet in shared memory; warp w finishes row w
#pragma unroll
  for (int r = 0; r < kSplitRows; ++r) {
    float* dst = mrg + (warp * kSplitRows + r) * (2 + Dv);
    if (lane == 0) { dst[0] = m[r]; dst[1] = l[r]; }
#pragma unroll
    for (int j = 0; j < DVJ; ++j) {
      const int d = lane + 32 * j;
      if (d < Dv) dst[2 + d] = acc[r][j];
    }
  }
  __syncthreads();
  if (warp < h_count) {
    const int r = warp;
    float mf = -INFINITY;
    for (int w = 0; w < 4; ++w) mf = fmaxf(mf, mrg[(w * kSplitRows + r) * (2 + Dv)]);
    float den = 0.f, sc4[4];
    for (int w = 0; w < 4; ++w) {
      const float mw = mrg[(w * kSplitRows + r) * (2 + Dv)];
      sc4[w] = mw == -INFINITY ? 0.f : expf(mw - mf);
      den += mrg[(w * kSplitRows + r) * (2 + Dv) + 1] * sc4[w];
    }
    float* dst = a.part + ((((int64_t)z * a.v_blocks + vb) * a.H + h_first + r) * a.nsplit + blockIdx.x) * (Dv + 2);
    if (lane == 0) { dst[0] = mf; dst[1] = den; }
    for (int d = lane; d < Dv; d += 32) {
      float v = 0.f;
      for (int w = 0; w < 4; ++w) v = fmaf(mrg[(w * kSplitRows + r) * (2 + Dv) + 2 + d], sc4[w], v);
      dst[2 + d] = v;
    }
  }
}

template <typename T>
int launch_attention_split(const AttnArgs& a, int64_t num_seqs, cudaStream_t st) {
  constexpr int VEC = 16 / (int)sizeof(T);
  const int Dp = (a.D + VEC - 1) / VEC * VEC + VEC, Dvp = (a.Dv + VEC - 1) / VEC * VEC;
  const int Dq = (a.D + 3) / 4 * 4;
  int mfl = 4 * kSplitRows * (2 + a.Dv);
  mfl += (4 - mfl % 4) % 4;
  const size_t smem = (size_t)(kSplitRows * Dq + mfl) * sizeof(float) + (size_t)4 * 32 * (Dp + Dvp) * sizeof(T);
  B2L_REQUIRE((int64_t)smem <= b2l_max_smem_optin(), "sink_attention: head sizes %d / %d need %lld bytes of shared memory",
              a.D, a.Dv, (long long)smem);
  const int dvj = (a.Dv + 31) / 32;
  B2L_REQUIRE(dvj <= 8, "sink_attention: value head size %d > 256", a.Dv);
  const int per = a.H / a.G, hchunks = (per + kSplitRows - 1) / kSplitRows;
  const dim3 grid((unsigned)a.nsplit, (unsigned)(a.G * hchunks * a.v_blocks), (unsigned)num_seqs);
#define B2L_SPLIT(J)                                                                                     \
  do {                                                                                                   \
    static int cache[64] = {0};                                                                          \
    B2L_CUDA_CHECK(b2l_ensure_dynamic_smem(sink_attention_split_kernel<T, J>, (int)smem, cache));        \
    b2l_launch(sink_attention_split_kernel<T, J>, grid, dim3(128), smem, st, a);                         \
  } while (0)
  if (dvj <= 2) B2L_SPLIT(2);
  else if (dvj <= 4) B2L_SPLIT(4);
  else B2L_SPLIT(8);
#undef B2L_SPLIT
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

// One CTA of 64 threads per (head, sequence): the ranges' maxima and sums are reduced across the threads, every range's
// weight exp(m_i - m) is computed once into shared memory, then thread d sums its value column over the ranges.
constexpr int kMergeCached = 256;      // ranges whose weights are kept in shared memory (more: recomputed per column)

template <typename T>
__global__ void __launch_bounds__(64) sink_attention_merge_kernel(T* __restrict__ out, int64_t out_stride,
                                                                  const float* __restrict__ part,
                                                                  const T* __restrict__ sink,
                                                                  const int* __restrict__ seq_start,
                                                                  const int* __restrict__ seq_list, int H, int Dv,
                                                                  int nsplit, int sink_heads) {
  pdl_prologue();
  __shared__ float wsm[kMergeCached];
  __shared__ float red[2];
  const int z = blockIdx.y, h = blockIdx.x, s = seq_list ? seq_list[z] : z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* p = part + ((int64_t)z * H + h) * nsplit * (Dv + 2);
  float mf = -INFINITY;
  for (int i = tid; i < nsplit; i += 64) mf = fmaxf(mf, p[i * (Dv + 2)]);
  mf = warp_reduce_max(mf);
  if (lane == 0) red[warp] = mf;
  __syncthreads();
  mf = fmaxf(red[0], red[1]);
  if (sink) mf = fmaxf(mf, to_f32(sink[h % sink_heads]));
  __syncthreads();
  float den = 0.f;
  for (int i = tid; i < nsplit; i += 64) {
    const float w = expf(p[i * (Dv + 2)] - mf);          // exp(-inf) = 0 for an empty range
    if (i < kMergeCached) wsm[i] = w;
    den += p[i * (Dv + 2) + 1] * w;
  }
  den = warp_reduce_sum(den);
  if (lane == 0) red[warp] = den;
  __syncthreads();
  den = red[0] + red[1];
  if (sink) den += expf(to_f32(sink[h % sink_heads]) - mf);
  T* o = out + (int64_t)seq_start[s] * out_stride + h * Dv;
  for (int d = tid; d < Dv; d += 64) {
    float v = 0.f;
    for (int i = 0; i < nsplit; ++i) {
      const float w = i < kMergeCached ? wsm[i] : expf(p[i * (Dv + 2)] - mf);
      v = fmaf(p[i * (Dv + 2) + 2 + d], w, v);
    }
    o[d] = from_f32<T>(v / den);
  }
}

// ---- one new token per sequence, softmax weights mixed ACROSS heads before they meet the values ---------------------
// p'_h(j) = sum_g M[h, g] p_g(j);  out_h = sum_j p'_h(j) v_kv(h)(j).  Two launches:
//   head_weights         CTA = (query head, sequence): thread j scores key j (its pool row read with 16-byte loads, q as
//                        fp32 in shared memory), softmax in fp32 over the CTA, NORMALISED weights to part [seq][H][chunk]
//   mixed_weights_values CTA = (query head h, sequence): the mixed weights of head h into shared memory (thread j sums
//                        over the heads), then warps over the keys and lanes over the value columns (16-byte loads) of
//                        the head's OWN kv head; the warps' sums meet in shared memory in a fixed order
// so the values are read once per query head, as in plain attention, and the mix costs H multiply-adds per key.
constexpr int kMixThreads = 256;

template <typename T>
__global__ void __launch_bounds__(128) head_weights_kernel(AttnArgs a) {
  pdl_prologue();
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __shared__ float red[4];
  constexpr int VEC = 16 / (int)sizeof(T);
  const int D = a.D, Dq = (D + 3) / 4 * 4;
  float* qs = reinterpret_cast<float*>(smem_raw);                        // [Dq]
  float* sc = qs + Dq;                                                    // [chunk]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int h = blockIdx.x, z = blockIdx.y, s = a.seq_list ? a.seq_list[z] : z;
  const int start = a.seq_start[s], ctx = a.seq_ctx[s];
  const int64_t slot = a.seq_slot[s];
  const int g = h / (a.H / a.G);
  const int lo = max(0, first_visible(a, ctx));
  const int n = min(ctx + 1 - lo, a.chunk);
  const T* q = (const T*)a.q + (int64_t)start * a.q_stride + h * D;
  for (int d = tid; d < D; d += 128) qs[d] = to_f32(q[d]);
  __syncthreads();
  const int* trow = a.table + slot * a.table_stride + lo;
  const T* kv = (const T*)a.kv + g * D;
  const float inv_cap = a.softcap > 0.f ? 1.0f / a.softcap : 0.f;
  const bool vec_ok = (D % VEC == 0) && (a.kv_stride % VEC == 0) && (((uintptr_t)a.kv % 16) == 0);
  float mx = -INFINITY;
  for (int j = tid; j < n; j += 128) {
    const T* kr = kv + (int64_t)trow[j] * a.kv_stride;
    float dot = 0.f;
    if (vec_ok) {                                  // 8 loads of the row in flight before the first product
      for (int d0 = 0; d0 < D; d0 += 8 * VEC) {
        uint4 raw[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) raw[u] = d0 + u * VEC < D ? ldg_128(kr + d0 + u * VEC) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const T* e = reinterpret_cast<const T*>(&raw[u]);
          if (d0 + u * VEC < D) {
#pragma unroll
            for (int c = 0; c < VEC; ++c) dot = fmaf(qs[d0 + u * VEC + c], to_f32(e[c]), dot);
          }
        }
      }
    } else {
      for (int d = 0; d < D; ++d) dot = fmaf(qs[d], to_f32(kr[d]), dot);
    }
    float sv = dot * a.scale;
    if (a.softcap > 0.f) sv = a.softcap * tanhf(sv * inv_cap);
    sc[j] = sv;
    mx = fmaxf(mx, sv);
  }
  mx = warp_reduce_max(mx);
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  __syncthreads();
  float sum = 0.f;
  for (int j = tid; j < n; j += 128) {
    const float p = expf(sc[j] - mx);
    sc[j] = p;
    sum += p;
  }
  sum = warp_reduce_sum(sum);
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  sum = (red[0] + red[1]) + (red[2] + red[3]);
  float* dst = a.part + ((int64_t)z * a.H + h) * a.chunk;
  for (int j = tid; j < n; j += 128) dst[j] = sc[j] / sum;
}

// lanes that share one key in mixed_weights_values (a power of two: enough 16-byte groups to cover the value head, at
// most a warp) and the floats of its merge buffer: one row of Dv sums per group of lanes
__host__ __device__ inline int mix_lanes_per_key(int Dv, int vec) {
  const int groups = (Dv + vec - 1) / vec;
  int l = 1;
  while (l < groups && l < 32) l *= 2;
  return l;
}
__host__ __device__ inline int mix_merge_floats(int Dv, int vec) { return kMixThreads / mix_lanes_per_key(Dv, vec) * Dv; }

template <typename T>
__global__ void __launch_bounds__(kMixThreads) mixed_weights_values_kernel(AttnArgs a, const T* __restrict__ mix) {
  pdl_prologue();
  extern __shared__ __align__(16) uint8_t smem_raw[];
  constexpr int VEC = 16 / (int)sizeof(T);
  const int Dv = a.Dv, H = a.H, chunk4 = (a.chunk + 3) / 4 * 4;
  float* pm = reinterpret_cast<float*>(smem_raw);                        // [chunk4] mixed weights
  int* rows = reinterpret_cast<int*>(pm + chunk4);                       // [chunk4] pool rows of the keys
  float* mrow = reinterpret_cast<float*>(rows + chunk4);                 // [H rounded to 4]
  float* mrg = mrow + (H + 3) / 4 * 4;                                   // [groups of lanes][Dv]
  const int tid = threadIdx.x;
  const int h = blockIdx.x, z = blockIdx.y, s = a.seq_list ? a.seq_list[z] : z;
  const int start = a.seq_start[s], ctx = a.seq_ctx[s];
  const int64_t slot = a.seq_slot[s];
  const int g = h / (H / a.G);
  const int lo = max(0, first_visible(a, ctx));
  const int n = min(ctx + 1 - lo, a.chunk);
  for (int i = tid; i < H; i += kMixThreads) mrow[i] = to_f32(mix[(int64_t)h * H + i]);
  __syncthreads();
  const float* P = a.part + (int64_t)z * H * a.chunk;
  const int* trow = a.table + slot * a.table_stride + lo;
  for (int j = tid; j < n; j += kMixThreads) {
    rows[j] = trow[j];
    float w = 0.f;
    for (int gg = 0; gg < H; ++gg) w = fmaf(mrow[gg], P[(int64_t)gg * a.chunk + j], w);
    pm[j] = w;
  }
  __syncthreads();
  const int v_col = a.v_col0 + g * a.v_hstride;
  const T* vbase = (const T*)a.kv + v_col;
  const bool vec_ok = (Dv % VEC == 0) && (a.kv_stride % VEC == 0) && (v_col % VEC == 0) && (((uintptr_t)a.kv % 16) == 0);
  const int lpk = mix_lanes_per_key(Dv, VEC), groups = kMixThreads / lpk;
  const int gi = tid / lpk, l = tid - gi * lpk;                          // group of lanes (one key at a time), lane in it
  for (int c0 = 0; c0 < Dv; c0 += lpk * VEC) {
    const int c = c0 + l * VEC;
    float acc[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
    if (vec_ok) {
      if (c < Dv) {
#pragma unroll 8
        for (int j = gi; j < n; j += groups) {
          const uint4 raw = ldg_128(vbase + (int64_t)rows[j] * a.kv_stride + c);
          const T* e = reinterpret_cast<const T*>(&raw);
          const float w = pm[j];
#pragma unroll
          for (int i = 0; i < VEC; ++i) acc[i] = fmaf(w, to_f32(e[i]), acc[i]);
        }
      }
    } else {
      for (int j = gi; j < n; j += groups) {
        const T* vr = vbase + (int64_t)rows[j] * a.kv_stride;
        const float w = pm[j];
#pragma unroll
        for (int i = 0; i < VEC; ++i)
          if (c + i < Dv) acc[i] = fmaf(w, to_f32(vr[c + i]), acc[i]);
      }
    }
#pragma unroll
    for (int i = 0; i < VEC; ++i)
      if (c + i < Dv) mrg[gi * Dv + c + i] = acc[i];
  }
  __syncthreads();
  T* o = (T*)a.out + (int64_t)start * a.out_stride + h * Dv;
  for (int d = tid; d < Dv; d += kMixThreads) {
    float v = 0.f;
    for (int w = 0; w < groups; ++w) v += mrg[w * Dv + d];             // a fixed order: the same sum in every batch
    o[d] = from_f32<T>(v);
  }
}

template <typename T>
int launch_mixed_head_attention(const AttnArgs& a, const void* mix, int64_t num_seqs, cudaStream_t st) {
  const size_t smem_w = (size_t)((a.D + 3) / 4 * 4 + a.chunk) * sizeof(float);
  const size_t smem_v = (size_t)(2 * ((a.chunk + 3) / 4 * 4) + (a.H + 3) / 4 * 4 +
                                 mix_merge_floats(a.Dv, 16 / (int)sizeof(T))) * sizeof(float);
  B2L_REQUIRE((int64_t)smem_w <= b2l_max_smem_optin() && (int64_t)smem_v <= b2l_max_smem_optin(),
              "mixed_head_attention: %d keys need %lld bytes of shared memory", a.chunk, (long long)(smem_w > smem_v ? smem_w : smem_v));
  const dim3 grid((unsigned)a.H, (unsigned)num_seqs);
  static int cache_w[64] = {0}, cache_v[64] = {0};
  B2L_CUDA_CHECK(b2l_ensure_dynamic_smem(head_weights_kernel<T>, (int)smem_w, cache_w));
  b2l_launch(head_weights_kernel<T>, grid, dim3(128), smem_w, st, a);
  B2L_CUDA_CHECK(b2l_ensure_dynamic_smem(mixed_weights_values_kernel<T>, (int)smem_v, cache_v));
  b2l_launch(mixed_weights_values_kernel<T>, grid, dim3(kMixThreads), smem_v, st, a, (const T*)mix);
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

__device__ __forceinline__ float block_sum2(float v, float* red) {
  v = warp_reduce_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : 0.f;
  t = warp_reduce_sum(t);
  __syncthreads();
  return t;
}

template <typename T>
__global__ void attn_prepare_kernel(T* __restrict__ qkv, int64_t stride, T* __restrict__ kv, int64_t kv_stride,
                                    const int* __restrict__ rows, const int* __restrict__ pos,
                                    const T* __restrict__ qw, const T* __restrict__ kw, const T* __restrict__ v_first_in,
                                    T* __restrict__ v_first_out, const T* __restrict__ lambda, int qn, int kn, int vn,
                                    float eps, float gain_coef, double gain_every) {
  pdl_prologue();
  __shared__ float red[32];
  const int64_t t = blockIdx.x;
  T* q = qkv + t * stride;
  T* k = q + qn;
  T* v = k + kn;
  T* dst = kv + (int64_t)rows[t] * kv_stride;
  float gain = 1.f;
  if (gain_every > 0.0) gain = 1.0f + gain_coef * logf((float)floor(((double)pos[t] + 1.0) / gain_every) + 1.0f);
  if (qw) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < qn; i += blockDim.x) { const float x = to_f32(q[i]); ss = fmaf(x, x, ss); }
    ss = block_sum2(ss, red);
    const float rr = 1.0f / sqrtf(ss / (float)qn + eps);
    for (int i = threadIdx.x; i < qn; i += blockDim.x) q[i] = from_f32<T>(to_f32(q[i]) * rr * to_f32(qw[i]) * gain);
  } else if (gain != 1.f) {
    for (int i = threadIdx.x; i < qn; i += blockDim.x) q[i] = from_f32<T>(to_f32(q[i]) * gain);
  }
  if (kw) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < kn; i += blockDim.x) { const float x = to_f32(k[i]); ss = fmaf(x, x, ss); }
    ss = block_sum2(ss, red);
    const float rr = 1.0f / sqrtf(ss / (float)kn + eps);
    for (int i = threadIdx.x; i < kn; i += blockDim.x) dst[i] = from_f32<T>(to_f32(k[i]) * rr * to_f32(kw[i]));
  } else {
    for (int i = threadIdx.x; i < kn; i += blockDim.x) dst[i] = k[i];
  }
  const float lam = (v_first_in && lambda) ? to_f32(lambda[0]) : 0.f;
  for (int i = threadIdx.x; i < vn; i += blockDim.x) {
    const T raw = v[i];
    if (v_first_out) v_first_out[t * vn + i] = raw;
    T val = raw;
    if (v_first_in) val = from_f32<T>((1.0f - lam) * to_f32(raw) + lam * to_f32(v_first_in[t * vn + i]));
    dst[kn + i] = val;
  }
}

// 16-byte version of attn_prepare: thread v owns vectors v, v + 256, ... of each part; q (at most kPrepQ vectors per
// thread) stays in registers between the statistic and the scaling.
constexpr int kPrepQ = 2;

template <typename T>
__global__ void __launch_bounds__(256) attn_prepare_vec_kernel(
    T* __restrict__ qkv, int64_t stride, T* __restrict__ kv, int64_t kv_stride, const int* __restrict__ rows,
    const int* __restrict__ pos, const T* __restrict__ qw, const T* __restrict__ kw, const T* __restrict__ v_first_in,
    T* __restrict__ v_first_out, const T* __restrict__ lambda, int qn, int kn, int vn, float eps, float gain_coef,
    double gain_every) {
  pdl_prologue();
  constexpr int VEC = 16 / (int)sizeof(T);
  __shared__ float red[32];
  const int64_t t = blockIdx.x;
  T* q = qkv + t * stride;
  T* k = q + qn;
  T* v = k + kn;
  T* dst = kv + (int64_t)rows[t] * kv_stride;
  float gain = 1.f;
  if (gain_every > 0.0) gain = 1.0f + gain_coef * logf((float)floor(((double)pos[t] + 1.0) / gain_every) + 1.0f);
  {
    uint4 raw[kPrepQ];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < kPrepQ; ++u) {
      const int i = (threadIdx.x + u * 256) * VEC;
      raw[u] = make_uint4(0u, 0u, 0u, 0u);
      if (i < qn) raw[u] = *reinterpret_cast<const uint4*>(q + i);
      const T* e = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
      for (int c = 0; c < VEC; ++c) { const float x = to_f32(e[c]); ss = fmaf(x, x, ss); }
    }
    float rr = 1.f;
    if (qw) rr = 1.0f / sqrtf(block_sum2(ss, red) / (float)qn + eps);
    if (qw || gain != 1.f) {
#pragma unroll
      for (int u = 0; u < kPrepQ; ++u) {
        const int i = (threadIdx.x + u * 256) * VEC;
        if (i >= qn) continue;
        const T* e = reinterpret_cast<const T*>(&raw[u]);
        uint4 wr = make_uint4(0u, 0u, 0u, 0u);
        if (qw) wr = ldg_128(qw + i);
        const T* we = reinterpret_cast<const T*>(&wr);
        uint4 res;
        T* re = reinterpret_cast<T*>(&res);
#pragma unroll
        for (int c = 0; c < VEC; ++c) re[c] = from_f32<T>(to_f32(e[c]) * rr * (qw ? to_f32(we[c]) : 1.f) * gain);
        *reinterpret_cast<uint4*>(q + i) = res;
      }
    }
  }
  {
    const int i = threadIdx.x * VEC;                 // kn <= 256 vectors (checked on the host)
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (i < kn) raw = *reinterpret_cast<const uint4*>(k + i);
    const T* e = reinterpret_cast<const T*>(&raw);
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < VEC; ++c) { const float x = to_f32(e[c]); ss = fmaf(x, x, ss); }
    float rr = 1.f;
    if (kw) rr = 1.0f / sqrtf(block_sum2(ss, red) / (float)kn + eps);
    if (i < kn) {
      uint4 res = raw;
      if (kw) {
        const uint4 wr = ldg_128(kw + i);
        const T* we = reinterpret_cast<const T*>(&wr);
        T* re = reinterpret_cast<T*>(&res);
#pragma unroll
        for (int c = 0; c < VEC; ++c) re[c] = from_f32<T>(to_f32(e[c]) * rr * to_f32(we[c]));
      }
      *reinterpret_cast<uint4*>(dst + i) = res;
    }
  }
  const float lam = (v_first_in && lambda) ? to_f32(lambda[0]) : 0.f;
  for (int i = threadIdx.x * VEC; i < vn; i += 256 * VEC) {
    const uint4 raw = *reinterpret_cast<const uint4*>(v + i);
    if (v_first_out) *reinterpret_cast<uint4*>(v_first_out + t * vn + i) = raw;
    uint4 res = raw;
    if (v_first_in) {
      const uint4 fr = ldg_128(v_first_in + t * vn + i);
      const T* e = reinterpret_cast<const T*>(&raw);
      const T* fe = reinterpret_cast<const T*>(&fr);
      T* re = reinterpret_cast<T*>(&res);
#pragma unroll
      for (int c = 0; c < VEC; ++c) re[c] = from_f32<T>((1.0f - lam) * to_f32(e[c]) + lam * to_f32(fe[c]));
    }
    *reinterpret_cast<uint4*>(dst + kn + i) = res;
  }
}

template <typename T>
int launch_attention(const AttnArgs& a, dim3 grid, cudaStream_t st) {
  const size_t smem = (size_t)(kRows * a.D + kKeys * (a.D + 1) + kKeys * a.Dv) * sizeof(float);
  B2L_REQUIRE((int64_t)smem <= b2l_max_smem_optin(), "sink_attention: head sizes %d / %d need %lld bytes of shared memory",
              a.D, a.Dv, (long long)smem);
  const int dvj = (a.Dv + 31) / 32;
  B2L_REQUIRE(dvj <= 8, "sink_attention: value head size %d > 256", a.Dv);
#define B2L_ATTN(J)                                                                                           \
  do {                                                                                                        \
    static int cache[64] = {0};                                                                               \
    B2L_CUDA_CHECK(b2l_ensure_dynamic_smem(sink_attention_kernel<T, J>, (int)smem, cache));                   \
    b2l_launch(sink_attention_kernel<T, J>, grid, dim3(kWarps * 32), smem, st, a);                            \
  } while (0)
  if (dvj <= 2) B2L_ATTN(2);
  else if (dvj <= 4) B2L_ATTN(4);
  else B2L_ATTN(8);
#undef B2L_ATTN
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

}  // namespace

extern "C" int b2l_attn_prepare(void* qkv, int64_t qkv_row_stride, void* kv_pool, int64_t kv_row_stride,
                                const void* kv_rows_i32, const void* pos_i32, const void* q_norm_weight,
                                const void* k_norm_weight, const void* v_first_in, void* v_first_out,
                                const void* v_lambda, int64_t tokens, int q_cols, int k_cols, int v_cols, float eps,
                                float gain_coef, float gain_every, int dtype, void* stream) {
  B2L_REQUIRE(qkv && kv_pool && kv_rows_i32 && pos_i32, "attn_prepare: null pointer");
  B2L_REQUIRE(q_cols > 0 && k_cols > 0 && v_cols > 0, "attn_prepare: bad shape");
  if (tokens <= 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  B2L_DISPATCH_FLOAT(dtype, "attn_prepare", {
    constexpr int VEC = 16 / (int)sizeof(T);
    auto al = [](const void* p) { return p == nullptr || (uintptr_t)p % 16 == 0; };
    const bool vec = q_cols % VEC == 0 && k_cols % VEC == 0 && v_cols % VEC == 0 && qkv_row_stride % VEC == 0 &&
                     kv_row_stride % VEC == 0 && q_cols <= kPrepQ * 256 * VEC && k_cols <= 256 * VEC && al(qkv) &&
                     al(kv_pool) && al(q_norm_weight) && al(k_norm_weight) && al(v_first_in) && al(v_first_out);
    if (vec)
      b2l_launch(attn_prepare_vec_kernel<T>, dim3((unsigned)tokens), dim3(256), (size_t)0, st, (T*)qkv, qkv_row_stride,
                 (T*)kv_pool, kv_row_stride, (const int*)kv_rows_i32, (const int*)pos_i32, (const T*)q_norm_weight,
                 (const T*)k_norm_weight, (const T*)v_first_in, (T*)v_first_out, (const T*)v_lambda, q_cols, k_cols,
                 v_cols, eps, gain_coef, (double)gain_every);
    else
    b2l_launch(attn_prepare_kernel<T>, dim3((unsigned)tokens), dim3(256), (size_t)0, st, (T*)qkv, qkv_row_stride,
               (T*)kv_pool, kv_row_stride, (const int*)kv_rows_i32, (const int*)pos_i32, (const T*)q_norm_weight,
               (const T*)k_norm_weight, (const T*)v_first_in, (T*)v_first_out, (const T*)v_lambda, q_cols, k_cols,
               v_cols, eps, gain_coef, (double)gain_every);
  });
  B2L_LAUNCH_CHECK();
  return B2L_OK;
}

extern "C" int64_t b2l_sink_attention_workspace_bytes(int64_t num_seqs, int heads, int v_head_dim, int num_splits) {
  if (num_splits <= 0) return 0;
  return num_seqs * heads * (int64_t)num_splits * (v_head_dim + 2) * 4;
}

/* num_splits == 0: tiled mode over `max_q_len`-token sequences; > 0: split mode, every listed sequence brings ONE token
 * and `split_keys` keys go to each of the num_splits ranges, counted from the token's first visible key
 * (num_splits * split_keys >= the most keys any listed token sees: context + 1, or the window if that is smaller).
 * window <= 0: no sliding window; block > 0 (window <= 0): block-diagonal mask; v_col0 < 0: the values follow the keys in a pool row (column kv_heads * head_dim);
 * v_head_stride < 0: kv head g's values start g * v_head_dim columns after v_col0 (0: all kv heads read the same columns).
 * v_blocks > 1 (split mode): block c of v_head_dim value columns starts c * v_head_dim columns further and is one more
 * set of `heads` results, out [v_blocks][heads][v_head_dim] per token, in the same two launches (workspace for
 * heads * v_blocks heads). */
extern "C" int b2l_sink_attention(void* out, int64_t out_row_stride, const void* q, int64_t q_row_stride,
                                  const void* kv_pool, int64_t kv_row_stride, const void* table_i32,
                                  int64_t table_row_stride, const void* seq_start, const void* seq_ctx,
                                  const void* seq_slot, const void* seq_list, int64_t num_seqs, int max_q_len,
                                  const void* sink, int heads, int kv_heads, int head_dim, int v_head_dim, float scale,
                                  float softcap, int window, int block, int v_col0, int v_head_stride, int v_blocks,
                                  int num_splits, int split_keys, void* workspace, int64_t workspace_bytes, int dtype, void* stream) {
  B2L_REQUIRE(out && q && kv_pool && table_i32 && seq_start && seq_ctx && seq_slot, "sink_attention: null pointer");
  B2L_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0, "sink_attention: %d heads must be a multiple of num_kv_heads %d",
              heads, kv_heads);
  B2L_REQUIRE(head_dim > 0 && v_head_dim > 0 && max_q_len >= 1, "sink_attention: bad shape");
  if (num_seqs <= 0) return B2L_OK;
  cudaStream_t st = (cudaStream_t)stream;
  AttnArgs a;
  a.q = q; a.q_stride = q_row_stride; a.kv = kv_pool; a.kv_stride = kv_row_stride;
  a.table = (const int*)table_i32; a.table_stride = table_row_stride;
  a.seq_start = (const int*)seq_start; a.seq_ctx = (const int*)seq_ctx; a.seq_slot = (const int*)seq_slot;
  a.seq_list = (const int*)seq_list; a.sink = sink; a.out = out; a.out_stride = out_row_stride;
  a.part = (float*)workspace;
  a.H = heads; a.G = kv_heads; a.D = head_dim; a.Dv = v_head_dim;
  const int per = heads / kv_heads;
  a.PH = per < kRows ? per : kRows;
  a.BQ = kRows / a.PH;
  a.nsplit = num_splits; a.chunk = split_keys; a.scale = scale; a.softcap = softcap;
  a.window = window > 0 ? window : 0;
  a.block = (window <= 0 && block > 0) ? block : 0;
  a.v_col0 = v_col0 >= 0 ? v_col0 : kv_heads * head_dim;
  a.v_hstride = v_head_stride >= 0 ? v_head_stride : v_head_dim;
  a.head_rows = 0;
  a.v_blocks = v_blocks > 1 ? v_blocks : 1;
  B2L_REQUIRE(a.v_blocks == 1 || num_splits > 0, "sink_attention: value blocks are for steps of single tokens");
  const int hchunks = (per + a.PH - 1) / a.PH;
  if (num_splits > 0) {
    B2L_REQUIRE(split_keys > 0, "sink_attention: split_keys must be positive");
    const int64_t need = b2l_sink_attention_workspace_bytes(num_seqs, heads * a.v_blocks, v_head_dim, num_splits);
    B2L_REQUIRE(workspace && workspace_bytes >= need, "sink_attention: workspace too small (%lld < %lld)",
                (long long)workspace_bytes, (long long)need);
    int rc = B2L_OK;
    // many query heads per kv head (latent caches: ALL heads share one row): the heads become the rows of a tensor-core
    // tile, so a cached row is read once and scored against every head by mma instead of 4 heads at a time on the
    // CUDA cores; same partials, same merge
    if (per > kSplitRows && a.v_blocks == 1 && mma_path_ok(a, dtype)) {
      a.head_rows = 1;
      rc = dtype == B2L_F16 ? dispatch_attention_mma<__half>(a, 1, num_seqs, st)
                            : dispatch_attention_mma<__nv_bfloat16>(a, 1, num_seqs, st);
    } else {
      B2L_DISPATCH_FLOAT(dtype, "sink_attention", { rc = launch_attention_split<T>(a, num_seqs, st); });
    }
    if (rc != B2L_OK) return rc;
    B2L_DISPATCH_FLOAT(dtype, "sink_attention", {
      b2l_launch(sink_attention_merge_kernel<T>, dim3((unsigned)(heads * a.v_blocks), (unsigned)num_seqs), dim3(64),
                 (size_t)0, st, (T*)out, out_row_stride, (const float*)workspace, (const T*)sink,
                 (const int*)seq_start, (const int*)seq_list, heads * a.v_blocks, v_head_dim, num_splits, heads);
    });
    B2L_LAUNCH_CHECK();
    return B2L_OK;
  }
  if (mma_path_ok(a, dtype)) {
    if (dtype == B2L_F16) return dispatch_attention_mma<__half>(a, max_q_len, num_seqs, st);
    return dispatch_attention_mma<__nv_bfloat16>(a, max_q_len, num_seqs, st);
  }
  const dim3 grid((unsigned)((max_q_len + a.BQ - 1) / a.BQ), (unsigned)(kv_heads * hchunks), (unsigned)num_seqs);
  int rc = B2L_OK;
  B2L_DISPATCH_FLOAT(dtype, "sink_attention", { rc = launch_attention<T>(a, grid, st); });
  return rc;
}

extern "C" int64_t b2l_mixed_head_attention_workspace_bytes(int64_t num_seqs, int heads, int max_keys) {
  return num_seqs * (int64_t)heads * max_keys * (int64_t)sizeof(float);
}

/* One new token per listed sequence; the heads' softmax weights are mixed by mix [heads, heads] (element type of q,
 * row h = the weights of head h's sum over the heads) before each head applies them to its own kv head's values.
 * max_keys: an upper bound of the keys any listed token sees (its window, or its context + 1). */
extern "C" int b2l_mixed_head_attention(void* out, int64_t out_row_stride, const void* q, int64_t q_row_stride,
                                        const void* kv_pool, int64_t kv_row_stride, const void* table_i32,
                                        int64_t table_row_stride, const void* seq_start, const void* seq_ctx,
                                        const void* seq_slot, const void* seq_list, int64_t num_seqs, const void* mix,
                                        int heads, int kv_heads, int head_dim, int v_head_dim, float scale, float softcap,
                                        int window, int block, int v_col0, int max_keys, void* workspace,
                                        int64_t workspace_bytes, int dtype, void* stream) {
  if (num_seqs <= 0) return B2L_OK;
  B2L_REQUIRE(out && q && kv_pool && table_i32 && seq_start && seq_ctx && seq_slot && mix, "mixed_head_attention: null pointer");
  B2L_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && head_dim > 0 && v_head_dim > 0 && max_keys > 0,
              "mixed_head_attention: bad geometry");
  const int64_t need = b2l_mixed_head_attention_workspace_bytes(num_seqs, heads, max_keys);
  B2L_REQUIRE(workspace && workspace_bytes >= need, "mixed_head_attention: workspace too small (%lld < %lld)",
              (long long)workspace_bytes, (long long)need);
  AttnArgs a{};
  a.q = q; a.q_stride = q_row_stride; a.kv = kv_pool; a.kv_stride = kv_row_stride;
  a.table = (const int*)table_i32; a.table_stride = table_row_stride;
  a.seq_start = (const int*)seq_start; a.seq_ctx = (const int*)seq_ctx; a.seq_slot = (const int*)seq_slot;
  a.seq_list = (const int*)seq_list;
  a.out = out; a.out_stride = out_row_stride; a.part = (float*)workspace;
  a.H = heads; a.G = kv_heads; a.D = head_dim; a.Dv = v_head_dim;
  a.chunk = max_keys; a.scale = scale; a.softcap = softcap;
  a.window = window > 0 ? window : 0;
  a.block = (window <= 0 && block > 0) ? block : 0;
  a.v_col0 = v_col0 >= 0 ? v_col0 : kv_heads * head_dim;
  a.v_hstride = v_head_dim;
  a.v_blocks = 1;
  cudaStream_t st = (cudaStream_t)stream;
  int rc = B2L_OK;
  B2L_DISPATCH_FLOAT(dtype, "mixed_head_attention", { rc = launch_mixed_head_attention<T>(a, mix, num_seqs, st); });
  return rc;
}
