// Causal FLARE: y_t = softmax_M(S[:, t]) . z_t with z_t = softmax_{n <= t}(S) v   (S = scale q k^T).
//
// The reference links this path without code, formula or test vector (figs/flare_decoder.py animates a
// decoder diagram, nothing more), so the definition above is this library's own choice: token t sees the
// latent summary of tokens 0..t inclusive, which makes token-by-token decoding on a per-(b, h) state
// (m[M], l[M], acc[M, D]) reproduce the prefill.  The state is the same split-N record the non-causal
// gather produces, so prefill is three passes:
//
//   1. flare_gather_partial with 128-token ranges: one record per chunk           (existing kernels)
//   2. k_causal_scan: exclusive log-sum-exp prefix of the records along the chunk axis, in place;
//      the inclusive total is the state after the last token
//   3. k_causal_walk: per (b, h, chunk), start from the chunk's prefix record and walk its tokens:
//      acc_m += e^{s_mt - mu_m} v_t,  y_t = sum_m softmax_M(s_:t)_m / l_mt * acc_m
//
// and decode is one launch of the same kernel per token on the caller's record.  Pass 3 and decode are fp32
// SIMT kernels: thread (d, g) keeps acc[m][d] of its latents m = g, g + G, ... in registers, scores and
// weights of a 32-token sub-chunk sit in shared memory (two CTAs per SM).  Scores are computed once per token; the
// sequential part is O(T M D) fused multiply-adds per chunk, the minimum for this recurrence.
#include <cstdarg>
#include <cstdio>
#include <cuda_runtime.h>
#include "common.cuh"
#include "launch.h"

namespace flare { void set_last_error(const char* msg); }

namespace {

using namespace flare;

constexpr int kThreads = 256;
constexpr int kSub = 32;          // tokens per sub-chunk (two CTAs per SM fit with this)
constexpr int kChunk = 128;       // tokens per record (pass 1 range length)
constexpr int kMaxLat = 32;       // latents per thread

int refuse(int code, const char* fmt, ...) {
  char msg[400];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(msg, sizeof(msg), fmt, ap);
  va_end(ap);
  flare::set_last_error(msg);
  return code;
}

// ---------------------------------------------------------------------------------------------
// pass 2: exclusive prefix of records along the chunk axis.  rec[c][row][D+2]; one warp per row.
// ---------------------------------------------------------------------------------------------
constexpr int kScanThreads = 128;
constexpr int kScanRows = 2;      // rows per warp, walked side by side

// The head dimension is a template parameter and a lane owns pairs of adjacent columns (one 8-byte access per 64
// columns; rows are D + 2 floats, so 8-byte aligned): about 25 instructions per row and chunk.  With D a run-time
// value, 4-byte accesses and 64-bit index arithmetic per access it was 109, and the kernel issue bound at a third of
// the memory bandwidth.
// COMPACT (behind the tensor-core record pass): the records are pacc[c][row][D] in 16 bits (what the tensor-core walk
// multiplies with anyway) and pml[c][row] = (m, l), scanned in place like the fp32 ones: half the bytes in every
// pass, and rows the walk can fetch in 16-byte pieces.  The sums themselves stay in fp32 registers.
template <int D, bool COMPACT>
__global__ void __launch_bounds__(kScanThreads, D == 128 ? 5 : 8)
k_causal_scan(float* __restrict__ rec, int n_chunks, long long rows, const float* __restrict__ state_in,
              float* __restrict__ state_out, __nv_bfloat16* __restrict__ pacc, float2* __restrict__ pml) {
  grid_dep_sync();
  constexpr int W = D + 2;
  constexpr int VEC = D >= 64 ? 2 : 1;             // floats per access
  constexpr int NLD = D >= 64 ? D / 64 : 1;        // accesses per row: columns 64 i + 2 lane (+1), or column lane
  const int lane = threadIdx.x % 32;
  const bool lane_on = D >= 32 || lane < D;
  const int col = VEC * lane;
  const long long row0 = ((long long)blockIdx.x * (kScanThreads / 32) + threadIdx.x / 32) * kScanRows;
  if (row0 >= rows) return;
  const long long cs = rows * W;
  // A warp's chain is latency bound and a record is only (D + 2) floats: two rows per warp and kAhead records of each
  // in flight keep the memory system busy, and half as many warps fit the GPU in one wave.
  constexpr int kAhead = 4;
  bool on[kScanRows];
  long long rw_[kScanRows];
  float* wp[kScanRows];                            // the record this row writes next
  const float* fp[kScanRows];                      // the record it fetches next
  float m[kScanRows], l[kScanRows], acc[kScanRows][NLD][VEC];
  float2 mlb[kScanRows][kAhead];
  float ab[kScanRows][kAhead][NLD][VEC];
  auto load_acc = [&](const float* r, float (&ao)[NLD][VEC]) {
#pragma unroll
    for (int i = 0; i < NLD; ++i) {
      if constexpr (VEC == 2) {
        const float2 t = *reinterpret_cast<const float2*>(r + 64 * i + col);
        ao[i][0] = t.x; ao[i][1] = t.y;
      } else {
        ao[i][0] = lane_on ? r[col] : 0.f;
      }
    }
  };
  auto store_acc = [&](float* r, const float (&ao)[NLD][VEC]) {
#pragma unroll
    for (int i = 0; i < NLD; ++i) {
      if constexpr (VEC == 2) *reinterpret_cast<float2*>(r + 64 * i + col) = make_float2(ao[i][0], ao[i][1]);
      else if (lane_on) r[col] = ao[i][0];
    }
  };
  // record c of row q into slot u
  auto fetch = [&](int q, int u, int c) {
    if constexpr (COMPACT) {
      const long long i = (long long)c * rows + rw_[q];
      mlb[q][u] = pml[i];
      const __nv_bfloat16* pr = pacc + i * D;
#pragma unroll
      for (int k = 0; k < NLD; ++k) {
        if constexpr (VEC == 2) {
          const float2 t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(pr + 64 * k + col));
          ab[q][u][k][0] = t.x; ab[q][u][k][1] = t.y;
        } else {
          ab[q][u][k][0] = lane_on ? __bfloat162float(pr[col]) : 0.f;
        }
      }
    } else {
      mlb[q][u] = *reinterpret_cast<const float2*>(fp[q] + D);
      load_acc(fp[q], ab[q][u]);
      fp[q] += cs;
    }
  };
#pragma unroll
  for (int q = 0; q < kScanRows; ++q) {
    on[q] = row0 + q < rows;
    const long long rw = on[q] ? row0 + q : row0;  // a row past the end repeats row0's loads and stores nothing
    rw_[q] = rw;
    wp[q] = rec + rw * W;
    fp[q] = wp[q];
    m[q] = -INFINITY; l[q] = 0.f;
#pragma unroll
    for (int i = 0; i < NLD; ++i)
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc[q][i][j] = 0.f;
    if (state_in) {
      const float* si = state_in + rw * W;
      const float2 ml = *reinterpret_cast<const float2*>(si + D);
      m[q] = ml.x; l[q] = ml.y;
      load_acc(si, acc[q]);
    }
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      mlb[q][u] = make_float2(-INFINITY, 0.f);
#pragma unroll
      for (int i = 0; i < NLD; ++i)
#pragma unroll
        for (int j = 0; j < VEC; ++j) ab[q][u][i][j] = 0.f;
      if (u < n_chunks) {
        fetch(q, u, u);
      }
    }
  }
  for (int c0 = 0; c0 < n_chunks; c0 += kAhead) {
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      const int c = c0 + u;
      if (c < n_chunks) {
#pragma unroll
        for (int q = 0; q < kScanRows; ++q) {
          const float mc = mlb[q][u].x, lc = mlb[q][u].y;
          float ac[NLD][VEC];
#pragma unroll
          for (int i = 0; i < NLD; ++i)
#pragma unroll
            for (int j = 0; j < VEC; ++j) ac[i][j] = ab[q][u][i][j];
          if (c + kAhead < n_chunks) {
            fetch(q, u, c + kAhead);
          }
          __syncwarp();
          if (on[q]) {                             // the record of everything before chunk c
            if constexpr (COMPACT) {
              __nv_bfloat16* pr = pacc + ((long long)c * rows + rw_[q]) * D;
#pragma unroll
              for (int i = 0; i < NLD; ++i) {
                if constexpr (VEC == 2)
                  *reinterpret_cast<__nv_bfloat162*>(pr + 64 * i + col) = __floats2bfloat162_rn(acc[q][i][0], acc[q][i][1]);
                else if (lane_on) pr[col] = __float2bfloat16_rn(acc[q][i][0]);
              }
              if (lane == 0) pml[(long long)c * rows + rw_[q]] = make_float2(m[q], l[q]);
            } else {
              store_acc(wp[q], acc[q]);
              if (lane == 0) *reinterpret_cast<float2*>(wp[q] + D) = make_float2(m[q], l[q]);
            }
          }
          wp[q] += cs;
          const float mn = fmaxf(m[q], mc);
          const float wa = (m[q] == -INFINITY) ? 0.f : __expf(m[q] - mn);
          const float wc = (mc == -INFINITY) ? 0.f : __expf(mc - mn);
          l[q] = wa * l[q] + wc * lc;
#pragma unroll
          for (int i = 0; i < NLD; ++i)
#pragma unroll
            for (int j = 0; j < VEC; ++j) acc[q][i][j] = wa * acc[q][i][j] + wc * ac[i][j];
          m[q] = mn;
        }
      }
    }
  }
  if (state_out) {
#pragma unroll
    for (int q = 0; q < kScanRows; ++q) {
      if (on[q]) {
        float* so = state_out + (row0 + q) * W;
        store_acc(so, acc[q]);
        if (lane == 0) *reinterpret_cast<float2*>(so + D) = make_float2(m[q], l[q]);
      }
    }
  }
}

void launch_scan(bool dependent, float* rec, int n_chunks, long long rows, int D, const float* state_in, float* state_out,
                 __nv_bfloat16* pacc, float2* pml, cudaStream_t st) {
  const int rpb = kScanThreads / 32 * kScanRows;
  const dim3 grid((unsigned)((rows + rpb - 1) / rpb)), block(kScanThreads);
  auto go = [&](auto kernel) {
    if (dependent) launch_dep(kernel, grid, block, 0, st, rec, n_chunks, rows, state_in, state_out, pacc, pml);
    else kernel<<<grid, block, 0, st>>>(rec, n_chunks, rows, state_in, state_out, pacc, pml);
  };
  if (pacc) {                                      // behind the tensor-core record pass: D is 32 or 64
    if (D == 32) go(k_causal_scan<32, true>); else go(k_causal_scan<64, true>);
    return;
  }
  switch (D) {                                     // fill_args admits exactly these
    case 16: go(k_causal_scan<16, false>); break;
    case 32: go(k_causal_scan<32, false>); break;
    case 64: go(k_causal_scan<64, false>); break;
    default: go(k_causal_scan<128, false>); break;
  }
}

// ---------------------------------------------------------------------------------------------
// pass 3 / decode: walk `cnt` tokens starting from a record.
// Shared memory: q [M][D] fp32, k/v sub-chunk [kSub][D] fp32, S->G [kSub][M], E [kSub][M],
// mu/l/a [M], cmax/csum [kSub], ypart [2][G][D] (rows padded by one float).
// ---------------------------------------------------------------------------------------------
struct CausalArgs {
  int B, H, N, M, D;
  float scale;
  long long qs[3], ks[3], vs[3], ys[3];
  const void* q; const void* k; const void* v; void* y;
  const float* prefix;         // [n_chunks][B][H][M][D+2]: the record before each chunk
  float* state;                // decode: [B][H][M][D+2], updated in place (prefix == nullptr)
  int tokens_per_cta;          // kChunk in prefill, N (usually 1) in decode
  const int* redo;             // prefill behind the tensor-core walk: [chunks][B*H], only the flagged units are walked
  int n_units;                 // chunks * B * H (redo mode)
  const __nv_bfloat16* pacc;   // redo mode: the prefix as the scan wrote it for the tensor-core walk,
  const float2* pml;           //   acc [chunks][B][H][M][D] in 16 bits and (m, l) [chunks][B][H][M]
};

template <typename T, int D>
__global__ void __launch_bounds__(kThreads)
k_causal_walk(CausalArgs a) {
  grid_dep_sync();
  constexpr int G = kThreads / D;                  // latent groups
  extern __shared__ __align__(16) float sm[];
  const int M = a.M;
  constexpr int DP = D + 1;                        // padded rows: no bank conflicts when a warp walks rows
  const int MP = M + 4;                            // keeps rows 16-byte aligned for the recurrence's vector loads
  float* sQ = sm;                                  // [M][DP]
  float* sK = sQ + M * DP;                         // [kSub][DP]
  float* sV = sK + kSub * DP;                      // [kSub][D]
  float* sS = sV + kSub * D;                       // [kSub][MP]  scores, then weights
  float* sE = sS + kSub * MP;                      // [kSub][MP]
  float* sMu = sE + kSub * MP;                     // [M]
  float* sL = sMu + M;                             // [M]
  float* sA = sL + M;                              // [M]
  float* sCm = sA + M;                             // [kSub]
  float* sCs = sCm + kSub;                         // [kSub]
  float* sY = sCs + kSub;                          // [2][G][D]

  const int tid = threadIdx.x;
  const int d = tid % D, g = tid / D;
  const int nlat = M / G;                          // latents of this thread: g * nlat ... g * nlat + nlat - 1
  // Redo mode (behind the tensor-core walk): a small one-dimensional grid strides over the (chunk, b*h) units and
  // takes the flagged ones; otherwise one CTA per unit.
  const int n_bh = a.B * a.H;
  int next_base = blockIdx.x, cur_base = 0;
  unsigned flagged = 0;                            // of the units cur_base + lane * gridDim.x: the same in every warp
  for (;;) {
  int chunk = blockIdx.x, bh = blockIdx.y;
  if (a.redo) {
    while (flagged == 0 && next_base < a.n_units) {                    // 32 flags per round, read side by side
      cur_base = next_base; next_base += 32 * (int)gridDim.x;
      const int u = cur_base + (tid & 31) * (int)gridDim.x;
      flagged = __ballot_sync(0xffffffffu, u < a.n_units && a.redo[u] != 0);
    }
    if (flagged == 0) break;
    const int unit = cur_base + (__ffs(flagged) - 1) * (int)gridDim.x;
    flagged &= flagged - 1;
    chunk = unit / n_bh; bh = unit % n_bh;
  }
  const int b = bh / a.H, h = bh % a.H;
  const int n0 = chunk * a.tokens_per_cta, n1 = min(a.N, n0 + a.tokens_per_cta);
  const int W = D + 2;

  const T* qp = reinterpret_cast<const T*>(a.q) + b * a.qs[0] + h * a.qs[1];
  const T* kp = reinterpret_cast<const T*>(a.k) + b * a.ks[0] + h * a.ks[1];
  const T* vp = reinterpret_cast<const T*>(a.v) + b * a.vs[0] + h * a.vs[1];
  T* yp = reinterpret_cast<T*>(a.y) + b * a.ys[0] + h * a.ys[1];
  const float* rec = a.prefix ? a.prefix + (((long long)chunk * a.B + b) * a.H + h) * M * W
                              : a.state + ((long long)b * a.H + h) * M * W;

  for (int i = tid; i < M * D; i += kThreads) sQ[(i / D) * DP + i % D] = to_f32(qp[(i / D) * a.qs[2] + i % D]);
  const long long prow = (((long long)chunk * a.B + b) * a.H + h) * M;      // first row of this unit in pacc / pml
  for (int m = tid; m < M; m += kThreads) {
    if (a.pacc) { const float2 ml = a.pml[prow + m]; sMu[m] = ml.x; sL[m] = ml.y; }
    else { sMu[m] = rec[m * W + D]; sL[m] = rec[m * W + D + 1]; }
  }
  float acc[kMaxLat];
#pragma unroll
  for (int j = 0; j < kMaxLat; ++j)
    acc[j] = (j < nlat) ? (a.pacc ? __bfloat162float(a.pacc[(prow + g * nlat + j) * D + d]) : rec[(g * nlat + j) * W + d]) : 0.f;
  __syncthreads();

  // E, l and acc of a sub-chunk are relative to the running maximum at its end, so l_mt >= e^{first - mu} with
  // `first` the running maximum after its first token.  Where the scores of some latent climb by more than
  // kSpread inside one sub-chunk that bound nears the underflow of fp32: from there on the chunk is walked token
  // by token (a one-token step has l >= l0 or e = 1).
  constexpr float kSpread = 60.f;
  int sub = kSub;
  for (int s0 = n0; s0 < n1;) {
    const int cnt = min(sub, n1 - s0);
    for (int i = tid; i < cnt * D; i += kThreads) {
      const int t = i / D, dd = i % D;
      sK[t * DP + dd] = to_f32(kp[(long long)(s0 + t) * a.ks[2] + dd]);
      sV[i] = to_f32(vp[(long long)(s0 + t) * a.vs[2] + dd]);
    }
    __syncthreads();
    // scores S[t][m] = scale q_m . k_t.  Few tokens (decode): one dot product per thread.
    if (cnt < 8) {
      for (int i = tid; i < cnt * M; i += kThreads) {
        const int t = i / M, m = i % M;
        const float* qr = sQ + m * DP;
        const float* kr = sK + t * DP;
        float sacc = 0.f;
#pragma unroll 8
        for (int dd = 0; dd < D; ++dd) sacc = fmaf(qr[dd], kr[dd], sacc);
        sS[t * MP + m] = sacc * a.scale;
      }
    } else {
      // thread (mg, tg) computes latents mg + 32a and tokens 4tg + b in registers, so every shared-memory
      // load feeds 4 (q) or up to 16 (k) multiply-adds
      const int mg = tid & 31, tg = tid >> 5;
      const int rm = (M + 31) >> 5;                // latents per thread, at most 16 (M <= 512)
      float sc[16][4];
#pragma unroll
      for (int a_ = 0; a_ < 16; ++a_)
#pragma unroll
        for (int b_ = 0; b_ < 4; ++b_) sc[a_][b_] = 0.f;
      const float* k0 = sK + (4 * tg) * DP;
      for (int dd = 0; dd < D; ++dd) {
        const float kv0 = k0[dd], kv1 = k0[DP + dd], kv2 = k0[2 * DP + dd], kv3 = k0[3 * DP + dd];
#pragma unroll
        for (int a_ = 0; a_ < 16; ++a_) {
          if (a_ < rm) {
            const int m = min(mg + 32 * a_, M - 1);
            const float qv = sQ[m * DP + dd];
            sc[a_][0] = fmaf(qv, kv0, sc[a_][0]); sc[a_][1] = fmaf(qv, kv1, sc[a_][1]);
            sc[a_][2] = fmaf(qv, kv2, sc[a_][2]); sc[a_][3] = fmaf(qv, kv3, sc[a_][3]);
          }
        }
      }
#pragma unroll
      for (int a_ = 0; a_ < 16; ++a_) {
        const int m = mg + 32 * a_;
        if (a_ < rm && m < M) {
#pragma unroll
          for (int b_ = 0; b_ < 4; ++b_)
            if (4 * tg + b_ < cnt) sS[(4 * tg + b_) * MP + m] = sc[a_][b_] * a.scale;
        }
      }
    }
    __syncthreads();
    {
      int wide = 0;
      for (int m = tid; m < M; m += kThreads) {
        const float mu0 = sMu[m];
        float mu = mu0;
        for (int t = 0; t < cnt; ++t) mu = fmaxf(mu, sS[t * MP + m]);
        sA[m] = mu;
        wide |= (mu - fmaxf(mu0, sS[m]) > kSpread);
      }
      if (cnt > 1 && __syncthreads_or(wide)) { sub = 1; continue; }    // again from s0, one token at a time
    }
    // per token: max and sum over the latents (the scatter softmax); eight threads per token, latents
    // part, part + 8, ... each, combined by shuffles
    {
      const int t = tid >> 3, part = tid & 7;
      float mx = -INFINITY;
      if (t < cnt) for (int m = part; m < M; m += 8) mx = fmaxf(mx, sS[t * MP + m]);
#pragma unroll
      for (int o = 1; o < 8; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      float su = 0.f;
      if (t < cnt) for (int m = part; m < M; m += 8) su += __expf(sS[t * MP + m] - mx);
#pragma unroll
      for (int o = 1; o < 8; o <<= 1) su += __shfl_xor_sync(0xffffffffu, su, o);
      if (t < cnt && part == 0) { sCm[t] = mx; sCs[t] = su; }
    }
    __syncthreads();
    // per latent: new running max over the sub-chunk, E = e^{S - mu}, running l, weights
    for (int m = tid; m < M; m += kThreads) {
      const float mu0 = sMu[m], mu = sA[m];
      const float al = (mu0 == -INFINITY) ? 0.f : __expf(mu0 - mu);
      float l = al * sL[m];
      for (int t = 0; t < cnt; ++t) {
        const float s = sS[t * MP + m];
        const float e = __expf(s - mu);
        l += e;
        sE[t * MP + m] = e;
        sS[t * MP + m] = __expf(s - sCm[t]) / (sCs[t] * l);     // softmax_M(s_:t)_m / l_mt
      }
      sMu[m] = mu; sL[m] = l; sA[m] = al;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kMaxLat; ++j) if (j < nlat) acc[j] *= sA[g * nlat + j];
    // the recurrence over the sub-chunk's tokens
    for (int t = 0; t < cnt; ++t) {
      const float vd = sV[t * D + d];
      const float* er = sE + t * MP + g * nlat;
      const float* gr = sS + t * MP + g * nlat;
      float y = 0.f;
      if ((nlat & 3) == 0) {                       // this thread's latents are contiguous: 16-byte broadcast loads
        float y0 = 0.f, y1 = 0.f, y2 = 0.f, y3 = 0.f;   // four chains instead of one of length nlat
#pragma unroll
        for (int j4 = 0; j4 < kMaxLat / 4; ++j4) {
          if (4 * j4 < nlat) {
            const float4 e4 = *reinterpret_cast<const float4*>(er + 4 * j4);
            const float4 g4 = *reinterpret_cast<const float4*>(gr + 4 * j4);
            acc[4 * j4] = fmaf(e4.x, vd, acc[4 * j4]);         y0 = fmaf(g4.x, acc[4 * j4], y0);
            acc[4 * j4 + 1] = fmaf(e4.y, vd, acc[4 * j4 + 1]); y1 = fmaf(g4.y, acc[4 * j4 + 1], y1);
            acc[4 * j4 + 2] = fmaf(e4.z, vd, acc[4 * j4 + 2]); y2 = fmaf(g4.z, acc[4 * j4 + 2], y2);
            acc[4 * j4 + 3] = fmaf(e4.w, vd, acc[4 * j4 + 3]); y3 = fmaf(g4.w, acc[4 * j4 + 3], y3);
          }
        }
        y = (y0 + y1) + (y2 + y3);
      } else {
#pragma unroll
        for (int j = 0; j < kMaxLat; ++j) {
          if (j < nlat) {
            acc[j] = fmaf(er[j], vd, acc[j]);
            y = fmaf(gr[j], acc[j], y);
          }
        }
      }
      float* yb = sY + (t & 1) * kThreads;         // two buffers: one barrier per token
      yb[g * D + d] = y;
      __syncthreads();
      if (g == 0) {
        float ys = 0.f;
#pragma unroll
        for (int gg = 0; gg < G; ++gg) ys += yb[gg * D + d];
        yp[(long long)(s0 + t) * a.ys[2] + d] = from_f32<T>(ys);
      }
    }
    __syncthreads();
    s0 += cnt;
  }
  if (!a.prefix) {                                 // decode: the record moves on
    float* st = a.state + ((long long)b * a.H + h) * M * W;
#pragma unroll
    for (int j = 0; j < kMaxLat; ++j) if (j < nlat) st[(g * nlat + j) * W + d] = acc[j];
    for (int m = tid; m < M; m += kThreads) { st[m * W + D] = sMu[m]; st[m * W + D + 1] = sL[m]; }
  }
  if (!a.redo) break;
  __syncthreads();                                 // the next unit reuses the shared arrays
  }
}

size_t walk_smem(int M, int D) {
  return sizeof(float) * ((size_t)(M + kSub) * (D + 1) + kSub * D + 2 * (size_t)kSub * (M + 4) + 3 * M + 2 * kSub + 2 * kThreads);
}

template <typename T, int D>
int launch_walk(const CausalArgs& a, int n_cta_x, cudaStream_t st) {
  const size_t smem = walk_smem(a.M, D);
  if (smem > 227 * 1024) return refuse(FLARE_EUNSUPPORTED, "causal: M=%d D=%d needs %zu bytes of shared memory", a.M, D, smem);
  cudaError_t e = cudaFuncSetAttribute(k_causal_walk<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return refuse(FLARE_ECUDA, "causal: %s", cudaGetErrorString(e));
  const dim3 grid = a.redo ? dim3((unsigned)(a.n_units < 2 * 148 ? a.n_units : 2 * 148))
                           : dim3((unsigned)n_cta_x, (unsigned)(a.B * a.H));
  launch_dep(k_causal_walk<T, D>, grid, dim3(kThreads), smem, st, a);
  e = cudaPeekAtLastError();
  if (e != cudaSuccess) return refuse(FLARE_ECUDA, "causal: %s", cudaGetErrorString(e));
  return FLARE_OK;
}

template <typename T>
int dispatch_walk(const CausalArgs& a, int n_cta_x, cudaStream_t st) {
  switch (a.D) {
    case 16: return launch_walk<T, 16>(a, n_cta_x, st);
    case 32: return launch_walk<T, 32>(a, n_cta_x, st);
    case 64: return launch_walk<T, 64>(a, n_cta_x, st);
    case 128: return launch_walk<T, 128>(a, n_cta_x, st);
  }
  return refuse(FLARE_EUNSUPPORTED, "causal: head dim %d not in {16,32,64,128}", a.D);
}

int fill_args(const FlareProblem* p, CausalArgs* a) {
  if (!p) return refuse(FLARE_EINVAL, "causal: null problem");
  if (p->B < 1 || p->H < 1 || p->M < 1 || p->N < 1) return refuse(FLARE_EINVAL, "causal: bad sizes");
  if ((long long)p->B * p->H > 65535) return refuse(FLARE_EUNSUPPORTED, "causal: B*H > 65535");
  if (!(p->scale > 0.f)) return refuse(FLARE_EINVAL, "causal: scale must be > 0");
  const int D = p->D;
  if (D != 16 && D != 32 && D != 64 && D != 128) return refuse(FLARE_EUNSUPPORTED, "causal: head dim %d not in {16,32,64,128}", D);
  const int G = kThreads / D;
  if (p->M % G != 0 || p->M / G > kMaxLat)
    return refuse(FLARE_EUNSUPPORTED, "causal: M=%d must be a multiple of %d and at most %d for D=%d", p->M, G, G * kMaxLat, D);
  a->B = p->B; a->H = p->H; a->N = p->N; a->M = p->M; a->D = D; a->scale = p->scale;
  a->redo = nullptr; a->n_units = 0; a->pacc = nullptr; a->pml = nullptr;
  for (int i = 0; i < 3; ++i) { a->qs[i] = p->q_stride[i]; a->ks[i] = p->k_stride[i]; a->vs[i] = p->v_stride[i]; a->ys[i] = p->y_stride[i]; }
  return FLARE_OK;
}

int run_walk(const FlareProblem* p, const CausalArgs& a, int n_cta_x, cudaStream_t st) {
  switch (p->dtype) {
    case FLARE_F32: return dispatch_walk<float>(a, n_cta_x, st);
    case FLARE_F16: return dispatch_walk<__half>(a, n_cta_x, st);
    case FLARE_BF16: return dispatch_walk<__nv_bfloat16>(a, n_cta_x, st);
  }
  return refuse(FLARE_EINVAL, "causal: bad dtype %d", p->dtype);
}

}  // namespace

namespace flare {
// pass 2 for the backward (flare_causal_bwd.cu), which needs the same chunk-start records
int launch_causal_scan(float* rec, int n_chunks, long long rows, int D, const float* state_in, float* state_out,
                       cudaStream_t st) {
  launch_scan(false, rec, n_chunks, rows, D, state_in, state_out, nullptr, nullptr, st);
  const cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) return refuse(FLARE_ECUDA, "causal scan: %s", cudaGetErrorString(e));
  return FLARE_OK;
}
}  // namespace flare

extern "C" {

size_t flare_causal_workspace_bytes(const FlareProblem* p) {
  if (!p || p->N < 1) return 0;
  const size_t chunks = ((size_t)p->N + kChunk - 1) / kChunk;
  const size_t rows = (size_t)p->B * p->H * p->M;
  // records, redo flags, and the compact prefix of the tensor-core path (16-byte aligned pieces)
  return chunks * rows * (p->D + 2) * sizeof(float) + ((chunks * p->B * p->H * sizeof(int) + 15) & ~size_t(15)) +
         chunks * rows * (p->D * 2 + sizeof(float2)) + 256;
}

int flare_causal_prefill(const FlareProblem* p, const void* q, const void* k, const void* v, void* y,
                         const float* state_in, float* state_out, float* workspace, flare_stream_t stream) {
  CausalArgs a;
  int rc = fill_args(p, &a);
  if (rc != FLARE_OK) return rc;
  if (!q || !k || !v || !y || !workspace) return refuse(FLARE_EINVAL, "causal_prefill: null pointer");
  if (reinterpret_cast<uintptr_t>(workspace) % 16) return refuse(FLARE_EINVAL, "causal_prefill: workspace must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int chunks = (p->N + kChunk - 1) / kChunk;
  // pass 1: one record per 128-token chunk
  const bool on_tc = flare::causal_tc_walk_supported(p, q, k, v, y);
  const long long rows = (long long)p->B * p->H * p->M;
  // workspace: fp32 records | redo flags | pml | pacc   (every piece a multiple of 16 bytes; the tensor-core path
  // keeps its records and prefixes in the last two, the others in the first)
  char* wsb = reinterpret_cast<char*>(workspace) + (size_t)chunks * rows * (p->D + 2) * sizeof(float);
  int* redo = reinterpret_cast<int*>(wsb);
  wsb += ((size_t)chunks * p->B * p->H * sizeof(int) + 15) & ~size_t(15);
  float2* pml = reinterpret_cast<float2*>(wsb);
  wsb += (size_t)chunks * rows * sizeof(float2);
  __nv_bfloat16* pacc = reinterpret_cast<__nv_bfloat16*>(wsb);
  if (on_tc) {
    rc = flare::causal_tc_record(p, q, k, v, pacc, pml, chunks, st);
    if (rc != FLARE_OK) return refuse(rc, "causal_prefill: tensor-core record pass could not be launched");
  } else {
    FlareProblem pp = *p;
    pp.n_splits = chunks;
    rc = flare_gather_partial(&pp, q, k, v, nullptr, workspace, st);
    if (rc != FLARE_OK) return rc;
  }
  // pass 2: exclusive prefix along the chunk axis
  launch_scan(true, workspace, chunks, rows, p->D, state_in, state_out, on_tc ? pacc : nullptr, on_tc ? pml : nullptr, st);
  // pass 3: the tokens of every chunk
  a.q = q; a.k = k; a.v = v; a.y = y;
  a.prefix = workspace; a.state = nullptr; a.tokens_per_cta = kChunk;
  if (on_tc) {
    // the tensor-core walk flags the chunks whose scores span too many octaves for its fixed reference
    // maximum; the fp32 walk, launched behind it, redoes exactly those (every other CTA returns at once)
    rc = flare::causal_tc_walk(p, q, k, v, y, pacc, pml, redo, chunks, st);
    if (rc != FLARE_OK) return refuse(rc, "causal_prefill: tensor-core walk could not be launched");
    const cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) return refuse(FLARE_ECUDA, "causal_prefill: %s", cudaGetErrorString(e));
    a.redo = redo; a.n_units = chunks * p->B * p->H; a.pacc = pacc; a.pml = pml;
  }
  return run_walk(p, a, chunks, st);
}

int flare_causal_decode(const FlareProblem* p, const void* q, const void* k, const void* v, void* y,
                        float* state, flare_stream_t stream) {
  CausalArgs a;
  int rc = fill_args(p, &a);
  if (rc != FLARE_OK) return rc;
  if (!q || !k || !v || !y || !state) return refuse(FLARE_EINVAL, "causal_decode: null pointer");
  a.q = q; a.k = k; a.v = v; a.y = y;
  a.prefix = nullptr; a.state = state; a.tokens_per_cta = p->N;
  return run_walk(p, a, 1, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
