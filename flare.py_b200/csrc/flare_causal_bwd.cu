// Backward of causal FLARE:  y_t = sum_m A_mt z_tm,  z_tm = acc_m(t) / l_m(t)  (the prefix softmax state
// after token t),  A = softmax_M(S),  S = scale q k^T.   dq, dk, dv from dy.
//
// The reference ships no code for the causal path (see flare_causal.cu); the algorithm is the reverse
// chunk scan that oracle/flare_oracle.py:causal_bwd_chunked states and checks against autograd.  With
// g_t = dy_t,  G = A / l  and  c_mt = g_t . z_tm:
//
//   scatter softmax:  dS2_mt = A_mt (c_mt - delta_t),  delta_t = sum_m A_mt c_mt
//   prefix softmax :  token n feeds z_tm of every t >= n, so its gradients need the suffix sums
//                     R_m = sum_{t > chunk} G_mt g_t  (M x D)  and  r_m = -sum_{t > chunk} G_mt c_mt,
//                     carried from the later chunks relative to the running maximum mu of the chunk that
//                     produced them (every rescaling factor is then at most one)
//   inside a chunk (E = e^{S - mu}, l = a l0 + cumsum E, X_nt = v_n . g_t):
//     c_mt  = (a_m acc0_m . g_t + sum_{n <= t} E_mn X_nt) / l_mt
//     dv_n  = sum_m E_mn Rin_m + sum_{t >= n} (sum_m G_mt E_mn) g_t
//     de_mn = Rin_m . v_n + rin_m + sum_{t >= n} G_mt (X_nt - c_mt)
//     dS    = E de + dS2,   dq_m += scale sum_n dS_mn k_n,   dk_n = scale sum_m dS_mn q_m
//     Rout  = Rin + G g,    rout = rin - sum_t G_mt c_mt
//
// One CTA per (b, h) walks the 128-token chunks from the last to the first.  The state before each
// chunk comes from the forward's own first two passes (records per chunk, exclusive prefix); inside a
// chunk the states before its 32-token sub-chunks are rebuilt by a short forward sweep, then the
// sub-chunks are taken in reverse.  Everything is fp32 arithmetic on shared-memory tiles: a correct,
// deterministic kernel (no atomics), far from the tensor cores.
#include <cstdarg>
#include <cstdio>
#include <cuda_runtime.h>
#include "common.cuh"

namespace flare { void set_last_error(const char* msg); }

namespace {

using namespace flare;

constexpr int kThreads = 512;
constexpr int kSub = 32;          // tokens per sub-chunk
constexpr int kChunk = 128;       // tokens per prefix record (the forward's chunk)
constexpr int kTP = kSub + 1;     // padded row of a [M][tokens] tile
constexpr int kMaxDq = 16;        // dq values per thread: M * D <= 8192

int refuse(int code, const char* fmt, ...) {
  char msg[400];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(msg, sizeof(msg), fmt, ap);
  va_end(ap);
  flare::set_last_error(msg);
  return code;
}

struct CausalBwdArgs {
  int B, H, N, M, D;
  float scale;
  long long qs[3], ks[3], vs[3], gs[3], dks[3], dvs[3];
  const void* q; const void* k; const void* v; const void* dy;
  void* dk; void* dv;
  float* dq;                   // [B][H][M][D] fp32: this (b, h)'s latent gradient
  const float* prefix;         // [n_chunks][B][H][M][D+2]: the record before each chunk
  float* sub;                  // [B*H][3][M][D+2]: records before sub-chunks 1..3 of the current chunk
};

__device__ __forceinline__ float exp_or_zero(float from, float to) {   // e^{from - to}, 0 for an empty prefix
  return from == -INFINITY ? 0.f : expf(from - to);
}

// out(r, c) = sum_k A(r, k) B(k, c) for r < R, c < Cn: every thread a TR x TC register tile, so that one pair of
// shared-memory loads feeds TR * TC / (TR + TC) multiply-adds instead of half of one.  A thread's rows are
// rt, rt + nr, ... and its columns ct, ct + nc, ...: neighbouring threads read neighbouring columns of B.
template <int TR, int TC, typename FA, typename FB, typename FS>
__device__ __forceinline__ void tile_mm(int R, int Cn, int Kn, FA A, FB B, FS store) {
  const int nr = (R + TR - 1) / TR, nc = (Cn + TC - 1) / TC;
  for (int tile = threadIdx.x; tile < nr * nc; tile += kThreads) {
    const int rt = tile / nc, ct = tile % nc;
    int rr[TR], cc[TC];
#pragma unroll
    for (int i = 0; i < TR; ++i) rr[i] = min(rt + i * nr, R - 1);
#pragma unroll
    for (int j = 0; j < TC; ++j) cc[j] = min(ct + j * nc, Cn - 1);
    float acc[TR][TC];
#pragma unroll
    for (int i = 0; i < TR; ++i)
#pragma unroll
      for (int j = 0; j < TC; ++j) acc[i][j] = 0.f;
#pragma unroll 4
    for (int k = 0; k < Kn; ++k) {
      float av[TR], bv[TC];
#pragma unroll
      for (int i = 0; i < TR; ++i) av[i] = A(rr[i], k);
#pragma unroll
      for (int j = 0; j < TC; ++j) bv[j] = B(k, cc[j]);
#pragma unroll
      for (int i = 0; i < TR; ++i)
#pragma unroll
        for (int j = 0; j < TC; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
#pragma unroll
    for (int i = 0; i < TR; ++i)
#pragma unroll
      for (int j = 0; j < TC; ++j)
        if (rt + i * nr < R && ct + j * nc < Cn) store(rt + i * nr, ct + j * nc, acc[i][j]);
  }
}

template <typename T, int D>
__global__ void __launch_bounds__(kThreads)
k_causal_bwd(CausalBwdArgs a) {
  extern __shared__ __align__(16) float sm[];
  const int M = a.M;
  constexpr int DP = D + 1, W = D + 2;
  float* sQ = sm;                                  // [M][DP]
  float* sRh = sQ + M * DP;                        // [M][DP]  suffix sum R (carried), Rin while a sub-chunk is worked
  float* sK = sRh + M * DP;                        // [kSub][DP]
  float* sV = sK + kSub * DP;                      // [kSub][DP]
  float* sG = sV + kSub * DP;                      // [kSub][DP]  dy rows
  float* sE = sG + kSub * DP;                      // [M][kTP]  S, then E
  float* sGm = sE + M * kTP;                       // [M][kTP]  A, then G = A / l
  float* sLp = sGm + M * kTP;                      // [M][kTP]  l_mt
  float* sC = sLp + M * kTP;                       // [M][kTP]  c_mt
  float* sDe = sC + M * kTP;                       // [M][kTP]  de, then dS
  float* sX = sDe + M * kTP;                       // [kSub][kTP]  X_nt
  float* sW = sX + kSub * kTP;                     // [kSub][kTP]  W_tn = sum_m G_mt E_mn
  float* sMu = sW + kSub * kTP;                    // [M]
  float* sAa = sMu + M;                            // [M]  a_m
  float* sAl0 = sAa + M;                           // [M]  a_m l0_m
  float* sRin = sAl0 + M;                          // [M]  r (carried), rin while a sub-chunk is worked
  float* sNu = sRin + M;                           // [M]  mu of the sub-chunk that produced the carry
  float* sCmax = sNu + M;                          // [kSub]
  float* sCsum = sCmax + kSub;                     // [kSub]
  float* sDelta = sCsum + kSub;                    // [kSub]

  const int tid = threadIdx.x;
  const int bh = blockIdx.x, b = bh / a.H, h = bh % a.H;
  const T* qp = reinterpret_cast<const T*>(a.q) + b * a.qs[0] + h * a.qs[1];
  const T* kp = reinterpret_cast<const T*>(a.k) + b * a.ks[0] + h * a.ks[1];
  const T* vp = reinterpret_cast<const T*>(a.v) + b * a.vs[0] + h * a.vs[1];
  const T* gp = reinterpret_cast<const T*>(a.dy) + b * a.gs[0] + h * a.gs[1];
  T* dkp = reinterpret_cast<T*>(a.dk) + b * a.dks[0] + h * a.dks[1];
  T* dvp = reinterpret_cast<T*>(a.dv) + b * a.dvs[0] + h * a.dvs[1];
  float* subst = a.sub + (long long)bh * 3 * M * W;
  const int MD = M * D;

  for (int i = tid; i < MD; i += kThreads) {
    sQ[(i / D) * DP + i % D] = to_f32(qp[(long long)(i / D) * a.qs[2] + i % D]);
    sRh[(i / D) * DP + i % D] = 0.f;
  }
  for (int m = tid; m < M; m += kThreads) { sRin[m] = 0.f; sNu[m] = INFINITY; }
  float dqr[kMaxDq];
#pragma unroll
  for (int i = 0; i < kMaxDq; ++i) dqr[i] = 0.f;
  __syncthreads();

  // k, v (and dy) rows of `cnt` tokens from token s0 on; rows past cnt are zero
  auto load_tokens = [&](int s0, int cnt, bool with_g) {
    for (int i = tid; i < kSub * D; i += kThreads) {
      const int t = i / D, dd = i % D;
      const bool in = t < cnt;
      sK[t * DP + dd] = in ? to_f32(kp[(long long)(s0 + t) * a.ks[2] + dd]) : 0.f;
      sV[t * DP + dd] = in ? to_f32(vp[(long long)(s0 + t) * a.vs[2] + dd]) : 0.f;
      if (with_g) sG[t * DP + dd] = in ? to_f32(gp[(long long)(s0 + t) * a.gs[2] + dd]) : 0.f;
    }
  };
  // S_mt = scale q_m . k_t into sE; -inf for the tokens past cnt
  auto scores = [&](int cnt) {
    tile_mm<4, 4>(M, kSub, D, [&](int m, int dd) { return sQ[m * DP + dd]; }, [&](int dd, int t) { return sK[t * DP + dd]; },
                  [&](int m, int t, float s) { sE[m * kTP + t] = t < cnt ? s * a.scale : -INFINITY; });
  };

  const int chunks = (a.N + kChunk - 1) / kChunk;
  for (int c = chunks - 1; c >= 0; --c) {
    const int n0 = c * kChunk, n1 = min(a.N, n0 + kChunk);
    const int nsub = (n1 - n0 + kSub - 1) / kSub;
    const float* pre = a.prefix + (((long long)c * a.B + b) * a.H + h) * M * W;

    // ---- forward sweep: the records before sub-chunks 1 .. nsub-1 -----------------------------------
    for (int j = 0; j + 1 < nsub; ++j) {
      const float* st = j == 0 ? pre : subst + (long long)(j - 1) * M * W;
      float* out = subst + (long long)j * M * W;
      load_tokens(n0 + j * kSub, kSub, false);
      __syncthreads();
      scores(kSub);
      __syncthreads();
      for (int m = tid; m < M; m += kThreads) {
        const float m0 = st[m * W + D], l0 = st[m * W + D + 1];
        float mu = m0;
        _Pragma("unroll 8") for (int t = 0; t < kSub; ++t) mu = fmaxf(mu, sE[m * kTP + t]);
        const float wa = exp_or_zero(m0, mu);
        float l = wa * l0;
        _Pragma("unroll 8") for (int t = 0; t < kSub; ++t) {
          const float e = expf(sE[m * kTP + t] - mu);
          sE[m * kTP + t] = e;
          l += e;
        }
        sAa[m] = wa;
        out[m * W + D] = mu; out[m * W + D + 1] = l;
      }
      __syncthreads();
      tile_mm<4, 4>(M, D, kSub, [&](int m, int t) { return sE[m * kTP + t]; }, [&](int t, int dd) { return sV[t * DP + dd]; },
                    [&](int m, int dd, float x) { out[m * W + dd] = fmaf(sAa[m], st[m * W + dd], x); });
      __syncthreads();
    }

    // ---- the sub-chunks in reverse ---------------------------------------------------------------------
    for (int j = nsub - 1; j >= 0; --j) {
      const float* st = j == 0 ? pre : subst + (long long)(j - 1) * M * W;
      const int s0 = n0 + j * kSub;
      const int cnt = min(kSub, n1 - s0);
      load_tokens(s0, cnt, true);
      __syncthreads();
      scores(cnt);
      __syncthreads();
      // per token: max and sum over the latents (scatter softmax); per latent: mu, a, a l0
      for (int t = tid; t < kSub; t += kThreads) {
        float mx = -INFINITY;
        _Pragma("unroll 8") for (int m = 0; m < M; ++m) mx = fmaxf(mx, sE[m * kTP + t]);
        float su = 0.f;
        if (t < cnt) _Pragma("unroll 8") for (int m = 0; m < M; ++m) su += expf(sE[m * kTP + t] - mx);
        sCmax[t] = mx; sCsum[t] = su;
      }
      for (int m = kThreads - 1 - tid; m < M; m += kThreads) {       // (the other end of the block than the loop above)
        const float m0 = st[m * W + D], l0 = st[m * W + D + 1];
        float mu = m0;
        for (int t = 0; t < cnt; ++t) mu = fmaxf(mu, sE[m * kTP + t]);
        const float aa = exp_or_zero(m0, mu);
        sMu[m] = mu; sAa[m] = aa; sAl0[m] = aa * l0;
      }
      __syncthreads();
      // A (into sGm), E (in place of S)
      for (int i = tid; i < M * kSub; i += kThreads) {
        const int m = i / kSub, t = i % kSub;
        const float s = sE[m * kTP + t];
        const bool in = t < cnt;
        sGm[m * kTP + t] = in ? expf(s - sCmax[t]) / sCsum[t] : 0.f;
        sE[m * kTP + t] = in ? expf(s - sMu[m]) : 0.f;
      }
      __syncthreads();
      // l_mt = a l0 + cumsum E; G = A / l.  X_nt = v_n . g_t.  Rin = w R, rin = w r with w = e^{mu - nu}.
      for (int m = tid; m < M; m += kThreads) {
        float l = sAl0[m];
        _Pragma("unroll 8") for (int t = 0; t < kSub; ++t) {
          l += sE[m * kTP + t];
          sLp[m * kTP + t] = l;
          sGm[m * kTP + t] = l > 0.f ? sGm[m * kTP + t] / l : 0.f;
        }
        const float w = sNu[m] == INFINITY ? 0.f : expf(sMu[m] - sNu[m]);
        sRin[m] *= w;
        sNu[m] = w;                                // kept until the rows of R are rescaled below
      }
      tile_mm<2, 2>(kSub, kSub, D, [&](int n, int dd) { return sV[n * DP + dd]; }, [&](int dd, int t) { return sG[t * DP + dd]; },
                    [&](int n, int t, float x) { sX[n * kTP + t] = x; });
      __syncthreads();
      for (int i = tid; i < MD; i += kThreads) sRh[(i / D) * DP + i % D] *= sNu[i / D];
      // c_mt
      // (one product over the concatenated axis [d | n]: a_m acc0_m against g_t, then E_mn against X_nt for n <= t)
      tile_mm<4, 4>(M, kSub, D + kSub,
                    [&](int m, int kk) { return kk < D ? sAa[m] * st[m * W + kk] : sE[m * kTP + kk - D]; },
                    [&](int kk, int t) { return kk < D ? sG[t * DP + kk] : (kk - D <= t ? sX[(kk - D) * kTP + t] : 0.f); },
                    [&](int m, int t, float x) {
                      const float l = sLp[m * kTP + t];
                      sC[m * kTP + t] = l > 0.f ? x / l : 0.f;
                    });
      __syncthreads();
      for (int m = tid; m < M; m += kThreads) sNu[m] = sMu[m];       // the carry leaves this sub-chunk relative to its mu
      // delta_t = sum_m A_mt c_mt (A = G l);  W_tn = sum_m G_mt E_mn
      for (int t = tid; t < kSub; t += kThreads) {
        float dl = 0.f;
        _Pragma("unroll 8") for (int m = 0; m < M; ++m) dl = fmaf(sGm[m * kTP + t] * sLp[m * kTP + t], sC[m * kTP + t], dl);
        sDelta[t] = dl;
      }
      tile_mm<2, 2>(kSub, kSub, M, [&](int t, int m) { return sGm[m * kTP + t]; }, [&](int m, int n) { return sE[m * kTP + n]; },
                    [&](int t, int n, float w) { sW[t * kTP + n] = w; });
      __syncthreads();
      // dv_n = sum_m E_mn Rin_m + sum_{t >= n} W_tn g_t
      tile_mm<2, 4>(cnt, D, M + cnt,
                    [&](int n, int kk) { return kk < M ? sE[kk * kTP + n] : (kk - M >= n ? sW[(kk - M) * kTP + n] : 0.f); },
                    [&](int kk, int dd) { return kk < M ? sRh[kk * DP + dd] : sG[(kk - M) * DP + dd]; },
                    [&](int n, int dd, float x) { dvp[(long long)(s0 + n) * a.dvs[2] + dd] = from_f32<T>(x); });
      // de_mn = Rin_m . v_n + rin_m + sum_{t >= n} G_mt (X_nt - c_mt);  dS = E de + A (c - delta)
      // (the c part of the sum is a reverse running sum along the row: rin_m - sum_{t >= n} G_mt c_mt into sDe first)
      for (int m = tid; m < M; m += kThreads) {
        float run = sRin[m];
#pragma unroll 8
        for (int n = kSub - 1; n >= 0; --n) {
          run -= sGm[m * kTP + n] * sC[m * kTP + n];
          sDe[m * kTP + n] = run;
        }
      }
      __syncthreads();
      tile_mm<4, 4>(M, kSub, D + kSub,
                    [&](int m, int kk) { return kk < D ? sRh[m * DP + kk] : sGm[m * kTP + kk - D]; },
                    [&](int kk, int n) { return kk < D ? sV[n * DP + kk] : (kk - D >= n ? sX[n * kTP + kk - D] : 0.f); },
                    [&](int m, int n, float x) {
                      const float de = x + sDe[m * kTP + n];
                      const float A = sGm[m * kTP + n] * sLp[m * kTP + n];
                      sDe[m * kTP + n] = n < cnt ? sE[m * kTP + n] * de + A * (sC[m * kTP + n] - sDelta[n]) : 0.f;
                    });
      __syncthreads();
      // dq_m += scale sum_n dS_mn k_n (registers);  dk_n = scale sum_m dS_mn q_m;
      // Rout = Rin + G g,  rout = rin - sum_t G_mt c_mt
      {
        // this thread's 4 x 4 tile of dq stays in registers over the whole sequence (M * D / 16 <= 512 tiles)
        const int nr = (M + 3) / 4, nc = D / 4;
        if (tid < nr * nc) {
          const int rt = tid / nc, ct = tid % nc;
#pragma unroll 4
          for (int n = 0; n < cnt; ++n) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = sDe[min(rt + i * nr, M - 1) * kTP + n];
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) bv[jj] = sK[n * DP + ct + jj * nc];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
              for (int jj = 0; jj < 4; ++jj) dqr[4 * i + jj] = fmaf(av[i], bv[jj], dqr[4 * i + jj]);
          }
        }
      }
      tile_mm<4, 4>(M, D, cnt, [&](int m, int t) { return sGm[m * kTP + t]; }, [&](int t, int dd) { return sG[t * DP + dd]; },
                    [&](int m, int dd, float x) { sRh[m * DP + dd] += x; });   // (one thread per element; its readers are done)
      tile_mm<2, 4>(cnt, D, M, [&](int n, int m) { return sDe[m * kTP + n]; }, [&](int m, int dd) { return sQ[m * DP + dd]; },
                    [&](int n, int dd, float x) { dkp[(long long)(s0 + n) * a.dks[2] + dd] = from_f32<T>(x * a.scale); });
      for (int m = tid; m < M; m += kThreads) {
        float r = sRin[m];
        for (int t = 0; t < cnt; ++t) r -= sGm[m * kTP + t] * sC[m * kTP + t];
        sRin[m] = r;
      }
      __syncthreads();
    }
  }
  float* dq = a.dq + (long long)bh * MD;
  {
    const int nr = (M + 3) / 4, nc = D / 4;
    if (tid < nr * nc) {
      const int rt = tid / nc, ct = tid % nc;
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int jj = 0; jj < 4; ++jj)
          if (rt + i * nr < M) dq[(rt + i * nr) * D + ct + jj * nc] = dqr[4 * i + jj] * a.scale;
    }
  }
}

size_t bwd_smem(int M, int D) {
  return sizeof(float) * ((size_t)(2 * M + 3 * kSub) * (D + 1) + (size_t)(5 * M + 2 * kSub) * kTP + 5 * (size_t)M + 3 * kSub);
}

template <typename T, int D>
int launch_d(const CausalBwdArgs& a, cudaStream_t st) {
  const size_t smem = bwd_smem(a.M, D);
  cudaError_t e = cudaFuncSetAttribute(k_causal_bwd<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return refuse(FLARE_ECUDA, "causal_bwd: %s", cudaGetErrorString(e));
  k_causal_bwd<T, D><<<(unsigned)(a.B * a.H), kThreads, smem, st>>>(a);
  e = cudaPeekAtLastError();
  if (e != cudaSuccess) return refuse(FLARE_ECUDA, "causal_bwd: %s", cudaGetErrorString(e));
  return FLARE_OK;
}

template <typename T>
int launch(const CausalBwdArgs& a, cudaStream_t st) {
  switch (a.D) {
    case 16: return launch_d<T, 16>(a, st);
    case 32: return launch_d<T, 32>(a, st);
    case 64: return launch_d<T, 64>(a, st);
  }
  return refuse(FLARE_EUNSUPPORTED, "causal_bwd: head dim %d not in {16,32,64}", a.D);
}

}  // namespace

// pass 2 of the forward (flare_causal.cu): exclusive prefix of the chunk records, in place
namespace flare {
int launch_causal_scan(float* rec, int n_chunks, long long rows, int D, const float* state_in, float* state_out,
                       cudaStream_t st);
}

extern "C" {

size_t flare_causal_bwd_workspace_bytes(const FlareProblem* p) {
  if (!p || p->N < 1) return 0;
  const size_t chunks = ((size_t)p->N + kChunk - 1) / kChunk;
  const size_t rec = (size_t)p->B * p->H * p->M * (p->D + 2) * sizeof(float);
  return chunks * rec + 3 * rec + 512;
}

int flare_causal_bwd(const FlareProblem* p, const void* q, const void* k, const void* v, const void* dy,
                     float* dq32, void* dk, void* dv, float* workspace, flare_stream_t stream) {
  if (!p) return refuse(FLARE_EINVAL, "causal_bwd: null problem");
  if (!q || !k || !v || !dy || !dq32 || !dk || !dv || !workspace) return refuse(FLARE_EINVAL, "causal_bwd: null pointer");
  if (p->B < 1 || p->H < 1 || p->M < 1 || p->N < 1) return refuse(FLARE_EINVAL, "causal_bwd: bad sizes");
  if (!(p->scale > 0.f)) return refuse(FLARE_EINVAL, "causal_bwd: scale must be > 0");
  const int D = p->D, M = p->M;
  if (D != 16 && D != 32 && D != 64) return refuse(FLARE_EUNSUPPORTED, "causal_bwd: head dim %d not in {16,32,64}", D);
  if ((long long)M * D > (long long)kMaxDq * kThreads)
    return refuse(FLARE_EUNSUPPORTED, "causal_bwd: M*D = %lld exceeds %d", (long long)M * D, kMaxDq * kThreads);
  if (bwd_smem(M, D) > 227 * 1024)
    return refuse(FLARE_EUNSUPPORTED, "causal_bwd: M=%d D=%d needs %zu bytes of shared memory", M, D, bwd_smem(M, D));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int chunks = (p->N + kChunk - 1) / kChunk;
  const long long rows = (long long)p->B * p->H * M;
  // the forward's first two passes again: one record per 128-token chunk, then their exclusive prefix
  FlareProblem pp = *p;
  pp.n_splits = chunks;
  int rc = flare_gather_partial(&pp, q, k, v, nullptr, workspace, st);
  if (rc != FLARE_OK) return rc;
  rc = launch_causal_scan(workspace, chunks, rows, D, nullptr, nullptr, st);
  if (rc != FLARE_OK) return rc;
  CausalBwdArgs a;
  a.B = p->B; a.H = p->H; a.N = p->N; a.M = M; a.D = D; a.scale = p->scale;
  for (int i = 0; i < 3; ++i) {
    a.qs[i] = p->q_stride[i]; a.ks[i] = p->k_stride[i]; a.vs[i] = p->v_stride[i];
    a.gs[i] = p->dy_stride[i]; a.dks[i] = p->dk_stride[i]; a.dvs[i] = p->dv_stride[i];
  }
  a.q = q; a.k = k; a.v = v; a.dy = dy; a.dk = dk; a.dv = dv; a.dq = dq32;
  a.prefix = workspace;
  a.sub = workspace + (size_t)chunks * rows * (D + 2);
  switch (p->dtype) {
    case FLARE_F32: return launch<float>(a, st);
    case FLARE_F16: return launch<__half>(a, st);
    case FLARE_BF16: return launch<__nv_bfloat16>(a, st);
  }
  return refuse(FLARE_EINVAL, "causal_bwd: bad dtype %d", p->dtype);
}

}  // extern "C"
