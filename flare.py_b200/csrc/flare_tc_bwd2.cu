// Main backward pass, one exponential per score (the fast form of flare_tc_bwd.cu).
//
// With P_mn = exp(S_mn - L_m) and A_mn = exp(S_mn - C_n) = P_mn * exp(L_m - C_n):
//
//   dS_mn = P_mn * T'_nm,     T'_nm = (V_n . dZ_m - Delta_m) + eC_n eL_m (dY_n . Z_m - delta_n)
//   eL_m = exp(L_m - mu),  eC_n = exp(mu - C_n),  mu = mid-range of L for this (b, h)
//
// and T' is ONE tensor-core product over an extended contraction axis:
//   A' row n = [ V_n | eC_n dY_n | 1, 1, g_hi, g_hi, g_lo, 0.. ]        g = eC_n delta_n
//   B' row m = [ dZ_m | eL_m Z_m | -Delta_hi, -Delta_lo, -eL_hi, -eL_lo, -eL_hi, 0.. ]
// (the subtractive terms are carried as bf16 hi+lo pairs so that the cancellation in
// dP - Delta and dA - delta keeps fp32-like accuracy).  The softmax threads then need one ex2,
// one multiply and two packs per score.  dV = P^T dZ, dK = scale dS^T Q, dQ = scale dS K as in
// the exact kernel.
//
// The factorisation is only valid while exp(L_m - C_n) and its two factors stay inside fp32's
// exponent range.  k_bwd_range checks that per (b, h) on the device (ranges of L and C) and
// writes a flag; this kernel runs the (b, h) whose flag is 0, k_tc_bwd (two exponentials, no
// factorisation) runs the others.  No host synchronisation is involved.
//
// One CTA of 512 threads per SM: thread (row, g) owns token row `row` (tensor-memory lane) and the
// 32 latent columns [32g, 32g+32) of the current 128-latent block.  Tensor memory: S^T [0,128),
// T' [128,256), dV 256, dK 288, dQ_j 320+32j.  Requires bf16, D in {16,32}, M <= 256.
#include "common.cuh"
#include "launch.h"
#include "tc_common.cuh"
#include "tma_host.h"

namespace flare {

using namespace tc;

// ------------------------------------------------------------------------------------------
// range check: flag[bh] = 1 when the one-exponential form is not safe for this (b, h)
// ------------------------------------------------------------------------------------------
constexpr int kRangeParts = 64;

__global__ void __launch_bounds__(256)
k_bwd_range_c(const float* __restrict__ lse_n, int N, float* __restrict__ part /*[BH][parts][2]*/) {
  const int bh = blockIdx.y, p = blockIdx.x;
  const float* c = lse_n + (long long)bh * N;
  float mx = -INFINITY, mn = INFINITY;
  for (long long i = (long long)p * blockDim.x + threadIdx.x; i < N; i += (long long)gridDim.x * blockDim.x) {
    const float v = c[i];
    mx = fmaxf(mx, v); mn = fminf(mn, v);
  }
  __shared__ float smx[256], smn[256];
  smx[threadIdx.x] = mx; smn[threadIdx.x] = mn;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (threadIdx.x < s) {
      smx[threadIdx.x] = fmaxf(smx[threadIdx.x], smx[threadIdx.x + s]);
      smn[threadIdx.x] = fminf(smn[threadIdx.x], smn[threadIdx.x + s]);
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    part[((long long)bh * kRangeParts + p) * 2] = smx[0];
    part[((long long)bh * kRangeParts + p) * 2 + 1] = smn[0];
  }
}

__global__ void __launch_bounds__(256)
k_bwd_range_final(const float* __restrict__ lse_m, int M, const float* __restrict__ part,
                  float* __restrict__ mu_out, int* __restrict__ flag_out) {
  const int bh = blockIdx.x;
  float lmx = -INFINITY, lmn = INFINITY, cmx = -INFINITY, cmn = INFINITY;
  for (int i = threadIdx.x; i < M; i += blockDim.x) {
    const float v = lse_m[(long long)bh * M + i];
    lmx = fmaxf(lmx, v); lmn = fminf(lmn, v);
  }
  for (int i = threadIdx.x; i < kRangeParts; i += blockDim.x) {
    cmx = fmaxf(cmx, part[((long long)bh * kRangeParts + i) * 2]);
    cmn = fminf(cmn, part[((long long)bh * kRangeParts + i) * 2 + 1]);
  }
  __shared__ float s[4][256];
  s[0][threadIdx.x] = lmx; s[1][threadIdx.x] = lmn; s[2][threadIdx.x] = cmx; s[3][threadIdx.x] = cmn;
  __syncthreads();
  for (int st = 128; st > 0; st >>= 1) {
    if (threadIdx.x < st) {
      s[0][threadIdx.x] = fmaxf(s[0][threadIdx.x], s[0][threadIdx.x + st]);
      s[1][threadIdx.x] = fminf(s[1][threadIdx.x], s[1][threadIdx.x + st]);
      s[2][threadIdx.x] = fmaxf(s[2][threadIdx.x], s[2][threadIdx.x + st]);
      s[3][threadIdx.x] = fminf(s[3][threadIdx.x], s[3][threadIdx.x + st]);
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const float Lmx = s[0][0] * kLog2e, Lmn = s[1][0] * kLog2e, Cmx = s[2][0] * kLog2e, Cmn = s[3][0] * kLog2e;
    const float mu = 0.5f * (Lmx + Lmn);
    // every factor within 2^+-50 and exp(L - C) within 2^+-100; anything non-finite takes the exact kernel
    const bool ok = (Lmx - mu < 50.f) && (mu - Lmn < 50.f) && (Cmx - mu < 50.f) && (mu - Cmn < 50.f) &&
                    isfinite(Lmx) && isfinite(Lmn) && isfinite(Cmx) && isfinite(Cmn);
    mu_out[bh] = ok ? mu : 0.f;
    flag_out[bh] = ok ? 0 : 1;
  }
}

// ------------------------------------------------------------------------------------------
struct Bwd2Args {
  int B, H, N, M;
  float scale, scale_log2;
  int q_batched;
  int n_splits, chunk;
  const float* z32;
  const float* dz32;
  const float* lse_m;
  const float* lse_n;
  const float* mu;             // [B*H] log2 units
  const int* flag;             // [B*H] 0 = this kernel, 1 = the exact kernel
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  long long dks[3], dvs[3];
  float* dq_part;              // [S,B,H,M,D]
  int* status;
};

template <int D>
struct Bwd2Smem {
  static constexpr int ROWB = 2 * D;
  static constexpr int kLat = 256 * ROWB;          // Q, dZ or eL*Z: all latents
  static constexpr int kExtB = 256 * 32;           // extension columns of B'
  static constexpr int kT = 128 * ROWB;            // one token tile
  static constexpr int kStage = 4 * kT;            // K, V, dY, Y
  static constexpr int kExtA = 128 * 32;           // extension columns of A'
  static constexpr int kDS = 2 * 128 * 128;        // dS^T [2 blocks of 64 latents][128 tok][128 B]
  static constexpr int kBytes = 3 * kLat + kExtB + 2 * kStage + kT + kExtA + kDS + 256 * 4 + 2 * 128 * 8 + 1024 + 128;
};

__device__ __forceinline__ void split_bf16(float x, __nv_bfloat16& hi, __nv_bfloat16& lo) {
  hi = __float2bfloat16_rn(x);
  lo = __float2bfloat16_rn(x - __bfloat162float(hi));
}

template <int D>
__global__ void __launch_bounds__(512, 1)
k_tc_bwd2(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
          const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmG,
          const __grid_constant__ CUtensorMap tmY, Bwd2Args a) {
  constexpr int ROWB = 2 * D;
  constexpr int CPR = ROWB / 16;
  using L = Bwd2Smem<D>;
  const int split = blockIdx.x % a.n_splits;
  const int bh = blockIdx.x / a.n_splits;
  if (a.flag[bh] != 0) return;                     // the exact kernel owns this (b, h)

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sDZ = sQ + L::kLat;
  uint8_t* sZe = sDZ + L::kLat;                    // eL_m * Z_m
  uint8_t* sXB = sZe + L::kLat;                    // B' extension [256][16]
  uint8_t* sTok = sXB + L::kExtB;                  // [2 stages][K | V | dY | Y]
  uint8_t* sGe = sTok + 2 * L::kStage;             // eC_n * dY_n
  uint8_t* sXA = sGe + L::kT;                      // A' extension [128][16]
  uint8_t* sDS = sXA + L::kExtA;
  float* sL2 = reinterpret_cast<float*>(sDS + L::kDS);        // [256] L_m in log2 units (+inf past M)
  float2* sCD = reinterpret_cast<float2*>(sL2 + 256);         // [2][128] {eC_n, eC_n delta_n}
  uint64_t* bars = reinterpret_cast<uint64_t*>(sCD + 256);
  uint64_t* bar_full = bars;                       // [2]
  uint64_t* bar_mma = bars + 2;
  uint64_t* bar_q = bars + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  int* abort_flag = reinterpret_cast<int*>(bars + 5);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = warp >> 2;                         // column group 0..3 (32 latent columns each)
  const int row = (warp & 3) * 32 + lane;          // token within the tile = tensor-memory lane
  const int b = bh / a.H, h = bh % a.H;
  const int M = a.M;
  const int n_mblk = (M + 127) / 128;
  const int n0 = split * a.chunk, n1 = min(a.N, n0 + a.chunk);
  const int n_tiles = n1 > n0 ? (n1 - n0 + 127) / 128 : 0;
  float* dq_out = a.dq_part + (((long long)split * a.B + b) * a.H + h) * M * D;

  if (n_tiles == 0) {
    for (int i = tid; i < M * D; i += 512) dq_out[i] = 0.f;
    return;
  }

  if (tid == 0) {
    mbar_init(&bar_full[0], 1); mbar_init(&bar_full[1], 1);
    mbar_init(bar_mma, 1); mbar_init(bar_q, 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmG); prefetch_tmap(&tmY);
  }
  if (warp == 0) tmem_alloc<512>(tmem_slot);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
  constexpr uint32_t cS = 0, cT = 128, cDV = 256, cDK = 288, cDQ = 320, cP = 384, cDSp = 448;

  auto load_tile = [&](int stage, int tok0) {
    uint8_t* dst = sTok + stage * L::kStage;
    mbar_expect_tx(&bar_full[stage], 4 * L::kT);
    tma_load_4d(dst, &tmK, &bar_full[stage], 0, tok0, h, b);
    tma_load_4d(dst + L::kT, &tmV, &bar_full[stage], 0, tok0, h, b);
    tma_load_4d(dst + 2 * L::kT, &tmG, &bar_full[stage], 0, tok0, h, b);
    tma_load_4d(dst + 3 * L::kT, &tmY, &bar_full[stage], 0, tok0, h, b);
  };

  if (tid == 0) {
    mbar_expect_tx(bar_q, L::kLat);
    tma_load_4d(sQ, &tmQ, bar_q, 0, 0, h, a.q_batched ? b : 0);
    load_tile(0, n0);
  }
  const float mu = a.mu[bh];
  // resident latent operands of B': dZ, eL*Z and the extension columns
  {
    const long long lrow = ((long long)b * a.H + h) * M;
    const float* zb = a.z32 + lrow * D;
    const float* dzb = a.dz32 + lrow * D;
    for (int i = tid; i < 256 * CPR; i += 512) {
      const int r = i / CPR, c = i % CPR;
      uint4 pz = make_uint4(0, 0, 0, 0), pd = make_uint4(0, 0, 0, 0);
      if (r < M) {
        const float el = ex2(a.lse_m[lrow + r] * kLog2e - mu);
        const float4 z0 = *reinterpret_cast<const float4*>(zb + r * D + c * 8);
        const float4 z1 = *reinterpret_cast<const float4*>(zb + r * D + c * 8 + 4);
        const float4 d0 = *reinterpret_cast<const float4*>(dzb + r * D + c * 8);
        const float4 d1 = *reinterpret_cast<const float4*>(dzb + r * D + c * 8 + 4);
        pz = make_uint4(pack_bf16(z0.x * el, z0.y * el), pack_bf16(z0.z * el, z0.w * el),
                        pack_bf16(z1.x * el, z1.y * el), pack_bf16(z1.z * el, z1.w * el));
        pd = make_uint4(pack_bf16(d0.x, d0.y), pack_bf16(d0.z, d0.w), pack_bf16(d1.x, d1.y), pack_bf16(d1.z, d1.w));
      }
      *reinterpret_cast<uint4*>(sZe + swz_off<ROWB>(r, c)) = pz;
      *reinterpret_cast<uint4*>(sDZ + swz_off<ROWB>(r, c)) = pd;
    }
    if (tid < 256) {
      const int m = tid;
      float l2 = INFINITY, dl = 0.f, el = 0.f;
      if (m < M) {
        for (int i = 0; i < D; ++i) dl = fmaf(dzb[m * D + i], zb[m * D + i], dl);
        l2 = a.lse_m[lrow + m] * kLog2e;
        el = ex2(l2 - mu);
      }
      sL2[m] = l2;
      __nv_bfloat16 e[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) e[i] = __float2bfloat16_rn(0.f);
      __nv_bfloat16 dh, dlw, eh, elw;
      split_bf16(-dl, dh, dlw);
      split_bf16(-el, eh, elw);
      e[0] = dh; e[1] = dlw; e[2] = eh; e[3] = elw; e[4] = eh;
      const uint4* src = reinterpret_cast<const uint4*>(e);
      *reinterpret_cast<uint4*>(sXB + swz_off<32>(m, 0)) = src[0];
      *reinterpret_cast<uint4*>(sXB + swz_off<32>(m, 1)) = src[1];
    }
  }
  fence_proxy_async();
  __syncthreads();
  mbar_wait(bar_q, 0, a.status, abort_flag);

  const uint32_t id_st = idesc_f16(128, 128, 1, 1, 0, 0);    // S^T, T': A, B K-major
  const uint32_t id_tv = idesc_f16(128, D, 1, 1, 0, 1);      // dV, dK: A in tensor memory, B MN-major
  const uint32_t id_dq = idesc_f16(128, D, 1, 1, 1, 1);      // dQ: A and B MN-major
  const float sl = a.scale_log2;
  const float* cb = a.lse_n + ((long long)b * a.H + h) * a.N;
  uint32_t ph_mma = 0;
  bool aborted = false;

  // Per-token operands of tile `t` (must have landed in stage t&1): eC_n, g_n = eC_n delta_n, the A'
  // extension columns and the eC_n * dY_n tile.  Called by all threads; ends with the writes fenced
  // for the tensor core but NOT with a CTA barrier (the caller's next barrier covers it).
  auto prep_tile = [&](int t) {
    const int st = t & 1;
    const int tok0 = n0 + t * 128;
    const uint8_t* tG = sTok + st * L::kStage + 2 * L::kT;
    const uint8_t* tY = sTok + st * L::kStage + 3 * L::kT;
    if (tid < 128) {
      const int n = tok0 + tid;
      float dl = 0.f, ec = 0.f;
      if (n < n1) {
        const float c2 = cb[n] * kLog2e;
#pragma unroll
        for (int c = 0; c < CPR; ++c) {
          const uint4 g4 = *reinterpret_cast<const uint4*>(tG + swz_off<ROWB>(tid, c));
          const uint4 y4 = *reinterpret_cast<const uint4*>(tY + swz_off<ROWB>(tid, c));
          const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g4);
          const __nv_bfloat162* yp = reinterpret_cast<const __nv_bfloat162*>(&y4);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 gf = __bfloat1622float2(gp[j]), yf = __bfloat1622float2(yp[j]);
            dl = fmaf(gf.x, yf.x, dl); dl = fmaf(gf.y, yf.y, dl);
          }
        }
        ec = ex2(mu - c2);
      }
      const float gg = ec * dl;
      sCD[tid] = make_float2(ec, gg);
      __nv_bfloat16 e[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) e[i] = __float2bfloat16_rn(0.f);
      __nv_bfloat16 gh, gl;
      split_bf16(gg, gh, gl);
      const __nv_bfloat16 one = __float2bfloat16_rn(n < n1 ? 1.f : 0.f);
      e[0] = one; e[1] = one; e[2] = gh; e[3] = gh; e[4] = gl;
      const uint4* src = reinterpret_cast<const uint4*>(e);
      *reinterpret_cast<uint4*>(sXA + swz_off<32>(tid, 0)) = src[0];
      *reinterpret_cast<uint4*>(sXA + swz_off<32>(tid, 1)) = src[1];
    }
    __syncthreads();
    for (int i = tid; i < 128 * CPR; i += 512) {
      const int r = i / CPR, c = i % CPR;
      const float ec = sCD[r].x;
      const uint4 g4 = *reinterpret_cast<const uint4*>(tG + swz_off<ROWB>(r, c));
      const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g4);
      uint4 o;
      uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 gf = __bfloat1622float2(gp[j]);
        op[j] = pack_bf16(gf.x * ec, gf.y * ec);
      }
      *reinterpret_cast<uint4*>(sGe + swz_off<ROWB>(r, c)) = o;
    }
    fence_proxy_async();
  };

  // S^T and T' of (tile in stage st, latent block j)
  auto issue_p1 = [&](int st, int j) {
    const uint8_t* tK = sTok + st * L::kStage;
    const uint32_t lo = (uint32_t)(j * 128 * ROWB);
    const uint64_t aK = smem_desc<ROWB>(smem_u32(tK)), aV = smem_desc<ROWB>(smem_u32(tK + L::kT)),
                   aG = smem_desc<ROWB>(smem_u32(sGe)), aX = smem_desc<32>(smem_u32(sXA));
    const uint64_t bQ = smem_desc<ROWB>(smem_u32(sQ) + lo), bDZ = smem_desc<ROWB>(smem_u32(sDZ) + lo),
                   bZe = smem_desc<ROWB>(smem_u32(sZe) + lo), bX = smem_desc<32>(smem_u32(sXB) + j * 128 * 32);
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) mma_ss(tmem + cS, aK + 2 * kk, bQ + 2 * kk, id_st, kk > 0);
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) mma_ss(tmem + cT, aV + 2 * kk, bDZ + 2 * kk, id_st, kk > 0);
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) mma_ss(tmem + cT, aG + 2 * kk, bZe + 2 * kk, id_st, true);
    mma_ss(tmem + cT, aX, bX, id_st, true);
  };

  // dV += P^T dZ_j, dK += dS^T Q_j, dQ_j += dS K_t
  auto issue_p2 = [&](int st, int j, bool first_tile) {
    const uint8_t* tK = sTok + st * L::kStage;
    const uint32_t lo = (uint32_t)(j * 128 * ROWB);
    const uint64_t bDZ = smem_desc<ROWB>(smem_u32(sDZ) + lo), bQ = smem_desc<ROWB>(smem_u32(sQ) + lo);
    const uint64_t bK = smem_desc<ROWB>(smem_u32(tK));
    const uint64_t aDS = smem_desc_mn128(smem_u32(sDS), 128 * 128, 1024);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {             // three independent accumulation chains, interleaved
      const uint64_t boff = (uint64_t)((kk * 16 * ROWB) >> 4);
      mma_ts(tmem + cDV, tmem + cP + 8 * kk, bDZ + boff, id_tv, (j > 0) || (kk > 0));      // over latents
      mma_ts(tmem + cDK, tmem + cDSp + 8 * kk, bQ + boff, id_tv, (j > 0) || (kk > 0));     // over latents
      mma_ss(tmem + cDQ + 32 * j, aDS + (uint64_t)((kk * 2048) >> 4), bK + boff, id_dq,    // over tokens
             !first_tile || (kk > 0));
    }
  };

  // dV (groups 0,1) and dK (groups 2,3) of tile t -> global, 16 columns per thread
  auto store_tile = [&](int t) {
    constexpr int HALVES = D / 16;
    const int which = g >> 1, piece = g & 1;
    if (piece < HALVES) {
      uint32_t r[16];
      tmem_ld16(lane_base + (which ? cDK : cDV) + 16 * piece, r);
      tmem_wait_ld();
      const int n = n0 + t * 128 + row;
      if (n < n1) {
        const float f = which ? a.scale : 1.f;
        __nv_bfloat16* op = which ? a.dk + b * a.dks[0] + h * a.dks[1] + (long long)n * a.dks[2]
                                  : a.dv + b * a.dvs[0] + h * a.dvs[1] + (long long)n * a.dvs[2];
        op += 16 * piece;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint4 o;
          o.x = pack_bf16(__uint_as_float(r[8 * c]) * f, __uint_as_float(r[8 * c + 1]) * f);
          o.y = pack_bf16(__uint_as_float(r[8 * c + 2]) * f, __uint_as_float(r[8 * c + 3]) * f);
          o.z = pack_bf16(__uint_as_float(r[8 * c + 4]) * f, __uint_as_float(r[8 * c + 5]) * f);
          o.w = pack_bf16(__uint_as_float(r[8 * c + 6]) * f, __uint_as_float(r[8 * c + 7]) * f);
          reinterpret_cast<uint4*>(op)[c] = o;
        }
      }
    }
  };

  // ---- prologue: operands of tile 0, then its first S^T / T' ------------------------------------
  mbar_wait(&bar_full[0], 0, a.status, abort_flag);
  prep_tile(0);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {                                // whole warp converged, one elected lane issues
    tc_fence_after();
    if (elect_one()) {
      issue_p1(0, 0);
      mma_commit(bar_mma);
    }
    __syncwarp();
  }

  // One step = (tile t, latent block j).  The single commit of a step covers the dV/dK/dQ products of
  // that step and the S^T/T' products of the next one, so there is one wait per step and the packed
  // P and dS live in their own columns (never overwritten by an S^T/T' product that is in flight).
  for (int t = 0; t < n_tiles && !aborted; ++t) {
    const int st = t & 1;
    for (int j = 0; j < n_mblk; ++j) {
      mbar_wait(bar_mma, ph_mma, a.status, abort_flag);
      ph_mma ^= 1;
      tc_fence_after();
      if (j == 0) {
        // every product that read stage st^1 (tile t-1) is complete: refill it, and write out tile t-1
        if (tid == 0 && t + 1 < n_tiles) load_tile(st ^ 1, n0 + (t + 1) * 128);
        if (t > 0) store_tile(t - 1);
      }

      // ---- P and dS = P * T' for this thread's token and its 32 latents of block j -------------
      {
        const uint32_t colb = 32 * g;
        const float* l2p = sL2 + j * 128 + colb;
        uint8_t* ds_row = sDS + (g >> 1) * (128 * 128);        // MN block of 64 latents
        uint32_t rs[32], rt[32];
        tmem_ld32(lane_base + cS + colb, rs);
        tmem_ld32(lane_base + cT + colb, rt);
        tmem_wait_ld();
        uint32_t pp[16], pd[16];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float4 l4 = *reinterpret_cast<const float4*>(l2p + 4 * e);
          const float p0 = ex2(fmaf(__uint_as_float(rs[4 * e]), sl, -l4.x));
          const float p1 = ex2(fmaf(__uint_as_float(rs[4 * e + 1]), sl, -l4.y));
          const float p2 = ex2(fmaf(__uint_as_float(rs[4 * e + 2]), sl, -l4.z));
          const float p3 = ex2(fmaf(__uint_as_float(rs[4 * e + 3]), sl, -l4.w));
          pp[2 * e] = pack_bf16(p0, p1);
          pp[2 * e + 1] = pack_bf16(p2, p3);
          pd[2 * e] = pack_bf16(p0 * __uint_as_float(rt[4 * e]), p1 * __uint_as_float(rt[4 * e + 1]));
          pd[2 * e + 1] = pack_bf16(p2 * __uint_as_float(rt[4 * e + 2]), p3 * __uint_as_float(rt[4 * e + 3]));
        }
        tmem_st16(lane_base + cP + 16 * g, pp);
        tmem_st16(lane_base + cDSp + 16 * g, pd);
        const int cb0 = 4 * (g & 1);                           // first 16-byte chunk within the 128-byte row
#pragma unroll
        for (int c = 0; c < 4; ++c)
          *reinterpret_cast<uint4*>(ds_row + swz_off<128>(row, cb0 + c)) =
              make_uint4(pd[4 * c], pd[4 * c + 1], pd[4 * c + 2], pd[4 * c + 3]);
      }
      const bool last_blk = (j + 1 == n_mblk);
      const bool has_next_tile = (t + 1 < n_tiles);
      if (last_blk && has_next_tile) {            // operands of the next tile, while this step's stores drain
        mbar_wait(&bar_full[st ^ 1], (uint32_t)((t + 1) >> 1) & 1, a.status, abort_flag);
        prep_tile(t + 1);
      }
      tmem_wait_st();
      fence_proxy_async();
      tc_fence_before();
      __syncthreads();
      aborted = *reinterpret_cast<volatile int*>(abort_flag) != 0;
      if (aborted) break;

      if (warp == 0) {                            // whole warp converged, one elected lane issues
        tc_fence_after();
        if (elect_one()) {
          issue_p2(st, j, t == 0);
          if (!last_blk) issue_p1(st, j + 1);
          else if (has_next_tile) issue_p1(st ^ 1, 0);
          mma_commit(bar_mma);
        }
        __syncwarp();
      }
    }
  }

  if (!aborted) {
    mbar_wait(bar_mma, ph_mma, a.status, abort_flag);
    tc_fence_after();
    store_tile(n_tiles - 1);
    // ---- dQ partial of this range: block g/2, 16-column piece g%2 -------------------------------
    const int j = g >> 1, piece = g & 1;
    if (j < n_mblk && piece < D / 16) {
      uint32_t r[16];
      tmem_ld16(lane_base + cDQ + 32 * j + 16 * piece, r);
      tmem_wait_ld();
      const int m = j * 128 + row;
      if (m < M) {
        float* o = dq_out + (long long)m * D + 16 * piece;
#pragma unroll
        for (int c = 0; c < 4; ++c)
          reinterpret_cast<float4*>(o)[c] = make_float4(__uint_as_float(r[4 * c]) * a.scale, __uint_as_float(r[4 * c + 1]) * a.scale,
                                                        __uint_as_float(r[4 * c + 2]) * a.scale, __uint_as_float(r[4 * c + 3]) * a.scale);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc<512>(tmem);
}

// ------------------------------------------------------------------------------------------
size_t tc_bwd2_scratch_bytes(const Ctx& c) {
  const size_t bh = (size_t)c.B * c.H;
  return ((bh * kRangeParts * 2 * sizeof(float) + 255) & ~size_t(255)) + ((bh * sizeof(float) + 255) & ~size_t(255)) +
         ((bh * sizeof(int) + 255) & ~size_t(255));
}

template <int D>
static int launch_bwd2(const Ctx& c, const void* q, const void* k, const void* v, const void* dy, const void* y,
                       const float* z32, const float* dz32, const float* lse_m, const float* lse_n, void* dk,
                       void* dv, float* dq_part, const float* mu, const int* flag, cudaStream_t st) {
  CUtensorMap tmQ, tmK, tmV, tmG, tmY;
  const uint64_t e = 2;
  const bool qb = c.qs[0] != 0;
  auto tokmap = [&](CUtensorMap* m, const void* p, const long long* s) {
    return make_tile_map(m, p, 1, D, (uint64_t)c.N, (uint64_t)c.H, (uint64_t)c.B, s[2] * e, s[1] * e,
                         (c.B > 1 ? s[0] : s[1] * c.H) * e, 128);
  };
  if (!make_tile_map(&tmQ, q, 1, D, (uint64_t)c.M, (uint64_t)c.H, (uint64_t)(qb ? c.B : 1), c.qs[2] * e, c.qs[1] * e,
                     (qb ? c.qs[0] : c.qs[1] * c.H) * e, 256) ||
      !tokmap(&tmK, k, c.ks) || !tokmap(&tmV, v, c.vs) || !tokmap(&tmG, dy, c.dys) || !tokmap(&tmY, y, c.ys))
    return FLARE_EUNSUPPORTED;
  Bwd2Args a;
  a.B = c.B; a.H = c.H; a.N = c.N; a.M = c.M;
  a.scale = c.scale; a.scale_log2 = c.scale * kLog2e;
  a.q_batched = qb ? 1 : 0;
  a.n_splits = c.n_splits; a.chunk = c.chunk;
  a.z32 = z32; a.dz32 = dz32; a.lse_m = lse_m; a.lse_n = lse_n;
  a.mu = mu; a.flag = flag;
  a.dk = reinterpret_cast<__nv_bfloat16*>(dk); a.dv = reinterpret_cast<__nv_bfloat16*>(dv);
  for (int i = 0; i < 3; ++i) { a.dks[i] = c.dks[i]; a.dvs[i] = c.dvs[i]; }
  a.dq_part = dq_part;
  a.status = tc_status_ptr();
  constexpr int smem = Bwd2Smem<D>::kBytes;
  if (tc_set_dyn_smem(reinterpret_cast<const void*>(&k_tc_bwd2<D>), smem) != FLARE_OK) return FLARE_ECUDA;
  const long long grid = (long long)c.n_splits * c.B * c.H;
  if (grid > 0x7fffffffLL) return FLARE_EUNSUPPORTED;
  k_tc_bwd2<D><<<(unsigned)grid, 512, smem, st>>>(tmQ, tmK, tmV, tmG, tmY, a);
  return FLARE_OK;
}

// Range check, then the one-exponential kernel; the caller launches the exact kernel behind it
// with the same flags.  scratch: tc_bwd2_scratch_bytes(c) bytes, 256-byte aligned.
int tc_bwd2_main(const Ctx& c, const void* q, const void* k, const void* v, const void* dy, const void* y,
                 const float* z32, const float* dz32, const float* lse_m, const float* lse_n, void* dk, void* dv,
                 float* dq_part, void* scratch, const int** flag_out, cudaStream_t st) {
  const size_t bh = (size_t)c.B * c.H;
  char* w = static_cast<char*>(scratch);
  float* part = reinterpret_cast<float*>(w);  w += (bh * kRangeParts * 2 * sizeof(float) + 255) & ~size_t(255);
  float* mu = reinterpret_cast<float*>(w);    w += (bh * sizeof(float) + 255) & ~size_t(255);
  int* flag = reinterpret_cast<int*>(w);
  k_bwd_range_c<<<dim3(kRangeParts, (unsigned)bh), 256, 0, st>>>(lse_n, c.N, part);
  k_bwd_range_final<<<(unsigned)bh, 256, 0, st>>>(lse_m, c.M, part, mu, flag);
  *flag_out = flag;
  // D = 32: the pipelined kernel with two issuing warps (flare_tc_bwd4.cu); D = 16: the step-serial one here
  if (tc_bwd4_supported(c, FLARE_BF16))
    return tc_bwd4_launch(c, q, k, v, dy, y, z32, dz32, lse_m, lse_n, dk, dv, dq_part, mu, flag, st);
  switch (c.D) {
    case 16: return launch_bwd2<16>(c, q, k, v, dy, y, z32, dz32, lse_m, lse_n, dk, dv, dq_part, mu, flag, st);
    case 32: return launch_bwd2<32>(c, q, k, v, dy, y, z32, dz32, lse_m, lse_n, dk, dv, dq_part, mu, flag, st);
  }
  return FLARE_EUNSUPPORTED;
}

}  // namespace flare
