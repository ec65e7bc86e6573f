// Main backward pass on tcgen05 tensor cores: dK, dV per token and the dQ partial of one token
// range, from one sweep over K, V, dY, Y.
//
//   P_mn = exp(S_mn - L_m)    A_mn = exp(S_mn - C_n)                    (S = scale q k^T)
//   dS   = P (dZ V^T - Delta_m) + A (Z dY^T - delta_n)      delta_n = dY_n . Y_n,  Delta_m = dZ_m . Z_m
//   dV_n = sum_m P_mn dZ_m     dK_n = scale sum_m dS_mn q_m     dQ_m = scale sum_n dS_mn k_n
//
// One CTA (256 threads, one per SM: it uses all 512 tensor-memory columns) owns one (b, h) and
// one token range and walks it in 128-token tiles; the latents are taken in blocks of 128.
// Per (tile, latent block j), token-major (tensor-memory lane = token):
//   MMA  : S^T = K_t Q_j^T,  T1 = V_t dZ_j^T,  T2 = dY_t Z_j^T      -> columns [0,128) [128,256) [256,384)
//   SIMT : two exponentials per score; P and dS are packed to bf16 over S and T1 (each half of the
//          threads keeps to its own 64 columns); dS also goes to shared memory, token-major rows,
//          which is the MN-major A operand of the dQ product
//   MMA  : dV += P^T dZ_j,  dK += dS^T Q_j   (A from tensor memory)     -> columns [384,384+D) [416,416+D)
//          dQ_j += dS K_t                     (A and B from shared memory) -> columns [448+32j, +D)
// Q, Z, dZ stay resident in shared memory for the whole range, each tile in one layout that
// serves both as a K-major and as an MN-major operand.  K, V, dY, Y tiles arrive by TMA in a
// two-stage ring.
//
// This is the general tensor-core backward: bf16 or fp16, D in {16, 32}, a key-padding mask (excluded
// tokens get P = A = 0, hence zero dK, dV and no share in dQ), either softmax term alone (the separate
// gather / scatter operators), and more than 256 latents as blocks of 256 per launch, each block adding
// its dK/dV to what the earlier ones wrote.  The one-exponential kernels (flare_tc_bwd_range.cu,
// flare_tc_bwd_fast.cu) are the fast form of its unmasked two-term bf16 case.
#include "common.cuh"
#include "launch.h"
#include "tc_common.cuh"
#include "tma_host.h"

namespace flare {

using namespace tc;

struct BwdArgs {
  int B, H, N, M;
  float scale, scale_log2;
  int q_batched;
  int n_splits, chunk;
  const float* z32;
  const float* dz32;
  const float* lse_m;
  const float* lse_n;
  void* dk;                    // 16-bit rows
  void* dv;
  long long dks[3], dvs[3];
  float* dq_part;              // [S,B,H,M_total,D]
  int M_total, m0;             // this launch covers latents [m0, m0 + M) of M_total
  int terms;                   // FLARE_TERM_GATHER | FLARE_TERM_SCATTER
  const uint8_t* mask;         // [B,N] key-padding mask (non-zero = keep) or null
  DropArgs drop;               // attention dropout: P' = D1 P / (1-p) feeds dV, A' = D2 A / (1-p); dS uses the masks too
  int* status;
  const int* flag;             // [B*H] or null: run only the (b, h) whose flag is 1
};

template <int D>
struct BwdSmem {
  static constexpr int ROWB = 2 * D;
  static constexpr int kLat = 256 * ROWB;          // Q, Z or dZ: all latents
  static constexpr int kT = 128 * ROWB;            // one token tile
  static constexpr int kStage = 4 * kT;            // K, V, dY, Y
  static constexpr int kDS = 2 * 128 * 128;        // dS^T [2 blocks of 64 latents][128 tok][128 B]
  static constexpr int kBytes = 3 * kLat + 2 * kStage + kDS + 256 * 8 + 2 * 128 * 8 + 2 * 128 * 4 + 1024 + 128;
};

template <int D, typename T16, bool ACC>          // ACC: add to the dK/dV an earlier latent block wrote
__global__ void __launch_bounds__(256, 1)
k_tc_bwd(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
         const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmG,
         const __grid_constant__ CUtensorMap tmY, BwdArgs a) {
  grid_dep_sync();
  constexpr int ROWB = 2 * D;
  constexpr int CPR = ROWB / 16;
  using L = BwdSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sZ = sQ + L::kLat;
  uint8_t* sDZ = sZ + L::kLat;
  uint8_t* sTok = sDZ + L::kLat;                   // [2 stages][K | V | dY | Y]
  uint8_t* sDS = sTok + 2 * L::kStage;
  float2* sLD = reinterpret_cast<float2*>(sDS + L::kDS);     // [256] {L_m log2e, Delta_m}
  float2* sCD = sLD + 256;                                    // [2][128] {C_n log2e, delta_n}
  float* sBias = reinterpret_cast<float*>(sCD + 256);         // [2][128] 0, or -inf for an excluded token
  uint64_t* bars = reinterpret_cast<uint64_t*>(sBias + 256);
  uint64_t* bar_full = bars;                       // [2]
  uint64_t* bar_mma = bars + 2;
  uint64_t* bar_q = bars + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  int* abort_flag = reinterpret_cast<int*>(bars + 5);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wg = warp >> 2;                        // which 64 of the 128 columns this thread handles
  const int row = (warp & 3) * 32 + lane;          // token within the tile = tensor-memory lane
  const int split = blockIdx.x % a.n_splits;
  const int bh = blockIdx.x / a.n_splits;
  if (a.flag && a.flag[bh] != 1) return;           // the one-exponential kernel owns this (b, h)
  const int b = bh / a.H, h = bh % a.H;
  const int M = a.M;
  const bool use_g = (a.terms & FLARE_TERM_GATHER) != 0, use_s = (a.terms & FLARE_TERM_SCATTER) != 0;
  const int n_mblk = (M + 127) / 128;
  const int n0 = split * a.chunk, n1 = min(a.N, n0 + a.chunk);
  const int n_tiles = n1 > n0 ? (n1 - n0 + 127) / 128 : 0;
  float* dq_out = a.dq_part + ((((long long)split * a.B + b) * a.H + h) * a.M_total + a.m0) * D;

  if (n_tiles == 0) {                              // empty range contributes nothing
    for (int i = tid; i < M * D; i += 256) dq_out[i] = 0.f;
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
  constexpr uint32_t cS = 0, cT1 = 128, cT2 = 256, cDV = 384, cDK = 416, cDQ = 448;

  auto load_tile = [&](int stage, int tok0) {
    uint8_t* dst = sTok + stage * L::kStage;
    mbar_expect_tx(&bar_full[stage], (1 + (use_g ? 1 : 0) + (use_s ? 2 : 0)) * L::kT);
    tma_load_4d(dst, &tmK, &bar_full[stage], 0, tok0, h, b);
    if (use_g) tma_load_4d(dst + L::kT, &tmV, &bar_full[stage], 0, tok0, h, b);
    if (use_s) {
      tma_load_4d(dst + 2 * L::kT, &tmG, &bar_full[stage], 0, tok0, h, b);
      tma_load_4d(dst + 3 * L::kT, &tmY, &bar_full[stage], 0, tok0, h, b);
    }
  };

  if (tid == 0) {
    mbar_expect_tx(bar_q, L::kLat);
    tma_load_4d(sQ, &tmQ, bar_q, 0, 0, h, a.q_batched ? b : 0);       // rows past M arrive as zeros
    load_tile(0, n0);
  }
  // resident latent operands: Z and dZ as bf16 in the swizzled tile layout; L and Delta per latent
  {
    const long long lrow = ((long long)b * a.H + h) * a.M_total + a.m0;
    const float* zb = a.z32 + lrow * D;
    const float* dzb = use_g ? a.dz32 + lrow * D : nullptr;
    // CPR consecutive lanes share a latent row (eight values each): coalesced reads, and Delta_m = dZ_m . Z_m is
    // summed over them by shuffles (whole warps run every iteration)
    for (int i = tid; i < 256 * CPR; i += 256) {
      const int r = i / CPR, c = i % CPR;
      uint4 pz = make_uint4(0, 0, 0, 0), pd = make_uint4(0, 0, 0, 0);
      float dl = 0.f;
      if (r < M) {
        const float4 z0 = *reinterpret_cast<const float4*>(zb + r * D + c * 8);
        const float4 z1 = *reinterpret_cast<const float4*>(zb + r * D + c * 8 + 4);
        pz = make_uint4(Op16<T16>::pack(z0.x, z0.y), Op16<T16>::pack(z0.z, z0.w), Op16<T16>::pack(z1.x, z1.y),
                        Op16<T16>::pack(z1.z, z1.w));
        if (use_g) {
          const float4 d0 = *reinterpret_cast<const float4*>(dzb + r * D + c * 8);
          const float4 d1 = *reinterpret_cast<const float4*>(dzb + r * D + c * 8 + 4);
          pd = make_uint4(Op16<T16>::pack(d0.x, d0.y), Op16<T16>::pack(d0.z, d0.w), Op16<T16>::pack(d1.x, d1.y),
                          Op16<T16>::pack(d1.z, d1.w));
          // Delta_m from dZ as the tensor core sees it (rounded to the operand type): sum_n P_mn (V_n . dZ_m) then
          // cancels against it exactly instead of leaving a rounding residue of one sign along the row
          const float zf[8] = {z0.x, z0.y, z0.z, z0.w, z1.x, z1.y, z1.z, z1.w};
          const uint32_t dw[4] = {pd.x, pd.y, pd.z, pd.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 df = Op16<T16>::unpack(dw[j]);
            dl = fmaf(df.x, zf[2 * j], dl);
            dl = fmaf(df.y, zf[2 * j + 1], dl);
          }
        }
      }
#pragma unroll
      for (int o = 1; o < CPR; o <<= 1) dl += __shfl_xor_sync(0xffffffffu, dl, o);
      *reinterpret_cast<uint4*>(sZ + swz_off<ROWB>(r, c)) = pz;
      *reinterpret_cast<uint4*>(sDZ + swz_off<ROWB>(r, c)) = pd;
      if (c == 0)                                  // without the gather term P = 0 (L = +inf)
        sLD[r] = make_float2(r < M && use_g ? a.lse_m[lrow + r] * kLog2e : INFINITY, dl);
    }
  }
  fence_proxy_async();
  __syncthreads();
  mbar_wait(bar_q, 0, a.status, abort_flag);

  constexpr int F = Op16<T16>::kFmt;
  const uint32_t id_st = idesc_f16(128, 128, F, F, 0, 0);    // S^T, T1, T2: A, B K-major
  const uint32_t id_tv = idesc_f16(128, D, F, F, 0, 1);      // dV, dK: A in tensor memory, B MN-major
  const uint32_t id_dq = idesc_f16(128, D, F, F, 1, 1);      // dQ: A and B MN-major
  const float sl = a.scale_log2;
  const float* cb = use_s ? a.lse_n + ((long long)b * a.H + h) * a.N : nullptr;
  const uint8_t* mrow = a.mask ? a.mask + (long long)b * a.N : nullptr;
  uint32_t ph_mma = 0;
  bool aborted = false;

  for (int t = 0; t < n_tiles && !aborted; ++t) {
    const int st = t & 1;
    const int tok0 = n0 + t * 128;
    uint8_t* tK = sTok + st * L::kStage;
    uint8_t* tV = tK + L::kT;
    uint8_t* tG = tK + 2 * L::kT;
    uint8_t* tY = tK + 3 * L::kT;
    if (tid == 0 && t + 1 < n_tiles) load_tile(st ^ 1, tok0 + 128);   // every MMA of tile t-1 is complete
    mbar_wait(&bar_full[st], (uint32_t)(t >> 1) & 1, a.status, abort_flag);

    // per-token scalars: C_n (log2 units) and delta_n = dY_n . Y_n from the tiles just loaded; the score
    // bias that removes a token (past the end of the range, or masked out): P = A = 0 for it
    if (tid < 128) {
      const int n = tok0 + tid;
      float dl = 0.f, c2 = INFINITY;
      const bool keep = n < n1 && (!mrow || mrow[n] != 0);
      if (keep && use_s) {
#pragma unroll
        for (int c = 0; c < CPR; ++c) {
          const uint4 g4 = *reinterpret_cast<const uint4*>(tG + swz_off<ROWB>(tid, c));
          const uint4 y4 = *reinterpret_cast<const uint4*>(tY + swz_off<ROWB>(tid, c));
          const uint32_t* gp = reinterpret_cast<const uint32_t*>(&g4);
          const uint32_t* yp = reinterpret_cast<const uint32_t*>(&y4);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 gf = Op16<T16>::unpack(gp[j]), yf = Op16<T16>::unpack(yp[j]);
            dl = fmaf(gf.x, yf.x, dl); dl = fmaf(gf.y, yf.y, dl);
          }
        }
        c2 = cb[n] * kLog2e;
      }
      sCD[st * 128 + tid] = make_float2(c2, dl);
      sBias[st * 128 + tid] = keep ? 0.f : -INFINITY;
    }
    __syncthreads();
    const float2 cd = sCD[st * 128 + row];
    const float c2n = cd.x, deln = cd.y, bias = sBias[st * 128 + row];
    const uint32_t ntok = (uint32_t)(tok0 + row);
    const uint32_t drow_g = (uint32_t)(1 * a.B * a.H + bh) * (uint32_t)a.M_total;     // gather weights' rows
    const uint32_t drow_s = (uint32_t)(2 * a.B * a.H + bh) * (uint32_t)a.M_total;     // scatter weights' rows

    for (int j = 0; j < n_mblk; ++j) {
      if (tid == 0) {
        tc_fence_after();
        const uint64_t dK_ = smem_desc<ROWB>(smem_u32(tK)), dV_ = smem_desc<ROWB>(smem_u32(tV)),
                       dG_ = smem_desc<ROWB>(smem_u32(tG));
        const uint32_t lo = (uint32_t)(j * 128 * ROWB);
        const uint64_t dQ_ = smem_desc<ROWB>(smem_u32(sQ) + lo), dZ_ = smem_desc<ROWB>(smem_u32(sZ) + lo),
                       dDZ_ = smem_desc<ROWB>(smem_u32(sDZ) + lo);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) mma_ss(tmem + cS, dK_ + 2 * kk, dQ_ + 2 * kk, id_st, kk > 0);
        if (use_g) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) mma_ss(tmem + cT1, dV_ + 2 * kk, dDZ_ + 2 * kk, id_st, kk > 0);
        }
        if (use_s) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) mma_ss(tmem + cT2, dG_ + 2 * kk, dZ_ + 2 * kk, id_st, kk > 0);
        }
        mma_commit(bar_mma);
      }
      mbar_wait(bar_mma, ph_mma, a.status, abort_flag);
      ph_mma ^= 1;
      tc_fence_after();

      // ---- P, A, dS for this thread's token and its 64 latents of block j ---------------------
      const uint32_t colb = 64 * wg;
      const float2* ld = sLD + j * 128 + colb;
      uint8_t* ds_row = sDS + wg * (128 * 128);    // MN block wg: [128 tok][128 B]
#pragma unroll 1
      for (int i = 0; i < 4; ++i) {
        uint32_t rs[16], r1[16], r2[16], pp[8], pd[8];
        tmem_ld16(lane_base + cS + colb + 16 * i, rs);
        if (use_g) tmem_ld16(lane_base + cT1 + colb + 16 * i, r1);
        if (use_s) tmem_ld16(lane_base + cT2 + colb + 16 * i, r2);
        tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float4 l4 = *reinterpret_cast<const float4*>(&ld[16 * i + 2 * e]);   // {L2,Dl} x 2
          const float x0 = fmaf(__uint_as_float(rs[2 * e]), sl, bias), x1 = fmaf(__uint_as_float(rs[2 * e + 1]), sl, bias);
          float p0 = ex2(x0 - l4.x), p1 = ex2(x1 - l4.z);
          float t10 = __uint_as_float(r1[2 * e]), t11 = __uint_as_float(r1[2 * e + 1]);
          float t20 = __uint_as_float(r2[2 * e]), t21 = __uint_as_float(r2[2 * e + 1]);
          float pv0 = p0, pv1 = p1;                 // the weights dV sees
          if (a.drop.on) {
            // z = (D1 P / (1-p)) V and y = (D2 A / (1-p))^T z: the upstream factors dZ V^T and Z dY^T pass the
            // same masks before Delta_m = dZ_m . Z_m and delta_n = dY_n . Y_n are subtracted
            const uint32_t mcol = (uint32_t)(a.m0 + j * 128 + colb + 16 * i + 2 * e);
            const float k10 = drop_hash(ntok, drow_g + mcol, a.drop.seed_lo, a.drop.seed_hi) >= a.drop.thresh ? a.drop.inv_keep : 0.f;
            const float k11 = drop_hash(ntok, drow_g + mcol + 1, a.drop.seed_lo, a.drop.seed_hi) >= a.drop.thresh ? a.drop.inv_keep : 0.f;
            const float k20 = drop_hash(ntok, drow_s + mcol, a.drop.seed_lo, a.drop.seed_hi) >= a.drop.thresh ? a.drop.inv_keep : 0.f;
            const float k21 = drop_hash(ntok, drow_s + mcol + 1, a.drop.seed_lo, a.drop.seed_hi) >= a.drop.thresh ? a.drop.inv_keep : 0.f;
            pv0 *= k10; pv1 *= k11; t10 *= k10; t11 *= k11; t20 *= k20; t21 *= k21;
          }
          float s0 = 0.f, s1 = 0.f;
          if (use_s) {
            const float a0 = ex2(x0 - c2n), a1 = ex2(x1 - c2n);
            s0 = a0 * (t20 - deln);
            s1 = a1 * (t21 - deln);
          }
          if (use_g) {
            s0 = fmaf(p0, t10 - l4.y, s0);
            s1 = fmaf(p1, t11 - l4.w, s1);
          }
          pp[e] = Op16<T16>::pack(pv0, pv1);
          pd[e] = Op16<T16>::pack(s0, s1);
        }
        tmem_st8(lane_base + cS + colb + 8 * i, pp);
        tmem_st8(lane_base + cT1 + colb + 8 * i, pd);
        *reinterpret_cast<uint4*>(ds_row + swz_off<128>(row, 2 * i)) = make_uint4(pd[0], pd[1], pd[2], pd[3]);
        *reinterpret_cast<uint4*>(ds_row + swz_off<128>(row, 2 * i + 1)) = make_uint4(pd[4], pd[5], pd[6], pd[7]);
      }
      tmem_wait_st();
      fence_proxy_async();
      tc_fence_before();
      __syncthreads();
      aborted = *reinterpret_cast<volatile int*>(abort_flag) != 0;
      if (aborted) break;

      if (tid == 0) {
        tc_fence_after();
        const uint32_t lo = (uint32_t)(j * 128 * ROWB);
        const uint64_t bDZ = smem_desc<ROWB>(smem_u32(sDZ) + lo), bQ = smem_desc<ROWB>(smem_u32(sQ) + lo);
        const uint64_t bK = smem_desc<ROWB>(smem_u32(tK));
        const uint64_t aDS = smem_desc_mn128(smem_u32(sDS), 128 * 128, 1024);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {           // contraction over the 128 latents of block j
          const uint32_t acol = (kk < 4) ? 8 * kk : 64 + 8 * (kk - 4);
          const uint64_t boff = (uint64_t)((kk * 16 * ROWB) >> 4);
          if (use_g) mma_ts(tmem + cDV, tmem + cS + acol, bDZ + boff, id_tv, (j > 0) || (kk > 0));
          mma_ts(tmem + cDK, tmem + cT1 + acol, bQ + boff, id_tv, (j > 0) || (kk > 0));
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)             // contraction over the 128 tokens of the tile
          mma_ss(tmem + cDQ + 32 * j, aDS + (uint64_t)((kk * 2048) >> 4), bK + (uint64_t)((kk * 16 * ROWB) >> 4),
                 id_dq, (t > 0) || (kk > 0));
        mma_commit(bar_mma);
      }
      mbar_wait(bar_mma, ph_mma, a.status, abort_flag);
      ph_mma ^= 1;
      tc_fence_after();
    }
    if (aborted) break;

    // ---- dV (first half of the threads) and dK (second half) of this tile -> global -------------
    if (wg == 1 || use_g) {
      uint32_t r[D];
      const uint32_t col = wg ? cDK : cDV;
      if constexpr (D == 16) tmem_ld16(lane_base + col, r);
      else tmem_ld32(lane_base + col, r);
      tmem_wait_ld();
      const int n = tok0 + row;
      if (n < n1) {
        const float f = wg ? a.scale : 1.f;
        uint16_t* op = wg ? static_cast<uint16_t*>(a.dk) + b * a.dks[0] + h * a.dks[1] + (long long)n * a.dks[2]
                          : static_cast<uint16_t*>(a.dv) + b * a.dvs[0] + h * a.dvs[1] + (long long)n * a.dvs[2];
#pragma unroll
        for (int c = 0; c < D / 8; ++c) {
          float g[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) g[j] = __uint_as_float(r[8 * c + j]) * f;
          if constexpr (ACC) {
            const uint4 old = reinterpret_cast<const uint4*>(op)[c];
            const uint32_t* o2 = reinterpret_cast<const uint32_t*>(&old);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 of = Op16<T16>::unpack(o2[j]);
              g[2 * j] += of.x; g[2 * j + 1] += of.y;
            }
          }
          uint4 o;
          o.x = Op16<T16>::pack(g[0], g[1]); o.y = Op16<T16>::pack(g[2], g[3]);
          o.z = Op16<T16>::pack(g[4], g[5]); o.w = Op16<T16>::pack(g[6], g[7]);
          reinterpret_cast<uint4*>(op)[c] = o;
        }
      }
    }
    tc_fence_before();
    __syncthreads();
  }

  // ---- dQ partial of this range: latent block wg by thread group wg -----------------------------
  if (!aborted && wg < n_mblk) {
    uint32_t r[D];
    if constexpr (D == 16) tmem_ld16(lane_base + cDQ + 32 * wg, r);
    else tmem_ld32(lane_base + cDQ + 32 * wg, r);
    tmem_wait_ld();
    const int m = wg * 128 + row;
    if (m < M) {
      float* o = dq_out + (long long)m * D;
#pragma unroll
      for (int c = 0; c < D / 4; ++c)
        reinterpret_cast<float4*>(o)[c] = make_float4(__uint_as_float(r[4 * c]) * a.scale, __uint_as_float(r[4 * c + 1]) * a.scale,
                                                      __uint_as_float(r[4 * c + 2]) * a.scale, __uint_as_float(r[4 * c + 3]) * a.scale);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc<512>(tmem);
}

// ------------------------------------------------------------------------------------------
bool tc_bwd_supported(const Ctx& c, int dtype) {
  return (dtype == FLARE_BF16 || dtype == FLARE_F16) && (c.D == 16 || c.D == 32) && c.M >= 1 && c.M <= 1024 && c.N >= 1 &&
         c.terms >= 1 && c.terms <= 3;
}

template <int D, typename T16>
static int launch_bwd(const Ctx& c, const void* q, const void* k, const void* v, const void* dy, const void* y,
                      const uint8_t* mask, const float* z32, const float* dz32, const float* lse_m, const float* lse_n,
                      void* dk, void* dv, float* dq_part, const int* flag, cudaStream_t st) {
  CUtensorMap tmK, tmV, tmG, tmY;
  const uint64_t e = 2;
  constexpr int F = Op16<T16>::kFmt;
  const bool qb = c.qs[0] != 0;
  const bool use_g = (c.terms & FLARE_TERM_GATHER) != 0, use_s = (c.terms & FLARE_TERM_SCATTER) != 0;
  auto tokmap = [&](CUtensorMap* m, const void* p, const long long* s) {
    return make_tile_map(m, p, F, D, (uint64_t)c.N, (uint64_t)c.H, (uint64_t)c.B, s[2] * e, s[1] * e,
                         (c.B > 1 ? s[0] : s[1] * c.H) * e, 128);
  };
  // a term that is switched off never loads its tiles: its maps stand in with K's
  if (!tokmap(&tmK, k, c.ks) || !tokmap(&tmV, use_g ? v : k, use_g ? c.vs : c.ks) ||
      !tokmap(&tmG, use_s ? dy : k, use_s ? c.dys : c.ks) || !tokmap(&tmY, use_s ? y : k, use_s ? c.ys : c.ks))
    return FLARE_EUNSUPPORTED;
  BwdArgs a;
  a.B = c.B; a.H = c.H; a.N = c.N; a.M_total = c.M;
  a.scale = c.scale; a.scale_log2 = c.scale * kLog2e;
  a.q_batched = qb ? 1 : 0;
  a.n_splits = c.n_splits; a.chunk = c.chunk;
  a.z32 = z32; a.dz32 = dz32; a.lse_m = lse_m; a.lse_n = lse_n;
  a.dk = dk; a.dv = dv;
  for (int i = 0; i < 3; ++i) { a.dks[i] = c.dks[i]; a.dvs[i] = c.dvs[i]; }
  a.dq_part = dq_part;
  a.terms = c.terms;
  a.mask = mask;
  a.drop = make_drop(c.drop_p, c.drop_seed);
  a.status = tc_status_ptr();
  a.flag = flag;
  constexpr int smem = BwdSmem<D>::kBytes;
  if (tc_set_dyn_smem(reinterpret_cast<const void*>(&k_tc_bwd<D, T16, false>), smem) != FLARE_OK ||
      tc_set_dyn_smem(reinterpret_cast<const void*>(&k_tc_bwd<D, T16, true>), smem) != FLARE_OK)
    return FLARE_ECUDA;
  const long long grid = (long long)c.n_splits * c.B * c.H;
  if (grid > 0x7fffffffLL) return FLARE_EUNSUPPORTED;
  for (int m0 = 0; m0 < c.M; m0 += 256) {
    const int mb = c.M - m0 < 256 ? c.M - m0 : 256;
    CUtensorMap tmQ;
    const char* qblk = static_cast<const char*>(q) + (long long)m0 * c.qs[2] * e;
    if (!make_tile_map(&tmQ, qblk, F, D, (uint64_t)mb, (uint64_t)c.H, (uint64_t)(qb ? c.B : 1), c.qs[2] * e, c.qs[1] * e,
                       (qb ? c.qs[0] : c.qs[1] * c.H) * e, 256))
      return FLARE_EUNSUPPORTED;
    a.M = mb; a.m0 = m0;
    if (m0 == 0) launch_dep(k_tc_bwd<D, T16, false>, dim3((unsigned)grid), dim3(256), smem, st, tmQ, tmK, tmV, tmG, tmY, a);
    else launch_dep(k_tc_bwd<D, T16, true>, dim3((unsigned)grid), dim3(256), smem, st, tmQ, tmK, tmV, tmG, tmY, a);
  }
  return FLARE_OK;
}

int tc_bwd_main(const Ctx& c, int dtype, const void* q, const void* k, const void* v, const void* dy, const void* y,
                const uint8_t* mask, const float* z32, const float* dz32, const float* lse_m, const float* lse_n,
                void* dk, void* dv, float* dq_part, const int* flag, cudaStream_t st) {
  const bool bf = dtype == FLARE_BF16;
  switch (c.D) {
    case 16: return bf ? launch_bwd<16, __nv_bfloat16>(c, q, k, v, dy, y, mask, z32, dz32, lse_m, lse_n, dk, dv, dq_part, flag, st)
                       : launch_bwd<16, __half>(c, q, k, v, dy, y, mask, z32, dz32, lse_m, lse_n, dk, dv, dq_part, flag, st);
    case 32: return bf ? launch_bwd<32, __nv_bfloat16>(c, q, k, v, dy, y, mask, z32, dz32, lse_m, lse_n, dk, dv, dq_part, flag, st)
                       : launch_bwd<32, __half>(c, q, k, v, dy, y, mask, z32, dz32, lse_m, lse_n, dk, dv, dq_part, flag, st);
  }
  return FLARE_EUNSUPPORTED;
}

}  // namespace flare
