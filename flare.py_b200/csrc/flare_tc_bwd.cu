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
// two-stage ring.  Requires bf16, D in {16, 32}, M <= 256.
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
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  long long dks[3], dvs[3];
  float* dq_part;              // [S,B,H,M,D]
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
  static constexpr int kBytes = 3 * kLat + 2 * kStage + kDS + 256 * 8 + 2 * 128 * 8 + 1024 + 128;
};

template <int D>
__global__ void __launch_bounds__(256, 1)
k_tc_bwd(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
         const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmG,
         const __grid_constant__ CUtensorMap tmY, BwdArgs a) {
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
  uint64_t* bars = reinterpret_cast<uint64_t*>(sCD + 256);
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
  const int n_mblk = (M + 127) / 128;
  const int n0 = split * a.chunk, n1 = min(a.N, n0 + a.chunk);
  const int n_tiles = n1 > n0 ? (n1 - n0 + 127) / 128 : 0;
  float* dq_out = a.dq_part + (((long long)split * a.B + b) * a.H + h) * M * D;

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
    mbar_expect_tx(&bar_full[stage], 4 * L::kT);
    tma_load_4d(dst, &tmK, &bar_full[stage], 0, tok0, h, b);
    tma_load_4d(dst + L::kT, &tmV, &bar_full[stage], 0, tok0, h, b);
    tma_load_4d(dst + 2 * L::kT, &tmG, &bar_full[stage], 0, tok0, h, b);
    tma_load_4d(dst + 3 * L::kT, &tmY, &bar_full[stage], 0, tok0, h, b);
  };

  if (tid == 0) {
    mbar_expect_tx(bar_q, L::kLat);
    tma_load_4d(sQ, &tmQ, bar_q, 0, 0, h, a.q_batched ? b : 0);       // rows past M arrive as zeros
    load_tile(0, n0);
  }
  // resident latent operands: Z and dZ as bf16 in the swizzled tile layout; L and Delta per latent
  {
    const long long lrow = ((long long)b * a.H + h) * M;
    const float* zb = a.z32 + lrow * D;
    const float* dzb = a.dz32 + lrow * D;
    for (int i = tid; i < 256 * CPR; i += 256) {
      const int r = i / CPR, c = i % CPR;
      uint4 pz = make_uint4(0, 0, 0, 0), pd = make_uint4(0, 0, 0, 0);
      if (r < M) {
        const float4 z0 = *reinterpret_cast<const float4*>(zb + r * D + c * 8);
        const float4 z1 = *reinterpret_cast<const float4*>(zb + r * D + c * 8 + 4);
        const float4 d0 = *reinterpret_cast<const float4*>(dzb + r * D + c * 8);
        const float4 d1 = *reinterpret_cast<const float4*>(dzb + r * D + c * 8 + 4);
        pz = make_uint4(pack_bf16(z0.x, z0.y), pack_bf16(z0.z, z0.w), pack_bf16(z1.x, z1.y), pack_bf16(z1.z, z1.w));
        pd = make_uint4(pack_bf16(d0.x, d0.y), pack_bf16(d0.z, d0.w), pack_bf16(d1.x, d1.y), pack_bf16(d1.z, d1.w));
      }
      *reinterpret_cast<uint4*>(sZ + swz_off<ROWB>(r, c)) = pz;
      *reinterpret_cast<uint4*>(sDZ + swz_off<ROWB>(r, c)) = pd;
    }
    {
      const int m = tid;                           // 256 threads, 256 latent slots
      float l2 = INFINITY, dl = 0.f;
      if (m < M) {
        for (int i = 0; i < D; ++i) dl = fmaf(dzb[m * D + i], zb[m * D + i], dl);
        l2 = a.lse_m[lrow + m] * kLog2e;
      }
      sLD[m] = make_float2(l2, dl);
    }
  }
  fence_proxy_async();
  __syncthreads();
  mbar_wait(bar_q, 0, a.status, abort_flag);

  const uint32_t id_st = idesc_f16(128, 128, 1, 1, 0, 0);    // S^T, T1, T2: A, B K-major
  const uint32_t id_tv = idesc_f16(128, D, 1, 1, 0, 1);      // dV, dK: A in tensor memory, B MN-major
  const uint32_t id_dq = idesc_f16(128, D, 1, 1, 1, 1);      // dQ: A and B MN-major
  const float sl = a.scale_log2;
  const float* cb = a.lse_n + ((long long)b * a.H + h) * a.N;
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

    // per-token scalars: C_n (log2 units) and delta_n = dY_n . Y_n from the tiles just loaded
    if (tid < 128) {
      const int n = tok0 + tid;
      float dl = 0.f, c2 = INFINITY;
      if (n < n1) {
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
        c2 = cb[n] * kLog2e;
      }
      sCD[st * 128 + tid] = make_float2(c2, dl);
    }
    __syncthreads();
    const float2 cd = sCD[st * 128 + row];
    const float c2n = cd.x, deln = cd.y;

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
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) mma_ss(tmem + cT1, dV_ + 2 * kk, dDZ_ + 2 * kk, id_st, kk > 0);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) mma_ss(tmem + cT2, dG_ + 2 * kk, dZ_ + 2 * kk, id_st, kk > 0);
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
        tmem_ld16(lane_base + cT1 + colb + 16 * i, r1);
        tmem_ld16(lane_base + cT2 + colb + 16 * i, r2);
        tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float4 l4 = *reinterpret_cast<const float4*>(&ld[16 * i + 2 * e]);   // {L2,Dl} x 2
          const float x0 = __uint_as_float(rs[2 * e]) * sl, x1 = __uint_as_float(rs[2 * e + 1]) * sl;
          const float p0 = ex2(x0 - l4.x), p1 = ex2(x1 - l4.z);
          const float a0 = ex2(x0 - c2n), a1 = ex2(x1 - c2n);
          const float s0 = fmaf(p0, __uint_as_float(r1[2 * e]) - l4.y, a0 * (__uint_as_float(r2[2 * e]) - deln));
          const float s1 = fmaf(p1, __uint_as_float(r1[2 * e + 1]) - l4.w, a1 * (__uint_as_float(r2[2 * e + 1]) - deln));
          pp[e] = pack_bf16(p0, p1);
          pd[e] = pack_bf16(s0, s1);
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
          mma_ts(tmem + cDV, tmem + cS + acol, bDZ + boff, id_tv, (j > 0) || (kk > 0));
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
    {
      uint32_t r[D];
      const uint32_t col = wg ? cDK : cDV;
      if constexpr (D == 16) tmem_ld16(lane_base + col, r);
      else tmem_ld32(lane_base + col, r);
      tmem_wait_ld();
      const int n = tok0 + row;
      if (n < n1) {
        const float f = wg ? a.scale : 1.f;
        __nv_bfloat16* op = wg ? a.dk + b * a.dks[0] + h * a.dks[1] + (long long)n * a.dks[2]
                               : a.dv + b * a.dvs[0] + h * a.dvs[1] + (long long)n * a.dvs[2];
#pragma unroll
        for (int c = 0; c < D / 8; ++c) {
          uint4 o;
          o.x = pack_bf16(__uint_as_float(r[8 * c]) * f, __uint_as_float(r[8 * c + 1]) * f);
          o.y = pack_bf16(__uint_as_float(r[8 * c + 2]) * f, __uint_as_float(r[8 * c + 3]) * f);
          o.z = pack_bf16(__uint_as_float(r[8 * c + 4]) * f, __uint_as_float(r[8 * c + 5]) * f);
          o.w = pack_bf16(__uint_as_float(r[8 * c + 6]) * f, __uint_as_float(r[8 * c + 7]) * f);
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
  return dtype == FLARE_BF16 && (c.D == 16 || c.D == 32) && c.M >= 1 && c.M <= 256 && c.N >= 1 &&
         c.terms == FLARE_TERM_BOTH;
}

template <int D>
static int launch_bwd(const Ctx& c, const void* q, const void* k, const void* v, const void* dy, const void* y,
                      const float* z32, const float* dz32, const float* lse_m, const float* lse_n, void* dk,
                      void* dv, float* dq_part, const int* flag, cudaStream_t st) {
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
  BwdArgs a;
  a.B = c.B; a.H = c.H; a.N = c.N; a.M = c.M;
  a.scale = c.scale; a.scale_log2 = c.scale * kLog2e;
  a.q_batched = qb ? 1 : 0;
  a.n_splits = c.n_splits; a.chunk = c.chunk;
  a.z32 = z32; a.dz32 = dz32; a.lse_m = lse_m; a.lse_n = lse_n;
  a.dk = reinterpret_cast<__nv_bfloat16*>(dk); a.dv = reinterpret_cast<__nv_bfloat16*>(dv);
  for (int i = 0; i < 3; ++i) { a.dks[i] = c.dks[i]; a.dvs[i] = c.dvs[i]; }
  a.dq_part = dq_part;
  a.status = tc_status_ptr();
  a.flag = flag;
  static bool attr_done = false;
  constexpr int smem = BwdSmem<D>::kBytes;
  if (!attr_done) {
    if (cudaFuncSetAttribute(k_tc_bwd<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return FLARE_ECUDA;
    attr_done = true;
  }
  const long long grid = (long long)c.n_splits * c.B * c.H;
  if (grid > 0x7fffffffLL) return FLARE_EUNSUPPORTED;
  k_tc_bwd<D><<<(unsigned)grid, 256, smem, st>>>(tmQ, tmK, tmV, tmG, tmY, a);
  return FLARE_OK;
}

int tc_bwd_main(const Ctx& c, const void* q, const void* k, const void* v, const void* dy, const void* y,
                const float* z32, const float* dz32, const float* lse_m, const float* lse_n, void* dk, void* dv,
                float* dq_part, const int* flag, cudaStream_t st) {
  switch (c.D) {
    case 16: return launch_bwd<16>(c, q, k, v, dy, y, z32, dz32, lse_m, lse_n, dk, dv, dq_part, flag, st);
    case 32: return launch_bwd<32>(c, q, k, v, dy, y, z32, dz32, lse_m, lse_n, dk, dv, dq_part, flag, st);
  }
  return FLARE_EUNSUPPORTED;
}

}  // namespace flare
