// Main backward pass, one exponential per score, 128-latent steps.
//
// dS = P * T' with T' from one extended-contraction product (the mathematics and the on-device range
// check that chooses the (b, h) this kernel may run are described in flare_tc_bwd_range.cu).  A step
// u = (token tile t, 128-latent block s); the score buffers are laid out so that the two halves of a
// step's arithmetic need different products:
//
//   tensor memory (512 columns): S^T double-buffered [0,128) [128,256); T' single [256,384);
//   dV 384, dK 416, dQ_0 448, dQ_1 480.  Thread (token row, c) owns columns [32c, 32c+32) of a step:
//   it packs P into the first 16 of its own S^T columns and dS into the last 16.
//
//   phase A (needs S^T(u) only):  P = ex2(.), packed in place                  <- overlaps the T'(u) product
//   phase B (needs T'(u))      :  dS = P * T', packed in place and to shared memory (for dQ)
//
//   two issuing warps, so that neither stream of products waits behind the other's instructions (a
//   lone warp that shares its scheduler with busy softmax warps issues a product every ~45 clocks):
//     warp 18: T'(u+1) as soon as the threads hold T'(u) in registers; the TMA loads
//     warp 19: once P/dS of step u are written: dV/dK(u), then S^T(u+2) into the buffer those just read
//              (products issued by one thread execute in issue order: no completion round trip between
//              them), then dQ(u)
//   helper warps 16, 17: per-token operands of the next tile (eC*dY, the A' extension with delta_n),
//   two token rows per thread.  dV/dK of finished tiles -> global: one lane quarter per warp 16-19.
// Token tiles (K, V, dY) arrive by TMA in a three-stage ring; Y is read from global memory a tile
// ahead.  Requires bf16, D = 32, 32 <= M <= 256.
#include "common.cuh"
#include "launch.h"
#include "tc_common.cuh"
#include "tma_host.h"

namespace flare {

using namespace tc;

struct BwdFastArgs {
  int B, H, N, M;
  float scale, scale_log2;
  int q_batched;
  int n_splits, chunk;
  const float* z32;
  const float* dz32;
  const float* lse_m;
  const float* lse_n;
  const float* mu;             // [B*H] log2 units (range check)
  const int* flag;             // [B*H] 0 = one-exponential kernels, 1 = exact kernel
  const __nv_bfloat16* y;
  long long ys[3];
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  long long dks[3], dvs[3];
  float* dq_part;              // [S,B,H,M_total,D]
  int M_total, m0;             // this launch covers latents [m0, m0 + M) of M_total
  int* status;
};

struct BwdFastSmem {
  static constexpr int D = 32, ROWB = 64;
  static constexpr int kLat = 256 * ROWB;          // Q, dZ or eL*Z: all latents
  static constexpr int kExtB = 256 * 32;           // extension columns of B'
  static constexpr int kT = 128 * ROWB;            // one token tile
  static constexpr int kStage = 3 * kT;            // K, V, dY
  static constexpr int kExtA = 128 * 32;           // extension columns of A'
  static constexpr int kDS = 2 * 128 * 128;        // dS^T of one 128-latent block
  static constexpr int kBytes = 3 * kLat + kExtB + 3 * kStage + 2 * kT + 2 * kExtA + 2 * kDS + 256 * 4 + 1024 + 256;
};

__device__ __forceinline__ void split_bf16_4(float x, __nv_bfloat16& hi, __nv_bfloat16& lo) {
  hi = __float2bfloat16_rn(x);
  lo = __float2bfloat16_rn(x - __bfloat162float(hi));
}
__device__ __forceinline__ void mbar_arrive4(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

constexpr int kBFSoftmax = 512, kBFHelpers = 96;   // + the issuer warp

template <bool ACC>                               // ACC: add to the dK/dV an earlier latent block wrote
__global__ void __launch_bounds__(kBFSoftmax + kBFHelpers + 32, 1)
k_tc_bwd_fast(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
          const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmG, BwdFastArgs a) {
  grid_dep_sync();
  constexpr int D = 32, ROWB = 64, CPR = 4;
  using L = BwdFastSmem;
  const int split = blockIdx.x % a.n_splits;
  const int bh = blockIdx.x / a.n_splits;
  if (a.flag[bh] != 0) return;                     // the exact kernel owns this (b, h)

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sDZ = sQ + L::kLat;
  uint8_t* sZe = sDZ + L::kLat;                    // eL_m * Z_m
  uint8_t* sXB = sZe + L::kLat;                    // B' extension [256][16]
  uint8_t* sTok = sXB + L::kExtB;                  // [3 stages][K | V | dY]
  uint8_t* sGe = sTok + 3 * L::kStage;             // [2] eC_n * dY_n
  uint8_t* sXA = sGe + 2 * L::kT;                  // [2] A' extension [128][16]
  uint8_t* sDS = sXA + 2 * L::kExtA;               // [2] dS^T of a step, by step parity
  float* sL2 = reinterpret_cast<float*>(sDS + 2 * L::kDS);    // [256] L_m in log2 units (+inf past M)
  uint64_t* bars = reinterpret_cast<uint64_t*>(sL2 + 256);
  uint64_t* bar_full = bars;                       // [3] TMA stages
  uint64_t* bar_s = bars + 3;                      // [2] S^T(u) complete, on bar_s[u&1]
  uint64_t* bar_t = bars + 5;                      // T'(u) complete (one phase per step)
  uint64_t* bar_tl = bars + 6;                     // T'(u) is in the softmax threads' registers (512 arrivals)
  uint64_t* bar_pd = bars + 7;                     // [2] P/dS of step u written (512 arrivals)
  uint64_t* bar_p2 = bars + 9;                     // [2] dV/dK/dQ products of step u complete
  uint64_t* bar_q = bars + 11;
  uint64_t* bar_free = bars + 12;                  // dV/dK of a finished tile have been read (warps 16-19: 128 arrivals)
  uint64_t* bar_tile = bars + 13;                  // the dV/dK products of a tile are complete
  uint64_t* bar_ge = bars + 14;                    // [2] every T' product of tile tau complete, on bar_ge[tau&1]
  uint64_t* bar_prep = bars + 16;                  // per-token operands of the next tile written (96 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
  int* abort_flag = reinterpret_cast<int*>(bars + 18);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool is_p2 = warp == kBFSoftmax / 32 + 3;  // issues dV/dK/dQ products, stores lane quarter 3
  const bool is_st = warp == kBFSoftmax / 32 + 2;  // issues S^T/T' products and the TMA loads, stores lane quarter 2
  const bool is_helper = warp == kBFSoftmax / 32 || warp == kBFSoftmax / 32 + 1;   // per-token operands, quarters 0, 1
  const int c4 = (warp >> 2) & 3;                  // column group: 32 latent columns of a step
  const int row = (warp & 3) * 32 + lane;          // token within the tile = tensor-memory lane
  const int b = bh / a.H, h = bh % a.H;
  const int M = a.M;
  const int n_sub = (M + 127) / 128;               // 1 or 2
  const int n0 = split * a.chunk, n1 = min(a.N, n0 + a.chunk);
  const int n_tiles = n1 > n0 ? (n1 - n0 + 127) / 128 : 0;
  const int U = n_tiles * n_sub;                   // steps
  float* dq_out = a.dq_part + ((((long long)split * a.B + b) * a.H + h) * a.M_total + a.m0) * D;

  if (n_tiles == 0) {
    for (int i = tid; i < M * D; i += blockDim.x) dq_out[i] = 0.f;
    return;
  }

  if (tid == 0) {
    for (int i = 0; i < 3; ++i) mbar_init(&bar_full[i], 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_s[i], 1); mbar_init(&bar_p2[i], 1); mbar_init(&bar_pd[i], kBFSoftmax); mbar_init(&bar_ge[i], 1);
    }
    mbar_init(bar_t, 1); mbar_init(bar_tl, kBFSoftmax);
    mbar_init(bar_q, 1); mbar_init(bar_free, 128); mbar_init(bar_tile, 1); mbar_init(bar_prep, 64);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmG);
  }
  if (warp == 0) tmem_alloc<512>(tmem_slot);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
  constexpr uint32_t cS = 0;                       // + 128*buf
  constexpr uint32_t cT = 256;
  constexpr uint32_t cDV = 384, cDK = 416, cDQ = 448;

  auto load_tile = [&](int tau) {
    const int stage = tau % 3;
    uint8_t* dst = sTok + stage * L::kStage;
    const int tok0 = n0 + tau * 128;
    mbar_expect_tx(&bar_full[stage], 3 * L::kT);
    tma_load_4d(dst, &tmK, &bar_full[stage], 0, tok0, h, b);
    tma_load_4d(dst + L::kT, &tmV, &bar_full[stage], 0, tok0, h, b);
    tma_load_4d(dst + 2 * L::kT, &tmG, &bar_full[stage], 0, tok0, h, b);
  };

  if (tid == 0) {
    mbar_expect_tx(bar_q, L::kLat);
    tma_load_4d(sQ, &tmQ, bar_q, 0, 0, h, a.q_batched ? b : 0);
    load_tile(0);
    if (n_tiles > 1) load_tile(1);
    if (n_tiles > 2) load_tile(2);
  }
  const float mu = a.mu[bh];
  // resident latent operands of B': dZ, eL*Z and the extension columns
  {
    const long long lrow = ((long long)b * a.H + h) * a.M_total + a.m0;
    const float* zb = a.z32 + lrow * D;
    const float* dzb = a.dz32 + lrow * D;
    // four consecutive lanes share a latent row (eight values each): coalesced reads, and Delta_m = dZ_m . Z_m
    // is summed over the four by shuffles (whole warps run every iteration: 256 * CPR and blockDim are
    // multiples of 32)
    for (int i = tid; i < 256 * CPR; i += blockDim.x) {
      const int r = i / CPR, c = i % CPR;
      uint4 pz = make_uint4(0, 0, 0, 0), pd = make_uint4(0, 0, 0, 0);
      float l2 = INFINITY, dl = 0.f, el = 0.f;
      if (r < M) {
        l2 = a.lse_m[lrow + r] * kLog2e;
        el = ex2(l2 - mu);
        const float4 z0 = *reinterpret_cast<const float4*>(zb + r * D + c * 8);
        const float4 z1 = *reinterpret_cast<const float4*>(zb + r * D + c * 8 + 4);
        const float4 d0 = *reinterpret_cast<const float4*>(dzb + r * D + c * 8);
        const float4 d1 = *reinterpret_cast<const float4*>(dzb + r * D + c * 8 + 4);
        pz = make_uint4(pack_bf16(z0.x * el, z0.y * el), pack_bf16(z0.z * el, z0.w * el),
                        pack_bf16(z1.x * el, z1.y * el), pack_bf16(z1.z * el, z1.w * el));
        pd = make_uint4(pack_bf16(d0.x, d0.y), pack_bf16(d0.z, d0.w), pack_bf16(d1.x, d1.y), pack_bf16(d1.z, d1.w));
        // Delta_m from dZ as the tensor core sees it (rounded to bf16): sum_n P_mn (V_n . dZ_m) then cancels
        // against it exactly instead of leaving a rounding residue of one sign along the row
        const float zf[8] = {z0.x, z0.y, z0.z, z0.w, z1.x, z1.y, z1.z, z1.w};
        const uint32_t dw[4] = {pd.x, pd.y, pd.z, pd.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 df = Op16<__nv_bfloat16>::unpack(dw[j]);
          dl = fmaf(df.x, zf[2 * j], dl);
          dl = fmaf(df.y, zf[2 * j + 1], dl);
        }
      }
      dl += __shfl_xor_sync(0xffffffffu, dl, 1);
      dl += __shfl_xor_sync(0xffffffffu, dl, 2);
      *reinterpret_cast<uint4*>(sZe + swz_off<ROWB>(r, c)) = pz;
      *reinterpret_cast<uint4*>(sDZ + swz_off<ROWB>(r, c)) = pd;
      if (c == 0) {
        sL2[r] = l2;
        __nv_bfloat16 e[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) e[j] = __float2bfloat16_rn(0.f);
        __nv_bfloat16 dh, dlw, eh, elw;
        split_bf16_4(-dl, dh, dlw);
        split_bf16_4(-el, eh, elw);
        e[0] = dh; e[1] = dlw; e[2] = eh; e[3] = elw; e[4] = eh;
        const uint4* src = reinterpret_cast<const uint4*>(e);
        *reinterpret_cast<uint4*>(sXB + swz_off<32>(r, 0)) = src[0];
        *reinterpret_cast<uint4*>(sXB + swz_off<32>(r, 1)) = src[1];
      }
    }
  }

  const uint32_t id_n128 = idesc_f16(128, 128, 1, 1, 0, 0);  // S^T, T': A, B K-major, N = 128 latents
  const uint32_t id_tv = idesc_f16(128, D, 1, 1, 0, 1);      // dV, dK: A in tensor memory, B MN-major
  const uint32_t id_dq = idesc_f16(128, D, 1, 1, 1, 1);      // dQ: A and B MN-major
  const float sl = a.scale_log2;
  const float* cb = a.lse_n + ((long long)b * a.H + h) * a.N;

  // Per-token operands of token row r of tile tau: eC_n, g_n = eC_n delta_n, the A' extension columns
  // and the eC_n * dY_n row.  yv = the row of Y (four 16-byte chunks), cbv = C_n.
  auto prep_row = [&](int tau, int r, const uint4 (&yv)[4], float cbv) {
    const int n = n0 + tau * 128 + r;
    const uint8_t* tG = sTok + (tau % 3) * L::kStage + 2 * L::kT;
    const bool valid = n < n1;
    const float ec = valid ? ex2(mu - cbv * kLog2e) : 0.f;
    // g_n = (eC_n dY_n) . Y_n with eC_n dY_n rounded to bf16 as the tensor core sees it, so that the scatter
    // term's cancellation sum_m A_mn (Z_m . dY_n - delta_n) is free of that rounding
    float dl = 0.f;
    uint8_t* ge = sGe + (tau & 1) * L::kT;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint4 g4 = *reinterpret_cast<const uint4*>(tG + swz_off<ROWB>(r, c));
      const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g4);
      const __nv_bfloat162* yp = reinterpret_cast<const __nv_bfloat162*>(&yv[c]);
      uint4 o;
      uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 gg2 = __bfloat1622float2(gp[j]), yf = __bfloat1622float2(yp[j]);
        const __nv_bfloat162 gs = __floats2bfloat162_rn(gg2.x * ec, gg2.y * ec);
        const float2 gsf = __bfloat1622float2(gs);
        dl = fmaf(gsf.x, yf.x, dl); dl = fmaf(gsf.y, yf.y, dl);
        ow[j] = *reinterpret_cast<const uint32_t*>(&gs);
      }
      *reinterpret_cast<uint4*>(ge + swz_off<ROWB>(r, c)) = o;
    }
    const float gg = valid ? dl : 0.f;
    __nv_bfloat16 gh, gl;
    split_bf16_4(gg, gh, gl);
    const __nv_bfloat16 one = __float2bfloat16_rn(valid ? 1.f : 0.f);
    const uint32_t w0 = (uint32_t)__bfloat16_as_ushort(one) | ((uint32_t)__bfloat16_as_ushort(one) << 16);
    const uint32_t w1 = (uint32_t)__bfloat16_as_ushort(gh) | ((uint32_t)__bfloat16_as_ushort(gh) << 16);
    const uint32_t w2 = (uint32_t)__bfloat16_as_ushort(gl);
    uint8_t* xa = sXA + (tau & 1) * L::kExtA;
    *reinterpret_cast<uint4*>(xa + swz_off<32>(r, 0)) = make_uint4(w0, w1, w2, 0u);
    *reinterpret_cast<uint4*>(xa + swz_off<32>(r, 1)) = make_uint4(0u, 0u, 0u, 0u);
  };
  auto fetch_row = [&](int tau, int r, uint4 (&yv)[4], float& cbv) {
    const int n = n0 + tau * 128 + r;
    cbv = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) yv[c] = make_uint4(0, 0, 0, 0);
    if (n < n1) {
      const uint4* yp = reinterpret_cast<const uint4*>(a.y + b * a.ys[0] + h * a.ys[1] + (long long)n * a.ys[2]);
#pragma unroll
      for (int c = 0; c < 4; ++c) yv[c] = yp[c];
      cbv = cb[n];
    }
  };

  // Descriptor words: the high word depends on the layout only; the low word is (address >> 4) plus a
  // constant (a 128-latent block of Q/dZ/eL*Z is 512 units on, of the B' extension 256, a token stage
  // 1536 with V +512 and dY +1024, the eC*dY buffers 512 apart, the A' extensions 256, the dS blocks 2048).
  const uint64_t dsc64 = smem_desc<ROWB>(smem_u32(sQ)), dsc32 = smem_desc<32>(smem_u32(sXB)),
                 dscmn = smem_desc_mn128(smem_u32(sDS), 128 * 128, 1024);
  const uint64_t hi64 = dsc64 & 0xffffffff00000000ull, hi32 = dsc32 & 0xffffffff00000000ull,
                 himn = dscmn & 0xffffffff00000000ull;
  const uint32_t q_lo = (uint32_t)dsc64, xb_lo = (uint32_t)dsc32, ds_lo = (uint32_t)dscmn;
  const uint32_t dz_lo = q_lo + (L::kLat >> 4), ze_lo = q_lo + 2 * (L::kLat >> 4);
  const uint32_t tok_lo = (uint32_t)smem_desc<ROWB>(smem_u32(sTok)), ge_lo = (uint32_t)smem_desc<ROWB>(smem_u32(sGe));
  const uint32_t xa_lo = (uint32_t)smem_desc<32>(smem_u32(sXA));

  // S^T of step u2 (tile in stage stg, latent block s) into buffer u2 & 1
  auto issue_s = [&](int u2, int stg, int s) {
    const uint32_t d = tmem + cS + 128 * (u2 & 1);
    const uint64_t aK = hi64 | (tok_lo + stg * (L::kStage >> 4)), bQ = hi64 | (q_lo + s * 512);
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) mma_ss(d, aK + 2 * kk, bQ + 2 * kk, id_n128, kk > 0);
  };
  // T' of the step (tile in stage stg, per-token buffers of parity par, latent block s)
  auto issue_t = [&](int stg, int par, int s) {
    const uint32_t d = tmem + cT;
    const uint64_t aV = hi64 | (tok_lo + stg * (L::kStage >> 4) + (L::kT >> 4)), aG = hi64 | (ge_lo + par * (L::kT >> 4)),
                   aX = hi32 | (xa_lo + par * (L::kExtA >> 4));
    const uint64_t bDZ = hi64 | (dz_lo + s * 512), bZe = hi64 | (ze_lo + s * 512), bX = hi32 | (xb_lo + s * 256);
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) mma_ss(d, aV + 2 * kk, bDZ + 2 * kk, id_n128, kk > 0);
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) mma_ss(d, aG + 2 * kk, bZe + 2 * kk, id_n128, true);
    mma_ss(d, aX, bX, id_n128, true);
  };
  // dV += P^T dZ_s, dK += dS^T Q_s  (P at +32(kk/2)+8(kk%2) of the step's buffer, dS 16 further): the
  // products that read the S^T buffer
  auto issue_dvdk = [&](int u, int s) {
    const uint32_t buf = tmem + cS + 128 * (u & 1);
    const uint64_t bDZ = hi64 | (dz_lo + s * 512), bQ = hi64 | (q_lo + s * 512);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const uint32_t pa = buf + 32 * (kk >> 1) + 8 * (kk & 1);
      mma_ts(tmem + cDV, pa, bDZ + 64 * kk, id_tv, (s > 0) || (kk > 0));
      mma_ts(tmem + cDK, pa + 16, bQ + 64 * kk, id_tv, (s > 0) || (kk > 0));
    }
  };
  // dQ_s += dS K_t  (dS from shared memory)
  auto issue_dq = [&](int u, int stg, int t, int s) {
    const uint64_t bK = hi64 | (tok_lo + stg * (L::kStage >> 4)), aDS = himn | (ds_lo + (u & 1) * (L::kDS >> 4));
#pragma unroll
    for (int kk = 0; kk < 8; ++kk)
      mma_ss(tmem + cDQ + 32 * s, aDS + 128 * kk, bK + 64 * kk, id_dq, (t > 0) || (kk > 0));
  };

  auto write_half = [&](__nv_bfloat16* op, const uint32_t (&r)[2][16], float f) {
#pragma unroll
    for (int pc = 0; pc < 2; ++pc) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float g[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] = __uint_as_float(r[pc][8 * c + j]) * f;
        if constexpr (ACC) {                       // a later latent block: add to what the earlier ones wrote
          const uint4 old = reinterpret_cast<const uint4*>(op + 16 * pc)[c];
          const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 of = __bfloat1622float2(o2[j]);
            g[2 * j] += of.x; g[2 * j + 1] += of.y;
          }
        }
        uint4 o;
        o.x = pack_bf16(g[0], g[1]); o.y = pack_bf16(g[2], g[3]);
        o.z = pack_bf16(g[4], g[5]); o.w = pack_bf16(g[6], g[7]);
        reinterpret_cast<uint4*>(op + 16 * pc)[c] = o;
      }
    }
  };

  // ---- prologue: per-token operands of tile 0 by the first 128 threads ---------------------------
  if (tid < 128) {
    uint4 yv[4]; float cbv;
    fetch_row(0, tid, yv, cbv);
    mbar_wait(&bar_full[0], 0, a.status, abort_flag);
    prep_row(0, tid, yv, cbv);
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();

  // One lane quarter of dV/dK of finished tile t: dV first (read, write out), then dK, so that only half
  // of the values sit in registers at a time.
  auto store_quarter = [&](int t) {
    const int n = n0 + t * 128 + row;
    {
      uint32_t r[2][16];
      tmem_ld16(lane_base + cDV, r[0]);
      tmem_ld16(lane_base + cDV + 16, r[1]);
      tmem_wait_ld();
      if (n < n1) write_half(a.dv + b * a.dvs[0] + h * a.dvs[1] + (long long)n * a.dvs[2], r, 1.f);
    }
    {
      uint32_t r[2][16];
      tmem_ld16(lane_base + cDK, r[0]);
      tmem_ld16(lane_base + cDK + 16, r[1]);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive4(bar_free);
      if (n < n1) write_half(a.dk + b * a.dks[0] + h * a.dks[1] + (long long)n * a.dks[2], r, a.scale);
    }
  };

  if (is_st) {
    // ================= S^T / T' issuer: the whole warp runs the code, one elected lane issues =================
    mbar_wait(bar_q, 0, a.status, abort_flag);
    mbar_wait(&bar_full[0], 0, a.status, abort_flag);
    tc_fence_after();
    if (elect_one()) {
      issue_s(0, 0, 0);
      mma_commit(&bar_s[0]);
      issue_t(0, 0, 0);
      mma_commit(bar_t);
      if (n_sub == 1) mma_commit(&bar_ge[0]);
    }
    __syncwarp();
    if (U > 1) {
      // S^T of step 1: the second latent block of tile 0, or tile 1
      const int t1 = n_sub > 1 ? 0 : 1, s1 = n_sub > 1 ? 1 : 0;
      if (t1 == 1) mbar_wait(&bar_full[1], 0, a.status, abort_flag);
      tc_fence_after();
      if (elect_one()) { issue_s(1, t1, s1); mma_commit(&bar_s[1]); }
      __syncwarp();
    }
    int t = 0, s = 0, stg = 0;                     // step u = (tile t in stage stg, latent block s)
    for (int u = 0; u < U; ++u) {
      const int xb = u & 1;
      int t1 = t, s1 = s + 1, stg1 = stg;          // step u+1
      if (s1 == n_sub) { s1 = 0; ++t1; stg1 = stg == 2 ? 0 : stg + 1; }
      // T'(u) is in the softmax threads' registers: its buffer takes T'(u+1)
      mbar_wait_hot(bar_tl, (uint32_t)u & 1, a.status, abort_flag);
      if (*reinterpret_cast<volatile int*>(abort_flag)) break;
      if (u + 1 < U) {
        if (s1 == 0) {                             // first step of a tile: its token data and per-token operands
          mbar_wait_hot(&bar_full[stg1], (uint32_t)(t1 / 3) & 1, a.status, abort_flag);
          mbar_wait_hot(bar_prep, (uint32_t)(t1 - 1) & 1, a.status, abort_flag);
        }
        tc_fence_after();
        if (elect_one()) {
          issue_t(stg1, t1 & 1, s1);
          mma_commit(bar_t);
          if (s1 == n_sub - 1) mma_commit(&bar_ge[t1 & 1]);   // the tile's per-token operands are dead after this
        }
        __syncwarp();
      }
      // After the last step of a tile: its dV/dK accumulators are read out once their products have
      // completed, and its token stage takes the tile three further on once dQ has read K too.
      if (s == n_sub - 1) {
        mbar_wait_hot(bar_tile, (uint32_t)t & 1, a.status, abort_flag);
        if (*reinterpret_cast<volatile int*>(abort_flag)) break;
        tc_fence_after();
        store_quarter(t);
        if (t + 3 < n_tiles) {
          mbar_wait_hot(&bar_p2[xb], (uint32_t)(u >> 1) & 1, a.status, abort_flag);
          if (elect_one()) load_tile(t + 3);
          __syncwarp();
        }
      }
      t = t1; s = s1; stg = stg1;
    }
  } else if (is_p2) {
    // ================= dV / dK / S^T / dQ issuer =================
    // dV/dK of step u, then S^T(u+2) into the buffer they read: products issued by one thread execute in
    // issue order, so no completion round trip sits between them; then dQ(u).  After the last step of a
    // tile this warp reads its lane quarter of dV/dK as soon as their products are complete, so that the
    // accumulators are free before the next tile's first dS is written.
    int t = 0, s = 0, stg = 0;
    for (int u = 0; u < U; ++u) {
      const int xb = u & 1;
      int t2 = t, s2 = s + 2, stg2 = stg;            // step u+2
      while (s2 >= n_sub) { s2 -= n_sub; ++t2; stg2 = stg2 == 2 ? 0 : stg2 + 1; }
      const bool next = u + 2 < U;
      const bool last = s == n_sub - 1;
      mbar_wait_hot(&bar_pd[xb], (uint32_t)(u >> 1) & 1, a.status, abort_flag);   // P and dS of step u are written
      if (*reinterpret_cast<volatile int*>(abort_flag)) break;
      if (s == 0 && t > 0) mbar_wait_hot(bar_free, (uint32_t)(t - 1) & 1, a.status, abort_flag);   // dV/dK of tile t-1 read out
      if (next && t2 != t) mbar_wait_hot(&bar_full[stg2], (uint32_t)(t2 / 3) & 1, a.status, abort_flag);
      tc_fence_after();
      if (elect_one()) {
        issue_dvdk(u, s);
        if (last) mma_commit(bar_tile);              // one phase per tile: the other warps follow it in order
        issue_dq(u, stg, t, s);
        if (next) { issue_s(u + 2, stg2, s2); mma_commit(&bar_s[xb]); }
        mma_commit(&bar_p2[xb]);
      }
      __syncwarp();
      if (last) {
        mbar_wait_hot(bar_tile, (uint32_t)t & 1, a.status, abort_flag);
        if (*reinterpret_cast<volatile int*>(abort_flag)) break;
        tc_fence_after();
        store_quarter(t);
      }
      if (++s == n_sub) { s = 0; ++t; stg = stg == 2 ? 0 : stg + 1; }
    }
  } else if (is_helper) {
    // ================= helper warps: per-token operands of tile t+1, then dV/dK of tile t -> global =========
    // Y rows and C_n of a tile are fetched one tile before they are needed, so that the DRAM latency
    // never sits between the end of a tile and the first product of the next one.
    const int j = tid - kBFSoftmax;                // 0..63: rows j and j + 64
    uint4 yv0[4], yv1[4];
    float cb0 = 0.f, cb1 = 0.f;
    if (n_tiles > 1) {
      fetch_row(1, j, yv0, cb0);
      fetch_row(1, j + 64, yv1, cb1);
    }
    for (int t = 0; t < n_tiles; ++t) {
      if (t + 1 < n_tiles) {
        const int tau = t + 1;
        // the buffers of tile tau were last read by the T' products of tile tau-2
        if (tau >= 2) mbar_wait(&bar_ge[tau & 1], (uint32_t)((tau - 2) >> 1) & 1, a.status, abort_flag);
        mbar_wait(&bar_full[tau % 3], (uint32_t)(tau / 3) & 1, a.status, abort_flag);
        prep_row(tau, j, yv0, cb0);
        prep_row(tau, j + 64, yv1, cb1);
        fence_proxy_async();
        mbar_arrive4(bar_prep);
        if (t + 2 < n_tiles) {
          fetch_row(t + 2, j, yv0, cb0);
          fetch_row(t + 2, j + 64, yv1, cb1);
        }
      }
      mbar_wait_hot(bar_tile, (uint32_t)t & 1, a.status, abort_flag);
      if (*reinterpret_cast<volatile int*>(abort_flag)) break;
      tc_fence_after();
      store_quarter(t);
    }
  } else {
    // ================= softmax threads =================
    int s = 0;
    for (int u = 0; u < U; ++u) {
      const int xb = u & 1;
      const uint32_t buf = lane_base + cS + 128 * xb + 32 * c4;
      const float* l2p = sL2 + s * 128 + 32 * c4;
      // ---- phase A: P = ex2(S^T sl - L), packed into the first 16 of this thread's 32 columns ------
      mbar_wait_hot(&bar_s[xb], (uint32_t)(u >> 1) & 1, a.status, abort_flag);
      tc_fence_after();
      uint32_t ra[16], rb[16];
      float p[32];
      tmem_ld16(buf, ra);
      tmem_ld16(buf + 16, rb);
      tmem_wait_ld();
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float4 l4 = *reinterpret_cast<const float4*>(l2p + 4 * e);
        p[4 * e] = ex2(fmaf(__uint_as_float(ra[4 * e]), sl, -l4.x));
        p[4 * e + 1] = ex2(fmaf(__uint_as_float(ra[4 * e + 1]), sl, -l4.y));
        p[4 * e + 2] = ex2(fmaf(__uint_as_float(ra[4 * e + 2]), sl, -l4.z));
        p[4 * e + 3] = ex2(fmaf(__uint_as_float(ra[4 * e + 3]), sl, -l4.w));
      }
      tmem_wait_ld();
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float4 l4 = *reinterpret_cast<const float4*>(l2p + 16 + 4 * e);
        p[16 + 4 * e] = ex2(fmaf(__uint_as_float(rb[4 * e]), sl, -l4.x));
        p[16 + 4 * e + 1] = ex2(fmaf(__uint_as_float(rb[4 * e + 1]), sl, -l4.y));
        p[16 + 4 * e + 2] = ex2(fmaf(__uint_as_float(rb[4 * e + 2]), sl, -l4.z));
        p[16 + 4 * e + 3] = ex2(fmaf(__uint_as_float(rb[4 * e + 3]), sl, -l4.w));
      }
      {
        uint32_t pp[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) pp[e] = pack_bf16(p[2 * e], p[2 * e + 1]);
        tmem_st16(buf, pp);
      }
      // ---- phase B: dS = P * T', packed into the last 16 columns and to shared memory ---------------
      mbar_wait_hot(bar_t, (uint32_t)u & 1, a.status, abort_flag);
      tc_fence_after();
      const uint32_t tcol = lane_base + cT + 32 * c4;
      tmem_ld16(tcol, ra);
      tmem_ld16(tcol + 16, rb);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive4(bar_tl);                        // the T' buffer may take the next step
      uint32_t pd[16];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        pd[e] = pack_bf16(p[2 * e] * __uint_as_float(ra[2 * e]), p[2 * e + 1] * __uint_as_float(ra[2 * e + 1]));
        pd[8 + e] = pack_bf16(p[16 + 2 * e] * __uint_as_float(rb[2 * e]), p[16 + 2 * e + 1] * __uint_as_float(rb[2 * e + 1]));
      }
      tmem_st16(buf + 16, pd);
      // (the shared-memory dS block of this step was last read by dQ(u-2), issued ahead of S^T(u) by the
      // same thread, hence complete)
      // dS^T of the step as the MN-major A operand of dQ: 64-latent half c4/2, 16-byte chunks 4(c4%2)..+3
      uint8_t* ds_row = sDS + xb * L::kDS + (c4 >> 1) * (128 * 128);
#pragma unroll
      for (int i = 0; i < 4; ++i)
        *reinterpret_cast<uint4*>(ds_row + swz_off<128>(row, 4 * (c4 & 1) + i)) =
            make_uint4(pd[4 * i], pd[4 * i + 1], pd[4 * i + 2], pd[4 * i + 3]);
      tmem_wait_st();
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive4(&bar_pd[xb]);
      if (*reinterpret_cast<volatile int*>(abort_flag)) break;
      if (++s == n_sub) s = 0;
    }

    // ---- tail: the dQ partial --------------------------------------------------------------------
    if (!*reinterpret_cast<volatile int*>(abort_flag)) {
      if (U >= 2) mbar_wait(&bar_p2[(U - 2) & 1], (uint32_t)((U - 2) >> 1) & 1, a.status, abort_flag);
      mbar_wait(&bar_p2[(U - 1) & 1], (uint32_t)((U - 1) >> 1) & 1, a.status, abort_flag);
      tc_fence_after();
      const int piece = c4 & 1, j = c4 >> 1;       // latent block j, 16-column piece
      if (j < n_sub) {
        uint32_t q[16];
        tmem_ld16(lane_base + cDQ + 32 * j + 16 * piece, q);
        tmem_wait_ld();
        const int m = j * 128 + row;
        if (m < M) {
          float* o = dq_out + (long long)m * D + 16 * piece;
#pragma unroll
          for (int c = 0; c < 4; ++c)
            reinterpret_cast<float4*>(o)[c] = make_float4(__uint_as_float(q[4 * c]) * a.scale, __uint_as_float(q[4 * c + 1]) * a.scale,
                                                          __uint_as_float(q[4 * c + 2]) * a.scale, __uint_as_float(q[4 * c + 3]) * a.scale);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc<512>(tmem);
}

// ------------------------------------------------------------------------------------------
bool tc_bwd_fast_supported(const Ctx& c, int dtype) {
  // more than 256 latents run as blocks of 256 that add into dK/dV
  return dtype == FLARE_BF16 && c.D == 32 && c.M >= 32 && c.M <= 1024 && c.N >= 1 && c.terms == FLARE_TERM_BOTH;
}

int tc_bwd_fast_launch(const Ctx& c, const void* q, const void* k, const void* v, const void* dy, const void* y,
                   const float* z32, const float* dz32, const float* lse_m, const float* lse_n, void* dk, void* dv,
                   float* dq_part, const float* mu, const int* flag, cudaStream_t st) {
  constexpr int D = 32;
  CUtensorMap tmK, tmV, tmG;
  const uint64_t e = 2;
  const bool qb = c.qs[0] != 0;
  auto tokmap = [&](CUtensorMap* m, const void* p, const long long* s) {
    return make_tile_map(m, p, 1, D, (uint64_t)c.N, (uint64_t)c.H, (uint64_t)c.B, s[2] * e, s[1] * e,
                         (c.B > 1 ? s[0] : s[1] * c.H) * e, 128);
  };
  if (!tokmap(&tmK, k, c.ks) || !tokmap(&tmV, v, c.vs) || !tokmap(&tmG, dy, c.dys)) return FLARE_EUNSUPPORTED;
  BwdFastArgs a;
  a.B = c.B; a.H = c.H; a.N = c.N; a.M_total = c.M;
  a.scale = c.scale; a.scale_log2 = c.scale * kLog2e;
  a.q_batched = qb ? 1 : 0;
  a.n_splits = c.n_splits; a.chunk = c.chunk;
  a.z32 = z32; a.dz32 = dz32; a.lse_m = lse_m; a.lse_n = lse_n;
  a.mu = mu; a.flag = flag;
  a.y = reinterpret_cast<const __nv_bfloat16*>(y);
  a.dk = reinterpret_cast<__nv_bfloat16*>(dk); a.dv = reinterpret_cast<__nv_bfloat16*>(dv);
  for (int i = 0; i < 3; ++i) { a.ys[i] = c.ys[i]; a.dks[i] = c.dks[i]; a.dvs[i] = c.dvs[i]; }
  a.dq_part = dq_part;
  a.status = tc_status_ptr();
  constexpr int smem = BwdFastSmem::kBytes;
  if (tc_set_dyn_smem(reinterpret_cast<const void*>(&k_tc_bwd_fast<false>), smem) != FLARE_OK) return FLARE_ECUDA;
  if (tc_set_dyn_smem(reinterpret_cast<const void*>(&k_tc_bwd_fast<true>), smem) != FLARE_OK) return FLARE_ECUDA;
  const long long grid = (long long)c.n_splits * c.B * c.H;
  if (grid > 0x7fffffffLL) return FLARE_EUNSUPPORTED;
  for (int m0 = 0; m0 < c.M; m0 += 256) {
    const int mb = c.M - m0 < 256 ? c.M - m0 : 256;
    CUtensorMap tmQ;
    const char* qblk = static_cast<const char*>(q) + (long long)m0 * c.qs[2] * e;
    if (!make_tile_map(&tmQ, qblk, 1, D, (uint64_t)mb, (uint64_t)c.H, (uint64_t)(qb ? c.B : 1), c.qs[2] * e, c.qs[1] * e,
                       (qb ? c.qs[0] : c.qs[1] * c.H) * e, 256))
      return FLARE_EUNSUPPORTED;
    a.M = mb; a.m0 = m0;
    if (m0 == 0) launch_dep(k_tc_bwd_fast<false>, dim3((unsigned)grid), dim3(kBFSoftmax + kBFHelpers + 32), smem, st, tmQ, tmK, tmV, tmG, a);
    else launch_dep(k_tc_bwd_fast<true>, dim3((unsigned)grid), dim3(kBFSoftmax + kBFHelpers + 32), smem, st, tmQ, tmK, tmV, tmG, a);
  }
  return FLARE_OK;
}

}  // namespace flare
