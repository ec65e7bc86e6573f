// Main backward pass, one exponential per score, software-pipelined: the tensor core and the
// softmax threads work on different steps at the same time.
//
// Same mathematics as flare_tc_bwd2.cu (dS = P * T', T' from one extended-contraction product;
// the (b, h) it may run are chosen by the same on-device range check).  What differs is the
// schedule.  A step u = (token tile t, 64-latent slice s):
//
//   issuer warp  : waits until the 512 softmax threads have finished step u, then issues
//                  P2(u)  : dV += P^T dZ_s, dK += dS^T Q_s, and every second slice dQ_j += dS K_t
//                  P1(u+2): S^T and T' of the step after next, into the buffer step u just freed
//                  and commits both onto one mbarrier.
//   softmax warps: wait for the commit of step u-2 (so S^T/T' of step u are there and the packed
//                  P/dS buffer of step u-2 is free), compute P = ex2(.), dS = P*T', write them packed
//                  to tensor memory and dS also to shared memory, prepare the next tile's per-token
//                  operands when one is due, and arrive on the issuer's mbarrier.
//
// Tensor memory (512 columns): S^T/T' double-buffered [0,128) [128,256); packed P/dS double-
// buffered [256,320) [320,384); dV 384, dK 416, dQ_0 448, dQ_1 480.  While the softmax threads are
// in step u+1 the tensor core runs P2(u) and P1(u+2): neither side waits for the other in steady
// state.  dV/dK of a tile are stored during the first step of the next tile.
// Token tiles (K, V, dY) arrive by TMA in a three-stage ring; Y is read straight from global
// memory for delta_n = dY_n . Y_n.  Requires bf16, D = 32, 128 < M <= 256.
#include "common.cuh"
#include "launch.h"
#include "tc_common.cuh"
#include "tma_host.h"

namespace flare {

using namespace tc;

struct Bwd3Args {
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
  float* dq_part;              // [S,B,H,M,D]
  int* status;
  long long* prof;             // optional phase counters, or null
};

struct Bwd3Smem {
  static constexpr int D = 32, ROWB = 64;
  static constexpr int kLat = 256 * ROWB;          // Q, dZ or eL*Z: all latents
  static constexpr int kExtB = 256 * 32;           // extension columns of B'
  static constexpr int kT = 128 * ROWB;            // one token tile
  static constexpr int kStage = 3 * kT;            // K, V, dY
  static constexpr int kExtA = 128 * 32;           // extension columns of A'
  static constexpr int kDS = 2 * 128 * 128;        // dS^T of one 128-latent block
  static constexpr int kBytes = 3 * kLat + kExtB + 3 * kStage + 2 * kT + 2 * kExtA + 2 * kDS + 256 * 4 + 1024 + 256;
};

__device__ __forceinline__ void split_bf16_3(float x, __nv_bfloat16& hi, __nv_bfloat16& lo) {
  hi = __float2bfloat16_rn(x);
  lo = __float2bfloat16_rn(x - __bfloat162float(hi));
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

constexpr int kSoftmaxThreads = 512, kStoreThreads = 96;   // the issuer warp stores the fourth lane quarter

__global__ void __launch_bounds__(kSoftmaxThreads + kStoreThreads + 32, 1)
k_tc_bwd3(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
          const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmG, Bwd3Args a) {
  constexpr int D = 32, ROWB = 64, CPR = 4;
  using L = Bwd3Smem;
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
  uint8_t* sDS = sXA + 2 * L::kExtA;               // [2 latent blocks]
  float* sL2 = reinterpret_cast<float*>(sDS + 2 * L::kDS);    // [256] L_m in log2 units (+inf past M)
  uint64_t* bars = reinterpret_cast<uint64_t*>(sL2 + 256);
  uint64_t* bar_full = bars;                       // [3] TMA stages
  uint64_t* bar_c = bars + 3;                      // [2] commit of step u on bar_c[u&1]
  uint64_t* bar_simt = bars + 5;                   // [2] softmax threads done with step u
  uint64_t* bar_pro = bars + 7;                    // first two S^T/T' products
  uint64_t* bar_q = bars + 8;
  uint64_t* bar_free = bars + 9;                   // dV/dK of a finished tile have been read (128 arrivals)
  uint64_t* bar_tile = bars + 10;                  // every product of a tile is complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  int* abort_flag = reinterpret_cast<int*>(bars + 12);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool is_issuer = warp == (kSoftmaxThreads + kStoreThreads) / 32;
  const bool is_store = !is_issuer && warp >= kSoftmaxThreads / 32;   // three warps that write dV/dK of finished tiles
  const int g = (warp >> 2) & 3;                   // column group 0..3 (16 latent columns of a slice)
  const int row = (warp & 3) * 32 + lane;          // token within the tile = tensor-memory lane
  const int b = bh / a.H, h = bh % a.H;
  const int M = a.M;
  const int n_sub = (M + 63) / 64;                 // 3 or 4
  const int n0 = split * a.chunk, n1 = min(a.N, n0 + a.chunk);
  const int n_tiles = n1 > n0 ? (n1 - n0 + 127) / 128 : 0;
  const int U = n_tiles * n_sub;                   // steps
  float* dq_out = a.dq_part + (((long long)split * a.B + b) * a.H + h) * M * D;

  if (n_tiles == 0) {
    for (int i = tid; i < M * D; i += blockDim.x) dq_out[i] = 0.f;
    return;
  }

  if (tid == 0) {
    for (int i = 0; i < 3; ++i) mbar_init(&bar_full[i], 1);
    mbar_init(&bar_c[0], 1); mbar_init(&bar_c[1], 1);
    mbar_init(&bar_simt[0], kSoftmaxThreads); mbar_init(&bar_simt[1], kSoftmaxThreads);
    mbar_init(bar_pro, 1); mbar_init(bar_q, 1); mbar_init(bar_free, kStoreThreads); mbar_init(bar_tile, 1);
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
  constexpr uint32_t cX = 0;                       // + 128*buf: S^T [0,64), T' [64,128)
  constexpr uint32_t cPD = 256;                    // + 64*buf:  P [0,32), dS [32,64)
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
  }
  const float mu = a.mu[bh];
  long long k_c0 = 0; unsigned long long k_t0 = 0;
  if (a.prof && tid == 0 && blockIdx.x == 0) { k_c0 = clock64(); asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(k_t0)); }
  // resident latent operands of B': dZ, eL*Z and the extension columns
  {
    const long long lrow = ((long long)b * a.H + h) * M;
    const float* zb = a.z32 + lrow * D;
    const float* dzb = a.dz32 + lrow * D;
    for (int i = tid; i < 256 * CPR; i += blockDim.x) {
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
      split_bf16_3(-dl, dh, dlw);
      split_bf16_3(-el, eh, elw);
      e[0] = dh; e[1] = dlw; e[2] = eh; e[3] = elw; e[4] = eh;
      const uint4* src = reinterpret_cast<const uint4*>(e);
      *reinterpret_cast<uint4*>(sXB + swz_off<32>(m, 0)) = src[0];
      *reinterpret_cast<uint4*>(sXB + swz_off<32>(m, 1)) = src[1];
    }
  }

  const uint32_t id_st = idesc_f16(128, 64, 1, 1, 0, 0);     // S^T, T' slices: A, B K-major, N = 64
  const uint32_t id_tv = idesc_f16(128, D, 1, 1, 0, 1);      // dV, dK: A in tensor memory, B MN-major
  const uint32_t id_dq = idesc_f16(128, D, 1, 1, 1, 1);      // dQ: A and B MN-major
  const float sl = a.scale_log2;
  const float* cb = a.lse_n + ((long long)b * a.H + h) * a.N;

  // Per-token operands of tile tau: eC_n, g_n = eC_n delta_n, the A' extension columns and the
  // eC_n * dY_n tile.  Thread (r, c) owns 16-byte chunk c of token row r; yv/cbv were loaded from
  // global memory at the start of the step.  No CTA barrier inside.
  auto prep_tile = [&](int tau, uint4 yv, float cbv) {
    const int r = tid >> 2, c = tid & 3;
    const int n = n0 + tau * 128 + r;
    const uint8_t* tG = sTok + (tau % 3) * L::kStage + 2 * L::kT;
    const uint4 g4 = *reinterpret_cast<const uint4*>(tG + swz_off<ROWB>(r, c));
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* yp = reinterpret_cast<const __nv_bfloat162*>(&yv);
    float gf[8];
    float dl = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 gg2 = __bfloat1622float2(gp[j]), yf = __bfloat1622float2(yp[j]);
      gf[2 * j] = gg2.x; gf[2 * j + 1] = gg2.y;
      dl = fmaf(gg2.x, yf.x, dl); dl = fmaf(gg2.y, yf.y, dl);
    }
    dl += __shfl_xor_sync(0xffffffffu, dl, 1);
    dl += __shfl_xor_sync(0xffffffffu, dl, 2);
    const bool valid = n < n1;
    const float ec = valid ? ex2(mu - cbv * kLog2e) : 0.f;
    uint4 o;
    o.x = pack_bf16(gf[0] * ec, gf[1] * ec); o.y = pack_bf16(gf[2] * ec, gf[3] * ec);
    o.z = pack_bf16(gf[4] * ec, gf[5] * ec); o.w = pack_bf16(gf[6] * ec, gf[7] * ec);
    *reinterpret_cast<uint4*>(sGe + (tau & 1) * L::kT + swz_off<ROWB>(r, c)) = o;
    if (c == 0) {
      const float gg = valid ? ec * dl : 0.f;
      __nv_bfloat16 e[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) e[i] = __float2bfloat16_rn(0.f);
      __nv_bfloat16 gh, gl;
      split_bf16_3(gg, gh, gl);
      const __nv_bfloat16 one = __float2bfloat16_rn(valid ? 1.f : 0.f);
      e[0] = one; e[1] = one; e[2] = gh; e[3] = gh; e[4] = gl;
      const uint4* src = reinterpret_cast<const uint4*>(e);
      uint8_t* xa = sXA + (tau & 1) * L::kExtA;
      *reinterpret_cast<uint4*>(xa + swz_off<32>(r, 0)) = src[0];
      *reinterpret_cast<uint4*>(xa + swz_off<32>(r, 1)) = src[1];
    }
    fence_proxy_async();
  };
  auto fetch_y = [&](int tau, uint4& yv, float& cbv) {
    const int r = tid >> 2, c = tid & 3;
    const int n = n0 + tau * 128 + r;
    yv = make_uint4(0, 0, 0, 0); cbv = 0.f;
    if (n < n1) {
      yv = *reinterpret_cast<const uint4*>(a.y + b * a.ys[0] + h * a.ys[1] + (long long)n * a.ys[2] + 8 * c);
      cbv = cb[n];
    }
  };

  // S^T and T' of step u2 into buffer (u2 & 1)
  auto issue_p1 = [&](int u2, int tau, int s) {
    const uint8_t* tK = sTok + (tau % 3) * L::kStage;
    const uint32_t lo = (uint32_t)(s * 64 * ROWB);
    const uint32_t cx = tmem + cX + 128 * (u2 & 1);
    const uint64_t aK = smem_desc<ROWB>(smem_u32(tK)), aV = smem_desc<ROWB>(smem_u32(tK + L::kT)),
                   aG = smem_desc<ROWB>(smem_u32(sGe + (tau & 1) * L::kT)),
                   aX = smem_desc<32>(smem_u32(sXA + (tau & 1) * L::kExtA));
    const uint64_t bQ = smem_desc<ROWB>(smem_u32(sQ) + lo), bDZ = smem_desc<ROWB>(smem_u32(sDZ) + lo),
                   bZe = smem_desc<ROWB>(smem_u32(sZe) + lo), bX = smem_desc<32>(smem_u32(sXB) + s * 64 * 32);
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) mma_ss(cx, aK + 2 * kk, bQ + 2 * kk, id_st, kk > 0);
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) mma_ss(cx + 64, aV + 2 * kk, bDZ + 2 * kk, id_st, kk > 0);
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) mma_ss(cx + 64, aG + 2 * kk, bZe + 2 * kk, id_st, true);
    mma_ss(cx + 64, aX, bX, id_st, true);
  };
  // dV += P^T dZ_s, dK += dS^T Q_s, and after the last slice of a 128-latent block dQ_j += dS K_t
  auto issue_p2 = [&](int u, int t, int s) {
    const uint8_t* tK = sTok + (t % 3) * L::kStage;
    const uint32_t lo = (uint32_t)(s * 64 * ROWB);
    const uint32_t cpd = tmem + cPD + 64 * (u & 1);
    const uint64_t bDZ = smem_desc<ROWB>(smem_u32(sDZ) + lo), bQ = smem_desc<ROWB>(smem_u32(sQ) + lo);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const uint64_t boff = (uint64_t)((kk * 16 * ROWB) >> 4);
      mma_ts(tmem + cDV, cpd + 8 * kk, bDZ + boff, id_tv, (s > 0) || (kk > 0));
      mma_ts(tmem + cDK, cpd + 32 + 8 * kk, bQ + boff, id_tv, (s > 0) || (kk > 0));
    }
    if ((s & 1) || s == n_sub - 1) {
      const int j = s >> 1;
      const uint64_t bK = smem_desc<ROWB>(smem_u32(tK));
      const uint64_t aDS = smem_desc_mn128(smem_u32(sDS + j * L::kDS), 128 * 128, 1024);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        mma_ss(tmem + cDQ + 32 * j, aDS + (uint64_t)((kk * 2048) >> 4), bK + (uint64_t)((kk * 16 * ROWB) >> 4),
               id_dq, (t > 0) || (kk > 0));
    }
  };

  if (a.prof && tid == 0 && blockIdx.x == 0) a.prof[11] = clock64() - k_c0;   // resident operands built
  // dV/dK rows of tile t for this warp's lane quarter: tensor memory -> registers, then -> global
  auto read_dvdk = [&](uint32_t (&r)[4][16]) {
    tmem_ld16(lane_base + cDV, r[0]);
    tmem_ld16(lane_base + cDV + 16, r[1]);
    tmem_ld16(lane_base + cDK, r[2]);
    tmem_ld16(lane_base + cDK + 16, r[3]);
    tmem_wait_ld();
    tc_fence_before();
  };
  auto write_dvdk = [&](int t, const uint32_t (&r)[4][16]) {
    const int n = n0 + t * 128 + row;
    if (n < n1) {
      __nv_bfloat16* pv = a.dv + b * a.dvs[0] + h * a.dvs[1] + (long long)n * a.dvs[2];
      __nv_bfloat16* pk = a.dk + b * a.dks[0] + h * a.dks[1] + (long long)n * a.dks[2];
#pragma unroll
      for (int pc = 0; pc < 4; ++pc) {
        const float f = pc >= 2 ? a.scale : 1.f;
        __nv_bfloat16* op = (pc >= 2 ? pk : pv) + 16 * (pc & 1);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint4 o;
          o.x = pack_bf16(__uint_as_float(r[pc][8 * c]) * f, __uint_as_float(r[pc][8 * c + 1]) * f);
          o.y = pack_bf16(__uint_as_float(r[pc][8 * c + 2]) * f, __uint_as_float(r[pc][8 * c + 3]) * f);
          o.z = pack_bf16(__uint_as_float(r[pc][8 * c + 4]) * f, __uint_as_float(r[pc][8 * c + 5]) * f);
          o.w = pack_bf16(__uint_as_float(r[pc][8 * c + 6]) * f, __uint_as_float(r[pc][8 * c + 7]) * f);
          reinterpret_cast<uint4*>(op)[c] = o;
        }
      }
    }
  };

  // ---- prologue --------------------------------------------------------------------------------
  // Y rows and C_n of the tile whose operands are prepared next; loaded a whole tile ahead so that the
  // DRAM latency never sits on the softmax threads' critical path
  uint4 yv_next = make_uint4(0, 0, 0, 0);
  float cb_next = 0.f;
  if (!is_issuer && !is_store) {
    fetch_y(0, yv_next, cb_next);
    mbar_wait(&bar_full[0], 0, a.status, abort_flag);
    prep_tile(0, yv_next, cb_next);
    if (n_tiles > 1) fetch_y(1, yv_next, cb_next);
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  if (is_issuer) {
    // the whole warp runs the issue code; one elected lane executes each TMA / MMA / commit
    mbar_wait(bar_q, 0, a.status, abort_flag);
    mbar_wait(&bar_full[0], 0, a.status, abort_flag);
    tc_fence_after();
    if (elect_one()) {
      issue_p1(0, 0, 0);
      if (U > 1) issue_p1(1, 0, 1);
      mma_commit(bar_pro);
    }
    __syncwarp();
  }

  if (a.prof && tid == 0 && blockIdx.x == 0) a.prof[12] = clock64() - k_c0;   // loop starts
  if (is_issuer) {
    // ================= issuer warp =================
    int t = 0, s = 0;                              // step u = (tile t, slice s), tracked without divisions
    for (int u = 0; u < U; ++u) {
      const int xb = u & 1;
      // token tile t+2 may be (re)loaded at slice 1 of tile t: every product that read its stage
      // (tile t-1) is complete once the commit of step u-2 has arrived
      if (s == 1 && t + 2 < n_tiles) {
        if (u >= 2) mbar_wait(&bar_c[xb], (uint32_t)((u >> 1) - 1) & 1, a.status, abort_flag);
        if (elect_one()) load_tile(t + 2);
        __syncwarp();
      }
      const long long i0 = (a.prof && lane == 0) ? clock64() : 0;
      mbar_wait(&bar_simt[xb], (uint32_t)(u >> 1) & 1, a.status, abort_flag);
      if (*reinterpret_cast<volatile int*>(abort_flag)) break;
      tc_fence_after();
      const long long i1 = (a.prof && lane == 0) ? clock64() : 0;
      int t2 = t, s2 = s + 2;                      // (tile, slice) of step u+2
      if (s2 >= n_sub) { s2 -= n_sub; ++t2; }
      if (s == 0 && t > 0) {
        // the dV/dK accumulators still hold tile t-1 until they have been read: run the independent
        // S^T/T' product first, read this warp's own lane quarter, wait for the three store warps,
        // then start this tile's accumulation and write the quarter out
        if (elect_one() && u + 2 < U) issue_p1(u + 2, t2, s2);
        __syncwarp();
        mbar_wait(bar_tile, (uint32_t)(t - 1) & 1, a.status, abort_flag);
        tc_fence_after();
        uint32_t r[4][16];
        read_dvdk(r);
        mbar_wait(bar_free, (uint32_t)(t - 1) & 1, a.status, abort_flag);
        tc_fence_after();
        if (elect_one()) {
          issue_p2(u, t, s);
          mma_commit(&bar_c[xb]);
        }
        __syncwarp();
        write_dvdk(t - 1, r);
      } else if (elect_one()) {
        issue_p2(u, t, s);
        if (u + 2 < U) issue_p1(u + 2, t2, s2);
        mma_commit(&bar_c[xb]);
        if (s == n_sub - 1) mma_commit(bar_tile);  // one phase per tile: the store warps follow it in order
      }
      __syncwarp();
      if (a.prof && lane == 0) {
        const long long i2 = clock64();
        atomicAdd((unsigned long long*)&a.prof[0], (unsigned long long)(i1 - i0));   // issuer waits for softmax
        atomicAdd((unsigned long long*)&a.prof[4], (unsigned long long)(i2 - i1));   // issue
      }
      if (++s == n_sub) { s = 0; ++t; }
    }
    if (!*reinterpret_cast<volatile int*>(abort_flag)) {   // this warp's quarter of the last tile
      mbar_wait(bar_tile, (uint32_t)(n_tiles - 1) & 1, a.status, abort_flag);
      tc_fence_after();
      uint32_t r[4][16];
      read_dvdk(r);
      write_dvdk(n_tiles - 1, r);
    }
  } else if (is_store) {
    // ================= store warps: dV/dK of every finished tile -> global =================
    for (int t = 0; t < n_tiles; ++t) {
      mbar_wait(bar_tile, (uint32_t)t & 1, a.status, abort_flag);
      if (*reinterpret_cast<volatile int*>(abort_flag)) break;
      tc_fence_after();
      uint32_t r[4][16];
      read_dvdk(r);
      mbar_arrive(bar_free);
      write_dvdk(t, r);
    }
  } else {
    // ================= softmax threads =================
    long long s_prev = 0;
    int t = 0, s = 0;                              // step u = (tile t, slice s), tracked without divisions
    for (int u = 0; u < U; ++u, s = (s + 1 == n_sub ? 0 : s + 1), t += (s == 0)) {
      const int xb = u & 1;
      // operands of the next tile are due when the product two steps ahead first belongs to it
      const int tau_p = t + 1;
      const bool do_prep = (s == n_sub - 2) && tau_p < n_tiles;

      const long long s0 = (a.prof && tid == 0) ? clock64() : 0;
      if (a.prof && tid == 0 && u > 0) atomicAdd((unsigned long long*)&a.prof[15], (unsigned long long)(s0 - s_prev));
      s_prev = s0;
      const long long sA = s0;
      (void)sA;
      if (u >= 2) mbar_wait(&bar_c[xb], (uint32_t)((u >> 1) - 1) & 1, a.status, abort_flag);
      else mbar_wait(bar_pro, 0, a.status, abort_flag);
      tc_fence_after();
      const long long s1 = (a.prof && tid == 0) ? clock64() : 0;

      // ---- P and dS = P * T' for this thread's token and its 16 latents of slice s --------------
      {
        const uint32_t cx = lane_base + cX + 128 * xb + 16 * g;
        const float* l2p = sL2 + s * 64 + 16 * g;
        uint32_t rs[16], rt[16];
        tmem_ld16(cx, rs);
        tmem_ld16(cx + 64, rt);
        float4 l4s[4];                             // L_m of the 16 latents: fetched while the loads are in flight
#pragma unroll
        for (int e = 0; e < 4; ++e) l4s[e] = *reinterpret_cast<const float4*>(l2p + 4 * e);
        tmem_wait_ld();
        uint32_t pp[8], pd[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float4 l4 = l4s[e];
          const float p0 = ex2(fmaf(__uint_as_float(rs[4 * e]), sl, -l4.x));
          const float p1 = ex2(fmaf(__uint_as_float(rs[4 * e + 1]), sl, -l4.y));
          const float p2 = ex2(fmaf(__uint_as_float(rs[4 * e + 2]), sl, -l4.z));
          const float p3 = ex2(fmaf(__uint_as_float(rs[4 * e + 3]), sl, -l4.w));
          pp[2 * e] = pack_bf16(p0, p1);
          pp[2 * e + 1] = pack_bf16(p2, p3);
          pd[2 * e] = pack_bf16(p0 * __uint_as_float(rt[4 * e]), p1 * __uint_as_float(rt[4 * e + 1]));
          pd[2 * e + 1] = pack_bf16(p2 * __uint_as_float(rt[4 * e + 2]), p3 * __uint_as_float(rt[4 * e + 3]));
        }
        const uint32_t cpd = lane_base + cPD + 64 * xb;
        tmem_st8(cpd + 8 * g, pp);
        tmem_st8(cpd + 32 + 8 * g, pd);
        uint8_t* ds_row = sDS + (s >> 1) * L::kDS + (s & 1) * (128 * 128);   // block s/2, 64-latent half s%2
        *reinterpret_cast<uint4*>(ds_row + swz_off<128>(row, 2 * g)) = make_uint4(pd[0], pd[1], pd[2], pd[3]);
        *reinterpret_cast<uint4*>(ds_row + swz_off<128>(row, 2 * g + 1)) = make_uint4(pd[4], pd[5], pd[6], pd[7]);
      }
      const long long s2 = (a.prof && tid == 0) ? clock64() : 0;
      if (do_prep) {
        mbar_wait(&bar_full[tau_p % 3], (uint32_t)(tau_p / 3) & 1, a.status, abort_flag);
        prep_tile(tau_p, yv_next, cb_next);
        if (tau_p + 1 < n_tiles) fetch_y(tau_p + 1, yv_next, cb_next);
      }
      const long long s3 = (a.prof && tid == 0) ? clock64() : 0;
      tmem_wait_st();
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(&bar_simt[xb]);
      if (a.prof && tid == 0) {
        const long long s4 = clock64();
        atomicAdd((unsigned long long*)&a.prof[1], (unsigned long long)(s1 - s0));   // softmax waits for products
        atomicAdd((unsigned long long*)&a.prof[2], (unsigned long long)(s2 - s1));   // softmax math
        atomicAdd((unsigned long long*)&a.prof[3], (unsigned long long)(s3 - s2));   // prep
        atomicAdd((unsigned long long*)&a.prof[6], (unsigned long long)(s4 - s3));   // store + drain
      }
      if (*reinterpret_cast<volatile int*>(abort_flag)) break;
    }

    if (a.prof && tid == 0 && blockIdx.x == 0) a.prof[10] = clock64() - k_c0;   // loop ends
    // ---- tail: last tile's dV/dK and the dQ partial ------------------------------------------------
    if (!*reinterpret_cast<volatile int*>(abort_flag)) {
      if (U >= 2) mbar_wait(&bar_c[(U - 2) & 1], (uint32_t)((U - 2) >> 1) & 1, a.status, abort_flag);
      mbar_wait(&bar_c[(U - 1) & 1], (uint32_t)((U - 1) >> 1) & 1, a.status, abort_flag);
      tc_fence_after();
      const int piece = g & 1;
      // dQ partial: latent block g/2, 16-column piece g%2
      const int j = g >> 1;
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
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc<512>(tmem);
  if (a.prof && tid == 0 && blockIdx.x == 0) {
    unsigned long long k_t1; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(k_t1));
    a.prof[13] = clock64() - k_c0; a.prof[14] = (long long)(k_t1 - k_t0);
  }
}

// ------------------------------------------------------------------------------------------
bool tc_bwd3_supported(const Ctx& c, int dtype) {
  return dtype == FLARE_BF16 && c.D == 32 && c.M > 128 && c.M <= 256 && c.N >= 1 && c.terms == FLARE_TERM_BOTH;
}

int tc_bwd3_launch(const Ctx& c, const void* q, const void* k, const void* v, const void* dy, const void* y,
                   const float* z32, const float* dz32, const float* lse_m, const float* lse_n, void* dk, void* dv,
                   float* dq_part, const float* mu, const int* flag, cudaStream_t st) {
  constexpr int D = 32;
  CUtensorMap tmQ, tmK, tmV, tmG;
  const uint64_t e = 2;
  const bool qb = c.qs[0] != 0;
  auto tokmap = [&](CUtensorMap* m, const void* p, const long long* s) {
    return make_tile_map(m, p, 1, D, (uint64_t)c.N, (uint64_t)c.H, (uint64_t)c.B, s[2] * e, s[1] * e,
                         (c.B > 1 ? s[0] : s[1] * c.H) * e, 128);
  };
  if (!make_tile_map(&tmQ, q, 1, D, (uint64_t)c.M, (uint64_t)c.H, (uint64_t)(qb ? c.B : 1), c.qs[2] * e, c.qs[1] * e,
                     (qb ? c.qs[0] : c.qs[1] * c.H) * e, 256) ||
      !tokmap(&tmK, k, c.ks) || !tokmap(&tmV, v, c.vs) || !tokmap(&tmG, dy, c.dys))
    return FLARE_EUNSUPPORTED;
  Bwd3Args a;
  a.B = c.B; a.H = c.H; a.N = c.N; a.M = c.M;
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
  a.prof = tc_phase_counters();
  static bool attr_done = false;
  constexpr int smem = Bwd3Smem::kBytes;
  if (!attr_done) {
    if (cudaFuncSetAttribute(k_tc_bwd3, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return FLARE_ECUDA;
    attr_done = true;
  }
  const long long grid = (long long)c.n_splits * c.B * c.H;
  if (grid > 0x7fffffffLL) return FLARE_EUNSUPPORTED;
  k_tc_bwd3<<<(unsigned)grid, kSoftmaxThreads + kStoreThreads + 32, smem, st>>>(tmQ, tmK, tmV, tmG, a);
  return FLARE_OK;
}

}  // namespace flare
