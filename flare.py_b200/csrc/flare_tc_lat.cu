// Latent-major split-N passes on tcgen05 tensor cores.
//
//   MODE 0  gather : record (acc, m, l) of z = softmax_N(S) v over one token range
//   MODE 1  dZ     : dz_part = sum_n exp(S_mn - C_n) dY_n over one token range
//
// One CTA (128 threads) owns 128 latents of one (b, h) and one token range and walks it in
// 128-token tiles.  Per tile:
//   TMA   : K tile and V (or dY) tile [128 x D] -> shared memory, two-stage ring
//   MMA S : S[128 lat x 128 tok] = Q_blk K_tile^T      (both K-major in shared memory)
//   SIMT  : thread t owns latent row t (= tensor-memory lane t).  MODE 0 keeps a running
//           maximum and sum per row; the accumulator in tensor memory is rescaled only when
//           the maximum grows by more than 2^8 (the weights stay well inside bf16/fp32 range).
//           MODE 1 subtracts the known per-token normaliser C_n.  One ex2 per score.  The bf16
//           weights are written over S, two per column.
//   MMA PV: acc[128 lat x D] += P[128 x 128] V_tile     (P from tensor memory, V MN-major)
// Tensor-memory columns: S of even tiles at [0,128) with P at [0,64); S of odd tiles at
// [64,192) with P at [128,192); accumulator at [192,192+D).  With this placement the S MMA of
// tile t+1 can be issued right behind the PV MMA of tile t (they touch disjoint columns), so
// one commit and one wait per tile suffice.  Two CTAs share an SM (256 columns each).
// Requires bf16, D in {16,32,64}; any M (blocks of 128 latents, rows past M are not stored).
#include "common.cuh"
#include "launch.h"
#include "tc_common.cuh"
#include "tma_host.h"

namespace flare {

using namespace tc;

struct LatArgs {
  int B, H, N, M;
  float scale_log2;
  int q_batched;
  int n_splits, chunk, n_mblk;
  const float* lse_n;          // MODE 1: [B,H,N]
  float* out;                  // MODE 0: rec [S,B,H,M,D+2]; MODE 1: dz_part [S,B,H,M,D]
  int* status;                 // device status word
};

template <int D>
struct LatSmem {
  static constexpr int ROWB = 2 * D;
  static constexpr int kQ = 128 * ROWB;
  static constexpr int kT = 128 * ROWB;            // one K or V tile
  static constexpr int kBytes = kQ + 4 * kT + 2 * 128 * 4 + 1024 + 128;
};

template <int D, int MODE>
__global__ void __launch_bounds__(128, 2)
k_tc_lat(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
         const __grid_constant__ CUtensorMap tmV, LatArgs a) {
  constexpr int ROWB = 2 * D;
  using L = LatSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + L::kQ;                        // [2]
  uint8_t* sV = sK + 2 * L::kT;                    // [2]
  float* sC2 = reinterpret_cast<float*>(sV + 2 * L::kT);   // [2][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sC2 + 256);
  uint64_t* bar_full = bars;                       // [2]
  uint64_t* bar_mma = bars + 2;
  uint64_t* bar_q = bars + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  int* abort_flag = reinterpret_cast<int*>(bars + 5);

  const int tid = threadIdx.x, warp = tid >> 5;
  // blockIdx.x = (bh * n_splits + split) * n_mblk + mblk : the latent blocks that read the same
  // K/V tiles are neighbours, so the second read of a tile comes from L2
  const int mblk = blockIdx.x % a.n_mblk;
  const int split = (blockIdx.x / a.n_mblk) % a.n_splits;
  const int bh = blockIdx.x / (a.n_splits * a.n_mblk);
  const int b = bh / a.H, h = bh % a.H;
  const int n0 = split * a.chunk, n1 = min(a.N, n0 + a.chunk);
  const int n_tiles = n1 > n0 ? (n1 - n0 + 127) / 128 : 0;
  const int lat = mblk * 128 + tid;

  constexpr int W = (MODE == 0) ? D + 2 : D;
  float* orow = a.out + ((((long long)split * a.B + b) * a.H + h) * a.M + lat) * W;

  if (n_tiles == 0) {                              // empty range: the neutral record
    if (lat < a.M) {
      for (int i = 0; i < D; ++i) orow[i] = 0.f;
      if (MODE == 0) { orow[D] = -INFINITY; orow[D + 1] = 0.f; }
    }
    return;
  }

  if (tid == 0) {
    mbar_init(&bar_full[0], 1); mbar_init(&bar_full[1], 1);
    mbar_init(bar_mma, 1); mbar_init(bar_q, 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
  }
  if (warp == 0) tmem_alloc<256>(tmem_slot);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
  constexpr uint32_t kAcc = 192;

  const uint32_t idesc_s = idesc_f16(128, 128, 1, 1, 0, 0);
  const uint32_t idesc_pv = idesc_f16(128, D, 1, 1, 0, 1);

  if (tid == 0) {
    mbar_expect_tx(bar_q, L::kQ);
    tma_load_4d(sQ, &tmQ, bar_q, 0, mblk * 128, h, a.q_batched ? b : 0);
    mbar_expect_tx(&bar_full[0], 2 * L::kT);
    tma_load_4d(sK, &tmK, &bar_full[0], 0, n0, h, b);
    tma_load_4d(sV, &tmV, &bar_full[0], 0, n0, h, b);
    mbar_wait(bar_q, 0, a.status, abort_flag);
    mbar_wait(&bar_full[0], 0, a.status, abort_flag);
    tc_fence_after();
    const uint64_t dq = smem_desc<ROWB>(smem_u32(sQ));
    const uint64_t dk = smem_desc<ROWB>(smem_u32(sK));
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) mma_ss(tmem, dq + 2 * kk, dk + 2 * kk, idesc_s, kk > 0);
    mma_commit(bar_mma);
  }

  const float sl = a.scale_log2;
  float m_run = -INFINITY, l_run = 0.f;
  uint32_t ph_mma = 0;
  bool aborted = false;
  const float* cb = (MODE == 1) ? a.lse_n + ((long long)b * a.H + h) * a.N : nullptr;

  for (int t = 0; t < n_tiles; ++t) {
    const int st = t & 1;
    const int tile0 = n0 + t * 128;
    const int cnt = min(128, n1 - tile0);
    if (MODE == 1) {
      const int n = tile0 + tid;
      sC2[st * 128 + tid] = (tid < cnt) ? cb[n] * kLog2e : INFINITY;
    }
    mbar_wait(bar_mma, ph_mma, a.status, abort_flag);
    ph_mma ^= 1;
    tc_fence_after();
    if (tid == 0 && t + 1 < n_tiles) {             // stage st^1 is free: S(t) and PV(t-1) are complete
      mbar_expect_tx(&bar_full[st ^ 1], 2 * L::kT);
      tma_load_4d(sK + (st ^ 1) * L::kT, &tmK, &bar_full[st ^ 1], 0, tile0 + 128, h, b);
      tma_load_4d(sV + (st ^ 1) * L::kT, &tmV, &bar_full[st ^ 1], 0, tile0 + 128, h, b);
    }
    __syncthreads();

    const uint32_t s_base = lane_base + (st ? 64 : 0);
    const uint32_t p_base = lane_base + (st ? 128 : 0);

    if (MODE == 0) {
      // running maximum; rescale only on the first tile or when it grew by more than 2^8
      float tmax = -INFINITY;
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(s_base + c * 32, r);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float x = __uint_as_float(r[j]);
          tmax = fmaxf(tmax, (c * 32 + j < cnt) ? x : -INFINITY);
        }
      }
      tmax *= sl;
      const bool grow = tmax > m_run + 8.f;
      if (__any_sync(0xffffffffu, grow) && t > 0) {
        const float f = grow ? ex2(m_run - tmax) : 1.f;    // ex2(-inf) = 0 on the first non-empty tile
        uint32_t r[D];
        if constexpr (D == 16) tmem_ld16(lane_base + kAcc, r);
        else {
#pragma unroll
          for (int c = 0; c < D / 32; ++c) tmem_ld32(lane_base + kAcc + c * 32, r + c * 32);
        }
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < D; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * f);
        if constexpr (D == 16) tmem_st16(lane_base + kAcc, r);
        else {
#pragma unroll
          for (int c = 0; c < D / 32; ++c) tmem_st32(lane_base + kAcc + c * 32, r + c * 32);
        }
        l_run *= f;
      }
      if (grow) m_run = tmax;
    }

    // one exponential per score; weights packed two per column over S
    float lsum = 0.f;
    for (int cc = 0; cc < 4; ++cc) {
      const int c = st ? 3 - cc : cc;              // odd tiles fill P from the top down
      uint32_t r[32], pk[16];
      tmem_ld32(s_base + c * 32, r);
      tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float x0, x1;
        if (MODE == 0) {
          x0 = fmaf(__uint_as_float(r[2 * j]), sl, -m_run);
          x1 = fmaf(__uint_as_float(r[2 * j + 1]), sl, -m_run);
        } else {
          const float2 cc2 = *reinterpret_cast<const float2*>(&sC2[st * 128 + c * 32 + 2 * j]);
          x0 = fmaf(__uint_as_float(r[2 * j]), sl, -cc2.x);
          x1 = fmaf(__uint_as_float(r[2 * j + 1]), sl, -cc2.y);
        }
        float e0 = ex2(x0), e1 = ex2(x1);
        if (MODE == 0 && cnt < 128) {
          if (c * 32 + 2 * j >= cnt) e0 = 0.f;
          if (c * 32 + 2 * j + 1 >= cnt) e1 = 0.f;
        }
        lsum += e0 + e1;
        pk[j] = pack_bf16(e0, e1);
      }
      tmem_st16(p_base + c * 16, pk);
    }
    l_run += lsum;
    tmem_wait_st();
    tc_fence_before();
    __syncthreads();
    aborted = *reinterpret_cast<volatile int*>(abort_flag) != 0;

    if (tid == 0 && !aborted) {
      tc_fence_after();
      const uint64_t dv = smem_desc<ROWB>(smem_u32(sV + st * L::kT));
      const uint32_t pa = tmem + (st ? 128 : 0);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        mma_ts(tmem + kAcc, pa + kk * 8, dv + (uint64_t)((kk * 16 * ROWB) >> 4), idesc_pv, (t > 0) || (kk > 0));
      if (t + 1 < n_tiles) {
        mbar_wait(&bar_full[st ^ 1], (uint32_t)((t + 1) >> 1) & 1, a.status, abort_flag);
        tc_fence_after();
        const uint64_t dq = smem_desc<ROWB>(smem_u32(sQ));
        const uint64_t dk = smem_desc<ROWB>(smem_u32(sK + (st ^ 1) * L::kT));
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_ss(tmem + (st ? 0 : 64), dq + 2 * kk, dk + 2 * kk, idesc_s, kk > 0);
      }
      mma_commit(bar_mma);
    }
    if (aborted) break;
  }

  if (!aborted) mbar_wait(bar_mma, ph_mma, a.status, abort_flag);
  tc_fence_after();
  {
    uint32_t r[D];
    if constexpr (D == 16) tmem_ld16(lane_base + kAcc, r);
    else {
#pragma unroll
      for (int c = 0; c < D / 32; ++c) tmem_ld32(lane_base + kAcc + c * 32, r + c * 32);
    }
    tmem_wait_ld();
    if (lat < a.M) {
#pragma unroll
      for (int j = 0; j < D / 4; ++j) {
        if constexpr (MODE == 1) {
          reinterpret_cast<float4*>(orow)[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                           __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
        } else {                                   // rows of D+2 floats are only 8-byte aligned
          reinterpret_cast<float2*>(orow)[2 * j] = make_float2(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]));
          reinterpret_cast<float2*>(orow)[2 * j + 1] = make_float2(__uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
        }
      }
      if (MODE == 0) { orow[D] = m_run * kLn2; orow[D + 1] = l_run; }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc<256>(tmem);
}

// ------------------------------------------------------------------------------------------
bool tc_lat_supported(const Ctx& c, int dtype) {
  return dtype == FLARE_BF16 && (c.D == 16 || c.D == 32 || c.D == 64) && c.N >= 1 && c.M >= 1;
}

template <int D, int MODE>
static int launch_lat(const Ctx& c, const void* q, const void* k, const void* v, const float* lse_n, float* out,
                      cudaStream_t st) {
  CUtensorMap tmQ, tmK, tmV;
  const uint64_t e = 2;
  const bool qb = c.qs[0] != 0;
  const long long* vs = (MODE == 0) ? c.vs : c.dys;
  if (!make_tile_map(&tmQ, q, 1, D, (uint64_t)c.M, (uint64_t)c.H, (uint64_t)(qb ? c.B : 1), c.qs[2] * e, c.qs[1] * e,
                     (qb ? c.qs[0] : c.qs[1] * c.H) * e, 128) ||
      !make_tile_map(&tmK, k, 1, D, (uint64_t)c.N, (uint64_t)c.H, (uint64_t)c.B, c.ks[2] * e, c.ks[1] * e,
                     (c.B > 1 ? c.ks[0] : c.ks[1] * c.H) * e, 128) ||
      !make_tile_map(&tmV, v, 1, D, (uint64_t)c.N, (uint64_t)c.H, (uint64_t)c.B, vs[2] * e, vs[1] * e,
                     (c.B > 1 ? vs[0] : vs[1] * c.H) * e, 128))
    return FLARE_EUNSUPPORTED;
  LatArgs a;
  a.B = c.B; a.H = c.H; a.N = c.N; a.M = c.M;
  a.scale_log2 = c.scale * kLog2e;
  a.q_batched = qb ? 1 : 0;
  a.n_splits = c.n_splits; a.chunk = c.chunk; a.n_mblk = (c.M + 127) / 128;
  a.lse_n = lse_n; a.out = out;
  a.status = tc_status_ptr();
  constexpr int smem = LatSmem<D>::kBytes;
  if (tc_set_dyn_smem(reinterpret_cast<const void*>(&k_tc_lat<D, MODE>), smem) != FLARE_OK) return FLARE_ECUDA;
  const long long grid = (long long)c.n_splits * a.n_mblk * c.B * c.H;
  if (grid > 0x7fffffffLL) return FLARE_EUNSUPPORTED;
  k_tc_lat<D, MODE><<<(unsigned)grid, 128, smem, st>>>(tmQ, tmK, tmV, a);
  return FLARE_OK;
}

int tc_gather_partial(const Ctx& c, const void* q, const void* k, const void* v, float* rec, cudaStream_t st) {
  switch (c.D) {
    case 16: return launch_lat<16, 0>(c, q, k, v, nullptr, rec, st);
    case 32: return launch_lat<32, 0>(c, q, k, v, nullptr, rec, st);
    case 64: return launch_lat<64, 0>(c, q, k, v, nullptr, rec, st);
  }
  return FLARE_EUNSUPPORTED;
}

int tc_dz_partial(const Ctx& c, const void* q, const void* k, const void* dy, const float* lse_n, float* dz_part,
                  cudaStream_t st) {
  switch (c.D) {
    case 16: return launch_lat<16, 1>(c, q, k, dy, lse_n, dz_part, st);
    case 32: return launch_lat<32, 1>(c, q, k, dy, lse_n, dz_part, st);
    case 64: return launch_lat<64, 1>(c, q, k, dy, lse_n, dz_part, st);
  }
  return FLARE_EUNSUPPORTED;
}

}  // namespace flare
