// Scatter pass on tcgen05 tensor cores:  y_n = softmax_M(S[:, n]) z,  C_n = logsumexp_m S_mn.
//
// One CTA (128 threads) owns a contiguous run of 128-token tiles.  Per tile:
//   TMA   : K tile [128 x D] -> shared memory (two-stage ring, next tile prefetched)
//   MMA 1 : S^T[128 x M] = K_tile Q^T              (both operands K-major in shared memory,
//                                                    fp32 accumulator in tensor memory cols [0, M))
//   SIMT  : thread t owns token row t (= tensor-memory lane t): exact row max, one ex2 per score,
//           row sum; the bf16 weights are written back over S (cols [0, M/2), two per column)
//   MMA 2 : Y[128 x D] = A^T[128 x M] Z[M x D]      (A from tensor memory, Z MN-major in shared
//                                                    memory, accumulator in cols [128, 128 + D))
//   SIMT  : y = Y / rowsum -> global, C_n -> global
// The steps of one tile run back to back; two CTAs share an SM (256 tensor-memory columns
// each) so that one CTA's exponentials overlap the other's MMAs, loads and stores.
// The N x M map never leaves the SM.  Requires bf16, M a multiple of 32 in [32, 256],
// D in {16, 32, 64}.
#include "common.cuh"
#include "launch.h"
#include "tc_common.cuh"
#include "tma_host.h"

namespace flare {

using namespace tc;


struct ScatterArgs {
  int B, H, N, M;
  float scale_log2;            // scale * log2(e)
  int q_batched;
  const float* z32;            // [B,H,M,D]
  const uint8_t* mask;         // [B,N] or null
  __nv_bfloat16* y;
  long long ys[3];
  float* lse_n;                // [B,H,N] or null
  int tiles_per_bh;
  long long total_tiles;
  int* status;                 // device status word
};

template <int D>
struct ScatterSmem {
  static constexpr int ROWB = 2 * D;
  static constexpr int kQ = 256 * ROWB;
  static constexpr int kZ = 256 * ROWB;
  static constexpr int kK = 128 * ROWB;
  static constexpr int kBytes = kQ + kZ + 2 * kK + 1024 /*alignment slack*/ + 128 /*barriers*/;
};

template <int D>
__global__ void __launch_bounds__(128, 2)
k_tc_scatter(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmQ, ScatterArgs a) {
  constexpr int ROWB = 2 * D;
  using L = ScatterSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sZ = sQ + L::kQ;
  uint8_t* sK = sZ + L::kZ;                       // two stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(sK + 2 * L::kK);
  uint64_t* bar_full = bars;                      // [2]
  uint64_t* bar_mma = bars + 2;
  uint64_t* bar_q = bars + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  int* abort_flag = reinterpret_cast<int*>(bars + 5);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int M = a.M;

  if (tid == 0) {
    mbar_init(&bar_full[0], 1); mbar_init(&bar_full[1], 1);
    mbar_init(bar_mma, 1); mbar_init(bar_q, 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmK); prefetch_tmap(&tmQ);
  }
  if (warp == 0) tmem_alloc<256>(tmem_slot);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);

  const long long per = (a.total_tiles + gridDim.x - 1) / gridDim.x;
  const long long t_begin = (long long)blockIdx.x * per;
  const long long t_end = min(a.total_tiles, t_begin + per);

  const uint32_t idesc1 = idesc_f16(128, M, 1, 1, 0, 0);
  const uint32_t idesc2 = idesc_f16(128, D, 1, 1, 0, 1);
  uint32_t ph_mma = 0, ph_q = 0;
  int cur_bh = -1;

  if (tid == 0 && t_begin < t_end) {
    const int bh = (int)(t_begin / a.tiles_per_bh), tile = (int)(t_begin % a.tiles_per_bh);
    mbar_expect_tx(&bar_full[0], L::kK);
    tma_load_4d(sK, &tmK, &bar_full[0], 0, tile * 128, bh % a.H, bh / a.H);
  }

  for (long long t = t_begin; t < t_end; ++t) {
    const int it = (int)(t - t_begin), stage = it & 1;
    const int bh = (int)(t / a.tiles_per_bh), tile = (int)(t % a.tiles_per_bh);
    const int b = bh / a.H, h = bh % a.H;

    if (bh != cur_bh) {
      // latents of this (b, h): Q by TMA, Z converted to bf16 into the swizzled operand layout
      if (tid == 0) {
        mbar_expect_tx(bar_q, (uint32_t)M * ROWB);
        tma_load_4d(sQ, &tmQ, bar_q, 0, 0, h, a.q_batched ? b : 0);
      }
      const float* zb = a.z32 + ((long long)b * a.H + h) * M * D;
      constexpr int CPR = ROWB / 16;               // 16-byte chunks per row
      for (int i = tid; i < M * CPR; i += 128) {
        const int r = i / CPR, c = i % CPR;
        const float4 lo = *reinterpret_cast<const float4*>(zb + r * D + c * 8);
        const float4 hi = *reinterpret_cast<const float4*>(zb + r * D + c * 8 + 4);
        uint4 pk;
        pk.x = pack_bf16(lo.x, lo.y); pk.y = pack_bf16(lo.z, lo.w);
        pk.z = pack_bf16(hi.x, hi.y); pk.w = pack_bf16(hi.z, hi.w);
        *reinterpret_cast<uint4*>(sZ + swz_off<ROWB>(r, c)) = pk;
      }
      fence_proxy_async();
      __syncthreads();
      mbar_wait(bar_q, ph_q, a.status, abort_flag);
      ph_q ^= 1;
      cur_bh = bh;
    }

    if (tid == 0 && t + 1 < t_end) {              // prefetch the next K tile into the other stage
      const int nbh = (int)((t + 1) / a.tiles_per_bh), ntile = (int)((t + 1) % a.tiles_per_bh);
      mbar_expect_tx(&bar_full[stage ^ 1], L::kK);
      tma_load_4d(sK + (stage ^ 1) * L::kK, &tmK, &bar_full[stage ^ 1], 0, ntile * 128, nbh % a.H, nbh / a.H);
    }
    mbar_wait(&bar_full[stage], (uint32_t)(it >> 1) & 1, a.status, abort_flag);

    if (tid == 0) {
      tc_fence_after();
      const uint64_t dk = smem_desc<ROWB>(smem_u32(sK + stage * L::kK));
      const uint64_t dq = smem_desc<ROWB>(smem_u32(sQ));
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) mma_ss(tmem, dk + 2 * kk, dq + 2 * kk, idesc1, kk > 0);
      mma_commit(bar_mma);
    }
    mbar_wait(bar_mma, ph_mma, a.status, abort_flag);
    ph_mma ^= 1;
    tc_fence_after();

    // ---- softmax over the M latents of this thread's token --------------------------------
    float mx = -INFINITY;
    for (int c = 0; c < M / 32; ++c) {
      uint32_t r[32];
      tmem_ld32(lane_base + c * 32, r);
      tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 32; ++j) mx = fmaxf(mx, __uint_as_float(r[j]));
    }
    const float sl = a.scale_log2, off = -mx * sl;
    float sum = 0.f;
    for (int c = 0; c < M / 32; ++c) {
      uint32_t r[32], pk[16];
      tmem_ld32(lane_base + c * 32, r);
      tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float e0 = ex2(fmaf(__uint_as_float(r[2 * j]), sl, off));
        const float e1 = ex2(fmaf(__uint_as_float(r[2 * j + 1]), sl, off));
        sum += e0 + e1;
        pk[j] = pack_bf16(e0, e1);
      }
      tmem_st16(lane_base + c * 16, pk);
    }
    tmem_wait_st();
    tc_fence_before();
    __syncthreads();

    if (tid == 0) {
      tc_fence_after();
      const uint64_t dz = smem_desc<ROWB>(smem_u32(sZ));
      for (int kk = 0; kk < M / 16; ++kk)
        mma_ts(tmem + 128, tmem + kk * 8, dz + (uint64_t)((kk * 16 * ROWB) >> 4), idesc2, kk > 0);
      mma_commit(bar_mma);
    }
    mbar_wait(bar_mma, ph_mma, a.status, abort_flag);
    ph_mma ^= 1;
    tc_fence_after();

    // ---- epilogue ---------------------------------------------------------------------------
    {
      const int tok = tile * 128 + tid;
      uint32_t r[D];
      if constexpr (D == 16) tmem_ld16(lane_base + 128, r);
      else {
#pragma unroll
        for (int c = 0; c < D / 32; ++c) tmem_ld32(lane_base + 128 + c * 32, r + c * 32);
      }
      tmem_wait_ld();
      if (tok < a.N) {
        const bool keep = !a.mask || a.mask[(long long)b * a.N + tok];
        const float inv = keep ? 1.f / sum : 0.f;
        __nv_bfloat16* yp = a.y + b * a.ys[0] + h * a.ys[1] + (long long)tok * a.ys[2];
#pragma unroll
        for (int c = 0; c < D / 8; ++c) {
          uint4 o;
          o.x = pack_bf16(__uint_as_float(r[8 * c]) * inv, __uint_as_float(r[8 * c + 1]) * inv);
          o.y = pack_bf16(__uint_as_float(r[8 * c + 2]) * inv, __uint_as_float(r[8 * c + 3]) * inv);
          o.z = pack_bf16(__uint_as_float(r[8 * c + 4]) * inv, __uint_as_float(r[8 * c + 5]) * inv);
          o.w = pack_bf16(__uint_as_float(r[8 * c + 6]) * inv, __uint_as_float(r[8 * c + 7]) * inv);
          reinterpret_cast<uint4*>(yp)[c] = o;
        }
        if (a.lse_n) a.lse_n[((long long)b * a.H + h) * a.N + tok] = (mx * sl + log2f(sum)) * kLn2;
      }
    }
    tc_fence_before();
    __syncthreads();
    if (*reinterpret_cast<volatile int*>(abort_flag)) break;
  }

  __syncthreads();
  if (warp == 0) tmem_dealloc<256>(tmem);
}

// ------------------------------------------------------------------------------------------
bool tc_scatter_supported(const Ctx& c, int dtype) {
  return dtype == FLARE_BF16 && (c.D == 16 || c.D == 32 || c.D == 64) && c.M >= 32 && c.M <= 256 &&
         c.M % 32 == 0 && c.N >= 1;
}

template <int D>
static int launch_scatter_d(const Ctx& c, const void* q, const void* k, const float* z32, const uint8_t* mask,
                            void* y, float* lse_n, cudaStream_t st) {
  CUtensorMap tmK, tmQ;
  const uint64_t e = 2;
  if (!make_tile_map(&tmK, k, 1, D, (uint64_t)c.N, (uint64_t)c.H, (uint64_t)c.B, c.ks[2] * e, c.ks[1] * e,
                     (c.B > 1 ? c.ks[0] : c.ks[1] * c.H) * e, 128))
    return FLARE_EUNSUPPORTED;
  const bool qb = c.qs[0] != 0;
  if (!make_tile_map(&tmQ, q, 1, D, (uint64_t)c.M, (uint64_t)c.H, (uint64_t)(qb ? c.B : 1), c.qs[2] * e,
                     c.qs[1] * e, (qb ? c.qs[0] : c.qs[1] * c.H) * e, (uint32_t)c.M))
    return FLARE_EUNSUPPORTED;
  ScatterArgs a;
  a.B = c.B; a.H = c.H; a.N = c.N; a.M = c.M;
  a.scale_log2 = c.scale * kLog2e;
  a.q_batched = qb ? 1 : 0;
  a.z32 = z32; a.mask = mask; a.y = reinterpret_cast<__nv_bfloat16*>(y);
  for (int i = 0; i < 3; ++i) a.ys[i] = c.ys[i];
  a.lse_n = lse_n;
  a.tiles_per_bh = (c.N + 127) / 128;
  a.total_tiles = (long long)a.tiles_per_bh * c.B * c.H;
  a.status = tc_status_ptr();
  constexpr int smem = ScatterSmem<D>::kBytes;
  if (tc_set_dyn_smem(reinterpret_cast<const void*>(&k_tc_scatter<D>), smem) != FLARE_OK) return FLARE_ECUDA;
  long long grid = 2LL * num_sms();
  if (grid > a.total_tiles) grid = a.total_tiles;
  k_tc_scatter<D><<<(unsigned)grid, 128, smem, st>>>(tmK, tmQ, a);
  return FLARE_OK;
}

int tc_scatter(const Ctx& c, const void* q, const void* k, const float* z32, const uint8_t* mask, void* y,
               float* lse_n, cudaStream_t st) {
  switch (c.D) {
    case 16: return launch_scatter_d<16>(c, q, k, z32, mask, y, lse_n, st);
    case 32: return launch_scatter_d<32>(c, q, k, z32, mask, y, lse_n, st);
    case 64: return launch_scatter_d<64>(c, q, k, z32, mask, y, lse_n, st);
  }
  return FLARE_EUNSUPPORTED;
}

}  // namespace flare
