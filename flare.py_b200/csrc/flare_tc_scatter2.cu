// Scatter pass on tcgen05 tensor cores, decoupled schedule:  y_n = softmax_M(S[:, n]) z,  C_n = lse_m S_mn.
//
// Same mathematics as flare_tc_scatter.cu; one CTA per SM owns one (b, h) and one token range, walks it
// in 128-token tiles and keeps two tiles in flight in the two halves of tensor memory:
//
//   issuer warp   : S^T(t) = K_t Q^T into buffer t&1 (as soon as the buffer's previous tile has been
//                   written out), Y(t) = A^T(t) Z once the softmax threads have packed A^T(t)
//   512 softmax   : two groups of 256 take alternate tiles, so one group's row-max pass overlaps the
//   threads         other's exponentials; two threads per token row, 128 latent columns each: row max
//                   (the two meet through shared memory), one ex2 per score, partial row sums, A^T
//                   packed to bf16 inside the thread's own score columns
//   4 epilogue    : one thread per token row: waits for Y(t), frees the buffer, divides by the row sum
//   warps           and stores y and C_n
// so the tensor core works on tile t+1 and the epilogue on tile t-1 while the exponentials of tile t
// run.  Buffer layout (256 columns): S^T at [0, M); half hf of a row packs A^T at [128hf, 128hf+64); Y goes
// to [64, 64+D), columns of half 0 that are dead by then.  K tiles arrive in a three-stage TMA ring.
// Requires bf16 or fp16, D in {16, 32}, M a multiple of 32 in [32, 256] per launch (more latents: blocks of 256).
#include "common.cuh"
#include "launch.h"
#include "tc_common.cuh"
#include "tma_host.h"

namespace flare {

using namespace tc;

struct Scatter2Args {
  int B, H, N, M;
  float scale_log2;
  int q_batched;
  int n_splits, chunk;
  const float* z32;            // [B,H,M,D]
  const uint8_t* mask;         // [B,N] or null
  void* y;                     // 16-bit rows
  long long ys[3];
  float* lse_n;                // [B,H,N] or null
  long long z_bh_stride;       // floats between the z32 blocks of consecutive (b, h)
  int accumulate;              // 1: merge with the y / lse_n a previous latent block left (log-sum-exp weights)
  int m0, M_total;             // this launch covers latents [m0, m0 + M) of M_total
  DropArgs drop;               // attention dropout of the scatter weights A
  int* status;
};

template <int D>
struct Scatter2Smem {
  static constexpr int ROWB = 2 * D;
  static constexpr int kQ = 256 * ROWB;
  static constexpr int kZ = 256 * ROWB;
  static constexpr int kK = 128 * ROWB;
  static constexpr int kBytes = kQ + kZ + 3 * kK + (2 * 4 * 128 + 2 * 4 * 128 + 2 * 128 + 16) * 4 + 1024 + 256;
};

__device__ __forceinline__ void mbar_arrive_s2(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void named_bar_sync_s2(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

constexpr int kS2Softmax = 512, kS2Epilogue = 128;

template <int D, typename T16, bool DROP>
__global__ void __launch_bounds__(kS2Softmax + kS2Epilogue + 32, 1)
k_tc_scatter2(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmQ, Scatter2Args a) {
  grid_dep_sync();
  constexpr int ROWB = 2 * D;
  using L = Scatter2Smem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sZ = sQ + L::kQ;
  uint8_t* sK = sZ + L::kZ;                        // [3]
  float* sMaxQ = reinterpret_cast<float*>(sK + 3 * L::kK);   // [2][4][128] quarter-row maxima
  float* sSum = sMaxQ + 2 * 4 * 128;               // [2][4][128] quarter-row sums
  float* sRowMax = sSum + 2 * 4 * 128;             // [2][128]
  float* sQmax = sRowMax + 2 * 128;                // [16] per-warp max |q_m|^2
  uint64_t* bars = reinterpret_cast<uint64_t*>(sQmax + 16);
  uint64_t* bar_full = bars;                       // [3]
  uint64_t* bar_s = bars + 3;                      // [2] S^T(t) complete
  uint64_t* bar_sm = bars + 5;                     // [2] softmax(t) done (512 arrivals)
  uint64_t* bar_pv = bars + 7;                     // [2] Y(t) complete
  uint64_t* bar_ep = bars + 9;                     // [2] buffer of tile t free (128 arrivals)
  uint64_t* bar_q = bars + 11;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  int* abort_flag = reinterpret_cast<int*>(bars + 13);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int role = warp < 16 ? 0 : (warp < 20 ? 1 : 2);      // softmax, epilogue, issuer
  const int row = (warp & 3) * 32 + lane;          // token within the tile = tensor-memory lane
  const int split = blockIdx.x % a.n_splits;
  const int bh = blockIdx.x / a.n_splits;
  const int b = bh / a.H, h = bh % a.H;
  const int M = a.M;
  const int n0 = split * a.chunk, n1 = min(a.N, n0 + a.chunk);
  const int T = n1 > n0 ? (n1 - n0 + 127) / 128 : 0;
  if (T == 0) return;

  if (tid == 0) {
    for (int i = 0; i < 3; ++i) mbar_init(&bar_full[i], 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_s[i], 1); mbar_init(&bar_sm[i], kS2Softmax / 2);
      mbar_init(&bar_pv[i], 1); mbar_init(&bar_ep[i], kS2Epilogue);
    }
    mbar_init(bar_q, 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmK); prefetch_tmap(&tmQ);
  }
  if (warp == 0) tmem_alloc<512>(tmem_slot);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
  constexpr uint32_t kY = 64;                      // Y columns inside a buffer

  // Q and the first K tiles are on their way while Z is converted
  if (tid == 0) {
    mbar_expect_tx(bar_q, (uint32_t)M * ROWB);
    tma_load_4d(sQ, &tmQ, bar_q, 0, 0, h, a.q_batched ? b : 0);
    for (int t = 0; t < 3 && t < T; ++t) {
      mbar_expect_tx(&bar_full[t], L::kK);
      tma_load_4d(sK + t * L::kK, &tmK, &bar_full[t], 0, n0 + t * 128, h, b);
    }
  }
  // Z of this (b, h) as bf16 in the swizzled operand layout (rows past M are never read)
  {
    const float* zb = a.z32 + ((long long)b * a.H + h) * a.z_bh_stride;
    constexpr int CPR = ROWB / 16;
    for (int i = tid; i < M * CPR; i += blockDim.x) {
      const int r = i / CPR, c = i % CPR;
      const float4 lo = *reinterpret_cast<const float4*>(zb + r * D + c * 8);
      const float4 hi = *reinterpret_cast<const float4*>(zb + r * D + c * 8 + 4);
      uint4 pk;
      pk.x = Op16<T16>::pack(lo.x, lo.y); pk.y = Op16<T16>::pack(lo.z, lo.w);
      pk.z = Op16<T16>::pack(hi.x, hi.y); pk.w = Op16<T16>::pack(hi.z, hi.w);
      *reinterpret_cast<uint4*>(sZ + swz_off<ROWB>(r, c)) = pk;
    }
  }
  fence_proxy_async();
  __syncthreads();

  if (role == 2) {
    // ================================ issuer warp ================================
    // The whole warp runs this code; one elected lane executes each TMA / MMA / commit.
    {
      constexpr int F = Op16<T16>::kFmt;
      const uint32_t idesc1 = idesc_f16(128, M, F, F, 0, 0);
      const uint32_t idesc2 = idesc_f16(128, D, F, F, 0, 1);
      const uint64_t dq = smem_desc<ROWB>(smem_u32(sQ));
      const uint64_t dz = smem_desc<ROWB>(smem_u32(sZ));
      const int ksteps = M / 16;
      auto load_tile = [&](int t) {
        const int st = t % 3;
        mbar_expect_tx(&bar_full[st], L::kK);
        tma_load_4d(sK + st * L::kK, &tmK, &bar_full[st], 0, n0 + t * 128, h, b);
      };
      auto issue_s = [&](int t) {
        mbar_wait(&bar_full[t % 3], (uint32_t)(t / 3) & 1, a.status, abort_flag);
        tc_fence_after();
        const uint64_t dk = smem_desc<ROWB>(smem_u32(sK + (t % 3) * L::kK));
        const uint32_t xb = tmem + 256 * (t & 1);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) mma_ss(xb, dk + 2 * kk, dq + 2 * kk, idesc1, kk > 0);
          mma_commit(&bar_s[t & 1]);
        }
        __syncwarp();
      };
      mbar_wait(bar_q, 0, a.status, abort_flag);
      issue_s(0);
      if (T > 1) issue_s(1);
      for (int t = 0; t < T; ++t) {
        const int p = t & 1;
        mbar_wait(&bar_sm[p], (uint32_t)(t >> 1) & 1, a.status, abort_flag);       // A^T(t) packed
        if (*reinterpret_cast<volatile int*>(abort_flag)) break;
        if (t + 3 < T && elect_one()) load_tile(t + 3);   // stage of tile t: S^T(t) has been consumed
        __syncwarp();
        tc_fence_after();
        const uint32_t xb = tmem + 256 * p;
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 16; ++kk)
            if (kk < ksteps)
              mma_ts(xb + kY, xb + 128 * (kk >> 3) + 8 * (kk & 7), dz + (uint64_t)((kk * 16 * ROWB) >> 4), idesc2, kk > 0);
          mma_commit(&bar_pv[p]);
        }
        __syncwarp();
        if (t + 2 < T) {
          mbar_wait(&bar_ep[p], (uint32_t)(t >> 1) & 1, a.status, abort_flag);     // Y(t) has been read
          issue_s(t + 2);
        }
      }
    }
    __syncwarp();
  } else if (role == 0) {
    // ================================ softmax threads ================================
    // Two groups of 256 threads take alternate tiles (group = tile parity = buffer), so one group's
    // row-max pass overlaps the other group's exponentials.  Inside a group two threads share a
    // token row: latent columns [128*hf, 128*hf + 128) each.
    const int grp = warp >> 3;                     // tile parity served by this thread
    const int hf = (warp >> 2) & 1;
    const int nv = max(0, min(128, M - 128 * hf)); // valid columns of this half: multiple of 32
    const float sl = a.scale_log2;
    const uint32_t cols = lane_base + 256 * grp + 128 * hf;
    // max_m |q_m| sl over the latents of this launch (every softmax thread computes it: 2 rows each, then
    // through shared memory)
    float qmax_sl;
    {
      mbar_wait(bar_q, 0, a.status, abort_flag);
      float mx2 = 0.f;
      for (int r = tid; r < M; r += kS2Softmax) {
        float q2 = 0.f;
#pragma unroll
        for (int c = 0; c < ROWB / 16; ++c) {
          const uint4 q4 = *reinterpret_cast<const uint4*>(sQ + swz_off<ROWB>(r, c));
          const uint32_t* qp = reinterpret_cast<const uint32_t*>(&q4);
#pragma unroll
          for (int j = 0; j < 4; ++j) { const float2 f = Op16<T16>::unpack(qp[j]); q2 = fmaf(f.x, f.x, q2); q2 = fmaf(f.y, f.y, q2); }
        }
        mx2 = fmaxf(mx2, q2);
      }
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) mx2 = fmaxf(mx2, __shfl_xor_sync(0xffffffffu, mx2, o));
      if (lane == 0) sQmax[warp] = mx2;
      named_bar_sync_s2(9, kS2Softmax);
      float m = 0.f;
      for (int w = 0; w < kS2Softmax / 32; ++w) m = fmaxf(m, sQmax[w]);
      qmax_sl = sqrtf(m) * sl * 1.0001f;
    }
    for (int t = grp; t < T; t += 2) {
      const int p = grp;
      mbar_wait(&bar_s[p], (uint32_t)(t >> 1) & 1, a.status, abort_flag);
      tc_fence_after();
      // Row maximum.  Every score of this token obeys |S_mn| sl <= |k_n| max_m |q_m| sl (Cauchy-Schwarz): when
      // that bound is small the exponentials cannot overflow or vanish without any shift, and the pass over
      // the scores that finds the maximum is skipped (rmax = 0).  The two threads of a row see the same
      // bound and the two warps that share 32 rows take the same branch.
      float rmax = 0.f;
      float kn2 = 0.f;
      {
        const uint8_t* kr = sK + (t % 3) * L::kK;
#pragma unroll
        for (int c = 0; c < ROWB / 16; ++c) {
          const uint4 k4 = *reinterpret_cast<const uint4*>(kr + swz_off<ROWB>(row, c));
          const uint32_t* kp = reinterpret_cast<const uint32_t*>(&k4);
#pragma unroll
          for (int j = 0; j < 4; ++j) { const float2 f = Op16<T16>::unpack(kp[j]); kn2 = fmaf(f.x, f.x, kn2); kn2 = fmaf(f.y, f.y, kn2); }
        }
      }
      // unshifted weights lie in [2^-bound, 2^bound]: far inside bf16's range; fp16 (largest value 2^16,
      // full precision down to 2^-14) gets a tighter bound
      constexpr float kBound = Op16<T16>::kFmt == 0 ? 8.f : 48.f;
      const bool exact = sqrtf(kn2) * qmax_sl > kBound;
      if (__any_sync(0xffffffffu, exact)) {
        float mx = -INFINITY;
        for (int c = 0; c < nv / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(cols + 32 * c, r);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) mx = fmaxf(mx, __uint_as_float(r[j]));
        }
        float* mq = sMaxQ + ((t >> 1) & 1) * 512 + p * 256;      // [tile-of-group parity][group][half][row]
        mq[hf * 128 + row] = mx;
        named_bar_sync_s2(1 + p * 4 + (warp & 3), 64);           // the two warps that share these rows
        rmax = fmaxf(mx, mq[(hf ^ 1) * 128 + row]);
      }
      const float off = -rmax * sl;
      float2 sum2 = make_float2(0.f, 0.f);
      const uint32_t ntok = (uint32_t)(n0 + t * 128 + row);
      const uint32_t drow0 = (uint32_t)(2 * a.B * a.H + bh) * (uint32_t)a.M_total + (uint32_t)(a.m0 + 128 * hf);
      for (int c = 0; c < nv / 32; ++c) {
        uint32_t r[32], pk[16];
        tmem_ld32(cols + 32 * c, r);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          // two scores per instruction (packed fp32 multiply-add and add)
          const float2 x2 = __ffma2_rn(make_float2(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1])), make_float2(sl, sl),
                                       make_float2(off, off));
          float e0 = ex2(x2.x), e1 = ex2(x2.y);
          sum2 = __fadd2_rn(sum2, make_float2(e0, e1));
          if (DROP) {                              // the row sum normalises before the dropout mask applies
            const uint32_t dr = drow0 + 32 * c + 2 * j;
            e0 = drop_hash(ntok, dr, a.drop.seed_lo, a.drop.seed_hi) >= a.drop.thresh ? e0 * a.drop.inv_keep : 0.f;
            e1 = drop_hash(ntok, dr + 1, a.drop.seed_lo, a.drop.seed_hi) >= a.drop.thresh ? e1 * a.drop.inv_keep : 0.f;
          }
          pk[j] = Op16<T16>::pack(e0, e1);
        }
        tmem_st16(cols + 16 * c, pk);
      }
      sSum[(p * 2 + hf) * 128 + row] = sum2.x + sum2.y;
      if (hf == 0) sRowMax[p * 128 + row] = rmax;
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive_s2(&bar_sm[p]);
      if (*reinterpret_cast<volatile int*>(abort_flag)) break;
    }
  } else {
    // ================================ epilogue warps ================================
    const float sl = a.scale_log2;
    for (int t = 0; t < T; ++t) {
      const int p = t & 1;
      mbar_wait(&bar_sm[p], (uint32_t)(t >> 1) & 1, a.status, abort_flag);         // row sums / max visible
      mbar_wait(&bar_pv[p], (uint32_t)(t >> 1) & 1, a.status, abort_flag);         // Y(t) complete
      if (*reinterpret_cast<volatile int*>(abort_flag)) break;
      tc_fence_after();
      uint32_t r[D];
      if constexpr (D == 16) tmem_ld16(lane_base + 256 * p + kY, r);
      else tmem_ld32(lane_base + 256 * p + kY, r);
      const float* sq = sSum + p * 2 * 128 + row;
      const float sum = sq[0] + sq[128];
      const float rmax = sRowMax[p * 128 + row];
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive_s2(&bar_ep[p]);                  // the buffer (and its shared-memory scalars) may be reused
      const int tok = n0 + t * 128 + row;
      if (tok < n1) {
        const bool keep = !a.mask || a.mask[(long long)b * a.N + tok];
        float inv = keep ? 1.f / sum : 0.f;
        float c_new = (rmax * sl + log2f(sum)) * kLn2;
        uint16_t* yp = static_cast<uint16_t*>(a.y) + b * a.ys[0] + h * a.ys[1] + (long long)tok * a.ys[2];
        float w_old = 0.f;
        if (a.accumulate) {
          // this launch covers one block of the latents: y = w_old y_old + w_new y_block, C = logaddexp
          const float c_old = a.lse_n[((long long)b * a.H + h) * a.N + tok];
          const float cm = fmaxf(c_old, c_new);
          const float e_old = __expf(c_old - cm), e_new = __expf(c_new - cm);
          const float tot = e_old + e_new;
          w_old = e_old / tot;
          inv *= e_new / tot;
          c_new = cm + __logf(tot);
        }
#pragma unroll
        for (int c = 0; c < D / 8; ++c) {
          float f[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[8 * c + j]) * inv;
          if (a.accumulate) {
            const uint4 old = reinterpret_cast<const uint4*>(yp)[c];
            const uint32_t* op = reinterpret_cast<const uint32_t*>(&old);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 of = Op16<T16>::unpack(op[j]);
              f[2 * j] = fmaf(w_old, of.x, f[2 * j]); f[2 * j + 1] = fmaf(w_old, of.y, f[2 * j + 1]);
            }
          }
          uint4 o;
          o.x = Op16<T16>::pack(f[0], f[1]); o.y = Op16<T16>::pack(f[2], f[3]);
          o.z = Op16<T16>::pack(f[4], f[5]); o.w = Op16<T16>::pack(f[6], f[7]);
          reinterpret_cast<uint4*>(yp)[c] = o;
        }
        if (a.lse_n) a.lse_n[((long long)b * a.H + h) * a.N + tok] = c_new;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc<512>(tmem);
}

// ------------------------------------------------------------------------------------------
bool tc_scatter2_supported(const Ctx& c, int dtype) {
  // more than 256 latents run as blocks of 256, each launch merging into y and C_n (needs C_n storage)
  return (dtype == FLARE_BF16 || dtype == FLARE_F16) && (c.D == 16 || c.D == 32) && c.M >= 32 && c.M <= 1024 &&
         c.M % 32 == 0 && c.N >= 1;
}

template <int D, typename T16>
static int launch_scatter2(const Ctx& c, const void* q, const void* k, const float* z32, const uint8_t* mask,
                           void* y, float* lse_n, cudaStream_t st) {
  CUtensorMap tmK;
  const uint64_t e = 2;
  if (c.M > 256 && !lse_n) return FLARE_EUNSUPPORTED;
  constexpr int F = Op16<T16>::kFmt;
  if (!make_tile_map(&tmK, k, F, D, (uint64_t)c.N, (uint64_t)c.H, (uint64_t)c.B, c.ks[2] * e, c.ks[1] * e,
                     (c.B > 1 ? c.ks[0] : c.ks[1] * c.H) * e, 128))
    return FLARE_EUNSUPPORTED;
  const bool qb = c.qs[0] != 0;
  // token ranges: two CTAs' worth of work per SM
  const long long bh = (long long)c.B * c.H;
  long long splits = (2LL * num_sms() + bh - 1) / bh;
  const long long tiles = (c.N + 127) / 128;
  if (splits > tiles) splits = tiles;
  if (splits < 1) splits = 1;
  const long long chunk = ((tiles + splits - 1) / splits) * 128;
  splits = (c.N + chunk - 1) / chunk;
  Scatter2Args a;
  a.B = c.B; a.H = c.H; a.N = c.N;
  a.scale_log2 = c.scale * kLog2e;
  a.q_batched = qb ? 1 : 0;
  a.n_splits = (int)splits; a.chunk = (int)chunk;
  a.mask = mask; a.y = y;
  a.z_bh_stride = (long long)c.M * D;
  for (int i = 0; i < 3; ++i) a.ys[i] = c.ys[i];
  a.lse_n = lse_n;
  a.status = tc_status_ptr();
  a.drop = make_drop(c.drop_p, c.drop_seed);
  constexpr int smem = Scatter2Smem<D>::kBytes;
  if (tc_set_dyn_smem(reinterpret_cast<const void*>(&k_tc_scatter2<D, T16, false>), smem) != FLARE_OK ||
      tc_set_dyn_smem(reinterpret_cast<const void*>(&k_tc_scatter2<D, T16, true>), smem) != FLARE_OK)
    return FLARE_ECUDA;
  const long long grid = splits * bh;
  if (grid > 0x7fffffffLL) return FLARE_EUNSUPPORTED;
  for (int m0 = 0; m0 < c.M; m0 += 256) {
    const int mb = c.M - m0 < 256 ? c.M - m0 : 256;
    CUtensorMap tmQ;
    const char* qblk = static_cast<const char*>(q) + (long long)m0 * c.qs[2] * e;
    if (!make_tile_map(&tmQ, qblk, F, D, (uint64_t)mb, (uint64_t)c.H, (uint64_t)(qb ? c.B : 1), c.qs[2] * e,
                       c.qs[1] * e, (qb ? c.qs[0] : c.qs[1] * c.H) * e, (uint32_t)mb))
      return FLARE_EUNSUPPORTED;
    a.M = mb; a.m0 = m0; a.M_total = c.M;
    a.z32 = z32 + (long long)m0 * D;
    a.accumulate = m0 > 0 ? 1 : 0;
    if (a.drop.on) launch_dep(k_tc_scatter2<D, T16, true>, dim3((unsigned)grid), dim3(kS2Softmax + kS2Epilogue + 32), smem, st, tmK, tmQ, a);
    else launch_dep(k_tc_scatter2<D, T16, false>, dim3((unsigned)grid), dim3(kS2Softmax + kS2Epilogue + 32), smem, st, tmK, tmQ, a);
  }
  return FLARE_OK;
}

int tc_scatter2(const Ctx& c, int dtype, const void* q, const void* k, const float* z32, const uint8_t* mask, void* y,
                float* lse_n, cudaStream_t st) {
  const bool bf = dtype == FLARE_BF16;
  switch (c.D) {
    case 16: return bf ? launch_scatter2<16, __nv_bfloat16>(c, q, k, z32, mask, y, lse_n, st)
                       : launch_scatter2<16, __half>(c, q, k, z32, mask, y, lse_n, st);
    case 32: return bf ? launch_scatter2<32, __nv_bfloat16>(c, q, k, z32, mask, y, lse_n, st)
                       : launch_scatter2<32, __half>(c, q, k, z32, mask, y, lse_n, st);
  }
  return FLARE_EUNSUPPORTED;
}

}  // namespace flare
