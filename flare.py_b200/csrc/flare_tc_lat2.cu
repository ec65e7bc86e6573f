// Latent-major split-N passes on tcgen05 tensor cores, decoupled schedule (D <= 32).
//
//   MODE 0  gather : record (acc, m, l) of z = softmax_N(S) v over one token range
//   MODE 1  dZ     : dz_part = sum_n exp(S_mn - C_n) dY_n over one token range
//
// Same mathematics and tiling as flare_tc_lat.cu (one CTA = 128 latents x one token range, 128-token
// tiles, S = Q K^T and acc += P V on the tensor core, P packed over S in tensor memory).  Differences:
//   * A dedicated issuer warp feeds the tensor core; the 256 softmax threads (two per latent row, 64
//     score columns each) never issue and never wait for more than the S product of their tile:
//     S(t+1) is committed on its own mbarrier ahead of P(t) V(t).
//   * No separate row-max pass in steady state.  The running maximum m_run only has to stay within
//     2^60 of the true one; a Cauchy-Schwarz bound |q_m| max_n |k_n| on the tile's scores (row norms of
//     the K tile, computed by the issuer warp two tiles ahead) tells when that is guaranteed.  Only the first
//     tile and tiles whose bound exceeds m_run + 60 take the exact max pass (two halves of a row meet
//     through shared memory) and rescale the accumulator.
//   * Tensor-memory columns: S of even tiles [0,128), of odd tiles [96,224); P of even tiles
//     {[0,32), [64,96)}, of odd tiles {[128,160), [192,224)}; accumulator [224,256).  Every thread
//     packs P inside its own score columns, S(t+1) never touches P(t), and S(t+2) is issued only after
//     P(t) V(t) has completed.
//   * K/V tiles arrive in a four-stage TMA ring (three tiles of prefetch distance); in MODE 1 the
//     tile's C_n row rides on the same mbarrier as an untiled bulk copy.
//   * The softmax threads read their 64 columns in four chunks of 16, one chunk ahead of the
//     arithmetic, so that few registers are live and the MUFU stays fed.
//   * A key-padding mask (and the ragged end of a range) reaches the softmax threads as one keep bit
//     per token of the tile, published with the norm bound; excluded tokens get probability zero and
//     do not enter the exact maximum.
// Two CTAs (288 threads each) share an SM.  bf16 or fp16 operands (fp16 probabilities must stay below
// 2^15, so its running maximum may lag the true one by 2^14 at most instead of 2^60).
#include "common.cuh"
#include "launch.h"
#include "tc_common.cuh"
#include "tma_host.h"

namespace flare {

using namespace tc;

struct Lat2Args {
  int B, H, N, M;
  float scale_log2;
  int q_batched;
  int n_splits, chunk, n_mblk;
  const float* lse_n;          // MODE 1: [B,H,N]
  float* out;                  // MODE 0: rec [S,B,H,M,D+2]; MODE 1: dz_part [S,B,H,M,D]
  int* status;
  int c_bulk;                  // MODE 1: C_n rows may be fetched with 16-byte-aligned bulk copies
  const uint8_t* mask;         // [B,N] key-padding mask (non-zero = keep) or null
  DropArgs drop;               // attention dropout of this pass's softmax weights
};

constexpr int kLat2Stages = 4;

template <int D>
struct Lat2Smem {
  static constexpr int ROWB = 2 * D;
  static constexpr int kQ = 128 * ROWB;
  static constexpr int kT = 128 * ROWB;            // one K or V tile
  static constexpr int kBytes = kQ + 2 * kLat2Stages * kT + kLat2Stages * 128 * 4 /*C*/ + 2 * 128 * 4 /*max*/ +
                                128 * 4 /*l*/ + 64 /*kmax*/ + 64 /*keep bits*/ + 1024 + 256;
};

__device__ __forceinline__ void mbar_arrive_l2(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
// Untiled bulk copy global -> shared, completing on an mbarrier.  Both addresses 16-byte aligned,
// size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

constexpr int kLat2Softmax = 256;

// One chunk of 16 score columns of one row: P = 2^(S sl - m) (MODE 0) or 2^(S sl - C2) (MODE 1, C2 = C log2e),
// packed to 16-bit pairs; the two running sums take alternate columns.  kbits: keep bit of each column.
// DROP: the packed weights (not the sums) additionally pass the dropout mask of row `drow`, tokens n16 .. n16 + 15.
template <int MODE, bool MASKED, bool DROP, typename T16>
__device__ __forceinline__ void lat2_chunk(const uint32_t* r, float sl, float m_run, const float* c16, uint32_t kbits,
                                           uint32_t* pk, float& s0, float& s1, const DropArgs& dr, uint32_t drow, uint32_t n16) {
  float cv[16];
  if (MODE == 1) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 c4 = *reinterpret_cast<const float4*>(c16 + 4 * j);
      cv[4 * j] = c4.x; cv[4 * j + 1] = c4.y; cv[4 * j + 2] = c4.z; cv[4 * j + 3] = c4.w;
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float x0, x1;
    if (MODE == 0) {
      x0 = fmaf(__uint_as_float(r[2 * j]), sl, -m_run);
      x1 = fmaf(__uint_as_float(r[2 * j + 1]), sl, -m_run);
    } else {
      x0 = fmaf(__uint_as_float(r[2 * j]), sl, -cv[2 * j]);
      x1 = fmaf(__uint_as_float(r[2 * j + 1]), sl, -cv[2 * j + 1]);
    }
    float e0 = ex2(x0), e1 = ex2(x1);
    if (MASKED) {
      if (!(kbits & (1u << (2 * j)))) e0 = 0.f;
      if (!(kbits & (2u << (2 * j)))) e1 = 0.f;
    }
    s0 += e0; s1 += e1;
    if (DROP) {
      e0 = drop_hash(n16 + 2 * j, drow, dr.seed_lo, dr.seed_hi) >= dr.thresh ? e0 * dr.inv_keep : 0.f;
      e1 = drop_hash(n16 + 2 * j + 1, drow, dr.seed_lo, dr.seed_hi) >= dr.thresh ? e1 * dr.inv_keep : 0.f;
    }
    pk[j] = Op16<T16>::pack(e0, e1);
  }
}

// The four chunks of this thread's 64 score columns, loads one chunk ahead of the arithmetic.
// Even tiles walk the chunks upwards and odd tiles downwards, so that the packed P of a chunk
// never lands on score columns that are still to be loaded (P sits in the lower half of the 64
// columns on even tiles, in the upper half on odd ones).  Registers are indexed statically; only
// addresses depend on the direction.  keep: one bit per column of this thread's 64.
template <int MODE, bool MASKED, bool DROP, typename T16>
__device__ __forceinline__ float lat2_row(uint32_t s_cols, uint32_t p_cols, int p, float sl, float m_run,
                                          const float* c64, uint64_t keep, const DropArgs& dr, uint32_t drow, uint32_t n64) {
  uint32_t ra[16], rb[16], pk[8];
  float s0 = 0.f, s1 = 0.f;
  const int c0 = p ? 3 : 0, dc = p ? -1 : 1;
  auto kb = [&](int c) { return (uint32_t)(keep >> (16 * c)) & 0xffffu; };
  tmem_ld16(s_cols + 16 * c0, ra);
  tmem_wait_ld();
  tmem_ld16(s_cols + 16 * (c0 + dc), rb);
  lat2_chunk<MODE, MASKED, DROP, T16>(ra, sl, m_run, c64 + 16 * c0, kb(c0), pk, s0, s1, dr, drow, n64 + 16 * c0);
  tmem_st8(p_cols + 8 * c0, pk);
  tmem_wait_ld();
  tmem_ld16(s_cols + 16 * (c0 + 2 * dc), ra);
  lat2_chunk<MODE, MASKED, DROP, T16>(rb, sl, m_run, c64 + 16 * (c0 + dc), kb(c0 + dc), pk, s0, s1, dr, drow, n64 + 16 * (c0 + dc));
  tmem_st8(p_cols + 8 * (c0 + dc), pk);
  tmem_wait_ld();
  tmem_ld16(s_cols + 16 * (c0 + 3 * dc), rb);
  lat2_chunk<MODE, MASKED, DROP, T16>(ra, sl, m_run, c64 + 16 * (c0 + 2 * dc), kb(c0 + 2 * dc), pk, s0, s1, dr, drow, n64 + 16 * (c0 + 2 * dc));
  tmem_st8(p_cols + 8 * (c0 + 2 * dc), pk);
  tmem_wait_ld();
  lat2_chunk<MODE, MASKED, DROP, T16>(rb, sl, m_run, c64 + 16 * (c0 + 3 * dc), kb(c0 + 3 * dc), pk, s0, s1, dr, drow, n64 + 16 * (c0 + 3 * dc));
  tmem_st8(p_cols + 8 * (c0 + 3 * dc), pk);
  return s0 + s1;
}

template <int D, int MODE, typename T16, bool DROP>
__global__ void __launch_bounds__(kLat2Softmax + 32, 2)
k_tc_lat2(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
          const __grid_constant__ CUtensorMap tmV, Lat2Args a) {
  grid_dep_sync();
  constexpr int ROWB = 2 * D;
  constexpr int CPR = ROWB / 16;
  constexpr int NS = kLat2Stages;
  using L = Lat2Smem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + L::kQ;                        // [NS]
  uint8_t* sV = sK + NS * L::kT;                   // [NS]
  float* sC = reinterpret_cast<float*>(sV + NS * L::kT);   // [NS][128]  C_n of the tile (MODE 1)
  float* sMax = sC + NS * 128;                     // [2][128] half-row maxima (exact pass)
  float* sLsum = sMax + 2 * 128;                   // [128]
  float* sKmax = sLsum + 128;                      // [NS] max_n |k_n|^2 of the tile in each stage
  uint32_t* sKeep = reinterpret_cast<uint32_t*>(sKmax + 16);   // [NS][4] keep bits of the tile's 128 tokens
  uint64_t* bars = reinterpret_cast<uint64_t*>(sKeep + 16);
  uint64_t* bar_full = bars;                       // [NS]
  uint64_t* bar_s = bars + NS;                     // [2][2] S(t), score columns of half hf, complete: bar_s[2 (t&1) + hf]
  uint64_t* bar_pv = bar_s + 4;                    // [2] P(t) V(t) complete
  uint64_t* bar_sm = bar_pv + 2;                   // [2] softmax(t) done (256 arrivals)
  uint64_t* bar_k = bar_sm + 2;                    // [2] tile norm bound of tile t written (MODE 0)
  uint64_t* bar_q = bar_k + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_q + 1);
  int* abort_flag = reinterpret_cast<int*>(bar_q + 2);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool is_issuer = warp == kLat2Softmax / 32;
  const int half = (warp >> 2) & 1;                // which 64 of the tile's 128 score columns
  const int row = (warp & 3) * 32 + lane;          // latent within the block = tensor-memory lane
  const int mblk = blockIdx.x % a.n_mblk;
  const int split = (blockIdx.x / a.n_mblk) % a.n_splits;
  const int bh = blockIdx.x / (a.n_splits * a.n_mblk);
  const int b = bh / a.H, h = bh % a.H;
  const int n0 = split * a.chunk, n1 = min(a.N, n0 + a.chunk);
  const int T = n1 > n0 ? (n1 - n0 + 127) / 128 : 0;
  const int lat = mblk * 128 + row;

  constexpr int W = (MODE == 0) ? D + 2 : D;
  float* orow = a.out + ((((long long)split * a.B + b) * a.H + h) * a.M + lat) * W;

  if (T == 0) {                                    // empty range: the neutral record
    if (!is_issuer && half == 0 && lat < a.M) {
      for (int i = 0; i < D; ++i) orow[i] = 0.f;
      if (MODE == 0) { orow[D] = -INFINITY; orow[D + 1] = 0.f; }
    }
    return;
  }

  if (tid == 0) {
    for (int i = 0; i < NS; ++i) mbar_init(&bar_full[i], 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_s[2 * i], 1); mbar_init(&bar_s[2 * i + 1], 1); mbar_init(&bar_pv[i], 1); mbar_init(&bar_sm[i], kLat2Softmax); mbar_init(&bar_k[i], 1);
    }
    mbar_init(bar_q, 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
  }
  if (warp == 0) tmem_alloc<256>(tmem_slot);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
  constexpr uint32_t kAcc = 224;
  const float* cb = (MODE == 1) ? a.lse_n + ((long long)b * a.H + h) * a.N : nullptr;
  const bool c_bulk = (MODE == 1) && a.c_bulk;
  const uint8_t* mrow = a.mask ? a.mask + (long long)b * a.N : nullptr;
  // lazy running maximum: how far (log2 units) the tile's score bound may exceed it before the exact pass
  constexpr float kLag = (sizeof(T16) == 2 && Op16<T16>::kFmt == 0) ? 14.f : 60.f;
  // keep bits of one 32-token quarter of a tile: token in range and not masked out (full warp)
  auto keep_word = [&](int tok) -> uint32_t {
    const bool k1 = tok < n1 && (!mrow || mrow[tok] != 0);
    return __ballot_sync(0xffffffffu, k1);
  };

  if (is_issuer) {
    // ================================ issuer warp ================================
    // The whole warp runs this code; one elected lane executes each TMA / MMA / commit.
    auto load_tile = [&](int t) {
      const int st = t % NS;
      const int tile0 = n0 + t * 128;
      const uint32_t cbytes = c_bulk ? (uint32_t)min(128, n1 - tile0) * 4u : 0u;
      mbar_expect_tx(&bar_full[st], 2 * L::kT + cbytes);
      tma_load_4d(sK + st * L::kT, &tmK, &bar_full[st], 0, tile0, h, b);
      tma_load_4d(sV + st * L::kT, &tmV, &bar_full[st], 0, tile0, h, b);
      if (c_bulk) bulk_load(sC + st * 128, cb + tile0, cbytes, &bar_full[st]);
    };
    // max_n |k_n|^2 of a landed tile (rows past the end are zero-filled), published to the softmax
    // threads through bar_k; lane l takes rows l, l+32, l+64, l+96
    auto tile_keep = [&](int t) {
      const int tile0 = n0 + t * 128;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t w = keep_word(tile0 + 32 * i + lane);
        if (lane == 0) sKeep[(t % NS) * 4 + i] = w;
      }
    };
    auto tile_kmax = [&](int t) {
      const int st = t % NS;
      float mx = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float s2 = 0.f;
#pragma unroll
        for (int c = 0; c < CPR; ++c) {
          const uint4 k4 = *reinterpret_cast<const uint4*>(sK + st * L::kT + swz_off<ROWB>(lane + 32 * i, c));
          const uint32_t* kp = reinterpret_cast<const uint32_t*>(&k4);
#pragma unroll
          for (int j = 0; j < 4; ++j) { const float2 f = Op16<T16>::unpack(kp[j]); s2 = fmaf(f.x, f.x, s2); s2 = fmaf(f.y, f.y, s2); }
        }
        mx = fmaxf(mx, s2);
      }
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      tile_keep(t);
      if (lane == 0) { sKmax[st] = mx; mbar_arrive_l2(&bar_k[t & 1]); }
      __syncwarp();
    };

    // MODE 1: the landed C_n row of a tile, converted to log2 units once for all 256 softmax threads
    // (lane l takes entries 4l..4l+3) and published through bar_k like the norm bound of MODE 0
    auto tile_cscale = [&](int t) {
      float4* c4 = reinterpret_cast<float4*>(sC + (t % NS) * 128) + lane;
      float4 c = *c4;
      c.x *= kLog2e; c.y *= kLog2e; c.z *= kLog2e; c.w *= kLog2e;
      *c4 = c;
      tile_keep(t);
      __syncwarp();
      if (lane == 0) mbar_arrive_l2(&bar_k[t & 1]);
      __syncwarp();
    };

    constexpr int F = Op16<T16>::kFmt;
    const uint32_t idesc_s = idesc_f16(128, 128, F, F, 0, 0);
    const uint32_t idesc_pv = idesc_f16(128, D, F, F, 0, 1);
    const uint64_t dq = smem_desc<ROWB>(smem_u32(sQ));
    if (elect_one()) {
      mbar_expect_tx(bar_q, L::kQ);
      tma_load_4d(sQ, &tmQ, bar_q, 0, mblk * 128, h, a.q_batched ? b : 0);
      for (int t = 0; t < NS - 1 && t < T; ++t) load_tile(t);
    }
    __syncwarp();
    mbar_wait(bar_q, 0, a.status, abort_flag);
    mbar_wait(&bar_full[0], 0, a.status, abort_flag);
    tc_fence_after();
    {
      const uint64_t dk = smem_desc<ROWB>(smem_u32(sK));
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) mma_ss(tmem, dq + 2 * kk, dk + 2 * kk, idesc_s, kk > 0);
        mma_commit(&bar_s[0]);
        mma_commit(&bar_s[1]);
      }
      __syncwarp();
    }
    if (MODE == 0) {
      tile_kmax(0);
      if (T > 1) { mbar_wait(&bar_full[1], 0, a.status, abort_flag); tile_kmax(1); }
    } else if (c_bulk) {
      tile_cscale(0);
      if (T > 1) { mbar_wait(&bar_full[1], 0, a.status, abort_flag); tile_cscale(1); }
    }
    // One half of the score product of tile t1 (64 token columns): S region of the tile + 64 hf.
    const uint32_t idesc_h = idesc_f16(128, 64, F, F, 0, 0);
    auto issue_s_half = [&](int t1, int hf) {
      const uint64_t dk = smem_desc<ROWB>(smem_u32(sK + (t1 % NS) * L::kT + hf * 64 * ROWB));
      const uint32_t sb = tmem + ((t1 & 1) ? 96 : 0) + 64 * hf;
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) mma_ss(sb, dq + 2 * kk, dk + 2 * kk, idesc_h, kk > 0);
        mma_commit(&bar_s[2 * (t1 & 1) + hf]);
      }
      __syncwarp();
    };
    for (int t = 0; t < T; ++t) {
      const int p = t & 1;
      // The score regions of consecutive tiles overlap in 32 columns only ([96,128)), which belong to one half of
      // either tile.  The half of S(t+1) that does not touch them (columns [160,224) after an even tile, [0,64)
      // after an odd one) is issued as soon as P(t-1) V(t-1) has completed -- while the softmax threads are
      // still on tile t -- and the other half once they are done: half of the threads find their scores
      // waiting, the others cover the product's latency with the first half's exponentials still running.
      if (t >= 1) mbar_wait_hot(&bar_pv[p ^ 1], (uint32_t)((t - 1) >> 1) & 1, a.status, abort_flag);
      const int early = p ? 0 : 1;                 // half of tile t+1 that is free of S(t)
      if (t + 1 < T) {
        mbar_wait_hot(&bar_full[(t + 1) % NS], (uint32_t)((t + 1) / NS) & 1, a.status, abort_flag);
        tc_fence_after();
        issue_s_half(t + 1, early);
      }
      mbar_wait_hot(&bar_sm[p], (uint32_t)(t >> 1) & 1, a.status, abort_flag);     // P(t) written, S(t) consumed
      if (*reinterpret_cast<volatile int*>(abort_flag)) break;
      // the stage of tile t-1 may take tile t+3 (its V was read by P(t-1) V(t-1))
      if (t + NS - 1 < T && elect_one()) load_tile(t + NS - 1);
      __syncwarp();
      tc_fence_after();
      if (t + 1 < T) issue_s_half(t + 1, early ^ 1);
      {
        const uint64_t dv = smem_desc<ROWB>(smem_u32(sV + (t % NS) * L::kT));
        const uint32_t p0 = tmem + (p ? 128 : 0), p1 = tmem + (p ? 192 : 64);       // packed P of the two halves
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            mma_ts(tmem + kAcc, (kk < 4 ? p0 + 8 * kk : p1 + 8 * (kk - 4)), dv + (uint64_t)((kk * 16 * ROWB) >> 4),
                   idesc_pv, (t > 0) || (kk > 0));
          mma_commit(&bar_pv[p]);
        }
        __syncwarp();
      }
      if ((MODE == 0 || c_bulk) && t + 2 < T) {
        // the bound (or the C_n row) of tile t+2, while the softmax threads work on tile t+1
        mbar_wait(&bar_full[(t + 2) % NS], (uint32_t)((t + 2) / NS) & 1, a.status, abort_flag);
        if (MODE == 0) tile_kmax(t + 2); else tile_cscale(t + 2);
      }
    }
    __syncwarp();
  } else {
    // ================================ softmax threads ================================
    const float sl = a.scale_log2;
    // dropout row of this thread's latent: gather weights (which = 1) in MODE 0, scatter weights (2) in MODE 1
    const uint32_t drow = ((uint32_t)((MODE == 0 ? 1 : 2) * a.B * a.H + bh) * (uint32_t)a.M + (uint32_t)lat);
    float m_run = (MODE == 0) ? -INFINITY : 0.f, l_run = 0.f, qn = 0.f;
    if (MODE == 0) {
      // |q_m| of this thread's latent row (both halves compute the same value)
      mbar_wait(bar_q, 0, a.status, abort_flag);
      float s2 = 0.f;
#pragma unroll
      for (int c = 0; c < CPR; ++c) {
        const uint4 q4 = *reinterpret_cast<const uint4*>(sQ + swz_off<ROWB>(row, c));
        const uint32_t* qp = reinterpret_cast<const uint32_t*>(&q4);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = Op16<T16>::unpack(qp[j]); s2 = fmaf(f.x, f.x, s2); s2 = fmaf(f.y, f.y, s2); }
      }
      qn = sqrtf(s2) * sl * 1.0001f;
    }

    for (int t = 0; t < T; ++t) {
      const int p = t & 1, st = t % NS;
      const int tile0 = n0 + t * 128;
      const int cnt = min(128, n1 - tile0);
      float bound = 0.f;
      if (MODE == 1) {
        // C_n of the tile in log2 units: landed with K and dY and scaled by the issuer warp, or
        // (unaligned rows) fetched by the first 128 threads
        if (c_bulk) {
          mbar_wait(&bar_k[p], (uint32_t)(t >> 1) & 1, a.status, abort_flag);
        } else {
          mbar_wait(&bar_full[st], (uint32_t)(t / NS) & 1, a.status, abort_flag);
          if (tid < 128) {
            sC[st * 128 + tid] = (tid < cnt) ? cb[tile0 + tid] * kLog2e : 0.f;
            const uint32_t w = keep_word(tile0 + tid);
            if (lane == 0) sKeep[st * 4 + warp] = w;
          }
          named_bar_sync(2, kLat2Softmax);
        }
      } else {
        mbar_wait(&bar_k[p], (uint32_t)(t >> 1) & 1, a.status, abort_flag);
        bound = qn * sqrtf(sKmax[st]);             // >= every score of this row in the tile, log2 units
      }

      mbar_wait_hot(&bar_s[2 * p + half], (uint32_t)(t >> 1) & 1, a.status, abort_flag);
      tc_fence_after();
      const uint64_t keep = (uint64_t)sKeep[st * 4 + 2 * half] | ((uint64_t)sKeep[st * 4 + 2 * half + 1] << 32);
      const bool masked = keep != ~0ull;
      const uint32_t s_cols = lane_base + (p ? 96 : 0) + 64 * half;   // this thread's 64 score columns
      const uint32_t p_cols = s_cols + (p ? 32 : 0);                  // where their packed P goes

      if (MODE == 0) {
        const bool need = (t == 0) || (bound > m_run + kLag);
        if (__any_sync(0xffffffffu, need)) {       // the partner warp holds the same rows: same vote
          float mx = -INFINITY;
          for (int i = 0; i < 4; ++i) {
            uint32_t r[16];
            tmem_ld16(s_cols + 16 * i, r);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j)
              mx = fmaxf(mx, ((keep >> (16 * i + j)) & 1) ? __uint_as_float(r[j]) : -INFINITY);
          }
          sMax[half * 128 + row] = mx;
          named_bar_sync(3 + (warp & 3), 64);      // the two warps of this lane quarter
          const float tmax = fmaxf(mx, sMax[(half ^ 1) * 128 + row]) * sl;
          const bool grow = tmax > m_run + 8.f;
          if (t > 0 && __any_sync(0xffffffffu, grow)) {
            const float f = grow ? ex2(m_run - tmax) : 1.f;
            if (half == 0) {                       // one thread per row rescales the accumulator
              mbar_wait(&bar_pv[p ^ 1], (uint32_t)((t - 1) >> 1) & 1, a.status, abort_flag);
              tc_fence_after();
              uint32_t r[D];
              if constexpr (D == 16) tmem_ld16(lane_base + kAcc, r); else tmem_ld32(lane_base + kAcc, r);
              tmem_wait_ld();
#pragma unroll
              for (int j = 0; j < D; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * f);
              if constexpr (D == 16) tmem_st16(lane_base + kAcc, r); else tmem_st32(lane_base + kAcc, r);
            }
            l_run *= f;
          }
          if (grow) m_run = tmax;
          named_bar_sync(3 + (warp & 3), 64);      // sMax may be rewritten next time only after both read it
        }
      }

      // ---- one exponential per score; P packed inside this thread's own columns ----------------
      const float* c64 = sC + st * 128 + 64 * half;
      const uint32_t n64 = (uint32_t)(tile0 + 64 * half);
      if (DROP)         l_run += lat2_row<MODE, true, true, T16>(s_cols, p_cols, p, sl, m_run, c64, keep, a.drop, drow, n64);
      else if (!masked) l_run += lat2_row<MODE, false, false, T16>(s_cols, p_cols, p, sl, m_run, c64, keep, a.drop, drow, n64);
      else              l_run += lat2_row<MODE, true, false, T16>(s_cols, p_cols, p, sl, m_run, c64, keep, a.drop, drow, n64);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive_l2(&bar_sm[p]);
      if (*reinterpret_cast<volatile int*>(abort_flag)) break;
    }

    // ---- epilogue ---------------------------------------------------------------------------
    if (!*reinterpret_cast<volatile int*>(abort_flag)) {
      if (MODE == 0) {
        if (half == 1) sLsum[row] = l_run;
        named_bar_sync(2, kLat2Softmax);
        if (half == 0) l_run += sLsum[row];
      }
      mbar_wait(&bar_pv[(T - 1) & 1], (uint32_t)((T - 1) >> 1) & 1, a.status, abort_flag);
      tc_fence_after();
      if (half == 0) {
        uint32_t r[D];
        if constexpr (D == 16) tmem_ld16(lane_base + kAcc, r); else tmem_ld32(lane_base + kAcc, r);
        tmem_wait_ld();
        if (lat < a.M) {
#pragma unroll
          for (int j = 0; j < D / 4; ++j) {
            if constexpr (MODE == 1) {
              reinterpret_cast<float4*>(orow)[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                               __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
            } else {
              reinterpret_cast<float2*>(orow)[2 * j] = make_float2(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]));
              reinterpret_cast<float2*>(orow)[2 * j + 1] = make_float2(__uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
            }
          }
          if (MODE == 0) { orow[D] = m_run * kLn2; orow[D + 1] = l_run; }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc<256>(tmem);
}

// ------------------------------------------------------------------------------------------
bool tc_lat2_supported(const Ctx& c, int dtype) {
  return (dtype == FLARE_BF16 || dtype == FLARE_F16) && (c.D == 16 || c.D == 32) && c.N >= 1 && c.M >= 1;
}

template <int D, int MODE, typename T16>
static int launch_lat2(const Ctx& c, const void* q, const void* k, const void* v, const uint8_t* mask, const float* lse_n,
                       float* out, cudaStream_t st) {
  CUtensorMap tmQ, tmK, tmV;
  const uint64_t e = 2;
  constexpr int F = Op16<T16>::kFmt;
  const bool qb = c.qs[0] != 0;
  const long long* vs = (MODE == 0) ? c.vs : c.dys;
  if (!make_tile_map(&tmQ, q, F, D, (uint64_t)c.M, (uint64_t)c.H, (uint64_t)(qb ? c.B : 1), c.qs[2] * e, c.qs[1] * e,
                     (qb ? c.qs[0] : c.qs[1] * c.H) * e, 128) ||
      !make_tile_map(&tmK, k, F, D, (uint64_t)c.N, (uint64_t)c.H, (uint64_t)c.B, c.ks[2] * e, c.ks[1] * e,
                     (c.B > 1 ? c.ks[0] : c.ks[1] * c.H) * e, 128) ||
      !make_tile_map(&tmV, v, F, D, (uint64_t)c.N, (uint64_t)c.H, (uint64_t)c.B, vs[2] * e, vs[1] * e,
                     (c.B > 1 ? vs[0] : vs[1] * c.H) * e, 128))
    return FLARE_EUNSUPPORTED;
  Lat2Args a;
  a.B = c.B; a.H = c.H; a.N = c.N; a.M = c.M;
  a.scale_log2 = c.scale * kLog2e;
  a.q_batched = qb ? 1 : 0;
  a.n_splits = c.n_splits; a.chunk = c.chunk; a.n_mblk = (c.M + 127) / 128;
  a.lse_n = lse_n; a.out = out;
  a.status = tc_status_ptr();
  a.c_bulk = (MODE == 1 && lse_n && (reinterpret_cast<uintptr_t>(lse_n) & 15) == 0 && (c.N & 3) == 0) ? 1 : 0;
  a.mask = mask;
  a.drop = make_drop(c.drop_p, c.drop_seed);
  constexpr int smem = Lat2Smem<D>::kBytes;
  if (tc_set_dyn_smem(reinterpret_cast<const void*>(&k_tc_lat2<D, MODE, T16, false>), smem) != FLARE_OK ||
      tc_set_dyn_smem(reinterpret_cast<const void*>(&k_tc_lat2<D, MODE, T16, true>), smem) != FLARE_OK)
    return FLARE_ECUDA;
  const long long grid = (long long)c.n_splits * a.n_mblk * c.B * c.H;
  if (grid > 0x7fffffffLL) return FLARE_EUNSUPPORTED;
  if (a.drop.on) launch_dep(k_tc_lat2<D, MODE, T16, true>, dim3((unsigned)grid), dim3(kLat2Softmax + 32), smem, st, tmQ, tmK, tmV, a);
  else launch_dep(k_tc_lat2<D, MODE, T16, false>, dim3((unsigned)grid), dim3(kLat2Softmax + 32), smem, st, tmQ, tmK, tmV, a);
  return FLARE_OK;
}

template <int MODE>
static int dispatch_lat2(const Ctx& c, int dtype, const void* q, const void* k, const void* v, const uint8_t* mask,
                         const float* lse_n, float* out, cudaStream_t st) {
  const bool bf = dtype == FLARE_BF16;
  switch (c.D) {
    case 16: return bf ? launch_lat2<16, MODE, __nv_bfloat16>(c, q, k, v, mask, lse_n, out, st)
                       : launch_lat2<16, MODE, __half>(c, q, k, v, mask, lse_n, out, st);
    case 32: return bf ? launch_lat2<32, MODE, __nv_bfloat16>(c, q, k, v, mask, lse_n, out, st)
                       : launch_lat2<32, MODE, __half>(c, q, k, v, mask, lse_n, out, st);
  }
  return FLARE_EUNSUPPORTED;
}

int tc_gather_partial2(const Ctx& c, int dtype, const void* q, const void* k, const void* v, const uint8_t* mask,
                       float* rec, cudaStream_t st) {
  return dispatch_lat2<0>(c, dtype, q, k, v, mask, nullptr, rec, st);
}

int tc_dz_partial2(const Ctx& c, int dtype, const void* q, const void* k, const void* dy, const uint8_t* mask,
                   const float* lse_n, float* dz_part, cudaStream_t st) {
  return dispatch_lat2<1>(c, dtype, q, k, dy, mask, lse_n, dz_part, st);
}

}  // namespace flare
