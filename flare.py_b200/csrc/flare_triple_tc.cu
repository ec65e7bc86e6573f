// Triple attention on the tensor cores (16-bit inputs, every feature dimension 32).
//
// Both shapes of work in lra/models/triton/triple.py (einsum forms :846-860, :887-931) are products with a
// 1024-long axis made of PAIRS of features, whose operand is never in memory: it is the per-token outer
// product u_n (x) w_n, built on the fly in shared memory, 128 pair columns (four u features x 32 w features)
// at a time:
//
//   outer     out[i][j][k] = alpha sum_n a[n,i] b[n,j] c[n,k]
//             = (P^T B)[(i,k), j]  with P[n,(i,k)] = a[n,i] c[n,k]:  for each block of four i the
//             128-token x 128-pair tile of P is the MN-major A operand (M = pairs, contraction = tokens),
//             the token tile of b the MN-major B operand; eight accumulators of 32 columns in tensor memory
//   contract  out[n,x] = alpha sum_{y,z} T[x,y,z] a[n,y] b[n,z]
//             = (P T')[n, x]  with P[n,(y,z)] = a[n,y] b[n,z], T'[(y,z), x]:  here the rows of P are the
//             tokens, so its tiles go straight into tensor memory (each thread packs the pairs of its own
//             token row) and are the A operand from there; T' is resident in shared memory as 16-bit
//             (scaled per (b,h) by a power of two so that fp16 cannot overflow)
//
// Eight producer warps build the tiles of P (one token row and half of the w features per thread: 4 packed
// multiplies per eight pairs) into four buffers; two warps issue the products (tcgen05.mma, fp32
// accumulation; alternate tiles, each warp into accumulators of its own, so nothing depends on the order of
// two threads' products) and recycle the buffers through mbarriers.  Every wait is bounded.
#include "common.cuh"
#include "launch.h"
#include "tc_common.cuh"

namespace flare {

using namespace tc;

namespace {

constexpr int kTD = 32;                            // every feature dimension
constexpr int kProd = 256;                         // producer threads
constexpr int kThreadsT = kProd + 64;              // + two issuing warps (alternate tiles of P, accumulators of their own)
constexpr int kPBytes = 128 * 128 * 2;             // one tile of P: 128 tokens x 128 pairs, 16-bit
constexpr int kNP = 4;                             // tiles of P in flight (building, waiting, being multiplied)
constexpr int kBBytes = 128 * 64;                  // one token tile of b (outer)
constexpr int kTBytes = 1024 * 64;                 // T' (contract): 1024 pair rows x 32 x, 16-bit

__device__ __forceinline__ void arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

template <typename T16> struct Pair16;
template <> struct Pair16<__nv_bfloat16> {
  using V2 = __nv_bfloat162;
  static __device__ __forceinline__ V2 splat(uint32_t word, int hi) {
    const uint32_t h = hi ? (word >> 16) : (word & 0xffffu);
    const uint32_t w = h | (h << 16);
    return *reinterpret_cast<const V2*>(&w);
  }
};
template <> struct Pair16<__half> {
  using V2 = __half2;
  static __device__ __forceinline__ V2 splat(uint32_t word, int hi) {
    const uint32_t h = hi ? (word >> 16) : (word & 0xffffu);
    const uint32_t w = h | (h << 16);
    return *reinterpret_cast<const V2*>(&w);
  }
};

// One 128-token x 128-pair tile of P into `dst` (two 64-pair halves of [128 rows][128 bytes], 128-byte
// swizzle): pairs (il, w) for the four u features 4*blk + il.  This thread: token row n, w features
// [16 hk, 16 hk + 16).  uw: the 32 u features of the token (16 words), ww: its 16 w features (8 words).
template <typename T16>
__device__ __forceinline__ void build_pairs(uint8_t* dst, int n, int hk, int blk, const uint32_t (&uw)[16],
                                            const uint32_t (&ww)[8]) {
  using V2 = typename Pair16<T16>::V2;
#pragma unroll
  for (int il = 0; il < 4; ++il) {
    const int i = 4 * blk + il;
    const V2 ui = Pair16<T16>::splat(uw[i >> 1], i & 1);
    uint8_t* half = dst + (il >> 1) * (128 * 128);
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const V2 p = __hmul2(ui, *reinterpret_cast<const V2*>(&ww[4 * cc + j]));
        o[j] = *reinterpret_cast<const uint32_t*>(&p);
      }
      *reinterpret_cast<uint4*>(half + swz_off<128>(n, 4 * (il & 1) + 2 * hk + cc)) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// The same tile as the K-major A operand of a product whose rows are the tokens: thread (token row = its
// tensor-memory lane, hk) writes its 16 pairs of every il as eight packed words at columns 16 il + 8 hk of
// the 64-column tile -- no shared memory on the way, and the product reads A at twice the rate.
template <typename T16>
__device__ __forceinline__ void build_pairs_tmem(uint32_t tile, int hk, int blk, const uint32_t (&uw)[16],
                                                 const uint32_t (&ww)[8]) {
  using V2 = typename Pair16<T16>::V2;
#pragma unroll
  for (int il = 0; il < 4; ++il) {
    const int i = 4 * blk + il;
    const V2 ui = Pair16<T16>::splat(uw[i >> 1], i & 1);
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const V2 p = __hmul2(ui, *reinterpret_cast<const V2*>(&ww[j]));
      o[j] = *reinterpret_cast<const uint32_t*>(&p);
    }
    tmem_st8(tile + 16 * il + 8 * hk, o);
  }
}

// features of token row `tok` (zeros past the end): all 32 of u, 16 of w
template <typename T16>
__device__ __forceinline__ void load_rows(const T16* u, const T16* w, long long tok, bool in, int hk, uint32_t (&uw)[16],
                                          uint32_t (&ww)[8]) {
  if (in) {
    const uint4* up = reinterpret_cast<const uint4*>(u + tok * kTD);
    const uint4* wp = reinterpret_cast<const uint4*>(w + tok * kTD + 16 * hk);
#pragma unroll
    for (int c = 0; c < 4; ++c) { const uint4 x = up[c]; uw[4 * c] = x.x; uw[4 * c + 1] = x.y; uw[4 * c + 2] = x.z; uw[4 * c + 3] = x.w; }
#pragma unroll
    for (int c = 0; c < 2; ++c) { const uint4 x = wp[c]; ww[4 * c] = x.x; ww[4 * c + 1] = x.y; ww[4 * c + 2] = x.z; ww[4 * c + 3] = x.w; }
  } else {
#pragma unroll
    for (int c = 0; c < 16; ++c) uw[c] = 0u;
#pragma unroll
    for (int c = 0; c < 8; ++c) ww[c] = 0u;
  }
}

struct TripleBars {
  uint64_t full[kNP], empty[kNP], acc_full[2], acc_free[2];
  uint32_t tmem_slot;
  int abort_flag;
};

// ---------------------------------------------------------------------------------------------------
// outer:  part[split][bh][i][j][k] = alpha * sum over the split's tokens of a[n,i] b[n,j] c[n,k]
// ---------------------------------------------------------------------------------------------------
template <typename T16>
__global__ void __launch_bounds__(kThreadsT, 1)
k_triple_tc_outer(const T16* __restrict__ A, const T16* __restrict__ Bm, const T16* __restrict__ Cm, int N, int chunk,
                  float alpha, float* __restrict__ part, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sP = smem;                              // [kNP] tiles of P
  uint8_t* sB = sP + kNP * kPBytes;                // [2] token tiles of b
  TripleBars* bars = reinterpret_cast<TripleBars*>(sB + 2 * kBBytes);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int split = blockIdx.x, bh = blockIdx.y;
  const int n0 = split * chunk, n1 = min(N, n0 + chunk);
  const int T = n1 > n0 ? (n1 - n0 + 127) / 128 : 0;
  float* out = part + ((long long)split * gridDim.y + bh) * (kTD * kTD * kTD);
  if (T == 0) {
    for (int i = tid; i < kTD * kTD * kTD; i += kThreadsT) out[i] = 0.f;
    return;
  }
  if (tid == 0) {
    for (int i = 0; i < kNP; ++i) { mbar_init(&bars->full[i], kProd); mbar_init(&bars->empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&bars->acc_full[i], 2); mbar_init(&bars->acc_free[i], kProd); }
    bars->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0) tmem_alloc<256>(&bars->tmem_slot);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_slot;
  int* abort_flag = &bars->abort_flag;
  const T16* a = A + (long long)bh * N * kTD;
  const T16* b = Bm + (long long)bh * N * kTD;
  const T16* c = Cm + (long long)bh * N * kTD;
  constexpr int F = Op16<T16>::kFmt;

  if (warp < kProd / 32) {
    // ================= producers =================
    const int n = tid & 127, hk = tid >> 7;
    // the rows of the next tile are fetched while the current one is worked: their latency never sits
    // between two tiles
    uint32_t uw[16], ww[8], un[16], wn[8];
    uint4 bn[2];
    auto fetch_b = [&](int t) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int e = tid + r * kProd, row = e >> 2, ch = e & 3;
        const long long tk = (long long)n0 + t * 128 + row;
        bn[r] = tk < n1 ? reinterpret_cast<const uint4*>(b + tk * kTD)[ch] : make_uint4(0, 0, 0, 0);
      }
    };
    load_rows<T16>(a, c, (long long)n0 + n, (long long)n0 + n < n1, hk, un, wn);
    fetch_b(0);
    for (int t = 0; t < T; ++t) {
#pragma unroll
      for (int i = 0; i < 16; ++i) uw[i] = un[i];
#pragma unroll
      for (int i = 0; i < 8; ++i) ww[i] = wn[i];
      const uint4 b0 = bn[0], b1 = bn[1];
      if (t + 1 < T) {
        const long long tok = (long long)n0 + (t + 1) * 128 + n;
        load_rows<T16>(a, c, tok, tok < n1, hk, un, wn);
        fetch_b(t + 1);
      }
#pragma unroll
      for (int blk = 0; blk < 8; ++blk) {
        const int g = 8 * t + blk, buf = g % kNP;
        if (g >= kNP) mbar_wait_hot(&bars->empty[buf], (uint32_t)(g / kNP - 1) & 1, status, abort_flag);
        if (blk == 0) {
          // the token tile of b (its buffer was last read by the products of tile t-2, complete by now)
          *reinterpret_cast<uint4*>(sB + (t & 1) * kBBytes + swz_off<64>(tid >> 2, tid & 3)) = b0;
          *reinterpret_cast<uint4*>(sB + (t & 1) * kBBytes + swz_off<64>((tid + kProd) >> 2, tid & 3)) = b1;
        }
        build_pairs<T16>(sP + buf * kPBytes, n, hk, blk, uw, ww);
        fence_proxy_async();
        arrive(&bars->full[buf]);
      }
      if (*reinterpret_cast<volatile int*>(abort_flag)) break;
    }
    // ---- the eight accumulators -> this split's partial sum ----
    mbar_wait(&bars->acc_full[0], 0, status, abort_flag);
    tc_fence_after();
    if (!*reinterpret_cast<volatile int*>(abort_flag)) {
      const int il = warp & 3;                     // lane quarter = which of the block's four i
      const uint32_t lane_base = tmem + ((uint32_t)(il * 32) << 16);
#pragma unroll 1
      for (int m4 = 0; m4 < 4; ++m4) {
        const int blk = (warp >> 2) * 4 + m4;
        uint32_t r[32];
        tmem_ld32(lane_base + 32 * blk, r);
        tmem_wait_ld();
        float* o = out + (long long)(4 * blk + il) * (kTD * kTD) + lane;      // [i][j][k = lane]
#pragma unroll
        for (int j = 0; j < 32; ++j) o[j * kTD] = __uint_as_float(r[j]) * alpha;
      }
    }
  } else {
    // ================= issuing warp =================
    const uint32_t idesc = idesc_f16(128, kTD, F, F, 1, 1);          // A (pairs x tokens) and B (tokens x j) MN-major
    const uint64_t pdesc = smem_desc_mn128(smem_u32(sP), 128 * 128, 1024);
    const uint64_t bdesc = smem_desc<64>(smem_u32(sB));
    const int iw = warp - kProd / 32;              // this issuing warp takes the blocks iw, iw + 2, ... (accumulators of their own)
    for (int t = 0; t < T; ++t) {
      for (int blk = iw; blk < 8; blk += 2) {
        const int g = 8 * t + blk, buf = g % kNP;
        mbar_wait_hot(&bars->full[buf], (uint32_t)(g / kNP) & 1, status, abort_flag);
        tc_fence_after();
        if (elect_one()) {
          const uint64_t pa = pdesc + (uint64_t)(buf * (kPBytes >> 4));
          const uint64_t pb = bdesc + (uint64_t)((t & 1) * (kBBytes >> 4));
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) mma_ss(tmem + 32 * blk, pa + 128 * kk, pb + 64 * kk, idesc, (t > 0) || (kk > 0));
          mma_commit(&bars->empty[buf]);
          if (t == T - 1 && blk >= 6) mma_commit(&bars->acc_full[0]);
        }
        __syncwarp();
        if (*reinterpret_cast<volatile int*>(abort_flag)) break;
      }
      if (*reinterpret_cast<volatile int*>(abort_flag)) break;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc<256>(tmem);
}

// ---------------------------------------------------------------------------------------------------
// contract:  out[bh][n][x] = alpha * sum_{y,z} T[x,y,z] a[n,y] b[n,z]
// ---------------------------------------------------------------------------------------------------
template <typename T16>
__global__ void __launch_bounds__(kThreadsT, 1)
k_triple_tc_contract(const float* __restrict__ Tm, long long sx, long long sy, long long sz, const T16* __restrict__ A,
                     const T16* __restrict__ Bm, int N, int chunk, float alpha, T16* __restrict__ O, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sT = smem;                              // T' [(y,z)][x], 16-bit, 64-byte swizzled rows
  TripleBars* bars = reinterpret_cast<TripleBars*>(sT + kTBytes);
  float* sRed = reinterpret_cast<float*>(bars + 1);                // [kThreadsT / 32] warp maxima
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int split = blockIdx.x, bh = blockIdx.y;
  const int n0 = split * chunk, n1 = min(N, n0 + chunk);
  const int T = n1 > n0 ? (n1 - n0 + 127) / 128 : 0;
  if (T == 0) return;
  if (tid == 0) {
    for (int i = 0; i < kNP; ++i) { mbar_init(&bars->full[i], kProd); mbar_init(&bars->empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&bars->acc_full[i], 2); mbar_init(&bars->acc_free[i], kProd); }
    bars->abort_flag = 0;
    fence_barrier_init();
  }
  // tensor memory: kNP tiles of P (64 columns each: 128 pairs, 16-bit), then the two accumulators
  if (warp == 0) tmem_alloc<512>(&bars->tmem_slot);
  // T of this (b, h): largest magnitude, then 16-bit copies scaled into [1, 2) at the top
  const float* tb = Tm + (long long)bh * (kTD * kTD * kTD);
  float mx = 0.f;
  for (int e = tid; e < kTD * kTD * kTD; e += kThreadsT) mx = fmaxf(mx, fabsf(tb[e]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) sRed[warp] = mx;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  mx = 0.f;
  for (int w = 0; w < kThreadsT / 32; ++w) mx = fmaxf(mx, sRed[w]);
  // a power of two: exact in every format
  int ex = 0;
  if (mx > 0.f && isfinite(mx)) frexpf(mx, &ex);
  const float tscale = ldexpf(1.f, 1 - ex), tinv = ldexpf(1.f, ex - 1);
  {
    // memory order of T is [d0][d1][d2] with strides (1024, 32, 1): which of x, y, z each one is follows from
    // the strides the caller gave
    const int xs = sx == 1024 ? 0 : (sx == 32 ? 1 : 2), ys = sy == 1024 ? 0 : (sy == 32 ? 1 : 2), zs = 3 - xs - ys;
    T16* tt = reinterpret_cast<T16*>(sT);
    for (int e = tid; e < kTD * kTD * kTD; e += kThreadsT) {
      const int d[3] = {e >> 10, (e >> 5) & 31, e & 31};
      const int x = d[xs], y = d[ys], z = d[zs];
      const int row = y * kTD + z;
      tt[(swz_off<64>(row, x >> 3) >> 1) + (x & 7)] = from_f32<T16>(tb[e] * tscale);
    }
  }
  fence_proxy_async();
  __syncthreads();
  const uint32_t tmem = bars->tmem_slot;
  int* abort_flag = &bars->abort_flag;
  const T16* a = A + (long long)bh * N * kTD;
  const T16* b = Bm + (long long)bh * N * kTD;
  T16* o = O + (long long)bh * N * kTD;
  constexpr int F = Op16<T16>::kFmt;
  const float oscale = alpha * tinv;
  constexpr uint32_t kAcc = 64 * kNP;              // + 64 iw + 32 par: one accumulator per issuing warp and tile parity

  if (warp < kProd / 32) {
    // ================= producers; they also write out the finished tile =================
    const int n = tid & 127, hk = tid >> 7;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    auto write_tile = [&](int t) {                 // tokens x 32 accumulator of tile t -> out (16 columns per thread)
      const int par = t & 1;
      mbar_wait(&bars->acc_full[par], (uint32_t)(t >> 1) & 1, status, abort_flag);
      tc_fence_after();
      uint32_t r[16], r2[16];
      tmem_ld16(lane_base + kAcc + 32 * par + 16 * hk, r);
      tmem_ld16(lane_base + kAcc + 64 + 32 * par + 16 * hk, r2);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) + __uint_as_float(r2[i]));
      tc_fence_before();
      arrive(&bars->acc_free[par]);
      const long long tok = (long long)n0 + t * 128 + n;
      if (tok < n1) {
        uint4 w0, w1;
        w0.x = Op16<T16>::pack(__uint_as_float(r[0]) * oscale, __uint_as_float(r[1]) * oscale);
        w0.y = Op16<T16>::pack(__uint_as_float(r[2]) * oscale, __uint_as_float(r[3]) * oscale);
        w0.z = Op16<T16>::pack(__uint_as_float(r[4]) * oscale, __uint_as_float(r[5]) * oscale);
        w0.w = Op16<T16>::pack(__uint_as_float(r[6]) * oscale, __uint_as_float(r[7]) * oscale);
        w1.x = Op16<T16>::pack(__uint_as_float(r[8]) * oscale, __uint_as_float(r[9]) * oscale);
        w1.y = Op16<T16>::pack(__uint_as_float(r[10]) * oscale, __uint_as_float(r[11]) * oscale);
        w1.z = Op16<T16>::pack(__uint_as_float(r[12]) * oscale, __uint_as_float(r[13]) * oscale);
        w1.w = Op16<T16>::pack(__uint_as_float(r[14]) * oscale, __uint_as_float(r[15]) * oscale);
        uint4* dst = reinterpret_cast<uint4*>(o + tok * kTD + 16 * hk);
        dst[0] = w0; dst[1] = w1;
      }
    };
    uint32_t uw[16], ww[8], un[16], wn[8];
    load_rows<T16>(a, b, (long long)n0 + n, (long long)n0 + n < n1, hk, un, wn);
    for (int t = 0; t < T; ++t) {
#pragma unroll
      for (int i = 0; i < 16; ++i) uw[i] = un[i];
#pragma unroll
      for (int i = 0; i < 8; ++i) ww[i] = wn[i];
      if (t + 1 < T) {                             // the next tile's rows, fetched while this one is worked
        const long long tok = (long long)n0 + (t + 1) * 128 + n;
        load_rows<T16>(a, b, tok, tok < n1, hk, un, wn);
      }
      // two tiles of P per round trip of the tensor-memory stores
#pragma unroll
      for (int blk = 0; blk < 8; blk += 2) {
        const int g = 8 * t + blk, buf = g % kNP, buf1 = (g + 1) % kNP;
        if (g >= kNP) {
          mbar_wait_hot(&bars->empty[buf], (uint32_t)(g / kNP - 1) & 1, status, abort_flag);
          mbar_wait_hot(&bars->empty[buf1], (uint32_t)((g + 1) / kNP - 1) & 1, status, abort_flag);
        }
        build_pairs_tmem<T16>(lane_base + 64 * buf, hk, blk, uw, ww);
        build_pairs_tmem<T16>(lane_base + 64 * buf1, hk, blk + 1, uw, ww);
        tmem_wait_st();
        tc_fence_before();
        arrive(&bars->full[buf]);
        arrive(&bars->full[buf1]);
      }
      if (*reinterpret_cast<volatile int*>(abort_flag)) break;
      if (t > 0) write_tile(t - 1);
    }
    if (!*reinterpret_cast<volatile int*>(abort_flag)) write_tile(T - 1);
  } else {
    // ================= issuing warp =================
    const uint32_t idesc = idesc_f16(128, kTD, F, F, 0, 1);          // A (tokens x pairs) in tensor memory, B (pairs x x) MN-major
    const uint64_t tdesc = smem_desc<64>(smem_u32(sT));
    const int iw = warp - kProd / 32;              // this issuing warp takes the blocks iw, iw + 2, ... into its own accumulator
    for (int t = 0; t < T; ++t) {
      const int par = t & 1;
      if (t >= 2) mbar_wait(&bars->acc_free[par], (uint32_t)((t - 2) >> 1) & 1, status, abort_flag);
      for (int blk = iw; blk < 8; blk += 2) {
        const int g = 8 * t + blk, buf = g % kNP;
        mbar_wait_hot(&bars->full[buf], (uint32_t)(g / kNP) & 1, status, abort_flag);
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            mma_ts(tmem + kAcc + 64 * iw + 32 * par, tmem + 64 * buf + 8 * kk, tdesc + (uint64_t)(64 * (8 * blk + kk)), idesc,
                   (blk > iw) || (kk > 0));
          mma_commit(&bars->empty[buf]);
          if (blk >= 6) mma_commit(&bars->acc_full[par]);
        }
        __syncwarp();
        if (*reinterpret_cast<volatile int*>(abort_flag)) break;
      }
      if (*reinterpret_cast<volatile int*>(abort_flag)) break;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc<512>(tmem);
}

int splits_for(int BH, int N) {
  long long s = num_sms() / BH;                    // one CTA per SM, one wave
  const long long max_s = (N + 511) / 512;         // at least four token tiles per CTA
  if (s > max_s) s = max_s;
  if (s < 1) s = 1;
  return (int)s;
}

}  // namespace

bool triple_tc_supported(int N, int D0, int D1, int D2, int dtype) {
  return (dtype == FLARE_BF16 || dtype == FLARE_F16) && D0 == kTD && D1 == kTD && D2 == kTD && N >= 128;
}

size_t triple_tc_outer_workspace(int BH, int N) {
  return (size_t)splits_for(BH, N) * BH * kTD * kTD * kTD * sizeof(float) + 256;
}

template <typename T16>
static int outer_launch(int BH, int N, const void* a, const void* b, const void* c, float alpha, float* out, float* ws,
                        cudaStream_t st) {
  const int S = splits_for(BH, N);
  const int chunk = ((N + S - 1) / S + 127) / 128 * 128;
  const int S2 = (N + chunk - 1) / chunk;
  float* part = S2 == 1 ? out : ws;
  constexpr int smem = kNP * kPBytes + 2 * kBBytes + 1024 + 256;
  if (tc_set_dyn_smem(reinterpret_cast<const void*>(&k_triple_tc_outer<T16>), smem) != FLARE_OK) return FLARE_ECUDA;
  k_triple_tc_outer<T16><<<dim3((unsigned)S2, (unsigned)BH), kThreadsT, smem, st>>>(
      reinterpret_cast<const T16*>(a), reinterpret_cast<const T16*>(b), reinterpret_cast<const T16*>(c), N, chunk, alpha,
      part, tc_status_ptr());
  if (S2 > 1) launch_reduce_sum(part, S2, (long long)BH * kTD * kTD * kTD, out, st);
  return FLARE_OK;
}

int triple_tc_outer(int BH, int N, int dtype, const void* a, const void* b, const void* c, float alpha, float* out,
                    float* ws, cudaStream_t st) {
  return dtype == FLARE_F16 ? outer_launch<__half>(BH, N, a, b, c, alpha, out, ws, st)
                            : outer_launch<__nv_bfloat16>(BH, N, a, b, c, alpha, out, ws, st);
}

template <typename T16>
static int contract_launch(int BH, int N, const float* t, long long sx, long long sy, long long sz, const void* a,
                           const void* b, float alpha, void* out, cudaStream_t st) {
  const int S = splits_for(BH, N);
  const int chunk = ((N + S - 1) / S + 127) / 128 * 128;
  const int S2 = (N + chunk - 1) / chunk;
  constexpr int smem = kTBytes + 1024 + 512;
  if (tc_set_dyn_smem(reinterpret_cast<const void*>(&k_triple_tc_contract<T16>), smem) != FLARE_OK) return FLARE_ECUDA;
  k_triple_tc_contract<T16><<<dim3((unsigned)S2, (unsigned)BH), kThreadsT, smem, st>>>(
      t, sx, sy, sz, reinterpret_cast<const T16*>(a), reinterpret_cast<const T16*>(b), N, chunk, alpha,
      reinterpret_cast<T16*>(out), tc_status_ptr());
  return FLARE_OK;
}

// T must be a permutation of a contiguous [32][32][32] tensor per (b, h): strides {1024, 32, 1} in some order
bool triple_tc_strides_ok(long long sx, long long sy, long long sz) {
  const long long s[3] = {sx, sy, sz};
  int seen = 0;
  for (int i = 0; i < 3; ++i) {
    if (s[i] == 1024) seen |= 1; else if (s[i] == 32) seen |= 2; else if (s[i] == 1) seen |= 4; else return false;
  }
  return seen == 7;
}

int triple_tc_contract(int BH, int N, int dtype, const float* t, long long sx, long long sy, long long sz, const void* a,
                       const void* b, float alpha, void* out, cudaStream_t st) {
  return dtype == FLARE_F16 ? contract_launch<__half>(BH, N, t, sx, sy, sz, a, b, alpha, out, st)
                            : contract_launch<__nv_bfloat16>(BH, N, t, sx, sy, sz, a, b, alpha, out, st);
}

}  // namespace flare
