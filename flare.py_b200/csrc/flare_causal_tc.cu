// Causal FLARE prefill, pass 3 on the tensor cores (bf16, M <= 128, D in {32, 64}).
//
// One CTA per (b, h, 128-token chunk) starts from the chunk's prefix (m0, l0 per latent, acc0 in 16 bits) and writes the
// chunk's y.  In the chunked form every contraction is a product (S = scale q k^T, mu = max(m0, rowmax S),
// a = e^{m0 - mu}, E = e^{S - mu}, l_mt = a l0 + cumsum_t E, A = softmax_M(S), G = A / l):
//
//   y_t = sum_m G_mt (a_m acc0_m)  +  sum_{n <= t} W_tn v_n,        W_tn = sum_m G_mt E_mn
//
//   1. S [latent lanes x token columns] and S^T [token lanes x latent columns]: two tcgen05 products, so that
//      the softmax over the latents (per token) and the running sum over the tokens (per latent) are both walks
//      along a thread's own tensor-memory row
//   2. token threads: column maximum and sum of S^T -> one factor w_t per token in shared memory
//   3. latent threads: mu, a, E, l (running sum), G' = E u_m / l (G = G' w_t: the token factor is common to row t
//      of W and Y and is applied to y at the end); E and G' rows as bf16 into shared memory, laid out as the
//      MN-major operands of the next product (contraction over the latents); a * acc0 as bf16 beside them
//   4. W = G^T E (token lanes x token columns) and Y = G^T (a acc0): products from shared memory
//   5. token threads: W masked to n <= t, packed to bf16 in place in tensor memory
//   6. Y += W V: A operand from tensor memory, V tile as loaded by TMA
//   7. token threads: w_t Y -> y
//
// 128 row threads (a thread is latent m in steps 3 and token t in steps 2, 5, 7) and one issuing warp; every
// wait is bounded.  bf16 only: E and G are relative to the chunk's final maximum and need the exponent range
// of fp32 before that maximum is reached.  A chunk whose scores climb by more than 64 octaves is flagged and
// redone by the fp32 walk, which carries a running maximum.  Two CTAs per SM (256 tensor-memory columns and
// under 100 KB of shared memory each) so that one chunk's products and loads overlap another's arithmetic.
#include <type_traits>
#include "common.cuh"
#include "launch.h"
#include "tc_common.cuh"
#include "tma_host.h"

namespace flare {

using namespace tc;

namespace {

constexpr int kRows = 128;                         // row threads = latents = tokens of a chunk
constexpr int kThreadsW = kRows + 32;

struct CausalTcArgs {
  int B, H, N, M;
  float scale_log2;
  int q_batched;
  const __nv_bfloat16* pacc;                       // [chunks][B][H][M][D]: acc of the prefix before every chunk
  const float2* pml;                               // [chunks][B][H][M]: its (m, l)
  __nv_bfloat16* y;
  long long ys[3];
  int* redo;                                       // [chunks][B*H]: 1 = this chunk's scores span too many octaves
  int* status;
};

__device__ __forceinline__ void arrive_w(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void rows_sync() {      // the 256 row threads
  asm volatile("bar.sync 1, 256;" ::: "memory");
}

// 256 row threads: thread (r, hb) owns row r (tensor-memory lane r) and the column half hb of every pass, so that a
// pass is two blocks of 32 columns per thread and eight warps share the latency of one chunk.
constexpr int kRowT = 256;
constexpr int kThreadsW2 = kRowT + 32;

template <int D>
__global__ void __launch_bounds__(kThreadsW2, 2)
k_causal_tc_walk(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, CausalTcArgs a) {
  grid_dep_sync();
  constexpr int ROWB = 2 * D, CPR = ROWB / 16, W = D + 2;
  constexpr int kTile = 128 * ROWB;                // Q, K, V, a*acc0
  constexpr int kHalf = 128 * 128;                 // 64-token half of the E / G tiles
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // Two CTAs per SM: Q and K are dead once S and S^T are complete, and G takes their place
  uint8_t* sG = smem;                              // [2 halves][latent rows][64 tokens]
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kTile;
  uint8_t* sE = sG + 2 * kHalf;
  uint8_t* sV = sE + 2 * kHalf;
  uint8_t* sA0 = sV + kTile;                       // a_m acc0_m as bf16: [latent][D]
  static_assert(2 * kTile <= 2 * kHalf, "Q and K must fit in the G tile");
  float* sCinv = reinterpret_cast<float*>(sA0 + kTile);      // [128] w_t (0 past the end of the sequence)
  float2* sPart = reinterpret_cast<float2*>(sCinv + 128);    // [2][128] (maximum, sum) of a token over half the latents
  float* sMuP = reinterpret_cast<float*>(sPart + 256);       // [2][128] maximum of a latent over half the tokens
  uint64_t* bars = reinterpret_cast<uint64_t*>(sMuP + 256);
  uint64_t* bar_load = bars;                       // Q, K, V landed
  uint64_t* bar_s = bars + 1;                      // S, S^T complete
  uint64_t* bar_ge = bars + 2;                     // E, G, a*acc0 written (256 arrivals)
  uint64_t* bar_w = bars + 3;                      // W and the first part of Y complete
  uint64_t* bar_wp = bars + 4;                     // masked W packed (256 arrivals)
  uint64_t* bar_y = bars + 5;                      // Y complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);
  int* abort_flag = reinterpret_cast<int*>(bars + 7);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int chunk = blockIdx.x, bh = blockIdx.y;
  const int b = bh / a.H, h = bh % a.H;
  const int n0 = chunk * 128;
  const int cnt = min(128, a.N - n0);
  const int M = a.M;

  if (tid == 0) {
    mbar_init(bar_load, 1); mbar_init(bar_s, 1); mbar_init(bar_ge, kRowT); mbar_init(bar_w, 1);
    mbar_init(bar_wp, kRowT); mbar_init(bar_y, 1);
    abort_flag[0] = 0;
    abort_flag[1] = 0;                             // range flag of this chunk
    fence_barrier_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
    // the loads start before tensor memory is allocated and the CTA has met
    mbar_expect_tx(bar_load, 3 * kTile);
    tma_load_4d(sQ, &tmQ, bar_load, 0, 0, h, a.q_batched ? b : 0);      // rows past M arrive as zeros
    tma_load_4d(sK, &tmK, bar_load, 0, n0, h, b);                       // rows past N arrive as zeros
    tma_load_4d(sV, &tmV, bar_load, 0, n0, h, b);
  }
  if (warp == 1) tmem_alloc<256>(tmem_slot);     // beside warp 0, whose first thread is issuing the loads
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // W takes the columns of S once every latent thread has read its row, Y those of S^T; the packed W sits behind Y
  constexpr uint32_t cS = 0, cST = 128, cW = 0, cY = 128, cWp = 192;

  if (warp == kRowT / 32) {
    // ================= issuing warp =================
    const uint32_t id_s = idesc_f16(128, 128, 1, 1, 0, 0);          // S, S^T: A, B K-major
    const uint32_t id_w = idesc_f16(128, 128, 1, 1, 1, 1);          // W: A = G, B = E, both MN-major over two 64-token blocks
    const uint32_t id_y0 = idesc_f16(128, D, 1, 1, 1, 1);           // Y = G^T (a acc0): A, B MN-major
    const uint32_t id_y1 = idesc_f16(128, D, 1, 1, 0, 1);           // Y += W V: A in tensor memory, B MN-major
    const uint64_t dQ = smem_desc<ROWB>(smem_u32(sQ)), dK = smem_desc<ROWB>(smem_u32(sK)), dV = smem_desc<ROWB>(smem_u32(sV)),
                   dA0 = smem_desc<ROWB>(smem_u32(sA0));
    const uint64_t dG = smem_desc_mn128(smem_u32(sG), kHalf, 1024);
    const uint64_t dE = smem_desc_mn128(smem_u32(sE), kHalf, 1024);
    mbar_wait(bar_load, 0, a.status, abort_flag);
    tc_fence_after();
    if (elect_one()) {
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) mma_ss(tmem + cS, dQ + 2 * kk, dK + 2 * kk, id_s, kk > 0);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) mma_ss(tmem + cST, dK + 2 * kk, dQ + 2 * kk, id_s, kk > 0);
      mma_commit(bar_s);
    }
    __syncwarp();
    mbar_wait(bar_ge, 0, a.status, abort_flag);
    tc_fence_after();
    if (elect_one()) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {             // contraction over the latents, 16 per product
        mma_ss(tmem + cW, dG + 128 * kk, dE + 128 * kk, id_w, kk > 0);
        mma_ss(tmem + cY, dG + 128 * kk, dA0 + (uint64_t)(kk * ROWB), id_y0, kk > 0);
      }
      mma_commit(bar_w);
    }
    __syncwarp();
    mbar_wait(bar_wp, 0, a.status, abort_flag);
    tc_fence_after();
    if (elect_one()) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)               // contraction over the chunk's tokens
        mma_ts(tmem + cY, tmem + cWp + 8 * kk, dV + (uint64_t)(kk * ROWB), id_y1, true);
      mma_commit(bar_y);
    }
    __syncwarp();
  } else {
    // ================= row threads: token r in steps 2, 5, 7, latent r in step 3; column half hb =================
    const int r = 32 * (warp & 3) + lane, hb = warp >> 2;
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const float sl = a.scale_log2;
    // the prefix of this chunk as the scan left it: (m, l) per latent, acc0 rows in 16 bits
    const long long prow = (((long long)chunk * a.B + b) * a.H + h) * M;
    const float2 ml0 = a.pml[prow + min(r, M - 1)];
    const float m0 = ml0.x, l0 = ml0.y;
    const bool live = r < M;
    // The acc0 rows are one contiguous block of M x D 16-bit values: the row threads fetch it with asynchronous
    // 16-byte copies now, while the tiles and the score products are on their way, into the bytes E takes later, in
    // the layout of the operand tile they become once scaled by a_m.  (A thread reading its own row of an fp32
    // record in the middle of step 3 cost 2600-4800 clocks per chunk.)
    {
      constexpr int NIT = 128 * CPR / kRowT;       // 16-byte pieces per thread: 4 (D = 64), 2 (D = 32)
      const uint4* blk = reinterpret_cast<const uint4*>(a.pacc + prow * D);
#pragma unroll
      for (int it = 0; it < NIT; ++it) {
        const int i16 = tid + kRowT * it;
        const int row = i16 / CPR, ch = i16 % CPR;
        if (row < M) {
          const uint32_t dst = smem_u32(sE + swz_off<ROWB>(row, ch));
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(blk + i16) : "memory");
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    }

    mbar_wait(bar_s, 0, a.status, abort_flag);
    tc_fence_after();
    // Steps 2 to 5, compiled twice: a full chunk with all 128 latents needs none of the per-score bounds tests.
    auto steps = [&](auto full_chunk) {
    constexpr bool FULL = decltype(full_chunk)::value;
    // ---- step 2: token r over the latents 64 hb ... 64 hb + 63: maximum and sum relative to it ----
    {
      float mx = -INFINITY, su = 0.f;
      row_half_pass(lane_base + cST + 64 * hb, [&](int c, const uint32_t (&v)[32]) {
#pragma unroll
        for (int j = 0; j < 32; ++j) if (FULL || 64 * hb + 32 * c + j < M) mx = fmaxf(mx, __uint_as_float(v[j]) * sl);
      });
      row_half_pass(lane_base + cST + 64 * hb, [&](int c, const uint32_t (&v)[32]) {
#pragma unroll
        for (int j = 0; j < 32; ++j) if (FULL || 64 * hb + 32 * c + j < M) su += ex2(fmaf(__uint_as_float(v[j]), sl, -mx));
      });
      sPart[hb * 128 + r] = make_float2(mx, su);
    }
    // ---- step 3, first pass: latent r over the tokens 64 hb ... 64 hb + 63: maximum ----
    float first = m0 * kLog2e;                     // hb == 0: the running maximum after the chunk's first token
    {
      float mp = -INFINITY;
      row_half_pass(lane_base + cS + 64 * hb, [&](int c, const uint32_t (&v)[32]) {
#pragma unroll
        for (int j = 0; j < 32; ++j) if (FULL || 64 * hb + 32 * c + j < cnt) mp = fmaxf(mp, __uint_as_float(v[j]) * sl);
        if (c == 0) first = fmaxf(first, __uint_as_float(v[0]) * sl);
      });
      sMuP[hb * 128 + r] = mp;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");       // this thread's part of the staged rows has landed
    rows_sync();
    // A_mt = 2^(S_mt - cmax_t) / csum_t is formed from the exponential that E needs anyway:
    //   A_mt = E_mt * u_m * w_t,   u_m = 2^(mu_m - c0),   w_t = 2^(c0 - cmax_t) / csum_t   (w_t applied in step 7),
    // with c0 the column maximum of the chunk's first token (every thread reads it from the same two words).
    // |mu_m - c0| and |cmax_t - c0| are kept within 50 octaves, so that no factor leaves fp32's range while A_mt
    // still matters; a chunk outside that is flagged and redone like one whose scores climb too far.
    const float c0 = fmaxf(sPart[0].x, sPart[128].x);
    if (hb == 0) {                                 // the two halves of token r's statistics
      const float2 p0 = sPart[r], p1 = sPart[128 + r];
      const float cm = fmaxf(p0.x, p1.x);
      const float cs = p0.y * ex2(p0.x - cm) + (p1.x == -INFINITY ? 0.f : p1.y * ex2(p1.x - cm));
      const bool in = r < cnt;
      sCinv[r] = in ? __fdividef(ex2(c0 - cm), cs) : 0.f;
      if (in && fabsf(c0 - cm) > 50.f) abort_flag[1] = 1;
    }
    const float mu = fmaxf(m0 * kLog2e, fmaxf(sMuP[r], sMuP[128 + r]));   // the record keeps m in natural-log units
    const float aa = (m0 == -INFINITY) ? 0.f : ex2(m0 * kLog2e - mu);
    // a * acc0 of this latent, half of its D values, from the staged rows (E overwrites them after the barrier)
#pragma unroll
    for (int cc = 0; cc < CPR / 2; ++cc) {
      const int c = hb * (CPR / 2) + cc;
      uint4 o = make_uint4(0, 0, 0, 0);
      if (FULL || live) {
        const uint4 x = *reinterpret_cast<const uint4*>(sE + swz_off<ROWB>(r, c));
        const uint32_t xw[4] = {x.x, x.y, x.z, x.w};
        uint32_t ow[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = Op16<__nv_bfloat16>::unpack(xw[j]);
          ow[j] = pack_bf16(f.x * aa, f.y * aa);
        }
        o = make_uint4(ow[0], ow[1], ow[2], ow[3]);
      }
      *reinterpret_cast<uint4*>(sA0 + swz_off<ROWB>(r, c)) = o;
    }
    rows_sync();

    // ---- step 3: latent r: a, E, running l, G over its half of the tokens; a * acc0 over its half of D ----
    {
      // E and l are relative to the chunk's final maximum: l_mt >= 2^(first - mu).  Past 64 octaves the chunk is
      // handed to the walk that carries a running maximum (flagged; its y overwrites this kernel's).
      if (hb == 0 && live && (mu - first > 64.f || fabsf(mu - c0) > 50.f)) abort_flag[1] = 1;
      const float um = live ? ex2(fminf(fmaxf(mu - c0, -60.f), 60.f)) : 0.f;
      float l = aa * l0;
      if (hb == 1) {                               // the sum over the first half, in the order its owner adds it
        row_half_pass(lane_base + cS, [&](int c, const uint32_t (&v)[32]) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            l += (FULL || (live && 32 * c + j < cnt)) ? ex2(fmaf(__uint_as_float(v[j]), sl, -mu)) : 0.f;
        });
      }
      uint8_t* eh = sE + hb * kHalf;
      uint8_t* gh = sG + hb * kHalf;
      row_half_pass(lane_base + cS + 64 * hb, [&](int c, const uint32_t (&v)[32]) {
        uint32_t pe[16], pg[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          float e2[2], g2[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int t = 64 * hb + 32 * c + j + u;
            const float x = __uint_as_float(v[j + u]);
            const bool in = FULL || (live && t < cnt);
            const float e = in ? ex2(fmaf(x, sl, -mu)) : 0.f;
            l += e;
            e2[u] = e;
            // G without its token factor w_t, which is common to row t of W and Y and applied to y in step 7
            g2[u] = (FULL || l > 0.f) ? e * __fdividef(um, l) : 0.f;   // l = 0 only in a chunk that is flagged and redone
          }
          pe[j >> 1] = pack_bf16(e2[0], e2[1]);
          pg[j >> 1] = pack_bf16(g2[0], g2[1]);
        }
        // 32 tokens = four 16-byte chunks of this thread's 64-token half
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const uint32_t off = swz_off<128>(r, 4 * c + q4);
          *reinterpret_cast<uint4*>(eh + off) = make_uint4(pe[4 * q4], pe[4 * q4 + 1], pe[4 * q4 + 2], pe[4 * q4 + 3]);
          *reinterpret_cast<uint4*>(gh + off) = make_uint4(pg[4 * q4], pg[4 * q4 + 1], pg[4 * q4 + 2], pg[4 * q4 + 3]);
        }
      });
      fence_proxy_async();
      tc_fence_before();
      arrive_w(bar_ge);
    }

    // ---- step 5: token r: its half of W masked to n <= r (and to the tokens that exist), packed behind Y ----
    mbar_wait(bar_w, 0, a.status, abort_flag);
    tc_fence_after();
    if (r == 0 && hb == 0) a.redo[chunk * gridDim.y + bh] = abort_flag[1];
    if (hb == 1 && (warp & 3) < 2) {               // tokens 0 ... 63 see none of the columns 64 ... 127
      uint32_t z[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) z[j] = 0u;
      tmem_st16(lane_base + cWp + 32, z);
      tmem_st16(lane_base + cWp + 48, z);
    } else {
      row_half_pass(lane_base + cW + 64 * hb, [&](int c, const uint32_t (&v)[32]) {
        uint32_t pw[16];
        const int cb = 2 * hb + c, rb = warp & 3;  // column block against this warp's row block: the same for all lanes
        if (FULL && cb < rb) {                     // below the diagonal: nothing to mask
#pragma unroll
          for (int j = 0; j < 32; j += 2) pw[j >> 1] = pack_bf16(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
        } else if (cb > rb) {                      // above it: nothing to keep
#pragma unroll
          for (int j = 0; j < 16; ++j) pw[j] = 0u;
        } else {
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const int n = 64 * hb + 32 * c + j;
            const float w0 = (n <= r && (FULL || n < cnt)) ? __uint_as_float(v[j]) : 0.f;
            const float w1 = (n + 1 <= r && (FULL || n + 1 < cnt)) ? __uint_as_float(v[j + 1]) : 0.f;
            pw[j >> 1] = pack_bf16(w0, w1);
          }
        }
        tmem_st16(lane_base + cWp + 32 * hb + 16 * c, pw);
      });
    }
    tmem_wait_st();
    tc_fence_before();
    arrive_w(bar_wp);
    };                                             // steps
    if (cnt == 128 && M == 128) steps(std::true_type{});
    else steps(std::false_type{});

    // ---- step 7: Y of token r, half of its D values -> y ----
    mbar_wait(bar_y, 0, a.status, abort_flag);
    tc_fence_after();
    if (!*reinterpret_cast<volatile int*>(abort_flag)) {
      __nv_bfloat16* yp = a.y + b * a.ys[0] + h * a.ys[1] + (long long)(n0 + r) * a.ys[2] + hb * (D / 2);
      uint32_t v[32];
      if constexpr (D == 64) tmem_ld32(lane_base + cY + 32 * hb, v);
      else tmem_ld16(lane_base + cY + 16 * hb, v);
      tmem_wait_ld();
      if (r < cnt) {
        const float wt = sCinv[r];                 // the token factor left out of G
#pragma unroll
        for (int q4 = 0; q4 < D / 16; ++q4) {
          uint4 o;
          o.x = pack_bf16(__uint_as_float(v[8 * q4]) * wt, __uint_as_float(v[8 * q4 + 1]) * wt);
          o.y = pack_bf16(__uint_as_float(v[8 * q4 + 2]) * wt, __uint_as_float(v[8 * q4 + 3]) * wt);
          o.z = pack_bf16(__uint_as_float(v[8 * q4 + 4]) * wt, __uint_as_float(v[8 * q4 + 5]) * wt);
          o.w = pack_bf16(__uint_as_float(v[8 * q4 + 6]) * wt, __uint_as_float(v[8 * q4 + 7]) * wt);
          reinterpret_cast<uint4*>(yp)[q4] = o;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc<256>(tmem);
}

// Pass 1 for the same shapes: the record (acc, m, l) of every 128-token chunk on its own.  S = scale q k^T,
// m = rowmax, E = e^{S - m} packed to bf16 in place in tensor memory, acc = E V.  128 tensor-memory columns and
// three operand tiles per CTA: four CTAs per SM.  acc leaves in 16 bits through shared memory as one contiguous block
// (the scan adds the records up in fp32; the walk multiplies 16-bit operands anyway), (m, l) as one pair per latent.
template <int D>
__global__ void __launch_bounds__(kThreadsW, 4)
k_causal_tc_record(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, CausalTcArgs a, __nv_bfloat16* __restrict__ racc,
                   float2* __restrict__ rml) {
  grid_dep_sync();
  constexpr int ROWB = 2 * D;
  constexpr int kTile = 128 * ROWB;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kTile;
  uint8_t* sV = sK + kTile;
  uint8_t* sOut = smem;                            // [128][D] in 16 bits (swizzled rows), over the operand tiles once the products are done
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + kTile);
  uint64_t* bar_load = bars;
  uint64_t* bar_s = bars + 1;
  uint64_t* bar_p = bars + 2;                      // E packed (128 arrivals)
  uint64_t* bar_acc = bars + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  int* abort_flag = reinterpret_cast<int*>(bars + 5);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int chunk = blockIdx.x, bh = blockIdx.y;
  const int b = bh / a.H, h = bh % a.H;
  const int n0 = chunk * 128;
  const int cnt = min(128, a.N - n0);
  const int M = a.M;

  if (tid == 0) {
    mbar_init(bar_load, 1); mbar_init(bar_s, 1); mbar_init(bar_p, kRows); mbar_init(bar_acc, 1);
    abort_flag[0] = 0;
    fence_barrier_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
    // the loads start before tensor memory is allocated and the CTA has met
    mbar_expect_tx(bar_load, 3 * kTile);
    tma_load_4d(sQ, &tmQ, bar_load, 0, 0, h, a.q_batched ? b : 0);
    tma_load_4d(sK, &tmK, bar_load, 0, n0, h, b);
    tma_load_4d(sV, &tmV, bar_load, 0, n0, h, b);
  }
  if (warp == 1) tmem_alloc<128>(tmem_slot);     // beside warp 0, whose first thread is issuing the loads
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  constexpr uint32_t cS = 0, cAcc = 64;            // E packed occupies columns [0, 64) when acc is written

  const int r = tid;
  const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
  float mx = -INFINITY, l = 0.f;
  if (warp == kRows / 32) {
    const uint32_t id_s = idesc_f16(128, 128, 1, 1, 0, 0);
    const uint32_t id_pv = idesc_f16(128, D, 1, 1, 0, 1);
    const uint64_t dQ = smem_desc<ROWB>(smem_u32(sQ)), dK = smem_desc<ROWB>(smem_u32(sK)), dV = smem_desc<ROWB>(smem_u32(sV));
    mbar_wait(bar_load, 0, a.status, abort_flag);
    tc_fence_after();
    if (elect_one()) {
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) mma_ss(tmem + cS, dQ + 2 * kk, dK + 2 * kk, id_s, kk > 0);
      mma_commit(bar_s);
    }
    __syncwarp();
    mbar_wait(bar_p, 0, a.status, abort_flag);
    tc_fence_after();
    if (elect_one()) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) mma_ts(tmem + cAcc, tmem + cS + 8 * kk, dV + (uint64_t)(kk * ROWB), id_pv, kk > 0);
      mma_commit(bar_acc);
    }
    __syncwarp();
    mbar_wait(bar_acc, 0, a.status, abort_flag);
  } else {
    const float sl = a.scale_log2;
    mbar_wait(bar_s, 0, a.status, abort_flag);
    tc_fence_after();
    row_pass(lane_base + cS, [&](int c, const uint32_t (&v)[32]) {
#pragma unroll
      for (int j = 0; j < 32; ++j) if (32 * c + j < cnt) mx = fmaxf(mx, __uint_as_float(v[j]) * sl);
    });
    row_pass(lane_base + cS, [&](int c, const uint32_t (&v)[32]) {
      uint32_t pe[16];
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        const float e0 = (32 * c + j < cnt) ? ex2(fmaf(__uint_as_float(v[j]), sl, -mx)) : 0.f;
        const float e1 = (32 * c + j + 1 < cnt) ? ex2(fmaf(__uint_as_float(v[j + 1]), sl, -mx)) : 0.f;
        l += e0 + e1;
        pe[j >> 1] = pack_bf16(e0, e1);
      }
      tmem_st16(lane_base + cS + 16 * c, pe);      // columns already read
    });
    tmem_wait_st();
    tc_fence_before();
    arrive_w(bar_p);
    mbar_wait(bar_acc, 0, a.status, abort_flag);
    tc_fence_after();
  }
  __syncthreads();                                 // the products are complete: the operand tiles are free
  const long long prow = (((long long)chunk * a.B + b) * a.H + h) * M;      // first row of this record
  if (warp < kRows / 32) {                         // whole warps: rows past M are staged and not copied out
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      uint32_t v[32];
      tmem_ld32(lane_base + cAcc + 32 * c, v);
      tmem_wait_ld();
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        uint4 o;
        o.x = pack_bf16(__uint_as_float(v[8 * q4]), __uint_as_float(v[8 * q4 + 1]));
        o.y = pack_bf16(__uint_as_float(v[8 * q4 + 2]), __uint_as_float(v[8 * q4 + 3]));
        o.z = pack_bf16(__uint_as_float(v[8 * q4 + 4]), __uint_as_float(v[8 * q4 + 5]));
        o.w = pack_bf16(__uint_as_float(v[8 * q4 + 6]), __uint_as_float(v[8 * q4 + 7]));
        *reinterpret_cast<uint4*>(sOut + swz_off<ROWB>(r, 4 * c + q4)) = o;
      }
    }
    if (r < M && !*reinterpret_cast<volatile int*>(abort_flag)) rml[prow + r] = make_float2(mx * kLn2, l);
  }
  __syncthreads();
  // acc of this (chunk, b, h): M x D contiguous 16-bit values
  if (!*reinterpret_cast<volatile int*>(abort_flag)) {
    uint4* dst = reinterpret_cast<uint4*>(racc + prow * D);
    constexpr int CPR = ROWB / 16;
    for (int i = tid; i < M * CPR; i += kThreadsW) dst[i] = *reinterpret_cast<const uint4*>(sOut + swz_off<ROWB>(i / CPR, i % CPR));
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc<128>(tmem);
}

struct TcLaunch {
  CUtensorMap tmQ, tmK, tmV;
  CausalTcArgs a;
};

template <int D>
int fill_launch(const FlareProblem* p, const void* q, const void* k, const void* v, TcLaunch* L) {
  CUtensorMap &tmQ = L->tmQ, &tmK = L->tmK, &tmV = L->tmV;
  const uint64_t e = 2;
  const bool qb = p->q_stride[0] != 0;
  if (!make_tile_map(&tmQ, q, 1, D, (uint64_t)p->M, (uint64_t)p->H, (uint64_t)(qb ? p->B : 1), p->q_stride[2] * e,
                     p->q_stride[1] * e, (qb ? p->q_stride[0] : p->q_stride[1] * p->H) * e, 128) ||
      !make_tile_map(&tmK, k, 1, D, (uint64_t)p->N, (uint64_t)p->H, (uint64_t)p->B, p->k_stride[2] * e, p->k_stride[1] * e,
                     (p->B > 1 ? p->k_stride[0] : p->k_stride[1] * p->H) * e, 128) ||
      !make_tile_map(&tmV, v, 1, D, (uint64_t)p->N, (uint64_t)p->H, (uint64_t)p->B, p->v_stride[2] * e, p->v_stride[1] * e,
                     (p->B > 1 ? p->v_stride[0] : p->v_stride[1] * p->H) * e, 128))
    return FLARE_EUNSUPPORTED;
  CausalTcArgs& a = L->a;
  a.B = p->B; a.H = p->H; a.N = p->N; a.M = p->M;
  a.scale_log2 = p->scale * kLog2e;
  a.q_batched = qb ? 1 : 0;
  a.pacc = nullptr; a.pml = nullptr; a.y = nullptr; a.redo = nullptr;
  for (int i = 0; i < 3; ++i) a.ys[i] = p->y_stride[i];
  a.status = tc_status_ptr();
  return FLARE_OK;
}

template <int D>
int launch_walk_tc(const FlareProblem* p, const void* q, const void* k, const void* v, void* y, const __nv_bfloat16* pacc,
                   const float2* pml, int* redo, int chunks, cudaStream_t st) {
  TcLaunch L;
  const int rc = fill_launch<D>(p, q, k, v, &L);
  if (rc != FLARE_OK) return rc;
  CausalTcArgs& a = L.a;
  const CUtensorMap &tmQ = L.tmQ, &tmK = L.tmK, &tmV = L.tmV;
  a.pacc = pacc; a.pml = pml;
  a.y = reinterpret_cast<__nv_bfloat16*>(y);
  a.redo = redo;
  constexpr int smem = 2 * 128 * 2 * D + 4 * 128 * 128 + 4096 + 256 + 1024;
  if (tc_set_dyn_smem(reinterpret_cast<const void*>(&k_causal_tc_walk<D>), smem) != FLARE_OK) return FLARE_ECUDA;
  launch_dep(k_causal_tc_walk<D>, dim3((unsigned)chunks, (unsigned)(p->B * p->H)), dim3(kThreadsW2), smem, st, tmQ, tmK, tmV, a);
  return FLARE_OK;
}

template <int D>
int launch_record_tc(const FlareProblem* p, const void* q, const void* k, const void* v, __nv_bfloat16* racc, float2* rml,
                     int chunks, cudaStream_t st) {
  TcLaunch L;
  const int rc = fill_launch<D>(p, q, k, v, &L);
  if (rc != FLARE_OK) return rc;
  constexpr int smem = 3 * 128 * 2 * D + 256 + 1024;
  if (tc_set_dyn_smem(reinterpret_cast<const void*>(&k_causal_tc_record<D>), smem) != FLARE_OK) return FLARE_ECUDA;
  launch_dep(k_causal_tc_record<D>, dim3((unsigned)chunks, (unsigned)(p->B * p->H)), dim3(kThreadsW), smem, st, L.tmQ, L.tmK,
             L.tmV, L.a, racc, rml);
  return FLARE_OK;
}

}  // namespace

// bf16, M <= 128, D in {32, 64}, rows the TMA can address (unit stride on D, 16-byte aligned strides)
bool causal_tc_walk_supported(const FlareProblem* p, const void* q, const void* k, const void* v, const void* y) {
  if (p->dtype != FLARE_BF16 || p->M < 1 || p->M > 128 || (p->D != 32 && p->D != 64)) return false;
  if ((long long)p->B * p->H > 65535) return false;
  auto ok = [&](const void* ptr, const int64_t* s) {
    if (reinterpret_cast<uintptr_t>(ptr) % 16) return false;
    for (int i = 0; i < 3; ++i) if ((s[i] * 2) % 16) return false;
    return true;
  };
  return ok(q, p->q_stride) && ok(k, p->k_stride) && ok(v, p->v_stride) && ok(y, p->y_stride);
}

int causal_tc_walk(const FlareProblem* p, const void* q, const void* k, const void* v, void* y, const __nv_bfloat16* pacc,
                   const float2* pml, int* redo, int chunks, cudaStream_t st) {
  return p->D == 32 ? launch_walk_tc<32>(p, q, k, v, y, pacc, pml, redo, chunks, st)
                    : launch_walk_tc<64>(p, q, k, v, y, pacc, pml, redo, chunks, st);
}

}  // namespace flare

namespace flare {
int causal_tc_record(const FlareProblem* p, const void* q, const void* k, const void* v, __nv_bfloat16* racc, float2* rml,
                     int chunks, cudaStream_t st) {
  return p->D == 32 ? launch_record_tc<32>(p, q, k, v, racc, rml, chunks, st)
                    : launch_record_tc<64>(p, q, k, v, racc, rml, chunks, st);
}
}  // namespace flare
