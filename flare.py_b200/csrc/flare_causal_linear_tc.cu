// Causal linear attention on the tensor cores: Y_t = Q_t . sum_{n <= t} K_n^T V_n / N for 16-bit inputs with
// Dk = 128 and Dv in {32, 64} (lra/models/triton/causal_linear.py:23-145; the shape of its main(): Dk 128, Dv 32).
//
// The token axis is cut into 128-token chunks, Y_c = Q_c P_c + tril(Q_c K_c^T) V_c / N with P_c the sum of K^T V / N
// over the chunks before c:
//   1. k_cl_tc_sums:   K_c^T V_c per chunk (one product, Dk lanes x Dv columns, fp32)            [chunks][Dk][Dv]
//   2. k_cl_tc_prefix: exclusive running sum over the chunks, scaled by 1/N, rounded to 16 bits   [chunks][Dk][Dv]
//   3. k_cl_tc_walk:   S = Q_c K_c^T and Y = Q_c P_c (shared-memory operands); the row threads mask S to n <= t,
//                      scale by 1/N and pack it to 16 bits in tensor memory; Y += S V_c takes it from there.
// A 128 x 128 row of 16-bit values is 256 bytes, two swizzle spans: Q and K arrive as two column blocks of 64, each a
// tile of its own.  Nothing of size N x Dk x Dv goes to HBM (the Triton path writes and re-reads two such fp32 arrays).
#include "common.cuh"
#include "launch.h"
#include "tc_common.cuh"
#include "tma_host.h"

namespace flare {

using namespace tc;

namespace {

constexpr int kDk = 128;
constexpr int kRowT = 256;                         // row threads of the walk: (row r, column half hb)
constexpr int kThreadsWalk = kRowT + 32;
constexpr int kThreadsSum = 128 + 32;

struct ClTcArgs {
  int B, H, N, chunks;
  float inv_n;
  float* sums;                                     // [B*H][chunks][Dk][Dv] fp32
  void* y;
  long long ys[3];
  int* status;
};

__device__ __forceinline__ void arrive_on(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// ---- pass 1: K_c^T V_c -------------------------------------------------------------------------------------------
template <typename T, int DV>
__global__ void __launch_bounds__(kThreadsSum, 4)
k_cl_tc_sums(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, ClTcArgs a) {
  grid_dep_sync();
  constexpr int F = Op16<T>::kFmt, ROWBV = 2 * DV;
  constexpr int kHalf = 128 * 128, kTileV = 128 * ROWBV;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;                              // [2 column blocks][128 tokens][64]
  uint8_t* sV = sK + 2 * kHalf;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + kTileV);
  uint64_t* bar_load = bars;
  uint64_t* bar_done = bars + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
  int* abort_flag = reinterpret_cast<int*>(bars + 3);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int chunk = blockIdx.x, bh = blockIdx.y;
  const int b = bh / a.H, h = bh % a.H;
  if (tid == 0) {
    mbar_init(bar_load, 1); mbar_init(bar_done, 1);
    abort_flag[0] = 0;
    fence_barrier_init();
    prefetch_tmap(&tmK); prefetch_tmap(&tmV);
    // the loads start before tensor memory is allocated and the CTA has met
    mbar_expect_tx(bar_load, 2 * kHalf + kTileV);
    tma_load_4d(sK, &tmK, bar_load, 0, chunk * 128, h, b);              // rows past N arrive as zeros
    tma_load_4d(sK + kHalf, &tmK, bar_load, 64, chunk * 128, h, b);
    tma_load_4d(sV, &tmV, bar_load, 0, chunk * 128, h, b);
  }
  if (warp == 1) tmem_alloc<64>(tmem_slot);       // beside warp 0, whose first thread is issuing the loads
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  if (warp == 4) {
    // A = K^T: contraction over the tokens (rows), Dk across two 64-column blocks; B = V rows, contiguous along Dv
    const uint32_t id = idesc_f16(128, DV, F, F, 1, 1);
    const uint64_t dK = smem_desc_mn128(smem_u32(sK), kHalf, 1024), dV = smem_desc<ROWBV>(smem_u32(sV));
    mbar_wait(bar_load, 0, a.status, abort_flag);
    tc_fence_after();
    if (elect_one()) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) mma_ss(tmem, dK + 128 * kk, dV + (uint64_t)(kk * ROWBV), id, kk > 0);
      mma_commit(bar_done);
    }
    __syncwarp();
  } else {
    const int r = tid;                             // row dk
    const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
    mbar_wait(bar_done, 0, a.status, abort_flag);
    tc_fence_after();
    if (!*reinterpret_cast<volatile int*>(abort_flag)) {
      float* out = a.sums + (((long long)bh * a.chunks + chunk) * kDk + r) * DV;
#pragma unroll
      for (int c = 0; c < DV / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(lane_base + 32 * c, v);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(out + 32 * c + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                                     __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc<64>(tmem);
}

// ---- pass 2: exclusive running sum over the chunks, scaled and rounded ---------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
k_cl_tc_prefix(const float* __restrict__ sums, T* __restrict__ prefix, int chunks, int per_chunk, long long total,
               float inv_n) {
  grid_dep_sync();
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;       // (bh, element pair of a chunk)
  if (i >= total) return;
  const long long bh = i / (per_chunk / 2);
  const int e = (int)(i % (per_chunk / 2)) * 2;
  const float* s = sums + bh * chunks * per_chunk + e;
  T* p = prefix + bh * chunks * per_chunk + e;
  float r0 = 0.f, r1 = 0.f;
  float2 nx = *reinterpret_cast<const float2*>(s);
  for (int c = 0; c < chunks; ++c) {
    const float2 cur = nx;
    if (c + 1 < chunks) nx = *reinterpret_cast<const float2*>(s + (long long)(c + 1) * per_chunk);
    *reinterpret_cast<uint32_t*>(p + (long long)c * per_chunk) = Op16<T>::pack(r0 * inv_n, r1 * inv_n);
    r0 += cur.x; r1 += cur.y;
  }
}

// ---- pass 3: the chunk itself --------------------------------------------------------------------------------------
template <typename T, int DV>
__global__ void __launch_bounds__(kThreadsWalk, 2)
k_cl_tc_walk(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
             const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmP, ClTcArgs a) {
  grid_dep_sync();
  constexpr int F = Op16<T>::kFmt, ROWBV = 2 * DV;
  constexpr int kHalf = 128 * 128, kTileV = 128 * ROWBV;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                              // [2 column blocks][128 tokens][64]
  uint8_t* sK = sQ + 2 * kHalf;
  uint8_t* sV = sK + 2 * kHalf;                    // [128 tokens][Dv]
  uint8_t* sP = sV + kTileV;                       // [128 dk][Dv]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + kTileV);
  uint64_t* bar_load = bars;
  uint64_t* bar_s = bars + 1;                      // S and Q P complete
  uint64_t* bar_p = bars + 2;                      // masked S packed (256 arrivals)
  uint64_t* bar_y = bars + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  int* abort_flag = reinterpret_cast<int*>(bars + 5);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int chunk = blockIdx.x, bh = blockIdx.y;
  const int b = bh / a.H, h = bh % a.H;
  const int n0 = chunk * 128;
  const int cnt = min(128, a.N - n0);
  if (tid == 0) {
    mbar_init(bar_load, 1); mbar_init(bar_s, 1); mbar_init(bar_p, kRowT); mbar_init(bar_y, 1);
    abort_flag[0] = 0;
    fence_barrier_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmP);
    // the loads start before tensor memory is allocated and the CTA has met
    mbar_expect_tx(bar_load, 4 * kHalf + 2 * kTileV);
    tma_load_4d(sQ, &tmQ, bar_load, 0, n0, h, b);
    tma_load_4d(sQ + kHalf, &tmQ, bar_load, 64, n0, h, b);
    tma_load_4d(sK, &tmK, bar_load, 0, n0, h, b);
    tma_load_4d(sK + kHalf, &tmK, bar_load, 64, n0, h, b);
    tma_load_4d(sV, &tmV, bar_load, 0, n0, h, b);
    tma_load_4d(sP, &tmP, bar_load, 0, 0, chunk, bh);
  }
  if (warp == 1) tmem_alloc<256>(tmem_slot);       // beside warp 0, whose first thread is issuing the loads
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  constexpr uint32_t cS = 0, cY = 128, cSp = 192;  // S fp32, Y, S masked and packed
  if (warp == kRowT / 32) {
    const uint32_t id_s = idesc_f16(128, 128, F, F, 0, 0);            // S: A = Q, B = K, both K-major
    const uint32_t id_y0 = idesc_f16(128, DV, F, F, 0, 1);            // Y = Q P: B rows are the contraction index
    const uint32_t id_y1 = idesc_f16(128, DV, F, F, 0, 1);            // Y += S V: A in tensor memory
    const uint64_t dQ0 = smem_desc<128>(smem_u32(sQ)), dQ1 = smem_desc<128>(smem_u32(sQ + kHalf));
    const uint64_t dK0 = smem_desc<128>(smem_u32(sK)), dK1 = smem_desc<128>(smem_u32(sK + kHalf));
    const uint64_t dV = smem_desc<ROWBV>(smem_u32(sV)), dP = smem_desc<ROWBV>(smem_u32(sP));
    mbar_wait(bar_load, 0, a.status, abort_flag);
    tc_fence_after();
    if (elect_one()) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint64_t aQ = (kk < 4 ? dQ0 : dQ1) + 2 * (kk & 3);
        mma_ss(tmem + cS, aQ, (kk < 4 ? dK0 : dK1) + 2 * (kk & 3), id_s, kk > 0);
        mma_ss(tmem + cY, aQ, dP + (uint64_t)(kk * ROWBV), id_y0, kk > 0);
      }
      mma_commit(bar_s);
    }
    __syncwarp();
    mbar_wait(bar_p, 0, a.status, abort_flag);
    tc_fence_after();
    if (elect_one()) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) mma_ts(tmem + cY, tmem + cSp + 8 * kk, dV + (uint64_t)(kk * ROWBV), id_y1, true);
      mma_commit(bar_y);
    }
    __syncwarp();
  } else {
    const int r = 32 * (warp & 3) + lane, hb = warp >> 2;             // token r, column half hb
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const float inv_n = a.inv_n;
    mbar_wait(bar_s, 0, a.status, abort_flag);
    tc_fence_after();
    if (hb == 1 && (warp & 3) < 2) {               // tokens 0 ... 63 see none of the columns 64 ... 127
      uint32_t z[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) z[j] = 0u;
      tmem_st16(lane_base + cSp + 32, z);
      tmem_st16(lane_base + cSp + 48, z);
    } else {
      row_half_pass(lane_base + cS + 64 * hb, [&](int c, const uint32_t (&v)[32]) {
        uint32_t pw[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const int n = 64 * hb + 32 * c + j;
          const float w0 = (n <= r) ? __uint_as_float(v[j]) * inv_n : 0.f;
          const float w1 = (n + 1 <= r) ? __uint_as_float(v[j + 1]) * inv_n : 0.f;
          pw[j >> 1] = Op16<T>::pack(w0, w1);
        }
        tmem_st16(lane_base + cSp + 32 * hb + 16 * c, pw);
      });
    }
    tmem_wait_st();
    tc_fence_before();
    arrive_on(bar_p);
    mbar_wait(bar_y, 0, a.status, abort_flag);
    tc_fence_after();
    if (!*reinterpret_cast<volatile int*>(abort_flag)) {
      T* yp = reinterpret_cast<T*>(a.y) + b * a.ys[0] + h * a.ys[1] + (long long)(n0 + r) * a.ys[2] + hb * (DV / 2);
      uint32_t v[32];
      if constexpr (DV == 64) tmem_ld32(lane_base + cY + 32 * hb, v);
      else tmem_ld16(lane_base + cY + 16 * hb, v);
      tmem_wait_ld();
      if (r < cnt) {
#pragma unroll
        for (int q4 = 0; q4 < DV / 16; ++q4) {
          uint4 o;
          o.x = Op16<T>::pack(__uint_as_float(v[8 * q4]), __uint_as_float(v[8 * q4 + 1]));
          o.y = Op16<T>::pack(__uint_as_float(v[8 * q4 + 2]), __uint_as_float(v[8 * q4 + 3]));
          o.z = Op16<T>::pack(__uint_as_float(v[8 * q4 + 4]), __uint_as_float(v[8 * q4 + 5]));
          o.w = Op16<T>::pack(__uint_as_float(v[8 * q4 + 6]), __uint_as_float(v[8 * q4 + 7]));
          reinterpret_cast<uint4*>(yp)[q4] = o;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc<256>(tmem);
}

template <typename T, int DV>
int launch_all(int B, int H, int N, const void* q, const int64_t* qs, const void* k, const int64_t* ks, const void* v,
               const int64_t* vs, void* y, const int64_t* ys, float* workspace, cudaStream_t st) {
  constexpr int F = Op16<T>::kFmt;
  const int chunks = (N + 127) / 128;
  const long long BH = (long long)B * H;
  const long long per_chunk = (long long)kDk * DV;
  float* sums = workspace;
  T* prefix = reinterpret_cast<T*>(workspace + BH * chunks * per_chunk);
  CUtensorMap tmQ, tmK, tmV, tmP;
  const uint64_t e = 2;
  auto b_stride = [&](const int64_t* s) { return (uint64_t)(B > 1 ? s[0] : s[1] * H) * e; };
  if (!make_tile_map_cols(&tmQ, q, F, kDk, 64, (uint64_t)N, (uint64_t)H, (uint64_t)B, qs[2] * e, qs[1] * e, b_stride(qs), 128) ||
      !make_tile_map_cols(&tmK, k, F, kDk, 64, (uint64_t)N, (uint64_t)H, (uint64_t)B, ks[2] * e, ks[1] * e, b_stride(ks), 128) ||
      !make_tile_map(&tmV, v, F, DV, (uint64_t)N, (uint64_t)H, (uint64_t)B, vs[2] * e, vs[1] * e, b_stride(vs), 128) ||
      !make_tile_map(&tmP, prefix, F, DV, (uint64_t)kDk, (uint64_t)chunks, (uint64_t)BH, DV * e, per_chunk * e,
                     chunks * per_chunk * e, 128))
    return FLARE_EUNSUPPORTED;
  ClTcArgs a;
  a.B = B; a.H = H; a.N = N; a.chunks = chunks;
  a.inv_n = 1.f / (float)N;
  a.sums = sums;
  a.y = y;
  for (int i = 0; i < 3; ++i) a.ys[i] = ys[i];
  a.status = tc_status_ptr();
  constexpr int smem1 = 2 * 128 * 128 + 128 * 2 * DV + 256 + 1024;
  constexpr int smem3 = 4 * 128 * 128 + 2 * 128 * 2 * DV + 256 + 1024;
  if (tc_set_dyn_smem(reinterpret_cast<const void*>(&k_cl_tc_sums<T, DV>), smem1) != FLARE_OK ||
      tc_set_dyn_smem(reinterpret_cast<const void*>(&k_cl_tc_walk<T, DV>), smem3) != FLARE_OK)
    return FLARE_ECUDA;
  const dim3 grid((unsigned)chunks, (unsigned)BH);
  launch_dep(k_cl_tc_sums<T, DV>, grid, dim3(kThreadsSum), smem1, st, tmK, tmV, a);
  const long long total = BH * (per_chunk / 2);
  launch_dep(k_cl_tc_prefix<T>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, (const float*)sums, prefix, chunks,
             (int)per_chunk, total, a.inv_n);
  launch_dep(k_cl_tc_walk<T, DV>, grid, dim3(kThreadsWalk), smem3, st, tmQ, tmK, tmV, tmP, a);
  return FLARE_OK;
}

}  // namespace

// 16-bit inputs, Dk = 128, Dv in {32, 64}, rows the TMA can address
bool causal_linear_tc_supported(int B, int H, int N, int Dk, int Dv, int dtype, const void* q, const int64_t* qs,
                                const void* k, const int64_t* ks, const void* v, const int64_t* vs, const void* y,
                                const int64_t* ys) {
  if (dtype != FLARE_BF16 && dtype != FLARE_F16) return false;
  if (Dk != kDk || (Dv != 32 && Dv != 64) || N < 1) return false;
  if ((long long)B * H > 65535) return false;
  auto ok = [&](const void* ptr, const int64_t* s) {
    if (reinterpret_cast<uintptr_t>(ptr) % 16) return false;
    for (int i = 0; i < 3; ++i) if ((s[i] * 2) % 16) return false;
    return true;
  };
  return ok(q, qs) && ok(k, ks) && ok(v, vs) && ok(y, ys);
}

size_t causal_linear_tc_workspace(int B, int H, int N, int Dk, int Dv) {
  const size_t chunks = ((size_t)N + 127) / 128;
  return (size_t)B * H * chunks * Dk * Dv * (sizeof(float) + 2) + 256;
}

int causal_linear_tc(int B, int H, int N, int Dv, int dtype, const void* q, const int64_t* qs, const void* k,
                     const int64_t* ks, const void* v, const int64_t* vs, void* y, const int64_t* ys, float* workspace,
                     cudaStream_t st) {
  if (dtype == FLARE_BF16)
    return Dv == 32 ? launch_all<__nv_bfloat16, 32>(B, H, N, q, qs, k, ks, v, vs, y, ys, workspace, st)
                    : launch_all<__nv_bfloat16, 64>(B, H, N, q, qs, k, ks, v, vs, y, ys, workspace, st);
  return Dv == 32 ? launch_all<__half, 32>(B, H, N, q, qs, k, ks, v, vs, y, ys, workspace, st)
                  : launch_all<__half, 64>(B, H, N, q, qs, k, ks, v, vs, y, ys, workspace, st);
}

}  // namespace flare
