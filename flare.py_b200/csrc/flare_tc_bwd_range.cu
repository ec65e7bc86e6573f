// The on-device range check in front of the one-exponential backward kernel (flare_tc_bwd_fast.cu).
//
// With P_mn = exp(S_mn - L_m) and A_mn = exp(S_mn - C_n) = P_mn * exp(L_m - C_n) the backward needs one
// exponential per score instead of two:
//
//   dS_mn = P_mn * T'_nm,     T'_nm = (V_n . dZ_m - Delta_m) + eC_n eL_m (dY_n . Z_m - delta_n)
//   eL_m = exp(L_m - mu),  eC_n = exp(mu - C_n),  mu = mid-range of L and C for this (b, h)
//
// and T' is ONE tensor-core product over an extended contraction axis:
//   A' row n = [ V_n | eC_n dY_n | 1, 1, g_hi, g_hi, g_lo, 0.. ]        g = (eC_n dY_n) . Y_n
//   B' row m = [ dZ_m | eL_m Z_m | -Delta_hi, -Delta_lo, -eL_hi, -eL_lo, -eL_hi, 0.. ]
// (the subtractive terms are carried as bf16 hi+lo pairs so that the cancellation in dP - Delta and
// dA - delta keeps fp32-like accuracy).
//
// The factorisation is only valid while exp(L_m - C_n) and its two factors stay inside the exponent
// range of fp32 and bf16.  The two kernels here check that per (b, h) on the device (ranges of L and C)
// and write mu and a flag; the one-exponential kernel runs the (b, h) whose flag is 0, the general
// kernel (flare_tc_bwd.cu: two exponentials, no factorisation) the others.  No host synchronisation.
#include "common.cuh"
#include "launch.h"
#include "tc_common.cuh"
#include "tma_host.h"

namespace flare {

using namespace tc;

// ------------------------------------------------------------------------------------------
// range check: flag[bh] = 1 when the one-exponential form is not safe for this (b, h)
// ------------------------------------------------------------------------------------------
constexpr int kRangeParts = 64;

__global__ void __launch_bounds__(256)
k_bwd_range_c(const float* __restrict__ lse_n, int N, float* __restrict__ part /*[BH][parts][2]*/) {
  grid_dep_sync();
  const int bh = blockIdx.y, p = blockIdx.x;
  const float* c = lse_n + (long long)bh * N;
  float mx = -INFINITY, mn = INFINITY;
  for (long long i = (long long)p * blockDim.x + threadIdx.x; i < N; i += (long long)gridDim.x * blockDim.x) {
    const float v = c[i];
    mx = fmaxf(mx, v); mn = fminf(mn, v);
  }
  __shared__ float smx[256], smn[256];
  smx[threadIdx.x] = mx; smn[threadIdx.x] = mn;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (threadIdx.x < s) {
      smx[threadIdx.x] = fmaxf(smx[threadIdx.x], smx[threadIdx.x + s]);
      smn[threadIdx.x] = fminf(smn[threadIdx.x], smn[threadIdx.x + s]);
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    part[((long long)bh * kRangeParts + p) * 2] = smx[0];
    part[((long long)bh * kRangeParts + p) * 2 + 1] = smn[0];
  }
}

__global__ void __launch_bounds__(256)
k_bwd_range_final(const float* __restrict__ lse_m, int M, const float* __restrict__ part,
                  float* __restrict__ mu_out, int* __restrict__ flag_out) {
  grid_dep_sync();
  const int bh = blockIdx.x;
  float lmx = -INFINITY, lmn = INFINITY, cmx = -INFINITY, cmn = INFINITY;
  for (int i = threadIdx.x; i < M; i += blockDim.x) {
    const float v = lse_m[(long long)bh * M + i];
    lmx = fmaxf(lmx, v); lmn = fminf(lmn, v);
  }
  for (int i = threadIdx.x; i < kRangeParts; i += blockDim.x) {
    cmx = fmaxf(cmx, part[((long long)bh * kRangeParts + i) * 2]);
    cmn = fminf(cmn, part[((long long)bh * kRangeParts + i) * 2 + 1]);
  }
  __shared__ float s[4][256];
  s[0][threadIdx.x] = lmx; s[1][threadIdx.x] = lmn; s[2][threadIdx.x] = cmx; s[3][threadIdx.x] = cmn;
  __syncthreads();
  for (int st = 128; st > 0; st >>= 1) {
    if (threadIdx.x < st) {
      s[0][threadIdx.x] = fmaxf(s[0][threadIdx.x], s[0][threadIdx.x + st]);
      s[1][threadIdx.x] = fminf(s[1][threadIdx.x], s[1][threadIdx.x + st]);
      s[2][threadIdx.x] = fmaxf(s[2][threadIdx.x], s[2][threadIdx.x + st]);
      s[3][threadIdx.x] = fminf(s[3][threadIdx.x], s[3][threadIdx.x + st]);
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const float Lmx = s[0][0] * kLog2e, Lmn = s[1][0] * kLog2e, Cmx = s[2][0] * kLog2e, Cmn = s[3][0] * kLog2e;
    const float mu = 0.5f * (Lmx + Lmn);
    // every factor within 2^+-50 and exp(L - C) within 2^+-100; anything non-finite takes the exact kernel
    const bool ok = (Lmx - mu < 50.f) && (mu - Lmn < 50.f) && (Cmx - mu < 50.f) && (mu - Cmn < 50.f) &&
                    isfinite(Lmx) && isfinite(Lmn) && isfinite(Cmx) && isfinite(Cmn);
    mu_out[bh] = ok ? mu : 0.f;
    flag_out[bh] = ok ? 0 : 1;
  }
}

// ------------------------------------------------------------------------------------------
size_t tc_bwd_fast_scratch_bytes(const Ctx& c) {
  const size_t bh = (size_t)c.B * c.H;
  return ((bh * kRangeParts * 2 * sizeof(float) + 255) & ~size_t(255)) + ((bh * sizeof(float) + 255) & ~size_t(255)) +
         ((bh * sizeof(int) + 255) & ~size_t(255));
}

// Range check, then the one-exponential kernel; the caller launches the general kernel behind it with the
// same flags.  scratch: tc_bwd_fast_scratch_bytes(c) bytes, 256-byte aligned.
int tc_bwd_fast_main(const Ctx& c, const void* q, const void* k, const void* v, const void* dy, const void* y,
                     const float* z32, const float* dz32, const float* lse_m, const float* lse_n, void* dk, void* dv,
                     float* dq_part, void* scratch, const int** flag_out, cudaStream_t st) {
  if (!tc_bwd_fast_supported(c, FLARE_BF16)) return FLARE_EUNSUPPORTED;
  const size_t bh = (size_t)c.B * c.H;
  char* w = static_cast<char*>(scratch);
  float* part = reinterpret_cast<float*>(w);  w += (bh * kRangeParts * 2 * sizeof(float) + 255) & ~size_t(255);
  float* mu = reinterpret_cast<float*>(w);    w += (bh * sizeof(float) + 255) & ~size_t(255);
  int* flag = reinterpret_cast<int*>(w);
  launch_dep(k_bwd_range_c, dim3(kRangeParts, (unsigned)bh), dim3(256), 0, st, lse_n, c.N, part);
  launch_dep(k_bwd_range_final, dim3((unsigned)bh), dim3(256), 0, st, lse_m, c.M, part, mu, flag);
  *flag_out = flag;
  return tc_bwd_fast_launch(c, q, k, v, dy, y, z32, dz32, lse_m, lse_n, dk, dv, dq_part, mu, flag, st);
}

}  // namespace flare
