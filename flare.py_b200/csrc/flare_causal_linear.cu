// Causal linear attention:  Y_t = Q_t . sum_{n <= t} K_n^T V_n / N     (lra/models/triton/causal_linear.py:23-145,
// reference form :317-336; forward only, as there).
//
// The token axis is cut into segments.  k_cl_segsum adds up K^T V of every segment (Dk x Dv fp32, a
// few KB); k_cl_walk starts each segment from the sum of the segments before it and walks it in
// 64-token sub-chunks:  Y_c = Q_c S + tril(Q_c K_c^T) V_c,  S += K_c^T V_c.  Nothing of size N x Dk x Dv
// goes to HBM (the reference's Triton path materialises two such fp32 arrays between its kernels);
// K and V are read twice, Q once.  fp32 SIMT arithmetic, inputs in fp32/fp16/bf16.
#include <cstdarg>
#include <cstdio>
#include <cuda_runtime.h>
#include "common.cuh"
#include "launch.h"

namespace flare { void set_last_error(const char* msg); }

namespace {

using namespace flare;

constexpr int kThreads = 256;
constexpr int kSub = 64;

int refuse(int code, const char* fmt, ...) {
  char msg[400];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(msg, sizeof(msg), fmt, ap);
  va_end(ap);
  flare::set_last_error(msg);
  return code;
}

struct ClArgs {
  int B, H, N, Dk, Dv;
  int n_seg, seg_len;          // seg_len a multiple of kSub
  long long qs[3], ks[3], vs[3], ys[3];
  const void* q; const void* k; const void* v; void* y;
  float* segsum;               // [B][H][n_seg][Dk][Dv]
};

// S[dk][dv] += sum_i K[i][dk] V[i][dv] over the rows of one sub-chunk (thread owns entries e, e + 256, ...)
__device__ __forceinline__ void add_ktv(float* sS, const float* sK, const float* sV, int cnt, int Dk, int Dv, int DkP) {
  for (int e = threadIdx.x; e < Dk * Dv; e += kThreads) {
    const int dk = e / Dv, dv = e % Dv;
    float a = sS[e];
    for (int i = 0; i < cnt; ++i) a = fmaf(sK[i * DkP + dk], sV[i * Dv + dv], a);
    sS[e] = a;
  }
}

template <typename T>
__device__ __forceinline__ void load_rows(float* dst, const T* src, long long row_stride, int row0, int cnt, int D, int DP) {
  for (int i = threadIdx.x; i < cnt * D; i += kThreads) {
    const int r = i / D, c = i % D;
    dst[r * DP + c] = to_f32(src[(long long)(row0 + r) * row_stride + c]);
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) k_cl_segsum(ClArgs a) {
  extern __shared__ __align__(16) float sm[];
  const int DkP = a.Dk + 1;
  float* sS = sm;                                  // [Dk][Dv]
  float* sK = sS + a.Dk * a.Dv;                    // [kSub][DkP]
  float* sV = sK + kSub * DkP;                     // [kSub][Dv]
  const int seg = blockIdx.x, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const T* kp = reinterpret_cast<const T*>(a.k) + b * a.ks[0] + h * a.ks[1];
  const T* vp = reinterpret_cast<const T*>(a.v) + b * a.vs[0] + h * a.vs[1];
  for (int e = threadIdx.x; e < a.Dk * a.Dv; e += kThreads) sS[e] = 0.f;
  const int n0 = seg * a.seg_len, n1 = min(a.N, n0 + a.seg_len);
  for (int s0 = n0; s0 < n1; s0 += kSub) {
    const int cnt = min(kSub, n1 - s0);
    __syncthreads();
    load_rows(sK, kp, a.ks[2], s0, cnt, a.Dk, DkP);
    load_rows(sV, vp, a.vs[2], s0, cnt, a.Dv, a.Dv);
    __syncthreads();
    add_ktv(sS, sK, sV, cnt, a.Dk, a.Dv, DkP);
  }
  __syncthreads();
  float* out = a.segsum + ((long long)bh * a.n_seg + seg) * a.Dk * a.Dv;
  for (int e = threadIdx.x; e < a.Dk * a.Dv; e += kThreads) out[e] = sS[e];
}

template <typename T>
__global__ void __launch_bounds__(kThreads) k_cl_walk(ClArgs a) {
  extern __shared__ __align__(16) float sm[];
  const int Dk = a.Dk, Dv = a.Dv, DkP = Dk + 1;
  float* sS = sm;                                  // [Dk][Dv]  state before the sub-chunk
  float* sQ = sS + Dk * Dv;                        // [kSub][DkP]
  float* sK = sQ + kSub * DkP;                     // [kSub][DkP]
  float* sV = sK + kSub * DkP;                     // [kSub][Dv]
  float* sA = sV + kSub * Dv;                      // [kSub][kSub+1]  tril(Q K^T)
  const int seg = blockIdx.x, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const T* qp = reinterpret_cast<const T*>(a.q) + b * a.qs[0] + h * a.qs[1];
  const T* kp = reinterpret_cast<const T*>(a.k) + b * a.ks[0] + h * a.ks[1];
  const T* vp = reinterpret_cast<const T*>(a.v) + b * a.vs[0] + h * a.vs[1];
  T* yp = reinterpret_cast<T*>(a.y) + b * a.ys[0] + h * a.ys[1];
  const float inv_n = 1.f / (float)a.N;

  // state at the start of the segment: the sums of the segments before it, in order
  const float* ss = a.segsum + (long long)bh * a.n_seg * Dk * Dv;
  for (int e = threadIdx.x; e < Dk * Dv; e += kThreads) {
    float s = 0.f;
    for (int p = 0; p < seg; ++p) s += ss[(long long)p * Dk * Dv + e];
    sS[e] = s;
  }
  const int n0 = seg * a.seg_len, n1 = min(a.N, n0 + a.seg_len);
  for (int s0 = n0; s0 < n1; s0 += kSub) {
    const int cnt = min(kSub, n1 - s0);
    __syncthreads();
    load_rows(sQ, qp, a.qs[2], s0, cnt, Dk, DkP);
    load_rows(sK, kp, a.ks[2], s0, cnt, Dk, DkP);
    load_rows(sV, vp, a.vs[2], s0, cnt, Dv, Dv);
    __syncthreads();
    // A[i][j] = q_i . k_j for j <= i
    for (int e = threadIdx.x; e < cnt * cnt; e += kThreads) {
      const int i = e / cnt, j = e % cnt;
      float s = 0.f;
      if (j <= i) {
        const float* qr = sQ + i * DkP;
        const float* kr = sK + j * DkP;
        for (int d = 0; d < Dk; ++d) s = fmaf(qr[d], kr[d], s);
      }
      sA[i * (kSub + 1) + j] = s;
    }
    __syncthreads();
    // Y[i][dv] = (sum_{j<=i} A[i][j] V[j][dv] + sum_dk Q[i][dk] S[dk][dv]) / N
    for (int e = threadIdx.x; e < cnt * Dv; e += kThreads) {
      const int i = e / Dv, dv = e % Dv;
      float s = 0.f;
      const float* ar = sA + i * (kSub + 1);
      for (int j = 0; j <= i; ++j) s = fmaf(ar[j], sV[j * Dv + dv], s);
      const float* qr = sQ + i * DkP;
      for (int d = 0; d < Dk; ++d) s = fmaf(qr[d], sS[d * Dv + dv], s);
      yp[(long long)(s0 + i) * a.ys[2] + dv] = from_f32<T>(s * inv_n);
    }
    __syncthreads();
    add_ktv(sS, sK, sV, cnt, Dk, Dv, DkP);
  }
}

template <typename T>
int run(const ClArgs& a, cudaStream_t st) {
  const size_t sm1 = sizeof(float) * ((size_t)a.Dk * a.Dv + kSub * (a.Dk + 1) + kSub * a.Dv);
  const size_t sm2 = sizeof(float) * ((size_t)a.Dk * a.Dv + 2 * kSub * (a.Dk + 1) + kSub * a.Dv + kSub * (kSub + 1));
  if (sm2 > 227 * 1024) return refuse(FLARE_EUNSUPPORTED, "causal_linear: Dk=%d Dv=%d needs %zu bytes of shared memory", a.Dk, a.Dv, sm2);
  if (cudaFuncSetAttribute(k_cl_segsum<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm1) != cudaSuccess ||
      cudaFuncSetAttribute(k_cl_walk<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm2) != cudaSuccess)
    return refuse(FLARE_ECUDA, "causal_linear: cudaFuncSetAttribute failed");
  const dim3 grid((unsigned)a.n_seg, (unsigned)(a.B * a.H));
  if (a.n_seg > 1) k_cl_segsum<T><<<grid, kThreads, sm1, st>>>(a);
  k_cl_walk<T><<<grid, kThreads, sm2, st>>>(a);
  const cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) return refuse(FLARE_ECUDA, "causal_linear: %s", cudaGetErrorString(e));
  return FLARE_OK;
}

int pick_segments(int B, int H, int N) {
  long long s = (2LL * 148 + (long long)B * H - 1) / ((long long)B * H);   // two CTAs' worth of work per SM
  const long long max_s = (N + 4 * kSub - 1) / (4 * kSub);                 // at least 256 tokens per segment
  if (s > max_s) s = max_s;
  if (s > 64) s = 64;
  if (s < 1) s = 1;
  return (int)s;
}

}  // namespace

extern "C" {

size_t flare_causal_linear_workspace_bytes(int B, int H, int N, int Dk, int Dv) {
  if (B < 1 || H < 1 || N < 1 || Dk < 1 || Dv < 1) return 0;
  const size_t simt = (size_t)B * H * pick_segments(B, H, N) * Dk * Dv * sizeof(float) + 256;
  const size_t tc = (Dk == 128 && (Dv == 32 || Dv == 64)) ? flare::causal_linear_tc_workspace(B, H, N, Dk, Dv) : 0;
  return simt > tc ? simt : tc;
}

int flare_causal_linear(int B, int H, int N, int Dk, int Dv, int dtype, const void* q, const int64_t* q_stride,
                        const void* k, const int64_t* k_stride, const void* v, const int64_t* v_stride, void* y,
                        const int64_t* y_stride, float* workspace, flare_stream_t stream) {
  if (B < 1 || H < 1 || N < 1) return refuse(FLARE_EINVAL, "causal_linear: bad sizes B=%d H=%d N=%d", B, H, N);
  if (Dk < 1 || Dv < 1 || Dk > 256 || Dv > 256) return refuse(FLARE_EUNSUPPORTED, "causal_linear: Dk=%d Dv=%d out of range", Dk, Dv);
  if ((long long)B * H > 65535) return refuse(FLARE_EUNSUPPORTED, "causal_linear: B*H > 65535");
  if (!q || !k || !v || !y || !workspace || !q_stride || !k_stride || !v_stride || !y_stride)
    return refuse(FLARE_EINVAL, "causal_linear: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (flare::causal_linear_tc_supported(B, H, N, Dk, Dv, dtype, q, q_stride, k, k_stride, v, v_stride, y, y_stride)) {
    const int rc = flare::causal_linear_tc(B, H, N, Dv, dtype, q, q_stride, k, k_stride, v, v_stride, y, y_stride, workspace, st);
    if (rc != FLARE_OK) return refuse(rc, "causal_linear: the tensor-core passes could not be launched");
    const cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) return refuse(FLARE_ECUDA, "causal_linear: %s", cudaGetErrorString(e));
    return FLARE_OK;
  }
  ClArgs a;
  a.B = B; a.H = H; a.N = N; a.Dk = Dk; a.Dv = Dv;
  a.n_seg = pick_segments(B, H, N);
  a.seg_len = (int)((((long long)N + a.n_seg - 1) / a.n_seg + kSub - 1) / kSub) * kSub;
  a.n_seg = (N + a.seg_len - 1) / a.seg_len;
  for (int i = 0; i < 3; ++i) { a.qs[i] = q_stride[i]; a.ks[i] = k_stride[i]; a.vs[i] = v_stride[i]; a.ys[i] = y_stride[i]; }
  a.q = q; a.k = k; a.v = v; a.y = y; a.segsum = workspace;
  switch (dtype) {
    case FLARE_F32: return run<float>(a, st);
    case FLARE_F16: return run<__half>(a, st);
    case FLARE_BF16: return run<__nv_bfloat16>(a, st);
  }
  return refuse(FLARE_EINVAL, "causal_linear: bad dtype %d", dtype);
}

}  // extern "C"
