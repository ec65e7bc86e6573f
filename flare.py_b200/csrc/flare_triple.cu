// Triple attention (lra/models/triton/triple.py:27-290; einsum references :846-860 and :887-931):
//
//   STATE[i,j,k] = (1/N) sum_n K1[n,i] V[n,j] K2[n,k]          O[n,j] = sum_{i,k} Q1[n,i] STATE[i,j,k] Q2[n,k]
//
// and its backward, which is the same two shapes of work with the operands permuted:
//   dSTATE = outer(Q1, dO, Q2);  dQ1, dQ2 contract STATE with (dO, Q2), (Q1, dO);
//   dK1, dK2, dV contract dSTATE with (V, K2), (K1, V), (K1, K2), times 1/N.
// Two kernels cover all of it:
//   k_triple_outer    out[i][j][k] = alpha * sum_n A[n,i] B[n,j] C[n,k] over one token range (partials are
//                     summed in range order by the library's reduce kernel).  A thread owns one (j, k)
//                     pair and every i in registers; tokens stream through shared memory once per
//                     block of 256 pairs.
//   k_triple_contract out[n,x] = alpha * sum_{y,z} T[x,y,z] A[n,y] B[n,z], T addressed through element
//                     strides so that every permutation of STATE is served without a copy.  A block
//                     of T (all y, z for a slab of x) sits in shared memory; lanes are tokens, warps
//                     are x, so every T element is a shared-memory broadcast.
// fp32 SIMT arithmetic (the reference upcasts to fp32 and uses TF32 dots); inputs fp32/fp16/bf16,
// [BH, N, D] contiguous as the reference makes them (triple.py:51-55).
#include <cstdarg>
#include <cstdio>
#include <cuda_runtime.h>
#include "common.cuh"
#include "launch.h"

namespace flare { void set_last_error(const char* msg); }

namespace {

using namespace flare;

int refuse(int code, const char* fmt, ...) {
  char msg[400];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(msg, sizeof(msg), fmt, ap);
  va_end(ap);
  flare::set_last_error(msg);
  return code;
}

constexpr int kPairs = 256;       // (j, k) pairs per CTA of the outer kernel
constexpr int kTok = 32;          // tokens per shared-memory tile

template <typename T, int DA>
__global__ void __launch_bounds__(kPairs)
k_triple_outer(const T* __restrict__ A, const T* __restrict__ Bm, const T* __restrict__ Cm, int N, int Db, int Dc,
               int n_splits, int chunk, float alpha, float* __restrict__ part) {
  extern __shared__ __align__(16) float sm[];
  float* sA = sm;                                  // [kTok][DA]
  float* sB = sA + kTok * DA;                      // [kTok][Db]
  float* sC = sB + kTok * Db;                      // [kTok][Dc]
  const int split = blockIdx.y, bh = blockIdx.z;
  const int pi = blockIdx.x * kPairs + threadIdx.x;
  const bool live = pi < Db * Dc;
  const int j = live ? pi / Dc : 0, k = live ? pi % Dc : 0;
  const T* a = A + (long long)bh * N * DA;
  const T* b = Bm + (long long)bh * N * Db;
  const T* c = Cm + (long long)bh * N * Dc;
  float acc[DA];
#pragma unroll
  for (int i = 0; i < DA; ++i) acc[i] = 0.f;
  const int n0 = split * chunk, n1 = min(N, n0 + chunk);
  for (int t0 = n0; t0 < n1; t0 += kTok) {
    const int cnt = min(kTok, n1 - t0);
    __syncthreads();
    for (int e = threadIdx.x; e < cnt * DA; e += kPairs) sA[e] = to_f32(a[(long long)t0 * DA + e]);
    for (int e = threadIdx.x; e < cnt * Db; e += kPairs) sB[e] = to_f32(b[(long long)t0 * Db + e]);
    for (int e = threadIdx.x; e < cnt * Dc; e += kPairs) sC[e] = to_f32(c[(long long)t0 * Dc + e]);
    __syncthreads();
    for (int n = 0; n < cnt; ++n) {
      const float p = sB[n * Db + j] * sC[n * Dc + k];
      const float4* ar = reinterpret_cast<const float4*>(sA + n * DA);
#pragma unroll
      for (int i = 0; i < DA / 4; ++i) {
        const float4 a4 = ar[i];
        acc[4 * i] = fmaf(a4.x, p, acc[4 * i]);
        acc[4 * i + 1] = fmaf(a4.y, p, acc[4 * i + 1]);
        acc[4 * i + 2] = fmaf(a4.z, p, acc[4 * i + 2]);
        acc[4 * i + 3] = fmaf(a4.w, p, acc[4 * i + 3]);
      }
    }
  }
  if (live) {
    float* o = part + (((long long)split * gridDim.z + bh) * DA) * Db * Dc + (long long)j * Dc + k;
#pragma unroll
    for (int i = 0; i < DA; ++i) o[(long long)i * Db * Dc] = acc[i] * alpha;
  }
}

constexpr int kCThreads = 256;

// NT tokens per lane (tokens lane, lane + 32, ...): every 16-byte load of T feeds 4 NT multiply-adds.
template <typename T, int DZ, int NT>
__global__ void __launch_bounds__(kCThreads)
k_triple_contract(const float* __restrict__ Tn, long long sx, long long sy, long long sz, int Dx, int Dy, int xb,
                  const T* __restrict__ A, const T* __restrict__ Bm, int N, int chunk, float alpha, T* __restrict__ out) {
  constexpr int TT = kTok * NT;                    // tokens per tile
  extern __shared__ __align__(16) float sm[];
  const int DyP = Dy + 1, xbP = xb + 1;
  float* sT = sm;                                  // [xb][Dy][DZ]
  float* sAt = sT + (size_t)xb * Dy * DZ;          // [TT][DyP]
  float* sO = sAt + TT * DyP;                      // [TT][xbP]
  const int x0 = blockIdx.x * xb, bh = blockIdx.z;
  const int nx = min(xb, Dx - x0);
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const float* tb = Tn + (long long)bh * Dx * Dy * DZ;
  for (int e = threadIdx.x; e < nx * Dy * DZ; e += kCThreads) {
    const int z = e % DZ, y = (e / DZ) % Dy, x = e / (DZ * Dy);
    sT[e] = tb[(x0 + x) * sx + y * sy + z * sz];
  }
  const T* a = A + (long long)bh * N * Dy;
  const T* b = Bm + (long long)bh * N * DZ;
  T* o = out + (long long)bh * N * Dx;
  const int n0 = blockIdx.y * chunk, n1 = min(N, n0 + chunk);
  for (int t0 = n0; t0 < n1; t0 += TT) {
    const int cnt = min(TT, n1 - t0);
    __syncthreads();
    for (int e = threadIdx.x; e < cnt * Dy; e += kCThreads) sAt[(e / Dy) * DyP + e % Dy] = to_f32(a[(long long)t0 * Dy + e]);
    float bn[NT][DZ];
#pragma unroll
    for (int q = 0; q < NT; ++q) {
      const int n = lane + 32 * q;
      if (n < cnt) {
#pragma unroll
        for (int z = 0; z < DZ; ++z) bn[q][z] = to_f32(b[(long long)(t0 + n) * DZ + z]);
      } else {
#pragma unroll
        for (int z = 0; z < DZ; ++z) bn[q][z] = 0.f;
      }
    }
    __syncthreads();
    for (int x = warp; x < nx; x += kCThreads / 32) {
      float ox[NT];
#pragma unroll
      for (int q = 0; q < NT; ++q) ox[q] = 0.f;
      const float* tx = sT + (size_t)x * Dy * DZ;
      for (int y = 0; y < Dy; ++y) {
        const float4* tr = reinterpret_cast<const float4*>(tx + y * DZ);
        float t[NT];
#pragma unroll
        for (int q = 0; q < NT; ++q) t[q] = 0.f;
#pragma unroll
        for (int z = 0; z < DZ / 4; ++z) {
          const float4 t4 = tr[z];
#pragma unroll
          for (int q = 0; q < NT; ++q) {
            t[q] = fmaf(t4.x, bn[q][4 * z], t[q]); t[q] = fmaf(t4.y, bn[q][4 * z + 1], t[q]);
            t[q] = fmaf(t4.z, bn[q][4 * z + 2], t[q]); t[q] = fmaf(t4.w, bn[q][4 * z + 3], t[q]);
          }
        }
#pragma unroll
        for (int q = 0; q < NT; ++q) ox[q] = fmaf(sAt[(lane + 32 * q) * DyP + y], t[q], ox[q]);
      }
#pragma unroll
      for (int q = 0; q < NT; ++q) sO[(lane + 32 * q) * xbP + x] = ox[q] * alpha;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < cnt * nx; e += kCThreads) {
      const int n = e / nx, x = e % nx;
      o[(long long)(t0 + n) * Dx + x0 + x] = from_f32<T>(sO[n * xbP + x]);
    }
  }
}

int pick_splits(int BH, int N, int pair_blocks) {
  long long s = (2LL * 148 + (long long)BH * pair_blocks - 1) / ((long long)BH * pair_blocks);
  const long long max_s = (N + 255) / 256;
  if (s > max_s) s = max_s;
  if (s > 256) s = 256;
  if (s < 1) s = 1;
  return (int)s;
}

template <typename T>
int run_outer(int BH, int N, int Da, int Db, int Dc, const void* a, const void* b, const void* c, float alpha,
              float* out, float* ws, cudaStream_t st) {
  const int pb = (Db * Dc + kPairs - 1) / kPairs;
  const int S = pick_splits(BH, N, pb);
  const int chunk = ((N + S - 1) / S + kTok - 1) / kTok * kTok;
  const int S2 = (N + chunk - 1) / chunk;
  float* part = S2 == 1 ? out : ws;
  const dim3 grid((unsigned)pb, (unsigned)S2, (unsigned)BH);
  const size_t smem = sizeof(float) * kTok * (size_t)(Da + Db + Dc);
  const T* A = reinterpret_cast<const T*>(a);
  const T* B = reinterpret_cast<const T*>(b);
  const T* C = reinterpret_cast<const T*>(c);
  switch (Da) {
    case 16: k_triple_outer<T, 16><<<grid, kPairs, smem, st>>>(A, B, C, N, Db, Dc, S2, chunk, alpha, part); break;
    case 32: k_triple_outer<T, 32><<<grid, kPairs, smem, st>>>(A, B, C, N, Db, Dc, S2, chunk, alpha, part); break;
    case 64: k_triple_outer<T, 64><<<grid, kPairs, smem, st>>>(A, B, C, N, Db, Dc, S2, chunk, alpha, part); break;
    default: return refuse(FLARE_EUNSUPPORTED, "triple_outer: first dimension %d not in {16,32,64}", Da);
  }
  if (S2 > 1) launch_reduce_sum(part, S2, (long long)BH * Da * Db * Dc, out, st);
  const cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) return refuse(FLARE_ECUDA, "triple_outer: %s", cudaGetErrorString(e));
  return FLARE_OK;
}

template <typename T, int DZ>
int launch_contract(int BH, int N, int Dx, int Dy, const float* t, long long sx, long long sy, long long sz, const void* a,
                    const void* b, float alpha, void* out, cudaStream_t st) {
  // slab of x whose [xb][Dy][DZ] block fits in 128 KB
  int xb = Dx;
  while ((size_t)xb * Dy * DZ * sizeof(float) > 128 * 1024 && xb > 1) xb = (xb + 1) / 2;
  const int nxb = (Dx + xb - 1) / xb;
  long long chunks = (2LL * 148 + (long long)BH * nxb - 1) / ((long long)BH * nxb);
  const long long maxc = (N + 4 * kTok - 1) / (4 * kTok);
  if (chunks > maxc) chunks = maxc;
  if (chunks < 1) chunks = 1;
  if (chunks > 65535) chunks = 65535;
  constexpr int NT = DZ <= 32 ? 2 : 1;             // tokens per lane: registers allow two up to DZ = 32
  constexpr int TT = kTok * NT;
  const int chunk = (int)(((N + chunks - 1) / chunks + TT - 1) / TT * TT);
  const int nch = (N + chunk - 1) / chunk;
  const size_t smem = sizeof(float) * ((size_t)xb * Dy * DZ + TT * (Dy + 1) + TT * (xb + 1));
  if (cudaFuncSetAttribute(k_triple_contract<T, DZ, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return refuse(FLARE_ECUDA, "triple_contract: cudaFuncSetAttribute failed (%zu bytes)", smem);
  k_triple_contract<T, DZ, NT><<<dim3((unsigned)nxb, (unsigned)nch, (unsigned)BH), kCThreads, smem, st>>>(
      t, sx, sy, sz, Dx, Dy, xb, reinterpret_cast<const T*>(a), reinterpret_cast<const T*>(b), N, chunk, alpha,
      reinterpret_cast<T*>(out));
  const cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) return refuse(FLARE_ECUDA, "triple_contract: %s", cudaGetErrorString(e));
  return FLARE_OK;
}

template <typename T>
int run_contract(int BH, int N, int Dx, int Dy, int Dz, const float* t, long long sx, long long sy, long long sz,
                 const void* a, const void* b, float alpha, void* out, cudaStream_t st) {
  switch (Dz) {
    case 16: return launch_contract<T, 16>(BH, N, Dx, Dy, t, sx, sy, sz, a, b, alpha, out, st);
    case 32: return launch_contract<T, 32>(BH, N, Dx, Dy, t, sx, sy, sz, a, b, alpha, out, st);
    case 64: return launch_contract<T, 64>(BH, N, Dx, Dy, t, sx, sy, sz, a, b, alpha, out, st);
  }
  return refuse(FLARE_EUNSUPPORTED, "triple_contract: last dimension %d not in {16,32,64}", Dz);
}

bool dim_ok(int d) { return d >= 4 && d <= 64 && d % 4 == 0; }

}  // namespace

extern "C" {

size_t flare_triple_workspace_bytes(int BH, int N, int Da, int Db, int Dc) {
  if (BH < 1 || N < 1) return 0;
  const int pb = (Db * Dc + kPairs - 1) / kPairs;
  const size_t simt = (size_t)pick_splits(BH, N, pb) * BH * Da * Db * Dc * sizeof(float) + 256;
  const size_t tc = triple_tc_outer_workspace(BH, N);                // dtype is not known here: room for either path
  return simt > tc ? simt : tc;
}

int flare_triple_outer(int BH, int N, int Da, int Db, int Dc, int dtype, const void* a, const void* b, const void* c,
                       float alpha, float* out, float* workspace, flare_stream_t stream) {
  if (BH < 1 || BH > 65535 || N < 1) return refuse(FLARE_EINVAL, "triple_outer: bad sizes BH=%d N=%d", BH, N);
  if (!dim_ok(Da) || !dim_ok(Db) || !dim_ok(Dc)) return refuse(FLARE_EUNSUPPORTED, "triple_outer: dims %d,%d,%d must be multiples of 4 up to 64", Da, Db, Dc);
  if (!a || !b || !c || !out || !workspace) return refuse(FLARE_EINVAL, "triple_outer: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (triple_tc_supported(N, Da, Db, Dc, dtype)) {
    const int rc = triple_tc_outer(BH, N, dtype, a, b, c, alpha, out, workspace, st);
    if (rc != FLARE_OK) return refuse(rc, "triple_outer (tcgen05): launch setup failed");
    const cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) return refuse(FLARE_ECUDA, "triple_outer: %s", cudaGetErrorString(e));
    return FLARE_OK;
  }
  switch (dtype) {
    case FLARE_F32: return run_outer<float>(BH, N, Da, Db, Dc, a, b, c, alpha, out, workspace, st);
    case FLARE_F16: return run_outer<__half>(BH, N, Da, Db, Dc, a, b, c, alpha, out, workspace, st);
    case FLARE_BF16: return run_outer<__nv_bfloat16>(BH, N, Da, Db, Dc, a, b, c, alpha, out, workspace, st);
  }
  return refuse(FLARE_EINVAL, "triple_outer: bad dtype %d", dtype);
}

int flare_triple_contract(int BH, int N, int Dx, int Dy, int Dz, int dtype, const float* t, int64_t sx, int64_t sy,
                          int64_t sz, const void* a, const void* b, float alpha, void* out, flare_stream_t stream) {
  if (BH < 1 || BH > 65535 || N < 1) return refuse(FLARE_EINVAL, "triple_contract: bad sizes BH=%d N=%d", BH, N);
  if (!dim_ok(Dx) || !dim_ok(Dy) || !dim_ok(Dz)) return refuse(FLARE_EUNSUPPORTED, "triple_contract: dims %d,%d,%d must be multiples of 4 up to 64", Dx, Dy, Dz);
  if (!t || !a || !b || !out) return refuse(FLARE_EINVAL, "triple_contract: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (triple_tc_supported(N, Dx, Dy, Dz, dtype) && triple_tc_strides_ok(sx, sy, sz)) {
    const int rc = triple_tc_contract(BH, N, dtype, t, sx, sy, sz, a, b, alpha, out, st);
    if (rc != FLARE_OK) return refuse(rc, "triple_contract (tcgen05): launch setup failed");
    const cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) return refuse(FLARE_ECUDA, "triple_contract: %s", cudaGetErrorString(e));
    return FLARE_OK;
  }
  switch (dtype) {
    case FLARE_F32: return run_contract<float>(BH, N, Dx, Dy, Dz, t, sx, sy, sz, a, b, alpha, out, st);
    case FLARE_F16: return run_contract<__half>(BH, N, Dx, Dy, Dz, t, sx, sy, sz, a, b, alpha, out, st);
    case FLARE_BF16: return run_contract<__nv_bfloat16>(BH, N, Dx, Dy, Dz, t, sx, sy, sz, a, b, alpha, out, st);
  }
  return refuse(FLARE_EINVAL, "triple_contract: bad dtype %d", dtype);
}

}  // extern "C"
