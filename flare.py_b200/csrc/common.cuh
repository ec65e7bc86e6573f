// Shared device/host helpers of the flare_b200 kernels.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "flare_b200.h"

namespace flare {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2   = 0.6931471805599453f;

// Device-side copy of a FlareProblem plus the derived token-range length.
struct Ctx {
  int B, H, N, M, D;
  float scale;
  int n_splits;
  int chunk;             // tokens per range (multiple of 128)
  int terms;
  long long qs[3], ks[3], vs[3], ys[3], dys[3], dks[3], dvs[3];
};

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// Load NE consecutive elements (16-byte aligned, NE*sizeof(T) a multiple of 16) as fp32.
template <typename T, int NE>
__device__ __forceinline__ void load_f32(const T* __restrict__ p, float* out) {
  if constexpr (sizeof(T) == 4) {
    static_assert(NE % 4 == 0, "row slice must be a multiple of 16 bytes");
#pragma unroll
    for (int i = 0; i < NE / 4; ++i) {
      float4 t = reinterpret_cast<const float4*>(p)[i];
      out[4 * i] = t.x; out[4 * i + 1] = t.y; out[4 * i + 2] = t.z; out[4 * i + 3] = t.w;
    }
  } else {
    static_assert(NE % 8 == 0, "row slice must be a multiple of 16 bytes");
#pragma unroll
    for (int i = 0; i < NE / 8; ++i) {
      uint4 t = reinterpret_cast<const uint4*>(p)[i];
      const T* e = reinterpret_cast<const T*>(&t);
#pragma unroll
      for (int j = 0; j < 8; ++j) out[8 * i + j] = to_f32(e[j]);
    }
  }
}

template <typename T, int NE>
__device__ __forceinline__ void store_from_f32(T* __restrict__ p, const float* in) {
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int i = 0; i < NE / 4; ++i)
      reinterpret_cast<float4*>(p)[i] = make_float4(in[4 * i], in[4 * i + 1], in[4 * i + 2], in[4 * i + 3]);
  } else {
#pragma unroll
    for (int i = 0; i < NE / 8; ++i) {
      uint4 t;
      T* e = reinterpret_cast<T*>(&t);
#pragma unroll
      for (int j = 0; j < 8; ++j) e[j] = from_f32<T>(in[8 * i + j]);
      reinterpret_cast<uint4*>(p)[i] = t;
    }
  }
}

// Sum over the TPT adjacent lanes that share one row.
template <int TPT>
__device__ __forceinline__ float group_sum(float x) {
#pragma unroll
  for (int o = TPT / 2; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

}  // namespace flare
