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
  float drop_p;                      // attention dropout probability (0 = off)
  unsigned long long drop_seed;
};

// Attention dropout: the keep decision of one softmax weight is a hash of (which softmax, b*H+h, m, n) and
// the seed -- any kernel, whatever its orientation, and the host can recompute it.  `which`: 1 = gather
// weights P_mn, 2 = scatter weights A_mn.
struct DropArgs {
  uint32_t seed_lo, seed_hi;
  uint32_t thresh;                   // keep iff hash >= thresh; thresh = p * 2^32
  float inv_keep;                    // 1 / (1 - p)
  int on;
};
inline DropArgs make_drop(float p, unsigned long long seed) {
  DropArgs d;
  d.seed_lo = (uint32_t)seed; d.seed_hi = (uint32_t)(seed >> 32);
  const double t = (double)p * 4294967296.0;
  d.thresh = t >= 4294967295.0 ? 4294967295u : (uint32_t)t;
  d.inv_keep = p < 1.f ? 1.f / (1.f - p) : 0.f;
  d.on = p > 0.f ? 1 : 0;
  return d;
}
// row = (which * BH + bh) * M + m
__host__ __device__ __forceinline__ uint32_t drop_hash(uint32_t n, uint32_t row, uint32_t seed_lo, uint32_t seed_hi) {
  uint32_t x = (n * 0x9E3779B1u) ^ seed_lo;
  const uint32_t y = (row * 0x85EBCA77u) ^ seed_hi;
  x ^= y + 0x165667B1u + (x << 6) + (x >> 2);
  x ^= x >> 16; x *= 0x85EBCA6Bu; x ^= x >> 13; x *= 0xC2B2AE35u; x ^= x >> 16;
  return x;
}

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

// Programmatic dependent launch.  A kernel launched with launch_dep() may be scheduled while the kernel
// before it in the stream is still running; its first statement, grid_dep_sync(), waits until that kernel
// has completed and its writes are visible, and lets the kernel after it be scheduled in turn.  What is
// hidden is the launch latency between consecutive kernels (a few microseconds each, a tenth of a
// context-parallel step at eight ranks).  Rules: every thread executes grid_dep_sync() before its first
// global-memory access and before any early return (a grid whose blocks all left without waiting would let
// its successor overtake the predecessor), and only kernels that do so are launched with launch_dep().
__device__ __forceinline__ void grid_dep_sync() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
template <typename... KArgs, typename... Args>
inline void launch_dep(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  (void)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);   // a failure stays in the last-error state the caller checks
}

}  // namespace flare
