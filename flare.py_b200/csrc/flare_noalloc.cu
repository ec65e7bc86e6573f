// flare_gather_noalloc: the gather pass (first SDPA call, z = softmax_N(scale q k^T) v) for
// callers that have no way to hand the library a workspace.
//
// Who needs it: code that runs where device allocation is off limits -- a plugin called inside
// a host framework's pre-planned memory arena, a real-time or interrupt-like service thread that
// must not enter the allocator (cudaMalloc takes locks and may synchronise the device), or a
// caller that only holds the tensors it was given.  Every other entry point of the library expects
// the split-N partial records in caller memory; here they live in a fixed array that is part of
// the library image, so the call touches no allocator at all (no cudaMalloc/cudaFree, no torch).
//
// Cost and limits: every GPU that loads the library carries the FLARE_NOALLOC_SCRATCH_BYTES array
// until the process exits.  One record set (B*H*M*(D+2) floats) must fit in it, otherwise the call
// is refused with FLARE_EWORKSPACE; when fewer token ranges fit than the library would normally
// use, it uses fewer (same result up to fp32 summation order, less parallelism).  All calls share
// the one array and it keeps the previous call's records: nothing in it has to start at zero
// (each call overwrites every record it later reads), but two calls that overlap on the GPU --
// different streams, or different host threads -- race on it and must be serialised by the caller; that
// includes the very first call on a device, which also fills the per-device address table below.
// The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
// that device current); make that first call outside any stream capture.
#include <cstdarg>
#include <cstdio>
#include <cuda_runtime.h>
#include "flare_b200.h"

namespace flare { void set_last_error(const char* msg); }   // text returned by flare_last_error()

namespace {

constexpr size_t kScratchFloats = FLARE_NOALLOC_SCRATCH_BYTES / sizeof(float);
static __device__ __align__(256) float g_gather_scratch[kScratchFloats];

constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {nullptr};   // device address of the array, per device

int refuse(int code, const char* fmt, ...) {
  char msg[400];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(msg, sizeof(msg), fmt, ap);
  va_end(ap);
  flare::set_last_error(msg);
  return code;
}

// In host code the name g_gather_scratch is only a handle for the runtime, not a device address:
// a kernel handed &g_gather_scratch[0] from the host would fault or scribble over unrelated memory.
// The address kernels may use comes from cudaGetSymbolAddress, per device, with that device current.
int scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return refuse(FLARE_ECUDA, "gather_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return refuse(FLARE_EUNSUPPORTED, "gather_noalloc: device index %d not supported", dev);
  if (!g_scratch_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_gather_scratch);
    if (e != cudaSuccess || !p)
      return refuse(FLARE_ECUDA, "gather_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    g_scratch_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_scratch_ptr[dev];
  return FLARE_OK;
}

}  // namespace

extern "C" int flare_gather_noalloc(const FlareProblem* p, const void* q, const void* k, const void* v,
                                    const uint8_t* key_mask, float* z32, void* z_out, float* lse_m,
                                    flare_stream_t stream) {
  if (!p) return refuse(FLARE_EINVAL, "gather_noalloc: null problem");
  if (!z32 && !z_out && !lse_m) return refuse(FLARE_EINVAL, "gather_noalloc: no output requested");
  if (p->B < 1 || p->H < 1 || p->M < 1 || p->D < 1 || p->N < 0)
    return refuse(FLARE_EINVAL, "gather_noalloc: bad sizes B=%d H=%d N=%d M=%d D=%d", p->B, p->H, p->N, p->M, p->D);
  const size_t per_split = (size_t)p->B * p->H * p->M * (size_t)(p->D + 2);
  if (per_split > kScratchFloats)
    return refuse(FLARE_EWORKSPACE,
                  "gather_noalloc: one record set needs B*H*M*(D+2) = %zu floats but the built-in scratch holds %zu "
                  "(%zu MiB); use flare_gather_partial + flare_combine with a caller workspace for this size",
                  per_split, kScratchFloats, (size_t)FLARE_NOALLOC_SCRATCH_BYTES >> 20);
  FlareProblem pp = *p;
  int splits = flare_pick_splits(p);
  const size_t fit = kScratchFloats / per_split;
  if ((size_t)splits > fit) splits = (int)fit;
  if (splits < 1) splits = 1;
  pp.n_splits = splits;
  float* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != FLARE_OK) return rc;
  rc = flare_gather_partial(&pp, q, k, v, key_mask, scratch, stream);
  if (rc != FLARE_OK) return rc;                 // flare_last_error() already describes it
  return flare_combine(&pp, scratch, splits, z32, z_out, lse_m, nullptr, stream);
}
