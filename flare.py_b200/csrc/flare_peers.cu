// Context-parallel exchanges over peer memory (GPUs of one node): the arrival barrier and the two whole
// passes with their exchanges inside.  The reference has no such mode (its only parallelism is replicas).
//
// Every rank owns an exchange buffer and an array of arrival flags in memory that its peers have mapped
// (symmetric memory, IPC).  An exchange is: write my contribution into my buffer -> barrier -> read all
// ranks' buffers with plain loads, in rank order, inside the kernel that consumes them (combine or sum).
// The barrier is one tiny kernel per rank: thread r stores this exchange's number into peer r's flag slot
// for this rank (release, system scope) and polls this rank's slot for peer r (acquire) until it has
// reached that number (the caller passes the number, or 0 and the barrier counts for itself).  The poll is bounded: after 2^30 clocks the kernel sets bit 1 of the device status
// word and returns, so a peer that has left never hangs this GPU; the step's result is then invalid and
// flare_device_status() says so.  Never launch two ranks' barriers on one GPU: they wait on each other.
#include "common.cuh"
#include "launch.h"

namespace flare {

constexpr int kErrPeerTimeout = 2;

__global__ void __launch_bounds__(32)
k_peer_barrier(int32_t* const* __restrict__ flags, int rank, int world, int epoch, int* __restrict__ status) {
  grid_dep_sync();
  const int r = threadIdx.x;
  // epoch 0: the barrier numbers itself with a count kept behind this rank's own flags (slot [world]); every
  // rank's count advances alike because every rank runs the same sequence of barriers.  A launch sequence
  // recorded once and replayed (a CUDA graph) then needs no new argument per replay.
  int32_t* count = flags[rank] + world;
  if (epoch == 0) epoch = *reinterpret_cast<volatile int32_t*>(count) + 1;
  __syncwarp();
  if (r < world) {
    __threadfence_system();                          // what earlier kernels wrote to my buffer is visible first
    int32_t* dst = flags[r] + rank;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(dst), "r"(epoch) : "memory");
    const int32_t* src = flags[rank] + r;
    const long long t0 = clock64();
    for (;;) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(src) : "memory");
      if (v - epoch >= 0) break;
      if (clock64() - t0 > (1LL << 30)) {
        if (status) atomicOr(status, kErrPeerTimeout);
        break;
      }
      __nanosleep(200);
    }
  }
  __syncwarp();
  if (r == 0) *reinterpret_cast<volatile int32_t*>(count) = epoch;
  __threadfence_system();
}

int launch_peer_barrier(int32_t* const* flags, int rank, int world, int epoch, cudaStream_t st) {
  launch_dep(k_peer_barrier, dim3(1), dim3(32), 0, st, flags, rank, world, epoch, tc_status_ptr());
  return FLARE_OK;
}

}  // namespace flare
