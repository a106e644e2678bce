// Cross-GPU completion barrier for the fused attention-output gather.
//
// Under tensor parallelism every rank's attention epilogue stores its [rows, cols] slice straight
// into the gathered [rows, world*cols] activation of every peer (plain peer stores over NVLink,
// no multicast loads).  This kernel then tells the peers "my slices have landed" and waits until
// every peer has said the same.  The wait is bounded: when it runs out the kernel sets
// GK_DEV_WAIT_EXPIRED in the status word and returns, it never traps or spins forever.
#include "gk_common.cuh"

namespace gk {
namespace {

struct PeerFlags {
  int32_t* ptr[GK_MAX_OUTPUTS];   // ptr[p] = rank p's flag array [world], mapped into this process
};

// With `counter` the epoch is kept on the device (this launch uses *counter + 1 and stores it back),
// so the same launch can be replayed from a CUDA graph; every rank must issue the same sequence of
// barriers.
__global__ void __launch_bounds__(32) peer_barrier_kernel(const PeerFlags flags, int rank, int world, int epoch,
                                                          int32_t* counter, long long max_cycles, int32_t* status) {
  const int lane = threadIdx.x;
  wait_for_predecessor();               // the kernels that wrote the peers' buffers have completed
  if (counter) {
    if (lane == 0) {
      epoch = *counter + 1;
      *counter = epoch;
    }
    epoch = __shfl_sync(0xffffffffu, epoch, 0);
  }
  if (lane >= world) return;
  // The launch is stream-ordered after the kernels that wrote the peers' buffers; the fence
  // orders those writes before the flag for observers on other GPUs.
  __threadfence_system();
  int32_t* remote = flags.ptr[lane] + rank;
  asm volatile("st.release.sys.global.s32 [%0], %1;\n" ::"l"(remote), "r"(epoch) : "memory");
  const int32_t* mine = flags.ptr[rank] + lane;
  const long long start = clock64();
  for (;;) {
    int seen;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];\n" : "=r"(seen) : "l"(mine) : "memory");
    if (seen - epoch >= 0) break;
    if (clock64() - start > max_cycles) {
      if (status) atomicOr(status, (int)GK_DEV_WAIT_EXPIRED);
      break;
    }
    __nanosleep(64);
  }
}

}  // namespace
}  // namespace gk

extern "C" int gk_peer_barrier(int32_t* const* flags, int rank, int world, int32_t epoch, int64_t max_cycles,
                               int32_t* status, gk_stream_t stream) {
  if (!flags || world <= 0 || world > GK_MAX_OUTPUTS || rank < 0 || rank >= world || max_cycles <= 0)
    return GK_ERR_INVALID_ARGUMENT;
  gk::PeerFlags f{};
  for (int p = 0; p < world; ++p) {
    if (!flags[p] || (reinterpret_cast<uintptr_t>(flags[p]) & 3)) return GK_ERR_INVALID_ARGUMENT;
    f.ptr[p] = flags[p];
  }
  gk::launch_after_predecessor(gk::peer_barrier_kernel, dim3(1), dim3(32), 0, reinterpret_cast<cudaStream_t>(stream), f, rank,
                               world, epoch, static_cast<int32_t*>(nullptr), (long long)max_cycles, status);
  return gk::check_launch();
}

extern "C" int gk_peer_barrier_counted(int32_t* const* flags, int rank, int world, int32_t* epoch_counter,
                                       int64_t max_cycles, int32_t* status, gk_stream_t stream) {
  if (!flags || !epoch_counter || world <= 0 || world > GK_MAX_OUTPUTS || rank < 0 || rank >= world || max_cycles <= 0)
    return GK_ERR_INVALID_ARGUMENT;
  gk::PeerFlags f{};
  for (int p = 0; p < world; ++p) {
    if (!flags[p] || (reinterpret_cast<uintptr_t>(flags[p]) & 3)) return GK_ERR_INVALID_ARGUMENT;
    f.ptr[p] = flags[p];
  }
  gk::launch_after_predecessor(gk::peer_barrier_kernel, dim3(1), dim3(32), 0, reinterpret_cast<cudaStream_t>(stream), f, rank,
                               world, 0, epoch_counter, (long long)max_cycles, status);
  return gk::check_launch();
}
