// Shared device helpers for the sm_100a kernels: PTX wrappers for asynchronous copies,
// shared-memory matrix loads and the bf16 warp-level MMA, plus launch-error bookkeeping.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/gaudirt_b200.h"

namespace gk {

// cudaError_t of the last failed launch on this host thread.
extern thread_local int g_last_cuda_error;

inline int check_launch() {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    g_last_cuda_error = static_cast<int>(e);
    return GK_ERR_CUDA;
  }
  return GK_OK;
}

// The opt-in for more than 48 KB of dynamic shared memory is per device and has to be made once
// before the first launch there.  `done` is one flag per device ordinal; the entry points may be
// called from several host threads, so the flags are atomics (setting the attribute twice is
// harmless, reading a half-written flag would not be).
template <typename Kernel>
inline int opt_in_shared_memory(Kernel kernel, int bytes, std::atomic<bool> (&done)[64]) {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return check_launch();
  const bool tracked = device >= 0 && device < 64;
  if (tracked && done[device].load(std::memory_order_acquire)) return GK_OK;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess)
    return check_launch();
  if (tracked) done[device].store(true, std::memory_order_release);
  return GK_OK;
}

// Programmatic dependent launch.  A kernel launched through launch_after_predecessor may be set up on
// the GPU while the kernel before it in the stream is still running; its first statement is
// wait_for_predecessor(), which lets the kernel AFTER it start its own set-up and then blocks until the
// kernel before it has completed and its writes are visible, so every access of the kernel body is
// ordered exactly as by plain stream order.  What overlaps is the launch latency and the scheduling of
// the CTAs, which is most of a decode layer's gap between kernels.  Launched the ordinary way (or with
// the switch off) both instructions do nothing.
extern std::atomic<int> g_programmatic_launch;

__device__ __forceinline__ void wait_for_predecessor() {
  asm volatile("griddepcontrol.launch_dependents;\ngriddepcontrol.wait;\n" ::: "memory");
}

template <typename... Params, typename... Args>
inline void launch_after_predecessor(void (*kernel)(Params...), dim3 grid, dim3 block, size_t shared_bytes,
                                     cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t config{};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = shared_bytes;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = g_programmatic_launch.load(std::memory_order_relaxed) ? 1 : 0;
  (void)cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);   // the caller reads the error with check_launch()
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte asynchronous global->shared copy, bypassing L1.  With src_bytes == 0 nothing is
// read and the 16 destination bytes are zero-filled.
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// D(16x8, fp32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);   // .x = lo (low 16 bits)
  return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

}  // namespace gk
