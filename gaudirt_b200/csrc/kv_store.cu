// Head-major KV store: scatter the new K/V rows of a step into their slots of the layer's
// [2, kv_heads, slots, head_dim] pool.  HBM-bound byte movement: one thread moves one 16-byte
// piece (or one element on the unaligned path), a warp covers two whole 256-byte head rows, so
// both the reads and the writes are full-sector coalesced.
#include "gk_common.cuh"

namespace gk {
thread_local int g_last_cuda_error = 0;
#ifndef GK_PROGRAMMATIC_LAUNCH_DEFAULT
#define GK_PROGRAMMATIC_LAUNCH_DEFAULT 0
#endif
std::atomic<int> g_programmatic_launch{GK_PROGRAMMATIC_LAUNCH_DEFAULT};

namespace {

// VEC = elements moved per thread (8 -> 16 bytes, 1 -> 2 bytes).
template <int VEC>
__global__ void __launch_bounds__(256) kv_store_kernel(const unsigned short* __restrict__ k,
                                                       const unsigned short* __restrict__ v,
                                                       int64_t k_stride, int64_t v_stride,
                                                       const int32_t* __restrict__ locations, int64_t rows,
                                                       unsigned short* __restrict__ pool_k,
                                                       unsigned short* __restrict__ pool_v, int64_t slots,
                                                       int kv_heads, int head_dim, int32_t* status) {
  const int pieces = head_dim / VEC;                           // per (row, head, K|V)
  const int64_t per_row = 2LL * kv_heads * pieces;
  const int64_t total = rows * per_row;
  // 32-bit index arithmetic whenever the launch allows it (a 64-bit division is a long subroutine) and a
  // shift for the usual power-of-two pieces per head
  const bool narrow = total <= 0x7fffffffLL;
  const int piece_shift = (pieces & (pieces - 1)) == 0 ? __ffs(pieces) - 1 : -1;
  const int per_kind = kv_heads * pieces;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t row;
    int rem;
    if (narrow) {
      const unsigned r = (unsigned)i / (unsigned)per_row;
      row = r;
      rem = (int)((unsigned)i - r * (unsigned)per_row);
    } else {
      row = i / per_row;
      rem = (int)(i - row * per_row);
    }
    const int kind = rem >= per_kind;
    rem -= kind * per_kind;
    const int head = piece_shift >= 0 ? rem >> piece_shift : rem / pieces, piece = rem - head * pieces;
    const int slot = __ldg(locations + row);
    if ((unsigned)slot >= (unsigned)slots) {
      if (status && piece == 0 && head == 0 && kind == 0) atomicOr(status, (int)GK_DEV_BAD_SLOT);
      continue;
    }
    const unsigned short* src = (kind ? v + row * v_stride : k + row * k_stride) + head * head_dim + piece * VEC;
    unsigned short* dst = (kind ? pool_v : pool_k) + ((int64_t)head * slots + slot) * head_dim + piece * VEC;
    if (VEC == 8) {
      *reinterpret_cast<uint4*>(dst) = __ldg(reinterpret_cast<const uint4*>(src));
    } else {
      *dst = __ldg(src);
    }
  }
}

}  // namespace
}  // namespace gk

extern "C" int gk_set_programmatic_launch(int on) {
  gk::g_programmatic_launch.store(on ? 1 : 0, std::memory_order_relaxed);
  return GK_OK;
}

extern "C" int gk_kv_store_head_major_bf16(const void* k, const void* v, int64_t k_row_stride, int64_t v_row_stride,
                                           const int32_t* locations, int64_t rows, void* pool_k, void* pool_v,
                                           int64_t slots, int kv_heads, int head_dim, int32_t* status,
                                           gk_stream_t stream) {
  if (rows == 0) return GK_OK;
  if (!k || !v || !locations || !pool_k || !pool_v || rows < 0 || slots <= 0 || kv_heads <= 0 || head_dim <= 0 ||
      k_row_stride < 0 || v_row_stride < 0)
    return GK_ERR_INVALID_ARGUMENT;
  if (kv_heads > 256 || head_dim % 8 != 0 || head_dim > 1024) return GK_ERR_UNSUPPORTED;
  const uintptr_t bits = reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                         reinterpret_cast<uintptr_t>(pool_k) | reinterpret_cast<uintptr_t>(pool_v);
  if (bits & 1) return GK_ERR_INVALID_ARGUMENT;
  const bool vec = !(bits & 15) && k_row_stride % 8 == 0 && v_row_stride % 8 == 0;
  const int64_t total = rows * 2 * kv_heads * (head_dim / (vec ? 8 : 1));
  const int threads = 256;
  const int64_t want = (total + threads - 1) / threads;
  const unsigned blocks = (unsigned)(want < 148 * 16 ? want : 148 * 16);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  auto* ks = static_cast<const unsigned short*>(k);
  auto* vs = static_cast<const unsigned short*>(v);
  auto* pk = static_cast<unsigned short*>(pool_k);
  auto* pv = static_cast<unsigned short*>(pool_v);
  if (vec)
    gk::kv_store_kernel<8><<<blocks, threads, 0, s>>>(ks, vs, k_row_stride, v_row_stride, locations, rows, pk, pv,
                                                      slots, kv_heads, head_dim, status);
  else
    gk::kv_store_kernel<1><<<blocks, threads, 0, s>>>(ks, vs, k_row_stride, v_row_stride, locations, rows, pk, pv,
                                                      slots, kv_heads, head_dim, status);
  return gk::check_launch();
}
