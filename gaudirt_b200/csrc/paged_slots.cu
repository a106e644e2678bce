// Steps either side of the attention path that the reference also runs on the device: paged
// slot allocation and release (src/bridge/paged_slot_allocator.cpp:91-209) and the per-step
// decode length update (src/bridge/eager_scheduler.cpp:51-82).  Integer work, bit-exact.
#include "gk_common.cuh"

namespace gk {
namespace {

constexpr int kThreads = 256;

// ---- decode length update -----------------------------------------------------------------
__global__ void advance_lengths_kernel(const int64_t* __restrict__ seq, const int32_t* __restrict__ orig,
                                       int64_t count, int64_t* __restrict__ next_seq,
                                       int32_t* __restrict__ next_orig) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  next_seq[i] = seq[i] + 1;
  next_orig[i] = orig[i] + 1;
}

// ---- allocation -----------------------------------------------------------------------------
// One thread per new token.  records[r] = {prefix, length, first token, first fresh page}.
// Token j of request r continues the partly filled page behind last_slots[r] while one is
// open (the first (-prefix) mod page_size tokens), then walks fresh pages in list order.
__global__ void allocate_kernel(const int64_t* __restrict__ last_slots, const int64_t* __restrict__ free_pages,
                                const int32_t* __restrict__ records, int n_requests, int64_t total,
                                int64_t page_size, int64_t* __restrict__ slots_out, int32_t* __restrict__ table,
                                int64_t table_stride, int64_t table_context,
                                const int32_t* __restrict__ table_rows, int64_t table_row_count,
                                int32_t* __restrict__ locations_out, int32_t* __restrict__ status) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= total) return;
  // Last record whose first token is <= t: records of empty requests share the first token
  // of the request that follows them and sort in front of it.
  int lo = 0, hi = n_requests - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if ((int64_t)records[4 * mid + 2] <= t) lo = mid; else hi = mid - 1;
  }
  const int4 rec = reinterpret_cast<const int4*>(records)[lo];
  const int64_t prefix = rec.x, j = t - rec.z;
  const int64_t open = (page_size - prefix % page_size) % page_size;
  const int64_t tail = open < (int64_t)rec.y ? open : (int64_t)rec.y;
  int64_t slot;
  if (j < tail) {
    slot = last_slots[lo] + 1 + j;
  } else {
    const int64_t k = j - tail;
    slot = free_pages[rec.w + k / page_size] * page_size + k % page_size;
  }
  slots_out[t] = slot;
  const bool narrow = slot >= 0 && slot <= INT32_MAX;
  if (locations_out) {
    locations_out[t] = narrow ? (int32_t)slot : 0;
    if (!narrow) atomicOr(status, GK_DEV_BAD_SLOT);
  }
  if (table) {
    const int64_t row = table_rows ? (int64_t)table_rows[lo] : (int64_t)lo;
    const int64_t position = prefix + j;
    if (!narrow || row < 0 || row >= table_row_count || position >= table_context) {
      if (status) atomicOr(status, narrow ? GK_DEV_BAD_TABLE : GK_DEV_BAD_SLOT);
    } else {
      table[row * table_stride + position] = (int32_t)slot;
    }
  }
}

// ---- release --------------------------------------------------------------------------------
// Slots -> pages in order of first occurrence, duplicates dropped.  first[page] is the smallest
// index of a slot on that page (atomicMin, so the order does not depend on scheduling); slot i
// emits its page iff first[page] == i; an ordered compaction writes the survivors.
constexpr int kReleaseThreads = 1024;
constexpr int kReleaseItems = 8;
constexpr int kReleaseTile = kReleaseThreads * kReleaseItems;

__device__ __forceinline__ bool slot_page(int64_t slot, int64_t page_size, int64_t max_pages, int64_t* page) {
  // Slot 0 is the padding slot and never belongs to a request (tests/paged_slots_device_smoke.py:42).
  if (slot <= 0) return false;
  *page = slot / page_size;
  return *page < max_pages;
}

__global__ void release_mark_kernel(const int64_t* __restrict__ slots, int64_t n, int64_t page_size, int64_t max_pages,
                                    unsigned* __restrict__ first, int32_t* __restrict__ count_out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  int64_t page;
  if (slot_page(slots[i], page_size, max_pages, &page)) atomicMin(first + page, (unsigned)i);
  else atomicAdd(count_out + 1, 1);
}

// Exclusive scan of one value per thread across the CTA; *total gets the CTA-wide sum.
__device__ int block_exclusive_scan(int value, int* total, int* warp_sums) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inclusive = value;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int up = __shfl_up_sync(0xffffffffu, inclusive, d);
    if (lane >= d) inclusive += up;
  }
  if (lane == 31) warp_sums[warp] = inclusive;
  __syncthreads();
  if (warp == 0) {
    int s = lane < (int)(blockDim.x >> 5) ? warp_sums[lane] : 0;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, s, d);
      if (lane >= d) s += up;
    }
    warp_sums[lane] = s;   // inclusive over warps
  }
  __syncthreads();
  const int before = warp ? warp_sums[warp - 1] : 0;
  *total = warp_sums[31];
  __syncthreads();
  return before + inclusive - value;
}

// Phase selected by `write`: 0 counts the survivors of each tile into tile_sums, 1 writes them
// behind the tile's offset.  A thread owns kReleaseItems consecutive slots, so positions inside
// the tile keep the input order.
template <bool kWrite>
__global__ void __launch_bounds__(kReleaseThreads)
release_compact_kernel(const int64_t* __restrict__ slots, int64_t n, int64_t page_size, int64_t max_pages,
                       const unsigned* __restrict__ first, int32_t* __restrict__ tile_sums,
                       int64_t* __restrict__ pages_out) {
  __shared__ int warp_sums[32];
  const int64_t base = (int64_t)blockIdx.x * kReleaseTile + (int64_t)threadIdx.x * kReleaseItems;
  int64_t pages[kReleaseItems];
  int keep = 0, mine = 0;
#pragma unroll
  for (int k = 0; k < kReleaseItems; ++k) {
    const int64_t i = base + k;
    int64_t page = 0;
    const bool hit = i < n && slot_page(slots[i], page_size, max_pages, &page) && first[page] == (unsigned)i;
    pages[k] = page;
    keep |= (int)hit << k;
    mine += hit;
  }
  int total;
  const int offset = block_exclusive_scan(mine, &total, warp_sums);
  if (!kWrite) {
    if (threadIdx.x == 0) tile_sums[blockIdx.x] = total;
    return;
  }
  int64_t at = (int64_t)tile_sums[blockIdx.x] + offset;
#pragma unroll
  for (int k = 0; k < kReleaseItems; ++k)
    if (keep >> k & 1) pages_out[at++] = pages[k];
}

// tile_sums -> exclusive offsets in place (one CTA walks all tiles); the grand total goes to
// count_out[0].
__global__ void __launch_bounds__(kReleaseThreads)
release_offsets_kernel(int32_t* __restrict__ tile_sums, int64_t n_tiles, int32_t* __restrict__ count_out) {
  __shared__ int warp_sums[32];
  int carry = 0;
  for (int64_t start = 0; start < n_tiles; start += kReleaseThreads) {
    const int64_t i = start + threadIdx.x;
    const int v = i < n_tiles ? tile_sums[i] : 0;
    int total;
    const int offset = block_exclusive_scan(v, &total, warp_sums);
    if (i < n_tiles) tile_sums[i] = carry + offset;
    carry += total;
  }
  if (threadIdx.x == 0) count_out[0] = carry;
}

// Everything in one CTA for a release of at most one tile (the usual case: the slots of a few
// finished requests).
__global__ void __launch_bounds__(kReleaseThreads)
release_small_kernel(const int64_t* __restrict__ slots, int n, int64_t page_size, int64_t max_pages,
                     unsigned* __restrict__ first, int64_t* __restrict__ pages_out, int32_t* __restrict__ count_out) {
  __shared__ int warp_sums[32];
  const int base = threadIdx.x * kReleaseItems;
  int64_t pages[kReleaseItems];
  int valid = 0, bad = 0;
#pragma unroll
  for (int k = 0; k < kReleaseItems; ++k) {
    const int i = base + k;
    pages[k] = 0;
    if (i >= n) continue;
    if (slot_page(slots[i], page_size, max_pages, &pages[k])) {
      valid |= 1 << k;
      atomicMin(first + pages[k], (unsigned)i);
    } else {
      ++bad;
    }
  }
  if (bad) atomicAdd(count_out + 1, bad);
  __syncthreads();
  int keep = 0, mine = 0;
#pragma unroll
  for (int k = 0; k < kReleaseItems; ++k) {
    const bool hit = (valid >> k & 1) && first[pages[k]] == (unsigned)(base + k);
    keep |= (int)hit << k;
    mine += hit;
  }
  int total;
  int at = block_exclusive_scan(mine, &total, warp_sums);
#pragma unroll
  for (int k = 0; k < kReleaseItems; ++k)
    if (keep >> k & 1) pages_out[at++] = pages[k];
  if (threadIdx.x == 0) count_out[0] = total;
}

inline uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

}  // namespace
}  // namespace gk

extern "C" int gk_advance_decode_lengths(const int64_t* seq_lens, const int32_t* orig_seq_lens, int64_t count,
                                         int64_t* next_seq_lens, int32_t* next_orig_seq_lens, gk_stream_t stream) {
  using namespace gk;
  if (!seq_lens || !orig_seq_lens || !next_seq_lens || !next_orig_seq_lens || count <= 0 || count > INT32_MAX)
    return GK_ERR_INVALID_ARGUMENT;
  const unsigned blocks = (unsigned)((count + kThreads - 1) / kThreads);
  advance_lengths_kernel<<<blocks, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      seq_lens, orig_seq_lens, count, next_seq_lens, next_orig_seq_lens);
  return check_launch();
}

extern "C" int gk_paged_slots_allocate(const int64_t* last_slots, const int64_t* free_pages, const int32_t* records,
                                       int64_t n_requests, int64_t total, int64_t page_size, int64_t* slots_out,
                                       int32_t* table, int64_t table_rows_count, int64_t table_stride,
                                       int64_t table_context, const int32_t* table_rows, int32_t* locations_out,
                                       int32_t* status, gk_stream_t stream) {
  using namespace gk;
  if (!last_slots || !free_pages || !records || !slots_out || n_requests <= 0 || n_requests > (int64_t{1} << 30) ||
      total <= 0 || total > (int64_t{1} << 30) || page_size < 1 || page_size > INT32_MAX ||
      (reinterpret_cast<uintptr_t>(records) & 15))
    return GK_ERR_INVALID_ARGUMENT;
  if (table && (table_rows_count <= 0 || table_context <= 0 || table_stride < table_context || !status))
    return GK_ERR_INVALID_ARGUMENT;
  if (locations_out && !status) return GK_ERR_INVALID_ARGUMENT;
  const unsigned blocks = (unsigned)((total + kThreads - 1) / kThreads);
  allocate_kernel<<<blocks, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      last_slots, free_pages, records, (int)n_requests, total, page_size, slots_out, table, table_stride,
      table_context, table_rows, table_rows_count, locations_out, status);
  return check_launch();
}

extern "C" int gk_paged_slots_release_workspace_bytes(int64_t n_slots, int64_t max_pages, uint64_t* bytes_out) {
  using namespace gk;
  if (!bytes_out || n_slots <= 0 || n_slots > (int64_t{1} << 30) || max_pages <= 0 || max_pages > INT32_MAX)
    return GK_ERR_INVALID_ARGUMENT;
  const uint64_t tiles = ((uint64_t)n_slots + kReleaseTile - 1) / kReleaseTile;
  *bytes_out = align_up((uint64_t)max_pages * 4, 256) + align_up(tiles * 4, 256);
  return GK_OK;
}

extern "C" int gk_paged_slots_release(const int64_t* slots, int64_t n_slots, int64_t page_size, int64_t max_pages,
                                      void* workspace, int64_t* pages_out, int32_t* count_out, gk_stream_t stream) {
  using namespace gk;
  if (!slots || !workspace || !pages_out || !count_out || n_slots <= 0 || n_slots > (int64_t{1} << 30) ||
      page_size < 1 || page_size > INT32_MAX || max_pages <= 0 || max_pages > INT32_MAX ||
      (reinterpret_cast<uintptr_t>(workspace) & 255))
    return GK_ERR_INVALID_ARGUMENT;
  auto s = static_cast<cudaStream_t>(stream);
  unsigned* first = static_cast<unsigned*>(workspace);
  int32_t* tile_sums = reinterpret_cast<int32_t*>(static_cast<char*>(workspace) + align_up((uint64_t)max_pages * 4, 256));
  const int64_t tiles = (n_slots + kReleaseTile - 1) / kReleaseTile;
  cudaError_t e = cudaMemsetAsync(first, 0xFF, (size_t)max_pages * 4, s);
  if (e == cudaSuccess) e = cudaMemsetAsync(count_out, 0, 2 * sizeof(int32_t), s);
  if (e != cudaSuccess) {
    g_last_cuda_error = (int)e;
    return GK_ERR_CUDA;
  }
  if (tiles == 1) {
    release_small_kernel<<<1, kReleaseThreads, 0, s>>>(slots, (int)n_slots, page_size, max_pages, first, pages_out,
                                                       count_out);
    return check_launch();
  }
  release_mark_kernel<<<(unsigned)((n_slots + kThreads - 1) / kThreads), kThreads, 0, s>>>(slots, n_slots, page_size,
                                                                                          max_pages, first, count_out);
  release_compact_kernel<false><<<(unsigned)tiles, kReleaseThreads, 0, s>>>(slots, n_slots, page_size, max_pages, first,
                                                                            tile_sums, pages_out);
  release_offsets_kernel<<<1, kReleaseThreads, 0, s>>>(tile_sums, tiles, count_out);
  release_compact_kernel<true><<<(unsigned)tiles, kReleaseThreads, 0, s>>>(slots, n_slots, page_size, max_pages, first,
                                                                           tile_sums, pages_out);
  return check_launch();
}
