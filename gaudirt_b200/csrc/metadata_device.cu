// Validation of device-resident scheduler metadata (the work of gk_paged_metadata_i32_v1 /
// gk_scheduler_metadata_i32_v1 / gk_token_indices_i32_v1 behind
// src/bridge/paged_metadata.cpp:176-430): narrows int64 index vectors to int32, expands
// per-sequence request ids to rows, and checks every row and every visible table entry without
// the step's indices ever visiting the host.
//
// Row codes (the ones tests/paged_device_metadata_smoke.py:130-150 observes are 1-4, 6, 7):
//   1  slot or position outside [0, slots) / [0, context) (includes a non-zero high word)
//   2  request id outside [0, n_requests)
//   3  table[request][position] is not the row's slot
//   4  two rows write the same slot
//   5  position is not prefix + offset of the row inside its sequence
//   6  a visible table entry is outside [0, slots)
//   7  a cached-prefix entry names a slot that this step writes
#include "gk_common.cuh"

#include <algorithm>

namespace gk {
namespace {

constexpr int kThreads = 256;
constexpr int kPrefixChunk = 2048;   // table entries one CTA of the prefix pass walks

__device__ __forceinline__ int64_t read_index(const void* p, bool wide, int64_t i) {
  return wide ? static_cast<const int64_t*>(p)[i] : (int64_t) static_cast<const int32_t*>(p)[i];
}

__device__ __forceinline__ void report(unsigned long long* first_error, int64_t row, int code) {
  atomicMin(first_error, ((unsigned long long)row << 8) | (unsigned)code);
}

struct RowArgs {
  const void *locations, *batch_requests, *positions, *token_ids;
  int wide;   // bit 0 locations, 1 batch_requests, 2 positions, 3 token_ids are int64
  int64_t vocabulary;
  const int32_t* table;
  int64_t n_requests, context, table_stride, slots;
  const int32_t* seq;
  int n_seq;
  int64_t rows;
  unsigned* written;   // one bit per slot
  int32_t *locations_out, *requests_out, *positions_out, *tokens_out, *last_token_out;
  int32_t *row_status, *token_status, *status;
  unsigned long long* first_error;
};

__global__ void rows_kernel(const RowArgs a) {
  const int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= a.rows) return;
  int lo = 0, hi = a.n_seq - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if ((int64_t)a.seq[4 * mid] <= row) lo = mid; else hi = mid - 1;
  }
  const int4 s = reinterpret_cast<const int4*>(a.seq)[lo];   // {first_row, n_rows, prefix, batch index}
  const int64_t slot = read_index(a.locations, a.wide & 1, row);
  const int64_t position = read_index(a.positions, a.wide & 4, row);
  const int64_t request = read_index(a.batch_requests, a.wide & 2, s.w);
  int code = 0;
  if (slot < 0 || slot >= a.slots || position < 0 || position >= a.context) code = 1;
  else if (request < 0 || request >= a.n_requests) code = 2;
  else if (position != (int64_t)s.z + (row - s.x)) code = 5;
  else if (a.table && a.table[request * a.table_stride + position] != (int32_t)slot) code = 3;
  else if (atomicOr(a.written + (slot >> 5), 1u << (slot & 31)) >> (slot & 31) & 1) code = 4;
  a.locations_out[row] = code == 1 ? 0 : (int32_t)slot;
  a.positions_out[row] = code == 1 ? 0 : (int32_t)position;
  a.requests_out[row] = (request < 0 || request >= a.n_requests) ? 0 : (int32_t)request;
  a.row_status[row] = code;
  if (code) {
    report(a.first_error, row, code);
    if (a.status) atomicOr(a.status, GK_DEV_BAD_METADATA);
  }
  if (a.token_ids) {
    const int64_t token = read_index(a.token_ids, a.wide & 8, row);
    const bool bad = token < 0 || token >= a.vocabulary;
    a.tokens_out[row] = bad ? 0 : (int32_t)token;
    a.token_status[row] = bad;
    if (bad) {
      atomicMin(a.first_error + 1, (unsigned long long)row);
      if (a.status) atomicOr(a.status, GK_DEV_BAD_METADATA);
    }
  }
  if (a.last_token_out && row == (int64_t)s.x + s.y - 1) a.last_token_out[lo] = (int32_t)row;
}

// Visible table entries of each sequence: grid (sequences, chunks).  Runs after rows_kernel,
// whose slot bits it reads.
__global__ void prefix_kernel(const RowArgs a) {
  const int4 s = reinterpret_cast<const int4*>(a.seq)[blockIdx.x];
  const int64_t request = read_index(a.batch_requests, a.wide & 2, s.w);
  if (request < 0 || request >= a.n_requests) return;
  const int prefix = s.z, end = s.z + s.y;
  const int32_t* row = a.table + request * a.table_stride;
  __shared__ int worst, page;
  if (threadIdx.x == 0) {
    worst = 0x7fffffff;
    page = 0x40000000;
  }
  __syncthreads();
  int code = 0x7fffffff, my_page = 0x40000000;
  for (int base = blockIdx.y * kPrefixChunk; base < end; base += gridDim.y * kPrefixChunk) {
    const int stop = min(end, base + kPrefixChunk);
    for (int p = base + threadIdx.x; p < stop; p += blockDim.x) {
      const int32_t slot = row[p];
      if (slot < 0 || (int64_t)slot >= a.slots) code = min(code, 6);
      else if (p < prefix && (a.written[slot >> 5] >> (slot & 31) & 1)) code = min(code, 7);
      // A break in slot contiguity at position p only allows pages that end there.
      if (p > 0 && slot != row[p - 1] + 1) my_page = min(my_page, p & -p);
    }
  }
  if (code != 0x7fffffff) atomicMin(&worst, code);
  if (my_page != 0x40000000) atomicMin(&page, my_page);
  __syncthreads();
  if (threadIdx.x == 0) {
    if (worst != 0x7fffffff) {
      atomicCAS(a.row_status + s.x, 0, worst);
      report(a.first_error, s.x, worst);
      if (a.status) atomicOr(a.status, GK_DEV_BAD_METADATA);
    }
    if (page != 0x40000000) atomicMin(a.first_error + 2, (unsigned long long)page);
  }
}

}  // namespace
}  // namespace gk

extern "C" int gk_paged_metadata_device_workspace_bytes(int64_t slots, uint64_t* bytes_out) {
  if (!bytes_out || slots <= 0 || slots > INT32_MAX) return GK_ERR_INVALID_ARGUMENT;
  *bytes_out = (((uint64_t)slots + 31) / 32 * 4 + 255) / 256 * 256;
  return GK_OK;
}

extern "C" int gk_paged_metadata_device_validate(
    const void* locations, const void* batch_requests, const void* positions, const void* token_ids, int wide_mask,
    int64_t vocabulary, const int32_t* table, int64_t n_requests, int64_t context, int64_t table_stride, int64_t slots,
    const int32_t* seq, int64_t n_seq, int64_t rows, void* workspace, int32_t* locations_out, int32_t* requests_out,
    int32_t* positions_out, int32_t* tokens_out, int32_t* last_token_out, int32_t* row_status, int32_t* token_status,
    uint64_t* first_error, int32_t* status, gk_stream_t stream) {
  using namespace gk;
  if (!locations || !batch_requests || !positions || !seq || !workspace || !locations_out || !requests_out ||
      !positions_out || !row_status || !first_error || n_seq <= 0 || rows <= 0 || n_seq > rows || rows > INT32_MAX ||
      slots <= 0 || slots > INT32_MAX || n_requests <= 0 || n_requests > INT32_MAX || context <= 0 ||
      context > INT32_MAX || (wide_mask & ~15) || (reinterpret_cast<uintptr_t>(seq) & 15) ||
      (reinterpret_cast<uintptr_t>(first_error) & 7))
    return GK_ERR_INVALID_ARGUMENT;
  if (table && table_stride < context) return GK_ERR_INVALID_ARGUMENT;
  if (token_ids && (!tokens_out || !token_status || vocabulary <= 0 || vocabulary > INT32_MAX))
    return GK_ERR_INVALID_ARGUMENT;
  auto s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(workspace, 0, (size_t)(((uint64_t)slots + 31) / 32 * 4), s);
  if (e == cudaSuccess) e = cudaMemsetAsync(first_error, 0xFF, 3 * sizeof(uint64_t), s);
  if (e != cudaSuccess) {
    g_last_cuda_error = (int)e;
    return GK_ERR_CUDA;
  }
  RowArgs a{locations, batch_requests, positions, token_ids, wide_mask, vocabulary, table, n_requests, context,
            table ? table_stride : 0, slots, seq, (int)n_seq, rows, static_cast<unsigned*>(workspace), locations_out,
            requests_out, positions_out, tokens_out, last_token_out, row_status, token_status, status,
            reinterpret_cast<unsigned long long*>(first_error)};
  rows_kernel<<<(unsigned)((rows + kThreads - 1) / kThreads), kThreads, 0, s>>>(a);
  if (table) {
    // Enough chunks per sequence to cover the longest possible range, capped so that the grid
    // stays near a few waves when there are many sequences.
    const int64_t per_seq = std::max<int64_t>(1, std::min<int64_t>((context + kPrefixChunk - 1) / kPrefixChunk,
                                                                    std::max<int64_t>(1, 1184 / n_seq)));
    prefix_kernel<<<dim3((unsigned)n_seq, (unsigned)per_seq), kThreads, 0, s>>>(a);
  }
  return check_launch();
}
