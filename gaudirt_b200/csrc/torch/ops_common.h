// Shared pieces of the PyTorch operator layer: error translation, the per-device status word, the
// attention plan carried by its device tensor, and the PagedMetadata class of the reference
// (src/bridge/paged_metadata.hpp) bound to CUDA tensors and to the C ABI of include/gaudirt_b200.h.
#pragma once

#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/custom_class.h>
#include <torch/library.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstring>
#include <memory>
#include <mutex>
#include <random>
#include <tuple>
#include <unordered_set>
#include <utility>
#include <vector>

#include "gaudirt_b200.h"


namespace gaudirt_b200 {


inline gk_stream_t stream_of(const c10::cuda::CUDAStream& s) { return reinterpret_cast<gk_stream_t>(s.stream()); }

inline void check_status(int status, const char* where) {
  if (status == GK_OK) return;
  if (status == GK_ERR_METADATA) TORCH_CHECK(false, gk_metadata_error());
  TORCH_CHECK(false, "GaudiRT: ", where, ": ", gk_status_string(status),
              status == GK_ERR_CUDA ? " (cudaError " + std::to_string(gk_last_cuda_error()) + ")" : std::string());
}

// One int32 status word per device; kernels OR gk_device_status bits into it.
inline at::Tensor& device_status(c10::DeviceIndex device) {
  static std::mutex mutex;
  static std::vector<at::Tensor> words(64);
  std::lock_guard<std::mutex> lock(mutex);
  TORCH_CHECK(device >= 0 && device < 64, "GaudiRT: device index out of range");
  if (!words[device].defined())
    words[device] = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(c10::Device(c10::kCUDA, device)));
  return words[device];
}

// Whether the KV store may ride in the attention launch (on by default; a test and tuning switch).
inline std::atomic<bool>& fuse_kv_store_flag() {
  static std::atomic<bool> flag{true};
  return flag;
}
inline bool fuse_kv_store() { return fuse_kv_store_flag().load(std::memory_order_relaxed); }

// Clears `bits` of the device status word, in stream order: for errors that were raised on the host.
inline void clear_status_bits(c10::DeviceIndex device, int bits) { device_status(device).bitwise_and_(~bits); }

// ---------------------------------------------------------------------------------------------
// attention plan carried by its device tensor (as in src/bridge/attention_plan.cpp:132-140,
// 319-322: the tensor's storage context owns the host-side schedule, so the tensor's lifetime
// is the plan's lifetime and a foreign or stale tensor is rejected).
// ---------------------------------------------------------------------------------------------
struct AttentionPlan {
  at::Tensor buffer;      // int32 device words: work records, then combine records
  at::Tensor part_ml;     // fp32 split state (m, l) per partial entry
  at::Tensor part_o;      // fp32 split state O per partial entry
  at::Tensor counters;    // int32 [rows * kv_heads] arrival counts of the fused combine (zero between launches)
  at::Tensor table;       // int32 slot table the work records index
  at::Tensor table_rows;  // optional int32 row indirection (device-resident request ids)
  void* address = nullptr;
  cudaStream_t stream = nullptr;
  c10::DeviceIndex device = -1;
  int64_t rows = 0, slots = 0, query_heads = 0, kv_heads = 0, head_dim = 0, sliding_window = -1;
  int64_t n_work = 0, n_combine = 0, combine_offset = 0, table_stride = 0, entry_stride = 1;
  int64_t n_prefill = 0, prefill_offset = 0;   // query tiles for the tensor-core prefill kernel
  int page_tokens = 1;
  // Every sequence of the step is one query block of the decode kernel (no other CTA reads a new row):
  // the KV store may then ride in the attention launch.
  bool single_block = false;
};

inline void release_plan(void* context) { delete static_cast<AttentionPlan*>(context); }

inline at::Tensor wrap_plan(std::unique_ptr<AttentionPlan> plan) {
  const auto bytes = static_cast<size_t>(plan->buffer.nbytes());
  const auto device = plan->buffer.device();
  void* address = plan->buffer.data_ptr();
  plan->address = address;
  c10::DataPtr data(address, plan.release(), &release_plan, device);
  auto storage = c10::make_intrusive<c10::StorageImpl>(c10::StorageImpl::use_byte_size_t(), bytes, std::move(data),
                                                       /*allocator=*/nullptr, /*resizable=*/false);
  auto tensor = at::detail::make_tensor<c10::TensorImpl>(std::move(storage), c10::DispatchKeySet(c10::DispatchKey::CUDA),
                                                         caffe2::TypeMeta::Make<int32_t>());
  tensor.unsafeGetTensorImpl()->set_sizes_contiguous({static_cast<int64_t>(bytes / sizeof(int32_t))});
  return tensor;
}

inline const AttentionPlan& plan_of(const at::Tensor& tensor) {
  TORCH_CHECK(tensor.defined() && tensor.is_cuda(), "GaudiRT attention: expected a device metadata plan");
  const auto* plan = tensor.storage().data_ptr().cast_context<AttentionPlan>(&release_plan);
  TORCH_CHECK(plan && tensor.data_ptr() == plan->address && tensor.device().index() == plan->device,
              "GaudiRT attention: invalid or expired metadata plan");
  return *plan;
}

inline std::vector<int32_t> host_i32(const at::Tensor& t) {
  std::vector<int32_t> out(static_cast<size_t>(t.numel()));
  if (t.scalar_type() == at::kInt) {
    std::memcpy(out.data(), t.data_ptr<int32_t>(), out.size() * sizeof(int32_t));
  } else {
    const int64_t* src = t.data_ptr<int64_t>();
    for (size_t i = 0; i < out.size(); ++i) {
      TORCH_CHECK(src[i] >= INT32_MIN && src[i] <= INT32_MAX, "GaudiRT: paged metadata index is out of range");
      out[i] = static_cast<int32_t>(src[i]);
    }
  }
  return out;
}


// ---------------------------------------------------------------------------------------------
// PagedMetadata
// ---------------------------------------------------------------------------------------------
class PagedMetadata : public torch::CustomClassHolder {
 public:
  // Host constructor (src/bridge/paged_metadata.cpp:82-174): validates on the host, then uploads
  // locations / requests / positions / mapping / header with ONE pinned staging buffer and one
  // asynchronous copy on the current stream.
  PagedMetadata(const at::Tensor& locations, const at::Tensor& requests, const at::Tensor& positions,
                const at::Tensor& mapping, int64_t slots) {
    for (const auto& t : {locations, requests, positions, mapping})
      TORCH_CHECK(t.device().is_cpu() && t.is_contiguous() && (t.scalar_type() == at::kInt || t.scalar_type() == at::kLong),
                  "GaudiRT: paged metadata must be contiguous CPU int32 or int64");
    TORCH_CHECK(locations.dim() == 1 && requests.dim() == 1 && positions.dim() == 1 && mapping.dim() == 2 &&
                    locations.size(0) == requests.size(0) && locations.size(0) == positions.size(0),
                "GaudiRT: invalid paged metadata ranks or row counts");
    const int64_t m = locations.size(0), n_req = mapping.size(0), context = mapping.size(1);
    const auto loc = host_i32(locations), req = host_i32(requests), pos = host_i32(positions), map = host_i32(mapping);
    sequences_.resize(static_cast<size_t>(std::max<int64_t>(m, 1)) * 4);
    int64_t n_seq = 0;
    int32_t page = 1;
    check_status(gk_paged_metadata_validate(loc.data(), req.data(), pos.data(), m, map.data(), n_req, context, slots,
                                            sequences_.data(), &n_seq, &page),
                 "paged metadata");
    sequences_.resize(static_cast<size_t>(n_seq) * 4);
    page_tokens_ = page;
    rows_ = m;
    slots_ = slots;
    request_count_ = n_req;
    context_ = context;
    {
      // No sequence reads a row another sequence of this step writes iff no request occurs twice
      // (a continuation chunk of the same request sees the earlier chunk's new rows).
      std::vector<int32_t> seen;
      for (int64_t i = 0; i < n_seq; ++i) seen.push_back(sequences_[static_cast<size_t>(i) * 4 + 3]);
      std::sort(seen.begin(), seen.end());
      rows_independent_ = std::adjacent_find(seen.begin(), seen.end()) == seen.end();
    }

    const auto device = c10::Device(c10::kCUDA, at::cuda::current_device());
    const int64_t words = 3 * m + n_req * context + 1;
    auto staging = at::empty({words}, at::TensorOptions().dtype(at::kInt).pinned_memory(true));
    int32_t* host = staging.data_ptr<int32_t>();
    std::memcpy(host, loc.data(), m * 4);
    std::memcpy(host + m, req.data(), m * 4);
    std::memcpy(host + 2 * m, pos.data(), m * 4);
    std::memcpy(host + 3 * m, map.data(), n_req * context * 4);
    host[words - 1] = static_cast<int32_t>(m);
    auto all = staging.to(device, /*non_blocking=*/true);
    locations_ = all.narrow(0, 0, m);
    requests_ = all.narrow(0, m, m);
    positions_ = all.narrow(0, 2 * m, m);
    mapping_ = all.narrow(0, 3 * m, n_req * context).view({n_req, context});
    header_ = all.narrow(0, words - 1, 1);
  }

  // Device-input constructor (src/bridge/paged_metadata.cpp:176-430): `batch_requests[batch]`
  // indexes a persistent device table `mapping[max_requests, max_context]`; `prefixes` and
  // `lengths` are the host lists of cached length and new-token count per sequence.  The index
  // vectors never visit the host: one validation pass on the device narrows them to int32,
  // expands request ids to rows and checks every row and visible table entry.  With
  // `scheduler_owned` the table is vouched for by the scheduler (not re-checked) and a rejection
  // only sets GK_DEV_BAD_METADATA in the device status word, so nothing synchronises; otherwise
  // the 24-byte verdict is read back and a rejection raises here.
  PagedMetadata(const at::Tensor& locations, const at::Tensor& batch_requests, const at::Tensor& positions,
                const at::Tensor& mapping, std::vector<int64_t> prefixes, std::vector<int64_t> lengths, int64_t slots,
                const at::Tensor& token_ids, int64_t vocabulary, bool scheduler_owned) {
    for (const auto& t : {locations, batch_requests, positions})
      TORCH_CHECK(t.is_cuda() && t.dim() == 1 && (t.scalar_type() == at::kInt || t.scalar_type() == at::kLong),
                  "GaudiRT device metadata: expected CUDA int32 or int64 vectors");
    TORCH_CHECK(mapping.is_cuda() && mapping.scalar_type() == at::kInt && mapping.dim() == 2 && mapping.is_contiguous(),
                "GaudiRT device metadata: expected a contiguous CUDA int32 request map");
    const bool has_tokens = token_ids.defined() && token_ids.numel() > 0;
    const int64_t m = locations.numel(), batch = batch_requests.numel();
    TORCH_CHECK((has_tokens && token_ids.is_cuda() && token_ids.dim() == 1 && token_ids.numel() == m &&
                 (token_ids.scalar_type() == at::kInt || token_ids.scalar_type() == at::kLong) && vocabulary > 0 &&
                 vocabulary <= INT32_MAX) || (!has_tokens && vocabulary == 0),
                "GaudiRT device metadata: invalid token IDs or vocabulary size");
    TORCH_CHECK(m > 0 && m <= INT32_MAX && positions.numel() == m && batch > 0 && batch <= m &&
                    static_cast<int64_t>(prefixes.size()) == batch && static_cast<int64_t>(lengths.size()) == batch &&
                    slots > 0 && slots <= INT32_MAX && mapping.numel() > 0 && mapping.numel() <= INT32_MAX,
                "GaudiRT device metadata: dimensions outside supported range");
    const int64_t context = mapping.size(1);
    const auto device = locations.device();
    c10::cuda::CUDAGuard guard(device);
    // Per-sequence records and last-row indices are host knowledge: one pinned buffer, one copy.
    auto staging = at::empty({batch * 4}, at::TensorOptions().dtype(at::kInt).pinned_memory(true));
    int32_t* records = staging.data_ptr<int32_t>();
    int64_t cursor = 0;
    for (int64_t i = 0; i < batch; ++i) {
      const int64_t prefix = prefixes[i], length = lengths[i];
      TORCH_CHECK(prefix >= 0 && prefix < context && length > 0 && length <= context - prefix && length <= m - cursor,
                  "GaudiRT device metadata: invalid sequence lengths");
      const int32_t record[4] = {static_cast<int32_t>(cursor), static_cast<int32_t>(length),
                                 static_cast<int32_t>(prefix), static_cast<int32_t>(i)};
      std::memcpy(records + 4 * i, record, sizeof(record));
      sequences_.insert(sequences_.end(), record, record + 4);
      cursor += length;
    }
    TORCH_CHECK(cursor == m, "GaudiRT device metadata: sequence lengths do not cover token rows");
    rows_ = m;
    slots_ = slots;
    request_count_ = mapping.size(0);
    context_ = context;
    mapping_ = mapping;
    // The validated form rejects (code 7) a batch in which a cached prefix names a slot this step
    // writes, so its sequences never read each other's new rows; the scheduler-owned form skips
    // that check and nothing is known here.
    rows_independent_ = !scheduler_owned;
    const auto i32 = at::TensorOptions().dtype(at::kInt).device(device);
    auto seq_device = staging.to(device, /*non_blocking=*/true);
    // Strided views (a column of a scheduler's packed buffer) are packed first, like the
    // reference's staged copy (src/bridge/paged_metadata.cpp:362-381).
    const at::Tensor loc = locations.contiguous(), req = batch_requests.contiguous(), pos = positions.contiguous();
    const at::Tensor tok = has_tokens ? token_ids.contiguous() : at::Tensor();
    // locations | requests | positions | tokens | row status | token status | last rows | batch ids
    const int64_t lanes = 4 + (has_tokens ? 2 : 0);
    auto out = at::empty({lanes * m + 2 * batch}, i32);
    locations_ = out.narrow(0, 0, m);
    requests_ = out.narrow(0, m, m);
    positions_ = out.narrow(0, 2 * m, m);
    auto row_status = out.narrow(0, 3 * m, m);
    at::Tensor token_status;
    if (has_tokens) {
      token_ids_ = out.narrow(0, 4 * m, m);
      token_status = out.narrow(0, 5 * m, m);
      vocabulary_ = vocabulary;
    }
    last_token_indices_ = out.narrow(0, lanes * m, batch);
    batch_requests_ = req.scalar_type() == at::kInt ? req : req.to(at::kInt);
    header_ = at::full({1}, rows_, i32);
    uint64_t workspace_bytes = 0;
    check_status(gk_paged_metadata_device_workspace_bytes(slots, &workspace_bytes), "device metadata");
    auto workspace = at::empty({static_cast<int64_t>(workspace_bytes)}, at::TensorOptions().dtype(at::kByte).device(device));
    auto verdict = at::empty({3}, at::TensorOptions().dtype(at::kLong).device(device));
    const int wide = (loc.scalar_type() == at::kLong ? 1 : 0) | (req.scalar_type() == at::kLong ? 2 : 0) |
                     (pos.scalar_type() == at::kLong ? 4 : 0) | (has_tokens && tok.scalar_type() == at::kLong ? 8 : 0);
    const auto stream = at::cuda::getCurrentCUDAStream(device.index());
    check_status(gk_paged_metadata_device_validate(
                     loc.data_ptr(), req.data_ptr(), pos.data_ptr(), has_tokens ? tok.data_ptr() : nullptr, wide,
                     vocabulary, scheduler_owned ? nullptr : mapping.data_ptr<int32_t>(), mapping.size(0), context,
                     mapping.stride(0), slots, seq_device.data_ptr<int32_t>(), batch, m, workspace.data_ptr(),
                     locations_.data_ptr<int32_t>(), requests_.data_ptr<int32_t>(), positions_.data_ptr<int32_t>(),
                     has_tokens ? token_ids_.data_ptr<int32_t>() : nullptr, last_token_indices_.data_ptr<int32_t>(),
                     row_status.data_ptr<int32_t>(), has_tokens ? token_status.data_ptr<int32_t>() : nullptr,
                     reinterpret_cast<uint64_t*>(verdict.data_ptr<int64_t>()),
                     device_status(device.index()).data_ptr<int32_t>(), stream_of(stream)),
                 "device metadata");
    dev_seq_ = seq_device;
    dev_workspace_ = workspace;
    dev_verdict_ = verdict;
    dev_row_status_ = row_status;
    table_checked_ = !scheduler_owned;
    if (!scheduler_owned) {
      const auto host = verdict.cpu();   // 24 bytes: the only read-back of the step
      const uint64_t first = static_cast<uint64_t>(host.data_ptr<int64_t>()[0]);
      const uint64_t token = static_cast<uint64_t>(host.data_ptr<int64_t>()[1]);
      // Largest page the visible table ranges are contiguous in: the kernels then walk one table
      // entry per page and the prefill kernel may fetch whole pages by TMA.
      const uint64_t page = static_cast<uint64_t>(host.data_ptr<int64_t>()[2]);
      page_tokens_ = static_cast<int64_t>(std::min<uint64_t>(page, 128));
      if (first != UINT64_MAX || token != UINT64_MAX) clear_status_bits(device.index(), GK_DEV_BAD_METADATA);
      uint64_t bad_row = first >> 8, bad_code = first & 255;
      if (first != UINT64_MAX && bad_code == 4) {
        // Two rows write one slot: on the device, which of them met the other's mark depends on arrival
        // order.  The error path can afford a walk on the host over the per-row codes: a duplicate is charged
        // to the later row of the pair, as the reference's host constructor does
        // (src/bridge/paged_metadata.cpp:104-140), and the first row in row order that carries any code is
        // the one reported.
        const auto slots_host = loc.to(at::kLong).cpu();
        const auto codes_host = row_status.cpu();
        const int64_t* sl = slots_host.data_ptr<int64_t>();
        const int32_t* codes = codes_host.data_ptr<int32_t>();
        std::unordered_set<int64_t> seen;
        for (int64_t r = 0; r < m; ++r) {
          // only a row that passed its own range and table checks marks its slot (as on the device)
          const bool passed = codes[r] == 0 || codes[r] == 4;
          const bool duplicate = passed && !seen.insert(sl[r]).second;
          const int32_t code = duplicate ? 4 : (passed ? 0 : codes[r]);
          if (code != 0) {
            bad_row = static_cast<uint64_t>(r);
            bad_code = static_cast<uint64_t>(code);
            break;
          }
        }
      }
      TORCH_CHECK(first == UINT64_MAX, "GaudiRT device metadata: invalid scheduler metadata at row ", bad_row,
                  ", code ", bad_code);
      TORCH_CHECK(token == UINT64_MAX, "GaudiRT device metadata: token ID outside vocabulary at row ", token);
    }
  }

  static c10::intrusive_ptr<PagedMetadata> from_device(const at::Tensor& locations, const at::Tensor& batch_requests,
                                                       const at::Tensor& positions, const at::Tensor& mapping,
                                                       std::vector<int64_t> prefixes, std::vector<int64_t> lengths,
                                                       int64_t slots) {
    return c10::make_intrusive<PagedMetadata>(locations, batch_requests, positions, mapping, std::move(prefixes),
                                              std::move(lengths), slots, at::Tensor(), 0, false);
  }
  static c10::intrusive_ptr<PagedMetadata> from_device_with_tokens(
      const at::Tensor& locations, const at::Tensor& batch_requests, const at::Tensor& positions,
      const at::Tensor& mapping, std::vector<int64_t> prefixes, std::vector<int64_t> lengths, int64_t slots,
      const at::Tensor& token_ids, int64_t vocabulary) {
    return c10::make_intrusive<PagedMetadata>(locations, batch_requests, positions, mapping, std::move(prefixes),
                                              std::move(lengths), slots, token_ids, vocabulary, false);
  }
  static c10::intrusive_ptr<PagedMetadata> from_scheduler(const at::Tensor& locations, const at::Tensor& batch_requests,
                                                          const at::Tensor& positions, const at::Tensor& mapping,
                                                          std::vector<int64_t> prefixes, std::vector<int64_t> lengths,
                                                          int64_t slots, const c10::optional<at::Tensor>& token_ids,
                                                          int64_t vocabulary) {
    return c10::make_intrusive<PagedMetadata>(locations, batch_requests, positions, mapping, std::move(prefixes),
                                              std::move(lengths), slots, token_ids.value_or(at::Tensor()), vocabulary,
                                              true);
  }
  static c10::intrusive_ptr<PagedMetadata> from_scheduler_fused(
      const at::Tensor& locations, const at::Tensor& batch_requests, const at::Tensor& positions,
      const at::Tensor& mapping, std::vector<int64_t> prefixes, std::vector<int64_t> lengths, int64_t slots,
      const c10::optional<at::Tensor>& token_ids, int64_t vocabulary, int64_t query_heads, int64_t kv_heads,
      int64_t head_dim) {
    auto md = from_scheduler(locations, batch_requests, positions, mapping, std::move(prefixes), std::move(lengths),
                             slots, token_ids, vocabulary);
    md->attention_plan(query_heads, kv_heads, head_dim);
    return md;
  }

  // Validates a NEW set of index vectors for a step of the SAME shape (same sequences, prefixes and
  // lengths) into this object's device tensors, so that everything bound to them -- the attention
  // plan, a captured CUDA graph -- stays valid.  Only kernel launches on the current stream: no
  // allocation, no host staging, no read-back, so the call can be captured and replayed with the
  // index vectors refreshed in place before every replay.  A rejection sets GK_DEV_BAD_METADATA in
  // the device status word (read it at the end of the step).  Not part of the reference surface,
  // whose fused scheduler form (src/bridge/paged_metadata.hpp:45-64) rebuilds the object instead.
  void revalidate_(const at::Tensor& locations, const at::Tensor& batch_requests, const at::Tensor& positions) {
    TORCH_CHECK(dev_seq_.defined(), "GaudiRT device metadata: only device-validated metadata can be revalidated");
    TORCH_CHECK(!token_ids_.defined(), "GaudiRT device metadata: revalidation with token IDs is not supported");
    const auto device = locations_.device();
    const int64_t batch = dev_seq_.numel() / 4;
    for (const auto& t : {locations, batch_requests, positions})
      TORCH_CHECK(t.is_cuda() && t.device() == device && t.dim() == 1 && t.is_contiguous() &&
                      (t.scalar_type() == at::kInt || t.scalar_type() == at::kLong),
                  "GaudiRT device metadata: expected CUDA int32 or int64 vectors");
    TORCH_CHECK(locations.numel() == rows_ && positions.numel() == rows_ && batch_requests.numel() == batch,
                "GaudiRT device metadata: dimensions outside supported range");
    TORCH_CHECK(batch_requests.scalar_type() == at::kInt && batch_requests.data_ptr() == batch_requests_.data_ptr(),
                "GaudiRT device metadata: revalidation needs the int32 request vector the metadata was built on");
    c10::cuda::CUDAGuard guard(device);
    const int wide = (locations.scalar_type() == at::kLong ? 1 : 0) | (positions.scalar_type() == at::kLong ? 4 : 0);
    check_status(gk_paged_metadata_device_validate(
                     locations.data_ptr(), batch_requests.data_ptr(), positions.data_ptr(), nullptr, wide, 0,
                     table_checked_ ? mapping_.data_ptr<int32_t>() : nullptr, mapping_.size(0), context_,
                     mapping_.stride(0), slots_, dev_seq_.data_ptr<int32_t>(), batch, rows_, dev_workspace_.data_ptr(),
                     locations_.data_ptr<int32_t>(), requests_.data_ptr<int32_t>(), positions_.data_ptr<int32_t>(),
                     nullptr, last_token_indices_.data_ptr<int32_t>(), dev_row_status_.data_ptr<int32_t>(), nullptr,
                     reinterpret_cast<uint64_t*>(dev_verdict_.data_ptr<int64_t>()),
                     device_status(device.index()).data_ptr<int32_t>(),
                     stream_of(at::cuda::getCurrentCUDAStream(device.index()))),
                 "device metadata");
  }

  int64_t rows() const { return rows_; }
  int64_t slots() const { return slots_; }
  int64_t context() const { return context_; }
  int64_t page_tokens() const { return page_tokens_; }
  at::Tensor rotary_positions() const { return positions_; }
  at::Tensor rotary_header() const { return header_; }
  at::Tensor row_locations() const { return locations_; }
  at::Tensor row_requests() const { return requests_; }
  at::Tensor request_mapping() const { return mapping_; }
  at::Tensor last_token_indices() const {
    TORCH_CHECK(last_token_indices_.defined(), "GaudiRT: last-token indices require batched metadata");
    return last_token_indices_;
  }
  at::Tensor token_ids() const {
    TORCH_CHECK(token_ids_.defined(), "GaudiRT: token IDs were not validated in this metadata");
    return token_ids_;
  }
  int64_t vocabulary() const { return vocabulary_; }
  std::vector<int64_t> sequences() const { return std::vector<int64_t>(sequences_.begin(), sequences_.end()); }

  at::Tensor attention_plan(int64_t query_heads, int64_t kv_heads, int64_t head_dim) {
    return attention_plan_for(query_heads, kv_heads, head_dim, -1);
  }

  // Schedule for one step, shared by all layers (src/bridge/attention_plan.cpp:146-361).
  at::Tensor attention_plan_for(int64_t query_heads, int64_t kv_heads, int64_t head_dim, int64_t sliding_window) {
    TORCH_CHECK(sliding_window == -1 || (sliding_window > 0 && sliding_window <= INT32_MAX),
                "GaudiRT attention: invalid sliding window size");
    for (const auto& entry : plans_) {
      if (entry.first != sliding_window) continue;
      const auto& plan = plan_of(entry.second);
      TORCH_CHECK(plan.query_heads == query_heads && plan.kv_heads == kv_heads && plan.head_dim == head_dim,
                  "GaudiRT attention: metadata already bound to different head geometry");
      return entry.second;
    }
    TORCH_CHECK(query_heads > 0 && query_heads <= 256 && kv_heads > 0 && kv_heads <= 256 &&
                    query_heads % kv_heads == 0 && (head_dim == 64 || head_dim == 128 || head_dim == 256),
                "GaudiRT attention: unsupported head or request-map geometry");
    const auto device = locations_.device();
    c10::cuda::CUDAGuard guard(device);
    const int sm_count = at::cuda::getDeviceProperties(device.index())->multiProcessorCount;
    const int64_t n_seq = static_cast<int64_t>(sequences_.size() / 4);
    const int window = static_cast<int>(sliding_window);
    // Multi-row sequences go to the tensor-core prefill kernel, the rest -- decode rows and very
    // short chunks -- to the split-KV decode kernel.
    int64_t n_prefill = 0, n_rest = n_seq;
    std::vector<int32_t> rest(sequences_);
    const bool tensor_core = prefill_min_rows_ >= 0;
    if (tensor_core)
      check_status(gk_prefill_plan_build(sequences_.data(), n_seq, (int)query_heads, (int)kv_heads, window,
                                         prefill_min_rows_, nullptr, 0, &n_prefill, rest.data(), &n_rest),
                   "prefill plan");
    int64_t n_work = 0, n_combine = 0, entries = 0;
    if (n_rest > 0)
      check_status(gk_attention_plan_build(rest.data(), n_rest, (int)query_heads, (int)kv_heads, (int)head_dim, window,
                                           sm_count, split_tokens_, nullptr, 0, &n_work, nullptr, 0, &n_combine, &entries),
                   "attention plan");
    const int64_t combine_offset = n_work * GK_WORK_WORDS;
    const int64_t prefill_offset = combine_offset + n_combine * GK_COMBINE_WORDS;
    const int64_t words = std::max<int64_t>(4, prefill_offset + n_prefill * GK_WORK_WORDS);
    auto staging = at::empty({words}, at::TensorOptions().dtype(at::kInt).pinned_memory(true));
    int32_t* host = staging.data_ptr<int32_t>();
    if (n_rest > 0)
      check_status(gk_attention_plan_build(rest.data(), n_rest, (int)query_heads, (int)kv_heads, (int)head_dim, window,
                                           sm_count, split_tokens_, host, n_work, &n_work, host + combine_offset,
                                           n_combine, &n_combine, &entries),
                   "attention plan");
    if (n_prefill > 0)
      check_status(gk_prefill_plan_build(sequences_.data(), n_seq, (int)query_heads, (int)kv_heads, window,
                                         prefill_min_rows_, host + prefill_offset, n_prefill, &n_prefill, rest.data(),
                                         &n_rest),
                   "prefill plan");
    auto plan = std::make_unique<AttentionPlan>();
    plan->buffer = staging.to(device, /*non_blocking=*/true);
    const auto f32 = at::TensorOptions().dtype(at::kFloat).device(device);
    plan->part_ml = at::empty({std::max<int64_t>(entries, 1) * 2}, f32);
    plan->part_o = at::empty({std::max<int64_t>(entries, 1) * head_dim}, f32);
    // Fused combine (the last split of a block to finish merges it inside the attention kernel) pays
    // when few blocks are split: it saves a launch whose grid would be small.  With many split
    // blocks the merges are better spread over the whole GPU by the separate combine kernel
    // (measured: 2-10 % faster fused at 4-59 split blocks, even at 61, 2-9 % slower at 64-256).
    // Blocks cut in two (the uneven cut that fills a tensor-parallel shard's single wave) merge so little state
    // that the fused form costs nothing even with hundreds of them, and it saves the launch.
    int32_t most_splits = 0;
    for (int64_t i = 0; i < n_combine; ++i) most_splits = std::max(most_splits, host[combine_offset + i * GK_COMBINE_WORDS + 3]);
    const bool fuse = fused_combine_ > 0 || (fused_combine_ < 0 && (n_combine * 5 <= sm_count * 2 || most_splits <= 2));
    last_plan_fused_ = n_combine > 0 && fuse;
    if (n_combine > 0 && fuse)
      plan->counters = at::zeros({rows_ * kv_heads}, at::TensorOptions().dtype(at::kInt).device(device));
    plan->table = mapping_;
    plan->table_rows = batch_requests_;
    plan->table_stride = mapping_.stride(0);
    plan->page_tokens = static_cast<int>(page_tokens_);
    plan->entry_stride = page_tokens_;
    plan->stream = at::cuda::getCurrentCUDAStream(device.index()).stream();
    plan->device = device.index();
    plan->rows = rows_;
    plan->slots = slots_;
    plan->query_heads = query_heads;
    plan->kv_heads = kv_heads;
    plan->head_dim = head_dim;
    plan->sliding_window = sliding_window;
    plan->n_work = n_work;
    plan->n_combine = n_combine;
    plan->combine_offset = combine_offset;
    plan->n_prefill = n_prefill;
    plan->prefill_offset = prefill_offset;
    {
      const int64_t block_rows = std::max<int64_t>(1, GK_MAX_PACKED_ROWS / (query_heads / kv_heads));
      bool single = n_prefill == 0 && n_work > 0 && rows_independent_;
      for (int64_t i = 0; single && i < n_seq; ++i) single = sequences_[static_cast<size_t>(i) * 4 + 1] <= block_rows;
      plan->single_block = single;
    }
    auto tensor = wrap_plan(std::move(plan));
    plans_.emplace_back(sliding_window, tensor);
    return tensor;
  }

  std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor, int64_t>
  forward_tensors(int64_t query_heads, int64_t kv_heads, int64_t head_dim) {
    return {token_ids(), last_token_indices(), rotary_positions(), rotary_header(), row_locations(),
            row_requests(), attention_plan(query_heads, kv_heads, head_dim), context_};
  }

  // Longest KV range of one work item for plans built after this call (0 = chosen from the SM
  // count).  Not part of the reference surface: a test and tuning hook.
  void set_split_tokens(int64_t tokens) {
    TORCH_CHECK(tokens >= 0 && tokens <= INT32_MAX, "GaudiRT attention: invalid split size");
    split_tokens_ = static_cast<int>(tokens);
  }

  // Fewest rows of a sequence that are sent to the tensor-core prefill kernel (0 = the library's
  // default, -1 = never).  Not part of the reference surface: a test and tuning hook.
  void set_prefill_min_rows(int64_t rows) {
    TORCH_CHECK(rows >= -1 && rows <= INT32_MAX, "GaudiRT attention: invalid prefill threshold");
    prefill_min_rows_ = static_cast<int>(rows);
  }

  int64_t rows_ = 0, slots_ = 0, request_count_ = 0, context_ = 0, vocabulary_ = 0, page_tokens_ = 1;
  // -1: decide from the schedule, 0: separate combine kernel, 1: combine fused into attention.
  bool last_plan_fuses_combine() const { return last_plan_fused_; }
  void set_fused_combine(int64_t mode) {
    TORCH_CHECK(mode >= -1 && mode <= 1, "GaudiRT attention: invalid combine mode");
    fused_combine_ = static_cast<int>(mode);
  }
  int split_tokens_ = 0, prefill_min_rows_ = 0, fused_combine_ = -1;
  bool last_plan_fused_ = false;       // whether the plan built last merges its splits inside the attention kernel
  bool rows_independent_ = false;   // no sequence of the step reads a row that another sequence writes
  at::Tensor locations_, requests_, positions_, mapping_, header_, batch_requests_, token_ids_, last_token_indices_;
  at::Tensor dev_seq_, dev_workspace_, dev_verdict_, dev_row_status_;   // device-validated forms only (revalidate_)
  bool table_checked_ = false;
  std::vector<int32_t> sequences_;   // {first_row, n_rows, first_position, table_row} per sequence
  std::vector<std::pair<int64_t, at::Tensor>> plans_;
};

// operators defined in ops_steps.cpp (registered in ops.cpp)
std::tuple<at::Tensor, int64_t> allocate_paged_slots(const at::Tensor& last_slots, const at::Tensor& free_pages,
                                                     std::vector<int64_t> prefixes, std::vector<int64_t> lengths,
                                                     int64_t page_size);
std::tuple<at::Tensor, at::Tensor, int64_t> allocate_paged_slots_into(
    const at::Tensor& last_slots, const at::Tensor& free_pages, std::vector<int64_t> prefixes,
    std::vector<int64_t> lengths, int64_t page_size, at::Tensor& mapping, const at::Tensor& batch_requests);
at::Tensor release_paged_slots(const at::Tensor& slots, int64_t page_size, int64_t max_pages);
std::tuple<at::Tensor, at::Tensor> advance_decode_lengths(const at::Tensor& seq_lens, const at::Tensor& orig_seq_lens);
at::Tensor oproj(const at::Tensor& input, const at::Tensor& weight);
void oproj_push(const at::Tensor& input, const at::Tensor& weight, at::TensorList outs);
at::Tensor rank_sum(at::TensorList parts);
std::tuple<at::Tensor, at::Tensor> rank_sum_add_rms_norm(at::TensorList parts, const at::Tensor& residual,
                                                         const at::Tensor& weight, double epsilon, double weight_offset);
at::Tensor vocabulary_argmax(const at::Tensor& logits);
at::Tensor sample_from_logits(const at::Tensor& logits, const at::Tensor& temperatures, const at::Tensor& top_ps,
                              const at::Tensor& top_ks, const at::Tensor& min_ps, const c10::optional<at::Tensor>& seeds,
                              const c10::optional<at::Tensor>& positions, bool nan_to_neg_inf);
at::Tensor& apply_token_bitmask_inplace_(at::Tensor& logits, const at::Tensor& bitmask,
                                         const c10::optional<at::Tensor>& indices, int64_t vocab_size, bool mask_tail);

}  // namespace gaudirt_b200
