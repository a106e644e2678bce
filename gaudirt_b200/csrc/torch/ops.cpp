// PyTorch operator layer: the `gaudirt` operator namespace and the PagedMetadata class of the
// reference (src/bridge/generic_private_use1.cpp:430-489, src/bridge/paged_metadata.hpp), bound
// to CUDA tensors and to the C ABI of include/gaudirt_b200.h.  This layer owns validation,
// allocation and error translation; the kernels behind the ABI never allocate or synchronise.
//
// Error behaviour follows the reference: TORCH_CHECK -> RuntimeError with a "GaudiRT ..."
// message raised before any pool write; there is no fallback path.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/custom_class.h>
#include <torch/library.h>

#include <cmath>
#include <cstring>
#include <memory>
#include <mutex>
#include <random>
#include <tuple>
#include <utility>
#include <vector>

#include "gaudirt_b200.h"

namespace gaudirt_b200 {
namespace {

gk_stream_t stream_of(const c10::cuda::CUDAStream& s) { return reinterpret_cast<gk_stream_t>(s.stream()); }

void check_status(int status, const char* where) {
  if (status == GK_OK) return;
  if (status == GK_ERR_METADATA) TORCH_CHECK(false, gk_metadata_error());
  TORCH_CHECK(false, "GaudiRT: ", where, ": ", gk_status_string(status),
              status == GK_ERR_CUDA ? " (cudaError " + std::to_string(gk_last_cuda_error()) + ")" : std::string());
}

// One int32 status word per device; kernels OR gk_device_status bits into it.
at::Tensor& device_status(c10::DeviceIndex device) {
  static std::mutex mutex;
  static std::vector<at::Tensor> words(64);
  std::lock_guard<std::mutex> lock(mutex);
  TORCH_CHECK(device >= 0 && device < 64, "GaudiRT: device index out of range");
  if (!words[device].defined())
    words[device] = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(c10::Device(c10::kCUDA, device)));
  return words[device];
}

// Clears `bits` of the device status word, in stream order: for errors that were raised on the host.
void clear_status_bits(c10::DeviceIndex device, int bits) { device_status(device).bitwise_and_(~bits); }

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
};

void release_plan(void* context) { delete static_cast<AttentionPlan*>(context); }

at::Tensor wrap_plan(std::unique_ptr<AttentionPlan> plan) {
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

const AttentionPlan& plan_of(const at::Tensor& tensor) {
  TORCH_CHECK(tensor.defined() && tensor.is_cuda(), "GaudiRT attention: expected a device metadata plan");
  const auto* plan = tensor.storage().data_ptr().cast_context<AttentionPlan>(&release_plan);
  TORCH_CHECK(plan && tensor.data_ptr() == plan->address && tensor.device().index() == plan->device,
              "GaudiRT attention: invalid or expired metadata plan");
  return *plan;
}

std::vector<int32_t> host_i32(const at::Tensor& t) {
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

}  // namespace

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
    if (!scheduler_owned) {
      const auto host = verdict.cpu();   // 24 bytes: the only read-back of the step
      const uint64_t first = static_cast<uint64_t>(host.data_ptr<int64_t>()[0]);
      const uint64_t token = static_cast<uint64_t>(host.data_ptr<int64_t>()[1]);
      // Largest page the visible table ranges are contiguous in: the kernels then walk one table
      // entry per page and the prefill kernel may fetch whole pages by TMA.
      const uint64_t page = static_cast<uint64_t>(host.data_ptr<int64_t>()[2]);
      page_tokens_ = static_cast<int64_t>(std::min<uint64_t>(page, 128));
      if (first != UINT64_MAX || token != UINT64_MAX) clear_status_bits(device.index(), GK_DEV_BAD_METADATA);
      TORCH_CHECK(first == UINT64_MAX, "GaudiRT device metadata: invalid scheduler metadata at row ", first >> 8,
                  ", code ", first & 255);
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
    // Multi-row sequences go to the tensor-core prefill kernel (head_dim 128 only), the rest --
    // decode rows and very short chunks -- to the split-KV decode kernel.
    int64_t n_prefill = 0, n_rest = n_seq;
    std::vector<int32_t> rest(sequences_);
    const bool tensor_core = head_dim == 128 && prefill_min_rows_ >= 0;
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
    // when only a few blocks are split: it saves a launch whose grid would be tiny.  With many split
    // blocks the merges are better spread over the whole GPU by the separate combine kernel
    // (measured: 2-5 % faster fused at 4-23 split blocks, 2-9 % slower at 64-256).
    const bool fuse = fused_combine_ > 0 || (fused_combine_ < 0 && n_combine * 4 <= sm_count);
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
  void set_fused_combine(int64_t mode) {
    TORCH_CHECK(mode >= -1 && mode <= 1, "GaudiRT attention: invalid combine mode");
    fused_combine_ = static_cast<int>(mode);
  }
  int split_tokens_ = 0, prefill_min_rows_ = 0, fused_combine_ = -1;
  at::Tensor locations_, requests_, positions_, mapping_, header_, batch_requests_, token_ids_, last_token_indices_;
  std::vector<int32_t> sequences_;   // {first_row, n_rows, first_position, table_row} per sequence
  std::vector<std::pair<int64_t, at::Tensor>> plans_;
};

// ---------------------------------------------------------------------------------------------
// operators
// ---------------------------------------------------------------------------------------------
at::Tensor allocate_paged_kv(int64_t layers, int64_t slots, int64_t heads, int64_t head_dim) {
  uint64_t bytes = 0;
  TORCH_CHECK(gk_paged_kv_pool_bytes(layers, slots, heads, head_dim, &bytes) == GK_OK,
              "GaudiRT: unsupported head-major KV pool geometry");
  return at::zeros({layers, 2, heads, slots, head_dim},
                   at::TensorOptions().dtype(at::kBFloat16).device(c10::Device(c10::kCUDA, at::cuda::current_device())));
}

int64_t paged_attn_kv_tile(int64_t) { return GK_REFERENCE_KV_TILE; }

// Shared body of the attention operators.  With `pushed` empty the result is a fresh tensor;
// otherwise every tensor of `pushed` (one per tensor-parallel rank, peer-mapped, same shape and
// strides) receives the rows and nothing is returned.
at::Tensor paged_attn_impl(const at::Tensor& query, const at::Tensor& key, const at::Tensor& value,
                           at::Tensor& key_pool, at::Tensor& value_pool, const at::Tensor& locations,
                           const at::Tensor& plan_tensor, int64_t head_dim, double scale, double softcap,
                           int64_t sliding_window, const std::vector<at::Tensor>& pushed) {
  const auto& plan = plan_of(plan_tensor);
  const auto device = plan_tensor.device();
  c10::cuda::CUDAGuard guard(device);
  const auto stream = at::cuda::getCurrentCUDAStream(device.index());
  const float scale_f = static_cast<float>(scale), softcap_f = static_cast<float>(softcap);
  TORCH_CHECK(plan.stream == stream.stream() && std::isfinite(scale) && std::isfinite(scale_f) && scale_f > 0 &&
                  std::isfinite(softcap) && std::isfinite(softcap_f) && softcap_f >= 0.0f &&
                  (sliding_window == -1 || (sliding_window > 0 && sliding_window <= INT32_MAX)) &&
                  head_dim == plan.head_dim,
              "GaudiRT attention: invalid scale, stream, or head dimension");
  TORCH_CHECK(plan.sliding_window == sliding_window, "GaudiRT attention: plan sliding_window mismatch");
  for (const auto& input : {query, key, value})
    TORCH_CHECK(input.is_cuda() && input.device() == device && input.scalar_type() == at::kBFloat16 &&
                    input.dim() == 2 && input.size(0) == plan.rows,
                "GaudiRT attention: Q/K/V must be BF16 device matrices with matching rows");
  TORCH_CHECK(query.size(1) == plan.query_heads * head_dim && key.size(1) == plan.kv_heads * head_dim &&
                  value.size(1) == key.size(1) && locations.dim() == 1 && locations.numel() == plan.rows &&
                  locations.scalar_type() == at::kInt && locations.device() == device && locations.is_contiguous(),
              "GaudiRT attention: Q/K/V or slot dimensions do not match metadata");
  for (const auto& pool : {key_pool, value_pool})
    TORCH_CHECK(pool.is_cuda() && pool.device() == device && pool.scalar_type() == at::kBFloat16 && pool.dim() == 3 &&
                    pool.size(0) == plan.slots && pool.size(1) == plan.kv_heads && pool.size(2) == head_dim &&
                    pool.stride(0) == head_dim && pool.stride(1) == plan.slots * head_dim && pool.stride(2) == 1,
                "GaudiRT attention: head-major combined KV pool is required");
  const auto key_address = reinterpret_cast<uintptr_t>(key_pool.data_ptr());
  const auto value_address = reinterpret_cast<uintptr_t>(value_pool.data_ptr());
  const uint64_t half_bytes = static_cast<uint64_t>(plan.slots) * plan.kv_heads * head_dim * sizeof(uint16_t);
  TORCH_CHECK(key_pool.storage().unsafeGetStorageImpl() == value_pool.storage().unsafeGetStorageImpl() &&
                  value_address == key_address + half_bytes && key_address % 16 == 0,
              "GaudiRT attention: KV pool descriptor is not backed by combined storage");
  // Row-strided column slices are read in place; anything else is packed first.
  const at::Tensor q = query.stride(1) == 1 ? query : query.contiguous();
  const at::Tensor k = key.stride(1) == 1 ? key : key.contiguous();
  const at::Tensor v = value.stride(1) == 1 ? value : value.contiguous();
  at::Tensor output;
  std::vector<void*> outs;
  int64_t out_stride = query.size(1);
  if (pushed.empty()) {
    output = at::empty({plan.rows, query.size(1)}, query.options().memory_format(at::MemoryFormat::Contiguous));
    outs.push_back(output.data_ptr());
  } else {
    TORCH_CHECK(pushed.size() <= GK_MAX_OUTPUTS, "GaudiRT attention: too many gather destinations");
    out_stride = pushed.front().stride(0);
    for (const auto& t : pushed) {
      TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 2 && t.size(0) == plan.rows &&
                      t.size(1) == query.size(1) && t.stride(1) == 1 && t.stride(0) == out_stride,
                  "GaudiRT attention: gather destinations must be BF16 [rows, q_width] column blocks of equal stride");
      outs.push_back(t.data_ptr());
    }
  }
  int32_t* status = device_status(device.index()).data_ptr<int32_t>();
  const gk_stream_t s = stream_of(stream);
  check_status(gk_kv_store_head_major_bf16(k.data_ptr(), v.data_ptr(), k.stride(0), v.stride(0),
                                           locations.data_ptr<int32_t>(), plan.rows, key_pool.data_ptr(),
                                           value_pool.data_ptr(), plan.slots, (int)plan.kv_heads, (int)head_dim, status, s),
               "KV store");
  const int32_t* words = plan.buffer.data_ptr<int32_t>();
  check_status(gk_paged_attn_multi_bf16(q.data_ptr(), q.stride(0), key_pool.data_ptr(), value_pool.data_ptr(), plan.slots,
                                        plan.table.data_ptr<int32_t>(), plan.table_stride, plan.entry_stride,
                                        plan.page_tokens,
                                        plan.table_rows.defined() ? plan.table_rows.data_ptr<int32_t>() : nullptr, words,
                                        plan.n_work, outs.data(), (int)outs.size(), out_stride,
                                        plan.part_ml.data_ptr<float>(), plan.part_o.data_ptr<float>(),
                                        plan.counters.defined() ? plan.counters.data_ptr<int32_t>() : nullptr, scale_f,
                                        softcap_f, (int)sliding_window, (int)plan.query_heads, (int)plan.kv_heads,
                                        (int)head_dim, status, s),
               "paged attention");
  if (!plan.counters.defined())     // otherwise the combine ran inside: the last split to finish merged its block
    check_status(gk_paged_attn_combine_multi_bf16(plan.part_ml.data_ptr<float>(), plan.part_o.data_ptr<float>(),
                                                  words + plan.combine_offset, plan.n_combine, outs.data(),
                                                  (int)outs.size(), out_stride, (int)plan.query_heads, (int)head_dim, s),
                 "split-KV combine");
  if (plan.n_prefill > 0) {
    // Query tiles of multi-row sequences: tcgen05 kernel, one destination.  With several gather
    // destinations the rows are staged once and copied to each of them.
    at::Tensor staged = pushed.empty() ? output : at::empty({plan.rows, query.size(1)}, query.options());
    check_status(gk_paged_prefill_tc_bf16(q.data_ptr(), q.stride(0), key_pool.data_ptr(), value_pool.data_ptr(), plan.slots,
                                          plan.table.data_ptr<int32_t>(), plan.table_stride, plan.entry_stride,
                                          plan.page_tokens,
                                          plan.table_rows.defined() ? plan.table_rows.data_ptr<int32_t>() : nullptr,
                                          words + plan.prefill_offset, plan.n_prefill, staged.data_ptr(), staged.stride(0),
                                          scale_f, softcap_f, (int)sliding_window, (int)plan.query_heads,
                                          (int)plan.kv_heads, (int)head_dim, status, s),
                 "tensor-core prefill");
    if (!pushed.empty()) {
      TORCH_CHECK(plan.n_work == 0, "GaudiRT attention: mixed prefill and decode rows are not supported with gather destinations");
      for (const auto& t : pushed) const_cast<at::Tensor&>(t).copy_(staged, /*non_blocking=*/true);
    }
  }
  return output;
}

at::Tensor paged_attn_validated(const at::Tensor& query, const at::Tensor& key, const at::Tensor& value,
                                at::Tensor& key_pool, at::Tensor& value_pool, const at::Tensor& locations,
                                const at::Tensor& /*requests*/, const at::Tensor& /*positions*/,
                                const at::Tensor& plan_tensor, const at::Tensor& /*header*/, int64_t head_dim,
                                double scale, double softcap, int64_t sliding_window) {
  return paged_attn_impl(query, key, value, key_pool, value_pool, locations, plan_tensor, head_dim, scale, softcap,
                         sliding_window, {});
}

// Attention whose epilogue is the tensor-parallel output gather: the rows are stored into every
// tensor of `outputs` (this rank's column block of each rank's gathered activation).  Not in the
// reference, which gathers with a separate collective (src/bridge/segmented_runner.cpp:170-191).
void paged_attn_push(const at::Tensor& query, const at::Tensor& key, const at::Tensor& value, at::Tensor& key_pool,
                     at::Tensor& value_pool, const at::Tensor& locations, const at::Tensor& plan_tensor,
                     at::TensorList outputs, int64_t head_dim, double scale, double softcap, int64_t sliding_window) {
  TORCH_CHECK(!outputs.empty(), "GaudiRT attention: gather destinations are required");
  paged_attn_impl(query, key, value, key_pool, value_pool, locations, plan_tensor, head_dim, scale, softcap,
                  sliding_window, outputs.vec());
}

// Completion barrier after the pushes: flags[p] aliases rank p's int32[world] flag array.
void peer_barrier(at::TensorList flags, int64_t rank, int64_t epoch, int64_t max_cycles) {
  TORCH_CHECK(!flags.empty() && flags.size() <= GK_MAX_OUTPUTS && rank >= 0 && rank < (int64_t)flags.size(),
              "GaudiRT: invalid peer barrier arguments");
  std::vector<int32_t*> ptrs;
  for (const auto& f : flags) {
    TORCH_CHECK(f.is_cuda() && f.scalar_type() == at::kInt && f.is_contiguous() && f.numel() >= (int64_t)flags.size(),
                "GaudiRT: peer barrier flags must be int32 device arrays of at least world entries");
    ptrs.push_back(f.data_ptr<int32_t>());
  }
  const auto device = flags[rank].device();
  c10::cuda::CUDAGuard guard(device);
  check_status(gk_peer_barrier(ptrs.data(), (int)rank, (int)flags.size(), (int32_t)epoch, max_cycles,
                               device_status(device.index()).data_ptr<int32_t>(),
                               stream_of(at::cuda::getCurrentCUDAStream(device.index()))),
               "peer barrier");
}

// The barrier with its epoch in device memory (`counter`, int32[1] on this rank): graph-replayable.
void peer_barrier_counted(at::TensorList flags, int64_t rank, at::Tensor& counter, int64_t max_cycles) {
  TORCH_CHECK(!flags.empty() && flags.size() <= GK_MAX_OUTPUTS && rank >= 0 && rank < (int64_t)flags.size(),
              "GaudiRT: invalid peer barrier arguments");
  std::vector<int32_t*> ptrs;
  for (const auto& f : flags) {
    TORCH_CHECK(f.is_cuda() && f.scalar_type() == at::kInt && f.is_contiguous() && f.numel() >= (int64_t)flags.size(),
                "GaudiRT: peer barrier flags must be int32 device arrays of at least world entries");
    ptrs.push_back(f.data_ptr<int32_t>());
  }
  const auto device = flags[rank].device();
  TORCH_CHECK(counter.is_cuda() && counter.device() == device && counter.scalar_type() == at::kInt && counter.numel() == 1,
              "GaudiRT: the barrier epoch counter must be one int32 on this rank's device");
  c10::cuda::CUDAGuard guard(device);
  check_status(gk_peer_barrier_counted(ptrs.data(), (int)rank, (int)flags.size(), counter.data_ptr<int32_t>(), max_cycles,
                                       device_status(device.index()).data_ptr<int32_t>(),
                                       stream_of(at::cuda::getCurrentCUDAStream(device.index()))),
               "peer barrier");
}

at::Tensor paged_attn(const at::Tensor& query, const at::Tensor& key, const at::Tensor& value, at::Tensor& key_pool,
                      at::Tensor& value_pool, const c10::intrusive_ptr<PagedMetadata>& metadata, int64_t head_dim,
                      double scale, double softcap, int64_t sliding_window) {
  TORCH_CHECK(metadata, "GaudiRT paged attention: metadata is required");
  TORCH_CHECK(query.dim() == 2 && key_pool.dim() == 3 && (head_dim == 64 || head_dim == 128 || head_dim == 256),
              "GaudiRT paged attention: invalid tensor ranks or head dimension");
  const auto q_heads = query.size(1) / head_dim;
  const auto kv_heads = key_pool.size(1);
  auto plan = sliding_window > 0 ? metadata->attention_plan_for(q_heads, kv_heads, head_dim, sliding_window)
                                 : metadata->attention_plan(q_heads, kv_heads, head_dim);
  return paged_attn_validated(query, key, value, key_pool, value_pool, metadata->row_locations(),
                              metadata->row_requests(), metadata->rotary_positions(), plan, metadata->rotary_header(),
                              head_dim, scale, softcap, sliding_window);
}

// ---------------------------------------------------------------------------------------------
// front of a decode layer
// ---------------------------------------------------------------------------------------------
namespace {
void check_norm_inputs(const at::Tensor& input, const at::Tensor* residual, const at::Tensor& weight, double epsilon,
                       double weight_offset, const char* what) {
  const float eps = static_cast<float>(epsilon), offset = static_cast<float>(weight_offset);
  TORCH_CHECK(std::isfinite(epsilon) && std::isfinite(eps) && eps > 0 && std::isfinite(weight_offset) &&
                  std::isfinite(offset),
              "GaudiRT: ", what, " epsilon must be positive finite and weight_offset finite");
  TORCH_CHECK(input.is_cuda() && weight.device() == input.device() && input.scalar_type() == at::kBFloat16 &&
                  weight.scalar_type() == at::kBFloat16 &&
                  (!residual || (residual->device() == input.device() && residual->scalar_type() == at::kBFloat16)),
              "GaudiRT: ", what, " requires same-device CUDA BF16 tensors");
  TORCH_CHECK(input.dim() >= 2 && input.dim() <= 5 && weight.dim() == 1 && weight.size(0) == input.size(-1) &&
                  input.size(-1) <= 8192 && (!residual || residual->sizes() == input.sizes()),
              "GaudiRT: invalid ", what, " tensor geometry");
}

// [.., hidden] -> 2-D [rows, hidden] with unit inner stride (a view when possible).
at::Tensor as_rows(const at::Tensor& t) {
  const auto hidden = t.size(-1);
  if (t.dim() == 2 && t.stride(1) == 1) return t;
  return t.contiguous().view({-1, hidden});
}
}  // namespace

at::Tensor rms_norm(const at::Tensor& input, const at::Tensor& weight, double epsilon, double weight_offset) {
  check_norm_inputs(input, nullptr, weight, epsilon, weight_offset, "RMSNorm");
  auto out = at::empty(input.sizes(), input.options().memory_format(at::MemoryFormat::Contiguous));
  if (!input.numel()) return out;
  c10::cuda::CUDAGuard guard(input.device());
  const auto x = as_rows(input);
  const auto w = weight.contiguous();
  check_status(gk_rms_norm_bf16(x.data_ptr(), w.data_ptr(), (float)epsilon, (float)weight_offset, x.size(0), x.size(1),
                                x.stride(0), out.data_ptr(), stream_of(at::cuda::getCurrentCUDAStream())),
               "RMSNorm");
  return out;
}

std::tuple<at::Tensor, at::Tensor> fused_add_rms_norm(const at::Tensor& input, const at::Tensor& residual,
                                                      const at::Tensor& weight, double epsilon, double weight_offset) {
  check_norm_inputs(input, &residual, weight, epsilon, weight_offset, "fused RMSNorm");
  auto norm = at::empty(input.sizes(), input.options().memory_format(at::MemoryFormat::Contiguous));
  auto updated = at::empty(residual.sizes(), residual.options().memory_format(at::MemoryFormat::Contiguous));
  if (!input.numel()) return {norm, updated};
  c10::cuda::CUDAGuard guard(input.device());
  const auto x = as_rows(input), r = as_rows(residual);
  const auto w = weight.contiguous();
  check_status(gk_fused_add_rms_norm_bf16(x.data_ptr(), r.data_ptr(), w.data_ptr(), (float)epsilon, (float)weight_offset,
                                          x.size(0), x.size(1), x.stride(0), r.stride(0), norm.data_ptr(),
                                          updated.data_ptr(), stream_of(at::cuda::getCurrentCUDAStream())),
               "fused RMSNorm");
  return {norm, updated};
}

std::tuple<at::Tensor, at::Tensor> rotary_embedding_validated(const at::Tensor& query, const at::Tensor& key,
                                                              const at::Tensor& cache, const at::Tensor& positions,
                                                              const at::Tensor& header, int64_t context, int64_t head_dim,
                                                              int64_t rotary_dim, bool is_neox) {
  TORCH_CHECK(head_dim > 0 && head_dim <= INT32_MAX && rotary_dim > 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0,
              "GaudiRT rotary: invalid head or rotary dimension");
  for (const auto& t : {query, key, cache})
    TORCH_CHECK(t.is_cuda() && t.device() == query.device() && t.scalar_type() == at::kBFloat16,
                "GaudiRT rotary: expected CUDA BF16 tensors");
  TORCH_CHECK(query.dim() == 2 && key.dim() == 2 && query.size(0) > 0 && key.size(0) == query.size(0) &&
                  query.size(1) > 0 && key.size(1) > 0 && query.size(1) % head_dim == 0 && key.size(1) % head_dim == 0,
              "GaudiRT rotary: invalid query or key geometry");
  TORCH_CHECK(cache.dim() == 2 && context > 0 && cache.size(0) >= context && cache.size(0) <= INT32_MAX &&
                  cache.size(1) == rotary_dim,
              "GaudiRT rotary: cache does not cover validated positions");
  const auto rows = query.size(0);
  TORCH_CHECK(positions.device() == query.device() && positions.scalar_type() == at::kInt && positions.dim() == 1 &&
                  positions.size(0) == rows && positions.is_contiguous() &&
                  (!header.defined() || (header.device() == query.device() && header.scalar_type() == at::kInt)),
              "GaudiRT rotary: invalid validated metadata tensors");
  c10::cuda::CUDAGuard guard(query.device());
  const at::Tensor q = query.stride(1) == 1 ? query : query.contiguous();
  const at::Tensor k = key.stride(1) == 1 ? key : key.contiguous();
  const at::Tensor table = cache.contiguous();
  auto q_out = at::empty({rows, query.size(1)}, query.options().memory_format(at::MemoryFormat::Contiguous));
  auto k_out = at::empty({rows, key.size(1)}, key.options().memory_format(at::MemoryFormat::Contiguous));
  check_status(gk_rotary_bf16(q.data_ptr(), k.data_ptr(), q.stride(0), k.stride(0), table.data_ptr(), table.size(0),
                              positions.data_ptr<int32_t>(), rows, query.size(1), key.size(1), (int)head_dim,
                              (int)rotary_dim, is_neox ? 1 : 0, q_out.data_ptr(), k_out.data_ptr(),
                              device_status(query.device().index()).data_ptr<int32_t>(),
                              stream_of(at::cuda::getCurrentCUDAStream())),
               "rotary");
  return {q_out, k_out};
}

std::tuple<at::Tensor, at::Tensor> rotary_embedding(const at::Tensor& query, const at::Tensor& key, const at::Tensor& cache,
                                                    const c10::intrusive_ptr<PagedMetadata>& metadata, int64_t head_dim,
                                                    int64_t rotary_dim, bool is_neox) {
  TORCH_CHECK(metadata, "GaudiRT rotary: metadata is required");
  return rotary_embedding_validated(query, key, cache, metadata->rotary_positions(), metadata->rotary_header(),
                                    metadata->context(), head_dim, rotary_dim, is_neox);
}

// Positions come from a device tensor: the range check happens in the kernel (status word).
std::tuple<at::Tensor, at::Tensor> rotary_embedding_positions(const at::Tensor& query, const at::Tensor& key,
                                                              const at::Tensor& cache, const at::Tensor& positions,
                                                              int64_t head_dim, int64_t rotary_dim, bool is_neox) {
  TORCH_CHECK(positions.is_cuda() && positions.dim() == 1 &&
                  (positions.scalar_type() == at::kInt || positions.scalar_type() == at::kLong),
              "GaudiRT rotary: invalid validated metadata tensors");
  return rotary_embedding_validated(query, key, cache, positions.to(at::kInt).contiguous(), at::Tensor(),
                                    cache.dim() == 2 ? cache.size(0) : 0, head_dim, rotary_dim, is_neox);
}

// ---------------------------------------------------------------------------------------------
// slot allocator and decode-length update (src/bridge/paged_slot_allocator.cpp,
// src/bridge/eager_scheduler.cpp)
// ---------------------------------------------------------------------------------------------
void require_indices(const at::Tensor& tensor) {
  TORCH_CHECK(tensor.is_cuda() && tensor.scalar_type() == at::kLong && tensor.dim() == 1 && tensor.is_contiguous(),
              "GaudiRT paged allocator: expected contiguous device int64 indices");
}

std::tuple<at::Tensor, int64_t> allocate_paged_slots(const at::Tensor& last_slots, const at::Tensor& free_pages,
                                                     std::vector<int64_t> prefixes, std::vector<int64_t> lengths,
                                                     int64_t page_size) {
  require_indices(last_slots);
  require_indices(free_pages);
  TORCH_CHECK(!prefixes.empty() && prefixes.size() == lengths.size() &&
                  last_slots.numel() == static_cast<int64_t>(prefixes.size()) && last_slots.device() == free_pages.device(),
              "GaudiRT paged allocator: unsupported page size or request count");
  const int64_t n = static_cast<int64_t>(prefixes.size());
  const auto device = last_slots.device();
  c10::cuda::CUDAGuard guard(device);
  auto staging = at::empty({n * 4}, at::TensorOptions().dtype(at::kInt).pinned_memory(true));
  int64_t total = 0, pages = 0;
  check_status(gk_paged_slots_layout(prefixes.data(), lengths.data(), n, page_size, free_pages.numel(),
                                     staging.data_ptr<int32_t>(), &total, &pages),
               "paged allocator");
  auto records = staging.to(device, /*non_blocking=*/true);
  auto result = at::empty({total}, last_slots.options());
  const auto stream = at::cuda::getCurrentCUDAStream(device.index());
  check_status(gk_paged_slots_allocate(last_slots.data_ptr<int64_t>(), free_pages.data_ptr<int64_t>(),
                                       records.data_ptr<int32_t>(), n, total, page_size, result.data_ptr<int64_t>(),
                                       nullptr, 0, 0, 0, nullptr, nullptr, nullptr, stream_of(stream)),
               "paged allocator");
  return {result, pages};
}

// Allocation fused with the two scatters a scheduler does next: the int32 slot list for the KV
// store and the request-to-token table rows the attention kernel walks.  Not part of the
// reference surface.
std::tuple<at::Tensor, at::Tensor, int64_t> allocate_paged_slots_into(
    const at::Tensor& last_slots, const at::Tensor& free_pages, std::vector<int64_t> prefixes,
    std::vector<int64_t> lengths, int64_t page_size, at::Tensor& mapping, const at::Tensor& batch_requests) {
  require_indices(last_slots);
  require_indices(free_pages);
  TORCH_CHECK(!prefixes.empty() && prefixes.size() == lengths.size() &&
                  last_slots.numel() == static_cast<int64_t>(prefixes.size()) && last_slots.device() == free_pages.device(),
              "GaudiRT paged allocator: unsupported page size or request count");
  const int64_t n = static_cast<int64_t>(prefixes.size());
  const auto device = last_slots.device();
  TORCH_CHECK(mapping.is_cuda() && mapping.device() == device && mapping.scalar_type() == at::kInt && mapping.dim() == 2 &&
                  mapping.stride(1) == 1 && batch_requests.is_cuda() && batch_requests.device() == device &&
                  batch_requests.scalar_type() == at::kInt && batch_requests.dim() == 1 && batch_requests.numel() == n &&
                  batch_requests.is_contiguous(),
              "GaudiRT paged allocator: expected an int32 request map and int32 request ids on the same device");
  for (int64_t i = 0; i < n; ++i)
    TORCH_CHECK(prefixes[i] >= 0 && lengths[i] >= 0 && prefixes[i] + lengths[i] <= mapping.size(1),
                "GaudiRT paged allocator: invalid request lengths");
  c10::cuda::CUDAGuard guard(device);
  auto staging = at::empty({n * 4}, at::TensorOptions().dtype(at::kInt).pinned_memory(true));
  int64_t total = 0, pages = 0;
  check_status(gk_paged_slots_layout(prefixes.data(), lengths.data(), n, page_size, free_pages.numel(),
                                     staging.data_ptr<int32_t>(), &total, &pages),
               "paged allocator");
  auto records = staging.to(device, /*non_blocking=*/true);
  auto result = at::empty({total}, last_slots.options());
  auto locations = at::empty({total}, batch_requests.options());
  const auto stream = at::cuda::getCurrentCUDAStream(device.index());
  check_status(gk_paged_slots_allocate(last_slots.data_ptr<int64_t>(), free_pages.data_ptr<int64_t>(),
                                       records.data_ptr<int32_t>(), n, total, page_size, result.data_ptr<int64_t>(),
                                       mapping.data_ptr<int32_t>(), mapping.size(0), mapping.stride(0), mapping.size(1),
                                       batch_requests.data_ptr<int32_t>(), locations.data_ptr<int32_t>(),
                                       device_status(device.index()).data_ptr<int32_t>(), stream_of(stream)),
               "paged allocator");
  return {result, locations, pages};
}

at::Tensor release_paged_slots(const at::Tensor& slots, int64_t page_size, int64_t max_pages) {
  require_indices(slots);
  TORCH_CHECK(page_size >= 1 && page_size <= INT32_MAX && max_pages > 0 && max_pages <= INT32_MAX && slots.numel() > 0 &&
                  slots.numel() <= (int64_t{1} << 30),
              "GaudiRT paged allocator: invalid release geometry");
  const auto device = slots.device();
  c10::cuda::CUDAGuard guard(device);
  uint64_t bytes = 0;
  check_status(gk_paged_slots_release_workspace_bytes(slots.numel(), max_pages, &bytes), "paged allocator");
  auto workspace = at::empty({static_cast<int64_t>(bytes)}, at::TensorOptions().dtype(at::kByte).device(device));
  auto result = at::empty_like(slots);
  auto count = at::empty({2}, at::TensorOptions().dtype(at::kInt).device(device));
  const auto stream = at::cuda::getCurrentCUDAStream(device.index());
  check_status(gk_paged_slots_release(slots.data_ptr<int64_t>(), slots.numel(), page_size, max_pages,
                                      workspace.data_ptr(), result.data_ptr<int64_t>(), count.data_ptr<int32_t>(),
                                      stream_of(stream)),
               "paged allocator");
  const auto host = count.cpu();   // the result's length is data dependent: one 8-byte read-back
  const int32_t released = host.data_ptr<int32_t>()[0], outside = host.data_ptr<int32_t>()[1];
  TORCH_CHECK(outside == 0 && released > 0 && released <= slots.numel(),
              "GaudiRT paged allocator: released slot is outside the KV pool");
  return result.narrow(0, 0, released);
}

std::tuple<at::Tensor, at::Tensor> advance_decode_lengths(const at::Tensor& seq_lens, const at::Tensor& orig_seq_lens) {
  TORCH_CHECK(seq_lens.is_cuda() && orig_seq_lens.device() == seq_lens.device() && seq_lens.scalar_type() == at::kLong &&
                  orig_seq_lens.scalar_type() == at::kInt && seq_lens.dim() == 1 &&
                  orig_seq_lens.sizes() == seq_lens.sizes() && seq_lens.numel() <= (int64_t{1} << 30) &&
                  seq_lens.is_contiguous() && orig_seq_lens.is_contiguous(),
              "GaudiRT decode lengths: expected matching contiguous int64 and int32 vectors");
  auto next = at::empty_like(seq_lens), orig_next = at::empty_like(orig_seq_lens);
  if (!seq_lens.numel()) return {next, orig_next};
  c10::cuda::CUDAGuard guard(seq_lens.device());
  const auto stream = at::cuda::getCurrentCUDAStream(seq_lens.device().index());
  check_status(gk_advance_decode_lengths(seq_lens.data_ptr<int64_t>(), orig_seq_lens.data_ptr<int32_t>(),
                                         seq_lens.numel(), next.data_ptr<int64_t>(), orig_next.data_ptr<int32_t>(),
                                         stream_of(stream)),
               "decode lengths");
  return {next, orig_next};
}

// ---------------------------------------------------------------------------------------------
// o_proj and its rank-ordered sum (the chain O-Proj -> AllReduce -> AddRMSNorm of the
// reference's tensor-parallel decoder; src/bridge/communicator.cpp:373-417)
// ---------------------------------------------------------------------------------------------
void oproj_into(const at::Tensor& input, const at::Tensor& weight, const std::vector<at::Tensor>& outs) {
  TORCH_CHECK(input.is_cuda() && weight.device() == input.device() && input.scalar_type() == at::kBFloat16 &&
                  weight.scalar_type() == at::kBFloat16 && input.dim() == 2 && weight.dim() == 2 &&
                  input.size(1) == weight.size(1) && input.stride(1) == 1 && weight.stride(1) == 1,
              "GaudiRT o_proj: expected BF16 device matrices input [rows, k] and weight [n, k]");
  TORCH_CHECK(!outs.empty() && outs.size() <= GK_MAX_OUTPUTS, "GaudiRT o_proj: invalid destination count");
  std::vector<void*> ptrs;
  for (const auto& t : outs) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 2 && t.size(0) == input.size(0) &&
                    t.size(1) == weight.size(0) && t.stride(1) == 1 && t.stride(0) == outs.front().stride(0),
                "GaudiRT o_proj: destinations must be BF16 [rows, n] blocks of equal stride");
    ptrs.push_back(t.data_ptr());
  }
  const auto device = input.device();
  c10::cuda::CUDAGuard guard(device);
  check_status(gk_oproj_bf16(input.data_ptr(), input.stride(0), weight.data_ptr(), weight.stride(0), input.size(0),
                             weight.size(0), input.size(1), ptrs.data(), (int)ptrs.size(), outs.front().stride(0),
                             device_status(device.index()).data_ptr<int32_t>(),
                             stream_of(at::cuda::getCurrentCUDAStream(device.index()))),
               "o_proj");
}

at::Tensor oproj(const at::Tensor& input, const at::Tensor& weight) {
  TORCH_CHECK(input.dim() == 2 && weight.dim() == 2, "GaudiRT o_proj: expected matrices");
  auto out = at::empty({input.size(0), weight.size(0)}, input.options().memory_format(at::MemoryFormat::Contiguous));
  oproj_into(input, weight, {out});
  return out;
}

void oproj_push(const at::Tensor& input, const at::Tensor& weight, at::TensorList outs) {
  oproj_into(input, weight, std::vector<at::Tensor>(outs.begin(), outs.end()));
}

std::vector<const void*> part_pointers(at::TensorList parts) {
  TORCH_CHECK(!parts.empty() && parts.size() <= GK_MAX_OUTPUTS, "GaudiRT rank sum: invalid rank count");
  std::vector<const void*> ptrs;
  for (const auto& t : parts) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.sizes() == parts.front().sizes() &&
                    t.strides() == parts.front().strides() && t.device() == parts.front().device(),
                "GaudiRT rank sum: partials must be BF16 device tensors of one shape and layout");
    ptrs.push_back(t.data_ptr());
  }
  return ptrs;
}

at::Tensor rank_sum(at::TensorList parts) {
  const auto ptrs = part_pointers(parts);
  TORCH_CHECK(parts.front().is_contiguous(), "GaudiRT rank sum: partials must be contiguous");
  auto out = at::empty_like(parts.front());
  const auto device = out.device();
  c10::cuda::CUDAGuard guard(device);
  check_status(gk_rank_sum_bf16(ptrs.data(), (int)ptrs.size(), out.numel(), out.data_ptr(),
                                stream_of(at::cuda::getCurrentCUDAStream(device.index()))),
               "rank sum");
  return out;
}

std::tuple<at::Tensor, at::Tensor> rank_sum_add_rms_norm(at::TensorList parts, const at::Tensor& residual,
                                                         const at::Tensor& weight, double epsilon, double weight_offset) {
  const auto ptrs = part_pointers(parts);
  const auto& first = parts.front();
  TORCH_CHECK(first.dim() == 2 && first.stride(1) == 1 && residual.is_cuda() && residual.device() == first.device() &&
                  residual.scalar_type() == at::kBFloat16 && residual.sizes() == first.sizes() && residual.stride(1) == 1 &&
                  weight.device() == first.device() && weight.scalar_type() == at::kBFloat16 && weight.dim() == 1 &&
                  weight.size(0) == first.size(1) && weight.is_contiguous() && std::isfinite(epsilon) && epsilon > 0,
              "GaudiRT rank sum: expected BF16 [rows, hidden] partials and residual, [hidden] weight");
  auto y = at::empty(first.sizes(), first.options().memory_format(at::MemoryFormat::Contiguous));
  auto u = at::empty_like(y);
  const auto device = first.device();
  c10::cuda::CUDAGuard guard(device);
  check_status(gk_rank_sum_add_rms_norm_bf16(ptrs.data(), (int)ptrs.size(), first.stride(0), residual.data_ptr(),
                                             weight.data_ptr(), (float)epsilon, (float)weight_offset, first.size(0),
                                             first.size(1), residual.stride(0), y.data_ptr(), u.data_ptr(),
                                             stream_of(at::cuda::getCurrentCUDAStream(device.index()))),
               "rank sum + norm");
  return {y, u};
}

// ---------------------------------------------------------------------------------------------
// after the LM head: argmax, grammar bitmask, sampling (src/bridge/sampler_vocab.cpp:333-485)
// ---------------------------------------------------------------------------------------------
void require_logits(const at::Tensor& logits, const char* what) {
  TORCH_CHECK(logits.defined() && logits.is_cuda() && logits.dim() == 2 && logits.stride(1) == 1 &&
                  (logits.scalar_type() == at::kBFloat16 || logits.scalar_type() == at::kFloat),
              "GaudiRT ", what, ": logits must be a 2D bf16 or fp32 tensor on the active device");
}

at::Tensor vocabulary_argmax(const at::Tensor& logits) {
  require_logits(logits, "argmax");
  TORCH_CHECK(logits.size(1) > 0, "GaudiRT argmax: empty vocabulary");
  auto out = at::empty({logits.size(0)}, logits.options().dtype(at::kLong));
  const auto device = logits.device();
  c10::cuda::CUDAGuard guard(device);
  check_status(gk_vocab_argmax(logits.data_ptr(), logits.scalar_type() == at::kFloat, logits.size(0), logits.size(1),
                               logits.stride(0), out.data_ptr<int64_t>(),
                               stream_of(at::cuda::getCurrentCUDAStream(device.index()))),
               "argmax");
  return out;
}

at::Tensor batch_vector(const at::Tensor& tensor, int64_t batch, at::ScalarType dtype, const char* name,
                        const c10::Device& device) {
  TORCH_CHECK(tensor.defined(), "GaudiRT sampler: missing required ", name);
  TORCH_CHECK(tensor.scalar_type() == dtype, "GaudiRT sampler: unexpected dtype for ", name);
  at::Tensor flat;
  if (tensor.dim() == 1 && tensor.size(0) == batch) flat = tensor;
  else if (tensor.dim() == 2 && tensor.size(0) == batch && tensor.size(1) == 1) flat = tensor.reshape({batch});
  else if (tensor.numel() == 1 && tensor.dim() <= 2) flat = tensor.reshape({1}).expand({batch});
  else TORCH_CHECK(false, "GaudiRT sampler: invalid shape for ", name);
  return flat.to(device, /*non_blocking=*/true).contiguous();
}

at::Tensor sample_from_logits(const at::Tensor& logits, const at::Tensor& temperatures, const at::Tensor& top_ps,
                              const at::Tensor& top_ks, const at::Tensor& min_ps, const c10::optional<at::Tensor>& seeds,
                              const c10::optional<at::Tensor>& positions, bool nan_to_neg_inf) {
  require_logits(logits, "sampler");
  const int64_t batch = logits.size(0), vocabulary = logits.size(1);
  TORCH_CHECK(batch > 0 && batch <= (int64_t{1} << 30) && vocabulary > 0 && vocabulary <= INT32_MAX,
              "GaudiRT sampler: logits shape outside supported range");
  const auto device = logits.device();
  c10::cuda::CUDAGuard guard(device);
  const auto temperature = batch_vector(temperatures, batch, at::kFloat, "temperatures", device);
  const auto top_p = batch_vector(top_ps, batch, at::kFloat, "top_ps", device);
  const auto top_k = batch_vector(top_ks, batch, at::kInt, "top_ks", device);
  const auto min_p = batch_vector(min_ps, batch, at::kFloat, "min_ps", device);
  at::Tensor seed, position;
  const bool has_seeds = seeds.has_value() && seeds->defined();
  if (has_seeds) {
    seed = batch_vector(*seeds, batch, at::kLong, "seeds", device);
    if (positions.has_value() && positions->defined()) {
      TORCH_CHECK(positions->scalar_type() == at::kInt || positions->scalar_type() == at::kLong,
                  "GaudiRT sampler: positions must be int32 or int64");
      position = batch_vector(*positions, batch, positions->scalar_type(), "positions", device);
    }
  }
  // Unseeded calls draw a fresh base from a process-wide generator, per call.
  static std::mutex mutex;
  static std::mt19937_64 generator{std::random_device{}()};
  uint64_t base = 0;
  if (!has_seeds) {
    std::lock_guard<std::mutex> lock(mutex);
    base = generator();
  }
  auto out = at::empty({batch}, logits.options().dtype(at::kInt));
  check_status(gk_sample_vocab(logits.data_ptr(), logits.scalar_type() == at::kFloat, batch, vocabulary, logits.stride(0),
                               temperature.data_ptr<float>(), top_p.data_ptr<float>(), top_k.data_ptr<int32_t>(),
                               min_p.data_ptr<float>(), has_seeds ? seed.data_ptr<int64_t>() : nullptr,
                               position.defined() ? position.data_ptr() : nullptr,
                               position.defined() && position.scalar_type() == at::kLong, base, nan_to_neg_inf,
                               out.data_ptr<int32_t>(), stream_of(at::cuda::getCurrentCUDAStream(device.index()))),
               "sampler");
  return out;
}

at::Tensor& apply_token_bitmask_inplace_(at::Tensor& logits, const at::Tensor& bitmask,
                                         const c10::optional<at::Tensor>& indices, int64_t vocab_size, bool mask_tail) {
  TORCH_CHECK(logits.defined() && logits.is_cuda() && (logits.dim() == 1 || logits.dim() == 2) &&
                  (logits.scalar_type() == at::kBFloat16 || logits.scalar_type() == at::kFloat),
              "GaudiRT bitmask: logits must be a 1D or 2D bf16/fp32 tensor on the active device");
  TORCH_CHECK(bitmask.defined() && bitmask.scalar_type() == at::kInt && (bitmask.dim() == 1 || bitmask.dim() == 2) &&
                  (bitmask.device().is_cpu() || bitmask.device() == logits.device()),
              "GaudiRT bitmask: bitmask must be a 1D or 2D int32 tensor on CPU or active device");
  auto work = logits.dim() == 1 ? logits.unsqueeze(0) : logits;
  TORCH_CHECK(work.stride(1) == 1, "GaudiRT bitmask: logits columns must be contiguous");
  const auto device = logits.device();
  c10::cuda::CUDAGuard guard(device);
  auto mask = (bitmask.dim() == 1 ? bitmask.unsqueeze(0) : bitmask).to(device, /*non_blocking=*/true).contiguous();
  const int64_t batch = work.size(0), cols = work.size(1), mask_rows = mask.size(0), mask_words = mask.size(1);
  TORCH_CHECK(cols > 0 && cols <= INT32_MAX && mask_words > 0 && mask_words <= INT32_MAX,
              "GaudiRT bitmask: invalid tensor dimensions");
  const int64_t mask_bits = mask_words * 32;
  int64_t active = std::min(cols, mask_bits);
  if (vocab_size >= 0) {
    TORCH_CHECK(vocab_size <= cols, "GaudiRT bitmask: vocab_size exceeds logits width");
    TORCH_CHECK(mask_tail || vocab_size <= mask_bits, "GaudiRT bitmask: bitmask is smaller than vocab_size");
    active = std::min(vocab_size, mask_bits);
  }
  at::Tensor rows;
  int64_t listed = 0;
  if (indices.has_value() && indices->defined()) {
    const auto& idx = *indices;
    TORCH_CHECK(idx.dim() <= 1 && (idx.scalar_type() == at::kInt || idx.scalar_type() == at::kLong) &&
                    (idx.device().is_cpu() || idx.device() == device),
                "GaudiRT bitmask: indices must be an int32 or int64 tensor on CPU or active device");
    if (idx.numel() == 0) return logits;
    if (idx.device().is_cpu()) {                              // host indices are checked here, device ones in the kernel
      const auto host = idx.reshape({-1}).to(at::kLong);
      for (int64_t i = 0; i < host.numel(); ++i) {
        const int64_t row = host.data_ptr<int64_t>()[i];
        TORCH_CHECK(row >= 0 && row < batch && row < mask_rows, "GaudiRT bitmask: index ", row,
                    " out of bounds for logits/bitmask rows (", batch, "/", mask_rows, ")");
      }
    }
    rows = idx.reshape({-1}).to(device, /*non_blocking=*/true).to(at::kInt).contiguous();
    listed = rows.numel();
  } else {
    TORCH_CHECK(mask_rows == batch, "GaudiRT bitmask: bitmask row count (", mask_rows, ") must match logits batch (", batch,
                ")");
    if (batch == 0) return logits;
  }
  check_status(gk_apply_vocab_bitmask(work.data_ptr(), work.scalar_type() == at::kFloat, batch, cols, work.stride(0),
                                      mask.data_ptr<int32_t>(), mask_rows, mask_words,
                                      rows.defined() ? rows.data_ptr<int32_t>() : nullptr, listed, active, mask_tail,
                                      device_status(device.index()).data_ptr<int32_t>(),
                                      stream_of(at::cuda::getCurrentCUDAStream(device.index()))),
               "bitmask");
  return logits;
}

// Reads and clears the device status word of the current device (synchronises the stream).
int64_t take_device_status() {
  auto& word = device_status(at::cuda::current_device());
  const int64_t value = word.item<int32_t>();
  if (value) word.zero_();
  return value;
}

}  // namespace gaudirt_b200

TORCH_LIBRARY(gaudirt, m) {
  using gaudirt_b200::PagedMetadata;
  m.class_<PagedMetadata>("PagedMetadata")
      .def(torch::init<at::Tensor, at::Tensor, at::Tensor, at::Tensor, int64_t>())
      .def_static("from_device", &PagedMetadata::from_device)
      .def_static("from_device_with_tokens", &PagedMetadata::from_device_with_tokens)
      .def_static("_from_scheduler", &PagedMetadata::from_scheduler)
      .def_static("_from_scheduler_fused", &PagedMetadata::from_scheduler_fused)
      .def("rows", &PagedMetadata::rows)
      .def("slots", &PagedMetadata::slots)
      .def("context", &PagedMetadata::context)
      .def("page_tokens", &PagedMetadata::page_tokens)
      .def("sequences", &PagedMetadata::sequences)
      .def("forward_tensors", &PagedMetadata::forward_tensors)
      .def("rotary_positions", &PagedMetadata::rotary_positions)
      .def("rotary_header", &PagedMetadata::rotary_header)
      .def("row_locations", &PagedMetadata::row_locations)
      .def("row_requests", &PagedMetadata::row_requests)
      .def("request_mapping", &PagedMetadata::request_mapping)
      .def("attention_plan", &PagedMetadata::attention_plan)
      .def("attention_plan_for", &PagedMetadata::attention_plan_for)
      .def("last_token_indices", &PagedMetadata::last_token_indices)
      .def("token_ids", &PagedMetadata::token_ids)
      .def("vocabulary", &PagedMetadata::vocabulary)
      .def("_set_split_tokens", &PagedMetadata::set_split_tokens)
      .def("_set_prefill_min_rows", &PagedMetadata::set_prefill_min_rows)
      .def("_set_fused_combine", &PagedMetadata::set_fused_combine);
  m.def("paged_attn(Tensor query, Tensor key, Tensor value, Tensor(a!) key_pool, Tensor(b!) value_pool, "
        "__torch__.torch.classes.gaudirt.PagedMetadata metadata, int head_dim, float scale, "
        "float softcap=0.0, int sliding_window=-1) -> Tensor");
  m.def("_paged_attn_validated(Tensor query, Tensor key, Tensor value, Tensor(a!) key_pool, Tensor(b!) value_pool, "
        "Tensor locations, Tensor requests, Tensor positions, Tensor mapping, Tensor header, "
        "int head_dim, float scale, float softcap=0.0, int sliding_window=-1) -> Tensor");
  m.def("_paged_attn_push(Tensor query, Tensor key, Tensor value, Tensor(a!) key_pool, Tensor(b!) value_pool, "
        "Tensor locations, Tensor plan, Tensor(c!)[] outputs, int head_dim, float scale, float softcap=0.0, "
        "int sliding_window=-1) -> ()");
  m.def("_peer_barrier(Tensor(a!)[] flags, int rank, int epoch, int max_cycles) -> ()");
  m.def("_peer_barrier_counted(Tensor(a!)[] flags, int rank, Tensor(b!) counter, int max_cycles) -> ()");
  m.def("rms_norm(Tensor input, Tensor weight, float epsilon, float weight_offset=0.0) -> Tensor");
  m.def("fused_add_rms_norm(Tensor input, Tensor residual, Tensor weight, float epsilon, float weight_offset=0.0) -> (Tensor, Tensor)");
  m.def("rotary_embedding(Tensor query, Tensor key, Tensor cache, "
        "__torch__.torch.classes.gaudirt.PagedMetadata metadata, int head_dim, int rotary_dim, bool is_neox) "
        "-> (Tensor, Tensor)");
  m.def("rotary_embedding_positions(Tensor query, Tensor key, Tensor cache, Tensor positions, "
        "int head_dim, int rotary_dim, bool is_neox) -> (Tensor, Tensor)");
  m.def("_rotary_embedding_validated(Tensor query, Tensor key, Tensor cache, Tensor positions, "
        "Tensor header, int context, int head_dim, int rotary_dim, bool is_neox) -> (Tensor, Tensor)");
  m.def("_allocate_paged_kv(int layers, int slots, int heads, int head_dim) -> Tensor", &gaudirt_b200::allocate_paged_kv);
  m.def("_paged_attn_kv_tile(int rows) -> int", &gaudirt_b200::paged_attn_kv_tile);
  m.def("_take_device_status() -> int", &gaudirt_b200::take_device_status);
  m.def("_allocate_paged_slots", &gaudirt_b200::allocate_paged_slots);
  m.def("_allocate_paged_slots_into", &gaudirt_b200::allocate_paged_slots_into);
  m.def("_release_paged_slots", &gaudirt_b200::release_paged_slots);
  m.def("_advance_decode_lengths(Tensor seq_lens, Tensor orig_seq_lens) -> (Tensor, Tensor)");
  m.def("sample_from_logits(Tensor logits, Tensor temperatures, Tensor top_ps, Tensor top_ks, Tensor min_ps, "
        "Tensor? seeds=None, Tensor? positions=None, bool nan_to_neg_inf=True) -> Tensor");
  m.def("apply_token_bitmask_inplace_(Tensor(a!) logits, Tensor bitmask, Tensor? indices=None, "
        "int vocab_size=-1, bool mask_tail=False) -> Tensor(a!)");
  m.def("_vocabulary_argmax(Tensor logits) -> Tensor");
  m.def("_oproj(Tensor input, Tensor weight) -> Tensor");
  m.def("_oproj_push(Tensor input, Tensor weight, Tensor(a!)[] outs) -> ()");
  m.def("_rank_sum(Tensor[] parts) -> Tensor");
  m.def("_rank_sum_add_rms_norm(Tensor[] parts, Tensor residual, Tensor weight, float epsilon, "
        "float weight_offset=0.0) -> (Tensor, Tensor)");
}

TORCH_LIBRARY_IMPL(gaudirt, CUDA, m) {
  m.impl("paged_attn", TORCH_FN(gaudirt_b200::paged_attn));
  m.impl("_paged_attn_validated", TORCH_FN(gaudirt_b200::paged_attn_validated));
  m.impl("_paged_attn_push", TORCH_FN(gaudirt_b200::paged_attn_push));
  m.impl("_peer_barrier", TORCH_FN(gaudirt_b200::peer_barrier));
  m.impl("_peer_barrier_counted", TORCH_FN(gaudirt_b200::peer_barrier_counted));
  m.impl("rms_norm", TORCH_FN(gaudirt_b200::rms_norm));
  m.impl("fused_add_rms_norm", TORCH_FN(gaudirt_b200::fused_add_rms_norm));
  m.impl("rotary_embedding", TORCH_FN(gaudirt_b200::rotary_embedding));
  m.impl("rotary_embedding_positions", TORCH_FN(gaudirt_b200::rotary_embedding_positions));
  m.impl("_rotary_embedding_validated", TORCH_FN(gaudirt_b200::rotary_embedding_validated));
  m.impl("_advance_decode_lengths", TORCH_FN(gaudirt_b200::advance_decode_lengths));
  m.impl("sample_from_logits", TORCH_FN(gaudirt_b200::sample_from_logits));
  m.impl("apply_token_bitmask_inplace_", TORCH_FN(gaudirt_b200::apply_token_bitmask_inplace_));
  m.impl("_vocabulary_argmax", TORCH_FN(gaudirt_b200::vocabulary_argmax));
  m.impl("_oproj", TORCH_FN(gaudirt_b200::oproj));
  m.impl("_oproj_push", TORCH_FN(gaudirt_b200::oproj_push));
  m.impl("_rank_sum", TORCH_FN(gaudirt_b200::rank_sum));
  m.impl("_rank_sum_add_rms_norm", TORCH_FN(gaudirt_b200::rank_sum_add_rms_norm));
}
