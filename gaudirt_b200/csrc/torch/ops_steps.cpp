// PyTorch operators for the steps either side of the attention path: slot allocator and
// decode-length update, o_proj with its rank-ordered sum, and the kernels behind the LM head.
// Registered in ops.cpp.
#include "ops_common.h"

namespace gaudirt_b200 {

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

}  // namespace gaudirt_b200
