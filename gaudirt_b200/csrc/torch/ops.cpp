// PyTorch operator layer: the `gaudirt` operator namespace and the PagedMetadata class of the
// reference (src/bridge/generic_private_use1.cpp:430-489, src/bridge/paged_metadata.hpp), bound
// to CUDA tensors and to the C ABI of include/gaudirt_b200.h.  This layer owns validation,
// allocation and error translation; the kernels behind the ABI never allocate or synchronise.
//
// Error behaviour follows the reference: TORCH_CHECK -> RuntimeError with a "GaudiRT ..."
// message raised before any pool write; there is no fallback path.
#include "ops_common.h"

namespace gaudirt_b200 {

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
// Without `key` / `value` the step's rows are already in the pool (stored by the rotary kernel) and no store runs.
at::Tensor paged_attn_impl(const at::Tensor& query, const c10::optional<at::Tensor>& key_in,
                           const c10::optional<at::Tensor>& value_in, at::Tensor& key_pool, at::Tensor& value_pool,
                           const at::Tensor& locations, const at::Tensor& plan_tensor, int64_t head_dim, double scale,
                           double softcap, int64_t sliding_window, const std::vector<at::Tensor>& pushed) {
  const bool store = key_in.has_value() && key_in->defined();
  TORCH_CHECK(store == (value_in.has_value() && value_in->defined()),
              "GaudiRT attention: Q/K/V must be BF16 device matrices with matching rows");
  const at::Tensor& key = store ? *key_in : query;        // stand-ins pass the shared checks when no store runs
  const at::Tensor& value = store ? *value_in : query;
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
  TORCH_CHECK(query.size(1) == plan.query_heads * head_dim && (!store || key.size(1) == plan.kv_heads * head_dim) &&
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
  const at::Tensor k = !store || key.stride(1) == 1 ? key : key.contiguous();
  const at::Tensor v = !store || value.stride(1) == 1 ? value : value.contiguous();
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
      TORCH_CHECK(plan.n_prefill == 0 || (reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0 && out_stride % 8 == 0),
                  "GaudiRT attention: gather destinations of a prefill step must be 16-byte aligned");
      outs.push_back(t.data_ptr());
    }
  }
  int32_t* status = device_status(device.index()).data_ptr<int32_t>();
  const gk_stream_t s = stream_of(stream);
  const int32_t* words = plan.buffer.data_ptr<int32_t>();
  const int32_t* table_rows = plan.table_rows.defined() ? plan.table_rows.data_ptr<int32_t>() : nullptr;
  int32_t* counters = plan.counters.defined() ? plan.counters.data_ptr<int32_t>() : nullptr;
  // The store rides in the attention launch when every sequence is one query block (any decode step) and
  // the rows can be moved 16 bytes at a time; otherwise it is its own launch first, as in the reference
  // (`separate_store`, src/bridge/paged_attention.cpp:251-263).
  const bool fused_store = store && plan.single_block && fuse_kv_store() &&
                           (reinterpret_cast<uintptr_t>(k.data_ptr()) | reinterpret_cast<uintptr_t>(v.data_ptr())) % 16 == 0 &&
                           k.stride(0) % 8 == 0 && v.stride(0) % 8 == 0;
  if (store && !fused_store)
    check_status(gk_kv_store_head_major_bf16(k.data_ptr(), v.data_ptr(), k.stride(0), v.stride(0),
                                             locations.data_ptr<int32_t>(), plan.rows, key_pool.data_ptr(),
                                             value_pool.data_ptr(), plan.slots, (int)plan.kv_heads, (int)head_dim, status, s),
                 "KV store");
  if (fused_store)
    check_status(gk_paged_attn_store_multi_bf16(q.data_ptr(), q.stride(0), k.data_ptr(), v.data_ptr(), k.stride(0),
                                                v.stride(0), locations.data_ptr<int32_t>(), key_pool.data_ptr(),
                                                value_pool.data_ptr(), plan.slots, plan.table.data_ptr<int32_t>(),
                                                plan.table_stride, plan.entry_stride, plan.page_tokens, table_rows, words,
                                                plan.n_work, outs.data(), (int)outs.size(), out_stride,
                                                plan.part_ml.data_ptr<float>(), plan.part_o.data_ptr<float>(), counters,
                                                scale_f, softcap_f, (int)sliding_window, (int)plan.query_heads,
                                                (int)plan.kv_heads, (int)head_dim, status, s),
                 "paged attention");
  else
    check_status(gk_paged_attn_multi_bf16(q.data_ptr(), q.stride(0), key_pool.data_ptr(), value_pool.data_ptr(), plan.slots,
                                          plan.table.data_ptr<int32_t>(), plan.table_stride, plan.entry_stride,
                                          plan.page_tokens, table_rows, words, plan.n_work, outs.data(), (int)outs.size(),
                                          out_stride, plan.part_ml.data_ptr<float>(), plan.part_o.data_ptr<float>(), counters,
                                          scale_f, softcap_f, (int)sliding_window, (int)plan.query_heads,
                                          (int)plan.kv_heads, (int)head_dim, status, s),
                 "paged attention");
  if (!plan.counters.defined())     // otherwise the combine ran inside: the last split to finish merged its block
    check_status(gk_paged_attn_combine_multi_bf16(plan.part_ml.data_ptr<float>(), plan.part_o.data_ptr<float>(),
                                                  words + plan.combine_offset, plan.n_combine, outs.data(),
                                                  (int)outs.size(), out_stride, (int)plan.query_heads, (int)head_dim, s),
                 "split-KV combine");
  if (plan.n_prefill > 0)
    // Query tiles of multi-row sequences: tcgen05 kernel, same destinations (a mixed prefill + decode
    // step is one call, as in src/bridge/paged_attention.cpp:251-345; the two kernels write disjoint rows).
    check_status(gk_paged_prefill_tc_multi_bf16(q.data_ptr(), q.stride(0), key_pool.data_ptr(), value_pool.data_ptr(),
                                                plan.slots, plan.table.data_ptr<int32_t>(), plan.table_stride,
                                                plan.entry_stride, plan.page_tokens,
                                                table_rows, words + plan.prefill_offset, plan.n_prefill, outs.data(), (int)outs.size(),
                                                out_stride, scale_f, softcap_f, (int)sliding_window, (int)plan.query_heads,
                                                (int)plan.kv_heads, (int)head_dim, status, s),
                 "tensor-core prefill");
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
void paged_attn_push(const at::Tensor& query, const c10::optional<at::Tensor>& key,
                     const c10::optional<at::Tensor>& value, at::Tensor& key_pool,
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

// Rotary fused with the head-major KV store: the rotated K row and the V row go straight to slot
// locations[row] of the pool, the rotated Q is returned; `_paged_attn_stored` then attends without
// a store of its own.  One launch where the reference's decoder layer runs two
// (tests/frozen_same_geometry_layer_smoke.py:22-37: rotary, then the store inside attention).
at::Tensor rotary_kv_store(const at::Tensor& query, const at::Tensor& key, const at::Tensor& value, const at::Tensor& cache,
                           const c10::intrusive_ptr<PagedMetadata>& metadata, at::Tensor& key_pool, at::Tensor& value_pool,
                           int64_t head_dim, int64_t rotary_dim, bool is_neox) {
  TORCH_CHECK(metadata, "GaudiRT rotary: metadata is required");
  TORCH_CHECK(head_dim > 0 && head_dim <= INT32_MAX && rotary_dim > 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0,
              "GaudiRT rotary: invalid head or rotary dimension");
  for (const auto& t : {query, key, value, cache})
    TORCH_CHECK(t.is_cuda() && t.device() == query.device() && t.scalar_type() == at::kBFloat16,
                "GaudiRT rotary: expected CUDA BF16 tensors");
  const auto rows = query.dim() == 2 ? query.size(0) : -1;
  TORCH_CHECK(query.dim() == 2 && key.dim() == 2 && value.dim() == 2 && rows > 0 && rows == metadata->rows() &&
                  key.size(0) == rows && value.size(0) == rows && query.size(1) > 0 && key.size(1) > 0 &&
                  query.size(1) % head_dim == 0 && key.size(1) % head_dim == 0 && value.size(1) == key.size(1),
              "GaudiRT rotary: invalid query or key geometry");
  TORCH_CHECK(cache.dim() == 2 && cache.size(0) >= metadata->context() && cache.size(0) <= INT32_MAX &&
                  cache.size(1) == rotary_dim,
              "GaudiRT rotary: cache does not cover validated positions");
  const int64_t kv_heads = key.size(1) / head_dim, slots = metadata->slots();
  for (const auto& pool : {key_pool, value_pool})
    TORCH_CHECK(pool.is_cuda() && pool.device() == query.device() && pool.scalar_type() == at::kBFloat16 &&
                    pool.dim() == 3 && pool.size(0) == slots && pool.size(1) == kv_heads && pool.size(2) == head_dim &&
                    pool.stride(0) == head_dim && pool.stride(1) == slots * head_dim && pool.stride(2) == 1,
                "GaudiRT attention: head-major combined KV pool is required");
  c10::cuda::CUDAGuard guard(query.device());
  const at::Tensor q = query.stride(1) == 1 ? query : query.contiguous();
  const at::Tensor k = key.stride(1) == 1 ? key : key.contiguous();
  const at::Tensor v = value.stride(1) == 1 ? value : value.contiguous();
  const at::Tensor table = cache.contiguous();
  auto q_out = at::empty({rows, query.size(1)}, query.options().memory_format(at::MemoryFormat::Contiguous));
  check_status(gk_rotary_kv_store_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), k.stride(0), v.stride(0),
                                       table.data_ptr(), table.size(0), metadata->rotary_positions().data_ptr<int32_t>(),
                                       metadata->row_locations().data_ptr<int32_t>(), rows, query.size(1), key.size(1),
                                       (int)head_dim, (int)rotary_dim, is_neox ? 1 : 0, q_out.data_ptr(), nullptr,
                                       key_pool.data_ptr(), value_pool.data_ptr(), slots,
                                       device_status(query.device().index()).data_ptr<int32_t>(),
                                       stream_of(at::cuda::getCurrentCUDAStream())),
               "rotary + KV store");
  return q_out;
}

// Attention over a pool that already holds the step's rows (after `_rotary_kv_store`).
at::Tensor paged_attn_stored(const at::Tensor& query, at::Tensor& key_pool, at::Tensor& value_pool,
                             const c10::intrusive_ptr<PagedMetadata>& metadata, int64_t head_dim, double scale,
                             double softcap, int64_t sliding_window) {
  TORCH_CHECK(metadata, "GaudiRT paged attention: metadata is required");
  TORCH_CHECK(query.dim() == 2 && key_pool.dim() == 3 && (head_dim == 64 || head_dim == 128 || head_dim == 256),
              "GaudiRT paged attention: invalid tensor ranks or head dimension");
  const auto q_heads = query.size(1) / head_dim;
  const auto kv_heads = key_pool.size(1);
  auto plan = sliding_window > 0 ? metadata->attention_plan_for(q_heads, kv_heads, head_dim, sliding_window)
                                 : metadata->attention_plan(q_heads, kv_heads, head_dim);
  return paged_attn_impl(query, c10::nullopt, c10::nullopt, key_pool, value_pool, metadata->row_locations(), plan,
                         head_dim, scale, softcap, sliding_window, {});
}

void set_fused_kv_store(bool on) { fuse_kv_store_flag().store(on); }

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
      .def("_revalidate_", &PagedMetadata::revalidate_)
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
      .def("_set_fused_combine", &PagedMetadata::set_fused_combine)
      .def("_last_plan_fuses_combine", &PagedMetadata::last_plan_fuses_combine);
  m.def("paged_attn(Tensor query, Tensor key, Tensor value, Tensor(a!) key_pool, Tensor(b!) value_pool, "
        "__torch__.torch.classes.gaudirt.PagedMetadata metadata, int head_dim, float scale, "
        "float softcap=0.0, int sliding_window=-1) -> Tensor");
  m.def("_paged_attn_validated(Tensor query, Tensor key, Tensor value, Tensor(a!) key_pool, Tensor(b!) value_pool, "
        "Tensor locations, Tensor requests, Tensor positions, Tensor mapping, Tensor header, "
        "int head_dim, float scale, float softcap=0.0, int sliding_window=-1) -> Tensor");
  m.def("_paged_attn_push(Tensor query, Tensor? key, Tensor? value, Tensor(a!) key_pool, Tensor(b!) value_pool, "
        "Tensor locations, Tensor plan, Tensor(c!)[] outputs, int head_dim, float scale, float softcap=0.0, "
        "int sliding_window=-1) -> ()");
  m.def("_paged_attn_stored(Tensor query, Tensor(a!) key_pool, Tensor(b!) value_pool, "
        "__torch__.torch.classes.gaudirt.PagedMetadata metadata, int head_dim, float scale, "
        "float softcap=0.0, int sliding_window=-1) -> Tensor");
  m.def("_rotary_kv_store(Tensor query, Tensor key, Tensor value, Tensor cache, "
        "__torch__.torch.classes.gaudirt.PagedMetadata metadata, Tensor(a!) key_pool, Tensor(b!) value_pool, "
        "int head_dim, int rotary_dim, bool is_neox) -> Tensor");
  m.def("_set_fused_kv_store(bool on) -> ()", &gaudirt_b200::set_fused_kv_store);
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
  m.impl("_paged_attn_stored", TORCH_FN(gaudirt_b200::paged_attn_stored));
  m.impl("_rotary_kv_store", TORCH_FN(gaudirt_b200::rotary_kv_store));
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
