/*
 * gaudirt_b200 -- C ABI of the B200 (sm_100a) paged KV-store / paged-attention path.
 *
 * This is the drop-in boundary: plain C, device pointers + sizes + a CUDA stream.  No entry
 * point allocates device memory, synchronises the device or throws; each returns a gk_status
 * (0 = success) and enqueues its work on `stream`.  Validation that needs tensor metadata,
 * allocation and error translation belong to the caller's framework layer.
 *
 * Citations are path:line inside the reference project (tracycam/GaudiRT); each entry point
 * names the reference interface it replaces.
 *
 * Memory layouts (all bf16 unless stated):
 *   pool      one layer of the combined KV pool, [2, kv_heads, slots, head_dim] contiguous
 *             (src/bridge/paged_kv_pool.cpp:15-41).  pool_k = &pool[0], pool_v = &pool[1];
 *             element (h, slot, c) of either half lives at (h*slots + slot)*head_dim + c.
 *   q / out   [rows, q_heads*head_dim], row stride given in elements.
 *   k / v     [rows, kv_heads*head_dim], row stride given in elements (column slices of a
 *             packed QKV projection are allowed).
 *   table     int32 slot table.  Row `t` starts at table + t*table_stride; page j of that row
 *             is described by the entry at j*table_entry_stride, which holds the slot of token
 *             j*page_tokens; the page_tokens tokens of a page occupy consecutive slots.
 *             page_tokens == 1, table_entry_stride == 1 is the reference's request-to-token
 *             `mapping[requests, context]` itself (src/bridge/paged_metadata.cpp:104-140);
 *             the same array with page_tokens == table_entry_stride == P reads one entry per
 *             page; a block table is table_entry_stride == 1 with page_tokens == block size.
 *   table_rows  optional int32 device array: the table row of a work record is
 *             table_rows[record.table_row] instead of record.table_row (request ids that only
 *             exist on the device, PagedMetadata::from_device, src/bridge/paged_metadata.hpp:26-64).
 */
#ifndef GAUDIRT_B200_H_
#define GAUDIRT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* gk_stream_t; /* cudaStream_t */

#if defined(__GNUC__)
#define GK_API __attribute__((visibility("default")))
#else
#define GK_API
#endif

enum gk_status {
  GK_OK = 0,
  GK_ERR_INVALID_ARGUMENT = 1,  /* null pointer, negative size, misaligned pointer or stride   */
  GK_ERR_UNSUPPORTED = 2,       /* geometry outside what the kernels implement: fail fast      */
  GK_ERR_CUDA = 3,              /* the CUDA runtime refused the launch; see gk_last_cuda_error */
  GK_ERR_CAPACITY = 4,          /* an output array or fixed scratch area is too small          */
  GK_ERR_METADATA = 5           /* host metadata validation failed; see the message accessor   */
};

/* Bits a kernel may OR into the caller's int32 device status word (never cleared by kernels). */
enum gk_device_status {
  GK_DEV_BAD_SLOT = 1,          /* a slot outside [0, slots) was met: the access was skipped   */
  GK_DEV_BAD_TABLE = 2,         /* a table entry outside [0, slots) was met: key left out      */
  GK_DEV_WAIT_EXPIRED = 4,      /* a bounded wait ran out                                      */
  GK_DEV_BAD_METADATA = 8       /* device-side metadata validation rejected a row              */
};

GK_API const char* gk_status_string(int status);
GK_API int gk_abi_version(void);
/* cudaError_t of the last failed launch on the calling thread (0 if none). */
GK_API int gk_last_cuda_error(void);

/* Size of a work record and of a combine record, in int32 words. */
#define GK_WORK_WORDS 8
#define GK_COMBINE_WORDS 4
/* Largest number of packed query rows (rows of one sequence x query heads of one KV head)
 * one work item may carry. */
#define GK_MAX_PACKED_ROWS 16
/* KV tile the independent tiled CPU reference must use for this implementation
 * (_C._paged_attn_kv_tile, src/bridge/generic_private_use1.cpp; 512 in the reference). */
#define GK_REFERENCE_KV_TILE 512

/* ---- pool -------------------------------------------------------------------------------
 * Replaces the geometry checks of allocate_paged_kv (src/bridge/paged_kv_pool.cpp:15-41).
 * Writes the byte size of [layers, 2, kv_heads, slots, head_dim] bf16.  The reference's
 * 131072-slot descriptor cap and descriptor tail do not exist here. */
GK_API int gk_paged_kv_pool_bytes(int64_t layers, int64_t slots, int64_t kv_heads, int64_t head_dim,
                           uint64_t* bytes_out);

/* ---- metadata (host) --------------------------------------------------------------------
 * Replaces the host half of the PagedMetadata constructor (src/bridge/paged_metadata.cpp:82-140):
 * range checks, mapping[request, position] == location, unique output slots, visible prefix
 * fully mapped and not aliased by an output slot.  Host arrays only.
 *   seq_out   [rows*4] receives {first_row, n_rows, first_position, request} per sequence
 *             (maximal runs of one request with consecutive positions).
 *   page_tokens_out  largest power of two <= 128 such that every visible prefix is made of
 *             slot-contiguous pages of that many tokens (1 if none).
 * On GK_ERR_METADATA, gk_metadata_error() returns the reference's message. */
GK_API int gk_paged_metadata_validate(const int32_t* locations, const int32_t* requests,
                               const int32_t* positions, int64_t rows, const int32_t* mapping,
                               int64_t n_requests, int64_t context, int64_t slots,
                               int32_t* seq_out, int64_t* n_seq_out, int32_t* page_tokens_out);
GK_API const char* gk_metadata_error(void);

/* ---- attention plan (host) --------------------------------------------------------------
 * Replaces PagedMetadata::attention_plan_for (src/bridge/attention_plan.cpp:146-361) and the
 * gk_attn_tile_indices_i32_v1 gather-index kernel: the schedule is a list of work records
 * (query block x KV range) balanced over the SMs; slots are looked up in the kernel.
 *   seq       [n_seq*4] as written by gk_paged_metadata_validate.
 *   window    sliding window (-1 = none): keys below position-window+1 are never scheduled.
 *   split_tokens  0 = choose from sm_count; otherwise the longest KV range of one work item.
 *   work_out  [work_cap*GK_WORK_WORDS] {first_row, n_rows, first_position, table_row,
 *             kv_begin, kv_end, partial_base (-1 = writes the output itself),
 *             n_splits | split_index << 16},
 *             longest first.  combine_out [combine_cap*GK_COMBINE_WORDS] {first_row, n_rows,
 *             partial_base, n_splits} for every query block cut into more than one range.
 *   partial_entries_out  number of (row, query head) entries of fp32 split state needed.
 * Pass work_out == NULL to obtain the three counts only. */
GK_API int gk_attention_plan_build(const int32_t* seq, int64_t n_seq, int q_heads, int kv_heads,
                            int head_dim, int window, int sm_count, int split_tokens,
                            int32_t* work_out, int64_t work_cap, int64_t* n_work_out,
                            int32_t* combine_out, int64_t combine_cap, int64_t* n_combine_out,
                            int64_t* partial_entries_out);

/* ---- KV store ---------------------------------------------------------------------------
 * Replaces gk_kv_store_head_major_bf16_v1 / launch_layer_kv_store
 * (src/bridge/paged_attention_tiles.cpp:37-55,236-260): for r < rows, h < kv_heads
 *   pool_k[(h*slots + locations[r])*d ...] = k[r*k_row_stride + h*d ...]   (same for v).
 * A bit copy; slots not named in `locations` are untouched.  `locations` must not repeat a
 * slot.  Rows whose slot is outside [0, slots) are skipped and GK_DEV_BAD_SLOT is set in
 * *status (status may be NULL).  Any row stride / 2-byte alignment is accepted; 16-byte
 * aligned inputs take the vector path. */
GK_API int gk_kv_store_head_major_bf16(const void* k, const void* v, int64_t k_row_stride,
                                int64_t v_row_stride, const int32_t* locations, int64_t rows,
                                void* pool_k, void* pool_v, int64_t slots, int kv_heads,
                                int head_dim, int32_t* status, gk_stream_t stream);

/* ---- paged attention --------------------------------------------------------------------
 * Replaces the fused single-tile recipe and the multi-tile chunk recipes
 * (src/bridge/paged_attention.cpp:39-127, src/bridge/paged_attention_tiles.cpp:57-195):
 *   S = Q K^T (fp32) ; s = scale*S ; softcap c*tanh(s/c) if softcap > 0 ;
 *   row at position p sees keys max(0, p-window+1) .. p ; P = softmax, rounded to bf16
 *   before P V ; fp32 accumulation ; out = bf16(O / l).
 * Query head h reads KV head h / (q_heads/kv_heads).  One CTA runs one work record for one
 * KV head; records with partial_base >= 0 leave (m, l, O) fp32 split state in the workspace
 * for gk_paged_attn_combine_bf16, the others write `out` directly.
 *   part_ml   fp32 [partial_entries*2] (m in log2 units, l), part_o fp32 [partial_entries*d].
 * head_dim in {64, 128, 256}; q_heads/kv_heads <= GK_MAX_PACKED_ROWS. */
GK_API int gk_paged_attn_bf16(const void* q, int64_t q_row_stride, const void* pool_k,
                       const void* pool_v, int64_t slots, const int32_t* table,
                       int64_t table_stride, int64_t table_entry_stride, int page_tokens,
                       const int32_t* table_rows, const int32_t* work,
                       int64_t n_work, void* out, int64_t out_row_stride, float* part_ml,
                       float* part_o, float scale, float softcap, int window, int q_heads,
                       int kv_heads, int head_dim, int32_t* status, gk_stream_t stream);

/* Programmatic dependent launch (on by default): the attention, combine, norm, rotary and barrier kernels
 * are launched so that the GPU may set them up while the kernel before them in the stream is still
 * running; their first statement waits until that kernel has completed and its writes are visible, so
 * every access keeps plain stream order and only launch latency overlaps.  0 switches back to ordinary
 * launches.  Process-wide; the reference has no such switch. */
GK_API int gk_set_programmatic_launch(int on);

/* How the attention kernel brings a 16-token group of K and V into shared memory.  BOXES: one
 * cp.async.bulk.tensor box per group (K and V, all columns; needs pages of at least 16 tokens, groups
 * that do not qualify -- ragged ends, ranges starting off a 16-token boundary -- are copied row by row).
 * ROWS: 16-byte cp.async copies for every group (the only form for token-granular tables).  AUTO (the
 * default) takes BOXES for launches of at most two CTAs per SM and ROWS otherwise, which is where each
 * measured faster.  Both forms produce the same bits.  Process-wide; not part of the reference, which has
 * no such choice (its gather runs in a separate index kernel, src/bridge/attention_plan.cpp:246-255). */
#define GK_ATTENTION_FORM_AUTO 0
#define GK_ATTENTION_FORM_ROWS 1
#define GK_ATTENTION_FORM_BOXES 2
GK_API int gk_set_attention_form(int form);

/* Replaces gk_attn_online_merge_f32_v1 + gk_attn_online_finalize_bf16_v1
 * (src/bridge/paged_attention_tiles.cpp:173-188): merges the n_splits partial states of every
 * combine record in split order (deterministic) and writes bf16(O / l); l == 0 gives 0. */
GK_API int gk_paged_attn_combine_bf16(const float* part_ml, const float* part_o, const int32_t* combine,
                               int64_t n_combine, void* out, int64_t out_row_stride, int q_heads,
                               int head_dim, gk_stream_t stream);

/* ---- chunked prefill on the tensor cores -----------------------------------------------------
 * The multi-row half of the same reference recipes (src/bridge/paged_attention_tiles.cpp:57-195:
 * prefill / extend blocks of up to 256-512 rows against 512-key tiles on the MME): query tiles of
 * GK_PREFILL_TILE_ROWS packed rows (rows x query heads of one KV head), GK_PREFILL_TILES_PER_ITEM
 * of them per work record, against 128-key tiles that are fetched once for all tiles of the
 * record; Q K^T and P V as tcgen05 UMMA contractions with fp32 accumulators in tensor memory (P is
 * the A operand straight from tensor memory), online softmax between them, causal inside the
 * chunk.  Same arithmetic contract as gk_paged_attn_bf16 (P rounded to bf16 before P V, fp32
 * accumulation, out = bf16(O / l)).  head_dim in {64, 128, 256}, the geometries of
 * tests/paged_attention_generalized_smoke.py:59-65; at 256 the two query tiles of a record run in
 * two CTAs against 64-key tiles (the accumulators of two tiles would not fit in tensor memory).
 *
 * gk_prefill_plan_build splits a step's sequences: those with at least min_rows rows
 * (0 = default, ceil(32 / (q_heads/kv_heads)) but at least 2) become tensor-core work records
 * {first_row, n_rows <= GK_PREFILL_TILES_PER_ITEM * (GK_PREFILL_TILE_ROWS / group), first_position,
 * table_row, kv_begin, kv_end, -1, 1}, longest KV range first; the others are copied to
 * rest_seq_out ([n_seq*4]) for gk_attention_plan_build.  Pass work_out == NULL to obtain the
 * counts only. */
#define GK_PREFILL_TILES_PER_ITEM 2
#define GK_PREFILL_TILE_ROWS 128
GK_API int gk_prefill_plan_build(const int32_t* seq, int64_t n_seq, int q_heads, int kv_heads,
                          int window, int min_rows, int32_t* work_out, int64_t work_cap,
                          int64_t* n_work_out, int32_t* rest_seq_out, int64_t* n_rest_out);
GK_API int gk_paged_prefill_tc_bf16(const void* q, int64_t q_row_stride, const void* pool_k,
                             const void* pool_v, int64_t slots, const int32_t* table,
                             int64_t table_stride, int64_t table_entry_stride, int page_tokens,
                             const int32_t* table_rows, const int32_t* work, int64_t n_work,
                             void* out, int64_t out_row_stride, float scale, float softcap,
                             int window, int q_heads, int kv_heads, int head_dim,
                             int32_t* status, gk_stream_t stream);

/* ---- tensor-parallel output gather fused into the attention epilogue ----------------------
 * Replaces AllGatherDimLast after attention (src/bridge/segmented_runner.cpp:170-191,
 * src/bridge/communicator.cpp:56-116: hcclAllGather into scratch + a transpose recipe): with KV
 * heads sharded over `world` ranks, rank r's kernels store their [rows, cols] result into
 * column block r of the gathered [rows, world*cols] activation of EVERY rank, i.e. `outs[p]`
 * is (peer p's gathered buffer) + r*cols with out_row_stride = world*cols.  Peer buffers are
 * ordinary peer-mapped device memory (CUDA IPC / symmetric memory); the kernels only issue
 * plain stores to them.  The multi forms are otherwise identical to the single-output forms,
 * except for split_counters: when not NULL it is an int32 array [rows * kv_heads], all zero, and
 * the attention kernel then also performs the combine -- the CTA that completes the last split of
 * a query block merges all of the block's splits in split order (the result does not depend on
 * which CTA that is) and leaves the counter at zero again; no combine launch is needed. */
#define GK_MAX_OUTPUTS 8
GK_API int gk_paged_attn_multi_bf16(const void* q, int64_t q_row_stride, const void* pool_k,
                             const void* pool_v, int64_t slots, const int32_t* table,
                             int64_t table_stride, int64_t table_entry_stride, int page_tokens,
                             const int32_t* table_rows, const int32_t* work, int64_t n_work,
                             void* const* outs, int n_outs, int64_t out_row_stride,
                             float* part_ml, float* part_o, int32_t* split_counters,
                             float scale, float softcap, int window, int q_heads, int kv_heads,
                             int head_dim, int32_t* status, gk_stream_t stream);
GK_API int gk_paged_attn_combine_multi_bf16(const float* part_ml, const float* part_o,
                                     const int32_t* combine, int64_t n_combine,
                                     void* const* outs, int n_outs, int64_t out_row_stride,
                                     int q_heads, int head_dim, gk_stream_t stream);
/* gk_kv_store_head_major_bf16 fused into the attention launch, as the reference's single-block
 * recipe does (src/bridge/paged_attention.cpp:74; `separate_store` at :251 decides): every CTA
 * first copies the new K/V rows whose positions fall into its own KV range to their pool slots,
 * then attends.  Valid only for a step whose sequences are ONE query block each (n_rows <=
 * GK_MAX_PACKED_ROWS / group, e.g. any decode step) and whose work records come from
 * gk_attention_plan_build for exactly those sequences, because then no other CTA reads the rows;
 * the caller decides that (the operator layer does, and launches the store separately otherwise).
 * new_k / new_v must be 16-byte aligned with row strides that are multiples of 8 elements
 * (GK_ERR_UNSUPPORTED otherwise).  The pool ends up bit-identical to the separate store. */
GK_API int gk_paged_attn_store_multi_bf16(const void* q, int64_t q_row_stride, const void* new_k,
                                   const void* new_v, int64_t new_k_row_stride,
                                   int64_t new_v_row_stride, const int32_t* locations,
                                   void* pool_k, void* pool_v, int64_t slots, const int32_t* table,
                                   int64_t table_stride, int64_t table_entry_stride,
                                   int page_tokens, const int32_t* table_rows, const int32_t* work,
                                   int64_t n_work, void* const* outs, int n_outs,
                                   int64_t out_row_stride, float* part_ml, float* part_o,
                                   int32_t* split_counters, float scale, float softcap, int window,
                                   int q_heads, int kv_heads, int head_dim, int32_t* status,
                                   gk_stream_t stream);
/* The tensor-core prefill kernel with the same multi-destination epilogue, so that a prefill or a
 * mixed prefill + decode step (one call in the reference, src/bridge/paged_attention.cpp:251-345)
 * is gathered by the kernels' own stores as well; destinations must be 16-byte aligned. */
GK_API int gk_paged_prefill_tc_multi_bf16(const void* q, int64_t q_row_stride, const void* pool_k,
                                   const void* pool_v, int64_t slots, const int32_t* table,
                                   int64_t table_stride, int64_t table_entry_stride,
                                   int page_tokens, const int32_t* table_rows, const int32_t* work,
                                   int64_t n_work, void* const* outs, int n_outs,
                                   int64_t out_row_stride, float scale, float softcap, int window,
                                   int q_heads, int kv_heads, int head_dim, int32_t* status,
                                   gk_stream_t stream);
/* Completion barrier that follows the pushes (replaces the wait on the collective,
 * src/bridge/segmented_runner.cpp:489-506): flags[p] is rank p's int32[world] flag array as
 * mapped in this process.  Writes `epoch` to slot `rank` of every peer's array, then waits
 * until all slots of its own array have reached `epoch` (epochs only grow).  The wait gives up
 * after max_cycles SM clock cycles and sets GK_DEV_WAIT_EXPIRED in *status; it never traps. */
GK_API int gk_peer_barrier(int32_t* const* flags, int rank, int world, int32_t epoch,
                    int64_t max_cycles, int32_t* status, gk_stream_t stream);
/* The same barrier with the epoch kept in device memory: the launch uses *epoch_counter + 1 and
 * stores it back, so it takes no per-call host value and can be replayed from a CUDA graph.  All
 * ranks must issue the same sequence of barriers on counters that start equal. */
GK_API int gk_peer_barrier_counted(int32_t* const* flags, int rank, int world, int32_t* epoch_counter,
                            int64_t max_cycles, int32_t* status, gk_stream_t stream);

/* ---- front of a decode layer ---------------------------------------------------------------
 * Replace gk_rms_norm_bf16_v1 / gk_fused_add_rms_norm_bf16_v1 (src/bridge/fx_op_lowering.cpp:450-478,
 * entry checks src/bridge/eager_ops.cpp:1140-1212):
 *   u = bf16(x + residual)              (fused form only; written to `u`)
 *   y = bf16(u * rsqrt(mean(u^2) + epsilon) * (weight + weight_offset))
 * x, residual: [rows, hidden] with the given row strides (elements); y, u: [rows, hidden]
 * contiguous; weight: [hidden]; hidden <= 8192.  Each boundary is rounded once from fp64. */
GK_API int gk_rms_norm_bf16(const void* x, const void* weight, float epsilon, float weight_offset,
                     int64_t rows, int64_t hidden, int64_t x_row_stride, void* y,
                     gk_stream_t stream);
GK_API int gk_fused_add_rms_norm_bf16(const void* x, const void* residual, const void* weight,
                               float epsilon, float weight_offset, int64_t rows, int64_t hidden,
                               int64_t x_row_stride, int64_t residual_row_stride, void* y,
                               void* u, gk_stream_t stream);

/* Replaces gk_rotary_bf16_v1 / gk_rotary_pos_bf16_v1 (src/bridge/generic_private_use1.cpp:295-418,
 * src/bridge/bucket_program.cpp:499-516): per head of q [rows, q_width] and k [rows, k_width],
 * with (cos, sin) = cache[positions[row]] (cache [cache_rows, rotary_dim] = cos || sin):
 *   neox: pairs (i, i + rotary_dim/2), otherwise pairs (2i, 2i+1);
 *   a' = bf16(a*cos - b*sin), b' = bf16(b*cos + a*sin); elements past rotary_dim are copied.
 * q_out / k_out are contiguous.  A position outside [0, cache_rows) passes the row through
 * unrotated and sets GK_DEV_BAD_SLOT in *status. */
GK_API int gk_rotary_bf16(const void* q, const void* k, int64_t q_row_stride, int64_t k_row_stride,
                   const void* cache, int64_t cache_rows, const int32_t* positions, int64_t rows,
                   int64_t q_width, int64_t k_width, int head_dim, int rotary_dim, int is_neox,
                   void* q_out, void* k_out, int32_t* status, gk_stream_t stream);

/* gk_rotary_bf16 fused with gk_kv_store_head_major_bf16 (the two reference kernels above it in
 * the decoder layer, tests/frozen_same_geometry_layer_smoke.py:22-37, as one launch): the rotated
 * K row and the V row go straight to slot locations[row] of the head-major pool; k_out may be
 * NULL when the rotated K is not needed elsewhere. */
GK_API int gk_rotary_kv_store_bf16(const void* q, const void* k, const void* v, int64_t q_row_stride,
                            int64_t k_row_stride, int64_t v_row_stride, const void* cache,
                            int64_t cache_rows, const int32_t* positions,
                            const int32_t* locations, int64_t rows, int64_t q_width,
                            int64_t k_width, int head_dim, int rotary_dim, int is_neox,
                            void* q_out, void* k_out, void* pool_k, void* pool_v, int64_t slots,
                            int32_t* status, gk_stream_t stream);

/* ---- the steps either side of the path ------------------------------------------------------
 * Slot allocation, replaces gk_paged_alloc_i32_v1 and its host set-up
 * (src/bridge/paged_slot_allocator.cpp:91-151; known answers tests/paged_slots_device_smoke.py:16-33).
 * gk_paged_slots_layout is the host half: it checks the request lists like the reference
 * (message through gk_metadata_error) and writes one int32 record {prefix, length, first token,
 * first fresh page} per request; *total_out = new tokens, *pages_out = fresh pages consumed
 * (must not exceed free_page_count).  records_out may be NULL for a sizing call.
 * gk_paged_slots_allocate takes those records in device memory (16-byte aligned) and writes
 * slots_out[total]: token j of request r gets last_slots[r] + 1 + j while it still fits the
 * partly filled page ((-prefix) mod page_size tokens), then
 * free_pages[first_page + k / page_size] * page_size + k % page_size.
 * Optional fused outputs, which save the scheduler two scatter launches: `locations_out`
 * (int32 copy of the slots, the KV store's input) and `table` (the request-to-token table of
 * the attention kernel: table[row(r)][prefix + j] = slot, row(r) = table_rows ? table_rows[r] : r).
 * A slot that does not fit int32 or a table cell out of range is skipped and reported in *status. */
GK_API int gk_paged_slots_layout(const int64_t* prefixes, const int64_t* lengths, int64_t n_requests,
                          int64_t page_size, int64_t free_page_count, int32_t* records_out,
                          int64_t* total_out, int64_t* pages_out);
GK_API int gk_paged_slots_allocate(const int64_t* last_slots, const int64_t* free_pages,
                            const int32_t* records, int64_t n_requests, int64_t total,
                            int64_t page_size, int64_t* slots_out, int32_t* table,
                            int64_t table_row_count, int64_t table_stride, int64_t table_context,
                            const int32_t* table_rows, int32_t* locations_out, int32_t* status,
                            gk_stream_t stream);

/* Slot release, replaces gk_paged_free_i32_v1 (src/bridge/paged_slot_allocator.cpp:153-209):
 * pages_out receives slot / page_size for every slot, in order of first occurrence, each page
 * once; count_out[0] = number of pages written, count_out[1] = number of slots that were not
 * inside (0, max_pages * page_size) (the reference raises "released slot is outside the KV
 * pool" for those; they are left out here).  pages_out holds n_slots entries; `workspace` is
 * 256-byte aligned device memory of gk_paged_slots_release_workspace_bytes bytes.  The result
 * does not depend on thread scheduling. */
GK_API int gk_paged_slots_release_workspace_bytes(int64_t n_slots, int64_t max_pages,
                                           uint64_t* bytes_out);
GK_API int gk_paged_slots_release(const int64_t* slots, int64_t n_slots, int64_t page_size,
                           int64_t max_pages, void* workspace, int64_t* pages_out,
                           int32_t* count_out, gk_stream_t stream);

/* Replaces advance_decode_lengths (src/bridge/eager_scheduler.cpp:51-82): next = current + 1
 * for both vectors in one launch, inputs left untouched, no host copy in either direction. */
GK_API int gk_advance_decode_lengths(const int64_t* seq_lens, const int32_t* orig_seq_lens,
                              int64_t count, int64_t* next_seq_lens, int32_t* next_orig_seq_lens,
                              gk_stream_t stream);

/* Validation of device-resident step metadata, replaces gk_paged_metadata_i32_v1 /
 * gk_scheduler_metadata_i32_v1 / gk_token_indices_i32_v1 (src/bridge/paged_metadata.cpp:26-79,
 * 326-430).  locations / positions [rows], batch_requests [n_seq] and token_ids [rows] are
 * int32, or int64 where their bit of wide_mask (1, 2, 4, 8 in that order: locations,
 * batch_requests, positions, token_ids) is set.  seq is a device copy of the host's per-sequence
 * int32 records {first_row, n_rows, prefix, index into batch_requests} (16-byte aligned).
 * Outputs: int32 locations / row-expanded requests / positions (/ tokens), last_token_out[n_seq]
 * (may be NULL), row_status[rows] with a code per row:
 *   1 slot or position out of range (or beyond int32)   2 request id out of range
 *   3 table[request][position] != slot                  4 slot written by two rows
 *   5 position != prefix + offset in its sequence       6 visible table entry outside [0, slots)
 *   7 cached-prefix entry names a slot this step writes
 * (6 and 7 are charged to the first row of the sequence), token_status[rows] (1 = token outside
 * [0, vocabulary)), first_error[3]: [0] = min over bad rows of (row << 8 | code), [1] = first row
 * with a bad token, both UINT64_MAX when clean, [2] = the smallest (p & -p) over the visible
 * positions p where table[p] != table[p-1] + 1, i.e. the largest power-of-two page size whose
 * pages are slot-contiguous in every visible range (UINT64_MAX: no break at all).  table == NULL (a table owned and
 * vouched for by the scheduler) skips 3, 6 and 7.  Any rejection also sets GK_DEV_BAD_METADATA
 * in *status (may be NULL).  `workspace`: gk_paged_metadata_device_workspace_bytes(slots) bytes.
 * Rejected entries are replaced by 0 in the int32 outputs so later kernels stay in bounds. */
GK_API int gk_paged_metadata_device_workspace_bytes(int64_t slots, uint64_t* bytes_out);
GK_API int gk_paged_metadata_device_validate(
    const void* locations, const void* batch_requests, const void* positions, const void* token_ids,
    int wide_mask, int64_t vocabulary, const int32_t* table, int64_t n_requests, int64_t context,
    int64_t table_stride, int64_t slots, const int32_t* seq, int64_t n_seq, int64_t rows,
    void* workspace, int32_t* locations_out, int32_t* requests_out, int32_t* positions_out,
    int32_t* tokens_out, int32_t* last_token_out, int32_t* row_status, int32_t* token_status,
    uint64_t* first_error, int32_t* status, gk_stream_t stream);

/* ---- o_proj and its rank-ordered sum --------------------------------------------------------
 * The step behind the attention block in tensor-parallel decode (the reference's design notes
 * name the chain O-Proj -> AllReduce -> AddRMSNorm): every rank multiplies its heads by its
 * slice of the o_proj weight, the partial results are summed in rank order
 * (src/bridge/communicator.cpp:373-417, expectation tests/tp4_gather_reduce_smoke.py:16-20), and
 * the sum enters the next layer's fused residual-add RMS norm.
 *
 * gk_oproj_bf16: out[m, n] = bf16(a[m, k] . weight[n, k]^T), bf16 operands, fp32 accumulation on
 * the tensor cores (tcgen05, accumulators in TMEM, operands by TMA).  n and k must be multiples
 * of 64, strides (elements) multiples of 8, pointers 16-byte aligned.  The same result is stored
 * to all n_outs destinations (host array of device pointers, common row stride): a destination
 * may be a peer GPU's receive buffer, which makes the exchange part of this kernel's epilogue.
 * gk_rank_sum_bf16: out[i] = bf16(((f32(parts[0][i]) + f32(parts[1][i])) + ...)), one fp32
 * rounding per add, rank order fixed, so every rank computes the same bits; count % 8 == 0.
 * gk_rank_sum_add_rms_norm_bf16: that sum as the `x` of gk_fused_add_rms_norm_bf16, without
 * writing it out: u = bf16(sum + residual), y = norm(u).  hidden % 8 == 0, hidden <= 8192. */
GK_API int gk_oproj_bf16(const void* a, int64_t a_row_stride, const void* weight,
                  int64_t weight_row_stride, int64_t m, int64_t n, int64_t k, void* const* outs,
                  int n_outs, int64_t out_row_stride, int32_t* status, gk_stream_t stream);
GK_API int gk_rank_sum_bf16(const void* const* parts, int world, int64_t count, void* out,
                     gk_stream_t stream);
GK_API int gk_rank_sum_add_rms_norm_bf16(const void* const* parts, int world, int64_t part_row_stride,
                                  const void* residual, const void* weight, float epsilon,
                                  float weight_offset, int64_t rows, int64_t hidden,
                                  int64_t residual_row_stride, void* y, void* u,
                                  gk_stream_t stream);

/* ---- after the LM head ------------------------------------------------------------------------
 * Replace gk_argmax_parts/finish, gk_apply_vocab_bitmask_{f32,bf16} and gk_sample_vocab_{f32,bf16}
 * (src/bridge/argmax_vocab.cpp, src/bridge/sampler_vocab.cpp:289-485).  logits: [rows, cols] bf16
 * (is_f32 = 0) or fp32 (is_f32 = 1), row stride in elements, columns contiguous.
 * gk_vocab_argmax: out[row] = index of the maximum with torch.argmax's rules (NaN is the largest
 * value, the first of equal values wins, -0 == +0).
 * gk_apply_vocab_bitmask: for every listed row (all rows, or row_indices[n_indices] on the device;
 * duplicates are harmless, an index outside the logits or the mask sets GK_DEV_BAD_METADATA and is
 * skipped) column c becomes -inf when c < active_cols and bit (c & 31) of bitmask[row][c >> 5] is 0,
 * or when c >= active_cols and mask_tail is set; every other element is left untouched.
 * gk_sample_vocab: one token per row.  temperature <= 0: the argmax (NaN counted as -inf when
 * nan_to_neg_inf).  Otherwise, with w = exp((x - max) / temperature): keep w >= the top_k-th
 * largest w (top_k outside [1, cols) keeps all), of those keep w >= the largest t whose mass
 * {w >= t} reaches top_p of the kept mass, keep w >= min_p; draw from the kept set in proportion to
 * w.  The draw is a pure function of (logits row, parameters, seeds[row], positions[row]):
 * u = splitmix64(splitmix64(seed ^ splitmix64(position))) scaled to the kept mass, masses summed
 * in 2^-40 fixed point.  seeds == NULL: rows are seeded from base_seed; positions may be NULL. */
GK_API int gk_vocab_argmax(const void* logits, int is_f32, int64_t rows, int64_t cols,
                    int64_t row_stride, int64_t* out, gk_stream_t stream);
GK_API int gk_apply_vocab_bitmask(void* logits, int is_f32, int64_t rows, int64_t cols,
                           int64_t row_stride, const int32_t* bitmask, int64_t mask_rows,
                           int64_t mask_words, const int32_t* row_indices, int64_t n_indices,
                           int64_t active_cols, int mask_tail, int32_t* status,
                           gk_stream_t stream);
GK_API int gk_sample_vocab(const void* logits, int is_f32, int64_t rows, int64_t cols,
                    int64_t row_stride, const float* temperatures, const float* top_ps,
                    const int32_t* top_ks, const float* min_ps, const int64_t* seeds,
                    const void* positions, int positions_are_i64, uint64_t base_seed,
                    int nan_to_neg_inf, int32_t* out, gk_stream_t stream);

/* ---- attention without any device allocation ---------------------------------------------
 * This entry point has no counterpart in the reference.  It is for callers that must not
 * allocate device memory on their hot path: a serving engine that has handed all HBM to its own
 * KV pool, a plugin called under a framework whose allocator it may not enter, a real-time loop
 * where cudaMalloc's implicit synchronisation is not acceptable.  It runs gk_paged_attn_bf16 and
 * then gk_paged_attn_combine_bf16 with the fp32 split state kept in an array that is part of
 * the library image itself (GK_STATIC_SCRATCH_MAX_ENTRIES entries of up to
 * GK_STATIC_SCRATCH_MAX_HEAD_DIM floats plus (m, l): about 8.5 MB, resident on every GPU that
 * loads the library until the process exits).  It calls no cudaMalloc, cudaFree or allocating
 * library routine.
 *   partial_entries   what gk_attention_plan_build reported for this schedule; more than
 *                     GK_STATIC_SCRATCH_MAX_ENTRIES (or head_dim above the maximum) is refused
 *                     with GK_ERR_CAPACITY before anything is launched.
 *   combine, n_combine  the schedule's combine records (may be empty).
 *                     A work or combine record that points past `partial_entries` is skipped on
 *                     the device and GK_DEV_BAD_SLOT is raised in *status: a schedule that
 *                     disagrees with the declared count cannot write outside the array.
 * All arguments are checked before the first launch; split state without combine records (or the
 * reverse), and combine records without work records, are GK_ERR_INVALID_ARGUMENT.
 * The first call on each device looks up the device address of the array.  The entry point itself
 * allocates nothing, but under CUDA's lazy module loading the first use of the library's device
 * code on a device is also the moment the driver loads the module and gives the array its memory,
 * so the very first call is not free of driver-side allocation: make it once per device at
 * start-up (a schedule with n_work = 0 will do), and before starting any stream capture.  All
 * calls share the one array: it keeps the previous call's contents (nothing in it needs clearing,
 * every entry a combine record reads is written by that call's attention kernel first), and two
 * calls whose kernels overlap on the GPU (different streams, or different threads) race on it. */
#define GK_STATIC_SCRATCH_MAX_ENTRIES 8192
#define GK_STATIC_SCRATCH_MAX_HEAD_DIM 256
GK_API int gk_paged_attn_static_scratch_bf16(const void* q, int64_t q_row_stride, const void* pool_k,
                                      const void* pool_v, int64_t slots, const int32_t* table,
                                      int64_t table_stride, int64_t table_entry_stride,
                                      int page_tokens, const int32_t* table_rows,
                                      const int32_t* work, int64_t n_work, const int32_t* combine,
                                      int64_t n_combine, int64_t partial_entries, void* out,
                                      int64_t out_row_stride, float scale, float softcap,
                                      int window, int q_heads, int kv_heads, int head_dim,
                                      int32_t* status, gk_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* GAUDIRT_B200_H_ */
