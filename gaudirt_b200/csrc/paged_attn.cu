// Paged attention over the head-major bf16 KV pool: the decode / short-query kernel and the
// split-KV combine.
//
// One CTA runs one work record (a query block of one sequence x a KV range) for one KV head.
// All query heads of the KV head's GQA group -- times the rows of the block -- are packed into
// the 16 rows of an m16n8k16 tile, so every K/V byte is read from HBM once per work item.
// The KV range is cut into 16-token groups dealt round-robin to the warps; each warp owns a
// private ring of staged groups and never meets a block-wide barrier until the final cross-warp
// merge.  The kernel exists in two forms that stage a group differently and are otherwise the same
// code (same bits):
//   boxes  a group that is 16 slot-contiguous tokens of one page (any page of at least 16 tokens) is
//          fetched by one lane as ONE 4-D TMA box (cp.async.bulk.tensor: K and V, every 64-column
//          panel, 16 rows, 128-byte swizzle, no multicast), completion by transaction bytes on the
//          stage's own mbarrier (bounded wait); the rare other group -- a ragged end, a range that does
//          not start on a 16-token boundary -- is copied row by row and waited for on the spot;
//   rows   every group row by row with 16-byte cp.async into the same layout (rows past the range
//          zero-filled), one cp.async group per stage; the only form for token-granular tables.
// The launcher takes boxes for launches that leave resident CTA slots idle and rows otherwise, which
// is where each measured faster.  The table entry of a group is loaded one iteration before its copies
// are issued and not touched until then, so the table read is never waited for.  Slots come from the
// slot table in the kernel, so there is no gather-index buffer and no gathered K/V copy as in the
// reference (src/bridge/attention_plan.cpp:246-255, src/bridge/paged_attention.cpp:89-100).
#include "tc_common.cuh"

#include <string.h>

#include <math_constants.h>

#include <mutex>

namespace gk {
namespace {

constexpr int kGroupTokens = 16;   // tokens one warp consumes per pipeline stage
constexpr float kLog2e = 1.4426950408889634f;

struct AttnParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* pool_k;
  const __nv_bfloat16* pool_v;
  const int32_t* table;
  const int32_t* table_rows;
  const int32_t* work;
  __nv_bfloat16* out[GK_MAX_OUTPUTS];   // every destination receives the same rows (peers under TP)
  float* part_ml;
  float* part_o;
  int32_t* status;
  int32_t* counters;                     // optional: per (first_row, kv_head) arrival counts for the fused combine
  // optional fused KV store: the step's new K/V rows and their slots.  A CTA first writes the rows whose
  // positions lie in its own KV range to the pool, then reads them back like any other token.
  const __nv_bfloat16* new_k;
  const __nv_bfloat16* new_v;
  const int32_t* locations;
  int64_t new_k_stride, new_v_stride;
  int64_t q_stride, out_stride, slots, table_stride, entry_stride;
  int64_t part_capacity;                 // entries part_ml / part_o hold; a record that points past it is skipped
  float scale, softcap;
  int window, page_shift, q_heads, kv_heads, group, n_out;
};

template <int D, int WARPS, int STAGES>
struct AttnConfig {
  static constexpr int kRowBytes = D * 2;
  static constexpr int kChunks = D / 8;                         // 16-byte chunks per row
  static constexpr int kTileBytes = kGroupTokens * kRowBytes;   // K (or V) of one group: D/64 panels
  static constexpr int kStageBytes = 2 * kTileBytes;
  static constexpr int kWarpBytes = STAGES * kStageBytes;
  static constexpr int kRingBytes = WARPS * kWarpBytes;
  static constexpr int kSmemBytes = kRingBytes + 128;           // + one mbarrier per warp and stage, the abort flag
  static_assert(WARPS * STAGES * 8 + 4 <= 128, "barrier area");
  static constexpr int kMergeStride = D + 8;                    // floats per merged row
  static_assert(STAGES >= 3, "the merge buffers reuse the ring and need three stages of room");
  static_assert(kWarpBytes >= (GK_MAX_PACKED_ROWS * kMergeStride + 2 * GK_MAX_PACKED_ROWS) * 4, "merge area");
};

// Byte offset of 16-byte chunk `chunk` of token `row` in a staged K or V tile: panels of 64 columns,
// rows 128 bytes apart, chunks exchanged by the 128-byte swizzle (what a TMA box writes; conflict-free
// for ldmatrix).
__device__ __forceinline__ uint32_t group_off(int row, int chunk) {
  return (chunk >> 3) * (kGroupTokens * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
}

template <int D, int WARPS, int STAGES, bool TMA>
__global__ void __launch_bounds__(WARPS * 32, 2) paged_attn_kernel(const AttnParams p,
                                                                   const __grid_constant__ CUtensorMap map_kv) {
  using C = AttnConfig<D, WARPS, STAGES>;
  extern __shared__ __align__(1024) uint8_t smem[];     // swizzle atoms of the TMA boxes are 1 KiB
  wait_for_predecessor();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int item = blockIdx.x / p.kv_heads, head = blockIdx.x - item * p.kv_heads;

  const int4 w0 = __ldg(reinterpret_cast<const int4*>(p.work) + 2 * item);
  const int4 w1 = __ldg(reinterpret_cast<const int4*>(p.work) + 2 * item + 1);
  const int first_row = w0.x, n_rows = w0.y, first_pos = w0.z, table_row = w0.w;
  const int kv_begin = w1.x, kv_end = w1.y, partial_base = w1.z;
  const int n_splits = w1.w & 0xffff, split_index = (w1.w >> 16) & 0x7fff;
  const int G = p.group;
  const int mv = n_rows * G;                                    // packed rows in use (<= 16)

  // ---- Q fragments (A operand of S = Q K^T), rows g and g+8 of the packed tile ----------
  uint32_t qf[D / 16][4];
  int lim0 = 0x7fffffff, lim1 = 0x7fffffff;                     // last visible key per row
  {
    const unsigned short* q0 = nullptr;
    const unsigned short* q1 = nullptr;
    if (g < mv) {
      const int r = g / G, gq = g - r * G;
      lim0 = first_pos + r;
      q0 = reinterpret_cast<const unsigned short*>(p.q) + (int64_t)(first_row + r) * p.q_stride +
           (int64_t)(head * G + gq) * D;
    }
    if (g + 8 < mv) {
      const int r = (g + 8) / G, gq = g + 8 - r * G;
      lim1 = first_pos + r;
      q1 = reinterpret_cast<const unsigned short*>(p.q) + (int64_t)(first_row + r) * p.q_stride +
           (int64_t)(head * G + gq) * D;
    }
    // two consecutive bf16 of a query row: one 32-bit load when the row is 4-byte aligned (col is even), else
    // two 16-bit loads (the reference's one-element-offset views are only 2-byte aligned)
    auto pair = [](const unsigned short* base, int col) -> uint32_t {
      if (base == nullptr) return 0u;
      if ((reinterpret_cast<uintptr_t>(base) & 3) == 0) return __ldg(reinterpret_cast<const uint32_t*>(base + col));
      return (uint32_t)__ldg(base + col) | ((uint32_t)__ldg(base + col + 1) << 16);
    };
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      qf[ks][0] = pair(q0, ks * 16 + 2 * t);
      qf[ks][1] = pair(q1, ks * 16 + 2 * t);
      qf[ks][2] = pair(q0, ks * 16 + 8 + 2 * t);
      qf[ks][3] = pair(q1, ks * 16 + 8 + 2 * t);
    }
  }

  const int n_groups = (kv_end - kv_begin + kGroupTokens - 1) / kGroupTokens;
  const int my_groups = n_groups > warp ? (n_groups - warp + WARPS - 1) / WARPS : 0;
  const uint32_t ring = smem_u32(smem) + warp * C::kWarpBytes;
  const __nv_bfloat16* kbase = p.pool_k + (int64_t)head * p.slots * D;
  const __nv_bfloat16* vbase = p.pool_v + (int64_t)head * p.slots * D;

  // ---- fused head-major KV store (gk_kv_store_head_major_bf16_v1 inside the attention launch, as the
  // reference's single-block recipe does, src/bridge/paged_attention.cpp:74) ----------------------------
  // Only offered for steps in which every sequence is one query block, so no other CTA reads these rows:
  // the KV ranges of a block's splits partition its positions and each CTA stores exactly the new rows it
  // will read.  Bytes are copied unchanged, 16 at a time.
  if (p.new_k != nullptr) {
    const int r_lo = max(0, kv_begin - first_pos), r_hi = min(n_rows, kv_end - first_pos);
    if (r_lo < r_hi) {
      const int per_kind = (r_hi - r_lo) * C::kChunks;
      for (int idx = threadIdx.x; idx < 2 * per_kind; idx += WARPS * 32) {
        const int kind = idx >= per_kind, rem = idx - kind * per_kind;
        const int row = first_row + r_lo + rem / C::kChunks, col = rem % C::kChunks;
        const int slot = __ldg(p.locations + row);
        if ((unsigned)slot < (unsigned)p.slots) {
          const __nv_bfloat16* src = (kind ? p.new_v + (int64_t)row * p.new_v_stride : p.new_k + (int64_t)row * p.new_k_stride) +
                                     (int64_t)head * D + col * 8;
          __nv_bfloat16* dst = const_cast<__nv_bfloat16*>(kind ? vbase : kbase) + (int64_t)slot * D + col * 8;
          *reinterpret_cast<uint4*>(dst) = __ldg(reinterpret_cast<const uint4*>(src));
        } else if (col == 0 && kind == 0 && p.status) {
          atomicOr(p.status, (int)GK_DEV_BAD_SLOT);
        }
      }
      asm volatile("fence.proxy.async;\n" ::: "memory");   // the rows may come back through a TMA box
      __threadfence_block();
      __syncthreads();                                  // uniform per CTA: the range is the CTA's
    }
  }
  const int32_t* trow =
      p.table + (int64_t)(p.table_rows ? __ldg(p.table_rows + table_row) : table_row) * p.table_stride;
  const int page_mask = (1 << p.page_shift) - 1;

  // TMA form: one mbarrier per ring stage, private to the warp, one arrival per fill.
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kRingBytes) + warp * STAGES;
  int* abort_flag = reinterpret_cast<int*>(smem + C::kRingBytes + WARPS * STAGES * 8);
  if (TMA) {
    if (lane == 0) {
#pragma unroll
      for (int s = 0; s < STAGES; ++s) bar_init(&bars[s], 1);
      if (warp == 0) *abort_flag = 0;
      asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();
  }
  const int head_row = head * (int)p.slots;
  const bool swizzle_ok = (smem_u32(smem) & 1023) == 0;     // a box lands where group_off expects it

  // Table entry of this lane's token (lanes 0..15 and 16..31 alike) of the warp's local group `local`.
  // The loaded value is not touched here -- not even by an add, which would wait for the load: it is
  // issued one iteration before stage_group turns it into a slot.
  auto lookup = [&](int local) -> int {
    const int tok = kv_begin + (warp + local * WARPS) * kGroupTokens + (lane & 15);
    const int32_t* entry = trow + (int64_t)(tok >> p.page_shift) * p.entry_stride;
    int raw;
    asm volatile("{\n.reg .pred p;\nsetp.ne.s32 p, %2, 0;\nmov.s32 %0, 0;\n@p ld.global.nc.s32 %0, [%1];\n}\n"
                 : "=&r"(raw)
                 : "l"(entry), "r"((int)(local < my_groups && tok < kv_end)));
    return raw;
  };
  // Asynchronously stage the K and V rows of the warp's local group `local` into ring stage `stage`;
  // `raw` is lookup(local).  Rows past the range are zero-filled so that a masked probability of 0 never
  // multiplies stale shared memory.  TMA form: a whole group inside one page is ONE box issued by lane 0
  // (completion by transaction bytes); the rare other group (a ragged end, a range that does not start on
  // a 16-token boundary) is copied row by row and waited for on the spot.  Plain form: row by row, one
  // cp.async group per call (committed by the caller).
  auto stage_group = [&](int local, int stage, int raw) {
    const int tok0 = kv_begin + (warp + local * WARPS) * kGroupTokens;
    const int tok = tok0 + (lane & 15);
    int slot = tok < kv_end ? raw + (tok & page_mask) : -1;
    if (slot != -1 && (unsigned)slot >= (unsigned)p.slots) {         // a table entry outside the pool
      if (p.status) atomicOr(p.status, (int)GK_DEV_BAD_TABLE);
      slot = -1;
    }
    const uint32_t dst_k = ring + stage * C::kStageBytes, dst_v = dst_k + C::kTileBytes;
    if (TMA) {
      const int slot0 = __shfl_sync(0xffffffffu, slot, 0);
      const bool boxed = swizzle_ok && (tok0 & (kGroupTokens - 1)) == 0 && tok0 + kGroupTokens <= kv_end && slot0 >= 0 &&
                         (int64_t)slot0 + kGroupTokens <= p.slots;
      if (boxed) {
        if (lane == 0) {                              // K and V, all panels: one box (see make_kv_group_map)
          bar_arrive_expect_tx(&bars[stage], 2 * C::kTileBytes);
          tma_load_kv_group(dst_k, &map_kv, head_row + slot0, &bars[stage]);
        }
        return;
      }
    }
#pragma unroll
    for (int j = 0; j < kGroupTokens * C::kChunks / 32; ++j) {
      const int c = j * 32 + lane;
      const int row = c / C::kChunks, col = c % C::kChunks;
      const int s = __shfl_sync(0xffffffffu, slot, row);
      const int64_t src = (int64_t)(s < 0 ? 0 : s) * D + col * 8;
      const int bytes = s < 0 ? 0 : 16;
      const uint32_t off = group_off(row, col);
      cp_async_16(dst_k + off, kbase + src, bytes);
      cp_async_16(dst_v + off, vbase + src, bytes);
    }
    if (TMA) {
      asm volatile("cp.async.wait_all;\n" ::: "memory");   // these copies belong to no committed group
      __syncwarp();
      if (lane == 0) bar_arrive(&bars[stage]);
    }
  };

  float o[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;

  const bool capped = p.softcap > 0.f;
  const float to_log2 = capped ? kLog2e : p.scale * kLog2e;
  const bool upper = mv > 8;

  int raw_next;
  {
    int first[STAGES - 1];
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) first[s] = lookup(s);
    raw_next = lookup(STAGES - 1);
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
      if (s < my_groups) stage_group(s, s, first[s]);
      if (!TMA) cp_async_commit();
    }
  }

  bool alive = true;
  int stage = 0, fill = STAGES - 1;                    // ring positions of group i and of group i + STAGES - 1
  uint32_t parity = 0;
  for (int i = 0; i < my_groups; ++i) {
    if (!TMA) cp_async_wait<STAGES - 2>();
    // the stage about to be refilled is the one group i - 1 was read from: those reads are complete
    // (their consumers have been issued) once every lane is here
    __syncwarp();
    if (i + STAGES - 1 < my_groups) stage_group(i + STAGES - 1, fill, raw_next);
    if (!TMA) cp_async_commit();
    raw_next = lookup(i + STAGES);
    if (++fill == STAGES) fill = 0;
    if (TMA) {
      // usually the box has landed: one try, one vote; the bounded wait only otherwise
      uint32_t landed;
      asm volatile("{\n.reg .pred P1;\nmbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\nselp.b32 %0, 1, 0, P1;\n}\n"
                   : "=r"(landed)
                   : "r"(smem_u32(&bars[stage])), "r"(parity)
                   : "memory");
      if (!__all_sync(0xffffffffu, landed)) {
        alive = __all_sync(0xffffffffu, bar_wait(&bars[stage], parity, abort_flag));
        if (!alive) break;
      }
    }
    const uint32_t ks_base = ring + stage * C::kStageBytes, vs_base = ks_base + C::kTileBytes;

    // ---- S = Q K^T for 16 keys: two n-tiles of 8 keys -----------------------------------
    float sc[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
#pragma unroll
    for (int kp = 0; kp < D / 32; ++kp) {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const int row = nt * 8 + (lane & 7), chunk = kp * 4 + (lane >> 3);
        uint32_t b[4];
        ldmatrix_x4(b, ks_base + group_off(row, chunk));
        mma_bf16_16816(sc[nt], qf[2 * kp], b[0], b[1]);
        mma_bf16_16816(sc[nt], qf[2 * kp + 1], b[2], b[3]);
      }
    }

    // ---- scale, softcap, mask -----------------------------------------------------------
    const int tok0 = kv_begin + (warp + i * WARPS) * kGroupTokens;
    if (capped) {
      const float inv = p.scale / p.softcap;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) sc[nt][e] = p.softcap * tanhf(sc[nt][e] * inv);
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) sc[nt][e] *= to_log2;
    const bool ragged = tok0 + kGroupTokens > kv_end || tok0 + kGroupTokens > first_pos + 1 ||
                        (p.window > 0 && tok0 <= first_pos + n_rows - 1 - p.window);
    if (ragged) {
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int tok = tok0 + nt * 8 + 2 * t + (e & 1);
          const int lim = e < 2 ? lim0 : lim1;
          const bool seen = tok < kv_end && tok <= lim && (p.window <= 0 || tok > lim - p.window);
          if (!seen) sc[nt][e] = -CUDART_INF_F;
        }
    }

    // ---- online softmax: rows g (lower) and g+8 (upper) ---------------------------------
    float mx0 = fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1]));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    const float mn0 = fmaxf(m0, mx0);
    const float mu0 = mn0 == -CUDART_INF_F ? 0.f : mn0;
    const float a0 = fast_exp2(m0 - mu0);
    m0 = mn0;
    float pr[2][4];
    pr[0][0] = fast_exp2(sc[0][0] - mu0);
    pr[0][1] = fast_exp2(sc[0][1] - mu0);
    pr[1][0] = fast_exp2(sc[1][0] - mu0);
    pr[1][1] = fast_exp2(sc[1][1] - mu0);
    l0 = l0 * a0 + ((pr[0][0] + pr[0][1]) + (pr[1][0] + pr[1][1]));
    float a1 = 1.f;
    pr[0][2] = pr[0][3] = pr[1][2] = pr[1][3] = 0.f;
    if (upper) {
      float mx1 = fmaxf(fmaxf(sc[0][2], sc[0][3]), fmaxf(sc[1][2], sc[1][3]));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn1 = fmaxf(m1, mx1);
      const float mu1 = mn1 == -CUDART_INF_F ? 0.f : mn1;
      a1 = fast_exp2(m1 - mu1);
      m1 = mn1;
      pr[0][2] = fast_exp2(sc[0][2] - mu1);
      pr[0][3] = fast_exp2(sc[0][3] - mu1);
      pr[1][2] = fast_exp2(sc[1][2] - mu1);
      pr[1][3] = fast_exp2(sc[1][3] - mu1);
      l1 = l1 * a1 + ((pr[0][2] + pr[0][3]) + (pr[1][2] + pr[1][3]));
    }
    if (__any_sync(0xffffffffu, a0 != 1.f || a1 != 1.f)) {       // the running maxima seldom move: skip the no-op
#pragma unroll
      for (int n = 0; n < D / 8; ++n) {
        o[n][0] *= a0;
        o[n][1] *= a0;
        o[n][2] *= a1;
        o[n][3] *= a1;
      }
    }

    // ---- O += P V, P rounded to bf16 (the reference's boundary before the second product) --
    uint32_t pa[4];
    pa[0] = pack_bf16(pr[0][0], pr[0][1]);
    pa[1] = pack_bf16(pr[0][2], pr[0][3]);
    pa[2] = pack_bf16(pr[1][0], pr[1][1]);
    pa[3] = pack_bf16(pr[1][2], pr[1][3]);
#pragma unroll
    for (int np = 0; np < D / 16; ++np) {
      const int row = ((lane >> 3) & 1) * 8 + (lane & 7), chunk = np * 2 + (lane >> 4);
      uint32_t b[4];
      ldmatrix_x4_trans(b, vs_base + group_off(row, chunk));
      mma_bf16_16816(o[2 * np], pa, b[0], b[1]);
      mma_bf16_16816(o[2 * np + 1], pa, b[2], b[3]);
    }
    if (++stage == STAGES) {
      stage = 0;
      parity ^= 1u;
    }
  }
  asm volatile("cp.async.wait_all;\n" ::: "memory");
  if (!alive && lane == 0 && p.status) atomicOr(p.status, (int)GK_DEV_WAIT_EXPIRED);

  // ---- merge the warps' partial states through the (now idle) rings ----------------------
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  __syncwarp();
  {
    float* wo = reinterpret_cast<float*>(smem + warp * C::kWarpBytes);
    float* wml = wo + GK_MAX_PACKED_ROWS * C::kMergeStride;
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      *reinterpret_cast<float2*>(wo + g * C::kMergeStride + n * 8 + 2 * t) = make_float2(o[n][0], o[n][1]);
      *reinterpret_cast<float2*>(wo + (g + 8) * C::kMergeStride + n * 8 + 2 * t) = make_float2(o[n][2], o[n][3]);
    }
    if (t == 0) {
      wml[2 * g] = m0;
      wml[2 * g + 1] = l0;
      wml[2 * (g + 8)] = m1;
      wml[2 * (g + 8) + 1] = l1;
    }
  }
  __syncthreads();

  for (int idx = threadIdx.x; idx < mv * (D / 4); idx += WARPS * 32) {
    const int prow = idx / (D / 4), c4 = idx - prow * (D / 4);
    float mstar = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float* wml = reinterpret_cast<const float*>(smem + w * C::kWarpBytes) + GK_MAX_PACKED_ROWS * C::kMergeStride;
      if (wml[2 * prow + 1] > 0.f) mstar = fmaxf(mstar, wml[2 * prow]);
    }
    float lsum = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float* wo = reinterpret_cast<const float*>(smem + w * C::kWarpBytes);
      const float* wml = wo + GK_MAX_PACKED_ROWS * C::kMergeStride;
      const float lw = wml[2 * prow + 1];
      if (lw > 0.f) {
        const float wgt = fast_exp2(wml[2 * prow] - mstar);
        const float4 v = *reinterpret_cast<const float4*>(wo + prow * C::kMergeStride + c4 * 4);
        lsum += wgt * lw;
        acc.x += wgt * v.x;
        acc.y += wgt * v.y;
        acc.z += wgt * v.z;
        acc.w += wgt * v.w;
      }
    }
    const int r = prow / G, gq = prow - r * G;
    if (partial_base < 0) {
      const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
      uint2 packed;
      packed.x = pack_bf16(acc.x * inv, acc.y * inv);
      packed.y = pack_bf16(acc.z * inv, acc.w * inv);
      const int64_t at = (int64_t)(first_row + r) * p.out_stride + (int64_t)(head * G + gq) * D + c4 * 4;
      for (int dst = 0; dst < p.n_out; ++dst) *reinterpret_cast<uint2*>(p.out[dst] + at) = packed;
    } else {
      const int64_t entry = (int64_t)partial_base + (int64_t)r * p.q_heads + head * G + gq;
      if (entry < p.part_capacity) {
        *reinterpret_cast<float4*>(p.part_o + entry * D + c4 * 4) = acc;
        if (c4 == 0) *reinterpret_cast<float2*>(p.part_ml + entry * 2) = make_float2(mstar, lsum);
      } else if (c4 == 0 && p.status) {
        atomicOr(p.status, (int)GK_DEV_BAD_SLOT);      // the record disagrees with the declared split state
      }
    }
  }

  // ---- fused combine: the CTA that completes a block's last split merges all of them ---------
  // Arrival order decides only WHO merges; the merge itself runs over the splits in split order, so
  // the result does not depend on scheduling.  The counter returns to zero for the next launch.
  if (partial_base >= 0 && p.counters != nullptr) {
    __shared__ int is_last;
    __threadfence();                                   // this CTA's split state before its arrival
    __syncthreads();
    if (threadIdx.x == 0) {
      int* counter = p.counters + (int64_t)first_row * p.kv_heads + head;
      const int seen = atomicAdd(counter, 1);
      is_last = seen == n_splits - 1;
      if (is_last) *counter = 0;
    }
    __syncthreads();
    if (is_last) {
      __threadfence();                                 // the other CTAs' split state after their arrivals
      const int stride = n_rows * p.q_heads;           // entries per split
      const int64_t base = (int64_t)partial_base - (int64_t)split_index * stride;
      for (int idx = threadIdx.x; idx < mv * (D / 4); idx += WARPS * 32) {
        const int prow = idx / (D / 4), c4 = idx - prow * (D / 4);
        const int r = prow / G, gq = prow - r * G;
        const int64_t e0 = base + (int64_t)r * p.q_heads + head * G + gq;
        if (e0 < 0 || e0 + (int64_t)(n_splits - 1) * stride >= p.part_capacity) continue;   // flagged by the writer
        float mstar = -CUDART_INF_F;
        for (int s = 0; s < n_splits; ++s) {
          const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml) + e0 + (int64_t)s * stride);
          if (ml.y > 0.f) mstar = fmaxf(mstar, ml.x);
        }
        float lsum = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
        for (int s = 0; s < n_splits; ++s) {
          const int64_t entry = e0 + (int64_t)s * stride;
          const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml) + entry);
          const float4 v = __ldcg(reinterpret_cast<const float4*>(p.part_o + entry * D) + c4);
          const float wgt = ml.y > 0.f ? fast_exp2(ml.x - mstar) : 0.f;
          lsum += wgt * ml.y;
          acc.x += wgt * v.x;
          acc.y += wgt * v.y;
          acc.z += wgt * v.z;
          acc.w += wgt * v.w;
        }
        const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
        uint2 packed;
        packed.x = pack_bf16(acc.x * inv, acc.y * inv);
        packed.y = pack_bf16(acc.z * inv, acc.w * inv);
        const int64_t at = (int64_t)(first_row + r) * p.out_stride + (int64_t)(head * G + gq) * D + c4 * 4;
        for (int dst = 0; dst < p.n_out; ++dst) *reinterpret_cast<uint2*>(p.out[dst] + at) = packed;
      }
    }
  }
}

struct OutputList {
  __nv_bfloat16* ptr[GK_MAX_OUTPUTS];
  int n;
};

// Merge the split states of each combine record in split order and write bf16(O / l).
// blockIdx.x = combine record, blockIdx.y = group of four query heads, one warp per
// (row, query head) entry; lanes stride over head_dim in float4 steps.
template <int D>
__global__ void __launch_bounds__(128) paged_attn_combine_kernel(const float* __restrict__ part_ml,
                                                                const float* __restrict__ part_o,
                                                                const int32_t* __restrict__ combine,
                                                                const OutputList outs, int64_t out_stride,
                                                                int q_heads, int64_t capacity, int32_t* status) {
  wait_for_predecessor();
  const int4 rec = __ldg(reinterpret_cast<const int4*>(combine) + blockIdx.x);
  const int first_row = rec.x, n_rows = rec.y, base = rec.z, n_splits = rec.w;
  const int entries = n_rows * q_heads;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // A record whose split state would lie outside the declared array is not read at all.
  if (base < 0 || n_splits <= 0 || n_rows <= 0 || (int64_t)base + (int64_t)n_splits * entries > capacity) {
    if (threadIdx.x == 0 && blockIdx.y == 0 && status) atomicOr(status, (int)GK_DEV_BAD_SLOT);
    return;
  }
  for (int e = blockIdx.y * 4 + warp; e < entries; e += gridDim.y * 4) {
    // (m, l) of up to 32 splits at a time, one per lane: the reference maximum and the weights come
    // from warp reductions, then the O rows (independent loads) are accumulated in split order.
    float mstar = -CUDART_INF_F;
    for (int s0 = 0; s0 < n_splits; s0 += 32) {
      const int sidx = s0 + lane;
      float2 ml = make_float2(-CUDART_INF_F, 0.f);
      if (sidx < n_splits) ml = __ldg(reinterpret_cast<const float2*>(part_ml) + (int64_t)base + (int64_t)sidx * entries + e);
      float mine = ml.y > 0.f ? ml.x : -CUDART_INF_F;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mine = fmaxf(mine, __shfl_xor_sync(0xffffffffu, mine, o));
      mstar = fmaxf(mstar, mine);
    }
    constexpr int kVec = D / 128 > 0 ? D / 128 : 1;              // float4 per lane
    float4 acc[kVec];
#pragma unroll
    for (int v = 0; v < kVec; ++v) acc[v] = make_float4(0.f, 0.f, 0.f, 0.f);
    float lsum = 0.f;
    const bool active = lane * 4 < D;
    for (int s0 = 0; s0 < n_splits; s0 += 32) {
      const int sidx = s0 + lane;
      float2 ml = make_float2(-CUDART_INF_F, 0.f);
      if (sidx < n_splits) ml = __ldg(reinterpret_cast<const float2*>(part_ml) + (int64_t)base + (int64_t)sidx * entries + e);
      const float wgt_mine = ml.y > 0.f ? fast_exp2(ml.x - mstar) : 0.f;
      float part = wgt_mine * ml.y;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
      lsum += part;
      const int n_here = n_splits - s0 < 32 ? n_splits - s0 : 32;
#pragma unroll 4
      for (int s = 0; s < n_here; ++s) {
        const float wgt = __shfl_sync(0xffffffffu, wgt_mine, s);
        if (active) {
          const int64_t entry = (int64_t)base + (int64_t)(s0 + s) * entries + e;
#pragma unroll
          for (int v = 0; v < kVec; ++v) {
            const float4 x = __ldg(reinterpret_cast<const float4*>(part_o + entry * D) + v * 32 + lane);
            acc[v].x += wgt * x.x;
            acc[v].y += wgt * x.y;
            acc[v].z += wgt * x.z;
            acc[v].w += wgt * x.w;
          }
        }
      }
    }
    const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
    const int r = e / q_heads, h = e - r * q_heads;
    if (active) {
#pragma unroll
      for (int v = 0; v < kVec; ++v) {
        uint2 packed;
        packed.x = pack_bf16(acc[v].x * inv, acc[v].y * inv);
        packed.y = pack_bf16(acc[v].z * inv, acc[v].w * inv);
        const int64_t at = (int64_t)(first_row + r) * out_stride + (int64_t)h * D + (v * 32 + lane) * 4;
        for (int dst = 0; dst < outs.n; ++dst) *reinterpret_cast<uint2*>(outs.ptr[dst] + at) = packed;
      }
    }
  }
}

constexpr int kWarps = 4;
constexpr int kStages = 3;

template <int D, bool TMA>
int launch_attn_form(const AttnParams& p, const CUtensorMap& map_kv, int64_t n_work, cudaStream_t stream) {
  using C = AttnConfig<D, kWarps, kStages>;
  auto kernel = paged_attn_kernel<D, kWarps, kStages, TMA>;
  static std::atomic<bool> configured[64];
  const int ready = opt_in_shared_memory(kernel, C::kSmemBytes, configured);
  if (ready != GK_OK) return ready;
  const int64_t blocks = n_work * p.kv_heads;
  launch_after_predecessor(kernel, dim3((unsigned)blocks), dim3(kWarps * 32), C::kSmemBytes, stream, p, map_kv);
  return check_launch();
}

std::atomic<int> attention_form{GK_ATTENTION_FORM_AUTO};

inline int sm_count_of_current_device() {
  static std::atomic<int> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

template <int D>
int launch_attn(const AttnParams& p, int64_t n_work, int page_tokens, cudaStream_t stream) {
  // One box per 16-token group needs pages of at least 16 slot-contiguous tokens, 32-bit row coordinates and
  // the V half at a positive 16-byte-aligned distance after the K half; without them (or without the driver's
  // encoder) the plain form copies every group row by row.
  alignas(64) CUtensorMap map_kv;
  memset(&map_kv, 0, sizeof(map_kv));
  const int64_t pool_rows = (int64_t)p.kv_heads * p.slots;
  const int64_t v_minus_k = reinterpret_cast<const char*>(p.pool_v) - reinterpret_cast<const char*>(p.pool_k);
  // Measured: the box form is 4 % faster per CTA while the grid leaves resident slots idle (the copies cost
  // one instruction instead of sixteen), the row form 1 % faster once the grid saturates the memory system.
  const int form = attention_form.load(std::memory_order_relaxed);
  const bool boxes = form == GK_ATTENTION_FORM_AUTO ? n_work * p.kv_heads <= 2 * sm_count_of_current_device()
                                                    : form == GK_ATTENTION_FORM_BOXES;
  const bool boxed = boxes && page_tokens >= kGroupTokens && pool_rows < 0x7fffffffLL &&
                     make_kv_group_map(&map_kv, p.pool_k, v_minus_k, pool_rows, kGroupTokens, D);
  return boxed ? launch_attn_form<D, true>(p, map_kv, n_work, stream) : launch_attn_form<D, false>(p, map_kv, n_work, stream);
}

// Argument checks + launch of the attention kernel.  `part_capacity` is the number of entries the
// split-state arrays hold (INT64_MAX when the caller sized them from the schedule itself).
int attn_entry(const void* q, int64_t q_row_stride, const void* pool_k, const void* pool_v, int64_t slots,
               const int32_t* table, int64_t table_stride, int64_t table_entry_stride, int page_tokens,
               const int32_t* table_rows, const int32_t* work, int64_t n_work, void* const* outs, int n_outs,
               int64_t out_row_stride, float* part_ml, float* part_o, int64_t part_capacity, int32_t* split_counters,
               float scale, float softcap, int window, int q_heads, int kv_heads, int head_dim, int32_t* status,
               gk_stream_t stream, const void* new_k = nullptr, const void* new_v = nullptr, int64_t new_k_stride = 0,
               int64_t new_v_stride = 0, const int32_t* locations = nullptr) {
  if (n_work == 0) return GK_OK;
  if (new_k || new_v || locations) {
    // the fused store moves whole 16-byte pieces
    if (!new_k || !new_v || !locations || new_k_stride < (int64_t)kv_heads * head_dim ||
        new_v_stride < (int64_t)kv_heads * head_dim)
      return GK_ERR_INVALID_ARGUMENT;
    if (((reinterpret_cast<uintptr_t>(new_k) | reinterpret_cast<uintptr_t>(new_v)) & 15) || (new_k_stride & 7) ||
        (new_v_stride & 7))
      return GK_ERR_UNSUPPORTED;
  }
  if (!outs || n_outs <= 0 || n_outs > GK_MAX_OUTPUTS) return GK_ERR_INVALID_ARGUMENT;
  for (int i = 0; i < n_outs; ++i)
    if (!outs[i] || (reinterpret_cast<uintptr_t>(outs[i]) & 7)) return GK_ERR_INVALID_ARGUMENT;
  if (!q || !pool_k || !pool_v || !table || !work || n_work < 0 || slots <= 0 || table_stride < 0 || table_entry_stride <= 0 ||
      page_tokens <= 0 || (page_tokens & (page_tokens - 1)) || q_heads <= 0 || kv_heads <= 0 ||
      !(scale > 0.f) || !(softcap >= 0.f) || (window != -1 && window <= 0))
    return GK_ERR_INVALID_ARGUMENT;
  if (q_heads % kv_heads != 0 || q_heads / kv_heads > GK_MAX_PACKED_ROWS ||
      (head_dim != 64 && head_dim != 128 && head_dim != 256))
    return GK_ERR_UNSUPPORTED;
  if (n_work * kv_heads > 0x7fffffffLL) return GK_ERR_UNSUPPORTED;
  // K/V rows are moved in 16-byte pieces and the result is stored 8 bytes at a time.
  if ((reinterpret_cast<uintptr_t>(pool_k) | reinterpret_cast<uintptr_t>(pool_v)) & 15) return GK_ERR_INVALID_ARGUMENT;
  if ((out_row_stride & 3) || (reinterpret_cast<uintptr_t>(work) & 15) || (reinterpret_cast<uintptr_t>(q) & 1))
    return GK_ERR_INVALID_ARGUMENT;
  if (part_ml && ((reinterpret_cast<uintptr_t>(part_ml) & 7) || (reinterpret_cast<uintptr_t>(part_o) & 15)))
    return GK_ERR_INVALID_ARGUMENT;
  AttnParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.pool_k = static_cast<const __nv_bfloat16*>(pool_k);
  p.pool_v = static_cast<const __nv_bfloat16*>(pool_v);
  p.table = table;
  p.table_rows = table_rows;
  p.entry_stride = table_entry_stride;
  p.work = work;
  for (int i = 0; i < n_outs; ++i) p.out[i] = static_cast<__nv_bfloat16*>(outs[i]);
  p.n_out = n_outs;
  p.part_ml = part_ml;
  p.part_o = part_o;
  p.status = status;
  p.counters = split_counters;
  p.part_capacity = part_ml ? part_capacity : 0;
  p.new_k = static_cast<const __nv_bfloat16*>(new_k);
  p.new_v = static_cast<const __nv_bfloat16*>(new_v);
  p.locations = locations;
  p.new_k_stride = new_k_stride;
  p.new_v_stride = new_v_stride;
  p.q_stride = q_row_stride;
  p.out_stride = out_row_stride;
  p.slots = slots;
  p.table_stride = table_stride;
  p.scale = scale;
  p.softcap = softcap;
  p.window = window;
  p.page_shift = __builtin_ctz((unsigned)page_tokens);
  p.q_heads = q_heads;
  p.kv_heads = kv_heads;
  p.group = q_heads / kv_heads;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  switch (head_dim) {
    case 64: return launch_attn<64>(p, n_work, page_tokens, s);
    case 128: return launch_attn<128>(p, n_work, page_tokens, s);
    default: return launch_attn<256>(p, n_work, page_tokens, s);
  }
}

}  // namespace
}  // namespace gk

extern "C" int gk_paged_attn_multi_bf16(const void* q, int64_t q_row_stride, const void* pool_k, const void* pool_v,
                                        int64_t slots, const int32_t* table, int64_t table_stride,
                                        int64_t table_entry_stride, int page_tokens, const int32_t* table_rows,
                                        const int32_t* work, int64_t n_work, void* const* outs, int n_outs,
                                        int64_t out_row_stride, float* part_ml, float* part_o,
                                        int32_t* split_counters, float scale, float softcap, int window, int q_heads,
                                        int kv_heads, int head_dim, int32_t* status, gk_stream_t stream) {
  return gk::attn_entry(q, q_row_stride, pool_k, pool_v, slots, table, table_stride, table_entry_stride, page_tokens,
                        table_rows, work, n_work, outs, n_outs, out_row_stride, part_ml, part_o, INT64_MAX,
                        split_counters, scale, softcap, window, q_heads, kv_heads, head_dim, status, stream);
}

extern "C" int gk_paged_attn_store_multi_bf16(const void* q, int64_t q_row_stride, const void* new_k, const void* new_v,
                                              int64_t new_k_row_stride, int64_t new_v_row_stride,
                                              const int32_t* locations, void* pool_k, void* pool_v, int64_t slots,
                                              const int32_t* table, int64_t table_stride, int64_t table_entry_stride,
                                              int page_tokens, const int32_t* table_rows, const int32_t* work,
                                              int64_t n_work, void* const* outs, int n_outs, int64_t out_row_stride,
                                              float* part_ml, float* part_o, int32_t* split_counters, float scale,
                                              float softcap, int window, int q_heads, int kv_heads, int head_dim,
                                              int32_t* status, gk_stream_t stream) {
  if (!new_k || !new_v || !locations) return GK_ERR_INVALID_ARGUMENT;
  return gk::attn_entry(q, q_row_stride, pool_k, pool_v, slots, table, table_stride, table_entry_stride, page_tokens,
                        table_rows, work, n_work, outs, n_outs, out_row_stride, part_ml, part_o, INT64_MAX,
                        split_counters, scale, softcap, window, q_heads, kv_heads, head_dim, status, stream, new_k, new_v,
                        new_k_row_stride, new_v_row_stride, locations);
}

extern "C" int gk_paged_attn_bf16(const void* q, int64_t q_row_stride, const void* pool_k, const void* pool_v,
                                  int64_t slots, const int32_t* table, int64_t table_stride,
                                  int64_t table_entry_stride, int page_tokens, const int32_t* table_rows,
                                  const int32_t* work, int64_t n_work, void* out, int64_t out_row_stride,
                                  float* part_ml, float* part_o, float scale, float softcap, int window,
                                  int q_heads, int kv_heads, int head_dim, int32_t* status, gk_stream_t stream) {
  void* const outs[1] = {out};
  return gk_paged_attn_multi_bf16(q, q_row_stride, pool_k, pool_v, slots, table, table_stride, table_entry_stride,
                                  page_tokens, table_rows, work, n_work, outs, 1, out_row_stride, part_ml, part_o, nullptr,
                                  scale, softcap, window, q_heads, kv_heads, head_dim, status, stream);
}

namespace gk {
namespace {
// Checks of the combine arguments alone, so that a caller can make them before launching anything.
int combine_check(const float* part_ml, const float* part_o, const int32_t* combine, int64_t n_combine,
                  void* const* outs, int n_outs, int64_t out_row_stride, int q_heads, int head_dim) {
  if (n_combine == 0) return GK_OK;
  if (!part_ml || !part_o || !combine || !outs || n_outs <= 0 || n_outs > GK_MAX_OUTPUTS || n_combine < 0 ||
      n_combine > 0x7fffffffLL || q_heads <= 0)
    return GK_ERR_INVALID_ARGUMENT;
  for (int i = 0; i < n_outs; ++i)
    if (!outs[i] || (reinterpret_cast<uintptr_t>(outs[i]) & 7)) return GK_ERR_INVALID_ARGUMENT;
  if ((out_row_stride & 3) || (reinterpret_cast<uintptr_t>(combine) & 15) ||
      (reinterpret_cast<uintptr_t>(part_ml) & 7) || (reinterpret_cast<uintptr_t>(part_o) & 15))
    return GK_ERR_INVALID_ARGUMENT;
  if (head_dim != 64 && head_dim != 128 && head_dim != 256) return GK_ERR_UNSUPPORTED;
  return GK_OK;
}

int combine_entry(const float* part_ml, const float* part_o, int64_t capacity, const int32_t* combine,
                  int64_t n_combine, void* const* outs, int n_outs, int64_t out_row_stride, int q_heads, int head_dim,
                  int32_t* status, gk_stream_t stream) {
  if (n_combine == 0) return GK_OK;
  const int checked = combine_check(part_ml, part_o, combine, n_combine, outs, n_outs, out_row_stride, q_heads, head_dim);
  if (checked != GK_OK) return checked;
  OutputList o{};
  o.n = n_outs;
  for (int i = 0; i < n_outs; ++i) o.ptr[i] = static_cast<__nv_bfloat16*>(outs[i]);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // Four entries per CTA; a decode record (one row) is covered in one pass, records with more
  // rows loop over them.
  const dim3 grid((unsigned)n_combine, (unsigned)((q_heads + 3) / 4));
  switch (head_dim) {
    case 64: launch_after_predecessor(paged_attn_combine_kernel<64>, grid, dim3(128), 0, s, part_ml, part_o, combine, o, out_row_stride, q_heads, capacity, status); break;
    case 128: launch_after_predecessor(paged_attn_combine_kernel<128>, grid, dim3(128), 0, s, part_ml, part_o, combine, o, out_row_stride, q_heads, capacity, status); break;
    default: launch_after_predecessor(paged_attn_combine_kernel<256>, grid, dim3(128), 0, s, part_ml, part_o, combine, o, out_row_stride, q_heads, capacity, status); break;
  }
  return check_launch();
}
}  // namespace
}  // namespace gk

extern "C" int gk_paged_attn_combine_multi_bf16(const float* part_ml, const float* part_o, const int32_t* combine,
                                                int64_t n_combine, void* const* outs, int n_outs,
                                                int64_t out_row_stride, int q_heads, int head_dim,
                                                gk_stream_t stream) {
  return gk::combine_entry(part_ml, part_o, INT64_MAX, combine, n_combine, outs, n_outs, out_row_stride, q_heads,
                           head_dim, nullptr, stream);
}

extern "C" int gk_paged_attn_combine_bf16(const float* part_ml, const float* part_o, const int32_t* combine,
                                          int64_t n_combine, void* out, int64_t out_row_stride, int q_heads,
                                          int head_dim, gk_stream_t stream) {
  void* const outs[1] = {out};
  return gk_paged_attn_combine_multi_bf16(part_ml, part_o, combine, n_combine, outs, 1, out_row_stride, q_heads,
                                          head_dim, stream);
}

// ---------------------------------------------------------------------------------------------
// Attention + combine for callers that cannot allocate device memory
// ---------------------------------------------------------------------------------------------
namespace gk {
namespace {
// Split state for gk_paged_attn_static_scratch_bf16: (m, l) pairs for every entry first, the
// O rows after them.  Lives in every GPU context that loads this library, until exit.
constexpr size_t kStaticMlFloats = (size_t)GK_STATIC_SCRATCH_MAX_ENTRIES * 2;
constexpr size_t kStaticFloats = kStaticMlFloats + (size_t)GK_STATIC_SCRATCH_MAX_ENTRIES * GK_STATIC_SCRATCH_MAX_HEAD_DIM;
static __device__ __align__(256) float g_static_scratch[kStaticFloats];

std::mutex g_static_mutex;
float* g_static_address[64] = {};   // device address of g_static_scratch, per device ordinal

// `g_static_scratch` names a host-side stand-in here, not device memory: the address a kernel may
// use has to be asked for, once per device, with that device current.
int static_scratch_address(float** out) {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return check_launch();
  if (device < 0 || device >= 64) return GK_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (!g_static_address[device]) {
    void* address = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&address, g_static_scratch);
    if (e != cudaSuccess || !address) {
      g_last_cuda_error = static_cast<int>(e);
      (void)cudaGetLastError();
      return GK_ERR_CUDA;
    }
    g_static_address[device] = static_cast<float*>(address);
  }
  *out = g_static_address[device];
  return GK_OK;
}
}  // namespace
}  // namespace gk

extern "C" int gk_paged_attn_static_scratch_bf16(const void* q, int64_t q_row_stride, const void* pool_k,
                                                 const void* pool_v, int64_t slots, const int32_t* table,
                                                 int64_t table_stride, int64_t table_entry_stride, int page_tokens,
                                                 const int32_t* table_rows, const int32_t* work, int64_t n_work,
                                                 const int32_t* combine, int64_t n_combine, int64_t partial_entries,
                                                 void* out, int64_t out_row_stride, float scale, float softcap,
                                                 int window, int q_heads, int kv_heads, int head_dim, int32_t* status,
                                                 gk_stream_t stream) {
  // Every argument is judged before the first launch, so a refused call leaves nothing half done.
  if (partial_entries < 0 || n_combine < 0 || n_work < 0) return GK_ERR_INVALID_ARGUMENT;
  // Split state and combine records come from one schedule: both present or both absent, and a
  // combine without this call's attention launch would merge what an earlier call left behind.
  if ((n_combine > 0) != (partial_entries > 0) || (n_combine > 0 && n_work == 0)) return GK_ERR_INVALID_ARGUMENT;
  if (partial_entries > GK_STATIC_SCRATCH_MAX_ENTRIES || head_dim > GK_STATIC_SCRATCH_MAX_HEAD_DIM) return GK_ERR_CAPACITY;
  float* base = nullptr;
  const int got = gk::static_scratch_address(&base);
  if (got != GK_OK) return got;
  float* part_ml = base;
  float* part_o = base + gk::kStaticMlFloats;
  void* const outs[1] = {out};
  const int checked = gk::combine_check(part_ml, part_o, combine, n_combine, outs, 1, out_row_stride, q_heads, head_dim);
  if (checked != GK_OK) return checked;
  // The kernels get the declared entry count: a work or combine record that points past it is
  // skipped and GK_DEV_BAD_SLOT is raised, so a schedule that disagrees with `partial_entries`
  // cannot write outside the array.
  const int rc = gk::attn_entry(q, q_row_stride, pool_k, pool_v, slots, table, table_stride, table_entry_stride,
                                page_tokens, table_rows, work, n_work, outs, 1, out_row_stride, part_ml, part_o,
                                partial_entries, nullptr, scale, softcap, window, q_heads, kv_heads, head_dim, status,
                                stream);
  if (rc != GK_OK) return rc;
  return gk::combine_entry(part_ml, part_o, partial_entries, combine, n_combine, outs, 1, out_row_stride, q_heads,
                           head_dim, status, stream);
}

extern "C" int gk_set_attention_form(int form) {
  if (form != GK_ATTENTION_FORM_AUTO && form != GK_ATTENTION_FORM_ROWS && form != GK_ATTENTION_FORM_BOXES)
    return GK_ERR_INVALID_ARGUMENT;
  gk::attention_form.store(form, std::memory_order_relaxed);
  return GK_OK;
}
