// Chunked-prefill paged attention on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// A work record here is a query tile of one sequence: up to 128/G consecutive rows whose G query
// heads of one KV head are packed into the 128 rows of a UMMA tile, against the KV range
// [kv_begin, kv_end) of the pool (prefix + the rows themselves, causal inside the chunk).
// Q.K^T (128 x 128 x d) and P.V (128 x d x 128) are real dense contractions, so they run as
// tcgen05.mma.kind::f16 with fp32 accumulators in tensor memory:
//
//   warps 0-7  softmax, two warpgroups: thread (wg, row) owns columns [64 wg, 64 wg + 64) of
//              packed row `row` (= TMEM lane).  It reads S with tcgen05.ld, the two halves of a
//              row exchange their maxima through shared memory, O is rescaled in TMEM only when
//              the running maximum moved by more than 2^8, P (bf16, the reference's rounding
//              point) goes to shared memory, and at the end O is normalised and written out
//   warps 8-11 loaders (8-9 for K, 10-11 for V) of a 128-token tile.  A tile made of whole,
//              slot-contiguous pages of >= 8 tokens is fetched by TMA: one elected thread issues
//              cp.async.bulk.tensor (2-D boxes of 64 columns x page rows, 128-byte swizzle, no
//              multicast) per page and panel, completion by transaction bytes on the mbarrier.
//              Any other tile (ragged tail, token-granular tables, window offsets) is gathered
//              row by row with 16-byte cp.async, completion by cp.async.mbarrier.arrive.  The
//              loaders never wait for their copies
//   warp 12    one thread issues the MMAs: S[j&1] = Q K_j^T, then O += P_{j-1} V_{j-1}, signalling
//              completion through tcgen05.commit -> mbarrier
//
// Shared-memory operand tiles are [128 rows x 128 bf16] as two panels of [128 x 64] with the
// 128-byte swizzle (16-byte chunk c of row r at chunk c ^ (r & 7)); the same bytes serve K as a
// K-major operand and V as an MN-major operand.  S and P are double-buffered, K and V have two
// stages each, so Q K_{j+1}^T and the loads run under softmax_j and P_j V_j under softmax_{j+1}.
// Every mbarrier wait is bounded: on expiry the CTA raises GK_DEV_WAIT_EXPIRED, drains its
// copies, frees its TMEM and returns.
#include "tc_common.cuh"

#include <string.h>
#include <math_constants.h>

namespace gk {
namespace {

constexpr int kTile = 128;             // packed query rows per CTA, KV tokens per tile, head_dim
constexpr int kPanelBytes = kTile * 128;
constexpr int kTileBytes = 2 * kPanelBytes;          // 32 KiB: one [128 x 128] bf16 operand
constexpr int kSoftmaxThreads = 256, kLoaderThreads = 64, kThreads = 512;   // loaders: 64 threads for K, 64 for V; 4 warpgroups
constexpr int kLaunchRegs = 128;     // what __launch_bounds__(512, 1) lets ptxas allocate per thread
constexpr int kSoftmaxRegs = 176, kOtherRegs = 80;
static_assert(kSoftmaxThreads * kSoftmaxRegs + (kThreads - kSoftmaxThreads) * kOtherRegs <= kThreads * kLaunchRegs,
              "register budgets exceed the pool the launch allocates");
constexpr float kLog2e = 1.4426950408889634f;

struct PrefillParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* pool_k;
  const __nv_bfloat16* pool_v;
  const int32_t* table;
  const int32_t* table_rows;
  const int32_t* work;
  __nv_bfloat16* out[GK_MAX_OUTPUTS];   // every destination receives the same rows (peers under TP)
  int32_t* status;
  int64_t q_stride, out_stride, slots, table_stride, entry_stride;
  float scale, softcap;
  int window, page_shift, q_heads, kv_heads, group;
  int tma_rows;          // rows of a TMA box (= page_tokens), 0 = TMA path off
  int n_out;
};

struct Shared {
  uint64_t k_full[2], v_full[2], s_full[2], p_full[2], pv_done[2], swap[3];   // swap: row-half exchanges
  uint32_t tmem_base;
  int abort;
  float exchange[2][2][kTile];     // [tile parity][warpgroup][row]: row maxima, finally row sums
};

__device__ __forceinline__ uint32_t tile_off(int r, int c) {
  return (c >> 3) * kPanelBytes + r * 128 + (((c & 7) ^ (r & 7)) << 4);
}

// kind::f16 instruction descriptor: fp32 accumulate, bf16 x bf16, M = 128, N = 128.
constexpr uint32_t kIdescQK = (1u << 4) | (1u << 7) | (1u << 10) | (16u << 17) | (8u << 24);   // A, B K-major
constexpr uint32_t kIdescPV = kIdescQK | (1u << 16);                                            // B (= V) MN-major

__global__ void __launch_bounds__(kThreads, 1) paged_prefill_tc_kernel(const PrefillParams p,
                                                                       const __grid_constant__ CUtensorMap map_k,
                                                                       const __grid_constant__ CUtensorMap map_v) {
  extern __shared__ __align__(1024) uint8_t tiles[];     // swizzle atoms need 1 KiB alignment
  uint8_t* s_q = tiles;
  uint8_t* s_p = tiles + kTileBytes;                     // two P buffers
  uint8_t* s_k = tiles + 3 * kTileBytes;                 // two K stages
  uint8_t* s_v = tiles + 5 * kTileBytes;                 // two V stages
  Shared* sh = reinterpret_cast<Shared*>(tiles + 7 * kTileBytes);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (smem_u32(tiles) & 1023) {                          // cannot build valid descriptors: report, leave
    if (tid == 0 && p.status) atomicOr(p.status, (int)GK_DEV_WAIT_EXPIRED);
    return;
  }
  const int item = blockIdx.x / p.kv_heads, head = blockIdx.x - item * p.kv_heads;
  const int4 w0 = __ldg(reinterpret_cast<const int4*>(p.work) + 2 * item);
  const int4 w1 = __ldg(reinterpret_cast<const int4*>(p.work) + 2 * item + 1);
  const int first_row = w0.x, n_rows = w0.y, first_pos = w0.z, table_row = w0.w;
  const int kv_begin = w1.x, kv_end = w1.y;
  const int G = p.group;
  const int mv = n_rows * G;                            // packed rows in use (<= 128)
  const int n_tiles = (kv_end - kv_begin + kTile - 1) / kTile;

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      bar_init(&sh->k_full[i], kLoaderThreads);
      bar_init(&sh->v_full[i], kLoaderThreads);
      bar_init(&sh->s_full[i], 1);
      bar_init(&sh->p_full[i], kSoftmaxThreads);
      bar_init(&sh->pv_done[i], 1);
    }
    for (int i = 0; i < 3; ++i) bar_init(&sh->swap[i], kSoftmaxThreads);
    sh->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&sh->tmem_base)), "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  // Q tile: packed row pr = (row pr / G, query head pr % G) of this KV head; unused rows are zero.
  for (int i = tid; i < kTile * 16; i += kThreads) {
    const int pr = i >> 4, c = i & 15;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (pr < mv) {
      const int r = pr / G, g = pr - r * G;
      const __nv_bfloat16* src = p.q + (int64_t)(first_row + r) * p.q_stride + (int64_t)(head * G + g) * kTile + c * 8;
      if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
        v = __ldg(reinterpret_cast<const uint4*>(src));
      } else {
        const unsigned short* s16 = reinterpret_cast<const unsigned short*>(src);
        unsigned short e[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) e[k] = __ldg(s16 + k);
        v = *reinterpret_cast<const uint4*>(e);
      }
    }
    *reinterpret_cast<uint4*>(s_q + tile_off(pr, c)) = v;
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_base;
  const uint32_t tmem_o = tmem + 256;

  // Registers move from the loader/MMA warpgroups (which need few) to the softmax warpgroups.
  // setmaxnreg.inc blocks until the CTA's register pool can satisfy it, and the pool is what the
  // launch allocated (kThreads x kLaunchRegs): the two budgets must fit in it or the softmax warps
  // would never start (checked at compile time and again on the host before every launch).
  if (warp < 8) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(kSoftmaxRegs));
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(kOtherRegs));
  }
  if (warp < 8) {
    // ================================ softmax ============================================
    const int wg = warp >> 2;                                    // which 64 columns of the row
    const int pr = tid & 127;                                    // packed row == TMEM lane
    const int lim = pr < mv ? first_pos + pr / G : 0x7fffffff;   // last visible key of this row
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const bool capped = p.softcap > 0.f;
    const float to_log2 = capped ? kLog2e : p.scale * kLog2e;
    const float cap_in = capped ? p.scale / p.softcap : 0.f;
    float m = -CUDART_INF_F, l = 0.f;                            // m: exponent reference of this row
    bool alive = true;
    for (int j = 0; j < n_tiles && alive; ++j) {
      const int st = j & 1;
      alive = __all_sync(0xffffffffu, bar_wait(&sh->s_full[st], (j >> 1) & 1, &sh->abort));
      if (!alive) break;
      tc_fence_after();
      const uint32_t s_addr = tmem + st * kTile + wg * 64 + lane_base;
      const int tok0 = kv_begin + j * kTile + wg * 64;
      float sc[64];
      {
        uint32_t r0[32], r1[32];
        tmem_ld32_nowait(s_addr, r0);
        tmem_ld32_nowait(s_addr + 32, r1);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          sc[e] = __uint_as_float(r0[e]);
          sc[32 + e] = __uint_as_float(r1[e]);
        }
      }
      const int tile_end = kv_begin + (j + 1) * kTile;
      const bool ragged = tile_end > kv_end || tile_end > first_pos + 1 ||
                          (p.window > 0 && kv_begin + j * kTile <= first_pos + n_rows - 1 - p.window);
      // After this block sc[] holds raw scores and `mult` the factor that takes them to log2
      // units; the uncommon cases (softcap, tiles that need masking) rewrite sc[] in place.
      float mult = to_log2;
      if (capped || ragged) {
#pragma unroll
        for (int e = 0; e < 64; ++e) {
          float v = sc[e];
          if (capped) v = p.softcap * tanhf(v * cap_in);
          v *= to_log2;
          const int tok = tok0 + e;
          const bool seen = tok < kv_end && tok <= lim && (p.window <= 0 || tok > lim - p.window);
          sc[e] = seen ? v : -CUDART_INF_F;
        }
        mult = 1.f;
      }
      float mx4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
      for (int e = 0; e < 64; e += 4) {
        mx4[0] = fmaxf(mx4[0], sc[e]);
        mx4[1] = fmaxf(mx4[1], sc[e + 1]);
        mx4[2] = fmaxf(mx4[2], sc[e + 2]);
        mx4[3] = fmaxf(mx4[3], sc[e + 3]);
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * mult;     // mult > 0
      // the two halves of a row meet through an mbarrier (a bounded wait, unlike bar.sync)
      sh->exchange[st][wg][pr] = mx;
      bar_arrive(&sh->swap[st]);
      alive = __all_sync(0xffffffffu, bar_wait(&sh->swap[st], (j >> 1) & 1, &sh->abort));
      if (!alive) break;
      mx = fmaxf(mx, sh->exchange[st][wg ^ 1][pr]);
      // The exponent reference only moves when the maximum grew by more than 2^8: P stays within
      // bf16/fp32 range and O needs rescaling (and the wait for the previous P.V) only then.
      float alpha = 1.f;
      if (mx > m + 8.f || m == -CUDART_INF_F) {
        if (mx > m) {
          alpha = fast_exp2(m - mx);                               // 0 on the first finite maximum
          m = mx;
        }
      }
      const float mu = m == -CUDART_INF_F ? 0.f : m;
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
        alive = __all_sync(0xffffffffu, bar_wait(&sh->pv_done[st ^ 1], ((j - 1) >> 1) & 1, &sh->abort));
        if (!alive) break;
        tc_fence_after();
#pragma unroll 1
        for (int cb = 0; cb < 2; ++cb) {
          uint32_t r[32];
          tmem_ld32(tmem_o + lane_base + wg * 64 + cb * 32, r);
#pragma unroll
          for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
          tmem_st32(tmem_o + lane_base + wg * 64 + cb * 32, r);
        }
        tc_fence_before();
      }
      if (j >= 2) {                                                // P[st] was last read by P.V of tile j-2
        alive = __all_sync(0xffffffffu, bar_wait(&sh->pv_done[st], ((j - 2) >> 1) & 1, &sh->abort));
        if (!alive) break;
      }
      // probabilities, rounded to bf16 for the second product; l from the fp32 values
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      uint8_t* p_tile = s_p + st * kTileBytes;
      const float neg_mu = -mu;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint32_t packed[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float a = fast_exp2(fmaf(sc[c * 8 + 2 * e], mult, neg_mu));
          const float b = fast_exp2(fmaf(sc[c * 8 + 2 * e + 1], mult, neg_mu));
          sum4[e] += a + b;
          packed[e] = pack_bf16(a, b);
        }
        *reinterpret_cast<uint4*>(p_tile + tile_off(pr, wg * 8 + c)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      }
      l = l * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
      fence_async_smem();
      tc_fence_before();
      bar_arrive(&sh->p_full[st]);
    }
    // epilogue: O / l -> bf16 rows of the output
    const int last = n_tiles - 1;
    if (alive) alive = __all_sync(0xffffffffu, bar_wait(&sh->pv_done[last & 1], (last >> 1) & 1, &sh->abort));
    sh->exchange[n_tiles & 1][wg][pr] = l;
    bar_arrive(&sh->swap[2]);
    if (alive) alive = __all_sync(0xffffffffu, bar_wait(&sh->swap[2], 0, &sh->abort));
    l += sh->exchange[n_tiles & 1][wg ^ 1][pr];
    if (alive) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const int r_q = pr / G, g = pr - r_q * G;
      const int64_t at = (int64_t)(first_row + r_q) * p.out_stride + (int64_t)(head * G + g) * kTile + wg * 64;
#pragma unroll 1
      for (int cb = 0; cb < 2; ++cb) {
        uint32_t r[32];
        tmem_ld32(tmem_o + lane_base + wg * 64 + cb * 32, r);
        if (pr < mv) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(r[c * 8 + 0]) * inv, __uint_as_float(r[c * 8 + 1]) * inv);
            v.y = pack_bf16(__uint_as_float(r[c * 8 + 2]) * inv, __uint_as_float(r[c * 8 + 3]) * inv);
            v.z = pack_bf16(__uint_as_float(r[c * 8 + 4]) * inv, __uint_as_float(r[c * 8 + 5]) * inv);
            v.w = pack_bf16(__uint_as_float(r[c * 8 + 6]) * inv, __uint_as_float(r[c * 8 + 7]) * inv);
            for (int dst = 0; dst < p.n_out; ++dst) *reinterpret_cast<uint4*>(p.out[dst] + at + cb * 32 + c * 8) = v;
          }
        }
      }
    }
  } else if (warp < 12) {
    // ================================ K/V loaders =========================================
    const bool is_v = warp >= 10;
    const int lwarp = (warp - 8) & 1;
    const __nv_bfloat16* kbase = p.pool_k + (int64_t)head * p.slots * kTile;
    const __nv_bfloat16* vbase = p.pool_v + (int64_t)head * p.slots * kTile;
    const int32_t* trow = p.table + (int64_t)(p.table_rows ? __ldg(p.table_rows + table_row) : table_row) * p.table_stride;
    const int page_mask = (1 << p.page_shift) - 1;
    bool alive = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int st = j & 1;
      // each loader warp stages 64 rows, 32 at a time: lanes resolve one slot each, then the
      // warp copies two 256-byte rows per instruction (16 lanes x 16 bytes each)
      int slot[2];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int tok = kv_begin + j * kTile + lwarp * 64 + half * 32 + lane;
        slot[half] = -1;
        if (tok < kv_end) {
          slot[half] = __ldg(trow + (int64_t)(tok >> p.page_shift) * p.entry_stride) + (tok & page_mask);
          if ((unsigned)slot[half] >= (unsigned)p.slots) {
            if (p.status) atomicOr(p.status, (int)GK_DEV_BAD_TABLE);
            slot[half] = -1;
          }
        }
      }
      auto stage_rows = [&](const __nv_bfloat16* base, uint32_t dst) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
#pragma unroll 4
          for (int i = 0; i < 16; ++i) {
            const int rr = 2 * i + (lane >> 4), c = lane & 15;
            const int s = __shfl_sync(0xffffffffu, slot[half], rr);
            cp_async_16(dst + tile_off(lwarp * 64 + half * 32 + rr, c), base + (int64_t)(s < 0 ? 0 : s) * kTile + c * 8,
                        s < 0 ? 0 : 16);
          }
        }
      };
      // This warp's 64 rows go by TMA when they are whole, in-range boxes of tma_rows slot-contiguous
      // tokens; the two warps of a tile decide independently (every thread arrives once either way).
      const int tok_first = kv_begin + j * kTile + lwarp * 64;
      bool by_tma = p.tma_rows > 0 && (tok_first & (p.tma_rows - 1)) == 0 && tok_first + 64 <= kv_end;
      by_tma = __all_sync(0xffffffffu, by_tma && slot[0] >= 0 && slot[1] >= 0);
      uint64_t* full = is_v ? &sh->v_full[st] : &sh->k_full[st];
      if (j >= 2) {   // stage free: K once Q.K^T of tile j-2 completed, V once P.V of tile j-2 completed
        uint64_t* freed = is_v ? &sh->pv_done[st] : &sh->s_full[st];
        alive = __all_sync(0xffffffffu, bar_wait_patient(freed, ((j - 2) >> 1) & 1, &sh->abort));
        if (!alive) break;
      }
      const uint32_t dst = smem_u32(is_v ? s_v : s_k) + st * kTileBytes;
      if (by_tma) {
        const CUtensorMap* map = is_v ? &map_v : &map_k;
        const int head_row = head * (int)p.slots;
        if (lane == 0) bar_arrive_expect_tx(full, 64 * 256);
        else bar_arrive(full);
        __syncwarp();
        // the lane that holds the first row of a box issues its two panels
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int row = half * 32 + lane;                       // row within this warp's 64
          if ((row & (p.tma_rows - 1)) == 0) {
            const uint32_t at = dst + (lwarp * 64 + row) * 128;
            tma_load_box(at, map, 0, head_row + slot[half], full);
            tma_load_box(at + kPanelBytes, map, 64, head_row + slot[half], full);
          }
        }
      } else {
        stage_rows(is_v ? vbase : kbase, dst);
        bar_arrive_on_copies(full);
      }
    }
    asm volatile("cp.async.wait_all;\n" ::: "memory");
  } else if (warp == 12 && lane == 0) {
    // ================================ MMA issue ===========================================
    const uint32_t q_addr = smem_u32(s_q), p_addr = smem_u32(s_p), k_base = smem_u32(s_k), v_base = smem_u32(s_v);
    bool alive = true;
    auto issue_pv = [&](int i) {
      const int st = i & 1;
      if (!bar_wait(&sh->p_full[st], (i >> 1) & 1, &sh->abort)) return false;
      if (!bar_wait(&sh->v_full[st], (i >> 1) & 1, &sh->abort)) return false;
      fence_async_smem();
      tc_fence_after();
      const uint32_t v_addr = v_base + st * kTileBytes, pa = p_addr + st * kTileBytes;
#pragma unroll
      for (int k = 0; k < 8; ++k) {                    // 16 tokens per step
        const uint64_t da = umma_desc(pa + (k >> 2) * kPanelBytes + (k & 3) * 32, 16, 1024);
        const uint64_t db = umma_desc(v_addr + k * 2048, kPanelBytes, 1024);
        umma_bf16(tmem_o, da, db, kIdescPV, (i > 0 || k > 0) ? 1u : 0u);
      }
      umma_commit(&sh->pv_done[st]);
      return true;
    };
    for (int j = 0; j < n_tiles && alive; ++j) {
      const int st = j & 1;
      alive = bar_wait(&sh->k_full[st], (j >> 1) & 1, &sh->abort);
      if (!alive) break;
      fence_async_smem();
      tc_fence_after();
      const uint32_t k_addr = k_base + st * kTileBytes;
#pragma unroll
      for (int k = 0; k < 8; ++k) {                    // 16 elements of head_dim per step
        const uint32_t koff = (k >> 2) * kPanelBytes + (k & 3) * 32;
        umma_bf16(tmem + st * kTile, umma_desc(q_addr + koff, 16, 1024), umma_desc(k_addr + koff, 16, 1024), kIdescQK,
                  k > 0 ? 1u : 0u);
      }
      umma_commit(&sh->s_full[st]);
      if (j > 0) alive = issue_pv(j - 1);
    }
    if (alive) issue_pv(n_tiles - 1);
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0 && sh->abort && p.status) atomicOr(p.status, (int)GK_DEV_WAIT_EXPIRED);
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512));
}

// 2-D view [kv_heads*slots rows, 128 bf16] of one pool half; boxes of 64 columns x box_rows rows.
bool make_pool_map(CUtensorMap* map, const void* pool, int64_t rows, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)kTile, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)kTile * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

constexpr int kSmemBytes = 7 * kTileBytes + 3072;   // 227 KiB: the whole opt-in shared memory of an SM

}  // namespace
}  // namespace gk

extern "C" int gk_paged_prefill_tc_multi_bf16(const void* q, int64_t q_row_stride, const void* pool_k,
                                              const void* pool_v, int64_t slots, const int32_t* table,
                                              int64_t table_stride, int64_t table_entry_stride, int page_tokens,
                                              const int32_t* table_rows, const int32_t* work, int64_t n_work,
                                              void* const* outs, int n_outs, int64_t out_row_stride, float scale,
                                              float softcap, int window, int q_heads, int kv_heads, int head_dim,
                                              int32_t* status, gk_stream_t stream) {
  if (n_work == 0) return GK_OK;
  if (!outs || n_outs <= 0 || n_outs > GK_MAX_OUTPUTS) return GK_ERR_INVALID_ARGUMENT;
  for (int i = 0; i < n_outs; ++i)
    if (!outs[i] || (reinterpret_cast<uintptr_t>(outs[i]) & 15)) return GK_ERR_INVALID_ARGUMENT;
  if (!q || !pool_k || !pool_v || !table || !work || n_work < 0 || slots <= 0 || table_stride < 0 ||
      table_entry_stride <= 0 || page_tokens <= 0 || (page_tokens & (page_tokens - 1)) || q_heads <= 0 || kv_heads <= 0 ||
      !(scale > 0.f) || !(softcap >= 0.f) || (window != -1 && window <= 0))
    return GK_ERR_INVALID_ARGUMENT;
  if (head_dim != 128 || q_heads % kv_heads != 0 || q_heads / kv_heads > GK_PREFILL_TILE_ROWS ||
      n_work * kv_heads > 0x7fffffffLL)
    return GK_ERR_UNSUPPORTED;
  if (((reinterpret_cast<uintptr_t>(pool_k) | reinterpret_cast<uintptr_t>(pool_v) | reinterpret_cast<uintptr_t>(work)) & 15) || (out_row_stride & 7) || (reinterpret_cast<uintptr_t>(q) & 1))
    return GK_ERR_INVALID_ARGUMENT;
  gk::PrefillParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.pool_k = static_cast<const __nv_bfloat16*>(pool_k);
  p.pool_v = static_cast<const __nv_bfloat16*>(pool_v);
  p.table = table;
  p.table_rows = table_rows;
  p.work = work;
  for (int i = 0; i < n_outs; ++i) p.out[i] = static_cast<__nv_bfloat16*>(outs[i]);
  p.n_out = n_outs;
  p.status = status;
  p.q_stride = q_row_stride;
  p.out_stride = out_row_stride;
  p.slots = slots;
  p.table_stride = table_stride;
  p.entry_stride = table_entry_stride;
  p.scale = scale;
  p.softcap = softcap;
  p.window = window;
  p.page_shift = __builtin_ctz((unsigned)page_tokens);
  p.q_heads = q_heads;
  p.kv_heads = kv_heads;
  p.group = q_heads / kv_heads;
  static std::atomic<bool> configured[64];
  const int ready = gk::opt_in_shared_memory(gk::paged_prefill_tc_kernel, gk::kSmemBytes, configured);
  if (ready != GK_OK) return ready;
  {
    // Never launch if the register pool of this build cannot satisfy the budgets (the kernel would hang).
    static std::atomic<int> launch_regs{-1};
    int regs = launch_regs.load(std::memory_order_acquire);
    if (regs < 0) {
      cudaFuncAttributes attr;
      if (cudaFuncGetAttributes(&attr, gk::paged_prefill_tc_kernel) != cudaSuccess) return gk::check_launch();
      regs = attr.numRegs;
      launch_regs.store(regs, std::memory_order_release);
    }
    if (regs * gk::kThreads <
        gk::kSoftmaxThreads * gk::kSoftmaxRegs + (gk::kThreads - gk::kSoftmaxThreads) * gk::kOtherRegs)
      return GK_ERR_UNSUPPORTED;
  }
  // TMA boxes need slot-contiguous pages of at least 8 tokens and 32-bit row coordinates.
  alignas(64) CUtensorMap map_k, map_v;
  memset(&map_k, 0, sizeof(map_k));
  memset(&map_v, 0, sizeof(map_v));
  const int box_rows = page_tokens < 64 ? page_tokens : 64;
  const int64_t pool_rows = (int64_t)kv_heads * slots;
  if (page_tokens >= 8 && pool_rows < 0x7fffffffLL && gk::make_pool_map(&map_k, pool_k, pool_rows, box_rows) &&
      gk::make_pool_map(&map_v, pool_v, pool_rows, box_rows))
    p.tma_rows = box_rows;
  gk::paged_prefill_tc_kernel<<<(unsigned)(n_work * kv_heads), gk::kThreads, gk::kSmemBytes,
                                reinterpret_cast<cudaStream_t>(stream)>>>(p, map_k, map_v);
  return gk::check_launch();
}

extern "C" int gk_paged_prefill_tc_bf16(const void* q, int64_t q_row_stride, const void* pool_k, const void* pool_v,
                                        int64_t slots, const int32_t* table, int64_t table_stride,
                                        int64_t table_entry_stride, int page_tokens, const int32_t* table_rows,
                                        const int32_t* work, int64_t n_work, void* out, int64_t out_row_stride,
                                        float scale, float softcap, int window, int q_heads, int kv_heads, int head_dim,
                                        int32_t* status, gk_stream_t stream) {
  void* const outs[1] = {out};
  return gk_paged_prefill_tc_multi_bf16(q, q_row_stride, pool_k, pool_v, slots, table, table_stride, table_entry_stride,
                                        page_tokens, table_rows, work, n_work, outs, 1, out_row_stride, scale, softcap,
                                        window, q_heads, kv_heads, head_dim, status, stream);
}
