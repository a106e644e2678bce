// Chunked-prefill paged attention on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// A work record is a run of up to 2 x (128/G) consecutive rows of one sequence.  The G query heads of
// one KV head of those rows are packed into TWO query tiles of 128 rows each (tile t = rows
// [t*128/G, (t+1)*128/G) of the record); both tiles attend to the KV range [kv_begin, kv_end) of the pool
// (prefix + the rows themselves, causal inside the chunk), so every K/V tile is fetched once for 256
// packed rows.  Q.K^T (128 x T x d) and P.V (128 x d x T) run as tcgen05.mma.kind::f16 with fp32
// accumulators in tensor memory.  The description below is head_dim 128 (KV tiles of T = 128 tokens);
// head_dim 64 is the same with 64-column accumulators, and head_dim 256, whose two 256-column accumulators
// would not fit beside the scores, runs ONE query tile per CTA (the record's two tiles go to two CTAs)
// against KV tiles of 64 tokens, so that two K and three V stages still fit in shared memory; there the two
// score buffers alternate between consecutive KV tiles and Q.K^T runs two tiles ahead of P.V:
//
//   TMEM (512 columns)   S0 | S1 | O0 | O1, 128 columns each; P_t (bf16, 64 columns) overwrites the lower
//                        half of S_t and is the A operand of P_t.V straight from tensor memory
//   warps 0-3 / 4-7      softmax of query tile 0 / 1: thread = one packed row = one TMEM lane, all 128
//                        columns, so the row maximum and the row sum need no exchange with anybody.
//                        S comes in with tcgen05.ld, P (rounded to bf16, the reference's boundary) goes
//                        back with tcgen05.st; O is rescaled in TMEM only when the running maximum moved
//                        by more than 2^8; at the end the same thread normalises its O row and stores it
//                        to every destination
//   warps 8-11           loaders (8-9 K, 10-11 V) of 128-token tiles: whole, slot-contiguous pages by TMA
//                        (cp.async.bulk.tensor 2-D boxes, 128-byte swizzle, no multicast), anything else
//                        row by row with 16-byte cp.async; two K stages, three V stages
//   warp 12              one thread issues the MMAs in the order  P0.V(j), Q0.K(j+1), P1.V(j), Q1.K(j+1):
//                        while one tile's softmax runs, the tensor pipe works on the other tile
//
// While one tile's softmax runs, the tensor pipe has the other tile's two products to do.  The softmax
// arithmetic is packed (fma.f32x2 / add.f32x2, three-input maxima) and the uncommon cases (softcap, tiles
// that need masking) rewrite S in tensor memory in a short loop first, so the common path stays small:
// the instruction cache is the first thing this kernel ran out of when every case was unrolled in place.
// Every mbarrier wait is bounded: on expiry the CTA raises GK_DEV_WAIT_EXPIRED, drains its copies,
// frees its TMEM and returns.
#include "tc_common.cuh"

#include <string.h>
#include <math_constants.h>

namespace gk {
namespace {

constexpr int kRows = 128;             // packed query rows per tile = lanes of tensor memory
constexpr int kKStages = 2, kVStages = 3;
constexpr int kSoftmaxThreads = 256, kLoaderThreads = 64, kThreads = 512;   // loaders: 64 threads for K, 64 for V
constexpr int kLaunchRegs = 128;     // what __launch_bounds__(512, 1) lets ptxas allocate per thread
constexpr int kSoftmaxRegs = 184, kLoaderRegs = 80, kIssueRegs = 64;
static_assert(kSoftmaxThreads * kSoftmaxRegs + 128 * kLoaderRegs + 128 * kIssueRegs <= kThreads * kLaunchRegs,
              "register budgets exceed the pool the launch allocates");

// Shapes that follow from head_dim D.  Operand tiles are stored as D/64 panels of [rows x 128 bytes] with the
// 128-byte swizzle; a query tile has 128 rows, a K or V tile kKv rows.
template <int D>
struct Geo {
  static_assert(D == 64 || D == 128 || D == 256, "head_dim");
  static constexpr int kKv = D == 256 ? 64 : 128;          // KV tokens per tile
  static constexpr int kTiles = D == 256 ? 1 : 2;          // query tiles per CTA
  static constexpr int kPanels = D / 64, kChunks = D / 8;  // 128-byte panels, 16-byte chunks per row
  static constexpr int kQPanelBytes = kRows * 128, kQTileBytes = kPanels * kQPanelBytes;
  static constexpr int kKvPanelBytes = kKv * 128, kKvTileBytes = kPanels * kKvPanelBytes;
  static constexpr int kSmemBytes = kTiles * kQTileBytes + (kKStages + kVStages) * kKvTileBytes + 3072;
  // kind::f16 instruction descriptors: fp32 accumulate, bf16 x bf16, M = 128; N = kKv (A, B K-major) for the
  // scores, N = D with B (= V) MN-major for the second product.
  static constexpr uint32_t kIdescQK = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kKv >> 3) << 17) | (8u << 24);
  static constexpr uint32_t kIdescPV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | (8u << 24);
};
static_assert(Geo<128>::kSmemBytes <= 227 * 1024 && Geo<256>::kSmemBytes <= 227 * 1024, "shared memory of an SM");
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
  int tma_rows;          // rows of a TMA box, 0 = TMA path off
  int n_out;
};

struct Shared {
  uint64_t k_full[kKStages], k_free[kKStages], v_full[kVStages], v_free[kVStages];
  uint64_t s_full[2], p_full[2], pv_done[2];
  uint32_t tmem_base;
  int abort;
};

// Byte offset of 16-byte chunk c of row r inside a tile whose panels are panel_bytes apart.
__device__ __forceinline__ uint32_t tile_off(int r, int c, int panel_bytes) {
  return (c >> 3) * panel_bytes + r * 128 + (((c & 7) ^ (r & 7)) << 4);
}

// The MMAs take each 64-bit shared-memory descriptor as its two halves: the upper half (strides, swizzle mode)
// is the same for every tile of one operand kind, the lower half is the address field plus the
// leading-dimension stride, so stepping through a tile or a ring is a 32-bit add.  The second form reads its
// A operand (P, bf16, two per 32-bit column) from tensor memory.
__device__ __forceinline__ void umma_bf16_ss_split(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                                   uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n.reg .b64 da, db;\nsetp.ne.b32 p, %6, 0;\nmov.b64 da, {%1, %2};\nmov.b64 db, {%3, %4};\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n}\n" ::"r"(tmem_d),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_ts_split(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                                   uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n.reg .b64 db;\nsetp.ne.b32 p, %5, 0;\nmov.b64 db, {%2, %3};\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n}\n" ::"r"(tmem_d),
      "r"(tmem_a), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st16_nowait(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

template <int D>
__global__ void __launch_bounds__(kThreads, 1) paged_prefill_tc_kernel(const PrefillParams p,
                                                                       const __grid_constant__ CUtensorMap map_k,
                                                                       const __grid_constant__ CUtensorMap map_v) {
  using G_ = Geo<D>;
  constexpr int kKv = G_::kKv, kTiles = G_::kTiles, kChunks = G_::kChunks;
  constexpr int kQPanelBytes = G_::kQPanelBytes, kQTileBytes = G_::kQTileBytes;
  constexpr int kKvPanelBytes = G_::kKvPanelBytes, kKvTileBytes = G_::kKvTileBytes;
  constexpr int kScoreChunks = kKv / 32;                 // 32-column pieces of a row of S
  extern __shared__ __align__(1024) uint8_t tiles[];     // swizzle atoms need 1 KiB alignment
  uint8_t* s_q = tiles;                                  // the query tiles
  uint8_t* s_k = s_q + kTiles * kQTileBytes;             // K stages
  uint8_t* s_v = s_k + kKStages * kKvTileBytes;          // V stages
  Shared* sh = reinterpret_cast<Shared*>(s_v + kVStages * kKvTileBytes);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (smem_u32(tiles) & 1023) {                          // cannot build valid descriptors: report, leave
    if (tid == 0 && p.status) atomicOr(p.status, (int)GK_DEV_WAIT_EXPIRED);
    return;
  }
  // With one query tile per CTA the record's two tiles go to two consecutive CTAs.
  const int unit = kTiles == 2 ? blockIdx.x : blockIdx.x >> 1, half = kTiles == 2 ? 0 : blockIdx.x & 1;
  const int item = unit / p.kv_heads, head = unit - item * p.kv_heads;
  const int4 w0 = __ldg(reinterpret_cast<const int4*>(p.work) + 2 * item);
  const int4 w1 = __ldg(reinterpret_cast<const int4*>(p.work) + 2 * item + 1);
  const int G = p.group;
  const int tile_rows = kRows / G;                          // rows of the record per query tile
  int first_row = w0.x, n_rows = w0.y, first_pos = w0.z, kv_begin = w1.x, kv_end = w1.y;
  const int table_row = w0.w;
  if (kTiles == 1) {                                        // this CTA's tile of the record, as a record of its own
    const int skip = half * tile_rows;
    n_rows = min(n_rows - skip, tile_rows);
    if (n_rows <= 0) return;                                // the whole CTA: nothing is allocated yet
    first_row += skip;
    first_pos += skip;
    kv_end = min(kv_end, first_pos + n_rows);               // causal: nothing after this tile's last row
    if (p.window > 0) kv_begin = max(kv_begin, first_pos - p.window + 1);
  }
  const int rows0 = min(n_rows, tile_rows), rows1 = n_rows - rows0;
  // KV tiles each query tile needs: tile 0 stops at its own last row (causal), tile 1 at the record's end
  const int nt1_all = (kv_end - kv_begin + kKv - 1) / kKv;
  const int nt0 = min(nt1_all, (first_pos + rows0 - kv_begin + kKv - 1) / kKv);
  const int nt1 = rows1 > 0 ? nt1_all : 0;
  const int n_tiles = max(nt0, nt1);

  if (tid == 0) {
    for (int i = 0; i < kKStages; ++i) {
      bar_init(&sh->k_full[i], kLoaderThreads);
      bar_init(&sh->k_free[i], 1);
    }
    for (int i = 0; i < kVStages; ++i) {
      bar_init(&sh->v_full[i], kLoaderThreads);
      bar_init(&sh->v_free[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      bar_init(&sh->s_full[i], 1);
      bar_init(&sh->p_full[i], 4);      // one arrival per softmax warp of the tile
      bar_init(&sh->pv_done[i], 1);
    }
    sh->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&sh->tmem_base)), "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  tc_fence_before();
  __syncthreads();                                       // barriers and the TMEM allocation are in place
  tc_fence_after();
  const bool is_loader = warp >= 8 && warp < 12;
  if (!is_loader) {
    // Q tiles: packed row pr of tile t = (row t*tile_rows + pr / G, query head pr % G) of this KV head; unused rows
    // are zero.  The loader warps do not take part: their first K/V tiles are already on the way meanwhile.
    const int filler = warp < 8 ? tid : tid - 128;       // 0..383
    for (int i = filler; i < kTiles * kRows * kChunks; i += kThreads - 128) {
      const int t = i / (kRows * kChunks), pr = (i / kChunks) & (kRows - 1), c = i & (kChunks - 1);
      uint4 v = make_uint4(0, 0, 0, 0);
      const int r = t * tile_rows + pr / G, g = pr % G;
      if (pr < tile_rows * G && r < n_rows) {
        const __nv_bfloat16* src = p.q + (int64_t)(first_row + r) * p.q_stride + (int64_t)(head * G + g) * D + c * 8;
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
      *reinterpret_cast<uint4*>(s_q + t * kQTileBytes + tile_off(pr, c, kQPanelBytes)) = v;
    }
    fence_async_smem();
    asm volatile("bar.sync 1, %0;\n" ::"n"(kThreads - 128) : "memory");      // the 384 threads that filled Q
  }
  const uint32_t tmem = sh->tmem_base;

  // Registers move from the loader / issue warpgroups (which need few) to the softmax warpgroups.
  // setmaxnreg.inc blocks until the CTA's register pool can satisfy it, and the pool is what the
  // launch allocated (kThreads x kLaunchRegs): the budgets must fit in it or the softmax warps
  // would never start (checked at compile time and again on the host before every launch).
  if (warp < 8) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(kSoftmaxRegs));
  } else if (warp < 12) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(kLoaderRegs));
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(kIssueRegs));
  }

  if (warp < 8) {
    // ================================ softmax of query tile t ===============================
    const int t = warp >> 2;
    const int pr = tid & 127;                                    // packed row == TMEM lane
    const int my_rows = t == 0 ? rows0 : rows1;
    const int mv = my_rows * G;                                  // packed rows of this tile in use
    const int my_tiles = t == 0 ? nt0 : nt1;
    const int tile_first_pos = first_pos + t * tile_rows;
    const int lim = pr < mv ? tile_first_pos + pr / G : 0x7fffffff;   // last visible key of this row
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t o_addr = tmem + 256 + t * D + lane_base;
    const bool capped = p.softcap > 0.f;
    const float to_log2 = capped ? kLog2e : p.scale * kLog2e;
    const float cap_in = capped ? p.scale / p.softcap : 0.f;
    float m = -CUDART_INF_F, l = 0.f;                            // m: exponent reference of this row
    bool alive = true;
    for (int j = 0; j < my_tiles && alive; ++j) {
      // Two query tiles: tile t owns score buffer t.  One query tile: the two buffers alternate between
      // consecutive KV tiles, so Q.K^T of the next tile is already there when this softmax ends.
      const int buf = kTiles == 2 ? t : (j & 1);
      const uint32_t use = kTiles == 2 ? j : (j >> 1);            // how often this buffer was filled before
      const uint32_t s_addr = tmem + buf * 128 + lane_base;       // S; P overwrites its lower half
      const uint32_t p_addr = s_addr;
      alive = __all_sync(0xffffffffu, bar_wait(&sh->s_full[buf], use & 1, &sh->abort));
      if (!alive) break;
      tc_fence_after();
      const int tok0 = kv_begin + j * kKv;
      const int tile_end = tok0 + kKv;
      const bool ragged = tile_end > kv_end || tile_end > tile_first_pos + 1 ||
                          (p.window > 0 && tok0 <= tile_first_pos + my_rows - 1 - p.window);
      // Softcap and tiles that need masking are uncommon: they first rewrite S in tensor memory (scores in
      // log2 units, masked keys at -inf), 32 columns at a time in a loop that is NOT unrolled, so that
      // the two passes below stay one short piece of code (the instruction cache is what this kernel
      // runs out of first when every variant is unrolled 128 times).
      float mult = to_log2;
      if (capped || ragged) {
#pragma unroll 1
        for (int c = 0; c < kScoreChunks; ++c) {
          uint32_t r[32];
          tmem_ld32(s_addr + c * 32, r);
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            float v = __uint_as_float(r[e]);
            if (capped) v = p.softcap * tanhf(v * cap_in);
            v *= to_log2;
            const int tok = tok0 + c * 32 + e;
            const bool seen = tok < kv_end && tok <= lim && (p.window <= 0 || tok > lim - p.window);
            r[e] = __float_as_uint(seen ? v : -CUDART_INF_F);
          }
          tmem_st32(s_addr + c * 32, r);
        }
        mult = 1.f;
      }
      // ---- the whole row comes in once (up to 128 registers) and stays until it has become P ----
      uint32_t sr[kScoreChunks][32];
#pragma unroll
      for (int c = 0; c < kScoreChunks; ++c) tmem_ld32_nowait(s_addr + c * 32, sr[c]);
      tmem_ld_wait();
      float mx;
      {
        float part[kScoreChunks];
#pragma unroll
        for (int c = 0; c < kScoreChunks; ++c) part[c] = -CUDART_INF_F;
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
#pragma unroll
          for (int c = 0; c < kScoreChunks; ++c)
            part[c] = max3(part[c], __uint_as_float(sr[c][e]), __uint_as_float(sr[c][e + 1]));
        }
        mx = fmaxf(part[0], part[1]);
        if (kScoreChunks == 4) mx = fmaxf(mx, fmaxf(part[2], part[3]));
        mx *= mult;                                                                 // mult > 0
      }
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
        alive = __all_sync(0xffffffffu, bar_wait(&sh->pv_done[t], (j - 1) & 1, &sh->abort));
        if (!alive) break;
        tc_fence_after();
#pragma unroll 1
        for (int cb = 0; cb < D / 32; ++cb) {
          uint32_t r[32];
          tmem_ld32(o_addr + cb * 32, r);
#pragma unroll
          for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
          tmem_st32(o_addr + cb * 32, r);
        }
      }
      // ---- probabilities, 32 columns at a time.  P (bf16, the reference's rounding point before the
      // second product) overwrites the LOWER half of S; every column of S is in registers by now.
      float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      const float2 mult2 = make_float2(mult, mult), neg_mu2 = make_float2(-mu, -mu);
#pragma unroll
      for (int c = 0; c < kScoreChunks; ++c) {
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float2 x = __ffma2_rn(make_float2(__uint_as_float(sr[c][2 * i]), __uint_as_float(sr[c][2 * i + 1])), mult2, neg_mu2);
          const float2 pr2 = make_float2(fast_exp2(x.x), fast_exp2(x.y));
          sum2[i & 1] = __fadd2_rn(sum2[i & 1], pr2);
          packed[i] = pack_bf16(pr2.x, pr2.y);
        }
        tmem_st16_nowait(p_addr + c * 16, packed);
      }
      l = l * alpha + ((sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y));
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();                                      // every lane's P is in tensor memory: one arrival per warp
      if (lane == 0) bar_arrive(&sh->p_full[buf]);
    }
    // epilogue: O / l -> bf16 rows of the output
    if (alive && my_tiles > 0) {
      alive = __all_sync(0xffffffffu, bar_wait(&sh->pv_done[t], (my_tiles - 1) & 1, &sh->abort));
      if (alive) {
        tc_fence_after();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const int r_q = t * tile_rows + pr / G, g = pr % G;
        const int64_t at = (int64_t)(first_row + r_q) * p.out_stride + (int64_t)(head * G + g) * D;
#pragma unroll 1
        for (int cb = 0; cb < D / 32; ++cb) {
          uint32_t r[32];
          tmem_ld32(o_addr + cb * 32, r);
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
    }
  } else if (warp < 12) {
    // ================================ K/V loaders =========================================
    const bool is_v = warp >= 10;
    const int lwarp = (warp - 8) & 1;
    const int stages = is_v ? kVStages : kKStages;
    const __nv_bfloat16* base = (is_v ? p.pool_v : p.pool_k) + (int64_t)head * p.slots * D;
    const int32_t* trow = p.table + (int64_t)(p.table_rows ? __ldg(p.table_rows + table_row) : table_row) * p.table_stride;
    const int page_mask = (1 << p.page_shift) - 1;
    const CUtensorMap* map = is_v ? &map_v : &map_k;
    const int head_row = head * (int)p.slots;
    int st = 0, round = 0;                                   // ring position of tile j: stage j % stages, round j / stages
    for (int j = 0; j < n_tiles; ++j) {
      // each loader warp stages half a tile, 32 rows at a time: lanes resolve one slot each, then the
      // warp copies 512 bytes of consecutive rows per instruction (16 bytes a lane)
      constexpr int kWarpRows = kKv / 2, kHalves = kWarpRows / 32;
      int slot[kHalves];
#pragma unroll
      for (int half = 0; half < kHalves; ++half) {
        const int tok = kv_begin + j * kKv + lwarp * kWarpRows + half * 32 + lane;
        slot[half] = -1;
        if (tok < kv_end) {
          slot[half] = __ldg(trow + (int64_t)(tok >> p.page_shift) * p.entry_stride) + (tok & page_mask);
          if ((unsigned)slot[half] >= (unsigned)p.slots) {
            if (p.status) atomicOr(p.status, (int)GK_DEV_BAD_TABLE);
            slot[half] = -1;
          }
        }
      }
      // This warp's rows go by TMA when they are whole, in-range boxes of tma_rows slot-contiguous
      // tokens; the two warps of a tile decide independently (every thread arrives once either way).
      const int tok_first = kv_begin + j * kKv + lwarp * kWarpRows;
      bool by_tma = p.tma_rows > 0 && (tok_first & (p.tma_rows - 1)) == 0 && tok_first + kWarpRows <= kv_end;
      by_tma = __all_sync(0xffffffffu, by_tma && slot[0] >= 0 && slot[kHalves - 1] >= 0);
      uint64_t* full = is_v ? &sh->v_full[st] : &sh->k_full[st];
      if (round > 0) {   // stage free: K once both Q.K^T of the tile that used it completed, V once both P.V did
        uint64_t* freed = is_v ? &sh->v_free[st] : &sh->k_free[st];
        if (!__all_sync(0xffffffffu, bar_wait_patient(freed, (round - 1) & 1, &sh->abort))) break;
      }
      const uint32_t dst = smem_u32(is_v ? s_v : s_k) + st * kKvTileBytes;
      if (by_tma) {
        if (lane == 0) bar_arrive_expect_tx(full, kWarpRows * D * 2);
        else bar_arrive(full);
        __syncwarp();
        // the lane that holds the first row of a box issues its panels
#pragma unroll
        for (int half = 0; half < kHalves; ++half) {
          const int row = half * 32 + lane;                       // row within this warp's share
          if ((row & (p.tma_rows - 1)) == 0) {
            const uint32_t at = dst + (lwarp * kWarpRows + row) * 128;
#pragma unroll
            for (int panel = 0; panel < G_::kPanels; ++panel)
              tma_load_box(at + panel * kKvPanelBytes, map, panel * 64, head_row + slot[half], full);
          }
        }
      } else {
#pragma unroll
        for (int half = 0; half < kHalves; ++half) {
#pragma unroll 4
          for (int i = 0; i < kChunks; ++i) {                     // 32 rows x kChunks chunks over 32 lanes
            const int at = i * 32 + lane, rr = at / kChunks, c = at & (kChunks - 1);
            const int s = __shfl_sync(0xffffffffu, slot[half], rr);
            cp_async_16(dst + tile_off(lwarp * kWarpRows + half * 32 + rr, c, kKvPanelBytes),
                        base + (int64_t)(s < 0 ? 0 : s) * D + c * 8, s < 0 ? 0 : 16);
          }
        }
        bar_arrive_on_copies(full);
      }
      if (++st == stages) {
        st = 0;
        ++round;
      }
    }
    asm volatile("cp.async.wait_all;\n" ::: "memory");
  } else if (warp == 12 && lane == 0) {
    // ================================ MMA issue ===========================================
    const uint32_t q_addr = smem_u32(s_q), k_base = smem_u32(s_k), v_base = smem_u32(s_v);
    const int nt[2] = {nt0, nt1};
    bool alive = true;
    // Operand descriptors are built once; a k-step or a ring stage only moves the 14-bit address field (units of
    // 16 bytes) in the lower half, so the issue loop is one 32-bit add per operand and the MMA itself.
    const uint64_t q_desc = umma_desc(q_addr, 16, 1024), k_desc = umma_desc(k_base, 16, 1024);
    const uint64_t v_desc = umma_desc(v_base, kKvPanelBytes, 1024);
    const uint32_t q_lo = (uint32_t)q_desc, k_lo = (uint32_t)k_desc, v_lo = (uint32_t)v_desc;
    const uint32_t qk_hi = (uint32_t)(q_desc >> 32), v_hi = (uint32_t)(v_desc >> 32);      // K's upper half equals Q's
    constexpr uint32_t kStageStep = kKvTileBytes >> 4;
    // S[buf] = Q[t] . K[stage]^T ; O[t] += P[buf] . V[stage]
    auto issue_qk = [&](int t, int buf, int stage) {
      const uint32_t a = q_lo + t * (kQTileBytes >> 4), b = k_lo + stage * kStageStep;
#pragma unroll
      for (int k = 0; k < D / 16; ++k) {               // 16 elements of head_dim per step
        const uint32_t a_step = ((k >> 2) * kQPanelBytes + (k & 3) * 32) >> 4;
        const uint32_t b_step = ((k >> 2) * kKvPanelBytes + (k & 3) * 32) >> 4;
        umma_bf16_ss_split(tmem + buf * 128, a + a_step, qk_hi, b + b_step, qk_hi, G_::kIdescQK, k > 0 ? 1u : 0u);
      }
      umma_commit(&sh->s_full[buf]);
    };
    auto issue_pv = [&](int t, int buf, int j, int stage) {
      const uint32_t b = v_lo + stage * kStageStep;
#pragma unroll
      for (int k = 0; k < kKv / 16; ++k) {             // 16 tokens per step: 8 columns of P, 16 rows of V
        umma_bf16_ts_split(tmem + 256 + t * D, tmem + buf * 128 + k * 8, b + k * (2048 >> 4), v_hi, G_::kIdescPV,
                           (j > 0 || k > 0) ? 1u : 0u);
      }
      umma_commit(&sh->pv_done[t]);
    };
    if (kTiles == 1) {
      // One query tile, two score buffers: Q.K^T runs two KV tiles ahead of P.V, so the tensor pipe has the next
      // tile's scores ready while this tile's softmax runs.  Order: QK(0), QK(1), then PV(j), QK(j+2) per tile.
      for (int a = 0; a < 2 && a < n_tiles && alive; ++a) {
        alive = bar_wait(&sh->k_full[a % kKStages], (a / kKStages) & 1, &sh->abort);
        if (!alive) break;
        fence_async_smem();
        tc_fence_after();
        issue_qk(0, a, a % kKStages);
        umma_commit(&sh->k_free[a % kKStages]);
      }
      int vs = 0, vround = 0;
      for (int j = 0; j < n_tiles && alive; ++j) {
        alive = bar_wait(&sh->v_full[vs], vround & 1, &sh->abort) &&
                bar_wait(&sh->p_full[j & 1], (j >> 1) & 1, &sh->abort);
        if (!alive) break;
        fence_async_smem();
        tc_fence_after();
        issue_pv(0, j & 1, j, vs);
        umma_commit(&sh->v_free[vs]);
        if (j + 2 < n_tiles) {                 // the buffer P.V(j) reads is free once that product has run: in order
          const int ks = (j + 2) % kKStages;
          alive = bar_wait(&sh->k_full[ks], ((j + 2) / kKStages) & 1, &sh->abort);
          if (!alive) break;
          fence_async_smem();
          tc_fence_after();
          issue_qk(0, j & 1, ks);
          umma_commit(&sh->k_free[ks]);
        }
        if (++vs == kVStages) {
          vs = 0;
          ++vround;
        }
      }
    } else {
    if (n_tiles > 0) {
      alive = bar_wait(&sh->k_full[0], 0, &sh->abort);
      if (alive) {
        fence_async_smem();
        tc_fence_after();
        for (int t = 0; t < 2; ++t)
          if (nt[t] > 0) issue_qk(t, t, 0);
        umma_commit(&sh->k_free[0]);
      }
    }
    int ks = 1 % kKStages, kround = 1 / kKStages, vs = 0, vround = 0;     // ring positions of K tile j+1 and V tile j
    for (int j = 0; j < n_tiles && alive; ++j) {
      const bool more = j + 1 < n_tiles;
      alive = bar_wait(&sh->v_full[vs], vround & 1, &sh->abort);
      if (alive && more) alive = bar_wait(&sh->k_full[ks], kround & 1, &sh->abort);
      if (!alive) break;
      fence_async_smem();
      tc_fence_after();
      for (int t = 0; t < 2 && alive; ++t) {
        if (j < nt[t]) {
          alive = bar_wait(&sh->p_full[t], j & 1, &sh->abort);
          if (!alive) break;
          tc_fence_after();
          issue_pv(t, t, j, vs);
        }
        if (j + 1 < nt[t]) issue_qk(t, t, ks);
      }
      if (!alive) break;
      umma_commit(&sh->v_free[vs]);
      if (more) umma_commit(&sh->k_free[ks]);
      if (++vs == kVStages) {
        vs = 0;
        ++vround;
      }
      if (++ks == kKStages) {
        ks = 0;
        ++kround;
      }
    }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0 && sh->abort && p.status) atomicOr(p.status, (int)GK_DEV_WAIT_EXPIRED);
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512));
}

template <int D>
int launch_prefill(PrefillParams& p, int64_t n_work, int page_tokens, cudaStream_t stream) {
  static std::atomic<bool> configured[64];
  const int ready = opt_in_shared_memory(paged_prefill_tc_kernel<D>, Geo<D>::kSmemBytes, configured);
  if (ready != GK_OK) return ready;
  {
    // Never launch if the register pool of this build cannot satisfy the budgets (the kernel would hang).
    static std::atomic<int> launch_regs{-1};
    int regs = launch_regs.load(std::memory_order_acquire);
    if (regs < 0) {
      cudaFuncAttributes attr;
      if (cudaFuncGetAttributes(&attr, paged_prefill_tc_kernel<D>) != cudaSuccess) return check_launch();
      regs = attr.numRegs;
      launch_regs.store(regs, std::memory_order_release);
    }
    if (regs * kThreads < kSoftmaxThreads * kSoftmaxRegs + 128 * kLoaderRegs + 128 * kIssueRegs) return GK_ERR_UNSUPPORTED;
  }
  // TMA boxes need slot-contiguous pages of at least 8 tokens and 32-bit row coordinates; a box is at most
  // the rows one loader warp stages.
  alignas(64) CUtensorMap map_k, map_v;
  memset(&map_k, 0, sizeof(map_k));
  memset(&map_v, 0, sizeof(map_v));
  constexpr int kWarpRows = Geo<D>::kKv / 2;
  const int box_rows = page_tokens < kWarpRows ? page_tokens : kWarpRows;
  const int64_t pool_rows = (int64_t)p.kv_heads * p.slots;
  if (page_tokens >= 8 && pool_rows < 0x7fffffffLL && make_pool_map(&map_k, p.pool_k, pool_rows, box_rows, D) &&
      make_pool_map(&map_v, p.pool_v, pool_rows, box_rows, D))
    p.tma_rows = box_rows;
  const int64_t ctas = n_work * p.kv_heads * (Geo<D>::kTiles == 2 ? 1 : 2);
  if (ctas > 0x7fffffffLL) return GK_ERR_UNSUPPORTED;
  paged_prefill_tc_kernel<D><<<(unsigned)ctas, kThreads, Geo<D>::kSmemBytes, stream>>>(p, map_k, map_v);
  return check_launch();
}

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
  if ((head_dim != 64 && head_dim != 128 && head_dim != 256) || q_heads % kv_heads != 0 || q_heads / kv_heads > GK_PREFILL_TILE_ROWS ||
      n_work * kv_heads > 0x7fffffffLL)
    return GK_ERR_UNSUPPORTED;
  if (((reinterpret_cast<uintptr_t>(pool_k) | reinterpret_cast<uintptr_t>(pool_v) | reinterpret_cast<uintptr_t>(work)) & 15) ||
      (out_row_stride & 7) || (reinterpret_cast<uintptr_t>(q) & 1))
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
  cudaStream_t at = reinterpret_cast<cudaStream_t>(stream);
  if (head_dim == 64) return gk::launch_prefill<64>(p, n_work, page_tokens, at);
  if (head_dim == 256) return gk::launch_prefill<256>(p, n_work, page_tokens, at);
  return gk::launch_prefill<128>(p, n_work, page_tokens, at);
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
