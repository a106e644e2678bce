// Output projection of the attention block on the 5th-generation tensor cores:
//   out[M, N] = bf16( A[M, K] . W[N, K]^T )      bf16 operands, fp32 accumulation in TMEM
// with A the attention output of this rank's heads and W this rank's column slice of the o_proj
// weight (row-parallel linear: every rank produces a partial [M, N] that the rank-ordered sum
// behind it adds up).  The result can be written to several destinations at once -- the same
// slot of every tensor-parallel peer's receive buffer -- so the exchange rides on the epilogue's
// stores and no separate collective moves the partials.
//
// One CTA owns a [128 * MT] x BN block of the output (MT = 1 or 2 accumulators of BN = 256, 128 or 64
// TMEM columns each; the 256 x 256 block uses all 512 columns) and walks its K range in steps of 64:
//   warp 0     one thread issues the TMA loads of a stage: MT boxes [128 x 64] of A and one box
//              [BN x 64] of W, 128-byte swizzle, no multicast; rows past M are zero-filled by TMA
//   warp 1     one thread issues tcgen05.mma.kind::f16 (M 128, N BN, K 16) four times per box and
//              commits the stage back to the loader, finally the accumulators to the epilogue
//   warps 2-5  epilogue: tcgen05.ld of the thread's row, rounding to bf16, the block staged in
//              shared memory and stored to every destination as whole contiguous row segments
// Wide blocks are for large problems: a 256 x 256 block needs 64 KB of operands per 64 of K where two
// 256 x 128 blocks need 96 KB, and a 128 x 256 x 16 MMA reads 96 bytes of shared-memory operands per cycle
// where the 128 x 128 x 16 one reads the SM's whole 128.
// A kernel of this shape is bound by how fast one SM takes in operand boxes, so small problems are
// cut along K over a thread-block cluster (2 or 4 CTAs per output block) until the grid fills the
// GPU; the cluster adds its fp32 accumulators through distributed shared memory in a fixed order.
// Every mbarrier wait is bounded; on expiry the CTA raises GK_DEV_WAIT_EXPIRED, frees its TMEM and
// returns.
#include "tc_common.cuh"

#include <string.h>

namespace gk {
namespace {

constexpr int kBM = 128, kBK = 64;
constexpr int kABytes = kBM * kBK * 2;   // 16 KiB
constexpr int kLinearThreads = 192;
constexpr int kMaxStages = 8;
constexpr int kMaxSplit = 4;
constexpr double kSplitOverheadUs = 6.0;

template <int MT, int BN>
struct LinearTile {
  static constexpr int kWBytes = BN * kBK * 2;
  static constexpr int kStageBytes = MT * kABytes + kWBytes;
  static constexpr int kStages = (192 * 1024) / kStageBytes > kMaxStages ? kMaxStages : (192 * 1024) / kStageBytes;
  static constexpr int kTmemCols = MT * BN < 32 ? 32 : MT * BN;
  static constexpr int kReduceBytes = MT * BN * kBM * 4;         // fp32 accumulators parked for the split-K sum
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /* alignment slack */ + 256 /* barriers */;
  // the split-K reduce buffer reuses the pipeline stages: tiles too large for that are never cut along K
  static constexpr bool kCanSplit = kReduceBytes <= kStages * kStageBytes;
  static_assert((kTmemCols & (kTmemCols - 1)) == 0 && kTmemCols <= 512, "TMEM columns: a power of two");
};

struct LinearShared {
  uint64_t full[kMaxStages], empty[kMaxStages], done;
  uint32_t tmem_base;
  int abort;
};

struct LinearParams {
  unsigned short* outs[GK_MAX_OUTPUTS];
  int n_outs;
  int64_t out_stride;
  int m, n, k;
  int32_t* status;
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;\n" : "=r"(r));
  return r;
}
// All threads of all CTAs of the cluster; release/acquire so that shared-memory writes before it are
// visible to remote reads after it.
__device__ __forceinline__ void cluster_sync() {
  __syncwarp();                                              // the elected threads rejoin their warps first
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ uint32_t peer_smem_addr(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(local_addr), "r"(rank));
  return remote;
}
// No memory clobber: the caller issues a batch of these before the first use so that they overlap;
// the cluster barrier in front of the batch (which has the clobber) orders them after the writes.
__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}

// Split-K: the CTAs of a cluster (gridDim.z of them) take consecutive K ranges of the same output
// block, park their fp32 accumulators in their own shared memory and, after a cluster barrier, each
// adds up a column slice over all CTAs in split order through distributed shared memory -- a fixed
// order, so the result does not depend on scheduling -- and stores it.
template <int MT, int BN>
__global__ void __launch_bounds__(kLinearThreads, 1)
linear_tc_kernel(const LinearParams p, const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w) {
  using T = LinearTile<MT, BN>;
  extern __shared__ unsigned char raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  LinearShared* sh = reinterpret_cast<LinearShared*>(base + T::kStages * T::kStageBytes);
  const uint32_t tiles = smem_u32(base);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * BN, m0 = blockIdx.y * (kBM * MT);
  const int split = (int)cluster_size(), part = (int)cluster_rank();
  const int all_steps = p.k / kBK, per = (all_steps + split - 1) / split;
  const int k_first = part * per, k_steps = max(0, min(all_steps, k_first + per) - k_first);

  if (tid == 0) {
    for (int s = 0; s < T::kStages; ++s) {
      bar_init(&sh->full[s], 1);
      bar_init(&sh->empty[s], 1);
    }
    bar_init(&sh->done, 1);
    sh->abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&sh->tmem_base)),
                 "r"(T::kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&sh->tmem_base);

  if (warp == 0) {
    if (lane == 0) {
      for (int kt = 0; kt < k_steps; ++kt) {
        const int s = kt % T::kStages;
        if (kt >= T::kStages && !bar_wait(&sh->empty[s], ((kt / T::kStages) - 1) & 1, &sh->abort)) break;
        bar_arrive_expect_tx(&sh->full[s], T::kStageBytes);
        const uint32_t dst = tiles + s * T::kStageBytes;
        const int x = (k_first + kt) * kBK;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) tma_load_box(dst + mt * kABytes, &map_a, x, m0 + mt * kBM, &sh->full[s]);
        tma_load_box(dst + MT * kABytes, &map_w, x, n0, &sh->full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BN);
      bool alive = true;
      for (int kt = 0; kt < k_steps && alive; ++kt) {
        const int s = kt % T::kStages;
        alive = bar_wait(&sh->full[s], (kt / T::kStages) & 1, &sh->abort);
        if (!alive) break;
        tc_fence_after();
        const uint32_t a = tiles + s * T::kStageBytes, w = a + MT * kABytes;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int k4 = 0; k4 < kBK / 16; ++k4)
            umma_bf16(tmem + mt * BN, umma_desc(a + mt * kABytes + k4 * 32, 16, 1024), umma_desc(w + k4 * 32, 16, 1024),
                      idesc, (kt > 0 || k4 > 0) ? 1u : 0u);
        umma_commit(&sh->empty[s]);
      }
      if (alive) umma_commit(&sh->done);
    }
  }

  // Epilogue warps: thread = one of the 128 accumulator rows (a warp reads TMEM lanes 32 * (warp % 4) ...).
  const int quarter = warp & 3, row = quarter * 32 + lane;
  float* park = reinterpret_cast<float*>(base);             // [mt][column][row] fp32, the stages are drained by now
  bool alive = true;
  if (warp >= 2) {
    alive = k_steps == 0 || __all_sync(0xffffffffu, bar_wait(&sh->done, 0, &sh->abort));
    if (alive) tc_fence_after();
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t acc[32];
        if (alive && k_steps > 0) {
          tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + mt * BN + c0, acc);
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c) acc[c] = 0u;
        }
        if (split > 1) {
#pragma unroll
          for (int c = 0; c < 32; ++c) park[(mt * BN + c0 + c) * kBM + row] = __uint_as_float(acc[c]);
        } else if (p.n_outs == 1) {                         // one (local) destination: straight from registers
          const int64_t out_row = (int64_t)m0 + mt * kBM + row;
          if (out_row < p.m) {
            uint4* dst = reinterpret_cast<uint4*>(p.outs[0] + out_row * p.out_stride + n0 + c0);
#pragma unroll
            for (int c = 0; c < 4; ++c)
              dst[c] = make_uint4(pack_bf16(__uint_as_float(acc[8 * c]), __uint_as_float(acc[8 * c + 1])),
                                  pack_bf16(__uint_as_float(acc[8 * c + 2]), __uint_as_float(acc[8 * c + 3])),
                                  pack_bf16(__uint_as_float(acc[8 * c + 4]), __uint_as_float(acc[8 * c + 5])),
                                  pack_bf16(__uint_as_float(acc[8 * c + 6]), __uint_as_float(acc[8 * c + 7])));
          }
        } else {
          // Several destinations (peers): the bf16 block is staged in shared memory ([mt][row][BN], 16-byte
          // chunks XOR-swizzled by the row so that a thread-per-row write pattern is conflict-free) and
          // stored row-contiguously below
          uint4* stage = reinterpret_cast<uint4*>(base) + (mt * kBM + row) * (BN / 8);
#pragma unroll
          for (int c = 0; c < 4; ++c)
            stage[(c0 / 8 + c) ^ (row & 7)] =
                make_uint4(pack_bf16(__uint_as_float(acc[8 * c]), __uint_as_float(acc[8 * c + 1])),
                           pack_bf16(__uint_as_float(acc[8 * c + 2]), __uint_as_float(acc[8 * c + 3])),
                           pack_bf16(__uint_as_float(acc[8 * c + 4]), __uint_as_float(acc[8 * c + 5])),
                           pack_bf16(__uint_as_float(acc[8 * c + 6]), __uint_as_float(acc[8 * c + 7])));
        }
      }
    }
    if (split == 1 && p.n_outs > 1) {
      // Coalesced stores: BN / 8 consecutive lanes write one row's BN * 2 contiguous bytes, to every
      // destination (a peer's receive buffer gets whole 128-byte lines instead of 16-byte fragments).
      asm volatile("bar.sync 1, 128;\n" ::: "memory");         // the four epilogue warps only
      constexpr int kChunks = BN / 8, kRowsPerPass = 128 / kChunks;
      const int t = tid - 64, chunk = t % kChunks;
      for (int r = t / kChunks; r < MT * kBM; r += kRowsPerPass) {
        const int64_t out_row = (int64_t)m0 + r;
        if (out_row >= p.m) break;                           // rows only grow with r
        const uint4 v = reinterpret_cast<const uint4*>(base)[r * kChunks + (chunk ^ (r & 7))];
        for (int o = 0; o < p.n_outs; ++o)
          *reinterpret_cast<uint4*>(p.outs[o] + out_row * p.out_stride + n0 + chunk * 8) = v;
      }
    }
  }
  if (split > 1) {
    cluster_sync();                                          // every CTA's accumulators are parked
    if (warp >= 2) {
      // This CTA adds up columns [part * width, (part + 1) * width) of the block.  A thread takes four
      // consecutive rows (one 16-byte load per column and CTA, a warp reads 512 contiguous bytes) of
      // every fourth 8-column group.
      const int width = BN / split, c_first = part * width;
      const int t = tid - 64, rows4 = (t & 31) * 4, group = t >> 5;
      uint32_t peer[kMaxSplit];
#pragma unroll
      for (int s = 0; s < kMaxSplit; ++s) peer[s] = peer_smem_addr(smem_u32(park), (uint32_t)min(s, split - 1));
#pragma unroll 1
      for (int mt = 0; mt < MT; ++mt) {
#pragma unroll 1
        for (int c0 = group * 8; c0 < width; c0 += 32) {
          float4 sum[8];
          const uint32_t offset = (uint32_t)(((mt * BN + c_first + c0) * kBM + rows4) * 4);
#pragma unroll
          for (int c = 0; c < 8; ++c) sum[c] = ld_cluster_f32x4(peer[0] + offset + c * kBM * 4);
#pragma unroll
          for (int s = 1; s < kMaxSplit; ++s) {
            if (s < split) {
              float4 next[8];
#pragma unroll
              for (int c = 0; c < 8; ++c) next[c] = ld_cluster_f32x4(peer[s] + offset + c * kBM * 4);
#pragma unroll
              for (int c = 0; c < 8; ++c) {
                sum[c].x = __fadd_rn(sum[c].x, next[c].x);
                sum[c].y = __fadd_rn(sum[c].y, next[c].y);
                sum[c].z = __fadd_rn(sum[c].z, next[c].z);
                sum[c].w = __fadd_rn(sum[c].w, next[c].w);
              }
            }
          }
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const int64_t out_row = (int64_t)m0 + mt * kBM + rows4 + r;
            if (out_row >= p.m) break;
            const float* f = reinterpret_cast<const float*>(sum) + r;          // element r of every column's float4
            const uint4 packed = make_uint4(pack_bf16(f[0], f[4]), pack_bf16(f[8], f[12]), pack_bf16(f[16], f[20]),
                                            pack_bf16(f[24], f[28]));
            for (int o = 0; o < p.n_outs; ++o)
              *reinterpret_cast<uint4*>(p.outs[o] + out_row * p.out_stride + n0 + c_first + c0) = packed;
          }
        }
      }
    }
    cluster_sync();                                          // nobody leaves while its memory is still being read
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0 && sh->abort && p.status) atomicOr(p.status, (int)GK_DEV_WAIT_EXPIRED);
  __syncwarp();
  if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(T::kTmemCols));
}

// Row-major [rows, cols] bf16 matrix with a row stride, boxes of 64 columns x box_rows rows.
bool make_matrix_map(CUtensorMap* map, const void* data, int64_t rows, int64_t cols, int64_t row_stride, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)row_stride * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(data), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int MT, int BN>
int launch_linear(const LinearParams& p, const CUtensorMap& map_a, const CUtensorMap& map_w, int split, cudaStream_t stream) {
  using T = LinearTile<MT, BN>;
  if (split > 1 && !T::kCanSplit) return GK_ERR_UNSUPPORTED;
  static std::atomic<bool> configured[64];
  const int ready = opt_in_shared_memory(linear_tc_kernel<MT, BN>, T::kSmemBytes, configured);
  if (ready != GK_OK) return ready;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((unsigned)(p.n / BN), (unsigned)((p.m + kBM * MT - 1) / (kBM * MT)), (unsigned)split);
  config.blockDim = dim3(kLinearThreads);
  config.dynamicSmemBytes = T::kSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute cluster;
  cluster.id = cudaLaunchAttributeClusterDimension;
  cluster.val.clusterDim.x = 1;
  cluster.val.clusterDim.y = 1;
  cluster.val.clusterDim.z = (unsigned)split;
  config.attrs = &cluster;
  config.numAttrs = 1;
  if (cudaLaunchKernelEx(&config, linear_tc_kernel<MT, BN>, p, map_a, map_w) != cudaSuccess) return check_launch();
  return check_launch();
}

// Block width and K cut, from a cost model fitted to measurements on B200: an SM takes in operand
// boxes at about 76 GB/s whatever the box sizes, a wave of CTAs therefore costs
// k-steps x stage bytes / 76 GB/s, and summing a cluster's accumulators through distributed shared
// memory costs a few microseconds once.
struct LinearChoice {
  int bn, split;
};
LinearChoice choose_linear(int64_t m, int64_t n, int64_t k, int mt, int sms) {
  const int64_t m_blocks = (m + kBM * mt - 1) / (kBM * mt), k_steps = k / kBK;
  LinearChoice best{64, 1};
  double best_us = 1e30;
  for (int bn = 256; bn >= 64; bn /= 2) {
    if (n % bn) continue;
    for (int split = 1; split <= kMaxSplit; split *= 2) {
      if (split > 1 && (bn / split < 32 || k_steps / split < 4 || mt * bn > 256)) break;
      const int64_t ctas = (n / bn) * m_blocks * split, waves = (ctas + sms - 1) / sms;
      const double stage_kb = mt * 16.0 + bn / 8.0;
      const double us = (double)waves * (double)((k_steps + split - 1) / split) * stage_kb * (1.0 / 76.0) +
                        (split > 1 ? kSplitOverheadUs : 0.0);
      if (us < best_us) {
        best_us = us;
        best = LinearChoice{bn, split};
      }
    }
  }
  return best;
}

}  // namespace
}  // namespace gk

extern "C" int gk_oproj_bf16(const void* a, int64_t a_row_stride, const void* weight, int64_t weight_row_stride,
                             int64_t m, int64_t n, int64_t k, void* const* outs, int n_outs, int64_t out_row_stride,
                             int32_t* status, gk_stream_t stream) {
  using namespace gk;
  if (m == 0) return GK_OK;
  if (!a || !weight || !outs || n_outs < 1 || n_outs > GK_MAX_OUTPUTS || m < 0 || n <= 0 || k <= 0)
    return GK_ERR_INVALID_ARGUMENT;
  if (n % 64 || k % kBK || m > INT32_MAX || n > INT32_MAX || k > INT32_MAX || (m + 255) / 256 > 65535)
    return GK_ERR_UNSUPPORTED;
  if (((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(weight)) & 15) || (a_row_stride & 7) ||
      (weight_row_stride & 7) || (out_row_stride & 7) || a_row_stride < k || weight_row_stride < k || out_row_stride < n)
    return GK_ERR_INVALID_ARGUMENT;
  LinearParams p{};
  for (int o = 0; o < n_outs; ++o) {
    if (!outs[o] || (reinterpret_cast<uintptr_t>(outs[o]) & 15)) return GK_ERR_INVALID_ARGUMENT;
    p.outs[o] = static_cast<unsigned short*>(outs[o]);
  }
  p.n_outs = n_outs;
  p.out_stride = out_row_stride;
  p.m = (int)m;
  p.n = (int)n;
  p.k = (int)k;
  p.status = status;
  static int sms[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return check_launch();
  if (!sms[device] && cudaDeviceGetAttribute(&sms[device], cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
    return check_launch();
  const int mt = m > kBM ? 2 : 1;
  const LinearChoice choice = choose_linear(m, n, k, mt, sms[device]);
  const int bn = choice.bn, split = choice.split;
  alignas(64) CUtensorMap map_a, map_w;
  memset(&map_a, 0, sizeof(map_a));
  memset(&map_w, 0, sizeof(map_w));
  if (!make_matrix_map(&map_a, a, m, k, a_row_stride, kBM) || !make_matrix_map(&map_w, weight, n, k, weight_row_stride, bn))
    return GK_ERR_UNSUPPORTED;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (bn == 256) return mt == 2 ? launch_linear<2, 256>(p, map_a, map_w, split, s) : launch_linear<1, 256>(p, map_a, map_w, split, s);
  if (bn == 128) return mt == 2 ? launch_linear<2, 128>(p, map_a, map_w, split, s) : launch_linear<1, 128>(p, map_a, map_w, split, s);
  return mt == 2 ? launch_linear<2, 64>(p, map_a, map_w, split, s) : launch_linear<1, 64>(p, map_a, map_w, split, s);
}
