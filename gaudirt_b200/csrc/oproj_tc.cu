// Output projection of the attention block on the 5th-generation tensor cores:
//   out[M, N] = bf16( A[M, K] . W[N, K]^T )      bf16 operands, fp32 accumulation in TMEM
// with A the attention output of this rank's heads and W this rank's column slice of the o_proj
// weight (row-parallel linear: every rank produces a partial [M, N] that the rank-ordered sum
// behind it adds up).  The result can be written to several destinations at once -- the same
// slot of every tensor-parallel peer's receive buffer -- so the exchange rides on the epilogue's
// stores and no separate collective moves the partials.
//
// One CTA owns a [128 * MT] x 64 block of the output (MT = 1 or 2 accumulators, 64 TMEM columns
// each) and walks K in steps of 64:
//   warp 0     one thread issues the TMA loads of a stage: MT boxes [128 x 64] of A and one box
//              [64 x 64] of W, 128-byte swizzle, no multicast; rows past M are zero-filled by TMA
//   warp 1     one thread issues tcgen05.mma.kind::f16 (M 128, N 64, K 16) four times per box and
//              commits the stage back to the loader, finally the accumulators to the epilogue
//   warps 2-5  epilogue: tcgen05.ld of the thread's row, rounding to bf16, 128-byte row segments
//              stored to every destination
// Every mbarrier wait is bounded; on expiry the CTA raises GK_DEV_WAIT_EXPIRED, frees its TMEM and
// returns.
#include "tc_common.cuh"

#include <string.h>

namespace gk {
namespace {

constexpr int kBM = 128, kBN = 64, kBK = 64;
constexpr int kABytes = kBM * kBK * 2;   // 16 KiB
constexpr int kWBytes = kBN * kBK * 2;   //  8 KiB
constexpr int kLinearThreads = 192;
constexpr int kMaxStages = 8;

template <int MT>
struct LinearTile {
  static constexpr int kStageBytes = MT * kABytes + kWBytes;
  static constexpr int kStages = MT == 1 ? 8 : 5;
  static constexpr int kTmemCols = MT == 1 ? 64 : 128;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /* alignment slack */ + 256 /* barriers */;
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

template <int MT>
__global__ void __launch_bounds__(kLinearThreads, 1)
linear_tc_kernel(const LinearParams p, const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w) {
  using T = LinearTile<MT>;
  extern __shared__ unsigned char raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  LinearShared* sh = reinterpret_cast<LinearShared*>(base + T::kStages * T::kStageBytes);
  const uint32_t tiles = smem_u32(base);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * kBN, m0 = blockIdx.y * (kBM * MT);
  const int k_steps = p.k / kBK;

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
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) tma_load_box(dst + mt * kABytes, &map_a, kt * kBK, m0 + mt * kBM, &sh->full[s]);
        tma_load_box(dst + MT * kABytes, &map_w, kt * kBK, n0, &sh->full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(kBN);
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
            umma_bf16(tmem + mt * kBN, umma_desc(a + mt * kABytes + k4 * 32, 16, 1024), umma_desc(w + k4 * 32, 16, 1024),
                      idesc, (kt > 0 || k4 > 0) ? 1u : 0u);
        umma_commit(&sh->empty[s]);
      }
      if (alive) umma_commit(&sh->done);
    }
  } else {
    const bool alive = __all_sync(0xffffffffu, bar_wait(&sh->done, 0, &sh->abort));
    if (alive) {
      tc_fence_after();
      const int quarter = warp & 3;                 // the TMEM lanes a warp may read: 32 * (warp % 4) ...
      const int row = quarter * 32 + lane;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int64_t out_row = (int64_t)m0 + mt * kBM + row;
        uint32_t packed[kBN / 2];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t acc[32];
          tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + mt * kBN + half * 32, acc);
#pragma unroll
          for (int c = 0; c < 16; ++c)
            packed[half * 16 + c] = pack_bf16(__uint_as_float(acc[2 * c]), __uint_as_float(acc[2 * c + 1]));
        }
        if (out_row < p.m) {
          for (int o = 0; o < p.n_outs; ++o) {
            uint4* dst = reinterpret_cast<uint4*>(p.outs[o] + out_row * p.out_stride + n0);
#pragma unroll
            for (int c = 0; c < kBN / 8; ++c)
              dst[c] = make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
          }
        }
      }
    }
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

template <int MT>
int launch_linear(const LinearParams& p, const CUtensorMap& map_a, const CUtensorMap& map_w, cudaStream_t stream) {
  using T = LinearTile<MT>;
  static bool configured[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return check_launch();
  if (device < 0 || device >= 64 || !configured[device]) {
    if (cudaFuncSetAttribute(linear_tc_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, T::kSmemBytes) != cudaSuccess)
      return check_launch();
    if (device >= 0 && device < 64) configured[device] = true;
  }
  const dim3 grid((unsigned)(p.n / kBN), (unsigned)((p.m + kBM * MT - 1) / (kBM * MT)));
  linear_tc_kernel<MT><<<grid, kLinearThreads, T::kSmemBytes, stream>>>(p, map_a, map_w);
  return check_launch();
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
  if (n % kBN || k % kBK || m > INT32_MAX || n > INT32_MAX || k > INT32_MAX || (m + 255) / 256 > 65535)
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
  alignas(64) CUtensorMap map_a, map_w;
  memset(&map_a, 0, sizeof(map_a));
  memset(&map_w, 0, sizeof(map_w));
  if (!make_matrix_map(&map_a, a, m, k, a_row_stride, kBM) || !make_matrix_map(&map_w, weight, n, k, weight_row_stride, kBN))
    return GK_ERR_UNSUPPORTED;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  return m > kBM ? launch_linear<2>(p, map_a, map_w, s) : launch_linear<1>(p, map_a, map_w, s);
}
