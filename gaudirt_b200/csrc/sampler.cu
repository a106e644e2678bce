// After the LM head: grammar bitmask, vocabulary argmax and temperature / top-k / top-p / min-p
// sampling over [rows, vocabulary] logits (src/bridge/sampler_vocab.cpp:333-485,
// src/bridge/argmax_vocab.cpp).  All three are single passes (or a fixed number of passes) of one
// CTA over a row that stays in L2 after the first pass; nothing here allocates or synchronises.
//
// Sampling semantics.  With w_i = exp((x_i - max x) / temperature) (NaN counted as -inf when asked):
//   top-k   keeps every w_i >= the k-th largest w          (ties at the threshold stay)
//   top-p   keeps, of those, every w_i >= the largest t with mass{w >= t} >= top_p * mass{kept}
//   min-p   keeps w_i >= min_p (w of the most likely token is 1)
// i.e. one threshold T = max of the three; a token is then drawn from {w_i >= T} in proportion to w
// by inverse transform in index order.  temperature == 0 is the argmax (lowest index on ties).
// Masses are summed as 2^-40 fixed point in 64-bit integers, so the result does not depend on the
// order threads add in: the same (seed, position) gives the same token.  The uniform variate comes
// from splitmix64(seed ^ splitmix64(position)) as in the reference's host set-up
// (src/bridge/sampler_vocab.cpp:272-279), evaluated on the device instead.
#include "gk_common.cuh"

#include <math_constants.h>

#include <algorithm>

namespace gk {
namespace {

constexpr int kRowThreads = 1024;

template <typename T>
__device__ __forceinline__ float load_logit(const T* row, int64_t i);
template <>
__device__ __forceinline__ float load_logit<float>(const float* row, int64_t i) { return row[i]; }
template <>
__device__ __forceinline__ float load_logit<unsigned short>(const unsigned short* row, int64_t i) {
  return __uint_as_float((uint32_t)row[i] << 16);
}

// Order-preserving key of a float for unsigned comparison; NaN sorts above +inf (torch.argmax
// treats NaN as the maximum), -0 and +0 tie.
__device__ __forceinline__ uint32_t order_key(float f) {
  if (f != f) return 0xffffffffu;
  const uint32_t b = __float_as_uint(f + 0.0f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// CTA-wide maximum of a 64-bit key; every thread gets the result.
__device__ unsigned long long block_max_u64(unsigned long long v, unsigned long long* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, o);
    v = other > v ? other : v;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  unsigned long long best = 0;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) best = scratch[w] > best ? scratch[w] : best;
  return best;
}

__device__ unsigned long long block_sum_u64(unsigned long long v, unsigned long long* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  unsigned long long total = 0;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) total += scratch[w];
  return total;
}

// (key << 32 | ~index): the maximum is the largest key at the lowest index.
template <typename T>
__device__ unsigned long long row_argmax(const T* row, int64_t cols, bool nan_is_lowest, unsigned long long* scratch) {
  unsigned long long best = 0;
  for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) {
    float f = load_logit(row, i);
    if (nan_is_lowest && f != f) f = -CUDART_INF_F;
    const unsigned long long key = ((unsigned long long)order_key(f) << 32) | (0xffffffffu - (uint32_t)i);
    best = key > best ? key : best;
  }
  return block_max_u64(best, scratch);
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads) argmax_kernel(const T* __restrict__ logits, int64_t cols, int64_t row_stride,
                                                             int64_t* __restrict__ out) {
  __shared__ unsigned long long scratch[32];
  const unsigned long long best = row_argmax(logits + (int64_t)blockIdx.x * row_stride, cols, false, scratch);
  if (threadIdx.x == 0) out[blockIdx.x] = (int64_t)(0xffffffffu - (uint32_t)best);
}

// ---- grammar bitmask -------------------------------------------------------------------------
// Column c of a listed row becomes -inf when c < active and bit c of the row's mask is 0, or when
// c >= active and mask_tail is set (tests/vocab_bitmask_device_smoke.py:14-33).  Allowed entries
// are not touched, so nothing is read from the logits at all.
template <typename T>
__global__ void __launch_bounds__(256) bitmask_kernel(T* __restrict__ logits, int64_t rows, int64_t cols, int64_t row_stride,
                                                      const int32_t* __restrict__ bitmask, int64_t mask_rows,
                                                      int64_t mask_words, const int32_t* __restrict__ indices,
                                                      int64_t active, int mask_tail, int32_t* __restrict__ status) {
  int64_t row = blockIdx.y;
  if (indices) {
    row = indices[blockIdx.y];
    if (row < 0 || row >= rows || row >= mask_rows) {
      if (threadIdx.x == 0 && blockIdx.x == 0 && status) atomicOr(status, (int)GK_DEV_BAD_METADATA);
      return;
    }
  }
  const uint32_t* mask = reinterpret_cast<const uint32_t*>(bitmask) + row * mask_words;
  T* out = logits + row * row_stride;
  T minus_inf;
  if (sizeof(T) == 2) *reinterpret_cast<unsigned short*>(&minus_inf) = 0xff80;
  else *reinterpret_cast<uint32_t*>(&minus_inf) = 0xff800000u;
  // One thread per 32 columns = one mask word.
  for (int64_t word = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; word * 32 < cols; word += (int64_t)gridDim.x * blockDim.x) {
    const int64_t c0 = word * 32;
    uint32_t banned;                                        // bit set: write -inf
    if (c0 >= active) banned = mask_tail ? 0xffffffffu : 0u;
    else {
      banned = ~mask[word];
      const int64_t live = active - c0;                     // columns of this word below `active`
      if (live < 32) {
        const uint32_t low = (1u << live) - 1u;
        banned = (banned & low) | (mask_tail ? ~low : 0u);
      }
    }
    if (cols - c0 < 32) banned &= (1u << (cols - c0)) - 1u;
    if (banned == 0xffffffffu && (reinterpret_cast<uintptr_t>(out + c0) & 15) == 0) {   // a whole word goes: 16-byte stores
      const uint32_t fill = sizeof(T) == 2 ? 0xff80ff80u : 0xff800000u;
      uint4* dst = reinterpret_cast<uint4*>(out + c0);
#pragma unroll
      for (int v = 0; v < (int)(32 * sizeof(T) / 16); ++v) dst[v] = make_uint4(fill, fill, fill, fill);
      continue;
    }
    while (banned) {
      const int bit = __ffs(banned) - 1;
      banned &= banned - 1;
      out[c0 + bit] = minus_inf;
    }
  }
}

// ---- sampling ----------------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
  x += 0x9e3779b97f4a7c15ull;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  return x ^ (x >> 31);
}

constexpr int kDigitBits = 11, kBins = 1 << kDigitBits;     // radix-select digit; 32 bits = 11 + 11 + 10
constexpr float kMassScale = 1099511627776.0f;              // 2^40

struct SampleShared {
  unsigned long long scratch[32];
  unsigned long long mass[kBins];
  unsigned int count[kBins];
  unsigned long long found_mass;
  unsigned int found_prefix, found_count;
  int found_index;
};

template <typename T>
__device__ __forceinline__ float weight_of(const T* row, int64_t i, float top, float inv_temp, bool nan_low) {
  float f = load_logit(row, i);
  if (f != f) f = nan_low ? -CUDART_INF_F : top;            // an unfiltered NaN is treated like the maximum
  return __expf((f - top) * inv_temp);                       // in [0, 1]; exp(-inf) = 0
}
__device__ __forceinline__ unsigned long long mass_of(float w) { return (unsigned long long)(w * kMassScale); }

// Threshold search over the bit pattern of w (non-negative floats order like unsigned integers),
// most significant digit first.  BY_MASS: the largest t with mass{floor <= w, w >= t} >= target;
// otherwise the largest t with count{w >= t} >= target (the k-th largest value).
template <typename T, bool BY_MASS>
__device__ uint32_t select_threshold(const T* row, int64_t cols, float top, float inv_temp, bool nan_low, uint32_t floor_bits,
                                     unsigned long long target, SampleShared* sh) {
  uint32_t prefix = 0;
  int shift = 32;
  for (int pass = 0; pass < 3; ++pass) {
    const int bits = pass < 2 ? kDigitBits : 32 - 2 * kDigitBits;
    shift -= bits;
    const uint32_t above = shift + bits >= 32 ? 0u : (0xffffffffu << (shift + bits));
    for (int b = threadIdx.x; b < kBins; b += blockDim.x) {
      sh->mass[b] = 0;
      sh->count[b] = 0;
    }
    __syncthreads();
    for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) {
      const float w = weight_of(row, i, top, inv_temp, nan_low);
      const uint32_t u = __float_as_uint(w);
      if (u < floor_bits || (u & above) != prefix) continue;
      const uint32_t digit = (u >> shift) & ((1u << bits) - 1u);
      if (BY_MASS) atomicAdd(&sh->mass[digit], mass_of(w));
      else atomicAdd(&sh->count[digit], 1u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {                                 // walk the bins from the top until the target is covered
      unsigned long long have = 0;
      int digit = (1 << bits) - 1;
      for (; digit > 0; --digit) {
        const unsigned long long here = BY_MASS ? sh->mass[digit] : (unsigned long long)sh->count[digit];
        if (have + here >= target) break;
        have += here;
      }
      sh->found_prefix = prefix | ((uint32_t)digit << shift);
      sh->found_mass = have;
    }
    __syncthreads();
    prefix = sh->found_prefix;
    target -= sh->found_mass;                               // what is still needed from inside the chosen bin
    __syncthreads();
  }
  return prefix > floor_bits ? prefix : floor_bits;
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads)
sample_kernel(const T* __restrict__ logits, int64_t cols, int64_t row_stride, const float* __restrict__ temperatures,
              const float* __restrict__ top_ps, const int32_t* __restrict__ top_ks, const float* __restrict__ min_ps,
              const int64_t* __restrict__ seeds, const void* __restrict__ positions, int positions_wide,
              unsigned long long base_seed, int nan_low, int32_t* __restrict__ out) {
  __shared__ SampleShared sh;
  const int64_t r = blockIdx.x;
  const T* row = logits + r * row_stride;
  const float temperature = temperatures[r];
  const unsigned long long best = row_argmax(row, cols, nan_low != 0, sh.scratch);
  const int greedy = (int)(0xffffffffu - (uint32_t)best);
  if (!(temperature > 0.f)) {
    if (threadIdx.x == 0) out[r] = greedy;
    return;
  }
  float top = load_logit(row, greedy);
  if (top != top || top == -CUDART_INF_F || top == CUDART_INF_F) {   // nothing to weigh against: the argmax it is
    if (threadIdx.x == 0) out[r] = greedy;
    return;
  }
  const float inv_temp = 1.0f / temperature;
  const bool nl = nan_low != 0;

  // min-p and top-k thresholds on w, then top-p inside what they leave.
  const float min_p = min_ps[r];
  uint32_t floor_bits = min_p > 0.f ? __float_as_uint(fminf(min_p, 1.0f)) : 0u;
  const int64_t k = top_ks[r];
  if (k >= 1 && k < cols) {
    const uint32_t kth = select_threshold<T, false>(row, cols, top, inv_temp, nl, 0u, (unsigned long long)k, &sh);
    floor_bits = kth > floor_bits ? kth : floor_bits;
  }
  unsigned long long kept = 0;
  for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) {
    const float w = weight_of(row, i, top, inv_temp, nl);
    if (__float_as_uint(w) >= floor_bits) kept += mass_of(w);
  }
  kept = block_sum_u64(kept, sh.scratch);
  const float top_p = top_ps[r];
  if (top_p < 1.0f && kept > 0) {
    const unsigned long long need = (unsigned long long)((double)kept * (double)fmaxf(top_p, 0.f));
    floor_bits = select_threshold<T, true>(row, cols, top, inv_temp, nl, floor_bits, need > 0 ? need : 1, &sh);
    kept = 0;
    for (int64_t i = threadIdx.x; i < cols; i += blockDim.x) {
      const float w = weight_of(row, i, top, inv_temp, nl);
      if (__float_as_uint(w) >= floor_bits) kept += mass_of(w);
    }
    kept = block_sum_u64(kept, sh.scratch);
  }
  if (kept == 0) {
    if (threadIdx.x == 0) out[r] = greedy;
    return;
  }

  // Inverse transform in index order: the first index whose running mass exceeds u * kept.
  unsigned long long seed = seeds ? (unsigned long long)seeds[r] : splitmix64(base_seed + (unsigned long long)r);
  if (seeds && positions) {
    const unsigned long long p = positions_wide ? (unsigned long long)static_cast<const int64_t*>(positions)[r]
                                                : (unsigned long long)(long long)static_cast<const int32_t*>(positions)[r];
    seed = splitmix64(seed ^ splitmix64(p));
  }
  const unsigned long long target = __umul64hi(splitmix64(seed), kept);      // uniform in [0, kept)
  if (threadIdx.x == 0) sh.found_index = greedy;
  unsigned long long running = 0;
  const int64_t tile = (int64_t)blockDim.x * 4;
  for (int64_t base = 0; base < cols; base += tile) {
    // thread t owns 4 consecutive columns of the tile, so index order = thread order
    unsigned long long mine[4], sum = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int64_t i = base + (int64_t)threadIdx.x * 4 + e;
      float w = 0.f;
      if (i < cols) {
        w = weight_of(row, i, top, inv_temp, nl);
        if (__float_as_uint(w) < floor_bits) w = 0.f;
      }
      mine[e] = mass_of(w);
      sum += mine[e];
    }
    // inclusive scan over threads
    unsigned long long incl = sum;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    __syncthreads();
    if (lane == 31) sh.scratch[warp] = incl;
    __syncthreads();
    unsigned long long before = 0, total = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) {
      if (w < warp) before += sh.scratch[w];
      total += sh.scratch[w];
    }
    const unsigned long long start = running + before + incl - sum;      // mass in front of this thread
    if (target >= start && target < start + sum) {
      unsigned long long at = start;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (target >= at && target < at + mine[e]) sh.found_index = (int)(base + (int64_t)threadIdx.x * 4 + e);
        at += mine[e];
      }
    }
    running += total;
    if (running > target) break;                             // uniform across the CTA
  }
  __syncthreads();
  if (threadIdx.x == 0) out[r] = sh.found_index;
}

}  // namespace
}  // namespace gk

extern "C" int gk_vocab_argmax(const void* logits, int is_f32, int64_t rows, int64_t cols, int64_t row_stride,
                               int64_t* out, gk_stream_t stream) {
  using namespace gk;
  if (rows == 0) return GK_OK;
  if (!logits || !out || rows < 0 || cols <= 0 || cols > INT32_MAX || rows > INT32_MAX || row_stride < cols)
    return GK_ERR_INVALID_ARGUMENT;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (is_f32) argmax_kernel<float><<<(unsigned)rows, kRowThreads, 0, s>>>(static_cast<const float*>(logits), cols, row_stride, out);
  else argmax_kernel<unsigned short><<<(unsigned)rows, kRowThreads, 0, s>>>(static_cast<const unsigned short*>(logits), cols, row_stride, out);
  return check_launch();
}

extern "C" int gk_apply_vocab_bitmask(void* logits, int is_f32, int64_t rows, int64_t cols, int64_t row_stride,
                                      const int32_t* bitmask, int64_t mask_rows, int64_t mask_words,
                                      const int32_t* row_indices, int64_t n_indices, int64_t active_cols, int mask_tail,
                                      int32_t* status, gk_stream_t stream) {
  using namespace gk;
  const int64_t listed = row_indices ? n_indices : rows;
  if (listed == 0 || rows == 0) return GK_OK;
  if (!logits || !bitmask || rows < 0 || cols <= 0 || cols > INT32_MAX || row_stride < cols || mask_rows <= 0 ||
      mask_words <= 0 || mask_words > INT32_MAX || listed < 0 || listed > 65535 * 32768LL || active_cols < 0 ||
      active_cols > cols || active_cols > mask_words * 32 || (!row_indices && mask_rows < rows))
    return GK_ERR_INVALID_ARGUMENT;
  if (listed > 65535) return GK_ERR_UNSUPPORTED;
  const int64_t words = (cols + 31) / 32;
  const dim3 grid((unsigned)std::min<int64_t>((words + 255) / 256, 64), (unsigned)listed);
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (is_f32)
    bitmask_kernel<float><<<grid, 256, 0, s>>>(static_cast<float*>(logits), rows, cols, row_stride, bitmask, mask_rows, mask_words,
                                               row_indices, active_cols, mask_tail, status);
  else
    bitmask_kernel<unsigned short><<<grid, 256, 0, s>>>(static_cast<unsigned short*>(logits), rows, cols, row_stride, bitmask,
                                                        mask_rows, mask_words, row_indices, active_cols, mask_tail, status);
  return check_launch();
}

extern "C" int gk_sample_vocab(const void* logits, int is_f32, int64_t rows, int64_t cols, int64_t row_stride,
                               const float* temperatures, const float* top_ps, const int32_t* top_ks, const float* min_ps,
                               const int64_t* seeds, const void* positions, int positions_are_i64, uint64_t base_seed,
                               int nan_to_neg_inf, int32_t* out, gk_stream_t stream) {
  using namespace gk;
  if (rows == 0) return GK_OK;
  if (!logits || !temperatures || !top_ps || !top_ks || !min_ps || !out || rows < 0 || rows > INT32_MAX || cols <= 0 ||
      cols > INT32_MAX || row_stride < cols || (positions && !seeds))
    return GK_ERR_INVALID_ARGUMENT;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (is_f32)
    sample_kernel<float><<<(unsigned)rows, kRowThreads, 0, s>>>(static_cast<const float*>(logits), cols, row_stride, temperatures,
                                                                top_ps, top_ks, min_ps, seeds, positions, positions_are_i64,
                                                                base_seed, nan_to_neg_inf, out);
  else
    sample_kernel<unsigned short><<<(unsigned)rows, kRowThreads, 0, s>>>(static_cast<const unsigned short*>(logits), cols,
                                                                         row_stride, temperatures, top_ps, top_ks, min_ps, seeds,
                                                                         positions, positions_are_i64, base_seed, nan_to_neg_inf,
                                                                         out);
  return check_launch();
}
