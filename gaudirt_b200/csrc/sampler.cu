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

constexpr int kRowThreads = 512;        // several rows share an SM, so one row's barriers hide behind another's loads

template <typename T>
__device__ __forceinline__ float load_logit(const T* row, int64_t i);
template <>
__device__ __forceinline__ float load_logit<float>(const float* row, int64_t i) { return row[i]; }
template <>
__device__ __forceinline__ float load_logit<unsigned short>(const unsigned short* row, int64_t i) {
  return __uint_as_float((uint32_t)row[i] << 16);
}

template <typename T>
__device__ __forceinline__ void unpack16(const uint4& q, float (&v)[16 / sizeof(T)]);
template <>
__device__ __forceinline__ void unpack16<float>(const uint4& q, float (&v)[4]) {
  v[0] = __uint_as_float(q.x); v[1] = __uint_as_float(q.y); v[2] = __uint_as_float(q.z); v[3] = __uint_as_float(q.w);
}
template <>
__device__ __forceinline__ void unpack16<unsigned short>(const uint4& q, float (&v)[8]) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    v[2 * e] = __uint_as_float(w[e] << 16);
    v[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
  }
}

// Visits every (index, value) of a row once, the whole CTA together: 16-byte loads when the row
// starts on a 16-byte boundary, element loads otherwise and for the tail.  The order of visits is
// not index order; every reduction built on it is order-independent.
template <typename T, typename F>
__device__ __forceinline__ void for_each_logit(const T* row, int64_t cols, F&& visit) {
  constexpr int V = 16 / sizeof(T);
  int64_t done = 0;
  if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    // Four loads are requested before the first is used: a row is read by one CTA, so memory
    // latency has to be covered by loads in flight per thread.
    const int64_t vectors = cols / V, stride = blockDim.x;
    int64_t v = threadIdx.x;
    for (; v + 3 * stride < vectors; v += 4 * stride) {
      uint4 q[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) q[u] = *reinterpret_cast<const uint4*>(row + (v + u * stride) * V);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float x[V];
        unpack16<T>(q[u], x);
#pragma unroll
        for (int e = 0; e < V; ++e) visit((v + u * stride) * V + e, x[e]);
      }
    }
    for (; v < vectors; v += stride) {
      float x[V];
      unpack16<T>(*reinterpret_cast<const uint4*>(row + v * V), x);
#pragma unroll
      for (int e = 0; e < V; ++e) visit(v * V + e, x[e]);
    }
    done = vectors * V;
  }
  for (int64_t i = done + threadIdx.x; i < cols; i += blockDim.x) visit(i, load_logit(row, i));
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

// CTA-wide exclusive prefix sum in thread order; *total gets the sum over all threads.
__device__ unsigned long long block_exclusive_scan_u64(unsigned long long v, unsigned long long* scratch,
                                                       unsigned long long* total) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned long long incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  __syncthreads();
  if (lane == 31) scratch[warp] = incl;
  __syncthreads();
  unsigned long long mine = lane < (int)(blockDim.x >> 5) ? scratch[lane] : 0ull, across = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long up = __shfl_up_sync(0xffffffffu, across, o);
    if (lane >= o) across += up;
  }
  *total = __shfl_sync(0xffffffffu, across, 31);
  return __shfl_sync(0xffffffffu, across - mine, warp) + incl - v;
}

// (key << 32 | ~index): the maximum is the largest key at the lowest index.
template <typename T>
__device__ unsigned long long row_argmax(const T* row, int64_t cols, bool nan_is_lowest, unsigned long long* scratch) {
  // Per thread: a float maximum with its index (a thread meets its columns in increasing index
  // order, so a strict comparison keeps the first of equals) and the first NaN; the 64-bit key is
  // only built once per thread, for the reduction across the CTA.
  float top = 0.f;
  int top_at = 0x7fffffff, nan_at = 0x7fffffff;
  for_each_logit(row, cols, [&](int64_t i, float f) {
    if (f != f) {
      if (!nan_is_lowest) {
        nan_at = min(nan_at, (int)i);
        return;
      }
      f = -CUDART_INF_F;
    }
    if (f > top || top_at == 0x7fffffff) {
      top = f;
      top_at = (int)i;
    }
  });
  unsigned long long best = 0;
  if (nan_at != 0x7fffffff) best = (0xffffffffull << 32) | (0xffffffffu - (uint32_t)nan_at);
  else if (top_at != 0x7fffffff) best = ((unsigned long long)order_key(top) << 32) | (0xffffffffu - (uint32_t)top_at);
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
// keep their bits: 16-byte groups without a banned column are neither read nor written.
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
    if (banned == 0u) continue;
    if ((reinterpret_cast<uintptr_t>(out + c0) & 15) == 0 && c0 + 32 <= cols) {
      // 16-byte groups: a fully banned group is stored, a mixed one is read, blended and stored back
      // (scattered 2- and 4-byte stores cost more than reading the sectors they would half-fill)
      constexpr int V = 16 / sizeof(T);
      const uint32_t fill = sizeof(T) == 2 ? 0xff80ff80u : 0xff800000u;
      uint4* dst = reinterpret_cast<uint4*>(out + c0);
#pragma unroll
      for (int g = 0; g < 32 / V; ++g) {
        const uint32_t bits = (banned >> (g * V)) & ((1u << V) - 1u);
        if (bits == 0u) continue;
        uint4 q = make_uint4(fill, fill, fill, fill);
        if (bits != (1u << V) - 1u) {
          q = dst[g];
          uint32_t w[4] = {q.x, q.y, q.z, q.w};
          if (sizeof(T) == 2) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              if (bits >> (2 * e) & 1u) w[e] = (w[e] & 0xffff0000u) | 0xff80u;
              if (bits >> (2 * e + 1) & 1u) w[e] = (w[e] & 0x0000ffffu) | 0xff800000u;
            }
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (bits >> e & 1u) w[e] = 0xff800000u;
          }
          q = make_uint4(w[0], w[1], w[2], w[3]);
        }
        dst[g] = q;
      }
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

struct SampleShared {
  unsigned long long scratch[32];
  unsigned int mass_lo[kBins], mass_hi[kBins];   // 64-bit bin masses as two words: 32-bit shared atomics are native
  unsigned int count[kBins];
  unsigned long long found_mass;
  unsigned int found_prefix;
};

__device__ __forceinline__ float weight_of(float f, float top, float inv_temp, bool nan_low) {
  if (f != f) f = nan_low ? -CUDART_INF_F : top;            // an unfiltered NaN is treated like the maximum
  return __expf((f - top) * inv_temp);                       // in [0, 1]; exp(-inf) = 0
}
// floor(w * 2^40) for 0 <= w <= 1, from the bits of w (a float -> 64-bit integer conversion
// instruction runs at a small fraction of the rate of these few integer operations).
__device__ __forceinline__ unsigned long long mass_of(float w) {
  const uint32_t bits = __float_as_uint(w);
  const int exponent = (int)(bits >> 23);                    // w >= 0: no sign bit
  if (exponent == 0) return 0ull;                            // zero and subnormals: below 2^-40 anyway
  const unsigned long long mantissa = (bits & 0x7fffffu) | 0x800000u;
  const int shift = exponent - 110;                          // (exponent - 127) + 40 - 23
  return shift >= 0 ? mantissa << shift : (shift > -24 ? mantissa >> -shift : 0ull);
}

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
      sh->mass_lo[b] = 0;
      sh->mass_hi[b] = 0;
      sh->count[b] = 0;
    }
    __syncthreads();
    for_each_logit(row, cols, [&](int64_t, float f) {
      const float w = weight_of(f, top, inv_temp, nan_low);
      const uint32_t u = __float_as_uint(w);
      if (u < floor_bits || (u & above) != prefix) return;
      const uint32_t digit = (u >> shift) & ((1u << bits) - 1u);
      if (BY_MASS) {
        // exact 64-bit add out of 32-bit atomics: the carry out of the low word is counted separately
        const unsigned long long mass = mass_of(w);
        const uint32_t low = (uint32_t)mass, high = (uint32_t)(mass >> 32);
        if (low) {
          const uint32_t before = atomicAdd(&sh->mass_lo[digit], low);
          if (before > 0xffffffffu - low) atomicAdd(&sh->mass_hi[digit], 1u);
        }
        if (high) atomicAdd(&sh->mass_hi[digit], high);
      } else {
        atomicAdd(&sh->count[digit], 1u);
      }
    });
    __syncthreads();
    // Find the bin, counted from the top, at which the running total first reaches the target: thread t
    // owns the four bins below 4t from the top, an exclusive scan over threads gives what lies above
    // them.  (No thread finds one when everything together falls short: bin 0 is taken then.)
    {
      const int n_bins = 1 << bits;
      unsigned long long value[4], mine = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int b = n_bins - 1 - (4 * (int)threadIdx.x + k);
        value[k] = b < 0 ? 0ull
                         : (BY_MASS ? ((unsigned long long)sh->mass_hi[b] << 32) | sh->mass_lo[b] : (unsigned long long)sh->count[b]);
        mine += value[k];
      }
      unsigned long long total;
      unsigned long long over = block_exclusive_scan_u64(mine, sh->scratch, &total);
      if (threadIdx.x == 0) {
        const unsigned long long lowest =
            BY_MASS ? ((unsigned long long)sh->mass_hi[0] << 32) | sh->mass_lo[0] : (unsigned long long)sh->count[0];
        sh->found_prefix = prefix;
        sh->found_mass = total - lowest;
      }
      __syncthreads();
      if (over < target && target <= over + mine) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (over < target && target <= over + value[k]) {
            sh->found_prefix = prefix | ((uint32_t)(n_bins - 1 - (4 * (int)threadIdx.x + k)) << shift);
            sh->found_mass = over;
          }
          over += value[k];
        }
      }
    }
    __syncthreads();
    prefix = sh->found_prefix;
    target -= sh->found_mass;                               // what is still needed from inside the chosen bin
    __syncthreads();
  }
  return prefix > floor_bits ? prefix : floor_bits;
}

// bf16 rows only: a row has at most 65 536 distinct values, and the thresholds of top-k / top-p sit
// among the largest of them.  One pass histograms count and mass over the 2 048 distinct bf16 values
// just below the maximum (bin = distance in order-preserving 16-bit keys; every element of a bin
// has the same weight, so a bin boundary is an exact threshold) and sums the rest as a tail; the
// k-th largest weight and the top-p cut are then prefix searches over the bins.  Returns false when
// a threshold falls into the tail, and the caller runs the general three-pass radix selects.
__device__ __forceinline__ uint32_t key_bf16(uint32_t bits) {          // bits of a non-NaN bf16, -0 already folded into +0
  return (bits & 0x8000u) ? (~bits & 0xffffu) : (bits | 0x8000u);
}
__device__ __forceinline__ float value_of_key_bf16(uint32_t key) {
  const uint32_t bits = (key & 0x8000u) ? (key & 0x7fffu) : (~key & 0xffffu);
  return __uint_as_float(bits << 16);
}

__device__ bool bf16_thresholds(const unsigned short* row, int64_t cols, float top, float inv_temp, bool nan_low, long long k,
                                float top_p, float min_p, SampleShared* sh, uint32_t* floor_out) {
  const uint32_t top_bits = __float_as_uint(top) >> 16;
  const uint32_t top_key = key_bf16(top_bits == 0x8000u ? 0u : top_bits);
  for (int b = threadIdx.x; b < kBins; b += blockDim.x) {
    sh->mass_lo[b] = 0;
    sh->mass_hi[b] = 0;
    sh->count[b] = 0;
  }
  __syncthreads();
  unsigned long long tail_count = 0, tail_mass = 0;
  for_each_logit(row, cols, [&](int64_t, float f) {
    if (f != f) {                                            // an unfiltered NaN weighs like the maximum (bin 0)
      if (nan_low) {
        ++tail_count;
        return;
      }
      f = top;
    }
    uint32_t bits = __float_as_uint(f) >> 16;
    if (bits == 0x8000u) bits = 0u;
    const uint32_t d = top_key - key_bf16(bits);
    const unsigned long long mass = mass_of(weight_of(f, top, inv_temp, nan_low));
    if (d < (uint32_t)kBins) {
      atomicAdd(&sh->count[d], 1u);
      const uint32_t low = (uint32_t)mass, high = (uint32_t)(mass >> 32);
      if (low) {
        const uint32_t before = atomicAdd(&sh->mass_lo[d], low);
        if (before > 0xffffffffu - low) atomicAdd(&sh->mass_hi[d], 1u);
      }
      if (high) atomicAdd(&sh->mass_hi[d], high);
    } else {
      ++tail_count;
      tail_mass += mass;
    }
  });
  __syncthreads();
  tail_count = block_sum_u64(tail_count, sh->scratch);
  tail_mass = block_sum_u64(tail_mass, sh->scratch);

  // Thread t owns bins 4t .. 4t+3 (weights fall as the bin index grows).
  unsigned long long count[4], mass[4], my_count = 0, my_mass = 0;
  uint32_t wbits[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int b = 4 * (int)threadIdx.x + q;
    count[q] = b < kBins ? sh->count[b] : 0ull;
    mass[q] = b < kBins ? ((unsigned long long)sh->mass_hi[b] << 32) | sh->mass_lo[b] : 0ull;
    wbits[q] = b < kBins && (uint32_t)b <= top_key ? __float_as_uint(weight_of(value_of_key_bf16(top_key - b), top, inv_temp, false)) : 0u;
    my_count += count[q];
    my_mass += mass[q];
  }
  unsigned long long binned_count, binned_mass;
  const unsigned long long count_before = block_exclusive_scan_u64(my_count, sh->scratch, &binned_count);
  const unsigned long long mass_before = block_exclusive_scan_u64(my_mass, sh->scratch, &binned_mass);

  // top-k: the bin in which the running count first reaches k
  uint32_t floor_bits = min_p > 0.f ? __float_as_uint(fminf(min_p, 1.0f)) : 0u;
  const bool has_k = k >= 1 && k < cols;
  if (threadIdx.x == 0) sh->found_prefix = 0xffffffffu;      // "not found"
  __syncthreads();
  if (has_k) {
    unsigned long long run = count_before;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (run < (unsigned long long)k && (unsigned long long)k <= run + count[q]) sh->found_prefix = wbits[q];
      run += count[q];
    }
  }
  __syncthreads();
  if (has_k) {
    if (sh->found_prefix == 0xffffffffu) return false;       // the k-th largest lies in the tail
    floor_bits = sh->found_prefix > floor_bits ? sh->found_prefix : floor_bits;
  }
  __syncthreads();
  // What the floor leaves: whole bins, plus the tail only when there is no floor at all.
  const uint32_t last_bin_bits =
      top_key >= (uint32_t)kBins - 1 ? __float_as_uint(weight_of(value_of_key_bf16(top_key - (kBins - 1)), top, inv_temp, false))
                                     : 0u;                   // fewer keys than bins below the maximum: nothing weighs in the tail
  if (floor_bits != 0u && floor_bits < last_bin_bits && tail_count > 0) return false;   // the floor cuts inside the tail
  if (!(top_p < 1.0f)) {
    *floor_out = floor_bits;
    return true;
  }
  unsigned long long kept_mine = 0;
#pragma unroll
  for (int q = 0; q < 4; ++q)
    if (wbits[q] >= floor_bits) kept_mine += mass[q];
  unsigned long long kept;
  const unsigned long long kept_before = block_exclusive_scan_u64(kept_mine, sh->scratch, &kept);
  const unsigned long long kept_all = kept + (floor_bits == 0u ? tail_mass : 0ull);
  if (kept_all == 0) {
    *floor_out = floor_bits;
    return true;
  }
  unsigned long long need = (unsigned long long)((double)kept_all * (double)fmaxf(top_p, 0.f));
  if (need == 0) need = 1;
  if (need > kept) return false;                             // the cut lies in the tail
  if (threadIdx.x == 0) sh->found_prefix = 0xffffffffu;
  __syncthreads();
  {
    unsigned long long run = kept_before;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const unsigned long long here = wbits[q] >= floor_bits ? mass[q] : 0ull;
      if (run < need && need <= run + here) sh->found_prefix = wbits[q];
      run += here;
    }
  }
  __syncthreads();
  const uint32_t cut = sh->found_prefix;
  __syncthreads();
  if (cut == 0xffffffffu) return false;
  *floor_out = cut > floor_bits ? cut : floor_bits;
  (void)mass_before;
  (void)binned_count;
  (void)binned_mass;
  return true;
}

template <typename T>
__device__ __forceinline__ bool fast_thresholds(const T*, int64_t, float, float, bool, long long, float, float, SampleShared*,
                                                uint32_t*) {
  return false;                                              // fp32 rows: the general path
}
template <>
__device__ __forceinline__ bool fast_thresholds<unsigned short>(const unsigned short* row, int64_t cols, float top, float inv_temp,
                                                                bool nan_low, long long k, float top_p, float min_p,
                                                                SampleShared* sh, uint32_t* floor_out) {
  return bf16_thresholds(row, cols, top, inv_temp, nan_low, k, top_p, min_p, sh, floor_out);
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
  const float top_p = top_ps[r];
  const bool filtered = (k >= 1 && k < cols) || top_p < 1.0f;
  if (filtered && !fast_thresholds<T>(row, cols, top, inv_temp, nl, k, top_p, min_p, &sh, &floor_bits)) {
    __syncthreads();
    floor_bits = min_p > 0.f ? __float_as_uint(fminf(min_p, 1.0f)) : 0u;
    if (k >= 1 && k < cols) {
      const uint32_t kth = select_threshold<T, false>(row, cols, top, inv_temp, nl, 0u, (unsigned long long)k, &sh);
      floor_bits = kth > floor_bits ? kth : floor_bits;
    }
    if (top_p < 1.0f) {
      unsigned long long kept = 0;
      for_each_logit(row, cols, [&](int64_t, float f) {
        const float w = weight_of(f, top, inv_temp, nl);
        if (__float_as_uint(w) >= floor_bits) kept += mass_of(w);
      });
      kept = block_sum_u64(kept, sh.scratch);
      if (kept > 0) {
        const unsigned long long need = (unsigned long long)((double)kept * (double)fmaxf(top_p, 0.f));
        floor_bits = select_threshold<T, true>(row, cols, top, inv_temp, nl, floor_bits, need > 0 ? need : 1, &sh);
      }
    }
  }

  // Inverse transform in index order.  Thread t owns a contiguous run of columns, so an exclusive scan
  // of the threads' kept masses is the running mass in index order; its total is the kept mass, the
  // thread whose run contains u * kept walks it.
  constexpr int V = 16 / sizeof(T);
  const bool aligned = (reinterpret_cast<uintptr_t>(row) & 15) == 0;
  const int64_t run = ((cols + blockDim.x - 1) / blockDim.x + V - 1) / V * V;
  const int64_t lo = (int64_t)threadIdx.x * run, hi = lo + run < cols ? lo + run : cols;
  auto kept_mass = [&](float f) {
    const float w = weight_of(f, top, inv_temp, nl);
    return __float_as_uint(w) >= floor_bits ? mass_of(w) : 0ull;
  };
  auto for_my_run = [&](auto&& visit) {                      // visit(index, value) in increasing index order
    int64_t i = lo;
    if (aligned) {
      for (; i + 4 * V <= hi; i += 4 * V) {                  // four loads in flight
        uint4 q[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) q[u] = *reinterpret_cast<const uint4*>(row + i + u * V);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          float x[V];
          unpack16<T>(q[u], x);
#pragma unroll
          for (int e = 0; e < V; ++e) visit(i + u * V + e, x[e]);
        }
      }
    }
    for (; i < hi; ++i) visit(i, load_logit(row, i));
  };
  unsigned long long mine = 0;
  for_my_run([&](int64_t, float f) { mine += kept_mass(f); });
  unsigned long long kept;
  const unsigned long long before = block_exclusive_scan_u64(mine, sh.scratch, &kept);
  if (kept == 0) {
    if (threadIdx.x == 0) out[r] = greedy;
    return;
  }
  unsigned long long seed = seeds ? (unsigned long long)seeds[r] : splitmix64(base_seed + (unsigned long long)r);
  if (seeds && positions) {
    const unsigned long long p = positions_wide ? (unsigned long long)static_cast<const int64_t*>(positions)[r]
                                                : (unsigned long long)(long long)static_cast<const int32_t*>(positions)[r];
    seed = splitmix64(seed ^ splitmix64(p));
  }
  const unsigned long long target = __umul64hi(splitmix64(seed), kept);      // uniform in [0, kept)
  if (target >= before && target < before + mine) {                          // exactly one thread
    unsigned long long at = before;
    int found = greedy;
    bool done = false;
    for_my_run([&](int64_t i, float f) {
      const unsigned long long mass = kept_mass(f);
      if (!done && target < at + mass) {
        found = (int)i;
        done = true;
      }
      at += mass;
    });
    out[r] = found;
  }
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
