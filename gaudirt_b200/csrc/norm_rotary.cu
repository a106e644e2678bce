// Front of a decode layer: (fused residual-add) RMS norm and rotary position embedding.
//
// Both are HBM-bound elementwise/row kernels.  Every bf16 boundary of the reference (the updated
// residual, the normalised output, each rotated element) is rounded ONCE from an exactly computed
// value, which reproduces the reference's binary64 truth (tests/fused_norm_midpoint_smoke.py:32-35,
// tests/rotary_runtime_smoke.py:28-40) bit for bit wherever fp64 itself is exact:
//   * the residual add: the fp32 sum of two bf16 values, rounded again to bf16, is always the rounding
//     of the exact sum (argument at add_bf16_exact);
//   * the norm's scaling u * inv * (w + offset): a packed fp32 evaluation with a 4.1-ulp error bound
//     first; only a result within 8 ulp of a bf16 rounding boundary (a few elements in 10^4) is
//     evaluated again in binary64.  The sum of squares is exact: squares of bf16 values are exact in
//     fp32 and are added in binary64;
//   * a rotation a*cos - b*sin: an exact fp32 product plus one fused multiply-add evaluated toward -inf
//     and toward +inf, with a sticky bit when the two differ (round-to-odd), then one rounding to bf16.
//     The vector kernel does this two elements per packed instruction and without a branch (rotate_word).
//     (A round-to-nearest evaluation with the exact one only for results on a bf16 midpoint was measured
//     slower, 72 against 54 us: sums of two 16-bit products land on a midpoint about once in 500 elements,
//     so four warps in ten took the exact path for some lane.)
#include "gk_common.cuh"

#include <algorithm>

namespace gk {
namespace {

// Correctly rounded binary64 -> bf16 (nearest, ties to even) through a round-to-odd fp32.  (Integer
// versions of these two conversions were measured slower than the hardware conversions.)
__device__ __forceinline__ unsigned short bf16_from_double(double v) {
  float f = __double2float_rz(v);
  if ((double)f != v) f = __uint_as_float(__float_as_uint(f) | 1u);      // inexact: sticky (odd) bit
  return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}
__device__ __forceinline__ double bf16_to_double(unsigned short b) {
  return (double)__uint_as_float((uint32_t)b << 16);
}

// bf16(x*c - y*s) resp. bf16(x*c + y*s), rounded once from the exact value, in fp32: the first
// product of two bf16 values is exact, the fused multiply-add is evaluated toward -inf and toward
// +inf; if the two differ the result is inexact, and the one nearer zero (the truncation of the
// exact value) gets a sticky bit (round-to-odd), which makes the final rounding to bf16 the
// rounding of the exact value.  (Toward-zero against toward +inf alone would miss every inexact
// negative result: both directions give the same float there.)
__device__ __forceinline__ unsigned short rotate_pair(unsigned short x, unsigned short c, unsigned short y,
                                                      unsigned short s, bool subtract) {
  const float xf = __uint_as_float((uint32_t)x << 16), cf = __uint_as_float((uint32_t)c << 16);
  float yf = __uint_as_float((uint32_t)y << 16);
  const float sf = __uint_as_float((uint32_t)s << 16);
  if (subtract) yf = -yf;
  const float first = xf * cf;                                  // exact
  const float down = __fmaf_rd(yf, sf, first), up = __fmaf_ru(yf, sf, first);
  float r = up;                                                 // exact result (an exact zero is +0, as in round-to-nearest)
  if (down != up) r = __uint_as_float(__float_as_uint(down < 0.f ? up : down) | 1u);   // toward zero, sticky bit
  return __bfloat16_as_ushort(__float2bfloat16_rn(r));
}

// bf16(a + b) of two bf16 values, rounded once from the exact sum: the fp32 sum rounded to nearest, rounded
// again to bf16, IS that.  Two 8-bit significands more than 16 binary places apart are the only way the fp32 sum
// is inexact, and then the small operand lies entirely below bit 7 of the 24-bit result, so the low half of the
// result can never read 1000...0 (the one pattern where a second rounding could go the other way); whenever it
// does read 1000...0 the fp32 sum was exact and ties-to-even is the right answer.  (Checked against the exact
// sum over 5 x 10^9 pairs covering every finite bf16 value.)
__device__ __forceinline__ unsigned short add_bf16_exact(unsigned short a, unsigned short b) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(__fadd_rn(__uint_as_float((uint32_t)a << 16), __uint_as_float((uint32_t)b << 16))));
}
// bf16(u * inv * (w + offset)): the norm's scaling step.  Fast evaluation in fp32: four roundings
// (w + offset, inv to fp32, two products), so the result is within 4.1 ulp of the exact product as
// long as nothing is subnormal; if it is more than 8 ulp away from every bf16 midpoint (bit pattern
// ...8000 in the low half), the exact product rounds to the same bf16.  Otherwise, and for tiny or
// non-finite values, the product is formed in binary64 and rounded once.
__device__ __forceinline__ unsigned short scale_to_bf16(unsigned short u, unsigned short w, float inv32, double inv,
                                                        float offset32, double offset) {
  const float uf = __uint_as_float((uint32_t)u << 16), wf = __uint_as_float((uint32_t)w << 16);
  const float a = uf * inv32, y = a * (wf + offset32);
  const uint32_t bits = __float_as_uint(y);
  const uint32_t away = ((bits & 0xffffu) - 0x8000u + 8u) & 0xffffu;      // < 17: within 8 ulp of a midpoint
  const bool safe = away > 16u && fabsf(a) > 1e-30f && fabsf(y) > 1e-30f && fabsf(y) < 1e38f;
  if (safe || uf == 0.f) return __bfloat16_as_ushort(__float2bfloat16_rn(y));
  return bf16_from_double(bf16_to_double(u) * inv * (bf16_to_double(w) + offset));
}

// u * u as a double: the square of a bf16 value has 16 significant bits, exact in fp32.
__device__ __forceinline__ double square_bf16(unsigned short u) {
  const float f = __uint_as_float((uint32_t)u << 16);
  return (double)(f * f);
}

// ---- word-wise forms: two bf16 per 32-bit word, packed fp32x2 arithmetic, no branch per element ------------
// A chunk of 8 elements is evaluated the short way as straight-line code while a flag collects "some
// element sits where the short way cannot decide its rounding"; only then is the chunk done again the
// exact way, element by element.  That is one rarely taken branch per 16 bytes instead of one per element.
__device__ __forceinline__ float2 unpack2(uint32_t w) {
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
__device__ __forceinline__ uint32_t pack2(float2 v) {
  const __nv_bfloat162 b = __float22bfloat162_rn(v);
  return *reinterpret_cast<const uint32_t*>(&b);
}

// rotate_pair for the two elements of a word, without a branch: bf16(x*c + y*s) rounded once from the exact
// value.  The packed multiply-add is taken toward -inf and toward +inf.  If the two agree the value is exact.
// If not, they are neighbouring floats, exactly one of them has an odd bit pattern, and that one IS the
// truncation of the exact value with a sticky bit (truncation | 1 either keeps an odd truncation or steps
// an even one to its neighbour away from zero): so "the odd one of the two, else either" is round-to-odd.
// An exact zero comes out as -0 | +0, and the even-patterned -0 yields to +0.
__device__ __forceinline__ uint32_t rotate_word(float2 x, float2 c, float2 y, float2 s) {
  const float2 a = __fmul2_rn(x, c);                                   // exact
  const float2 down = __ffma2_rd(y, s, a), up = __ffma2_ru(y, s, a);
  float2 r;
  r.x = (__float_as_uint(down.x) & 1u) ? down.x : up.x;
  r.y = (__float_as_uint(down.y) & 1u) ? down.y : up.y;
  return pack2(r);
}

// u = bf16(a + b) for the 4 words of a chunk (see add_bf16_exact for why one fp32 rounding is enough)
__device__ __forceinline__ uint4 add_chunk(uint4 a, uint4 b) {
  const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
  uint32_t out[4];
#pragma unroll
  for (int w = 0; w < 4; ++w) out[w] = pack2(__fadd2_rn(unpack2(aw[w]), unpack2(bw[w])));
  return make_uint4(out[0], out[1], out[2], out[3]);
}

// sum of the 8 squares of a chunk, exact: every square of a bf16 value is exact in fp32, the sum runs in binary64
__device__ __forceinline__ double square_chunk(uint4 u) {
  const uint32_t uw[4] = {u.x, u.y, u.z, u.w};
  double sum = 0.0;
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    const float2 f = unpack2(uw[w]);
    const float2 q = __fmul2_rn(f, f);
    sum += (double)q.x + (double)q.y;
  }
  return sum;
}

// y = bf16(u * inv * (w + offset)) for a chunk: the bounded fp32 evaluation of scale_to_bf16, word-wise
__device__ __forceinline__ uint4 scale_chunk(uint4 u, uint4 w, float inv32, double inv, float offset32, double offset) {
  const uint32_t uw[4] = {u.x, u.y, u.z, u.w}, ww[4] = {w.x, w.y, w.z, w.w};
  uint32_t out[4];
  bool hard = false;
  const float2 inv2 = make_float2(inv32, inv32), off2 = make_float2(offset32, offset32);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 uf = unpack2(uw[i]);
    const float2 a = __fmul2_rn(uf, inv2);
    const float2 y = __fmul2_rn(a, __fadd2_rn(unpack2(ww[i]), off2));
    const float av[2] = {a.x, a.y}, yv[2] = {y.x, y.y};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t bits = __float_as_uint(yv[h]);
      const bool near_midpoint = (((bits & 0xffffu) - 0x7ff8u) & 0xffffu) <= 16u;             // within 8 ulp
      // exponent fields of y and of the intermediate product in [32, 254): nothing subnormal, nothing infinite
      const bool sized = ((bits & 0x7f800000u) - 0x10000000u) < 0x6f000000u &&
                         ((__float_as_uint(av[h]) & 0x7f800000u) - 0x10000000u) < 0x6f000000u;
      const bool zero = ((uw[i] >> (16 * h)) & 0x7fffu) == 0u;                                // u = +-0 gives y = +-0 exactly
      hard |= !zero && (near_midpoint || !sized);
    }
    out[i] = pack2(y);
  }
  if (hard) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      out[i] = (uint32_t)scale_to_bf16((unsigned short)uw[i], (unsigned short)ww[i], inv32, inv, offset32, offset) |
               (uint32_t)scale_to_bf16((unsigned short)(uw[i] >> 16), (unsigned short)(ww[i] >> 16), inv32, inv, offset32, offset) << 16;
  }
  return make_uint4(out[0], out[1], out[2], out[3]);
}

__device__ __forceinline__ double block_sum(double v, double* shared) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  if (lane == 0) shared[warp] = v;
  __syncthreads();
  double total = 0.0;
  for (int w = 0; w < warps; ++w) total += shared[w];          // same order in every thread
  return total;
}

// One CTA per row.  VEC = 8: 16-byte loads, the row is held in registers between the reduction
// and the write (hidden <= 256 threads * 8 * 4).  VEC = 1: any alignment, second pass re-reads.
// Partial results of the tensor-parallel ranks, summed in rank order (PARTS variant below).
struct PartList {
  const unsigned short* p[GK_MAX_OUTPUTS];
  int n;
};

// Rank-ordered sum of bf16 partials the way the reference's all-reduce defines it
// (tests/tp4_gather_reduce_smoke.py:16-20): fp32 accumulator seeded with rank 0, one fp32 add per
// further rank, one rounding to bf16.  Loads bypass L1: the partials were written by other GPUs.
__device__ __forceinline__ void rank_sum8(const PartList& parts, int64_t offset, unsigned short (&out)[8]) {
  // All ranks' vectors are requested before the first add, so their latencies overlap; the adds then
  // run in rank order.
  uint4 v[GK_MAX_OUTPUTS];
#pragma unroll
  for (int r = 0; r < GK_MAX_OUTPUTS; ++r)
    if (r < parts.n) v[r] = __ldcg(reinterpret_cast<const uint4*>(parts.p[r] + offset));
  float acc[8];
  {
    const unsigned short* av = reinterpret_cast<const unsigned short*>(&v[0]);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = __uint_as_float((uint32_t)av[e] << 16);
  }
#pragma unroll
  for (int r = 1; r < GK_MAX_OUTPUTS; ++r) {
    if (r < parts.n) {
      const unsigned short* bv = reinterpret_cast<const unsigned short*>(&v[r]);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = __fadd_rn(acc[e], __uint_as_float((uint32_t)bv[e] << 16));
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) out[e] = __bfloat16_as_ushort(__float2bfloat16_rn(acc[e]));
}

__global__ void __launch_bounds__(256) rank_sum_kernel(const PartList parts, int64_t vectors, unsigned short* __restrict__ out) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < vectors; i += (int64_t)gridDim.x * blockDim.x) {
    unsigned short v[8];
    rank_sum8(parts, i * 8, v);
    *reinterpret_cast<uint4*>(out + i * 8) = *reinterpret_cast<const uint4*>(v);
  }
}

// Five CTAs per SM (48 registers, no spills): 101 us at 8192 x 8192 against 102 us with the compiler's own
// choice and 108 us with no occupancy target; six CTAs spill and gain nothing more.
#ifndef GK_NORM_MIN_BLOCKS
#define GK_NORM_MIN_BLOCKS 5
#endif
// PARTS: x is not read; the row comes from rank_sum8 over parts (row stride x_stride).
template <int VEC, bool FUSED, bool PARTS = false>
__global__ void __launch_bounds__(256, GK_NORM_MIN_BLOCKS) rms_norm_kernel(const unsigned short* __restrict__ x,
                                                       const unsigned short* __restrict__ residual,
                                                       const unsigned short* __restrict__ weight,
                                                       unsigned short* __restrict__ y, unsigned short* __restrict__ u_out,
                                                       int64_t x_stride, int64_t r_stride, int hidden, double epsilon,
                                                       double weight_offset, const PartList parts = PartList{}) {
  static_assert(!PARTS || (VEC == 8 && FUSED), "the rank-sum front exists for the vectorised fused form only");
  __shared__ double partial[8];
  wait_for_predecessor();
  const int64_t row = blockIdx.x;
  const unsigned short* xr = PARTS ? nullptr : x + row * x_stride;
  const unsigned short* rr = FUSED ? residual + row * r_stride : nullptr;
  unsigned short* yr = y + row * (int64_t)hidden;
  unsigned short* ur = FUSED ? u_out + row * (int64_t)hidden : nullptr;
  double sumsq = 0.0;
  if (VEC == 8) {
    constexpr int kItems = 4;
    uint4 u[kItems];
#pragma unroll
    for (int it = 0; it < kItems; ++it) {
      const int col = (it * 256 + threadIdx.x) * 8;
      if (col < hidden) {
        uint4 a;
        if (PARTS) {
          unsigned short summed[8];
          rank_sum8(parts, row * x_stride + col, summed);
          a = *reinterpret_cast<const uint4*>(summed);
        } else {
          a = __ldg(reinterpret_cast<const uint4*>(xr + col));
        }
        if (FUSED) {
          u[it] = add_chunk(a, __ldg(reinterpret_cast<const uint4*>(rr + col)));
          *reinterpret_cast<uint4*>(ur + col) = u[it];
        } else {
          u[it] = a;
        }
        sumsq += square_chunk(u[it]);
      }
    }
    const double total = block_sum(sumsq, partial);
    const double inv = rsqrt(total / (double)hidden + epsilon);
    const float inv32 = (float)inv, offset32 = (float)weight_offset;
#pragma unroll
    for (int it = 0; it < kItems; ++it) {
      const int col = (it * 256 + threadIdx.x) * 8;
      if (col < hidden)
        *reinterpret_cast<uint4*>(yr + col) =
            scale_chunk(u[it], __ldg(reinterpret_cast<const uint4*>(weight + col)), inv32, inv, offset32, weight_offset);
    }
  } else {
    for (int col = threadIdx.x; col < hidden; col += 256) {
      unsigned short v = __ldg(xr + col);
      if (FUSED) {
        v = add_bf16_exact(v, __ldg(rr + col));
        ur[col] = v;
      }
      sumsq += square_bf16(v);
    }
    const double total = block_sum(sumsq, partial);
    const double inv = rsqrt(total / (double)hidden + epsilon);
    for (int col = threadIdx.x; col < hidden; col += 256) {
      // each thread re-reads only what it wrote (or the untouched input)
      const unsigned short v = FUSED ? ur[col] : __ldg(xr + col);
      yr[col] = bf16_from_double(bf16_to_double(v) * inv * (bf16_to_double(__ldg(weight + col)) + weight_offset));
    }
  }
}

struct RotaryParams {
  const unsigned short* q;
  const unsigned short* k;
  const unsigned short* cache;
  const int32_t* positions;
  unsigned short* q_out;
  unsigned short* k_out;
  // fused store (optional): rotated K and the untouched V go straight to their pool slots
  const unsigned short* v;
  const int32_t* locations;
  unsigned short* pool_k;
  unsigned short* pool_v;
  int32_t* status;
  int64_t rows, q_stride, k_stride, v_stride, cache_rows, slots;
  int q_heads, k_heads, head_dim, rotary_dim, is_neox;
};

__device__ __forceinline__ unsigned short rotate_element(const unsigned short* head, const unsigned short* table,
                                                         int e, int rotary_dim, int is_neox) {
  if (e >= rotary_dim) return __ldg(head + e);
  const int half = rotary_dim >> 1;
  int i, partner;
  bool first;
  if (is_neox) {
    first = e < half;
    i = first ? e : e - half;
    partner = first ? e + half : e - half;
  } else {
    first = !(e & 1);
    i = e >> 1;
    partner = e ^ 1;
  }
  // first of a pair: a*cos - b*sin ; second: b*cos + a*sin   (self is a resp. b)
  return rotate_pair(__ldg(head + e), __ldg(table + i), __ldg(head + partner), __ldg(table + half + i), first);
}

// One thread per element of q, k (and v when the store is fused).
template <bool STORE>
__global__ void __launch_bounds__(256) rotary_kernel(const RotaryParams p) {
  wait_for_predecessor();
  const int heads = p.q_heads + p.k_heads + (STORE ? p.k_heads : 0);
  const int64_t per_row = (int64_t)heads * p.head_dim;
  const int64_t total = p.rows * per_row;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = idx / per_row;
    const int rem = (int)(idx - row * per_row);
    const int head = rem / p.head_dim, e = rem - head * p.head_dim;
    int pos = __ldg(p.positions + row);
    int rotary_dim = p.rotary_dim;
    if ((unsigned)pos >= (unsigned)p.cache_rows) {          // position outside the table: pass through, report
      if (p.status && rem == 0) atomicOr(p.status, (int)GK_DEV_BAD_SLOT);
      pos = 0;
      rotary_dim = 0;
    }
    const unsigned short* table = p.cache + (int64_t)pos * p.rotary_dim;
    if (head < p.q_heads) {
      const unsigned short* src = p.q + row * p.q_stride + (int64_t)head * p.head_dim;
      p.q_out[row * (int64_t)p.q_heads * p.head_dim + rem] = rotate_element(src, table, e, rotary_dim, p.is_neox);
      continue;
    }
    const int kh = head - p.q_heads;
    if (kh < p.k_heads) {
      const unsigned short* src = p.k + row * p.k_stride + (int64_t)kh * p.head_dim;
      const unsigned short out = rotate_element(src, table, e, rotary_dim, p.is_neox);
      if (p.k_out) p.k_out[row * (int64_t)p.k_heads * p.head_dim + kh * p.head_dim + e] = out;
      if (STORE) {
        const int slot = __ldg(p.locations + row);
        if ((unsigned)slot < (unsigned)p.slots) {
          p.pool_k[((int64_t)kh * p.slots + slot) * p.head_dim + e] = out;
        } else if (p.status && e == 0 && kh == 0) {
          atomicOr(p.status, (int)GK_DEV_BAD_SLOT);
        }
      }
      continue;
    }
    if (STORE) {
      const int vh = kh - p.k_heads;
      const int slot = __ldg(p.locations + row);
      if ((unsigned)slot < (unsigned)p.slots)
        p.pool_v[((int64_t)vh * p.slots + slot) * p.head_dim + e] = __ldg(p.v + row * p.v_stride + (int64_t)vh * p.head_dim + e);
    }
  }
}

// Vector form: one thread per 16-byte chunk (8 elements) of q, k (and v when the store is fused).
// Needs 16-byte aligned rows, head_dim % 8 == 0 and whole chunks on each side of a rotation
// (rotary_dim % 16 == 0 for neox pairs, % 8 == 0 for interleaved pairs).
template <bool STORE>
__global__ void __launch_bounds__(256) rotary_vec_kernel(const RotaryParams p) {
  wait_for_predecessor();
  const int chunks = p.head_dim >> 3;
  const int heads = p.q_heads + p.k_heads + (STORE ? p.k_heads : 0);
  const int per_row = heads * chunks;
  const int64_t total = p.rows * (int64_t)per_row;
  const int half = p.rotary_dim >> 1;
  // Index arithmetic in 32 bits whenever the launch allows it (a 64-bit division is a long subroutine, and
  // this kernel is bound by instruction issue), and a shift for the usual power-of-two chunks per head.
  const bool narrow = total <= 0x7fffffffLL;
  const int chunk_shift = (chunks & (chunks - 1)) == 0 ? __ffs(chunks) - 1 : -1;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    int64_t row;
    int rem;
    if (narrow) {
      const unsigned i = (unsigned)idx, r = i / (unsigned)per_row;
      row = r;
      rem = (int)(i - r * (unsigned)per_row);
    } else {
      row = idx / per_row;
      rem = (int)(idx - row * per_row);
    }
    const int head = chunk_shift >= 0 ? rem >> chunk_shift : rem / chunks, ch = rem - head * chunks;
    const int kh = head - p.q_heads;
    if (STORE && kh >= p.k_heads) {                              // V: straight to its slot
      const int vh = kh - p.k_heads;
      const int slot = __ldg(p.locations + row);
      if ((unsigned)slot < (unsigned)p.slots)
        *reinterpret_cast<uint4*>(p.pool_v + ((int64_t)vh * p.slots + slot) * p.head_dim + ch * 8) =
            __ldg(reinterpret_cast<const uint4*>(p.v + row * p.v_stride + (int64_t)vh * p.head_dim + ch * 8));
      continue;
    }
    int pos = __ldg(p.positions + row);
    int rotary_dim = p.rotary_dim;
    if ((unsigned)pos >= (unsigned)p.cache_rows) {                // position outside the table: pass through, report
      if (p.status && rem == 0) atomicOr(p.status, (int)GK_DEV_BAD_SLOT);
      pos = 0;
      rotary_dim = 0;
    }
    const unsigned short* table = p.cache + (int64_t)pos * p.rotary_dim;
    const bool is_q = head < p.q_heads;
    const unsigned short* src = is_q ? p.q + row * p.q_stride + (int64_t)head * p.head_dim
                                     : p.k + row * p.k_stride + (int64_t)kh * p.head_dim;
    uint4 self4 = __ldg(reinterpret_cast<const uint4*>(src + ch * 8));
    uint32_t outw[4];
    if (ch * 8 >= rotary_dim) {
      outw[0] = self4.x;
      outw[1] = self4.y;
      outw[2] = self4.z;
      outw[3] = self4.w;
    } else if (p.is_neox) {
      const bool first = ch * 8 < half;
      const int i0 = first ? ch * 8 : ch * 8 - half;
      uint4 other4 = __ldg(reinterpret_cast<const uint4*>(src + (first ? ch * 8 + half : ch * 8 - half)));
      uint4 cos4 = __ldg(reinterpret_cast<const uint4*>(table + i0)), sin4 = __ldg(reinterpret_cast<const uint4*>(table + half + i0));
      // first half: x*cos - y*sin, second half: x*cos + y*sin (x = this element, y = its partner), two per word
      const uint32_t sw[4] = {self4.x, self4.y, self4.z, self4.w}, ow[4] = {other4.x, other4.y, other4.z, other4.w};
      const uint32_t cw[4] = {cos4.x, cos4.y, cos4.z, cos4.w}, nw[4] = {sin4.x, sin4.y, sin4.z, sin4.w};
      const uint32_t flip = first ? 0x80008000u : 0u;
#pragma unroll
      for (int k = 0; k < 4; ++k)
        outw[k] = rotate_word(unpack2(sw[k]), unpack2(cw[k]), unpack2(ow[k]), unpack2(nw[k] ^ flip));
    } else {
      uint2 cos2 = __ldg(reinterpret_cast<const uint2*>(table + ch * 4)), sin2 = __ldg(reinterpret_cast<const uint2*>(table + half + ch * 4));
      // a word holds the pair (a, b): a*cos - b*sin | b*cos + a*sin
      const uint32_t sw[4] = {self4.x, self4.y, self4.z, self4.w};
      const uint32_t cpair[2] = {cos2.x, cos2.y}, spair[2] = {sin2.x, sin2.y};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 v = unpack2(sw[k]);
        const float cf = __uint_as_float((cpair[k >> 1] >> ((k & 1) * 16)) << 16);
        const float sf = __uint_as_float((spair[k >> 1] >> ((k & 1) * 16)) << 16);
        outw[k] = rotate_word(v, make_float2(cf, cf), make_float2(v.y, v.x), make_float2(-sf, sf));
      }
    }
    const uint4 packed = make_uint4(outw[0], outw[1], outw[2], outw[3]);
    if (is_q) {
      *reinterpret_cast<uint4*>(p.q_out + row * (int64_t)p.q_heads * p.head_dim + (int64_t)head * p.head_dim + ch * 8) = packed;
    } else {
      if (p.k_out) *reinterpret_cast<uint4*>(p.k_out + row * (int64_t)p.k_heads * p.head_dim + (int64_t)kh * p.head_dim + ch * 8) = packed;
      if (STORE) {
        const int slot = __ldg(p.locations + row);
        if ((unsigned)slot < (unsigned)p.slots) {
          *reinterpret_cast<uint4*>(p.pool_k + ((int64_t)kh * p.slots + slot) * p.head_dim + ch * 8) = packed;
        } else if (p.status && ch == 0 && kh == 0) {
          atomicOr(p.status, (int)GK_DEV_BAD_SLOT);
        }
      }
    }
  }
}

// Neox layout, vector form: one thread per PAIR of 16-byte chunks (chunk c of the first half of the rotated
// part and its partner c + rotary_dim/16), so every input chunk, cosine and sine is loaded and unpacked once
// for the two chunks it feeds; chunks past the rotated part and (with the store) the V rows are plain copies.
// A head is `units` work units: rotary_dim/16 pairs, then (head_dim - rotary_dim)/8 single chunks.
#ifndef GK_ROTARY_MIN_BLOCKS
#define GK_ROTARY_MIN_BLOCKS 5   // 48 registers: 35.4 us at 8192 rows; 37.5 us with no target (62 registers), 39.4 us at eight CTAs (spills)
#endif
template <bool STORE>
__global__ void __launch_bounds__(256, GK_ROTARY_MIN_BLOCKS) rotary_neox_pair_kernel(const RotaryParams p) {
  wait_for_predecessor();
  const int chunks = p.head_dim >> 3, pairs = p.rotary_dim >> 4, units = pairs + chunks - 2 * pairs;
  const int rotated = (p.q_heads + p.k_heads) * units;                      // units of a row that are q or k
  const int per_row = rotated + (STORE ? p.k_heads * chunks : 0);
  const int64_t total = p.rows * (int64_t)per_row;
  const int half = p.rotary_dim >> 1;
  const bool narrow = total <= 0x7fffffffLL;
  const int unit_shift = (units & (units - 1)) == 0 ? __ffs(units) - 1 : -1;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    int64_t row;
    int rem;
    if (narrow) {
      const unsigned i = (unsigned)idx, r = i / (unsigned)per_row;
      row = r;
      rem = (int)(i - r * (unsigned)per_row);
    } else {
      row = idx / per_row;
      rem = (int)(idx - row * per_row);
    }
    if (STORE && rem >= rotated) {                                 // V: straight to its slot
      const int at = rem - rotated, vh = at / chunks, ch = at - vh * chunks;
      const int slot = __ldg(p.locations + row);
      if ((unsigned)slot < (unsigned)p.slots)
        *reinterpret_cast<uint4*>(p.pool_v + ((int64_t)vh * p.slots + slot) * p.head_dim + ch * 8) =
            __ldg(reinterpret_cast<const uint4*>(p.v + row * p.v_stride + (int64_t)vh * p.head_dim + ch * 8));
      continue;
    }
    const int head = unit_shift >= 0 ? rem >> unit_shift : rem / units, unit = rem - head * units;
    const int kh = head - p.q_heads;
    const bool is_q = kh < 0;
    int pos = __ldg(p.positions + row);
    bool rotate = unit < pairs;
    if ((unsigned)pos >= (unsigned)p.cache_rows) {                // position outside the table: pass through, report
      if (p.status && rem == 0) atomicOr(p.status, (int)GK_DEV_BAD_SLOT);
      pos = 0;
      rotate = false;
    }
    const unsigned short* src = is_q ? p.q + row * p.q_stride + (int64_t)head * p.head_dim
                                     : p.k + row * p.k_stride + (int64_t)kh * p.head_dim;
    unsigned short* dst = is_q ? p.q_out + (row * p.q_heads + head) * (int64_t)p.head_dim
                               : (p.k_out ? p.k_out + (row * p.k_heads + kh) * (int64_t)p.head_dim : nullptr);
    unsigned short* pooled = nullptr;
    if (STORE && !is_q) {
      const int slot = __ldg(p.locations + row);
      if ((unsigned)slot < (unsigned)p.slots) {
        pooled = p.pool_k + ((int64_t)kh * p.slots + slot) * p.head_dim;
      } else if (p.status && unit == 0 && kh == 0) {
        atomicOr(p.status, (int)GK_DEV_BAD_SLOT);
      }
    }
    // a unit below `pairs` covers chunks `unit` and `unit + pairs`; the others are one chunk each
    const int ch_a = unit < pairs ? unit : 2 * pairs + (unit - pairs);
    const uint4 a4 = __ldg(reinterpret_cast<const uint4*>(src + ch_a * 8));
    if (unit >= pairs) {                                          // past the rotated part: a copy
      if (dst) *reinterpret_cast<uint4*>(dst + ch_a * 8) = a4;
      if (pooled) *reinterpret_cast<uint4*>(pooled + ch_a * 8) = a4;
      continue;
    }
    const int ch_b = unit + pairs;
    const uint4 b4 = __ldg(reinterpret_cast<const uint4*>(src + ch_b * 8));
    uint4 out_a = a4, out_b = b4;
    if (rotate) {
      const unsigned short* table = p.cache + (int64_t)pos * p.rotary_dim;
      const uint4 cos4 = __ldg(reinterpret_cast<const uint4*>(table + unit * 8));
      const uint4 sin4 = __ldg(reinterpret_cast<const uint4*>(table + half + unit * 8));
      const uint32_t aw[4] = {a4.x, a4.y, a4.z, a4.w}, bw[4] = {b4.x, b4.y, b4.z, b4.w};
      const uint32_t cw[4] = {cos4.x, cos4.y, cos4.z, cos4.w}, sw[4] = {sin4.x, sin4.y, sin4.z, sin4.w};
      uint32_t oa[4], ob[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 a = unpack2(aw[k]), b = unpack2(bw[k]), c = unpack2(cw[k]), sn = unpack2(sw[k]);
        oa[k] = rotate_word(a, c, b, make_float2(-sn.x, -sn.y));      // a*cos - b*sin
        ob[k] = rotate_word(b, c, a, sn);                             // b*cos + a*sin
      }
      out_a = make_uint4(oa[0], oa[1], oa[2], oa[3]);
      out_b = make_uint4(ob[0], ob[1], ob[2], ob[3]);
    }
    if (dst) {
      *reinterpret_cast<uint4*>(dst + ch_a * 8) = out_a;
      *reinterpret_cast<uint4*>(dst + ch_b * 8) = out_b;
    }
    if (pooled) {
      *reinterpret_cast<uint4*>(pooled + ch_a * 8) = out_a;
      *reinterpret_cast<uint4*>(pooled + ch_b * 8) = out_b;
    }
  }
}

bool rotary_vectorisable(const RotaryParams& p, bool store) {
  uintptr_t bits = reinterpret_cast<uintptr_t>(p.q) | reinterpret_cast<uintptr_t>(p.k) | reinterpret_cast<uintptr_t>(p.cache) |
                   reinterpret_cast<uintptr_t>(p.q_out) | reinterpret_cast<uintptr_t>(p.k_out);
  if (store) bits |= reinterpret_cast<uintptr_t>(p.v) | reinterpret_cast<uintptr_t>(p.pool_k) | reinterpret_cast<uintptr_t>(p.pool_v);
  const int64_t strides = p.q_stride | p.k_stride | (store ? p.v_stride : 0);
  return !(bits & 15) && !(strides & 7) && p.head_dim % 8 == 0 && p.rotary_dim % (p.is_neox ? 16 : 8) == 0;
}

int launch_rotary(const RotaryParams& p, bool store, cudaStream_t stream) {
  if (p.is_neox && rotary_vectorisable(p, store)) {
    const int chunks = p.head_dim / 8, pairs = p.rotary_dim / 16, units = chunks - pairs;
    const int64_t total = p.rows * ((int64_t)(p.q_heads + p.k_heads) * units + (store ? p.k_heads * chunks : 0));
    const int64_t want = (total + 255) / 256;
    const unsigned blocks = (unsigned)(want < 148 * 16 ? want : 148 * 16);
    if (store)
      launch_after_predecessor(rotary_neox_pair_kernel<true>, dim3(blocks), dim3(256), 0, stream, p);
    else
      launch_after_predecessor(rotary_neox_pair_kernel<false>, dim3(blocks), dim3(256), 0, stream, p);
    return check_launch();
  }
  if (rotary_vectorisable(p, store)) {
    const int heads = p.q_heads + p.k_heads + (store ? p.k_heads : 0);
    const int64_t total = p.rows * heads * (p.head_dim / 8);
    const int64_t want = (total + 255) / 256;
    const unsigned blocks = (unsigned)(want < 148 * 16 ? want : 148 * 16);
    if (store)
      launch_after_predecessor(rotary_vec_kernel<true>, dim3(blocks), dim3(256), 0, stream, p);
    else
      launch_after_predecessor(rotary_vec_kernel<false>, dim3(blocks), dim3(256), 0, stream, p);
    return check_launch();
  }
  const int heads = p.q_heads + p.k_heads + (store ? p.k_heads : 0);
  const int64_t total = p.rows * heads * p.head_dim;
  const int64_t want = (total + 255) / 256;
  const unsigned blocks = (unsigned)(want < 148 * 16 ? want : 148 * 16);
  if (store)
    launch_after_predecessor(rotary_kernel<true>, dim3(blocks), dim3(256), 0, stream, p);
  else
    launch_after_predecessor(rotary_kernel<false>, dim3(blocks), dim3(256), 0, stream, p);
  return check_launch();
}

bool rotary_args_ok(const void* q, const void* k, const void* cache, const int32_t* positions, int64_t rows,
                    int64_t q_width, int64_t k_width, int64_t cache_rows, int head_dim, int rotary_dim) {
  return q && k && cache && positions && rows >= 0 && q_width > 0 && k_width > 0 && cache_rows > 0 && head_dim > 0 &&
         rotary_dim > 0 && rotary_dim <= head_dim && rotary_dim % 2 == 0 && q_width % head_dim == 0 &&
         k_width % head_dim == 0;
}

}  // namespace
}  // namespace gk

static int norm_common(const void* x, const void* residual, const void* weight, double epsilon, double weight_offset,
                       int64_t rows, int64_t hidden, int64_t x_row_stride, int64_t residual_row_stride, void* y,
                       void* u, gk_stream_t stream) {
  const bool fused = residual != nullptr;
  if (rows == 0) return GK_OK;
  if (!x || !weight || !y || (fused && !u) || rows < 0 || hidden <= 0 || !(epsilon > 0.0) || x_row_stride < hidden ||
      (fused && residual_row_stride < hidden))
    return GK_ERR_INVALID_ARGUMENT;
  if (hidden > 8192 || rows > 0x7fffffffLL) return GK_ERR_UNSUPPORTED;   // bound of the reference's op (eager_ops.cpp:1147)
  const uintptr_t bits = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(weight) |
                         reinterpret_cast<uintptr_t>(y) | (fused ? reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(u) : 0);
  if (bits & 1) return GK_ERR_INVALID_ARGUMENT;
  const bool vec = !(bits & 15) && hidden % 8 == 0 && x_row_stride % 8 == 0 && (!fused || residual_row_stride % 8 == 0);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  auto xs = static_cast<const unsigned short*>(x);
  auto rs = static_cast<const unsigned short*>(residual);
  auto ws = static_cast<const unsigned short*>(weight);
  auto ys = static_cast<unsigned short*>(y);
  auto us = static_cast<unsigned short*>(u);
  const unsigned grid = (unsigned)rows;
  const int h = (int)hidden;
  if (fused) {
    if (vec) gk::launch_after_predecessor(gk::rms_norm_kernel<8, true, false>, dim3(grid), dim3(256), 0, s, xs, rs, ws, ys, us, x_row_stride, residual_row_stride, h, epsilon, weight_offset, gk::PartList{});
    else gk::launch_after_predecessor(gk::rms_norm_kernel<1, true, false>, dim3(grid), dim3(256), 0, s, xs, rs, ws, ys, us, x_row_stride, residual_row_stride, h, epsilon, weight_offset, gk::PartList{});
  } else {
    if (vec) gk::launch_after_predecessor(gk::rms_norm_kernel<8, false, false>, dim3(grid), dim3(256), 0, s, xs, nullptr, ws, ys, nullptr, x_row_stride, 0, h, epsilon, weight_offset, gk::PartList{});
    else gk::launch_after_predecessor(gk::rms_norm_kernel<1, false, false>, dim3(grid), dim3(256), 0, s, xs, nullptr, ws, ys, nullptr, x_row_stride, 0, h, epsilon, weight_offset, gk::PartList{});
  }
  return gk::check_launch();
}

extern "C" int gk_rms_norm_bf16(const void* x, const void* weight, float epsilon, float weight_offset, int64_t rows,
                                int64_t hidden, int64_t x_row_stride, void* y, gk_stream_t stream) {
  return norm_common(x, nullptr, weight, (double)epsilon, (double)weight_offset, rows, hidden, x_row_stride, 0, y,
                     nullptr, stream);
}

extern "C" int gk_fused_add_rms_norm_bf16(const void* x, const void* residual, const void* weight, float epsilon,
                                          float weight_offset, int64_t rows, int64_t hidden, int64_t x_row_stride,
                                          int64_t residual_row_stride, void* y, void* u, gk_stream_t stream) {
  if (!residual) return GK_ERR_INVALID_ARGUMENT;
  return norm_common(x, residual, weight, (double)epsilon, (double)weight_offset, rows, hidden, x_row_stride,
                     residual_row_stride, y, u, stream);
}

static int parts_ok(const void* const* parts, int world, gk::PartList* list) {
  if (!parts || world < 1 || world > GK_MAX_OUTPUTS) return GK_ERR_INVALID_ARGUMENT;
  list->n = world;
  for (int r = 0; r < world; ++r) {
    if (!parts[r] || (reinterpret_cast<uintptr_t>(parts[r]) & 15)) return GK_ERR_INVALID_ARGUMENT;
    list->p[r] = static_cast<const unsigned short*>(parts[r]);
  }
  return GK_OK;
}

extern "C" int gk_rank_sum_bf16(const void* const* parts, int world, int64_t count, void* out, gk_stream_t stream) {
  if (count == 0) return GK_OK;
  gk::PartList list{};
  if (const int bad = parts_ok(parts, world, &list)) return bad;
  if (!out || count < 0 || (reinterpret_cast<uintptr_t>(out) & 15)) return GK_ERR_INVALID_ARGUMENT;
  if (count % 8) return GK_ERR_UNSUPPORTED;
  const int64_t vectors = count / 8;
  const unsigned blocks = (unsigned)std::min<int64_t>((vectors + 255) / 256, 148 * 8);
  gk::rank_sum_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(list, vectors,
                                                                                 static_cast<unsigned short*>(out));
  return gk::check_launch();
}

extern "C" int gk_rank_sum_add_rms_norm_bf16(const void* const* parts, int world, int64_t part_row_stride,
                                             const void* residual, const void* weight, float epsilon,
                                             float weight_offset, int64_t rows, int64_t hidden,
                                             int64_t residual_row_stride, void* y, void* u, gk_stream_t stream) {
  if (rows == 0) return GK_OK;
  gk::PartList list{};
  if (const int bad = parts_ok(parts, world, &list)) return bad;
  if (!residual || !weight || !y || !u || rows < 0 || hidden <= 0 || !(epsilon > 0.f) || part_row_stride < hidden ||
      residual_row_stride < hidden)
    return GK_ERR_INVALID_ARGUMENT;
  if (hidden > 8192 || rows > 0x7fffffffLL || hidden % 8 || part_row_stride % 8 || residual_row_stride % 8)
    return GK_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(y) |
       reinterpret_cast<uintptr_t>(u)) & 15)
    return GK_ERR_INVALID_ARGUMENT;
  gk::launch_after_predecessor(gk::rms_norm_kernel<8, true, true>, dim3((unsigned)rows), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream),
      nullptr, static_cast<const unsigned short*>(residual), static_cast<const unsigned short*>(weight),
      static_cast<unsigned short*>(y), static_cast<unsigned short*>(u), part_row_stride, residual_row_stride, (int)hidden,
      (double)epsilon, (double)weight_offset, list);
  return gk::check_launch();
}

extern "C" int gk_rotary_bf16(const void* q, const void* k, int64_t q_row_stride, int64_t k_row_stride,
                              const void* cache, int64_t cache_rows, const int32_t* positions, int64_t rows,
                              int64_t q_width, int64_t k_width, int head_dim, int rotary_dim, int is_neox, void* q_out,
                              void* k_out, int32_t* status, gk_stream_t stream) {
  if (rows == 0) return GK_OK;
  if (!gk::rotary_args_ok(q, k, cache, positions, rows, q_width, k_width, cache_rows, head_dim, rotary_dim) || !q_out ||
      !k_out || q_row_stride < q_width || k_row_stride < k_width)
    return GK_ERR_INVALID_ARGUMENT;
  gk::RotaryParams p{};
  p.q = static_cast<const unsigned short*>(q);
  p.k = static_cast<const unsigned short*>(k);
  p.cache = static_cast<const unsigned short*>(cache);
  p.positions = positions;
  p.q_out = static_cast<unsigned short*>(q_out);
  p.k_out = static_cast<unsigned short*>(k_out);
  p.status = status;
  p.rows = rows;
  p.q_stride = q_row_stride;
  p.k_stride = k_row_stride;
  p.cache_rows = cache_rows;
  p.q_heads = (int)(q_width / head_dim);
  p.k_heads = (int)(k_width / head_dim);
  p.head_dim = head_dim;
  p.rotary_dim = rotary_dim;
  p.is_neox = is_neox ? 1 : 0;
  return gk::launch_rotary(p, false, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int gk_rotary_kv_store_bf16(const void* q, const void* k, const void* v, int64_t q_row_stride,
                                       int64_t k_row_stride, int64_t v_row_stride, const void* cache,
                                       int64_t cache_rows, const int32_t* positions, const int32_t* locations,
                                       int64_t rows, int64_t q_width, int64_t k_width, int head_dim, int rotary_dim,
                                       int is_neox, void* q_out, void* k_out, void* pool_k, void* pool_v, int64_t slots,
                                       int32_t* status, gk_stream_t stream) {
  if (rows == 0) return GK_OK;
  if (!gk::rotary_args_ok(q, k, cache, positions, rows, q_width, k_width, cache_rows, head_dim, rotary_dim) || !q_out ||
      !v || !locations || !pool_k || !pool_v || slots <= 0 || q_row_stride < q_width || k_row_stride < k_width ||
      v_row_stride < k_width)
    return GK_ERR_INVALID_ARGUMENT;
  gk::RotaryParams p{};
  p.q = static_cast<const unsigned short*>(q);
  p.k = static_cast<const unsigned short*>(k);
  p.v = static_cast<const unsigned short*>(v);
  p.cache = static_cast<const unsigned short*>(cache);
  p.positions = positions;
  p.locations = locations;
  p.q_out = static_cast<unsigned short*>(q_out);
  p.k_out = static_cast<unsigned short*>(k_out);   // may be NULL: the rotated K is only needed in the pool
  p.pool_k = static_cast<unsigned short*>(pool_k);
  p.pool_v = static_cast<unsigned short*>(pool_v);
  p.status = status;
  p.rows = rows;
  p.q_stride = q_row_stride;
  p.k_stride = k_row_stride;
  p.v_stride = v_row_stride;
  p.cache_rows = cache_rows;
  p.slots = slots;
  p.q_heads = (int)(q_width / head_dim);
  p.k_heads = (int)(k_width / head_dim);
  p.head_dim = head_dim;
  p.rotary_dim = rotary_dim;
  p.is_neox = is_neox ? 1 : 0;
  return gk::launch_rotary(p, true, reinterpret_cast<cudaStream_t>(stream));
}
