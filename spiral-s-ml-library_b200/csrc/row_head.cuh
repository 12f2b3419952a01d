// Row heads finished in registers, shared by the GEMM epilogue and the fused
// multi-layer kernel: one thread holds one output row (up to 64 values) and
// applies masked softmax, masked regret matching, arg-max, discrete sampling with
// a counter-based random stream, and the sign hash.
//
// Reference arithmetic: local_masked_softmax / local_masked_regret_matching
// (ml/primitives.spi:748-780), local_argmax (:705-708), local_discrete_sampling
// (:782-800), local_binarize (:816-821); the layers instantiate the mask as the
// prefix j < size (ml/layers.spi:409,416,422-431).  The softmax subtracts the masked
// maximum (the reference subtracts the masked mean: identical in exact arithmetic,
// and this form cannot overflow).
//
// Random numbers.  The reference gives every thread a cuRAND Philox4_32_10 state
// initialised as curand_init(seed, subsequence = thread index in the grid, offset = 0)
// (corecuda/random.spi:22-24, game/leduc/tests/train.spi:118) and draws
// curand_uniform, a value in (0, 1] (corecuda/random.spi:84).  Here the same
// generator is written out as a pure function: Philox4x32 with 10 rounds (Salmon,
// Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC 2011), key =
// the 64-bit seed, counter = (position / 4 as 64 bits, subsequence as 64 bits), and
// 32-bit output number `position` of a stream is word position % 4 of that block.
// Nothing is carried between kernels: a draw is named by (seed, subsequence,
// position), so the host-side checker can recompute every one of them.
#pragma once

#include "common.cuh"

struct SbPhilox4 {
  uint32_t v[4];
};

__host__ __device__ inline void sb_mulhilo32(uint32_t a, uint32_t b, uint32_t& hi, uint32_t& lo) {
  const unsigned long long p = (unsigned long long)a * (unsigned long long)b;
  hi = (uint32_t)(p >> 32);
  lo = (uint32_t)p;
}

// One block of Philox4x32-10: counter c[0..3], key (k0, k1).
__host__ __device__ inline SbPhilox4 sb_philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                                      uint32_t k1) {
#pragma unroll
  for (int round = 0; round < 10; ++round) {
    uint32_t hi0, lo0, hi1, lo1;
    sb_mulhilo32(0xD2511F53u, c0, hi0, lo0);
    sb_mulhilo32(0xCD9E8D57u, c2, hi1, lo1);
    const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  SbPhilox4 out;
  out.v[0] = c0; out.v[1] = c1; out.v[2] = c2; out.v[3] = c3;
  return out;
}

// 32-bit output number `position` of the stream (seed, subsequence).
__host__ __device__ inline uint32_t sb_philox_u32(unsigned long long seed, unsigned long long subsequence,
                                                  unsigned long long position) {
  const unsigned long long block = position >> 2;
  const SbPhilox4 r = sb_philox4x32_10((uint32_t)block, (uint32_t)(block >> 32), (uint32_t)subsequence,
                                       (uint32_t)(subsequence >> 32), (uint32_t)seed, (uint32_t)(seed >> 32));
  return r.v[position & 3ull];
}

// A 32-bit draw as a float in (0, 1]: x * 2^-32 + 2^-33, rounded once (the mapping of curand_uniform).
__host__ __device__ inline float sb_uniform_open_closed(uint32_t x) {
#ifdef __CUDA_ARCH__
  return __fmaf_rn((float)x, 2.3283064365386963e-10f, 1.1641532182693481e-10f);
#else
  return (float)((double)(float)x * 2.3283064365386963e-10 + 1.1641532182693481e-10);
#endif
}

// Unbiased integer in [0, range) from a stream, the rejection form of corecuda/random.spi:53-59
// (draw r; x = r mod range; accept when r - x <= 2^32 - range).  Draws are taken at
// position, position + 1, ...; after 8 rejections (probability below range^8 / 2^256) the last
// draw is used as it is, so the loop is bounded.
__host__ __device__ inline uint32_t sb_philox_below(unsigned long long seed, unsigned long long subsequence,
                                                    unsigned long long position, uint32_t range) {
  uint32_t x = 0u;
  for (int attempt = 0; attempt < 8; ++attempt) {
    const uint32_t r = sb_philox_u32(seed, subsequence, position + (unsigned long long)attempt);
    x = r % range;
    if (r - x <= 0u - range) break;
  }
  return x;
}

#ifdef __CUDACC__

struct SbRowHead {
  int n;                    // columns of the row
  int flags;                // SB_EPI_MASKED_SOFTMAX | SB_EPI_REGRET_MATCHING | SB_EPI_ARGMAX | SB_EPI_SAMPLE | SB_EPI_BINARIZE
  int prefix;               // >= 0: legal iff column < prefix; < 0: the byte mask (or everything) is legal
  const uint8_t* mask;      // uint8 [rows, n] or null
  int32_t* argmax_out;      // int32 [rows]
  int32_t* sample_out;      // int32 [rows]
  uint32_t* hash_out;       // uint32 [rows]
  uint32_t modulo;          // of the sign hash
  unsigned long long seed, row_offset, position;   // the sampling draw of row r: stream (seed, row_offset + r), output `position`
};

// v[0..W) holds the row's first W values (everything else the caller has applied already: scale,
// bias, ReLU).  When n > W the caller guarantees 0 <= prefix <= W: columns from W on are illegal
// and come out as zeros.  Writes the finished row to crow[0..n) and the per-row results.  Returns
// the sampled index (or -1) so that callers can go on with it.
template <int W>
__device__ __forceinline__ int sb_row_head_finish(const SbRowHead& h, float* v, long long row, float* crow) {
  static_assert(W == 16 || W == 32 || W == 64, "a row head holds 16, 32 or 64 values");
  const int n = h.n;
  const int live = n < W ? n : W;            // values of this row held in v
  unsigned long long legal = 0ull;
  if (h.prefix >= 0) {
    const int p = h.prefix < live ? h.prefix : live;
    legal = p >= 64 ? ~0ull : ((1ull << p) - 1ull);
  } else if (h.mask) {
    const uint8_t* mrow = h.mask + row * (long long)n;
#pragma unroll
    for (int j = 0; j < W; ++j)
      if (j < live && mrow[j] != 0) legal |= 1ull << j;
  } else {
    legal = live >= 64 ? ~0ull : ((1ull << live) - 1ull);
  }
  if (h.flags & SB_EPI_BINARIZE) {
    // Bit j = (value j > 0) over the first 32 values, before any other head (the hash is of the logits).
    uint32_t bits = 0u;
#pragma unroll
    for (int j = 0; j < (W < 32 ? W : 32); ++j)
      if (j < live && v[j] > 0.f) bits |= 1u << j;
    h.hash_out[row] = bits % h.modulo;
  }
  const int count = __popcll(legal);
  if (h.flags & SB_EPI_MASKED_SOFTMAX) {
    float mx = -3.402823466e38f;
#pragma unroll
    for (int j = 0; j < W; ++j)
      if ((legal >> j) & 1ull) mx = fmaxf(mx, v[j]);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < W; ++j) {
      const float e = ((legal >> j) & 1ull) ? __expf(v[j] - mx) : 0.f;
      v[j] = e;
      s += e;
    }
    const float inv = s > 0.f ? 1.f / s : 0.f;
#pragma unroll
    for (int j = 0; j < W; ++j) v[j] *= inv;
  }
  if (h.flags & SB_EPI_REGRET_MATCHING) {
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < W; ++j) {
      const float q = ((legal >> j) & 1ull) ? fmaxf(v[j], 0.f) : 0.f;
      v[j] = q;
      s += q;
    }
    const float inv_len = count > 0 ? 1.f / (float)count : 0.f;
#pragma unroll
    for (int j = 0; j < W; ++j) v[j] = !((legal >> j) & 1ull) ? 0.f : (s != 0.f ? v[j] / s : inv_len);
  }
  // The finished row.  16-byte stores when the row pitch allows them.
  if ((n & 3) == 0 && (reinterpret_cast<uintptr_t>(crow) & 15) == 0) {
#pragma unroll
    for (int q = 0; q < W / 4; ++q)
      if (4 * q < n) *reinterpret_cast<float4*>(crow + 4 * q) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    for (int j = W; j < n; j += 4) *reinterpret_cast<float4*>(crow + j) = make_float4(0.f, 0.f, 0.f, 0.f);
  } else {
#pragma unroll
    for (int j = 0; j < W; ++j)
      if (j < n) crow[j] = v[j];
    for (int j = W; j < n; ++j) crow[j] = 0.f;
  }
  if (h.flags & SB_EPI_ARGMAX) {
    int best = 0;
    float bv = v[0];
#pragma unroll
    for (int j = 1; j < W; ++j) {
      if (j < n && v[j] > bv) {
        bv = v[j];
        best = j;
      }
    }
    h.argmax_out[row] = best;
  }
  int pick = -1;
  if (h.flags & SB_EPI_SAMPLE) {
    // cdf = running sum in index order; top = the cdf at the last positive entry; the first j with
    // a positive weight and cdf[j] - u * top >= 0.  Each operation is rounded on its own (no fused
    // multiply-add) so that the host-side checker reproduces the comparison bit for bit.
    const float u = sb_uniform_open_closed(sb_philox_u32(h.seed, h.row_offset + (unsigned long long)row, h.position));
    float s = 0.f, top = 0.f;
#pragma unroll
    for (int j = 0; j < W; ++j) {
      if (j < live) {
        s = __fadd_rn(s, v[j]);
        if (v[j] > 0.f) top = s;
      }
    }
    const float threshold = __fmul_rn(u, top);
    s = 0.f;
#pragma unroll
    for (int j = 0; j < W; ++j) {
      if (j < live) {
        s = __fadd_rn(s, v[j]);
        if (pick < 0 && v[j] > 0.f && __fsub_rn(s, threshold) >= 0.f) pick = j;
      }
    }
    h.sample_out[row] = pick;
  }
  return pick;
}

#endif  // __CUDACC__
