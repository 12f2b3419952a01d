// Tensor-core GEMM for sm_100a: C <- alpha * op(A) * op(B) + beta * C with a
// fused epilogue.  Replaces matmul_tf32_template (ml/matmul/kernel.spi:25-240,
// nvcuda::wmma m16n16k8 TF32 with one-deep cuda::memcpy_async prefetch).
//
// Structure of one CTA (192 threads, persistent over output tiles):
//   warp 0, lane 0 : TMA producer.  Per k-block it arms full[stage] with the
//                    stage's byte count and issues plain 2-D tiled TMA loads
//                    (128-byte swizzle) of the A and B tiles.
//   warp 1, lane 0 : MMA issuer.  Waits full[stage], issues 4 tcgen05.mma
//                    (M=128, N=block_n, 32 bytes of K each) on shared-memory
//                    descriptors, commits to empty[stage]; after the last
//                    k-block commits to tmem_full[acc].  Warp 1 also owns the
//                    TMEM allocation.
//   warps 2..5     : epilogue.  Wait tmem_full[acc], read the fp32 accumulator
//                    from TMEM (tcgen05.ld, one output row per thread), apply
//                    alpha/beta/bias/ReLU/row head, store, arrive on
//                    tmem_empty[acc].  Two accumulators in TMEM let the
//                    epilogue of tile i overlap the main loop of tile i+1.
//
// Operand layouts.  "K-major" = the K index is contiguous in global memory
// (A stored [M,K]; B stored [N,K]); "MN-major" = the M or N index is contiguous
// (A stored [K,M]; B stored [K,N]).  Either way one stage holds 128 bytes of K
// (64 16-bit or 32 32-bit elements) per row for K-major, or block_k rows of
// 128-byte MN segments for MN-major, always in the canonical 128-byte-swizzle
// UMMA layout that TMA produces, so no operand is transposed or re-tiled in
// shared memory.
#include "common.cuh"

namespace {

constexpr int UG_BLOCK_M = 128;
constexpr int UG_THREADS = 192;
constexpr int UG_MAX_STAGES = 8;
constexpr int UG_SMEM_LIMIT = 227 * 1024;
constexpr int UG_HEAD_MAX_N = 32;  // widest row a fused head keeps in registers
constexpr int UG_EPI_STAGING = 4 * 2 * 4096;  // 4 epilogue warps x 2 boxes x (32 rows x 128 B)

struct UmmaGemmParams {
  int M, N, K;
  int block_n;
  int acc_stride;  // TMEM columns between the two accumulators
  int tmem_cols;   // allocated TMEM columns (power of two >= 32)
  int stages;
  int kind_tf32;
  int a_mn, b_mn;
  int block_k;  // elements of K per stage
  int k_blocks;
  int tiles_m, tiles_n, num_tiles;
  int splits;          // split-K factor: work item = (split, tile); 1 = no split
  int kb_per_split;    // k-blocks per split
  int num_work;        // num_tiles * splits
  long long split_stride;  // elements between the partial outputs of two splits
  uint32_t idesc;
  uint32_t a_stage_bytes, b_stage_bytes;
  int a_boxes, b_boxes;    // TMA boxes per stage (1 when K-major)
  int mn_box_elems;        // MN extent of one MN-major box (128 bytes)
  uint32_t mn_box_bytes;   // bytes of one MN-major box = block_k * 128
  uint32_t a_kstep, b_kstep;  // descriptor start-address step per MMA, in 16-byte units
  uint32_t a_sbo, b_sbo;      // stride byte offset of the smem descriptors
  uint32_t a_layout, b_layout;  // descriptor layout type (2 = SW128, 1 = SW128 with 32-byte chunks)
  float alpha, beta;
  void* C;
  long long ldc;
  int out_dtype;
  int epi;
  const float* bias;
  const uint8_t* mask;
  const void* aux_in;
  void* aux_out;
  int tma_store;       // 1: full 32-column chunks leave through shared memory + TMA store
  uint32_t epi_offset; // byte offset of the epilogue staging area from the stage base
};

__device__ __forceinline__ void tile_coords(const UmmaGemmParams& p, int tile, int& m_blk, int& n_blk) {
  constexpr int GROUP = 8;
  const int per_group = GROUP * p.tiles_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP;
  const int gsz = min(GROUP, p.tiles_m - first_m);
  const int r = tile - g * per_group;
  m_blk = first_m + r % gsz;
  n_blk = r / gsz;
}

// ------------------------------ epilogue -----------------------------------
template <typename T>
__device__ __forceinline__ float load_as_float(const T* p);
template <>
__device__ __forceinline__ float load_as_float<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}
template <>
__device__ __forceinline__ float load_as_float<__half>(const __half* p) { return __half2float(*p); }

template <typename T>
__device__ __forceinline__ T float_to(float v);
template <>
__device__ __forceinline__ float float_to<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 float_to<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ __half float_to<__half>(float v) { return __float2half_rn(v); }

__device__ __forceinline__ float round_tf32_rn(float v) {
  uint32_t u = __float_as_uint(v);
  if ((u & 0x7f800000u) == 0x7f800000u) return v;
  u += 0x0fffu + ((u >> 13) & 1u);
  return __uint_as_float(u & 0xffffe000u);
}

// One thread finishes `w` (16 or 32) consecutive columns of its output row.
// ROUND_TF32: fp32 output rounded to 10 mantissa bits (nearest even), so that a
// following TF32 GEMM reads exactly the value stored.
template <typename OutT, bool ROUND_TF32>
__device__ __forceinline__ void finish_chunk(const UmmaGemmParams& p, float* v, int w, long long row,
                                             int col0, long long c_off) {
  const int valid = min(w, p.N - col0);
  if (valid <= 0) return;
  OutT* crow = reinterpret_cast<OutT*>(p.C) + c_off + row * p.ldc + col0;
  const OutT* arow = reinterpret_cast<const OutT*>(p.aux_in) + row * p.ldc + col0;
  constexpr int VEC = 16 / sizeof(OutT);
  const bool vec_ok = (valid == w) && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0);
  const bool has_beta = p.beta != 0.0f;
  const bool has_bias = (p.epi & SB_EPI_BIAS) != 0;
  const bool relu = (p.epi & SB_EPI_RELU) != 0;
  const bool relu_grad = (p.epi & SB_EPI_RELU_GRAD) != 0;
  const bool avec_ok = relu_grad && ((reinterpret_cast<uintptr_t>(arow) & 15) == 0) && (valid == w);

#pragma unroll
  for (int j0 = 0; j0 < 32; j0 += VEC) {
    if (j0 < w) {
      float old[VEC];
      float act[VEC];
      if (has_beta) {
        if (vec_ok) {
          uint4 raw = *reinterpret_cast<const uint4*>(crow + j0);
          const OutT* e = reinterpret_cast<const OutT*>(&raw);
#pragma unroll
          for (int t = 0; t < VEC; ++t) old[t] = load_as_float<OutT>(e + t);
        } else {
#pragma unroll
          for (int t = 0; t < VEC; ++t) old[t] = (j0 + t < valid) ? load_as_float<OutT>(crow + j0 + t) : 0.f;
        }
      }
      if (relu_grad) {
        if (avec_ok) {
          uint4 raw = *reinterpret_cast<const uint4*>(arow + j0);
          const OutT* e = reinterpret_cast<const OutT*>(&raw);
#pragma unroll
          for (int t = 0; t < VEC; ++t) act[t] = load_as_float<OutT>(e + t);
        } else {
#pragma unroll
          for (int t = 0; t < VEC; ++t) act[t] = (j0 + t < valid) ? load_as_float<OutT>(arow + j0 + t) : 0.f;
        }
      }
      OutT outv[VEC];
#pragma unroll
      for (int t = 0; t < VEC; ++t) {
        float x = p.alpha * v[j0 + t];
        if (has_beta) x += p.beta * old[t];
        if (has_bias) x += (j0 + t < valid) ? __ldg(p.bias + col0 + j0 + t) : 0.f;
        if (relu) x = fmaxf(x, 0.f);
        if (relu_grad) x = act[t] > 0.f ? x : 0.f;
        if (ROUND_TF32) x = round_tf32_rn(x);
        outv[t] = float_to<OutT>(x);
      }
      if (vec_ok) {
        *reinterpret_cast<uint4*>(crow + j0) = *reinterpret_cast<const uint4*>(outv);
      } else {
#pragma unroll
        for (int t = 0; t < VEC; ++t)
          if (j0 + t < valid) crow[j0 + t] = outv[t];
      }
    }
  }
}

// Staged variant for a full 32-column chunk: the warp's 32 rows x 32 columns are
// written to a swizzled shared-memory box and leave through one TMA store, so
// global memory sees whole 128-byte (fp32) or 64-byte (16-bit) row segments
// instead of one 16-byte piece per thread.  `sbuf` is this warp's staging box
// (two alternate; a box is reused only after the store that read it retired).
template <typename OutT, bool ROUND_TF32>
__device__ __forceinline__ void stage_chunk(const UmmaGemmParams& p, const CUtensorMap* tmap_c, float* v,
                                            long long row, bool row_ok, int row0_warp, int col0,
                                            long long c_off, uint32_t sbuf, int lane) {
  constexpr int VEC = 16 / sizeof(OutT);      // elements per 16-byte piece
  constexpr int PIECES = 32 / VEC;            // 16-byte pieces per row of the box
  constexpr uint32_t ROW_BYTES = 32 * sizeof(OutT);
  const bool has_beta = p.beta != 0.0f;
  const bool has_bias = (p.epi & SB_EPI_BIAS) != 0;
  const bool relu = (p.epi & SB_EPI_RELU) != 0;
  const bool relu_grad = (p.epi & SB_EPI_RELU_GRAD) != 0;
  const OutT* crow = reinterpret_cast<const OutT*>(p.C) + c_off + row * p.ldc + col0;
  const OutT* arow = reinterpret_cast<const OutT*>(p.aux_in) + row * p.ldc + col0;
  const int valid = min(32, p.N - col0);     // columns of this chunk inside the matrix
  uint4 packed[PIECES];
#pragma unroll
  for (int q = 0; q < PIECES; ++q) {
    float old[VEC], act[VEC];
    const bool piece_full = (q + 1) * VEC <= valid;
    if (has_beta && row_ok) {
      if (piece_full) {
        uint4 raw = *reinterpret_cast<const uint4*>(crow + q * VEC);
        const OutT* e = reinterpret_cast<const OutT*>(&raw);
#pragma unroll
        for (int t = 0; t < VEC; ++t) old[t] = load_as_float<OutT>(e + t);
      } else {
#pragma unroll
        for (int t = 0; t < VEC; ++t) old[t] = (q * VEC + t < valid) ? load_as_float<OutT>(crow + q * VEC + t) : 0.f;
      }
    }
    if (relu_grad && row_ok) {
      if (piece_full) {
        uint4 raw = *reinterpret_cast<const uint4*>(arow + q * VEC);
        const OutT* e = reinterpret_cast<const OutT*>(&raw);
#pragma unroll
        for (int t = 0; t < VEC; ++t) act[t] = load_as_float<OutT>(e + t);
      } else {
#pragma unroll
        for (int t = 0; t < VEC; ++t) act[t] = (q * VEC + t < valid) ? load_as_float<OutT>(arow + q * VEC + t) : 0.f;
      }
    }
    OutT outv[VEC];
#pragma unroll
    for (int t = 0; t < VEC; ++t) {
      float x = p.alpha * v[q * VEC + t];
      if (has_beta && row_ok) x += p.beta * old[t];
      if (has_bias) x += (q * VEC + t < valid) ? __ldg(p.bias + col0 + q * VEC + t) : 0.f;
      if (relu) x = fmaxf(x, 0.f);
      if (relu_grad && row_ok) x = act[t] > 0.f ? x : 0.f;
      if (ROUND_TF32) x = round_tf32_rn(x);
      outv[t] = float_to<OutT>(x);
    }
    packed[q] = *reinterpret_cast<const uint4*>(outv);
  }
  // The box about to be overwritten was read by the store issued two chunks ago.
  if (lane == 0) bulk_wait_group_read<1>();
  __syncwarp();
  const uint32_t swz_mask = ROW_BYTES == 128 ? 7u : 3u;
#pragma unroll
  for (int q = 0; q < PIECES; ++q) {
    const uint32_t lin = (uint32_t)lane * ROW_BYTES + (uint32_t)q * 16u;
    st_shared_v4(sbuf + (lin ^ (((lin >> 7) & swz_mask) << 4)), packed[q]);
  }
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) {
    tma_store_2d(tmap_c, sbuf, col0, row0_warp);
    bulk_commit_group();
  }
}

// Row head on a full row (N <= 32) held by one thread; fp32 output.
// Follows local_masked_softmax / local_masked_regret_matching / local_argmax
// (ml/primitives.spi:748-780, 705-708); the softmax subtracts the masked
// maximum, which equals the reference's masked-mean form exactly in exact
// arithmetic and cannot overflow.
__device__ __forceinline__ void finish_head(const UmmaGemmParams& p, float* v, long long row) {
  const int n = p.N;
  float* crow = reinterpret_cast<float*>(p.C) + row * p.ldc;
  const uint8_t* mrow = p.mask ? p.mask + row * (long long)n : nullptr;
  const bool has_beta = p.beta != 0.0f;
  uint32_t legal = 0;
#pragma unroll
  for (int j = 0; j < UG_HEAD_MAX_N; ++j) {
    if (j < n) {
      float x = p.alpha * v[j];
      if (has_beta) x += p.beta * crow[j];
      if (p.epi & SB_EPI_BIAS) x += __ldg(p.bias + j);
      if (p.epi & SB_EPI_RELU) x = fmaxf(x, 0.f);
      v[j] = x;
      if (!mrow || mrow[j] != 0) legal |= (1u << j);
    }
  }
  const int count = __popc(legal);
  if (p.epi & SB_EPI_MASKED_SOFTMAX) {
    float mx = -3.402823466e38f;
#pragma unroll
    for (int j = 0; j < UG_HEAD_MAX_N; ++j)
      if (j < n && ((legal >> j) & 1u)) mx = fmaxf(mx, v[j]);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < UG_HEAD_MAX_N; ++j) {
      if (j < n) {
        float e = ((legal >> j) & 1u) ? __expf(v[j] - mx) : 0.f;
        v[j] = e;
        s += e;
      }
    }
    const float inv = s > 0.f ? 1.f / s : 0.f;
#pragma unroll
    for (int j = 0; j < UG_HEAD_MAX_N; ++j)
      if (j < n) v[j] *= inv;
  }
  if (p.epi & SB_EPI_REGRET_MATCHING) {
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < UG_HEAD_MAX_N; ++j) {
      if (j < n) {
        float q = ((legal >> j) & 1u) ? fmaxf(v[j], 0.f) : 0.f;
        v[j] = q;
        s += q;
      }
    }
    const float inv_len = count > 0 ? 1.f / (float)count : 0.f;
#pragma unroll
    for (int j = 0; j < UG_HEAD_MAX_N; ++j) {
      if (j < n) {
        const bool lg = (legal >> j) & 1u;
        v[j] = !lg ? 0.f : (s != 0.f ? v[j] / s : inv_len);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < UG_HEAD_MAX_N; ++j)
    if (j < n) crow[j] = v[j];
  if (p.epi & SB_EPI_ARGMAX) {
    int best = 0;
    float bv = v[0];
#pragma unroll
    for (int j = 1; j < UG_HEAD_MAX_N; ++j) {
      if (j < n && v[j] > bv) {
        bv = v[j];
        best = j;
      }
    }
    reinterpret_cast<int32_t*>(p.aux_out)[row] = best;
  }
}

constexpr int EPI_HEAD_MASK = SB_EPI_MASKED_SOFTMAX | SB_EPI_REGRET_MATCHING | SB_EPI_ARGMAX;

__global__ void __launch_bounds__(UG_THREADS, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a,
                 const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_c, const UmmaGemmParams p) {
  extern __shared__ uint8_t ug_smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[UG_MAX_STAGES];
  __shared__ __align__(8) uint64_t bar_empty[UG_MAX_STAGES];
  __shared__ __align__(8) uint64_t bar_tmem_full[2];
  __shared__ __align__(8) uint64_t bar_tmem_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // Stage buffers start on a 1024-byte boundary (one swizzle atom).
  const uint32_t raw_addr = smem_u32(ug_smem_raw);
  const uint32_t stage_base = (raw_addr + 1023u) & ~1023u;
  const uint32_t stage_bytes = p.a_stage_bytes + p.b_stage_bytes;

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bar_tmem_full[a]), 1);
      mbar_init(smem_u32(&bar_tmem_empty[a]), 4);
    }
    abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_slot), (uint32_t)p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  volatile int* abortp = &abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int work = blockIdx.x; ok && work < p.num_work; work += gridDim.x) {
        const int split = work / p.num_tiles;
        int m_blk, n_blk;
        tile_coords(p, work - split * p.num_tiles, m_blk, n_blk);
        const int m0 = m_blk * UG_BLOCK_M;
        const int n0 = n_blk * p.block_n;
        const int kb_begin = split * p.kb_per_split;
        const int kb_end = min(p.k_blocks, kb_begin + p.kb_per_split);
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, abortp, SB_SITE_PRODUCER_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&bar_full[stage]);
          mbar_arrive_expect_tx(full, stage_bytes);
          const uint32_t a_dst = stage_base + (uint32_t)stage * stage_bytes;
          const uint32_t b_dst = a_dst + p.a_stage_bytes;
          const int k0 = kb * p.block_k;
          if (!p.a_mn) {
            tma_load_2d(a_dst, &tmap_a, k0, m0, full);
          } else {
            for (int i = 0; i < p.a_boxes; ++i)
              tma_load_2d(a_dst + (uint32_t)i * p.mn_box_bytes, &tmap_a, m0 + i * p.mn_box_elems, k0, full);
          }
          if (!p.b_mn) {
            tma_load_2d(b_dst, &tmap_b, k0, n0, full);
          } else {
            for (int i = 0; i < p.b_boxes; ++i)
              tma_load_2d(b_dst + (uint32_t)i * p.mn_box_bytes, &tmap_b, n0 + i * p.mn_box_elems, k0, full);
          }
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      // K-major: LBO unused (1), SBO = 1024 (8 rows x 128 B).
      // MN-major: LBO = bytes between 128-byte MN segments (one TMA box),
      //           SBO = bytes between k-row groups: 1024 (8 rows) for 16-bit
      //           types, 512 (4 rows) for the 32-byte-chunk swizzle of TF32.
      const uint32_t a_lbo = p.a_mn ? p.mn_box_bytes : 16u;
      const uint32_t b_lbo = p.b_mn ? p.mn_box_bytes : 16u;
      for (int work = blockIdx.x; ok && work < p.num_work; work += gridDim.x) {
        const int split = work / p.num_tiles;
        const int kb_begin = split * p.kb_per_split;
        const int kb_end = min(p.k_blocks, kb_begin + p.kb_per_split);
        if (!mbar_wait(smem_u32(&bar_tmem_empty[acc]), acc_phase ^ 1u, abortp, SB_SITE_MMA_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * p.acc_stride);
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(smem_u32(&bar_full[stage]), phase, abortp, SB_SITE_MMA_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_src = stage_base + (uint32_t)stage * stage_bytes;
          const uint32_t b_src = a_src + p.a_stage_bytes;
          const uint64_t a_desc = umma_smem_desc(a_src, a_lbo, p.a_sbo, p.a_layout);
          const uint64_t b_desc = umma_smem_desc(b_src, b_lbo, p.b_sbo, p.b_layout);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint32_t accumulate = (kb > kb_begin || ks > 0) ? 1u : 0u;
            const uint64_t ad = a_desc + (uint64_t)(ks * p.a_kstep);
            const uint64_t bd = b_desc + (uint64_t)(ks * p.b_kstep);
            if (p.kind_tf32)
              umma_tf32(d_tmem, ad, bd, p.idesc, accumulate);
            else
              umma_f16(d_tmem, ad, bd, p.idesc, accumulate);
          }
          tc_commit(smem_u32(&bar_empty[stage]));
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        tc_commit(smem_u32(&bar_tmem_full[acc]));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // Epilogue warps 2..5; TMEM lane quadrant = warp index modulo 4.
    const int quad = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool head = (p.epi & EPI_HEAD_MASK) != 0;
    const uint32_t sbuf0 = stage_base + p.epi_offset + (uint32_t)(warp - 2) * 8192u;
    int sbuf_sel = 0;
    for (int work = blockIdx.x; work < p.num_work; work += gridDim.x) {
      const int split = work / p.num_tiles;
      const long long c_off = (long long)split * p.split_stride;
      int m_blk, n_blk;
      tile_coords(p, work - split * p.num_tiles, m_blk, n_blk);
      if (!mbar_wait(smem_u32(&bar_tmem_full[acc]), acc_phase, abortp, SB_SITE_EPI_TMEM_FULL)) break;
      tc_fence_after_sync();
      const long long row = (long long)m_blk * UG_BLOCK_M + quad * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * p.acc_stride);
      if (head) {
        uint32_t raw[32];
        if (p.block_n >= 32) tmem_ld32(t_row, raw); else tmem_ld16(t_row, raw);
        tmem_ld_wait();
        if (row_ok) finish_head(p, reinterpret_cast<float*>(raw), row);
      } else {
        for (int c0 = 0; c0 < p.block_n; c0 += 32) {
          const int w = min(32, p.block_n - c0);
          uint32_t raw[32];
          if (w == 32) tmem_ld32(t_row + (uint32_t)c0, raw); else tmem_ld16(t_row + (uint32_t)c0, raw);
          tmem_ld_wait();
          const int col0 = n_blk * p.block_n + c0;
          float* v = reinterpret_cast<float*>(raw);
          const int row0_warp = m_blk * UG_BLOCK_M + quad * 32;
          if (p.tma_store && w == 32 && col0 < p.N) {
            // Clipped by the tensor map: rows >= M (per split) and columns >= N.
            if (row0_warp < p.M) {
              const uint32_t sbuf = sbuf0 + (uint32_t)sbuf_sel * 4096u;
              const int y = split * p.M + row0_warp;
              if (p.out_dtype == SB_F32) stage_chunk<float, false>(p, &tmap_c, v, row, row_ok, y, col0, c_off, sbuf, lane);
              else if (p.out_dtype == SB_TF32) stage_chunk<float, true>(p, &tmap_c, v, row, row_ok, y, col0, c_off, sbuf, lane);
              else if (p.out_dtype == SB_BF16) stage_chunk<__nv_bfloat16, false>(p, &tmap_c, v, row, row_ok, y, col0, c_off, sbuf, lane);
              else stage_chunk<__half, false>(p, &tmap_c, v, row, row_ok, y, col0, c_off, sbuf, lane);
              sbuf_sel ^= 1;
            }
          } else if (row_ok) {
            if (p.out_dtype == SB_F32) finish_chunk<float, false>(p, v, w, row, col0, c_off);
            else if (p.out_dtype == SB_TF32) finish_chunk<float, true>(p, v, w, row, col0, c_off);
            else if (p.out_dtype == SB_BF16) finish_chunk<__nv_bfloat16, false>(p, v, w, row, col0, c_off);
            else finish_chunk<__half, false>(p, v, w, row, col0, c_off);
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_tmem_empty[acc]));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  // Teardown.  Stores still reading the staging boxes must retire first; after
  // an expired wait, also give copies and MMAs in flight time to land before
  // shared and tensor memory are released.
  if (warp >= 2 && lane == 0) bulk_wait_group<0>();
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (*abortp != 0) {
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) { }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

// ------------------------------- host side ----------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// 2-D row-major tensor [rows, cols] -> tensor map with box [box_rows, box_cols],
// 128-byte swizzle (box_cols * elem size must be 128 bytes), zero fill outside.
// `swz`: SWZ_128 (16-byte chunks), SWZ_128_CHUNK32 (32-byte chunks, MN-major
// TF32 operands) or SWZ_64 (64-byte rows, 16-bit output boxes).
enum TmapSwizzle { SWZ_128 = 0, SWZ_128_CHUNK32 = 1, SWZ_64 = 2 };

int make_tmap_2d(CUtensorMap* map, const void* base, int in_dtype, long long rows, long long cols,
                 int box_rows, int box_cols, int swz) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return sb_fail(SB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const int es = sb_dtype_size(in_dtype);
  CUtensorMapDataType dt = in_dtype == SB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : in_dtype == SB_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)cols * (cuuint64_t)es};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swz == SWZ_128_CHUNK32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                   : swz == SWZ_64      ? CU_TENSOR_MAP_SWIZZLE_64B
                                        : CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return sb_fail(SB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (rows=%lld cols=%lld box=%dx%d)",
                   (int)r, rows, cols, box_rows, box_cols);
  return SB_OK;
}

int round_up_int(int x, int m) { return (x + m - 1) / m * m; }
int next_pow2(int x) {
  int p = 32;
  while (p < x) p <<= 1;
  return p;
}

int cached_sm_count() {
  static int sms[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return SB_NUM_SMS_FALLBACK;
  if (sms[dev] == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0)
      v = SB_NUM_SMS_FALLBACK;
    sms[dev] = v;
  }
  return sms[dev];
}

// Chooses block_n / stages / grid for a problem; `sms` = SM count to plan for.
void plan_umma(UmmaGemmParams& p, int in_dtype, int sms) {
  const int es = sb_dtype_size(in_dtype);
  p.block_k = 128 / es;
  p.k_blocks = (p.K + p.block_k - 1) / p.block_k;
  p.tiles_m = (p.M + UG_BLOCK_M - 1) / UG_BLOCK_M;
  p.mn_box_elems = 128 / es;
  p.mn_box_bytes = (uint32_t)p.block_k * 128u;
  const int gran = p.b_mn ? p.mn_box_elems : 16;
  int best_bn = 0;
  if (p.N <= 256) {
    best_bn = round_up_int(p.N, gran);
  } else {
    // Minimise (waves of tiles over the SMs) x (cost of one tile); tiles
    // narrower than 192 columns are shared-memory-bandwidth bound for
    // single-CTA MMAs, so they are not considered for wide problems.
    double best_cost = 1e30;
    for (int bn = 256; bn >= 192; bn -= gran) {
      if (bn % gran) continue;
      const long long tiles = (long long)p.tiles_m * ((p.N + bn - 1) / bn);
      const long long waves = (tiles + sms - 1) / sms;
      const double cost = (double)waves * (bn + 16);
      if (cost < best_cost - 1e-9) {
        best_cost = cost;
        best_bn = bn;
      }
    }
  }
  p.block_n = best_bn;
  p.tiles_n = (p.N + p.block_n - 1) / p.block_n;
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.splits = 1;
  p.kb_per_split = p.k_blocks;
  p.num_work = p.num_tiles;
  p.split_stride = 0;
  p.acc_stride = next_pow2(p.block_n);
  p.tmem_cols = next_pow2(2 * p.acc_stride);
  p.a_stage_bytes = UG_BLOCK_M * 128u;
  p.b_stage_bytes = (uint32_t)p.block_n * 128u;
  // Keep every stage 1024-byte aligned: block_n * 128 is a multiple of 1024
  // only when block_n % 8 == 0, which holds (multiples of 16).
  p.a_boxes = p.a_mn ? UG_BLOCK_M / p.mn_box_elems : 1;
  p.b_boxes = p.b_mn ? p.block_n / p.mn_box_elems : 1;
  const int stage_bytes = (int)(p.a_stage_bytes + p.b_stage_bytes);
  int stages = (UG_SMEM_LIMIT - 2048 - UG_EPI_STAGING) / stage_bytes;
  if (stages > UG_MAX_STAGES) stages = UG_MAX_STAGES;
  if (stages > p.k_blocks && p.k_blocks >= 2) stages = max(2, p.k_blocks);
  if (stages < 2) stages = 2;
  p.stages = stages;
  p.epi_offset = (uint32_t)stages * (uint32_t)stage_bytes;
  // Per-MMA descriptor step: K-major advances 32 bytes inside the swizzle
  // atom; MN-major advances (UMMA_K / 8) groups of 8 k-rows (1024 B each).
  const int umma_k = 32 / es;
  p.a_kstep = p.a_mn ? (uint32_t)((umma_k / 8) * 1024 / 16) : 2u;
  p.b_kstep = p.b_mn ? (uint32_t)((umma_k / 8) * 1024 / 16) : 2u;
  p.kind_tf32 = (in_dtype == SB_TF32) ? 1 : 0;
  const bool a32 = p.a_mn && es == 4, b32 = p.b_mn && es == 4;
  p.a_layout = a32 ? 1u : 2u;
  p.b_layout = b32 ? 1u : 2u;
  p.a_sbo = a32 ? 512u : 1024u;
  p.b_sbo = b32 ? 512u : 1024u;
  p.idesc = sb_umma_idesc(in_dtype, p.a_mn, p.b_mn, UG_BLOCK_M, p.block_n);
}

size_t umma_dyn_smem(const UmmaGemmParams& p) {
  return (size_t)p.stages * (p.a_stage_bytes + p.b_stage_bytes) + UG_EPI_STAGING + 1024;
}

__global__ void scale_rows_kernel(void* C, long long total, float beta, int out_dtype) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long step = (long long)gridDim.x * blockDim.x;
  for (; i < total; i += step) {
    if (out_dtype == SB_F32 || out_dtype == SB_TF32) {
      float* c = reinterpret_cast<float*>(C);
      c[i] = beta == 0.f ? 0.f : beta * c[i];
    } else if (out_dtype == SB_BF16) {
      __nv_bfloat16* c = reinterpret_cast<__nv_bfloat16*>(C);
      c[i] = __float2bfloat16_rn(beta == 0.f ? 0.f : beta * __bfloat162float(c[i]));
    } else {
      __half* c = reinterpret_cast<__half*>(C);
      c[i] = __float2half_rn(beta == 0.f ? 0.f : beta * __half2float(c[i]));
    }
  }
}

}  // namespace

// Launches the tensor-core GEMM.  All argument validation happens here, so a
// bad call never reaches the device.
int sb_umma_gemm_launch(int a_trans, int b_trans, float alpha, const void* A, const void* B,
                        float beta, void* C, int M, int N, int K, int in_dtype, int out_dtype,
                        int epi, const float* bias, const uint8_t* mask, const void* aux_in,
                        void* aux_out, cudaStream_t stream, int splits, int* splits_used) {
  const int es = sb_dtype_size(in_dtype);
  UmmaGemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K;
  p.a_mn = a_trans ? 1 : 0;   // A stored [K,M]: M contiguous
  p.b_mn = b_trans ? 0 : 1;   // B stored [K,N]: N contiguous
  plan_umma(p, in_dtype, cached_sm_count());
  p.alpha = alpha; p.beta = beta;
  p.C = C; p.ldc = N; p.out_dtype = out_dtype;
  p.epi = epi; p.bias = bias; p.mask = mask; p.aux_in = aux_in; p.aux_out = aux_out;

  // TMA needs 16-byte aligned bases and row pitches.
  const long long lda = a_trans ? M : K;
  const long long ldb = b_trans ? K : N;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return sb_fail(SB_ERR_MISALIGNED, "GEMM operand base pointers must be 16-byte aligned");
  if ((lda * es) % 16 != 0 || (ldb * es) % 16 != 0)
    return sb_fail(SB_ERR_MISALIGNED,
                   "GEMM operand row pitch must be a multiple of 16 bytes (lda=%lld ldb=%lld elem=%d B)",
                   lda, ldb, es);

  CUtensorMap ta, tb;
  int rc;
  if (!p.a_mn) rc = make_tmap_2d(&ta, A, in_dtype, M, K, UG_BLOCK_M, p.block_k, SWZ_128);
  else rc = make_tmap_2d(&ta, A, in_dtype, K, M, p.block_k, p.mn_box_elems, p.a_layout == 1u ? SWZ_128_CHUNK32 : SWZ_128);
  if (rc != SB_OK) return rc;
  if (!p.b_mn) rc = make_tmap_2d(&tb, B, in_dtype, N, K, p.block_n, p.block_k, SWZ_128);
  else rc = make_tmap_2d(&tb, B, in_dtype, K, N, p.block_k, p.mn_box_elems, p.b_layout == 1u ? SWZ_128_CHUNK32 : SWZ_128);
  if (rc != SB_OK) return rc;

  if (splits > 1) {
    // Split-K: each split writes its own [M,N] partial at C + split * M * N.
    int kbps = (p.k_blocks + splits - 1) / splits;
    if (kbps < 1) kbps = 1;
    p.kb_per_split = kbps;
    p.splits = (p.k_blocks + kbps - 1) / kbps;   // every split owns at least one k-block
    p.num_work = p.num_tiles * p.splits;
    p.split_stride = (long long)M * N;
  }
  if (splits_used) *splits_used = p.splits;

  // Output through shared memory + TMA store when C allows it: 16-byte aligned
  // base and row pitch, no row head, and -- with split-K, where the partials
  // form one [splits * M, N] tensor -- no 32-row box may straddle two partials.
  const int es_out = out_dtype == SB_BF16 || out_dtype == SB_F16 ? 2 : 4;
  CUtensorMap tc;
  memset(&tc, 0, sizeof(tc));
  p.tma_store = 0;
  if (!(epi & EPI_HEAD_MASK) && ((long long)N * es_out) % 16 == 0 && N >= 32 &&
      (reinterpret_cast<uintptr_t>(C) & 15) == 0 && (p.splits == 1 || M % 32 == 0)) {
    const int cdt = es_out == 4 ? SB_F32 : out_dtype;
    rc = make_tmap_2d(&tc, C, cdt, (long long)M * p.splits, N, 32, 32, es_out == 4 ? SWZ_128 : SWZ_64);
    if (rc != SB_OK) return rc;
    p.tma_store = 1;
  }

  const size_t smem = umma_dyn_smem(p);
  static bool attr_set[64] = {false};
  int dev = 0;
  SB_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    SB_CUDA(cudaFuncSetAttribute(umma_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 UG_SMEM_LIMIT - 1024));
    attr_set[dev] = true;
  }
  const int grid = min(p.num_work, cached_sm_count());
  sb_prof_before(stream);
  umma_gemm_kernel<<<grid, UG_THREADS, smem, stream>>>(ta, tb, tc, p);
  sb_prof_after(stream, 2.0 * M * N * K);
  SB_COUNT_LAUNCH();
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

int sb_umma_plan(int a_trans, int b_trans, int M, int N, int K, int in_dtype, int sms, int* plan5) {
  UmmaGemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K;
  p.a_mn = a_trans ? 1 : 0;
  p.b_mn = b_trans ? 0 : 1;
  plan_umma(p, in_dtype, sms);
  plan5[0] = UG_BLOCK_M;
  plan5[1] = p.block_n;
  plan5[2] = p.block_k;
  plan5[3] = p.stages;
  plan5[4] = min(p.num_tiles, sms);
  return SB_OK;
}

int sb_scale_launch(void* C, long long total, float beta, int out_dtype, cudaStream_t stream) {
  if (total <= 0) return SB_OK;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  scale_rows_kernel<<<(int)blocks, 256, 0, stream>>>(C, total, beta, out_dtype);
  SB_COUNT_LAUNCH();
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

int sb_umma_head_max_n() { return UG_HEAD_MAX_N; }
