// Persistent fused multi-layer forward for narrow policy networks (the Leduc-sized
// 32-256-256-256-3 net of the benchmark): one launch runs every layer, and hidden
// activations never leave the SM.
//
// The reference runs such a net as block_matmul -> block_map -> block_row_map device
// functions with a global-memory round trip per node (ml/layers.spi:181-252,
// generated ml/layers.py:4500-4546).  Here a CTA owns 128 batch rows at a time:
//   warp 0, lane 0 : TMA producer -- the input tile, then every layer's weights in
//                    64-column K-chunks through a ring of shared-memory stages
//                    (weights come from L2: the whole net is a few hundred KB).
//   warp 1, lane 0 : tcgen05.mma issuer -- layer l multiplies the activation tile in
//                    shared memory (A, K-major, 128-byte swizzle) by the weight chunk
//                    (B) into one TMEM accumulator of up to 256 fp32 columns.
//   warps 2..9     : epilogue -- read the accumulator (one row per thread), add bias,
//                    ReLU, round to the 16-bit storage type and write the result back
//                    into the activation tile in exactly the swizzled K-major layout
//                    the next layer's MMAs read; the last layer ends in the row head
//                    (masked softmax / regret matching / argmax) written to global.
// 16-bit arithmetic classes only (SB_F16, SB_BF16); widths: input <= 256 and a
// multiple of 8, hidden layers multiples of 64 up to 256, output <= 32.
#include "common.cuh"

namespace {

constexpr int FM_MAX_LAYERS = 8;
constexpr int FM_THREADS = 320;
constexpr int FM_EPI_WARPS = 8;
constexpr int FM_W_STAGES = 4;
constexpr uint32_t FM_CHUNK_BYTES = 128u * 128u;       // activation chunk: 128 rows x 64 elements x 2 B
constexpr uint32_t FM_STAGE_BYTES = 256u * 128u;       // weight stage: up to 256 rows x 64 elements x 2 B

struct FusedMaps {
  CUtensorMap x;                      // [batch, in] box {64, 128}
  CUtensorMap w[FM_MAX_LAYERS];       // W_l [members, out_l, in_l] box {64, rows_l, 1}
};

struct FusedParams {
  int n_layers;
  int batch;
  int width[FM_MAX_LAYERS + 1];       // width[0] = input features
  int n_pad[FM_MAX_LAYERS];           // MMA N of layer l (hidden: width; last: padded to 16 or 32)
  int k_chunks[FM_MAX_LAYERS];        // ceil(in_l / 64)
  uint32_t idesc[FM_MAX_LAYERS];
  uint32_t w_bytes[FM_MAX_LAYERS];    // bytes of one weight chunk of layer l
  const float* bias[FM_MAX_LAYERS];   // may be null
  int is_bf16;
  int tmem_cols;
  int num_tiles;                      // 128-row tiles of the batch
  int num_items;                      // work items = tiles x ensemble members
  long long member_stride;            // elements between two members' parameter vectors
  long long out_stride;               // elements between two members' outputs (batch x n_out)
  uint32_t x_chunks;                  // chunks of the input tile
  uint32_t act_offset, w_offset;      // byte offsets of the activation tile and the weight ring
  // head
  float* out;
  const uint8_t* mask;
  int32_t* actions;
  int head;
};

struct HeadArgsF {
  float* out;
  const float* bias;
  const uint8_t* mask;
  int32_t* actions;
  int N, epi;
};

// Row head on one full row held by a thread (same math as the GEMM's fused head;
// ml/primitives.spi:705-708, 748-780).
template <int W>
__device__ __forceinline__ void fused_head_row(const HeadArgsF& h, float* v, long long row) {
  const int n = h.N;
  float* crow = h.out + row * n;
  const uint8_t* mrow = h.mask ? h.mask + row * (long long)n : nullptr;
  uint32_t legal = 0;
#pragma unroll
  for (int j = 0; j < W; ++j) {
    if (j < n) {
      if (h.bias) v[j] += __ldg(h.bias + j);
      if (!mrow || mrow[j] != 0) legal |= (1u << j);
    }
  }
  const int count = __popc(legal);
  if (h.epi & SB_EPI_MASKED_SOFTMAX) {
    float mx = -3.402823466e38f;
#pragma unroll
    for (int j = 0; j < W; ++j)
      if (j < n && ((legal >> j) & 1u)) mx = fmaxf(mx, v[j]);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < W; ++j) {
      if (j < n) {
        const float e = ((legal >> j) & 1u) ? __expf(v[j] - mx) : 0.f;
        v[j] = e;
        s += e;
      }
    }
    const float inv = s > 0.f ? 1.f / s : 0.f;
#pragma unroll
    for (int j = 0; j < W; ++j)
      if (j < n) v[j] *= inv;
  }
  if (h.epi & SB_EPI_REGRET_MATCHING) {
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < W; ++j) {
      if (j < n) {
        const float q = ((legal >> j) & 1u) ? fmaxf(v[j], 0.f) : 0.f;
        v[j] = q;
        s += q;
      }
    }
    const float inv_len = count > 0 ? 1.f / (float)count : 0.f;
#pragma unroll
    for (int j = 0; j < W; ++j)
      if (j < n) v[j] = !((legal >> j) & 1u) ? 0.f : (s != 0.f ? v[j] / s : inv_len);
  }
#pragma unroll
  for (int j = 0; j < W; ++j)
    if (j < n) crow[j] = v[j];
  if (h.epi & SB_EPI_ARGMAX) {
    int best = 0;
    float bv = v[0];
#pragma unroll
    for (int j = 1; j < W; ++j) {
      if (j < n && v[j] > bv) {
        bv = v[j];
        best = j;
      }
    }
    h.actions[row] = best;
  }
}

template <int W>
__device__ __noinline__ void fused_head(HeadArgsF h, uint32_t t_row, long long row, int batch) {
  uint32_t raw[W];
  if (W == 32) tmem_ld32(t_row, raw); else tmem_ld16(t_row, raw);
  tmem_ld_wait();
  if (row < batch) fused_head_row<W>(h, reinterpret_cast<float*>(raw), row);
}

// One warp's share of a hidden layer: chunks `half`, half+2, ... of 32 columns.
// Writes relu(acc + bias) in the storage type into the activation tile, in the
// 128-byte-swizzled K-major layout the next layer's A descriptors expect:
// element (row, j) -> chunk j / 64, byte row * 128 + (((j % 64) / 8) ^ (row % 8)) * 16 + (j % 8) * 2.
template <bool BF16>
__device__ __noinline__ void fused_hidden(uint32_t t_row, int n_cols, const float* bias, uint32_t act_base,
                                          uint32_t bias_smem, int row_in_tile, int lane, int half) {
  const int nchunks = n_cols >> 5;
  float bias_cur = 0.f, bias_nxt = 0.f;
  if (bias && half < nchunks) bias_cur = __ldg(bias + half * 32 + lane);
  for (int c = half; c < nchunks; c += 2) {
    uint32_t raw[32];
    tmem_ld32(t_row + (uint32_t)(c * 32), raw);
    if (bias && c + 2 < nchunks) bias_nxt = __ldg(bias + (c + 2) * 32 + lane);
    tmem_ld_wait();
    float* v = reinterpret_cast<float*>(raw);
    if (bias) {
      asm volatile("st.shared.f32 [%0], %1;" ::"r"(bias_smem + 4u * (uint32_t)lane), "f"(bias_cur) : "memory");
      __syncwarp();
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        uint4 b;
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w)
                     : "r"(bias_smem + 16u * (uint32_t)q) : "memory");
        v[4 * q + 0] += __uint_as_float(b.x);
        v[4 * q + 1] += __uint_as_float(b.y);
        v[4 * q + 2] += __uint_as_float(b.z);
        v[4 * q + 3] += __uint_as_float(b.w);
      }
      __syncwarp();
    }
    const int col0 = c * 32;
    const uint32_t chunk_base = act_base + (uint32_t)(col0 >> 6) * FM_CHUNK_BYTES + (uint32_t)row_in_tile * 128u;
    const uint32_t piece0 = (uint32_t)((col0 & 63) >> 3);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t packed[4];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float lo = fmaxf(v[q * 8 + 2 * t], 0.f), hi = fmaxf(v[q * 8 + 2 * t + 1], 0.f);
        if (BF16) {
          __nv_bfloat162 h2 = __floats2bfloat162_rn(lo, hi);
          packed[t] = *reinterpret_cast<uint32_t*>(&h2);
        } else {
          __half2 h2 = __floats2half2_rn(lo, hi);
          packed[t] = *reinterpret_cast<uint32_t*>(&h2);
        }
      }
      const uint32_t addr = chunk_base + (((piece0 + (uint32_t)q) ^ ((uint32_t)row_in_tile & 7u)) << 4);
      st_shared_v4(addr, make_uint4(packed[0], packed[1], packed[2], packed[3]));
    }
    bias_cur = bias_nxt;
  }
}

__global__ void __launch_bounds__(FM_THREADS, 1)
mlp_fused_kernel(const __grid_constant__ FusedMaps maps, const __grid_constant__ FusedParams p) {
  extern __shared__ uint8_t fm_smem_raw[];
  __shared__ __align__(8) uint64_t bar_x_full, bar_x_empty, bar_acc_full, bar_act_ready;
  __shared__ __align__(8) uint64_t bar_w_full[FM_W_STAGES], bar_w_empty[FM_W_STAGES];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ __align__(16) float bias_spread[FM_EPI_WARPS][32];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t base = (smem_u32(fm_smem_raw) + 1023u) & ~1023u;
  const uint32_t x_base = base;                      // input tile: x_chunks x 16 KB
  const uint32_t act_base = base + p.act_offset;     // activation tile: up to 4 chunks
  const uint32_t w_base = base + p.w_offset;         // weight ring

  if (tid == 0) {
    mbar_init(smem_u32(&bar_x_full), 1);
    mbar_init(smem_u32(&bar_x_empty), 1);
    mbar_init(smem_u32(&bar_acc_full), 1);
    mbar_init(smem_u32(&bar_act_ready), FM_EPI_WARPS);
    for (int s = 0; s < FM_W_STAGES; ++s) {
      mbar_init(smem_u32(&bar_w_full[s]), 1);
      mbar_init(smem_u32(&bar_w_empty[s]), 1);
    }
    abort_flag = 0;
    fence_mbar_init();
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
  const int L = p.n_layers;
  // Set-up above touched only this CTA's shared and tensor memory; everything below reads or writes
  // global memory and therefore waits for the kernel before it on the stream.
  sb_grid_dependency_wait();
  sb_grid_dependents_launch();

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t w_phase = 0, x_phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x) {
        const int member = item / p.num_tiles, tile = item - member * p.num_tiles;
        if (!mbar_wait(smem_u32(&bar_x_empty), x_phase ^ 1u, abortp, SB_SITE_MLP_ACT)) break;
        x_phase ^= 1u;
        mbar_arrive_expect_tx(smem_u32(&bar_x_full), p.x_chunks * FM_CHUNK_BYTES);
        for (uint32_t c = 0; c < p.x_chunks; ++c)
          tma_load_2d(x_base + c * FM_CHUNK_BYTES, &maps.x, (int)(c * 64), tile * 128, smem_u32(&bar_x_full));
        for (int l = 0; ok && l < L; ++l) {
          for (int c = 0; c < p.k_chunks[l]; ++c) {
            if (!mbar_wait(smem_u32(&bar_w_empty[stage]), w_phase ^ 1u, abortp, SB_SITE_MLP_WEIGHTS)) {
              ok = false;
              break;
            }
            mbar_arrive_expect_tx(smem_u32(&bar_w_full[stage]), p.w_bytes[l]);
            tma_load_3d(w_base + (uint32_t)stage * FM_STAGE_BYTES, &maps.w[l], c * 64, 0, member, smem_u32(&bar_w_full[stage]));
            if (++stage == FM_W_STAGES) {
              stage = 0;
              w_phase ^= 1u;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t w_phase = 0, x_phase = 0, act_phase = 0;
      bool ok = true;
      const uint32_t hi = (uint32_t)(umma_smem_desc(0u, 16u, 1024u, 2u) >> 32);
      for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x) {
        for (int l = 0; ok && l < L; ++l) {
          uint32_t a_base;
          if (l == 0) {
            if (!mbar_wait(smem_u32(&bar_x_full), x_phase, abortp, SB_SITE_MLP_ACT)) { ok = false; break; }
            x_phase ^= 1u;
            a_base = x_base;
          } else {
            // the epilogue has drained the accumulator and written this layer's input
            if (!mbar_wait(smem_u32(&bar_act_ready), act_phase, abortp, SB_SITE_MLP_ACT)) { ok = false; break; }
            act_phase ^= 1u;
            a_base = act_base;
          }
          tc_fence_after_sync();
          uint32_t accumulate = 0u;
          for (int c = 0; c < p.k_chunks[l]; ++c) {
            if (!mbar_wait(smem_u32(&bar_w_full[stage]), w_phase, abortp, SB_SITE_MLP_WEIGHTS)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t a_lo = (uint32_t)umma_smem_desc(a_base + (uint32_t)c * FM_CHUNK_BYTES, 16u, 1024u, 2u);
            const uint32_t b_lo = (uint32_t)umma_smem_desc(w_base + (uint32_t)stage * FM_STAGE_BYTES, 16u, 1024u, 2u);
#pragma unroll
            for (uint32_t ks = 0; ks < 4; ++ks) {
              umma_issue<false, false>(tmem_base, a_lo + 2u * ks, hi, b_lo + 2u * ks, hi, p.idesc[l], accumulate);
              accumulate = 1u;
            }
            tc_commit(smem_u32(&bar_w_empty[stage]));
            if (++stage == FM_W_STAGES) {
              stage = 0;
              w_phase ^= 1u;
            }
          }
          if (!ok) break;
          if (l == 0) tc_commit(smem_u32(&bar_x_empty));     // the input tile may be refilled
          tc_commit(smem_u32(&bar_acc_full));
        }
        // The next tile's first layer overwrites the accumulator: wait until the head has read it.
        if (ok && item + (int)gridDim.x < p.num_items) {
          if (!mbar_wait(smem_u32(&bar_act_ready), act_phase, abortp, SB_SITE_MLP_ACT)) break;
          act_phase ^= 1u;
        }
      }
    }
  } else {
    const int quad = warp & 3, half = (warp - 2) >> 2;
    const int row_in_tile = quad * 32 + lane;
    const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16);
    const uint32_t bias_smem = smem_u32(&bias_spread[warp - 2][0]);
    uint32_t acc_phase = 0;
    HeadArgsF h;
    h.out = p.out; h.bias = p.bias[L - 1]; h.mask = p.mask; h.actions = p.actions;
    h.N = p.width[L]; h.epi = p.head;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x) {
      const int member = item / p.num_tiles, tile = item - member * p.num_tiles;
      const long long pofs = (long long)member * p.member_stride;
      h.out = p.out + (long long)member * p.out_stride;
      h.actions = p.actions ? p.actions + (long long)member * p.batch : nullptr;
      h.bias = p.bias[L - 1] ? p.bias[L - 1] + pofs : nullptr;
      for (int l = 0; l < L; ++l) {
        if (!mbar_wait(smem_u32(&bar_acc_full), acc_phase, abortp, SB_SITE_MLP_ACC)) { ok = false; break; }
        acc_phase ^= 1u;
        tc_fence_after_sync();
        if (l < L - 1) {
          const float* bias_l = p.bias[l] ? p.bias[l] + pofs : nullptr;
          if (p.is_bf16) fused_hidden<true>(t_row, p.n_pad[l], bias_l, act_base, bias_smem, row_in_tile, lane, half);
          else fused_hidden<false>(t_row, p.n_pad[l], bias_l, act_base, bias_smem, row_in_tile, lane, half);
          // generic-proxy writes of the activation tile must be visible to the MMA's async-proxy reads
          fence_proxy_async_smem();
        } else if (half == 0) {
          const long long row = (long long)tile * 128 + row_in_tile;
          if (p.n_pad[l] >= 32) fused_head<32>(h, t_row, row, p.batch);
          else fused_head<16>(h, t_row, row, p.batch);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_act_ready));
      }
    }
  }

  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (*abortp != 0) {
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) { }
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

}  // namespace

// 3-D tensor map over the weights of one layer of every ensemble member: [members, rows, cols] with
// `member_stride` elements between members, box {64 columns, box_rows, 1 member}, 128-byte swizzle.
static int make_tmap_members(CUtensorMap* map, const void* base, int in_dtype, int members, long long member_stride,
                             int rows, int cols, int box_rows) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return sb_fail(SB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  CUtensorMapDataType dt = in_dtype == SB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  cuuint64_t gdim[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)members};
  cuuint64_t gstride[2] = {(cuuint64_t)cols * 2u, (cuuint64_t)member_stride * 2u};
  cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, 1u};
  cuuint32_t estr[3] = {1, 1, 1};
  if (members == 1) gstride[1] = (cuuint64_t)rows * cols * 2u;      // unused dimension: any legal stride
  gstride[1] = (gstride[1] + 15u) / 16u * 16u;
  CUresult r = enc(map, dt, 3, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return sb_fail(SB_ERR_CUDA, "cuTensorMapEncodeTiled (3-D) failed with CUresult %d (members=%d rows=%d cols=%d)",
                   (int)r, members, rows, cols);
  return SB_OK;
}

extern "C" int sb_mlp_forward_fused_ensemble(int n_layers, const int* sizes, int batch, int members, int in_dtype,
                                             const void* x, const void* w_compute, const float* params, int head,
                                             const uint8_t* mask, float* out, int32_t* actions, void* stream);

extern "C" int sb_mlp_forward_fused(int n_layers, const int* sizes, int batch, int in_dtype, const void* x,
                                    const void* w_compute, const float* params, int head, const uint8_t* mask,
                                    float* out, int32_t* actions, void* stream) {
  return sb_mlp_forward_fused_ensemble(n_layers, sizes, batch, 1, in_dtype, x, w_compute, params, head, mask, out,
                                       actions, stream);
}

extern "C" int sb_mlp_forward_fused_ensemble(int n_layers, const int* sizes, int batch, int members, int in_dtype,
                                             const void* x, const void* w_compute, const float* params, int head,
                                             const uint8_t* mask, float* out, int32_t* actions, void* stream) {
  if (members < 1 || members > 1024) return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_forward_fused: 1..1024 ensemble members");
  if (n_layers < 1 || n_layers > FM_MAX_LAYERS) return sb_fail(SB_ERR_UNSUPPORTED, "sb_mlp_forward_fused: 1..%d layers", FM_MAX_LAYERS);
  if (!sizes) return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_forward_fused: sizes is null");
  if (in_dtype != SB_F16 && in_dtype != SB_BF16)
    return sb_fail(SB_ERR_UNSUPPORTED, "sb_mlp_forward_fused: 16-bit arithmetic classes only (SB_F16, SB_BF16)");
  if (batch < 0) return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_forward_fused: negative batch");
  if (head & ~(SB_EPI_MASKED_SOFTMAX | SB_EPI_REGRET_MATCHING | SB_EPI_ARGMAX))
    return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_forward_fused: head may hold only row-head flags");
  if (sizes[0] < 8 || sizes[0] > 256 || sizes[0] % 8) return sb_fail(SB_ERR_UNSUPPORTED, "sb_mlp_forward_fused: input width %d (8..256, multiple of 8)", sizes[0]);
  for (int i = 1; i < n_layers; ++i)
    if (sizes[i] < 64 || sizes[i] > 256 || sizes[i] % 64)
      return sb_fail(SB_ERR_UNSUPPORTED, "sb_mlp_forward_fused: hidden width %d (64..256, multiple of 64)", sizes[i]);
  if (sizes[n_layers] < 1 || sizes[n_layers] > 32) return sb_fail(SB_ERR_UNSUPPORTED, "sb_mlp_forward_fused: output width %d (1..32)", sizes[n_layers]);
  if (batch == 0) return SB_OK;
  if (!x || !w_compute || !out) return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_forward_fused: null pointer");
  if ((head & SB_EPI_ARGMAX) && !actions) return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_forward_fused: SB_EPI_ARGMAX without an actions buffer");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w_compute)) & 15)
    return sb_fail(SB_ERR_MISALIGNED, "sb_mlp_forward_fused: x and w_compute must be 16-byte aligned");

  long long off[2 * FM_MAX_LAYERS + 1];
  int rc = sb_mlp_param_offsets(n_layers, sizes, off);
  if (rc != SB_OK) return rc;

  FusedMaps maps;
  FusedParams p;
  memset(&p, 0, sizeof(p));
  p.n_layers = n_layers;
  p.batch = batch;
  p.is_bf16 = in_dtype == SB_BF16;
  p.num_tiles = (batch + 127) / 128;
  p.num_items = p.num_tiles * members;
  p.member_stride = off[2 * n_layers];
  p.out_stride = (long long)batch * sizes[n_layers];
  int max_n = 32;
  uint32_t max_act_chunks = 1;
  for (int l = 0; l <= n_layers; ++l) p.width[l] = sizes[l];
  for (int l = 0; l < n_layers; ++l) {
    const bool last = l == n_layers - 1;
    p.n_pad[l] = last ? (sizes[l + 1] <= 16 ? 16 : 32) : sizes[l + 1];
    p.k_chunks[l] = (sizes[l] + 63) / 64;
    p.idesc[l] = sb_umma_idesc(in_dtype, 0, 0, 128, p.n_pad[l]);
    p.w_bytes[l] = (uint32_t)p.n_pad[l] * 128u;
    p.bias[l] = params ? params + off[2 * l + 1] : nullptr;
    if (p.n_pad[l] > max_n) max_n = p.n_pad[l];
    if (l > 0 && (uint32_t)p.k_chunks[l] > max_act_chunks) max_act_chunks = (uint32_t)p.k_chunks[l];
    const void* w = reinterpret_cast<const char*>(w_compute) + off[2 * l] * 2;
    rc = make_tmap_members(&maps.w[l], w, in_dtype, members, p.member_stride, sizes[l + 1], sizes[l], p.n_pad[l]);
    if (rc != SB_OK) return rc;
  }
  for (int l = n_layers; l < FM_MAX_LAYERS; ++l) maps.w[l] = maps.w[0];
  rc = make_tmap_2d(&maps.x, x, in_dtype, batch, sizes[0], 128, 64, SWZ_128);
  if (rc != SB_OK) return rc;
  p.x_chunks = (uint32_t)p.k_chunks[0];
  p.act_offset = p.x_chunks * FM_CHUNK_BYTES;
  p.w_offset = p.act_offset + max_act_chunks * FM_CHUNK_BYTES;
  p.tmem_cols = 32;
  while (p.tmem_cols < max_n) p.tmem_cols <<= 1;
  p.out = out; p.mask = mask; p.actions = actions; p.head = head;
  const size_t smem = (size_t)p.w_offset + (size_t)FM_W_STAGES * FM_STAGE_BYTES + 1024;

  static std::atomic<bool> attr_set[64];
  int dev = 0;
  SB_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[dev].load(std::memory_order_acquire)) {
    SB_CUDA(cudaFuncSetAttribute(mlp_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024));
    attr_set[dev].store(true, std::memory_order_release);
  }
  if (smem > 225 * 1024) return sb_fail(SB_ERR_UNSUPPORTED, "sb_mlp_forward_fused: %zu bytes of shared memory needed", smem);
  const int sms = sb_sm_count();
  const int grid = p.num_items < sms ? p.num_items : sms;
  double flops = 0.0;
  for (int l = 0; l < n_layers; ++l) flops += 2.0 * batch * (double)sizes[l] * sizes[l + 1] * members;
  sb_prof_before((cudaStream_t)stream);
  SB_CUDA(sb_launch(mlp_fused_kernel, dim3(grid), dim3(FM_THREADS), smem, (cudaStream_t)stream, 1, maps, p));
  sb_prof_after((cudaStream_t)stream, flops);
  SB_COUNT_LAUNCH();
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}
