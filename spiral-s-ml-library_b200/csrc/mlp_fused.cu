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
// 16-bit arithmetic classes only (SB_F16, SB_BF16); widths: input <= 512 and a
// multiple of 8 (inputs beyond 256 as far as shared memory allows: the reference's Hold'em
// policy net is 512 -> 64, game/nl_hu_holdem/model_cem.spi:71-98), hidden layers multiples of 64 up to 256, output <= 64 (<= 256 when a
// prefix mask confines the head to its first 64 columns, the shape of the reference's
// own policy nets, game/leduc/model_cem.spi:37,52-60).
//
// Optional, for the reference's graphs: ln_l2 before every ReLU (ml/layers.spi:562-568), a
// sampling head that draws from a Philox stream per row (ml/layers.spi:422-431), and the
// per-decision tail of ml/models.spi:51-76 (pick a member per row, report its action and the
// probabilities every member gave that action), done by whichever CTA finishes the last member
// of a row tile.
#include "common.cuh"
#include "row_head.cuh"

namespace {

constexpr int FM_MAX_LAYERS = 8;
constexpr int FM_THREADS = 320;
constexpr int FM_EPI_WARPS = 8;
constexpr int FM_W_STAGES = 4;
constexpr uint32_t FM_CHUNK_BYTES = 128u * 128u;       // activation chunk: 128 rows x 64 elements x 2 B
// A weight stage holds one 64-column K-chunk of a layer: (widest layer's rows) x 128 bytes, at most 256 rows.

struct FusedMaps {
  CUtensorMap x;                      // [batch, in] box {64, 128}
  CUtensorMap w[FM_MAX_LAYERS];       // W_l [members, out_l, in_l] box {64, rows_l, 1}
  CUtensorMap act[FM_MAX_LAYERS];     // training forward: hidden activations of layer l, [batch, width_l] box {64, 128}
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
  int acc_stride;                     // TMEM columns between the two accumulators (layers alternate between them)
  int num_tiles;                      // 128-row tiles of the batch
  int num_items;                      // work items = tiles x ensemble members
  long long member_stride;            // elements between two members' parameter vectors
  long long out_stride;               // elements between two members' outputs (batch x n_out)
  uint32_t x_chunks;                  // chunks of the input tile
  uint32_t stage_bytes;               // bytes of one weight stage
  uint32_t act_offset, w_offset;      // byte offsets of the activation tile and the weight ring
  // head
  float* out;
  SbRowHead head;                     // n, flags, prefix, mask, seed, ...; argmax_out / sample_out are [members, batch]
  int hidden_norm;                    // 1: x / sum(x^2) over the row before every ReLU
  // training forward: the hidden activations and their ReLU sign words are also written to global
  // memory for the backward pass (single net only)
  int store_acts;
  uint32_t* bits[FM_MAX_LAYERS];      // uint32 [width_l / 32, batch] per hidden layer, or null
  // decision tail (null counters = off)
  int members;
  int* tile_counters;                 // int32 [num_tiles], zero between calls
  int32_t* ensemble_id;               // [batch]
  int32_t* action;                    // [batch]
  float* prob_selected;               // [batch]
  float* prob_ensemble;               // [batch, members]
};

// The last layer: a thread takes the first W values of its row out of tensor memory, adds the bias and
// hands over to the shared row head.
template <int W>
__device__ __noinline__ void fused_head(const SbRowHead& h, const float* bias, float* out, uint32_t t_row, long long row,
                                        int batch) {
  uint32_t raw[W];
  if constexpr (W == 64) {
    tmem_ld32(t_row, raw);
    tmem_ld32(t_row + 32u, raw + 32);
  } else if constexpr (W == 32) {
    tmem_ld32(t_row, raw);
  } else {
    tmem_ld16(t_row, raw);
  }
  tmem_ld_wait();
  if (row >= batch) return;
  float* v = reinterpret_cast<float*>(raw);
  if (bias) {
#pragma unroll
    for (int j = 0; j < W; ++j)
      if (j < h.n) v[j] += __ldg(bias + j);
  }
  sb_row_head_finish<W>(h, v, row, out + row * h.n);
}

// One warp's share of a hidden layer: chunks `half`, half+2, ... of 32 columns.
// Writes relu(acc + bias) in the storage type into the activation tile, in the
// 128-byte-swizzled K-major layout the next layer's A descriptors expect:
// element (row, j) -> chunk j / 64, byte row * 128 + (((j % 64) / 8) ^ (row % 8)) * 16 + (j % 8) * 2.
// After each 32-column chunk the warp arrives on the barrier of the 64-column activation chunk it
// belongs to (`chunk_bar0` + 8 bytes per chunk): the next layer's MMAs on that K-chunk start as soon as
// all eight warps have delivered it, while the later chunks of this layer are still being finished.
template <bool BF16>
__device__ __noinline__ void fused_hidden(uint32_t t_row, int n_cols, const float* bias, uint32_t act_base,
                                          uint32_t bias_smem, int row_in_tile, int lane, int half, int norm,
                                          uint32_t chunk_bar0, uint32_t* bits_out, long long row, int batch) {
  const int nchunks = n_cols >> 5;
  // Row normalisation (local_ln_l2, ml/primitives.spi:701-703; no bias in this mode): a first pass
  // over the whole accumulator row sums the squares; both warps of a quadrant do it for themselves.
  float sumsq = 0.f;
  if (norm) {
    for (int c = 0; c < nchunks; ++c) {
      uint32_t raw[32];
      tmem_ld32(t_row + (uint32_t)(c * 32), raw);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) sumsq = fmaf(__uint_as_float(raw[j]), __uint_as_float(raw[j]), sumsq);
    }
  }
  float bias_cur = 0.f, bias_nxt = 0.f;
  if (bias && half < nchunks) bias_cur = __ldg(bias + half * 32 + lane);
  for (int c = half; c < nchunks; c += 2) {
    uint32_t raw[32];
    tmem_ld32(t_row + (uint32_t)(c * 32), raw);
    if (bias && c + 2 < nchunks) bias_nxt = __ldg(bias + (c + 2) * 32 + lane);
    tmem_ld_wait();
    float* v = reinterpret_cast<float*>(raw);
    if (norm) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = sumsq != 0.f ? v[j] / sumsq : 0.f;
    }
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
    if (bits_out) {
      // ReLU sign word of this row and chunk (bit j = value j > 0), stored [chunk, row]: the 32 rows of
      // the warp are 32 consecutive words.  The backward pass gates its gradients by these words.
      uint32_t signs = 0u;
#pragma unroll
      for (int j = 0; j < 32; ++j) signs |= (v[j] > 0.f ? 1u : 0u) << j;
      if (row < batch) bits_out[(long long)c * batch + row] = signs;
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
    // generic-proxy writes of the activation tile must be visible to the MMA's async-proxy reads
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) mbar_arrive(chunk_bar0 + 8u * (uint32_t)(c >> 1));
  }
}

// The per-decision tail for one state, once every member's probabilities and sampled index are in
// global memory: draw a member, report its action, the probability it gave the action and the
// probability every member gave it (ml/models.spi:51-76).
__device__ __noinline__ void decide_row(const FusedParams& p, long long row) {
  if (row >= p.batch) return;
  const int n = p.head.n;
  const unsigned long long stream = p.head.row_offset + (unsigned long long)row;
  // drawn after the members' sampling draws (outputs position .. position + members - 1 of the stream)
  const int e_id = (int)sb_philox_below(p.head.seed, stream, p.head.position + (unsigned long long)p.members,
                                        (uint32_t)p.members);
  const int a = __ldcg(p.head.sample_out + (long long)e_id * p.batch + row);
  p.ensemble_id[row] = e_id;
  p.action[row] = a;
  const float* prow = p.out + row * n;
  p.prob_selected[row] = a >= 0 ? __ldcg(prow + (long long)e_id * p.out_stride + a) : 0.f;
  for (int e = 0; e < p.members; ++e)
    p.prob_ensemble[row * p.members + e] = a >= 0 ? __ldcg(prow + (long long)e * p.out_stride + a) : 0.f;
}

__global__ void __launch_bounds__(FM_THREADS, 1)
mlp_fused_kernel(const __grid_constant__ FusedMaps maps, const __grid_constant__ FusedParams p) {
  extern __shared__ uint8_t fm_smem_raw[];
  __shared__ __align__(8) uint64_t bar_x_full, bar_x_empty, bar_acc_full, bar_item_done, bar_tail_in, bar_tail_out;
  __shared__ __align__(8) uint64_t bar_chunk[4];       // 64-column chunk k of the activation tile is written (8 warps each)
  __shared__ __align__(8) uint64_t bar_w_full[FM_W_STAGES], bar_w_empty[FM_W_STAGES];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ int tile_is_complete;
  __shared__ SbRowHead head_slot[FM_EPI_WARPS];
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
    mbar_init(smem_u32(&bar_item_done), FM_EPI_WARPS);
    for (int k = 0; k < 4; ++k) mbar_init(smem_u32(&bar_chunk[k]), FM_EPI_WARPS);
    mbar_init(smem_u32(&bar_tail_in), 4);       // the four warps that finish head rows
    mbar_init(smem_u32(&bar_tail_out), 1);
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
            tma_load_3d(w_base + (uint32_t)stage * p.stage_bytes, &maps.w[l], c * 64, 0, member, smem_u32(&bar_w_full[stage]));
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
      uint32_t w_phase = 0, x_phase = 0, item_phase = 0, chunk_phase = 0;     // chunk_phase: one parity bit per chunk barrier
      bool ok = true;
      const uint32_t hi = (uint32_t)(umma_smem_desc(0u, 16u, 1024u, 2u) >> 32);
      for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x) {
        const int tile = item % p.num_tiles;
        for (int l = 0; ok && l < L; ++l) {
          uint32_t a_base;
          if (l == 0) {
            if (!mbar_wait(smem_u32(&bar_x_full), x_phase, abortp, SB_SITE_MLP_ACT)) { ok = false; break; }
            x_phase ^= 1u;
            a_base = x_base;
          } else {
            a_base = act_base;
          }
          tc_fence_after_sync();
          // Layers alternate between two accumulators: the epilogue of layer l-1 still reads its own while
          // this layer's first MMAs run.  (Layer l+1 reuses the accumulator of layer l-1 only after every
          // chunk of this layer's input -- the whole of layer l-1's epilogue -- has been delivered.)
          const uint32_t d_tmem = tmem_base + (uint32_t)((l & 1) * p.acc_stride);
          uint32_t accumulate = 0u;
          for (int c = 0; c < p.k_chunks[l]; ++c) {
            if (l > 0) {
              // K-chunk c of this layer's input = 64-column chunk c of the previous layer's output
              if (!mbar_wait(smem_u32(&bar_chunk[c]), (chunk_phase >> c) & 1u, abortp, SB_SITE_MLP_ACT)) { ok = false; break; }
              chunk_phase ^= 1u << c;
              tc_fence_after_sync();
              // Training forward: the delivered chunk of the previous layer's output also leaves for global
              // memory; the tile in shared memory already has the layout of a TMA box.
              if (p.store_acts) {
                tma_store_2d(&maps.act[l - 1], a_base + (uint32_t)c * FM_CHUNK_BYTES, c * 64, tile * 128);
                bulk_commit_group();
              }
            }
            if (!mbar_wait(smem_u32(&bar_w_full[stage]), w_phase, abortp, SB_SITE_MLP_WEIGHTS)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t a_lo = (uint32_t)umma_smem_desc(a_base + (uint32_t)c * FM_CHUNK_BYTES, 16u, 1024u, 2u);
            const uint32_t b_lo = (uint32_t)umma_smem_desc(w_base + (uint32_t)stage * p.stage_bytes, 16u, 1024u, 2u);
#pragma unroll
            for (uint32_t ks = 0; ks < 4; ++ks) {
              umma_issue<false, false>(d_tmem, a_lo + 2u * ks, hi, b_lo + 2u * ks, hi, p.idesc[l], accumulate);
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
          // This layer's epilogue overwrites the activation tile: the stores of its chunks must have read it.
          if (p.store_acts && l > 0) bulk_wait_group_read<0>();
          tc_commit(smem_u32(&bar_acc_full));
        }
        // The next tile's layers overwrite the accumulators and the activation tile: wait until the head
        // has read the last accumulator.
        if (ok && item + (int)gridDim.x < p.num_items) {
          if (!mbar_wait(smem_u32(&bar_item_done), item_phase, abortp, SB_SITE_MLP_ACT)) break;
          item_phase ^= 1u;
        }
      }
    }
  } else {
    const int quad = warp & 3, half = (warp - 2) >> 2;
    const int row_in_tile = quad * 32 + lane;
    const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16);
    const uint32_t bias_smem = smem_u32(&bias_spread[warp - 2][0]);
    uint32_t acc_phase = 0, tail_phase = 0;
    // This warp's copy of the head description (in shared memory: the head code reads a field where it
    // needs it instead of holding the whole structure in registers); member-specific fields are set per item.
    SbRowHead& h = head_slot[warp - 2];
    if (lane == 0) h = p.head;
    __syncwarp();
    bool ok = true;
    for (int item = blockIdx.x; ok && item < p.num_items; item += gridDim.x) {
      const int member = item / p.num_tiles, tile = item - member * p.num_tiles;
      const long long pofs = (long long)member * p.member_stride;
      float* out_m = p.out + (long long)member * p.out_stride;
      if (lane == 0) {
        h.argmax_out = p.head.argmax_out ? p.head.argmax_out + (long long)member * p.batch : nullptr;
        h.sample_out = p.head.sample_out ? p.head.sample_out + (long long)member * p.batch : nullptr;
        h.position = p.head.position + (unsigned long long)member;      // one draw per member from the row's stream
      }
      __syncwarp();
      const float* head_bias = p.bias[L - 1] ? p.bias[L - 1] + pofs : nullptr;
      for (int l = 0; l < L; ++l) {
        if (!mbar_wait(smem_u32(&bar_acc_full), acc_phase, abortp, SB_SITE_MLP_ACC)) { ok = false; break; }
        acc_phase ^= 1u;
        tc_fence_after_sync();
        const uint32_t t_acc = t_row + (uint32_t)((l & 1) * p.acc_stride);
        if (l < L - 1) {
          const float* bias_l = p.bias[l] ? p.bias[l] + pofs : nullptr;
          const long long grow = (long long)tile * 128 + row_in_tile;
          if (p.is_bf16) fused_hidden<true>(t_acc, p.n_pad[l], bias_l, act_base, bias_smem, row_in_tile, lane, half, p.hidden_norm, smem_u32(&bar_chunk[0]), p.bits[l], grow, p.batch);
          else fused_hidden<false>(t_acc, p.n_pad[l], bias_l, act_base, bias_smem, row_in_tile, lane, half, p.hidden_norm, smem_u32(&bar_chunk[0]), p.bits[l], grow, p.batch);
        } else {
          if (half == 0) {
            const long long row = (long long)tile * 128 + row_in_tile;
            if (p.n_pad[l] > 32) fused_head<64>(h, head_bias, out_m, t_acc, row, p.batch);
            else if (p.n_pad[l] > 16) fused_head<32>(h, head_bias, out_m, t_acc, row, p.batch);
            else fused_head<16>(h, head_bias, out_m, t_acc, row, p.batch);
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bar_item_done));
        }
      }
      if (ok && p.tile_counters && half == 0) {
        // Decision tail (ml/models.spi:51-76).  The four head warps publish their rows of this member, count
        // the member in; the CTA that counts the last member of the tile in sees every member's results.
        // The two meeting points are mbarriers with bounded waits, like every other wait of the kernel.
        __threadfence();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_tail_in));
        if (warp == 2 && lane == 0) {
          if (mbar_wait(smem_u32(&bar_tail_in), tail_phase, abortp, SB_SITE_MLP_ACT)) {
            __threadfence();
            const int before = atomicAdd(p.tile_counters + tile, 1);
            __threadfence();
            tile_is_complete = before == p.members - 1 ? 1 : 0;
          } else {
            tile_is_complete = 0;
          }
          mbar_arrive(smem_u32(&bar_tail_out));
        }
        if (!mbar_wait(smem_u32(&bar_tail_out), tail_phase, abortp, SB_SITE_MLP_ACT)) break;
        tail_phase ^= 1u;
        if (tile_is_complete) {
          __threadfence();
          decide_row(p, (long long)tile * 128 + row_in_tile);
          if (warp == 2 && lane == 0) p.tile_counters[tile] = 0;        // ready for the next call
        }
        // tile_is_complete is rewritten only after all four warps have arrived for the next item.
      }
    }
  }

  if (warp == 1 && lane == 0 && p.store_acts) bulk_wait_group<0>();
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

// What the per-decision tail writes (all null = no tail).
struct FusedDecide {
  int* tile_counters;
  int32_t* ensemble_id;
  int32_t* action;
  float* prob_selected;
  float* prob_ensemble;
};

// Validates and launches the fused kernel.  `head`: n is set here; argmax_out / sample_out are
// [members, batch].  `who` names the entry point in error texts.
static int fused_launch(const char* who, int n_layers, const int* sizes, int batch, int members, int in_dtype,
                        const void* x, const void* w_compute, const float* params, SbRowHead head, int hidden_norm,
                        float* out, const FusedDecide* decide, void* stream, void* const* acts_out = nullptr,
                        void* const* bits_out = nullptr) {
  if (members < 1 || members > 1024) return sb_fail(SB_ERR_BAD_ARG, "%s: 1..1024 ensemble members", who);
  if (n_layers < 1 || n_layers > FM_MAX_LAYERS) return sb_fail(SB_ERR_UNSUPPORTED, "%s: 1..%d layers", who, FM_MAX_LAYERS);
  if (!sizes) return sb_fail(SB_ERR_BAD_ARG, "%s: sizes is null", who);
  if (in_dtype != SB_F16 && in_dtype != SB_BF16)
    return sb_fail(SB_ERR_UNSUPPORTED, "%s: 16-bit arithmetic classes only (SB_F16, SB_BF16)", who);
  if (batch < 0) return sb_fail(SB_ERR_BAD_ARG, "%s: negative batch", who);
  if (head.flags & ~(SB_EPI_MASKED_SOFTMAX | SB_EPI_REGRET_MATCHING | SB_EPI_ARGMAX | SB_EPI_SAMPLE))
    return sb_fail(SB_ERR_BAD_ARG, "%s: the head may hold softmax, regret matching, arg-max and sampling", who);
  if (sizes[0] < 8 || sizes[0] > 512 || sizes[0] % 8) return sb_fail(SB_ERR_UNSUPPORTED, "%s: input width %d (8..512, multiple of 8)", who, sizes[0]);
  for (int i = 1; i < n_layers; ++i)
    if (sizes[i] < 64 || sizes[i] > 256 || sizes[i] % 64)
      return sb_fail(SB_ERR_UNSUPPORTED, "%s: hidden width %d (64..256, multiple of 64)", who, sizes[i]);
  const int n_out = sizes[n_layers];
  if (head.prefix > n_out) return sb_fail(SB_ERR_BAD_ARG, "%s: prefix %d beyond the %d output columns", who, head.prefix, n_out);
  if (n_out < 1 || !(n_out <= 64 || (n_out <= 256 && head.prefix >= 0 && head.prefix <= 64)))
    return sb_fail(SB_ERR_UNSUPPORTED, "%s: output width %d (1..64, or up to 256 under a prefix mask of at most 64 columns)", who, n_out);
  if (hidden_norm && params) return sb_fail(SB_ERR_UNSUPPORTED, "%s: row-normalised hidden layers take no bias (params must be null)", who);
  if (batch == 0) return SB_OK;
  if (!x || !w_compute || !out) return sb_fail(SB_ERR_BAD_ARG, "%s: null pointer", who);
  if ((head.flags & SB_EPI_ARGMAX) && !head.argmax_out) return sb_fail(SB_ERR_BAD_ARG, "%s: SB_EPI_ARGMAX without an actions buffer", who);
  if ((head.flags & SB_EPI_SAMPLE) && !head.sample_out) return sb_fail(SB_ERR_BAD_ARG, "%s: SB_EPI_SAMPLE without an indices buffer", who);
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w_compute)) & 15)
    return sb_fail(SB_ERR_MISALIGNED, "%s: x and w_compute must be 16-byte aligned", who);

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
  p.out_stride = (long long)batch * n_out;
  int max_n = 32;
  uint32_t max_act_chunks = 1;
  for (int l = 0; l <= n_layers; ++l) p.width[l] = sizes[l];
  for (int l = 0; l < n_layers; ++l) {
    const bool last = l == n_layers - 1;
    p.n_pad[l] = last ? (sizes[l + 1] + 15) / 16 * 16 : sizes[l + 1];
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
  if (acts_out) {
    if (members != 1) return sb_fail(SB_ERR_UNSUPPORTED, "%s: the training forward runs one net", who);
    for (int l = 0; l + 1 < n_layers; ++l) {
      if (!acts_out[l] || (reinterpret_cast<uintptr_t>(acts_out[l]) & 15))
        return sb_fail(SB_ERR_BAD_ARG, "%s: activations[%d] is null or not 16-byte aligned", who, l);
      rc = make_tmap_2d(&maps.act[l], acts_out[l], in_dtype, batch, sizes[l + 1], 128, 64, SWZ_128);
      if (rc != SB_OK) return rc;
      p.bits[l] = (bits_out && bits_out[l]) ? reinterpret_cast<uint32_t*>(bits_out[l]) : nullptr;
    }
    p.store_acts = 1;
  }
  for (int l = acts_out ? (n_layers > 1 ? n_layers - 1 : 0) : 0; l < FM_MAX_LAYERS; ++l) maps.act[l] = maps.w[0];
  rc = make_tmap_2d(&maps.x, x, in_dtype, batch, sizes[0], 128, 64, SWZ_128);
  if (rc != SB_OK) return rc;
  p.x_chunks = (uint32_t)p.k_chunks[0];
  p.act_offset = p.x_chunks * FM_CHUNK_BYTES;
  p.w_offset = p.act_offset + max_act_chunks * FM_CHUNK_BYTES;
  p.acc_stride = 32;
  while (p.acc_stride < max_n) p.acc_stride <<= 1;
  p.tmem_cols = 2 * p.acc_stride;            // two accumulators (at most 2 x 256 columns)
  head.n = n_out;
  p.out = out; p.head = head; p.hidden_norm = hidden_norm ? 1 : 0;
  p.members = members;
  if (decide) {
    p.tile_counters = decide->tile_counters; p.ensemble_id = decide->ensemble_id; p.action = decide->action;
    p.prob_selected = decide->prob_selected; p.prob_ensemble = decide->prob_ensemble;
  }
  p.stage_bytes = ((uint32_t)max_n * 128u + 1023u) / 1024u * 1024u;     // stages stay 1024-byte aligned (swizzle atoms)
  const size_t smem = (size_t)p.w_offset + (size_t)FM_W_STAGES * p.stage_bytes + 1024;

  static std::atomic<bool> attr_set[64];
  int dev = 0;
  SB_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[dev].load(std::memory_order_acquire)) {
    SB_CUDA(cudaFuncSetAttribute(mlp_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 225 * 1024));
    attr_set[dev].store(true, std::memory_order_release);
  }
  if (smem > 225 * 1024)
    return sb_fail(SB_ERR_UNSUPPORTED, "%s: the input tile, the widest hidden tile and the weight ring need %zu bytes of "
                                       "shared memory (inputs wider than 256 fit with hidden layers of at most 128)", who, smem);
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

static SbRowHead fused_head_from_spec(const sb_head_spec* spec) {
  SbRowHead h;
  memset(&h, 0, sizeof(h));
  h.flags = spec->flags; h.prefix = spec->prefix < 0 ? -1 : spec->prefix; h.mask = spec->mask;
  h.argmax_out = spec->argmax_out; h.sample_out = spec->sample_out;
  h.seed = spec->seed; h.row_offset = spec->row_offset; h.position = spec->position;
  return h;
}

extern "C" int sb_mlp_forward_fused_ensemble(int n_layers, const int* sizes, int batch, int members, int in_dtype,
                                             const void* x, const void* w_compute, const float* params, int head,
                                             const uint8_t* mask, float* out, int32_t* actions, void* stream) {
  if (head & ~(SB_EPI_MASKED_SOFTMAX | SB_EPI_REGRET_MATCHING | SB_EPI_ARGMAX))
    return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_forward_fused: head may hold only row-head flags");
  SbRowHead h;
  memset(&h, 0, sizeof(h));
  h.flags = head; h.prefix = -1; h.mask = mask; h.argmax_out = actions;
  return fused_launch("sb_mlp_forward_fused", n_layers, sizes, batch, members, in_dtype, x, w_compute, params, h, 0, out,
                      nullptr, stream);
}

extern "C" int sb_mlp_forward_fused(int n_layers, const int* sizes, int batch, int in_dtype, const void* x,
                                    const void* w_compute, const float* params, int head, const uint8_t* mask,
                                    float* out, int32_t* actions, void* stream) {
  return sb_mlp_forward_fused_ensemble(n_layers, sizes, batch, 1, in_dtype, x, w_compute, params, head, mask, out,
                                       actions, stream);
}

extern "C" int sb_mlp_forward_fused_head(int n_layers, const int* sizes, int batch, int members, int in_dtype,
                                         const void* x, const void* w_compute, const float* params, int hidden_norm,
                                         const sb_head_spec* head, float* out, void* stream) {
  if (!head) return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_forward_fused_head: head is null");
  if (head->flags & SB_EPI_BINARIZE) return sb_fail(SB_ERR_UNSUPPORTED, "sb_mlp_forward_fused_head: no sign hash in the fused kernel");
  return fused_launch("sb_mlp_forward_fused_head", n_layers, sizes, batch, members, in_dtype, x, w_compute, params,
                      fused_head_from_spec(head), hidden_norm, out, nullptr, stream);
}

extern "C" int sb_policy_decide(const sb_decide_args* a, void* stream) {
  if (!a) return sb_fail(SB_ERR_BAD_ARG, "sb_policy_decide: null arguments");
  if (a->rows < 0 || a->rows > 0x7fffffffLL) return sb_fail(SB_ERR_BAD_ARG, "sb_policy_decide: rows out of range");
  if (a->rows == 0) return SB_OK;
  if (!a->sizes || a->n_layers < 1) return sb_fail(SB_ERR_BAD_ARG, "sb_policy_decide: no network");
  if (!a->output_probs || !a->output_indices || !a->ensemble_id || !a->action || !a->sampling_prob_selected ||
      !a->sampling_prob_ensemble || !a->tile_counters || !a->x)
    return sb_fail(SB_ERR_BAD_ARG, "sb_policy_decide: every output buffer, the input workspace x and tile_counters are required");
  if (a->head_flags & ~(SB_EPI_MASKED_SOFTMAX | SB_EPI_REGRET_MATCHING))
    return sb_fail(SB_ERR_BAD_ARG, "sb_policy_decide: head_flags may hold SB_EPI_MASKED_SOFTMAX and SB_EPI_REGRET_MATCHING");
  int rc;
  if (a->fields) {
    int features = a->n_dense;
    for (int j = 0; j < a->n_fields; ++j) features += a->widths ? a->widths[j] : 0;
    if (features != a->sizes[0])
      return sb_fail(SB_ERR_BAD_ARG, "sb_policy_decide: the state layout describes %d features, the net takes %d", features, a->sizes[0]);
    rc = sb_encode_states(a->fields, a->n_fields, a->widths, a->dense, a->n_dense, a->x, a->rows, a->in_dtype, stream);
    if (rc != SB_OK) return rc;
  }
  SbRowHead h;
  memset(&h, 0, sizeof(h));
  h.flags = a->head_flags | SB_EPI_SAMPLE;
  h.prefix = a->prefix < 0 ? -1 : a->prefix;
  h.mask = a->mask;
  h.sample_out = a->output_indices;
  h.seed = a->seed; h.row_offset = a->row_offset; h.position = 0;
  FusedDecide d;
  d.tile_counters = a->tile_counters; d.ensemble_id = a->ensemble_id; d.action = a->action;
  d.prob_selected = a->sampling_prob_selected; d.prob_ensemble = a->sampling_prob_ensemble;
  return fused_launch("sb_policy_decide", a->n_layers, a->sizes, (int)a->rows, a->members, a->in_dtype, a->x, a->w_compute,
                      a->params, h, a->hidden_norm, a->output_probs, &d, stream);
}

// True when the fused kernel can run this net (the checks of fused_launch that depend on the shape only).
static bool fused_shape_ok(int n_layers, const int* sizes, int in_dtype) {
  if (n_layers < 1 || n_layers > FM_MAX_LAYERS || !sizes) return false;
  if (in_dtype != SB_F16 && in_dtype != SB_BF16) return false;
  if (sizes[0] < 8 || sizes[0] > 512 || sizes[0] % 8) return false;
  uint32_t max_act_chunks = 1;
  int max_n = 32;
  for (int i = 1; i < n_layers; ++i) {
    if (sizes[i] < 64 || sizes[i] > 256 || sizes[i] % 64) return false;
    if ((uint32_t)(sizes[i] / 64) > max_act_chunks) max_act_chunks = (uint32_t)(sizes[i] / 64);
    if (sizes[i] > max_n) max_n = sizes[i];
  }
  const int n_out = sizes[n_layers];
  if (n_out < 1 || n_out > 64) return false;
  if ((n_out + 15) / 16 * 16 > max_n) max_n = (n_out + 15) / 16 * 16;
  const size_t stage = ((size_t)max_n * 128 + 1023) / 1024 * 1024;
  const size_t smem = (size_t)((sizes[0] + 63) / 64 + max_act_chunks) * FM_CHUNK_BYTES + FM_W_STAGES * stage + 1024;
  return smem <= 225 * 1024;
}

extern "C" int sb_mlp_fused_supported(int n_layers, const int* sizes, int in_dtype) {
  return fused_shape_ok(n_layers, sizes, in_dtype) ? 1 : 0;
}

extern "C" int sb_mlp_forward_fused_train(int n_layers, const int* sizes, int batch, int in_dtype, const void* x,
                                          const void* w_compute, const float* params, void* const* activations,
                                          void* const* relu_bits, int head, const uint8_t* mask, float* out,
                                          int32_t* actions, void* stream) {
  if (head & ~(SB_EPI_MASKED_SOFTMAX | SB_EPI_REGRET_MATCHING | SB_EPI_ARGMAX))
    return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_forward_fused_train: head may hold only row-head flags");
  if (n_layers > 1 && !activations) return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_forward_fused_train: activations is null");
  for (int l = 0; l + 1 < n_layers; ++l)
    if (relu_bits && relu_bits[l] && sizes && sizes[l + 1] % 32 != 0)
      return sb_fail(SB_ERR_UNSUPPORTED, "sb_mlp_forward_fused_train: sign words need widths that are multiples of 32");
  SbRowHead h;
  memset(&h, 0, sizeof(h));
  h.flags = head; h.prefix = -1; h.mask = mask; h.argmax_out = actions;
  static void* const no_acts[1] = {nullptr};
  return fused_launch("sb_mlp_forward_fused_train", n_layers, sizes, batch, 1, in_dtype, x, w_compute, params, h, 0, out,
                      nullptr, stream, n_layers > 1 ? activations : no_acts, relu_bits);
}
