// Dense policy-network path: forward chain, backward (cross-entropy on a masked
// softmax head), split-K weight gradients and the fused SGD update.
//
// Forward replaces the per-node device functions the reference's graph
// interpreter emits (BlockMatmul -> BlockMap relu -> BlockRowMap head,
// ml/layers.spi:181-252, one global-memory pass per node): here every layer is
// one tensor-core GEMM whose epilogue applies bias, ReLU, the storage rounding
// of the next layer's input and, on the last layer, the row head.
//
// The reference has no backward pass, loss or optimiser (its training is CEM /
// tabular CFR, ml/cem.spi:99-146); dgrad (NN), wgrad (TN) and SGD below follow
// the benchmark's training configurations and are pinned by the NumPy oracle.
//
// Memory model (caller-owned, as in ml/layers.spi:127-172): a flat fp32 master
// parameter buffer [W0 | b0 | W1 | b1 | ...] with 64-element aligned segments,
// a compute copy of the same layout in the storage type of the arithmetic class,
// a flat fp32 gradient buffer of the same layout (the unit of the data-parallel
// all-reduce), per-layer activation buffers and one scratch buffer.
#include "common.cuh"


namespace {

constexpr int MLP_MAX_LAYERS = 16;
constexpr long long SEG_ALIGN = 64;  // elements; 256 B in fp32, 128 B in 16-bit storage

long long align_up(long long x, long long a) { return (x + a - 1) / a * a; }

int storage_dtype(int in_dtype) { return in_dtype == SB_TF32 ? SB_TF32 : in_dtype; }

int check_layout(const char* who, int n_layers, const int* sizes, int batch, int in_dtype) {
  if (n_layers < 1 || n_layers > MLP_MAX_LAYERS) return sb_fail(SB_ERR_BAD_ARG, "%s: n_layers must be in [1, %d]", who, MLP_MAX_LAYERS);
  if (!sizes) return sb_fail(SB_ERR_BAD_ARG, "%s: sizes is null", who);
  for (int i = 0; i <= n_layers; ++i)
    if (sizes[i] < 1) return sb_fail(SB_ERR_BAD_ARG, "%s: sizes[%d] = %d", who, i, sizes[i]);
  if (batch < 0) return sb_fail(SB_ERR_BAD_ARG, "%s: negative batch", who);
  if (in_dtype != SB_TF32 && in_dtype != SB_BF16 && in_dtype != SB_F16)
    return sb_fail(SB_ERR_UNSUPPORTED, "%s: arithmetic class must be SB_TF32, SB_BF16 or SB_F16", who);
  return SB_OK;
}

// Rows of a weight segment: the fan-out padded to a multiple of 8 so that the
// transposed uses of dY (wgrad A operand, dgrad inner dimension) have 16-byte
// row pitches.  Padding rows stay zero: their gradients are zero.
int padded_out(int fan_out) { return (fan_out + 7) / 8 * 8; }

void param_offsets(int n_layers, const int* sizes, long long* off) {
  long long cur = 0;
  for (int i = 0; i < n_layers; ++i) {
    off[2 * i] = cur;
    cur = align_up(cur + (long long)padded_out(sizes[i + 1]) * sizes[i], SEG_ALIGN);
    off[2 * i + 1] = cur;
    cur = align_up(cur + sizes[i + 1], SEG_ALIGN);
  }
  off[2 * n_layers] = cur;
}

// d logits of cross-entropy(masked softmax): (p * sum(t) - t) / global_batch on
// legal entries, 0 elsewhere; also accumulates the loss.  One thread per row.
// LD > 0: the padded row width is the compile-time LD and the column sums of
// d logits -- the head layer's bias gradient -- are added to db here (a CTA-wide
// reduction, then LD atomics per CTA) instead of in a pass of their own over dY.
template <typename DyT, bool ROUND_TF32, int LD>
__global__ void ce_grad_kernel(const float* __restrict__ probs, const float* __restrict__ target,
                               const uint8_t* __restrict__ mask, DyT* __restrict__ dy, int rows, int n,
                               int ld, float inv_batch, float* __restrict__ loss, float* __restrict__ db) {
  constexpr int NACC = LD > 0 ? LD : 1;
  __shared__ float colpart[8][NACC];
  sb_grid_dependency_wait();
  sb_grid_dependents_launch();
  float local = 0.f;
  float colacc[NACC];
#pragma unroll
  for (int j = 0; j < NACC; ++j) colacc[j] = 0.f;
  for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < rows;
       r += (long long)gridDim.x * blockDim.x) {
    const float* pr = probs + r * n;
    const float* tr = target + r * n;
    const uint8_t* mr = mask ? mask + r * n : nullptr;
    if (LD > 0 && sizeof(DyT) == 2) {
      // The whole row in registers first (an even row length keeps every row 8-byte aligned:
      // probabilities and targets then come as two-float loads); then one or two 16-byte stores of
      // the padded 16-bit row instead of LD two-byte ones 2 * LD bytes apart.
      float pv[NACC], tv[NACC];
      if ((n & 1) == 0) {
#pragma unroll
        for (int j = 0; j < NACC; j += 2) {
          float2 a = make_float2(0.f, 0.f), b = a;
          if (j < n) {
            a = __ldg(reinterpret_cast<const float2*>(pr + j));
            b = __ldg(reinterpret_cast<const float2*>(tr + j));
          }
          pv[j] = a.x; pv[j + 1] = a.y;
          tv[j] = b.x; tv[j + 1] = b.y;
        }
      } else {
#pragma unroll
        for (int j = 0; j < NACC; ++j) {
          pv[j] = j < n ? __ldg(pr + j) : 0.f;
          tv[j] = j < n ? __ldg(tr + j) : 0.f;
        }
      }
      bool legal[NACC];
      float ts = 0.f;
#pragma unroll
      for (int j = 0; j < NACC; ++j) {
        legal[j] = j < n && (!mr || mr[j]);
        if (legal[j]) ts += tv[j];
      }
      __align__(16) DyT packed[NACC];
#pragma unroll
      for (int j = 0; j < NACC; ++j) {
        float g = 0.f;
        if (legal[j]) {
          g = (pv[j] * ts - tv[j]) * inv_batch;
          local -= tv[j] * __logf(fmaxf(pv[j], 1e-38f));
        }
        colacc[j] += g;
        packed[j] = (DyT)g;
      }
      uint4* dst = reinterpret_cast<uint4*>(dy + r * ld);
#pragma unroll
      for (int q = 0; q < NACC / 8; ++q) dst[q] = reinterpret_cast<const uint4*>(packed)[q];
      continue;
    }
    float tsum = 0.f;
    for (int j = 0; j < n; ++j)
      if (!mr || mr[j]) tsum += tr[j];
    auto one = [&](int j) {
      const bool lg = j < n && (!mr || mr[j]);
      float g = 0.f;
      if (lg) {
        const float pj = pr[j], tj = tr[j];
        g = (pj * tsum - tj) * inv_batch;
        local -= tj * __logf(fmaxf(pj, 1e-38f));
      }
      if (ROUND_TF32) {
        uint32_t u = __float_as_uint(g);
        u += 0x0fffu + ((u >> 13) & 1u);
        g = __uint_as_float(u & 0xffffe000u);
      }
      if (sizeof(DyT) == 4) reinterpret_cast<float*>(dy)[r * ld + j] = g;
      else if (sizeof(DyT) == 2) dy[r * ld + j] = (DyT)g;
      return g;
    };
    if (LD > 0) {
#pragma unroll
      for (int j = 0; j < NACC; ++j) colacc[j] += one(j);
    } else {
      for (int j = 0; j < ld; ++j) one(j);
    }
  }
  if (loss) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
    if ((threadIdx.x & 31) == 0 && local != 0.f) atomicAdd(loss, local * inv_batch);
  }
  if (LD > 0 && db) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int j = 0; j < NACC; ++j) {
      float v = colacc[j];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) colpart[warp][j] = v;
    }
    __syncthreads();
    if (threadIdx.x < NACC && (int)threadIdx.x < n) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) t += colpart[w][threadIdx.x];
      if (t != 0.f) atomicAdd(db + threadIdx.x, t);
    }
  }
}

// Column sums of dY [rows, n] -> db[n] (bias gradient).  A block owns a slab of
// rows and a strip of 32 * VEC columns; each thread reads 16-byte pieces (VEC
// elements) so that a warp covers 512 contiguous bytes of a row, the 8 warps
// take alternate rows, and the block's partial sums are combined with atomics
// into a zeroed output (fp32, run-dependent order over a few hundred terms).
template <typename DyT>
__global__ void __launch_bounds__(256)
colsum_kernel(const DyT* __restrict__ dy, float* __restrict__ db, int rows, int n, int rows_per_block) {
  constexpr int VEC = 16 / sizeof(DyT);
  __shared__ float part[8][32 * VEC + 1];
  sb_grid_dependency_wait();
  sb_grid_dependents_launch();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col0 = (blockIdx.x * 32 + lane) * VEC;
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(rows, r0 + rows_per_block);
  float s[VEC];
#pragma unroll
  for (int t = 0; t < VEC; ++t) s[t] = 0.f;
  const bool vec_ok = (n % VEC == 0) && ((reinterpret_cast<uintptr_t>(dy) & 15) == 0) && col0 + VEC <= n;
  if (vec_ok) {
    for (int r = r0 + warp; r < r1; r += 8) {
      const uint4 raw = *reinterpret_cast<const uint4*>(dy + (long long)r * n + col0);
      const DyT* e = reinterpret_cast<const DyT*>(&raw);
#pragma unroll
      for (int t = 0; t < VEC; ++t) s[t] += (float)e[t];
    }
  } else {
    for (int r = r0 + warp; r < r1; r += 8)
#pragma unroll
      for (int t = 0; t < VEC; ++t)
        if (col0 + t < n) s[t] += (float)dy[(long long)r * n + col0 + t];
  }
#pragma unroll
  for (int t = 0; t < VEC; ++t) part[warp][lane * VEC + t] = s[t];
  __syncthreads();
  for (int j = threadIdx.x; j < 32 * VEC; j += 256) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += part[w][j];
    const int col = blockIdx.x * 32 * VEC + j;
    if (col < n && t != 0.f) atomicAdd(db + col, t);
  }
}

// dgrad of a layer with at most 16 outputs (the head): dX[r, n] = gate(r, n) * sum_k dY[r, k] * W[k, n],
// k < KV.  With so short an inner dimension the tensor-core kernel is all epilogue (it drains a
// 128 x 256 accumulator in 4.4 us whatever K is); here a thread keeps its 8 columns of W in
// registers, 8 * KV fused multiply-adds make one 16-byte store, rows are taken eight at a time so
// that the sign words of a column block (stored [N / 32, rows]) come as two 16-byte loads, and the
// output leaves in whole rows.  Column sums of the output (the bias gradient of the layer below) are
// kept per thread over all its rows and added once per block and column.  (A form of this kernel
// with the multiply-adds on warp-level MMAs, m16n8k16, was built and measured: 4 us faster at
// 32768 x 1024 with 10 outputs, 28 us slower for a 3-output head -- gating, packing, column sums
// and stores cost the same either way and the MMA does 16 multiply-adds whatever K is.)
// Two fp32 fused multiply-adds in one instruction (the packed form sm_100 adds): c += a * b on register pairs.
__device__ __forceinline__ unsigned long long pack_f32x2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ void fma_f32x2(unsigned long long& c, unsigned long long a, unsigned long long b) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(c) : "l"(a), "l"(b));
}

constexpr int ND_THREADS = 384;
constexpr int ND_MAX_SLOTS = ND_THREADS / 32;
template <typename T, int KV>
__global__ void __launch_bounds__(ND_THREADS, 1)
narrow_dgrad_kernel(const T* __restrict__ dy, int ldy, const T* __restrict__ w, int n, const uint32_t* __restrict__ bits,
                    T* __restrict__ dx, float* __restrict__ colsum, int rows) {
  __shared__ float sums[1024];
  // The dY rows of the next eight rows of every slot arrive here (cp.async) while this eight are computed.
  __shared__ __align__(16) uint4 dy_s[2][ND_MAX_SLOTS][8][2];
  sb_grid_dependency_wait();
  sb_grid_dependents_launch();
  const int groups = n >> 3;                                    // 16-byte column groups of a row
  const int tpr = groups < 128 ? ((groups + 31) & ~31) : 128;   // threads per row slot: whole warps
  const int slots = ND_THREADS / tpr;                           // row slots of a block (3 when n >= 1024)
  const int slot = (int)threadIdx.x / tpr, t = (int)threadIdx.x % tpr;
  const long long stride = (long long)gridDim.x * slots * 8;
  const int iters = (int)((rows + stride - 1) / stride);        // the same for every thread: the loop holds barriers
  const int halves = ldy >= 16 ? 2 : 1;                         // 16-byte pieces of a dY row that are read
  for (int cg0 = 0; cg0 < groups; cg0 += 128) {                 // n > 1024: one pass per 1024 columns
    const int cg = cg0 + t;
    const bool live = cg < groups && slot < slots;
    unsigned long long wr[KV][4];            // the thread's 8 columns of W as four fp32 pairs per k
#pragma unroll
    for (int k = 0; k < KV; ++k) {
      uint4 raw = make_uint4(0u, 0u, 0u, 0u);
      if (live) raw = *reinterpret_cast<const uint4*>(w + (long long)k * n + cg * 8);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) wr[k][j] = pack_f32x2((float)e[2 * j], (float)e[2 * j + 1]);
    }
    float cs[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) cs[j] = 0.f;
    const int shift = (cg & 3) * 8;                // this thread's 8 bits inside its 32-column sign word
    const long long first = ((long long)blockIdx.x * slots + slot) * 8;

    // Thread t < 16 of a slot fetches piece (t & 1) of row (t >> 1) of the slot's eight rows.
    auto fetch_dy = [&](int it) {
      if (slot < slots && t < 16) {
        const long long r = first + (long long)it * stride + (t >> 1);
        if (r < rows && (t & 1) < halves)
          cp_async_16(smem_u32(&dy_s[it & 1][slot][t >> 1][t & 1]), dy + r * ldy + (t & 1) * 8);
      }
      cp_async_commit();
    };
    auto fetch_gate = [&](int it, uint32_t* gate) {
      const long long r0 = first + (long long)it * stride;
      if (!live || r0 >= rows) return;
      if (bits) {
        const uint32_t* g = bits + (long long)(cg >> 2) * rows + r0;
        if (r0 + 8 <= rows && ((reinterpret_cast<uintptr_t>(g) & 15) == 0)) {
          const uint4 a = __ldg(reinterpret_cast<const uint4*>(g)), b = __ldg(reinterpret_cast<const uint4*>(g) + 1);
          gate[0] = a.x; gate[1] = a.y; gate[2] = a.z; gate[3] = a.w;
          gate[4] = b.x; gate[5] = b.y; gate[6] = b.z; gate[7] = b.w;
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) gate[i] = r0 + i < rows ? __ldg(g + i) : 0u;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) gate[i] = 0xffffffffu;
      }
    };

    uint32_t gate[8], gate_next[8];
    fetch_dy(0);
    fetch_gate(0, gate);
    for (int it = 0; it < iters; ++it) {
      cp_async_wait_all();
      __syncthreads();                       // this iteration's dY rows are in; the other buffer is free
      if (it + 1 < iters) {
        fetch_dy(it + 1);
        fetch_gate(it + 1, gate_next);
      }
      const long long r0 = first + (long long)it * stride;
      if (live && r0 < rows) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const long long r = r0 + i;
          if (r < rows) {
            float d[KV];
#pragma unroll
            for (int k8 = 0; k8 < KV; k8 += 8) {
              const uint4 raw = dy_s[it & 1][slot][i][k8 >> 3];      // the same address for the whole warp
              const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (k8 + j < KV) d[k8 + j] = (float)e[j];
            }
            unsigned long long acc2[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
            for (int k = 0; k < KV; ++k) {
              const unsigned long long dd = pack_f32x2(d[k], d[k]);
#pragma unroll
              for (int j = 0; j < 4; ++j) fma_f32x2(acc2[j], dd, wr[k][j]);
            }
            float acc[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) unpack_f32x2(acc2[j], acc[2 * j], acc[2 * j + 1]);
            const uint32_t gb = gate[i] >> shift;
            uint4 out;
            T* o = reinterpret_cast<T*>(&out);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float v = ((gb >> j) & 1u) ? acc[j] : 0.f;
              cs[j] += v;
              o[j] = (T)v;
            }
            *reinterpret_cast<uint4*>(dx + r * n + cg * 8) = out;
          }
        }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) gate[i] = gate_next[i];
    }
    __syncthreads();
    if (colsum) {
      // One addition per block and column: the row slots fold in shared memory first.
      for (int c = (int)threadIdx.x; c < tpr * 8; c += ND_THREADS) sums[c] = 0.f;
      __syncthreads();
      if (live) {
#pragma unroll
        for (int j = 0; j < 8; ++j) atomicAdd(&sums[t * 8 + j], cs[j]);
      }
      __syncthreads();
      for (int c = (int)threadIdx.x; c < tpr * 8; c += ND_THREADS) {
        const int col = cg0 * 8 + c;
        const float v = sums[c];
        if (col < n && v != 0.f) atomicAdd(colsum + col, v);
      }
      __syncthreads();
    }
  }
}

// Whether the narrow dgrad kernel serves a layer: a 16-bit storage type, at most 16 (real) outputs,
// rows of whole 16-byte groups.
bool narrow_dgrad_ok(int fan_out_real, int fan_in, int in_dtype) {
  static int off = -1;
  if (off < 0) {
    const char* e = getenv("SB_NARROW_DGRAD");          // SB_NARROW_DGRAD=0: the tensor-core kernel for every layer
    off = (e && e[0] == '0') ? 1 : 0;
  }
  return !off && (in_dtype == SB_BF16 || in_dtype == SB_F16) && fan_out_real >= 1 && fan_out_real <= 16 && fan_in % 8 == 0;
}

template <typename T>
int narrow_dgrad_launch(const void* dy, int ldy, const void* w, int fan_out_real, int n, const uint32_t* bits, void* dx,
                        float* colsum, int rows, cudaStream_t s) {
  const int groups = n / 8;
  const int tpr = groups < 128 ? ((groups + 31) & ~31) : 128;
  const int slots = ND_THREADS / tpr;
  long long want = ((long long)rows + slots * 8 - 1) / (slots * 8);
  const int grid = (int)(want < sb_sm_count() ? (want < 1 ? 1 : want) : sb_sm_count());
  const T* dyp = reinterpret_cast<const T*>(dy);
  const T* wp = reinterpret_cast<const T*>(w);
  T* dxp = reinterpret_cast<T*>(dx);
#define SB_ND(KV) SB_CUDA(sb_launch(narrow_dgrad_kernel<T, KV>, dim3(grid), dim3(ND_THREADS), 0, s, 1, dyp, ldy, wp, n, bits, dxp, colsum, rows))
  if (fan_out_real <= 4) SB_ND(4);
  else if (fan_out_real <= 8) SB_ND(8);
  else if (fan_out_real <= 10) SB_ND(10);
  else if (fan_out_real <= 12) SB_ND(12);
  else SB_ND(16);
#undef SB_ND
  SB_COUNT_LAUNCH();
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

// grads[i] = sum over splits of partial[s][i]; deterministic order.
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                     long long n, int splits) {
  sb_grid_dependency_wait();
  sb_grid_dependents_launch();
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
    float s = 0.f;
    for (int k = 0; k < splits; ++k) s += partial[(long long)k * n + i];
    out[i] = s;
  }
}

// params -= lr * grads ; compute copy = params rounded to the storage type.
__global__ void sgd_kernel(float* __restrict__ params, const float* __restrict__ grads,
                           void* __restrict__ compute, long long n, float lr, int dt) {
  sb_grid_dependency_wait();
  sb_grid_dependents_launch();
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
    const float w = params[i] - lr * grads[i];
    params[i] = w;
    if (!compute) continue;
    if (dt == SB_BF16) reinterpret_cast<__nv_bfloat16*>(compute)[i] = __float2bfloat16_rn(w);
    else if (dt == SB_F16) reinterpret_cast<__half*>(compute)[i] = __float2half_rn(w);
    else if (dt == SB_TF32) {
      uint32_t u = __float_as_uint(w);
      if ((u & 0x7f800000u) != 0x7f800000u) { u += 0x0fffu + ((u >> 13) & 1u); u &= 0xffffe000u; }
      reinterpret_cast<float*>(compute)[i] = __uint_as_float(u);
    } else reinterpret_cast<float*>(compute)[i] = w;
  }
}

int blocks_for(long long n, int per_block, int cap = 0) {
  if (cap <= 0) cap = sb_sm_count() * 8;
  long long b = (n + per_block - 1) / per_block;
  if (b < 1) b = 1;
  return (int)(b > cap ? cap : b);
}

// Split factor of a wgrad GEMM [out, in] with inner dimension = batch.  A GEMM with more than
// 128 output rows runs on CTA pairs (256 x 256 tiles, 74 pairs).  Model of its time, in k-blocks:
// (waves of work items over the pairs) x (k-blocks per item + a fixed part per item for pipeline
// fill and the tile's reduce-add).  For a 1024 x 1024 layer at a batch of 262144 that picks 9 splits
// (144 items, two full waves) instead of 4 (64 items on 74 pairs, 14 % of the GPU idle), at 32768
// rows still 4; a 256 x 256 layer (one tile) is cut into as many items as there are pairs, which
// measured 23 us against 37 us with 11.  Narrow outputs run on single CTAs, one item each.
int wgrad_splits(int out, int in, int batch, int in_dtype) {
  static int forced = -1;                  // SB_WGRAD_SPLITS=n in the environment fixes the factor (tuning runs)
  if (forced < 0) {
    const char* e = getenv("SB_WGRAD_SPLITS");
    forced = e ? atoi(e) : 0;
    if (forced < 0 || forced > 128) forced = 0;
  }
  const int es = sb_dtype_size(in_dtype);
  const int block_k = 128 / es;
  const int k_blocks = (batch + block_k - 1) / block_k;
  const int max_by_k = k_blocks / 8 > 0 ? k_blocks / 8 : 1;  // keep >= 8 k-blocks per split
  if (forced > 0) return forced < max_by_k ? forced : max_by_k;
  if (out > 128) {
    const int tiles = ((out + 255) / 256) * ((in + 255) / 256);
    const int workers = sb_sm_count() / 2;
    // The fixed part of an item, in k-blocks (about 6 us against 0.55 us per k-block of a pair tile).
    const int item_fixed = 10;
    int best = 1;
    long long best_cost = -1;
    for (int s = 1; s <= 128 && s <= max_by_k; ++s) {
      const long long waves = ((long long)tiles * s + workers - 1) / workers;
      const long long cost = waves * ((k_blocks + s - 1) / s + item_fixed);
      if (best_cost < 0 || cost < best_cost) {
        best_cost = cost;
        best = s;
      }
    }
    return best;
  }
  const int tiles = ((out + 127) / 128) * ((in + 255) / 256);
  int s = sb_sm_count() / (tiles > 0 ? tiles : 1);
  if (s < 1) s = 1;
  if (s > max_by_k) s = max_by_k;
  if (s > 128) s = 128;
  return s;
}

bool wgrad_partials_forced() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("SB_WGRAD_PARTIALS");
    v = (e && e[0] == '1') ? 1 : 0;
  }
  return v == 1;
}

size_t backward_scratch_bytes(int n_layers, const int* sizes, int batch, int in_dtype) {
  const int es = sb_dtype_size(in_dtype);
  int max_w = 0;
  long long max_partial = 0;
  for (int i = 0; i < n_layers; ++i) {
    const int op = padded_out(sizes[i + 1]);
    if (op > max_w) max_w = op;
    const long long p = (long long)wgrad_splits(op, sizes[i], batch, in_dtype) * op * sizes[i];
    if (p > max_partial) max_partial = p;
  }
  const size_t dy = (size_t)align_up((long long)batch * max_w * es, 256);
  return 2 * dy + (size_t)max_partial * 4 + 256;
}

}  // namespace

extern "C" {

int sb_mlp_param_offsets(int n_layers, const int* sizes, long long* offsets) {
  if (!offsets) return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_param_offsets: null output");
  int rc = check_layout("sb_mlp_param_offsets", n_layers, sizes, 0, SB_BF16);
  if (rc != SB_OK) return rc;
  param_offsets(n_layers, sizes, offsets);
  return SB_OK;
}

int sb_mlp_forward(int n_layers, const int* sizes, int batch, int in_dtype, const void* x,
                   const void* w_compute, const float* params, void* const* activations,
                   void* const* relu_bits, int head, const uint8_t* mask, float* out, int32_t* actions,
                   void* stream) {
  int rc = check_layout("sb_mlp_forward", n_layers, sizes, batch, in_dtype);
  if (rc != SB_OK) return rc;
  if (batch == 0) return SB_OK;
  if (!x || !w_compute || !out) return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_forward: null pointer");
  if (n_layers > 1 && !activations) return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_forward: activations is null");
  if (head & ~(SB_EPI_MASKED_SOFTMAX | SB_EPI_REGRET_MATCHING | SB_EPI_ARGMAX))
    return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_forward: head may hold only row-head flags");
  if ((head & SB_EPI_ARGMAX) && !actions) return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_forward: SB_EPI_ARGMAX without an actions buffer");
  long long off[2 * MLP_MAX_LAYERS + 1];
  param_offsets(n_layers, sizes, off);
  const int es = sb_dtype_size(in_dtype);
  const int st = storage_dtype(in_dtype);
  const void* h = x;
  for (int i = 0; i < n_layers; ++i) {
    const bool last = i == n_layers - 1;
    const void* w = reinterpret_cast<const char*>(w_compute) + off[2 * i] * es;
    const float* b = params ? params + off[2 * i + 1] : nullptr;
    int epi = b ? SB_EPI_BIAS : 0;
    void* dst;
    int odt;
    if (last) {
      epi |= head;
      dst = out;
      odt = SB_F32;
    } else {
      if (!activations[i]) return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_forward: activations[%d] is null", i);
      epi |= SB_EPI_RELU;
      dst = activations[i];
      odt = st;
      if (relu_bits && relu_bits[i] && sizes[i + 1] % 32 == 0) epi |= SB_EPI_RELU_MASK_OUT;
    }
    void* aux_out = last ? (void*)actions : ((epi & SB_EPI_RELU_MASK_OUT) ? relu_bits[i] : nullptr);
    rc = sb_matmul_ex(0, 1, 1.0f, h, w, 0.0f, dst, batch, sizes[i + 1], sizes[i], in_dtype, odt, epi, b,
                      last ? mask : nullptr, nullptr, aux_out, stream);
    if (rc != SB_OK) return rc;
    h = dst;
  }
  return SB_OK;
}

// ---------------------------------------------------------------------------
// Forward pass for hosts that cannot allocate device memory.
//
// Some callers of this library have no way to obtain the hidden-activation
// workspace that sb_mlp_forward wants: a per-decision game loop that only
// holds the reference's three arenas, a plugin running inside someone else's
// CUDA context with allocation forbidden, or code between cudaStreamBeginCapture
// and EndCapture, where cudaMalloc is illegal.  For them the hidden activations
// live in the fixed array below, which is part of the library image: every GPU
// that loads the library holds these SB_STATIC_WORKSPACE_BYTES until the
// process exits.
//
// In host code the name `g_static_workspace` is only a host-side stand-in for
// the symbol, not a device address; the real address is looked up once per
// device with cudaGetSymbolAddress and that pointer is what the kernels get.
// ---------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_static_workspace[SB_STATIC_WORKSPACE_BYTES];

namespace {
unsigned char* g_static_workspace_addr[64] = {nullptr};

// Device address of the static workspace on the current device (looked up on
// the first call per device, with that device current).
int static_workspace_address(unsigned char** out) {
  int dev = 0;
  SB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return sb_fail(SB_ERR_UNSUPPORTED, "sb_mlp_forward_static: device index %d out of range", dev);
  if (!g_static_workspace_addr[dev]) {
    void* p = nullptr;
    SB_CUDA(cudaGetSymbolAddress(&p, g_static_workspace));
    if (!p) return sb_fail(SB_ERR_CUDA, "sb_mlp_forward_static: cudaGetSymbolAddress returned a null address");
    g_static_workspace_addr[dev] = reinterpret_cast<unsigned char*>(p);
  }
  *out = g_static_workspace_addr[dev];
  return SB_OK;
}
}  // namespace

int sb_mlp_forward_static(int n_layers, const int* sizes, int batch, int in_dtype, const void* x,
                          const void* w_compute, const float* params, int head, const uint8_t* mask,
                          float* out, int32_t* actions, void* stream) {
  int rc = check_layout("sb_mlp_forward_static", n_layers, sizes, batch, in_dtype);
  if (rc != SB_OK) return rc;
  // Carve one 256-byte aligned slab per hidden layer out of the fixed array.
  const int es = sb_dtype_size(in_dtype);
  void* acts[MLP_MAX_LAYERS];
  size_t offset = 0;
  size_t offsets[MLP_MAX_LAYERS];
  for (int i = 0; i + 1 < n_layers; ++i) {
    offsets[i] = offset;
    offset += (size_t)align_up((long long)batch * sizes[i + 1] * es, 256);
  }
  if (offset > (size_t)SB_STATIC_WORKSPACE_BYTES)
    return sb_fail(SB_ERR_TOO_LARGE,
                   "sb_mlp_forward_static: hidden activations need %zu bytes, the built-in workspace holds %zu; "
                   "use sb_mlp_forward with caller memory for this batch", offset, (size_t)SB_STATIC_WORKSPACE_BYTES);
  unsigned char* base = nullptr;
  rc = static_workspace_address(&base);
  if (rc != SB_OK) return rc;
  for (int i = 0; i + 1 < n_layers; ++i) acts[i] = base + offsets[i];
  // Every slab is completely overwritten by its layer before the next layer
  // reads it, so nothing left behind by an earlier call needs clearing.
  return sb_mlp_forward(n_layers, sizes, batch, in_dtype, x, w_compute, params, n_layers > 1 ? acts : nullptr,
                        nullptr, head, mask, out, actions, stream);
}

int sb_mlp_backward_scratch_bytes(int n_layers, const int* sizes, int batch, int in_dtype, size_t* bytes) {
  if (!bytes) return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_backward_scratch_bytes: null output");
  int rc = check_layout("sb_mlp_backward_scratch_bytes", n_layers, sizes, batch, in_dtype);
  if (rc != SB_OK) return rc;
  *bytes = backward_scratch_bytes(n_layers, sizes, batch, in_dtype);
  return SB_OK;
}

int sb_mlp_backward_dy_offset(int n_layers, const int* sizes, int batch, int in_dtype, int layer, size_t* offset) {
  if (!offset) return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_backward_dy_offset: null output");
  int rc = check_layout("sb_mlp_backward_dy_offset", n_layers, sizes, batch, in_dtype);
  if (rc != SB_OK) return rc;
  if (layer < 0 || layer >= n_layers) return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_backward_dy_offset: layer %d of %d", layer, n_layers);
  int max_w = 0;
  for (int i = 0; i < n_layers; ++i) max_w = max(max_w, padded_out(sizes[i + 1]));
  const size_t dy_bytes = (size_t)align_up((long long)batch * max_w * sb_dtype_size(in_dtype), 256);
  *offset = ((n_layers - 1 - layer) & 1) ? dy_bytes : 0;
  return SB_OK;
}

// Which layers' weight gradients a data-parallel backward pass adds straight into the owners' copies.
static bool layer_grads_go_to_peers(int fan_out_padded, int fan_in, int world) {
  return world > 1 && sb_umma_peer_out_ok(fan_out_padded, fan_in, world);
}

int sb_mlp_dp_fused_layers(int n_layers, const int* sizes, int world_size, int* fused) {
  if (!fused) return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_dp_fused_layers: null output");
  int rc = check_layout("sb_mlp_dp_fused_layers", n_layers, sizes, 0, SB_BF16);
  if (rc != SB_OK) return rc;
  for (int i = 0; i < n_layers; ++i) fused[i] = layer_grads_go_to_peers(padded_out(sizes[i + 1]), sizes[i], world_size) ? 1 : 0;
  return SB_OK;
}

static int backward_impl(int n_layers, const int* sizes, int batch, float inv_global_batch, int in_dtype,
                         const void* x, const void* w_compute, void* const* activations,
                         void* const* relu_bits, const float* probs, const uint8_t* mask,
                         const float* target, float* grads, int with_bias, void* scratch,
                         size_t scratch_bytes, float* loss, int first_layer, int last_layer, void* stream,
                         float* const* grads_peers, int world);

int sb_mlp_backward_range(int n_layers, const int* sizes, int batch, float inv_global_batch, int in_dtype,
                          const void* x, const void* w_compute, void* const* activations,
                          void* const* relu_bits, const float* probs, const uint8_t* mask,
                          const float* target, float* grads, int with_bias, void* scratch,
                          size_t scratch_bytes, float* loss, int first_layer, int last_layer, void* stream) {
  return backward_impl(n_layers, sizes, batch, inv_global_batch, in_dtype, x, w_compute, activations, relu_bits, probs,
                       mask, target, grads, with_bias, scratch, scratch_bytes, loss, first_layer, last_layer, stream,
                       nullptr, 1);
}

int sb_mlp_backward_dp(int n_layers, const int* sizes, int batch, float inv_global_batch, int in_dtype,
                       const void* x, const void* w_compute, void* const* activations,
                       void* const* relu_bits, const float* probs, const uint8_t* mask, const float* target,
                       float* const* grads_peers, int world_size, int rank, int with_bias, void* scratch,
                       size_t scratch_bytes, float* loss, void* stream) {
  if (world_size < 1 || world_size > 16 || rank < 0 || rank >= world_size || !grads_peers)
    return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_backward_dp: rank %d of world size %d, or no table of gradient buffers", rank, world_size);
  for (int r = 0; r < world_size; ++r)
    if (!grads_peers[r]) return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_backward_dp: gradient buffer of rank %d is null", r);
  // This rank's own buffer comes first in the peers table handed down: the launcher's C.
  return backward_impl(n_layers, sizes, batch, inv_global_batch, in_dtype, x, w_compute, activations, relu_bits, probs,
                       mask, target, grads_peers[rank], with_bias, scratch, scratch_bytes, loss, n_layers - 1, 0, stream,
                       grads_peers, world_size);
}

static int backward_impl(int n_layers, const int* sizes, int batch, float inv_global_batch, int in_dtype,
                         const void* x, const void* w_compute, void* const* activations,
                         void* const* relu_bits, const float* probs, const uint8_t* mask,
                         const float* target, float* grads, int with_bias, void* scratch,
                         size_t scratch_bytes, float* loss, int first_layer, int last_layer, void* stream,
                         float* const* grads_peers, int world) {
  int rc = check_layout("sb_mlp_backward", n_layers, sizes, batch, in_dtype);
  if (rc != SB_OK) return rc;
  if (!grads) return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_backward: grads is null");
  if (first_layer < last_layer || first_layer >= n_layers || last_layer < 0)
    return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_backward: layer range [%d, %d] of %d layers", last_layer, first_layer, n_layers);
  const bool from_top = first_layer == n_layers - 1;
  long long off[2 * MLP_MAX_LAYERS + 1];
  param_offsets(n_layers, sizes, off);
  cudaStream_t s = (cudaStream_t)stream;
  // Zeroes the gradient vector before a pass.  Weight segments that peers add into (data-parallel
  // pass) are left alone: their owner slices are zeroed by the update kernel that consumed them, and a
  // faster rank may already be adding this step's tiles.
  auto zero_grads = [&]() -> int {
    if (!grads_peers || world <= 1) {
      SB_CUDA(cudaMemsetAsync(grads, 0, (size_t)off[2 * n_layers] * 4, s));
      return SB_OK;
    }
    for (int i = 0; i < n_layers; ++i) {
      const bool fused = layer_grads_go_to_peers(padded_out(sizes[i + 1]), sizes[i], world);
      const long long begin = fused ? off[2 * i + 1] : off[2 * i];
      SB_CUDA(cudaMemsetAsync(grads + begin, 0, (size_t)(off[2 * i + 2] - begin) * 4, s));
    }
    return SB_OK;
  };
  if (batch == 0) {
    if (from_top) return zero_grads();
    return SB_OK;
  }
  if (!x || !w_compute || !probs || !target || !scratch)
    return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_backward: null pointer");
  if (n_layers > 1 && !activations) return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_backward: activations is null");
  for (int i = 1; i < n_layers; ++i)
    if (sizes[i] % 8 != 0)
      return sb_fail(SB_ERR_UNSUPPORTED, "sb_mlp_backward: hidden width %d is not a multiple of 8", sizes[i]);
  const size_t need = backward_scratch_bytes(n_layers, sizes, batch, in_dtype);
  if (scratch_bytes < need)
    return sb_fail(SB_ERR_BAD_ARG, "sb_mlp_backward: scratch of %zu bytes, %zu needed", scratch_bytes, need);
  if (reinterpret_cast<uintptr_t>(scratch) & 255) return sb_fail(SB_ERR_MISALIGNED, "sb_mlp_backward: scratch must be 256-byte aligned");
  const int es = sb_dtype_size(in_dtype);
  const int st = storage_dtype(in_dtype);
  int max_w = 0;
  for (int i = 0; i < n_layers; ++i) max_w = max(max_w, padded_out(sizes[i + 1]));
  const size_t dy_bytes = (size_t)align_up((long long)batch * max_w * es, 256);
  char* sc = reinterpret_cast<char*>(scratch);
  // The two dY buffers alternate once per dgrad: layer i reads the buffer chosen by the number of
  // dgrads above it, so a pass split into several calls finds its input where the last call left it.
  const bool odd = ((n_layers - 1 - first_layer) & 1) != 0;
  void* dy_cur = odd ? sc + dy_bytes : sc;
  void* dy_next = odd ? sc : sc + dy_bytes;
  float* partial = reinterpret_cast<float*>(sc + 2 * dy_bytes);

  // Bias gradients and split-K weight gradients are accumulated into zeroed memory.  Zero the whole buffer (padding included) so that
  // the all-reduce and the SGD update can treat it as one flat vector.
  if (from_top) {
    rc = zero_grads();
    if (rc != SB_OK) return rc;
  }

  const int n_out = sizes[n_layers];
  const int ld_out = padded_out(n_out);
  bool head_bias_done = false;
  if (from_top) {
    const int blocks = blocks_for(batch, 256);
    // The head layer's bias gradient is summed by this kernel when its padded width is 8 or 16.
    head_bias_done = with_bias && first_layer == n_layers - 1 && (ld_out == 8 || ld_out == 16);
    float* db_head = head_bias_done ? grads + off[2 * (n_layers - 1) + 1] : nullptr;
#define SB_CE_LAUNCH(T, R, L)                                                                                     \
  SB_CUDA(sb_launch(ce_grad_kernel<T, R, L>, dim3(blocks), dim3(256), 0, s, 1, probs, target, mask, (T*)dy_cur, \
                    batch, n_out, ld_out, inv_global_batch, loss, db_head))
#define SB_CE_BY_LD(T, R)                                     \
  do {                                                        \
    if (head_bias_done && ld_out == 8) SB_CE_LAUNCH(T, R, 8); \
    else if (head_bias_done) SB_CE_LAUNCH(T, R, 16);          \
    else SB_CE_LAUNCH(T, R, 0);                               \
  } while (0)
    if (in_dtype == SB_BF16) SB_CE_BY_LD(__nv_bfloat16, false);
    else if (in_dtype == SB_F16) SB_CE_BY_LD(__half, false);
    else SB_CE_BY_LD(float, true);
#undef SB_CE_BY_LD
#undef SB_CE_LAUNCH
    SB_COUNT_LAUNCH();
    SB_CUDA(cudaGetLastError());
  }

  // True when dY of the current layer came out of a dgrad whose epilogue already added its column
  // sums to the bias gradient, so that the stand-alone column-sum pass (a second read of dY) is skipped.
  // A pass split into several calls: the dgrad of the layer above ran in an earlier call.
  bool bias_done = from_top ? head_bias_done
                            : (with_bias && relu_bits && relu_bits[first_layer] && sizes[first_layer + 1] % 32 == 0);
  for (int i = first_layer; i >= last_layer; --i) {
    const int fan_out = padded_out(sizes[i + 1]), fan_in = sizes[i];
    const void* h_in = i == 0 ? x : activations[i - 1];
    if (with_bias && !bias_done) {
      // Enough blocks to fill the GPU a few times over, each with a long row slab.
      const int strip = 32 * (16 / es);
      const int strips = (fan_out + strip - 1) / strip;
      int slabs = (sb_sm_count() * 4 + strips - 1) / strips;
      int rows_per_block = (batch + slabs - 1) / slabs;
      if (rows_per_block < 64) rows_per_block = 64;
      dim3 grid(strips, (batch + rows_per_block - 1) / rows_per_block);
      float* db = grads + off[2 * i + 1];
      if (in_dtype == SB_BF16) SB_CUDA(sb_launch(colsum_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, s, 1, (const __nv_bfloat16*)dy_cur, db, batch, fan_out, rows_per_block));
      else if (in_dtype == SB_F16) SB_CUDA(sb_launch(colsum_kernel<__half>, dim3(grid), dim3(256), 0, s, 1, (const __half*)dy_cur, db, batch, fan_out, rows_per_block));
      else SB_CUDA(sb_launch(colsum_kernel<float>, dim3(grid), dim3(256), 0, s, 1, (const float*)dy_cur, db, batch, fan_out, rows_per_block));
      SB_COUNT_LAUNCH();
  SB_CUDA(cudaGetLastError());
    }
    // wgrad (TN): dW[out, in] = dY^T [out, B] * H_in [B, in]
    float* dw = grads + off[2 * i];
    const int want = wgrad_splits(fan_out, fan_in, batch, in_dtype);
    int used = 1;
    // The splits add their tiles straight into dW (zeroed above) through TMA reduce-add stores: no
    // partial matrices, no reduction kernel.  The order of those fp32 additions is not fixed, so the
    // last bits of dW can differ between runs; SB_WGRAD_PARTIALS=1 in the environment selects the
    // older form, partials reduced in a fixed order by a kernel of their own.
    const bool may_accumulate = want > 1 && !wgrad_partials_forced();
    if (grads_peers && layer_grads_go_to_peers(fan_out, fan_in, world)) {
      // Data-parallel pass: every tile is added to the copy of dW on the rank that owns its rows (the
      // reduce-scatter of the gradient all-reduce, done by the GEMM's own stores over peer memory).
      SbPeerOut po;
      po.n = world;
      for (int r = 0; r < world; ++r) po.c[r] = grads_peers[r] + off[2 * i];
      rc = sb_umma_gemm_launch(1, 0, 1.0f, dy_cur, h_in, 0.0f, nullptr, fan_out, fan_in, batch, in_dtype, SB_F32, 0, nullptr,
                               nullptr, nullptr, nullptr, s, want, &used, nullptr, nullptr, &po);
    } else {
      rc = sb_umma_gemm_launch(1, 0, 1.0f, dy_cur, h_in, 0.0f, (want > 1 && !may_accumulate) ? (void*)partial : (void*)dw,
                               fan_out, fan_in, batch, in_dtype, SB_F32, 0, nullptr, nullptr, nullptr, nullptr, s, want,
                               &used, nullptr, may_accumulate ? (void*)partial : nullptr);
    }
    if (rc != SB_OK) return rc;
    if (used > 1) {
      const long long n = (long long)fan_out * fan_in;
      SB_CUDA(sb_launch(splitk_reduce_kernel, dim3(blocks_for(n, 256)), dim3(256), 0, s, 1, partial, dw, n, used));
      SB_COUNT_LAUNCH();
  SB_CUDA(cudaGetLastError());
    }
    // dgrad (NN): dH[B, in] = dY [B, out] * W [out, in], gated by ReLU'(H_in)
    if (i > 0) {
      const void* w = reinterpret_cast<const char*>(w_compute) + off[2 * i] * es;
      // The gate is ReLU'(H_in): read from the sign bits the forward pass recorded
      // when they exist (4 bytes per row and 32 columns), else from H_in itself.
      const bool bits = relu_bits && relu_bits[i - 1] && fan_in % 32 == 0;
      // The output is dY of layer i-1, whose column sums are that layer's bias gradient
      // (fan_in = sizes[i] is its unpadded width: hidden widths are multiples of 8 and, here, of 32).
      const bool sum_cols = bits && with_bias;
      float* db_below = grads + off[2 * (i - 1) + 1];
      if (bits && narrow_dgrad_ok(sizes[i + 1], fan_in, in_dtype) && st == in_dtype) {
        // A head layer: the inner dimension is at most 16, nothing for the tensor cores to do.
        const uint32_t* gate = reinterpret_cast<const uint32_t*>(relu_bits[i - 1]);
        rc = in_dtype == SB_BF16
                 ? narrow_dgrad_launch<__nv_bfloat16>(dy_cur, fan_out, w, sizes[i + 1], fan_in, gate, dy_next, sum_cols ? db_below : nullptr, batch, s)
                 : narrow_dgrad_launch<__half>(dy_cur, fan_out, w, sizes[i + 1], fan_in, gate, dy_next, sum_cols ? db_below : nullptr, batch, s);
      } else
      rc = sb_umma_gemm_launch(0, 0, 1.0f, dy_cur, w, 0.0f, dy_next, batch, fan_in, fan_out, in_dtype, st,
                               bits ? (SB_EPI_RELU_GRAD_MASK | (sum_cols ? SB_EPI_COLSUM_OUT : 0)) : SB_EPI_RELU_GRAD,
                               nullptr, nullptr, bits ? (const void*)relu_bits[i - 1] : h_in,
                               sum_cols ? (void*)db_below : nullptr, s, 1, nullptr);
      if (rc != SB_OK) return rc;
      bias_done = sum_cols;
      void* t = dy_cur; dy_cur = dy_next; dy_next = t;
    }
  }
  return SB_OK;
}

int sb_mlp_backward(int n_layers, const int* sizes, int batch, float inv_global_batch, int in_dtype,
                    const void* x, const void* w_compute, void* const* activations,
                    void* const* relu_bits, const float* probs, const uint8_t* mask, const float* target,
                    float* grads, int with_bias, void* scratch, size_t scratch_bytes, float* loss,
                    void* stream) {
  return sb_mlp_backward_range(n_layers, sizes, batch, inv_global_batch, in_dtype, x, w_compute, activations,
                               relu_bits, probs, mask, target, grads, with_bias, scratch, scratch_bytes, loss,
                               n_layers - 1, 0, stream);
}

int sb_sgd_update(float* params, const float* grads, void* w_compute, long long n, float lr,
                  int compute_dtype, void* stream) {
  if (n < 0) return sb_fail(SB_ERR_BAD_ARG, "sb_sgd_update: negative length");
  if (n == 0) return SB_OK;
  if (!params || !grads) return sb_fail(SB_ERR_BAD_ARG, "sb_sgd_update: null pointer");
  SB_CUDA(sb_launch(sgd_kernel, dim3(blocks_for(n, 256)), dim3(256), 0, (cudaStream_t)stream, 1, params, grads, w_compute, n, lr, compute_dtype));
  SB_COUNT_LAUNCH();
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

int sb_mlp_train_step(int n_layers, const int* sizes, int batch, int in_dtype, const void* x,
                      float* params, void* w_compute, void* const* activations, void* const* relu_bits,
                      const uint8_t* mask,
                      const float* target, float* probs, float* grads, int with_bias, float lr,
                      void* scratch, size_t scratch_bytes, float* loss, void* stream) {
  // Narrow nets run the whole forward pass as one fused launch that also writes what backward needs.
  int rc;
  if (sb_mlp_fused_supported(n_layers, sizes, in_dtype) && batch > 0)
    rc = sb_mlp_forward_fused_train(n_layers, sizes, batch, in_dtype, x, w_compute, with_bias ? params : nullptr,
                                    activations, relu_bits, SB_EPI_MASKED_SOFTMAX, mask, probs, nullptr, stream);
  else
    rc = sb_mlp_forward(n_layers, sizes, batch, in_dtype, x, w_compute, with_bias ? params : nullptr,
                        activations, relu_bits, SB_EPI_MASKED_SOFTMAX, mask, probs, nullptr, stream);
  if (rc != SB_OK) return rc;
  rc = sb_mlp_backward(n_layers, sizes, batch, batch > 0 ? 1.0f / (float)batch : 0.f, in_dtype, x, w_compute,
                       activations, relu_bits, probs, mask, target, grads, with_bias, scratch, scratch_bytes, loss,
                       stream);
  if (rc != SB_OK) return rc;
  long long off[2 * MLP_MAX_LAYERS + 1];
  param_offsets(n_layers, sizes, off);
  return sb_sgd_update(params, grads, w_compute, off[2 * n_layers], lr, storage_dtype(in_dtype), stream);
}

}  // extern "C"
