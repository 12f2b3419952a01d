// Stand-alone elementwise and per-row operations: the unfused forms of the
// epilogues, for rows wider than a fused head can hold and for callers that
// run them as separate graph nodes the way the reference does
// (BlockMap / BlockRowMap / BlockRowReduce, ml/layers.spi:195-210;
// row math ml/primitives.spi:701-722,748-780).
//
// Rows of at most 64 columns (the policy heads) take one thread per row with the
// row in registers; wider rows one warp per row, lanes striding over the columns
// with warp-shuffle reductions, so any column count works.
#include "common.cuh"
#include "row_head.cuh"

namespace {

constexpr float NEG_MAX = -3.402823466e38f;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ int warp_sum_int(int v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ bool is_legal(const uint8_t* mrow, int prefix, int j) {
  if (prefix >= 0) return j < prefix;
  if (mrow) return mrow[j] != 0;
  return true;
}

enum RowOp { ROW_SOFTMAX = 0, ROW_REGRET = 1, ROW_LN_L2 = 2 };

template <int OP>
__global__ void row_map_kernel(const float* x, float* out, int rows, int cols,
                               const uint8_t* __restrict__ mask, int prefix) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  for (long long row = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows;
       row += (long long)gridDim.x * warps_per_block) {
    const float* xr = x + row * cols;
    float* orow = out + row * cols;
    const uint8_t* mrow = mask ? mask + row * cols : nullptr;
    if (OP == ROW_SOFTMAX) {
      float mx = NEG_MAX;
      for (int j = lane; j < cols; j += 32)
        if (is_legal(mrow, prefix, j)) mx = fmaxf(mx, xr[j]);
      mx = warp_max(mx);
      float s = 0.f;
      for (int j = lane; j < cols; j += 32)
        if (is_legal(mrow, prefix, j)) s += __expf(xr[j] - mx);
      s = warp_sum(s);
      const float inv = s > 0.f ? 1.f / s : 0.f;
      for (int j = lane; j < cols; j += 32)
        orow[j] = is_legal(mrow, prefix, j) ? __expf(xr[j] - mx) * inv : 0.f;
    } else if (OP == ROW_REGRET) {
      float s = 0.f;
      int count = 0;
      for (int j = lane; j < cols; j += 32) {
        if (is_legal(mrow, prefix, j)) {
          s += fmaxf(xr[j], 0.f);
          ++count;
        }
      }
      s = warp_sum(s);
      count = warp_sum_int(count);
      const float inv_len = count > 0 ? 1.f / (float)count : 0.f;
      for (int j = lane; j < cols; j += 32) {
        const bool lg = is_legal(mrow, prefix, j);
        const float q = fmaxf(xr[j], 0.f);
        orow[j] = !lg ? 0.f : (s != 0.f ? q / s : inv_len);
      }
    } else {
      float s = 0.f;
      for (int j = lane; j < cols; j += 32) s += xr[j] * xr[j];
      s = warp_sum(s);
      for (int j = lane; j < cols; j += 32) orow[j] = s != 0.f ? xr[j] / s : 0.f;
    }
  }
}

// Narrow rows (at most 64 columns, the policy heads): one THREAD per row with the row in registers, the
// same code the fused GEMM heads run (row_head.cuh), instead of a warp per row with most lanes idle.
// x and out are [rows, cols] fp32 and may alias (a row is read whole before it is written).
template <int W>
__global__ void __launch_bounds__(128) row_head_kernel(const float* x, float* out, int rows, SbRowHead h) {
  for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += (long long)gridDim.x * blockDim.x) {
    float v[W];
    const float* xr = x + r * h.n;
#pragma unroll
    for (int j = 0; j < W; ++j) v[j] = j < h.n ? xr[j] : 0.f;
    sb_row_head_finish<W>(h, v, r, out + r * h.n);
  }
}

__global__ void row_argmax_kernel(const float* __restrict__ x, int32_t* __restrict__ out, int rows,
                                  int cols) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  for (long long row = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows;
       row += (long long)gridDim.x * warps_per_block) {
    const float* xr = x + row * cols;
    float bv = NEG_MAX;
    int bi = 0x7fffffff;
    for (int j = lane; j < cols; j += 32) {
      const float v = xr[j];
      if (v > bv || (v == bv && j < bi)) {
        bv = v;
        bi = j;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    if (lane == 0) out[row] = bi == 0x7fffffff ? 0 : bi;
  }
}

__global__ void relu_kernel(const float* x, float* out, size_t n) {
  const size_t n4 = n / 4;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (aligned) {
    const float4* x4 = reinterpret_cast<const float4*>(x);
    float4* o4 = reinterpret_cast<float4*>(out);
    for (size_t q = i; q < n4; q += step) {
      float4 v = x4[q];
      v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f);
      o4[q] = v;
    }
    for (size_t q = n4 * 4 + i; q < n; q += step) out[q] = fmaxf(x[q], 0.f);
  } else {
    for (size_t q = i; q < n; q += step) out[q] = fmaxf(x[q], 0.f);
  }
}

__device__ __forceinline__ float round_to_tf32(float v) {
  // Round-to-nearest-even to 10 explicit mantissa bits; the result is an
  // fp32 value whose low 13 bits are zero, so the tensor core's own operand
  // truncation leaves it unchanged.
  uint32_t u = __float_as_uint(v);
  if ((u & 0x7f800000u) == 0x7f800000u) return v;
  const uint32_t lsb = (u >> 13) & 1u;
  u += 0x0fffu + lsb;
  u &= 0xffffe000u;
  return __uint_as_float(u);
}

__global__ void convert_kernel(const float* __restrict__ x, void* __restrict__ out, size_t n, int dt) {
  const size_t step = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
    const float v = x[i];
    if (dt == SB_BF16) reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
    else if (dt == SB_F16) reinterpret_cast<__half*>(out)[i] = __float2half_rn(v);
    else if (dt == SB_TF32) reinterpret_cast<float*>(out)[i] = round_to_tf32(v);
    else reinterpret_cast<float*>(out)[i] = v;
  }
}

// Game-state encoder.  The reference zeroes the input tensor and pickles each
// game state into it on the device (ml/models.spi:30-41): a bounded int becomes
// a one-hot group (corebase/pickler.spi:20-37).  Here the host ships compact
// records -- one byte per one-hot field plus the dense values -- and this kernel
// writes the dense network input [rows, features] in the storage type: field j
// with value v < widths[j] sets feature (offset_j + v), any other value leaves
// the group zero; `dense` [rows, n_dense] follows unchanged.
constexpr int ENC_MAX_FIELDS = 64;
constexpr int ENC_MAX_ONEHOT = 2048;
struct EncodeLayout {
  int n_fields;
  int onehot;                       // sum of widths
  unsigned char widths[ENC_MAX_FIELDS];
};

template <typename T>
__global__ void __launch_bounds__(256)
encode_states_kernel(const uint8_t* __restrict__ fields, const T* __restrict__ dense, T* __restrict__ x,
                     long long rows, int n_dense, EncodeLayout lay) {
  constexpr int VEC = 16 / sizeof(T);
  __shared__ unsigned char field_of[ENC_MAX_ONEHOT];   // which field owns a one-hot feature
  __shared__ unsigned char pos_of[ENC_MAX_ONEHOT];     // and which value of the field sets it
  for (int j = 0, col = 0; j < lay.n_fields; ++j) {
    const int w = lay.widths[j];
    for (int t = threadIdx.x; t < w; t += blockDim.x) {
      field_of[col + t] = (unsigned char)j;
      pos_of[col + t] = (unsigned char)t;
    }
    col += w;
  }
  __syncthreads();
  const int features = lay.onehot + n_dense;
  const int pieces = (features + VEC - 1) / VEC;           // 16-byte pieces per output row
  const long long total = rows * pieces;
  const long long step = (long long)gridDim.x * blockDim.x;
  const bool vec_ok = features % VEC == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    const long long r = i / pieces;
    const int f0 = (int)(i - r * pieces) * VEC;
    T out[VEC];
#pragma unroll
    for (int t = 0; t < VEC; ++t) {
      const int f = f0 + t;
      T v = (T)0.f;
      if (f < lay.onehot) {
        if (fields[r * lay.n_fields + field_of[f]] == pos_of[f]) v = (T)1.f;
      } else if (f < features) {
        v = dense[r * n_dense + (f - lay.onehot)];
      }
      out[t] = v;
    }
    if (vec_ok) {
      *reinterpret_cast<uint4*>(x + r * features + f0) = *reinterpret_cast<const uint4*>(out);
    } else {
#pragma unroll
      for (int t = 0; t < VEC; ++t)
        if (f0 + t < features) x[r * features + f0 + t] = out[t];
    }
  }
}

// Discrete sampling of one index per row from non-negative weights (probabilities), with the
// caller's uniform number u in (0, 1] per row: local_discrete_sampling, ml/primitives.spi:782-800 --
// cdf = running sum of the row, top = the cdf at the last positive entry, result = the first j
// with x[j] > 0 and cdf[j] >= u * top; -1 for a row without a positive entry (the reference
// returns its integer maximum there).  The reference draws u inside the kernel; here the random
// stream stays with the caller, which makes the result a pure function of (row, u).  One thread per
// row, sums in index order.
__global__ void row_sample_kernel(const float* __restrict__ x, const float* __restrict__ u,
                                  int32_t* __restrict__ out, int rows, int cols) {
  for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < rows;
       r += (long long)gridDim.x * blockDim.x) {
    const float* row = x + r * cols;
    float s = 0.f, top = 0.f;
    for (int j = 0; j < cols; ++j) {
      const float v = row[j];
      s += v;
      if (v > 0.f) top = s;
    }
    const float threshold = u[r] * top;
    int pick = -1;
    s = 0.f;
    for (int j = 0; j < cols; ++j) {
      const float v = row[j];
      s += v;
      if (v > 0.f && s - threshold >= 0.f) {
        pick = j;
        break;
      }
    }
    out[r] = pick;
  }
}

// The same with the uniform number drawn on the device: row r uses output `position` of the Philox
// stream (seed, row_offset + r), the draw the fused sampling heads make (row_head.cuh).
__global__ void row_sample_seeded_kernel(const float* __restrict__ x, int32_t* __restrict__ out, int rows, int cols,
                                         unsigned long long seed, unsigned long long row_offset,
                                         unsigned long long position) {
  for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < rows;
       r += (long long)gridDim.x * blockDim.x) {
    const float* row = x + r * cols;
    const float u = sb_uniform_open_closed(sb_philox_u32(seed, row_offset + (unsigned long long)r, position));
    float s = 0.f, top = 0.f;
    for (int j = 0; j < cols; ++j) {
      const float v = row[j];
      s = __fadd_rn(s, v);
      if (v > 0.f) top = s;
    }
    const float threshold = __fmul_rn(u, top);
    int pick = -1;
    s = 0.f;
    for (int j = 0; j < cols; ++j) {
      const float v = row[j];
      s = __fadd_rn(s, v);
      if (v > 0.f && __fsub_rn(s, threshold) >= 0.f) {
        pick = j;
        break;
      }
    }
    out[r] = pick;
  }
}

__global__ void philox_uniform_kernel(float* __restrict__ out, long long n, unsigned long long seed,
                                      unsigned long long row_offset, unsigned long long position) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = sb_uniform_open_closed(sb_philox_u32(seed, row_offset + (unsigned long long)i, position));
}

// Hash of a row: bit j = (x[r, j] > 0), the word taken modulo `modulo` (local_binarize,
// ml/primitives.spi:816-821; rows of at most 32 values, where the shift is defined).
__global__ void row_binarize_kernel(const float* __restrict__ x, uint32_t* __restrict__ out, int rows, int cols,
                                    uint32_t modulo) {
  for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < rows;
       r += (long long)gridDim.x * blockDim.x) {
    const float* row = x + r * cols;
    uint32_t bits = 0u;
    for (int j = 0; j < cols; ++j) bits |= (row[j] > 0.f ? 1u : 0u) << j;
    out[r] = bits % modulo;
  }
}

int grid_for(long long work_items, int per_block) {
  long long b = (work_items + per_block - 1) / per_block;
  if (b < 1) b = 1;
  const long long cap = (long long)sb_sm_count() * 16;
  return (int)(b > cap ? cap : b);
}

}  // namespace

extern "C" {

int sb_relu(const float* x, float* out, size_t n, void* stream) {
  if (n == 0) return SB_OK;
  if (!x || !out) return sb_fail(SB_ERR_BAD_ARG, "sb_relu: null pointer");
  relu_kernel<<<grid_for((long long)(n / 4 + 1), 256), 256, 0, (cudaStream_t)stream>>>(x, out, n);
  SB_COUNT_LAUNCH();
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

static int row_args_ok(const char* who, const void* x, const void* out, int rows, int cols) {
  if (rows < 0 || cols < 0) return sb_fail(SB_ERR_BAD_ARG, "%s: negative size", who);
  if (rows == 0 || cols == 0) return 1;
  if (!x || !out) return sb_fail(SB_ERR_BAD_ARG, "%s: null pointer", who);
  return SB_OK;
}

// Softmax / regret matching of rows of at most 64 columns through the thread-per-row kernel.
static int launch_narrow_head(const float* x, float* out, int rows, int cols, const uint8_t* mask, int prefix, int flag,
                              void* stream) {
  SbRowHead h;
  memset(&h, 0, sizeof(h));
  h.n = cols; h.flags = flag; h.prefix = prefix < 0 ? -1 : (prefix > cols ? cols : prefix); h.mask = mask;
  const int grid = grid_for(rows, 128);
  cudaStream_t s = (cudaStream_t)stream;
  if (cols <= 16) row_head_kernel<16><<<grid, 128, 0, s>>>(x, out, rows, h);
  else if (cols <= 32) row_head_kernel<32><<<grid, 128, 0, s>>>(x, out, rows, h);
  else row_head_kernel<64><<<grid, 128, 0, s>>>(x, out, rows, h);
  SB_COUNT_LAUNCH();
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

int sb_row_softmax(const float* x, float* out, int rows, int cols, const uint8_t* mask, int prefix,
                   void* stream) {
  int rc = row_args_ok("sb_row_softmax", x, out, rows, cols);
  if (rc != SB_OK) return rc > 0 ? SB_OK : rc;
  if (cols <= 64) return launch_narrow_head(x, out, rows, cols, mask, prefix, SB_EPI_MASKED_SOFTMAX, stream);
  row_map_kernel<ROW_SOFTMAX><<<grid_for(rows, 8), 256, 0, (cudaStream_t)stream>>>(x, out, rows, cols, mask, prefix);
  SB_COUNT_LAUNCH();
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

int sb_row_regret_matching(const float* x, float* out, int rows, int cols, const uint8_t* mask,
                           int prefix, void* stream) {
  int rc = row_args_ok("sb_row_regret_matching", x, out, rows, cols);
  if (rc != SB_OK) return rc > 0 ? SB_OK : rc;
  if (cols <= 64) return launch_narrow_head(x, out, rows, cols, mask, prefix, SB_EPI_REGRET_MATCHING, stream);
  row_map_kernel<ROW_REGRET><<<grid_for(rows, 8), 256, 0, (cudaStream_t)stream>>>(x, out, rows, cols, mask, prefix);
  SB_COUNT_LAUNCH();
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

int sb_row_ln_l2(const float* x, float* out, int rows, int cols, void* stream) {
  int rc = row_args_ok("sb_row_ln_l2", x, out, rows, cols);
  if (rc != SB_OK) return rc > 0 ? SB_OK : rc;
  row_map_kernel<ROW_LN_L2><<<grid_for(rows, 8), 256, 0, (cudaStream_t)stream>>>(x, out, rows, cols, nullptr, -1);
  SB_COUNT_LAUNCH();
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

int sb_row_argmax(const float* x, int32_t* out, int rows, int cols, void* stream) {
  int rc = row_args_ok("sb_row_argmax", x, out, rows, cols);
  if (rc != SB_OK) return rc > 0 ? SB_OK : rc;
  row_argmax_kernel<<<grid_for(rows, 8), 256, 0, (cudaStream_t)stream>>>(x, out, rows, cols);
  SB_COUNT_LAUNCH();
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

int sb_row_sample(const float* probs, const float* uniforms, int32_t* out, int rows, int cols, void* stream) {
  int rc = row_args_ok("sb_row_sample", probs, out, rows, cols);
  if (rc != SB_OK) return rc > 0 ? SB_OK : rc;
  if (!uniforms) return sb_fail(SB_ERR_BAD_ARG, "sb_row_sample: uniforms is null");
  row_sample_kernel<<<grid_for(rows, 256), 256, 0, (cudaStream_t)stream>>>(probs, uniforms, out, rows, cols);
  SB_COUNT_LAUNCH();
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

int sb_row_sample_seeded(const float* probs, int32_t* out, int rows, int cols, unsigned long long seed,
                         unsigned long long row_offset, unsigned long long position, void* stream) {
  int rc = row_args_ok("sb_row_sample_seeded", probs, out, rows, cols);
  if (rc != SB_OK) return rc > 0 ? SB_OK : rc;
  row_sample_seeded_kernel<<<grid_for(rows, 256), 256, 0, (cudaStream_t)stream>>>(probs, out, rows, cols, seed, row_offset,
                                                                                  position);
  SB_COUNT_LAUNCH();
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

int sb_philox_uniform(float* out, long long n, unsigned long long seed, unsigned long long row_offset,
                      unsigned long long position, void* stream) {
  if (n < 0) return sb_fail(SB_ERR_BAD_ARG, "sb_philox_uniform: negative length");
  if (n == 0) return SB_OK;
  if (!out) return sb_fail(SB_ERR_BAD_ARG, "sb_philox_uniform: null output");
  philox_uniform_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(out, n, seed, row_offset, position);
  SB_COUNT_LAUNCH();
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

int sb_row_binarize(const float* x, uint32_t* out, int rows, int cols, uint32_t modulo, void* stream) {
  int rc = row_args_ok("sb_row_binarize", x, out, rows, cols);
  if (rc != SB_OK) return rc > 0 ? SB_OK : rc;
  if (cols > 32) return sb_fail(SB_ERR_UNSUPPORTED, "sb_row_binarize: rows of at most 32 values (cols=%d)", cols);
  if (modulo == 0u) return sb_fail(SB_ERR_BAD_ARG, "sb_row_binarize: modulo must be positive");
  row_binarize_kernel<<<grid_for(rows, 256), 256, 0, (cudaStream_t)stream>>>(x, out, rows, cols, modulo);
  SB_COUNT_LAUNCH();
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

int sb_convert(const float* x, void* out, size_t n, int out_dtype, void* stream) {
  if (n == 0) return SB_OK;
  if (!x || !out) return sb_fail(SB_ERR_BAD_ARG, "sb_convert: null pointer");
  if (out_dtype != SB_BF16 && out_dtype != SB_F16 && out_dtype != SB_TF32 && out_dtype != SB_F32)
    return sb_fail(SB_ERR_BAD_ARG, "sb_convert: unknown output dtype %d", out_dtype);
  convert_kernel<<<grid_for((long long)n, 256), 256, 0, (cudaStream_t)stream>>>(x, out, n, out_dtype);
  SB_COUNT_LAUNCH();
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

int sb_encode_states(const uint8_t* fields, int n_fields, const int* widths, const void* dense, int n_dense,
                     void* x, long long rows, int dtype, void* stream) {
  if (rows < 0 || n_fields < 0 || n_dense < 0) return sb_fail(SB_ERR_BAD_ARG, "sb_encode_states: negative size");
  if (n_fields > ENC_MAX_FIELDS) return sb_fail(SB_ERR_TOO_LARGE, "sb_encode_states: at most %d one-hot fields", ENC_MAX_FIELDS);
  if (n_fields > 0 && !widths) return sb_fail(SB_ERR_BAD_ARG, "sb_encode_states: widths is null");
  if (dtype != SB_F32 && dtype != SB_TF32 && dtype != SB_BF16 && dtype != SB_F16)
    return sb_fail(SB_ERR_BAD_ARG, "sb_encode_states: unknown storage dtype %d", dtype);
  EncodeLayout lay;
  memset(&lay, 0, sizeof(lay));
  lay.n_fields = n_fields;
  for (int j = 0; j < n_fields; ++j) {
    if (widths[j] < 1 || widths[j] > 255) return sb_fail(SB_ERR_BAD_ARG, "sb_encode_states: widths[%d] = %d is outside [1, 255]", j, widths[j]);
    lay.widths[j] = (unsigned char)widths[j];
    lay.onehot += widths[j];
  }
  if (lay.onehot > ENC_MAX_ONEHOT) return sb_fail(SB_ERR_TOO_LARGE, "sb_encode_states: at most %d one-hot features", ENC_MAX_ONEHOT);
  if (rows == 0 || lay.onehot + n_dense == 0) return SB_OK;
  if (!x || (n_fields > 0 && !fields) || (n_dense > 0 && !dense)) return sb_fail(SB_ERR_BAD_ARG, "sb_encode_states: null pointer");
  const int es = sb_dtype_size(dtype);
  const long long pieces = (long long)rows * ((lay.onehot + n_dense + 16 / es - 1) / (16 / es));
  const int grid = grid_for(pieces, 256);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == SB_BF16)
    encode_states_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(fields, (const __nv_bfloat16*)dense, (__nv_bfloat16*)x, rows, n_dense, lay);
  else if (dtype == SB_F16)
    encode_states_kernel<__half><<<grid, 256, 0, s>>>(fields, (const __half*)dense, (__half*)x, rows, n_dense, lay);
  else
    encode_states_kernel<float><<<grid, 256, 0, s>>>(fields, (const float*)dense, (float*)x, rows, n_dense, lay);
  SB_COUNT_LAUNCH();
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

}  // extern "C"
