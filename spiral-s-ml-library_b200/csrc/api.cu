// Public GEMM entry points: argument validation and dispatch between the
// tensor-core path (TF32 / BF16 / FP16 inputs) and the fp32 FFMA path.
// Mirrors the call surface of matmul_tf32 / matmul_tf32'
// (ml/matmul/run.spi:21-26): C's shape gives M and N, A gives K, all tensors
// row-major and written in place.
#include "common.cuh"
#include "row_head.cuh"

int sb_umma_plan(int a_trans, int b_trans, int M, int N, int K, int in_dtype, int sms, int* plan5);
int sb_scale_launch(void* C, long long total, float beta, int out_dtype, cudaStream_t stream);
int sb_sgemm_launch(int a_trans, int b_trans, float alpha, const float* A, const float* B, float beta,
                    float* C, int M, int N, int K, int epi, const float* bias, cudaStream_t stream);

namespace {
constexpr int HEAD_FLAGS = SB_EPI_MASKED_SOFTMAX | SB_EPI_REGRET_MATCHING | SB_EPI_ARGMAX;   // heads sb_matmul_ex accepts
constexpr int SPEC_HEAD_FLAGS = HEAD_FLAGS | SB_EPI_SAMPLE | SB_EPI_BINARIZE;                  // heads sb_matmul_head accepts
constexpr int GATE_FLAGS = SB_EPI_RELU_MASK_OUT | SB_EPI_RELU_GRAD_MASK;
constexpr int ALL_FLAGS = SB_EPI_BIAS | SB_EPI_RELU | SB_EPI_RELU_GRAD | HEAD_FLAGS | GATE_FLAGS | SB_EPI_COLSUM_OUT |
                          SB_EPI_LN_L2;

// The head as kernels of its own on the finished C (rows too wide for the fused head).
int run_heads_unfused(float* C, int M, int N, const SbRowHead& h, void* stream) {
  int rc = SB_OK;
  if (h.flags & SB_EPI_BINARIZE) {
    rc = sb_row_binarize(C, h.hash_out, M, N, h.modulo, stream);
    if (rc != SB_OK) return rc;
  }
  if (h.flags & SB_EPI_MASKED_SOFTMAX) {
    rc = sb_row_softmax(C, C, M, N, h.mask, h.prefix, stream);
    if (rc != SB_OK) return rc;
  }
  if (h.flags & SB_EPI_REGRET_MATCHING) {
    rc = sb_row_regret_matching(C, C, M, N, h.mask, h.prefix, stream);
    if (rc != SB_OK) return rc;
  }
  if (h.flags & SB_EPI_ARGMAX) {
    rc = sb_row_argmax(C, h.argmax_out, M, N, stream);
    if (rc != SB_OK) return rc;
  }
  if (h.flags & SB_EPI_SAMPLE) rc = sb_row_sample_seeded(C, h.sample_out, M, N, h.seed, h.row_offset, h.position, stream);
  return rc;
}

SbRowHead legacy_head(int epilogue, int N, const uint8_t* mask, void* aux_out) {
  SbRowHead h;
  memset(&h, 0, sizeof(h));
  h.n = N; h.flags = epilogue & HEAD_FLAGS; h.prefix = -1; h.mask = mask;
  h.argmax_out = reinterpret_cast<int32_t*>(aux_out);
  return h;
}

int check_head(const char* who, const SbRowHead& h, int N) {
  if (h.flags & ~SPEC_HEAD_FLAGS) return sb_fail(SB_ERR_BAD_ARG, "%s: head flags 0x%x hold something that is not a row head", who, h.flags);
  if ((h.flags & SB_EPI_ARGMAX) && !h.argmax_out) return sb_fail(SB_ERR_BAD_ARG, "%s: SB_EPI_ARGMAX without argmax_out", who);
  if ((h.flags & SB_EPI_SAMPLE) && !h.sample_out) return sb_fail(SB_ERR_BAD_ARG, "%s: SB_EPI_SAMPLE without sample_out", who);
  if (h.flags & SB_EPI_BINARIZE) {
    if (!h.hash_out || h.modulo == 0) return sb_fail(SB_ERR_BAD_ARG, "%s: SB_EPI_BINARIZE needs hash_out and a non-zero modulo", who);
    if (N > 32) return sb_fail(SB_ERR_UNSUPPORTED, "%s: the sign hash is defined for rows of at most 32 values (N=%d)", who, N);
  }
  if (h.prefix > N) return sb_fail(SB_ERR_BAD_ARG, "%s: prefix %d beyond the %d columns", who, h.prefix, N);
  return SB_OK;
}
}  // namespace

// ---------------------------------------------------------------------------
// fp32 class on the tensor cores: the "3 x TF32" split.
//
// An fp32 value x is written hi + lo with hi = tf32(x) and lo = tf32(x - hi) (both rounded to
// nearest); then A * B = Ah*Bh + Ah*Bl + Al*Bh up to terms of relative size 2^-22.  The three products
// are ONE tensor-core GEMM over operands concatenated along K:
//     [Ah | Ah | Al] (M x 3K)   times   [Bh ; Bl ; Bh] (3K x N),
// accumulated in fp32 in tensor memory.  A pre-pass kernel writes the concatenated operands (in the
// same storage order as the originals, so every layout flag carries over) into a caller workspace.
// ---------------------------------------------------------------------------
namespace {

__device__ __forceinline__ float tf32_rn(float v) {
  uint32_t u = __float_as_uint(v);
  if ((u & 0x7f800000u) == 0x7f800000u) return v;
  u += 0x0fffu + ((u >> 13) & 1u);
  return __uint_as_float(u & 0xffffe000u);
}

// `src` is [rows, cols] row-major.  k_is_col: K runs along the columns (dst [rows, 3 * cols], the three
// parts side by side in every row); otherwise K runs along the rows (dst [3 * rows, cols], the parts
// stacked).  Part order p0, p1, p2 with 0 = hi, 1 = lo.  Two matrices per launch (A then B).
struct SplitJob {
  const float* src;
  float* dst;
  long long rows, cols;
  int k_is_col;
  int part[3];
};

// c_init: when non-null the same launch also brings C to beta * C (zero for beta == 0), the state the
// split-K tiles are then added to.
__global__ void split3_kernel(SplitJob ja, SplitJob jb, float* c_init, long long c_count, float beta) {
  sb_grid_dependency_wait();
  sb_grid_dependents_launch();
  const long long na = ja.rows * ja.cols, total = na + jb.rows * jb.cols;
  const long long step = (long long)gridDim.x * blockDim.x;
  if (c_init) {
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < c_count; t += step)
      c_init[t] = beta == 0.0f ? 0.0f : beta * c_init[t];
  }
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += step) {
    const bool first = t < na;
    const SplitJob& j = first ? ja : jb;
    const long long i = first ? t : t - na;
    const float x = j.src[i];
    const float hi = tf32_rn(x);
    const float lo = tf32_rn(x - hi);
    const long long r = i / j.cols, c = i - r * j.cols;
#pragma unroll
    for (int p = 0; p < 3; ++p) {
      const float v = j.part[p] ? lo : hi;
      if (j.k_is_col) j.dst[r * (3 * j.cols) + p * j.cols + c] = v;
      else j.dst[(p * j.rows + r) * j.cols + c] = v;
    }
  }
}

}  // namespace

extern "C" {

int sb_matmul_f32_workspace_bytes(int M, int N, int K, size_t* bytes) {
  if (!bytes) return sb_fail(SB_ERR_BAD_ARG, "sb_matmul_f32_workspace_bytes: null output");
  if (M < 0 || N < 0 || K < 0) return sb_fail(SB_ERR_BAD_ARG, "sb_matmul_f32_workspace_bytes: negative dimension");
  const size_t a = ((size_t)3 * M * K * 4 + 255) / 256 * 256, b = ((size_t)3 * N * K * 4 + 255) / 256 * 256;
  *bytes = a + b + 256;
  return SB_OK;
}

int sb_matmul_f32x3(int a_trans, int b_trans, float alpha, const float* A, const float* B, float beta, float* C,
                    int M, int N, int K, int epilogue, const float* bias, void* workspace, size_t workspace_bytes,
                    void* stream) {
  if (M < 0 || N < 0 || K <= 0) return sb_fail(SB_ERR_BAD_ARG, "sb_matmul_f32x3: dimensions M=%d N=%d K=%d", M, N, K);
  if (epilogue & ~(SB_EPI_BIAS | SB_EPI_RELU)) return sb_fail(SB_ERR_UNSUPPORTED, "sb_matmul_f32x3: epilogue may hold SB_EPI_BIAS and SB_EPI_RELU");
  if ((epilogue & SB_EPI_BIAS) && !bias) return sb_fail(SB_ERR_BAD_ARG, "sb_matmul_f32x3: SB_EPI_BIAS without a bias pointer");
  if (M == 0 || N == 0) return SB_OK;
  if (!A || !B || !C || !workspace) return sb_fail(SB_ERR_BAD_ARG, "sb_matmul_f32x3: null pointer");
  size_t need = 0;
  sb_matmul_f32_workspace_bytes(M, N, K, &need);
  if (workspace_bytes < need) return sb_fail(SB_ERR_BAD_ARG, "sb_matmul_f32x3: workspace of %zu bytes, %zu needed", workspace_bytes, need);
  if ((long long)3 * K > 0x7fffffffLL) return sb_fail(SB_ERR_TOO_LARGE, "sb_matmul_f32x3: 3 * K exceeds the index range");
  // Row pitches of the concatenated operands must be multiples of 16 bytes (TMA): K % 4 == 0 where K is
  // contiguous, M (N) % 4 == 0 where M (N) is.
  const long long lda = a_trans ? M : 3LL * K, ldb = b_trans ? 3LL * K : N;
  if ((lda * 4) % 16 != 0 || (ldb * 4) % 16 != 0 || ((long long)N * 4) % 16 != 0 || (reinterpret_cast<uintptr_t>(C) & 15))
    return sb_fail(SB_ERR_MISALIGNED, "sb_matmul_f32x3: contiguous dimensions must be multiples of 4 elements and C 16-byte "
                                      "aligned (use the SB_F32 class of sb_matmul_ex for other shapes)");
  char* ws = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~(uintptr_t)255);
  float* a3 = reinterpret_cast<float*>(ws);
  float* b3 = reinterpret_cast<float*>(ws + ((size_t)3 * M * K * 4 + 255) / 256 * 256);
  SplitJob ja, jb;
  ja.src = A; ja.dst = a3; ja.rows = a_trans ? K : M; ja.cols = a_trans ? M : K; ja.k_is_col = a_trans ? 0 : 1;
  ja.part[0] = 0; ja.part[1] = 0; ja.part[2] = 1;                     // Ah | Ah | Al
  jb.src = B; jb.dst = b3; jb.rows = b_trans ? N : K; jb.cols = b_trans ? K : N; jb.k_is_col = b_trans ? 1 : 0;
  jb.part[0] = 0; jb.part[1] = 1; jb.part[2] = 0;                     // Bh ; Bl ; Bh
  const long long total = (long long)M * K + (long long)N * K;
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)sb_sm_count() * 16;
  if (blocks > cap) blocks = cap;
  cudaStream_t s = (cudaStream_t)stream;
  // Split-K with the tiles ADDED to C (TMA reduce-add) serves two ends.  Accuracy: the tensor core's
  // fp32 accumulator does not round to nearest, so a long chain of accumulations drifts (4e-5 at
  // K = 4096 in one pass); chains of at most 256 elements of K per part stay far below 1e-5 and the
  // additions between chains are ordinary fp32 additions.  Parallelism: a 512 x 512 output is four
  // tiles; with the splits it is spread over the whole GPU.  Needs a plain product (no bias / ReLU)
  // and whole 32-column chunks; C is first brought to beta * C (zero for beta == 0).
  int splits = 1;
  if (epilogue == 0 && N % 32 == 0 && 3 * K >= 512) {
    const int by_accuracy = (K + 255) / 256;
    const long long tiles = (long long)((M + 255) / 256) * ((N + 255) / 256);
    long long by_fill = tiles > 0 ? (sb_sm_count() / 2) / tiles : 1;                // one wave of CTA pairs
    if (by_fill > 8) by_fill = 8;             // every split adds a whole tile to C: more than a few cost more than they spread
    const int by_k = (3 * K) / 128 > 0 ? (3 * K) / 128 : 1;                          // at least two k-blocks of 64 per split
    long long want = by_accuracy > by_fill ? by_accuracy : by_fill;
    if (want > by_k) want = by_k;
    if (want > 128) want = 128;
    splits = (int)(want < 1 ? 1 : want);
  }
  const bool init_c = splits > 1 && beta != 1.0f;
  SB_CUDA(sb_launch(split3_kernel, dim3((int)blocks), dim3(256), 0, s, 1, ja, jb, init_c ? C : (float*)nullptr,
                    (long long)M * N, beta));
  SB_COUNT_LAUNCH();
  SB_CUDA(cudaGetLastError());
  if (splits > 1) {
    int used = 0;
    // `C` doubles as the partials pointer: every condition for adding into C holds here by construction
    // (fp32 output, no epilogue, aligned rows, whole chunks), so no partial is ever written.
    int rc = sb_umma_gemm_launch(a_trans, b_trans, alpha, a3, b3, 0.0f, C, M, N, 3 * K, SB_TF32, SB_F32, 0, nullptr, nullptr,
                                 nullptr, nullptr, s, splits, &used, nullptr, C);
    if (rc != SB_OK) return rc;
    if (used != 1) return sb_fail(SB_ERR_UNSUPPORTED, "internal: sb_matmul_f32x3 expected its splits to be added into C");
    return SB_OK;
  }
  return sb_umma_gemm_launch(a_trans, b_trans, alpha, a3, b3, beta, C, M, N, 3 * K, SB_TF32, SB_F32, epilogue, bias, nullptr,
                             nullptr, nullptr, s);
}

int sb_matmul_ex(int a_trans, int b_trans, float alpha, const void* A, const void* B, float beta,
                 void* C, int M, int N, int K, int in_dtype, int out_dtype, int epilogue,
                 const float* bias, const uint8_t* mask, const void* aux_in, void* aux_out,
                 void* stream) {
  if (M < 0 || N < 0 || K < 0) return sb_fail(SB_ERR_BAD_ARG, "sb_matmul: negative dimension (M=%d N=%d K=%d)", M, N, K);
  if (in_dtype != SB_F32 && in_dtype != SB_TF32 && in_dtype != SB_BF16 && in_dtype != SB_F16)
    return sb_fail(SB_ERR_BAD_ARG, "sb_matmul: unknown input dtype %d", in_dtype);
  if (out_dtype != SB_F32 && out_dtype != SB_BF16 && out_dtype != SB_F16 && out_dtype != SB_TF32)
    return sb_fail(SB_ERR_BAD_ARG, "sb_matmul: unknown output dtype %d", out_dtype);
  if (epilogue & ~ALL_FLAGS) return sb_fail(SB_ERR_BAD_ARG, "sb_matmul: unknown epilogue flag in 0x%x", epilogue);
  if (M == 0 || N == 0) return SB_OK;
  if (!C) return sb_fail(SB_ERR_BAD_ARG, "sb_matmul: C is null");
  if (K > 0 && (!A || !B)) return sb_fail(SB_ERR_BAD_ARG, "sb_matmul: A or B is null");
  if ((epilogue & SB_EPI_BIAS) && !bias) return sb_fail(SB_ERR_BAD_ARG, "sb_matmul: SB_EPI_BIAS without a bias pointer");
  if ((epilogue & SB_EPI_RELU_GRAD) && !aux_in) return sb_fail(SB_ERR_BAD_ARG, "sb_matmul: SB_EPI_RELU_GRAD without aux_in");
  if ((epilogue & SB_EPI_ARGMAX) && !aux_out) return sb_fail(SB_ERR_BAD_ARG, "sb_matmul: SB_EPI_ARGMAX without aux_out");
  if (epilogue & GATE_FLAGS) {
    if (N % 32 != 0) return sb_fail(SB_ERR_UNSUPPORTED, "sb_matmul: ReLU sign-bit epilogues need N %% 32 == 0 (N=%d)", N);
    if (in_dtype == SB_F32) return sb_fail(SB_ERR_UNSUPPORTED, "sb_matmul: ReLU sign-bit epilogues need a tensor-core input class");
    if (epilogue & HEAD_FLAGS) return sb_fail(SB_ERR_UNSUPPORTED, "sb_matmul: ReLU sign-bit epilogues cannot be combined with a row head");
    if ((epilogue & SB_EPI_RELU_MASK_OUT) && !aux_out) return sb_fail(SB_ERR_BAD_ARG, "sb_matmul: SB_EPI_RELU_MASK_OUT without aux_out");
    if ((epilogue & SB_EPI_RELU_GRAD_MASK) && (!aux_in || (epilogue & SB_EPI_RELU_GRAD)))
      return sb_fail(SB_ERR_BAD_ARG, "sb_matmul: SB_EPI_RELU_GRAD_MASK needs aux_in and excludes SB_EPI_RELU_GRAD");
  }
  if (epilogue & SB_EPI_COLSUM_OUT) {
    if (!aux_out) return sb_fail(SB_ERR_BAD_ARG, "sb_matmul: SB_EPI_COLSUM_OUT without aux_out");
    if (N % 32 != 0) return sb_fail(SB_ERR_UNSUPPORTED, "sb_matmul: SB_EPI_COLSUM_OUT needs N %% 32 == 0 (N=%d)", N);
    if (in_dtype == SB_F32) return sb_fail(SB_ERR_UNSUPPORTED, "sb_matmul: SB_EPI_COLSUM_OUT needs a tensor-core input class");
    if (epilogue & ~(SB_EPI_COLSUM_OUT | SB_EPI_RELU_GRAD_MASK))
      return sb_fail(SB_ERR_UNSUPPORTED, "sb_matmul: SB_EPI_COLSUM_OUT combines only with SB_EPI_RELU_GRAD_MASK");
    if (beta != 0.0f || alpha != 1.0f)
      return sb_fail(SB_ERR_UNSUPPORTED, "sb_matmul: SB_EPI_COLSUM_OUT needs alpha == 1 and beta == 0");
  }
  if (epilogue & SB_EPI_LN_L2) {
    if (in_dtype == SB_F32) return sb_fail(SB_ERR_UNSUPPORTED, "sb_matmul: SB_EPI_LN_L2 needs a tensor-core input class");
    if (alpha != 1.0f || beta != 0.0f || (epilogue & ~(SB_EPI_LN_L2 | SB_EPI_RELU)))
      return sb_fail(SB_ERR_UNSUPPORTED, "sb_matmul: SB_EPI_LN_L2 needs alpha == 1, beta == 0 and combines only with SB_EPI_RELU");
  }
  if (in_dtype == SB_F32 && out_dtype == SB_TF32) out_dtype = SB_F32;
  if ((epilogue & HEAD_FLAGS) && out_dtype != SB_F32)
    return sb_fail(SB_ERR_UNSUPPORTED, "sb_matmul: row heads write fp32 output only");
  if ((epilogue & HEAD_FLAGS) && (epilogue & SB_EPI_RELU_GRAD))
    return sb_fail(SB_ERR_UNSUPPORTED, "sb_matmul: a row head cannot be combined with SB_EPI_RELU_GRAD");
  if (reinterpret_cast<uintptr_t>(C) & 15) return sb_fail(SB_ERR_MISALIGNED, "sb_matmul: C must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;

  if (K == 0) {
    // Empty inner dimension: op(A) * op(B) is the zero matrix.
    if (epilogue != SB_EPI_NONE) return sb_fail(SB_ERR_UNSUPPORTED, "sb_matmul: K == 0 with an epilogue");
    return sb_scale_launch(C, (long long)M * N, beta, out_dtype, s);
  }

  if (in_dtype == SB_F32) {
    if (out_dtype != SB_F32) return sb_fail(SB_ERR_UNSUPPORTED, "sb_matmul: the fp32 path writes fp32 output only");
    if (epilogue & SB_EPI_RELU_GRAD) return sb_fail(SB_ERR_UNSUPPORTED, "sb_matmul: SB_EPI_RELU_GRAD needs a tensor-core input class");
    int rc = sb_sgemm_launch(a_trans, b_trans, alpha, (const float*)A, (const float*)B, beta, (float*)C,
                             M, N, K, epilogue & (SB_EPI_BIAS | SB_EPI_RELU), bias, s);
    if (rc != SB_OK) return rc;
    if (epilogue & HEAD_FLAGS) return run_heads_unfused((float*)C, M, N, legacy_head(epilogue, N, mask, aux_out), stream);
    return SB_OK;
  }

  if ((epilogue & HEAD_FLAGS) && !sb_umma_head_fits(N, -1)) {
    int rc = sb_umma_gemm_launch(a_trans, b_trans, alpha, A, B, beta, C, M, N, K, in_dtype, out_dtype,
                                 epilogue & ~HEAD_FLAGS, bias, nullptr, aux_in, nullptr, s);
    if (rc != SB_OK) return rc;
    return run_heads_unfused((float*)C, M, N, legacy_head(epilogue, N, mask, aux_out), stream);
  }
  return sb_umma_gemm_launch(a_trans, b_trans, alpha, A, B, beta, C, M, N, K, in_dtype, out_dtype,
                             epilogue, bias, mask, aux_in, aux_out, s);
}

int sb_matmul_head(int a_trans, int b_trans, float alpha, const void* A, const void* B, float beta,
                   float* C, int M, int N, int K, int in_dtype, int epilogue, const float* bias,
                   const sb_head_spec* head, void* stream) {
  if (!head) return sb_fail(SB_ERR_BAD_ARG, "sb_matmul_head: head is null");
  if (M < 0 || N < 0 || K <= 0) return sb_fail(SB_ERR_BAD_ARG, "sb_matmul_head: dimensions M=%d N=%d K=%d", M, N, K);
  if (epilogue & ~(SB_EPI_BIAS | SB_EPI_RELU))
    return sb_fail(SB_ERR_BAD_ARG, "sb_matmul_head: epilogue may hold SB_EPI_BIAS and SB_EPI_RELU (the head comes through head->flags)");
  if ((epilogue & SB_EPI_BIAS) && !bias) return sb_fail(SB_ERR_BAD_ARG, "sb_matmul_head: SB_EPI_BIAS without a bias pointer");
  if (in_dtype != SB_F32 && in_dtype != SB_TF32 && in_dtype != SB_BF16 && in_dtype != SB_F16)
    return sb_fail(SB_ERR_BAD_ARG, "sb_matmul_head: unknown input dtype %d", in_dtype);
  if (M == 0 || N == 0) return SB_OK;
  if (!A || !B || !C) return sb_fail(SB_ERR_BAD_ARG, "sb_matmul_head: null pointer");
  if (reinterpret_cast<uintptr_t>(C) & 15) return sb_fail(SB_ERR_MISALIGNED, "sb_matmul_head: C must be 16-byte aligned");
  SbRowHead h;
  h.n = N; h.flags = head->flags; h.prefix = head->prefix < 0 ? -1 : head->prefix; h.mask = head->mask;
  h.argmax_out = head->argmax_out; h.sample_out = head->sample_out; h.hash_out = head->hash_out;
  h.modulo = head->modulo; h.seed = head->seed; h.row_offset = head->row_offset; h.position = head->position;
  int rc = check_head("sb_matmul_head", h, N);
  if (rc != SB_OK) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  if (in_dtype == SB_F32) {
    rc = sb_sgemm_launch(a_trans, b_trans, alpha, (const float*)A, (const float*)B, beta, C, M, N, K, epilogue, bias, s);
    if (rc != SB_OK) return rc;
    return run_heads_unfused(C, M, N, h, stream);
  }
  if (h.flags == 0 || !sb_umma_head_fits(N, h.prefix)) {
    rc = sb_umma_gemm_launch(a_trans, b_trans, alpha, A, B, beta, C, M, N, K, in_dtype, SB_F32, epilogue, bias, nullptr,
                             nullptr, nullptr, s);
    if (rc != SB_OK) return rc;
    return run_heads_unfused(C, M, N, h, stream);
  }
  return sb_umma_gemm_launch(a_trans, b_trans, alpha, A, B, beta, C, M, N, K, in_dtype, SB_F32, epilogue | h.flags, bias,
                             nullptr, nullptr, nullptr, s, 1, nullptr, &h);
}

int sb_matmul_tf32(int a_trans, int b_trans, float alpha, const float* A, const float* B,
                   float beta, float* C, int M, int N, int K, void* stream) {
  return sb_matmul_ex(a_trans, b_trans, alpha, A, B, beta, C, M, N, K, SB_TF32, SB_F32, SB_EPI_NONE,
                      nullptr, nullptr, nullptr, nullptr, stream);
}

int sb_matmul_plan(int a_trans, int b_trans, int M, int N, int K, int in_dtype, int epilogue,
                   int* plan5) {
  (void)epilogue;
  if (!plan5) return sb_fail(SB_ERR_BAD_ARG, "sb_matmul_plan: null output");
  if (M <= 0 || N <= 0 || K <= 0) return sb_fail(SB_ERR_BAD_ARG, "sb_matmul_plan: dimensions must be positive");
  if (in_dtype != SB_TF32 && in_dtype != SB_BF16 && in_dtype != SB_F16)
    return sb_fail(SB_ERR_BAD_ARG, "sb_matmul_plan: tensor-core input classes only");
  return sb_umma_plan(a_trans, b_trans, M, N, K, in_dtype, sb_sm_count(), plan5);
}

}  // extern "C"
