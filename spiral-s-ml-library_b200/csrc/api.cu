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

extern "C" {

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
