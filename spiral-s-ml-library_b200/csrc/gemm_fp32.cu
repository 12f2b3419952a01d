// fp32-exact GEMM (FFMA, fp32 accumulate) for the 1e-5 accuracy class.
// The reference has no such mode (its only arithmetic is TF32,
// corecuda/wmma.spi:20); it exists because single-pass TF32 cannot meet a
// 1e-5 relative error.  Same contract as the tensor-core path:
// C <- alpha * op(A) * op(B) + beta * C, any M, N, K, no alignment demands.
#include "common.cuh"

namespace {

constexpr int F_BM = 64;
constexpr int F_BN = 64;
constexpr int F_BK = 16;
constexpr int F_THREADS = 256;

template <bool A_TRANS, bool B_TRANS>
__global__ void __launch_bounds__(F_THREADS)
sgemm_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, int M,
             int N, int K, float alpha, float beta, int epi, const float* __restrict__ bias) {
  __shared__ __align__(16) float As[F_BK][F_BM + 4];
  __shared__ __align__(16) float Bs[F_BK][F_BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15;   // column group
  const int ty = tid >> 4;   // row group
  const int m0 = blockIdx.y * F_BM;
  const int n0 = blockIdx.x * F_BN;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += F_BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + i * F_THREADS;  // 0..1023
      int m, k;
      if (A_TRANS) { k = e / F_BM; m = e % F_BM; } else { m = e / F_BK; k = e % F_BK; }
      const int gm = m0 + m, gk = k0 + k;
      float v = 0.f;
      if (gm < M && gk < K) v = A_TRANS ? A[(size_t)gk * M + gm] : A[(size_t)gm * K + gk];
      As[k][m] = v;
      int n, kk;
      if (B_TRANS) { n = e / F_BK; kk = e % F_BK; } else { kk = e / F_BN; n = e % F_BN; }
      const int gn = n0 + n, gk2 = k0 + kk;
      float w = 0.f;
      if (gn < N && gk2 < K) w = B_TRANS ? B[(size_t)gn * K + gk2] : B[(size_t)gk2 * N + gn];
      Bs[kk][n] = w;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < F_BK; ++k) {
      // one 16-byte shared-memory load per operand (rows are 272 bytes apart, a multiple of 16)
      const float4 av = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float4 bv = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
      const float a[4] = {av.x, av.y, av.z, av.w};
      const float b[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float v = alpha * acc[i][j];
      float* c = C + (size_t)gm * N + gn;
      if (beta != 0.f) v += beta * *c;
      if (epi & SB_EPI_BIAS) v += bias[gn];
      if (epi & SB_EPI_RELU) v = fmaxf(v, 0.f);
      *c = v;
    }
  }
}

}  // namespace

int sb_sgemm_launch(int a_trans, int b_trans, float alpha, const float* A, const float* B, float beta,
                    float* C, int M, int N, int K, int epi, const float* bias, cudaStream_t stream) {
  dim3 grid((N + F_BN - 1) / F_BN, (M + F_BM - 1) / F_BM);
  if (grid.y > 65535) return sb_fail(SB_ERR_TOO_LARGE, "fp32 GEMM: M too large for this launch shape");
  if (a_trans && b_trans)
    sgemm_kernel<true, true><<<grid, F_THREADS, 0, stream>>>(A, B, C, M, N, K, alpha, beta, epi, bias);
  else if (a_trans)
    sgemm_kernel<true, false><<<grid, F_THREADS, 0, stream>>>(A, B, C, M, N, K, alpha, beta, epi, bias);
  else if (b_trans)
    sgemm_kernel<false, true><<<grid, F_THREADS, 0, stream>>>(A, B, C, M, N, K, alpha, beta, epi, bias);
  else
    sgemm_kernel<false, false><<<grid, F_THREADS, 0, stream>>>(A, B, C, M, N, K, alpha, beta, epi, bias);
  SB_COUNT_LAUNCH();
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}
