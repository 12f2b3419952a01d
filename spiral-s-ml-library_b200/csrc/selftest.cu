// Self-test of the bounded device-side wait: a tiny kernel waits on an mbarrier
// that nothing ever arrives on.  The wait gives up after SB_WAIT_LIMIT_NS, records
// the wait site in the device status word, raises the CTA's abort flag (which
// releases the second waiter at once) and the kernel returns normally -- the same
// path every kernel of the library takes if one of its waits should ever expire.
// No trap, no device assert, no unbounded loop: the context stays usable.
#include "common.cuh"

namespace {

__global__ void wait_selftest_kernel(int* out) {
  __shared__ __align__(8) uint64_t never_signalled;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&never_signalled), 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0 && warp < 2) {
    const unsigned long long t0 = global_timer_ns();
    const bool ok = mbar_wait(smem_u32(&never_signalled), 0u, &abort_flag, SB_SITE_DRAIN);
    out[warp] = ok ? 1 : 0;
    out[2 + warp] = (int)((global_timer_ns() - t0) / 1000000ull);   // milliseconds waited
  }
  __syncthreads();
  if (threadIdx.x == 0) out[4] = abort_flag;
}

}  // namespace

extern "C" int sb_selftest_bounded_wait(int* result5) {
  if (!result5) return sb_fail(SB_ERR_BAD_ARG, "sb_selftest_bounded_wait: null output");
  int* dev = nullptr;
  SB_CUDA(cudaMalloc(&dev, 5 * sizeof(int)));
  cudaMemset(dev, 0xff, 5 * sizeof(int));
  wait_selftest_kernel<<<1, 64>>>(dev);
  SB_COUNT_LAUNCH();
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpy(result5, dev, 5 * sizeof(int), cudaMemcpyDeviceToHost);
  cudaFree(dev);
  return sb_check_cuda(e, "sb_selftest_bounded_wait");
}
