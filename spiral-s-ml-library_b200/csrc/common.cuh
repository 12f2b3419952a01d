// Shared device/host helpers for the sm_100a kernels of libspiral_b200.
//
// Everything here is either a thin wrapper over one PTX instruction
// (mbarrier, TMA bulk-tensor copies, tcgen05 alloc/mma/commit/ld) or host-side
// error bookkeeping.  Every device-side wait is bounded in time: when the
// bound runs out the waiter records a code in a device status word and the
// kernel drains and returns instead of spinning forever.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <atomic>

#include "../../include/spiral_b200.h"

// ---------------------------------------------------------------------------
// Host-side error bookkeeping
// ---------------------------------------------------------------------------
void sb_set_error(const char* fmt, ...);
int sb_fail(int code, const char* fmt, ...);
int sb_check_cuda(cudaError_t e, const char* what);

#define SB_CUDA(call)                                                          \
  do {                                                                         \
    int _rc = sb_check_cuda((call), #call);                                    \
    if (_rc != SB_OK) return _rc;                                              \
  } while (0)

// Device status word (one per loaded library per device).  0 = healthy.
// Kernels record the first bounded wait that expired here.  The library is
// built as one translation unit, so the definition lives in this header.
__device__ int g_sb_status[4] = {0, 0, 0, 0};

enum SbWaitSite : int {
  SB_SITE_PRODUCER_EMPTY = 1,
  SB_SITE_MMA_FULL = 2,
  SB_SITE_MMA_TMEM_EMPTY = 3,
  SB_SITE_EPI_TMEM_FULL = 4,
  SB_SITE_MLP_WEIGHTS = 5,
  SB_SITE_MLP_ACT = 6,
  SB_SITE_MLP_ACC = 7,
  SB_SITE_DRAIN = 8,
};

// Launch accounting: every kernel launch of the library goes through
// SB_COUNT_LAUNCH so that a host can report how many kernels a region issued.
// The counter is atomic: entry points may be called from several host threads.
void sb_count_launch();
#define SB_COUNT_LAUNCH() sb_count_launch()

// Multiprocessor count of the current device (cached per device); SB_NUM_SMS_FALLBACK when no
// device can be asked (planning calls on a host without a GPU).
int sb_sm_count();

// Optional GEMM profiling: when enabled, the tensor-core GEMM launcher records
// a CUDA event pair around each launch on the launching stream.
void sb_prof_before(cudaStream_t s);
void sb_prof_after(cudaStream_t s, double flops);

// The tensor-core GEMM launcher (gemm_umma.cu); every argument is validated there.  `head`
// describes the row head when `epi` holds a head flag (null: the legacy form -- byte mask in
// `mask`, arg-max indices to `aux_out`).  Split-K: by default split s writes its own partial at
// C + s * M * N.  With `split_partials` (room for splits * M * N floats) the launcher chooses: when C
// can take TMA boxes every split ADDS its tile to the one fp32 matrix C (which the caller has zeroed)
// through TMA reduce-add stores and *splits_used comes back as 1; otherwise the partials go to
// `split_partials`, *splits_used tells how many, and the caller reduces them into C.
// `peer_out` (see SbPeerOut; the caller has checked sb_umma_peer_out_ok): every tile, split or not, is
// added to the copy of C on the rank that owns its rows -- the reduce-scatter half of a gradient
// all-reduce done by the GEMM's own TMA reduce-add stores over peer memory.  C is ignored then.
struct SbRowHead;
// Copies of the output matrix on several ranks (data-parallel weight gradients): c[r] is rank r's
// copy of C, the same [M, N] fp32 matrix in that rank's memory (its own for this rank, peer pointers
// for the others).  Rows [r * M / n, (r + 1) * M / n) of the product are ADDED to c[r] only.
struct SbPeerOut {
  int n;
  void* c[8];
};
// True when a GEMM with an [M, N] fp32 output can add its rows to n ranks' copies (sb_umma_gemm_launch
// with peer_out): whole 128-row blocks per rank, at most 8 ranks, rows that can leave as TMA boxes.
bool sb_umma_peer_out_ok(int M, int N, int n);
int sb_umma_gemm_launch(int a_trans, int b_trans, float alpha, const void* A, const void* B,
                        float beta, void* C, int M, int N, int K, int in_dtype, int out_dtype,
                        int epi, const float* bias, const uint8_t* mask, const void* aux_in,
                        void* aux_out, cudaStream_t stream, int splits = 1, int* splits_used = nullptr,
                        const SbRowHead* head = nullptr, void* split_partials = nullptr,
                        const SbPeerOut* peer_out = nullptr);
// True when a row head over N columns (legal columns j < prefix when prefix >= 0) runs inside the GEMM.
bool sb_umma_head_fits(int N, int prefix);

static inline int sb_dtype_size(int dt) {
  switch (dt) {
    case SB_F32: case SB_TF32: return 4;
    case SB_BF16: case SB_F16: return 2;
    default: return 0;
  }
}

constexpr int SB_NUM_SMS_FALLBACK = 148;

#ifdef __CUDACC__

// Programmatic dependent launch.  A kernel launched through sb_launch() may
// become resident while the kernel before it on the stream is still draining:
// its CTAs set themselves up (barriers, tensor memory, descriptor prefetch) and
// then block in sb_grid_dependency_wait() until the earlier grid has completed
// and its writes are visible.  Every kernel launched this way must call
// sb_grid_dependency_wait() before its first access to global memory, and
// calls sb_grid_dependents_launch() right after it so that its own successor
// can move up the same way.  SB_NO_PDL=1 in the environment turns the
// attribute off (plain stream order); the device calls are then no-ops.
__device__ __forceinline__ void sb_grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void sb_grid_dependents_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool sb_pdl_enabled();

template <typename... KArgs, typename... Args>
cudaError_t sb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                      int cluster_x, Args... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = (unsigned)cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (sb_pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Wall-clock limit of one device-side wait (nanoseconds of %globaltimer).
constexpr unsigned long long SB_WAIT_LIMIT_NS = 400ull * 1000ull * 1000ull;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ------------------------------- mbarrier ----------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// Makes generic-proxy writes to shared memory visible to the async proxy
// (TMA, tcgen05.mma operand reads).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait on an mbarrier phase.  `abort_flag` lives in shared memory and
// is shared by every role of the CTA: the first waiter whose time runs out
// sets it (and the device status word); every other waiter polls it, so one
// expired wait drains the whole CTA in bounded time.  Returns false when the
// caller must stop issuing work and fall through to the teardown.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                            int site) {
#pragma unroll 1
  for (int i = 0; i < 2048; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  const unsigned long long t0 = global_timer_ns();
#pragma unroll 1
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag != 0) return false;
    if (global_timer_ns() - t0 > SB_WAIT_LIMIT_NS) {
      *abort_flag = 1;
      atomicCAS(&g_sb_status[0], 0, site);
      atomicAdd(&g_sb_status[1], 1);
      return false;
    }
  }
}

// The common case (phase already complete, or completing within one try_wait)
// costs a single instruction in the caller; everything else is out of line so
// that the single-thread issue loops stay short.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int site) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag, site);
}

// --------------------------------- TMA --------------------------------------
// Plain (non-multicast) 2-D tiled bulk-tensor load into this CTA's shared
// memory; completion is reported to `bar` as transaction bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* tmap, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// 16 bytes from global to shared memory without passing through registers (cp.async); the copies
// of a thread complete in the order of their commit groups.
__device__ __forceinline__ void cp_async_16(uint32_t dst_smem, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
// The same for a 3-D tensor (x innermost).
__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const CUtensorMap* tmap, int x, int y, int z,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}
// 2-D tiled bulk-tensor store from this CTA's shared memory; elements outside
// the tensor are clipped.  Completion is tracked by the issuing thread's
// bulk async-group.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tmap, uint32_t src_smem, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
               ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(src_smem)
               : "memory");
}
// The same box added to the tensor in global memory (fp32 adds done by the memory system, so boxes
// from different CTAs may target the same elements; the order of the additions is not fixed).
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* tmap, uint32_t src_smem, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];"
               ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(src_smem)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Waits until at most N of this thread's bulk groups still read shared memory.
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// ------------------------------- tcgen05 ------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrives once on `bar` when every tcgen05.mma issued so far by this thread
// has finished reading shared memory and writing tensor memory.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]; `accumulate == 0` overwrites D.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
      "}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Variants taking each 64-bit shared-memory descriptor as (lo, hi) words: the
// hi word is constant per operand and the lo word (start address) is the only
// part that moves, so the issuing thread does 32-bit adds only.
template <bool PAIR, bool TF32>
__device__ __forceinline__ void umma_issue(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                           uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  if (PAIR) {
    if (TF32)
      asm volatile(
          "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
          "setp.ne.b32 p, %6, 0;\n\ttcgen05.mma.cta_group::2.kind::tf32 [%0], da, db, %5, p;\n\t}"
          ::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
    else
      asm volatile(
          "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
          "setp.ne.b32 p, %6, 0;\n\ttcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n\t}"
          ::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
  } else {
    if (TF32)
      asm volatile(
          "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
          "setp.ne.b32 p, %6, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], da, db, %5, p;\n\t}"
          ::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
    else
      asm volatile(
          "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
          "setp.ne.b32 p, %6, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
          ::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
  }
}

// 32 lanes x 32-bit, 16 / 32 consecutive columns: thread t of the warp gets
// TMEM lane (lane_base + t), columns [col, col + n).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ------------------ CTA pairs (cluster of 2, cta_group::2) ------------------
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Cluster-wide barrier: every thread of every CTA of the cluster arrives, then waits.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address, in the shared::cluster window, of the same shared-memory location in CTA `rank`.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load issued by either CTA of a pair: data lands in the issuing CTA's shared
// memory, the transaction bytes are reported to `bar`, which may live in the
// pair's leader CTA (a shared::cluster address).  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst_smem, const CUtensorMap* tmap, int x, int y,
                                                 uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(bar_cluster_addr)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
// Commit of the pair's MMAs: arrives on the barrier at this shared-memory offset
// in every CTA named by `cta_mask` (bit r = CTA rank r of the cluster).
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"(cta_mask)
      : "memory");
}
// M = 256 MMA of a CTA pair: each CTA supplies its 128 rows of A and half of the
// N columns of B from the same shared-memory offsets, and keeps its 128 rows of D.
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                              uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_tf32_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t"
      "}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// ---------------------- UMMA descriptors (sm_100) ---------------------------
// Shared-memory matrix descriptor, 128-byte swizzle.  Fields (bit ranges):
//   [0,14)  start address >> 4       [16,30) leading byte offset >> 4
//   [32,46) stride byte offset >> 4  [46,48) version = 1
//   [61,64) layout type: 2 = SWIZZLE_128B (16-byte chunks XORed with the row
//           index modulo 8); 1 = SWIZZLE_128B with 32-byte chunks XORed with
//           the row index modulo 4, the only layout tcgen05 accepts for
//           MN-major 32-bit (TF32) operands.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes, uint32_t layout_type) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(layout_type & 7u) << 61;
  return d;
}

// 128-byte swizzle as TMA and tcgen05 apply it: the 16-byte chunk index
// (address bits [4,7)) is XORed with the row-in-atom index (bits [7,10)).
// `row_stride` is 128 bytes; atoms of 8 rows are 1024 bytes and the tile base
// must be 1024-byte aligned.
__device__ __forceinline__ uint32_t swizzle128_offset(uint32_t row, uint32_t byte_in_row) {
  const uint32_t chunk = (byte_in_row >> 4) ^ (row & 7u);
  return row * 128u + (chunk << 4) + (byte_in_row & 15u);
}

#endif  // __CUDACC__

// Instruction descriptor for tcgen05.mma kind::f16 / kind::tf32 with an fp32
// accumulator.  Fields: [4,6) D format (1 = f32); [7,10) A format; [10,13) B
// format (0 = f16, 1 = bf16, 2 = tf32); bit 15 / 16 = A / B is MN-major;
// [17,23) N >> 3; [24,29) M >> 4.
static inline uint32_t sb_umma_idesc(int in_dtype, int a_mn_major, int b_mn_major, int m, int n) {
  uint32_t fmt = in_dtype == SB_F16 ? 0u : (in_dtype == SB_BF16 ? 1u : 2u);
  uint32_t d = 0;
  d |= 1u << 4;
  d |= fmt << 7;
  d |= fmt << 10;
  d |= (a_mn_major ? 1u : 0u) << 15;
  d |= (b_mn_major ? 1u : 0u) << 16;
  d |= (static_cast<uint32_t>(n) >> 3) << 17;
  d |= (static_cast<uint32_t>(m) >> 4) << 24;
  return d;
}
