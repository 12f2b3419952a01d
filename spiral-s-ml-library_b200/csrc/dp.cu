// Data-parallel weight update over peer memory: gradient reduction, SGD and the
// redistribution of the new weights in ONE kernel, instead of a library
// all-reduce followed by an update kernel on every rank.
//
// Every rank (one process per GPU) holds the whole model: fp32 master
// parameters, the compute copy and an fp32 gradient buffer of its batch shard.
// The flat parameter vector is cut into world_size contiguous slices.  Rank r
//   1. waits until every rank's gradients are complete (flag barrier),
//   2. for its own slice reads the gradients of all ranks through peer
//      pointers (NVLink loads, summed in rank order: every element is reduced by
//      exactly one rank, so all ranks end with bit-identical weights),
//   3. applies the SGD step to its slice of the master parameters and
//   4. stores the new master values and their compute copies into every rank's
//      buffers (NVLink stores),
// and a second flag barrier, run by the CTA that finishes last, closes the step:
// after it every rank's weights are complete and nobody still reads anybody's
// gradients.  One launch per step.  Bytes crossing NVLink
// per rank and step: (W-1)/W of the gradient vector in, (W-1)/W of 6 (or 8)
// bytes per parameter out -- the same as a ring all-reduce moves, without its
// 2(W-1) latency steps.
//
// The reference has no multi-GPU path (single device, corecuda/base.spi:7);
// this follows the benchmark's data-parallel training configurations.
//
// Waits: a rank spins on flags in its OWN memory that peers write; every spin
// is bounded by `timeout_ms` of %globaltimer.  When it expires the kernel
// records it in the flag block's status word, skips the update and returns:
// no trap, the context stays usable, the host reads the word with
// sb_dp_status.  Two ranks never share a GPU, so the waiting kernels of
// different ranks always run at the same time.
#include "common.cuh"

namespace {

constexpr int DP_MAX_WORLD = 16;
constexpr int DP_MAX_RANGES = 16;
constexpr int DP_MAX_SEGMENTS = 34;    // element ranges one launch may cover (weights and bias of up to 17 layers)
constexpr int DP_THREADS = 128;
constexpr int DP_STATUS_WORD = 16;     // index of the status word in a flag block
constexpr int DP_COUNTER_WORD = 17;    // CTAs of the running update that have finished their stores
constexpr int DP_FLAG_WORDS = 32;      // words per flag block: [0, 16) peer epochs, [16] status, [17] counter

struct DpPeers {
  const float* grads[DP_MAX_WORLD];
  float* params[DP_MAX_WORLD];
  void* compute[DP_MAX_WORLD];
  unsigned int* flags[DP_MAX_WORLD];
  // With a sharded master only these element ranges of the master parameters are stored to every
  // rank (the biases, which the forward pass reads in fp32); elsewhere only the owner's are.
  long long rep_begin[DP_MAX_RANGES];
  long long rep_end[DP_MAX_RANGES];
  int n_ranges;
  int shard_master;   // 0: every rank receives the whole master vector
  int gather_only;    // 1: no gradients, no step: the owners' master slices are copied to every rank
};

// The element ranges one launch covers.  Every range is cut into world_size slices of whole
// 4-element vectors of its own; rank r reduces, updates and redistributes slice r of every range.
// reduced[s] != 0: the gradients of range s were already summed into the owners' buffers by the
// backward pass (its weight-gradient GEMMs add their tiles to the owner's copy over peer memory), so
// the owner reads only its own buffer -- and zeroes what it has read, ready for the next step's tiles.
struct DpSegments {
  int n;
  long long begin[DP_MAX_SEGMENTS];
  long long end[DP_MAX_SEGMENTS];
  unsigned char reduced[DP_MAX_SEGMENTS];
};

__device__ __forceinline__ void dp_slice_of(long long begin, long long end, int world, int rank, long long& v_begin,
                                            long long& v_end) {
  const long long nvec = (end - begin) >> 2;
  const long long per = (nvec + world - 1) / world;
  v_begin = (begin >> 2) + min(nvec, per * rank);
  v_end = (begin >> 2) + min(nvec, per * rank + per);
}

__device__ __forceinline__ float4 ld_volatile_f4(const float* p) {
  float4 v;
  asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ unsigned int ld_volatile_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
// Release / acquire fence at system scope: orders without the full sequential-consistency cost of
// __threadfence_system().
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ void st_volatile_u32(unsigned int* p, unsigned int v) {
  asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Thread t < world publishes `epoch` in rank t's flag block (slot = this rank).
__device__ __forceinline__ void dp_signal(const DpPeers& peers, int world, int rank, unsigned int epoch) {
  if ((int)threadIdx.x < world) {
    fence_acq_rel_sys();
    st_volatile_u32(peers.flags[threadIdx.x] + rank, epoch);
  }
}

// Thread t < world waits until rank t has published an epoch >= `epoch` in this
// rank's flag block.  Returns false (and records it) when the wait expired or a
// wait of this rank expired before.
__device__ __forceinline__ bool dp_wait(unsigned int* my_flags, int world, unsigned int epoch,
                                        unsigned long long timeout_ns) {
  __shared__ int ok_shared;
  if (threadIdx.x == 0) ok_shared = 1;
  __syncthreads();
  if ((int)threadIdx.x < world) {
    const unsigned long long t0 = global_timer_ns();
    bool ok = true;
    unsigned int polls = 0;
    // Epochs only grow; the signed difference tolerates wrap-around.  The clock and the status word
    // are looked at every 16th poll only: the common case is a flag that arrives within microseconds.
    while ((int)(ld_volatile_u32(my_flags + threadIdx.x) - epoch) < 0) {
      if ((++polls & 15u) == 0u &&
          (global_timer_ns() - t0 > timeout_ns || ld_volatile_u32(my_flags + DP_STATUS_WORD) != 0u)) {
        ok = false;
        break;
      }
      __nanosleep(20);
    }
    if (!ok) {
      atomicCAS(my_flags + DP_STATUS_WORD, 0u, 0x100u + threadIdx.x);   // 0x100 + the rank that never arrived
      ok_shared = 0;
    }
    fence_acq_rel_sys();
  }
  __syncthreads();
  return ok_shared != 0;
}

__device__ __forceinline__ void store_compute4(void* base, long long i, float4 w, int dt) {
  if (dt == SB_BF16) {
    uint2 o;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o.x) : "f"(w.y), "f"(w.x));
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o.y) : "f"(w.w), "f"(w.z));
    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(base) + i) = o;
  } else if (dt == SB_F16) {
    uint2 o;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(o.x) : "f"(w.y), "f"(w.x));
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(o.y) : "f"(w.w), "f"(w.z));
    *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(base) + i) = o;
  } else {
    if (dt == SB_TF32) {
      float* e = reinterpret_cast<float*>(&w);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        uint32_t u = __float_as_uint(e[t]);
        if ((u & 0x7f800000u) != 0x7f800000u) { u += 0x0fffu + ((u >> 13) & 1u); u &= 0xffffe000u; }
        e[t] = __uint_as_float(u);
      }
    }
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + i) = w;
  }
}

// One launch per step and rank.  `n` is a multiple of 4; slices are whole
// 4-element vectors.  barriers = 0 skips both barriers (single rank, or a
// caller that ordered the ranks by other means).
__global__ void __launch_bounds__(DP_THREADS)
dp_update_kernel(DpPeers peers, DpSegments segs, int world, int rank, unsigned int epoch, float lr,
                 int dt, unsigned long long timeout_ns, int barriers) {
  unsigned int* my_flags = peers.flags[rank];
  __shared__ int is_last;
  if (barriers) {
    if (blockIdx.x == 0) dp_signal(peers, world, rank, epoch);
    if (!dp_wait(my_flags, world, epoch, timeout_ns)) return;
  } else if (ld_volatile_u32(my_flags + DP_STATUS_WORD) != 0u) {
    return;
  }
  long long total = 0;                     // vectors of this rank over all ranges
  for (int s = 0; s < segs.n; ++s) {
    long long b, e;
    dp_slice_of(segs.begin[s], segs.end[s], world, rank, b, e);
    total += e - b;
  }
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += step) {
    // which range, and which vector of this rank's slice of it
    long long local = t, v = 0;
    bool reduced = false;
    for (int s = 0; s < segs.n; ++s) {
      long long b, e;
      dp_slice_of(segs.begin[s], segs.end[s], world, rank, b, e);
      if (local < e - b) {
        v = b + local;
        reduced = segs.reduced[s] != 0;
        break;
      }
      local -= e - b;
    }
    const long long i = v << 2;
    float4 w = *reinterpret_cast<const float4*>(peers.params[rank] + i);
    bool master_everywhere = peers.shard_master == 0;
    if (!peers.gather_only && reduced) {
      // The sum over ranks is already in this rank's buffer (added there tile by tile by every rank's
      // weight-gradient GEMM); read it, and leave zeros for the next step's tiles.
      float* mine = const_cast<float*>(peers.grads[rank]) + i;
      const float4 s4 = ld_volatile_f4(mine);
      *reinterpret_cast<float4*>(mine) = make_float4(0.f, 0.f, 0.f, 0.f);
      w.x -= lr * s4.x; w.y -= lr * s4.y; w.z -= lr * s4.z; w.w -= lr * s4.w;
      if (!master_everywhere)
        for (int k = 0; k < peers.n_ranges; ++k)
          if (i >= peers.rep_begin[k] && i < peers.rep_end[k]) master_everywhere = true;
    } else if (!peers.gather_only) {
      // Eight loads in flight before the first add (two rounds for more than eight ranks): a CTA of
      // this kernel must fit beside a resident GEMM CTA, which leaves it some 90 registers a thread.
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int r0 = 0; r0 < DP_MAX_WORLD; r0 += 8) {
        if (r0 < world) {
          float4 g[8];
#pragma unroll
          for (int r = 0; r < 8; ++r)
            if (r0 + r < world) g[r] = ld_volatile_f4(peers.grads[r0 + r] + i);
#pragma unroll
          for (int r = 0; r < 8; ++r)
            if (r0 + r < world) { s.x += g[r].x; s.y += g[r].y; s.z += g[r].z; s.w += g[r].w; }
        }
      }
      w.x -= lr * s.x; w.y -= lr * s.y; w.z -= lr * s.z; w.w -= lr * s.w;
      if (!master_everywhere)
        for (int k = 0; k < peers.n_ranges; ++k)     // ranges are whole vectors (64-element aligned segments)
          if (i >= peers.rep_begin[k] && i < peers.rep_end[k]) master_everywhere = true;
    } else {
      master_everywhere = true;
    }
#pragma unroll
    for (int r = 0; r < DP_MAX_WORLD; ++r)
      if (r < world) {
        if (master_everywhere || r == rank) *reinterpret_cast<float4*>(peers.params[r] + i) = w;
        if (peers.compute[r]) store_compute4(peers.compute[r], i, w, dt);
      }
  }
  // Closing barrier.  Every CTA releases its stores at device scope and counts itself; the CTA that
  // arrives last has thereby observed all of them, and its system-wide fences (one per signalling
  // thread, in dp_signal) order them before the flags it publishes.  A system-wide fence in every
  // thread, or even in every CTA, costs more than the update itself.
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int before = atomicAdd(my_flags + DP_COUNTER_WORD, 1u);
    __threadfence();
    is_last = before == gridDim.x - 1u ? 1 : 0;
  }
  __syncthreads();
  if (!is_last) return;
  if (threadIdx.x == 0) st_volatile_u32(my_flags + DP_COUNTER_WORD, 0u);   // ready for the next launch
  if (barriers) {
    dp_signal(peers, world, rank, epoch + 1u);
    dp_wait(my_flags, world, epoch + 1u, timeout_ns);
  }
}

}  // namespace

extern "C" {

int sb_ipc_export(void* dev_ptr, void* handle64) {
  if (!dev_ptr || !handle64) return sb_fail(SB_ERR_BAD_ARG, "sb_ipc_export: null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the C ABI promises 64-byte handles");
  cudaIpcMemHandle_t h;
  SB_CUDA(cudaIpcGetMemHandle(&h, dev_ptr));
  memcpy(handle64, &h, sizeof(h));
  return SB_OK;
}

int sb_ipc_open(const void* handle64, void** dev_ptr) {
  if (!handle64 || !dev_ptr) return sb_fail(SB_ERR_BAD_ARG, "sb_ipc_open: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  SB_CUDA(cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return SB_OK;
}

int sb_ipc_close(void* dev_ptr) {
  if (!dev_ptr) return SB_OK;
  SB_CUDA(cudaIpcCloseMemHandle(dev_ptr));
  return SB_OK;
}

int sb_dp_flag_bytes(void) { return DP_FLAG_WORDS * (int)sizeof(unsigned int); }

int sb_dp_slice(long long begin, long long end, int world_size, int rank, long long* begin_end) {
  if (!begin_end) return sb_fail(SB_ERR_BAD_ARG, "sb_dp_slice: null output");
  if (begin < 0 || end < begin || begin % 4 != 0 || end % 4 != 0)
    return sb_fail(SB_ERR_BAD_ARG, "sb_dp_slice: [begin, end) must be whole 4-element vectors");
  if (world_size < 1 || world_size > DP_MAX_WORLD || rank < 0 || rank >= world_size)
    return sb_fail(SB_ERR_BAD_ARG, "sb_dp_slice: rank %d of world size %d (at most %d ranks)", rank, world_size, DP_MAX_WORLD);
  const long long nvec = (end - begin) >> 2;
  const long long per = (nvec + world_size - 1) / world_size;
  long long b = per * rank, e = b + per;
  if (b > nvec) b = nvec;
  if (e > nvec) e = nvec;
  begin_end[0] = begin + (b << 2);
  begin_end[1] = begin + (e << 2);
  return SB_OK;
}

int sb_dp_sgd_update_segments(int world_size, int rank, const float* const* grads, float* const* params,
                              void* const* w_compute, void* const* flags, unsigned int epoch, int n_segments,
                              const long long* segments, const int* reduced, float lr, int compute_dtype, int mode,
                              const long long* replicate, int n_replicate, int max_blocks, int timeout_ms, int barriers,
                              void* stream) {
  if (world_size < 1 || world_size > DP_MAX_WORLD || rank < 0 || rank >= world_size)
    return sb_fail(SB_ERR_BAD_ARG, "sb_dp_sgd_update: rank %d of world size %d (at most %d ranks)", rank, world_size, DP_MAX_WORLD);
  if (n_segments < 1 || n_segments > DP_MAX_SEGMENTS || !segments)
    return sb_fail(SB_ERR_BAD_ARG, "sb_dp_sgd_update: between 1 and %d element ranges", DP_MAX_SEGMENTS);
  if (max_blocks < 0) return sb_fail(SB_ERR_BAD_ARG, "sb_dp_sgd_update: negative max_blocks");
  if (mode != SB_DP_REPLICATED && mode != SB_DP_SHARDED_MASTER && mode != SB_DP_GATHER_MASTER)
    return sb_fail(SB_ERR_BAD_ARG, "sb_dp_sgd_update: unknown mode %d", mode);
  if ((!grads && mode != SB_DP_GATHER_MASTER) || !params || !flags) return sb_fail(SB_ERR_BAD_ARG, "sb_dp_sgd_update: null pointer table");
  if (n_replicate < 0 || n_replicate > DP_MAX_RANGES || (n_replicate > 0 && !replicate))
    return sb_fail(SB_ERR_BAD_ARG, "sb_dp_sgd_update: between 0 and %d replicated ranges", DP_MAX_RANGES);
  if (timeout_ms < 1 || timeout_ms > 60000) return sb_fail(SB_ERR_BAD_ARG, "sb_dp_sgd_update: timeout_ms must be in [1, 60000]");
  if (compute_dtype != SB_F32 && compute_dtype != SB_TF32 && compute_dtype != SB_BF16 && compute_dtype != SB_F16)
    return sb_fail(SB_ERR_BAD_ARG, "sb_dp_sgd_update: unknown compute dtype %d", compute_dtype);
  DpSegments segs;
  memset(&segs, 0, sizeof(segs));
  segs.n = n_segments;
  long long slice_vecs = 0;
  for (int k = 0; k < n_segments; ++k) {
    const long long begin = segments[2 * k], end = segments[2 * k + 1];
    if (begin < 0 || end < begin || begin % 4 != 0 || end % 4 != 0)
      return sb_fail(SB_ERR_BAD_ARG, "sb_dp_sgd_update: range %d must be [begin, end) in whole 4-element vectors", k);
    segs.begin[k] = begin;
    segs.end[k] = end;
    segs.reduced[k] = (reduced && reduced[k]) ? 1 : 0;
    slice_vecs += (((end - begin) >> 2) + world_size - 1) / world_size;
  }
  DpPeers peers;
  memset(&peers, 0, sizeof(peers));
  for (int r = 0; r < world_size; ++r) {
    const float* gr = mode == SB_DP_GATHER_MASTER ? params[r] : grads[r];
    if (!gr || !params[r] || !flags[r]) return sb_fail(SB_ERR_BAD_ARG, "sb_dp_sgd_update: null buffer of rank %d", r);
    if ((reinterpret_cast<uintptr_t>(gr) | reinterpret_cast<uintptr_t>(params[r])) & 15)
      return sb_fail(SB_ERR_MISALIGNED, "sb_dp_sgd_update: buffers of rank %d must be 16-byte aligned", r);
    if (w_compute && w_compute[r] && (reinterpret_cast<uintptr_t>(w_compute[r]) & 15))
      return sb_fail(SB_ERR_MISALIGNED, "sb_dp_sgd_update: compute copy of rank %d must be 16-byte aligned", r);
    peers.grads[r] = gr;
    peers.params[r] = params[r];
    peers.compute[r] = w_compute ? w_compute[r] : nullptr;
    peers.flags[r] = reinterpret_cast<unsigned int*>(flags[r]);
  }
  peers.shard_master = mode == SB_DP_SHARDED_MASTER ? 1 : 0;
  peers.gather_only = mode == SB_DP_GATHER_MASTER ? 1 : 0;
  peers.n_ranges = n_replicate;
  for (int k = 0; k < n_replicate; ++k) {
    peers.rep_begin[k] = replicate[2 * k];
    peers.rep_end[k] = replicate[2 * k + 1];
    if (peers.rep_begin[k] % 4 != 0 || peers.rep_end[k] % 4 != 0 || peers.rep_begin[k] > peers.rep_end[k])
      return sb_fail(SB_ERR_BAD_ARG, "sb_dp_sgd_update: replicated range %d must be [begin, end) in whole 4-element vectors", k);
  }
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned long long timeout_ns = (unsigned long long)timeout_ms * 1000000ull;
  long long blocks = (slice_vecs + DP_THREADS - 1) / DP_THREADS;
  if (blocks < 1) blocks = 1;
  const long long cap = max_blocks > 0 ? max_blocks : (long long)sb_sm_count() * 8;
  if (blocks > cap) blocks = cap;
  // A plain launch (no programmatic dependent launch): the first thing this kernel does is to tell
  // its peers that the gradients of this rank -- the work of the kernels before it -- are complete.
  dp_update_kernel<<<(int)blocks, DP_THREADS, 0, s>>>(peers, segs, world_size, rank, epoch, lr, compute_dtype, timeout_ns,
                                                      barriers ? 1 : 0);
  SB_COUNT_LAUNCH();
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

int sb_dp_sgd_update(int world_size, int rank, const float* const* grads, float* const* params,
                     void* const* w_compute, void* const* flags, unsigned int epoch, long long begin, long long end,
                     float lr, int compute_dtype, int mode, const long long* replicate, int n_replicate,
                     int max_blocks, int timeout_ms, int barriers, void* stream) {
  const long long seg[2] = {begin, end};
  return sb_dp_sgd_update_segments(world_size, rank, grads, params, w_compute, flags, epoch, 1, seg, nullptr, lr,
                                   compute_dtype, mode, replicate, n_replicate, max_blocks, timeout_ms, barriers, stream);
}

int sb_dp_status(const void* flags, int* status) {
  if (!flags || !status) return sb_fail(SB_ERR_BAD_ARG, "sb_dp_status: null pointer");
  unsigned int v = 0;
  SB_CUDA(cudaMemcpy(&v, reinterpret_cast<const unsigned int*>(flags) + DP_STATUS_WORD, sizeof(v), cudaMemcpyDeviceToHost));
  *status = (int)v;
  return SB_OK;
}

}  // extern "C"
