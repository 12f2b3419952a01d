// Tensor-core GEMM for sm_100a: C <- alpha * op(A) * op(B) + beta * C with a
// fused epilogue.  Replaces matmul_tf32_template (ml/matmul/kernel.spi:25-240,
// nvcuda::wmma m16n16k8 TF32 with one-deep cuda::memcpy_async prefetch).
//
// Structure of one CTA (352 threads = 11 warps, persistent over output tiles):
//   warp 0, lane 0 : TMA producer of A.  Per k-block it arms full[stage] with the
//                    stage's byte count and issues plain 2-D tiled TMA loads
//                    (128-byte swizzle) of the A tile; a stage holds one or two
//                    128-byte sub-blocks of K per operand.
//   warp 10, lane 0: TMA producer of B (the same loop, the B tile's loads).
//   warp 1, lane 0 : MMA issuer.  Waits full[stage], issues 4 or 8 tcgen05.mma
//                    (M=128, or 256 for a CTA pair; N=block_n; 32 bytes of K
//                    each) on shared-memory descriptors, commits to
//                    empty[stage]; after the last k-block commits to
//                    tmem_full[acc].  Warp 1 also owns the TMEM allocation.
//   warps 2..9     : epilogue, two warps per TMEM lane quadrant taking alternate
//                    32-column chunks (or chunk pairs).  Wait tmem_full[acc],
//                    read the fp32 accumulator from TMEM (tcgen05.ld, one output
//                    row per thread), apply alpha/beta/bias/ReLU/row head, store
//                    through a swizzled shared-memory box and a TMA store,
//                    arrive on tmem_empty[acc].  Two accumulators in TMEM let
//                    the epilogue of tile i overlap the main loop of tile i+1.
//
// Operand layouts.  "K-major" = the K index is contiguous in global memory
// (A stored [M,K]; B stored [N,K]); "MN-major" = the M or N index is contiguous
// (A stored [K,M]; B stored [K,N]).  Either way one stage holds 128 bytes of K
// (64 16-bit or 32 32-bit elements) per row for K-major, or block_k rows of
// 128-byte MN segments for MN-major, always in the canonical 128-byte-swizzle
// UMMA layout that TMA produces, so no operand is transposed or re-tiled in
// shared memory.
#include "common.cuh"
#include "row_head.cuh"

#include <stdlib.h>
#include <string.h>

#include <atomic>

namespace {

constexpr int UG_BLOCK_M = 128;
// Epilogue warps per CTA (template parameter EW of the kernel): 8 = two warps per TMEM lane quadrant, the
// general form; 16 = four per quadrant, for 16-bit outputs of CTA-pair tiles whose K is so short (at most
// two k-blocks: the narrow nets' layers) that the launch is all epilogue; measured on a 262144 x 1024
// output with K = 16: 277 -> 242 us.  A warp takes
// every (EW / 4)-th 32-column chunk and owns a staging slot of 32 KB / EW.  Measured: with a real main
// loop (K = 1024) sixteen warps are 4 % SLOWER than eight although the drain alone is 10 % faster -- the
// MMA-issuing thread shares its scheduler with twice as many busy warps and the tensor pipe waits for it.
constexpr int UG_EPI_WARPS = 8;
constexpr int UG_EPI_WARPS_MAX = 16;
constexpr int ug_threads(int ew) { return 96 + 32 * ew; }   // A-producer warp, MMA warp, epilogue warps, B-producer warp
constexpr int UG_MAX_STAGES = 8;
constexpr int UG_SMEM_LIMIT = 227 * 1024;
constexpr int UG_MAX_PEERS = 8;         // ranks whose copies of C one launch can add its tiles to
constexpr int UG_HEAD_MAX_N = 64;       // widest row a fused head keeps in registers
constexpr int UG_HEAD_MAX_TILE_N = 256; // widest row a fused head may belong to when a prefix mask confines it to UG_HEAD_MAX_N columns
constexpr int UG_EPI_STAGING = UG_EPI_WARPS * 4096;  // one 32-row x 128-byte box per epilogue warp (8 warps), or 2 KB each (16)

// Tensor maps of the output: m[0] is C itself; with peer_rows > 0, m[r] is rank r's copy of C (the
// same matrix in that rank's memory) and a CTA adds its rows to the copy of the rank that owns them.
struct UmmaOutMaps {
  CUtensorMap m[UG_MAX_PEERS];
  CUtensorMap b_tail;     // a K-major B with boxes of half as many rows: the half-width tiles of the last wave
};

struct UmmaGemmParams {
  int M, N, K;
  int block_n;
  int acc_stride;  // TMEM columns between the two accumulators
  int tmem_cols;   // allocated TMEM columns (power of two >= 32)
  int stages;
  int kind_tf32;
  int a_mn, b_mn;
  int block_k;  // elements of K per stage
  int k_blocks;
  int tiles_m, tiles_n, num_tiles;
  int splits;          // split-K factor: work item = (split, tile); 1 = no split
  int kb_per_split;    // k-blocks per split
  int num_work;        // num_tiles * splits
  long long split_stride;  // elements between the partial outputs of two splits
  uint32_t idesc;
  uint32_t a_stage_bytes, b_stage_bytes;
  int a_boxes, b_boxes;    // TMA boxes per stage (1 when K-major)
  int mn_box_elems;        // MN extent of one MN-major box (128 bytes)
  uint32_t mn_box_bytes;   // bytes of one MN-major box = block_k * 128
  uint32_t a_kstep, b_kstep;  // descriptor start-address step per MMA, in 16-byte units
  int subs;                   // 128-byte K sub-blocks per stage (1 or 2): 4 * subs MMAs per barrier round
  uint32_t a_sub_step, b_sub_step;  // descriptor step between the two sub-blocks, in 16-byte units
  uint32_t a_sub_bytes, b_sub_bytes;  // bytes of one K-major sub-block (rows * 128)
  uint32_t a_sbo, b_sbo;      // stride byte offset of the smem descriptors
  uint32_t a_layout, b_layout;  // descriptor layout type (2 = SW128, 1 = SW128 with 32-byte chunks)
  float alpha, beta;
  void* C;
  long long ldc;
  int out_dtype;
  int epi;
  const float* bias;
  const uint8_t* mask;
  const void* aux_in;
  void* aux_out;
  int pair;            // 1: CTA pairs (cta_group::2), 256-row tiles
  int coalesced;       // 1: 32-column chunks are transposed through shared memory for row-contiguous stores
  int tma_store;       // 1: and the finished boxes are written by TMA stores
  int wide;            // 1: 16-bit output boxes span two chunks (64 columns, 128-byte rows)
  uint32_t epi_offset; // byte offset of the epilogue staging area from the stage base
  SbRowHead head;      // the row head, when epi holds a head flag
  int epi_warps;       // 8 or 16 epilogue warps (the kernel instance launched)
  int reduce_add;      // 1: tiles are added to C through TMA reduce-add stores (split-K into one matrix, peer copies)
  int peer_rows;       // > 0: rows [r * peer_rows, (r + 1) * peer_rows) of C are added to rank r's copy (out map r)
  int tail_first;      // work items from this one on are HALF tiles (block_n / 2 columns); == num_work: none
  uint32_t idesc_tail; // instruction descriptor of a half tile
};

// Walks the work of one worker (a CTA, or a CTA pair): work items (split, tile) strided over the
// workers.  Items of one split sit side by side, so the workers that run at the same time read the same
// K range of different tiles and share the operands through L2.  (Cutting the k-blocks of all tiles
// into one equal range per worker -- "stream-K" -- was measured: no worker idles, but no two workers
// are at the same K at the same time, every operand byte comes from DRAM once per tile column instead
// of once, and the Hold'em weight-gradient GEMM went from 0.36 to 0.49 ms.)
struct WorkIter {
  int work, stride;
  __device__ __forceinline__ WorkIter(const UmmaGemmParams&, int worker, int num_workers) {
    work = worker;
    stride = num_workers;
  }
  // The next item: tile index, split index, k-block range.  False when done.
  // `half`: -1 for a whole tile; 0 / 1 for the left / right half of one (the last wave of a launch whose
  // tiles would fill less than half of the workers is cut into half-width tiles, so that it takes about
  // half as long; only launches without split-K have such items).
  __device__ __forceinline__ bool next(const UmmaGemmParams& p, int& tile, int& split, int& kb_begin, int& kb_end,
                                       int& half) {
    if (work >= p.num_work) return false;
    if (work >= p.tail_first) {
      const int t = work - p.tail_first;
      split = 0;
      tile = p.tail_first + (t >> 1);
      half = t & 1;
      kb_begin = 0;
      kb_end = p.k_blocks;
    } else {
      half = -1;
      split = work / p.num_tiles;
      tile = work - split * p.num_tiles;
      kb_begin = split * p.kb_per_split;
      kb_end = min(p.k_blocks, kb_begin + p.kb_per_split);
    }
    work += stride;
    return true;
  }
};

__device__ __forceinline__ void tile_coords(const UmmaGemmParams& p, int tile, int& m_blk, int& n_blk) {
  constexpr int GROUP = 8;
  const int per_group = GROUP * p.tiles_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP;
  const int gsz = min(GROUP, p.tiles_m - first_m);
  const int r = tile - g * per_group;
  m_blk = first_m + r % gsz;
  n_blk = r / gsz;
}

// ------------------------------ epilogue -----------------------------------
template <typename T>
__device__ __forceinline__ float load_as_float(const T* p);
template <>
__device__ __forceinline__ float load_as_float<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}
template <>
__device__ __forceinline__ float load_as_float<__half>(const __half* p) { return __half2float(*p); }

template <typename T>
__device__ __forceinline__ T float_to(float v);
template <>
__device__ __forceinline__ float float_to<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 float_to<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ __half float_to<__half>(float v) { return __float2half_rn(v); }

// Two floats -> one 32-bit word of two 16-bit values (lo in the low half), round to nearest even,
// optionally with the ReLU folded into the conversion.  The packed form is one ALU-class
// instruction per pair; scalar conversions go through the quarter-rate conversion pipe, which an
// epilogue of 32768 values per tile saturates.
template <typename OutT, bool RELU>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16, false>(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16, true>(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.relu.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
template <>
__device__ __forceinline__ uint32_t pack2<__half, false>(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
template <>
__device__ __forceinline__ uint32_t pack2<__half, true>(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.relu.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
template <>
__device__ __forceinline__ uint32_t pack2<float, false>(float lo, float) { return __float_as_uint(lo); }
template <>
__device__ __forceinline__ uint32_t pack2<float, true>(float lo, float) { return __float_as_uint(lo); }

__device__ __forceinline__ float round_tf32_rn(float v) {
  uint32_t u = __float_as_uint(v);
  if ((u & 0x7f800000u) == 0x7f800000u) return v;
  u += 0x0fffu + ((u >> 13) & 1u);
  return __uint_as_float(u & 0xffffe000u);
}

// Coalescing variant for a 32-column chunk.  TMEM hands each thread one output
// row, so a direct store would touch 32 rows per instruction with 16 bytes
// each.  Instead the warp's 32 rows x 32 columns go through a swizzled
// shared-memory box (conflict-free both ways) and are written so that one
// store instruction covers whole row segments: 4 rows x 128 B (32-bit output)
// or 8 rows x 64 B (16-bit output).  Old C values (beta) and the activation
// tile of the ReLU-gradient gate come in through the same box, read with the
// same coalesced pattern.  `sbuf` is this warp's private 4 KB box.
template <typename OutT>
__device__ __forceinline__ uint32_t box_offset(uint32_t row, uint32_t piece) {
  constexpr uint32_t ROW_BYTES = 32 * sizeof(OutT);
  constexpr uint32_t PIECES = ROW_BYTES / 16;
  const uint32_t key = ROW_BYTES == 128 ? (row & 7u) : ((row >> 1) & 3u);
  return row * ROW_BYTES + (((piece ^ key) & (PIECES - 1)) << 4);
}

__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}

// Brings the chunk [row0_warp .. +32) x [col0 .. +32) of a row-major matrix
// (row pitch ld elements; rows valid below row_limit, columns below n; zeros
// elsewhere) into the box with coalesced loads.  Afterwards lane r finds its
// own row r at box_offset(r, piece).
template <typename OutT>
__device__ __forceinline__ void load_chunk_to_box(const OutT* base, long long ld, long long row0_warp,
                                                  long long row_limit, int col0, int n, uint32_t sbuf,
                                                  int lane) {
  constexpr int VEC = 16 / sizeof(OutT);
  constexpr int PIECES = 32 / VEC;
  constexpr int ROWS_PER_INST = 32 / PIECES;
#pragma unroll
  for (int i = 0; i < PIECES; ++i) {
    const int r = i * ROWS_PER_INST + lane / PIECES;
    const int q = lane % PIECES;
    const long long grow = row0_warp + r;
    const int gcol = col0 + q * VEC;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (grow < row_limit) {
      const OutT* src = base + grow * ld + gcol;
      if (gcol + VEC <= n) {
        val = *reinterpret_cast<const uint4*>(src);
      } else {
        OutT tmp[VEC];
#pragma unroll
        for (int t = 0; t < VEC; ++t) tmp[t] = (gcol + t < n) ? src[t] : float_to<OutT>(0.f);
        val = *reinterpret_cast<const uint4*>(tmp);
      }
    }
    st_shared_v4(sbuf + box_offset<OutT>((uint32_t)r, (uint32_t)q), val);
  }
  __syncwarp();
}

// Per-launch epilogue constants.  They live in shared memory, written once by
// thread 0: the out-of-line epilogue reads a field where it needs it (a shared
// memory load) instead of carrying some twenty-five values in registers through
// code that is already at the register budget of a 10-warp CTA, and instead of
// reading the kernel's parameter block through a pointer (with the L1 carved out
// as shared memory each such read would be an L2 round trip).
struct EpiShared {
  void* c;                  // output matrix (split partials follow each other)
  const void* aux;          // activation tile for the ReLU-gradient gate (SB_EPI_RELU_GRAD)
  const float* bias;
  const uint32_t* gate_in;  // ReLU sign bits, uint32 [N / 32, M]: one word per 32 columns and row (SB_EPI_RELU_GRAD_MASK)
  uint32_t* gate_out;       // where the forward pass records them (SB_EPI_RELU_MASK_OUT)
  float* colsum;            // column sums of the output are added here (SB_EPI_COLSUM_OUT)
  const CUtensorMap* tma_c; // non-null: finished boxes leave through TMA stores (32 x 32 element boxes over C)
  long long ldc;
  long long split_stride;
  int M, N;
  int block_n;
  float alpha, beta;
  int has_bias, relu, relu_grad, coalesced;
  int reduce_add;           // finished boxes are ADDED to C (split-K accumulating into one matrix)
  int peer_rows;            // > 0: the boxes of rows [r * peer_rows, ...) go to out map r (rank r's copy of C)
  int split_rows;           // rows between two splits' outputs in the store map (0 when they share C)
  int ln_l2;                // divide every row by its sum of squares before the ReLU (SB_EPI_LN_L2; the tile spans the row)
  uint32_t box_base;        // shared-memory address of the first epilogue warp's 4 KB box
};
__shared__ EpiShared g_epi;
__shared__ int g_abort_flag;
__shared__ __align__(16) float g_bias_spread[8][32];

// Finishes one 32-column chunk.  `bias_lane` = bias[col0 + lane]; `gate` = this
// row's 32 ReLU sign bits of the chunk (when gating by bits).  Returns the sign
// bits of the values this row produced (bit j = value j > 0 before the ReLU).
// MODE selects how much is decided at compile time, because every run-time flag
// tested inside the unrolled per-element code costs instructions and registers
// in a loop that is issue-bound:
//   MODE >= 0 : alpha = 1, beta = 0 and exactly the features in the bit mask
//               (1 bias, 2 ReLU, 4 record sign bits, 8 gate by sign bits);
//   MODE = -1 : run-time flags, no second tile read;
//   MODE = -2 : run-time flags plus the two features that read a second tile
//               through the box (beta != 0, gate by the activation tile).
template <typename OutT, bool ROUND_TF32, int MODE, int EW = UG_EPI_WARPS>
__device__ __forceinline__ uint32_t coalesced_chunk(float* v, float bias_lane, uint32_t gate, int split,
                                                    int row0_warp, int col0, uint32_t sbuf,
                                                    uint32_t bias_smem, int lane) {
  constexpr int VEC = 16 / sizeof(OutT);      // elements per 16-byte piece
  constexpr int PIECES = 32 / VEC;            // 16-byte pieces per row of the box
  constexpr int ROWS_PER_INST = 32 / PIECES;
  constexpr bool GENERAL = MODE == -2;
  const bool has_bias = MODE >= 0 ? (MODE & 1) != 0 : g_epi.has_bias != 0;
  const bool relu = MODE >= 0 ? (MODE & 2) != 0 : g_epi.relu != 0;
  const bool gate_out = MODE >= 0 ? (MODE & 4) != 0 : g_epi.gate_out != nullptr;
  const bool gate_in = MODE >= 0 ? (MODE & 8) != 0 : g_epi.gate_in != nullptr;
  if (GENERAL && g_epi.beta != 0.0f) {
    // v <- alpha * acc + beta * C_old, with the old tile read through the box.
    OutT* cbase = reinterpret_cast<OutT*>(g_epi.c) + (long long)split * g_epi.split_stride;
    load_chunk_to_box<OutT>(cbase, g_epi.ldc, row0_warp, g_epi.M, col0, g_epi.N, sbuf, lane);
    const float alpha = g_epi.alpha, beta = g_epi.beta;
#pragma unroll
    for (int q = 0; q < PIECES; ++q) {
      const uint4 raw = ld_shared_v4(sbuf + box_offset<OutT>((uint32_t)lane, (uint32_t)q));
      const OutT* o = reinterpret_cast<const OutT*>(&raw);
#pragma unroll
      for (int t = 0; t < VEC; ++t) v[q * VEC + t] = alpha * v[q * VEC + t] + beta * load_as_float<OutT>(o + t);
    }
    __syncwarp();
  } else if (MODE < 0 && g_epi.alpha != 1.0f) {
    const float alpha = g_epi.alpha;
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] *= alpha;
  }
  if (has_bias && EW == 16) {
    // Lane j holds bias[col0 + j]; every lane needs all 32.  With sixteen epilogue warps there is no
    // shared memory left for a spread buffer per warp: the values go round by shuffles.
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] += __shfl_sync(0xffffffffu, bias_lane, j);
  } else if (has_bias) {
    // Lane j holds bias[col0 + j]; every lane needs all 32: spread them through
    // 128 bytes of shared memory and read them back as broadcasts.
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(bias_smem + 4u * (uint32_t)lane), "f"(bias_lane) : "memory");
    __syncwarp();
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const uint4 b = ld_shared_v4(bias_smem + 16u * (uint32_t)q);
      v[4 * q + 0] += __uint_as_float(b.x);
      v[4 * q + 1] += __uint_as_float(b.y);
      v[4 * q + 2] += __uint_as_float(b.z);
      v[4 * q + 3] += __uint_as_float(b.w);
    }
  }
  uint32_t signs = 0u;
  if (gate_in) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = ((gate >> j) & 1u) ? v[j] : 0.f;
  }
  const bool tile_gate = GENERAL && g_epi.relu_grad != 0;
  if (tile_gate)
    load_chunk_to_box<OutT>(reinterpret_cast<const OutT*>(g_epi.aux), g_epi.ldc, row0_warp, g_epi.M, col0, g_epi.N,
                            sbuf, lane);
  const bool tma_out = !GENERAL && g_epi.tma_c != nullptr;
  // A 16-bit box here is 32 rows x 32 columns (64-byte swizzle).
  if (tma_out) {
    // The store that last read this box must have finished reading it.  A 16-bit box is 2 KB,
    // so the warp's 4 KB slot holds two that alternate and only the store before last is awaited.
    if (lane == 0) {
      if (sizeof(OutT) == 2 && EW == 8) bulk_wait_group_read<1>(); else bulk_wait_group_read<0>();
    }
    __syncwarp();
  }
#pragma unroll
  for (int q = 0; q < PIECES; ++q) {
    const uint32_t mine = sbuf + box_offset<OutT>((uint32_t)lane, (uint32_t)q);
    uint4 araw = make_uint4(0u, 0u, 0u, 0u);
    if (tile_gate) araw = ld_shared_v4(mine);     // this lane's piece of the activation tile
    const OutT* acte = reinterpret_cast<const OutT*>(&araw);
    // ReLU of a compile-time mode rides on the 16-bit conversion itself.
    constexpr bool RELU_IN_CVT = sizeof(OutT) == 2 && MODE >= 0 && (MODE & 2) != 0;
    float x[VEC];
#pragma unroll
    for (int t = 0; t < VEC; ++t) {
      x[t] = v[q * VEC + t];
      if (relu && !RELU_IN_CVT) x[t] = fmaxf(x[t], 0.f);
      if (tile_gate) x[t] = load_as_float<OutT>(acte + t) > 0.f ? x[t] : 0.f;
      if (ROUND_TF32) x[t] = round_tf32_rn(x[t]);
    }
    uint4 outw;
    if (sizeof(OutT) == 2) {
      outw.x = pack2<OutT, RELU_IN_CVT>(x[0], x[1]);
      outw.y = pack2<OutT, RELU_IN_CVT>(x[2], x[3]);
      outw.z = pack2<OutT, RELU_IN_CVT>(x[4 % VEC], x[5 % VEC]);
      outw.w = pack2<OutT, RELU_IN_CVT>(x[6 % VEC], x[7 % VEC]);
    } else {
      outw = make_uint4(__float_as_uint(x[0]), __float_as_uint(x[1]), __float_as_uint(x[2]), __float_as_uint(x[3]));
    }
    if (gate_out) {
      // Sign bits of this piece from the values just consumed (v is not needed afterwards).
      uint32_t s = 0u;
#pragma unroll
      for (int t = 0; t < VEC; ++t) s |= (__float_as_int(v[q * VEC + t]) > 0 ? 1u : 0u) << t;
      signs |= s << (q * VEC);
    }
    st_shared_v4(mine, outw);   // overwrites only what this lane just read
  }
  if (tma_out) {
    // The box already has the layout of a swizzled TMA box: one asynchronous bulk store writes
    // it (clipped at the matrix edges) without occupying the load/store pipe.
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      if (g_epi.reduce_add)
        tma_reduce_add_2d(g_epi.tma_c + (g_epi.peer_rows > 0 ? row0_warp / g_epi.peer_rows : 0), sbuf, col0, row0_warp);
      else tma_store_2d(g_epi.tma_c, sbuf, col0, split * g_epi.split_rows + row0_warp);
      bulk_commit_group();
    }
    return signs;
  }
  __syncwarp();
  // Not fully unrolled: eight independent 64-bit store addresses at once would
  // push the 32-bit-output variant past its register budget.
  OutT* cbase = reinterpret_cast<OutT*>(g_epi.c) + (long long)split * g_epi.split_stride;
  const long long ldc = g_epi.ldc;
  const int M = g_epi.M, N = g_epi.N;
#pragma unroll 2
  for (int i = 0; i < PIECES; ++i) {
    const int r = i * ROWS_PER_INST + lane / PIECES;
    const int q = lane % PIECES;
    const long long grow = (long long)row0_warp + r;
    const int gcol = col0 + q * VEC;
    if (grow < M && gcol < N) {
      const uint4 val = ld_shared_v4(sbuf + box_offset<OutT>((uint32_t)r, (uint32_t)q));
      OutT* dst = cbase + grow * ldc + gcol;
      if (gcol + VEC <= N) {
        *reinterpret_cast<uint4*>(dst) = val;
      } else {
        const OutT* o = reinterpret_cast<const OutT*>(&val);
#pragma unroll
        for (int t = 0; t < VEC; ++t)
          if (gcol + t < N) dst[t] = o[t];
      }
    }
  }
  __syncwarp();
  return signs;
}

// Adds the column sums of a finished 32-row x 32-column chunk to g_epi.colsum.
// Each lane holds one row (v[0..31], already scaled, biased and gated); a
// butterfly of 31 shuffles folds the 32 rows so that lane j ends with the sum
// of column j, and the warp issues one 128-byte vector reduction to global
// memory.  The sums are taken before the rounding to the storage type.
template <int MODE>
__device__ __forceinline__ void chunk_colsum(float* v, int col0, int lane) {
  static_assert(MODE >= 0 && (MODE & 3) == 0, "column sums are built for the modes without bias and ReLU");
  // Rows beyond M are zero: their rows of A were zero-filled and nothing was added to them.
#define SB_FOLD(HALF)                                                      \
  {                                                                        \
    const bool up = (lane & HALF) != 0;                                    \
    _Pragma("unroll") for (int i = 0; i < HALF; ++i) {                     \
      const float send = up ? v[i] : v[i + HALF];                          \
      const float keep = up ? v[i + HALF] : v[i];                          \
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, HALF);              \
    }                                                                      \
  }
  SB_FOLD(16) SB_FOLD(8) SB_FOLD(4) SB_FOLD(2) SB_FOLD(1)
#undef SB_FOLD
  if (col0 + lane < g_epi.N) atomicAdd(g_epi.colsum + col0 + lane, v[0]);
}

// Per-thread stores of 16 columns of one row: the fallback when C's row pitch or base is not
// 16-byte aligned, and the 16-column tail chunk.  The sign-bit and column-sum epilogues never come
// here (they need N % 32 == 0 and an aligned C, which always takes the coalesced path).
template <typename OutT, bool ROUND_TF32>
__device__ __forceinline__ void direct_chunk16(float* v, long long row, int col0, int split) {
  const int valid = min(16, g_epi.N - col0);
  if (valid <= 0) return;
  const long long ldc = g_epi.ldc;
  OutT* crow = reinterpret_cast<OutT*>(g_epi.c) + (long long)split * g_epi.split_stride + row * ldc + col0;
  const OutT* arow = reinterpret_cast<const OutT*>(g_epi.aux) + row * ldc + col0;
  const float alpha = g_epi.alpha, beta = g_epi.beta;
  const float* bias = g_epi.has_bias ? g_epi.bias : nullptr;
  const bool relu = g_epi.relu != 0, relu_grad = g_epi.relu_grad != 0;
#pragma unroll
  for (int j = 0; j < 16; ++j) {      // static indices keep v[] in registers
    if (j < valid) {
      float x = alpha * v[j];
      if (beta != 0.0f) x += beta * load_as_float<OutT>(crow + j);
      if (bias) x += __ldg(bias + col0 + j);
      if (relu) x = fmaxf(x, 0.f);
      if (relu_grad) x = load_as_float<OutT>(arow + j) > 0.f ? x : 0.f;
      if (ROUND_TF32) x = round_tf32_rn(x);
      crow[j] = float_to<OutT>(x);
    }
  }
}

// Chunks that cannot take the coalesced path, from chunk `c` on: per-thread stores, 16 columns at
// a time.  A function of its own so that its registers do not add to the fast path's.
template <typename OutT, bool ROUND_TF32, int EW>
__device__ __noinline__ void epilogue_rest(uint32_t t_row, int row0_warp, int n0, int block_n, int split, int c) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)row0_warp + lane;
  const bool row_ok = row < g_epi.M;
  const int nchunks = (block_n + 31) >> 5;
  for (; c < nchunks; c += EW / 4) {
    const int w = min(32, block_n - c * 32);
    for (int h = 0; h < w; h += 16) {
      uint32_t raw[16];
      tmem_ld16(t_row + (uint32_t)(c * 32 + h), raw);
      tmem_ld_wait();
      const int col0 = n0 + c * 32 + h;
      if (row_ok && col0 < g_epi.N) direct_chunk16<OutT, ROUND_TF32>(reinterpret_cast<float*>(raw), row, col0, split);
    }
  }
}

// One warp drains its share of a tile: its 32 accumulator rows (TMEM lane
// quadrant) and every UG_EPI_STRIDE-th 32-column chunk starting at its `half`
// (with 8 epilogue warps two warps share a quadrant).  The bias values and ReLU
// sign word of a chunk are requested one chunk ahead (the first before the wait
// for the accumulator).  Out of line, one instance per output type and mode; it
// must not spill: with the L1 carved out as shared memory a spilled register
// costs an L2 round trip.  Returns false when the wait for the accumulator expired.
template <typename OutT, bool ROUND_TF32, int MODE, int EW>
__device__ __noinline__ bool epilogue_tile(uint32_t t_row, int row0_warp, int n0, int block_n, int split,
                                           uint32_t bar_full, uint32_t parity) {
  static_assert(EW == 8 || (EW == 16 && sizeof(OutT) == 2), "sixteen epilogue warps: 2 KB staging slots, 16-bit outputs only");
  constexpr int STRIDE = EW / 4;
  const int lane = threadIdx.x & 31;
  const int ewarp = (int)(threadIdx.x >> 5) - 2;
  const int half = ewarp >> 2;
  const uint32_t sbuf = g_epi.box_base + (uint32_t)ewarp * (EW == 8 ? 4096u : 2048u);
  const uint32_t bias_smem = smem_u32(&g_bias_spread[ewarp & 7][0]);
  const bool has_bias = MODE >= 0 ? (MODE & 1) != 0 : g_epi.has_bias != 0;
  const bool want_gate_in = MODE >= 0 ? (MODE & 8) != 0 : g_epi.gate_in != nullptr;
  const bool want_gate_out = MODE >= 0 ? (MODE & 4) != 0 : g_epi.gate_out != nullptr;
  const int N = g_epi.N;
  const bool row_ok = row0_warp + lane < g_epi.M;
  const bool rows_live = row0_warp < g_epi.M;
  const int nchunks = (block_n + 31) >> 5;
  const int nfull = g_epi.coalesced ? (block_n >> 5) : 0;     // chunks that take the coalesced path
  // The sign-bit matrices are stored [N / 32, M]: the 32 rows of a warp are 32 consecutive words,
  // so a chunk's words move as one 128-byte transaction.
  const long long gate_row = (long long)(row0_warp + lane);
  const long long gate_pitch = g_epi.M;

  auto fetch = [&](int c, float& bias_lane, uint32_t& gate) {
    bias_lane = 0.f;
    gate = 0u;
    const int col0 = n0 + c * 32;
    if (c < nchunks) {
      if (has_bias && col0 + lane < N) bias_lane = __ldg(g_epi.bias + col0 + lane);
      if (want_gate_in && row_ok && col0 < N) gate = __ldg(g_epi.gate_in + (col0 >> 5) * gate_pitch + gate_row);
    }
  };

  int c = half;
  float bias_cur, bias_nxt;
  uint32_t gate_cur, gate_nxt;
  fetch(c, bias_cur, gate_cur);
  if (!mbar_wait(bar_full, parity, &g_abort_flag, SB_SITE_EPI_TMEM_FULL)) return false;
  tc_fence_after_sync();

  uint32_t raw_a[32];
  uint32_t box_sel = 0u;
  // Row normalisation (local_ln_l2, ml/primitives.spi:701-703): a first pass over the whole
  // accumulator row sums the squares (both warps of a quadrant do it, each for itself); the tile
  // spans the row (one column tile, N a multiple of 32), columns beyond N are zero.
  float sumsq = 0.f;
  const bool ln_l2 = MODE == -1 && g_epi.ln_l2 != 0;
  if (ln_l2) {
    for (int cc = 0; cc < nfull; ++cc) {
      tmem_ld32(t_row + (uint32_t)(cc * 32), raw_a);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) sumsq = fmaf(__uint_as_float(raw_a[j]), __uint_as_float(raw_a[j]), sumsq);
    }
  }
  for (; c < nfull; c += STRIDE) {
    tmem_ld32(t_row + (uint32_t)(c * 32), raw_a);
    fetch(c + STRIDE, bias_nxt, gate_nxt);    // in flight while this chunk is finished
    tmem_ld_wait();
    if (ln_l2) {
#pragma unroll
      for (int j = 0; j < 32; ++j) raw_a[j] = __float_as_uint(sumsq != 0.f ? __uint_as_float(raw_a[j]) / sumsq : 0.f);
    }
    const int col0 = n0 + c * 32;
    if (rows_live && col0 < N) {
      const uint32_t box = sbuf + ((EW == 8 && MODE != -2 && sizeof(OutT) == 2 && g_epi.tma_c) ? box_sel : 0u);
      box_sel ^= 2048u;
      const uint32_t signs = coalesced_chunk<OutT, ROUND_TF32, MODE, EW>(reinterpret_cast<float*>(raw_a), bias_cur, gate_cur,
                                                              split, row0_warp, col0, box, bias_smem, lane);
      if (want_gate_out && row_ok) g_epi.gate_out[(col0 >> 5) * gate_pitch + gate_row] = signs;
      if constexpr (MODE >= 0 && (MODE & 16) != 0) chunk_colsum<MODE>(reinterpret_cast<float*>(raw_a), col0, lane);
    }
    bias_cur = bias_nxt;
    gate_cur = gate_nxt;
  }
  // What is left for this warp: a 16-column tail chunk, or every chunk when C
  // cannot take row-contiguous 16-byte stores.
  if (c < nchunks) epilogue_rest<OutT, ROUND_TF32, EW>(t_row, row0_warp, n0, block_n, split, c);
  return true;
}

// Finishes one 32-column chunk of a 16-bit output in registers: scale, bias, gate, ReLU, rounding to
// the storage type.  out[0..3] are the row's four 16-byte pieces of the chunk; returns the sign bits
// (bit j = value j > 0 before the ReLU).  v[] keeps the gated fp32 values (the column sums use them).
template <typename OutT, int MODE>
__device__ __forceinline__ uint32_t wide_prepare(float* v, float bias_lane, uint32_t gate, uint32_t bias_smem, int lane,
                                                 uint4* out) {
  const bool has_bias = MODE >= 0 ? (MODE & 1) != 0 : g_epi.has_bias != 0;
  const bool relu = MODE >= 0 ? (MODE & 2) != 0 : g_epi.relu != 0;
  const bool gate_out = MODE >= 0 ? (MODE & 4) != 0 : g_epi.gate_out != nullptr;
  const bool gate_in = MODE >= 0 ? (MODE & 8) != 0 : g_epi.gate_in != nullptr;
  if (MODE < 0 && g_epi.alpha != 1.0f) {
    const float alpha = g_epi.alpha;
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] *= alpha;
  }
  if (has_bias) {
    // Lane j holds bias[col0 + j]; every lane needs all 32: spread them through 128 bytes of shared
    // memory and read them back as broadcasts.
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(bias_smem + 4u * (uint32_t)lane), "f"(bias_lane) : "memory");
    __syncwarp();
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const uint4 b = ld_shared_v4(bias_smem + 16u * (uint32_t)q);
      v[4 * q + 0] += __uint_as_float(b.x);
      v[4 * q + 1] += __uint_as_float(b.y);
      v[4 * q + 2] += __uint_as_float(b.z);
      v[4 * q + 3] += __uint_as_float(b.w);
    }
    __syncwarp();      // every lane has read them: the next chunk may overwrite the spread buffer
  }
  if (gate_in) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = ((gate >> j) & 1u) ? v[j] : 0.f;
  }
  uint32_t signs = 0u;
  if (gate_out) {
#pragma unroll
    for (int j = 0; j < 32; ++j) signs |= (__float_as_int(v[j]) > 0 ? 1u : 0u) << j;
  }
  // ReLU of a compile-time mode rides on the 16-bit conversion itself.
  constexpr bool RELU_IN_CVT = MODE >= 0 && (MODE & 2) != 0;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    float x[8];
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      x[t] = v[q * 8 + t];
      if (relu && !RELU_IN_CVT) x[t] = fmaxf(x[t], 0.f);
    }
    out[q].x = pack2<OutT, RELU_IN_CVT>(x[0], x[1]);
    out[q].y = pack2<OutT, RELU_IN_CVT>(x[2], x[3]);
    out[q].z = pack2<OutT, RELU_IN_CVT>(x[4], x[5]);
    out[q].w = pack2<OutT, RELU_IN_CVT>(x[6], x[7]);
  }
  return signs;
}

// The same for a 16-bit output whose tile is a whole number of 64-column chunk pairs and leaves
// through TMA stores: the two warps of a quadrant take alternate PAIRS of adjacent chunks
// (warp 0: chunks 0 1 4 5 ..., warp 1: 2 3 6 7 ...).  Both accumulator chunks of a pair are
// requested from tensor memory at once and finished in registers; only then does the warp wait for
// its box -- 32 rows x 64 columns, 128-byte rows in the 128-byte swizzle, chunk e = 0 / 1 filling
// pieces 4e .. 4e+3 of every row -- to be free, so that the store of the previous pair reads the
// box while this pair is computed.  One store (one proxy fence) serves the pair.
template <typename OutT, int MODE>
__device__ __noinline__ bool epilogue_tile_wide(uint32_t t_row, int row0_warp, int n0, int block_n, int split,
                                                uint32_t bar_full, uint32_t parity) {
  static_assert(sizeof(OutT) == 2 && MODE != -2, "wide boxes: 16-bit output through TMA stores only");
  const int lane = threadIdx.x & 31;
  const int ewarp = (int)(threadIdx.x >> 5) - 2;
  const int half = ewarp >> 2;
  const uint32_t sbuf = g_epi.box_base + (uint32_t)ewarp * 4096u;
  const uint32_t bias_smem = smem_u32(&g_bias_spread[ewarp][0]);
  const bool has_bias = MODE >= 0 ? (MODE & 1) != 0 : g_epi.has_bias != 0;
  const bool want_gate_in = MODE >= 0 ? (MODE & 8) != 0 : g_epi.gate_in != nullptr;
  const bool want_gate_out = MODE >= 0 ? (MODE & 4) != 0 : g_epi.gate_out != nullptr;
  const int N = g_epi.N;
  const bool row_ok = row0_warp + lane < g_epi.M;
  const bool rows_live = row0_warp < g_epi.M;
  const int nchunks = block_n >> 5;     // even
  const long long gate_row = (long long)(row0_warp + lane);
  const long long gate_pitch = g_epi.M;

  auto fetch = [&](int c, float& bias_lane, uint32_t& gate) {
    bias_lane = 0.f;
    gate = 0u;
    const int col0 = n0 + c * 32;
    if (c < nchunks) {
      if (has_bias && col0 + lane < N) bias_lane = __ldg(g_epi.bias + col0 + lane);
      if (want_gate_in && row_ok && col0 < N) gate = __ldg(g_epi.gate_in + (col0 >> 5) * gate_pitch + gate_row);
    }
  };

  int c = 2 * half;
  float bias_a, bias_b, bias_na, bias_nb;
  uint32_t gate_a, gate_b, gate_na, gate_nb;
  fetch(c, bias_a, gate_a);
  fetch(c + 1, bias_b, gate_b);
  if (!mbar_wait(bar_full, parity, &g_abort_flag, SB_SITE_EPI_TMEM_FULL)) return false;
  tc_fence_after_sync();

  // With the column sums (a 32-register butterfly per chunk) or with run-time flags both chunks do
  // not fit in the register budget at once: those modes read the second chunk after the first is
  // finished.
  constexpr bool BOTH_AT_ONCE = MODE >= 0 && (MODE & 16) == 0;
  uint32_t raw_a[32], raw_b[32];
  constexpr int UG_EPI_STRIDE = UG_EPI_WARPS / 4;
  const uint32_t wide_row = sbuf + (uint32_t)lane * 128u;
  const uint32_t key = (uint32_t)lane & 7u;
  for (; c < nchunks; c += 2 * UG_EPI_STRIDE) {
    tmem_ld32(t_row + (uint32_t)(c * 32), raw_a);
    if (BOTH_AT_ONCE) tmem_ld32(t_row + (uint32_t)(c * 32 + 32), raw_b);
    fetch(c + 2 * UG_EPI_STRIDE, bias_na, gate_na);      // the next pair's, in flight meanwhile
    fetch(c + 2 * UG_EPI_STRIDE + 1, bias_nb, gate_nb);
    tmem_ld_wait();
    const int col0 = n0 + c * 32;
    // A second chunk beyond N is all zeros and the store clips it; it is still written into the box.
    if (rows_live && col0 < N) {
      uint4 out_a[4], out_b[4];
      const uint32_t sa = wide_prepare<OutT, MODE>(reinterpret_cast<float*>(raw_a), bias_a, gate_a, bias_smem, lane, out_a);
      if (want_gate_out && row_ok) g_epi.gate_out[(col0 >> 5) * gate_pitch + gate_row] = sa;
      if constexpr (MODE >= 0 && (MODE & 16) != 0) chunk_colsum<MODE>(reinterpret_cast<float*>(raw_a), col0, lane);
      if (!BOTH_AT_ONCE) {
        tmem_ld32(t_row + (uint32_t)(c * 32 + 32), raw_b);
        tmem_ld_wait();
      }
      const uint32_t sb = wide_prepare<OutT, MODE>(reinterpret_cast<float*>(raw_b), bias_b, gate_b, bias_smem, lane, out_b);
      if (want_gate_out && row_ok && col0 + 32 < N) g_epi.gate_out[((col0 >> 5) + 1) * gate_pitch + gate_row] = sb;
      if constexpr (MODE >= 0 && (MODE & 16) != 0) chunk_colsum<MODE>(reinterpret_cast<float*>(raw_b), col0 + 32, lane);
      // The store that last read this box must have finished reading it.
      if (lane == 0) bulk_wait_group_read<0>();
      __syncwarp();
#pragma unroll
      for (int q = 0; q < 4; ++q) {        // piece 4e + q of the row sits at ((4e + q) ^ key) * 16
        st_shared_v4(wide_row + (((uint32_t)q ^ key) << 4), out_a[q]);
        st_shared_v4(wide_row + (((uint32_t)(4 + q) ^ key) << 4), out_b[q]);
      }
      // The box has the layout of a swizzled TMA box: one asynchronous bulk store writes it (clipped
      // at the matrix edges) without occupying the load/store pipe.
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(g_epi.tma_c, sbuf, col0, split * g_epi.split_rows + row0_warp);
        bulk_commit_group();
      }
    }
    bias_a = bias_na; bias_b = bias_nb;
    gate_a = gate_na; gate_b = gate_nb;
  }
  return true;
}

// What the row-head epilogue needs, in shared memory like EpiShared (written once by thread 0).
struct HeadShared {
  float* C;
  const float* bias;
  long long ldc;
  int epi;                 // SB_EPI_BIAS / SB_EPI_RELU applied before the head
  float alpha, beta;
  SbRowHead rh;
};
__shared__ HeadShared g_head;

// One warp finishes the head rows of its TMEM lane quadrant: a thread holds the first W values of
// its row (the whole row when N <= W), applies scale / old C / bias / ReLU and hands over to the
// shared row head.  Out of line for the same reason as epilogue_tile.
template <int W>
__device__ __noinline__ void epilogue_head(uint32_t t_row, long long row, int M) {
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
  if (row >= M) return;
  float* v = reinterpret_cast<float*>(raw);
  const int n = g_head.rh.n;
  float* crow = g_head.C + row * g_head.ldc;
  const float alpha = g_head.alpha, beta = g_head.beta;
  const bool has_beta = beta != 0.0f, has_bias = (g_head.epi & SB_EPI_BIAS) != 0, relu = (g_head.epi & SB_EPI_RELU) != 0;
  const float* bias = g_head.bias;
#pragma unroll
  for (int j = 0; j < W; ++j) {
    if (j < n) {
      float x = alpha * v[j];
      if (has_beta) x += beta * crow[j];
      if (has_bias) x += __ldg(bias + j);
      if (relu) x = fmaxf(x, 0.f);
      v[j] = x;
    }
  }
  sb_row_head_finish<W>(g_head.rh, v, row, crow);
}

constexpr int EPI_HEAD_MASK = SB_EPI_MASKED_SOFTMAX | SB_EPI_REGRET_MATCHING | SB_EPI_ARGMAX | SB_EPI_SAMPLE | SB_EPI_BINARIZE;
constexpr int EPI_GATE_MASK = SB_EPI_RELU_MASK_OUT | SB_EPI_RELU_GRAD_MASK;

// PAIR = false: one CTA per 128 x block_n tile (cta_group::1).
// PAIR = true : a cluster of two CTAs per 256 x block_n tile (cta_group::2).
//   Each CTA loads its own 128 rows of A and its own half of the B columns
//   (plain TMA loads whose completion bytes are reported to the leader CTA's
//   full barrier); the leader CTA (cluster rank 0) issues every MMA with M = 256
//   and commits to the barriers of both CTAs; each CTA's epilogue drains its own
//   128 accumulator rows and arrives on the leader's tmem_empty barrier.  Halving
//   the B bytes each SM stages is what lifts the shared-memory ceiling of the
//   single-CTA form.
template <bool PAIR, bool TF32, int EW = UG_EPI_WARPS>
__global__ void __launch_bounds__(ug_threads(EW), 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a,
                 const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ UmmaOutMaps out_maps,
                 const __grid_constant__ UmmaGemmParams p) {
  extern __shared__ uint8_t ug_smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[UG_MAX_STAGES];
  __shared__ __align__(8) uint64_t bar_empty[UG_MAX_STAGES];
  __shared__ __align__(8) uint64_t bar_tmem_full[2];
  __shared__ __align__(8) uint64_t bar_tmem_empty[2];
  __shared__ uint32_t tmem_slot;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const uint32_t cta_rank = PAIR ? cluster_cta_rank() : 0u;
  const bool leader = cta_rank == 0u;
  // Work items are strided over CTAs (single) or over CTA pairs.
  const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int num_workers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  constexpr int TILE_M = PAIR ? 2 * UG_BLOCK_M : UG_BLOCK_M;

  // Stage buffers start on a 1024-byte boundary (one swizzle atom).
  const uint32_t raw_addr = smem_u32(ug_smem_raw);
  const uint32_t stage_base = (raw_addr + 1023u) & ~1023u;
  const uint32_t stage_bytes = p.a_stage_bytes + p.b_stage_bytes;

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bar_tmem_full[a]), 1);
      mbar_init(smem_u32(&bar_tmem_empty[a]), PAIR ? 2 * EW : EW);
    }
    g_abort_flag = 0;
    g_epi.c = p.C; g_epi.aux = p.aux_in; g_epi.bias = p.bias;
    g_epi.gate_in = (p.epi & SB_EPI_RELU_GRAD_MASK) ? reinterpret_cast<const uint32_t*>(p.aux_in) : nullptr;
    g_epi.gate_out = (p.epi & SB_EPI_RELU_MASK_OUT) ? reinterpret_cast<uint32_t*>(p.aux_out) : nullptr;
    g_epi.colsum = (p.epi & SB_EPI_COLSUM_OUT) ? reinterpret_cast<float*>(p.aux_out) : nullptr;
    g_epi.tma_c = p.tma_store ? &out_maps.m[0] : nullptr;
    g_epi.peer_rows = p.peer_rows;
    g_epi.ldc = p.ldc;
    g_epi.split_stride = p.split_stride;
    g_epi.M = p.M; g_epi.N = p.N; g_epi.block_n = p.block_n;
    g_epi.alpha = p.alpha; g_epi.beta = p.beta;
    g_epi.has_bias = (p.epi & SB_EPI_BIAS) ? 1 : 0; g_epi.relu = (p.epi & SB_EPI_RELU) ? 1 : 0;
    g_epi.relu_grad = (p.epi & SB_EPI_RELU_GRAD) ? 1 : 0; g_epi.coalesced = p.coalesced;
    g_epi.ln_l2 = (p.epi & SB_EPI_LN_L2) ? 1 : 0;
    g_epi.reduce_add = p.reduce_add; g_epi.split_rows = p.reduce_add ? 0 : p.M;
    g_epi.box_base = stage_base + p.epi_offset;
    g_head.C = reinterpret_cast<float*>(p.C); g_head.bias = p.bias; g_head.ldc = p.ldc; g_head.epi = p.epi;
    g_head.alpha = p.alpha; g_head.beta = p.beta; g_head.rh = p.head;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(smem_u32(&tmem_slot), (uint32_t)p.tmem_cols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(&tmem_slot), (uint32_t)p.tmem_cols);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  if (PAIR) cluster_sync_all(); else __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  volatile int* abortp = &g_abort_flag;
  // Everything above touched only this CTA's shared and tensor memory; from here on the
  // kernel reads what earlier kernels on the stream wrote.
  sb_grid_dependency_wait();
  sb_grid_dependents_launch();

  if (warp == 0 || warp == 2 + EW) {
    // Two producer threads: warp 0 arms the stage's barrier and loads A, the last warp loads B.  One thread
    // issuing all four loads of a stage measured 3 % slower on main-loop-bound GEMMs (4096^3: 1307 ->
    // 1346 TFLOP/s): a TMA instruction occupies its thread for long enough to matter.  A load whose
    // bytes land before the barrier is armed is in order: the transaction count may run negative.
    const bool do_a = warp == 0, do_b = !do_a;
    if (lane == 0) {
      // The issue loop of a single thread: keep it to a handful of instructions
      // per k-block (addresses advance by adds, nothing is recomputed).
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const int b_cols = PAIR ? p.block_n / 2 : p.block_n;   // half of the B columns per CTA in a pair
      const uint32_t full0_local = smem_u32(&bar_full[0]);
      const uint32_t full0 = PAIR ? map_to_cta(full0_local, 0u) : full0_local;
      const uint32_t empty0 = smem_u32(&bar_empty[0]);
      const bool a_mn = p.a_mn != 0, b_mn = p.b_mn != 0;
      const int a_boxes = p.a_boxes, mn_box_elems = p.mn_box_elems, block_k = p.block_k;
      const uint32_t mn_box_bytes = p.mn_box_bytes, a_stage_bytes = p.a_stage_bytes;
      const int subs = p.subs;
      const uint32_t a_sub_bytes = p.a_sub_bytes, b_sub_bytes = p.b_sub_bytes;
      const int stages = p.stages;
      uint32_t a_dst = stage_base;
      WorkIter it(p, worker, num_workers);
      int tile, split, kb_begin, kb_end, half;
      while (ok && it.next(p, tile, split, kb_begin, kb_end, half)) {
        int m_blk, n_blk;
        tile_coords(p, tile, m_blk, n_blk);
        const int m0 = m_blk * TILE_M + (int)cta_rank * UG_BLOCK_M;
        // A half tile: half as many B columns per CTA (half the boxes, or a tensor map with half-height boxes).
        const int item_cols = half < 0 ? b_cols : b_cols / 2;
        const int n0 = n_blk * p.block_n + (half > 0 ? p.block_n / 2 : 0) + (int)cta_rank * item_cols;
        const CUtensorMap* map_b = half < 0 ? &tmap_b : &out_maps.b_tail;
        const int b_boxes = half < 0 ? p.b_boxes : p.b_boxes / 2;
        const uint32_t item_b_bytes = half < 0 ? p.b_stage_bytes : p.b_stage_bytes / 2u;
        const uint32_t tx_bytes = PAIR ? 2u * (a_stage_bytes + item_b_bytes) : a_stage_bytes + item_b_bytes;
        int k0 = kb_begin * block_k;
        for (int kb = kb_begin; kb < kb_end; ++kb, k0 += block_k) {
          if (!mbar_wait(empty0 + 8u * (uint32_t)stage, phase ^ 1u, abortp, SB_SITE_PRODUCER_EMPTY)) {
            ok = false;
            break;
          }
          // In a pair only the leader arms its full barrier, with the bytes of both CTAs.
          if (do_a && (!PAIR || leader)) mbar_arrive_expect_tx(full0_local + 8u * (uint32_t)stage, tx_bytes);
          const uint32_t full = full0 + 8u * (uint32_t)stage;
          const uint32_t b_dst = a_dst + a_stage_bytes;
          if (!do_a) {
          } else if (!a_mn) {
            for (int s = 0; s < subs; ++s) {
              if (PAIR) tma_load_2d_pair(a_dst + (uint32_t)s * a_sub_bytes, &tmap_a, k0 + s * mn_box_elems, m0, full);
              else tma_load_2d(a_dst + (uint32_t)s * a_sub_bytes, &tmap_a, k0 + s * mn_box_elems, m0, full);
            }
          } else {
            for (int i = 0; i < a_boxes; ++i) {
              if (PAIR) tma_load_2d_pair(a_dst + (uint32_t)i * mn_box_bytes, &tmap_a, m0 + i * mn_box_elems, k0, full);
              else tma_load_2d(a_dst + (uint32_t)i * mn_box_bytes, &tmap_a, m0 + i * mn_box_elems, k0, full);
            }
          }
          if (!do_b) {
          } else if (!b_mn) {
            for (int s = 0; s < subs; ++s) {
              if (PAIR) tma_load_2d_pair(b_dst + (uint32_t)s * b_sub_bytes, map_b, k0 + s * mn_box_elems, n0, full);
              else tma_load_2d(b_dst + (uint32_t)s * b_sub_bytes, map_b, k0 + s * mn_box_elems, n0, full);
            }
          } else {
            for (int i = 0; i < b_boxes; ++i) {
              if (PAIR) tma_load_2d_pair(b_dst + (uint32_t)i * mn_box_bytes, &tmap_b, n0 + i * mn_box_elems, k0, full);
              else tma_load_2d(b_dst + (uint32_t)i * mn_box_bytes, &tmap_b, n0 + i * mn_box_elems, k0, full);
            }
          }
          a_dst += stage_bytes;
          if (++stage == stages) {
            stage = 0;
            phase ^= 1u;
            a_dst = stage_base;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      // tcgen05.mma issue blocks while the tensor pipe's short queue is full, so
      // every other instruction of this thread is time the pipe may run dry:
      // descriptors are kept as (lo, hi) words, the lo word advances by adds.
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      // K-major: LBO unused (1), SBO = 1024 (8 rows x 128 B).
      // MN-major: LBO = bytes between 128-byte MN segments (one TMA box),
      //           SBO = bytes between k-row groups: 1024 (8 rows) for 16-bit
      //           types, 512 (4 rows) for the 32-byte-chunk swizzle of TF32.
      const uint64_t a_desc0 = umma_smem_desc(stage_base, p.a_mn ? p.mn_box_bytes : 16u, p.a_sbo, p.a_layout);
      const uint64_t b_desc0 = umma_smem_desc(stage_base + p.a_stage_bytes, p.b_mn ? p.mn_box_bytes : 16u, p.b_sbo, p.b_layout);
      const uint32_t a_hi = (uint32_t)(a_desc0 >> 32), b_hi = (uint32_t)(b_desc0 >> 32);
      const uint32_t a_lo0 = (uint32_t)a_desc0, b_lo0 = (uint32_t)b_desc0;
      const uint32_t stage_step = stage_bytes >> 4;
      const uint32_t a_kstep = p.a_kstep, b_kstep = p.b_kstep;
      const uint32_t a_sub_step = p.a_sub_step, b_sub_step = p.b_sub_step;
      const bool two_subs = p.subs == 2;
      const uint32_t full0 = smem_u32(&bar_full[0]), empty0 = smem_u32(&bar_empty[0]);
      const int stages = p.stages;
      uint32_t a_lo = a_lo0, b_lo = b_lo0;
      WorkIter it(p, worker, num_workers);
      int tile, split, kb_begin, kb_end, half;
      while (ok && it.next(p, tile, split, kb_begin, kb_end, half)) {
        const uint32_t idesc = half < 0 ? p.idesc : p.idesc_tail;
        if (!mbar_wait(smem_u32(&bar_tmem_empty[acc]), acc_phase ^ 1u, abortp, SB_SITE_MMA_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * p.acc_stride);
        uint32_t accumulate = 0u;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(full0 + 8u * (uint32_t)stage, phase, abortp, SB_SITE_MMA_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          umma_issue<PAIR, TF32>(d_tmem, a_lo, a_hi, b_lo, b_hi, idesc, accumulate);
          umma_issue<PAIR, TF32>(d_tmem, a_lo + a_kstep, a_hi, b_lo + b_kstep, b_hi, idesc, 1u);
          umma_issue<PAIR, TF32>(d_tmem, a_lo + 2u * a_kstep, a_hi, b_lo + 2u * b_kstep, b_hi, idesc, 1u);
          umma_issue<PAIR, TF32>(d_tmem, a_lo + 3u * a_kstep, a_hi, b_lo + 3u * b_kstep, b_hi, idesc, 1u);
          if (two_subs) {
            const uint32_t a2 = a_lo + a_sub_step, b2 = b_lo + b_sub_step;
            umma_issue<PAIR, TF32>(d_tmem, a2, a_hi, b2, b_hi, idesc, 1u);
            umma_issue<PAIR, TF32>(d_tmem, a2 + a_kstep, a_hi, b2 + b_kstep, b_hi, idesc, 1u);
            umma_issue<PAIR, TF32>(d_tmem, a2 + 2u * a_kstep, a_hi, b2 + 2u * b_kstep, b_hi, idesc, 1u);
            umma_issue<PAIR, TF32>(d_tmem, a2 + 3u * a_kstep, a_hi, b2 + 3u * b_kstep, b_hi, idesc, 1u);
          }
          accumulate = 1u;
          if (PAIR) tc_commit_pair(empty0 + 8u * (uint32_t)stage, (uint16_t)3);
          else tc_commit(empty0 + 8u * (uint32_t)stage);
          a_lo += stage_step;
          b_lo += stage_step;
          if (++stage == stages) {
            stage = 0;
            phase ^= 1u;
            a_lo = a_lo0;
            b_lo = b_lo0;
          }
        }
        if (!ok) break;
        if (PAIR) tc_commit_pair(smem_u32(&bar_tmem_full[acc]), (uint16_t)3);
        else tc_commit(smem_u32(&bar_tmem_full[acc]));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else if (warp < 2 + EW) {
    // Epilogue warps.  A warp may only read the TMEM lane quadrant given by its index
    // modulo 4; with 8 warps the two warps of a quadrant take alternate 32-column chunks.
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool head = (p.epi & EPI_HEAD_MASK) != 0;
    // Which compile-time variant of the epilogue serves this launch (see coalesced_chunk).
    int epi_mode = (p.beta != 0.0f || (p.epi & SB_EPI_RELU_GRAD)) ? -2 : -1;
    if (epi_mode == -1 && p.alpha == 1.0f && !(p.epi & SB_EPI_LN_L2)) {
      const int flags = ((p.epi & SB_EPI_BIAS) ? 1 : 0) | ((p.epi & SB_EPI_RELU) ? 2 : 0) |
                        ((p.epi & SB_EPI_RELU_MASK_OUT) ? 4 : 0) | ((p.epi & SB_EPI_RELU_GRAD_MASK) ? 8 : 0) |
                        ((p.epi & SB_EPI_COLSUM_OUT) ? 16 : 0);
      if (flags == 0 || flags == 3 || flags == 7 || flags == 8 || flags == 16 || flags == 24) epi_mode = flags;
    }
    WorkIter it(p, worker, num_workers);
    int tile, split, kb_begin, kb_end, half_tile;
    while (it.next(p, tile, split, kb_begin, kb_end, half_tile)) {
      int m_blk, n_blk;
      tile_coords(p, tile, m_blk, n_blk);
      const int item_n = half_tile < 0 ? p.block_n : p.block_n / 2;
      const int row0_warp = m_blk * TILE_M + (int)cta_rank * UG_BLOCK_M + quad * 32;
      const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * p.acc_stride);
      const uint32_t full_bar = smem_u32(&bar_tmem_full[acc]);
      if (EW == 8 && head) {           // row heads always run on the eight-warp instance
        if constexpr (EW == 8) {
          if (!mbar_wait(full_bar, acc_phase, abortp, SB_SITE_EPI_TMEM_FULL)) break;
          tc_fence_after_sync();
          if (half == 0) {               // a thread finishes a whole head row: the second warp of the quadrant idles
            if (p.block_n > 32) epilogue_head<64>(t_row, (long long)row0_warp + lane, p.M);
            else if (p.block_n > 16) epilogue_head<32>(t_row, (long long)row0_warp + lane, p.M);
            else epilogue_head<16>(t_row, (long long)row0_warp + lane, p.M);
          }
        }
      } else {
        const int n0 = n_blk * p.block_n + (half_tile > 0 ? item_n : 0);
        bool ok;
#define SB_EPI_CALL(T, R, G) epilogue_tile<T, R, G, EW>(t_row, row0_warp, n0, item_n, split, full_bar, acc_phase)
#define SB_EPI_WIDE(T, G) epilogue_tile_wide<T, (G) == -2 ? -1 : (G)>(t_row, row0_warp, n0, item_n, split, full_bar, acc_phase)
#define SB_EPI_BY_TYPE(G)                                                        \
  do {                                                                           \
    if constexpr (EW == 16) {            /* 16-bit outputs only, one 32 x 32 box per chunk */ \
      if (p.out_dtype == SB_BF16) ok = SB_EPI_CALL(__nv_bfloat16, false, G);     \
      else ok = SB_EPI_CALL(__half, false, G);                                   \
    } else {                                                                     \
      if (p.out_dtype == SB_F32) ok = SB_EPI_CALL(float, false, G);              \
      else if (p.out_dtype == SB_TF32) ok = SB_EPI_CALL(float, true, G);         \
      else if (p.out_dtype == SB_BF16)                                           \
        ok = (p.wide && (G) != -2) ? SB_EPI_WIDE(__nv_bfloat16, G) : SB_EPI_CALL(__nv_bfloat16, false, G); \
      else ok = (p.wide && (G) != -2) ? SB_EPI_WIDE(__half, G) : SB_EPI_CALL(__half, false, G);            \
    }                                                                            \
  } while (0)
        switch (epi_mode) {
          case 0: SB_EPI_BY_TYPE(0); break;        // plain: standalone GEMMs, wgrad partials
          case 3: SB_EPI_BY_TYPE(3); break;        // bias + ReLU: inference layers
          case 7: SB_EPI_BY_TYPE(7); break;        // bias + ReLU + sign bits: training forward
          case 8: SB_EPI_BY_TYPE(8); break;        // gate by sign bits: dgrad
          case 16: SB_EPI_BY_TYPE(16); break;      // plain + column sums
          case 24: SB_EPI_BY_TYPE(24); break;      // dgrad that also sums its output columns (bias gradient)
          case -2: SB_EPI_BY_TYPE(-2); break;
          default: SB_EPI_BY_TYPE(-1); break;
        }
#undef SB_EPI_BY_TYPE
#undef SB_EPI_WIDE
#undef SB_EPI_CALL
        if (!ok) break;
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        // The MMA issuer (leader CTA) owns the tmem_empty barrier of the pair.
        if (PAIR) mbar_arrive_cluster(map_to_cta(smem_u32(&bar_tmem_empty[acc]), 0u));
        else mbar_arrive(smem_u32(&bar_tmem_empty[acc]));
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  // Teardown.  Bulk stores of the epilogue must have completed; after an expired wait, give copies and MMAs in flight time to
  // land before shared and tensor memory are released.  In a pair neither CTA
  // may leave while its peer can still touch its shared memory or barriers.
  if (warp >= 2 && warp < 2 + EW && lane == 0) bulk_wait_group<0>();
  __syncwarp();
  tc_fence_before_sync();
  if (PAIR) cluster_sync_all(); else __syncthreads();
  if (*abortp != 0) {
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) { }
  }
  if (PAIR) cluster_sync_all(); else __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    if (PAIR) tmem_dealloc_pair(tmem_base, (uint32_t)p.tmem_cols);
    else tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

// ------------------------------- host side ----------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// 2-D row-major tensor [rows, cols] -> tensor map with box [box_rows, box_cols],
// 128-byte swizzle (box_cols * elem size must be 128 bytes), zero fill outside.
// `swz`: SWZ_128 (16-byte chunks), SWZ_128_CHUNK32 (32-byte chunks, MN-major
// TF32 operands) or SWZ_64 (64-byte rows, 16-bit output boxes).
enum TmapSwizzle { SWZ_128 = 0, SWZ_128_CHUNK32 = 1, SWZ_64 = 2 };

int make_tmap_2d(CUtensorMap* map, const void* base, int in_dtype, long long rows, long long cols,
                 int box_rows, int box_cols, int swz) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return sb_fail(SB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const int es = sb_dtype_size(in_dtype);
  CUtensorMapDataType dt = in_dtype == SB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : in_dtype == SB_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)cols * (cuuint64_t)es};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swz == SWZ_128_CHUNK32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                   : swz == SWZ_64      ? CU_TENSOR_MAP_SWIZZLE_64B
                                        : CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return sb_fail(SB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (rows=%lld cols=%lld box=%dx%d)",
                   (int)r, rows, cols, box_rows, box_cols);
  return SB_OK;
}

// Shared memory per SM that the GEMM's pipeline leaves unused so that CTAs of another kernel can be
// resident beside a GEMM CTA (sb_gemm_reserve_smem).
std::atomic<int> g_gemm_smem_reserve{0};

// SB_NO_PAIR=1 in the environment keeps every GEMM on single-CTA tiles.
bool sb_pair_mode_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("SB_NO_PAIR");
    v = (e && e[0] == '1') ? 0 : 1;
  }
  return v == 1;
}

// SB_EPI_WARPS=8 in the environment keeps every GEMM on eight epilogue warps.
bool tail_split_enabled() {
  static const bool on = [] {
    const char* e = getenv("SB_TAIL_SPLIT");     // SB_TAIL_SPLIT=0 keeps whole tiles in the last wave (tuning runs)
    return !(e && e[0] == '0');
  }();
  return on;
}

bool epi16_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("SB_EPI_WARPS");
    v = (e && atoi(e) == 8) ? 0 : 1;
  }
  return v == 1;
}

int round_up_int(int x, int m) { return (x + m - 1) / m * m; }
int next_pow2(int x) {
  int p = 32;
  while (p < x) p <<= 1;
  return p;
}

int cached_sm_count() { return sb_sm_count(); }

// Chooses block_n / stages / grid for a problem; `sms` = SM count to plan for.
// `allow_pair`: CTA pairs may be used (needs at least two 128-row blocks and a
// tile at least 64 columns wide; row heads stay on single CTAs).
void plan_umma(UmmaGemmParams& p, int in_dtype, int sms, bool allow_pair, bool chunks32 = false) {
  const int es = sb_dtype_size(in_dtype);
  p.mn_box_elems = 128 / es;
  p.pair = (allow_pair && p.M > UG_BLOCK_M && p.N >= 64 && sms >= 2) ? 1 : 0;
  const int tile_m = p.pair ? 2 * UG_BLOCK_M : UG_BLOCK_M;
  const int workers = p.pair ? sms / 2 : sms;
  p.tiles_m = (p.M + tile_m - 1) / tile_m;
  // Column granularity of a tile: 16 for a K-major B (32 in a pair, 16 per CTA);
  // an MN-major B needs whole 128-byte boxes per CTA.
  int gran = (p.b_mn ? p.mn_box_elems : 16) * (p.pair ? 2 : 1);
  if (chunks32 && gran < 32) gran = 32;   // the ReLU sign words cover whole 32-column chunks
  int best_bn = 0;
  if (p.N <= 256) {
    best_bn = round_up_int(p.N, gran);
  } else {
    // Minimise (waves of tiles over the workers) x (cost of one tile); tiles
    // narrower than 192 columns stage too many operand bytes per flop, so they
    // are not considered for wide problems.
    double best_cost = 1e30;
    for (int bn = 256; bn >= 192; bn -= 16) {
      if (bn % gran) continue;
      const long long tiles = (long long)p.tiles_m * ((p.N + bn - 1) / bn);
      const long long waves = (tiles + workers - 1) / workers;
      // a tile's time grows with its width plus a fixed part (pipeline fill, drain of the last chunk pair,
      // and the operand bytes staged per flop, which rise as the tile narrows): 256 x 192 tiles in five
      // waves measured 9 % slower than 256 x 256 in four on 4096^3
      const double cost = (double)waves * (bn + 96);
      if (cost < best_cost - 1e-9) {
        best_cost = cost;
        best_bn = bn;
      }
    }
  }
  p.block_n = best_bn;
  p.tiles_n = (p.N + p.block_n - 1) / p.block_n;
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.splits = 1;
  p.kb_per_split = p.k_blocks;
  p.num_work = p.num_tiles;
  p.split_stride = 0;
  p.acc_stride = next_pow2(p.block_n);
  p.tmem_cols = next_pow2(2 * p.acc_stride);
  // Per CTA: 128 rows of A and all (single) or half (pair) of the B columns.
  const int b_cols = p.pair ? p.block_n / 2 : p.block_n;
  // A stage holds one or two 128-byte sub-blocks of K.  Two halve the barrier
  // rounds per flop (the issue thread's fixed cost per round is what keeps the
  // tensor pipe from running back to back); they are used when at least three
  // such stages still fit and K is long enough to fill them.
  const int sub_bytes = (UG_BLOCK_M + b_cols) * 128;
  const int budget = UG_SMEM_LIMIT - 2048 - UG_EPI_STAGING - g_gemm_smem_reserve.load(std::memory_order_relaxed);
  const int sub_k = 128 / es;
  p.subs = (budget / (2 * sub_bytes) >= 3 && p.K >= 6 * sub_k) ? 2 : 1;
  p.block_k = p.subs * sub_k;
  p.k_blocks = (p.K + p.block_k - 1) / p.block_k;
  p.kb_per_split = p.k_blocks;
  p.mn_box_bytes = (uint32_t)p.block_k * 128u;
  p.a_sub_bytes = UG_BLOCK_M * 128u;
  p.b_sub_bytes = (uint32_t)b_cols * 128u;
  p.a_stage_bytes = (uint32_t)p.subs * p.a_sub_bytes;
  p.b_stage_bytes = (uint32_t)p.subs * p.b_sub_bytes;
  // Every stage stays 1024-byte aligned: b_cols is a multiple of 16.
  p.a_boxes = p.a_mn ? UG_BLOCK_M / p.mn_box_elems : 1;
  p.b_boxes = p.b_mn ? b_cols / p.mn_box_elems : 1;
  const int stage_bytes = (int)(p.a_stage_bytes + p.b_stage_bytes);
  int stages = budget / stage_bytes;
  if (stages > UG_MAX_STAGES) stages = UG_MAX_STAGES;
  if (stages > p.k_blocks && p.k_blocks >= 2) stages = max(2, p.k_blocks);
  if (stages < 2) stages = 2;
  p.stages = stages;
  p.epi_offset = (uint32_t)stages * (uint32_t)stage_bytes;
  // Per-MMA descriptor step: K-major advances 32 bytes inside the swizzle
  // atom; MN-major advances (UMMA_K / 8) groups of 8 k-rows (1024 B each).
  const int umma_k = 32 / es;
  p.a_kstep = p.a_mn ? (uint32_t)((umma_k / 8) * 1024 / 16) : 2u;
  p.b_kstep = p.b_mn ? (uint32_t)((umma_k / 8) * 1024 / 16) : 2u;
  // Second sub-block: MN-major tiles simply continue along K (4 more k-steps);
  // K-major tiles start a new [rows x 128 B] slab.
  p.a_sub_step = p.a_mn ? 4u * p.a_kstep : p.a_sub_bytes / 16u;
  p.b_sub_step = p.b_mn ? 4u * p.b_kstep : p.b_sub_bytes / 16u;
  p.kind_tf32 = (in_dtype == SB_TF32) ? 1 : 0;
  const bool a32 = p.a_mn && es == 4, b32 = p.b_mn && es == 4;
  p.a_layout = a32 ? 1u : 2u;
  p.b_layout = b32 ? 1u : 2u;
  p.a_sbo = a32 ? 512u : 1024u;
  p.b_sbo = b32 ? 512u : 1024u;
  p.idesc = sb_umma_idesc(in_dtype, p.a_mn, p.b_mn, tile_m, p.block_n);
}

size_t umma_dyn_smem(const UmmaGemmParams& p) {
  return (size_t)p.stages * (p.a_stage_bytes + p.b_stage_bytes) + UG_EPI_STAGING + 1024;
}

__global__ void scale_rows_kernel(void* C, long long total, float beta, int out_dtype) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long step = (long long)gridDim.x * blockDim.x;
  for (; i < total; i += step) {
    if (out_dtype == SB_F32 || out_dtype == SB_TF32) {
      float* c = reinterpret_cast<float*>(C);
      c[i] = beta == 0.f ? 0.f : beta * c[i];
    } else if (out_dtype == SB_BF16) {
      __nv_bfloat16* c = reinterpret_cast<__nv_bfloat16*>(C);
      c[i] = __float2bfloat16_rn(beta == 0.f ? 0.f : beta * __bfloat162float(c[i]));
    } else {
      __half* c = reinterpret_cast<__half*>(C);
      c[i] = __float2half_rn(beta == 0.f ? 0.f : beta * __half2float(c[i]));
    }
  }
}

}  // namespace

// Launches the tensor-core GEMM.  All argument validation happens here, so a
// bad call never reaches the device.
int sb_umma_gemm_launch(int a_trans, int b_trans, float alpha, const void* A, const void* B,
                        float beta, void* C, int M, int N, int K, int in_dtype, int out_dtype,
                        int epi, const float* bias, const uint8_t* mask, const void* aux_in,
                        void* aux_out, cudaStream_t stream, int splits, int* splits_used, const SbRowHead* head,
                        void* split_partials, const SbPeerOut* peer_out) {
  const bool to_peers = peer_out && peer_out->n > 1;
  if (to_peers) {
    if (!sb_umma_peer_out_ok(M, N, peer_out->n) || out_dtype != SB_F32 || epi != 0 || beta != 0.0f || alpha != 1.0f)
      return sb_fail(SB_ERR_UNSUPPORTED, "GEMM into peer copies: plain fp32 product with whole 128-row blocks per rank only");
    for (int r = 0; r < peer_out->n; ++r)
      if (!peer_out->c[r] || (reinterpret_cast<uintptr_t>(peer_out->c[r]) & 15))
        return sb_fail(SB_ERR_MISALIGNED, "GEMM into peer copies: copy %d is null or not 16-byte aligned", r);
    C = peer_out->c[0];
  }
  const int es = sb_dtype_size(in_dtype);
  UmmaGemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K;
  p.a_mn = a_trans ? 1 : 0;   // A stored [K,M]: M contiguous
  p.b_mn = b_trans ? 0 : 1;   // B stored [K,N]: N contiguous
  // Whole 32-column chunks per tile where every chunk must leave as a box: sign words, column sums, and
  // tiles that are added to C (split-K accumulation, peer copies).
  plan_umma(p, in_dtype, cached_sm_count(), !(epi & EPI_HEAD_MASK) && sb_pair_mode_enabled(),
            (epi & (EPI_GATE_MASK | SB_EPI_COLSUM_OUT)) != 0 || (split_partials && splits > 1) || to_peers);
  p.alpha = alpha; p.beta = beta;
  p.C = C; p.ldc = N; p.out_dtype = out_dtype;
  p.epi = epi; p.bias = bias; p.mask = mask; p.aux_in = aux_in; p.aux_out = aux_out;
  if (epi & EPI_HEAD_MASK) {
    if (head) {
      p.head = *head;
    } else {
      p.head.prefix = -1;
      p.head.mask = mask;
      p.head.argmax_out = reinterpret_cast<int32_t*>(aux_out);
    }
    p.head.n = N;
    p.head.flags = epi & EPI_HEAD_MASK;
    if (!sb_umma_head_fits(N, p.head.prefix))
      return sb_fail(SB_ERR_UNSUPPORTED, "a fused row head holds %d columns (%d under a prefix mask of at most %d)",
                     UG_HEAD_MAX_N, UG_HEAD_MAX_TILE_N, UG_HEAD_MAX_N);
  }

  // TMA needs 16-byte aligned bases and row pitches.
  const long long lda = a_trans ? M : K;
  const long long ldb = b_trans ? K : N;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return sb_fail(SB_ERR_MISALIGNED, "GEMM operand base pointers must be 16-byte aligned");
  if ((lda * es) % 16 != 0 || (ldb * es) % 16 != 0)
    return sb_fail(SB_ERR_MISALIGNED,
                   "GEMM operand row pitch must be a multiple of 16 bytes (lda=%lld ldb=%lld elem=%d B)",
                   lda, ldb, es);

  CUtensorMap ta, tb;
  int rc;
  if (!p.a_mn) rc = make_tmap_2d(&ta, A, in_dtype, M, K, UG_BLOCK_M, p.mn_box_elems, SWZ_128);
  else rc = make_tmap_2d(&ta, A, in_dtype, K, M, p.block_k, p.mn_box_elems, p.a_layout == 1u ? SWZ_128_CHUNK32 : SWZ_128);
  if (rc != SB_OK) return rc;
  if (!p.b_mn) rc = make_tmap_2d(&tb, B, in_dtype, N, K, p.pair ? p.block_n / 2 : p.block_n, p.mn_box_elems, SWZ_128);
  else rc = make_tmap_2d(&tb, B, in_dtype, K, N, p.block_k, p.mn_box_elems, p.b_layout == 1u ? SWZ_128_CHUNK32 : SWZ_128);
  if (rc != SB_OK) return rc;

  if (splits > 1) {
    // Split-K: each split writes its own [M,N] partial at C + split * M * N.
    int kbps = (p.k_blocks + splits - 1) / splits;
    if (kbps < 1) kbps = 1;
    p.kb_per_split = kbps;
    p.splits = (p.k_blocks + kbps - 1) / kbps;   // every split owns at least one k-block
    p.num_work = p.num_tiles * p.splits;
    p.split_stride = (long long)M * N;
    if (split_partials && p.splits > 1 && !to_peers) {
      // Accumulating form: fp32 output, every chunk of a tile leaves as a TMA box (whole 32-column
      // chunks, 16-byte aligned rows), nothing else in the epilogue.
      if (out_dtype == SB_F32 && epi == 0 && beta == 0.0f && p.block_n % 32 == 0 &&
          ((long long)N * 4) % 16 == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0) {
        p.reduce_add = 1;
        p.split_stride = 0;
      } else {
        p.C = C = split_partials;
      }
    }
  }
  if (to_peers) {
    if (p.block_n % 32 != 0) return sb_fail(SB_ERR_UNSUPPORTED, "GEMM into peer copies: the tile plan leaves a 16-column tail");
    p.reduce_add = 1;
    p.split_stride = 0;
    p.peer_rows = M / peer_out->n;
  }
  if (splits_used) *splits_used = p.reduce_add ? 1 : p.splits;

  // Row-contiguous (coalesced) stores need a 16-byte aligned base and row pitch;
  // anything else falls back to per-thread stores.  Row heads write directly.
  const int es_out = out_dtype == SB_BF16 || out_dtype == SB_F16 ? 2 : 4;
  p.coalesced = (!(epi & EPI_HEAD_MASK) && ((long long)N * es_out) % 16 == 0 &&
                 (reinterpret_cast<uintptr_t>(C) & 15) == 0 &&
                 (!(epi & SB_EPI_RELU_GRAD) || (reinterpret_cast<uintptr_t>(aux_in) & 15) == 0)) ? 1 : 0;

  if (!p.coalesced && (epi & (EPI_GATE_MASK | SB_EPI_COLSUM_OUT)))
    return sb_fail(SB_ERR_MISALIGNED, "the sign-bit and column-sum epilogues need a 16-byte aligned C");
  if (epi & SB_EPI_LN_L2) {
    if (epi & EPI_HEAD_MASK) return sb_fail(SB_ERR_UNSUPPORTED, "SB_EPI_LN_L2 cannot be combined with a row head");
    if (p.tiles_n != 1 || N % 32 != 0 || !p.coalesced)
      return sb_fail(SB_ERR_UNSUPPORTED, "SB_EPI_LN_L2 needs N <= 256, N %% 32 == 0 and a 16-byte aligned C (N=%d)", N);
  }

  // TMA stores of the finished boxes: no second tile is read (beta, activation gate), and with
  // split-K -- the partials form one [splits * M, N] tensor -- no 32-row box may straddle two partials.
  UmmaOutMaps tc;
  memset(&tc, 0, sizeof(tc));
  p.tma_store = 0;
  if (p.coalesced && beta == 0.0f && !(epi & SB_EPI_RELU_GRAD) && (p.splits == 1 || p.reduce_add || M % 32 == 0)) {
    const int cdt = es_out == 4 ? SB_F32 : out_dtype;
    // Sixteen epilogue warps: CTA-pair tiles with a 16-bit output and next to no main loop; one 32 x 32
    // box per chunk, no 64-column boxes.
    p.epi_warps = (p.pair && es_out == 2 && !(epi & EPI_HEAD_MASK) && p.block_n % 32 == 0 && p.k_blocks <= 2 &&
                   epi16_enabled()) ? 16 : 8;
    p.wide = (es_out == 2 && p.block_n % 64 == 0 && !(epi & SB_EPI_LN_L2) && p.epi_warps == 8) ? 1 : 0;
    for (int r = 0; r < (to_peers ? peer_out->n : 1); ++r) {
      rc = make_tmap_2d(&tc.m[r], to_peers ? peer_out->c[r] : C, cdt, p.reduce_add ? (long long)M : (long long)M * p.splits, N,
                        32, p.wide ? 64 : 32, (es_out == 4 || p.wide) ? SWZ_128 : SWZ_64);
      if (rc != SB_OK) return rc;
    }
    p.tma_store = 1;
  }
  if (p.epi_warps == 0) p.epi_warps = 8;
  // A last wave that would fill at most half of the pairs is cut into half-width tiles (twice as many
  // items, each about half as long): 4096^3 is 256 tiles on 74 pairs, three full waves and 34 tiles.
  p.tail_first = p.num_work;
  p.idesc_tail = p.idesc;
  if (p.pair && p.splits == 1 && !to_peers && !(epi & (EPI_HEAD_MASK | SB_EPI_LN_L2)) && p.block_n % 128 == 0 &&
      tail_split_enabled()) {
    const int workers = cached_sm_count() / 2;
    const int rem = workers > 0 ? p.num_tiles % workers : 0;
    if (p.num_tiles > workers && rem > 0 && 2 * rem <= workers) {
      p.tail_first = p.num_tiles - rem;
      p.num_work = p.num_tiles + rem;
      p.idesc_tail = sb_umma_idesc(in_dtype, p.a_mn, p.b_mn, 2 * UG_BLOCK_M, p.block_n / 2);
      if (!p.b_mn) {
        rc = make_tmap_2d(&tc.b_tail, B, in_dtype, N, K, p.block_n / 4, p.mn_box_elems, SWZ_128);
        if (rc != SB_OK) return rc;
      }
    }
  }
  if (p.reduce_add && !p.tma_store)
    return sb_fail(SB_ERR_UNSUPPORTED, "internal: split-K accumulation was chosen for a C that cannot take TMA stores");
  const size_t smem = umma_dyn_smem(p);
  static std::atomic<bool> attr_set[64];
  int dev = 0;
  SB_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[dev].load(std::memory_order_acquire)) {   // setting it twice is harmless
    SB_CUDA(cudaFuncSetAttribute(umma_gemm_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, UG_SMEM_LIMIT - 2048));
    SB_CUDA(cudaFuncSetAttribute(umma_gemm_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, UG_SMEM_LIMIT - 2048));
    SB_CUDA(cudaFuncSetAttribute(umma_gemm_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, UG_SMEM_LIMIT - 2048));
    SB_CUDA(cudaFuncSetAttribute(umma_gemm_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, UG_SMEM_LIMIT - 2048));
    SB_CUDA(cudaFuncSetAttribute(umma_gemm_kernel<true, false, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, UG_SMEM_LIMIT - 2048));
    attr_set[dev].store(true, std::memory_order_release);
  }
  sb_prof_before(stream);
  if (!p.pair) {
    const int grid = min(p.num_work, cached_sm_count());
    if (p.kind_tf32) SB_CUDA(sb_launch(umma_gemm_kernel<false, true>, dim3(grid), dim3(ug_threads(8)), smem, stream, 1, ta, tb, tc, p));
    else SB_CUDA(sb_launch(umma_gemm_kernel<false, false>, dim3(grid), dim3(ug_threads(8)), smem, stream, 1, ta, tb, tc, p));
  } else {
    // One cluster of two CTAs per worker; the two CTAs of a cluster share a TPC.
    const int workers = min(p.num_work, cached_sm_count() / 2);
    if (p.kind_tf32) SB_CUDA(sb_launch(umma_gemm_kernel<true, true>, dim3(2 * workers), dim3(ug_threads(8)), smem, stream, 2, ta, tb, tc, p));
    else if (p.epi_warps == 16) SB_CUDA(sb_launch(umma_gemm_kernel<true, false, 16>, dim3(2 * workers), dim3(ug_threads(16)), smem, stream, 2, ta, tb, tc, p));
    else SB_CUDA(sb_launch(umma_gemm_kernel<true, false>, dim3(2 * workers), dim3(ug_threads(8)), smem, stream, 2, ta, tb, tc, p));
  }
  sb_prof_after(stream, 2.0 * M * N * K);
  SB_COUNT_LAUNCH();
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

extern "C" int sb_gemm_reserve_smem(int bytes) {
  if (bytes < 0 || bytes > 64 * 1024) return sb_fail(SB_ERR_BAD_ARG, "sb_gemm_reserve_smem: between 0 and 65536 bytes");
  g_gemm_smem_reserve.store((bytes + 1023) / 1024 * 1024, std::memory_order_relaxed);
  return SB_OK;
}

int sb_umma_plan(int a_trans, int b_trans, int M, int N, int K, int in_dtype, int sms, int* plan5) {
  UmmaGemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K;
  p.a_mn = a_trans ? 1 : 0;
  p.b_mn = b_trans ? 0 : 1;
  plan_umma(p, in_dtype, sms, sb_pair_mode_enabled());
  plan5[0] = p.pair ? 2 * UG_BLOCK_M : UG_BLOCK_M;
  plan5[1] = p.block_n;
  plan5[2] = p.block_k;
  plan5[3] = p.stages;
  plan5[4] = p.pair ? 2 * min(p.num_tiles, sms / 2) : min(p.num_tiles, sms);
  return SB_OK;
}

int sb_scale_launch(void* C, long long total, float beta, int out_dtype, cudaStream_t stream) {
  if (total <= 0) return SB_OK;
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)sb_sm_count() * 8;
  if (blocks > cap) blocks = cap;
  scale_rows_kernel<<<(int)blocks, 256, 0, stream>>>(C, total, beta, out_dtype);
  SB_COUNT_LAUNCH();
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

bool sb_umma_peer_out_ok(int M, int N, int n) {
  return n >= 2 && n <= UG_MAX_PEERS && M % n == 0 && (M / n) % UG_BLOCK_M == 0 && ((long long)N * 4) % 16 == 0;
}

bool sb_umma_head_fits(int N, int prefix) {
  return N <= UG_HEAD_MAX_N || (N <= UG_HEAD_MAX_TILE_N && prefix >= 0 && prefix <= UG_HEAD_MAX_N);
}
