/* libspiral_b200 -- C ABI of the B200 (sm_100a) dense-matmul / policy-MLP path.
 *
 * Every entry point takes plain device pointers and sizes, writes its results
 * in place into caller-owned memory and returns an int status (SB_OK or a
 * negative sb_status code; sb_last_error_string() holds the text).  Launches
 * are asynchronous on the given stream (NULL = the legacy default stream).
 * Unless a comment says otherwise no entry point allocates device memory.
 *
 * Each declaration cites the reference interface (file:line inside
 * mrakgr/Spiral-s-ML-Library) that it replaces.
 */
#ifndef SPIRAL_B200_H
#define SPIRAL_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum sb_status {
  SB_OK = 0,
  SB_ERR_BAD_ARG = -1,       /* null pointer, negative size, unknown enum */
  SB_ERR_MISALIGNED = -2,    /* base or leading dimension not 16-byte aligned */
  SB_ERR_UNSUPPORTED = -3,   /* dtype / layout / epilogue combination not built */
  SB_ERR_CUDA = -4,          /* a CUDA runtime or driver call failed */
  SB_ERR_DEVICE_TIMEOUT = -5,/* a bounded device-side wait expired */
  SB_ERR_TOO_LARGE = -6,     /* size beyond a documented fixed limit */
  SB_ERR_NO_DEVICE = -7      /* no CUDA device / driver */
} sb_status;

/* Arithmetic classes of the GEMM inputs.  SB_F32 = fp32 storage, fp32 FMA
 * math (1e-5 class).  SB_TF32 = fp32 storage, TF32 tensor-core multiply, the
 * reference's own arithmetic (corecuda/wmma.spi:20,78-82).  SB_BF16 / SB_F16
 * = 16-bit storage.  Accumulation is always fp32. */
typedef enum sb_dtype { SB_F32 = 0, SB_TF32 = 1, SB_BF16 = 2, SB_F16 = 3, SB_I32 = 4, SB_U8 = 5 } sb_dtype;

/* Epilogue flags, OR-ed.  Order of application on one output row:
 *   v = alpha * acc + beta * C_old ; v += bias[col] ; v = relu(v) ;
 *   v = (aux_in[row,col] > 0) ? v : 0   (RELU_GRAD) ;
 *   row head: masked softmax, then regret matching, then argmax.
 *   row head: sign hash, masked softmax, then regret matching, then argmax and sampling.
 * Row heads are fused into the GEMM for N <= 64 (and for N <= 256 under a prefix mask of at
 * most 64 columns) and run as further kernels on C for wider rows. */
enum {
  SB_EPI_NONE = 0,
  SB_EPI_BIAS = 1,            /* bias: fp32[N] */
  SB_EPI_RELU = 2,            /* ml/layers.spi:355 (BlockMap max 0), fused */
  SB_EPI_RELU_GRAD = 4,       /* aux_in: activation [M,N] in out_dtype */
  SB_EPI_MASKED_SOFTMAX = 8,  /* ml/primitives.spi:748-759; mask: uint8[M,N] or NULL = all legal */
  SB_EPI_REGRET_MATCHING = 16,/* ml/primitives.spi:761-780, same mask */
  SB_EPI_ARGMAX = 32,         /* ml/primitives.spi:705-708; aux_out: int32[M], lowest index on ties */
  /* ReLU sign bits instead of the activation tile (N % 32 == 0): word
   * [c, row] of a uint32[N/32, M] matrix, bit j = (value[row, 32c + j] > 0).
   * Stored column-block-major so that the 32 rows a warp finishes together
   * are 32 consecutive words. */
  SB_EPI_RELU_MASK_OUT = 64,  /* with SB_EPI_RELU: also write the sign bits to aux_out */
  SB_EPI_RELU_GRAD_MASK = 128,/* gate by the sign bits in aux_in (the backward twin of the above) */
  /* Column sums of the finished values (after the sign-bit gate, before storage
   * rounding) are ADDED to aux_out: fp32[N], which the caller zeroes.  This is
   * the bias gradient of the layer below when the GEMM is a dgrad.  N % 32 == 0,
   * alpha == 1, beta == 0, tensor-core classes; combines only with
   * SB_EPI_RELU_GRAD_MASK.  The additions are atomic: their order, hence the
   * last bits of the sums, can differ between runs. */
  SB_EPI_COLSUM_OUT = 256,
  /* The next three are given through sb_matmul_head / sb_head_spec. */
  SB_EPI_SAMPLE = 512,        /* ml/primitives.spi:782-800: one index per row drawn from the finished row */
  SB_EPI_BINARIZE = 1024,     /* ml/primitives.spi:816-821: sign hash of the logits (N <= 32) */
  /* x / sum(x^2) over the whole row (local_ln_l2, ml/primitives.spi:701-703), applied before the
   * ReLU: the reference's test nets put ln_l2 between every matmul and relu
   * (ml/layers.spi:562-568).  N <= 256, alpha == 1, beta == 0, no bias, tensor-core classes. */
  SB_EPI_LN_L2 = 2048
};

/* A row head with everything it may need.  `flags`: SB_EPI_MASKED_SOFTMAX, SB_EPI_REGRET_MATCHING,
 * SB_EPI_ARGMAX, SB_EPI_SAMPLE, SB_EPI_BINARIZE.  Legal columns: j < prefix when prefix >= 0 (the way
 * layers.masked_softmax / masked_regret_matching / masked_softmax_and_discrete_sample instantiate
 * their mask, ml/layers.spi:409,416,426), else mask[row, j] != 0, else all.  Sampling draws, for row
 * r, output number `position` of the Philox4x32-10 stream (key = seed, subsequence = row_offset + r)
 * -- the generator the reference initialises per thread with curand_init(seed, thread index, 0)
 * (corecuda/random.spi:22-24) -- as a uniform number in (0, 1] (corecuda/random.spi:84), and takes the
 * first j with a positive weight and cdf[j] >= u * total; -1 for a row without a positive weight. */
typedef struct sb_head_spec {
  int flags;
  int prefix;                    /* -1: no prefix mask */
  const uint8_t* mask;           /* uint8 [rows, N] or NULL */
  int32_t* argmax_out;           /* int32 [rows], SB_EPI_ARGMAX */
  int32_t* sample_out;           /* int32 [rows], SB_EPI_SAMPLE */
  uint32_t* hash_out;            /* uint32 [rows], SB_EPI_BINARIZE */
  uint32_t modulo;               /* SB_EPI_BINARIZE: the hash is taken modulo this (> 0) */
  unsigned long long seed;
  unsigned long long row_offset;
  unsigned long long position;
} sb_head_spec;

/* ---- runtime ------------------------------------------------------------ */
const char* sb_last_error_string(void);
int sb_version(void);
int sb_device_count(int* count);
int sb_set_device(int device);
int sb_device_sm_count(int* sms);
/* cupy.empty / cp.cuda memory calls of corecuda/cupy.spi:20-58 are replaced by
 * the caller's own allocator; these exist so that hosts without one (tests,
 * bench) can still obtain device memory. */
int sb_malloc(void** ptr, size_t bytes);
int sb_free(void* ptr);
int sb_malloc_host(void** ptr, size_t bytes);   /* pinned host memory */
int sb_free_host(void* ptr);
int sb_memcpy_h2d(void* dst, const void* src, size_t bytes, void* stream);
int sb_memcpy_d2h(void* dst, const void* src, size_t bytes, void* stream);
int sb_memcpy_d2d(void* dst, const void* src, size_t bytes, void* stream);
int sb_memset(void* dst, int value, size_t bytes, void* stream);
int sb_stream_create(void** stream);
int sb_stream_destroy(void* stream);
int sb_stream_sync(void* stream);               /* corecuda/base.spi:45 device_sync */
int sb_device_sync(void);
int sb_event_create(void** event);
int sb_event_destroy(void* event);
int sb_event_record(void* event, void* stream);
int sb_event_elapsed_ms(void* start, void* stop, float* ms);  /* syncs on stop */
int sb_stream_wait_event(void* stream, void* event);        /* later work on stream waits for event */
/* Host-side check of the bounded device waits: synchronises `stream`, then returns
 * SB_ERR_DEVICE_TIMEOUT when any kernel of this library gave up a wait since the status word
 * was last cleared (the outputs of those kernels are then incomplete), else SB_OK.  Stands
 * where the reference learns of a failed device assert at its next synchronisation
 * (ml/matmul/run.py:1240).  The Python host calls it at its read-back points. */
int sb_check_device(void* stream);
/* Free and total bytes of device memory (cudaMemGetInfo); corecuda/cupy.spi:20-58 leaves this
 * to CuPy's memory pool. */
int sb_mem_info(size_t* free_bytes, size_t* total_bytes);
/* Reads (and optionally clears) the device status word written by bounded
 * waits: status[0] = first wait site that expired (0 = healthy), status[1] =
 * count of expired waits.  Synchronises the device. */
int sb_device_status(int* status2, int clear);
/* Exercises the bounded device-side wait on purpose: one small kernel waits on
 * a barrier nothing signals; after the library's wait limit (0.4 s) it must
 * return with result5 = {0, 0, ms waited by the first waiter, ms waited by the
 * second, 1} and sb_device_status must report wait site 8.  The context stays
 * usable.  No counterpart in the reference (a failed device assert kills its
 * context, ml/matmul/run.py:1240).  Allocates 20 bytes for the duration of the call. */
int sb_selftest_bounded_wait(int* result5);
/* Number of kernels this library has launched in this process so far. */
unsigned long long sb_launch_count(void);
/* Device-side timing of the tensor-core GEMM launches between begin and end:
 * a CUDA event pair is recorded around each launch on its own stream (at most
 * 4096 launches).  end synchronises and returns the launch count, the summed
 * kernel time and the summed algorithmic flops (2*M*N*K each).  Stands where
 * the reference times by hand with time.perf_counter around a synchronised
 * launch (game/leduc/full.spi:21-34). */
int sb_gemm_profile_begin(void);
int sb_gemm_profile_end(int* launches, double* total_ms, double* total_flops);
/* Time and flops of launch `index` of the profile that sb_gemm_profile_end just closed. */
int sb_gemm_profile_entry(int index, double* ms, double* flops);

/* ---- GEMM ---------------------------------------------------------------
 * C[M,N] <- alpha * op(A) * op(B) + beta * C, row-major, in place.
 * a_trans = 0: A stored [M,K]; 1: stored [K,M].  b_trans = 0: B stored [K,N];
 * 1: stored [N,K].  Replaces matmul_tf32 a_trans b_trans alpha a b beta c
 * (ml/matmul/run.spi:21-26; template ml/matmul/kernel.spi:25-240; argument
 * order A, B, C as in ml/matmul/run.py:1228-1232). */
int sb_matmul_tf32(int a_trans, int b_trans, float alpha, const float* A, const float* B,
                   float beta, float* C, int M, int N, int K, void* stream);

/* Same contract with explicit input class, output dtype (SB_F32, SB_BF16,
 * SB_F16) and fused epilogue; the dense layer of ml/layers.spi:227-240 is
 * a_trans=0, b_trans=1, alpha=1, beta=0.  bias / mask / aux_in / aux_out may
 * be NULL when their flag is absent. */
int sb_matmul_ex(int a_trans, int b_trans, float alpha, const void* A, const void* B, float beta,
                 void* C, int M, int N, int K, int in_dtype, int out_dtype, int epilogue,
                 const float* bias, const uint8_t* mask, const void* aux_in, void* aux_out,
                 void* stream);

/* The fp32 accuracy class (1e-5 relative Frobenius error against a float32 product) on the tensor
 * cores: every operand is split into a TF32 head and a TF32 tail and the product is taken as
 * Ah*Bh + Ah*Bl + Al*Bh in one tcgen05 GEMM with fp32 accumulation ("3 x TF32"; the reference's own
 * arithmetic is single-pass TF32, corecuda/wmma.spi:20,78-82, which cannot meet 1e-5).  Two launches:
 * the split into `workspace` (caller memory, at least sb_matmul_f32_workspace_bytes) and the GEMM.
 * Contiguous dimensions must be multiples of 4 elements; other shapes use the SB_F32 class of
 * sb_matmul_ex (FFMA).  epilogue: SB_EPI_BIAS, SB_EPI_RELU. */
int sb_matmul_f32_workspace_bytes(int M, int N, int K, size_t* bytes);
int sb_matmul_f32x3(int a_trans, int b_trans, float alpha, const float* A, const float* B, float beta, float* C,
                    int M, int N, int K, int epilogue, const float* bias, void* workspace, size_t workspace_bytes,
                    void* stream);

/* The dense layer with a row head described by `head` (ml/layers.spi:408-436 on top of :227-240):
 * C <- head(alpha * op(A) * op(B) + beta * C (+ bias) (ReLU)), fp32 output.  `epilogue` may hold
 * SB_EPI_BIAS, SB_EPI_RELU and SB_EPI_LN_L2; the head flags come from head->flags.  One launch when
 * N <= 64, or N <= 256 with 0 <= prefix <= 64 (the reference's policy nets end in 64 columns of
 * which the first few are legal, game/leduc/model_cem.spi:37,52-60); wider rows run the head as
 * further kernels on C.  Nothing is allocated and no mask matrix is needed for a prefix. */
int sb_matmul_head(int a_trans, int b_trans, float alpha, const void* A, const void* B, float beta,
                   float* C, int M, int N, int K, int in_dtype, int epilogue, const float* bias,
                   const sb_head_spec* head, void* stream);

/* Keeps `bytes` of shared memory per SM out of the GEMM's pipeline (0 = use all of it; rounded up to a
 * KiB, at most 64 KiB) so that a CTA of another kernel -- the data-parallel update of the layers whose
 * gradients are already complete -- can be resident beside a GEMM CTA and run in its idle issue
 * slots.  A process-wide setting read at every GEMM launch; the pipeline gets shallower (a few per
 * cent of GEMM throughput).  No counterpart in the reference (single device, one kernel at a time). */
int sb_gemm_reserve_smem(int bytes);

/* Tile-shape heuristic of the tensor-core path, exposed for tests: the
 * counterpart of matmul_config_tf32 (ml/matmul/run.spi:8-19).  Writes
 * {block_m, block_n, block_k_elems, stages, grid}. */
int sb_matmul_plan(int a_trans, int b_trans, int M, int N, int K, int in_dtype, int epilogue,
                   int* plan5);

/* ---- elementwise / row operations (stand-alone forms) ---------------------
 * relu: ml/layers.spi:355 + ml/primitives.spi:115-129.  Row heads:
 * ml/primitives.spi:705-722,748-780 over x[rows, cols] fp32 row-major;
 * `mask` uint8[rows, cols] or NULL, or prefix masking j < prefix when
 * prefix >= 0 (ml/layers.spi:409,416).  out may alias x. */
int sb_relu(const float* x, float* out, size_t n, void* stream);
int sb_row_softmax(const float* x, float* out, int rows, int cols, const uint8_t* mask, int prefix,
                   void* stream);
int sb_row_regret_matching(const float* x, float* out, int rows, int cols, const uint8_t* mask,
                           int prefix, void* stream);
int sb_row_argmax(const float* x, int32_t* out, int rows, int cols, void* stream);
int sb_row_ln_l2(const float* x, float* out, int rows, int cols, void* stream);  /* ml/primitives.spi:701-703 */
/* Discrete sampling, local_discrete_sampling ml/primitives.spi:782-800 (the sampling heads of
 * ml/layers.spi:422-431): out[r] = the first j with probs[r,j] > 0 and cdf[r,j] >= uniforms[r] *
 * (cdf at the last positive entry), -1 for a row without a positive entry.  The uniform numbers in
 * (0, 1] come from the caller (the reference draws them inside the kernel). */
int sb_row_sample(const float* probs, const float* uniforms, int32_t* out, int rows, int cols, void* stream);
/* The same with the uniform numbers drawn on the device, as the reference does: row r uses output
 * number `position` of the Philox4x32-10 stream (seed, row_offset + r), see sb_head_spec. */
int sb_row_sample_seeded(const float* probs, int32_t* out, int rows, int cols, unsigned long long seed,
                         unsigned long long row_offset, unsigned long long position, void* stream);
/* The uniform numbers themselves (fp32 [n], each in (0, 1]): element i = output `position` of stream
 * (seed, row_offset + i).  For callers and tests that want to see what a sampling head drew. */
int sb_philox_uniform(float* out, long long n, unsigned long long seed, unsigned long long row_offset,
                      unsigned long long position, void* stream);
/* Row hash, local_binarize ml/primitives.spi:816-821 (layers.binarize, ml/layers.spi:433-436): out[r] =
 * (sum over j of (x[r,j] > 0) << j) mod modulo; cols <= 32. */
int sb_row_binarize(const float* x, uint32_t* out, int rows, int cols, uint32_t modulo, void* stream);
/* Rounds fp32 to the storage type of a tensor-core input class (SB_BF16,
 * SB_F16 -> 16-bit; SB_TF32 -> fp32 with the low 13 mantissa bits cleared,
 * round-to-nearest-even). */
int sb_convert(const float* x, void* out, size_t n, int out_dtype, void* stream);
/* Game-state encoder: compact records -> the dense network input x [rows,
 * sum(widths) + n_dense] in storage type `dtype`.  Replaces the device-side
 * serialisation of ml/models.spi:30-41 (zero the input tensor, then pickle each
 * state into it) for states made of bounded ints (one-hot groups,
 * corebase/pickler.spi:20-37) followed by real values.  fields: uint8 [rows,
 * n_fields], value v < widths[j] sets feature offset_j + v of group j, any
 * other value leaves the group zero; widths: HOST array, each in [1, 255],
 * at most 64 fields and 2048 one-hot features; dense: [rows, n_dense] in
 * `dtype`, copied unchanged behind the one-hot groups (may be NULL when
 * n_dense == 0). */
int sb_encode_states(const uint8_t* fields, int n_fields, const int* widths, const void* dense, int n_dense,
                     void* x, long long rows, int dtype, void* stream);

/* ---- dense policy network ---------------------------------------------------
 * A ReLU MLP `sizes[0] -> sizes[1] -> ... -> sizes[n_layers]` with a row head
 * on the last layer; every layer is y = x W^T (+ b) with W stored [out, in]
 * (layers.matmul, ml/layers.spi:227-240,467).  All buffers are caller-owned,
 * like the reference's weight / workspace / adjoint arenas
 * (ml/layers.spi:6-12,127-172).
 *
 * Parameter layout: one flat vector [W0 | b0 | W1 | b1 | ...]; offsets (in
 * elements) from sb_mlp_param_offsets: offsets[2i] = W_i, offsets[2i+1] = b_i,
 * offsets[2*n_layers] = total length.  A weight segment holds
 * round_up(out, 8) rows (padding rows must be zero and stay zero).  `params`
 * is the fp32 master copy, `w_compute` the same layout in the storage type of
 * `in_dtype` (SB_TF32: fp32 rounded to TF32; SB_BF16; SB_F16). */
int sb_mlp_param_offsets(int n_layers, const int* sizes, long long* offsets);

/* Forward pass; replaces graph_run_host / graph_run_device for a dense chain
 * (ml/layers.spi:339-344, generated block_matmul/block_map/block_row_map
 * sequence ml/layers.py:4500-4546).  x: [batch, sizes[0]] in the storage type;
 * activations: host array of n_layers-1 device pointers, activations[i] =
 * [batch, sizes[i+1]] in the storage type (workspace, overwritten); params may
 * be NULL (no bias, as in the reference); relu_bits: NULL, or a host array of
 * n_layers-1 device pointers, relu_bits[i] = uint32 [sizes[i+1]/32, batch]
 * receiving the ReLU sign bits of hidden layer i (SB_EPI_RELU_MASK_OUT; used
 * when the width is a multiple of 32, so that backward need not re-read the
 * activations to gate its gradients); head: SB_EPI_MASKED_SOFTMAX |
 * SB_EPI_REGRET_MATCHING | SB_EPI_ARGMAX; out: fp32 [batch, sizes[n_layers]];
 * actions: int32 [batch] when SB_EPI_ARGMAX. */
int sb_mlp_forward(int n_layers, const int* sizes, int batch, int in_dtype, const void* x,
                   const void* w_compute, const float* params, void* const* activations,
                   void* const* relu_bits, int head, const uint8_t* mask, float* out, int32_t* actions,
                   void* stream);

/* The same forward pass as ONE persistent kernel for narrow nets (the Leduc-sized
 * policy MLP): hidden activations stay in shared memory / TMEM, so no activations
 * buffer is needed.  Replaces the same reference chain (ml/layers.py:4500-4546).
 * Limits: in_dtype SB_F16 or SB_BF16; sizes[0] in 8..512 and a multiple of 8 (the
 * input tile, the widest hidden tile and the weight ring share 225 KB of shared memory:
 * inputs beyond 256 fit with hidden layers of at most 128 columns); hidden widths
 * multiples of 64 up to 256; sizes[n_layers] <= 64; n_layers <= 8; otherwise
 * SB_ERR_UNSUPPORTED (use sb_mlp_forward). */
int sb_mlp_forward_fused(int n_layers, const int* sizes, int batch, int in_dtype, const void* x,
                         const void* w_compute, const float* params, int head, const uint8_t* mask,
                         float* out, int32_t* actions, void* stream);
/* The same for an ensemble of `members` nets of one architecture on ONE input batch, the way the
 * reference's games run their policies (layers.matmul_ensemble, ml/layers.spi:468-471: weights
 * [ensemble, out, in], the graph run once per member, ml/layers.spi:339-344): here all members are
 * one launch, a CTA works on (row tile, member) pairs.  w_compute and params hold the members'
 * flat parameter vectors one after the other (member e at element e * sb_mlp_param_offsets(...)
 * [2 * n_layers]); out: fp32 [members, batch, n_out]; actions: int32 [members, batch]; mask
 * [batch, n_out] is shared by the members. */
int sb_mlp_forward_fused_ensemble(int n_layers, const int* sizes, int batch, int members, int in_dtype,
                                  const void* x, const void* w_compute, const float* params, int head,
                                  const uint8_t* mask, float* out, int32_t* actions, void* stream);

/* The training form of the fused forward (one net): the same single launch, and the hidden
 * activations (activations[l]: [batch, sizes[l+1]] in the storage type) and their ReLU sign words
 * (relu_bits[l]: uint32 [sizes[l+1]/32, batch], may be NULL) are also written to global memory, in the
 * layout sb_mlp_forward leaves them, so that sb_mlp_backward can follow.  The activation tile in
 * shared memory already has the layout of a TMA box and leaves through one TMA store per 64-column
 * chunk.  sb_mlp_fused_supported tells (1 / 0) whether a net is within the fused kernel's limits;
 * sb_mlp_train_step takes this path by itself when it is. */
int sb_mlp_fused_supported(int n_layers, const int* sizes, int in_dtype);
int sb_mlp_forward_fused_train(int n_layers, const int* sizes, int batch, int in_dtype, const void* x,
                               const void* w_compute, const float* params, void* const* activations,
                               void* const* relu_bits, int head, const uint8_t* mask, float* out,
                               int32_t* actions, void* stream);

/* The fused ensemble forward with the head given as an sb_head_spec and the reference's other
 * graph pieces: hidden_norm = 1 puts ln_l2 (x / sum(x^2) over the row, ml/primitives.spi:701-703)
 * before every ReLU as the reference's nets do (ml/layers.spi:594-603; then params must be NULL:
 * those nets have no bias); the head may be prefix-masked (ml/layers.spi:409,416) and may sample
 * (SB_EPI_SAMPLE, ml/layers.spi:422-431): member e draws output number head->position + e of the row's
 * stream, the way the reference's per-thread generator advances from one member's run to the next
 * (ml/models.spi:47-49).  Output widths up to 64, or up to 256 under a prefix of at most 64 columns
 * (game/leduc/model_cem.spi:37,52-60: 64 columns, 3 legal).  head->argmax_out / sample_out are
 * int32 [members, batch]; out is fp32 [members, batch, n_out].  No sign hash here. */
int sb_mlp_forward_fused_head(int n_layers, const int* sizes, int batch, int members, int in_dtype,
                              const void* x, const void* w_compute, const float* params, int hidden_norm,
                              const sb_head_spec* head, float* out, void* stream);

/* One policy decision per game state, the whole of models.noinline_run (ml/models.spi:9-76): the states
 * are serialised into the input tensor on the device (sb_encode_states; fields == NULL: x already holds
 * the input), every ensemble member's net runs on them, each member samples an action per state from
 * its head, a member is drawn per state, and the call reports that member's action together with the
 * probability the drawn member gave it (sampling_prob_selected) and the probability EVERY member gave
 * it (sampling_prob_ensemble) -- what the reference returns as {action, sampling_prob_selected,
 * sampling_prob_ensemble} and leaves in its output_probs / output_indices tensors.  Two launches:
 * the encoder and one fused kernel (nets within the limits of sb_mlp_forward_fused_head).
 * Random stream of state r: Philox4x32-10 (seed, row_offset + r); outputs 0 .. members-1 are the
 * members' sampling draws, the outputs from `members` on pick the member (unbiased rejection,
 * corecuda/random.spi:53-59).  tile_counters: int32 [ceil(rows / 128)] that the caller zeroes once;
 * every call leaves it zero again.  Calls that overlap on the GPU need counters of their own. */
typedef struct sb_decide_args {
  int n_layers;
  const int* sizes;              /* HOST: n_layers + 1 widths */
  int members;
  int in_dtype;                  /* SB_F16 or SB_BF16 */
  const void* w_compute;         /* members' flat parameter vectors, one after the other */
  const float* params;           /* fp32 copies for the biases, or NULL: no bias */
  int hidden_norm;               /* 1: ln_l2 before every ReLU (params must be NULL) */
  long long rows;
  const uint8_t* fields;         /* uint8 [rows, n_fields] or NULL */
  int n_fields;
  const int* widths;             /* HOST */
  const void* dense;             /* [rows, n_dense] in the storage type, or NULL */
  int n_dense;
  void* x;                       /* [rows, sizes[0]] storage type: the network input (written when fields != NULL) */
  int head_flags;                /* SB_EPI_MASKED_SOFTMAX and / or SB_EPI_REGRET_MATCHING */
  int prefix;                    /* legal iff column < prefix; -1: use mask (or all) */
  const uint8_t* mask;           /* uint8 [rows, n_out] or NULL */
  unsigned long long seed;
  unsigned long long row_offset;
  float* output_probs;           /* fp32 [members, rows, n_out] */
  int32_t* output_indices;       /* int32 [members, rows] */
  int32_t* ensemble_id;          /* int32 [rows]: the member drawn for each state */
  int32_t* action;               /* int32 [rows] */
  float* sampling_prob_selected; /* fp32 [rows] */
  float* sampling_prob_ensemble; /* fp32 [rows, members] */
  int32_t* tile_counters;        /* int32 [ceil(rows / 128)], zero */
} sb_decide_args;
int sb_policy_decide(const sb_decide_args* args, void* stream);

/* The same forward pass for callers that cannot allocate device memory (a host
 * that owns no allocator, a plugin in a context where allocation is forbidden,
 * code inside a stream capture): the hidden activations live in a fixed array
 * inside the library image instead of caller memory.  It has no counterpart in
 * the reference.  Limit: the 256-byte aligned hidden activations,
 * sum over hidden layers of batch * sizes[i+1] * element size, must fit in
 * SB_STATIC_WORKSPACE_BYTES (32 MiB, held by every GPU that loads the library
 * until the process exits); larger requests return SB_ERR_TOO_LARGE.  It calls
 * no cudaMalloc / cudaFree.  The first call on a device looks up the array's
 * device address and sets kernel attributes; make that call before starting any
 * stream capture.  All calls share the one array and it keeps the last call's
 * contents (every byte used is rewritten before it is read, so nothing needs
 * clearing): two calls that overlap on the GPU -- different streams, or
 * different host threads -- race on it. */
#define SB_STATIC_WORKSPACE_BYTES (32u * 1024u * 1024u)
int sb_mlp_forward_static(int n_layers, const int* sizes, int batch, int in_dtype, const void* x,
                          const void* w_compute, const float* params, int head, const uint8_t* mask,
                          float* out, int32_t* actions, void* stream);

/* Backward pass of mean cross-entropy over `1/inv_global_batch` rows on a
 * masked-softmax head, after sb_mlp_forward with SB_EPI_MASKED_SOFTMAX on the
 * same buffers.  No counterpart in the reference (it trains by CEM / CFR,
 * ml/cem.spi:99-146).  Writes the flat fp32 gradient vector `grads` (layout of
 * sb_mlp_param_offsets, padding zeroed) -- the buffer a data-parallel caller
 * all-reduces -- and adds this shard's share of the loss to *loss (device
 * float, caller zeroes it; NULL to skip).  scratch: 256-byte aligned, at least
 * sb_mlp_backward_scratch_bytes. */
int sb_mlp_backward_scratch_bytes(int n_layers, const int* sizes, int batch, int in_dtype, size_t* bytes);
int sb_mlp_backward(int n_layers, const int* sizes, int batch, float inv_global_batch, int in_dtype,
                    const void* x, const void* w_compute, void* const* activations,
                    void* const* relu_bits, const float* probs, const uint8_t* mask, const float* target,
                    float* grads, int with_bias, void* scratch, size_t scratch_bytes, float* loss,
                    void* stream);

/* Where the backward pass keeps d(loss)/d(output of layer `layer`) inside `scratch`: byte offset
 * of a [batch, round_up(sizes[layer+1], 8)] matrix in the storage type.  The two dY buffers
 * alternate from layer to layer, so the matrix is intact from the moment layer `layer` has been
 * processed until layer `layer - 2` is; a caller that runs sb_mlp_backward_range one layer at a
 * time can inspect every layer's dY (the counterpart of reading the reference's adjoint arena,
 * ml/layers.spi:6-12).  Used by the full-size parity tests. */
int sb_mlp_backward_dy_offset(int n_layers, const int* sizes, int batch, int in_dtype, int layer, size_t* offset);

/* The same pass restricted to layers first_layer, first_layer-1, ..., last_layer
 * (first_layer = n_layers-1 zeroes grads and computes d logits and the loss
 * first).  Successive calls that together cover n_layers-1 .. 0 equal one
 * sb_mlp_backward; a data-parallel caller uses them to start the all-reduce of
 * a layer's gradient segment while the layers below are still being computed. */
int sb_mlp_backward_range(int n_layers, const int* sizes, int batch, float inv_global_batch, int in_dtype,
                          const void* x, const void* w_compute, void* const* activations,
                          void* const* relu_bits, const float* probs, const uint8_t* mask,
                          const float* target, float* grads, int with_bias, void* scratch,
                          size_t scratch_bytes, float* loss, int first_layer, int last_layer, void* stream);

/* params -= lr * grads over n elements, and w_compute (may be NULL) = params
 * rounded to compute_dtype.  No counterpart in the reference. */
int sb_sgd_update(float* params, const float* grads, void* w_compute, long long n, float lr,
                  int compute_dtype, void* stream);

/* Single-GPU training step: forward, backward over this batch, SGD. */
int sb_mlp_train_step(int n_layers, const int* sizes, int batch, int in_dtype, const void* x,
                      float* params, void* w_compute, void* const* activations, void* const* relu_bits,
                      const uint8_t* mask,
                      const float* target, float* probs, float* grads, int with_bias, float lr,
                      void* scratch, size_t scratch_bytes, float* loss, void* stream);

/* ---- data-parallel update over peer memory ---------------------------------
 * No reference counterpart (the reference is single-device, corecuda/base.spi:7);
 * follows the benchmark's data-parallel training configurations.  One process
 * per GPU.  Each rank exports its gradient, master-parameter, compute-copy and
 * flag buffers (sb_ipc_export), sends the 64-byte handles to its peers by any
 * host channel, and opens theirs (sb_ipc_open): the tables passed below are HOST
 * arrays of world_size DEVICE pointers, entry [rank] being the rank's own
 * buffer.  Buffers come from sb_malloc / cudaMalloc (whole allocations). */
int sb_ipc_export(void* dev_ptr, void* handle64);
int sb_ipc_open(const void* handle64, void** dev_ptr);
int sb_ipc_close(void* dev_ptr);
/* Size of one rank's flag block; the caller zero-fills it once before the first step. */
int sb_dp_flag_bytes(void);
/* The part of the element range [begin, end) (whole 4-element vectors) that rank `rank` reduces and
 * updates when the range is handled by one sb_dp_sgd_update call. */
int sb_dp_slice(long long begin, long long end, int world_size, int rank, long long* begin_end);
/* Gradient reduction + SGD + redistribution in one kernel for the elements
 * [begin, end) of the flat vectors: waits until every rank has reached this
 * call (flag barrier), then for this rank's slice of the range
 *   g = sum over ranks (in rank order) of grads[r][i];  w = params[rank][i] - lr * g;
 *   params[r][i] = w and w_compute[r][i] = round(w) for every rank r,
 * and closes with a second barrier, after which every rank holds the complete
 * new weights.  Replaces all-reduce + sb_sgd_update.  `epoch` must be odd and
 * grow by 2 per call, the same on every rank (the call uses epoch and epoch+1).
 * mode: SB_DP_REPLICATED as above; SB_DP_SHARDED_MASTER stores the fp32 master
 * value only on the owner of a slice, except inside the `replicate` ranges
 * (HOST array of n_replicate [begin, end) element pairs in whole 4-element
 * vectors -- the biases, which the forward pass reads in fp32): a third of the
 * bytes leave the GPU, and a rank's master vector is current only in its own
 * slice until SB_DP_GATHER_MASTER (no gradients, no step: every owner's slice
 * is copied to all ranks) is called.  Every wait is bounded by timeout_ms; when
 * one expires the waiting CTAs return without updating, sb_dp_status reports
 * 0x100 + the rank that did not arrive, and the flag block must be zeroed
 * before it is used again.  The update of that step may then be PARTIAL (a CTA
 * that still saw the late flag has stored its part): restore the weights from a
 * checkpoint.  barriers = 0 runs the update without either barrier (single rank, or
 * ranks ordered by the caller).  A step may be split into several calls over
 * disjoint ranges; calls that can be in flight at the same time need flag
 * blocks of their own.  max_blocks caps the grid (0 = no cap). */
enum { SB_DP_REPLICATED = 0, SB_DP_SHARDED_MASTER = 1, SB_DP_GATHER_MASTER = 2 };
int sb_dp_sgd_update(int world_size, int rank, const float* const* grads, float* const* params,
                     void* const* w_compute, void* const* flags, unsigned int epoch, long long begin, long long end,
                     float lr, int compute_dtype, int mode, const long long* replicate, int n_replicate,
                     int max_blocks, int timeout_ms, int barriers, void* stream);
/* The same over several element ranges in ONE launch (one pair of barriers): `segments` = HOST array of
 * n_segments [begin, end) pairs; every range is cut into world_size slices of its own and rank r handles
 * slice r of each.  reduced[k] != 0 (HOST array, may be NULL): the gradients of range k have already
 * been summed into the owners' buffers by sb_mlp_backward_dp, so a rank reads only its own buffer there
 * -- and zeroes what it read, which is what the next step's tiles are added to. */
int sb_dp_sgd_update_segments(int world_size, int rank, const float* const* grads, float* const* params,
                              void* const* w_compute, void* const* flags, unsigned int epoch, int n_segments,
                              const long long* segments, const int* reduced, float lr, int compute_dtype, int mode,
                              const long long* replicate, int n_replicate, int max_blocks, int timeout_ms, int barriers,
                              void* stream);
int sb_dp_status(const void* flags, int* status);

/* Data-parallel backward pass that does the reduce-scatter half of the gradient all-reduce itself:
 * grads_peers = HOST array of world_size DEVICE pointers, entry r = rank r's flat gradient vector
 * (own buffer at [rank], peers' buffers opened with sb_ipc_open).  For every layer that
 * sb_mlp_dp_fused_layers marks (weight matrix of at least 128 * world_size padded rows, at most 8
 * ranks) the weight-gradient GEMM adds each output tile straight into the copy of the rank that owns
 * its rows (rows [r * out / world, (r + 1) * out / world) belong to rank r: the slice r of that layer's
 * weight range in sb_dp_sgd_update_segments) through TMA reduce-add stores over peer memory, tile by
 * tile while the GEMM runs; after all ranks' passes the owner holds the summed gradient and
 * sb_dp_sgd_update_segments(reduced = 1 for those ranges) needs no remote reads.  Other gradients
 * (narrow layers, biases) are written to this rank's own vector as in sb_mlp_backward.  The marked
 * weight ranges of every rank's vector must be zero before the first pass (a fresh sb_memset) and are
 * left zero by the update.  No counterpart in the reference (single device). */
int sb_mlp_dp_fused_layers(int n_layers, const int* sizes, int world_size, int* fused);
int sb_mlp_backward_dp(int n_layers, const int* sizes, int batch, float inv_global_batch, int in_dtype,
                       const void* x, const void* w_compute, void* const* activations,
                       void* const* relu_bits, const float* probs, const uint8_t* mask, const float* target,
                       float* const* grads_peers, int world_size, int rank, int with_bias, void* scratch,
                       size_t scratch_bytes, float* loss, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SPIRAL_B200_H */
