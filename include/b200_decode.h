/*
 * C ABI of the B200 (sm_100a) decode-step kernels.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream, launches on that
 * stream, never synchronises, never allocates, and returns 0 or a negative B200_ERR_* code
 * (no exceptions, no exit, no trap).  All tensors are row-major and dense unless a leading
 * dimension is passed.  "bf16" means CUDA __nv_bfloat16 bits.
 *
 * Each declaration cites the reference (Megatron Core 0.15) call it replaces, by path inside
 * the reference project.
 */
#ifndef B200_DECODE_H_
#define B200_DECODE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* b200_stream_t; /* same type as cudaStream_t */

enum {
  B200_OK = 0,
  B200_ERR_INVALID_ARGUMENT = -1, /* null pointer, bad size, unsupported head dim ...            */
  B200_ERR_ALIGNMENT = -2,        /* pointer or leading dimension not 16-byte aligned            */
  B200_ERR_WORKSPACE = -3,        /* workspace too small                                         */
  B200_ERR_LAUNCH = -4,           /* the CUDA runtime refused the launch                         */
  B200_ERR_DRIVER = -5,           /* tensor-map encode entry point missing or failed             */
  B200_ERR_DEVICE_TIMEOUT = -6,   /* a bounded device-side wait gave up (see b200_device_status) */
  B200_ERR_SCRATCH_LIMIT = -7     /* the problem needs more scratch than the library's built-in array */
};

/* Library / ABI version (major*1000 + minor). */
int b200_version(void);
const char* b200_error_string(int code);

/*
 * Status word that kernels set when a bounded wait (mbarrier) ran out.  Reading it copies one
 * int from the device (this call synchronises the device); `reset` != 0 clears it afterwards.
 * 0 = no kernel has given up since the last reset.
 */
int b200_device_status(int reset, int* status_out);
/* Bound, in nanoseconds, of every device-side wait of the library on the current device (mbarrier waits inside a
 * CTA, waits for a tensor-parallel peer's flag).  Default 2 s.  When a wait runs out the kernel records a code in the
 * status word (1 GEMM pipeline, 2 attention pipeline, 4 tensor-parallel peer), carries on without the missing data
 * and ends normally, so the context stays usable.  Not to be changed while kernels are in flight. */
int b200_set_wait_limit_ns(uint64_t limit_ns);
/* `rows` rows of `width_bytes` from (pinned) host memory to the device in ONE asynchronous copy: the per-step index
 * arrays of the context (token -> position / chunk / slot, lengths; dynamic_context.py:656-825, 1284-1296) are rows
 * of one staging matrix, and a step updates the first n entries of each. */
int b200_copy_rows_h2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes, size_t rows,
                       b200_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Embedding / row gather.  out[i, :] = table[ids[i] - vocab_start, :] if vocab_start <= ids[i]
 * < vocab_end else 0.
 * Replaces VocabParallelEmbedding.forward (megatron/core/tensor_parallel/layers.py:262-295,
 * masked lookup before the all-reduce) and the last-token gather of
 * DynamicInferenceContext.last_token_logits (megatron/core/inference/contexts/dynamic_context.py:890-918).
 * Optional `add_table`/`add_ids`: a second table gathered and added in bf16 (learned absolute
 * position embedding, megatron/core/models/common/embeddings/language_model_embedding.py:99-149).
 */
int b200_gather_rows_bf16(const void* table, const int64_t* ids, void* out, int n_rows, int row_elems,
                          int64_t vocab_start, int64_t vocab_end, const void* add_table,
                          const int64_t* add_ids, b200_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Fused residual add + RMSNorm / LayerNorm over rows of `hidden` elements.
 *   h = x (+ bias, bf16 add) (+ residual, bf16 add);  if hidden_out: hidden_out = h
 *   normed_out = bf16( normalise_fp32(h) * gamma (+ beta) )
 * beta == NULL selects RMSNorm, otherwise LayerNorm.  normed_out may be NULL (residual add only).
 * Replaces bias_dropout_add (megatron/core/fusions/fused_bias_dropout.py:11-57, eval mode) followed by
 * WrappedTorchNorm (megatron/core/transformer/torch_norm.py:38-51) / TENorm
 * (megatron/core/extensions/transformer_engine.py:204-238).
 */
int b200_add_norm_bf16(const void* x, const void* bias, const void* residual, const void* gamma,
                       const void* beta, void* hidden_out, void* normed_out, int rows, int hidden, float eps,
                       b200_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Activation between fc1 and fc2.
 *   kind 0 (SwiGLU): in [rows, 2*F] = [gate | up]; out[r, f] = bf16(bf16(silu(gate)) * up)
 *                    (megatron/core/fusions/fused_bias_swiglu.py:15-26, eager bf16 rounding points)
 *   kind 1 (GELU):   in [rows, F] (+ bias[F]); out = bf16(gelu_erf(in + bias))
 *                    (megatron/core/transformer/mlp.py:200-213)
 *   kind 2 (SwiGLU, tile-interleaved input): of every 128 input columns the first 64 are gate features 64j..64j+63
 *                    and the last 64 the matching up features - the output of an fc1 whose weight rows were
 *                    arranged for b200_gemm_bf16_swiglu; F a multiple of 64.
 */
int b200_activation_bf16(const void* in, const void* bias, void* out, int rows, int F, int kind,
                         b200_stream_t stream);
/* fc1 + SwiGLU in one kernel (mlp.py:140-234 with fused_bias_swiglu.py:15-26): w [N, K] with N = 2F and rows arranged
 * per 128-row tile j as [gate rows 64j..64j+63 ; up rows 64j..64j+63] of the reference's [gate ; up] weight;
 * y [M, F] = bf16(bf16(silu(x w_gate^T)) * bf16(x w_up^T)), the same bits as b200_gemm_bf16 + b200_activation_bf16.
 * Only shapes whose GEMM is not split along K (b200_gemm_bf16_swiglu_supported returns 1); otherwise use
 * b200_gemm_bf16 and b200_activation_bf16 kind 2. */
int b200_gemm_bf16_swiglu_supported(int M, int N, int K);
int b200_gemm_bf16_swiglu(const void* x, int64_t ldx, const void* w, void* y, int64_t ldy, int M, int N, int K,
                          b200_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * y[M, N] = x[M, K] * w[N, K]^T (+ bias[N]), bf16 in, fp32 accumulate in tensor memory (tcgen05),
 * bf16 out.  x row stride ldx elements, y row stride ldy elements; w is dense.
 * Replaces ColumnParallelLinear.forward / RowParallelLinear.forward local GEMM
 * (megatron/core/tensor_parallel/layers.py:317-336, 946-1043, 1225-1281; torch.matmul(x, W.t())).
 * The all-reduce of the row-parallel variant stays with the caller.
 * `workspace`: split-K partial sums (fp32), see b200_gemm_bf16_workspace_bytes; its contents need no
 * initialisation and it must be 16-byte aligned (0 bytes are needed when K is not split).  When K is split a
 * second kernel on the same stream sums the partials in a fixed order, so results are deterministic.
 *
 * b200_set_gemm_split_policy: tuning of the K split shared by all GEMM entry points (no counterpart in the
 * reference; cuBLAS picks its own).  A shape with fewer output tiles than `ctas_per_sm` CTAs per SM is split along K
 * until it has that many CTAs, keeping at least `min_k_blocks_per_split` K blocks (64 bf16 / 128 FP8 elements
 * each) per split and at most `max_splits` (<= 32) splits.  Defaults 2, 4, 32.  Process-wide; change it only
 * between, not inside, a *_workspace_bytes / *_splitk_bytes query and the launch it sizes.
 */
int b200_set_gemm_split_policy(int ctas_per_sm, int min_k_blocks_per_split, int max_splits);
size_t b200_gemm_bf16_workspace_bytes(int M, int N, int K);
int b200_gemm_bf16(const void* x, int64_t ldx, const void* w, const void* bias, void* y, int64_t ldy, int M,
                   int N, int K, void* workspace, size_t workspace_bytes, b200_stream_t stream);

/*
 * The same GEMM for callers that cannot allocate device memory.  (No counterpart in the reference.)
 *
 * Who needs it: code that runs where cudaMalloc is not an option - a latency-critical serving loop that must
 * not take the allocator's locks or its implicit synchronisation, a server that has given the whole device to
 * its own memory pool, or a plugin that is handed nothing but input and output pointers.  The split-K scratch that b200_gemm_bf16 takes as `workspace` is here a fixed array inside
 * the library (b200_gemm_bf16_static_scratch_limit() bytes: 16 MiB of partial sums,
 * resident on every GPU that loads the library until the process exits).  The call performs no device or host
 * allocation; the caller still owns x, w, bias and y.
 *
 *  - Limit: returns B200_ERR_SCRATCH_LIMIT when b200_gemm_bf16_workspace_bytes(M, N, K) exceeds the array
 *    (decode shapes with few tokens fit; e.g. M = 256, N = 4096, K = 14336 does not).
 *  - The first call on each device looks up the array's device address (cudaGetSymbolAddress, once per
 *    device, with that device current).  Make that first call outside any stream capture.
 *  - Every call uses the same array and finds whatever the last call left in it.  Nothing in it has to start
 *    at zero: the partial sums of a call are always fully overwritten before they are read.  Two calls whose kernels can overlap on the GPU (different streams without an ordering
 *    between them) race on the array: order them.
 *  - Results are bit-identical to b200_gemm_bf16 for the same arguments.
 */
size_t b200_gemm_bf16_static_scratch_limit(void);
int b200_gemm_bf16_static_scratch(const void* x, int64_t ldx, const void* w, const void* bias, void* y, int64_t ldy,
                                  int M, int N, int K, b200_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * MXFP8 linears: E4M3 values with one E8M0 (power-of-two) scale per 32 elements along K, for weights and
 * activations alike; fp32 accumulation on tcgen05 (kind::mxf8f6f4.block_scale), bf16 output.
 * Replaces the FP8 path of TELayerNormColumnParallelLinear / TERowParallelLinear under the `mxfp8` recipe
 * (megatron/core/extensions/transformer_engine.py:453-640, 736-828; recipe choice megatron/core/fp8_utils.py:451-468;
 * the arithmetic itself lives in Transformer Engine 2.7, absent from the reference tree).
 *
 * Scale storage ("tile layout"): for a [rows, K] matrix, b200_mxfp8_scale_bytes(rows, K) bytes arranged as
 * [ceil(rows/128)][K/128][512]; inside a tile the scale of (row r, 32-block b) is byte
 * (r % 32) * 16 + ((r % 128) / 32) * 4 + (b % 4).  Scale byte e means 2^(e - 127); a block's scale is the smallest
 * power of two >= amax / 448.  K must be a multiple of 128.
 *
 * Weight bytes are stored TILE-MAJOR by both FP8 recipes: [ceil(N/128)][K/128] tiles of 128 rows x 128 bytes, 16 KiB of
 * consecutive memory each (byte (n, k) at ((n/128) * (K/128) + k/128) * 16384 + (n%128) * 128 + k%128;
 * b200_fp8_weight_bytes(N, K) bytes; rows past N are padding), so that a GEMM CTA's 128-row x 128-byte operand
 * box is one contiguous DRAM read.  Activations stay row-major [rows, K].
 *
 * b200_quantize_mxfp8    bf16 activations [rows, K] (row stride ldx) -> q [rows, K] + scales (activations whose
 *                        producer is not fused).
 * b200_quantize_mxfp8_weight  bf16 weight [N, K] (dense) -> tile-major q + scales (once, at load).
 * b200_add_norm_mxfp8    b200_add_norm_bf16 whose normalised output is written as MXFP8 instead of bf16
 *                        (the quantisation of the next linear's input fused into its producer).
 * b200_activation_mxfp8  b200_activation_bf16 with MXFP8 output (input of fc2).
 * b200_gemm_mxfp8        y[M, N] = dq(xq)[M, K] * dq(wq)[N, K]^T (+ bias); workspace as for b200_gemm_bf16.
 * (b200_gemm_mxfp8_swiglu is declared below, after the plain entry points.)
 */
size_t b200_mxfp8_scale_bytes(int rows, int K);
size_t b200_fp8_weight_bytes(int N, int K);
int b200_quantize_mxfp8_weight(const void* w, void* q, void* sf, int N, int K, b200_stream_t stream);
int b200_quantize_mxfp8(const void* x, int64_t ldx, void* q, void* sf, int rows, int K, b200_stream_t stream);
int b200_add_norm_mxfp8(const void* x, const void* bias, const void* residual, const void* gamma, const void* beta,
                        void* hidden_out, void* q_out, void* sf_out, int rows, int hidden, float eps,
                        b200_stream_t stream);
int b200_activation_mxfp8(const void* in, const void* bias, void* q_out, void* sf_out, int rows, int F, int kind,
                          b200_stream_t stream);
/*
 * b200_gemm_mxfp8_swiglu fc1 + SwiGLU (+ MXFP8 quantisation) in one kernel for the gated MLP (MLP.forward, mlp.py:140-213;
 *                        TE's fused fc1 path, extensions/transformer_engine.py:561-583): wq is the fc1 weight [2F, K] in
 *                        the reference's [gate ; up] row order.  One CTA multiplies 128 gate rows and the 128 matching
 *                        up rows by the same token tile; the epilogue writes bf16(bf16(silu(gate)) * up) either as
 *                        MXFP8 (q_out [M, F] + sf_out, the fc2 input) or as bf16 (y_out, row stride ldy) - exactly
 *                        one of the two.  Bit-identical to b200_gemm_mxfp8 + b200_activation_mxfp8 / _bf16 when that GEMM is not split
 *                        along K either (split-K sums its partial sums in another order).  K is not
 *                        split: meant for shapes with F / 128 CTAs enough to fill the GPU.  F % 128 == 0.
 */
int b200_gemm_mxfp8_swiglu(const void* xq, const void* x_sf, const void* wq, const void* w_sf, void* q_out, void* sf_out,
                           void* y_out, int64_t ldy, int M, int F, int K, b200_stream_t stream);
size_t b200_gemm_mxfp8_workspace_bytes(int M, int N, int K);
int b200_gemm_mxfp8(const void* xq, const void* x_sf, const void* wq, const void* w_sf, const void* bias, void* y,
                    int64_t ldy, int M, int N, int K, void* workspace, size_t workspace_bytes, b200_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Block-scaled FP8 linears with fp32 scales: E4M3 weights (tile-major bytes, see above) with one scale per
 * 128 x 128 block (w_scale [ceil(N/128)][K/128]) and E4M3 activations with one scale per token per 128 elements of K
 * (x_scale [K/128][m_pad], m_pad >= M a multiple of 4); scale = amax / 448, value = RNE-saturate(x / scale).
 * Replaces the FP8 path of the TE linears under the `blockwise` recipe (Float8BlockScaling,
 * megatron/core/fp8_utils.py:451-468; arithmetic in Transformer Engine 2.7, absent from the reference tree).
 * Each 128-wide K block is multiplied on tcgen05 (kind::f8f6f4) into its own TMEM accumulator and promoted
 * with w_scale * x_scale[token] in fp32 registers.  K must be a multiple of 128.
 */
int b200_quantize_fp8_weight_block128(const void* w, void* q, float* scale, int N, int K, b200_stream_t stream);
int b200_quantize_fp8_rowblock(const void* x, int64_t ldx, void* q, float* scale, int rows, int K, int m_pad,
                               b200_stream_t stream);
int b200_add_norm_fp8_rowblock(const void* x, const void* bias, const void* residual, const void* gamma,
                               const void* beta, void* hidden_out, void* q_out, float* scale_out, int m_pad, int rows,
                               int hidden, float eps, b200_stream_t stream);
int b200_activation_fp8_rowblock(const void* in, const void* bias, void* q_out, float* scale_out, int m_pad, int rows,
                                 int F, int kind, b200_stream_t stream);
/* 129..256 tokens and N a multiple of 256: optionally (off by default; process-wide switch) the GEMM runs as pairs of
 * CTAs on two SMs that share one tcgen05.mma.cta_group::2 per K step over a 256-token x 256-row output tile - each CTA
 * stages its 128 tokens and its 128 weight rows, so the SMs take in two instead of three times the weight bytes.  Same
 * arithmetic, same split-K workspace sizes, bit-identical results. */
int b200_set_fp8_block_cta_pairs(int enable);
size_t b200_gemm_fp8_block_workspace_bytes(int M, int N, int K);
int b200_gemm_fp8_block(const void* xq, const float* x_scale, int m_pad, const void* wq, const float* w_scale,
                        const void* bias, void* y, int64_t ldy, int M, int N, int K, void* workspace,
                        size_t workspace_bytes, b200_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Row-parallel linear -> residual add -> norm without the split-K reduction launch.
 *
 * At decode sizes the out-projection and fc2 GEMMs (RowParallelLinear.forward, layers.py:1225-1281) are split
 * along K; their fp32 partial sums are normally reduced by a second kernel, and the residual add + norm that
 * follows in the layer (transformer_layer.py:433-660: bias-dropout-add, then pre_mlp_layernorm / the next
 * layer's input_layernorm) is a third.  The *_splitk entry points leave the partial sums
 * [num_splits][M][N] fp32 in `partials` (b200_gemm_*_splitk_bytes gives the size; *num_splits is written on the
 * host before the call returns; one split is possible), and b200_add_norm_splitk_* read them in place of `x`:
 * x = bf16(sum of the splits in split order), then exactly what b200_add_norm_* does (`bias` here is the linear's
 * bias).  Results are bit-identical to b200_gemm_* followed by b200_add_norm_*.  hidden <= 8192.
 *
 * b200_activation_splitk_* do the same for the column-parallel fc1 -> activation pair (MLP.forward,
 * megatron/core/transformer/mlp.py:140-213): `partials` [num_splits][rows][2F] (gated kinds) or [num_splits][rows][F]
 * replace the bf16 input of b200_activation_*; bit-identical to GEMM + reduction + b200_activation_*.
 */
size_t b200_gemm_bf16_splitk_bytes(int M, int N, int K);
int b200_gemm_bf16_splitk(const void* x, int64_t ldx, const void* w, int M, int N, int K, float* partials,
                          size_t partials_bytes, int* num_splits, b200_stream_t stream);
size_t b200_gemm_mxfp8_splitk_bytes(int M, int N, int K);
int b200_gemm_mxfp8_splitk(const void* xq, const void* x_sf, const void* wq, const void* w_sf, int M, int N, int K,
                           float* partials, size_t partials_bytes, int* num_splits, b200_stream_t stream);
size_t b200_gemm_fp8_block_splitk_bytes(int M, int N, int K);
int b200_gemm_fp8_block_splitk(const void* xq, const float* x_scale, int m_pad, const void* wq, const float* w_scale,
                               int M, int N, int K, float* partials, size_t partials_bytes, int* num_splits,
                               b200_stream_t stream);
int b200_add_norm_splitk_bf16(const float* partials, int num_splits, const void* bias, const void* residual,
                              const void* gamma, const void* beta, void* hidden_out, void* normed_out, int rows, int hidden,
                              float eps, b200_stream_t stream);
int b200_add_norm_splitk_mxfp8(const float* partials, int num_splits, const void* bias, const void* residual,
                               const void* gamma, const void* beta, void* hidden_out, void* q_out, void* sf_out, int rows,
                               int hidden, float eps, b200_stream_t stream);
int b200_add_norm_splitk_fp8_rowblock(const float* partials, int num_splits, const void* bias, const void* residual,
                                      const void* gamma, const void* beta, void* hidden_out, void* q_out, float* scale_out,
                                      int m_pad, int rows, int hidden, float eps, b200_stream_t stream);
int b200_activation_splitk_bf16(const float* partials, int num_splits, const void* bias, void* out, int rows, int F, int kind,
                                b200_stream_t stream);
int b200_activation_splitk_mxfp8(const float* partials, int num_splits, const void* bias, void* q_out, void* sf_out, int rows,
                                 int F, int kind, b200_stream_t stream);
int b200_activation_splitk_fp8_rowblock(const float* partials, int num_splits, const void* bias, void* q_out, float* scale_out,
                                        int m_pad, int rows, int F, int kind, b200_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Tensor parallelism: the all-reduce after a row-parallel linear (mappings.py:22-33 called from
 * RowParallelLinear.forward, layers.py:1225-1281) fused into the residual-add + norm kernel that follows it.
 *
 * Every rank of the node owns a data buffer of two slots [max_rows][hidden] bf16 and a flag array
 * [world_size][max_rows] int32 (zero-initialised), both created with b200_peer_buffer_create and mapped by the
 * other ranks through the 64-byte CUDA IPC handle (b200_peer_buffer_open); `counters` is 2 local int32 (zeroed).
 * A rank writes the bf16 output of its row-parallel GEMM into its own slot; b200_allreduce_add_norm_* then
 * (per token row) tells the peers the row is ready, waits - at most 2 s, then B200 device status 4 - until theirs
 * are, reads all ranks' rows with peer loads and uses x = bf16(sum in rank order, fp32) exactly like
 * b200_add_norm_*'s x.  All ranks obtain identical bits.  Consecutive calls must alternate the slot (0, 1, 0, ...)
 * and every rank must issue the same sequence of calls.  hidden <= 8192, world_size 2..8; plain peer loads and stores only.
 * The slot must have been written by an EARLIER kernel launch on the same stream (the GEMM): the ready flags are relaxed
 * stores that rely on that kernel's completion for the visibility of the rows.
 */
typedef struct {
  int32_t world_size, rank;
  int32_t max_rows, hidden;
  void* data[8];        /* data[r]: rank r's data buffer (two slots); data[rank] is local memory */
  int32_t* flags[8];    /* flags[r]: rank r's flag array */
  int32_t* counters;    /* local */
} b200_tp_comm;
int b200_peer_buffer_create(size_t bytes, void** ptr, unsigned char handle[64]);
int b200_peer_buffer_open(const unsigned char handle[64], void** ptr);
int b200_peer_buffer_close(void* ptr);
int b200_peer_buffer_destroy(void* ptr);
int b200_allreduce_add_norm_bf16(const b200_tp_comm* comm, int slot, const void* bias, const void* residual,
                                 const void* gamma, const void* beta, void* hidden_out, void* normed_out, int rows,
                                 int hidden, float eps, b200_stream_t stream);
int b200_allreduce_add_norm_mxfp8(const b200_tp_comm* comm, int slot, const void* bias, const void* residual,
                                  const void* gamma, const void* beta, void* hidden_out, void* q_out, void* sf_out, int rows,
                                  int hidden, float eps, b200_stream_t stream);
int b200_allreduce_add_norm_fp8_rowblock(const b200_tp_comm* comm, int slot, const void* bias, const void* residual,
                                         const void* gamma, const void* beta, void* hidden_out, void* q_out,
                                         float* scale_out, int m_pad, int rows, int hidden, float eps,
                                         b200_stream_t stream);

/*
 * Two-shot form of the same fusion, for larger groups (the reference's symmetric-memory all-reduce has the same
 * choice: `two_shot` / `one_shot`, megatron/training/arguments.py:1437-1442).  The token rows are divided among the
 * ranks (rank r owns rows [r * ceil(rows / w), ...)); a rank sums ITS rows from all ranks' `in` buffers (peer loads),
 * adds bias + residual, normalises (+ quantises: q_mode 0 bf16, 1 MXFP8, 2 the 128-block recipe) and stores the
 * finished rows into EVERY rank's output buffers (peer stores): `hidden_out` [max_rows][hidden] bf16, `normed_out`
 * ([max_rows][hidden] bf16, or E4M3 bytes) and `scales_out` (MXFP8 tile-layout scale bytes of a [max_rows, hidden]
 * matrix, or fp32 [hidden / 128][m_pad]).  Each row is computed exactly once, so all ranks hold identical bits.
 * `flags[r]`: 16 int32 of rank r (zero-initialised, peer-mapped); `counters`: 4 local int32 (zeroed).  Two flag
 * exchanges per call (inputs complete / outputs stored), each wait bounded by b200_set_wait_limit_ns (device status
 * 4 on expiry); the kernel completes only after every rank's rows have arrived, so later kernels on the stream may
 * read the local output buffers.  `residual` is local memory and may be this rank's `hidden_out` buffer itself.
 * One buffer of each kind is enough (no slot alternation); every rank must issue the same sequence of calls.  `in[rank]`
 * must have been written by an EARLIER kernel launch on the same stream (see above).
 */
typedef struct {
  int32_t world_size, rank;
  int32_t max_rows, hidden;
  int32_t m_pad;           /* row stride of the fp32 scale matrix (q_mode 2): >= max_rows, multiple of 4 */
  void* in[8];             /* in[r]: rank r's partial GEMM output [max_rows][hidden] bf16; in[rank] is local */
  void* hidden_out[8];
  void* normed_out[8];
  void* scales_out[8];     /* may be NULL when q_mode 0 is the only mode used */
  int32_t* flags[8];
  int32_t* counters;
} b200_tp_exchange;
int b200_allreduce2_add_norm(const b200_tp_exchange* comm, const void* bias, const void* residual, const void* gamma,
                             const void* beta, int q_mode, int rows, int hidden, float eps, b200_stream_t stream);
/* The same with the row-parallel GEMM's split-K partial sums as input (b200_gemm_*_splitk: `partials`
 * [num_splits][rows][hidden] fp32, local memory): the kernel first sums them in split order into this rank's `in` buffer
 * (what the GEMM's own reduction kernel would have written there) and then proceeds as above - one launch fewer per
 * linear, bit-identical results. */
int b200_allreduce2_add_norm_splitk(const b200_tp_exchange* comm, const float* partials, int num_splits, const void* bias,
                                    const void* residual, const void* gamma, const void* beta, int q_mode, int rows,
                                    int hidden, float eps, b200_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Paged-KV attention for the dynamic context.
 *
 * qkv        [T, nkv, (g+2)*d] bf16: per KV group g query heads, then the key, then the value
 *            (layout of SelfAttention.get_query_key_value_tensors, megatron/core/transformer/attention.py:985-1021)
 * k_cache/v_cache  [n_chunks, chunk, nkv, d] bf16: one layer of the context's memory_buffer
 *            (megatron/core/inference/contexts/dynamic_context.py:296-308, 547-564)
 * block_table [rows, max_chunks] int32, kv_seq_lengths [T] int32 (kv length INCLUDING this step's token),
 * row_of_token [T] int32 or NULL (NULL: token t uses block-table row t)
 * out        [T, nq*d] bf16
 *
 * b200_rope_append: RoPE on q (in place in qkv) and k, then scatter k, v into the cache at
 *   (token_to_chunk_idx[t], token_to_local_pos[t]).  Replaces apply_rotary_emb_key/query + append_key_value_cache
 *   (dynamic_context.py:511-545, 566-631; megatron/core/models/common/embeddings/rope_utils.py:92-126).
 *   cos/sin: bf16 tables [max_pos, d/2] or NULL for no RoPE.
 * b200_paged_attention: softmax(q k^T / sqrt(d)) v over each row's paged KV; replaces
 *   flash_attn_with_kvcache / flash_attn_varlen_func with block_table
 *   (megatron/core/transformer/attention.py:470-601).  With fuse_rope_append != 0 it also does the work of
 *   b200_rope_append for decode steps (one new token per request) inside the same kernel.
 *   num_splits > 1 splits every row's context into that many ranges (flash-decoding) and needs
 *   `workspace` of b200_paged_attention_workspace_bytes.
 * FP8 pool (kv_cache_fp8; an extension, the reference's pool is always params_dtype; head_dim 128, chunk_size a
 *   multiple of 128): keys and values are stored as E4M3 bytes with one fp32 scale per KV head; both kernels
 *   quantise what they append (RNE-saturate(x / scale)) and the attention kernel multiplies E4M3 by E4M3 on the
 *   tensor cores (queries and probabilities as two E4M3 terms each).  Keys keep the layout
 *   [chunk][token][head][dim]; the value bytes of a chunk are stored transposed and permuted,
 *   [chunk][head][dim][b200_fp8_value_position(token)], so that the kernel needs no transposition.
 */
typedef struct {
  const void* qkv;
  void* k_cache;
  void* v_cache;
  const int32_t* block_table;
  const int32_t* kv_seq_lengths;
  const int32_t* row_of_token;
  const int64_t* token_to_pos_ids;          /* RoPE position of q  */
  const int64_t* token_to_pos_in_request;   /* RoPE position of k  */
  const int64_t* token_to_chunk_idx;
  const int64_t* token_to_local_pos;
  const void* rope_cos;
  const void* rope_sin;
  void* out;
  void* workspace;
  size_t workspace_bytes;
  int32_t num_tokens;     /* T */
  int32_t num_q_heads;    /* nq (this rank) */
  int32_t num_kv_heads;   /* nkv (this rank) */
  int32_t head_dim;       /* 64 or 128 */
  int32_t chunk_size;     /* tokens per chunk, multiple of 64 */
  int32_t num_chunks;     /* chunks in the pool */
  int32_t max_chunks_per_row; /* block_table row stride */
  int32_t num_splits;
  int32_t fuse_rope_append;
  float softmax_scale;    /* 0 = 1/sqrt(d) */
  int32_t kv_cache_fp8;   /* != 0: k_cache / v_cache hold E4M3 bytes (head_dim 128), value = byte * scale[head];
                             1: queries and probabilities as two E4M3 terms (adds ~1e-3 to the pool's own ~4e-2 error);
                             2: one term each (total ~5e-2, 1.6x faster) */
  const float* k_scale;   /* [nkv] fp32, FP8 pool only */
  const float* v_scale;   /* [nkv] fp32, FP8 pool only */
  const float* qkv_partials; /* NULL, or [qkv_num_splits][T][nkv*(g+2)*d] fp32: the split-K partial sums of the QKV GEMM
                                (b200_gemm_*_splitk) for b200_paged_attention to use instead of `qkv`: every unit sums its own
                                head vectors in split order and rounds once to bf16, the bits the GEMM's reduction kernel
                                would have produced (no QKV bias then).  b200_rope_append and the prefill kernel need `qkv`. */
  int32_t qkv_num_splits;
  const int32_t* row_order; /* [T] int32 or NULL: a permutation of 0..T-1; the attention kernel starts its work on the
                               rows in this order (longest context first balances the SMs).  Results do not depend on it. */
  void* out_q;              /* NULL, or E4M3 bytes [T][nq * d]: b200_paged_attention writes its output quantised as the
                               FP8 input of the out-projection instead of bf16 `out` (which is then not written): the
                               bits b200_quantize_mxfp8 / b200_quantize_fp8_rowblock would produce from the bf16 output
                               (TE quantises the attention output inside its row-parallel linear,
                               megatron/core/extensions/transformer_engine.py:736-828).  Decode kernels only. */
  void* out_scales;         /* out_q_mode 1: E8M0 scales in the MXFP8 tile layout (b200_mxfp8_scale_bytes(T, nq * d));
                               out_q_mode 2: fp32 [nq][out_m_pad], one scale per token per head (head_dim 128 only) */
  int32_t out_q_mode;       /* 1: MXFP8, 2: 128-block recipe */
  int32_t out_m_pad;        /* out_q_mode 2: row stride of out_scales (>= T, multiple of 4) */
} b200_attention_args;

size_t b200_paged_attention_workspace_bytes(int num_tokens, int num_q_heads, int head_dim, int num_splits);
int b200_fp8_value_position(int token_in_chunk);
int b200_rope_append(const b200_attention_args* args, b200_stream_t stream);
int b200_paged_attention(const b200_attention_args* args, b200_stream_t stream);
/* Prefill / mixed steps (flash_attn_varlen_func with block_table, attention.py:501-558), after b200_rope_append:
 * `units` [num_units][4] int32 on the device = {block-table row, first token, number of tokens, 0}; the tokens of a
 * unit are consecutive tokens of ONE request, at most 64 / (nq / nkv) of them; entries with 0 tokens are skipped (so a
 * fixed-size list can be padded).  kv_seq_lengths[t] is the number of keys token t sees (its position + 1).  Same
 * result as b200_paged_attention with row_of_token (one CTA per token) up to summation order, but every K/V tile is
 * read once per unit instead of once per token.  bf16 pool, nq / nkv in {1, 2, 4, 8, 16}. */
int b200_paged_prefill_attention(const b200_attention_args* args, const int32_t* units, int num_units,
                                 b200_stream_t stream);

/* ---------------------------------------------------------------------------------------
 * Sampling over [rows, vocab] bf16 logits (row stride ld elements).
 * b200_argmax_bf16: greedy token (smallest index among equal maxima) -> int64; replaces torch.argmax in
 *   TextGenerationController.sample_from_logits (megatron/core/inference/text_generation_controllers/
 *   text_generation_controller.py:288-290).
 * b200_topk_probs_bf16: temperature, keep logits >= k-th largest, softmax -> fp32 probs [rows, vocab];
 *   replaces modify_logits_for_top_k_filtering + softmax (same file :216-219, 292-305).  The draw itself
 *   (torch.multinomial on the controller's generator) stays with the caller.
 * b200_topp_probs_bf16: temperature, nucleus filter, softmax over the kept set -> fp32 probs; replaces
 *   modify_logits_for_top_p_filtering + softmax (same file :221-240, 306-309): with tokens in descending order
 *   of logit (equal logits by ascending index) a token is kept iff the probability mass strictly ahead of it is
 *   <= top_p.  Computed in fp32 (the reference's cumulative sum runs in the logits' dtype).
 */
int b200_argmax_bf16(const void* logits, int64_t ld, int64_t* out, int rows, int vocab, b200_stream_t stream);
/* Greedy sampling over VOCAB-PARALLEL logits without gathering them (the reference all-gathers [B, V/tp] logits on
 * every step, megatron/core/tensor_parallel/layers.py:1037-1039 -> mappings.py:80-96, and then takes the argmax of the
 * full row).  b200_argmax_shard_bf16: per row of this rank's shard [rows, vocab_shard] one 64-bit key =
 * (order-preserving code of the largest value << 32) | (2^32 - 1 - (index_offset + its smallest index)).  The keys of
 * all ranks ([shards][rows], 8 bytes per row and rank - an all-gather of a few KB) go to b200_argmax_merge, whose
 * maximum per row is the token torch.argmax would pick on the gathered row (ties: smallest index). */
int b200_argmax_shard_bf16(const void* logits, int64_t ld, uint64_t* keys, int rows, int vocab, int64_t index_offset,
                           b200_stream_t stream);
int b200_argmax_merge(const uint64_t* keys, int shards, int rows, int64_t* out, b200_stream_t stream);
int b200_topk_probs_bf16(const void* logits, int64_t ld, float* probs, int rows, int vocab, int top_k,
                         float temperature, b200_stream_t stream);
int b200_topp_probs_bf16(const void* logits, int64_t ld, float* probs, int rows, int vocab, float top_p,
                         float temperature, b200_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_DECODE_H_ */
