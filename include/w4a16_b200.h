/*
 * w4a16_b200 -- C ABI of the B200 (sm_100a) W4A16 linear library.
 *
 * Packed weight format (shared with the reference project, w4a16/quantization.py:4-113):
 *   packed  uint8  [N, K/2] row-major; byte j of a row = code(2j) in bits 0-3, code(2j+1) in
 *           bits 4-7, 4-bit two's complement (all 16 values decode, 0x8 -> -8)
 *   scales  fp16   [N, K/group_size] row-major, one scale per group_size consecutive k
 *   x       fp16   [M, K] row-major        y  fp16 [M, N] row-major
 *   y[m][n] = half( sum_k float(x[m][k]) * code[n][k] * float(scale[n][k/group_size]) )
 *
 * Conventions for every entry point:
 *   - all pointers are DEVICE pointers on the current device unless a name ends in _host;
 *   - the call enqueues work on `stream` and returns; it never synchronises, allocates or frees;
 *   - inputs are read-only, outputs are fully overwritten;
 *   - the return value is W4A16_OK (0) or a negative W4A16_ERR_* code; nothing is launched on error.
 *
 * The torch operator shim (nibble_b200/csrc/int4_linear.cpp) binds exactly these functions.
 */
#ifndef W4A16_B200_H_
#define W4A16_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* A cudaStream_t, spelled without the CUDA headers. */
typedef struct CUstream_st* w4a16_stream_t;

enum {
    W4A16_OK = 0,
    W4A16_ERR_NULL_POINTER = -1,  /* a required pointer is NULL                                  */
    W4A16_ERR_BAD_SHAPE = -2,     /* negative size, odd K, K % group_size != 0                    */
    W4A16_ERR_BAD_GROUP = -3,     /* group_size <= 0 or odd (dequantize: not a multiple of 32)    */
    W4A16_ERR_MISALIGNED = -4,    /* a pointer misses the alignment this entry point requires     */
    W4A16_ERR_WORKSPACE = -5,     /* workspace missing or too small for the requested split       */
    W4A16_ERR_BAD_CONFIG = -6,    /* an explicit launch configuration is not one the library has  */
    W4A16_ERR_LAUNCH = -7,        /* the CUDA runtime refused the launch (see cudaGetLastError)   */
    W4A16_ERR_TOO_LARGE = -8      /* a size exceeds what this entry point supports                */
};

/* Flags for w4a16_linear_f16. */
enum {
    /* Launch with programmatic stream serialisation: the kernel may start, and prefetch packed
     * weights and scales, while the preceding kernel of the stream is still running; it waits for
     * that kernel before it reads x or writes y.  Only valid when nothing earlier in the stream
     * that may still be running writes `packed` or `scales`. */
    W4A16_FLAG_PROGRAMMATIC_LAUNCH = 1u << 0,
    /* Route to the generic kernel even when the fast path applies (testing / A-B). */
    W4A16_FLAG_FORCE_GENERIC = 1u << 1,
    /* y is float [M, N] and receives the unrounded FP32 sums: for K-sharded layers whose partial
     * results are added across devices before the single rounding to FP16. */
    W4A16_FLAG_OUTPUT_F32 = 1u << 2,
    /* Keep batches of 65 rows and more on the mma.sync kernel instead of the tcgen05 GEMM (A/B, tests). */
    W4A16_FLAG_NO_TCGEN05 = 1u << 3,
    /* Route to the tcgen05 GEMM whatever the batch size, when the fast path applies and y is FP16 (A/B, tests). */
    W4A16_FLAG_FORCE_TCGEN05 = 1u << 4
};

/* Explicit launch shape of the fused tensor-core kernel; zero fields mean "choose for me". */
typedef struct w4a16_linear_config {
    int32_t row_tiles;   /* 16-row tiles owned by one warp: 1 or 2                                 */
    int32_t k_warps;     /* warps of a CTA that split K of one row tile between them: 1, 2, 4, 8   */
    int32_t k_splits;    /* CTAs that split K of one row tile: 1..8 (>1 needs the workspace)       */
    int32_t unroll;      /* 128-wide K chunks per pipeline step: 1 or 2 (2 needs K/128 even and    */
                         /* 4-byte aligned scales)                                                 */
    int32_t stages;      /* slots of the asynchronous-copy ring each thread keeps in flight: 3..8  */
} w4a16_linear_config;

/*
 * Fused unpack + dequantise + matmul:  y = x . dequant(packed, scales)^T.
 * Replaces the reference's int4_linear_cuda (csrc/int4_linear_kernel.cu:641-802) and the kernels
 * it dispatches to (decode_multirow :325-404, small_batch :542-617, naive :20-69).
 *
 * Fast path when group_size == 128 and x, packed are 16-byte aligned: M <= 8 runs the mma.sync
 * streaming kernel, M >= 65 (and 9..64 on layers of N >= 4096 where a cost model built from measurements
 * favours it) a tcgen05 GEMM whose producer warps dequantise into the operand tiles
 * (no FP16 weight matrix in memory; weights enter the product as half(code * scale), the arithmetic of
 * the reference's dequantise-then-matmul prefill route, w4a16/linear.py:132-152).
 * Otherwise a generic kernel that accepts any even group_size and any alignment.
 * The GEMM shares the K of an output tile between up to four CTAs when a layer has too few 128-row tiles for the
 * SMs (FP32 partial sums in the workspace, added in order and rounded once by a second small kernel); without
 * enough workspace it runs unsplit.
 * `workspace` may be NULL (then K is never split across CTAs); if given it must be 16-byte aligned,
 * hold at least w4a16_linear_workspace_bytes(M, N, K) bytes, be zero-filled before its first use
 * and not be shared by calls that may run concurrently.  The library leaves it ready for re-use, by calls
 * of any shape: the arrival counters live in a fixed 256 KB prefix that partial sums never touch (problems
 * with more than 65536 pairs of 16-row tile x 8-row batch block use a longer prefix; re-zero a workspace that
 * such a problem shares with others).
 * M == 0 or N == 0 returns W4A16_OK without launching.
 */
int w4a16_linear_f16(const void* x, const void* packed, const void* scales, void* y,
                     int64_t M, int64_t N, int64_t K, int64_t group_size,
                     void* workspace, size_t workspace_bytes,
                     uint32_t flags, w4a16_stream_t stream);

/* Same as w4a16_linear_f16 with an explicit launch shape for the fast path (tuning, tests).
 * Returns W4A16_ERR_BAD_CONFIG when the fast path does not apply or the shape is not built. */
int w4a16_linear_f16_config(const void* x, const void* packed, const void* scales, void* y,
                            int64_t M, int64_t N, int64_t K, int64_t group_size,
                            void* workspace, size_t workspace_bytes,
                            uint32_t flags, const w4a16_linear_config* config,
                            w4a16_stream_t stream);

/* Bytes of workspace that let w4a16_linear_f16 split K across CTAs for this problem
 * (FP32 partial sums plus arrival counters).  Never fails; returns 0 for empty problems. */
size_t w4a16_linear_workspace_bytes(int64_t M, int64_t N, int64_t K);
/* The same for a call made with `flags`: batches that w4a16_linear_f16 sends to the tcgen05 GEMM
 * (M >= 65 without W4A16_FLAG_OUTPUT_F32 / W4A16_FLAG_NO_TCGEN05) or to the generic kernel need none.
 * w4a16_linear_workspace_bytes(M, N, K) is this function with flags == 0. */
size_t w4a16_linear_workspace_bytes_flags(int64_t M, int64_t N, int64_t K, uint32_t flags);

/*
 * Tensor-parallel exchange (no counterpart in the reference, which is single-GPU).  A layer sharded over
 * `world` GPUs of one node hands its result to every GPU from the kernel epilogue -- plain stores into
 * peer-mapped memory over NVLink -- and the kernel that consumes the result picks it up while it stages its
 * activations, with its weight prefetch already in flight.  No collective library call, no host involvement,
 * and no fence or flag round trip on the way: every element travels together with a tag that says which
 * publication it belongs to, in one naturally atomic store, and the reader simply re-reads an element until
 * its tag is the one it expects (the low-latency scheme collective libraries use for small messages).
 *
 * Element format in a result buffer:
 *   FP16 results   uint32 = half bits | tag << 16            (element (m, n) at index m * ld + n)
 *   FP32 partials  uint64 = float bits | (uint64)tag << 32
 *   tag of publication e = 0x8000 | (e & 0x7FFF); zero-filled memory therefore never looks published.
 *
 * Memory a sharded layer owns on every rank (mapped on all ranks by the caller: CUDA IPC, cuMem, or
 * torch's symmetric memory; zero-filled at start):
 *   two result buffers, `buffer_stride` bytes apart (publication e goes to buffer e & 1),
 *   consumed[world]   uint32: consumed[c] = latest publication that reader c has finished reading in ITS
 *                     buffers (readers write it on every rank, so that senders learn when a buffer is free).
 * And private device words on each rank, zero at start: done_counter, send_epoch, staged_counter, status.
 *
 * Sender (w4a16_peer_target): e = *send_epoch + 1.  Before its first store the kernel waits (bounded) until
 * consumed[r] >= e - 2 for all r on this rank; then every output element (m, n) of this rank's result goes,
 * tagged, to outputs[r] + (e & 1) * buffer_stride at index m * ld + column_offset + n, for every rank r; the
 * launch ends by setting *send_epoch = e.  It does not wait for anybody else.
 * Column-parallel layers use it as an all-gather (ld = full N, column_offset = rank * N_local); row-parallel
 * layers push FP32 partials (outputs[r] = staging[r] + rank * M * N elements) and finish with
 * w4a16_sum_partials_f16.
 *
 * Reader (w4a16_peer_source): after the preceding kernel of the stream has completed it reads
 * e = *epoch (the send_epoch word of the layer that produced the data, on this rank -- so that layer's
 * launch must precede the reader in the stream), reads buffer e & 1, re-reading (bounded) every element whose
 * tag is not yet that of e, and when every CTA has read writes e to consumed[rank] on every rank.
 *
 * Every wait gives up after max_polls polls and records who was missing in *status -- 1 + sender for an
 * element that never arrived (the sender is worked out from the element's column: first_column and
 * columns_per_rank; for FP32 partials it is the slot), 33 + reader for a reader that never released a buffer --
 * so a missing rank ends in an error the host can read, never in a hung GPU.  Every rank must issue the same
 * sequence of launches for a layer, and every publication must be read (by one reader) on every rank.
 */
typedef struct w4a16_peer_target {
    void* const* outputs;         /* [world] result buffer 0 of this layer on each rank (plus this rank's offset)   */
    const uint32_t* consumed;     /* this rank's consumed[] array                                                     */
    uint32_t* done_counter;
    uint32_t* send_epoch;
    uint32_t* status;
    int64_t buffer_stride;        /* bytes between result buffer 0 and 1                                              */
    int64_t ld;
    int64_t column_offset;
    int64_t max_polls;
    int32_t rank;
    int32_t world;
} w4a16_peer_target;

typedef struct w4a16_peer_source {
    const uint32_t* epoch;        /* send_epoch word of the producing layer on this rank                              */
    uint32_t* const* consumed;    /* [world] the consumed[] array of each rank                                        */
    uint32_t* staged_counter;
    uint32_t* status;
    int64_t buffer_stride;
    int64_t max_polls;
    int64_t first_column;         /* column of the gathered result that x (or the copy) starts at                     */
    int64_t columns_per_rank;     /* columns each sender contributes (0: unknown, failures are reported as sender 0)  */
    int32_t rank;
    int32_t world;
} w4a16_peer_source;

/* w4a16_linear_f16 as one stage of a tensor-parallel chain (fast path only: group 128, aligned pointers,
 * M <= 64; otherwise W4A16_ERR_BAD_CONFIG).  `target` non-NULL: the result goes to every rank as described
 * above and y is ignored; NULL: the result goes to y.  `source` non-NULL: x points at tagged FP16 elements
 * (4 bytes each) in result buffer 0 of the producing layer on this rank and the kernel adds the parity
 * offset itself; NULL: plain FP16 x.
 * x_ld is the distance between batch rows of x in elements (>= K, a multiple of 8), so that a column slice of
 * a wider gathered result can be the input. */
int w4a16_linear_f16_peers(const void* x, int64_t x_ld, const void* packed, const void* scales, void* y,
                           int64_t M, int64_t N, int64_t K, int64_t group_size,
                           void* workspace, size_t workspace_bytes, uint32_t flags,
                           const w4a16_peer_target* target, const w4a16_peer_source* source,
                           w4a16_stream_t stream);

/* Reader as a kernel of its own: copies `count` FP16 elements (a multiple of 8) of the publication described
 * by `source` from the current result buffer (`buffer0` + parity offset, tagged elements) to `out` (plain
 * FP16), waiting for elements that have not arrived yet, then releases the buffer.  count may be 0 (release
 * only: for a result nobody needs). */
int w4a16_wait_peers(const w4a16_peer_source* source, const void* buffer0, void* out, int64_t count,
                     uint32_t flags, w4a16_stream_t stream);

/* y[i] = half(sum_r partials[r * count + i]), r ascending: the finish of a row-parallel layer.
 * With `source` non-NULL `partials` is result buffer 0 of the layer (tagged FP32 elements, 8 bytes each) and
 * the kernel is the reader of the publication (parity offset, wait per element, release) as above; NULL: a
 * plain sum over a local float array.
 * flags (here and for w4a16_wait_peers): W4A16_FLAG_PROGRAMMATIC_LAUNCH only. */
int w4a16_sum_partials_f16(const void* partials, void* y, int64_t count, int32_t world,
                           const w4a16_peer_source* source, uint32_t flags, w4a16_stream_t stream);

/*
 * packed + scales -> FP16 [N, K], bit-identical to half(float(code) * float(scale)).
 * Replaces the reference's int4_dequantize_cuda (csrc/int4_linear_kernel.cu:805-867).
 * Requires group_size a positive multiple of 32 and `packed` 16-byte aligned, as the reference does.
 */
int w4a16_dequantize_f16(const void* packed, const void* scales, void* weights,
                         int64_t N, int64_t K, int64_t group_size, w4a16_stream_t stream);

/*
 * FP16 / FP32 weights [N, K] -> packed codes [N, K/2] and FP16 scales [N, K/group_size] on the device,
 * bit-identical to the reference's host quantiser quantize_and_pack_weights
 * (w4a16/quantization.py:65-113): step = absmax/7 in FP32 (1 for an all-zero group),
 * code = clamp(round_half_even(w / step), -7, 7), scale = half(step).  group_size: positive, even,
 * dividing K.  The reference has no device version of this step.
 */
int w4a16_quantize_pack_f16(const void* weights, void* packed, void* scales,
                            int64_t N, int64_t K, int64_t group_size, w4a16_stream_t stream);
int w4a16_quantize_pack_f32(const void* weights, void* packed, void* scales,
                            int64_t N, int64_t K, int64_t group_size, w4a16_stream_t stream);

/*
 * w4a16_linear_f16 whose activations are computed while they are staged on chip, so that the
 * producer of x needs no kernel of its own (no counterpart in the reference):
 *   W4A16_INPUT_SILU_MUL     x[m][k] = half(silu(g[m][k])) * u[m][k], where the `x` argument points at
 *                            rows [g | u] of 2K values (the output of a fused gate/up projection);
 *   W4A16_INPUT_ADD_RMSNORM  M must be 1; s = half(x + second) (second may be NULL),
 *                            x'[k] = norm_weight[k] * half(float(s[k]) * rsqrt(mean(s^2) + eps)); s is also
 *                            written to stream_out (K values; must not alias x or second) when non-NULL.
 * Same arithmetic as w4a16_silu_mul_f16 / w4a16_add_rmsnorm_f16 followed by w4a16_linear_f16.
 * Only the tensor-core path takes a transform: group_size 128 and 16-byte aligned x, packed, second,
 * norm_weight and stream_out, M <= 64; otherwise W4A16_ERR_BAD_CONFIG.  transform == NULL is w4a16_linear_f16.
 */
enum { W4A16_INPUT_PLAIN = 0, W4A16_INPUT_SILU_MUL = 1, W4A16_INPUT_ADD_RMSNORM = 2 };
typedef struct w4a16_input_transform {
    int32_t kind;
    const void* second;
    const void* norm_weight;
    void* stream_out;
    float eps;
} w4a16_input_transform;
int w4a16_linear_f16_input(const void* x, const void* packed, const void* scales, void* y,
                           int64_t M, int64_t N, int64_t K, int64_t group_size,
                           void* workspace, size_t workspace_bytes, uint32_t flags,
                           const w4a16_input_transform* transform, w4a16_stream_t stream);

/*
 * The three kernels either side of the linears in one LLaMA decode step (batch 1), for a runner
 * that replaces the framework's decoder-layer code (the reference drives HuggingFace's
 * model.generate, scripts/generate.py:260-365; the arithmetic restated is transformers'
 * LlamaRMSNorm, apply_rotary_pos_emb, grouped-KV scaled-dot-product attention and LlamaMLP).
 *
 * add_rmsnorm: s = half(stream_in + delta) (delta may be NULL); stream_out = s (may be NULL or alias
 *   stream_in); normed = weight * half(float(s) * rsqrt(mean(float(s)^2) + eps)).  One row of `hidden`.
 * silu_mul: out[i] = half(silu(gate_up[i])) * gate_up[intermediate + i].
 * attention_decode: qkv = [q_heads*d | kv_heads*d | kv_heads*d] of the token at *position (device
 *   scalar); applies RoPE (cos, sin of position * inv_freq[j], times rope_scale, rounded to FP16) to
 *   q and k, writes k and v into caches laid out [kv_heads][max_len][d], and writes
 *   softmax(q k^T * softmax_scale) v over positions 0..*position to out [q_heads*d].  d is 64 or
 *   128.  A position outside [0, max_len) sets *status to 1 and nothing is written.
 * flags: W4A16_FLAG_PROGRAMMATIC_LAUNCH as for the linear (each kernel waits for its predecessor before
 *   it reads or writes memory).  One exception, for latency: attention_decode reads *position, inv_freq and
 *   the cache rows below the position BEFORE that wait.  A programmatic chain only orders a kernel after its
 *   immediate predecessor, so nothing launched programmatically ahead of an attention_decode may write
 *   `position` or the caches without a fully serialising (ordinary) launch in between -- e.g. put the kernel
 *   that advances the position at the end of a step and start the next step with an ordinary launch.
 */
int w4a16_add_rmsnorm_f16(const void* stream_in, const void* delta, const void* weight, void* stream_out,
                          void* normed, int64_t hidden, float eps, uint32_t flags, w4a16_stream_t stream);
int w4a16_silu_mul_f16(const void* gate_up, void* out, int64_t intermediate, uint32_t flags, w4a16_stream_t stream);
/* *token = index of the first maximum of `count` FP16 logits (NaNs are never chosen); when `position` is
 * non-NULL, *position += 1: the end of a greedy decode step in one launch. */
int w4a16_argmax_advance_f16(const void* logits, int64_t count, int64_t* token, int64_t* position,
                             uint32_t flags, w4a16_stream_t stream);
int w4a16_attention_decode_f16(const void* qkv, void* k_cache, void* v_cache, void* out,
                               const int64_t* position, const float* inv_freq, int32_t q_heads,
                               int32_t kv_heads, int32_t head_dim, int32_t max_len, float rope_scale,
                               float softmax_scale, uint32_t* status, uint32_t flags, w4a16_stream_t stream);

/*
 * One whole decode step (batch 1) of a LLaMA-architecture model as ONE cooperative kernel launch: resident
 * CTAs walk a prebuilt list of operations (per block: fused q/k/v with add + RMSNorm inside, attention, o_proj,
 * fused gate/up with add + RMSNorm inside, down_proj with SiLU * up inside; then lm_head with the final norm and
 * the arg-max), handing over between operations through one counter in L2 instead of a kernel boundary, the next
 * operation's weights already being fetched while the hand-off is waited for.  Same arithmetic as the kernels
 * above.  No counterpart in the reference (it drives HuggingFace's generate(), scripts/generate.py:260-365).
 *
 * The caller describes the model once (device pointers; q/k/v and gate/up packed as single matrices: rows
 * [q | k | v] and [gate | up]; all group size 128; hidden, intermediate and q_heads * head_dim multiples of 256;
 * head_dim 64 or 128; KV caches [kv_heads][max_len][head_dim] per layer), provides w4a16_decode_plan_bytes()
 * bytes of 256-byte aligned device memory, and builds the plan (this copies the operation list to the device and
 * synchronises `stream`).  The plan also holds the step's work buffers.  `token` and `position` are device
 * scalars: a step consumes *token at *position, appends to the caches, leaves the greedy next token in *token and
 * adds 1 to *position.  info->logits (FP16 [vocab]) and info->status (uint32: 0 healthy, 1 the position was outside
 * the cache, 0x100 + n: the hand-off before operation n was not seen within its poll limit -- the step still ends)
 * point into the plan.  Steps on one plan must be ordered on one stream.
 */
typedef struct w4a16_decode_layer {
    const void* norm1;            /* input_layernorm weight, FP16 [hidden]                         */
    const void* qkv_packed;       /* [(q_heads + 2 kv_heads) * head_dim, hidden / 2]                */
    const void* qkv_scales;
    const void* o_packed;         /* [hidden, q_heads * head_dim / 2]                              */
    const void* o_scales;
    const void* norm2;            /* post_attention_layernorm weight                               */
    const void* gate_up_packed;   /* [2 * intermediate, hidden / 2]                                */
    const void* gate_up_scales;
    const void* down_packed;      /* [hidden, intermediate / 2]                                    */
    const void* down_scales;
    void* k_cache;
    void* v_cache;
} w4a16_decode_layer;

typedef struct w4a16_decode_model {
    int32_t layers, hidden, q_heads, kv_heads, head_dim, intermediate, vocab, max_len;
    float eps, rope_scale, softmax_scale;
    const void* embed;            /* FP16 [vocab, hidden]                                          */
    const void* final_norm;
    const void* lm_head_packed;   /* [vocab, hidden / 2]                                           */
    const void* lm_head_scales;
    const float* inv_freq;        /* [head_dim / 2]                                                */
    const w4a16_decode_layer* layer;   /* HOST array of `layers` entries                           */
} w4a16_decode_model;

typedef struct w4a16_decode_plan_info {
    const void* logits;
    const void* status;
    int32_t operations;
    int32_t grid;
    int32_t head_dim;
    uint32_t smem_bytes;
} w4a16_decode_plan_info;

size_t w4a16_decode_plan_bytes(const w4a16_decode_model* model);   /* 0 when the model does not fit the kernel */
int w4a16_decode_plan_build(const w4a16_decode_model* model, void* plan, size_t plan_bytes,
                            int64_t* token, int64_t* position, w4a16_decode_plan_info* info,
                            w4a16_stream_t stream);
int w4a16_decode_step_f16(void* plan, const w4a16_decode_plan_info* info, w4a16_stream_t stream);

/*
 * w4a16_linear_f16 for callers that cannot allocate device memory (no cudaMalloc after start-up,
 * no workspace handed to a plugin, an open stream capture): the split-K scratch is a fixed array
 * inside the library's device image, w4a16_static_scratch_bytes() bytes per GPU, instead of a
 * caller workspace.  This entry point has no counterpart in the reference project, which never
 * splits K and so never needs scratch.
 *
 * Same arguments and results as w4a16_linear_f16 without the workspace pair.  It allocates and frees
 * nothing.  Calls that need no scratch (other group sizes, misaligned pointers, batches that go to the
 * tcgen05 GEMM) are simply forwarded.  Problems whose split-K scratch, as
 * w4a16_linear_workspace_bytes_flags reports it, exceeds the array return W4A16_ERR_TOO_LARGE and launch
 * nothing.  All calls on a device share the one array: calls that may overlap on the GPU (several
 * streams, parallel graph branches) race; calls ordered on one stream do not.  The first call on
 * each device resolves the array's address and should be made outside stream capture.
 */
int w4a16_linear_f16_static_scratch(const void* x, const void* packed, const void* scales, void* y,
                                    int64_t M, int64_t N, int64_t K, int64_t group_size,
                                    uint32_t flags, w4a16_stream_t stream);

/* Size in bytes of the built-in scratch array used by w4a16_linear_f16_static_scratch. */
size_t w4a16_static_scratch_bytes(void);

/* Device-side health word of the tcgen05 kernel: 0 while healthy; non-zero identifies a barrier wait
 * that gave up after its spin limit (the kernel then still ran to completion of its clean-up, with an
 * unfinished result).  Reading synchronises the device and clears the word.  No reference counterpart. */
int w4a16_device_status(uint32_t* value);

/* Checked build only (the library compiled with -DW4A16_BOUNDS_CHECK, `python nibble_b200/_build.py --bounds-check`):
 * the streaming kernel compares every shared- and global-memory index it computes with the extent it must stay
 * inside, skips an access that would leave it and counts it.  *count = violations since the last call, *site = the
 * highest site code among them (1 activation staging, 2 output, 3 split-K partial, 4 weight copy, 5 scale copy);
 * reading synchronises and clears.  The ordinary build returns W4A16_ERR_BAD_CONFIG.  No reference counterpart
 * (the reference relies on compute-sanitizer, README.md:199-210). */
int w4a16_bounds_check_status(uint32_t* site, uint32_t* count);

/* Number of kernels this library has launched in this process (all entry points, all devices). */
uint64_t w4a16_launch_count(void);

/* Static description of an error code. */
const char* w4a16_status_string(int status);

/* ABI version: bumped when a signature above changes. */
int w4a16_abi_version(void);   /* currently 2 */

#ifdef __cplusplus
}
#endif
#endif /* W4A16_B200_H_ */
