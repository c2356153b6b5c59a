// Internal interface between the C-ABI layer (capi.cu) and the kernel translation units.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/w4a16_b200.h"

namespace w4a16 {

// Kernels launched by this library since it was loaded.
extern std::atomic<uint64_t> g_launch_count;

constexpr int kGroupFast = 128;        // group size the tensor-core kernel is built for
constexpr int kMaxKSplits = 8;          // upper bound on CTAs splitting K of one row block
constexpr int kBatchPerTile = 8;        // batch rows covered by one n8 MMA tile
constexpr int kMaxBatchTiles = 4;       // n8 tiles per warp (so up to 32 batch rows per CTA pass)

struct LinearProblem {
    const __half* x;          // [M, K]
    const uint8_t* packed;    // [N, K/2]
    const __half* scales;     // [N, K/group]
    void* y;                  // [M, N], FP16 or FP32
    int64_t M, N, K, group;
    void* workspace;          // may be null
    size_t workspace_bytes;
    const w4a16_peer_target* peers = nullptr;   // fan the result out to a tensor-parallel group
    const w4a16_input_transform* input = nullptr;   // x is derived from other buffers while it is staged
    const w4a16_peer_source* source = nullptr;  // x is another sharded layer's published result
    int64_t x_ld = 0;                           // elements between batch rows of x (0: K)
};

// Workspace layout for split-K: arrival counters first, FP32 partials after them.
size_t linear_counter_bytes(int64_t M, int64_t N);
size_t linear_workspace_bytes_for(int64_t M, int64_t N, int splits);

// Picks a launch shape for the tensor-core kernel.  `max_splits` caps k_splits (1 = no workspace).
w4a16_linear_config choose_linear_config(int64_t M, int64_t N, int64_t K, int max_splits);

// Tensor-core path: requires group == 128 and 16-byte aligned x / packed.  Returns a W4A16_* code.
// `out_f32` makes y an FP32 [M, N] matrix (unrounded sums, for partial results that are added up).
int launch_linear_mma(const LinearProblem& p, const w4a16_linear_config& cfg, bool programmatic,
                      bool out_f32, cudaStream_t stream);

// Bounds-check word of the streaming kernel; W4A16_ERR_BAD_CONFIG in builds without -DW4A16_BOUNDS_CHECK.
int read_bounds_check(unsigned* site, unsigned* count);

// Prefill-sized batches: dequantisation fused into a tcgen05 GEMM (group == 128, aligned x / packed).
int launch_linear_tcgen05(const LinearProblem& p, cudaStream_t stream);
// Status word of that kernel (non-zero: a bounded barrier wait gave up); reading clears it and synchronises.
int read_tcgen05_status(unsigned* value);
constexpr int kTcgen05MinRows = 65;     // from here on every fast-path call with FP16 output takes the GEMM
// Scratch the GEMM wants (FP32 partial sums of K ranges, for layers with few tiles); it runs unsplit without.
size_t tcgen05_workspace_bytes(int64_t M, int64_t N, int64_t K);
// K ranges per output tile the GEMM uses when it has that scratch (1: none); *split_k receives the width of a range.
int tcgen05_k_splits(int64_t M, int64_t N, int64_t K, int64_t* split_k);
// Whether w4a16_linear_f16 sends a fast-path call with these sizes and flags to the GEMM (capi.cu).
bool linear_routes_to_tcgen05(int64_t M, int64_t N, int64_t K, uint32_t flags);

// Any even group size, any alignment, any M.
int launch_linear_generic(const LinearProblem& p, bool out_f32, cudaStream_t stream);

// Tensor-parallel helpers: a reader kernel (bounded wait for every rank's publication, optional copy, release)
// and the rank-ordered sum of FP32 partials into FP16.
int launch_wait_peers(const w4a16_peer_source* source, const void* buffer0, void* out, int64_t count, int64_t ld,
                      bool programmatic, cudaStream_t stream);
int launch_sum_partials(const void* partials, __half* y, int64_t count, int world, const w4a16_peer_source* source,
                        bool programmatic, cudaStream_t stream);

int launch_dequantize(const uint8_t* packed, const __half* scales, __half* weights, int64_t N,
                      int64_t K, int64_t group, cudaStream_t stream);

// Kernels either side of the linears in a LLaMA decode step (decode_ops.cu).
int launch_add_rmsnorm(const __half* stream_in, const __half* delta, const __half* weight, __half* stream_out,
                       __half* normed, int hidden, float eps, bool programmatic, cudaStream_t stream);
int launch_argmax_advance(const __half* logits, int count, long long* token, long long* position, bool programmatic,
                          cudaStream_t stream);
int launch_silu_mul(const __half* gate_up, __half* out, int inter, bool programmatic, cudaStream_t stream);
int launch_attention_decode(const __half* qkv, __half* k_cache, __half* v_cache, __half* out, const long long* position,
                            const float* inv_freq, int q_heads, int kv_heads, int head_dim, int max_len, float rope_scale,
                            float softmax_scale, unsigned* status, bool programmatic, cudaStream_t stream);

// One decode step as one cooperative launch over a prebuilt plan (decode_persistent.cu).
size_t decode_plan_bytes(const w4a16_decode_model* model);
int decode_plan_build(const w4a16_decode_model* model, void* plan, size_t plan_bytes, int64_t* token, int64_t* position,
                      w4a16_decode_plan_info* info, cudaStream_t stream);
int launch_decode_step(const void* plan, int32_t n_ops, int32_t grid, int32_t head_dim, uint32_t smem_bytes, cudaStream_t stream);

// Quantise + pack on the device (quantize.cu): FP16 or FP32 weights -> packed codes and FP16 scales.
int launch_quantize_pack(const void* weights, bool is_f32, uint8_t* packed, __half* scales, int64_t N, int64_t K,
                         int64_t group, cudaStream_t stream);

}  // namespace w4a16
