// extern "C" boundary of libw4a16_b200: argument validation and kernel routing only.
// The declarations, their contracts and the reference functions they replace are in
// include/w4a16_b200.h.
#include <cuda_runtime.h>

#include "kernels.h"

namespace w4a16 {
std::atomic<uint64_t> g_launch_count{0};
}

namespace {

bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

int validate_linear(const void* x, const void* packed, const void* scales, const void* y, int64_t M,
                    int64_t N, int64_t K, int64_t group) {
    if (M < 0 || N < 0 || K < 0 || (K & 1)) return W4A16_ERR_BAD_SHAPE;
    if (group <= 0 || (group & 1)) return W4A16_ERR_BAD_GROUP;
    if (K % group != 0) return W4A16_ERR_BAD_SHAPE;
    if (M == 0 || N == 0) return W4A16_OK;
    if (y == nullptr) return W4A16_ERR_NULL_POINTER;
    if (K > 0 && (x == nullptr || packed == nullptr || scales == nullptr)) return W4A16_ERR_NULL_POINTER;
    return W4A16_OK;
}

bool fast_path_applies(const void* x, const void* packed, int64_t K, int64_t group) {
    return group == w4a16::kGroupFast && K > 0 && aligned16(x) && aligned16(packed);
}

}  // namespace

namespace {

// Whether a fast-path call with FP16 output goes to the tcgen05 GEMM rather than the streaming kernel.
// From 65 rows on always, up to 8 rows never.  Between 9 and 64 rows the streaming kernel still wins on small layers, but its cost
// grows with the batch and with K (every CTA stages batch x K activations, K is split ever further and the partial
// sums travel through memory) while the GEMM's does not.  Both sides of the comparison are fits to measurements
// on B200: the GEMM takes about 0.6 us per 128-wide K step of a round of 148 weight tiles whatever the batch; the
// streaming kernel about 5 us plus (8 + 1.5 * K/1024) us per 1e9 multiply-adds of the batch padded to 32 or 64
// rows.  Layers of fewer than 32 weight tiles leave most SMs of the GEMM idle and stay on the streaming kernel.
bool routes_to_tcgen05(int64_t M, int64_t N, int64_t K, uint32_t flags) {
    if (flags & (W4A16_FLAG_OUTPUT_F32 | W4A16_FLAG_NO_TCGEN05 | W4A16_FLAG_FORCE_GENERIC)) return false;
    if ((flags & W4A16_FLAG_FORCE_TCGEN05) || M >= w4a16::kTcgen05MinRows) return true;
    if (M <= 8) return false;
    if (N < 4096) {
        // Narrow layers: the fits below do not hold (few row tiles, so the streaming kernel leans on K splits whose
        // partial sums and repeated activation staging grow with the batch).  Measured: with K = 5632, N = 2048 the
        // GEMM, sharing K between CTAs, takes 14-15 us at 24..64 rows where the streaming kernel takes 22-42 us;
        // with K = 2048 the streaming kernel wins throughout.  So: from 17 rows on, when the streaming kernel
        // would split K four ways or more and the layer has at least eight weight tiles.
        // (with N = 1024 and K = 8192 the streaming kernel is still ahead at 17..32 rows, 14-15 us against 18 us,
        // and behind from 33 on, 24 us against 19 us)
        if (M <= 16 || N < 1024 || K < 4096 || (N < 2048 && M <= 32)) return false;
        return w4a16::choose_linear_config(M, N, K, w4a16::kMaxKSplits).k_splits >= 4;
    }
    const double padded = M <= 16 ? 16.0 : M <= 32 ? 32.0 : 64.0;
    const double giga_macs = padded * static_cast<double>(K) * static_cast<double>(N) * 1e-9;
    const double streaming_us = 5.0 + giga_macs * (8.0 + 1.5 * static_cast<double>(K) / 1024.0);
    const int64_t rounds = ((N + 127) / 128 + 147) / 148;
    // (a layer of few tiles shares the K of a tile between CTAs and pays a second small launch for the sum)
    const int splits = w4a16::tcgen05_k_splits(M, N, K, nullptr);
    const double gemm_us = 3.5 + 0.6 * static_cast<double>(rounds) * static_cast<double>(K) / (128.0 * splits) +
                           (splits > 1 ? 3.0 : 0.0);
    // 9..16 rows are close to the streaming kernel's best case: only a clear win moves them (K = 28672: 94 -> 71 us)
    return gemm_us < (M <= 16 ? 0.85 : 1.0) * streaming_us;
}

}  // namespace

bool w4a16::linear_routes_to_tcgen05(int64_t M, int64_t N, int64_t K, uint32_t flags) {
    return routes_to_tcgen05(M, N, K, flags);
}

extern "C" {

int w4a16_abi_version(void) { return 2; }

uint64_t w4a16_launch_count(void) { return w4a16::g_launch_count.load(std::memory_order_relaxed); }

const char* w4a16_status_string(int status) {
    switch (status) {
        case W4A16_OK: return "ok";
        case W4A16_ERR_NULL_POINTER: return "a required pointer is NULL";
        case W4A16_ERR_BAD_SHAPE: return "invalid shape: sizes must be non-negative, K even and divisible by group_size";
        case W4A16_ERR_BAD_GROUP: return "invalid group_size for this entry point";
        case W4A16_ERR_MISALIGNED: return "a pointer misses the required 16-byte alignment";
        case W4A16_ERR_WORKSPACE: return "workspace missing or too small";
        case W4A16_ERR_BAD_CONFIG: return "launch configuration not available";
        case W4A16_ERR_LAUNCH: return "CUDA kernel launch failed";
        case W4A16_ERR_TOO_LARGE: return "problem size exceeds what this entry point supports";
        default: return "unknown status";
    }
}

size_t w4a16_linear_workspace_bytes_flags(int64_t M, int64_t N, int64_t K, uint32_t flags) {
    if (M <= 0 || N <= 0 || K <= 0 || K % w4a16::kGroupFast != 0) return 0;
    // The generic kernel uses no scratch; the tcgen05 GEMM wants some only for layers with few tiles.
    if (flags & W4A16_FLAG_FORCE_GENERIC) return 0;
    if (routes_to_tcgen05(M, N, K, flags)) return w4a16::tcgen05_workspace_bytes(M, N, K);
    const w4a16_linear_config c = w4a16::choose_linear_config(M, N, K, w4a16::kMaxKSplits);
    return w4a16::linear_workspace_bytes_for(M, N, c.k_splits);
}

size_t w4a16_linear_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    return w4a16_linear_workspace_bytes_flags(M, N, K, 0);
}

int w4a16_linear_f16(const void* x, const void* packed, const void* scales, void* y, int64_t M, int64_t N,
                     int64_t K, int64_t group_size, void* workspace, size_t workspace_bytes, uint32_t flags,
                     w4a16_stream_t stream) {
    const int status = validate_linear(x, packed, scales, y, M, N, K, group_size);
    if (status != W4A16_OK || M == 0 || N == 0) return status;
    w4a16::LinearProblem p{static_cast<const __half*>(x), static_cast<const uint8_t*>(packed),
                           static_cast<const __half*>(scales), y, M, N, K, group_size,
                           workspace, workspace_bytes};
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const bool out_f32 = (flags & W4A16_FLAG_OUTPUT_F32) != 0;
    if (K == 0) {
        const size_t element = out_f32 ? sizeof(float) : sizeof(__half);
        return cudaMemsetAsync(y, 0, static_cast<size_t>(M) * N * element, s) == cudaSuccess
                   ? W4A16_OK
                   : W4A16_ERR_LAUNCH;
    }
    if ((flags & W4A16_FLAG_FORCE_GENERIC) || !fast_path_applies(x, packed, K, group_size)) {
        return w4a16::launch_linear_generic(p, out_f32, s);
    }
    // Prefill-sized batches, and medium ones on large layers: dense enough for the tcgen05 tensor cores.
    if (routes_to_tcgen05(M, N, K, flags)) return w4a16::launch_linear_tcgen05(p, s);
    // Split K across CTAs only as far as the caller's workspace allows.
    int max_splits = 1;
    if (workspace != nullptr && aligned16(workspace)) {
        for (int splits = w4a16::kMaxKSplits; splits > 1; splits >>= 1) {
            if (workspace_bytes >= w4a16::linear_workspace_bytes_for(M, N, splits)) {
                max_splits = splits;
                break;
            }
        }
    }
    w4a16_linear_config cfg = w4a16::choose_linear_config(M, N, K, max_splits);
    if (reinterpret_cast<uintptr_t>(scales) % 4 != 0) cfg.unroll = 1;
    const int launched =
        w4a16::launch_linear_mma(p, cfg, (flags & W4A16_FLAG_PROGRAMMATIC_LAUNCH) != 0, out_f32, s);
    // Too much activation data for one CTA's shared memory and no workspace to split K further: the tcgen05 GEMM
    // has no such limit (nor has the generic kernel, for FP32 output or when the GEMM is switched off).
    if (launched == W4A16_ERR_WORKSPACE) {
        if (!out_f32 && !(flags & W4A16_FLAG_NO_TCGEN05)) return w4a16::launch_linear_tcgen05(p, s);
        return w4a16::launch_linear_generic(p, out_f32, s);
    }
    return launched;
}

int w4a16_linear_f16_input(const void* x, const void* packed, const void* scales, void* y, int64_t M, int64_t N,
                           int64_t K, int64_t group_size, void* workspace, size_t workspace_bytes, uint32_t flags,
                           const w4a16_input_transform* transform, w4a16_stream_t stream) {
    if (transform == nullptr || transform->kind == W4A16_INPUT_PLAIN) {
        return w4a16_linear_f16(x, packed, scales, y, M, N, K, group_size, workspace, workspace_bytes, flags, stream);
    }
    const int status = validate_linear(x, packed, scales, y, M, N, K, group_size);
    if (status != W4A16_OK || M == 0 || N == 0) return status;
    if (K == 0 || M > 64 || !fast_path_applies(x, packed, K, group_size)) return W4A16_ERR_BAD_CONFIG;
    w4a16::LinearProblem p{static_cast<const __half*>(x), static_cast<const uint8_t*>(packed),
                           static_cast<const __half*>(scales), y, M, N, K, group_size,
                           workspace, workspace_bytes, nullptr, transform};
    int max_splits = 1;
    if (workspace != nullptr && aligned16(workspace)) {
        for (int splits = w4a16::kMaxKSplits; splits > 1; splits >>= 1) {
            if (workspace_bytes >= w4a16::linear_workspace_bytes_for(M, N, splits)) {
                max_splits = splits;
                break;
            }
        }
    }
    w4a16_linear_config cfg = w4a16::choose_linear_config(M, N, K, max_splits);
    if (reinterpret_cast<uintptr_t>(scales) % 4 != 0) cfg.unroll = 1;
    return w4a16::launch_linear_mma(p, cfg, (flags & W4A16_FLAG_PROGRAMMATIC_LAUNCH) != 0,
                                    (flags & W4A16_FLAG_OUTPUT_F32) != 0, reinterpret_cast<cudaStream_t>(stream));
}

int w4a16_linear_f16_config(const void* x, const void* packed, const void* scales, void* y, int64_t M,
                            int64_t N, int64_t K, int64_t group_size, void* workspace,
                            size_t workspace_bytes, uint32_t flags, const w4a16_linear_config* config,
                            w4a16_stream_t stream) {
    const int status = validate_linear(x, packed, scales, y, M, N, K, group_size);
    if (status != W4A16_OK || M == 0 || N == 0) return status;
    if (config == nullptr) return W4A16_ERR_NULL_POINTER;
    if (!fast_path_applies(x, packed, K, group_size)) return W4A16_ERR_BAD_CONFIG;
    w4a16_linear_config cfg = w4a16::choose_linear_config(M, N, K, 1);
    if (config->row_tiles) cfg.row_tiles = config->row_tiles;
    if (config->k_warps) cfg.k_warps = config->k_warps;
    if (config->k_splits) cfg.k_splits = config->k_splits;
    if (config->unroll) cfg.unroll = config->unroll;
    if (config->stages) cfg.stages = config->stages;
    w4a16::LinearProblem p{static_cast<const __half*>(x), static_cast<const uint8_t*>(packed),
                           static_cast<const __half*>(scales), y, M, N, K, group_size,
                           workspace, workspace_bytes};
    return w4a16::launch_linear_mma(p, cfg, (flags & W4A16_FLAG_PROGRAMMATIC_LAUNCH) != 0,
                                    (flags & W4A16_FLAG_OUTPUT_F32) != 0, reinterpret_cast<cudaStream_t>(stream));
}

int w4a16_linear_f16_peers(const void* x, int64_t x_ld, const void* packed, const void* scales, void* y, int64_t M,
                           int64_t N, int64_t K, int64_t group_size, void* workspace, size_t workspace_bytes,
                           uint32_t flags, const w4a16_peer_target* target, const w4a16_peer_source* source,
                           w4a16_stream_t stream) {
    // with a target the results go to the ranks' buffers and y is not used
    const int status = validate_linear(x, packed, scales, target != nullptr ? static_cast<const void*>(target) : y, M, N,
                                       K, group_size);
    if (status != W4A16_OK) return status;
    if (M == 0 || N == 0 || K == 0) return W4A16_ERR_BAD_SHAPE;
    if (M > 64 || !fast_path_applies(x, packed, K, group_size)) return W4A16_ERR_BAD_CONFIG;
    w4a16::LinearProblem p{static_cast<const __half*>(x), static_cast<const uint8_t*>(packed),
                           static_cast<const __half*>(scales), target != nullptr ? nullptr : y, M, N, K, group_size,
                           workspace, workspace_bytes, target, nullptr, source, x_ld};
    int max_splits = 1;
    if (workspace != nullptr && aligned16(workspace)) {
        for (int splits = w4a16::kMaxKSplits; splits > 1; splits >>= 1) {
            if (workspace_bytes >= w4a16::linear_workspace_bytes_for(M, N, splits)) {
                max_splits = splits;
                break;
            }
        }
    }
    w4a16_linear_config cfg = w4a16::choose_linear_config(M, N, K, max_splits);
    if (reinterpret_cast<uintptr_t>(scales) % 4 != 0) cfg.unroll = 1;
    return w4a16::launch_linear_mma(p, cfg, (flags & W4A16_FLAG_PROGRAMMATIC_LAUNCH) != 0,
                                    (flags & W4A16_FLAG_OUTPUT_F32) != 0, reinterpret_cast<cudaStream_t>(stream));
}

int w4a16_wait_peers(const w4a16_peer_source* source, const void* buffer0, void* out, int64_t count, uint32_t flags,
                     w4a16_stream_t stream) {
    const int64_t ld = source != nullptr && source->columns_per_rank > 0
                           ? source->columns_per_rank * static_cast<int64_t>(source->world)
                           : 0;
    return w4a16::launch_wait_peers(source, buffer0, out, count, ld, (flags & W4A16_FLAG_PROGRAMMATIC_LAUNCH) != 0,
                                    reinterpret_cast<cudaStream_t>(stream));
}

int w4a16_sum_partials_f16(const void* partials, void* y, int64_t count, int32_t world, const w4a16_peer_source* source,
                           uint32_t flags, w4a16_stream_t stream) {
    if (count < 0 || world < 1 || world > 32) return W4A16_ERR_BAD_SHAPE;
    if (count == 0) return W4A16_OK;
    if (partials == nullptr || y == nullptr) return W4A16_ERR_NULL_POINTER;
    if (source != nullptr && source->world != world) return W4A16_ERR_BAD_SHAPE;
    return w4a16::launch_sum_partials(partials, static_cast<__half*>(y), count, world, source,
                                      (flags & W4A16_FLAG_PROGRAMMATIC_LAUNCH) != 0, reinterpret_cast<cudaStream_t>(stream));
}

int w4a16_bounds_check_status(uint32_t* site, uint32_t* count) {
    if (site == nullptr || count == nullptr) return W4A16_ERR_NULL_POINTER;
    unsigned s = 0, c = 0;
    const int status = w4a16::read_bounds_check(&s, &c);
    *site = s;
    *count = c;
    return status;
}

int w4a16_device_status(uint32_t* value) {
    if (value == nullptr) return W4A16_ERR_NULL_POINTER;
    unsigned v = 0;
    const int status = w4a16::read_tcgen05_status(&v);
    *value = v;
    return status;
}

int w4a16_dequantize_f16(const void* packed, const void* scales, void* weights, int64_t N, int64_t K,
                         int64_t group_size, w4a16_stream_t stream) {
    if (N < 0 || K < 0 || (K & 1)) return W4A16_ERR_BAD_SHAPE;
    if (group_size <= 0 || group_size % 32 != 0) return W4A16_ERR_BAD_GROUP;
    if (K % group_size != 0) return W4A16_ERR_BAD_SHAPE;
    if (N == 0 || K == 0) return W4A16_OK;
    if (packed == nullptr || scales == nullptr || weights == nullptr) return W4A16_ERR_NULL_POINTER;
    if (!aligned16(packed) || !aligned16(weights)) return W4A16_ERR_MISALIGNED;
    return w4a16::launch_dequantize(static_cast<const uint8_t*>(packed), static_cast<const __half*>(scales),
                                    static_cast<__half*>(weights), N, K, group_size,
                                    reinterpret_cast<cudaStream_t>(stream));
}

static int quantize_pack(const void* weights, bool is_f32, void* packed, void* scales, int64_t N, int64_t K,
                         int64_t group_size, w4a16_stream_t stream) {
    if (N < 0 || K < 0 || (K & 1)) return W4A16_ERR_BAD_SHAPE;
    if (group_size <= 0 || (group_size & 1) || group_size > INT32_MAX) return W4A16_ERR_BAD_GROUP;
    if (K % group_size != 0) return W4A16_ERR_BAD_SHAPE;
    if (N == 0 || K == 0) return W4A16_OK;
    if (weights == nullptr || packed == nullptr || scales == nullptr) return W4A16_ERR_NULL_POINTER;
    if (reinterpret_cast<uintptr_t>(packed) % 2 != 0 || reinterpret_cast<uintptr_t>(scales) % 2 != 0 ||
        reinterpret_cast<uintptr_t>(weights) % (is_f32 ? 4 : 2) != 0) {
        return W4A16_ERR_MISALIGNED;
    }
    return w4a16::launch_quantize_pack(weights, is_f32, static_cast<uint8_t*>(packed), static_cast<__half*>(scales), N, K,
                                       group_size, reinterpret_cast<cudaStream_t>(stream));
}

int w4a16_quantize_pack_f16(const void* weights, void* packed, void* scales, int64_t N, int64_t K, int64_t group_size,
                            w4a16_stream_t stream) {
    return quantize_pack(weights, false, packed, scales, N, K, group_size, stream);
}

int w4a16_quantize_pack_f32(const void* weights, void* packed, void* scales, int64_t N, int64_t K, int64_t group_size,
                            w4a16_stream_t stream) {
    return quantize_pack(weights, true, packed, scales, N, K, group_size, stream);
}

int w4a16_add_rmsnorm_f16(const void* stream_in, const void* delta, const void* weight, void* stream_out, void* normed,
                          int64_t hidden, float eps, uint32_t flags, w4a16_stream_t stream) {
    if (hidden <= 0 || hidden > 24576) return W4A16_ERR_BAD_SHAPE;
    if (stream_in == nullptr || weight == nullptr || normed == nullptr) return W4A16_ERR_NULL_POINTER;
    return w4a16::launch_add_rmsnorm(static_cast<const __half*>(stream_in), static_cast<const __half*>(delta),
                                     static_cast<const __half*>(weight), static_cast<__half*>(stream_out),
                                     static_cast<__half*>(normed), static_cast<int>(hidden), eps,
                                     (flags & W4A16_FLAG_PROGRAMMATIC_LAUNCH) != 0, reinterpret_cast<cudaStream_t>(stream));
}

int w4a16_silu_mul_f16(const void* gate_up, void* out, int64_t intermediate, uint32_t flags, w4a16_stream_t stream) {
    if (intermediate <= 0 || intermediate > (1 << 30)) return W4A16_ERR_BAD_SHAPE;
    if (gate_up == nullptr || out == nullptr) return W4A16_ERR_NULL_POINTER;
    return w4a16::launch_silu_mul(static_cast<const __half*>(gate_up), static_cast<__half*>(out),
                                  static_cast<int>(intermediate), (flags & W4A16_FLAG_PROGRAMMATIC_LAUNCH) != 0,
                                  reinterpret_cast<cudaStream_t>(stream));
}

int w4a16_argmax_advance_f16(const void* logits, int64_t count, int64_t* token, int64_t* position, uint32_t flags,
                             w4a16_stream_t stream) {
    if (count <= 0 || count > INT32_MAX - 8192) return W4A16_ERR_BAD_SHAPE;
    if (logits == nullptr || token == nullptr) return W4A16_ERR_NULL_POINTER;
    return w4a16::launch_argmax_advance(static_cast<const __half*>(logits), static_cast<int>(count),
                                        reinterpret_cast<long long*>(token), reinterpret_cast<long long*>(position),
                                        (flags & W4A16_FLAG_PROGRAMMATIC_LAUNCH) != 0, reinterpret_cast<cudaStream_t>(stream));
}

size_t w4a16_decode_plan_bytes(const w4a16_decode_model* model) { return w4a16::decode_plan_bytes(model); }

int w4a16_decode_plan_build(const w4a16_decode_model* model, void* plan, size_t plan_bytes, int64_t* token,
                            int64_t* position, w4a16_decode_plan_info* info, w4a16_stream_t stream) {
    return w4a16::decode_plan_build(model, plan, plan_bytes, token, position, info, reinterpret_cast<cudaStream_t>(stream));
}

int w4a16_decode_step_f16(void* plan, const w4a16_decode_plan_info* info, w4a16_stream_t stream) {
    if (plan == nullptr || info == nullptr) return W4A16_ERR_NULL_POINTER;
    return w4a16::launch_decode_step(plan, info->operations, info->grid, info->head_dim, info->smem_bytes,
                                     reinterpret_cast<cudaStream_t>(stream));
}

int w4a16_attention_decode_f16(const void* qkv, void* k_cache, void* v_cache, void* out, const int64_t* position,
                               const float* inv_freq, int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t max_len,
                               float rope_scale, float softmax_scale, uint32_t* status, uint32_t flags,
                               w4a16_stream_t stream) {
    if (q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0 || (head_dim != 64 && head_dim != 128) || max_len <= 0) {
        return W4A16_ERR_BAD_SHAPE;
    }
    if (qkv == nullptr || k_cache == nullptr || v_cache == nullptr || out == nullptr || position == nullptr ||
        inv_freq == nullptr || status == nullptr) {
        return W4A16_ERR_NULL_POINTER;
    }
    if (reinterpret_cast<uintptr_t>(k_cache) % 4 != 0 || reinterpret_cast<uintptr_t>(v_cache) % 4 != 0) return W4A16_ERR_MISALIGNED;
    return w4a16::launch_attention_decode(static_cast<const __half*>(qkv), static_cast<__half*>(k_cache),
                                          static_cast<__half*>(v_cache), static_cast<__half*>(out),
                                          reinterpret_cast<const long long*>(position), inv_freq, q_heads, kv_heads, head_dim,
                                          max_len, rope_scale, softmax_scale, status,
                                          (flags & W4A16_FLAG_PROGRAMMATIC_LAUNCH) != 0, reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
