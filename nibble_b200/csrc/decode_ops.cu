// The small kernels either side of the linear layers in one LLaMA decode step (batch 1), so that a
// token is ~8 launches per decoder block instead of the several dozen elementwise kernels a
// framework issues:
//   add_rmsnorm   residual add (FP16) + RMSNorm with FP32 statistics          -> input of q/k/v or gate/up
//   attention     RoPE on q and k, append k/v to the cache, softmax(q k^T / sqrt(d)) v over the cache
//   silu_mul      silu(gate) * up on the fused gate/up output                   -> input of down_proj
// They restate what the reference's generation script gets from HuggingFace's LlamaDecoderLayer
// (scripts/generate.py:260-365 drives model.generate; the arithmetic is transformers' modeling_llama:
// LlamaRMSNorm, apply_rotary_pos_emb / rotate_half, scaled dot product attention with grouped KV heads,
// LlamaMLP).  Roundings follow that code: the residual sum, the normalised value, the rotary
// products and silu(gate) are each rounded to FP16 where the framework rounds them.
//
// The position is read from device memory, so one captured graph serves every step.
//
// Every kernel releases its successor at once (griddepcontrol.launch_dependents) and waits for its
// predecessor (griddepcontrol.wait) before it touches memory: when launched with the programmatic
// attribute, the next kernel's blocks are resident and -- for the linears -- already streaming weights
// while this one computes.  Both instructions do nothing under an ordinary launch.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "kernels.h"
#include "unpack.cuh"

namespace w4a16 {
namespace {

__device__ __forceinline__ float block_sum(float v, float* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    __syncthreads();                       // scratch may still be read from a previous call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.0f;
    for (int w = 0; w < warps; ++w) total += scratch[w];
    return total;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float best = scratch[0];
    for (int w = 1; w < warps; ++w) best = fmaxf(best, scratch[w]);
    return best;
}

// stream_out = half(stream_in + delta) (or stream_in when delta is null); normed = weight * half(s * rsqrt(mean(s^2) + eps))
__global__ void __launch_bounds__(256)
add_rmsnorm_kernel(const __half* __restrict__ stream_in, const __half* __restrict__ delta, const __half* __restrict__ weight,
                   __half* __restrict__ stream_out, __half* __restrict__ normed, int hidden, float eps) {
    __shared__ float scratch[8];
    extern __shared__ __half row[];        // the summed stream, kept for the second pass
    pdl_release_downstream();
    pdl_wait_for_upstream();
    float sq = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        __half s = stream_in[i];
        if (delta != nullptr) s = __hadd(s, delta[i]);
        row[i] = s;
        const float f = __half2float(s);
        sq += f * f;
    }
    const float inv = rsqrtf(block_sum(sq, scratch) / static_cast<float>(hidden) + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const __half s = row[i];
        if (stream_out != nullptr) stream_out[i] = s;
        normed[i] = __hmul(weight[i], __float2half_rn(__half2float(s) * inv));
    }
}

__global__ void __launch_bounds__(256)
silu_mul_kernel(const __half* __restrict__ gate_up, __half* __restrict__ out, int inter) {
    pdl_release_downstream();
    pdl_wait_for_upstream();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= inter) return;
    const __half2 act = silu_half2(__half2half2(gate_up[i]));
    out[i] = __hmul(__low2half(act), gate_up[inter + i]);
}

// token = index of the first largest logit (what argmax returns); the position moves on by one.
__global__ void __launch_bounds__(1024)
argmax_advance_kernel(const __half* __restrict__ logits, int count, long long* __restrict__ token,
                      long long* __restrict__ position) {
    __shared__ float best_value[32];
    __shared__ int best_index[32];
    pdl_release_downstream();
    pdl_wait_for_upstream();
    float value = -INFINITY;
    int index = 0x7fffffff;
    for (int i = threadIdx.x * 8; i < count; i += blockDim.x * 8) {
        if (i + 8 <= count && (reinterpret_cast<uintptr_t>(logits + i) & 15) == 0) {
            const uint4 q = *reinterpret_cast<const uint4*>(logits + i);
            const __half2* h = reinterpret_cast<const __half2*>(&q);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(h[j]);
                if (f.x > value) { value = f.x; index = i + 2 * j; }
                if (f.y > value) { value = f.y; index = i + 2 * j + 1; }
            }
        } else {
            for (int j = i; j < min(i + 8, count); ++j) {
                const float f = __half2float(logits[j]);
                if (f > value) { value = f; index = j; }
            }
        }
    }
    auto merge = [&](float other_value, int other_index) {
        if (other_value > value || (other_value == value && other_index < index)) { value = other_value; index = other_index; }
    };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) merge(__shfl_xor_sync(0xffffffffu, value, o), __shfl_xor_sync(0xffffffffu, index, o));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { best_value[warp] = value; best_index[warp] = index; }
    __syncthreads();
    if (warp == 0) {
        const int warps = blockDim.x >> 5;
        value = lane < warps ? best_value[lane] : -INFINITY;
        index = lane < warps ? best_index[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) merge(__shfl_xor_sync(0xffffffffu, value, o), __shfl_xor_sync(0xffffffffu, index, o));
        if (lane == 0) {
            *token = index == 0x7fffffff ? 0 : index;
            if (position != nullptr) *position += 1;
        }
    }
}

struct AttentionParams {
    const __half* qkv;        // [q heads * d | kv heads * d | kv heads * d] of this token
    __half* k_cache;          // [kv heads][max_len][d]
    __half* v_cache;
    __half* out;              // [q heads * d]
    const long long* position;  // device scalar: index of this token
    const float* inv_freq;    // [d / 2]
    int q_heads, kv_heads, head_dim, max_len;
    float rope_scale;         // multiplies cos and sin (1 for plain RoPE)
    float softmax_scale;
    unsigned* status;         // set to 1 when the position does not fit the cache
};

// One CTA per query head, 128 threads.  D/8 consecutive lanes share a cached position: each reads 16
// bytes of its K (then V) row, so a row is one coalesced 128- or 256-byte read, and the 128 threads
// cover 16 (D = 64) or 8 (D = 128) positions per pass with independent loads in flight.
template <int D>
__global__ void __launch_bounds__(128)
attention_decode_kernel(const AttentionParams p) {
    constexpr int kLanesPerPos = D / 8;
    constexpr int kPosPerPass = 128 / kLanesPerPos;
    extern __shared__ float scores[];                 // max_len floats
    __shared__ float scratch[4];
    __shared__ float q[D];
    __shared__ __align__(16) __half k_new[D];
    __shared__ __align__(16) __half v_new[D];
    __shared__ float partial[kPosPerPass][D];
    constexpr int kEarlyPasses = 2;                   // passes whose cache rows are requested before anything else
    const int head = blockIdx.x;
    constexpr int half_d = D / 2;
    const int kv_head = head / (p.q_heads / p.kv_heads);
    const int sub = threadIdx.x % kLanesPerPos;       // which 8 of the D dims
    const int slot = threadIdx.x / kLanesPerPos;      // which position of a pass
    const uint4* k_rows = reinterpret_cast<const uint4*>(p.k_cache + static_cast<size_t>(kv_head) * p.max_len * D) + sub;
    const uint4* v_rows = reinterpret_cast<const uint4*>(p.v_cache + static_cast<size_t>(kv_head) * p.max_len * D) + sub;
    pdl_release_downstream();
    // Nothing below depends on the kernel just before this one (it produces qkv): the position was set
    // and the older cache rows were written by earlier steps.  So the first rows of K and V, the position
    // and the rotary frequencies are requested before waiting for that kernel.  Rows at or past the
    // position hold stale data; they are fetched (inside the cache) and never used.
    uint4 k_early[kEarlyPasses], v_early[kEarlyPasses];
#pragma unroll
    for (int e = 0; e < kEarlyPasses; ++e) {
        const int t = min(e * kPosPerPass + slot, p.max_len - 1);
        k_early[e] = k_rows[static_cast<size_t>(t) * kLanesPerPos];
        v_early[e] = v_rows[static_cast<size_t>(t) * kLanesPerPos];
    }
    const long long pos = *p.position;
    const float freq = p.inv_freq[threadIdx.x % half_d];
    pdl_wait_for_upstream();
    if (pos < 0 || pos >= p.max_len) {
        if (threadIdx.x == 0) atomicMax(p.status, 1u);
        return;
    }
    const __half* q_in = p.qkv + head * D;
    const __half* k_in = p.qkv + p.q_heads * D + kv_head * D;
    const __half* v_in = p.qkv + (p.q_heads + p.kv_heads) * D + kv_head * D;
    // rotary embedding, rounded as the framework rounds it: cos/sin to FP16, two FP16 products, one FP16 sum
    if (threadIdx.x < D) {
        const int i = threadIdx.x;
        const float angle = static_cast<float>(pos) * freq;
        float sn, cs;
        sincosf(angle, &sn, &cs);
        const __half c = __float2half_rn(cs * p.rope_scale);
        const __half s = __float2half_rn(sn * p.rope_scale);
        const __half q_rot = i < half_d ? __hneg(q_in[i + half_d]) : q_in[i - half_d];
        const __half k_rot = i < half_d ? __hneg(k_in[i + half_d]) : k_in[i - half_d];
        // the _rn forms are never contracted into one fused multiply-add: two roundings, then a third
        q[i] = __half2float(__hadd_rn(__hmul_rn(q_in[i], c), __hmul_rn(q_rot, s)));
        const __half k_val = __hadd_rn(__hmul_rn(k_in[i], c), __hmul_rn(k_rot, s));
        k_new[i] = k_val;
        v_new[i] = v_in[i];
        if (head % (p.q_heads / p.kv_heads) == 0) {   // one CTA per KV head appends to the cache
            p.k_cache[(static_cast<size_t>(kv_head) * p.max_len + pos) * D + i] = k_val;
            p.v_cache[(static_cast<size_t>(kv_head) * p.max_len + pos) * D + i] = v_in[i];
        }
    }
    __syncthreads();

    const int length = static_cast<int>(pos) + 1;
    // The newest position comes from shared memory, not from the cache: another CTA writes it there.
    auto row_piece = [&](const uint4* rows, const __half* newest, const uint4 (&early)[kEarlyPasses], int base, int t) {
        if (t == length - 1) return reinterpret_cast<const uint4*>(newest)[sub];
        if (base == 0) return early[0];
        if (base == kPosPerPass) return early[1];
        return rows[static_cast<size_t>(t) * kLanesPerPos];
    };
    float qf[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) qf[i] = q[sub * 8 + i];

    float local_max = -INFINITY;
#pragma unroll 4
    for (int base = 0; base < length; base += kPosPerPass) {
        const int t = base + slot;
        float dot = 0.0f;
        if (t < length) {
            const uint4 piece = row_piece(k_rows, k_new, k_early, base, t);
            const __half2* h = reinterpret_cast<const __half2*>(&piece);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 kk = __half22float2(h[i]);
                dot += qf[2 * i] * kk.x + qf[2 * i + 1] * kk.y;
            }
        }
#pragma unroll
        for (int o = kLanesPerPos / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if (t < length) {
            dot *= p.softmax_scale;
            if (sub == 0) scores[t] = dot;
            local_max = fmaxf(local_max, dot);
        }
    }
    const float top = block_max(local_max, scratch);  // its barriers also publish the scores
    float local_sum = 0.0f;
    for (int t = threadIdx.x; t < length; t += blockDim.x) {
        const float e = expf(scores[t] - top);
        scores[t] = e;
        local_sum += e;
    }
    const float denom = block_sum(local_sum, scratch);

    float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 4
    for (int base = 0; base < length; base += kPosPerPass) {
        const int t = base + slot;
        if (t < length) {
            const float w = scores[t];
            const uint4 piece = row_piece(v_rows, v_new, v_early, base, t);
            const __half2* h = reinterpret_cast<const __half2*>(&piece);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 vv = __half22float2(h[i]);
                acc[2 * i] += w * vv.x;
                acc[2 * i + 1] += w * vv.y;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) partial[slot][sub * 8 + i] = acc[i];
    __syncthreads();
    if (threadIdx.x < D) {
        float total = 0.0f;
#pragma unroll
        for (int g = 0; g < kPosPerPass; ++g) total += partial[g][threadIdx.x];
        p.out[head * D + threadIdx.x] = __float2half_rn(total / denom);
    }
}

template <typename... Params, typename... Args>
int launch_kernel(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, bool programmatic, cudaStream_t stream,
                  Args... args) {
    cudaLaunchConfig_t launch = {};
    launch.gridDim = grid;
    launch.blockDim = block;
    launch.dynamicSmemBytes = smem;
    launch.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    launch.attrs = attr;
    launch.numAttrs = programmatic ? 1 : 0;
    if (cudaLaunchKernelEx(&launch, kernel, static_cast<Params>(args)...) != cudaSuccess) return W4A16_ERR_LAUNCH;
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    return W4A16_OK;
}

}  // namespace

int launch_add_rmsnorm(const __half* stream_in, const __half* delta, const __half* weight, __half* stream_out,
                       __half* normed, int hidden, float eps, bool programmatic, cudaStream_t stream) {
    return launch_kernel(add_rmsnorm_kernel, dim3(1), dim3(256), static_cast<size_t>(hidden) * sizeof(__half), programmatic,
                         stream, stream_in, delta, weight, stream_out, normed, hidden, eps);
}

int launch_silu_mul(const __half* gate_up, __half* out, int inter, bool programmatic, cudaStream_t stream) {
    return launch_kernel(silu_mul_kernel, dim3((inter + 255) / 256), dim3(256), 0, programmatic, stream, gate_up, out, inter);
}

int launch_argmax_advance(const __half* logits, int count, long long* token, long long* position, bool programmatic,
                          cudaStream_t stream) {
    return launch_kernel(argmax_advance_kernel, dim3(1), dim3(1024), 0, programmatic, stream, logits, count, token, position);
}

int launch_attention_decode(const __half* qkv, __half* k_cache, __half* v_cache, __half* out, const long long* position,
                            const float* inv_freq, int q_heads, int kv_heads, int head_dim, int max_len, float rope_scale,
                            float softmax_scale, unsigned* status, bool programmatic, cudaStream_t stream) {
    AttentionParams params{qkv, k_cache, v_cache, out, position, inv_freq, q_heads, kv_heads, head_dim, max_len,
                           rope_scale, softmax_scale, status};
    const size_t smem = static_cast<size_t>(max_len) * sizeof(float);      // the scores; the rest is static
    auto kernel = head_dim == 64 ? attention_decode_kernel<64> : attention_decode_kernel<128>;
    if (smem > 32 * 1024) {
        if (smem > 160 * 1024) return W4A16_ERR_TOO_LARGE;
        static bool raised[64][2] = {};
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return W4A16_ERR_LAUNCH;
        const int which = head_dim == 64 ? 0 : 1;
        if (!raised[device][which]) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess) {
                return W4A16_ERR_LAUNCH;
            }
            raised[device][which] = true;
        }
    }
    return launch_kernel(kernel, dim3(q_heads), dim3(128), smem, programmatic, stream, params);
}

}  // namespace w4a16
