// Group-wise symmetric INT4 quantisation and packing on the device: FP16 or FP32 weights [N, K] ->
// packed codes [N, K/2] + FP16 scales [N, K/group], bit-identical to the reference's host routine
// (w4a16/quantization.py:65-113):
//   step  = amax(|w| over the group) / 7 in FP32, 1 for an all-zero group
//   code  = clamp(round_half_even(w / step), -7, 7)        (FP32 IEEE division, rint)
//   scale = half(step)                                     (rounded after the codes are made)
// byte j of a row holds code 2j in its low nibble and code 2j+1 in its high nibble.
//
// 128-wide groups (the format's default): half a warp per group, a lane keeps its eight consecutive
// weights in registers (one 16-byte load for FP16, two for FP32), the group maximum is a four-step
// shuffle reduction inside the half warp, and the eight codes leave as one 4-byte store.  Bound: HBM,
// 2.5 (FP16 input) or 4.5 (FP32) bytes per weight; the IEEE divisions keep it near the issue limit.
// Other group sizes: one warp per group, weights read twice (maximum, then codes).
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "kernels.h"

namespace w4a16 {
namespace {

template <typename T>
__device__ __forceinline__ float load_weight(const T* p);
template <>
__device__ __forceinline__ float load_weight<__half>(const __half* p) { return __half2float(*p); }
template <>
__device__ __forceinline__ float load_weight<float>(const float* p) { return *p; }

__device__ __forceinline__ unsigned code_of(float w, float step) {
    float q = rintf(__fdiv_rn(w, step));
    q = fminf(fmaxf(q, -7.0f), 7.0f);
    return static_cast<unsigned>(static_cast<int>(q)) & 0xFu;
}

template <typename T>
__global__ void __launch_bounds__(256)
quantize_pack_kernel(const T* __restrict__ weights, uint8_t* __restrict__ packed, __half* __restrict__ scales,
                     int64_t total_groups, int group) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
    for (int64_t g = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); g < total_groups; g += warps) {
        const T* src = weights + g * group;              // groups of a row-major matrix are consecutive in memory
        float amax = 0.0f;
        for (int i = lane; i < group; i += 32) amax = fmaxf(amax, fabsf(load_weight(src + i)));
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
        const float step = amax == 0.0f ? 1.0f : __fdiv_rn(amax, 7.0f);
        uint8_t* dst = packed + g * (group >> 1);
        if ((group & 3) == 0) {
            for (int q = lane; q < (group >> 2); q += 32) {
                const unsigned c0 = code_of(load_weight(src + 4 * q), step);
                const unsigned c1 = code_of(load_weight(src + 4 * q + 1), step);
                const unsigned c2 = code_of(load_weight(src + 4 * q + 2), step);
                const unsigned c3 = code_of(load_weight(src + 4 * q + 3), step);
                // (g * group / 2 + 2 q) is even: the two bytes are 2-byte aligned when `packed` is
                *reinterpret_cast<uint16_t*>(dst + 2 * q) = static_cast<uint16_t>(c0 | (c1 << 4) | (c2 << 8) | (c3 << 12));
            }
        } else {
            for (int q = lane; q < (group >> 1); q += 32) {
                const unsigned c0 = code_of(load_weight(src + 2 * q), step);
                const unsigned c1 = code_of(load_weight(src + 2 * q + 1), step);
                dst[q] = static_cast<uint8_t>(c0 | (c1 << 4));
            }
        }
        if (lane == 0) scales[g] = __float2half_rn(step);
    }
}

__device__ __forceinline__ void load8(const __half* p, float (&w)[8]) {
    const uint4 q = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        w[2 * i] = f.x;
        w[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void load8(const float* p, float (&w)[8]) {
    const float4 a = reinterpret_cast<const float4*>(p)[0];
    const float4 b = reinterpret_cast<const float4*>(p)[1];
    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
    w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
}

// group == 128 and 16-byte aligned weights: sixteen lanes per group, eight weights per lane
template <typename T>
__global__ void __launch_bounds__(256)
quantize_pack_128_kernel(const T* __restrict__ weights, uint8_t* __restrict__ packed, __half* __restrict__ scales,
                         int64_t total_groups) {
    const int lane16 = threadIdx.x & 15;
    const int64_t halves = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 4);
    // every lane of a warp runs the same number of rounds: the shuffles below name the whole warp
    const int64_t rounds = (total_groups + halves - 1) / halves;
    int64_t g = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 4) + (threadIdx.x >> 4);
    for (int64_t r = 0; r < rounds; ++r, g += halves) {
        const bool live = g < total_groups;
        float w[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
        if (live) load8(weights + g * 128 + lane16 * 8, w);
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(w[i]));
#pragma unroll
        for (int offset = 8; offset > 0; offset >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
        if (!live) continue;
        const float step = amax == 0.0f ? 1.0f : __fdiv_rn(amax, 7.0f);
        const float inv_step = __fdiv_rn(1.0f, step);
        // Fast route for all eight codes: t = w * (1/step) + 1.5 * 2^23 in one FMA leaves round-half-even of the
        // exact product in the low mantissa bits of t (|w / step| <= 7, so the low nibble of t's bit pattern IS the
        // two's-complement code).  The product and the reference's fl(w / step) differ by a few ulp at most, so
        // both round to the same integer unless the quotient sits within 1e-4 of a tie k + 0.5; a lane that sees
        // such a weight redoes its eight codes with the IEEE division (about one lane in 600).
        constexpr float kMagic = 12582912.0f;
        unsigned word = 0;
        bool near_tie = false;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float t = fmaf(w[i], inv_step, kMagic);
            const float q = w[i] * inv_step;
            near_tie |= fabsf(q - (t - kMagic)) > 0.4999f;
            word |= (__float_as_uint(t) & 0xFu) << (4 * i);
        }
        if (near_tie) {
            word = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) word |= code_of(w[i], step) << (4 * i);
        }
        reinterpret_cast<uint32_t*>(packed + g * 64)[lane16] = word;
        if (lane16 == 0) scales[g] = __float2half_rn(step);
    }
}

template <typename T>
int launch(const T* weights, uint8_t* packed, __half* scales, int64_t N, int64_t K, int64_t group, cudaStream_t stream) {
    const int64_t total_groups = N * (K / group);
    if (group == 128 && reinterpret_cast<uintptr_t>(weights) % 16 == 0 && reinterpret_cast<uintptr_t>(packed) % 4 == 0) {
        const int64_t fast_blocks = std::min<int64_t>((total_groups + 15) / 16, 148 * 32);
        quantize_pack_128_kernel<T><<<static_cast<unsigned>(fast_blocks), 256, 0, stream>>>(weights, packed, scales, total_groups);
        if (cudaGetLastError() != cudaSuccess) return W4A16_ERR_LAUNCH;
        g_launch_count.fetch_add(1, std::memory_order_relaxed);
        return W4A16_OK;
    }
    const int64_t blocks = std::min<int64_t>((total_groups + 7) / 8, 148 * 64);
    quantize_pack_kernel<T><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(weights, packed, scales, total_groups,
                                                                              static_cast<int>(group));
    if (cudaGetLastError() != cudaSuccess) return W4A16_ERR_LAUNCH;
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    return W4A16_OK;
}

}  // namespace

int launch_quantize_pack(const void* weights, bool is_f32, uint8_t* packed, __half* scales, int64_t N, int64_t K,
                         int64_t group, cudaStream_t stream) {
    if (is_f32) return launch(static_cast<const float*>(weights), packed, scales, N, K, group, stream);
    return launch(static_cast<const __half*>(weights), packed, scales, N, K, group, stream);
}

}  // namespace w4a16
