// Generic W4A16 linear: any even group size, any pointer alignment, any batch size.
// Correctness path for the cases the tensor-core kernel declines (group_size != 128 or x / packed
// not 16-byte aligned), like the reference's one-thread-per-output kernel
// (csrc/int4_linear_kernel.cu:20-69) -- but a warp walks one output row with byte-wide coalesced
// loads and keeps up to eight batch rows in registers, so the packed row is read once per eight.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "kernels.h"
#include "unpack.cuh"

namespace w4a16 {
namespace {

constexpr int kGenericBatch = 8;
constexpr int kGenericWarps = 4;

__global__ void __launch_bounds__(kGenericWarps * 32)
linear_generic_kernel(const __half* __restrict__ x, const uint8_t* __restrict__ packed,
                      const __half* __restrict__ scales, void* __restrict__ y, int64_t M, int64_t N,
                      int64_t K, int64_t group, int out_f32) {
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kGenericWarps + (threadIdx.x >> 5);
    if (row >= N) return;
    const int64_t m0 = static_cast<int64_t>(blockIdx.y) * kGenericBatch;
    const int64_t bytes_per_row = K >> 1;
    const int64_t groups = K / group;
    const uint8_t* wrow = packed + row * bytes_per_row;
    const __half* srow = scales + row * groups;

    float total[kGenericBatch];
#pragma unroll
    for (int m = 0; m < kGenericBatch; ++m) total[m] = 0.f;

    // group is even, so the two codes of a byte always share a scale.
    for (int64_t b = lane; b < bytes_per_row; b += 32) {
        const uint32_t byte = wrow[b];
        const float c_even = static_cast<float>(static_cast<int>((byte & 0xFu) ^ 8u) - 8);
        const float c_odd = static_cast<float>(static_cast<int>((byte >> 4) ^ 8u) - 8);
        const float s = __half2float(srow[(2 * b) / group]);
#pragma unroll
        for (int m = 0; m < kGenericBatch; ++m) {
            if (m0 + m < M) {
                const __half* xr = x + (m0 + m) * K + 2 * b;
                const float dot = fmaf(c_odd, __half2float(xr[1]), c_even * __half2float(xr[0]));
                total[m] = fmaf(dot, s, total[m]);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < kGenericBatch; ++m) {
        float v = total[m];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (lane == 0 && m0 + m < M) {
            if (out_f32) {
                static_cast<float*>(y)[(m0 + m) * N + row] = v;
            } else {
                static_cast<__half*>(y)[(m0 + m) * N + row] = __float2half_rn(v);
            }
        }
    }
}

}  // namespace

int launch_linear_generic(const LinearProblem& p, bool out_f32, cudaStream_t stream) {
    const int64_t row_blocks = (p.N + kGenericWarps - 1) / kGenericWarps;
    const int64_t batch_blocks = (p.M + kGenericBatch - 1) / kGenericBatch;
    if (row_blocks > INT32_MAX || batch_blocks > 65535) return W4A16_ERR_TOO_LARGE;
    const dim3 grid(static_cast<unsigned>(row_blocks), static_cast<unsigned>(batch_blocks), 1);
    linear_generic_kernel<<<grid, kGenericWarps * 32, 0, stream>>>(p.x, p.packed, p.scales, p.y, p.M, p.N,
                                                                   p.K, p.group, out_f32 ? 1 : 0);
    if (cudaGetLastError() != cudaSuccess) return W4A16_ERR_LAUNCH;
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    return W4A16_OK;
}

}  // namespace w4a16
