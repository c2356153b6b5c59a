// packed INT4 + FP16 scales -> FP16 [N, K], bit-identical to half(float(code) * float(scale)).
// Replaces the reference's int4_dequantize_kernel (csrc/int4_linear_kernel.cu:419-451).
//
// Pure streaming: N*K/2 bytes in, 2*N*K bytes out.  A thread owns one 32-bit word (8 codes) at a time
// and writes one 16-byte vector, so a warp reads 128 contiguous bytes and writes 512 contiguous bytes;
// the grid is a multiple of the SM count and strides over the matrix.
// code * scale in a single FP16 multiply rounds once from the exact product, which is what
// rounding the FP32 product to FP16 does (|code| <= 8 needs 4 bits, an FP16 significand 11).
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "kernels.h"
#include "unpack.cuh"

namespace w4a16 {
namespace {

constexpr int kDequantThreads = 256;
constexpr int kWordsPerThread = 4;   // independent 4-byte loads in flight per thread

__global__ void __launch_bounds__(kDequantThreads)
dequantize_kernel(const uint32_t* __restrict__ packed_words, const __half* __restrict__ scales,
                  uint4* __restrict__ out, int64_t total_words, int words_per_row, int words_per_group,
                  int groups_per_row) {
    // A warp owns 128 consecutive words per round: lane l takes words l, l+32, l+64, l+96 of them, so
    // every load instruction reads 128 contiguous bytes and every store writes 512.  Row and column
    // are divided out once per round and walked forward for the other three words.
    const int lane = threadIdx.x & 31;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * (kDequantThreads / 32);
    const int64_t first_warp = static_cast<int64_t>(blockIdx.x) * (kDequantThreads / 32) + (threadIdx.x >> 5);
    for (int64_t chunk = first_warp * 128; chunk < total_words; chunk += warps * 128) {
        uint32_t word[kWordsPerThread];
        uint32_t scale2[kWordsPerThread];
        const int64_t w0 = chunk + lane;
        int64_t row = w0 / words_per_row;
        int col = static_cast<int>(w0 - row * words_per_row);
#pragma unroll
        for (int i = 0; i < kWordsPerThread; ++i) {
            const int64_t w = w0 + i * 32;
            if (w < total_words) {
                word[i] = ldg_stream4(packed_words + w);
                const uint32_t s = ldg_nc_u16(scales + row * groups_per_row + col / words_per_group);
                scale2[i] = s | (s << 16);
            }
            col += 32;
            while (col >= words_per_row) {
                col -= words_per_row;
                ++row;
            }
        }
#pragma unroll
        for (int i = 0; i < kWordsPerThread; ++i) {
            const int64_t w = w0 + i * 32;
            if (w < total_words) {
                uint32_t h[4];
                unpack8(word[i], h);   // (c0,c4) (c1,c5) (c2,c6) (c3,c7)
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] = hmul2_u32(h[j], scale2[i]);
                uint4 v;               // back to memory order (c0,c1) (c2,c3) (c4,c5) (c6,c7)
                v.x = prmt(h[0], h[1], 0x5410u);
                v.y = prmt(h[2], h[3], 0x5410u);
                v.z = prmt(h[0], h[1], 0x7632u);
                v.w = prmt(h[2], h[3], 0x7632u);
                out[w] = v;
            }
        }
    }
}

}  // namespace

int launch_dequantize(const uint8_t* packed, const __half* scales, __half* weights, int64_t N, int64_t K,
                      int64_t group, cudaStream_t stream) {
    const int64_t total_words = N * K / 8;
    if (total_words == 0) return W4A16_OK;
    if (K / 8 > INT32_MAX) return W4A16_ERR_TOO_LARGE;
    constexpr int kSms = 148;
    const int64_t per_block = static_cast<int64_t>(kDequantThreads) * kWordsPerThread;
    int64_t blocks = (total_words + per_block - 1) / per_block;
    const int64_t cap = static_cast<int64_t>(kSms) * 8 * 4;   // a few waves of 8 resident CTAs per SM
    if (blocks > cap) blocks = cap;
    dequantize_kernel<<<static_cast<unsigned>(blocks), kDequantThreads, 0, stream>>>(
        reinterpret_cast<const uint32_t*>(packed), scales, reinterpret_cast<uint4*>(weights), total_words,
        static_cast<int>(K / 8), static_cast<int>(group / 8), static_cast<int>(K / group));
    if (cudaGetLastError() != cudaSuccess) return W4A16_ERR_LAUNCH;
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    return W4A16_OK;
}

}  // namespace w4a16
