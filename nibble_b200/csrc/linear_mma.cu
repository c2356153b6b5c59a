// Fused W4A16 linear for sm_100a: packed INT4 weights are streamed from HBM straight into
// registers, unpacked to exact FP16 integers with two-instruction-per-pair bit tricks, and fed to
// the tensor cores as the 16-row operand of m16n8k16 MMAs whose 8-wide axis carries the batch.
// The group scale multiplies the FP32 accumulator once per 128 k, never the individual weights.
//
// Replaces the reference's M=1 decode kernel (csrc/int4_linear_kernel.cu:325-404), its M=2..8
// small-batch kernel (:542-617) and, for larger M, its dequantise-then-cuBLAS route
// (w4a16/linear.py:132-152); one design covers all of them because the work per weight byte is
// independent of M as long as the batch fits the MMA's n axis.
//
// Data movement per CTA
//   rows      : 16*TILES consecutive output rows; row-major [N, K/2] makes each row's K range a
//               contiguous byte run, read with 16-byte no-L1-allocate loads
//   K         : one 128-wide chunk = 64 packed bytes of a row = the 4 lanes of a quad x 16 bytes,
//               i.e. one scale group; the KW warps of a CTA take interleaved chunks, so together
//               they sweep 64*KW contiguous bytes of every row per step
//   x         : read from global through L1 (it is re-read by every warp of the SM) and permuted
//               in registers to the (k, k+4) pairing the unpack produces
//   reduction : K-split warps combine through shared memory; optional K-split CTAs combine
//               through an FP32 workspace, the last-arriving CTA summing in a fixed order
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "kernels.h"
#include "unpack.cuh"

namespace w4a16 {
namespace {

struct MmaParams {
    const __half* x;
    const uint8_t* packed;
    const __half* scales;
    __half* y;
    float* partial;        // [k_splits][M][N] when k_splits > 1
    unsigned* counters;    // one per (row block, batch block) when k_splits > 1
    int M, N, K;
    int chunks;            // K / 128
    int chunks_per_split;  // chunks handled by one K-split CTA
    int k_splits;
};

// Packed words and scales of U chunks for the warp's TILES*16 rows.
template <int TILES, int U>
struct WeightRegs {
    uint4 w[U][TILES][2];
    uint16_t s[U][TILES][2];
};

template <int NT, int TILES, int KW, int U>
__global__ void __launch_bounds__(KW * 32)
linear_mma_kernel(const MmaParams p) {
    constexpr int kRowsPerCta = 16 * TILES;
    constexpr int kAccPerLane = TILES * NT * 4;

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int g = lane >> 2;   // row within an 8-row half tile / batch column of the B operand
    const int t = lane & 3;    // which 16 bytes of the 64-byte chunk this lane owns

    const int row0 = blockIdx.x * kRowsPerCta;
    const int split = blockIdx.y;
    const int m0 = blockIdx.z * (8 * NT);

    const int c_begin = split * p.chunks_per_split;
    const int c_end = min(p.chunks, c_begin + p.chunks_per_split);
    const size_t row_bytes = static_cast<size_t>(p.K) >> 1;

    // Rows past N are clamped for the loads and dropped at the store.
    const uint8_t* wrow[TILES][2];
    const __half* srow[TILES][2];
#pragma unroll
    for (int tile = 0; tile < TILES; ++tile) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = min(row0 + tile * 16 + h * 8 + g, p.N - 1);
            wrow[tile][h] = p.packed + static_cast<size_t>(r) * row_bytes + t * 16;
            srow[tile][h] = p.scales + static_cast<size_t>(r) * p.chunks;
        }
    }

    const __half* xrow[NT];
    bool xvalid[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int n = m0 + nt * 8 + g;
        xvalid[nt] = n < p.M;
        xrow[nt] = p.x + static_cast<size_t>(xvalid[nt] ? n : 0) * p.K + t * 32;
    }

    float total[TILES][NT][4];
#pragma unroll
    for (int tile = 0; tile < TILES; ++tile)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int j = 0; j < 4; ++j) total[tile][nt][j] = 0.f;

    auto fetch = [&](WeightRegs<TILES, U>& regs, int c_first) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = c_first + u * KW;
            const bool live = c < c_end;
#pragma unroll
            for (int tile = 0; tile < TILES; ++tile) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (live) {
                        regs.w[u][tile][h] = ldg_stream16(wrow[tile][h] + static_cast<size_t>(c) * kChunkBytes);
                        regs.s[u][tile][h] = ldg_nc_u16(srow[tile][h] + c);
                    } else {
                        regs.w[u][tile][h] = make_uint4(0u, 0u, 0u, 0u);
                        regs.s[u][tile][h] = 0;
                    }
                }
            }
        }
    };

    auto consume = [&](const WeightRegs<TILES, U>& regs, int c_first) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = c_first + u * KW;
            if (c >= c_end) break;   // warp-uniform
            // Activations of this chunk for the lane's batch column(s): 32 halves = 4 x 16 bytes.
            uint4 xq[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    xq[nt][i] = xvalid[nt]
                        ? ldg_keep16(xrow[nt] + static_cast<size_t>(c) * kGroup + i * 8)
                        : make_uint4(0u, 0u, 0u, 0u);
                }
            }
            float acc[TILES][NT][4];
#pragma unroll
            for (int tile = 0; tile < TILES; ++tile)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[tile][nt][j] = 0.f;

#pragma unroll
            for (int i = 0; i < 4; ++i) {
                // B fragments: (x0,x4) (x1,x5) (x2,x6) (x3,x7) of the word's eight k.
                uint32_t b[NT][4];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const uint4 q = xq[nt][i];
                    b[nt][0] = prmt(q.x, q.z, 0x5410u);
                    b[nt][1] = prmt(q.x, q.z, 0x7632u);
                    b[nt][2] = prmt(q.y, q.w, 0x5410u);
                    b[nt][3] = prmt(q.y, q.w, 0x7632u);
                }
#pragma unroll
                for (int tile = 0; tile < TILES; ++tile) {
                    const uint4 lo = regs.w[u][tile][0];
                    const uint4 hi = regs.w[u][tile][1];
                    const uint32_t word_lo = i == 0 ? lo.x : i == 1 ? lo.y : i == 2 ? lo.z : lo.w;
                    const uint32_t word_hi = i == 0 ? hi.x : i == 1 ? hi.y : i == 2 ? hi.z : hi.w;
                    uint32_t a_lo[4], a_hi[4];
                    unpack8(word_lo, a_lo);
                    unpack8(word_hi, a_hi);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        mma_m16n8k16(acc[tile][nt], a_lo[0], a_hi[0], a_lo[1], a_hi[1], b[nt][0], b[nt][1]);
                        mma_m16n8k16(acc[tile][nt], a_lo[2], a_hi[2], a_lo[3], a_hi[3], b[nt][2], b[nt][3]);
                    }
                }
            }
#pragma unroll
            for (int tile = 0; tile < TILES; ++tile) {
                const float s_lo = __half2float(__ushort_as_half(regs.s[u][tile][0]));
                const float s_hi = __half2float(__ushort_as_half(regs.s[u][tile][1]));
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    total[tile][nt][0] = fmaf(acc[tile][nt][0], s_lo, total[tile][nt][0]);
                    total[tile][nt][1] = fmaf(acc[tile][nt][1], s_lo, total[tile][nt][1]);
                    total[tile][nt][2] = fmaf(acc[tile][nt][2], s_hi, total[tile][nt][2]);
                    total[tile][nt][3] = fmaf(acc[tile][nt][3], s_hi, total[tile][nt][3]);
                }
            }
        }
    };

    // Weights and scales never depend on the previous kernel of the stream, so the first batch is
    // requested before waiting for it; x and y may, so they are touched only after the wait.
    WeightRegs<TILES, U> cur, nxt;
    int c = c_begin + warp;
    fetch(cur, c);
    pdl_release_downstream();
    pdl_wait_for_upstream();
    for (; c < c_end; c += KW * U) {
        fetch(nxt, c + KW * U);
        consume(cur, c);
        cur = nxt;
    }

    // ---- combine the KW warps of the CTA ---------------------------------------------------
    __shared__ float red[KW][kAccPerLane][32];
#pragma unroll
    for (int tile = 0; tile < TILES; ++tile)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int j = 0; j < 4; ++j) red[warp][(tile * NT + nt) * 4 + j][lane] = total[tile][nt][j];
    __syncthreads();

    const int batch_here = min(8 * NT, p.M - m0);            // live batch columns of this CTA
    const int outputs = kRowsPerCta * batch_here;
    const bool split_k = p.k_splits > 1;

    for (int e = threadIdx.x; e < outputs; e += KW * 32) {
        const int rl = e % kRowsPerCta;        // consecutive threads -> consecutive rows of y
        const int col = e / kRowsPerCta;
        const int tile = rl >> 4, rr = rl & 15;
        const int nt = col >> 3, cc = col & 7;
        const int j = (rr >> 3) * 2 + (cc & 1);
        const int src_lane = (rr & 7) * 4 + (cc >> 1);
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < KW; ++w) sum += red[w][(tile * NT + nt) * 4 + j][src_lane];
        const int row = row0 + rl;
        const int m = m0 + col;
        if (row < p.N) {
            if (!split_k) {
                p.y[static_cast<size_t>(m) * p.N + row] = __float2half_rn(sum);
            } else {
                p.partial[(static_cast<size_t>(split) * p.M + m) * p.N + row] = sum;
            }
        }
    }
    if (!split_k) return;

    // ---- combine K-split CTAs: the last one to arrive sums all partials in split order ------
    __shared__ bool is_last;
    __threadfence();
    __syncthreads();
    unsigned* counter = p.counters + (static_cast<size_t>(blockIdx.z) * gridDim.x + blockIdx.x);
    if (threadIdx.x == 0) {
        const unsigned arrived = atomicAdd(counter, 1u);
        is_last = arrived == static_cast<unsigned>(p.k_splits - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int e = threadIdx.x; e < outputs; e += KW * 32) {
        const int rl = e % kRowsPerCta;
        const int col = e / kRowsPerCta;
        const int row = row0 + rl;
        const int m = m0 + col;
        if (row >= p.N) continue;
        float sum = 0.f;
        for (int s = 0; s < p.k_splits; ++s) {
            sum += __ldcg(p.partial + (static_cast<size_t>(s) * p.M + m) * p.N + row);
        }
        p.y[static_cast<size_t>(m) * p.N + row] = __float2half_rn(sum);
    }
    if (threadIdx.x == 0) *counter = 0u;   // ready for the next call that shares the workspace
}

template <int NT, int TILES, int KW, int U>
int launch_one(const MmaParams& params, dim3 grid, bool programmatic, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(KW * 32, 1, 1);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    const cudaError_t err = cudaLaunchKernelEx(&cfg, linear_mma_kernel<NT, TILES, KW, U>, params);
    if (err != cudaSuccess) return W4A16_ERR_LAUNCH;
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    return W4A16_OK;
}

template <int NT, int TILES, int KW>
int dispatch_unroll(int unroll, const MmaParams& params, dim3 grid, bool programmatic, cudaStream_t stream) {
    switch (unroll) {
        case 1: return launch_one<NT, TILES, KW, 1>(params, grid, programmatic, stream);
        case 2: return launch_one<NT, TILES, KW, 2>(params, grid, programmatic, stream);
        default: return W4A16_ERR_BAD_CONFIG;
    }
}

template <int NT, int TILES>
int dispatch_kw(int kw, int unroll, const MmaParams& params, dim3 grid, bool programmatic, cudaStream_t stream) {
    switch (kw) {
        case 4: return dispatch_unroll<NT, TILES, 4>(unroll, params, grid, programmatic, stream);
        case 8: return dispatch_unroll<NT, TILES, 8>(unroll, params, grid, programmatic, stream);
        default: return W4A16_ERR_BAD_CONFIG;
    }
}

template <int NT>
int dispatch_tiles(const w4a16_linear_config& c, const MmaParams& params, dim3 grid, bool programmatic,
                   cudaStream_t stream) {
    switch (c.row_tiles) {
        case 1: return dispatch_kw<NT, 1>(c.k_warps, c.unroll, params, grid, programmatic, stream);
        case 2: return dispatch_kw<NT, 2>(c.k_warps, c.unroll, params, grid, programmatic, stream);
        default: return W4A16_ERR_BAD_CONFIG;
    }
}

int batch_tiles_for(int64_t M) { return M <= 8 ? 1 : (M <= 16 ? 2 : 4); }

}  // namespace

size_t linear_counter_bytes(int64_t M, int64_t N) {
    const int64_t row_blocks = (N + 15) / 16;
    const int64_t batch_blocks = (M + 7) / 8;
    const size_t bytes = static_cast<size_t>(row_blocks * batch_blocks) * sizeof(unsigned);
    return (bytes + 255) & ~static_cast<size_t>(255);
}

size_t linear_workspace_bytes_for(int64_t M, int64_t N, int splits) {
    if (M <= 0 || N <= 0 || splits <= 1) return 0;
    return linear_counter_bytes(M, N) + static_cast<size_t>(splits) * M * N * sizeof(float);
}

w4a16_linear_config choose_linear_config(int64_t M, int64_t N, int64_t K, int max_splits) {
    constexpr int kSms = 148;
    w4a16_linear_config c;
    const int nt = batch_tiles_for(M);
    const int64_t batch_blocks = (M + 8 * nt - 1) / (8 * nt);
    const int64_t chunks = K / kGroup;
    const int64_t tiles16 = (N + 15) / 16;
    // Two tiles per warp halve the x traffic and the CTA count; only worth it when there are
    // plenty of row blocks to go round.
    c.row_tiles = (tiles16 * batch_blocks >= 8 * kSms && nt <= 2) ? 2 : 1;
    c.k_warps = chunks >= 8 ? 8 : 4;
    int64_t ctas = ((N + 16 * c.row_tiles - 1) / (16 * c.row_tiles)) * batch_blocks;
    int splits = 1;
    if (M <= 32) {
        while (splits * 2 <= max_splits && splits * 2 <= kMaxKSplits && ctas * splits < 2 * kSms &&
               chunks / (splits * 2) >= 2 * c.k_warps) {
            splits *= 2;
        }
    }
    c.k_splits = splits;
    const int64_t per_warp = (chunks / splits + c.k_warps - 1) / c.k_warps;
    c.unroll = per_warp >= 2 ? 2 : 1;
    return c;
}

int launch_linear_mma(const LinearProblem& prob, const w4a16_linear_config& cfg, bool programmatic,
                      cudaStream_t stream) {
    if (prob.group != kGroup || prob.K % kGroup != 0) return W4A16_ERR_BAD_CONFIG;
    if (prob.M > INT32_MAX || prob.N > INT32_MAX || prob.K > INT32_MAX) return W4A16_ERR_TOO_LARGE;
    const int nt = batch_tiles_for(prob.M);
    const int chunks = static_cast<int>(prob.K / kGroup);
    const int splits = cfg.k_splits;
    if (splits < 1 || splits > kMaxKSplits || splits > chunks) return W4A16_ERR_BAD_CONFIG;

    MmaParams params;
    params.x = prob.x;
    params.packed = prob.packed;
    params.scales = prob.scales;
    params.y = prob.y;
    params.partial = nullptr;
    params.counters = nullptr;
    params.M = static_cast<int>(prob.M);
    params.N = static_cast<int>(prob.N);
    params.K = static_cast<int>(prob.K);
    params.chunks = chunks;
    params.chunks_per_split = (chunks + splits - 1) / splits;
    params.k_splits = splits;
    if (splits > 1) {
        const size_t need = linear_workspace_bytes_for(prob.M, prob.N, splits);
        if (prob.workspace == nullptr || prob.workspace_bytes < need) return W4A16_ERR_WORKSPACE;
        if (reinterpret_cast<uintptr_t>(prob.workspace) % 16 != 0) return W4A16_ERR_MISALIGNED;
        params.counters = static_cast<unsigned*>(prob.workspace);
        params.partial = reinterpret_cast<float*>(static_cast<char*>(prob.workspace) +
                                                  linear_counter_bytes(prob.M, prob.N));
    }
    const int64_t row_blocks = (prob.N + 16 * cfg.row_tiles - 1) / (16 * cfg.row_tiles);
    const int64_t batch_blocks = (prob.M + 8 * nt - 1) / (8 * nt);
    if (batch_blocks > 65535) return W4A16_ERR_TOO_LARGE;
    const dim3 grid(static_cast<unsigned>(row_blocks), static_cast<unsigned>(splits),
                    static_cast<unsigned>(batch_blocks));
    switch (nt) {
        case 1: return dispatch_tiles<1>(cfg, params, grid, programmatic, stream);
        case 2: return dispatch_tiles<2>(cfg, params, grid, programmatic, stream);
        default: return dispatch_tiles<4>(cfg, params, grid, programmatic, stream);
    }
}

}  // namespace w4a16
