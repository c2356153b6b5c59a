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
// Shape of a launch
//   CTA        : 8 warps = RW row groups x KW warps; the KW warps of a group split the K range of
//                one row tile between them (contiguous sub-ranges), the RW groups own different
//                row tiles.  CTAs are persistent: the grid is sized to what is resident at once
//                and every group strides over the row tiles.
//   row tile   : 16*TILES consecutive output rows.  Row-major [N, K/2] makes a row's K range one
//                contiguous byte run; lane (g, t) reads 16 bytes of rows g and g+8 per 128-wide K
//                chunk with L1-bypassing loads, so a quad covers the 64 bytes of one scale group.
//   x          : copied once per CTA into shared memory, already permuted to the (k, k+4) pairing
//                the unpack produces and laid out so a warp's B-fragment read is one conflict-free
//                512-byte row.
//   scales     : U consecutive FP16 scales of a row in one 2*U-byte load.
//   reduction  : warps of a group combine through shared memory (one named barrier per group and
//                tile); optional K-split CTAs (grid.y) combine through an FP32 workspace, the
//                group that arrives last summing the partials in split order.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <map>
#include <mutex>
#include <utility>

#include "kernels.h"
#include "unpack.cuh"

namespace w4a16 {
namespace {

constexpr int kWarpsPerCta = 8;
constexpr int kThreads = kWarpsPerCta * 32;
constexpr int kSmemBudget = 220 * 1024;   // dynamic shared memory a CTA may ask for
constexpr int kSmemPerSm = 228 * 1024;    // shared memory of one SM; every resident CTA also reserves 1 KB
constexpr int kMaxStages = 8;

struct MmaParams {
    const __half* x;
    const uint8_t* packed;
    const __half* scales;
    void* y;               // __half [M, N], or float [M, N] when out_f32
    float* partial;        // [k_splits][M][N] when k_splits > 1
    unsigned* counters;    // one per (row tile, batch block) when k_splits > 1
    int M, N, K;
    int chunks;            // K / 128
    int chunks_per_split;  // multiple of U
    int k_splits;
    int row_tiles_total;   // ceil(N / (16 * TILES))
    int out_f32;
    int stages;            // slots of the per-thread copy ring (2..8)
};

__device__ __forceinline__ void group_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ unsigned smem_addr(const void* p) {
    return static_cast<unsigned>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint4 lds16(unsigned addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ uint32_t lds4(unsigned addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// Asynchronous global -> shared copies (no register staging).  The 16-byte form bypasses L1.
__device__ __forceinline__ void cp_async16(unsigned dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(unsigned dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }

// Wait until at most `pending` of this thread's committed copy groups are still in flight.
__device__ __forceinline__ void cp_async_wait(int pending) {
    if (pending <= 0) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else if (pending == 1) {
        asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else if (pending == 2) {
        asm volatile("cp.async.wait_group 2;" ::: "memory");
    } else if (pending == 3) {
        asm volatile("cp.async.wait_group 3;" ::: "memory");
    } else if (pending == 4) {
        asm volatile("cp.async.wait_group 4;" ::: "memory");
    } else if (pending == 5) {
        asm volatile("cp.async.wait_group 5;" ::: "memory");
    } else if (pending == 6) {
        asm volatile("cp.async.wait_group 6;" ::: "memory");
    } else {
        asm volatile("cp.async.wait_group 7;" ::: "memory");
    }
}

// Bytes one pipeline stage occupies per CTA: every thread parks U chunks x 2*TILES rows x 16 bytes
// of packed weights plus (U == 2) one 4-byte scale pair per row.
template <int TILES, int U>
__host__ __device__ constexpr int stage_bytes() {
    return kThreads * (2 * TILES * U * 16 + (U == 2 ? 2 * TILES * 4 : 0));
}

// Resident CTAs per SM the register allocation aims for.
template <int NT, int TILES>
__host__ __device__ constexpr int min_ctas_per_sm() {
    return (NT * TILES <= 2) ? 2 : 1;
}

template <int NT, int TILES, int KW, int U>
__global__ void __launch_bounds__(kThreads, min_ctas_per_sm<NT, TILES>())
linear_mma_kernel(const MmaParams p) {
    constexpr int RW = kWarpsPerCta / KW;
    constexpr int kRowsPerTile = 16 * TILES;
    constexpr int kAccPerLane = TILES * NT * 4;
    constexpr int kRedFloats = KW > 1 ? 2 * KW * kAccPerLane * 32 : 0;   // per group, double buffered
    constexpr int kStageBytes = stage_bytes<TILES, U>();
    constexpr int kItemBytes = kThreads * 16;                            // one 16-byte item of every thread
    constexpr int kScaleOffset = 2 * TILES * U * kItemBytes;             // scales follow the weights

    extern __shared__ __align__(16) unsigned char smem[];
    float* red_all = reinterpret_cast<float*>(smem);
    const unsigned ring = smem_addr(smem + sizeof(float) * kRedFloats * RW);
    const unsigned ring_end = ring + static_cast<unsigned>(p.stages) * kStageBytes;
    const unsigned xs = ring_end;
    __shared__ int last_flag[RW];

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int group = warp / KW;          // which row tile of the CTA
    const int kw = warp % KW;             // which K sub-range of the tile
    const int g = lane >> 2;
    const int t = lane & 3;

    const int split = blockIdx.y;
    const int m0 = blockIdx.z * (8 * NT);
    const int batch_here = min(8 * NT, p.M - m0);

    const int c_begin = split * p.chunks_per_split;
    const int c_end = min(p.chunks, c_begin + p.chunks_per_split);
    // Contiguous sub-range of this warp.  Every range is a whole number of U-chunk steps: the host
    // only selects U = 2 when K/128 is even, and chunks_per_split and per_warp are multiples of U.
    const int span = c_end - c_begin;
    const int per_warp = ((span + KW - 1) / KW + U - 1) / U * U;
    const int w_begin = min(c_end, c_begin + kw * per_warp);
    const int w_end = min(c_end, w_begin + per_warp);
    const int steps_per_tile = (w_end - w_begin) / U;
    const size_t row_bytes = static_cast<size_t>(p.K) >> 1;

    const int tile_stride = gridDim.x * RW;
    const int first_tile = blockIdx.x * RW + group;

    const int tid = threadIdx.x;

    // ---- producer side: a private ring of `stages` slots per thread ---------------------------
    // Each thread copies exactly the bytes it will later feed to its own MMAs, so completion of its
    // own copy groups is the only synchronisation the weight stream needs.
    const uint8_t* p_src[TILES][2];
    const __half* p_scl[TILES][2];
    int p_tile = first_tile;
    int p_left = 0;                                          // steps still to issue for p_tile
    unsigned p_waddr = ring + tid * 16;                      // this thread's first weight item of the slot
    unsigned p_saddr = ring + kScaleOffset + tid * 4;        // this thread's first scale pair of the slot
    const unsigned ring_bytes = static_cast<unsigned>(p.stages) * kStageBytes;
    auto point_producer_at = [&](int tile_index) {
        const int row0 = tile_index * kRowsPerTile;
#pragma unroll
        for (int tl = 0; tl < TILES; ++tl) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int r = min(row0 + tl * 16 + h * 8 + g, p.N - 1);   // rows past N: load the last row
                p_src[tl][h] = p.packed + static_cast<size_t>(r) * row_bytes +
                               static_cast<size_t>(w_begin) * kChunkBytes + t * 16;
                p_scl[tl][h] = p.scales + static_cast<size_t>(r) * p.chunks + w_begin;
            }
        }
        p_left = steps_per_tile;
    };
    if (steps_per_tile > 0 && p_tile < p.row_tiles_total) point_producer_at(p_tile);

    auto issue_step = [&]() {
        if (p_left > 0) {
#pragma unroll
            for (int tl = 0; tl < TILES; ++tl) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        cp_async16(p_waddr + ((tl * 2 + h) * U + u) * kItemBytes, p_src[tl][h] + u * kChunkBytes);
                    }
                    if constexpr (U == 2) {
                        cp_async4(p_saddr + (tl * 2 + h) * (kThreads * 4), p_scl[tl][h]);
                        p_scl[tl][h] += U;
                    }
                    p_src[tl][h] += U * kChunkBytes;
                }
            }
            if (--p_left == 0) {
                p_tile += tile_stride;
                if (p_tile < p.row_tiles_total) point_producer_at(p_tile);
            }
        }
        cp_async_commit();   // an empty group keeps the group count in step with the slot count
        p_waddr += kStageBytes;
        p_saddr += kStageBytes;
        if (p_waddr >= ring_end) {
            p_waddr -= ring_bytes;
            p_saddr -= ring_bytes;
        }
    };

    // Weights and scales never depend on the previous kernel of the stream, so the whole ring is
    // requested before waiting for it; x and y may, so they are touched only after the wait.
    for (int s = 0; s < p.stages; ++s) issue_step();
    pdl_release_downstream();
    pdl_wait_for_upstream();

    // ---- stage this CTA's slice of x in shared memory, in B-fragment order --------------------
    // 16-byte unit ((c * 4 + i) * batch_here + n) * 4 + t  holds, for batch row n, the eight
    // activations k = c*128 + t*32 + i*8 .. +8 re-paired as (x0,x4)(x1,x5)(x2,x6)(x3,x7).
    {
        const int units_per_row = span * 16;   // 16-byte pieces of one batch row in this K slice
        for (int n = 0; n < batch_here; ++n) {
            const uint4* src = reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(m0 + n) * p.K +
                                                              static_cast<size_t>(c_begin) * kGroup);
            for (int j = tid; j < units_per_row; j += kThreads) {
                const uint4 q = ldg_keep16(src + j);
                const int c = j >> 4, tt = (j >> 2) & 3, i = j & 3;
                const unsigned dst = xs + (((c * 4 + i) * batch_here + n) * 4 + tt) * 16;
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(prmt(q.x, q.z, 0x5410u)),
                             "r"(prmt(q.x, q.z, 0x7632u)), "r"(prmt(q.y, q.w, 0x5410u)),
                             "r"(prmt(q.y, q.w, 0x7632u))
                             : "memory");
            }
        }
    }
    __syncthreads();

    // B-fragment addressing: lane (g, t) reads unit (i * batch_here + n) * 4 + t of a chunk, n being
    // its batch column nt*8 + g.  Columns past the batch re-read the last live row instead of being
    // zero-filled: their products land in output columns that are never stored.
    unsigned x_lane[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int n = min(nt * 8 + g, batch_here - 1);
        x_lane[nt] = xs + static_cast<unsigned>(w_begin - c_begin) * batch_here * 256 + (n * 4 + t) * 16;
    }
    const unsigned x_i_stride = static_cast<unsigned>(batch_here) * 64;
    const unsigned x_chunk_stride = static_cast<unsigned>(batch_here) * 256;

    // Four registers that stay zero: the C operand of the first MMA of every chunk.
    float zero[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) asm volatile("mov.f32 %0, 0f00000000;" : "=f"(zero[j]));

    float* red = red_all + group * kRedFloats;
    int parity = 0;
    unsigned c_waddr = ring + tid * 16;
    unsigned c_saddr = ring + kScaleOffset + tid * 4;

    // Registers of one step: U chunks of packed words for 2*TILES rows, and their scale pairs.
    struct StepRegs {
        uint4 w[U][TILES][2];
        uint32_t s[TILES][2];
    };
    int my_tiles = 0;
    if (first_tile < p.row_tiles_total) my_tiles = (p.row_tiles_total - 1 - first_tile) / tile_stride + 1;
    int steps_left = my_tiles * steps_per_tile;   // steps this warp still has to consume
    int scale_row0 = first_tile * kRowsPerTile;   // only used by the U == 1 scale loads
    int scale_step = 0;

    auto load_step = [&](StepRegs& regs) {
#pragma unroll
        for (int tl = 0; tl < TILES; ++tl) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
#pragma unroll
                for (int u = 0; u < U; ++u) regs.w[u][tl][h] = lds16(c_waddr + ((tl * 2 + h) * U + u) * kItemBytes);
                if constexpr (U == 2) {
                    regs.s[tl][h] = lds4(c_saddr + (tl * 2 + h) * (kThreads * 4));
                } else {
                    const int r = min(scale_row0 + tl * 16 + h * 8 + g, p.N - 1);
                    regs.s[tl][h] = ldg_nc_u16(p.scales + static_cast<size_t>(r) * p.chunks + w_begin + scale_step);
                }
            }
        }
        if constexpr (U == 1) {
            if (++scale_step == steps_per_tile) {
                scale_step = 0;
                scale_row0 += tile_stride * kRowsPerTile;
            }
        }
        c_waddr += kStageBytes;
        c_saddr += kStageBytes;
        if (c_waddr >= ring_end) {
            c_waddr -= ring_bytes;
            c_saddr -= ring_bytes;
        }
    };

    StepRegs cur, nxt;
    if (steps_left > 0) {
        cp_async_wait(p.stages - 1);   // the oldest group has landed
        load_step(cur);
    }

    for (int tile = first_tile; tile < p.row_tiles_total; tile += tile_stride) {
        float total[TILES][NT][4];
#pragma unroll
        for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) total[tl][nt][j] = 0.f;
        const int row0 = tile * kRowsPerTile;
        unsigned x_chunk[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) x_chunk[nt] = x_lane[nt];

        for (int step = 0; step < steps_per_tile; ++step) {
            // Pull the next step's words out of shared memory before computing on this one, so the
            // shared-memory latency hides behind the unpack/MMA work of the current step.
            if (steps_left > 1) {
                cp_async_wait(p.stages - 2);
                load_step(nxt);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                float acc[TILES][NT][4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint4 b[NT];
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) b[nt] = lds16(x_chunk[nt] + i * x_i_stride);
#pragma unroll
                    for (int tl = 0; tl < TILES; ++tl) {
                        const uint4 lo = cur.w[u][tl][0];
                        const uint4 hi = cur.w[u][tl][1];
                        const uint32_t word_lo = i == 0 ? lo.x : i == 1 ? lo.y : i == 2 ? lo.z : lo.w;
                        const uint32_t word_hi = i == 0 ? hi.x : i == 1 ? hi.y : i == 2 ? hi.z : hi.w;
                        uint32_t a_lo[4], a_hi[4];
                        unpack8(word_lo, a_lo);
                        unpack8(word_hi, a_hi);
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            if (i == 0) {   // the chunk's first product starts from the zero registers
                                mma_m16n8k16_from(acc[tl][nt], zero, a_lo[0], a_hi[0], a_lo[1], a_hi[1], b[nt].x, b[nt].y);
                            } else {
                                mma_m16n8k16(acc[tl][nt], a_lo[0], a_hi[0], a_lo[1], a_hi[1], b[nt].x, b[nt].y);
                            }
                            mma_m16n8k16(acc[tl][nt], a_lo[2], a_hi[2], a_lo[3], a_hi[3], b[nt].z, b[nt].w);
                        }
                    }
                }
#pragma unroll
                for (int tl = 0; tl < TILES; ++tl) {
                    const __half2 pair_lo = *reinterpret_cast<const __half2*>(&cur.s[tl][0]);
                    const __half2 pair_hi = *reinterpret_cast<const __half2*>(&cur.s[tl][1]);
                    const float s_lo = u == 0 ? __low2float(pair_lo) : __high2float(pair_lo);
                    const float s_hi = u == 0 ? __low2float(pair_hi) : __high2float(pair_hi);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        total[tl][nt][0] = fmaf(acc[tl][nt][0], s_lo, total[tl][nt][0]);
                        total[tl][nt][1] = fmaf(acc[tl][nt][1], s_lo, total[tl][nt][1]);
                        total[tl][nt][2] = fmaf(acc[tl][nt][2], s_hi, total[tl][nt][2]);
                        total[tl][nt][3] = fmaf(acc[tl][nt][3], s_hi, total[tl][nt][3]);
                    }
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) x_chunk[nt] += x_chunk_stride;
            }
            // The slot this step came from was emptied into registers one step ago: refill it.
            issue_step();
            --steps_left;
            cur = nxt;
        }

        // ---- combine the KW warps of the group ------------------------------------------------
        const int outputs = kRowsPerTile * batch_here;
        const bool split_k = p.k_splits > 1;
        float* buf = red + parity * (KW * kAccPerLane * 32);
        if constexpr (KW > 1) {
#pragma unroll
            for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        buf[(kw * kAccPerLane + (tl * NT + nt) * 4 + j) * 32 + lane] = total[tl][nt][j];
            group_barrier(1 + group, KW * 32);
        }
        const int gthread = kw * 32 + lane;   // thread index inside the group
        if constexpr (KW > 1) {
            for (int e = gthread; e < outputs; e += KW * 32) {
                const int rl = e % kRowsPerTile;   // consecutive threads -> consecutive rows of y
                const int col = e / kRowsPerTile;
                const int tl = rl >> 4, rr = rl & 15;
                const int nt = col >> 3, cc = col & 7;
                const int j = (rr >> 3) * 2 + (cc & 1);
                const int src_lane = (rr & 7) * 4 + (cc >> 1);
                float sum = 0.f;
#pragma unroll
                for (int w = 0; w < KW; ++w) sum += buf[(w * kAccPerLane + (tl * NT + nt) * 4 + j) * 32 + src_lane];
                const int row = row0 + rl;
                const size_t m = m0 + col;
                if (row < p.N) {
                    if (split_k) {
                        p.partial[(static_cast<size_t>(split) * p.M + m) * p.N + row] = sum;
                    } else if (p.out_f32) {
                        static_cast<float*>(p.y)[m * p.N + row] = sum;
                    } else {
                        static_cast<__half*>(p.y)[m * p.N + row] = __float2half_rn(sum);
                    }
                }
            }
        } else {
            // one warp owns the tile: write straight from the accumulator registers
#pragma unroll
            for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int row = row0 + tl * 16 + (j >> 1) * 8 + g;
                        const int col = nt * 8 + 2 * t + (j & 1);
                        const size_t m = m0 + col;
                        if (row < p.N && col < batch_here) {
                            const float sum = total[tl][nt][j];
                            if (split_k) {
                                p.partial[(static_cast<size_t>(split) * p.M + m) * p.N + row] = sum;
                            } else if (p.out_f32) {
                                static_cast<float*>(p.y)[m * p.N + row] = sum;
                            } else {
                                static_cast<__half*>(p.y)[m * p.N + row] = __float2half_rn(sum);
                            }
                        }
                    }
        }
        parity ^= 1;

        if (split_k) {
            // ---- combine K-split CTAs: the group arriving last sums the partials in split order
            __threadfence();
            group_barrier(1 + group, KW * 32);
            unsigned* counter = p.counters + (static_cast<size_t>(blockIdx.z) * p.row_tiles_total + tile);
            if (gthread == 0) {
                const unsigned arrived = atomicAdd(counter, 1u);
                last_flag[group] = arrived == static_cast<unsigned>(p.k_splits - 1);
            }
            group_barrier(1 + group, KW * 32);
            const bool is_last = last_flag[group] != 0;
            if (is_last) {
                __threadfence();
                for (int e = gthread; e < outputs; e += KW * 32) {
                    const int rl = e % kRowsPerTile;
                    const int col = e / kRowsPerTile;
                    const int row = row0 + rl;
                    const size_t m = m0 + col;
                    if (row >= p.N) continue;
                    float sum = 0.f;
                    for (int s = 0; s < p.k_splits; ++s) {
                        sum += __ldcg(p.partial + (static_cast<size_t>(s) * p.M + m) * p.N + row);
                    }
                    if (p.out_f32) {
                        static_cast<float*>(p.y)[m * p.N + row] = sum;
                    } else {
                        static_cast<__half*>(p.y)[m * p.N + row] = __float2half_rn(sum);
                    }
                }
                if (gthread == 0) *counter = 0u;   // ready for the next call sharing the workspace
            }
            group_barrier(1 + group, KW * 32);   // last_flag may be rewritten by the next tile
        }
    }
    cp_async_wait(0);   // nothing of this thread may still be landing in shared memory at exit
}

// ------------------------------------------------------------------------------------------------
struct Variant {
    const void* fn;
    int red_bytes;     // shared memory for the cross-warp reduction
    int stage_bytes;   // shared memory of one pipeline stage
};

template <int NT, int TILES, int KW, int U>
Variant variant_of() {
    constexpr int RW = kWarpsPerCta / KW;
    constexpr int red = KW > 1 ? 2 * KW * TILES * NT * 4 * 32 * RW * static_cast<int>(sizeof(float)) : 0;
    return {reinterpret_cast<const void*>(&linear_mma_kernel<NT, TILES, KW, U>), red, stage_bytes<TILES, U>()};
}

template <int NT, int TILES, int KW>
bool pick_unroll(int unroll, Variant* v) {
    switch (unroll) {
        case 1: *v = variant_of<NT, TILES, KW, 1>(); return true;
        case 2: *v = variant_of<NT, TILES, KW, 2>(); return true;
        default: return false;
    }
}

template <int NT, int TILES>
bool pick_kw(int kw, int unroll, Variant* v) {
    switch (kw) {
        case 1: return pick_unroll<NT, TILES, 1>(unroll, v);
        case 2: return pick_unroll<NT, TILES, 2>(unroll, v);
        case 4: return pick_unroll<NT, TILES, 4>(unroll, v);
        case 8: return pick_unroll<NT, TILES, 8>(unroll, v);
        default: return false;
    }
}

template <int NT>
bool pick_tiles(const w4a16_linear_config& c, Variant* v) {
    switch (c.row_tiles) {
        case 1: return pick_kw<NT, 1>(c.k_warps, c.unroll, v);
        case 2: return NT <= 2 ? pick_kw<(NT <= 2 ? NT : 1), 2>(c.k_warps, c.unroll, v) : false;
        default: return false;
    }
}

bool pick_variant(int nt, const w4a16_linear_config& c, Variant* v) {
    switch (nt) {
        case 1: return pick_tiles<1>(c, v);
        case 2: return pick_tiles<2>(c, v);
        case 4: return pick_tiles<4>(c, v);
        default: return false;
    }
}

int batch_tiles_for(int64_t M) { return M <= 8 ? 1 : (M <= 16 ? 2 : 4); }

int sm_count() {
    static int cached = 0;
    if (cached == 0) {
        int device = 0, count = 0;
        if (cudaGetDevice(&device) == cudaSuccess &&
            cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) == cudaSuccess && count > 0) {
            cached = count;
        } else {
            return 148;
        }
    }
    return cached;
}

// Bytes of x a CTA must hold for `batch` rows of a K slice of `chunks` chunks.
size_t x_slice_bytes(int batch, int chunks) { return static_cast<size_t>(batch) * chunks * kGroup * sizeof(__half); }

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
    const int sms = 148;
    w4a16_linear_config c;
    const int nt = batch_tiles_for(M);
    const int batch = static_cast<int>(M < 8 * nt ? M : 8 * nt);
    const int64_t batch_blocks = (M + 8 * nt - 1) / (8 * nt);
    const int chunks = static_cast<int>(K / kGroup);
    const int64_t tiles16 = (N + 15) / 16;

    c.row_tiles = 1;
    // Warps needed to keep every SM streaming: about 16 per SM.  Split K inside the CTA first
    // (free), across CTAs second (costs a round trip through the workspace).
    const int64_t want_warps = static_cast<int64_t>(sms) * 16;
    int kw = 1;
    while (kw < 8 && tiles16 * batch_blocks * kw < want_warps && chunks >= kw * 2) kw *= 2;
    c.k_warps = kw;
    int splits = 1;
    if (M <= 32) {
        while (splits * 2 <= max_splits && splits * 2 <= kMaxKSplits &&
               tiles16 * batch_blocks * kw * splits < want_warps && chunks >= splits * 2 * kw * 2) {
            splits *= 2;
        }
    }
    // The activation slice of a CTA has to fit in shared memory.
    while (x_slice_bytes(batch, (chunks + splits - 1) / splits) > static_cast<size_t>(kSmemBudget - 80 * 1024) &&
           splits * 2 <= max_splits && splits * 2 <= kMaxKSplits && chunks >= splits * 2) {
        splits *= 2;
    }
    c.k_splits = splits;
    c.unroll = chunks % 2 == 0 ? 2 : 1;
    c.stages = 0;   // sized at launch from the shared memory left over
    return c;
}

int launch_linear_mma(const LinearProblem& prob, const w4a16_linear_config& cfg, bool programmatic,
                      bool out_f32, cudaStream_t stream) {
    if (prob.group != kGroup || prob.K % kGroup != 0) return W4A16_ERR_BAD_CONFIG;
    if (prob.M > INT32_MAX || prob.N > INT32_MAX || prob.K > INT32_MAX) return W4A16_ERR_TOO_LARGE;
    const int nt = batch_tiles_for(prob.M);
    const int chunks = static_cast<int>(prob.K / kGroup);
    const int splits = cfg.k_splits;
    if (splits < 1 || splits > kMaxKSplits || splits > chunks) return W4A16_ERR_BAD_CONFIG;
    // With unroll 2 the two scales of a step travel as one 4-byte copy: that needs K/128 even and
    // the scale matrix 4-byte aligned.
    if (cfg.unroll == 2 && (chunks % 2 != 0 || reinterpret_cast<uintptr_t>(prob.scales) % 4 != 0)) {
        return W4A16_ERR_BAD_CONFIG;
    }
    if (cfg.stages < 0 || (cfg.stages > 0 && cfg.stages < 3) || cfg.stages > kMaxStages) return W4A16_ERR_BAD_CONFIG;

    Variant variant;
    if (!pick_variant(nt, cfg, &variant)) return W4A16_ERR_BAD_CONFIG;

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
    const int per_split = (chunks + splits - 1) / splits;
    params.chunks_per_split = (per_split + cfg.unroll - 1) / cfg.unroll * cfg.unroll;
    params.k_splits = splits;
    params.row_tiles_total = static_cast<int>((prob.N + 16 * cfg.row_tiles - 1) / (16 * cfg.row_tiles));
    params.out_f32 = out_f32 ? 1 : 0;
    if ((splits - 1) * params.chunks_per_split >= chunks) return W4A16_ERR_BAD_CONFIG;   // an empty split
    if (splits > 1) {
        const size_t need = linear_workspace_bytes_for(prob.M, prob.N, splits);
        if (prob.workspace == nullptr || prob.workspace_bytes < need) return W4A16_ERR_WORKSPACE;
        if (reinterpret_cast<uintptr_t>(prob.workspace) % 16 != 0) return W4A16_ERR_MISALIGNED;
        params.counters = static_cast<unsigned*>(prob.workspace);
        params.partial = reinterpret_cast<float*>(static_cast<char*>(prob.workspace) +
                                                  linear_counter_bytes(prob.M, prob.N));
    }

    const int batch = static_cast<int>(prob.M < 8 * nt ? prob.M : 8 * nt);
    const size_t fixed = static_cast<size_t>(variant.red_bytes) + x_slice_bytes(batch, params.chunks_per_split);
    int stages = cfg.stages;
    if (stages == 0) {
        // Deepest ring that still lets three, else two, else one CTA share an SM; at least three
        // slots in flight per thread before giving up residency.
        for (int ctas = 3; ctas >= 1 && stages == 0; --ctas) {
            const int64_t room = static_cast<int64_t>(kSmemPerSm / ctas - 1024) - static_cast<int64_t>(fixed);
            const int64_t fit = room / variant.stage_bytes;
            if (fit >= (ctas > 1 ? 4 : 3)) stages = static_cast<int>(fit < kMaxStages ? fit : kMaxStages);
        }
        if (stages == 0) return W4A16_ERR_WORKSPACE;   // activation slice too large: needs more K splits
    }
    const size_t smem = fixed + static_cast<size_t>(stages) * variant.stage_bytes;
    if (smem > static_cast<size_t>(kSmemBudget)) return W4A16_ERR_WORKSPACE;
    params.stages = stages;

    // Opt in to large dynamic shared memory once per kernel variant, and learn its occupancy
    // (cached per variant and shared-memory size; one process drives one device).
    static std::mutex mutex;
    static std::map<std::pair<const void*, size_t>, int> occupancy;
    int blocks_per_sm = 0;
    {
        std::lock_guard<std::mutex> lock(mutex);
        const auto key = std::make_pair(variant.fn, smem);
        const auto found = occupancy.find(key);
        if (found != occupancy.end()) {
            blocks_per_sm = found->second;
        } else {
            if (cudaFuncSetAttribute(variant.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget) !=
                cudaSuccess) {
                return W4A16_ERR_LAUNCH;
            }
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks_per_sm, variant.fn, kThreads, smem) !=
                    cudaSuccess || blocks_per_sm < 1) {
                return W4A16_ERR_LAUNCH;
            }
            occupancy.emplace(key, blocks_per_sm);
        }
    }

    const int rw = kWarpsPerCta / cfg.k_warps;
    const int64_t batch_blocks = (prob.M + 8 * nt - 1) / (8 * nt);
    if (batch_blocks > 65535) return W4A16_ERR_TOO_LARGE;
    const int64_t tile_ctas = (params.row_tiles_total + rw - 1) / rw;
    int64_t resident = static_cast<int64_t>(sm_count()) * blocks_per_sm / (splits * batch_blocks);
    if (resident < 1) resident = 1;
    const int64_t grid_x = tile_ctas < resident ? tile_ctas : resident;
    const dim3 grid(static_cast<unsigned>(grid_x), static_cast<unsigned>(splits), static_cast<unsigned>(batch_blocks));

    cudaLaunchConfig_t launch = {};
    launch.gridDim = grid;
    launch.blockDim = dim3(kThreads, 1, 1);
    launch.dynamicSmemBytes = smem;
    launch.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    launch.attrs = attr;
    launch.numAttrs = programmatic ? 1 : 0;
    void* args[] = {const_cast<MmaParams*>(&params)};
    if (cudaLaunchKernelExC(&launch, variant.fn, args) != cudaSuccess) return W4A16_ERR_LAUNCH;
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    return W4A16_OK;
}

}  // namespace w4a16
