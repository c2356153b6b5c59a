// Prefill-sized W4A16 linear on the 5th-generation tensor cores: packed INT4 weights are
// dequantised by the producer warps straight into the swizzled shared-memory operand layout of
// tcgen05.mma, so the FP16 weight matrix is never written to (or re-read from) HBM.
//
// Replaces, for large M, the reference's dequantise-to-FP16-then-cuBLAS route
// (w4a16/linear.py:132-152 over csrc/int4_linear_kernel.cu:419-451).  The arithmetic is that route's:
// weights are half(code * scale) -- one FP16 rounding per weight -- multiplied with FP16
// activations and accumulated in FP32.
//
//   D[128 x BN] (TMEM, FP32)  +=  A[128 x 64] (W rows, K-major, SWIZZLE_128B)  x  B[BN x 64] (x rows, K-major)
//
// so the output channels sit on the MMA's M axis and the batch on its N axis; the epilogue writes
// the transposed tile back as y[m][n].
//
// CTA = 5 warps.  Warps 0-3: one thread per weight row -- load 32 packed bytes per 64-wide K block,
// unpack, scale, re-pair to memory order and store eight 16-byte pieces at their swizzled places;
// the same threads copy the x tile with cp.async.  Warp 4: allocates TMEM, and one of its lanes issues
// the MMAs and the commits that recycle pipeline stages.  After the last K block warps 0-3 read the
// accumulator with tcgen05.ld and store FP16.
//
// Every wait on an mbarrier is bounded; a wait that gives up sets a device status word and the CTA
// still runs to its TMEM deallocation, so a logic error ends in a reported failure, not a hung GPU.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "kernels.h"
#include "unpack.cuh"

namespace w4a16 {
namespace {

constexpr int kBM = 128;          // output channels per CTA (MMA M)
constexpr int kBN = 128;          // batch rows per CTA (MMA N)
constexpr int kBK = 64;           // K per pipeline stage: one 128-byte swizzle row of FP16
constexpr int kStagesTc = 4;
constexpr int kTileBytes = kBM * kBK * 2;                 // 16 KB, A and B tiles alike (kBM == kBN)
constexpr int kProducerThreads = 128;
constexpr int kThreadsTc = kProducerThreads + 32;
constexpr unsigned kSpinLimit = 1u << 20;

// Set when a bounded wait inside the tensor-core kernel gives up (which barrier: low byte).
__device__ unsigned g_tcgen05_status = 0;

__device__ __forceinline__ unsigned smem_u32(const void* p) {
    return static_cast<unsigned>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait for the phase with the given parity to complete.  False (and a status code) on give-up.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, unsigned code) {
    for (unsigned spin = 0; spin < kSpinLimit; ++spin) {
        unsigned done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
    }
    atomicMax(&g_tcgen05_status, code);
    return false;
}

// Shared-memory operand descriptor: K-major tile, 128-byte swizzle, rows 128 bytes apart, 8-row
// groups 1024 bytes apart, descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t operand_desc(unsigned smem_address) {
    uint64_t desc = (smem_address & 0x3FFFFu) >> 4;   // start address, 16-byte units
    desc |= static_cast<uint64_t>(1) << 16;           // leading byte offset (unused with swizzle): 1
    desc |= static_cast<uint64_t>(1024 >> 4) << 32;   // stride byte offset between 8-row groups
    desc |= static_cast<uint64_t>(1) << 46;           // version
    desc |= static_cast<uint64_t>(2) << 61;           // SWIZZLE_128B
    return desc;
}

// Instruction descriptor: FP32 accumulate, FP16 A and B, both K-major, N = kBN, M = 128.
constexpr uint32_t kInstrDesc = (1u << 4) | (static_cast<uint32_t>(kBN >> 3) << 17) | (static_cast<uint32_t>(kBM >> 4) << 24);

__device__ __forceinline__ void umma_f16(unsigned tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(kInstrDesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

struct TcParams {
    const __half* x;
    const uint8_t* packed;
    const __half* scales;
    __half* y;
    int M, N, K;
};

__global__ void __launch_bounds__(kThreadsTc, 1)
linear_tcgen05_kernel(const TcParams p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // 1024-byte aligned tiles (the swizzle pattern is a function of address bits 4-9)
    const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const unsigned a_tiles = base;
    const unsigned b_tiles = base + kStagesTc * kTileBytes;
    const unsigned bars = b_tiles + kStagesTc * kTileBytes;      // full[stages], empty[stages], done
    const unsigned tmem_slot = bars + (2 * kStagesTc + 1) * 8;
    auto full_bar = [&](int s) { return bars + s * 8; };
    auto empty_bar = [&](int s) { return bars + (kStagesTc + s) * 8; };
    const unsigned done_bar = bars + 2 * kStagesTc * 8;

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int n0 = blockIdx.x * kBM;
    const int m0 = blockIdx.y * kBN;
    const int k_blocks = p.K / kBK;

    if (tid == 0) {
        for (int s = 0; s < kStagesTc; ++s) {
            mbar_init(full_bar(s), kProducerThreads);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(done_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(kBN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    unsigned tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

    bool healthy = true;
    if (warp < 4) {
        // ---------------- producers: thread r owns weight row n0 + r and batch row m0 + r ----------
        const int r = tid;
        const int w_row = min(n0 + r, p.N - 1);
        const int x_row = min(m0 + r, p.M - 1);
        const uint8_t* w_ptr = p.packed + static_cast<size_t>(w_row) * (p.K >> 1);
        const __half* s_ptr = p.scales + static_cast<size_t>(w_row) * (p.K / kGroup);
        const __half* x_ptr = p.x + static_cast<size_t>(x_row) * p.K;
        const unsigned row_offset = (r >> 3) * 1024 + (r & 7) * 128;   // this row inside a tile
        const unsigned swz = r & 7;
        for (int kb = 0; kb < k_blocks && healthy; ++kb) {
            const int stage = kb % kStagesTc;
            const unsigned round = kb / kStagesTc;
            if (round > 0) healthy = mbar_wait(empty_bar(stage), (round - 1) & 1, 0x10u + stage);
            if (!healthy) break;
            const unsigned a_row = a_tiles + stage * kTileBytes + row_offset;
            const unsigned b_row = b_tiles + stage * kTileBytes + row_offset;
            // x tile: eight 16-byte pieces of this batch row, asynchronously
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(b_row + ((c ^ swz) << 4)),
                             "l"(x_ptr + kb * kBK + c * 8)
                             : "memory");
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            // weight tile: 64 codes of this row -> FP16 * scale, in memory order
            const uint4 lo = ldg_stream16(w_ptr + kb * 32);
            const uint4 hi = ldg_stream16(w_ptr + kb * 32 + 16);
            const uint32_t s16 = ldg_nc_u16(s_ptr + (kb >> 1));
            const uint32_t scale2 = s16 | (s16 << 16);
            const uint32_t words[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                uint32_t h[4];
                unpack8(words[c], h);                       // (c0,c4) (c1,c5) (c2,c6) (c3,c7)
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] = hmul2_u32(h[j], scale2);
                const uint32_t v0 = prmt(h[0], h[1], 0x5410u);   // (c0,c1)
                const uint32_t v1 = prmt(h[2], h[3], 0x5410u);   // (c2,c3)
                const uint32_t v2 = prmt(h[0], h[1], 0x7632u);   // (c4,c5)
                const uint32_t v3 = prmt(h[2], h[3], 0x7632u);   // (c6,c7)
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a_row + ((c ^ swz) << 4)), "r"(v0), "r"(v1),
                             "r"(v2), "r"(v3)
                             : "memory");
            }
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> tensor-core reads
            mbar_arrive(full_bar(stage));
        }
    } else if (lane == 0) {
        // ---------------- one thread issues the MMAs ------------------------------------------------
        for (int kb = 0; kb < k_blocks && healthy; ++kb) {
            const int stage = kb % kStagesTc;
            const unsigned round = kb / kStagesTc;
            healthy = mbar_wait(full_bar(stage), round & 1, 0x20u + stage);
            if (!healthy) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t a_desc = operand_desc(a_tiles + stage * kTileBytes);
            const uint64_t b_desc = operand_desc(b_tiles + stage * kTileBytes);
#pragma unroll
            for (int j = 0; j < kBK / 16; ++j) {
                // 16 k = 32 bytes further along the swizzled row: +2 in 16-byte address units
                umma_f16(tmem_base, a_desc + 2 * j, b_desc + 2 * j, (kb > 0 || j > 0) ? 1u : 0u);
            }
            umma_commit(empty_bar(stage));   // arrives when these MMAs have finished reading the stage
        }
        umma_commit(done_bar);               // arrives when every MMA above has completed
    }

    // ---------------- epilogue: warps 0-3 read their 32 TMEM lanes (= 32 output channels) ---------------
    if (warp < 4) {
        const bool ready = mbar_wait(done_bar, 0, 0x30u);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int n = n0 + warp * 32 + lane;
        if (ready) {
            for (int col = 0; col < kBN; col += 8) {
                uint32_t v[8];
                const unsigned taddr = tmem_base + (static_cast<unsigned>(warp * 32) << 16) + col;
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                             : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                             : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (n < p.N) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int m = m0 + col + j;
                        if (m < p.M) p.y[static_cast<size_t>(m) * p.N + n] = __float2half_rn(__uint_as_float(v[j]));
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 4) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kBN) : "memory");
    }
}

}  // namespace

int launch_linear_tcgen05(const LinearProblem& prob, cudaStream_t stream) {
    if (prob.group != kGroup || prob.K % kGroup != 0 || prob.K <= 0) return W4A16_ERR_BAD_CONFIG;
    if (prob.M > INT32_MAX || prob.N > INT32_MAX || prob.K > INT32_MAX) return W4A16_ERR_TOO_LARGE;
    const int64_t grid_n = (prob.N + kBM - 1) / kBM;
    const int64_t grid_m = (prob.M + kBN - 1) / kBN;
    if (grid_m > 65535) return W4A16_ERR_TOO_LARGE;
    TcParams params{prob.x, prob.packed, prob.scales, static_cast<__half*>(prob.y), static_cast<int>(prob.M),
                    static_cast<int>(prob.N), static_cast<int>(prob.K)};
    const size_t smem = 2 * kStagesTc * kTileBytes + 1024 /* alignment slack */ + 256 /* barriers, TMEM slot */;
    // the attribute is kept per device
    static bool configured[64] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return W4A16_ERR_LAUNCH;
    if (!configured[device]) {
        if (cudaFuncSetAttribute(linear_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem)) != cudaSuccess) {
            return W4A16_ERR_LAUNCH;
        }
        configured[device] = true;
    }
    linear_tcgen05_kernel<<<dim3(static_cast<unsigned>(grid_n), static_cast<unsigned>(grid_m)), kThreadsTc, smem, stream>>>(params);
    if (cudaGetLastError() != cudaSuccess) return W4A16_ERR_LAUNCH;
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    return W4A16_OK;
}

// Reads (and clears) the status word of the tensor-core kernel.  Synchronises the device.
int read_tcgen05_status(unsigned* value) {
    unsigned zero = 0;
    if (cudaMemcpyFromSymbol(value, g_tcgen05_status, sizeof(unsigned)) != cudaSuccess) return W4A16_ERR_LAUNCH;
    if (cudaMemcpyToSymbol(g_tcgen05_status, &zero, sizeof(unsigned)) != cudaSuccess) return W4A16_ERR_LAUNCH;
    return W4A16_OK;
}

}  // namespace w4a16
