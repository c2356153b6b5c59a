// Prefill-sized W4A16 linear on the 5th-generation tensor cores: packed INT4 weights are
// dequantised by producer warps straight into the swizzled shared-memory operand layout of
// tcgen05.mma, so the FP16 weight matrix is never written to (or re-read from) HBM.
//
// Replaces, for large M, the reference's dequantise-to-FP16-then-cuBLAS route
// (w4a16/linear.py:132-152 over csrc/int4_linear_kernel.cu:419-451).  The arithmetic is that route's:
// weights are half(code * scale) -- one FP16 rounding per weight -- multiplied with FP16
// activations and accumulated in FP32.
//
//   D[128 x BN] (TMEM, FP32)  +=  A[128 x 64] (W rows, K-major, SWIZZLE_128B)  x  B[BN x 64] (x rows, K-major)
//
// The output channels sit on the MMA's M axis (TMEM lanes) and the batch on its N axis (TMEM
// columns, BN a multiple of 16 up to 256 chosen per call), so one pass of dequantisation feeds up to
// 256 batch rows.
//
// Persistent CTAs, one per SM, each walking a strided list of output tiles; 23 warps with fixed roles:
//   warp 0      one lane issues the TMA loads of the x tiles, one per operand stage
//   warp 22     one lane issues the TMA loads of the packed codes into a ring of its own (two tensor
//               maps built per call on the host)
//   warp 1      allocates TMEM; one lane issues the MMAs and the commits that recycle pipeline stages
//   warps 2-5   epilogue: tcgen05.ld the accumulator of the finished tile, round to FP16, store
//   warps 6-21  dequantisers, four groups of four warps; a group takes every fourth 64-wide K block and a
//               thread of it one weight row: 64 codes read from the packed tile -> unpack, scale, re-pair
//               to memory order, eight 16-byte stores at their swizzled places in the stage's FP16 tile
// The accumulator is double buffered (2 x 256 TMEM columns), so the epilogue of one tile runs under
// the main loop of the next.
//
// Two rings.  The codes are the only operand that comes from HBM, 4 KB per K block, and their slot is
// free again as soon as the dequantisers hold it in registers: eight slots keep eight K blocks of codes
// in flight whatever the tensor cores are doing.  An operand stage (the FP16 weight tile the
// dequantisers write plus the x tile) is held until its MMAs have finished; its x tile comes out of L2.
// The x tile is sized for the call's batch tile, so small batches get more operand stages (up to eight)
// out of the same shared memory.
//
// Every wait on an mbarrier is bounded; a wait that gives up sets a device status word and the CTA
// still runs to its TMEM deallocation, so a logic error ends in a reported failure, not a hung GPU.
// A give-up always follows a wait far longer than a bulk copy takes, so no copy is in flight when
// the CTA leaves.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>

#include "kernels.h"
#include "unpack.cuh"

namespace w4a16 {
namespace {

constexpr int kBM = 128;          // output channels per tile (MMA M)
constexpr int kMaxBN = 256;       // batch rows per tile at most (MMA N)
constexpr int kBK = 64;           // K of one operand sub-tile: one 128-byte swizzle row of FP16
// A pipeline stage holds SUB such sub-tiles (a template parameter of the kernel): two -- one 128-wide scale
// group per stage -- when the batch tile leaves room for three stages of that size, else one.
constexpr int kMaxStagesTc = 8;                   // operand stages at most (fewer when the x tile is large)
constexpr int kCodeCopyK = 256;                   // K of one copy of codes: 128 bytes of every row
constexpr int kCodeSlots = 2;                     // ring of such copies
constexpr int kASubTileBytes = kBM * kBK * 2;     // 16 KB
constexpr int kPackedTileBytes = kBM * kCodeCopyK / 2;   // 16 KB: whole 128-byte lines of 128 weight rows
constexpr int kDequantGroups = 4;                 // groups of dequantisers at most, taking the stages in turn
constexpr int kDequantGroupWarps = kBM / 32;      // one thread per weight row
constexpr int kDequantThreads = kDequantGroups * kBM;
constexpr int kEpilogueThreads = 128;
constexpr int kFirstDequantWarp = 6;
constexpr int kCodesWarp = kFirstDequantWarp + kDequantThreads / 32;          // 22
constexpr int kThreadsTc = (kCodesWarp + 1) * 32;                             // 736
constexpr int kBarrierBytes = 512;
constexpr int kSmemLimitTc = 227 * 1024;
constexpr int kTmemColumns = 2 * kMaxBN;
constexpr int kGroupM = 4;        // batch tiles walked together before moving along N
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
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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

__device__ __forceinline__ void umma_f16(unsigned tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t instr_desc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(instr_desc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

struct TcParams {
    const uint8_t* packed;
    const __half* scales;
    __half* y;
    int M, N, K;
    int bn;            // batch rows per tile (multiple of 16)
    int m_tiles, n_tiles, total_tiles;
    int stages;        // operand stages in use, 2..kMaxStagesTc
    int dequant_groups;   // groups of dequantisers in use: a divisor of `stages`, see the kernel
    int k_splits;         // CTAs that share one output tile, each taking a range of K (1: none)
    int split_k;          // K of one such range: a multiple of 256 (whole copies of codes)
    float* partial;       // [k_splits, M, N] FP32 sums of the ranges when k_splits > 1, else null
};

// A position in a ring of `size` slots together with the parity of the mbarrier phase it is in.
struct RingCursor {
    int slot = 0;
    unsigned phase = 0;
    bool first_round = true;
    __device__ __forceinline__ void advance(int size) {
        if (++slot == size) {
            slot = 0;
            phase ^= 1u;
            first_round = false;
        }
    }
};

// Tiles are numbered so that kGroupM batch tiles sharing one slab of weights are adjacent: CTAs
// running at the same time then read a small set of x tiles and weight slabs out of L2.
__device__ __forceinline__ void tile_coords(int tile, const TcParams& p, int& m_tile, int& n_tile) {
    const int per_group = kGroupM * p.n_tiles;
    const int g = tile / per_group;
    const int first = g * kGroupM;
    const int gm = min(kGroupM, p.m_tiles - first);
    const int local = tile - g * per_group;
    n_tile = local / gm;
    m_tile = first + (local - n_tile * gm);
}

template <int SUB>
__global__ void __launch_bounds__(kThreadsTc, 1)
linear_tcgen05_kernel(const TcParams p, const __grid_constant__ CUtensorMap x_map,
                      const __grid_constant__ CUtensorMap w_map) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // 1024-byte aligned tiles (the swizzle pattern is a function of address bits 4-9)
    const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const unsigned x_sub_tile_bytes = static_cast<unsigned>(p.bn) * (kBK * 2);   // a multiple of 2 KB
    constexpr int kStageK = SUB * kBK;
    constexpr int kATileBytes = SUB * kASubTileBytes;
    constexpr int kCodeBlocks = kCodeCopyK / kStageK;                      // stages served by one copy of codes
    const unsigned x_tile_bytes = SUB * x_sub_tile_bytes;
    const unsigned stage_bytes = kATileBytes + x_tile_bytes;
    auto a_tile = [&](int s) { return base + s * stage_bytes; };
    auto b_tile = [&](int s) { return base + s * stage_bytes + kATileBytes; };
    const unsigned codes_ring = base + p.stages * stage_bytes;
    auto packed_tile = [&](int c) { return codes_ring + c * kPackedTileBytes; };
    const unsigned bars = codes_ring + kCodeSlots * kPackedTileBytes;
    auto full_bar = [&](int s) { return bars + s * 8; };                          // operands of the stage are ready
    auto empty_bar = [&](int s) { return bars + (kMaxStagesTc + s) * 8; };        // the MMAs are done with the stage
    auto codes_bar = [&](int c) { return bars + (2 * kMaxStagesTc + c) * 8; };    // the packed codes have landed
    auto codes_free_bar = [&](int c) { return bars + (2 * kMaxStagesTc + kCodeSlots + c) * 8; };   // ... and are in registers
    constexpr int kRingBars = 2 * kMaxStagesTc + 2 * kCodeSlots;
    auto acc_full_bar = [&](int b) { return bars + (kRingBars + b) * 8; };
    auto acc_empty_bar = [&](int b) { return bars + (kRingBars + 2 + b) * 8; };
    const unsigned tmem_slot = bars + (kRingBars + 4) * 8;
    static_assert((kRingBars + 4) * 8 + 4 <= kBarrierBytes, "barrier block too small");

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    // A work item is one output tile, or one K range of it when the layer has too few tiles for the SMs: item
    // t is range t % k_splits of tile t / k_splits, so the CTAs that share a tile run side by side.
    struct Item {
        int m_tile, n_tile, split;
        int first_block;   // first pipeline stage of the range, in stages of the whole K
        int k_blocks;      // stages in the range
        int code_chunks;   // copies of codes in the range
    };
    auto item_of = [&](int item) {
        Item it;
        it.split = item % p.k_splits;
        tile_coords(item / p.k_splits, p, it.m_tile, it.n_tile);
        const int k_begin = it.split * p.split_k;
        const int k_end = min(p.K, k_begin + p.split_k);
        it.first_block = k_begin / kStageK;
        it.k_blocks = (k_end - k_begin) / kStageK;
        it.code_chunks = (it.k_blocks + kCodeBlocks - 1) / kCodeBlocks;
        return it;
    };

    if (tid == 0) {
        for (int s = 0; s < kMaxStagesTc; ++s) {
            mbar_init(full_bar(s), kDequantGroupWarps + 1);   // one lane per warp of a dequantiser group + the TMA issuer
            mbar_init(empty_bar(s), 1);                    // one tcgen05.commit
        }
        for (int c = 0; c < kCodeSlots; ++c) {
            mbar_init(codes_bar(c), 1);                    // the TMA issuer
            mbar_init(codes_free_bar(c), p.dequant_groups * kDequantGroupWarps);   // one lane per working dequantiser warp
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full_bar(b), 1);
            mbar_init(acc_empty_bar(b), kEpilogueThreads);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&x_map)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&w_map)) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(kTmemColumns) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    unsigned tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

    bool healthy = true;
    if (warp == 0) {
        // ---------------- TMA: the x tile of every operand stage ----------------------------------------
        if (lane == 0) {
            RingCursor at;
            for (int tile = blockIdx.x; tile < p.total_tiles && healthy; tile += gridDim.x) {
                const Item item = item_of(tile);
                const int m0 = item.m_tile * p.bn;
                for (int kb = item.first_block; kb < item.first_block + item.k_blocks; ++kb, at.advance(p.stages)) {
                    if (!at.first_round) healthy = mbar_wait(empty_bar(at.slot), at.phase ^ 1u, 0x10u + at.slot);
                    if (!healthy) break;
                    mbar_arrive_expect_tx(full_bar(at.slot), x_tile_bytes);
#pragma unroll
                    for (int sub = 0; sub < SUB; ++sub) {
                        asm volatile(
                            "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
                            "[%0], [%1, {%2, %3}], [%4];"
                            ::"r"(b_tile(at.slot) + sub * x_sub_tile_bytes), "l"(reinterpret_cast<uint64_t>(&x_map)),
                            "r"(kb * kStageK + sub * kBK), "r"(m0), "r"(full_bar(at.slot))
                            : "memory");
                    }
                }
            }
        }
    } else if (warp == kCodesWarp) {
        // ---------------- TMA: the packed codes, as far ahead as their ring allows ------------------------
        if (lane == 0) {
            RingCursor at;
            for (int tile = blockIdx.x; tile < p.total_tiles && healthy; tile += gridDim.x) {
                const Item item = item_of(tile);
                const int n0 = item.n_tile * kBM;
                const int first_chunk = item.first_block / kCodeBlocks;      // ranges start at whole copies
                for (int chunk = first_chunk; chunk < first_chunk + item.code_chunks; ++chunk, at.advance(kCodeSlots)) {
                    if (!at.first_round) healthy = mbar_wait(codes_free_bar(at.slot), at.phase ^ 1u, 0x60u + at.slot);
                    if (!healthy) break;
                    mbar_arrive_expect_tx(codes_bar(at.slot), kPackedTileBytes);
                    // (a box that reaches past K/2 bytes is filled with zero codes and still counts in full)
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
                        "[%0], [%1, {%2, %3}], [%4];"
                        ::"r"(packed_tile(at.slot)), "l"(reinterpret_cast<uint64_t>(&w_map)), "r"(chunk * (kCodeCopyK / 2)),
                        "r"(n0), "r"(codes_bar(at.slot))
                        : "memory");
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- one thread issues the MMAs ----------------------------------------------------
        if (lane == 0) {
            const uint32_t instr_desc = (1u << 4)                                        // FP32 accumulate
                                        | (static_cast<uint32_t>(p.bn >> 3) << 17)       // N
                                        | (static_cast<uint32_t>(kBM >> 4) << 24);       // M; FP16, K-major A and B
            unsigned done_tiles = 0;
            RingCursor at;
            for (int tile = blockIdx.x; tile < p.total_tiles && healthy; tile += gridDim.x, ++done_tiles) {
                const unsigned buf = done_tiles & 1, use = done_tiles >> 1;
                if (use > 0) healthy = mbar_wait(acc_empty_bar(buf), (use - 1) & 1, 0x40u + buf);
                if (!healthy) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned acc = tmem_base + buf * kMaxBN;
                const int k_blocks = item_of(tile).k_blocks;
                for (int kb = 0; kb < k_blocks; ++kb, at.advance(p.stages)) {
                    const int stage = at.slot;
                    healthy = mbar_wait(full_bar(stage), at.phase, 0x20u + stage);
                    if (!healthy) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                    for (int sub = 0; sub < SUB; ++sub) {
                        const uint64_t a_desc = operand_desc(a_tile(stage) + sub * kASubTileBytes);
                        const uint64_t b_desc = operand_desc(b_tile(stage) + sub * x_sub_tile_bytes);
#pragma unroll
                        for (int j = 0; j < kBK / 16; ++j) {
                            // 16 k = 32 bytes further along the swizzled row: +2 in 16-byte address units
                            umma_f16(acc, a_desc + 2 * j, b_desc + 2 * j, instr_desc, (kb > 0 || sub > 0 || j > 0) ? 1u : 0u);
                        }
                    }
                    umma_commit(empty_bar(stage));   // arrives when these MMAs have finished reading the stage
                }
                if (!healthy) break;
                umma_commit(acc_full_bar(buf));      // arrives when the whole tile has been accumulated
            }
        }
    } else if (warp < kFirstDequantWarp) {
        // ---------------- epilogue: each warp owns the 32 TMEM lanes (output channels) it may address ----
        const int quarter = warp & 3;
        unsigned done_tiles = 0;
        for (int tile = blockIdx.x; tile < p.total_tiles && healthy; tile += gridDim.x, ++done_tiles) {
            const Item item = item_of(tile);
            const int m0 = item.m_tile * p.bn;
            const int n = item.n_tile * kBM + quarter * 32 + lane;
            const unsigned buf = done_tiles & 1, use = done_tiles >> 1;
            healthy = mbar_wait(acc_full_bar(buf), use & 1, 0x30u + buf);
            if (!healthy) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned taddr = tmem_base + (static_cast<unsigned>(quarter * 32) << 16) + buf * kMaxBN;
            __half* out = p.y + static_cast<size_t>(m0) * p.N + n;
            // a K range leaves its unrounded sums; a small kernel adds the ranges in order and rounds once
            float* out_partial = p.partial == nullptr ? nullptr
                : p.partial + (static_cast<size_t>(item.split) * p.M + m0) * static_cast<size_t>(p.N) + n;
            for (int col = 0; col < p.bn; col += 16) {
                uint32_t v[16];
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                    "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                    : "r"(taddr + col));
                // the registers pass through the wait so that no use of them can be scheduled before it
                asm volatile("tcgen05.wait::ld.sync.aligned;"
                             : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]),
                               "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15])
                             :
                             : "memory");
                if (n < p.N) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (m0 + col + j < p.M) {
                            if (out_partial != nullptr) {
                                out_partial[static_cast<size_t>(col + j) * p.N] = __uint_as_float(v[j]);
                            } else {
                                out[static_cast<size_t>(col + j) * p.N] = __float2half_rn(__uint_as_float(v[j]));
                            }
                        }
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(acc_empty_bar(buf));         // this thread's part of the accumulator is in registers or stored
        }
    } else {
        // ---------------- dequantisers: group g takes K blocks g, g+4, ...; thread r of it weight row r ----
        // What a thread spends per K block is mostly waiting -- about 0.1 us per mbarrier wait, whatever the
        // barrier's state, and the latency of its own chain of instructions -- not issue slots.  So the four
        // groups work on four K blocks at once, each warp on its own (one lane waits and signals for it);
        // the MMA issuer takes the stages in order whichever group fills them.
        const int t = tid - kFirstDequantWarp * 32;
        const int group = t / kBM;
        const int r = t % kBM;
        const unsigned row_offset = (r >> 3) * 1024 + (r & 7) * 128;     // row r inside a swizzled tile
        const unsigned swz = r & 7;
        // The codes of a stage are 2*SUB of the eight 16-byte units of the row's 128 bytes in a copy, each at the
        // place the copy's 128-byte swizzle gave it.
        //
        // A parity wait is exact only for a waiter that is within one phase of the barrier.  So every working
        // group waits for every copy of codes and gives every slot back, also the copies none of its stages lie
        // in (the slot's barrier counts one arrival per working warp); and the host picks the number of working
        // groups as a divisor of the number of operand stages, so that a group meets each of its stages in
        // every round of the ring.
        constexpr int kUnits = 2 * SUB;
        const int active = p.dequant_groups;
        const int groups = p.K / kGroup;
        unsigned blocks_before = 0;                                      // stages of the tiles already done
        unsigned chunks_before = 0;                                      // ... and copies of codes
        int k_blocks = 0, code_chunks = 0;
        for (int tile = blockIdx.x; tile < p.total_tiles && healthy && group < active;
             tile += gridDim.x, blocks_before += k_blocks, chunks_before += code_chunks) {
            const Item item = item_of(tile);
            k_blocks = item.k_blocks;
            code_chunks = item.code_chunks;
            // rows past N hold zero codes (the tensor map fills them); their scale is the last row's
            const int w_row = min(item.n_tile * kBM + r, p.N - 1);
            const __half* s_ptr = p.scales + static_cast<size_t>(w_row) * groups;
            // scales (one per 128 K) are requested three of this group's stages before their use
            auto scale_of = [&](int kb) {
                return static_cast<uint32_t>(ldg_nc_u16(s_ptr + min((item.first_block + kb) * kStageK / kGroup, groups - 1)));
            };
            uint32_t s_now = scale_of(group);
            uint32_t s_next = scale_of(group + active);
            uint32_t s_after = scale_of(group + 2 * active);
            int kb = group;                                              // this group's next stage of the tile
            for (int c = 0; c < code_chunks && healthy; ++c) {
                const unsigned chunk = chunks_before + static_cast<unsigned>(c);
                const int code_slot = static_cast<int>(chunk % kCodeSlots);
                int ok = 1;
                if (lane == 0) ok = mbar_wait(codes_bar(code_slot), (chunk / kCodeSlots) & 1u, 0x50u + code_slot) ? 1 : 0;
                healthy = __shfl_sync(0xffffffffu, ok, 0) != 0;      // also orders the lanes' reads after lane 0's wait
                if (!healthy) break;
                const int chunk_end = min(k_blocks, (c + 1) * kCodeBlocks);
                for (; kb < chunk_end; kb += active) {
                    const unsigned first_unit = static_cast<unsigned>(kb % kCodeBlocks) * kUnits;
                    const unsigned it = blocks_before + static_cast<unsigned>(kb);      // position in the operand ring
                    const int stage = static_cast<int>(it % static_cast<unsigned>(p.stages));
                    const unsigned round = it / static_cast<unsigned>(p.stages);
                    const uint32_t s16 = s_now;
                    s_now = s_next;
                    s_next = s_after;
                    s_after = scale_of(kb + 3 * active);
                    uint4 words[kUnits];
#pragma unroll
                    for (int u = 0; u < kUnits; ++u) {
                        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                                     : "=r"(words[u].x), "=r"(words[u].y), "=r"(words[u].z), "=r"(words[u].w)
                                     : "r"(packed_tile(code_slot) + row_offset + (((first_unit + u) ^ swz) << 4))
                                     : "memory");
                    }
                    // the operand tile may be overwritten once the MMAs that last read this stage are done
                    if (round > 0) {
                        if (lane == 0) ok = mbar_wait(empty_bar(stage), (round - 1u) & 1u, 0x70u + stage) ? 1 : 0;
                        healthy = __shfl_sync(0xffffffffu, ok, 0) != 0;
                        if (!healthy) break;
                    }
                    const uint32_t scale2 = s16 | (s16 << 16);
#pragma unroll
                    for (int w = 0; w < 4 * kUnits; ++w) {
                        const uint4 quad = words[w >> 2];
                        const uint32_t word = (w & 3) == 0 ? quad.x : (w & 3) == 1 ? quad.y : (w & 3) == 2 ? quad.z : quad.w;
                        uint32_t h[4];
                        unpack8(word, h);                           // (c0,c4) (c1,c5) (c2,c6) (c3,c7)
#pragma unroll
                        for (int j = 0; j < 4; ++j) h[j] = hmul2_u32(h[j], scale2);
                        const uint32_t v0 = prmt(h[0], h[1], 0x5410u);   // (c0,c1)
                        const uint32_t v1 = prmt(h[2], h[3], 0x5410u);   // (c2,c3)
                        const uint32_t v2 = prmt(h[0], h[1], 0x7632u);   // (c4,c5)
                        const uint32_t v3 = prmt(h[2], h[3], 0x7632u);   // (c6,c7)
                        // word w holds k = 8w .. 8w+7 of the stage: sub-tile w / 8, 16-byte piece w % 8 of the row
                        const unsigned piece = static_cast<unsigned>(w & 7) ^ swz;
                        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a_tile(stage) + (w >> 3) * kASubTileBytes +
                                                                                       row_offset + (piece << 4)),
                                     "r"(v0), "r"(v1), "r"(v2), "r"(v3)
                                     : "memory");
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> tensor-core reads
                    __syncwarp();                                    // every lane has written its row and fenced
                    if (lane == 0) mbar_arrive(full_bar(stage));     // (release: the stores come first)
                }
                if (!healthy) break;
                __syncwarp();                                        // every lane holds the codes it wanted of this copy
                if (lane == 0) mbar_arrive(codes_free_bar(code_slot));
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns) : "memory");
    }
}

// y = half(sum of the K ranges' partial sums, in range order): four outputs per thread, 16-byte loads.
__global__ void sum_ranges_kernel(const float* __restrict__ partial, __half* __restrict__ y, long long count, int ranges) {
    const long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
    if (i >= count) return;
    float4 sum = __ldcg(reinterpret_cast<const float4*>(partial + i));
    for (int r = 1; r < ranges; ++r) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(partial + static_cast<long long>(r) * count + i));
        sum.x += v.x;
        sum.y += v.y;
        sum.z += v.z;
        sum.w += v.w;
    }
    const __half2 lo = __floats2half2_rn(sum.x, sum.y);
    const __half2 hi = __floats2half2_rn(sum.z, sum.w);
    uint2 out;
    out.x = *reinterpret_cast<const uint32_t*>(&lo);
    out.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(y + i) = out;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up through the runtime so that libcuda is not a link dependency.
EncodeTiledFn tensor_map_encoder() {
    static EncodeTiledFn fn = [] {
        void* entry = nullptr;
        cudaDriverEntryPointQueryResult found;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &found) != cudaSuccess ||
            found != cudaDriverEntryPointSuccess) {
            entry = nullptr;
        }
        return reinterpret_cast<EncodeTiledFn>(entry);
    }();
    return fn;
}

}  // namespace

// K ranges per output tile that the GEMM wants for a problem: more than one when the layer has so few tiles that
// half the SMs or more would idle and K is long enough to share (ranges of 1024 or more, a multiple of 256, and
// K of 4096 or more: below that the second launch, which adds the ranges, costs more than the shorter loop saves).
int tcgen05_k_splits(int64_t M, int64_t N, int64_t K, int64_t* split_k) {
    const int64_t m_tiles = (M + kMaxBN - 1) / kMaxBN;
    const int64_t tiles = m_tiles * ((N + kBM - 1) / kBM);
    int64_t splits = tiles > 0 ? std::min<int64_t>(4, 148 / tiles) : 1;
    splits = std::max<int64_t>(1, std::min<int64_t>(splits, K / (K >= 4096 ? 1024 : 2048)));
    int64_t width = ((K + splits - 1) / splits + 255) / 256 * 256;
    splits = (K + width - 1) / width;
    if (split_k != nullptr) *split_k = splits > 1 ? width : K;
    return static_cast<int>(splits);
}

size_t tcgen05_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    const int splits = tcgen05_k_splits(M, N, K, nullptr);
    return splits > 1 ? linear_workspace_bytes_for(M, N, splits) : 0;
}

int launch_linear_tcgen05(const LinearProblem& prob, cudaStream_t stream) {
    if (prob.group != kGroup || prob.K % kGroup != 0 || prob.K <= 0) return W4A16_ERR_BAD_CONFIG;
    if (prob.M > INT32_MAX || prob.N > INT32_MAX || prob.K > INT32_MAX) return W4A16_ERR_TOO_LARGE;
    if (reinterpret_cast<uintptr_t>(prob.x) % 16 != 0 || reinterpret_cast<uintptr_t>(prob.packed) % 16 != 0) {
        return W4A16_ERR_MISALIGNED;
    }
    const int64_t m_tiles = (prob.M + kMaxBN - 1) / kMaxBN;
    const int64_t bn = (((prob.M + m_tiles - 1) / m_tiles) + 15) / 16 * 16;     // even split, multiple of 16, <= 256
    const int64_t n_tiles = (prob.N + kBM - 1) / kBM;
    if (m_tiles * n_tiles > INT32_MAX) return W4A16_ERR_TOO_LARGE;

    const EncodeTiledFn encode = tensor_map_encoder();
    if (encode == nullptr) return W4A16_ERR_LAUNCH;
    CUtensorMap x_map;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(prob.K), static_cast<cuuint64_t>(prob.M)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(prob.K) * 2};
    const cuuint32_t box[2] = {kBK, static_cast<cuuint32_t>(bn)};
    const cuuint32_t element_strides[2] = {1, 1};
    // rows past M read as zero; the swizzle matches the MMA operand descriptor
    if (encode(&x_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(prob.x), dims, strides, box,
               element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
        return W4A16_ERR_LAUNCH;
    }

    // packed codes as a byte matrix [N, K/2]; rows past N read as zero codes
    CUtensorMap w_map;
    const cuuint64_t w_dims[2] = {static_cast<cuuint64_t>(prob.K / 2), static_cast<cuuint64_t>(prob.N)};
    const cuuint64_t w_strides[1] = {static_cast<cuuint64_t>(prob.K / 2)};
    const cuuint32_t w_box[2] = {kCodeCopyK / 2, kBM};   // 128 bytes of 128 rows, swizzled like an operand tile
    if (encode(&w_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(prob.packed), w_dims, w_strides, w_box,
               element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
        return W4A16_ERR_LAUNCH;
    }

    TcParams params{prob.packed, prob.scales, static_cast<__half*>(prob.y),
                    static_cast<int>(prob.M), static_cast<int>(prob.N), static_cast<int>(prob.K),
                    static_cast<int>(bn), static_cast<int>(m_tiles), static_cast<int>(n_tiles),
                    static_cast<int>(m_tiles * n_tiles), 0};
    // K split across CTAs when the caller's workspace has room for the partial sums (they follow the counter prefix
    // that the streaming kernel keeps at zero there)
    int64_t split_k = prob.K;
    int splits = tcgen05_k_splits(prob.M, prob.N, prob.K, &split_k);
    if (splits > 1 && (prob.workspace == nullptr || reinterpret_cast<uintptr_t>(prob.workspace) % 16 != 0 ||
                       prob.workspace_bytes < linear_workspace_bytes_for(prob.M, prob.N, splits))) {
        splits = 1;
        split_k = prob.K;
    }
    params.k_splits = splits;
    params.split_k = static_cast<int>(split_k);
    params.partial = splits > 1 ? reinterpret_cast<float*>(static_cast<char*>(prob.workspace) + linear_counter_bytes(prob.M, prob.N))
                                : nullptr;
    params.total_tiles *= splits;
    // as many operand stages as fit beside the code ring: 4 with a 256-row batch tile, 8 up to 80 rows
    const size_t fixed = static_cast<size_t>(kCodeSlots) * kPackedTileBytes + 1024 /* alignment slack */ + kBarrierBytes;
    const size_t sub_bytes = kASubTileBytes + static_cast<size_t>(bn) * (kBK * 2);      // A and x sub-tile
    // 128-wide stages (half as many waits, fences and commits for the thread that issues the MMAs, which sets the
    // pace of small batch tiles) when three of them fit: batch tiles of up to 128 rows
    const int sub_tiles = (kSmemLimitTc - fixed) / (2 * sub_bytes) >= 3 ? 2 : 1;
    const size_t stage_bytes = sub_tiles * sub_bytes;
    // stages in use / dequantiser groups in use (a divisor of the former): 2/2, 3/3, 4/4, 6/3, 8/4
    const size_t fit = (kSmemLimitTc - fixed) / stage_bytes;
    params.stages = fit >= 8 ? 8 : fit >= 6 ? 6 : fit >= 4 ? 4 : fit >= 3 ? 3 : 2;
    params.dequant_groups = params.stages == 8 ? 4 : params.stages == 6 ? 3 : params.stages;
    if (fit < 2) return W4A16_ERR_TOO_LARGE;
    const size_t smem = params.stages * stage_bytes + fixed;
    const void* kernel = sub_tiles == 2 ? reinterpret_cast<const void*>(linear_tcgen05_kernel<2>)
                                        : reinterpret_cast<const void*>(linear_tcgen05_kernel<1>);
    // the shared-memory attribute and the SM count are kept per device
    static int sm_count[64] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return W4A16_ERR_LAUNCH;
    if (sm_count[device] == 0) {
        int sms = 0;
        if (cudaFuncSetAttribute(linear_tcgen05_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kSmemLimitTc) != cudaSuccess ||
            cudaFuncSetAttribute(linear_tcgen05_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kSmemLimitTc) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) {
            return W4A16_ERR_LAUNCH;
        }
        sm_count[device] = sms;
    }
    const int grid = static_cast<int>(std::min<int64_t>(params.total_tiles, sm_count[device]));
    void* args[] = {&params, &x_map, &w_map};
    if (cudaLaunchKernel(kernel, dim3(grid), dim3(kThreadsTc), args, smem, stream) != cudaSuccess) return W4A16_ERR_LAUNCH;
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    if (splits > 1) {
        // y = half(sum of the ranges, in order)
        const long long count = static_cast<long long>(prob.M) * prob.N;
        if (count % 4 != 0 || reinterpret_cast<uintptr_t>(prob.y) % 8 != 0) {
            return launch_sum_partials(params.partial, static_cast<__half*>(prob.y), count, splits, nullptr, false, stream);
        }
        const long long blocks = (count / 4 + 255) / 256;
        if (blocks > INT32_MAX) return W4A16_ERR_TOO_LARGE;
        sum_ranges_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(params.partial, static_cast<__half*>(prob.y), count, splits);
        if (cudaGetLastError() != cudaSuccess) return W4A16_ERR_LAUNCH;
        g_launch_count.fetch_add(1, std::memory_order_relaxed);
    }
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
