// The fused W4A16 streaming linear as a device function, shared by the stand-alone kernel
// (linear_mma.cu) and the persistent decode-step kernel (decode_persistent.cu).  See linear_mma.cu for
// the description of the design.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <type_traits>
#include <utility>

#include "kernels.h"
#include "unpack.cuh"

namespace w4a16 {
namespace {

// -DW4A16_BOUNDS_CHECK: every computed shared- or global-memory index of the kernel body is compared with the
// extent it must stay inside; a violation is counted and its site recorded in a device word (read through
// w4a16_bounds_check_status) and the access is skipped -- never a trap.  Stands in for compute-sanitizer where
// that tool is not available; the ordinary build compiles none of it.
#ifdef W4A16_BOUNDS_CHECK
static __device__ unsigned g_bounds_word[2];   // [0] highest site code seen, [1] number of violations
#define W4A16_IN_BOUNDS(cond, site) \
    ((cond) ? true : (atomicMax(&g_bounds_word[0], static_cast<unsigned>(site)), atomicAdd(&g_bounds_word[1], 1u), false))
#else
#define W4A16_IN_BOUNDS(cond, site) true
#endif

constexpr int kWarpsPerCta = 8;
constexpr int kThreads = kWarpsPerCta * 32;
constexpr int kSmemBudget = 220 * 1024;   // dynamic shared memory a CTA may ask for
constexpr int kFlagBytes = 128;           // split-K arrival flags at the head of the dynamic shared memory
constexpr int kSmemPerSm = 228 * 1024;    // shared memory of one SM; every resident CTA also reserves 1 KB

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
    // Optional fan-out of the result to every GPU of a tensor-parallel group (null: plain y).
    void* const* peer_out;          // [world] result buffer 0 of this layer on each rank
    const unsigned* consumed;       // this rank's consumed[] flags, indexed by reader
    unsigned* done_counter;         // CTAs of this launch that finished; left at zero
    unsigned* send_epoch;           // publications made so far by this layer on this rank
    unsigned* peer_status;          // zero while healthy; see wait_for_flags
    long long out_stride;           // bytes between the two result buffers (publication e uses buffer e & 1)
    long long ld_out;               // elements between batch rows of the peers' buffers
    long long col_out;              // first column this rank writes there
    long long wait_polls;           // bound of every flag wait
    int rank, world;
    // Optional: x is the published result of another sharded layer (null: plain x).
    const unsigned* src_epoch;      // that layer's send_epoch word on this rank
    unsigned* const* src_consumed;  // [world] consumed[] flags of that layer on each rank
    unsigned* staged_counter;       // CTAs of this launch that have read x; left at zero
    long long src_stride;           // bytes between that layer's two result buffers
    long long src_col0;             // column of the gathered result x starts at, and columns per sender:
    long long src_cols_per_rank;    //   they name the sender of an element that never arrives
    // Activations derived while they are staged (W4A16_INPUT_*): see the staging code.
    int x_mode;
    long long x_ld;                 // elements between batch rows of x (2K for [gate | up] rows)
    const long long* x_row_index;   // optional device scalar: x starts at row *x_row_index of a [rows, x_ld] table
    const __half* x_second;         // delta of the residual stream, or null
    const __half* norm_weight;
    __half* stream_out;
    float eps;
};

// Eight FP16 values at once.
struct Half8 {
    __half2 v[4];
};
__device__ __forceinline__ Half8 as_half8(const uint4& q) {
    Half8 h;
    h.v[0] = *reinterpret_cast<const __half2*>(&q.x);
    h.v[1] = *reinterpret_cast<const __half2*>(&q.y);
    h.v[2] = *reinterpret_cast<const __half2*>(&q.z);
    h.v[3] = *reinterpret_cast<const __half2*>(&q.w);
    return h;
}
__device__ __forceinline__ uint4 as_uint4(const Half8& h) {
    uint4 q;
    q.x = *reinterpret_cast<const uint32_t*>(&h.v[0]);
    q.y = *reinterpret_cast<const uint32_t*>(&h.v[1]);
    q.z = *reinterpret_cast<const uint32_t*>(&h.v[2]);
    q.w = *reinterpret_cast<const uint32_t*>(&h.v[3]);
    return q;
}
// half(silu(g)) * u, elementwise, rounded as a framework rounds it: silu in FP32, to FP16, then an FP16 product
__device__ __forceinline__ uint4 silu_mul8(const uint4& gate, const uint4& up) {
    const Half8 g = as_half8(gate), u = as_half8(up);
    Half8 out;
#pragma unroll
    for (int i = 0; i < 4; ++i) out.v[i] = __hmul2(silu_half2(g.v[i]), u.v[i]);
    return as_uint4(out);
}

// True once some wait of this layer has already given up: later waits then do not spend their own limit, so a
// missing rank costs one time-out, not one per element.
__device__ __forceinline__ bool already_failed(const unsigned* status) {
    if (status == nullptr) return false;
    unsigned seen;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(seen) : "l"(status));
    return seen != 0u;
}

// Bounded wait, by the first `world` lanes of one warp, until flags[lane] has reached `epoch`.  A flag that
// never gets there is recorded in *status as code_base + lane + 1 and the wait moves on: the caller then
// computes on unfinished data and the host reads the status word, but the GPU never hangs.
__device__ __forceinline__ void wait_for_flags(const unsigned* flags, int world, unsigned epoch, long long max_polls,
                                               unsigned* status, unsigned code_base) {
    const int lane = threadIdx.x & 31;
    if (lane < world) {
        bool arrived = false;
        for (long long poll = 0; poll < max_polls; ++poll) {
            unsigned seen;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flags + lane) : "memory");
            if (static_cast<int>(seen - epoch) >= 0) {
                arrived = true;
                break;
            }
            if ((poll & 255) == 255 && already_failed(status)) break;
            __nanosleep(20);
        }
        if (!arrived && status != nullptr) atomicMax(status, code_base + static_cast<unsigned>(lane) + 1u);
    }
    __syncwarp();
}
constexpr unsigned kReaderCodeBase = 32;   // status codes 33.. name a reader that never released a buffer

// Tells every rank that this rank has finished reading publication `epoch` of a layer.  The reads are
// complete (their values have been used) before the caller gets here, so a relaxed store is enough.
__device__ __forceinline__ void release_buffers(unsigned* const* consumed, int rank, int world, unsigned epoch) {
    for (int peer = 0; peer < world; ++peer) {
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(consumed[peer] + rank), "r"(epoch) : "memory");
    }
}

// Results travel between GPUs as tagged elements: a 32-bit word holding an FP16 value and the 16-bit tag of
// the publication it belongs to, or a 64-bit word holding an FP32 value and the tag.  One aligned store of
// such a word is atomic, so a reader that sees the expected tag also sees the value: no fence, no flag.
__device__ __forceinline__ unsigned tag_of(unsigned epoch) { return 0x8000u | (epoch & 0x7FFFu); }

__device__ __forceinline__ void store_tagged_half(void* buffer, size_t index, float value, unsigned tag) {
    const unsigned word = static_cast<unsigned>(__half_as_ushort(__float2half_rn(value))) | (tag << 16);
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(static_cast<unsigned*>(buffer) + index), "r"(word) : "memory");
}
__device__ __forceinline__ void store_tagged_float(void* buffer, size_t index, float value, unsigned tag) {
    const unsigned long long word = static_cast<unsigned long long>(__float_as_uint(value)) |
                                    (static_cast<unsigned long long>(tag) << 32);
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(static_cast<unsigned long long*>(buffer) + index), "l"(word)
                 : "memory");
}

// Eight tagged FP16 elements (32 bytes, 32-byte aligned), read past L1.
struct Tagged8 {
    uint4 a, b;
};
__device__ __forceinline__ Tagged8 load_tagged8(const uint4* src) {
    Tagged8 t;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(t.a.x), "=r"(t.a.y), "=r"(t.a.z), "=r"(t.a.w) : "l"(src));
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(t.b.x), "=r"(t.b.y), "=r"(t.b.z), "=r"(t.b.w) : "l"(src + 1));
    return t;
}
// True when all eight carry `tag2` (the tag in both halves of a word).
__device__ __forceinline__ bool tags_match(const Tagged8& t, unsigned tag2) {
    return prmt(t.a.x, t.a.y, 0x7632u) == tag2 && prmt(t.a.z, t.a.w, 0x7632u) == tag2 &&
           prmt(t.b.x, t.b.y, 0x7632u) == tag2 && prmt(t.b.z, t.b.w, 0x7632u) == tag2;
}
// The eight FP16 values, in order.
__device__ __forceinline__ uint4 values_of(const Tagged8& t) {
    return make_uint4(prmt(t.a.x, t.a.y, 0x5410u), prmt(t.a.z, t.a.w, 0x5410u), prmt(t.b.x, t.b.y, 0x5410u),
                      prmt(t.b.z, t.b.w, 0x5410u));
}
// Re-reads (bounded) until the eight elements at `src` carry the tag; false when the wait ran out.
__device__ __forceinline__ bool wait_tagged8(const uint4* src, unsigned tag2, long long max_polls, const unsigned* status,
                                             Tagged8& t) {
    for (long long poll = 0; poll < max_polls; ++poll) {
        if (tags_match(t, tag2)) return true;
        if ((poll & 255) == 255 && already_failed(status)) break;
        __nanosleep(20);
        t = load_tagged8(src);
    }
    return tags_match(t, tag2);
}
// Which sender owns `column` of a gathered result (for the status word).
__device__ __forceinline__ unsigned sender_of(long long column, long long columns_per_rank, int world) {
    if (columns_per_rank <= 0) return 0u;
    const long long sender = column / columns_per_rank;
    return static_cast<unsigned>(sender < world ? sender : world - 1);
}

__device__ __forceinline__ void group_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ unsigned smem_addr(const void* p) {
    return static_cast<unsigned>(__cvta_generic_to_shared(p));
}

template <int OFFSET>
__device__ __forceinline__ uint4 lds16(unsigned addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(addr), "n"(OFFSET));
    return v;
}

template <int OFFSET>
__device__ __forceinline__ uint32_t lds4(unsigned addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFFSET));
    return v;
}

// Asynchronous global -> shared copies (no register staging).  The 16-byte form bypasses L1.
template <int DST_OFFSET, int SRC_OFFSET>
__device__ __forceinline__ void cp_async16(unsigned dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0+%1], [%2+%3], 16;" ::"r"(dst), "n"(DST_OFFSET), "l"(src),
                 "n"(SRC_OFFSET)
                 : "memory");
}
template <int DST_OFFSET, int SRC_OFFSET>
__device__ __forceinline__ void cp_async4(unsigned dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0+%1], [%2+%3], 4;" ::"r"(dst), "n"(DST_OFFSET), "l"(src),
                 "n"(SRC_OFFSET)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }

// Wait until at most PENDING of this thread's committed copy groups are still in flight.
template <int PENDING>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory");
}

// Bytes one pipeline stage occupies per CTA: per thread U chunks x 2*TILES rows x 16 bytes of
// packed weights, plus (U == 2) per warp one 4-byte scale pair for each of its 16*TILES rows.
template <int TILES, int U>
__host__ __device__ constexpr int stage_bytes() {
    return kThreads * (2 * TILES * U * 16) + (U == 2 ? kWarpsPerCta * 16 * TILES * 4 : 0);
}

// Resident CTAs per SM the register allocation aims for.
template <int NT, int TILES>
__host__ __device__ constexpr int min_ctas_per_sm() {
    return (NT * TILES <= 2) ? 2 : 1;
}

// Stages x from another sharded layer's result buffer: tagged elements arriving from every rank.  Four pieces
// are requested per round, then the ones whose tag is not yet this publication's are re-read (bounded).
// Kept out of line so that its registers do not count against the streaming loop of the kernel.
// Destination layout: see the staging comment in the kernel (16-byte unit ((c*4 + i) * XB + n) * 4 + t).
template <int XB>
__device__ __noinline__ void stage_tagged(const uint4* base, size_t row_units, int units_per_row, int rows, unsigned tag,
                                          unsigned xs, long long max_polls, unsigned* status, long long first_column,
                                          long long cols_per_rank, int world) {
    const unsigned tag2 = tag | (tag << 16);
    const int total = units_per_row * rows;
    for (int i0 = threadIdx.x; i0 < total; i0 += 4 * kThreads) {
        Tagged8 t[4];
        const uint4* src[4];
        int at[4], row[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int i = i0 + r * kThreads;
            if (i < total) {
                row[r] = XB == 1 ? 0 : i / units_per_row;
                at[r] = XB == 1 ? i : i - row[r] * units_per_row;
                src[r] = base + row[r] * row_units + 2 * at[r];
                t[r] = load_tagged8(src[r]);
            }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            if (i0 + r * kThreads < total) {
                if (!wait_tagged8(src[r], tag2, max_polls, status, t[r]) && status != nullptr) {
                    atomicMax(status, sender_of(first_column + at[r] * 8, cols_per_rank, world) + 1u);
                }
                const uint4 q = values_of(t[r]);
                const int j = at[r];
                const int c = j >> 4, tt = (j >> 2) & 3, i = j & 3;
                const unsigned dst = xs + (((c * 4 + i) * XB + row[r]) * 4 + tt) * 16;
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(prmt(q.x, q.z, 0x5410u)),
                             "r"(prmt(q.x, q.z, 0x7632u)), "r"(prmt(q.y, q.w, 0x5410u)), "r"(prmt(q.y, q.w, 0x7632u))
                             : "memory");
            }
        }
    }
}

// NT     n8 tiles of the batch a CTA handles per pass (batch rows = up to 8*NT)
// XB     batch rows stored per chunk in the shared copy of x: 1 (M == 1) or 8*NT (padded)
// TILES  16-row tiles per warp           KW  warps splitting K of one row tile
// U      chunks per pipeline step        STAGES  ring depth
// `smem` is the CTA's dynamic shared memory (128-byte aligned).  `hooks.before_activations()` runs once the
// whole weight ring has been requested and must return only when x may be read and y written;
// `hooks.after_outputs()` runs when this CTA has written its last output.  The function may be called
// repeatedly by a persistent kernel: it leaves no copy in flight and no state in shared memory.
//
// FEATURES selects optional code at compile time, so that the plain kernel -- whose small launches are bound by
// instruction fetch and prologue latency -- carries none of it: kFeatExchange = the tensor-parallel sender and
// reader paths (peer_out / src_* parameters), kFeatRowIndex = the x_row_index parameter.
constexpr int kFeatExchange = 1;
constexpr int kFeatRowIndex = 2;

template <int NT, int XB, int TILES, int KW, int U, int STAGES, int FEATURES, typename Hooks>
__device__ __forceinline__ void linear_mma_body(const MmaParams& p, unsigned char* smem, Hooks& hooks) {
    constexpr int RW = kWarpsPerCta / KW;
    constexpr int kRowsPerTile = 16 * TILES;
    constexpr int kAccPerLane = TILES * NT * 4;
    constexpr int kRedFloats = KW > 1 ? 2 * KW * kAccPerLane * 32 : 0;   // per group, double buffered
    constexpr int kStageBytes = stage_bytes<TILES, U>();
    constexpr int kItemBytes = kThreads * 16;                            // one 16-byte item of every thread
    constexpr int kScaleOffset = 2 * TILES * U * kItemBytes;             // scales follow the weights
    constexpr int kPeriod = (STAGES % 2 == 0) ? STAGES : 2 * STAGES;     // steps per unrolled loop body
    static_assert(STAGES >= 3, "the step loop prefetches one slot ahead of the one it computes on");

    // All shared memory is dynamic and 128-byte aligned, and so is every region in it: a 16-byte
    // cp.async whose destination straddles two 32-byte shared-memory sectors cannot be merged with
    // its neighbour lane's and costs a second sector fetch from L2.
    int* last_flag = reinterpret_cast<int*>(smem);                      // [RW], first 128 bytes
    float* red_all = reinterpret_cast<float*>(smem + kFlagBytes);
    const unsigned ring = smem_addr(smem + kFlagBytes + sizeof(float) * kRedFloats * RW);
    const unsigned xs = ring + STAGES * kStageBytes;

    hooks.at_start();
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
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
    int my_tiles = 0;
    if (first_tile < p.row_tiles_total) my_tiles = (p.row_tiles_total - 1 - first_tile) / tile_stride + 1;

    // ---- producer side ------------------------------------------------------------------------
    // U == 2: a step is 128 contiguous bytes of each of the warp's 16*TILES rows.  Copy j of a lane
    // moves piece (lane & 7) of row 4j + lane/8, so every warp-wide cp.async covers four whole
    // 128-byte lines; the bytes land where the lane that will consume them expects them
    // (item (chunk, row half), entry row%8 * 4 + piece%4).  The warp therefore shares its slots:
    // one __syncwarp after the wait publishes them, and orders the refill after everyone's reads.
    // U == 1: a step is 64 bytes per row and every lane copies exactly what it consumes itself.
    constexpr int kCopies = U == 2 ? 4 * TILES : 2 * TILES;   // 16-byte copies per lane per step
    const unsigned ring_w = ring + tid * 16;                  // consumer view: this lane's entry of item 0
    const unsigned ring_s = ring + kScaleOffset + warp * (16 * TILES * 4);   // this warp's scale pairs
    const unsigned copy_dst = U == 2
        ? ring + ((lane >> 2) & 1) * kItemBytes + (warp * 32 + (lane >> 3) * 4 + (lane & 3)) * 16
        : ring_w;
    // Source pointers are kept "as of position 0 of the unrolled period": the copy issued at
    // position POS reads p_src + POS * (bytes per step), an immediate, so the pointers move once per
    // period instead of once per step.
    constexpr int kStepBytes = U * kChunkBytes;               // packed bytes of one row per step
    const uint8_t* p_src[kCopies];
    const __half* p_scl = nullptr;
    int p_tile = first_tile;
    int p_left = 0;                                           // steps still to issue for p_tile
    const bool scale_lane = lane < 16 * TILES;
    auto point_producer_at = [&](int tile_index, int pos) {
        const int row0 = tile_index * kRowsPerTile;
#pragma unroll
        for (int j = 0; j < kCopies; ++j) {
            // rows past N re-read the last row; their results are never stored
            const int local = U == 2 ? 4 * j + (lane >> 3) : 8 * j + g;
            const int piece = U == 2 ? (lane & 7) : t;
            const int r = min(row0 + local, p.N - 1);
            p_src[j] = p.packed + static_cast<size_t>(r) * row_bytes + static_cast<size_t>(w_begin) * kChunkBytes +
                       piece * 16 - pos * kStepBytes;
        }
        if constexpr (U == 2) {
            const int r = min(row0 + (lane & (16 * TILES - 1)), p.N - 1);
            p_scl = p.scales + static_cast<size_t>(r) * p.chunks + w_begin - pos * U;
        }
        p_left = steps_per_tile;
    };
    if (steps_per_tile > 0 && my_tiles > 0) point_producer_at(p_tile, 0);

    auto copy_at = [&](auto pos_tag, auto j_tag) {
        constexpr int POS = decltype(pos_tag)::value;
        constexpr int SLOT = POS % STAGES;
        constexpr int j = decltype(j_tag)::value;
        if constexpr (j < kCopies) {
            // U == 2: copy j -> tile j/4, row half (j/2)%2, rows (j%2)*4 .. +3 of that half
            constexpr int OFFSET = U == 2
                ? SLOT * kStageBytes + ((j >> 2) * 2 + ((j >> 1) & 1)) * U * kItemBytes + (j & 1) * 256
                : SLOT * kStageBytes + j * kItemBytes;
            // source: 16 bytes inside the packed matrix; destination: inside the ring
            if (!W4A16_IN_BOUNDS(p_src[j] + POS * kStepBytes >= p.packed &&
                                     p_src[j] + POS * kStepBytes + 16 <= p.packed + static_cast<size_t>(p.N) * row_bytes &&
                                     copy_dst + OFFSET + 16 <= ring + STAGES * kStageBytes, 4)) {
                return;
            }
            cp_async16<OFFSET, POS * kStepBytes>(copy_dst, p_src[j]);
        }
    };
    // Requests the next step of this warp's stream into the ring slot of period position POS and
    // commits the group (an empty group when the stream is exhausted keeps group count and slot
    // count in step).
    auto issue_step = [&](auto pos_tag) {
        constexpr int POS = decltype(pos_tag)::value;
        constexpr int SLOT = POS % STAGES;
        constexpr int NEXT_POS = (POS + 1) % kPeriod;
        if (p_left > 0) {
            copy_at(pos_tag, std::integral_constant<int, 0>{});
            copy_at(pos_tag, std::integral_constant<int, 1>{});
            copy_at(pos_tag, std::integral_constant<int, 2>{});
            copy_at(pos_tag, std::integral_constant<int, 3>{});
            copy_at(pos_tag, std::integral_constant<int, 4>{});
            copy_at(pos_tag, std::integral_constant<int, 5>{});
            copy_at(pos_tag, std::integral_constant<int, 6>{});
            copy_at(pos_tag, std::integral_constant<int, 7>{});
            if constexpr (U == 2) {
                if (scale_lane && W4A16_IN_BOUNDS(p_scl + POS * U >= p.scales &&
                                                      p_scl + POS * U + 2 <= p.scales + static_cast<size_t>(p.N) * p.chunks, 5)) {
                    cp_async4<SLOT * kStageBytes, POS * U * 2>(ring_s + lane * 4, p_scl);
                }
            }
            if (--p_left == 0) {
                p_tile += tile_stride;
                if (p_tile < p.row_tiles_total) point_producer_at(p_tile, NEXT_POS);
            } else if constexpr (NEXT_POS == 0) {
#pragma unroll
                for (int j = 0; j < kCopies; ++j) p_src[j] += kPeriod * kStepBytes;
                if constexpr (U == 2) p_scl += kPeriod * U;
            }
        }
        cp_async_commit();
    };
    auto issue_all_slots = [&]<int... S>(std::integer_sequence<int, S...>) {
        (issue_step(std::integral_constant<int, S>{}), ...);
    };

    // Weights and scales never depend on the previous kernel of the stream, so the whole ring is
    // requested before waiting for it; x and y may, so they are touched only after the wait.
    issue_all_slots(std::make_integer_sequence<int, STAGES>{});
    hooks.before_activations();

    // Tensor-parallel hand-shakes, with the weight ring already in flight.  As a sender: wait until every rank
    // has let go of the result buffer this launch will overwrite (two publications back, so this is normally
    // satisfied long ago).  As a reader nothing is waited for here: the staging loop below re-reads elements
    // of x that have not arrived yet.
    const __half* x_in = p.x;
    constexpr bool kExchange = (FEATURES & kFeatExchange) != 0;
    if constexpr ((FEATURES & kFeatRowIndex) != 0) {
        if (p.x_row_index != nullptr) x_in += static_cast<size_t>(__ldcg(p.x_row_index)) * static_cast<size_t>(p.x_ld);
    }
    unsigned src_epoch = 0, out_epoch = 0, out_tag = 0;
    size_t out_offset = 0;
    if (kExchange && p.src_epoch != nullptr) {
        src_epoch = __ldcg(p.src_epoch);
        x_in = reinterpret_cast<const __half*>(reinterpret_cast<const char*>(p.x) + (src_epoch & 1u) * p.src_stride);
    }
    if (kExchange && p.peer_out != nullptr) {
        out_epoch = __ldcg(p.send_epoch) + 1u;
        out_tag = tag_of(out_epoch);
        if (warp == 1) wait_for_flags(p.consumed, p.world, out_epoch - 2u, p.wait_polls, p.peer_status, kReaderCodeBase);
        out_offset = static_cast<size_t>(out_epoch & 1u) * static_cast<size_t>(p.out_stride);
        __syncthreads();
    }

    // ---- stage this CTA's slice of x in shared memory, in B-fragment order --------------------
    // 16-byte unit ((c * 4 + i) * XB + n) * 4 + t holds, for batch row n, the eight activations
    // k = c*128 + t*32 + i*8 .. +8 re-paired as (x0,x4)(x1,x5)(x2,x6)(x3,x7).
    // With p.x_mode set, the activations are computed here from what produced them: silu(gate) * up of
    // a fused gate/up output, or the RMSNorm of the residual stream plus the last block's output (one
    // CTA also writes the summed stream back).
    {
        const int units_per_row = span * 16;   // 16-byte pieces of one batch row in this K slice
        auto put = [&](const uint4& q, int j, int n) {
            const int c = j >> 4, tt = (j >> 2) & 3, i = j & 3;
            const unsigned dst = xs + (((c * 4 + i) * XB + n) * 4 + tt) * 16;
            if (!W4A16_IN_BOUNDS(n >= 0 && n < XB && j >= 0 && dst + 16 <= xs + static_cast<unsigned>(span) * (XB * 256), 1)) return;
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(prmt(q.x, q.z, 0x5410u)),
                         "r"(prmt(q.x, q.z, 0x7632u)), "r"(prmt(q.y, q.w, 0x5410u)),
                         "r"(prmt(q.y, q.w, 0x7632u))
                         : "memory");
        };
        if (kExchange && p.src_epoch != nullptr) {
            const int staged_rows = XB == 1 ? 1 : batch_here;
            const uint4* base = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned*>(x_in) +
                                                               static_cast<size_t>(m0) * p.x_ld +
                                                               static_cast<size_t>(c_begin) * kGroup);
            stage_tagged<XB>(base, static_cast<size_t>(p.x_ld) >> 2, units_per_row, staged_rows, tag_of(src_epoch), xs,
                             p.wait_polls, p.peer_status, p.src_col0 + static_cast<long long>(c_begin) * kGroup,
                             p.src_cols_per_rank, p.world);
        } else if (p.x_mode == W4A16_INPUT_ADD_RMSNORM) {
            // pass 1, whole row: s = half(stream + delta), sum of squares in FP32
            const uint4* s_in = reinterpret_cast<const uint4*>(x_in);
            const uint4* d_in = reinterpret_cast<const uint4*>(p.x_second);
            const bool writer = p.stream_out != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
            auto summed = [&](int j) {
                Half8 s8 = as_half8(ldg_keep16(s_in + j));
                if (d_in != nullptr) {
                    const Half8 d8 = as_half8(ldg_keep16(d_in + j));
#pragma unroll
                    for (int i = 0; i < 4; ++i) s8.v[i] = __hadd2(s8.v[i], d8.v[i]);
                }
                return s8;
            };
            float sq = 0.0f;
            for (int j = tid; j < (p.K >> 3); j += kThreads) {
                const Half8 s8 = summed(j);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __half22float2(s8.v[i]);
                    sq += f.x * f.x + f.y * f.y;
                }
                if (writer) reinterpret_cast<uint4*>(p.stream_out)[j] = as_uint4(s8);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            float* scratch = reinterpret_cast<float*>(smem + 64);     // second half of the flag header: free until the epilogue
            if (lane == 0) scratch[warp] = sq;
            __syncthreads();
            float total = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarpsPerCta; ++w) total += scratch[w];
            const float inv = rsqrtf(total / static_cast<float>(p.K) + p.eps);
            // pass 2, this CTA's K slice: weight * half(s * inv)
            const uint4* w_in = reinterpret_cast<const uint4*>(p.norm_weight);
            for (int j = tid; j < units_per_row; j += kThreads) {
                const int at = c_begin * 16 + j;
                const Half8 s8 = summed(at);
                const Half8 w8 = as_half8(ldg_keep16(w_in + at));
                Half8 x8;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __half22float2(s8.v[i]);
                    x8.v[i] = __hmul2(w8.v[i], __floats2half2_rn(f.x * inv, f.y * inv));
                }
                put(as_uint4(x8), j, 0);
            }
        } else {
            // Only the rows that exist are staged.  The B-fragment columns of the rows past the batch then hold
            // whatever the shared memory held; each output column depends on its own activation row alone and
            // those columns are never stored.
            const int staged_rows = XB == 1 ? 1 : batch_here;
            // Up to eight rows' loads are issued before the first store (the stores are ordered against later
            // loads, so a row-at-a-time loop would pay one L2 round trip per row).
            constexpr int kRowBatch = XB < 8 ? XB : 8;
            const bool silu = p.x_mode == W4A16_INPUT_SILU_MUL;
            const uint4* base = reinterpret_cast<const uint4*>(x_in + static_cast<size_t>(m0) * p.x_ld +
                                                               static_cast<size_t>(c_begin) * kGroup);
            const size_t row_units = static_cast<size_t>(p.x_ld) >> 3;       // 16-byte units between batch rows
            if constexpr (XB == 1) {
                // one row: four pieces of it per round
                for (int j0 = tid; j0 < units_per_row; j0 += 4 * kThreads) {
                    uint4 q[4], u[4];
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const int j = j0 + r * kThreads;
                        if (j < units_per_row) {
                            q[r] = ldg_keep16(base + j);
                            if (silu) u[r] = ldg_keep16(base + j + (p.K >> 3));   // the second K values of the row
                        }
                    }
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const int j = j0 + r * kThreads;
                        if (j < units_per_row) put(silu ? silu_mul8(q[r], u[r]) : q[r], j, 0);
                    }
                }
            } else {
                for (int j = tid; j < units_per_row; j += kThreads) {
                    for (int n0 = 0; n0 < staged_rows; n0 += kRowBatch) {
                        uint4 q[kRowBatch], u[kRowBatch];
#pragma unroll
                        for (int r = 0; r < kRowBatch; ++r) {
                            if (n0 + r < staged_rows) {
                                const uint4* src = base + (n0 + r) * row_units + j;
                                q[r] = ldg_keep16(src);
                                if (silu) u[r] = ldg_keep16(src + (p.K >> 3));
                            }
                        }
#pragma unroll
                        for (int r = 0; r < kRowBatch; ++r) {
                            if (n0 + r < staged_rows) put(silu ? silu_mul8(q[r], u[r]) : q[r], j, n0 + r);
                        }
                    }
                }
            }
        }
    }
    __syncthreads();
    if (kExchange && p.src_epoch != nullptr && tid == 0) {
        // the last CTA to have read its part of x gives the buffer back to the senders
        const unsigned ctas = gridDim.x * gridDim.y * gridDim.z;
        if (atomicAdd(p.staged_counter, 1u) == ctas - 1) {
            *p.staged_counter = 0u;
            release_buffers(p.src_consumed, p.rank, p.world, src_epoch);
        }
    }

    // B-fragment base of this lane: batch column g of n-tile 0 (every lane reads row 0 when XB == 1).
    const unsigned x_lane = xs + static_cast<unsigned>(w_begin - c_begin) * (XB * 256) +
                            ((XB == 1 ? 0 : g) * 4 + t) * 16;

    // Four registers that stay zero: the C operand of the first MMA of every chunk.
    float zero[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) asm volatile("mov.f32 %0, 0f00000000;" : "=f"(zero[j]));

    // Registers of one step: U chunks of packed words for 2*TILES rows, and their scale pairs.
    struct StepRegs {
        uint4 w[U][TILES][2];
        uint32_t s[TILES][2];
    };
    StepRegs buf[2];

    int steps_left = my_tiles * steps_per_tile;   // steps this warp still has to consume
    int scale_row0 = first_tile * kRowsPerTile;   // walked only by the U == 1 scale loads
    int scale_step = 0;

    auto load_step = [&](StepRegs& regs, auto slot_tag) {
        constexpr int SLOT = decltype(slot_tag)::value;
        auto item = [&](auto index_tag) -> uint4 {
            return lds16<SLOT * kStageBytes + decltype(index_tag)::value * kItemBytes>(ring_w);
        };
        auto scale = [&](auto index_tag) -> uint32_t {
            return lds4<SLOT * kStageBytes + decltype(index_tag)::value * 32>(ring_s + g * 4);
        };
        if constexpr (U == 2) {
            // item (tile, half, chunk) = ((tile*2 + half) * 2 + chunk); scale pair of row tile*16 + half*8 + g
            regs.w[0][0][0] = item(std::integral_constant<int, 0>{});
            regs.w[1][0][0] = item(std::integral_constant<int, 1>{});
            regs.w[0][0][1] = item(std::integral_constant<int, 2>{});
            regs.w[1][0][1] = item(std::integral_constant<int, 3>{});
            regs.s[0][0] = scale(std::integral_constant<int, 0>{});
            regs.s[0][1] = scale(std::integral_constant<int, 1>{});
            if constexpr (TILES == 2) {
                regs.w[0][1][0] = item(std::integral_constant<int, 4>{});
                regs.w[1][1][0] = item(std::integral_constant<int, 5>{});
                regs.w[0][1][1] = item(std::integral_constant<int, 6>{});
                regs.w[1][1][1] = item(std::integral_constant<int, 7>{});
                regs.s[1][0] = scale(std::integral_constant<int, 2>{});
                regs.s[1][1] = scale(std::integral_constant<int, 3>{});
            }
        } else {
            regs.w[0][0][0] = item(std::integral_constant<int, 0>{});
            regs.w[0][0][1] = item(std::integral_constant<int, 1>{});
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int r = min(scale_row0 + h * 8 + g, p.N - 1);
                regs.s[0][h] = ldg_nc_u16(p.scales + static_cast<size_t>(r) * p.chunks + w_begin + scale_step);
            }
            if (++scale_step == steps_per_tile) {
                scale_step = 0;
                scale_row0 += tile_stride * kRowsPerTile;
            }
        }
    };

    float total[TILES][NT][4];
#pragma unroll
    for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int j = 0; j < 4; ++j) total[tl][nt][j] = 0.f;

    unsigned x_step = x_lane;   // B-fragment address of the current step's first chunk

    // B fragment of (chunk u of the step, word i, n-tile nt): compile-time offsets from x_step.
    auto load_b = [&](auto u_tag, auto i_tag, auto nt_tag) -> uint4 {
        constexpr int OFFSET = decltype(u_tag)::value * (XB * 256) + decltype(i_tag)::value * (XB * 64) +
                               decltype(nt_tag)::value * 512;
        return lds16<OFFSET>(x_step);
    };

    auto compute_chunk = [&](const StepRegs& regs, auto u_tag) {
        constexpr int u = decltype(u_tag)::value;
        float acc[TILES][NT][4];
        auto word_step = [&](auto i_tag) {
            constexpr int i = decltype(i_tag)::value;
            uint4 b[NT];
            if constexpr (NT >= 1) b[0] = load_b(u_tag, i_tag, std::integral_constant<int, 0>{});
            if constexpr (NT >= 2) b[1] = load_b(u_tag, i_tag, std::integral_constant<int, 1>{});
            if constexpr (NT >= 4) {
                b[2] = load_b(u_tag, i_tag, std::integral_constant<int, 2>{});
                b[3] = load_b(u_tag, i_tag, std::integral_constant<int, 3>{});
            }
#pragma unroll
            for (int tl = 0; tl < TILES; ++tl) {
                const uint4 lo = regs.w[u][tl][0];
                const uint4 hi = regs.w[u][tl][1];
                const uint32_t word_lo = i == 0 ? lo.x : i == 1 ? lo.y : i == 2 ? lo.z : lo.w;
                const uint32_t word_hi = i == 0 ? hi.x : i == 1 ? hi.y : i == 2 ? hi.z : hi.w;
                uint32_t a_lo[4], a_hi[4];
                unpack8(word_lo, a_lo);
                unpack8(word_hi, a_hi);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    if constexpr (i == 0) {   // the chunk's first product starts from the zero registers
                        mma_m16n8k16_from(acc[tl][nt], zero, a_lo[0], a_hi[0], a_lo[1], a_hi[1], b[nt].x, b[nt].y);
                    } else {
                        mma_m16n8k16(acc[tl][nt], a_lo[0], a_hi[0], a_lo[1], a_hi[1], b[nt].x, b[nt].y);
                    }
                    mma_m16n8k16(acc[tl][nt], a_lo[2], a_hi[2], a_lo[3], a_hi[3], b[nt].z, b[nt].w);
                }
            }
        };
        word_step(std::integral_constant<int, 0>{});
        word_step(std::integral_constant<int, 1>{});
        word_step(std::integral_constant<int, 2>{});
        word_step(std::integral_constant<int, 3>{});
#pragma unroll
        for (int tl = 0; tl < TILES; ++tl) {
            const __half2 pair_lo = *reinterpret_cast<const __half2*>(&regs.s[tl][0]);
            const __half2 pair_hi = *reinterpret_cast<const __half2*>(&regs.s[tl][1]);
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
    };
    auto compute_step = [&](const StepRegs& regs) {
        compute_chunk(regs, std::integral_constant<int, 0>{});
        if constexpr (U == 2) compute_chunk(regs, std::integral_constant<int, 1>{});
        x_step += U * XB * 256;
    };

    float* red = red_all + group * kRedFloats;
    int parity = 0;
    const int gthread = kw * 32 + lane;   // thread index inside the group
    const bool split_k = p.k_splits > 1;

    // Final destination of one output element: this rank's y, or the same position in the result
    // buffer of every rank of the group (plain stores over NVLink into peer-mapped memory).
    auto write_out = [&](int row, size_t m, float sum) {
        if (!W4A16_IN_BOUNDS(row >= 0 && row < p.N && m < static_cast<size_t>(p.M), 2)) return;
        if (!kExchange || p.peer_out == nullptr) {
            if (p.out_f32) {
                static_cast<float*>(p.y)[m * p.N + row] = sum;
            } else {
                static_cast<__half*>(p.y)[m * p.N + row] = __float2half_rn(sum);
            }
        } else {
            const size_t at = m * static_cast<size_t>(p.ld_out) + static_cast<size_t>(p.col_out) + row;
            for (int peer = 0; peer < p.world; ++peer) {
                char* buffer = static_cast<char*>(p.peer_out[peer]) + out_offset;
                if (p.out_f32) {
                    store_tagged_float(buffer, at, sum, out_tag);
                } else {
                    store_tagged_half(buffer, at, sum, out_tag);
                }
            }
        }
    };

    // Combines the group's warps for one finished row tile and writes it out (or hands it to the
    // split-K reduction); leaves `total` cleared for the next tile.
    auto finish_tile = [&](int tile) {
        const int row0 = tile * kRowsPerTile;
        const int outputs = kRowsPerTile * batch_here;
        float* stage = red + parity * (KW * kAccPerLane * 32);
        auto store = [&](int row, size_t m, float sum) {
            if (split_k) {
                if (!W4A16_IN_BOUNDS(row >= 0 && row < p.N && m < static_cast<size_t>(p.M) && split < p.k_splits, 3)) return;
                p.partial[(static_cast<size_t>(split) * p.M + m) * p.N + row] = sum;
            } else {
                write_out(row, m, sum);
            }
        };
        if constexpr (KW > 1) {
#pragma unroll
            for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        stage[(kw * kAccPerLane + (tl * NT + nt) * 4 + j) * 32 + lane] = total[tl][nt][j];
            group_barrier(1 + group, KW * 32);
            for (int e = gthread; e < outputs; e += KW * 32) {
                const int rl = e % kRowsPerTile;   // consecutive threads -> consecutive rows of y
                const int col = e / kRowsPerTile;
                const int tl = rl >> 4, rr = rl & 15;
                const int nt = col >> 3, cc = col & 7;
                const int j = (rr >> 3) * 2 + (cc & 1);
                const int src_lane = (rr & 7) * 4 + (cc >> 1);
                float sum = 0.f;
#pragma unroll
                for (int w = 0; w < KW; ++w) sum += stage[(w * kAccPerLane + (tl * NT + nt) * 4 + j) * 32 + src_lane];
                if (row0 + rl < p.N) store(row0 + rl, m0 + col, sum);
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
                        if (row < p.N && col < batch_here) store(row, m0 + col, total[tl][nt][j]);
                    }
        }
        parity ^= 1;
#pragma unroll
        for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) total[tl][nt][j] = 0.f;

        if (split_k) {
            // The group arriving last at this tile sums the partials of all K splits in split order.
            __threadfence();
            group_barrier(1 + group, KW * 32);
            unsigned* counter = p.counters + (static_cast<size_t>(blockIdx.z) * p.row_tiles_total + tile);
            if (gthread == 0) {
                const unsigned arrived = atomicAdd(counter, 1u);
                last_flag[group] = arrived == static_cast<unsigned>(p.k_splits - 1);
            }
            group_barrier(1 + group, KW * 32);
            if (last_flag[group] != 0) {
                __threadfence();
                for (int e = gthread; e < outputs; e += KW * 32) {
                    const int row = row0 + e % kRowsPerTile;
                    const size_t m = m0 + e / kRowsPerTile;
                    if (row >= p.N) continue;
                    float sum = 0.f;
                    for (int s = 0; s < p.k_splits; ++s) {
                        sum += __ldcg(p.partial + (static_cast<size_t>(s) * p.M + m) * p.N + row);
                    }
                    write_out(row, m, sum);
                }
                if (gthread == 0) *counter = 0u;   // ready for the next call sharing the workspace
            }
            group_barrier(1 + group, KW * 32);   // last_flag may be rewritten at the next tile
        }
    };

    if (steps_per_tile == 0) {
        // A warp without a share of K still meets its group at every tile's barrier.
        for (int tile = first_tile; tile < p.row_tiles_total; tile += tile_stride) finish_tile(tile);
    }

    if (steps_left > 0) {
        cp_async_wait<STAGES - 1>();   // the oldest group, slot 0, has landed
        __syncwarp();                  // ... for every lane of the warp
        load_step(buf[0], std::integral_constant<int, 0>{});
    }
    int tile = first_tile;
    int tile_steps_left = steps_per_tile;

    // One position of the unrolled step loop: POS fixes the ring slot and the register buffer.
    // Returns true when the step completed the current row tile.
    auto step_at = [&](auto pos_tag) -> bool {
        constexpr int POS = decltype(pos_tag)::value;
        constexpr int NEXT_SLOT = (POS + 1) % STAGES;
        constexpr int PRODUCER_POS = (POS + STAGES) % kPeriod;   // the producer runs STAGES steps ahead
        // The warp-wide sync publishes the lanes' landed copies to each other; it also orders the
        // refill below after every lane's reads of that slot (done one step ago).
        cp_async_wait<STAGES - 2>();
        __syncwarp();
        // Pull the next step's words out of shared memory before computing on this one, so the
        // shared-memory latency hides behind the current step's unpack and MMA work.
        // (Past the last step this reads a stale slot into registers nobody uses.)
        load_step(buf[(POS + 1) & 1], std::integral_constant<int, NEXT_SLOT>{});
        compute_step(buf[POS & 1]);
        // This step's slot was emptied into registers one step ago: refill it.
        issue_step(std::integral_constant<int, PRODUCER_POS>{});
        --steps_left;
        return --tile_steps_left == 0;
    };

    // The step code exists once per ring position and the tile epilogue once: a step that finishes
    // a tile leaves the switch, the epilogue runs, and the switch is re-entered at the next position.
    int pos = 0;
    while (steps_left > 0) {
        bool tile_done = false;
        switch (pos) {
            case 0:
                tile_done = step_at(std::integral_constant<int, 0>{});
                pos = 1;
                if (tile_done || steps_left == 0) break;
                [[fallthrough]];
            case 1:
                tile_done = step_at(std::integral_constant<int, 1>{});
                pos = 2;
                if (tile_done || steps_left == 0) break;
                [[fallthrough]];
            case 2:
                tile_done = step_at(std::integral_constant<int, 2>{});
                pos = 3;
                if (tile_done || steps_left == 0) break;
                [[fallthrough]];
            case 3:
                tile_done = step_at(std::integral_constant<int, 3>{});
                pos = kPeriod == 4 ? 0 : 4;
                if (kPeriod == 4 || tile_done || steps_left == 0) break;
                [[fallthrough]];
            case 4:
                if constexpr (kPeriod == 6) {
                    tile_done = step_at(std::integral_constant<int, 4>{});
                    pos = 5;
                    if (tile_done || steps_left == 0) break;
                }
                [[fallthrough]];
            default:
                if constexpr (kPeriod == 6) {
                    tile_done = step_at(std::integral_constant<int, 5>{});
                    pos = 0;
                }
                break;
        }
        if (tile_done) {
            finish_tile(tile);
            tile += tile_stride;
            tile_steps_left = steps_per_tile;
            x_step = x_lane;
        }
    }
    cp_async_wait<0>();   // nothing of this thread may still be landing in shared memory at exit

    if (kExchange && p.peer_out != nullptr && tid == 0) {
        // The tagged elements need no flag behind them; the last CTA only counts the publication, for this
        // rank's readers (which run after this kernel has completed) and for the next launch.
        const unsigned ctas = gridDim.x * gridDim.y * gridDim.z;
        if (atomicAdd(p.done_counter, 1u) == ctas - 1) {
            *p.done_counter = 0u;
            *p.send_epoch = out_epoch;
        }
    }
    hooks.after_outputs();
}

}  // namespace
}  // namespace w4a16
