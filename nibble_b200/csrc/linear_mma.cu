// Fused W4A16 linear for sm_100a: packed INT4 weights are streamed from HBM, unpacked to exact FP16
// integers with two-instruction-per-pair bit tricks, and fed to the tensor cores as the 16-row
// operand of m16n8k16 MMAs whose 8-wide axis carries the batch.  The group scale multiplies the
// FP32 accumulator once per 128 k, never the individual weights.
//
// Replaces the reference's M=1 decode kernel (csrc/int4_linear_kernel.cu:325-404), its M=2..8
// small-batch kernel (:542-617) and, for larger M, its dequantise-then-cuBLAS route
// (w4a16/linear.py:132-152); one design covers all of them because the work per weight byte is
// independent of M as long as the batch fits the MMA's n axis.
//
// Shape of a launch
//   CTA        : 8 warps = RW row groups x KW warps; the KW warps of a group split the K range of
//                one row tile between them (contiguous sub-ranges), the RW groups own different
//                row tiles.  CTAs are persistent: the grid is what is resident at once and every
//                group strides over the row tiles.
//   row tile   : 16*TILES consecutive output rows.  Row-major [N, K/2] makes a row's K range one
//                contiguous byte run; lane (g, t) owns 16 bytes of rows g and g+8 per 128-wide K
//                chunk, so a quad covers the 64 bytes of one scale group.
//   weights    : each thread keeps a ring of STAGES slots in shared memory, filled with 16-byte
//                cp.async copies of exactly the bytes its own MMAs will consume (plus one 4-byte
//                scale pair per row).  The thread's own cp.async.wait_group is the only
//                synchronisation of the stream, and the bytes in flight per SM are set by the ring
//                depth, not by registers.  Slot addresses are compile-time offsets: the step loop
//                is unrolled over the ring.
//   x          : copied once per CTA into shared memory, already permuted to the (k, k+4) pairing
//                the unpack produces; a warp's B-fragment read is one conflict-free 512-byte row.
//   reduction  : warps of a group combine through shared memory (one named barrier per group and
//                tile); optional K-split CTAs (grid.y) combine through an FP32 workspace, the
//                group that arrives last summing the partials in split order.
//
// The instruction budget is what bounds this kernel on B200: at 6.5 TB/s an SM has about 43 clocks
// per KB of packed weights, lop3/shf/prmt and fma.f16x2 each issue at 2 warp-instructions per clock
// per SM, and the unpack alone needs 40 + 32 of them per KB.  Hence no per-step address arithmetic,
// no register clearing and no register-to-register copies in the step loop.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <map>
#include <mutex>
#include <tuple>
#include <utility>

#include "kernels.h"
#include "linear_mma_body.cuh"
#include "unpack.cuh"

namespace w4a16 {
namespace {

// Hooks of the stand-alone kernel: programmatic dependent launch on the way in, nothing on the way out.
struct KernelHooks {
    // The successor is released with the very first instruction: its CTAs only take SM resources this grid does not
    // use, and the earlier they are resident the more of their prologue and weight prefetch hides under this grid.
    __device__ __forceinline__ void at_start() { pdl_release_downstream(); }
    __device__ __forceinline__ void before_activations() { pdl_wait_for_upstream(); }
    __device__ __forceinline__ void after_outputs() {}
};

template <int NT, int XB, int TILES, int KW, int U, int STAGES>
__global__ void __launch_bounds__(kThreads, min_ctas_per_sm<NT, TILES>())
linear_mma_kernel(const MmaParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    KernelHooks hooks;
    linear_mma_body<NT, XB, TILES, KW, U, STAGES, 0>(p, smem, hooks);
}

// The same kernel with the tensor-parallel sender and reader paths compiled in (launches that carry a
// w4a16_peer_target or a w4a16_peer_source).
template <int NT, int XB, int TILES, int KW, int U, int STAGES>
__global__ void __launch_bounds__(kThreads, min_ctas_per_sm<NT, TILES>())
linear_mma_exchange_kernel(const MmaParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    KernelHooks hooks;
    linear_mma_body<NT, XB, TILES, KW, U, STAGES, kFeatExchange>(p, smem, hooks);
}


// What a kernel needs to be the reader of a sharded layer's publication.
struct ReaderParams {
    const unsigned* epoch;
    unsigned* const* consumed;
    unsigned* staged_counter;
    unsigned* status;
    long long stride;
    long long max_polls;
    long long col0, cols_per_rank;
    int rank, world;
};

// Block-wide: the last block of the grid to get here gives the buffers back to the senders.
__device__ __forceinline__ void reader_release(const ReaderParams& r, unsigned epoch) {
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned blocks = gridDim.x * gridDim.y * gridDim.z;
        if (atomicAdd(r.staged_counter, 1u) == blocks - 1) {
            *r.staged_counter = 0u;
            release_buffers(r.consumed, r.rank, r.world, epoch);
        }
    }
}

// A reader as a kernel of its own: copies `units` groups of eight FP16 values of the publication out of the
// result buffer (tagged elements -> plain FP16), re-reading what has not arrived yet, then releases the buffer.
// `ld` is the row length of the gathered result in elements (names the sender of a missing element).
__global__ void wait_peers_kernel(const ReaderParams r, const uint4* buffer0, uint4* out, long long units, long long ld) {
    pdl_release_downstream();
    pdl_wait_for_upstream();
    const unsigned epoch = __ldcg(r.epoch);
    const unsigned tag = tag_of(epoch);
    const unsigned tag2 = tag | (tag << 16);
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(buffer0) + (epoch & 1u) * r.stride);
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < units;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        Tagged8 t = load_tagged8(src + 2 * i);
        if (!wait_tagged8(src + 2 * i, tag2, r.max_polls, r.status, t)) {
            const long long column = r.col0 + (ld > 0 ? (i * 8) % ld : 0);
            atomicMax(r.status, sender_of(column, r.cols_per_rank, r.world) + 1u);
        }
        out[i] = values_of(t);
    }
    reader_release(r, epoch);
}

// y = half(sum over ranks of partials[rank]), summed in rank order so every rank gets identical bits.
// With a reader description the partials are tagged 64-bit elements of a publication: each is re-read
// (bounded) until it has arrived, and the buffer is released afterwards.
__global__ void sum_partials_kernel(const void* __restrict__ partials, __half* __restrict__ y, long long count,
                                    int world, const ReaderParams r) {
    pdl_release_downstream();
    pdl_wait_for_upstream();
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (r.epoch == nullptr) {
        if (i < count) {
            float sum = 0.f;
            for (int k = 0; k < world; ++k) sum += __ldcg(static_cast<const float*>(partials) + static_cast<long long>(k) * count + i);
            y[i] = __float2half_rn(sum);
        }
        return;
    }
    const unsigned epoch = __ldcg(r.epoch);
    const unsigned long long tag = tag_of(epoch);
    const unsigned long long* src = reinterpret_cast<const unsigned long long*>(
        static_cast<const char*>(partials) + (epoch & 1u) * r.stride);
    if (i < count) {
        float sum = 0.f;
        for (int k0 = 0; k0 < world; k0 += 8) {
            unsigned long long v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (k0 + j < world) {
                    asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v[j]) : "l"(src + static_cast<long long>(k0 + j) * count + i));
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (k0 + j < world) {
                    const unsigned long long* at = src + static_cast<long long>(k0 + j) * count + i;
                    long long poll = 0;
                    while ((v[j] >> 32) != tag && poll++ < r.max_polls) {
                        if ((poll & 255) == 255 && already_failed(r.status)) break;
                        __nanosleep(20);
                        asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v[j]) : "l"(at));
                    }
                    if ((v[j] >> 32) != tag) atomicMax(r.status, static_cast<unsigned>(k0 + j) + 1u);
                    sum += __uint_as_float(static_cast<unsigned>(v[j]));
                }
            }
        }
        y[i] = __float2half_rn(sum);
    }
    reader_release(r, epoch);
}

// ------------------------------------------------------------------------------------------------
struct Variant {
    const void* fn;
    const void* fn_exchange;   // the build with the tensor-parallel paths; null where it is not instantiated
    int red_bytes;     // shared memory for the cross-warp reduction
    int stage_bytes;   // shared memory of one pipeline stage
    int stages;
    int x_rows;        // batch rows stored per chunk of x (XB)
};

template <int NT, int XB, int TILES, int KW, int U, int STAGES>
Variant variant_of() {
    constexpr int RW = kWarpsPerCta / KW;
    constexpr int red = KW > 1 ? 2 * KW * TILES * NT * 4 * 32 * RW * static_cast<int>(sizeof(float)) : 0;
    const void* exchange = nullptr;
    if constexpr (TILES == 1) {   // sharded layers always run one 16-row tile per warp
        exchange = reinterpret_cast<const void*>(&linear_mma_exchange_kernel<NT, XB, TILES, KW, U, STAGES>);
    }
    return {reinterpret_cast<const void*>(&linear_mma_kernel<NT, XB, TILES, KW, U, STAGES>), exchange, red,
            stage_bytes<TILES, U>(), STAGES, XB};
}

template <int NT, int XB, int TILES, int KW>
bool pick_pipeline(int unroll, int stages, Variant* v) {
    if (unroll == 1) {   // odd K/128: the slow-scale path, one tile per warp and one ring depth only
        if constexpr (TILES == 1) {
            if (stages != 3) return false;
            *v = variant_of<NT, XB, 1, KW, 1, 3>();
            return true;
        } else {
            return false;
        }
    }
    if (unroll != 2) return false;
    if (stages == 3) { *v = variant_of<NT, XB, TILES, KW, 2, 3>(); return true; }
    if (stages == 4) { *v = variant_of<NT, XB, TILES, KW, 2, 4>(); return true; }
    return false;
}

template <int NT, int XB, int TILES>
bool pick_kw(int kw, int unroll, int stages, Variant* v) {
    switch (kw) {
        case 1: return pick_pipeline<NT, XB, TILES, 1>(unroll, stages, v);
        case 2: return pick_pipeline<NT, XB, TILES, 2>(unroll, stages, v);
        case 4: return pick_pipeline<NT, XB, TILES, 4>(unroll, stages, v);
        case 8: return pick_pipeline<NT, XB, TILES, 8>(unroll, stages, v);
        default: return false;
    }
}

template <int NT, int XB>
bool pick_tiles(const w4a16_linear_config& c, Variant* v) {
    switch (c.row_tiles) {
        case 1: return pick_kw<NT, XB, 1>(c.k_warps, c.unroll, c.stages, v);
        case 2:
            if constexpr (NT <= 2) {
                return pick_kw<NT, XB, 2>(c.k_warps, c.unroll, c.stages, v);
            } else {
                return false;
            }
        default: return false;
    }
}

bool pick_variant(int nt, bool single_row, const w4a16_linear_config& c, Variant* v) {
    switch (nt) {
        case 1: return single_row ? pick_tiles<1, 1>(c, v) : pick_tiles<1, 8>(c, v);
        case 2: return pick_tiles<2, 16>(c, v);
        case 4: return pick_tiles<4, 32>(c, v);
        default: return false;
    }
}

int batch_tiles_for(int64_t M) { return M <= 8 ? 1 : (M <= 16 ? 2 : 4); }
int x_rows_for(int64_t M) { return M == 1 ? 1 : 8 * batch_tiles_for(M); }

constexpr int kMaxDevices = 64;

// SM count of `device`, looked up once per device.
int sm_count(int device) {
    static std::atomic<int> cached[kMaxDevices] = {};
    if (device < 0 || device >= kMaxDevices) return 148;
    int count = cached[device].load(std::memory_order_relaxed);
    if (count == 0) {
        if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0) return 148;
        cached[device].store(count, std::memory_order_relaxed);
    }
    return count;
}

// Bytes of x a CTA holds for `rows` stored batch rows of a K slice of `chunks` chunks.
size_t x_slice_bytes(int rows, int chunks) { return static_cast<size_t>(rows) * chunks * kGroup * sizeof(__half); }

}  // namespace

// The arrival counters occupy a prefix of the workspace whose size does not depend on the problem (as long as
// the problem has at most kCounterSlots row-tile x batch-block pairs): one workspace may then serve calls of
// different shapes one after the other, because the FP32 partial sums of one call can never land where another
// call keeps its counters (they used to, when the prefix was sized per problem: leftover partials of an N = 2048
// call sat in the counter slots of tiles 128.. of a following N = 2560 call, whose last arriver was then never
// recognised and whose outputs were never written).
constexpr int64_t kCounterSlots = 65536;

size_t linear_counter_bytes(int64_t M, int64_t N) {
    const int64_t row_blocks = (N + 15) / 16;
    const int64_t batch_blocks = (M + 7) / 8;
    const int64_t slots = std::max<int64_t>(row_blocks * batch_blocks, kCounterSlots);
    const size_t bytes = static_cast<size_t>(slots) * sizeof(unsigned);
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
    const int x_rows = x_rows_for(M);
    const int64_t batch_blocks = (M + 8 * nt - 1) / (8 * nt);
    const int chunks = static_cast<int>(K / kGroup);
    const int64_t tiles16 = (N + 15) / 16;

    c.row_tiles = 1;
    c.unroll = chunks % 2 == 0 ? 2 : 1;
    // Warps of a CTA that share one row tile: the fewest that still give about 12 streaming warps
    // per SM (more only shortens each warp's share of a tile and multiplies the per-tile epilogue).
    const int64_t want_warps = static_cast<int64_t>(sms) * 12;
    int kw = 1;
    while (kw < 8 && tiles16 * batch_blocks * kw < want_warps && chunks >= kw * 2 * c.unroll) kw *= 2;
    // Single-row launches with at most ~3 row tiles per resident CTA: all eight warps on each tile.  In a
    // chain of dependent layers the whole share of a CTA is then prefetched before its activations
    // arrive, and what remains after the wait is at most three short steps per warp instead of four
    // (measured inside a decode step: 2 us per launch on the fused gate/up layer; within 2 % either
    // way for independent launches).
    if (M == 1 && tiles16 <= 1024) {
        while (kw < 8 && chunks >= kw * 2 * c.unroll) kw *= 2;
    }
    // Shapes measured on B200 where a different split of the same work is clearly faster (sweeps over
    // every k_warps x k_splits combination; Llama-70B gate/up and down projections).
    struct Tuned { int64_t n, k; int k_warps, k_splits; };
    static const Tuned tuned[] = {
        {28672, 8192, 8, 1},   // 1792 row tiles: eight warps per tile halve the quarter-full last wave
        {8192, 28672, 1, 4},   // long K: split across CTAs so the activation slice stays small
    };
    int tuned_splits = 0;
    if (M <= 8) {
        for (const Tuned& entry : tuned) {
            if (entry.n == N && entry.k == K && entry.k_splits <= max_splits) {
                kw = entry.k_warps;
                tuned_splits = entry.k_splits;
            }
        }
    }
    c.k_warps = kw;
    // Splitting K across CTAs costs a round trip through the workspace; do it when the row tiles
    // alone cannot fill the machine ...
    int splits = tuned_splits > 0 ? tuned_splits : 1;
    if (M <= 32 && tuned_splits == 0) {
        while (splits * 2 <= max_splits && splits * 2 <= kMaxKSplits &&
               tiles16 * batch_blocks * kw * splits < want_warps && chunks >= splits * 2 * kw * 2 * c.unroll) {
            splits *= 2;
        }
    }
    // ... or, for the single-row case, when the activation slice would crowd the copy ring out of
    // shared memory (two CTAs per SM want it at or below 32 KB) ...
    if (M == 1 && tuned_splits == 0) {
        while (x_slice_bytes(x_rows, (chunks + splits - 1) / splits) > 32u * 1024 && splits * 2 <= max_splits &&
               splits * 2 <= kMaxKSplits && chunks >= splits * 2 * kw * c.unroll) {
            splits *= 2;
        }
    }
    // ... and always when the slice would not fit next to a three-slot ring at all.
    while (x_slice_bytes(x_rows, (chunks + splits - 1) / splits) > static_cast<size_t>(kSmemBudget - 64 * 1024) &&
           splits * 2 <= max_splits && splits * 2 <= kMaxKSplits && chunks >= splits * 2) {
        splits *= 2;
    }
    c.k_splits = splits;
    c.stages = 0;   // chosen at launch from the shared memory left over
    return c;
}

namespace {

int reader_params(const w4a16_peer_source* source, ReaderParams* r) {
    *r = ReaderParams{};
    if (source == nullptr) return W4A16_OK;
    if (source->epoch == nullptr || source->consumed == nullptr || source->staged_counter == nullptr ||
        source->status == nullptr) {
        return W4A16_ERR_NULL_POINTER;
    }
    if (source->world < 1 || source->world > 32 || source->rank < 0 || source->rank >= source->world ||
        source->max_polls <= 0 || source->buffer_stride < 0 || source->first_column < 0 || source->columns_per_rank < 0) {
        return W4A16_ERR_BAD_SHAPE;
    }
    *r = ReaderParams{source->epoch, source->consumed, source->staged_counter, source->status, source->buffer_stride,
                      source->max_polls, source->first_column, source->columns_per_rank, source->rank, source->world};
    return W4A16_OK;
}

template <typename Kernel, typename... Args>
int launch_small(Kernel kernel, unsigned blocks, unsigned threads, bool programmatic, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t launch = {};
    launch.gridDim = dim3(blocks, 1, 1);
    launch.blockDim = dim3(threads, 1, 1);
    launch.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    launch.attrs = attr;
    launch.numAttrs = programmatic ? 1 : 0;
    if (cudaLaunchKernelEx(&launch, kernel, args...) != cudaSuccess) return W4A16_ERR_LAUNCH;
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    return W4A16_OK;
}

}  // namespace

int launch_wait_peers(const w4a16_peer_source* source, const void* buffer0, void* out, int64_t count, int64_t ld,
                      bool programmatic, cudaStream_t stream) {
    if (source == nullptr) return W4A16_ERR_NULL_POINTER;
    ReaderParams r;
    const int status = reader_params(source, &r);
    if (status != W4A16_OK) return status;
    if (count < 0 || count % 8 != 0) return W4A16_ERR_BAD_SHAPE;
    if (count > 0) {
        if (buffer0 == nullptr || out == nullptr) return W4A16_ERR_NULL_POINTER;
        if (reinterpret_cast<uintptr_t>(buffer0) % 32 != 0 || reinterpret_cast<uintptr_t>(out) % 16 != 0 ||
            source->buffer_stride % 32 != 0) {
            return W4A16_ERR_MISALIGNED;
        }
    }
    const long long units = count / 8;
    const unsigned blocks = static_cast<unsigned>(std::min<long long>(64, std::max<long long>(1, (units + 255) / 256)));
    return launch_small(wait_peers_kernel, blocks, 256, programmatic, stream, r, static_cast<const uint4*>(buffer0),
                        static_cast<uint4*>(out), units, static_cast<long long>(ld));
}

int launch_sum_partials(const void* partials, __half* y, int64_t count, int world, const w4a16_peer_source* source,
                        bool programmatic, cudaStream_t stream) {
    if (count <= 0) return W4A16_OK;
    ReaderParams r;
    const int status = reader_params(source, &r);
    if (status != W4A16_OK) return status;
    if (source != nullptr && (reinterpret_cast<uintptr_t>(partials) % 8 != 0 || source->buffer_stride % 8 != 0)) {
        return W4A16_ERR_MISALIGNED;
    }
    const int threads = 256;
    const int64_t blocks = (count + threads - 1) / threads;
    if (blocks > INT32_MAX) return W4A16_ERR_TOO_LARGE;
    return launch_small(sum_partials_kernel, static_cast<unsigned>(blocks), threads, programmatic, stream, partials, y,
                        static_cast<long long>(count), world, r);
}

// Reads and clears the bounds-check word of the streaming kernel (builds with -DW4A16_BOUNDS_CHECK only).
int read_bounds_check(unsigned* site, unsigned* count) {
#ifdef W4A16_BOUNDS_CHECK
    unsigned word[2] = {0u, 0u};
    const unsigned zero[2] = {0u, 0u};
    if (cudaMemcpyFromSymbol(word, g_bounds_word, sizeof(word)) != cudaSuccess ||
        cudaMemcpyToSymbol(g_bounds_word, zero, sizeof(zero)) != cudaSuccess) {
        return W4A16_ERR_LAUNCH;
    }
    *site = word[0];
    *count = word[1];
    return W4A16_OK;
#else
    *site = 0u;
    *count = 0u;
    return W4A16_ERR_BAD_CONFIG;
#endif
}

int launch_linear_mma(const LinearProblem& prob, const w4a16_linear_config& cfg_in, bool programmatic,
                      bool out_f32, cudaStream_t stream) {
    if (prob.group != kGroup || prob.K % kGroup != 0) return W4A16_ERR_BAD_CONFIG;
    if (prob.M > INT32_MAX || prob.N > INT32_MAX || prob.K > INT32_MAX) return W4A16_ERR_TOO_LARGE;
    w4a16_linear_config cfg = cfg_in;
    const int nt = batch_tiles_for(prob.M);
    const int x_rows = x_rows_for(prob.M);
    const int chunks = static_cast<int>(prob.K / kGroup);
    const int splits = cfg.k_splits;
    if (splits < 1 || splits > kMaxKSplits || splits > chunks) return W4A16_ERR_BAD_CONFIG;
    // With unroll 2 the two scales of a step travel as one 4-byte copy: that needs K/128 even and
    // the scale matrix 4-byte aligned.
    if (cfg.unroll == 2 && (chunks % 2 != 0 || reinterpret_cast<uintptr_t>(prob.scales) % 4 != 0)) {
        return W4A16_ERR_BAD_CONFIG;
    }
    if (cfg.unroll != 1 && cfg.unroll != 2) return W4A16_ERR_BAD_CONFIG;
    if (cfg.stages != 0 && cfg.stages != 3 && cfg.stages != 4) return W4A16_ERR_BAD_CONFIG;

    const int per_split = (chunks + splits - 1) / splits;
    const int chunks_per_split = (per_split + cfg.unroll - 1) / cfg.unroll * cfg.unroll;
    if ((splits - 1) * chunks_per_split >= chunks) return W4A16_ERR_BAD_CONFIG;   // an empty split

    // Ring depth: four slots when two CTAs still fit on an SM with them; else three if that is what lets two CTAs fit;
    // and when the activation slice is so large that only one CTA fits either way, four again (as many bytes in flight
    // as the budget allows, and the step loop is unrolled over 4 positions instead of 6: with eight warps per SM the
    // longer loop showed up as instruction-fetch stalls, `no_instruction` 1.26 per issue at M = 8 on 8192-wide layers).
    Variant variant;
    if (cfg.stages == 0) {
        cfg.stages = cfg.unroll == 1 ? 3 : 4;
        if (cfg.unroll == 2) {
            if (!pick_variant(nt, prob.M == 1, cfg, &variant)) return W4A16_ERR_BAD_CONFIG;
            const size_t fixed = kFlagBytes + variant.red_bytes + x_slice_bytes(x_rows, chunks_per_split);
            const size_t half_sm = static_cast<size_t>(kSmemPerSm / 2 - 1024);
            const bool two_with_four = fixed + 4u * variant.stage_bytes <= half_sm;
            const bool two_with_three = fixed + 3u * variant.stage_bytes <= half_sm;
            const bool four_fit = fixed + 4u * variant.stage_bytes <= static_cast<size_t>(kSmemBudget);
            if (!two_with_four && (two_with_three || !four_fit)) cfg.stages = 3;
        }
    }
    if (!pick_variant(nt, prob.M == 1, cfg, &variant)) return W4A16_ERR_BAD_CONFIG;

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
    params.chunks_per_split = chunks_per_split;
    params.k_splits = splits;
    params.row_tiles_total = static_cast<int>((prob.N + 16 * cfg.row_tiles - 1) / (16 * cfg.row_tiles));
    params.out_f32 = out_f32 ? 1 : 0;
    params.peer_out = nullptr;
    params.done_counter = nullptr;
    params.send_epoch = nullptr;
    params.peer_status = nullptr;
    params.wait_polls = 0;
    params.ld_out = 0;
    params.col_out = 0;
    params.rank = 0;
    params.world = 1;
    params.x_mode = W4A16_INPUT_PLAIN;
    params.x_ld = prob.K;
    params.x_row_index = nullptr;
    params.x_second = nullptr;
    params.norm_weight = nullptr;
    params.stream_out = nullptr;
    params.eps = 0.0f;
    if (prob.input != nullptr && prob.input->kind != W4A16_INPUT_PLAIN) {
        const w4a16_input_transform& in = *prob.input;
        auto aligned = [](const void* q) { return reinterpret_cast<uintptr_t>(q) % 16 == 0; };
        if (in.kind == W4A16_INPUT_SILU_MUL) {
            params.x_ld = 2 * prob.K;
        } else if (in.kind == W4A16_INPUT_ADD_RMSNORM) {
            if (prob.M != 1) return W4A16_ERR_BAD_SHAPE;
            if (in.norm_weight == nullptr) return W4A16_ERR_NULL_POINTER;
            if (!aligned(in.second) || !aligned(in.norm_weight) || !aligned(in.stream_out)) return W4A16_ERR_MISALIGNED;
            if (in.stream_out != nullptr && (in.stream_out == prob.x || in.stream_out == in.second)) return W4A16_ERR_BAD_CONFIG;
            params.x_second = static_cast<const __half*>(in.second);
            params.norm_weight = static_cast<const __half*>(in.norm_weight);
            params.stream_out = static_cast<__half*>(in.stream_out);
            params.eps = in.eps;
        } else {
            return W4A16_ERR_BAD_CONFIG;
        }
        params.x_mode = in.kind;
    }
    params.consumed = nullptr;
    params.out_stride = 0;
    params.src_epoch = nullptr;
    params.src_consumed = nullptr;
    params.src_col0 = 0;
    params.src_cols_per_rank = 0;
    params.staged_counter = nullptr;
    params.src_stride = 0;
    if (prob.x_ld != 0) {
        if (prob.x_ld < prob.K || prob.x_ld % 8 != 0 || params.x_mode != W4A16_INPUT_PLAIN) return W4A16_ERR_BAD_SHAPE;
        params.x_ld = prob.x_ld;
    }
    if (prob.peers != nullptr) {
        const w4a16_peer_target& t = *prob.peers;
        if (t.outputs == nullptr || t.consumed == nullptr || t.done_counter == nullptr ||
            t.send_epoch == nullptr || t.status == nullptr) {
            return W4A16_ERR_NULL_POINTER;
        }
        if (t.world < 1 || t.world > 32 || t.rank < 0 || t.rank >= t.world || t.ld < prob.N || t.column_offset < 0 ||
            t.max_polls <= 0 || t.buffer_stride < 0) {
            return W4A16_ERR_BAD_SHAPE;
        }
        params.peer_out = t.outputs;
        params.consumed = t.consumed;
        params.done_counter = t.done_counter;
        params.send_epoch = t.send_epoch;
        params.peer_status = t.status;
        params.out_stride = t.buffer_stride;
        params.wait_polls = t.max_polls;
        params.ld_out = t.ld;
        params.col_out = t.column_offset;
        params.rank = t.rank;
        params.world = t.world;
    }
    if (prob.source != nullptr) {
        ReaderParams r;
        const int status = reader_params(prob.source, &r);
        if (status != W4A16_OK) return status;
        // tagged elements are 4 bytes each and are read 32 bytes at a time
        if (params.x_mode != W4A16_INPUT_PLAIN || r.stride % 32 != 0 || reinterpret_cast<uintptr_t>(prob.x) % 32 != 0) {
            return W4A16_ERR_BAD_CONFIG;
        }
        if (prob.peers != nullptr && (prob.peers->world != r.world || prob.peers->rank != r.rank)) return W4A16_ERR_BAD_SHAPE;
        params.src_epoch = r.epoch;
        params.src_col0 = r.col0;
        params.src_cols_per_rank = r.cols_per_rank;
        params.src_consumed = r.consumed;
        params.staged_counter = r.staged_counter;
        params.src_stride = r.stride;
        params.rank = r.rank;
        params.world = r.world;
        if (params.peer_status == nullptr) params.peer_status = r.status;
        if (params.wait_polls == 0) params.wait_polls = r.max_polls;
    }
    if (splits > 1) {
        const size_t need = linear_workspace_bytes_for(prob.M, prob.N, splits);
        if (prob.workspace == nullptr || prob.workspace_bytes < need) return W4A16_ERR_WORKSPACE;
        if (reinterpret_cast<uintptr_t>(prob.workspace) % 16 != 0) return W4A16_ERR_MISALIGNED;
        params.counters = static_cast<unsigned*>(prob.workspace);
        params.partial = reinterpret_cast<float*>(static_cast<char*>(prob.workspace) +
                                                  linear_counter_bytes(prob.M, prob.N));
    }

    const size_t smem = kFlagBytes + static_cast<size_t>(variant.red_bytes) + x_slice_bytes(x_rows, chunks_per_split) +
                        static_cast<size_t>(variant.stages) * variant.stage_bytes;
    if (smem > static_cast<size_t>(kSmemBudget)) return W4A16_ERR_WORKSPACE;   // x slice too large: more K splits

    // Opt in to large dynamic shared memory once per device and kernel variant (the attribute belongs to
    // the function as loaded on one device), and learn its occupancy there (cached per device, variant
    // and shared-memory size).
    const void* kernel = variant.fn;
    if (prob.peers != nullptr || prob.source != nullptr) {
        if (variant.fn_exchange == nullptr) return W4A16_ERR_BAD_CONFIG;
        kernel = variant.fn_exchange;
    }
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return W4A16_ERR_LAUNCH;
    static std::mutex mutex;
    static std::map<std::tuple<int, const void*, size_t>, int> occupancy;
    int blocks_per_sm = 0;
    {
        std::lock_guard<std::mutex> lock(mutex);
        const auto key = std::make_tuple(device, kernel, smem);
        const auto found = occupancy.find(key);
        if (found != occupancy.end()) {
            blocks_per_sm = found->second;
        } else {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget) !=
                cudaSuccess) {
                return W4A16_ERR_LAUNCH;
            }
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks_per_sm, kernel, kThreads, smem) !=
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
    int64_t resident = static_cast<int64_t>(sm_count(device)) * blocks_per_sm / (splits * batch_blocks);
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
    if (cudaLaunchKernelExC(&launch, kernel, args) != cudaSuccess) return W4A16_ERR_LAUNCH;
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    return W4A16_OK;
}

}  // namespace w4a16
