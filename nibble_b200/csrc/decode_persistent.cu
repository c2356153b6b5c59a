// One LLaMA decode step (batch 1) as ONE cooperative kernel launch: the CTAs stay resident for the whole
// token and walk a device-side list of operations -- per decoder block the fused q/k/v linear (with the
// residual add + RMSNorm computed while its activations are staged), attention (RoPE, cache append, softmax,
// values), o_proj, the fused gate/up linear (add + RMSNorm inside), down_proj (SiLU * up inside); then lm_head
// (final norm inside) and the arg-max that advances the token and the position.
//
// Replaces, for the decode step, the chain of ~5 launches per block of the graph-replayed runner and, before
// it, what the reference gets from HuggingFace's generate() (scripts/generate.py:260-365).  A dependent launch
// costs about 2 us even with programmatic launch; a grid-wide hand-off through one L2 counter costs well under
// that, and the next operation's weight ring is requested BEFORE the hand-off is waited for, so weight
// streaming never stops at an operation boundary.
//
// Hand-off between operations: every CTA adds 1 to a global counter when it has finished its part of an
// operation (after a __threadfence); an operation that consumes the result waits until the counter has reached
// (operations so far) x (CTAs).  The launch is cooperative, so all CTAs are resident and the wait always ends;
// it is bounded all the same: after kBarrierSpinLimit polls it records the operation's index in the status word
// and goes on, so that a logic error ends in a wrong token and a reported status, never in a hung GPU.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <vector>

#include "kernels.h"
#include "linear_mma_body.cuh"
#include "unpack.cuh"

namespace w4a16 {
namespace {

constexpr unsigned kBarrierSpinLimit = 1u << 22;   // polls of one L2 round trip each: a few seconds
constexpr int kStepKW = 8;          // all eight warps of a CTA share one 16-row tile
constexpr int kStepStages = 4;

enum : int { kOpLinear = 0, kOpAttention = 1, kOpArgmax = 2 };

struct AttentionOp {
    const __half* qkv;
    __half* k_cache;
    __half* v_cache;
    __half* out;
    const long long* position;
    const float* inv_freq;
    int q_heads, kv_heads, max_len;
    float rope_scale, softmax_scale;
};

struct ArgmaxOp {
    const __half* logits;
    int count;
    long long* token;
    long long* position;
    unsigned* step_count;
};

struct DecodeOp {
    int kind;
    MmaParams linear;
    AttentionOp attention;
    ArgmaxOp argmax;
};

struct StepParams {
    const DecodeOp* ops;
    int n_ops;
    unsigned* counter;          // arrivals of all CTAs at all operations, since the plan was built
    const unsigned* step_count; // steps run so far with this plan
    unsigned* status;           // 0 healthy; 1 position outside the cache; 0x100 + op: a hand-off wait gave up
};

// Grid-wide hand-off through one counter (see the head of the file).
struct GridSync {
    unsigned* counter;
    unsigned* status;
    unsigned base;        // counter value when this step started
    unsigned ctas;
    unsigned op;          // index of the operation being run

    // This CTA has finished its part of operation `op` (call with all threads).
    __device__ __forceinline__ void arrive() {
        __syncthreads();
        if (threadIdx.x == 0) {
            // release at GPU scope: orders this CTA's writes (made visible to this thread by the barrier above)
            asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
        }
    }
    // Everything before operation `op` is complete and visible (call with all threads).
    __device__ __forceinline__ void wait_for_previous() {
        if (op > 0 && threadIdx.x == 0) {
            const unsigned target = base + op * ctas;
            bool done = false;
            for (unsigned spin = 0; spin < kBarrierSpinLimit; ++spin) {
                unsigned seen;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
                if (static_cast<int>(seen - target) >= 0) {
                    done = true;
                    break;
                }
            }
            if (!done) atomicMax(status, 0x100u + op);
            __threadfence();   // nothing read below may come from a line this SM cached before the hand-off
        }
        __syncthreads();
    }
};

// Hooks that make the streaming linear one operation of the step: its weight ring is requested first, then
// the previous operation is waited for, and its end is announced to the next one.
struct StepHooks {
    GridSync& sync;
    __device__ __forceinline__ void at_start() {}
    __device__ __forceinline__ void before_activations() { sync.wait_for_previous(); }
    __device__ __forceinline__ void after_outputs() { sync.arrive(); }
};

__device__ __forceinline__ float cta_sum(float v, float* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.0f;
    for (int w = 0; w < kWarpsPerCta; ++w) total += scratch[w];
    return total;
}
__device__ __forceinline__ float cta_max(float v, float* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float best = scratch[0];
    for (int w = 1; w < kWarpsPerCta; ++w) best = fmaxf(best, scratch[w]);
    return best;
}

// Attention of one query head by one CTA of 256 threads (same arithmetic and roundings as
// attention_decode_kernel in decode_ops.cu: RoPE with FP16 cos/sin and uncontracted FP16 products, FP32
// scores and softmax, FP32 accumulation of the values).  D/8 consecutive lanes share a cached position.
// Shared memory (all inside `smem`): scores[max_len] floats, then the fixed part below.
template <int D>
__device__ __forceinline__ void attention_head(const AttentionOp& p, int head, unsigned char* smem, unsigned* status,
                                               GridSync& sync) {
    constexpr int kLanesPerPos = D / 8;
    constexpr int kPosPerPass = kThreads / kLanesPerPos;
    constexpr int half_d = D / 2;
    float* scores = reinterpret_cast<float*>(smem);
    float* scratch = scores + ((p.max_len + 3) & ~3);          // [8]
    float* q = scratch + 8;                                     // [D]
    float* partial = q + D;                                     // [kPosPerPass][D]
    __half* k_new = reinterpret_cast<__half*>(partial + kPosPerPass * D);   // [D], 16-byte aligned
    __half* v_new = k_new + D;
    const int tid = threadIdx.x;
    const int kv_head = head / (p.q_heads / p.kv_heads);
    const int sub = tid % kLanesPerPos;
    const int slot = tid / kLanesPerPos;
    const uint4* k_rows = reinterpret_cast<const uint4*>(p.k_cache + static_cast<size_t>(kv_head) * p.max_len * D) + sub;
    const uint4* v_rows = reinterpret_cast<const uint4*>(p.v_cache + static_cast<size_t>(kv_head) * p.max_len * D) + sub;
    // Nothing requested here depends on the operation before this one (it produces qkv): the position only moves
    // at the end of a step and the older cache rows were written by earlier steps.  So the first pass of K and V
    // rows is requested before the hand-off is waited for; rows at or past the position are fetched (inside the
    // cache) and never used.
    const long long pos = __ldcg(p.position);
    const int early_t = min(slot, p.max_len - 1);
    const uint4 k_early = __ldcg(k_rows + static_cast<size_t>(early_t) * kLanesPerPos);
    const uint4 v_early = __ldcg(v_rows + static_cast<size_t>(early_t) * kLanesPerPos);
    sync.wait_for_previous();
    if (pos < 0 || pos >= p.max_len) {
        if (tid == 0) atomicMax(status, 1u);
        return;
    }
    const __half* q_in = p.qkv + head * D;
    const __half* k_in = p.qkv + p.q_heads * D + kv_head * D;
    const __half* v_in = p.qkv + (p.q_heads + p.kv_heads) * D + kv_head * D;
    if (tid < D) {
        const int i = tid;
        const float angle = static_cast<float>(pos) * p.inv_freq[i % half_d];
        float sn, cs;
        sincosf(angle, &sn, &cs);
        const __half c = __float2half_rn(cs * p.rope_scale);
        const __half s = __float2half_rn(sn * p.rope_scale);
        const __half qv = __ldcg(q_in + i), kv = __ldcg(k_in + i);
        const __half q_rot = i < half_d ? __hneg(__ldcg(q_in + i + half_d)) : __ldcg(q_in + i - half_d);
        const __half k_rot = i < half_d ? __hneg(__ldcg(k_in + i + half_d)) : __ldcg(k_in + i - half_d);
        q[i] = __half2float(__hadd_rn(__hmul_rn(qv, c), __hmul_rn(q_rot, s)));
        const __half k_val = __hadd_rn(__hmul_rn(kv, c), __hmul_rn(k_rot, s));
        const __half v_val = __ldcg(v_in + i);
        k_new[i] = k_val;
        v_new[i] = v_val;
        if (head % (p.q_heads / p.kv_heads) == 0) {   // one CTA per KV head appends to the cache
            p.k_cache[(static_cast<size_t>(kv_head) * p.max_len + pos) * D + i] = k_val;
            p.v_cache[(static_cast<size_t>(kv_head) * p.max_len + pos) * D + i] = v_val;
        }
    }
    __syncthreads();

    const int length = static_cast<int>(pos) + 1;
    // The newest position comes from shared memory, not from the cache: another CTA writes it there.
    auto row_piece = [&](const uint4* rows, const __half* newest, const uint4& early, int t) {
        if (t == length - 1) return reinterpret_cast<const uint4*>(newest)[sub];
        if (t < kPosPerPass) return early;
        return __ldcg(rows + static_cast<size_t>(t) * kLanesPerPos);
    };
    float qf[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) qf[i] = q[sub * 8 + i];

    float local_max = -INFINITY;
#pragma unroll 2
    for (int base = 0; base < length; base += kPosPerPass) {
        const int t = base + slot;
        float dot = 0.0f;
        if (t < length) {
            const uint4 piece = row_piece(k_rows, k_new, k_early, t);
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
    const float top = cta_max(local_max, scratch);   // its barriers also publish the scores
    float local_sum = 0.0f;
    for (int t = tid; t < length; t += kThreads) {
        const float e = expf(scores[t] - top);
        scores[t] = e;
        local_sum += e;
    }
    const float denom = cta_sum(local_sum, scratch);

    float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 2
    for (int base = 0; base < length; base += kPosPerPass) {
        const int t = base + slot;
        if (t < length) {
            const float w = scores[t];
            const uint4 piece = row_piece(v_rows, v_new, v_early, t);
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
    for (int i = 0; i < 8; ++i) partial[slot * D + sub * 8 + i] = acc[i];
    __syncthreads();
    if (tid < D) {
        float total = 0.0f;
#pragma unroll 4
        for (int g = 0; g < kPosPerPass; ++g) total += partial[g * D + tid];
        p.out[head * D + tid] = __float2half_rn(total / denom);
    }
}

// token = index of the first largest logit; position and the step count move on by one.  One CTA.
__device__ __forceinline__ void argmax_advance(const ArgmaxOp& p, unsigned char* smem) {
    float* best_value = reinterpret_cast<float*>(smem);            // [8]
    int* best_index = reinterpret_cast<int*>(best_value + 8);      // [8]
    float value = -INFINITY;
    int index = 0x7fffffff;
    auto merge = [&](float other_value, int other_index) {
        if (other_value > value || (other_value == value && other_index < index)) { value = other_value; index = other_index; }
    };
    for (int i = threadIdx.x * 8; i < p.count; i += kThreads * 8) {
        if (i + 8 <= p.count && (reinterpret_cast<uintptr_t>(p.logits + i) & 15) == 0) {
            const uint4 q = __ldcg(reinterpret_cast<const uint4*>(p.logits + i));
            const __half2* h = reinterpret_cast<const __half2*>(&q);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(h[j]);
                if (f.x > value) { value = f.x; index = i + 2 * j; }
                if (f.y > value) { value = f.y; index = i + 2 * j + 1; }
            }
        } else {
            for (int j = i; j < min(i + 8, p.count); ++j) {
                const float f = __half2float(__ldcg(p.logits + j));
                if (f > value) { value = f; index = j; }
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) merge(__shfl_xor_sync(0xffffffffu, value, o), __shfl_xor_sync(0xffffffffu, index, o));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) { best_value[warp] = value; best_index[warp] = index; }
    __syncthreads();
    if (warp == 0) {
        value = lane < kWarpsPerCta ? best_value[lane] : -INFINITY;
        index = lane < kWarpsPerCta ? best_index[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) merge(__shfl_xor_sync(0xffffffffu, value, o), __shfl_xor_sync(0xffffffffu, index, o));
        if (lane == 0) {
            *p.token = index == 0x7fffffff ? 0 : index;
            *p.position += 1;
            *p.step_count += 1u;
        }
    }
}

__global__ void __launch_bounds__(kThreads, 2)
decode_step_kernel(const StepParams s, const int head_dim) {
    extern __shared__ __align__(128) unsigned char smem[];
    const unsigned ctas = gridDim.x;
    // the step count only changes at the very end of a step (by the arg-max), so every CTA reads the same value
    GridSync sync{s.counter, s.status, __ldcg(s.step_count) * static_cast<unsigned>(s.n_ops) * ctas, ctas, 0u};
    for (int i = 0; i < s.n_ops; ++i) {
        sync.op = static_cast<unsigned>(i);
        const int kind = s.ops[i].kind;
        if (kind == kOpLinear) {
            const MmaParams p = s.ops[i].linear;
            StepHooks hooks{sync};
            linear_mma_body<1, 1, 1, kStepKW, 2, kStepStages, kFeatRowIndex>(p, smem, hooks);
        } else if (kind == kOpAttention) {
            const AttentionOp p = s.ops[i].attention;
            if (static_cast<int>(blockIdx.x) < p.q_heads) {
                if (head_dim == 64) {
                    attention_head<64>(p, blockIdx.x, smem, s.status, sync);
                } else {
                    attention_head<128>(p, blockIdx.x, smem, s.status, sync);
                }
            } else {
                // A CTA without a head still waits: the counter only means "operation i - 1 is complete" while no
                // CTA arrives at operation i before it has seen that itself.
                sync.wait_for_previous();
            }
            sync.arrive();
        } else {
            sync.wait_for_previous();
            if (blockIdx.x == 0) argmax_advance(s.ops[i].argmax, smem);
            sync.arrive();
        }
    }
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------
// Host side: the plan (operation list + work buffers, all inside one caller-owned device allocation).
namespace {

constexpr size_t kPlanAlign = 256;
size_t aligned(size_t bytes) { return (bytes + kPlanAlign - 1) / kPlanAlign * kPlanAlign; }

struct PlanLayout {
    size_t header, ops, stream_a, stream_b, qkv, attn, o, gate_up, down, logits, total;
    int n_ops;
};

// The first 256 bytes of a plan.
struct PlanHeader {
    unsigned counter;
    unsigned step_count;
    unsigned status;
    int n_ops;
    int grid;
    int head_dim;
    unsigned smem_bytes;
    unsigned magic;
};
constexpr unsigned kPlanMagic = 0x57344450u;

bool layout_of(const w4a16_decode_model& m, PlanLayout* out) {
    if (m.layers <= 0 || m.hidden <= 0 || m.q_heads <= 0 || m.kv_heads <= 0 || m.q_heads % m.kv_heads != 0 ||
        (m.head_dim != 64 && m.head_dim != 128) || m.intermediate <= 0 || m.vocab <= 0 || m.max_len <= 0) {
        return false;
    }
    // every linear runs the 128-wide-group kernel two chunks per step
    if (m.hidden % 256 != 0 || m.intermediate % 256 != 0 || (m.q_heads * m.head_dim) % 256 != 0) return false;
    PlanLayout l{};
    l.n_ops = 5 * m.layers + 2;
    size_t at = 0;
    auto take = [&](size_t bytes) { const size_t here = at; at += aligned(bytes); return here; };
    l.header = take(sizeof(PlanHeader));
    l.ops = take(sizeof(DecodeOp) * l.n_ops);
    l.stream_a = take(2 * static_cast<size_t>(m.hidden));
    l.stream_b = take(2 * static_cast<size_t>(m.hidden));
    l.qkv = take(2 * static_cast<size_t>(m.q_heads + 2 * m.kv_heads) * m.head_dim);
    l.attn = take(2 * static_cast<size_t>(m.q_heads) * m.head_dim);
    l.o = take(2 * static_cast<size_t>(m.hidden));
    l.gate_up = take(4 * static_cast<size_t>(m.intermediate));
    l.down = take(2 * static_cast<size_t>(m.hidden));
    l.logits = take(2 * static_cast<size_t>(m.vocab));
    l.total = at;
    *out = l;
    return true;
}

// Parameters of one M = 1 linear in the step's launch shape (one 16-row tile per CTA pass, eight warps across K).
MmaParams step_linear(const void* x, const void* packed, const void* scales, void* y, int n, int k) {
    MmaParams p{};
    p.x = static_cast<const __half*>(x);
    p.packed = static_cast<const uint8_t*>(packed);
    p.scales = static_cast<const __half*>(scales);
    p.y = y;
    p.M = 1;
    p.N = n;
    p.K = k;
    p.chunks = k / kGroup;
    p.chunks_per_split = p.chunks;
    p.k_splits = 1;
    p.row_tiles_total = (n + 15) / 16;
    p.world = 1;
    p.x_mode = W4A16_INPUT_PLAIN;
    p.x_ld = k;
    return p;
}

size_t step_smem_bytes(const w4a16_decode_model& m) {
    const int max_k = std::max(std::max(m.hidden, m.intermediate), m.q_heads * m.head_dim);
    const size_t linear = kFlagBytes + sizeof(float) * 2 * kStepKW * 4 * 32 + static_cast<size_t>(kStepStages) * stage_bytes<1, 2>() +
                          static_cast<size_t>(max_k) * sizeof(__half);
    const int lanes_per_pos = m.head_dim / 8;
    const size_t attention = sizeof(float) * (((m.max_len + 3) & ~3) + 8 + m.head_dim + (kThreads / lanes_per_pos) * m.head_dim) +
                             4 * static_cast<size_t>(m.head_dim);
    return std::max(linear, attention);
}

}  // namespace

size_t decode_plan_bytes(const w4a16_decode_model* model) {
    PlanLayout l;
    if (model == nullptr || !layout_of(*model, &l)) return 0;
    return l.total;
}

int decode_plan_build(const w4a16_decode_model* model, void* plan, size_t plan_bytes, int64_t* token, int64_t* position,
                      w4a16_decode_plan_info* info, cudaStream_t stream) {
    if (model == nullptr || plan == nullptr || token == nullptr || position == nullptr || model->layer == nullptr ||
        info == nullptr) {
        return W4A16_ERR_NULL_POINTER;
    }
    const w4a16_decode_model& m = *model;
    PlanLayout l;
    if (!layout_of(m, &l)) return W4A16_ERR_BAD_SHAPE;
    if (plan_bytes < l.total) return W4A16_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(plan) % kPlanAlign != 0) return W4A16_ERR_MISALIGNED;
    if (m.embed == nullptr || m.final_norm == nullptr || m.lm_head_packed == nullptr || m.lm_head_scales == nullptr ||
        m.inv_freq == nullptr) {
        return W4A16_ERR_NULL_POINTER;
    }
    const size_t smem = step_smem_bytes(m);
    if (smem > static_cast<size_t>(kSmemBudget)) return W4A16_ERR_TOO_LARGE;

    char* base = static_cast<char*>(plan);
    auto at = [&](size_t offset) { return static_cast<void*>(base + offset); };
    __half* stream_a = static_cast<__half*>(at(l.stream_a));
    __half* stream_b = static_cast<__half*>(at(l.stream_b));
    PlanHeader* header = static_cast<PlanHeader*>(at(l.header));
    const int qkv_n = (m.q_heads + 2 * m.kv_heads) * m.head_dim;
    const int attn_n = m.q_heads * m.head_dim;

    std::vector<DecodeOp> ops;
    ops.reserve(l.n_ops);
    auto aligned16 = [](const void* q) { return reinterpret_cast<uintptr_t>(q) % 16 == 0; };
    const __half* delta = nullptr;
    for (int i = 0; i < m.layers; ++i) {
        const w4a16_decode_layer& w = m.layer[i];
        if (w.norm1 == nullptr || w.qkv_packed == nullptr || w.qkv_scales == nullptr || w.o_packed == nullptr ||
            w.o_scales == nullptr || w.norm2 == nullptr || w.gate_up_packed == nullptr || w.gate_up_scales == nullptr ||
            w.down_packed == nullptr || w.down_scales == nullptr || w.k_cache == nullptr || w.v_cache == nullptr) {
            return W4A16_ERR_NULL_POINTER;
        }
        if (!aligned16(w.qkv_packed) || !aligned16(w.o_packed) || !aligned16(w.gate_up_packed) || !aligned16(w.down_packed) ||
            !aligned16(w.norm1) || !aligned16(w.norm2) || !aligned16(w.k_cache) || !aligned16(w.v_cache)) {
            return W4A16_ERR_MISALIGNED;
        }
        DecodeOp op{};
        // q/k/v: x = norm1 * rmsnorm(a + delta); the summed stream goes to b.  In the first block the stream is the
        // embedding row of the token.
        op.kind = kOpLinear;
        op.linear = step_linear(i == 0 ? m.embed : stream_a, w.qkv_packed, w.qkv_scales, at(l.qkv), qkv_n, m.hidden);
        op.linear.x_mode = W4A16_INPUT_ADD_RMSNORM;
        op.linear.x_row_index = i == 0 ? reinterpret_cast<const long long*>(token) : nullptr;
        op.linear.x_second = delta;
        op.linear.norm_weight = static_cast<const __half*>(w.norm1);
        op.linear.stream_out = stream_b;
        op.linear.eps = m.eps;
        ops.push_back(op);
        op = DecodeOp{};
        op.kind = kOpAttention;
        op.attention = AttentionOp{static_cast<const __half*>(at(l.qkv)), static_cast<__half*>(w.k_cache),
                                   static_cast<__half*>(w.v_cache), static_cast<__half*>(at(l.attn)),
                                   reinterpret_cast<const long long*>(position), m.inv_freq, m.q_heads, m.kv_heads, m.max_len,
                                   m.rope_scale, m.softmax_scale};
        ops.push_back(op);
        op = DecodeOp{};
        op.kind = kOpLinear;
        op.linear = step_linear(at(l.attn), w.o_packed, w.o_scales, at(l.o), m.hidden, attn_n);
        ops.push_back(op);
        // gate/up: x = norm2 * rmsnorm(b + o); the summed stream goes back to a
        op.linear = step_linear(stream_b, w.gate_up_packed, w.gate_up_scales, at(l.gate_up), 2 * m.intermediate, m.hidden);
        op.linear.x_mode = W4A16_INPUT_ADD_RMSNORM;
        op.linear.x_second = static_cast<const __half*>(at(l.o));
        op.linear.norm_weight = static_cast<const __half*>(w.norm2);
        op.linear.stream_out = stream_a;
        op.linear.eps = m.eps;
        ops.push_back(op);
        // down: x = silu(gate) * up
        op.linear = step_linear(at(l.gate_up), w.down_packed, w.down_scales, at(l.down), m.hidden, m.intermediate);
        op.linear.x_mode = W4A16_INPUT_SILU_MUL;
        op.linear.x_ld = 2 * m.intermediate;
        ops.push_back(op);
        delta = static_cast<const __half*>(at(l.down));
    }
    DecodeOp op{};
    op.kind = kOpLinear;
    op.linear = step_linear(stream_a, m.lm_head_packed, m.lm_head_scales, at(l.logits), m.vocab, m.hidden);
    op.linear.x_mode = W4A16_INPUT_ADD_RMSNORM;
    op.linear.x_second = delta;
    op.linear.norm_weight = static_cast<const __half*>(m.final_norm);
    op.linear.eps = m.eps;
    ops.push_back(op);
    op = DecodeOp{};
    op.kind = kOpArgmax;
    op.argmax = ArgmaxOp{static_cast<const __half*>(at(l.logits)), m.vocab, reinterpret_cast<long long*>(token),
                         reinterpret_cast<long long*>(position), &header->step_count};
    ops.push_back(op);
    if (static_cast<int>(ops.size()) != l.n_ops) return W4A16_ERR_BAD_CONFIG;

    // grid: as many CTAs as are resident at once (the launch is cooperative), at most one per 16-row tile of the
    // narrowest linear ... and at least one per query head
    int device = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
        cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_step_kernel, kThreads, smem) != cudaSuccess || per_sm < 1) {
        return W4A16_ERR_LAUNCH;
    }
    int ctas_per_sm = 2;
    if (const char* knob = std::getenv("W4A16_STEP_CTAS_PER_SM")) ctas_per_sm = std::atoi(knob) == 1 ? 1 : 2;
    const int grid = sms * std::min(per_sm, ctas_per_sm);
    if (grid < m.q_heads) return W4A16_ERR_TOO_LARGE;

    PlanHeader host_header{0u, 0u, 0u, l.n_ops, grid, m.head_dim, static_cast<unsigned>(smem), kPlanMagic};
    if (cudaMemsetAsync(plan, 0, l.total, stream) != cudaSuccess ||
        cudaMemcpyAsync(at(l.ops), ops.data(), sizeof(DecodeOp) * ops.size(), cudaMemcpyHostToDevice, stream) != cudaSuccess ||
        cudaMemcpyAsync(header, &host_header, sizeof(PlanHeader), cudaMemcpyHostToDevice, stream) != cudaSuccess ||
        cudaStreamSynchronize(stream) != cudaSuccess) {     // `ops` and `host_header` are about to go out of scope
        return W4A16_ERR_LAUNCH;
    }
    info->logits = at(l.logits);
    info->status = &header->status;
    info->operations = l.n_ops;
    info->grid = grid;
    info->head_dim = m.head_dim;
    info->smem_bytes = static_cast<uint32_t>(smem);
    return W4A16_OK;
}

int launch_decode_step(const void* plan, int32_t n_ops, int32_t grid, int32_t head_dim, uint32_t smem_bytes, cudaStream_t stream) {
    if (plan == nullptr) return W4A16_ERR_NULL_POINTER;
    if (n_ops <= 0 || grid <= 0 || smem_bytes > static_cast<uint32_t>(kSmemBudget)) return W4A16_ERR_BAD_SHAPE;
    char* base = static_cast<char*>(const_cast<void*>(plan));
    PlanHeader* header = reinterpret_cast<PlanHeader*>(base);
    StepParams params{reinterpret_cast<const DecodeOp*>(base + aligned(sizeof(PlanHeader))), n_ops, &header->counter,
                      &header->step_count, &header->status};
    int hd = head_dim;
    void* args[] = {&params, &hd};
    if (cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(decode_step_kernel), dim3(grid), dim3(kThreads), args,
                                    smem_bytes, stream) != cudaSuccess) {
        return W4A16_ERR_LAUNCH;
    }
    g_launch_count.fetch_add(1, std::memory_order_relaxed);
    return W4A16_OK;
}

}  // namespace w4a16
