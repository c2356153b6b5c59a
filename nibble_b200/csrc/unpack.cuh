// Device helpers shared by the W4A16 kernels: INT4 -> FP16 unpack, cache-hinted loads,
// the m16n8k16 tensor-core instruction and programmatic-dependent-launch controls.
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

namespace w4a16 {

constexpr int kGroup = 128;        // K elements per scale on the fast path
constexpr int kChunkBytes = 64;    // packed bytes of one 128-wide K chunk of one row

// lop3 with truth table (a & b) ^ c.
__device__ __forceinline__ uint32_t and_xor(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// One 32-bit word = 8 codes, code j in nibble j.  Returns four half2 registers holding the exact
// signed values as FP16, paired (c0,c4) (c1,c5) (c2,c6) (c3,c7).
//
// A nibble n (two's complement code c) satisfies n ^ 8 == c + 8.  OR-ing that into the mantissa of
// 1024.0 (0x6400, ulp 1) gives 1032 + c, so (word & 0x000F000F) ^ 0x64086408 is the pair
// (1032 + c0, 1032 + c4) in one instruction; subtracting 1032 is exact.  A nibble four bits higher
// lands as 1024 + 16*(c + 8); multiplying by 1/16 and subtracting 72 in one FMA is exact too.
__device__ __forceinline__ void unpack8(uint32_t word, uint32_t (&out)[4]) {
    const uint32_t lo0 = and_xor(word, 0x000F000Fu, 0x64086408u);
    const uint32_t hi0 = and_xor(word, 0x00F000F0u, 0x64806480u);
    const uint32_t next = word >> 8;
    const uint32_t lo1 = and_xor(next, 0x000F000Fu, 0x64086408u);
    const uint32_t hi1 = and_xor(next, 0x00F000F0u, 0x64806480u);
    out[0] = hsub2_u32(lo0, 0x64086408u);                     // (c0, c4)
    out[1] = hfma2_u32(hi0, 0x2C002C00u, 0xD480D480u);        // (c1, c5)
    out[2] = hsub2_u32(lo1, 0x64086408u);                     // (c2, c6)
    out[3] = hfma2_u32(hi1, 0x2C002C00u, 0xD480D480u);        // (c3, c7)
}

// Byte permute: pick bytes of {b:a} by selector nibbles.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// 16-byte streaming load of read-only data that is touched once: skip L1 allocation.
__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t ldg_stream4(const void* p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

// 16-byte load of data every warp of the SM re-reads (activations): keep it in L1.
__device__ __forceinline__ uint4 ldg_keep16(const void* p) {
    uint4 v;
    asm volatile("ld.global.ca.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ uint16_t ldg_nc_u16(const void* p) {
    uint16_t v;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}

// D = A(16x16, row) * B(16x8, col) + D, FP16 operands, FP32 accumulate.
// Lane (g = lane/4, t = lane%4) supplies
//   a0: A[g][2t,2t+1]   a1: A[g+8][2t,2t+1]   a2: A[g][2t+8,2t+9]   a3: A[g+8][2t+8,2t+9]
//   b0: B[2t,2t+1][g]   b1: B[2t+8,2t+9][g]
// and owns d0,d1 = D[g][2t,2t+1], d2,d3 = D[g+8][2t,2t+1].
__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                             uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// D = A * B + C with C read from caller-kept registers (e.g. four that stay zero) and D written
// elsewhere: lets the first MMA of a sum skip clearing its accumulator.
__device__ __forceinline__ void mma_m16n8k16_from(float (&d)[4], const float (&c)[4], uint32_t a0, uint32_t a1,
                                                  uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

// half(silu(g)) for a pair: FP32 with the fast exponential and division (a few ulp of FP32, far below
// the FP16 rounding that follows), then one rounding to FP16 -- where a framework rounds silu's result.
__device__ __forceinline__ __half2 silu_half2(__half2 gate) {
    const float2 f = __half22float2(gate);
    return __floats2half2_rn(__fdividef(f.x, 1.0f + __expf(-f.x)), __fdividef(f.y, 1.0f + __expf(-f.y)));
}

// Programmatic dependent launch.  Both are no-ops for a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait_for_upstream() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void pdl_release_downstream() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

}  // namespace w4a16
