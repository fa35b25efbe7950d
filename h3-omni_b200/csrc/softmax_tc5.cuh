// Online-softmax building blocks shared by the tcgen05 attention kernels. One thread owns one
// query row: its S values arrive from TMEM with tcgen05.ld.32x32b (32 columns per load), its
// P values go back as packed bf16 pairs over the columns S occupied.
#pragma once
#include "sm100_ptx.cuh"

namespace h3b {

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ void max_chunk(const uint32_t (&v)[32], float &m0, float &m1) {
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
        m0 = max3(m0, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
        m1 = max3(m1, __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
    }
}
// The same over four independent chains (a lone warp on its scheduler is bound by the latency of
// the chain, not by issue slots).
__device__ __forceinline__ void max_chunk4(const uint32_t (&v)[32], float (&m)[4]) {
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
#pragma unroll
        for (int k = 0; k < 4; k++)
            m[k] = max3(m[k], __uint_as_float(v[i + 2 * k]), __uint_as_float(v[i + 2 * k + 1]));
    }
}
// Row maximum over a full tile. Loads of the next 32 columns are in flight while the
// current 32 are reduced.
template <int BN>
__device__ __forceinline__ float row_max_full(uint32_t s_addr) {
    constexpr int NC = BN / 32;
    uint32_t a[32], b[32];
    float m0 = -INFINITY, m1 = -INFINITY;
    tmem_ld32(s_addr, a);
    tmem_wait_ld();
#pragma unroll
    for (int c = 0; c < NC; c += 2) {
        if (c + 1 < NC) tmem_ld32(s_addr + (c + 1) * 32, b);
        max_chunk(a, m0, m1);
        if (c + 1 < NC) {
            tmem_wait_ld();
            if (c + 2 < NC) tmem_ld32(s_addr + (c + 2) * 32, a);
            max_chunk(b, m0, m1);
            if (c + 2 < NC) tmem_wait_ld();
        }
    }
    return fmaxf(m0, m1);
}
template <int BN>
__device__ __forceinline__ float row_max_masked(uint32_t s_addr, int nvalid) {
    float mx = -INFINITY;
#pragma unroll
    for (int c = 0; c < BN / 32; c++) {
        uint32_t v[32];
        tmem_ld32(s_addr + c * 32, v);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i++)
            if (c * 32 + i < nvalid) mx = fmaxf(mx, __uint_as_float(v[i]));
    }
    return mx;
}
// p = exp2(s * scale_log2 + neg) for 32 columns, packed pairwise to bf16; partial row sums
// accumulate in two float2 chains (packed f32x2 arithmetic halves the FMA-pipe work).
__device__ __forceinline__ void exp_chunk(const uint32_t (&v)[32], uint32_t (&packed)[16],
                                          float2 scale2, float2 neg2, float2 &sum0, float2 &sum1) {
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
        const float2 x0 = __ffma2_rn(make_float2(__uint_as_float(v[i]), __uint_as_float(v[i + 1])),
                                     scale2, neg2);
        const float2 x1 = __ffma2_rn(
            make_float2(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3])), scale2, neg2);
        const float2 p0 = make_float2(fast_exp2(x0.x), fast_exp2(x0.y));
        const float2 p1 = make_float2(fast_exp2(x1.x), fast_exp2(x1.y));
        sum0 = __fadd2_rn(sum0, p0);
        sum1 = __fadd2_rn(sum1, p1);
        packed[i / 2] = pack_bf16(p0.x, p0.y);
        packed[i / 2 + 1] = pack_bf16(p1.x, p1.y);
    }
}
// Full tile: P (bf16 pairs, half the columns) goes to p_addr - over columns of S that were
// already consumed - with the loads running one chunk ahead.
template <int BN>
__device__ __forceinline__ float exp_store_full(uint32_t s_addr, uint32_t p_addr, float scale_log2,
                                                float neg) {
    constexpr int NC = BN / 32;
    uint32_t a[32], b[32], packed[16];
    float2 sum0 = make_float2(0.f, 0.f), sum1 = make_float2(0.f, 0.f);
    const float2 scale2 = make_float2(scale_log2, scale_log2), neg2 = make_float2(neg, neg);
    tmem_ld32(s_addr, a);
    tmem_wait_ld();
#pragma unroll
    for (int c = 0; c < NC; c += 2) {
        if (c + 1 < NC) tmem_ld32(s_addr + (c + 1) * 32, b);
        exp_chunk(a, packed, scale2, neg2, sum0, sum1);
        tmem_st16(p_addr + c * 16, packed);
        if (c + 1 < NC) {
            tmem_wait_ld();
            if (c + 2 < NC) tmem_ld32(s_addr + (c + 2) * 32, a);
            exp_chunk(b, packed, scale2, neg2, sum0, sum1);
            tmem_st16(p_addr + (c + 1) * 16, packed);
            if (c + 2 < NC) tmem_wait_ld();
        }
    }
    return (sum0.x + sum0.y) + (sum1.x + sum1.y);
}
template <int BN>
__device__ __forceinline__ float exp_store_masked(uint32_t s_addr, uint32_t p_addr, float scale_log2,
                                                  float neg, int nvalid) {
    float sum = 0.0f;
#pragma unroll
    for (int c = 0; c < BN / 32; c++) {
        uint32_t v[32], packed[16];
        tmem_ld32(s_addr + c * 32, v);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
            float p0 = fast_exp2(fmaf(__uint_as_float(v[i]), scale_log2, neg));
            float p1 = fast_exp2(fmaf(__uint_as_float(v[i + 1]), scale_log2, neg));
            if (c * 32 + i >= nvalid) p0 = 0.0f;
            if (c * 32 + i + 1 >= nvalid) p1 = 0.0f;
            sum += p0 + p1;
            packed[i / 2] = pack_bf16(p0, p1);
        }
        tmem_st16(p_addr + c * 16, packed);
    }
    return sum;
}
template <int BN>
__device__ __forceinline__ void store_zero_p(uint32_t p_addr) {
    uint32_t zero[16];
#pragma unroll
    for (int i = 0; i < 16; i++) zero[i] = 0u;
#pragma unroll
    for (int c = 0; c < BN / 32; c++) tmem_st16(p_addr + c * 16, zero);
}


// 2^x for a pair of finite x <= 2^7 on the FMA pipe instead of the exponential unit:
// x = n + f with n = round(x), f in [-0.5, 0.5]; 2^f by a degree-3 minimax polynomial
// (relative error 7.5e-5, an order of magnitude below the bf16 rounding applied to P next);
// 2^n by adding n to the exponent field. Used for a fixed fraction of the columns so the
// exponential unit stops being the critical resource of the softmax.
__device__ __forceinline__ float2 exp2_poly2(float2 x) {
    const float magic = 12582912.0f;  // 1.5 * 2^23: x + magic holds round(x) in its low mantissa bits
    x.x = fmaxf(x.x, -126.0f);
    x.y = fmaxf(x.y, -126.0f);
    const float2 t = __fadd2_rn(x, make_float2(magic, magic));
    const float2 n = __fadd2_rn(t, make_float2(-magic, -magic));
    const float2 f = __fadd2_rn(x, make_float2(-n.x, -n.y));
    float2 p = __ffma2_rn(make_float2(0.0551716685f, 0.0551716685f), f,
                          make_float2(0.2426111251f, 0.2426111251f));
    p = __ffma2_rn(p, f, make_float2(0.6932609677f, 0.6932609677f));
    p = __ffma2_rn(p, f, make_float2(0.9999280572f, 0.9999280572f));
    float2 r;
    r.x = __int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23));
    r.y = __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23));
    return r;
}
// exp_chunk where, in the groups of four columns named by POLY_MASK (bit g = group g of the
// chunk's eight), the second pair is evaluated by exp2_poly2: 0x55 -> 25 % of the columns,
// 0x6d -> 31 %, 0xff -> 50 %, 0 -> none.
template <int POLY_MASK>
__device__ __forceinline__ void exp_chunk_mixed(const uint32_t (&v)[32], uint32_t (&packed)[16],
                                                float2 scale2, float2 neg2, float2 &sum0,
                                                float2 &sum1) {
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
        const float2 x0 = __ffma2_rn(make_float2(__uint_as_float(v[i]), __uint_as_float(v[i + 1])),
                                     scale2, neg2);
        const float2 x1 = __ffma2_rn(
            make_float2(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3])), scale2, neg2);
        const float2 p0 = make_float2(fast_exp2(x0.x), fast_exp2(x0.y));
        const bool poly = (POLY_MASK >> (i / 4)) & 1;
        const float2 p1 = poly ? exp2_poly2(x1) : make_float2(fast_exp2(x1.x), fast_exp2(x1.y));
        sum0 = __fadd2_rn(sum0, p0);
        sum1 = __fadd2_rn(sum1, p1);
        packed[i / 2] = pack_bf16(p0.x, p0.y);
        packed[i / 2 + 1] = pack_bf16(p1.x, p1.y);
    }
}

}  // namespace h3b
