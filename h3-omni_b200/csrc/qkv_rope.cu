// Q/K RMS-norm + rotary embedding on the fused QKV projection output, head dim 128, writing
// straight into the layout the attention step wants. Three sinks share one arithmetic core:
//   token-major   q, k, v [rows][heads][128]                 (h3_gpu_qkv_rope_bf16 and the grouped
//                 variant; the reference's cuda/h3_gpu_cuda.cu:989-1031)
//   head shards   each (row, head) vector goes to the peer rank that owns the head, at the place
//                 the Ulysses scatter would have put it (replaces rope + three exchange kernels)
//   VSA tiles     q, k, v in 64-row tile order plus the FP32 tile means (replaces rope + the
//                 gather of tile_pool: the token-major copies are never written or re-read)
// The arithmetic is the reference's, operation for operation (cuda/primitives.cuh:897-962 and
// cuda/fast_primitives.cuh:184-265), so outputs are bit-identical to it: one warp per
// (row, head) vector, lane t owns dimensions 4t..4t+3; sum of squares as a 4-step fmaf chain
// per lane then a shuffle-down tree; x * rsqrt(mean + eps) * weight rounded to bf16; rotation
// of dimension d < rope_half with d + rope_half from two bf16-rounded products.
// Every kernel here is bound by HBM traffic: 6 bytes moved per bf16 element of q, k and v.
#include <algorithm>

#include <cuda_bf16.h>

#include "attn_kernels.h"
#include "sm100_ptx.cuh"

namespace h3b {
namespace {

constexpr int RD = 128;        // head dimension
constexpr int TILE_ROWS = 64;  // rows of a VSA tile

struct RopeArgs {
    const uint16_t *qkv, *q_weight, *k_weight, *rope_cos, *rope_sin;
    unsigned rows, heads, rope_half, grouped;
    float epsilon;
    uint16_t *out[3];          // token-major sink
    uint16_t *peer[3][16];     // head-shard sink: tensor x rank windows, [ranks*rows][heads/ranks][128]
    unsigned rank, ranks;
    const int *map, *sizes;    // tile sink
    int tiles;
    uint16_t *tiled[3];
    float *pooled[3];
};

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ void unpack4(uint2 raw, float (&x)[4]) {
    x[0] = bf16_lo(raw.x);
    x[1] = bf16_hi(raw.x);
    x[2] = bf16_lo(raw.y);
    x[3] = bf16_hi(raw.y);
}

// What a lane needs that does not depend on the head: norm weights, its rotation partner and
// the row's angles. The sine carries the sign of the rotation (minus for dimensions below
// rope_half), so both halves compute round(y cos) + round(z sin'); a - b and a + (-b) are the
// same IEEE operation and negation commutes with rounding.
struct LaneSetup {
    float qw[4], kw[4];
    uint2 c, s;   // four cosines / signed sines of the row, packed bf16
    unsigned partner;
    int role;   // 0: dimension d < rope_half, 1: rope_half <= d < 2 rope_half, 2: not rotated
};

__device__ __forceinline__ void lane_weights(const RopeArgs &a, unsigned lane, LaneSetup &u) {
    unpack4(__ldg(reinterpret_cast<const uint2 *>(a.q_weight) + lane), u.qw);
    unpack4(__ldg(reinterpret_cast<const uint2 *>(a.k_weight) + lane), u.kw);
    const unsigned quarter = a.rope_half / 4;
    u.role = lane < quarter ? 0 : lane < 2 * quarter ? 1 : 2;
    u.partner = u.role == 0 ? lane + quarter : u.role == 1 ? lane - quarter : lane;
    u.c = u.s = make_uint2(0u, 0u);
}
// The row's four cosines and sines of this lane, still packed (lanes that do not rotate: zeros).
__device__ __forceinline__ void load_angles(const RopeArgs &a, unsigned lane, const LaneSetup &u, size_t row,
                                            uint2 &c, uint2 &s) {
    c = s = make_uint2(0u, 0u);
    if (u.role == 2) return;
    const size_t angle = row * a.rope_half + (u.role == 0 ? lane * 4 : lane * 4 - a.rope_half);
    c = __ldg(reinterpret_cast<const uint2 *>(a.rope_cos + angle));
    s = __ldg(reinterpret_cast<const uint2 *>(a.rope_sin + angle));
}
__device__ __forceinline__ void set_angles(LaneSetup &u, uint2 c, uint2 s) {
    u.c = c;
    if (u.role == 0) {   // flip the sign bits of the four sines
        s.x ^= 0x80008000u;
        s.y ^= 0x80008000u;
    }
    u.s = s;
}
// Products of two bf16 values rounded to bf16, a pair at a time. The exact product of two
// 8-bit significands has 16 bits, so the reference's fp32 product is exact and its rounding to
// bf16 is the single rounding mul.rn.bf16x2 performs.
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// One vector of 128 values across the warp. Explicit _rn intrinsics: no contraction may merge
// a product with the add that follows it, each product is rounded on its own as in the
// reference build (--fmad=false). Roundings to bf16 go two at a time through cvt.rn.bf16x2.
__device__ __forceinline__ uint2 norm_rope(uint2 raw, const float (&w)[4], const LaneSetup &u, float epsilon,
                                           bool rotate) {
    float x[4];
    unpack4(raw, x);
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; i++) sum = fmaf(x[i], x[i], sum);
#pragma unroll
    for (int distance = 16; distance; distance >>= 1)
        sum = __fadd_rn(sum, __shfl_down_sync(0xffffffffu, sum, distance));
    sum = __shfl_sync(0xffffffffu, sum, 0);
    // sum / 128 as a multiplication: the same correctly rounded value for every input
    const float inverse = rsqrtf(__fadd_rn(__fmul_rn(sum, 1.0f / (float)RD), epsilon));
    uint2 y;   // normalised, weighted, rounded to bf16
    y.x = pack_bf16(__fmul_rn(__fmul_rn(x[0], inverse), w[0]), __fmul_rn(__fmul_rn(x[1], inverse), w[1]));
    y.y = pack_bf16(__fmul_rn(__fmul_rn(x[2], inverse), w[2]), __fmul_rn(__fmul_rn(x[3], inverse), w[3]));
    if (!rotate) return y;   // rope_half == 0: uniform over the launch
    uint2 z;
    z.x = __shfl_sync(0xffffffffu, y.x, u.partner);
    z.y = __shfl_sync(0xffffffffu, y.y, u.partner);
    if (u.role == 2) return y;
    const uint32_t m01 = mul_bf16x2(y.x, u.c.x), m23 = mul_bf16x2(y.y, u.c.y);
    const uint32_t o01 = mul_bf16x2(z.x, u.s.x), o23 = mul_bf16x2(z.y, u.s.y);
    y.x = pack_bf16(__fadd_rn(bf16_lo(m01), bf16_lo(o01)), __fadd_rn(bf16_hi(m01), bf16_hi(o01)));
    y.y = pack_bf16(__fadd_rn(bf16_lo(m23), bf16_lo(o23)), __fadd_rn(bf16_hi(m23), bf16_hi(o23)));
    return y;
}

// Offsets (in uint2 units) of the q, k, v vectors of (row, head) inside the projection output:
// [row][q|k|v][head][128] or, grouped, [row][head][q|k|v][128] (the checkpoint's layout).
__device__ __forceinline__ void input_offsets(const RopeArgs &a, size_t row, unsigned head, size_t (&off)[3]) {
    const size_t inner = (size_t)a.heads * RD, base = row * inner * 3;
    if (a.grouped) {
        off[0] = (base + (size_t)head * RD * 3) / 4;
        off[1] = off[0] + RD / 4;
        off[2] = off[1] + RD / 4;
    } else {
        off[0] = (base + (size_t)head * RD) / 4;
        off[1] = off[0] + inner / 4;
        off[2] = off[1] + inner / 4;
    }
}

// One warp per (row, chunk of up to eight heads), four heads (twelve 256-byte loads) in flight
// per pass; the chunks keep warps short so the last wave of CTAs drains evenly. Registers are
// capped at 64 for four CTAs per SM: at three the kernel reached 82 % of the HBM copy rate, at
// four 92 %.
// PEER: stores go to the window of the rank that owns the head.
constexpr unsigned HEAD_CHUNK = 8, HEADS_IN_FLIGHT = 4;

template <bool PEER>
__global__ void __launch_bounds__(256, 4)
qkv_rope_rows_kernel(const RopeArgs a) {
    const unsigned lane = threadIdx.x & 31;
    const unsigned chunks = (a.heads + HEAD_CHUNK - 1) / HEAD_CHUNK;
    const size_t item = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (item >= (size_t)a.rows * chunks) return;   // whole warps leave
    const size_t row = item / chunks;
    const unsigned first = (unsigned)(item % chunks) * HEAD_CHUNK, last = min(a.heads, first + HEAD_CHUNK);
    const bool rotate = a.rope_half != 0;
    LaneSetup u;
    lane_weights(a, lane, u);
    uint2 craw, sraw;
    load_angles(a, lane, u, row, craw, sraw);
    const uint2 *in = reinterpret_cast<const uint2 *>(a.qkv);
    const unsigned per_rank = PEER ? a.heads / a.ranks : a.heads;
    bool angles_set = false;
    for (unsigned head = first; head < last; head += HEADS_IN_FLIGHT) {
        uint2 raw[HEADS_IN_FLIGHT][3];
#pragma unroll
        for (unsigned h = 0; h < HEADS_IN_FLIGHT; h++)
            if (head + h < last) {
                size_t off[3];
                input_offsets(a, row, head + h, off);
#pragma unroll
                for (int t = 0; t < 3; t++) raw[h][t] = __ldcs(in + off[t] + lane);
            }
        if (!angles_set) {
            set_angles(u, craw, sraw);
            angles_set = true;
        }
#pragma unroll
        for (unsigned h = 0; h < HEADS_IN_FLIGHT; h++)
            if (head + h < last) {
                const uint2 q = norm_rope(raw[h][0], u.qw, u, a.epsilon, rotate);
                const uint2 k = norm_rope(raw[h][1], u.kw, u, a.epsilon, rotate);
                size_t at;
                uint2 *dst[3];
                if (PEER) {
                    const unsigned owner = (head + h) / per_rank;
                    at = (((size_t)a.rank * a.rows + row) * per_rank + (head + h) % per_rank) * (RD / 4) + lane;
#pragma unroll
                    for (int t = 0; t < 3; t++) dst[t] = reinterpret_cast<uint2 *>(a.peer[t][owner]);
                } else {
                    at = (row * a.heads + head + h) * (RD / 4) + lane;
#pragma unroll
                    for (int t = 0; t < 3; t++) dst[t] = reinterpret_cast<uint2 *>(a.out[t]);
                }
                __stcs(dst[0] + at, q);
                __stcs(dst[1] + at, k);
                __stcs(dst[2] + at, raw[h][2]);
            }
    }
}

// One CTA per (tile, head): the 64 token rows the tile map names are normalised and rotated and
// written in tile order; the tile means follow the summation order of the tile-pooling kernel
// (cuda/vsa.cuh:18-43): row i feeds accumulator i % 16, in the order i = a, a + 16, a + 32,
// a + 48; accumulators a = l, l + 4, l + 8, l + 12 are added left to right into lane sum l, the
// mean is ((lane0 + lane2) + (lane1 + lane3)) / valid rows.
// Warp w owns accumulators w and w + 8 and works through their rows in order, two rows requested
// at a time, so the sums stay in registers and only the sixteen partial sums per tensor meet in
// shared memory; registers are capped for four CTAs per SM (occupancy hides the gather latency). The kernel issues about as
// many instructions as the two kernels it replaces; what it saves is their memory round trip.
__global__ void __launch_bounds__(256, 4)
qkv_rope_tiles_kernel(const RopeArgs a) {
    __shared__ float4 partial[16][3][32];   // [accumulator][tensor][lane]
    __shared__ int rows[TILE_ROWS];
    const int tile = blockIdx.x, head = blockIdx.y;
    const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x < TILE_ROWS) rows[threadIdx.x] = a.map[tile * TILE_ROWS + threadIdx.x];
    __syncthreads();
    const bool rotate = a.rope_half != 0;
    LaneSetup u;
    lane_weights(a, lane, u);
    const uint2 *in = reinterpret_cast<const uint2 *>(a.qkv);
#pragma unroll
    for (int which = 0; which < 2; which++) {
        const int acc_id = warp + 8 * which;
        float acc[3][4];
#pragma unroll
        for (int t = 0; t < 3; t++)
#pragma unroll
            for (int d = 0; d < 4; d++) acc[t][d] = 0.0f;
#pragma unroll
        for (int half = 0; half < 2; half++) {   // two rows (six vectors and their angles) requested at once
            uint2 raw[2][3], craw[2], sraw[2];
            int row[2];
#pragma unroll
            for (int i = 0; i < 2; i++) {
                row[i] = rows[acc_id + 16 * (2 * half + i)];   // the same for the whole warp
#pragma unroll
                for (int t = 0; t < 3; t++) raw[i][t] = make_uint2(0u, 0u);
                craw[i] = sraw[i] = make_uint2(0u, 0u);
                if (row[i] >= 0) {
                    size_t off[3];
                    input_offsets(a, (size_t)row[i], head, off);
#pragma unroll
                    for (int t = 0; t < 3; t++) raw[i][t] = __ldcs(in + off[t] + lane);
                    load_angles(a, lane, u, (size_t)row[i], craw[i], sraw[i]);
                }
            }
#pragma unroll
            for (int i = 0; i < 2; i++) {
                if (row[i] >= 0) {
                    set_angles(u, craw[i], sraw[i]);
                    raw[i][0] = norm_rope(raw[i][0], u.qw, u, a.epsilon, rotate);
                    raw[i][1] = norm_rope(raw[i][1], u.kw, u, a.epsilon, rotate);
                }
                const size_t at =
                    (((size_t)head * a.tiles + tile) * TILE_ROWS + acc_id + 16 * (2 * half + i)) * (RD / 4) + lane;
#pragma unroll
                for (int t = 0; t < 3; t++) {
                    __stcs(reinterpret_cast<uint2 *>(a.tiled[t]) + at, raw[i][t]);
                    acc[t][0] = __fadd_rn(acc[t][0], bf16_lo(raw[i][t].x));
                    acc[t][1] = __fadd_rn(acc[t][1], bf16_hi(raw[i][t].x));
                    acc[t][2] = __fadd_rn(acc[t][2], bf16_lo(raw[i][t].y));
                    acc[t][3] = __fadd_rn(acc[t][3], bf16_hi(raw[i][t].y));
                }
            }
        }
#pragma unroll
        for (int t = 0; t < 3; t++)
            partial[acc_id][t][lane] = make_float4(acc[t][0], acc[t][1], acc[t][2], acc[t][3]);
    }
    __syncthreads();
    // tile means: warp = tensor, lane = four dimensions
    if (warp >= 3) return;
    const int t = warp;
    float4 lane_sum[4];
#pragma unroll
    for (int l = 0; l < 4; l++) {
        float4 s4 = partial[l][t][lane];
#pragma unroll
        for (int slot = 1; slot < 4; slot++) {
            const float4 x = partial[l + 4 * slot][t][lane];
            s4.x = __fadd_rn(s4.x, x.x);
            s4.y = __fadd_rn(s4.y, x.y);
            s4.z = __fadd_rn(s4.z, x.z);
            s4.w = __fadd_rn(s4.w, x.w);
        }
        lane_sum[l] = s4;
    }
    const float size = (float)a.sizes[tile];
    float4 mean;
    mean.x = __fdiv_rn(__fadd_rn(__fadd_rn(lane_sum[0].x, lane_sum[2].x), __fadd_rn(lane_sum[1].x, lane_sum[3].x)), size);
    mean.y = __fdiv_rn(__fadd_rn(__fadd_rn(lane_sum[0].y, lane_sum[2].y), __fadd_rn(lane_sum[1].y, lane_sum[3].y)), size);
    mean.z = __fdiv_rn(__fadd_rn(__fadd_rn(lane_sum[0].z, lane_sum[2].z), __fadd_rn(lane_sum[1].z, lane_sum[3].z)), size);
    mean.w = __fdiv_rn(__fadd_rn(__fadd_rn(lane_sum[0].w, lane_sum[2].w), __fadd_rn(lane_sum[1].w, lane_sum[3].w)), size);
    reinterpret_cast<float4 *>(a.pooled[t])[((size_t)head * a.tiles + tile) * (RD / 4) + lane] = mean;
}

cudaError_t fill(RopeArgs &a, const QkvRopeInput &in) {
    if (!in.qkv || !in.q_weight || !in.k_weight || !in.rope_cos || !in.rope_sin || !in.rows ||
        !in.heads || in.rope_half % 4 || in.rope_half * 2 > (unsigned)RD)
        return cudaErrorInvalidValue;
    for (const void *p : {in.qkv, in.q_weight, in.k_weight, in.rope_cos, in.rope_sin})
        if (reinterpret_cast<uintptr_t>(p) % 8) return cudaErrorMisalignedAddress;
    a.qkv = static_cast<const uint16_t *>(in.qkv);
    a.q_weight = static_cast<const uint16_t *>(in.q_weight);
    a.k_weight = static_cast<const uint16_t *>(in.k_weight);
    a.rope_cos = static_cast<const uint16_t *>(in.rope_cos);
    a.rope_sin = static_cast<const uint16_t *>(in.rope_sin);
    a.rows = in.rows;
    a.heads = in.heads;
    a.rope_half = in.rope_half;
    a.grouped = in.grouped ? 1u : 0u;
    a.epsilon = in.epsilon;
    return cudaSuccess;
}

unsigned rows_grid(const QkvRopeInput &in) {
    const size_t items = (size_t)in.rows * ((in.heads + HEAD_CHUNK - 1) / HEAD_CHUNK);
    return (unsigned)((items + 7) / 8);
}

}  // namespace

cudaError_t qkv_rope_token_major(const QkvRopeInput &in, void *q, void *k, void *v, cudaStream_t stream) {
    RopeArgs a{};
    cudaError_t e = fill(a, in);
    if (e != cudaSuccess) return e;
    void *out[3] = {q, k, v};
    for (int t = 0; t < 3; t++) {
        if (!out[t]) return cudaErrorInvalidValue;
        if (reinterpret_cast<uintptr_t>(out[t]) % 8) return cudaErrorMisalignedAddress;
        a.out[t] = static_cast<uint16_t *>(out[t]);
    }
    qkv_rope_rows_kernel<false><<<rows_grid(in), 256, 0, stream>>>(a);
    return cudaGetLastError();
}

cudaError_t qkv_rope_head_shards(const QkvRopeInput &in, void *const window_q[], void *const window_k[],
                                 void *const window_v[], int rank, int ranks, cudaStream_t stream) {
    RopeArgs a{};
    cudaError_t e = fill(a, in);
    if (e != cudaSuccess) return e;
    if (ranks < 1 || ranks > 16 || rank < 0 || rank >= ranks || in.heads % ranks) return cudaErrorInvalidValue;
    for (int p = 0; p < ranks; p++) {
        void *w[3] = {window_q[p], window_k[p], window_v[p]};
        for (int t = 0; t < 3; t++) {
            if (!w[t] || reinterpret_cast<uintptr_t>(w[t]) % 8) return cudaErrorInvalidValue;
            a.peer[t][p] = static_cast<uint16_t *>(w[t]);
        }
    }
    a.rank = (unsigned)rank;
    a.ranks = (unsigned)ranks;
    qkv_rope_rows_kernel<true><<<rows_grid(in), 256, 0, stream>>>(a);
    return cudaGetLastError();
}

cudaError_t qkv_rope_vsa_tiles(const QkvRopeInput &in, const int *map, const int *sizes, int tiles,
                               void *const tiled[3], float *const pooled[3], cudaStream_t stream) {
    RopeArgs a{};
    cudaError_t e = fill(a, in);
    if (e != cudaSuccess) return e;
    if (!map || !sizes || tiles < 1) return cudaErrorInvalidValue;
    for (int t = 0; t < 3; t++) {
        if (!tiled[t] || !pooled[t]) return cudaErrorInvalidValue;
        a.tiled[t] = static_cast<uint16_t *>(tiled[t]);
        a.pooled[t] = pooled[t];
    }
    a.map = map;
    a.sizes = sizes;
    a.tiles = tiles;
    dim3 grid(tiles, in.heads);
    qkv_rope_tiles_kernel<<<grid, 256, 0, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace h3b
