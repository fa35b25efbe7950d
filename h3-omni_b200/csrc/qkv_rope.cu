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

#include "attn_kernels.h"
#include "sm100_ptx.cuh"

namespace h3b {
namespace {

constexpr int RD = 128;        // head dimension
constexpr int TILE_ROWS = 64;  // rows of a VSA tile
constexpr int TILE_HEADS = 2;  // heads per CTA of the tile sink (96 KB of staging, two CTAs per SM)

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
__device__ __forceinline__ float round_bf16(float x) {
    return __bfloat162float(__float2bfloat16_rn(x));
}
__device__ __forceinline__ void unpack4(uint2 raw, float (&x)[4]) {
    x[0] = bf16_lo(raw.x);
    x[1] = bf16_hi(raw.x);
    x[2] = bf16_lo(raw.y);
    x[3] = bf16_hi(raw.y);
}
__device__ __forceinline__ uint32_t bits2(float lo, float hi) {
    return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(lo)) |
           ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(hi)) << 16);
}

// What a lane needs that does not depend on the head: norm weights, its rotation partner and
// the row's angles.
struct LaneSetup {
    float qw[4], kw[4], c[4], s[4];
    unsigned partner;
    int role;   // 0: dimension d < rope_half, 1: rope_half <= d < 2 rope_half, 2: not rotated
};

__device__ __forceinline__ void lane_weights(const RopeArgs &a, unsigned lane, LaneSetup &u) {
    unpack4(__ldg(reinterpret_cast<const uint2 *>(a.q_weight) + lane), u.qw);
    unpack4(__ldg(reinterpret_cast<const uint2 *>(a.k_weight) + lane), u.kw);
    const unsigned quarter = a.rope_half / 4;
    u.role = lane < quarter ? 0 : lane < 2 * quarter ? 1 : 2;
    u.partner = u.role == 0 ? lane + quarter : u.role == 1 ? lane - quarter : lane;
}
__device__ __forceinline__ void lane_angles(const RopeArgs &a, unsigned lane, size_t row, LaneSetup &u) {
    if (u.role == 2) return;
    const size_t angle = row * a.rope_half + (u.role == 0 ? lane * 4 : lane * 4 - a.rope_half);
    unpack4(__ldg(reinterpret_cast<const uint2 *>(a.rope_cos + angle)), u.c);
    unpack4(__ldg(reinterpret_cast<const uint2 *>(a.rope_sin + angle)), u.s);
}

// One vector of 128 values across the warp. Explicit _rn intrinsics: no contraction may merge
// a product with the add that follows it, each product is rounded on its own as in the
// reference build (--fmad=false).
__device__ __forceinline__ uint2 norm_rope(uint2 raw, const float (&w)[4], const LaneSetup &u, float epsilon) {
    float x[4];
    unpack4(raw, x);
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; i++) sum = fmaf(x[i], x[i], sum);
#pragma unroll
    for (int distance = 16; distance; distance >>= 1)
        sum = __fadd_rn(sum, __shfl_down_sync(0xffffffffu, sum, distance));
    sum = __shfl_sync(0xffffffffu, sum, 0);
    const float inverse = rsqrtf(__fadd_rn(__fdiv_rn(sum, (float)RD), epsilon));
    float y[4], z[4];
#pragma unroll
    for (int i = 0; i < 4; i++) y[i] = round_bf16(__fmul_rn(__fmul_rn(x[i], inverse), w[i]));
#pragma unroll
    for (int i = 0; i < 4; i++) z[i] = __shfl_sync(0xffffffffu, y[i], u.partner);
    if (u.role != 2) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float mine = round_bf16(__fmul_rn(y[i], u.c[i]));
            const float other = round_bf16(__fmul_rn(z[i], u.s[i]));
            y[i] = u.role == 0 ? __fsub_rn(mine, other) : __fadd_rn(mine, other);
        }
    }
    return make_uint2(bits2(y[0], y[1]), bits2(y[2], y[3]));
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

// One warp per row, walking its heads two at a time (six 256-byte loads in flight per warp).
// PEER: stores go to the window of the rank that owns the head.
template <bool PEER>
__global__ void __launch_bounds__(256)
qkv_rope_rows_kernel(const RopeArgs a) {
    const unsigned lane = threadIdx.x & 31;
    const size_t row = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= a.rows) return;   // whole warps leave
    LaneSetup u;
    lane_weights(a, lane, u);
    lane_angles(a, lane, row, u);
    const uint2 *in = reinterpret_cast<const uint2 *>(a.qkv);
    const unsigned per_rank = PEER ? a.heads / a.ranks : a.heads;
    auto store = [&](unsigned head, uint2 q, uint2 k, uint2 v) {
        size_t at;
        uint2 *dst[3];
        if (PEER) {
            const unsigned owner = head / per_rank;
            at = (((size_t)a.rank * a.rows + row) * per_rank + head % per_rank) * (RD / 4) + lane;
#pragma unroll
            for (int t = 0; t < 3; t++) dst[t] = reinterpret_cast<uint2 *>(a.peer[t][owner]);
        } else {
            at = (row * a.heads + head) * (RD / 4) + lane;
#pragma unroll
            for (int t = 0; t < 3; t++) dst[t] = reinterpret_cast<uint2 *>(a.out[t]);
        }
        dst[0][at] = q;
        dst[1][at] = k;
        dst[2][at] = v;
    };
    unsigned head = 0;
    for (; head + 1 < a.heads; head += 2) {
        size_t o0[3], o1[3];
        input_offsets(a, row, head, o0);
        input_offsets(a, row, head + 1, o1);
        const uint2 q0 = __ldg(in + o0[0] + lane), k0 = __ldg(in + o0[1] + lane), v0 = __ldg(in + o0[2] + lane);
        const uint2 q1 = __ldg(in + o1[0] + lane), k1 = __ldg(in + o1[1] + lane), v1 = __ldg(in + o1[2] + lane);
        store(head, norm_rope(q0, u.qw, u, a.epsilon), norm_rope(k0, u.kw, u, a.epsilon), v0);
        store(head + 1, norm_rope(q1, u.qw, u, a.epsilon), norm_rope(k1, u.kw, u, a.epsilon), v1);
    }
    if (head < a.heads) {
        size_t o0[3];
        input_offsets(a, row, head, o0);
        const uint2 q0 = __ldg(in + o0[0] + lane), k0 = __ldg(in + o0[1] + lane), v0 = __ldg(in + o0[2] + lane);
        store(head, norm_rope(q0, u.qw, u, a.epsilon), norm_rope(k0, u.kw, u, a.epsilon), v0);
    }
}

// One CTA per (tile, pair of heads): the 64 token rows the tile map names are normalised and
// rotated, written in tile order, and kept in shared memory for the tile means, which follow
// the summation order of the tile-pooling kernel (cuda/vsa.cuh:18-43): row i feeds accumulator
// (i % 4, (i / 4) % 4); the four accumulators of a lane are added left to right, then
// (lane0 + lane2) + (lane1 + lane3), then divided by the number of valid rows.
__global__ void __launch_bounds__(256)
qkv_rope_tiles_kernel(const RopeArgs a) {
    extern __shared__ uint2 staged[];   // [tensor][slot][head of the pair][32 lanes]
    __shared__ int rows[TILE_ROWS];
    const int tile = blockIdx.x, head0 = blockIdx.y * TILE_HEADS;
    const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x < TILE_ROWS) rows[threadIdx.x] = a.map[tile * TILE_ROWS + threadIdx.x];
    __syncthreads();
    LaneSetup u;
    lane_weights(a, lane, u);
    const uint2 *in = reinterpret_cast<const uint2 *>(a.qkv);
    const int pair = min(TILE_HEADS, (int)a.heads - head0);
    for (int slot = warp; slot < TILE_ROWS; slot += 8) {
        const int row = rows[slot];   // the same for the whole warp
        if (row >= 0) lane_angles(a, lane, (size_t)row, u);
        for (int h = 0; h < pair; h++) {
            uint2 r[3] = {make_uint2(0u, 0u), make_uint2(0u, 0u), make_uint2(0u, 0u)};
            if (row >= 0) {
                size_t off[3];
                input_offsets(a, (size_t)row, head0 + h, off);
                const uint2 q = __ldg(in + off[0] + lane), k = __ldg(in + off[1] + lane);
                r[2] = __ldg(in + off[2] + lane);
                r[0] = norm_rope(q, u.qw, u, a.epsilon);
                r[1] = norm_rope(k, u.kw, u, a.epsilon);
            }
            const size_t at = (((size_t)(head0 + h) * a.tiles + tile) * TILE_ROWS + slot) * (RD / 4) + lane;
#pragma unroll
            for (int t = 0; t < 3; t++) {
                reinterpret_cast<uint2 *>(a.tiled[t])[at] = r[t];
                staged[((t * TILE_ROWS + slot) * TILE_HEADS + h) * 32 + lane] = r[t];
            }
        }
    }
    __syncthreads();
    // tile means: thread = (tensor, head of the pair, four dimensions)
    const int item = threadIdx.x >> 5;   // 0 .. 3 * TILE_HEADS - 1 are used
    if (item >= 3 * TILE_HEADS) return;
    const int t = item / TILE_HEADS, h = item % TILE_HEADS;
    if (h >= pair) return;
    float lane_sum[4][4];
#pragma unroll
    for (int l = 0; l < 4; l++) {
        float acc[4][4];
#pragma unroll
        for (int slot = 0; slot < 4; slot++)
#pragma unroll
            for (int d = 0; d < 4; d++) acc[slot][d] = 0.0f;
#pragma unroll
        for (int round = 0; round < 4; round++) {
#pragma unroll
            for (int slot = 0; slot < 4; slot++) {
                const int i = l + slot * 4 + round * 16;
                const uint2 x = staged[((t * TILE_ROWS + i) * TILE_HEADS + h) * 32 + lane];
                acc[slot][0] = __fadd_rn(acc[slot][0], bf16_lo(x.x));
                acc[slot][1] = __fadd_rn(acc[slot][1], bf16_hi(x.x));
                acc[slot][2] = __fadd_rn(acc[slot][2], bf16_lo(x.y));
                acc[slot][3] = __fadd_rn(acc[slot][3], bf16_hi(x.y));
            }
        }
#pragma unroll
        for (int d = 0; d < 4; d++)
            lane_sum[l][d] = __fadd_rn(__fadd_rn(__fadd_rn(acc[0][d], acc[1][d]), acc[2][d]), acc[3][d]);
    }
    const float size = (float)a.sizes[tile];
    float4 mean;
    mean.x = __fdiv_rn(__fadd_rn(__fadd_rn(lane_sum[0][0], lane_sum[2][0]), __fadd_rn(lane_sum[1][0], lane_sum[3][0])), size);
    mean.y = __fdiv_rn(__fadd_rn(__fadd_rn(lane_sum[0][1], lane_sum[2][1]), __fadd_rn(lane_sum[1][1], lane_sum[3][1])), size);
    mean.z = __fdiv_rn(__fadd_rn(__fadd_rn(lane_sum[0][2], lane_sum[2][2]), __fadd_rn(lane_sum[1][2], lane_sum[3][2])), size);
    mean.w = __fdiv_rn(__fadd_rn(__fadd_rn(lane_sum[0][3], lane_sum[2][3]), __fadd_rn(lane_sum[1][3], lane_sum[3][3])), size);
    reinterpret_cast<float4 *>(a.pooled[t])[((size_t)(head0 + h) * a.tiles + tile) * (RD / 4) + lane] = mean;
}

constexpr size_t TILES_SMEM = (size_t)3 * TILE_ROWS * TILE_HEADS * 32 * sizeof(uint2);

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
    qkv_rope_rows_kernel<false><<<(in.rows + 7) / 8, 256, 0, stream>>>(a);
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
    qkv_rope_rows_kernel<true><<<(in.rows + 7) / 8, 256, 0, stream>>>(a);
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
    static thread_local int configured_device = -1;
    int device = 0;
    e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    if (configured_device != device) {
        e = cudaFuncSetAttribute(qkv_rope_tiles_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)TILES_SMEM);
        if (e != cudaSuccess) return e;
        configured_device = device;
    }
    dim3 grid(tiles, (in.heads + TILE_HEADS - 1) / TILE_HEADS);
    qkv_rope_tiles_kernel<<<grid, 256, TILES_SMEM, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace h3b
