// Video sparse attention, coarse stage and merge: token-cube pooling, pooled scores with
// warp-level top-k tile selection, the pooled-softmax compression branch, and the gated
// merge back to token-major rows. These are HBM-bound passes; they replace tile_pool,
// the two cuBLAS SGEMMs, select_blocks, pooled_softmax and untile_merge of the reference's
// cuda/vsa.cuh:18-181,263-300 with three launches (pool x3 fused, score+select+compress,
// merge) and never materialise the [heads][tiles][tiles] score matrix unless asked to.
#include <cuda_bf16.h>
#include <math_constants.h>

#include <cstdio>

#include "attn_kernels.h"

namespace h3b {
namespace {

constexpr int VD = 128, VT = 64;

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t x) { return __uint_as_float(x << 16); }
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float x) {
    return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(x));
}
__device__ __forceinline__ float bf16_round(float x) { return bf16_bits_to_f32(f32_to_bf16_bits(x)); }

// ---- pooling ---------------------------------------------------------------------
// One CTA = one tile x 8 heads x one of {Q, K, V}; thread = (head, four dims = 8 bytes), so
// every token row contributes one contiguous 2 KB read per CTA and each thread keeps 64
// independent 8-byte loads in flight. The per-dimension summation order is the reference's
// (cuda/vsa.cuh:22-42): 4 lanes x 4 slot accumulators, element i = lane + 4*slot + 16*round,
// ((a0+a1)+a2)+a3 per lane, (l0+l2)+(l1+l3), then / size.
struct PoolArgs {
    const uint2 *src[3];
    uint2 *tiled[3];
    float *pooled[3];
};

__global__ void __launch_bounds__(256)
tile_pool_kernel(PoolArgs a, const int *__restrict__ map, const int *__restrict__ sizes, int tiles,
                 int heads) {
    __shared__ int rows[VT];
    const int tile = blockIdx.x, which = blockIdx.z;
    const int head = blockIdx.y * 8 + (threadIdx.x >> 5), dq = threadIdx.x & 31;
    if (threadIdx.x < VT) rows[threadIdx.x] = map[tile * VT + threadIdx.x];
    __syncthreads();
    if (head >= heads) return;
    const uint2 *src = which == 0 ? a.src[0] : which == 1 ? a.src[1] : a.src[2];
    uint2 *tiled = which == 0 ? a.tiled[0] : which == 1 ? a.tiled[1] : a.tiled[2];
    float *pooled = which == 0 ? a.pooled[0] : which == 1 ? a.pooled[1] : a.pooled[2];
    float lane_sum[4][4];   // [lane][dim]
#pragma unroll
    for (int lane = 0; lane < 4; lane++) {
        float acc[4][4];    // [slot][dim]
#pragma unroll
        for (int slot = 0; slot < 4; slot++)
#pragma unroll
            for (int d = 0; d < 4; d++) acc[slot][d] = 0.0f;
#pragma unroll
        for (int round = 0; round < 4; round++) {
#pragma unroll
            for (int slot = 0; slot < 4; slot++) {
                const int i = lane + slot * 4 + round * 16;
                const int row = rows[i];
                uint2 x = make_uint2(0u, 0u);
                if (row >= 0) x = __ldg(src + ((size_t)row * heads + head) * (VD / 4) + dq);
                if (tiled) tiled[((size_t)head * tiles * VT + tile * VT + i) * (VD / 4) + dq] = x;
                acc[slot][0] += bf16_bits_to_f32(x.x & 0xffffu);
                acc[slot][1] += bf16_bits_to_f32(x.x >> 16);
                acc[slot][2] += bf16_bits_to_f32(x.y & 0xffffu);
                acc[slot][3] += bf16_bits_to_f32(x.y >> 16);
            }
        }
#pragma unroll
        for (int d = 0; d < 4; d++)
            lane_sum[lane][d] = ((acc[0][d] + acc[1][d]) + acc[2][d]) + acc[3][d];
    }
    const float size = (float)sizes[tile];
    float4 mean;
    mean.x = ((lane_sum[0][0] + lane_sum[2][0]) + (lane_sum[1][0] + lane_sum[3][0])) / size;
    mean.y = ((lane_sum[0][1] + lane_sum[2][1]) + (lane_sum[1][1] + lane_sum[3][1])) / size;
    mean.z = ((lane_sum[0][2] + lane_sum[2][2]) + (lane_sum[1][2] + lane_sum[3][2])) / size;
    mean.w = ((lane_sum[0][3] + lane_sum[2][3]) + (lane_sum[1][3] + lane_sum[3][3])) / size;
    reinterpret_cast<float4 *>(pooled)[((size_t)head * tiles + tile) * (VD / 4) + dq] = mean;
}

// ---- scores + top-k selection + compression -----------------------------------------
constexpr int CHUNK = 64;    // pooled K/V rows staged per step
constexpr int PADDED = VD + 4;  // 16-byte aligned rows; float4 reads of 8 consecutive rows hit 32 distinct banks

// Order-preserving key of a float, the one cub's radix sort uses: larger float -> larger key.
__device__ __forceinline__ uint32_t sort_key(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// One CTA = 8 * QPW query tiles of one head, 8 warps; warp w owns query tiles w, w + 8, ...
// for selection, softmax and compression. Pooled K (then V) rows stream through shared
// memory in chunks of 32, the next chunk's global loads in flight while the current one is
// used, so each pooled row is read from L2 once per 8 * QPW query tiles.
//   scores row = scale * fmaf-chain over d = 0..127 (ascending), one fixed order.
//   Selection (cuda/vsa.cuh:47-76): prefix query tiles keep all tiles; video query tiles keep
//   all prefix tiles plus the `keep` best video tiles (ties: lower index first), ascending.
//   Compression (cuda/vsa.cuh:80-166,291-294): softmax over the whole row in the ATen lane
//   order, then sum_k p[k] * poolv[k][:] as one fmaf chain over k ascending.
template <int QPW>
__global__ void __launch_bounds__(256)
score_select_kernel(const float *__restrict__ poolq, const float *__restrict__ poolk,
                    const float *__restrict__ poolv, float *__restrict__ scores_out,
                    int *__restrict__ indices, int *__restrict__ counts,
                    float *__restrict__ compression, int tiles, int prefix, int keep, float scale) {
    constexpr int QT = 8 * QPW;
    extern __shared__ float sm[];
    float *row_scores = sm;                               // [QT][tiles]
    float *stage = row_scores + (size_t)QT * tiles;       // [CHUNK][PADDED]
    float *qrows = stage + CHUNK * PADDED;                // [QT][VD]

    const int head = blockIdx.y, qt0 = blockIdx.x * QT;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nq = min(QT, tiles - qt0);
    const float *pk = poolk + (size_t)head * tiles * VD;

    for (int i = tid; i < QT * VD; i += 256) {
        const int qi = i / VD;
        qrows[i] = qi < nq ? poolq[((size_t)head * tiles + qt0 + qi) * VD + (i % VD)] : 0.0f;
    }
    // ---- scores: thread = (key row r of the chunk, query group); 4 * QPW dot products per
    // thread from float4 shared-memory reads (the pass is bound by shared-memory wavefronts:
    // 4 for the key vector + 1 per broadcast query vector feed 16 * QPW FMAs) ----
    {
        constexpr int NQ = 4 * QPW;            // query rows per thread: group + 4 g... (QT / 4)
        constexpr int PER_THREAD = CHUNK * VD / 256;
        float next[PER_THREAD];   // this thread's elements of the chunk being fetched
        auto fetch = [&](int k0) {
#pragma unroll
            for (int u = 0; u < PER_THREAD; u++) {
                const int i = tid + u * 256, r = i / VD, d = i % VD;
                next[u] = k0 + r < tiles ? __ldg(pk + (size_t)(k0 + r) * VD + d) : 0.0f;
            }
        };
        fetch(0);
        const int r = tid & (CHUNK - 1), group = tid / CHUNK;   // 64 key rows x 4 query groups
        for (int k0 = 0; k0 < tiles; k0 += CHUNK) {
            __syncthreads();   // previous chunk fully consumed
#pragma unroll
            for (int u = 0; u < PER_THREAD; u++) {
                const int i = tid + u * 256;
                stage[(i / VD) * PADDED + (i % VD)] = next[u];
            }
            __syncthreads();
            if (k0 + CHUNK < tiles) fetch(k0 + CHUNK);
            if (k0 + r < tiles) {
                const float4 *kr = reinterpret_cast<const float4 *>(stage + r * PADDED);
                float dot[NQ];
#pragma unroll
                for (int g = 0; g < NQ; g++) dot[g] = 0.0f;
#pragma unroll 4
                for (int d4 = 0; d4 < VD / 4; d4++) {
                    const float4 kv = kr[d4];
#pragma unroll
                    for (int g = 0; g < NQ; g++) {
                        const float4 qv = reinterpret_cast<const float4 *>(qrows + (group + 4 * g) * VD)[d4];
                        dot[g] = fmaf(qv.x, kv.x, dot[g]);
                        dot[g] = fmaf(qv.y, kv.y, dot[g]);
                        dot[g] = fmaf(qv.z, kv.z, dot[g]);
                        dot[g] = fmaf(qv.w, kv.w, dot[g]);
                    }
                }
#pragma unroll
                for (int g = 0; g < NQ; g++)
                    if (group + 4 * g < nq) row_scores[(size_t)(group + 4 * g) * tiles + k0 + r] = scale * dot[g];
            }
        }
    }
    __syncthreads();

    // ---- selection and pooled softmax: warp `warp` owns query tiles qt0 + warp + 8 g ----
#pragma unroll 1
    for (int g = 0; g < QPW; g++) {
        const int qi = warp + 8 * g;
        if (qi >= nq) break;
        const int qt = qt0 + qi;
        float *mine = row_scores + (size_t)qi * tiles;
        const size_t row = (size_t)head * tiles + qt;
        if (scores_out)
            for (int j = lane; j < tiles; j += 32) scores_out[row * tiles + j] = mine[j];
        int *dst = indices + row * tiles;
        if (qt < prefix) {
            for (int j = lane; j < tiles; j += 32) dst[j] = j;
            if (lane == 0) counts[row] = tiles;
        } else {
            // The keep-th largest key among the video tiles, found bit by bit from the top:
            // `want` grows by a bit whenever at least `keep` keys are still >= the candidate.
            // Counting is a compare per key and one warp reduction per bit - no shared-memory
            // histogram, no atomics.
            uint32_t want = 0u;
            int greater = 0;
            if (tiles - prefix <= 32 * 32) {
                // up to 1024 video tiles: this lane's keys live in registers for all 33 passes
                uint32_t key[32];
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    const int j = prefix + lane + 32 * i;
                    key[i] = j < tiles ? sort_key(mine[j]) : 0u;   // 0 is below every real key
                }
                for (int bit = 31; bit >= 0; bit--) {
                    const uint32_t candidate = want | (1u << bit);
                    int count = 0;
#pragma unroll
                    for (int i = 0; i < 32; i++) count += key[i] >= candidate;
                    if (__reduce_add_sync(0xffffffffu, count) >= keep) want = candidate;
                }
#pragma unroll
                for (int i = 0; i < 32; i++) greater += key[i] > want;
                greater = __reduce_add_sync(0xffffffffu, greater);
            } else {
                for (int bit = 31; bit >= 0; bit--) {
                    const uint32_t candidate = want | (1u << bit);
                    int count = 0;
                    for (int j = prefix + lane; j < tiles; j += 32) count += sort_key(mine[j]) >= candidate;
                    if (__reduce_add_sync(0xffffffffu, count) >= keep) want = candidate;
                }
                for (int j = prefix + lane; j < tiles; j += 32) greater += sort_key(mine[j]) > want;
                greater = __reduce_add_sync(0xffffffffu, greater);
            }
            const int remaining = keep - greater;   // how many keys equal to `want` to take
            // Take every larger key and the first `remaining` equal keys in index order;
            // emit ascending.
            int written = 0, equal_seen = 0;
            for (int base = 0; base < tiles; base += 32) {
                const int j = base + lane;
                bool take = false, equal = false;
                if (j < tiles) {
                    if (j < prefix) {
                        take = true;
                    } else {
                        const uint32_t key = sort_key(mine[j]);
                        take = key > want;
                        equal = key == want;
                    }
                }
                const unsigned eq_mask = __ballot_sync(0xffffffffu, equal);
                if (equal && equal_seen + __popc(eq_mask & ((1u << lane) - 1u)) < remaining)
                    take = true;
                equal_seen += __popc(eq_mask);
                const unsigned take_mask = __ballot_sync(0xffffffffu, take);
                if (take) dst[written + __popc(take_mask & ((1u << lane) - 1u))] = j;
                written += __popc(take_mask);
            }
            if (lane == 0) counts[row] = written;
        }
        if (!compression) continue;

        // pooled softmax, in place, ATen reduction order
        float largest = -CUDART_INF_F, total = 0.0f;
        for (int j = lane; j < tiles; j += 32) largest = fmaxf(largest, mine[j]);
#pragma unroll
        for (int o = 16; o; o >>= 1)
            largest = fmaxf(largest, __shfl_xor_sync(0xffffffffu, largest, o));
        if (tiles <= 2048) {
            for (int j = lane; j < tiles; j += 32) {
                const float e = expf(mine[j] - largest);
                mine[j] = e;
                total += e;
            }
#pragma unroll
            for (int o = 16; o; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
        } else {
            // 1024-thread two-level shuffle-down order of the reference's block variant:
            // virtual thread t = w*32 + lane sums columns t, t+1024, ...
            float warp_sums = 0.0f;  // lane w keeps virtual warp w's sum
            for (int w = 0; w < 32; w++) {
                float part = 0.0f;
                for (int i = 0; i < 4; i++) {
                    const int col = w * 32 + lane + i * 1024;
                    if (col < tiles) part += expf(mine[col] - largest);
                }
#pragma unroll
                for (int o = 16; o; o >>= 1) part += __shfl_down_sync(0xffffffffu, part, o);
                part = __shfl_sync(0xffffffffu, part, 0);
                if (lane == w) warp_sums = part;
            }
#pragma unroll
            for (int o = 16; o; o >>= 1) warp_sums += __shfl_down_sync(0xffffffffu, warp_sums, o);
            total = __shfl_sync(0xffffffffu, warp_sums, 0);
            for (int j = lane; j < tiles; j += 32) mine[j] = expf(mine[j] - largest);
        }
        __syncwarp();
        for (int j = lane; j < tiles; j += 32) mine[j] = mine[j] / total;
    }
    if (!compression) return;

    // ---- compression: lane owns dims 4*lane..4*lane+3 of each of its warp's query tiles ----
    const float *pv = poolv + (size_t)head * tiles * VD;
    float4 acc[QPW];
#pragma unroll
    for (int g = 0; g < QPW; g++) acc[g] = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 *stage4 = reinterpret_cast<float4 *>(stage);  // [CHUNK][VD/4], unpadded reuse
    constexpr int PER_THREAD4 = CHUNK * (VD / 4) / 256;
    float4 next4[PER_THREAD4];
    auto fetch4 = [&](int k0) {
#pragma unroll
        for (int u = 0; u < PER_THREAD4; u++) {
            const int i = tid + u * 256, r = i / (VD / 4);
            next4[u] = k0 + r < tiles
                           ? __ldg(reinterpret_cast<const float4 *>(pv + (size_t)(k0 + r) * VD) + i % (VD / 4))
                           : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    fetch4(0);
    for (int k0 = 0; k0 < tiles; k0 += CHUNK) {
        __syncthreads();
#pragma unroll
        for (int u = 0; u < PER_THREAD4; u++) stage4[tid + u * 256] = next4[u];
        __syncthreads();
        if (k0 + CHUNK < tiles) fetch4(k0 + CHUNK);
        const int n = min(CHUNK, tiles - k0);
        for (int r = 0; r < n; r++) {
            const float4 vv = stage4[r * (VD / 4) + lane];
#pragma unroll
            for (int g = 0; g < QPW; g++) {
                const float pr = row_scores[(size_t)(warp + 8 * g) * tiles + k0 + r];
                acc[g].x = fmaf(pr, vv.x, acc[g].x);
                acc[g].y = fmaf(pr, vv.y, acc[g].y);
                acc[g].z = fmaf(pr, vv.z, acc[g].z);
                acc[g].w = fmaf(pr, vv.w, acc[g].w);
            }
        }
    }
#pragma unroll
    for (int g = 0; g < QPW; g++)
        if (warp + 8 * g < nq)
            reinterpret_cast<float4 *>(compression + ((size_t)head * tiles + qt0 + warp + 8 * g) * VD)[lane] = acc[g];
}

// ---- merge ---------------------------------------------------------------------------
// out[row][h][:] = bf16(fmaf(bf16_round(compression[h][tile][:]), gate[row][h][:], sparse))
// for every non-padded tiled row (cuda/vsa.cuh:168-181); one 16-byte vector per thread.
__global__ void __launch_bounds__(256)
untile_merge_kernel(uint4 *__restrict__ output, const uint4 *__restrict__ tiled,
                    const uint4 *__restrict__ gate, const float *__restrict__ compression,
                    const int *__restrict__ map, int tiles, int heads) {
    const size_t total = (size_t)tiles * VT * heads * (VD / 8);
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int v = (int)(i % (VD / 8));
    const int head = (int)((i / (VD / 8)) % heads);
    const int padded = (int)(i / ((size_t)(VD / 8) * heads));
    const int row = map[padded];
    if (row < 0) return;
    const uint4 x = tiled[((size_t)head * tiles * VT + padded) * (VD / 8) + v];
    const size_t dst = ((size_t)row * heads + head) * (VD / 8) + v;
    const uint4 gt = gate[dst];
    const float4 *cp = reinterpret_cast<const float4 *>(
        compression + ((size_t)head * tiles + padded / VT) * VD + v * 8);
    const float4 c0 = cp[0], c1 = cp[1];
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const uint32_t xs[4] = {x.x, x.y, x.z, x.w}, gs[4] = {gt.x, gt.y, gt.z, gt.w};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const float lo = fmaf(bf16_round(c[2 * k]), bf16_bits_to_f32(gs[k] & 0xffffu),
                              bf16_bits_to_f32(xs[k] & 0xffffu));
        const float hi = fmaf(bf16_round(c[2 * k + 1]), bf16_bits_to_f32(gs[k] >> 16),
                              bf16_bits_to_f32(xs[k] >> 16));
        o[k] = f32_to_bf16_bits(lo) | (f32_to_bf16_bits(hi) << 16);
    }
    output[dst] = make_uint4(o[0], o[1], o[2], o[3]);
}

}  // namespace

cudaError_t vsa_tile_pool3(const void *const src[3], void *const tiled[3], float *const pooled[3],
                           const int *map, const int *sizes, int tiles, int heads, int count,
                           cudaStream_t stream) {
    PoolArgs a{};
    for (int i = 0; i < count; i++) {
        a.src[i] = static_cast<const uint2 *>(src[i]);
        a.tiled[i] = static_cast<uint2 *>(tiled[i]);
        a.pooled[i] = pooled[i];
    }
    dim3 grid(tiles, (heads + 7) / 8, count);
    tile_pool_kernel<<<grid, 256, 0, stream>>>(a, map, sizes, tiles, heads);
    return cudaGetLastError();
}

static size_t score_select_smem(int tiles, int qt) {
    return sizeof(float) * ((size_t)qt * tiles + CHUNK * PADDED + (size_t)qt * VD);
}

template <int QPW>
static cudaError_t launch_score_select(const float *poolq, const float *poolk, const float *poolv,
                                       float *scores, int *indices, int *counts, float *compression,
                                       int tiles, int prefix, int keep, int heads, float scale,
                                       cudaStream_t stream) {
    constexpr int QT = 8 * QPW;
    static thread_local int configured_device = -1;
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    if (configured_device != device) {
        e = cudaFuncSetAttribute(score_select_kernel<QPW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)score_select_smem(QPW == 1 ? 4096 : 2048, QT));
        if (e != cudaSuccess) return e;
        configured_device = device;
    }
    dim3 grid((tiles + QT - 1) / QT, heads);
    score_select_kernel<QPW><<<grid, 256, score_select_smem(tiles, QT), stream>>>(
        poolq, poolk, poolv, scores, indices, counts, compression, tiles, prefix, keep, scale);
    return cudaGetLastError();
}

cudaError_t vsa_score_select_compress(const float *poolq, const float *poolk, const float *poolv,
                                      float *scores, int *indices, int *counts,
                                      float *compression, int tiles, int prefix, int keep,
                                      int heads, float scale, cudaStream_t stream) {
    if (tiles < 1 || tiles > 4096 || keep < 1 || prefix < 0 || prefix > tiles)
        return cudaErrorInvalidValue;
    // 16 query tiles per CTA up to 1400 tiles (two such CTAs share an SM up to about 1130 tiles,
    // one beyond), 8 per CTA beyond that: the score rows of a CTA must fit its shared memory.
    // The kernel is latency-bound (fixed-order fmaf chains, a 32-round threshold search), so its
    // time is about one CTA's time as long as every CTA is resident: with few heads (a rank's share
    // under sequence parallelism) 8 tiles per CTA halve that time and still fill the GPU.
    static thread_local int sms_device = -1, sms = 0;
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e == cudaSuccess && device != sms_device) {
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (e == cudaSuccess) sms_device = device;
    }
    if (e != cudaSuccess) return e;
    if (tiles <= 1400 && (size_t)((tiles + 15) / 16) * heads >= (size_t)4 * sms)
        return launch_score_select<2>(poolq, poolk, poolv, scores, indices, counts, compression, tiles,
                                      prefix, keep, heads, scale, stream);
    return launch_score_select<1>(poolq, poolk, poolv, scores, indices, counts, compression, tiles,
                                  prefix, keep, heads, scale, stream);
}

cudaError_t vsa_untile_merge(void *output, const void *tiled, const void *gate,
                             const float *compression, const int *map, int tiles, int heads,
                             cudaStream_t stream) {
    const size_t total = (size_t)tiles * VT * heads * (VD / 8);
    const size_t blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffu) return cudaErrorInvalidValue;
    untile_merge_kernel<<<(unsigned)blocks, 256, 0, stream>>>(
        static_cast<uint4 *>(output), static_cast<const uint4 *>(tiled),
        static_cast<const uint4 *>(gate), compression, map, tiles, heads);
    return cudaGetLastError();
}

}  // namespace h3b

// ---- top-k tile selection without any allocation -----------------------------------
// For callers that may not allocate device memory at the point of the call: code running
// inside someone else's memory plan (a fixed arena handed out once at start-up), under a
// memory-capped container where a late allocation can fail, or on a real-time path where
// the driver's allocator lock is not acceptable. The pooled means of Q and K - the only
// intermediate the selection needs - live in one file-scope device array instead of buffers
// owned by an h3_gpu_vsa object.
namespace h3b {
namespace {
constexpr unsigned STATIC_TOPK_MAX_ROWS = 8192;  // heads * tiles
// [2][heads * tiles][128] f32 = 8 MiB, resident on every GPU that loads the library.
static __device__ __align__(256) float g_topk_pool[2 * (size_t)STATIC_TOPK_MAX_ROWS * VD];
thread_local char g_topk_error[160] = "";
}  // namespace
}  // namespace h3b

extern "C" const char *h3b_vsa_topk_static_error(void) { return h3b::g_topk_error; }

extern "C" cudaError_t h3b_vsa_topk_static(const void *query, const void *key, const int *map,
                                           const int *sizes, int *indices, int *counts,
                                           unsigned tiles, unsigned prefix, unsigned keep,
                                           unsigned heads, cudaStream_t stream) {
    using namespace h3b;
    g_topk_error[0] = 0;
    if (!query || !key || !map || !sizes || !indices || !counts) {
        snprintf(g_topk_error, sizeof g_topk_error, "h3b_vsa_topk_static: null pointer argument");
        return cudaErrorInvalidValue;
    }
    if (!tiles || !heads || tiles > 4096u || prefix > tiles || !keep || keep > tiles - prefix) {
        snprintf(g_topk_error, sizeof g_topk_error,
                 "h3b_vsa_topk_static: bad geometry (tiles %u, prefix %u, keep %u, heads %u)", tiles,
                 prefix, keep, heads);
        return cudaErrorInvalidValue;
    }
    if ((size_t)heads * tiles > STATIC_TOPK_MAX_ROWS) {
        snprintf(g_topk_error, sizeof g_topk_error,
                 "h3b_vsa_topk_static: heads * tiles = %zu exceeds the static scratch limit of %u",
                 (size_t)heads * tiles, STATIC_TOPK_MAX_ROWS);
        return cudaErrorInvalidValue;
    }
    // Device address of the scratch array, resolved once per device with that device current.
    // (In host code the array's name is only a handle for the runtime, not an address.)
    static float *pool_of_device[64] = {};
    // every failing return leaves its reason in the thread's error text
    auto failed = [](cudaError_t code, const char *where) {
        snprintf(g_topk_error, sizeof g_topk_error, "h3b_vsa_topk_static: %s: %s", where, cudaGetErrorString(code));
        return code;
    };
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return failed(e, "current device");
    if (device < 0 || device >= 64) return failed(cudaErrorInvalidDevice, "device ordinal above 63");
    float *pool = __atomic_load_n(&pool_of_device[device], __ATOMIC_ACQUIRE);
    if (!pool) {
        e = cudaGetSymbolAddress(reinterpret_cast<void **>(&pool), g_topk_pool);
        if (e != cudaSuccess) return failed(e, "address of the static scratch");
        __atomic_store_n(&pool_of_device[device], pool, __ATOMIC_RELEASE);
    }
    float *poolq = pool, *poolk = pool + (size_t)STATIC_TOPK_MAX_ROWS * VD;
    const void *src[3] = {query, key, nullptr};
    void *no_tiled[3] = {nullptr, nullptr, nullptr};
    float *pooled[3] = {poolq, poolk, nullptr};
    e = vsa_tile_pool3(src, no_tiled, pooled, map, sizes, (int)tiles, (int)heads, 2, stream);
    if (e != cudaSuccess) return failed(e, "pooling launch");
    e = vsa_score_select_compress(poolq, poolk, nullptr, nullptr, indices, counts, nullptr, (int)tiles,
                                  (int)prefix, (int)keep, (int)heads, 1.0f / sqrtf(128.0f), stream);
    return e == cudaSuccess ? e : failed(e, "selection launch");
}
