/*
 * CPU oracle for the H3-omni DiT attention path. TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C with FP32 arithmetic, what the reference's
 * GPU attention path computes. It is the checker for the CUDA library: only
 * the test-suite, the smoke check and the CPU-baseline leg of the benchmark
 * may load it. Nothing the library ships calls into it.
 *
 * The reference has no CPU attention path. Pins of this restatement:
 *   - golden outputs of the reference's own CUDA code (FP32 fallback attention, tile pooling,
 *     cuBLAS pooled scores + softmax, block selection, compression), produced on a B200 by
 *     tests/golden/make_reference_fixtures.py and checked on CPU by tests/test_golden.py;
 *   - the same reference code run live on the GPU box (oracle/ref_build.py,
 *     tests/test_reference_backend.py).
 * The reference's dense and fine-stage kernels live in un-vendored third-party trees
 * (FlashAttention 979702c / v2.8.3 060c918, ThunderKittens 6c27e28) and are sm_90a-only:
 * bit-level parity with THOSE kernels is unpinned; for them the reference's own acceptance
 * thresholds apply (tests/pytorch/acceptance.json:5-8, tests/live/attention.py:38,
 * tests/fasth3/vsa.py:131).
 *
 * Each function cites the reference file:line it follows.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_API __attribute__((visibility("default")))
#define VSA_D 128
#define VSA_TILE 64

/* ---- bf16 / fp16 scalar conversions ------------------------------------ */

/* cuda/primitives.cuh:218-224: widen by shifting; narrow with round-to-nearest-even. */
static inline float bf16_to_f32(uint16_t x) {
    uint32_t u = (uint32_t)x << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff; /* NaN, as __float2bfloat16_rn */
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
static inline float bf16_round(float f) { return bf16_to_f32(f32_to_bf16(f)); }
static inline float f16_to_f32(uint16_t x) {
    _Float16 h;
    memcpy(&h, &x, 2);
    return (float)h;
}
static inline uint16_t f32_to_f16(float f) {
    _Float16 h = (_Float16)f;
    uint16_t x;
    memcpy(&x, &h, 2);
    return x;
}

ORACLE_API void oracle_f32_to_bf16(const float *in, uint16_t *out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = f32_to_bf16(in[i]);
}
ORACLE_API void oracle_bf16_to_f32(const uint16_t *in, float *out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = bf16_to_f32(in[i]);
}
ORACLE_API void oracle_f32_to_f16(const float *in, uint16_t *out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = f32_to_f16(in[i]);
}
ORACLE_API void oracle_f16_to_f32(const uint16_t *in, float *out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = f16_to_f32(in[i]);
}

/* ---- seeded synthetic inputs -------------------------------------------- */

static inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
/* Counter-based N(0,1) -> bf16: element i of stream `seed` depends on (seed, i) only. */
ORACLE_API void oracle_fill_normal_bf16(uint16_t *out, size_t n, uint64_t seed, float sigma) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i += 2) {
        uint64_t r = splitmix64(seed * 0xD1342543DE82EF95ull + (i >> 1));
        float u1 = ((float)(uint32_t)(r >> 40) + 0.5f) * (1.0f / 16777216.0f);
        float u2 = ((float)(uint32_t)((r >> 8) & 0xffffffu) + 0.5f) * (1.0f / 16777216.0f);
        float radius = sqrtf(-2.0f * logf(u1)) * sigma;
        float angle = 6.28318530717958647692f * u2;
        out[i] = f32_to_bf16(radius * cosf(angle));
        if (i + 1 < n) out[i + 1] = f32_to_bf16(radius * sinf(angle));
    }
}

/* ---- dense / rectangular / causal / GQA attention ----------------------- */

/*
 * FP32 attention over token-major tensors, the arithmetic of the reference's
 * FP32 fallback (cuda/h3_gpu_cuda.cu:1131-1180): S = scale * (Q.K^T) in fp32,
 * row max, expf(x - max), row sum, divide (softmax_rows, :1065-1101), then
 * P.V in fp32. Causal masks key > query (:1071). GQA maps query head h to
 * kv head h / (heads / kv_heads) (pack_heads, :1055).
 *
 * q, out: [batch][lq][heads][dim]; k, v: [batch][lk][kv_heads][dim].
 * elem: 0 = bf16, 1 = fp16. out_f32 may be NULL; out_16 may be NULL.
 * lse (may be NULL): [batch][heads][lq] = max*scale + log(sum), the
 * FlashAttention convention written by h3_flash*_bf16.
 */
ORACLE_API void oracle_attention(float *out_f32, uint16_t *out_16, float *lse, const uint16_t *q,
                                 const uint16_t *k, const uint16_t *v, int batch, int lq, int lk,
                                 int heads, int kv_heads, int dim, float scale, int causal,
                                 int elem) {
    const int group = heads / kv_heads;
#pragma omp parallel
    {
        float *s = (float *)malloc(sizeof(float) * (size_t)lk);
        float qf[256], acc[256];
#pragma omp for collapse(3) schedule(dynamic, 8)
        for (int b = 0; b < batch; b++)
            for (int h = 0; h < heads; h++)
                for (int i = 0; i < lq; i++) {
                    const int kh = h / group;
                    const uint16_t *qrow = q + (((size_t)b * lq + i) * heads + h) * dim;
                    for (int d = 0; d < dim; d++)
                        qf[d] = elem ? f16_to_f32(qrow[d]) : bf16_to_f32(qrow[d]);
                    int limit = causal ? (i + 1 < lk ? i + 1 : lk) : lk;
                    float m = -INFINITY;
                    for (int j = 0; j < limit; j++) {
                        const uint16_t *krow = k + (((size_t)b * lk + j) * kv_heads + kh) * dim;
                        float dot = 0.0f;
                        if (elem) {
#pragma omp simd reduction(+ : dot)
                            for (int d = 0; d < dim; d++) dot += qf[d] * f16_to_f32(krow[d]);
                        } else {
#pragma omp simd reduction(+ : dot)
                            for (int d = 0; d < dim; d++) dot += qf[d] * bf16_to_f32(krow[d]);
                        }
                        s[j] = scale * dot;
                        m = fmaxf(m, s[j]);
                    }
                    float sum = 0.0f;
                    for (int j = 0; j < limit; j++) {
                        s[j] = expf(s[j] - m);
                        sum += s[j];
                    }
                    for (int d = 0; d < dim; d++) acc[d] = 0.0f;
                    for (int j = 0; j < limit; j++) {
                        const uint16_t *vrow = v + (((size_t)b * lk + j) * kv_heads + kh) * dim;
                        float p = s[j] / sum;
                        for (int d = 0; d < dim; d++)
                            acc[d] += p * (elem ? f16_to_f32(vrow[d]) : bf16_to_f32(vrow[d]));
                    }
                    size_t o = (((size_t)b * lq + i) * heads + h) * dim;
                    for (int d = 0; d < dim; d++) {
                        if (out_f32) out_f32[o + d] = acc[d];
                        if (out_16) out_16[o + d] = elem ? f32_to_f16(acc[d]) : f32_to_bf16(acc[d]);
                    }
                    if (lse) lse[((size_t)b * heads + h) * lq + i] = m + logf(sum);
                }
        free(s);
    }
}

/*
 * Sampled-row check with FP64 accumulation, the scheme of the reference's
 * attention microbenchmark (tests/serving/profile/attn_bench.cu:23-55): for
 * `count` query rows listed in `rows`, every head, recompute the output row
 * in double precision. out: [count][heads][dim] f32.
 */
ORACLE_API void oracle_attention_rows_f64(float *out, const int *rows, int count,
                                          const uint16_t *q, const uint16_t *k,
                                          const uint16_t *v, int lq, int lk, int heads,
                                          int kv_heads, int dim, float scale) {
    const int group = heads / kv_heads;
    (void)lq;
#pragma omp parallel
    {
        double *s = (double *)malloc(sizeof(double) * (size_t)lk);
        double acc[256];
#pragma omp for collapse(2) schedule(dynamic, 1)
        for (int r = 0; r < count; r++)
            for (int h = 0; h < heads; h++) {
                const int kh = h / group;
                const uint16_t *qrow = q + ((size_t)rows[r] * heads + h) * dim;
                double m = -INFINITY;
                for (int j = 0; j < lk; j++) {
                    const uint16_t *krow = k + ((size_t)j * kv_heads + kh) * dim;
                    double dot = 0.0;
                    for (int d = 0; d < dim; d++)
                        dot += (double)bf16_to_f32(qrow[d]) * (double)bf16_to_f32(krow[d]);
                    s[j] = dot * (double)scale;
                    if (s[j] > m) m = s[j];
                }
                double sum = 0.0;
                for (int j = 0; j < lk; j++) {
                    s[j] = exp(s[j] - m);
                    sum += s[j];
                }
                for (int d = 0; d < dim; d++) acc[d] = 0.0;
                for (int j = 0; j < lk; j++) {
                    const uint16_t *vrow = v + ((size_t)j * kv_heads + kh) * dim;
                    for (int d = 0; d < dim; d++) acc[d] += s[j] * (double)bf16_to_f32(vrow[d]);
                }
                for (int d = 0; d < dim; d++)
                    out[((size_t)r * heads + h) * dim + d] = (float)(acc[d] / sum);
            }
        free(s);
    }
}

/* ---- video sparse attention: tile map ------------------------------------ */

/*
 * cuda/vsa.cuh:192-242. Text rows, then audio rows, in dense 64-row chunks
 * (prefix tiles); then 4x4x4 cubes of the (time, height, width) token grid in
 * (t, y, x) raster order, tokens inside a cube in (dt, dy, dx) order, padded
 * with -1 to 64. keep = max(1, (video_tiles + 9) / 10) (:242).
 * Returns the tile count, or -1 if the limits of :195-205 are violated.
 * map must hold tiles*64 ints and sizes tiles ints; call with map == NULL to
 * size them. info: [0] rows, [1] tiles, [2] prefix, [3] keep.
 */
ORACLE_API int oracle_vsa_map(int *map, int *sizes, int *info, unsigned text, unsigned audio,
                              unsigned time, unsigned height, unsigned width, unsigned heads) {
    if (!text || !audio || !time || !height || !width || !heads) return -1;
    uint64_t blocks = ((uint64_t)text + 63) / 64 + ((uint64_t)audio + 63) / 64;
    uint64_t nt = ((uint64_t)time + 3) / 4, nh = ((uint64_t)height + 3) / 4,
             nw = ((uint64_t)width + 3) / 4;
    if (blocks >= 4096 || nt > 4096 || nh > 4096 || nw > 4096 || blocks + nt * nh * nw > 4096 ||
        heads > 56)
        return -1;
    int tiles = 0, prefix = 0, cursor = 0;
    unsigned counts[2] = {text, audio};
    for (int c = 0; c < 2; c++) {
        unsigned count = counts[c];
        for (unsigned i = 0; i < count; i += 64) {
            int valid = (int)(count - i < 64 ? count - i : 64);
            if (map) {
                sizes[tiles] = valid;
                for (int j = 0; j < 64; j++)
                    map[tiles * 64 + j] = j < valid ? cursor + (int)i + j : -1;
            }
            tiles++;
            prefix++;
        }
        cursor += (int)count;
    }
    for (unsigned t = 0; t < time; t += 4)
        for (unsigned y = 0; y < height; y += 4)
            for (unsigned x = 0; x < width; x += 4) {
                int valid = 0;
                for (unsigned dt = t; dt < (time < t + 4 ? time : t + 4); dt++)
                    for (unsigned dy = y; dy < (height < y + 4 ? height : y + 4); dy++)
                        for (unsigned dx = x; dx < (width < x + 4 ? width : x + 4); dx++) {
                            if (map)
                                map[tiles * 64 + valid] =
                                    cursor + (int)((dt * height + dy) * width + dx);
                            valid++;
                        }
                if (map) {
                    sizes[tiles] = valid;
                    for (int j = valid; j < 64; j++) map[tiles * 64 + j] = -1;
                }
                tiles++;
            }
    int keep = (tiles - prefix + 9) / 10;
    if (keep < 1) keep = 1;
    info[0] = cursor + (int)(time * height * width);
    info[1] = tiles;
    info[2] = prefix;
    info[3] = keep;
    return tiles;
}

/* ---- VSA coarse stage ------------------------------------------------------ */

/*
 * cuda/vsa.cuh:18-43 (tile_pool): gather token rows into head-major tiles
 * [heads][tiles*64][128] (zero for padding) and the FP32 mean per tile with
 * the fixed order: four lanes, element i = lane + slot*4 + round*16, four
 * slot accumulators per lane summed ((a0+a1)+a2)+a3, lanes summed
 * (l0+l2)+(l1+l3), then divided by sizes[tile]. tiled may be NULL.
 */
ORACLE_API void oracle_vsa_tile_pool(const uint16_t *src, uint16_t *tiled, float *pooled,
                                     const int *map, const int *sizes, int tiles, int heads) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int tile = 0; tile < tiles; tile++)
        for (int head = 0; head < heads; head++)
            for (int d = 0; d < VSA_D; d++) {
                float lane_sum[4];
                for (int lane = 0; lane < 4; lane++) {
                    float acc[4] = {0, 0, 0, 0};
                    for (int round = 0; round < 4; round++)
                        for (int slot = 0; slot < 4; slot++) {
                            int i = lane + slot * 4 + round * 16;
                            int row = map[tile * VSA_TILE + i];
                            uint16_t x =
                                row < 0 ? 0 : src[((size_t)row * heads + head) * VSA_D + d];
                            if (tiled)
                                tiled[((size_t)head * tiles * VSA_TILE + tile * VSA_TILE + i) *
                                          VSA_D + d] = x;
                            acc[slot] += bf16_to_f32(x);
                        }
                    lane_sum[lane] = ((acc[0] + acc[1]) + acc[2]) + acc[3];
                }
                float sum = (lane_sum[0] + lane_sum[2]) + (lane_sum[1] + lane_sum[3]);
                pooled[((size_t)head * tiles + tile) * VSA_D + d] = sum / (float)sizes[tile];
            }
}

/*
 * cuda/vsa.cuh:281-284: scores[h][q][k] = scale * dot(poolq[h][q], poolk[h][k])
 * in FP32. The reference computes this with cuBLAS SGEMM, whose summation
 * order is not documented; this oracle fixes ONE order - a sequential fmaf
 * chain over d = 0..127 starting from 0, then one multiply by scale - which
 * the CUDA selection kernel reproduces exactly.
 */
ORACLE_API void oracle_vsa_scores(float *scores, const float *poolq, const float *poolk, int tiles,
                                  int heads, float scale) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int h = 0; h < heads; h++)
        for (int qt = 0; qt < tiles; qt++) {
            const float *a = poolq + ((size_t)h * tiles + qt) * VSA_D;
            for (int kt = 0; kt < tiles; kt++) {
                const float *b = poolk + ((size_t)h * tiles + kt) * VSA_D;
                float dot = 0.0f;
                for (int d = 0; d < VSA_D; d++) dot = fmaf(a[d], b[d], dot);
                scores[((size_t)h * tiles + qt) * tiles + kt] = scale * dot;
            }
        }
}

/* Radix-sort key order of cub::BlockRadixSort on floats: sign-flipped bit pattern. */
static inline uint32_t float_sort_key(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

/*
 * cuda/vsa.cuh:47-76 (select_blocks). Prefix query tiles keep every tile.
 * A video query tile keeps every prefix tile plus the `keep` video tiles with
 * the largest score; a stable descending sort decides ties (the lower tile
 * index wins, as a stable LSD radix sort over ascending input does); indices
 * are emitted ascending. indices: [heads][tiles][tiles], counts: [heads][tiles].
 */
ORACLE_API void oracle_vsa_select(const float *scores, int *indices, int *counts, int tiles,
                                  int prefix, int keep, int heads) {
#pragma omp parallel
    {
        uint32_t *key = (uint32_t *)malloc(sizeof(uint32_t) * (size_t)tiles);
        unsigned char *chosen = (unsigned char *)malloc((size_t)tiles);
#pragma omp for collapse(2) schedule(static)
        for (int h = 0; h < heads; h++)
            for (int qt = 0; qt < tiles; qt++) {
                size_t row = (size_t)h * tiles + qt;
                int *dst = indices + row * tiles;
                if (qt < prefix) {
                    for (int j = 0; j < tiles; j++) dst[j] = j;
                    counts[row] = tiles;
                    continue;
                }
                for (int j = 0; j < tiles; j++) {
                    chosen[j] = j < prefix;
                    key[j] = float_sort_key(scores[row * tiles + j]);
                }
                /* keep-times selection of the best remaining (largest key, lowest index) */
                for (int pick = 0; pick < keep; pick++) {
                    int best = -1;
                    for (int j = prefix; j < tiles; j++)
                        if (!chosen[j] && (best < 0 || key[j] > key[best])) best = j;
                    if (best < 0) break;
                    chosen[best] = 1;
                }
                int count = 0;
                for (int j = 0; j < tiles; j++)
                    if (chosen[j]) dst[count++] = j;
                counts[row] = count;
            }
        free(key);
        free(chosen);
    }
}

/* ---- VSA fine stage --------------------------------------------------------- */

/*
 * cuda/vendor/vsa_hopper_forward.cuh:68-270 (fwd_attend_ker<128>). For each
 * (query tile, head) walk indices[h][q][0..counts) in order; per KV tile:
 * S = Q.K^T (fp32), keys >= sizes[kv] set to -inf (:160), running max,
 * exp2((s - max) * scale*log2e) (:163-172), running sum rescaled by
 * exp2(old - new), P rounded to bf16 before P.V (:181), O rescaled (:182);
 * finally O / sum (:244) and lse = -sqrt(128) * (log(sum) + max*scale) (:254-259).
 * round_p = 0 keeps P in fp32 (the "exact" variant used as a second opinion).
 * q, k, v, out: [heads][tiles*64][128] bf16 (out_f32 optional, same shape).
 */
ORACLE_API void oracle_vsa_fine(uint16_t *out, float *out_f32, float *lse, const uint16_t *q,
                                const uint16_t *k, const uint16_t *v, const int *indices,
                                const int *counts, const int *sizes, int tiles, int heads,
                                int round_p) {
    const float c = 1.44269504089f * 0.08838834764f;
#pragma omp parallel for collapse(2) schedule(dynamic, 4)
    for (int h = 0; h < heads; h++)
        for (int qt = 0; qt < tiles; qt++) {
            size_t row = (size_t)h * tiles + qt;
            int n = counts[row];
            const int *list = indices + row * tiles;
            for (int r = 0; r < VSA_TILE; r++) {
                size_t qoff = ((size_t)h * tiles * VSA_TILE + (size_t)qt * VSA_TILE + r) * VSA_D;
                float qf[VSA_D], acc[VSA_D], s[VSA_TILE];
                for (int d = 0; d < VSA_D; d++) {
                    qf[d] = bf16_to_f32(q[qoff + d]);
                    acc[d] = 0.0f;
                }
                float m = -INFINITY, sum = 0.0f;
                for (int t = 0; t < n; t++) {
                    int kt = list[t];
                    int valid = sizes[kt];
                    size_t koff = ((size_t)h * tiles * VSA_TILE + (size_t)kt * VSA_TILE) * VSA_D;
                    float last = m;
                    for (int j = 0; j < VSA_TILE; j++) {
                        float dot = 0.0f;
                        for (int d = 0; d < VSA_D; d++)
                            dot += qf[d] * bf16_to_f32(k[koff + (size_t)j * VSA_D + d]);
                        s[j] = j < valid ? dot : -INFINITY;
                        m = fmaxf(m, s[j]);
                    }
                    float ms = m * c;
                    float rescale = exp2f(last * c - ms);
                    if (last == -INFINITY) rescale = 0.0f;
                    sum *= rescale;
                    for (int d = 0; d < VSA_D; d++) acc[d] *= rescale;
                    for (int j = 0; j < VSA_TILE; j++) {
                        float p = exp2f(s[j] * c - ms);
                        sum += p;
                        if (round_p) p = bf16_round(p);
                        if (p != 0.0f)
                            for (int d = 0; d < VSA_D; d++)
                                acc[d] += p * bf16_to_f32(v[koff + (size_t)j * VSA_D + d]);
                    }
                }
                for (int d = 0; d < VSA_D; d++) {
                    float o = acc[d] / sum;
                    if (out) out[qoff + d] = f32_to_bf16(o);
                    if (out_f32) out_f32[qoff + d] = o;
                }
                if (lse)
                    lse[(size_t)h * tiles * VSA_TILE + (size_t)qt * VSA_TILE + r] =
                        (logf(sum) + m * c * 0.69314718056f) * -11.313708499f;
            }
        }
}

/* ---- VSA compression branch and merge ------------------------------------- */

/*
 * cuda/vsa.cuh:80-166 (pooled softmax, ATen lane order) for tiles <= 2048:
 * lane l of 32 holds columns l, l+32, ...; max then sum are reduced per lane
 * in column order and across lanes by XOR butterflies 16,8,4,2,1. Above 2048
 * tiles the 1024-thread two-level shuffle-down order of :110-156 is used.
 * In place on scores [rows][tiles].
 */
static float butterfly(float *lanes, int is_max) {
    float cur[32], nxt[32];
    memcpy(cur, lanes, sizeof cur);
    for (int offset = 16; offset; offset /= 2) {
        for (int l = 0; l < 32; l++)
            nxt[l] = is_max ? fmaxf(cur[l], cur[l ^ offset]) : cur[l] + cur[l ^ offset];
        memcpy(cur, nxt, sizeof cur);
    }
    return cur[0];
}
/* __shfl_down reduction of 32 lanes; the value of lane 0 is the result (:114-118). */
static float shuffle_down(float *lanes, int is_max) {
    float cur[32], nxt[32];
    memcpy(cur, lanes, sizeof cur);
    for (int offset = 16; offset; offset /= 2) {
        for (int l = 0; l < 32; l++) {
            float other = l + offset < 32 ? cur[l + offset] : cur[l];
            nxt[l] = is_max ? fmaxf(cur[l], other) : cur[l] + other;
        }
        memcpy(cur, nxt, sizeof cur);
    }
    return cur[0];
}
static float block_reduce_1024(const float *values, int is_max) {
    float warp[32], tmp[32];
    for (int w = 0; w < 32; w++) {
        memcpy(tmp, values + w * 32, sizeof tmp);
        warp[w] = shuffle_down(tmp, is_max);
    }
    return shuffle_down(warp, is_max);
}
ORACLE_API void oracle_vsa_pooled_softmax(float *scores, int tiles, int rows) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++) {
        float *x = scores + (size_t)r * tiles;
        if (tiles <= 2048) {
            float lanes[32];
            for (int l = 0; l < 32; l++) {
                float m = -INFINITY;
                for (int col = l; col < tiles; col += 32) m = fmaxf(m, x[col]);
                lanes[l] = m;
            }
            float largest = butterfly(lanes, 1);
            for (int l = 0; l < 32; l++) {
                float sum = 0.0f;
                for (int col = l; col < tiles; col += 32) {
                    x[col] = expf(x[col] - largest);
                    sum += x[col];
                }
                /* padded columns hold expf(-inf - max) = 0 and add nothing */
                lanes[l] = sum;
            }
            float total = butterfly(lanes, 0);
            for (int col = 0; col < tiles; col++) x[col] = x[col] / total;
        } else {
            float part[1024];
            for (int t = 0; t < 1024; t++) {
                float m = -INFINITY;
                for (int i = 0; i < 4; i++) {
                    int col = t + i * 1024;
                    if (col < tiles) m = fmaxf(m, x[col]);
                }
                part[t] = m;
            }
            float largest = block_reduce_1024(part, 1);
            for (int t = 0; t < 1024; t++) {
                float sum = 0.0f;
                for (int i = 0; i < 4; i++) {
                    int col = t + i * 1024;
                    if (col < tiles) sum += expf(x[col] - largest);
                }
                part[t] = sum;
            }
            float total = block_reduce_1024(part, 0);
            for (int col = 0; col < tiles; col++) x[col] = expf(x[col] - largest) / total;
        }
    }
}

/*
 * cuda/vsa.cuh:291-294: compression[h][q][d] = sum_k prob[h][q][k] * poolv[h][k][d]
 * in FP32 (cuBLAS SGEMM in the reference; this oracle fixes a sequential fmaf
 * chain over k = 0..tiles-1, which the CUDA kernel reproduces).
 */
ORACLE_API void oracle_vsa_compress(float *compression, const float *prob, const float *poolv,
                                    int tiles, int heads) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int h = 0; h < heads; h++)
        for (int qt = 0; qt < tiles; qt++) {
            float acc[VSA_D];
            for (int d = 0; d < VSA_D; d++) acc[d] = 0.0f;
            const float *p = prob + ((size_t)h * tiles + qt) * tiles;
            for (int kt = 0; kt < tiles; kt++) {
                const float *vv = poolv + ((size_t)h * tiles + kt) * VSA_D;
                for (int d = 0; d < VSA_D; d++) acc[d] = fmaf(p[kt], vv[d], acc[d]);
            }
            memcpy(compression + ((size_t)h * tiles + qt) * VSA_D, acc, sizeof acc);
        }
}

/*
 * cuda/vsa.cuh:168-181 (untile_merge): for every non-padded tiled row,
 * out[row][h][d] = bf16(fmaf(bf16_round(compression[h][tile][d]), gate[row][h][d], sparse)).
 */
ORACLE_API void oracle_vsa_untile_merge(uint16_t *output, const uint16_t *tiled,
                                        const uint16_t *gate, const float *compression,
                                        const int *map, int tiles, int heads) {
#pragma omp parallel for schedule(static)
    for (int padded = 0; padded < tiles * VSA_TILE; padded++) {
        int row = map[padded];
        if (row < 0) continue;
        for (int h = 0; h < heads; h++)
            for (int d = 0; d < VSA_D; d++) {
                float x = bf16_to_f32(tiled[((size_t)h * tiles * VSA_TILE + padded) * VSA_D + d]);
                size_t dst = ((size_t)row * heads + h) * VSA_D + d;
                float c = bf16_round(
                    compression[((size_t)h * tiles + padded / VSA_TILE) * VSA_D + d]);
                output[dst] = f32_to_bf16(fmaf(c, bf16_to_f32(gate[dst]), x));
            }
    }
}

/* ---- Ulysses index algebra -------------------------------------------------- */

/* ---- Q/K RMS-norm + rotary embedding (the producer of q, k, v) ---------------- */

/*
 * cuda/primitives.cuh:897-962 with head_dim == 128 (and cuda/fast_primitives.cuh:184-265,
 * which the reference requires to be bit-identical to it). qkv: [rows][3][heads][128] or,
 * grouped, [rows][heads][3][128]; weights [128]; cos/sin [rows][rope_half]; outputs
 * [rows][heads][128]. Order of the sum of squares (:914-925): lane t of 32 chains fmaf over
 * dimensions 4t..4t+3, then a shuffle-down tree 16,8,4,2,1 whose lane 0 is the sum.
 * x * inverse * weight is rounded to bf16 (:935-939); dimension d < rope_half rotates with
 * d + rope_half, each product rounded to bf16 before the subtraction / addition (:940-959).
 * One deliberate difference: the GPU takes rsqrtf (an approximation, <= 2 ulp); this file
 * uses 1/sqrtf, so single outputs may differ from the GPU by one bf16 ulp where that last
 * bit of the inverse decides a rounding. Bit-level parity of the CUDA kernel is pinned
 * against the reference's own kernel run on the same GPU instead.
 */
ORACLE_API void oracle_qkv_rope(uint16_t *query, uint16_t *key, uint16_t *value, const uint16_t *qkv,
                                const uint16_t *q_weight, const uint16_t *k_weight,
                                const uint16_t *rope_cos, const uint16_t *rope_sin, int rows,
                                int heads, int rope_half, float epsilon, int grouped) {
    const size_t inner = (size_t)heads * 128;
#pragma omp parallel for schedule(static)
    for (int row = 0; row < rows; row++)
        for (int head = 0; head < heads; head++) {
            size_t base[3];
            base[0] = (size_t)row * inner * 3 + (size_t)head * 128;
            base[1] = base[0] + inner;
            base[2] = base[0] + inner * 2;
            if (grouped) {
                base[0] = (size_t)row * inner * 3 + (size_t)head * 128 * 3;
                base[1] = base[0] + 128;
                base[2] = base[1] + 128;
            }
            const size_t out = ((size_t)row * heads + head) * 128;
            for (int which = 0; which < 2; which++) {
                const uint16_t *x = qkv + base[which];
                const uint16_t *w = which ? k_weight : q_weight;
                uint16_t *y = (which ? key : query) + out;
                float lanes[32];
                for (int t = 0; t < 32; t++) {
                    float sum = 0.0f;
                    for (int d = 4 * t; d < 4 * t + 4; d++) sum = fmaf(bf16_to_f32(x[d]), bf16_to_f32(x[d]), sum);
                    lanes[t] = sum;
                }
                const float inverse = 1.0f / sqrtf(shuffle_down(lanes, 0) / 128.0f + epsilon);
                float normed[128];
                for (int d = 0; d < 128; d++)
                    normed[d] = bf16_round(bf16_to_f32(x[d]) * inverse * bf16_to_f32(w[d]));
                for (int d = 0; d < 128; d++) {
                    float r = normed[d];
                    if (d < rope_half) {
                        const float c = bf16_to_f32(rope_cos[(size_t)row * rope_half + d]);
                        const float s = bf16_to_f32(rope_sin[(size_t)row * rope_half + d]);
                        r = bf16_round(normed[d] * c) - bf16_round(normed[d + rope_half] * s);
                    } else if (d < 2 * rope_half) {
                        const float c = bf16_to_f32(rope_cos[(size_t)row * rope_half + d - rope_half]);
                        const float s = bf16_to_f32(rope_sin[(size_t)row * rope_half + d - rope_half]);
                        r = bf16_round(normed[d] * c) + bf16_round(normed[d - rope_half] * s);
                    }
                    y[d] = f32_to_bf16(r);
                }
            }
            memcpy(value + out, qkv + base[2], 128 * sizeof(uint16_t));
        }
}

/*
 * cuda/parallel.cuh:67-143. All ranks' buffers live in one address space here:
 * in: [ranks][rows][heads][dim] (rank r's row shard), out:
 * [ranks][ranks*rows][heads/ranks][dim] (rank r holds every row of its head
 * group). scatter: out[r][s*rows + i][g][:] = in[s][i][r*(heads/ranks) + g][:].
 * gather (inverse = 1) undoes it. Elements are 16-bit words.
 */
ORACLE_API void oracle_ulysses(uint16_t *out, const uint16_t *in, int ranks, int rows, int heads,
                               int dim, int inverse) {
    int hg = heads / ranks;
    for (int r = 0; r < ranks; r++)
        for (int s = 0; s < ranks; s++)
            for (int i = 0; i < rows; i++)
                for (int g = 0; g < hg; g++) {
                    size_t row_major = (((size_t)s * rows + i) * heads + (size_t)r * hg + g) * dim;
                    size_t head_major =
                        (((size_t)r * ranks * rows + (size_t)s * rows + i) * hg + g) * dim;
                    if (inverse)
                        memcpy(out + row_major, in + head_major, (size_t)dim * 2);
                    else
                        memcpy(out + head_major, in + row_major, (size_t)dim * 2);
                }
}

/* ---- timed CPU baseline ----------------------------------------------------- */

#include <time.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* Attention output projection, gate and AdaLN: h3_dit.c:2573-2597.
 *   y = bf16(x . w^T) with FP32 accumulation (cuda/h3_gpu_cuda.cu:774-777; cuBLAS' summation order is
 *       not knowable, a plain ascending fmaf chain is used), w [hidden][inner];
 *   gated = bf16(residual + bf16(y * gate)), gate = gate_mod[map[row]][gate_slot]
 *       (cuda/fast_primitives.cuh:74-90);
 *   out = bf16(bf16(bf16(gated * inverse * weight) * bf16(1 + scale)) + shift) with the row's sum of
 *       squares in the kernel's order: thread t < 128 owns the 4-value groups at 4t + 512c, fmaf in
 *       index order, shuffle-down tree over 32 lanes, warp sums paired 0+2, 1+3, then 0+1
 *       (cuda/fast_primitives.cuh:64-124). inverse = 1/sqrtf (the GPU uses the approximate rsqrtf). */
static float adaln_row_sum(const uint16_t *x, unsigned width) {
    float lane[128];
    for (unsigned t = 0; t < 128; t++) {
        float sum = 0.0f;
        for (unsigned c = 0; 4 * t + 512 * c < width; c++)
            for (unsigned i = 0; i < 4; i++) {
                const float v = bf16_to_f32(x[4 * t + 512 * c + i]);
                sum = fmaf(v, v, sum);
            }
        lane[t] = sum;
    }
    float warp_sums[4];
    for (unsigned w = 0; w < 4; w++) {
        float v[32];
        for (unsigned l = 0; l < 32; l++) v[l] = lane[32 * w + l];
        for (unsigned distance = 16; distance; distance >>= 1)
            for (unsigned l = 0; l < 32; l++)       /* ascending l reads not yet updated partners */
                v[l] = v[l] + (l + distance < 32 ? v[l + distance] : v[l]);
        warp_sums[w] = v[0];
    }
    warp_sums[0] += warp_sums[2];
    warp_sums[1] += warp_sums[3];
    return warp_sums[0] + warp_sums[1];
}
ORACLE_API void oracle_out_proj_gate_adaln(uint16_t *gated, uint16_t *out, const uint16_t *residual,
                                           const uint16_t *x, const uint16_t *w, const uint16_t *norm_weight,
                                           const uint16_t *gate_mod, const uint16_t *mod, const uint32_t *map,
                                           unsigned rows, unsigned inner, unsigned hidden, unsigned slots,
                                           unsigned gate_slot, unsigned shift_slot, unsigned scale_slot,
                                           float epsilon) {
#pragma omp parallel for schedule(static)
    for (long r = 0; r < (long)rows; r++) {
        const size_t base = (size_t)map[r] * slots * hidden;
        for (unsigned n = 0; n < hidden; n++) {
            float acc = 0.0f;
            for (unsigned k = 0; k < inner; k++)
                acc = fmaf(bf16_to_f32(x[(size_t)r * inner + k]), bf16_to_f32(w[(size_t)n * inner + k]), acc);
            const float y = bf16_round(acc);
            const float g = bf16_to_f32(gate_mod[base + (size_t)gate_slot * hidden + n]);
            gated[(size_t)r * hidden + n] = f32_to_bf16(bf16_to_f32(residual[(size_t)r * hidden + n]) + bf16_round(y * g));
        }
        if (!out) continue;
        const float total = adaln_row_sum(gated + (size_t)r * hidden, hidden);
        const float inverse = 1.0f / sqrtf(total / (float)hidden + epsilon);
        for (unsigned n = 0; n < hidden; n++) {
            const float xv = bf16_to_f32(gated[(size_t)r * hidden + n]);
            const float normalized = xv * inverse * bf16_to_f32(norm_weight[n]);
            const float shift = bf16_to_f32(mod[base + (size_t)shift_slot * hidden + n]);
            const float scale = bf16_to_f32(mod[base + (size_t)scale_slot * hidden + n]);
            out[(size_t)r * hidden + n] = f32_to_bf16(bf16_round(bf16_round(normalized) * bf16_round(1.0f + scale)) + shift);
        }
    }
}

/* Thread count of the OpenMP loops above, for the benchmark's CPU-baseline legs: a launcher may
 * have exported OMP_NUM_THREADS=1 to its children, so the count is set and read back explicitly. */
ORACLE_API void oracle_set_threads(int threads) {
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#else
    (void)threads;
#endif
}
ORACLE_API int oracle_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
/*
 * Times oracle_attention (bf16 in, bf16 out) on `threads` OpenMP threads and
 * returns seconds for one pass; used only by the benchmark's cpu_baseline leg.
 */
ORACLE_API double oracle_time_attention(uint16_t *out, const uint16_t *q, const uint16_t *k,
                                        const uint16_t *v, int lq, int lk, int heads, int dim,
                                        float scale) {
    struct timespec a, b;
    clock_gettime(CLOCK_MONOTONIC, &a);
    oracle_attention(NULL, out, NULL, q, k, v, 1, lq, lk, heads, heads, dim, scale, 0, 0);
    clock_gettime(CLOCK_MONOTONIC, &b);
    return (double)(b.tv_sec - a.tv_sec) + 1e-9 * (double)(b.tv_nsec - a.tv_nsec);
}
