// Host side of the library, part 2: video sparse attention. The h3_gpu_vsa object of the
// primitive ABI (reference cuda/h3_cuda.h:70-76, cuda/vsa.cuh:192-300), the same pipeline fed by the
// QKV projection output, and raw-pointer entry points of the individual stages for callers that
// keep their own tensor objects (a backend that adopts the stages one by one).
#include <algorithm>
#include <cmath>
#include <new>
#include <vector>

#include "attn_kernels.h"
#include "h3_gpu_internal.h"

using h3b::bf16;
using h3b::cuda_good;
using h3b::fail;
using h3b::new_tensor;
using h3b::satisfied;

namespace h3b {
int rope_input(h3_gpu *g, QkvRopeInput &in, const h3_gpu_tensor *qkv, const h3_gpu_tensor *qn,
               const h3_gpu_tensor *kn, const h3_gpu_tensor *co, const h3_gpu_tensor *si, uint32_t rows,
               uint32_t heads, uint32_t dim, uint32_t half, float eps, int grouped);
}

namespace {

constexpr uint64_t MAX_TILES = 4096, MAX_HEADS = 56;   // limits of cuda/vsa.cuh:195-205
constexpr float VSA_SCALE = 0.08838834764831845f;      // 1/sqrt(128)

// Tile geometry of video sparse attention (what cuda/vsa.cuh:214-234 builds): the sequence is
// text rows, audio rows, then a (time, height, width) grid of video tokens. Text and audio are
// cut into dense 64-row tiles; the video grid into 4x4x4 cubes in raster order (width fastest),
// tokens inside a cube again in (time, height, width) order, edge cubes partial.
struct TileGeometry {
    uint32_t text, audio, time, height, width;
    uint32_t text_tiles, audio_tiles, cubes_t, cubes_h, cubes_w;

    TileGeometry(uint32_t te, uint32_t au, uint32_t t, uint32_t h, uint32_t w)
        : text(te), audio(au), time(t), height(h), width(w), text_tiles((te + 63) / 64),
          audio_tiles((au + 63) / 64), cubes_t((t + 3) / 4), cubes_h((h + 3) / 4), cubes_w((w + 3) / 4) {}
    uint64_t prefix() const { return (uint64_t)text_tiles + audio_tiles; }
    uint64_t tiles() const { return prefix() + (uint64_t)cubes_t * cubes_h * cubes_w; }
    uint64_t rows() const { return (uint64_t)text + audio + (uint64_t)time * height * width; }
    // Token row held by slot `slot` (0..63) of tile `tile`, or -1 for padding.
    int token(uint32_t tile, uint32_t slot) const {
        if (tile < text_tiles) {
            const uint32_t row = tile * 64 + slot;
            return row < text ? (int)row : -1;
        }
        if (tile < prefix()) {
            const uint32_t row = (tile - text_tiles) * 64 + slot;
            return row < audio ? (int)(text + row) : -1;
        }
        const uint32_t cube = tile - (uint32_t)prefix();
        const uint32_t x0 = 4 * (cube % cubes_w), y0 = 4 * ((cube / cubes_w) % cubes_h),
                       t0 = 4 * (cube / (cubes_w * cubes_h));
        const uint32_t ex = std::min(4u, width - x0), ey = std::min(4u, height - y0), et = std::min(4u, time - t0);
        if (slot >= ex * ey * et) return -1;
        const uint32_t x = x0 + slot % ex, y = y0 + (slot / ex) % ey, t = t0 + slot / (ex * ey);
        return (int)(text + audio + (t * height + y) * width + x);
    }
};

}  // namespace

struct h3_gpu_vsa {
    h3_gpu *gpu{};
    int rows{}, heads{}, tiles{}, prefix{}, keep{};
    bool trace_scores{};
    cudaEvent_t stage[5]{};   // optional stage timing: before pooling, after pooling, selection, fine stage, merge
    bool time_stages{};
    h3_gpu_tensor *map{}, *sizes{}, *q{}, *k{}, *v{}, *out{};
    h3_gpu_tensor *poolq{}, *poolk{}, *poolv{}, *scores{}, *compression{}, *indices{}, *counts{};
};

extern "C" void h3_gpu_vsa_free(h3_gpu_vsa *s) {
    if (!s) return;
    for (auto *t : {s->map, s->sizes, s->q, s->k, s->v, s->out, s->poolq, s->poolk, s->poolv, s->scores,
                    s->compression, s->indices, s->counts})
        h3_gpu_tensor_free(t);
    for (cudaEvent_t e : s->stage)
        if (e) cudaEventDestroy(e);
    delete s;
}

extern "C" h3_gpu_vsa *h3_gpu_vsa_new(h3_gpu *g, uint32_t text, uint32_t audio, uint32_t time, uint32_t height,
                                      uint32_t width, uint32_t heads) {
    if (!g || !text || !audio || !time || !height || !width || !heads) return nullptr;
    const TileGeometry geo(text, audio, time, height, width);
    // every factor is bounded before the product is formed
    if (geo.prefix() >= MAX_TILES || geo.cubes_t > MAX_TILES || geo.cubes_h > MAX_TILES || geo.cubes_w > MAX_TILES ||
        geo.tiles() > MAX_TILES || heads > MAX_HEADS) {
        fail(g, "VSA requires at most %d tiles and 56 heads", (int)MAX_TILES);
        return nullptr;
    }
    const size_t tiles = (size_t)geo.tiles();
    std::vector<int> map, sizes;
    try {
        map.resize(tiles * 64);
        sizes.resize(tiles);
    } catch (const std::bad_alloc &) {
        fail(g, "out of host memory constructing VSA tiles");
        return nullptr;
    }
    for (size_t tile = 0; tile < tiles; tile++) {
        int valid = 0;
        for (uint32_t slot = 0; slot < 64; slot++) {
            const int row = geo.token((uint32_t)tile, slot);
            map[tile * 64 + slot] = row;
            valid += row >= 0;
        }
        sizes[tile] = valid;
    }
    auto *s = new (std::nothrow) h3_gpu_vsa{};
    if (!s) return nullptr;
    s->gpu = g;
    s->rows = (int)geo.rows();
    s->heads = (int)heads;
    s->tiles = (int)tiles;
    s->prefix = (int)geo.prefix();
    s->keep = std::max(1, (s->tiles - s->prefix + 9) / 10);   // ceil(10 %) of the video tiles, cuda/vsa.cuh:242
    const size_t tiled = tiles * 64 * heads * 128, pooled = tiles * heads * 128;
    struct {
        h3_gpu_tensor **slot;
        size_t elements;
        h3_gpu_dtype dtype;
    } const buffers[] = {
        {&s->map, tiles * 64, H3_GPU_U32},      {&s->sizes, tiles, H3_GPU_U32},
        {&s->q, tiled, H3_GPU_BF16},            {&s->k, tiled, H3_GPU_BF16},
        {&s->v, tiled, H3_GPU_BF16},            {&s->out, tiled, H3_GPU_BF16},
        {&s->poolq, pooled, H3_GPU_F32},        {&s->poolk, pooled, H3_GPU_F32},
        {&s->poolv, pooled, H3_GPU_F32},        {&s->compression, pooled, H3_GPU_F32},
        {&s->indices, tiles * tiles * heads, H3_GPU_U32}, {&s->counts, tiles * heads, H3_GPU_U32},
    };
    bool ok = true;
    for (const auto &b : buffers) ok = ok && (*b.slot = new_tensor(g, b.elements, b.dtype)) != nullptr;
    ok = ok && cuda_good(g, cudaMemcpyAsync(s->map->data, map.data(), map.size() * sizeof(int), cudaMemcpyHostToDevice,
                                            g->stream)) &&
         cuda_good(g, cudaMemcpyAsync(s->sizes->data, sizes.data(), sizes.size() * sizeof(int),
                                      cudaMemcpyHostToDevice, g->stream)) &&
         cuda_good(g, cudaStreamSynchronize(g->stream));
    if (!ok) {
        h3_gpu_vsa_free(s);
        return nullptr;
    }
    return s;
}

extern "C" int h3b_vsa_info(const h3_gpu_vsa *s, int *rows, int *tiles, int *prefix, int *keep) {
    if (!s) return 0;
    if (rows) *rows = s->rows;
    if (tiles) *tiles = s->tiles;
    if (prefix) *prefix = s->prefix;
    if (keep) *keep = s->keep;
    return 1;
}
extern "C" int h3b_vsa_set_keep(h3_gpu_vsa *s, int keep) {
    if (!s || keep < 1 || keep > s->tiles - s->prefix) return 0;
    s->keep = keep;
    return 1;
}
extern "C" int h3b_vsa_trace_scores(h3_gpu_vsa *s, int enable) {
    if (!s) return 0;
    if (enable && !s->scores) {
        s->scores = new_tensor(s->gpu, (size_t)s->tiles * s->tiles * s->heads, H3_GPU_F32);
        if (!s->scores) return 0;
    }
    s->trace_scores = enable != 0;
    return 1;
}
// Stage timing with CUDA events on the context's stream (off by default).
extern "C" int h3b_vsa_time_stages(h3_gpu_vsa *s, int enable) {
    if (!s) return 0;
    if (enable)
        for (cudaEvent_t &e : s->stage)
            if (!e && !cuda_good(s->gpu, cudaEventCreate(&e))) return 0;
    s->time_stages = enable != 0;
    return 1;
}
// Milliseconds of the last call's four stages: pooling (or norm + RoPE + pooling), scores +
// selection + compression, block-sparse attention, merge. Waits for that call to finish.
extern "C" int h3b_vsa_stage_ms(h3_gpu_vsa *s, float *ms) {
    if (!s || !ms || !s->time_stages) return 0;
    if (!cuda_good(s->gpu, cudaEventSynchronize(s->stage[4]))) return 0;
    for (int i = 0; i < 4; i++)
        if (!cuda_good(s->gpu, cudaEventElapsedTime(&ms[i], s->stage[i], s->stage[i + 1]))) return 0;
    return 1;
}
extern "C" void *h3b_vsa_buffer(const h3_gpu_vsa *s, int which) {
    if (!s) return nullptr;
    const h3_gpu_tensor *all[] = {s->map, s->sizes, s->q, s->k, s->v, s->out, s->poolq, s->poolk,
                                  s->poolv, s->indices, s->counts, s->compression, s->scores};
    if (which < 0 || which >= (int)(sizeof all / sizeof all[0]) || !all[which]) return nullptr;
    return all[which]->data;
}

// ---- the stages on raw device pointers --------------------------------------------------------

extern "C" cudaError_t h3b_vsa_pool_raw(const void *const source[3], void *const tiled[3], float *const pooled[3],
                                        const int *map, const int *sizes, unsigned tiles, unsigned heads,
                                        cudaStream_t stream) {
    if (!source || !tiled || !pooled || !map || !sizes || !tiles || tiles > MAX_TILES || !heads)
        return cudaErrorInvalidValue;
    for (int i = 0; i < 3; i++)
        if (!source[i] || !tiled[i] || !pooled[i]) return cudaErrorInvalidValue;
    return h3b::vsa_tile_pool3(source, tiled, pooled, map, sizes, (int)tiles, (int)heads, 3, stream);
}
extern "C" cudaError_t h3b_vsa_select_raw(const float *pooled_q, const float *pooled_k, const float *pooled_v,
                                          float *scores, int *indices, int *counts, float *compression,
                                          unsigned tiles, unsigned prefix, unsigned keep, unsigned heads,
                                          cudaStream_t stream) {
    if (!pooled_q || !pooled_k || !indices || !counts || (compression && !pooled_v) || !heads)
        return cudaErrorInvalidValue;
    return h3b::vsa_score_select_compress(pooled_q, pooled_k, pooled_v, scores, indices, counts, compression,
                                          (int)tiles, (int)prefix, (int)keep, (int)heads, VSA_SCALE, stream);
}
extern "C" cudaError_t h3b_vsa_merge_raw(void *output, const void *tiled_sparse, const void *gate,
                                         const float *compression, const int *map, unsigned tiles, unsigned heads,
                                         cudaStream_t stream) {
    if (!output || !tiled_sparse || !gate || !compression || !map || !tiles || !heads) return cudaErrorInvalidValue;
    return h3b::vsa_untile_merge(output, tiled_sparse, gate, compression, map, (int)tiles, (int)heads, stream);
}
extern "C" cudaError_t h3b_qkv_rope_raw(void *query, void *key, void *value, const void *qkv, const void *q_norm,
                                        const void *k_norm, const void *rope_cos, const void *rope_sin,
                                        unsigned sequence, unsigned heads, unsigned rope_half, float epsilon,
                                        int grouped, cudaStream_t stream) {
    const h3b::QkvRopeInput in{qkv, q_norm, k_norm, rope_cos, rope_sin, sequence, heads, rope_half, grouped != 0,
                               epsilon};
    return h3b::qkv_rope_token_major(in, query, key, value, stream);
}

// ---- the pipeline -------------------------------------------------------------------------------

static bool mark(h3_gpu_vsa *s, int which) {
    return !s->time_stages || cuda_good(s->gpu, cudaEventRecord(s->stage[which], s->gpu->stream));
}

// Everything after the tiled copies and tile means exist: scores + selection + compression, the
// block-sparse kernel, merge back to token order (the work of cuda/vsa.cuh:281-299).
static int after_tiling(h3_gpu_vsa *s, h3_gpu_tensor *out, const h3_gpu_tensor *gate) {
    h3_gpu *g = s->gpu;
    cudaStream_t stream = g->stream;
    auto f32 = [](h3_gpu_tensor *t) { return static_cast<float *>(t->data); };
    auto i32 = [](h3_gpu_tensor *t) { return static_cast<int *>(t->data); };
    return mark(s, 1) &&
           cuda_good(g, h3b_vsa_select_raw(f32(s->poolq), f32(s->poolk), f32(s->poolv),
                                           s->trace_scores ? f32(s->scores) : nullptr, i32(s->indices),
                                           i32(s->counts), f32(s->compression), s->tiles, s->prefix, s->keep,
                                           s->heads, stream)) &&
           mark(s, 2) &&
           cuda_good(g, h3_vsa_hopper(s->out->data, s->q->data, s->k->data, s->v->data, nullptr, i32(s->indices),
                                      i32(s->counts), i32(s->sizes), s->tiles, s->heads, stream)) &&
           mark(s, 3) &&
           cuda_good(g, h3b_vsa_merge_raw(out->data, s->out->data, gate->data, f32(s->compression), i32(s->map),
                                          s->tiles, s->heads, stream)) &&
           mark(s, 4);
}

// cuda/vsa.cuh:263-300 as four launches: pooling of Q, K and V; scores + selection + pooled
// softmax + compression; the block-sparse kernel; merge.
extern "C" int h3_gpu_vsa_bf16(h3_gpu_vsa *s, h3_gpu_tensor *out, const h3_gpu_tensor *q, const h3_gpu_tensor *k,
                               const h3_gpu_tensor *value, const h3_gpu_tensor *gate) {
    if (!s) return 0;
    h3_gpu *g = s->gpu;
    const size_t elements = (size_t)s->rows * s->heads * 128;
    const char *what = "VSA input/output";
    if (!satisfied(g, {bf16(out, elements, what), bf16(q, elements, what), bf16(k, elements, what),
                       bf16(value, elements, what), bf16(gate, elements, what)}))
        return 0;
    const void *source[3] = {q->data, k->data, value->data};
    void *tiled[3] = {s->q->data, s->k->data, s->v->data};
    float *pooled[3] = {(float *)s->poolq->data, (float *)s->poolk->data, (float *)s->poolv->data};
    return mark(s, 0) &&
           cuda_good(g, h3b_vsa_pool_raw(source, tiled, pooled, (const int *)s->map->data,
                                         (const int *)s->sizes->data, s->tiles, s->heads, g->stream)) &&
           after_tiling(s, out, gate);
}

// The same pipeline fed by the QKV projection output: norm + rotation write the tiled copies and
// the tile means themselves (csrc/qkv_rope.cu), then the shared remainder.
extern "C" int h3b_vsa_qkv_rope_bf16(h3_gpu_vsa *s, h3_gpu_tensor *out, const h3_gpu_tensor *qkv,
                                     const h3_gpu_tensor *qn, const h3_gpu_tensor *kn, const h3_gpu_tensor *co,
                                     const h3_gpu_tensor *si, const h3_gpu_tensor *gate, uint32_t rope_half,
                                     float eps, int grouped) {
    if (!s) return 0;
    h3_gpu *g = s->gpu;
    const size_t elements = (size_t)s->rows * s->heads * 128;
    if (!satisfied(g, {bf16(out, elements, "VSA output"), bf16(gate, elements, "VSA gate")})) return 0;
    h3b::QkvRopeInput in{};
    if (!h3b::rope_input(g, in, qkv, qn, kn, co, si, (uint32_t)s->rows, (uint32_t)s->heads, 128, rope_half, eps,
                         grouped))
        return 0;
    void *tiled[3] = {s->q->data, s->k->data, s->v->data};
    float *pooled[3] = {(float *)s->poolq->data, (float *)s->poolk->data, (float *)s->poolv->data};
    return mark(s, 0) &&
           cuda_good(g, h3b::qkv_rope_vsa_tiles(in, (const int *)s->map->data, (const int *)s->sizes->data, s->tiles,
                                                tiled, pooled, g->stream)) &&
           after_tiling(s, out, gate);
}
