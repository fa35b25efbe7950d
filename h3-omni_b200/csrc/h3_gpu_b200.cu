// Host side of the library, part 1: the five kernel-adapter entry points, the context and tensor
// objects, and the dense / rectangular / host-buffer attention calls and the Q/K norm + RoPE
// calls of the primitive ABI. Argument meaning, return conventions and error strings follow the
// reference's CUDA backend (cuda/h3_gpu_cuda.cu) so a caller cannot tell the two apart on this
// path. (Video sparse attention: vsa_object.cu. Communicators and Ulysses: multi_gpu.cu.)
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>

#include "attn_kernels.h"
#include "h3_gpu_internal.h"

namespace h3b {
// One status word per device, written by kernels whose bounded waits or bounds checks fail.
__device__ int g_device_status = 0;

cudaError_t device_status_word(int **word) {
    static thread_local int cached_device = -1;
    static thread_local int *cached = nullptr;
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    if (device != cached_device) {
        e = cudaGetSymbolAddress(reinterpret_cast<void **>(&cached), g_device_status);
        if (e != cudaSuccess) return e;
        cached_device = device;
    }
    *word = cached;
    return cudaSuccess;
}

void fail(h3_gpu *g, const char *format, ...) {
    if (!g) return;
    va_list args;
    va_start(args, format);
    vsnprintf(g->error, sizeof g->error, format, args);
    va_end(args);
}
bool cuda_good(h3_gpu *g, cudaError_t e) {
    if (e != cudaSuccess) fail(g, "CUDA: %s", cudaGetErrorString(e));
    return e == cudaSuccess;
}
size_t dtype_bytes(h3_gpu_dtype t) {
    switch (t) {
        case H3_GPU_I8: return 1;
        case H3_GPU_BF16:
        case H3_GPU_F16: return 2;
        default: return 4;
    }
}
bool satisfied(h3_gpu *g, std::initializer_list<Need> needs) {
    static const char *const names[] = {"F32", "BF16", "I8", "U32", "FP16"};
    for (const Need &need : needs) {
        const h3_gpu_tensor *t = need.tensor;
        if (!t || t->owner != g || t->elements < need.elements) {
            fail(g, "invalid tensor: %s (need %zu elements)", need.what, need.elements);
            return false;
        }
        if (!need.any_dtype && t->dtype != need.dtype) {
            fail(g, "expected %s: %s", names[need.dtype], need.what);
            return false;
        }
    }
    return true;
}
h3_gpu_tensor *new_tensor(h3_gpu *g, size_t elements, h3_gpu_dtype dtype) {
    if (!g || !elements) return nullptr;
    auto *t = new (std::nothrow) h3_gpu_tensor{nullptr, elements, elements * dtype_bytes(dtype), dtype, g, true};
    // stream-ordered, like the reference's pool (cuda/h3_gpu_cuda.cu:215-249)
    if (t && !cuda_good(g, cudaMallocAsync(&t->data, t->bytes, g->stream))) {
        delete t;
        t = nullptr;
    }
    return t;
}
}  // namespace h3b

using h3b::bf16;
using h3b::cuda_good;
using h3b::fail;
using h3b::new_tensor;
using h3b::satisfied;
using h3b::sized;

// ======================= 1. kernel-adapter entry points =======================

extern "C" cudaError_t h3_flash_bf16(void *output, const void *query, const void *key,
                                     const void *value, float *logsumexp, unsigned batch,
                                     unsigned sequence, unsigned heads, unsigned kv_heads,
                                     float scale, bool causal, cudaStream_t stream) {
    if (!output || !query || !key || !value) return cudaErrorInvalidValue;
    if (!causal)
        return h3b::attn_dense_tc5(output, query, key, value, logsumexp, batch, sequence, sequence,
                                   heads, kv_heads, scale, stream);
    return h3b::attn_mma(output, query, key, value, logsumexp, batch, sequence, sequence, heads,
                         kv_heads, scale, true, 0, stream);
}

extern "C" cudaError_t h3_flash3_bf16(void *output, const void *query, const void *key,
                                      const void *value, float *logsumexp, unsigned batch,
                                      unsigned sequence, unsigned heads, unsigned kv_heads,
                                      float scale, cudaStream_t stream) {
    if (!output || !query || !key || !value) return cudaErrorInvalidValue;
    return h3b::attn_dense_tc5(output, query, key, value, logsumexp, batch, sequence, sequence,
                               heads, kv_heads, scale, stream);
}

extern "C" cudaError_t h3_flash3_f16_d64(void *output, const void *query, const void *key,
                                         const void *value, float *logsumexp, unsigned batch,
                                         unsigned sequence, unsigned heads, float scale,
                                         cudaStream_t stream) {
    if (!output || !query || !key || !value) return cudaErrorInvalidValue;
    return h3b::attn_mma(output, query, key, value, logsumexp, batch, sequence, sequence, heads,
                         heads, scale, false, 1, stream);
}

extern "C" cudaError_t h3_flash3_cross_bf16(void *output, const void *query, const void *key,
                                            const void *value, float *logsumexp,
                                            unsigned query_rows, unsigned key_rows, unsigned heads,
                                            float scale, cudaStream_t stream) {
    if (!output || !query || !key || !value) return cudaErrorInvalidValue;
    return h3b::attn_dense_tc5(output, query, key, value, logsumexp, 1, query_rows, key_rows, heads,
                               heads, scale, stream);
}

extern "C" cudaError_t h3_vsa_hopper(void *out, const void *q, const void *k, const void *v,
                                     float *lse, int *indices, int *counts, int *sizes,
                                     unsigned tiles, unsigned heads, cudaStream_t stream) {
    if (!out || !q || !k || !v || !indices || !counts || !sizes) return cudaErrorInvalidValue;
    if (!tiles || !heads) return cudaErrorNotSupported;  // as cuda/vsa_hopper.cu:13
    return h3b::attn_sparse_tc5(out, q, k, v, lse, indices, counts, sizes, tiles, heads, stream);
}

extern "C" void h3b_vsa_fine_mode(int mode) { h3b::attn_sparse_set_mode(mode < 0 || mode > 3 ? 0 : mode); }

extern "C" cudaError_t h3b_device_status(int *status, int reset) {
    if (!status) return cudaErrorInvalidValue;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return e;
    e = cudaMemcpyFromSymbol(status, h3b::g_device_status, sizeof(int));
    if (e != cudaSuccess || !reset) return e;
    const int zero = 0;
    return cudaMemcpyToSymbol(h3b::g_device_status, &zero, sizeof(int));
}

// ======================= 2. context and tensors =======================

extern "C" h3_gpu *h3_gpu_create(const char *, char *error, size_t error_size) {
    auto refuse = [&](const char *format, auto... values) -> h3_gpu * {
        if (error && error_size) snprintf(error, error_size, format, values...);
        return nullptr;
    };
    int device = 0, major = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return refuse("no CUDA device: %s", cudaGetErrorString(e));
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
    if (e != cudaSuccess) return refuse("device query: %s", cudaGetErrorString(e));
    // No fallback: this library holds sm_100a code only.
    if (major != 10) return refuse("libh3b200_attn needs a B200-class GPU (sm_100), found sm_%d0", major);
    auto *g = new (std::nothrow) h3_gpu{};
    if (!g) return refuse("out of host memory");
    g->device = device;
    e = cudaStreamCreateWithFlags(&g->own_stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
        delete g;
        return refuse("stream: %s", cudaGetErrorString(e));
    }
    g->stream = g->own_stream;
    return g;
}
static void pipeline_release(h3_gpu *g) {
    host_pipeline &p = g->pipe;
    if (!p.ready) return;
    cudaStreamSynchronize(p.h2d);
    cudaStreamSynchronize(p.d2h);
    for (cudaStream_t stream : p.compute) cudaStreamSynchronize(stream);
    for (auto &slot : p.slot)
        for (void *&buffer : slot) {
            if (buffer) cudaFree(buffer);
            buffer = nullptr;
        }
    for (int s = 0; s < 2; s++) {
        cudaEventDestroy(p.loaded[s]);
        cudaEventDestroy(p.computed[s]);
        cudaEventDestroy(p.stored[s]);
    }
    cudaEventDestroy(p.entry);
    cudaStreamDestroy(p.h2d);
    cudaStreamDestroy(p.d2h);
    for (cudaStream_t stream : p.compute) cudaStreamDestroy(stream);
    p = host_pipeline{};
}
extern "C" void h3_gpu_free(h3_gpu *g) {
    if (!g) return;
    cudaStreamSynchronize(g->stream);
    pipeline_release(g);
    cudaStreamDestroy(g->own_stream);
    delete g;
}
extern "C" int h3b_gpu_set_stream(h3_gpu *g, cudaStream_t stream) {
    if (g) g->stream = stream ? stream : g->own_stream;
    return g != nullptr;
}
extern "C" cudaStream_t h3b_gpu_stream(const h3_gpu *g) { return g ? g->stream : nullptr; }

extern "C" h3_gpu_tensor *h3_gpu_tensor_new_f32(h3_gpu *g, size_t n) { return new_tensor(g, n, H3_GPU_F32); }
extern "C" h3_gpu_tensor *h3_gpu_tensor_new_bf16(h3_gpu *g, size_t n) { return new_tensor(g, n, H3_GPU_BF16); }
extern "C" h3_gpu_tensor *h3b_tensor_new_f16(h3_gpu *g, size_t n) { return new_tensor(g, n, H3_GPU_F16); }

// Host <-> device moves of whole tensors or ranges; all of them wait for the copy.
static bool move(h3_gpu *g, void *dst, const void *src, size_t bytes, cudaMemcpyKind kind) {
    return cuda_good(g, cudaMemcpyAsync(dst, src, bytes, kind, g->stream)) &&
           cuda_good(g, cudaStreamSynchronize(g->stream));
}
static h3_gpu_tensor *uploaded(h3_gpu *g, const void *values, size_t n, h3_gpu_dtype dtype) {
    h3_gpu_tensor *t = values ? new_tensor(g, n, dtype) : nullptr;
    if (t && !move(g, t->data, values, t->bytes, cudaMemcpyHostToDevice)) {
        h3_gpu_tensor_free(t);
        t = nullptr;
    }
    return t;
}
extern "C" h3_gpu_tensor *h3_gpu_tensor_from_f32(h3_gpu *g, const float *v, size_t n) {
    return uploaded(g, v, n, H3_GPU_F32);
}
extern "C" h3_gpu_tensor *h3_gpu_tensor_from_bf16(h3_gpu *g, const uint16_t *v, size_t n) {
    return uploaded(g, v, n, H3_GPU_BF16);
}
extern "C" h3_gpu_tensor *h3_gpu_tensor_from_u32(h3_gpu *g, const uint32_t *v, size_t n) {
    return uploaded(g, v, n, H3_GPU_U32);
}
extern "C" h3_gpu_tensor *h3b_tensor_wrap(h3_gpu *g, void *device_pointer, size_t elements, h3_gpu_dtype dtype) {
    if (!g || !device_pointer || !elements) return nullptr;
    return new (std::nothrow)
        h3_gpu_tensor{device_pointer, elements, elements * h3b::dtype_bytes(dtype), dtype, g, false};
}
extern "C" void *h3b_tensor_data(const h3_gpu_tensor *t) { return t ? t->data : nullptr; }
extern "C" void h3_gpu_tensor_free(h3_gpu_tensor *t) {
    if (!t) return;
    if (t->owns && t->data) cudaFreeAsync(t->data, t->owner->stream);
    delete t;
}
extern "C" size_t h3_gpu_tensor_elements(const h3_gpu_tensor *t) { return t ? t->elements : 0; }
extern "C" h3_gpu_dtype h3_gpu_tensor_dtype(const h3_gpu_tensor *t) { return t ? t->dtype : H3_GPU_F32; }

static int read_range(const h3_gpu_tensor *t, void *values, size_t n, h3_gpu_dtype dtype) {
    if (!t || !values || t->dtype != dtype || n > t->elements) return 0;
    return move(t->owner, values, t->data, n * h3b::dtype_bytes(dtype), cudaMemcpyDeviceToHost);
}
static int write_range(h3_gpu_tensor *t, size_t offset, const void *values, size_t n, h3_gpu_dtype dtype) {
    if (!t || !values || t->dtype != dtype || offset > t->elements || n > t->elements - offset) return 0;
    const size_t size = h3b::dtype_bytes(dtype);
    return move(t->owner, static_cast<char *>(t->data) + offset * size, values, n * size, cudaMemcpyHostToDevice);
}
extern "C" int h3_gpu_tensor_read_f32(const h3_gpu_tensor *t, float *v, size_t n) { return read_range(t, v, n, H3_GPU_F32); }
extern "C" int h3_gpu_tensor_read_bf16(const h3_gpu_tensor *t, uint16_t *v, size_t n) { return read_range(t, v, n, H3_GPU_BF16); }
extern "C" int h3_gpu_tensor_write_f32(h3_gpu_tensor *t, const float *v, size_t n) { return write_range(t, 0, v, n, H3_GPU_F32); }
extern "C" int h3_gpu_tensor_write_bf16(h3_gpu_tensor *t, const uint16_t *v, size_t n) { return write_range(t, 0, v, n, H3_GPU_BF16); }
extern "C" int h3_gpu_tensor_write_bf16_range(h3_gpu_tensor *t, size_t offset, const uint16_t *v, size_t n) {
    return write_range(t, offset, v, n, H3_GPU_BF16);
}
extern "C" int h3_gpu_begin(h3_gpu *g) { return g != nullptr; }
extern "C" int h3_gpu_continue(h3_gpu *g) { return g != nullptr; }
// Waits for the context's stream, then reports the status word of the context's device: a
// bounded device-side wait that gave up or a refused access fails this call once (the word is
// cleared after it has been reported, so the next submit starts clean).
extern "C" int h3_gpu_submit(h3_gpu *g) {
    if (!g) return 0;
    int current = -1;
    if (!cuda_good(g, cudaGetDevice(&current))) return 0;
    if (current != g->device) {
        fail(g, "context of device %d used while device %d is current", g->device, current);
        return 0;
    }
    if (!cuda_good(g, cudaStreamSynchronize(g->stream))) return 0;
    int status = 0;
    if (!cuda_good(g, cudaMemcpyFromSymbol(&status, h3b::g_device_status, sizeof(int)))) return 0;
    if (!status) return 1;
    const int zero = 0;
    cudaMemcpyToSymbol(h3b::g_device_status, &zero, sizeof(int));
    if (status == 1) fail(g, "device-side wait timed out (status 1)");
    else fail(g, "device-side bounds check failed (status %d)", status);
    return 0;
}
extern "C" const char *h3_gpu_error(const h3_gpu *g) { return g ? g->error : "no GPU context"; }
extern "C" int h3_gpu_zero(h3_gpu *g, h3_gpu_tensor *t) {
    return t && t->owner == g && cuda_good(g, cudaMemsetAsync(t->data, 0, t->bytes, g->stream));
}
extern "C" int h3_gpu_copy_bf16(h3_gpu *g, h3_gpu_tensor *dst, size_t dst_offset, const h3_gpu_tensor *src,
                                size_t src_offset, size_t n) {
    if (!satisfied(g, {bf16(dst, dst_offset + n, "copy destination"), bf16(src, src_offset + n, "copy source")}))
        return 0;
    return cuda_good(g, cudaMemcpyAsync(static_cast<uint16_t *>(dst->data) + dst_offset,
                                        static_cast<const uint16_t *>(src->data) + src_offset, n * 2,
                                        cudaMemcpyDeviceToDevice, g->stream));
}
extern "C" int h3_gpu_download(h3_gpu *g, const h3_gpu_tensor *t, size_t offset, void *host, size_t count) {
    if (!g || !t || t->owner != g || !host || offset > t->bytes || count > t->bytes - offset) return 0;
    return move(g, host, static_cast<const char *>(t->data) + offset, count, cudaMemcpyDeviceToHost);
}

// ======================= dense / rectangular attention =======================

// The shape of one bf16 attention call of the primitive ABI (cuda/h3_gpu_cuda.cu:1109-1130,
// 1216-1246). The reference allocates a logsumexp tensor per call and frees it right after the
// enqueue without ever reading it; the kernels here take NULL instead.
struct DenseCall {
    unsigned sequence, heads, kv_heads, dim;
    float scale;
    bool causal, flash3;
};
static int dense_attention(h3_gpu *g, h3_gpu_tensor *y, const h3_gpu_tensor *q, const h3_gpu_tensor *k,
                           const h3_gpu_tensor *v, const DenseCall &c) {
    if (!g || !c.sequence || !c.heads || !c.kv_heads || c.heads % c.kv_heads || !c.dim) return 0;
    if (c.dim != 128) {
        fail(g, "BF16 attention supports head dimension 128 only");
        return 0;
    }
    const size_t per_head = (size_t)c.sequence * c.dim;
    if (!satisfied(g, {bf16(q, per_head * c.heads, "attention query"), bf16(k, per_head * c.kv_heads, "attention key"),
                       bf16(v, per_head * c.kv_heads, "attention value"),
                       bf16(y, per_head * c.heads, "attention output")}))
        return 0;
    const cudaError_t e =
        (c.flash3 && !c.causal)
            ? h3_flash3_bf16(y->data, q->data, k->data, v->data, nullptr, 1, c.sequence, c.heads, c.kv_heads,
                             c.scale, g->stream)
            : h3_flash_bf16(y->data, q->data, k->data, v->data, nullptr, 1, c.sequence, c.heads, c.kv_heads,
                            c.scale, c.causal, g->stream);
    return cuda_good(g, e);
}
extern "C" int h3_gpu_sdpa_bf16(h3_gpu *g, h3_gpu_tensor *y, const h3_gpu_tensor *q, const h3_gpu_tensor *k,
                                const h3_gpu_tensor *v, uint32_t n, uint32_t h, uint32_t d, float s) {
    return dense_attention(g, y, q, k, v, DenseCall{n, h, h, d, s, false, true});
}
extern "C" int h3_gpu_sdpa_fa2_bf16(h3_gpu *g, h3_gpu_tensor *y, const h3_gpu_tensor *q, const h3_gpu_tensor *k,
                                    const h3_gpu_tensor *v, uint32_t n, uint32_t h, uint32_t d, float s) {
    return dense_attention(g, y, q, k, v, DenseCall{n, h, h, d, s, false, false});
}
extern "C" int h3_gpu_gqa_causal_bf16(h3_gpu *g, h3_gpu_tensor *y, const h3_gpu_tensor *q, const h3_gpu_tensor *k,
                                      const h3_gpu_tensor *v, uint32_t n, uint32_t h, uint32_t kh, uint32_t d,
                                      float s) {
    return dense_attention(g, y, q, k, v, DenseCall{n, h, kh, d, s, true, true});
}
extern "C" int h3_gpu_sdpa_f16_d64(h3_gpu *g, h3_gpu_tensor *y, const h3_gpu_tensor *q, const h3_gpu_tensor *k,
                                   const h3_gpu_tensor *v, uint32_t n, uint32_t h, uint32_t d, float s) {
    if (!g) return 0;
    if (d != 64 || !n || !h) {
        fail(g, "FP16 attention supports head dimension 64 only");
        return 0;
    }
    const size_t count = (size_t)n * h * d;
    if (!satisfied(g, {h3b::Need{q, count, "FP16 attention query", H3_GPU_F16, false},
                       h3b::Need{k, count, "FP16 attention key", H3_GPU_F16, false},
                       h3b::Need{v, count, "FP16 attention value", H3_GPU_F16, false},
                       h3b::Need{y, count, "FP16 attention output", H3_GPU_F16, false}}))
        return 0;
    return cuda_good(g, h3_flash3_f16_d64(y->data, q->data, k->data, v->data, nullptr, 1, n, h, s, g->stream));
}

// Row `row` of a token-major [rows][heads][128] bf16 tensor.
static uint16_t *row_of(const h3_gpu_tensor *t, size_t row, uint32_t heads) {
    return static_cast<uint16_t *>(t->data) + row * heads * 128;
}
static const float LIVE_SCALE = 0.08838834764831845f;   // 1/sqrt(128), fixed for the live calls

extern "C" int h3_gpu_cross_attention_bf16(h3_gpu *g, h3_gpu_tensor *y, size_t yo, const h3_gpu_tensor *q, size_t qo,
                                           const h3_gpu_tensor *k, const h3_gpu_tensor *v, size_t ko, uint32_t nq,
                                           uint32_t nk, uint32_t heads) {
    if (!g || !nq || !nk || !heads) return 0;
    const size_t width = (size_t)heads * 128;
    if (!satisfied(g, {sized(y, (yo + nq) * width, "live output"), sized(q, (qo + nq) * width, "live query"),
                       sized(k, (ko + nk) * width, "live key"), sized(v, (ko + nk) * width, "live value")}))
        return 0;
    if (y->dtype != H3_GPU_BF16 || q->dtype != H3_GPU_BF16 || k->dtype != H3_GPU_BF16 || v->dtype != H3_GPU_BF16) {
        fail(g, "live attention requires BF16");
        return 0;
    }
    return cuda_good(g, h3_flash3_cross_bf16(row_of(y, yo, heads), row_of(q, qo, heads), row_of(k, ko, heads),
                                             row_of(v, ko, heads), nullptr, nq, nk, heads, LIVE_SCALE, g->stream));
}

// Live-mode attention without the per-layer concatenation copies (an addition; the reference
// builds text | sink | recent0 | recent1 | current by device copies first, h3_dit_live.inc:81-94):
// query rows attend the listed K/V row ranges as if they were one tensor. Every range is
// [>= kv_row[s] + kv_rows[s]][heads][128] bf16; at most six ranges; scale 1/sqrt(128) as in
// h3_gpu_cross_attention_bf16.
extern "C" int h3b_cross_attention_segments_bf16(h3_gpu *g, h3_gpu_tensor *y, size_t yo, const h3_gpu_tensor *q,
                                                 size_t qo, uint32_t nq, uint32_t heads, uint32_t segments,
                                                 const h3_gpu_tensor *const *k, const h3_gpu_tensor *const *v,
                                                 const size_t *kv_row, const uint32_t *kv_rows) {
    if (!g) return 0;
    const size_t width = (size_t)heads * 128;
    if (!nq || !heads || !segments || segments > 6 || !k || !v || !kv_row || !kv_rows) {
        fail(g, "segmented live attention: 1 to 6 key/value ranges and a non-empty query");
        return 0;
    }
    if (!satisfied(g, {bf16(y, (yo + nq) * width, "live output"), bf16(q, (qo + nq) * width, "live query")})) return 0;
    const void *kp[6], *vp[6];
    for (uint32_t s = 0; s < segments; s++) {
        if (!kv_rows[s]) {
            fail(g, "segmented live attention: range %u is empty", s);
            return 0;
        }
        const size_t need = (kv_row[s] + kv_rows[s]) * width;
        if (!satisfied(g, {bf16(k[s], need, "live key"), bf16(v[s], need, "live value")})) return 0;
        kp[s] = row_of(k[s], kv_row[s], heads);
        vp[s] = row_of(v[s], kv_row[s], heads);
    }
    return cuda_good(g, h3b::attn_segments_tc5(row_of(y, yo, heads), row_of(q, qo, heads), kp, vp, kv_rows, segments,
                                               nq, heads, LIVE_SCALE, g->stream));
}

// Dense attention straight from and to host memory (an addition; the reference has no
// host-buffer attention call). The heads are independent, so the work is cut into head groups
// and pipelined over three streams: while group g is computed, group g+1 is copied in and
// group g-1 is copied out. Host tensors are token-major [sequence][heads][128]; each group's
// strided slice is packed into a compact device buffer by a 2-D copy, so the kernel sees a
// plain [sequence][heads/groups][128] tensor. With pinned host memory the copies overlap the
// kernel and the call costs about max(copy time, kernel time) instead of their sum; with
// pageable memory it still works but the copies serialise. Returns after `out` is complete.
static int pipeline_prepare(h3_gpu *g, size_t slot_bytes) {
    host_pipeline &p = g->pipe;
    if (p.ready && p.slot_bytes >= slot_bytes) return 1;
    pipeline_release(g);
    if (!cuda_good(g, cudaStreamCreateWithFlags(&p.h2d, cudaStreamNonBlocking)) ||
        !cuda_good(g, cudaStreamCreateWithFlags(&p.d2h, cudaStreamNonBlocking)) ||
        !cuda_good(g, cudaStreamCreateWithFlags(&p.compute[0], cudaStreamNonBlocking)) ||
        !cuda_good(g, cudaStreamCreateWithFlags(&p.compute[1], cudaStreamNonBlocking)) ||
        !cuda_good(g, cudaEventCreateWithFlags(&p.entry, cudaEventDisableTiming)))
        return 0;
    for (int s = 0; s < 2; s++) {
        if (!cuda_good(g, cudaEventCreateWithFlags(&p.loaded[s], cudaEventDisableTiming)) ||
            !cuda_good(g, cudaEventCreateWithFlags(&p.computed[s], cudaEventDisableTiming)) ||
            !cuda_good(g, cudaEventCreateWithFlags(&p.stored[s], cudaEventDisableTiming)))
            return 0;
        for (int t = 0; t < 4; t++)
            if (!cuda_good(g, cudaMalloc(&p.slot[s][t], slot_bytes))) return 0;
    }
    p.slot_bytes = slot_bytes;
    p.ready = true;
    return 1;
}
// How the heads of a host-buffer call are cut into chunks. The copy-in before the first kernel
// and the copy-out after the last one are the only transfers nothing overlaps, so the chunks at
// both ends are short. head_groups > 0: equal groups, the two outer ones halved. head_groups == 0:
// two one-head chunks at either end and inner chunks of at least two heads and about 24 MB per
// tensor (large enough for the copy engines; small chunks cost nothing on the compute side
// because the kernels of consecutive chunks run on two streams and overlap, so no chunk's last,
// partly empty wave of CTAs leaves SMs idle).
extern "C" uint32_t h3b_sdpa_host_plan(uint32_t sequence, uint32_t heads, uint32_t head_groups, uint32_t *head_count,
                                       uint32_t capacity) {
    uint32_t chunks = 0;
    auto push = [&](uint32_t n) {
        if (n && chunks < capacity) head_count[chunks] = n;
        chunks += n ? 1 : 0;
    };
    if (!heads || !sequence) return 0;
    if (head_groups) {
        if (heads % head_groups || head_groups > 64) return 0;
        const uint32_t hg = heads / head_groups;
        for (uint32_t group = 0; group < head_groups; group++) {
            const bool edge = (group == 0 || group + 1 == head_groups) && hg >= 2;
            if (edge) {
                push(hg / 2);
                push(hg - hg / 2);
            } else {
                push(hg);
            }
        }
    } else {
        const uint32_t edge = heads >= 8 ? 2 : heads >= 4 ? 1 : 0, inner = heads - 2 * edge;
        const uint64_t head_bytes = (uint64_t)sequence * 256;
        uint32_t best = (uint32_t)((24ull << 20) / head_bytes);
        best = best < 2 ? 2 : best > 8 ? 8 : best;
        if (best < (inner + 59) / 60) best = (inner + 59) / 60;   // never more than 64 chunks
        if (best > inner) best = inner;
        for (uint32_t i = 0; i < edge; i++) push(1);
        if (inner) {
            const uint32_t n = (inner + best - 1) / best, base = inner / n, extra = inner % n;
            for (uint32_t i = 0; i < n; i++) push(i < extra ? base + 1 : base);
        }
        for (uint32_t i = 0; i < edge; i++) push(1);
    }
    return chunks <= capacity ? chunks : 0;
}

extern "C" int h3b_sdpa_bf16_host(h3_gpu *g, uint16_t *out, const uint16_t *q, const uint16_t *k,
                                  const uint16_t *v, uint32_t sequence, uint32_t heads,
                                  uint32_t head_dim, float scale, uint32_t head_groups) {
    if (!g) return 0;
    if (!out || !q || !k || !v || !sequence || !heads) {
        fail(g, "host attention: null pointer or empty shape");
        return 0;
    }
    if (head_dim != 128) {
        fail(g, "BF16 attention supports head dimension 128 only");
        return 0;
    }
    uint32_t first_head[66], head_count[66];
    const uint32_t chunks = h3b_sdpa_host_plan(sequence, heads, head_groups, head_count, 66);
    if (!chunks) {
        fail(g, "host attention: %u heads do not split into %u groups (at most 64)", heads, head_groups);
        return 0;
    }
    uint32_t widest = 0;
    for (uint32_t c = 0, at = 0; c < chunks; at += head_count[c++]) {
        first_head[c] = at;
        widest = head_count[c] > widest ? head_count[c] : widest;
    }
    const size_t pitch = (size_t)heads * 256;
    if (!pipeline_prepare(g, (size_t)widest * 256 * sequence)) return 0;
    host_pipeline &p = g->pipe;
    // everything already queued on the context's stream comes first
    if (!cuda_good(g, cudaEventRecord(p.entry, g->stream)) || !cuda_good(g, cudaStreamWaitEvent(p.h2d, p.entry, 0)) ||
        !cuda_good(g, cudaStreamWaitEvent(p.compute[0], p.entry, 0)) ||
        !cuda_good(g, cudaStreamWaitEvent(p.compute[1], p.entry, 0)))
        return 0;
    for (uint32_t chunk = 0; chunk < chunks; chunk++) {
        // Slot s and stream s belong to the chunks of parity s. The kernels of two consecutive
        // chunks may overlap: the CTAs of the later one fill the SMs the earlier one's last
        // wave leaves idle, which is what makes one-head chunks at both ends affordable.
        const int s = chunk & 1;
        cudaStream_t compute = p.compute[s];
        const uint32_t n = head_count[chunk];
        const size_t offset = (size_t)first_head[chunk] * 128;   // elements into a host row
        const size_t row_bytes = (size_t)n * 256;
        if (chunk >= 2) {
            // slot reuse: inputs after the kernel of chunk-2, output after its copy-out
            if (!cuda_good(g, cudaStreamWaitEvent(p.h2d, p.computed[s], 0)) ||
                !cuda_good(g, cudaStreamWaitEvent(compute, p.stored[s], 0)))
                return 0;
        }
        const uint16_t *src[3] = {q, k, v};
        for (int t = 0; t < 3; t++)
            if (!cuda_good(g, cudaMemcpy2DAsync(p.slot[s][t], row_bytes, src[t] + offset, pitch,
                                              row_bytes, sequence, cudaMemcpyHostToDevice, p.h2d)))
                return 0;
        if (!cuda_good(g, cudaEventRecord(p.loaded[s], p.h2d)) ||
            !cuda_good(g, cudaStreamWaitEvent(compute, p.loaded[s], 0)) ||
            !cuda_good(g, h3_flash3_bf16(p.slot[s][3], p.slot[s][0], p.slot[s][1], p.slot[s][2], nullptr,
                                       1, sequence, n, n, scale, compute)) ||
            !cuda_good(g, cudaEventRecord(p.computed[s], compute)) ||
            !cuda_good(g, cudaStreamWaitEvent(p.d2h, p.computed[s], 0)) ||
            !cuda_good(g, cudaMemcpy2DAsync(out + offset, pitch, p.slot[s][3], row_bytes, row_bytes,
                                          sequence, cudaMemcpyDeviceToHost, p.d2h)) ||
            !cuda_good(g, cudaEventRecord(p.stored[s], p.d2h)))
            return 0;
    }
    return cuda_good(g, cudaStreamSynchronize(p.d2h)) && cuda_good(g, cudaStreamSynchronize(p.compute[0])) &&
           cuda_good(g, cudaStreamSynchronize(p.compute[1])) && cuda_good(g, cudaStreamSynchronize(g->stream));
}

// ======================= Q/K norm + rotary embedding (attention's producer) =======================

namespace h3b {
// Checks the inputs of the norm + RoPE operator and fills the kernel's argument block.
int rope_input(h3_gpu *g, QkvRopeInput &in, const h3_gpu_tensor *qkv, const h3_gpu_tensor *qn,
               const h3_gpu_tensor *kn, const h3_gpu_tensor *co, const h3_gpu_tensor *si, uint32_t rows,
               uint32_t heads, uint32_t dim, uint32_t half, float eps, int grouped) {
    if (dim != 128 || half % 4 || half * 2 > dim || !rows || !heads) {
        fail(g, "qkv_rope: head_dim %u / rope_half %u not supported (128; multiple of 4, <= 64)", dim, half);
        return 0;
    }
    if (!satisfied(g, {bf16(qkv, (size_t)rows * heads * dim * 3, "QKV projection"), bf16(qn, dim, "query norm weight"),
                       bf16(kn, dim, "key norm weight"), bf16(co, (size_t)rows * half, "RoPE cosine"),
                       bf16(si, (size_t)rows * half, "RoPE sine")}))
        return 0;
    in = QkvRopeInput{qkv->data, qn->data, kn->data, co->data, si->data, rows, heads, half, grouped != 0, eps};
    return 1;
}
}  // namespace h3b

static int qkv_rope(h3_gpu *g, h3_gpu_tensor *q, h3_gpu_tensor *k, h3_gpu_tensor *v, const h3_gpu_tensor *x,
                    const h3_gpu_tensor *qn, const h3_gpu_tensor *kn, const h3_gpu_tensor *co,
                    const h3_gpu_tensor *si, uint32_t rows, uint32_t heads, uint32_t dim, uint32_t half, float eps,
                    int grouped) {
    if (!g) return 0;
    h3b::QkvRopeInput in{};
    if (!h3b::rope_input(g, in, x, qn, kn, co, si, rows, heads, dim, half, eps, grouped)) return 0;
    const size_t n = (size_t)rows * heads * dim;
    if (!satisfied(g, {bf16(q, n, "query"), bf16(k, n, "key"), bf16(v, n, "value")})) return 0;
    return cuda_good(g, h3b::qkv_rope_token_major(in, q->data, k->data, v->data, g->stream));
}
extern "C" int h3_gpu_qkv_rope_bf16(h3_gpu *g, h3_gpu_tensor *q, h3_gpu_tensor *k, h3_gpu_tensor *v,
                                    const h3_gpu_tensor *x, const h3_gpu_tensor *qn, const h3_gpu_tensor *kn,
                                    const h3_gpu_tensor *co, const h3_gpu_tensor *si, uint32_t s, uint32_t h,
                                    uint32_t d, uint32_t rh, float eps) {
    return qkv_rope(g, q, k, v, x, qn, kn, co, si, s, h, d, rh, eps, 0);
}
extern "C" int h3_gpu_grouped_qkv_rope_bf16(h3_gpu *g, h3_gpu_tensor *q, h3_gpu_tensor *k, h3_gpu_tensor *v,
                                            const h3_gpu_tensor *x, const h3_gpu_tensor *qn,
                                            const h3_gpu_tensor *kn, const h3_gpu_tensor *co,
                                            const h3_gpu_tensor *si, uint32_t s, uint32_t h, uint32_t d,
                                            uint32_t rh, float eps) {
    return qkv_rope(g, q, k, v, x, qn, kn, co, si, s, h, d, rh, eps, 1);
}
