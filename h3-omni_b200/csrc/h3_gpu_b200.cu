// Host side of the library: the five kernel-adapter entry points, and the attention subset of
// the reference's GPU primitive ABI (context, tensors, dense / rectangular / sparse attention,
// Ulysses exchanges) written against them. Argument checks, error strings and return
// conventions follow the reference's CUDA backend (cuda/h3_gpu_cuda.cu, cuda/vsa.cuh,
// cuda/parallel.cuh) so a caller cannot tell the two apart on this path.
#include <nccl.h>

#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>
#include <vector>

#include "../../include/h3b200_attn.h"
#include "attn_kernels.h"

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
}  // namespace h3b

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

extern "C" void h3b_vsa_fine_mode(int mode) { h3b::attn_sparse_set_mode(mode < 0 || mode > 2 ? 0 : mode); }

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

// Staging for h3b_sdpa_bf16_host: two slots of compact per-head-group device buffers,
// a stream for each copy direction and the events that order the three streams.
struct host_pipeline {
    void *slot[2][4]{};            // q, k, v, out per slot
    size_t slot_bytes{};
    cudaStream_t h2d{}, d2h{};
    cudaEvent_t loaded[2]{}, computed[2]{}, stored[2]{};
    bool ready{};
};
struct h3_gpu {
    int device{};
    cudaStream_t own_stream{}, stream{};
    char error[512]{};
    host_pipeline pipe;
};
struct h3_gpu_tensor {
    void *data{};
    size_t elements{}, bytes{};
    h3_gpu_dtype dtype{};
    h3_gpu *owner{};
    bool owns{};
};

static void set_error(h3_gpu *g, const char *format, ...) {
    if (!g) return;
    va_list args;
    va_start(args, format);
    vsnprintf(g->error, sizeof g->error, format, args);
    va_end(args);
}
static int cuda_ok(h3_gpu *g, cudaError_t e) {
    if (e == cudaSuccess) return 1;
    set_error(g, "CUDA: %s", cudaGetErrorString(e));
    return 0;
}
static size_t dtype_size(h3_gpu_dtype t) {
    return t == H3_GPU_F32 || t == H3_GPU_U32 ? 4 : t == H3_GPU_I8 ? 1 : 2;
}
static h3_gpu_tensor *allocate(h3_gpu *g, size_t elements, h3_gpu_dtype dtype) {
    if (!g || !elements) return nullptr;
    auto *t = new (std::nothrow) h3_gpu_tensor{};
    if (!t) return nullptr;
    t->elements = elements;
    t->bytes = elements * dtype_size(dtype);
    t->dtype = dtype;
    t->owner = g;
    t->owns = true;
    // Stream-ordered allocation, as the reference's pool (cuda/h3_gpu_cuda.cu:215-249).
    if (!cuda_ok(g, cudaMallocAsync(&t->data, t->bytes, g->stream))) {
        delete t;
        return nullptr;
    }
    return t;
}
static int require_elements(h3_gpu *g, const h3_gpu_tensor *t, size_t n, const char *what) {
    if (t && t->owner == g && t->elements >= n) return 1;
    set_error(g, "invalid tensor: %s (need %zu elements)", what, n);
    return 0;
}
static int require_bf16(h3_gpu *g, const h3_gpu_tensor *t, size_t n, const char *what) {
    if (!require_elements(g, t, n, what)) return 0;
    if (t->dtype == H3_GPU_BF16) return 1;
    set_error(g, "expected BF16: %s", what);
    return 0;
}

extern "C" h3_gpu *h3_gpu_create(const char *, char *error, size_t error_size) {
    auto fail = [&](const char *what, cudaError_t e) -> h3_gpu * {
        if (error && error_size) snprintf(error, error_size, "%s: %s", what, cudaGetErrorString(e));
        return nullptr;
    };
    int device = 0, major = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return fail("no CUDA device", e);
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
    if (e != cudaSuccess) return fail("device query", e);
    if (major != 10) {
        // No fallback: this library holds sm_100a code only.
        if (error && error_size)
            snprintf(error, error_size, "libh3b200_attn needs a B200-class GPU (sm_100), found sm_%d0",
                     major);
        return nullptr;
    }
    auto *g = new (std::nothrow) h3_gpu{};
    if (!g) return nullptr;
    g->device = device;
    e = cudaStreamCreateWithFlags(&g->own_stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
        delete g;
        return fail("stream", e);
    }
    g->stream = g->own_stream;
    return g;
}
static void pipeline_release(h3_gpu *g) {
    host_pipeline &p = g->pipe;
    if (!p.ready) return;
    cudaStreamSynchronize(p.h2d);
    cudaStreamSynchronize(p.d2h);
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
    cudaStreamDestroy(p.h2d);
    cudaStreamDestroy(p.d2h);
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
    if (!g) return 0;
    g->stream = stream ? stream : g->own_stream;
    return 1;
}
extern "C" cudaStream_t h3b_gpu_stream(const h3_gpu *g) { return g ? g->stream : nullptr; }

extern "C" h3_gpu_tensor *h3_gpu_tensor_new_f32(h3_gpu *g, size_t n) { return allocate(g, n, H3_GPU_F32); }
extern "C" h3_gpu_tensor *h3_gpu_tensor_new_bf16(h3_gpu *g, size_t n) { return allocate(g, n, H3_GPU_BF16); }
extern "C" h3_gpu_tensor *h3b_tensor_new_f16(h3_gpu *g, size_t n) { return allocate(g, n, H3_GPU_F16); }
static h3_gpu_tensor *from_host(h3_gpu *g, const void *values, size_t n, h3_gpu_dtype dtype) {
    if (!values) return nullptr;
    auto *t = allocate(g, n, dtype);
    if (!t) return nullptr;
    if (!cuda_ok(g, cudaMemcpyAsync(t->data, values, t->bytes, cudaMemcpyHostToDevice, g->stream)) ||
        !cuda_ok(g, cudaStreamSynchronize(g->stream))) {
        h3_gpu_tensor_free(t);
        return nullptr;
    }
    return t;
}
extern "C" h3_gpu_tensor *h3_gpu_tensor_from_f32(h3_gpu *g, const float *v, size_t n) {
    return from_host(g, v, n, H3_GPU_F32);
}
extern "C" h3_gpu_tensor *h3_gpu_tensor_from_bf16(h3_gpu *g, const uint16_t *v, size_t n) {
    return from_host(g, v, n, H3_GPU_BF16);
}
extern "C" h3_gpu_tensor *h3_gpu_tensor_from_u32(h3_gpu *g, const uint32_t *v, size_t n) {
    return from_host(g, v, n, H3_GPU_U32);
}
extern "C" h3_gpu_tensor *h3b_tensor_wrap(h3_gpu *g, void *device_pointer, size_t elements,
                                          h3_gpu_dtype dtype) {
    if (!g || !device_pointer || !elements) return nullptr;
    auto *t = new (std::nothrow) h3_gpu_tensor{};
    if (!t) return nullptr;
    t->data = device_pointer;
    t->elements = elements;
    t->bytes = elements * dtype_size(dtype);
    t->dtype = dtype;
    t->owner = g;
    t->owns = false;
    return t;
}
extern "C" void *h3b_tensor_data(const h3_gpu_tensor *t) { return t ? t->data : nullptr; }
extern "C" void h3_gpu_tensor_free(h3_gpu_tensor *t) {
    if (!t) return;
    if (t->owns && t->data) cudaFreeAsync(t->data, t->owner->stream);
    delete t;
}
extern "C" size_t h3_gpu_tensor_elements(const h3_gpu_tensor *t) { return t ? t->elements : 0; }
extern "C" h3_gpu_dtype h3_gpu_tensor_dtype(const h3_gpu_tensor *t) { return t ? t->dtype : H3_GPU_F32; }

static int read_back(const h3_gpu_tensor *t, void *values, size_t n, h3_gpu_dtype dtype) {
    if (!t || !values || t->dtype != dtype || n > t->elements) return 0;
    h3_gpu *g = t->owner;
    return cuda_ok(g, cudaMemcpyAsync(values, t->data, n * dtype_size(dtype), cudaMemcpyDeviceToHost,
                                      g->stream)) &&
           cuda_ok(g, cudaStreamSynchronize(g->stream));
}
extern "C" int h3_gpu_tensor_read_f32(const h3_gpu_tensor *t, float *v, size_t n) {
    return read_back(t, v, n, H3_GPU_F32);
}
extern "C" int h3_gpu_tensor_read_bf16(const h3_gpu_tensor *t, uint16_t *v, size_t n) {
    return read_back(t, v, n, H3_GPU_BF16);
}
static int write_range(h3_gpu_tensor *t, size_t offset, const void *values, size_t n,
                       h3_gpu_dtype dtype) {
    if (!t || !values || t->dtype != dtype || offset > t->elements || n > t->elements - offset)
        return 0;
    h3_gpu *g = t->owner;
    const size_t size = dtype_size(dtype);
    return cuda_ok(g, cudaMemcpyAsync(static_cast<char *>(t->data) + offset * size, values, n * size,
                                      cudaMemcpyHostToDevice, g->stream)) &&
           cuda_ok(g, cudaStreamSynchronize(g->stream));
}
extern "C" int h3_gpu_tensor_write_f32(h3_gpu_tensor *t, const float *v, size_t n) {
    return write_range(t, 0, v, n, H3_GPU_F32);
}
extern "C" int h3_gpu_tensor_write_bf16(h3_gpu_tensor *t, const uint16_t *v, size_t n) {
    return write_range(t, 0, v, n, H3_GPU_BF16);
}
extern "C" int h3_gpu_tensor_write_bf16_range(h3_gpu_tensor *t, size_t offset, const uint16_t *v,
                                              size_t n) {
    return write_range(t, offset, v, n, H3_GPU_BF16);
}
extern "C" int h3_gpu_begin(h3_gpu *g) { return g != nullptr; }
extern "C" int h3_gpu_continue(h3_gpu *g) { return g != nullptr; }
extern "C" int h3_gpu_submit(h3_gpu *g) {
    if (!g) return 0;
    if (!cuda_ok(g, cudaStreamSynchronize(g->stream))) return 0;
    int status = 0;
    if (!cuda_ok(g, cudaMemcpyFromSymbol(&status, h3b::g_device_status, sizeof(int)))) return 0;
    if (status) {
        set_error(g, status == 1 ? "device-side wait timed out (status 1)"
                                 : "device-side bounds check failed (status %d)", status);
        return 0;
    }
    return 1;
}
extern "C" const char *h3_gpu_error(const h3_gpu *g) { return g ? g->error : "no GPU context"; }
extern "C" int h3_gpu_zero(h3_gpu *g, h3_gpu_tensor *t) {
    return t && t->owner == g && cuda_ok(g, cudaMemsetAsync(t->data, 0, t->bytes, g->stream));
}
extern "C" int h3_gpu_copy_bf16(h3_gpu *g, h3_gpu_tensor *dst, size_t dst_offset,
                                const h3_gpu_tensor *src, size_t src_offset, size_t n) {
    if (!require_bf16(g, dst, dst_offset + n, "copy destination") ||
        !require_bf16(g, src, src_offset + n, "copy source"))
        return 0;
    return cuda_ok(g, cudaMemcpyAsync(static_cast<uint16_t *>(dst->data) + dst_offset,
                                      static_cast<const uint16_t *>(src->data) + src_offset, n * 2,
                                      cudaMemcpyDeviceToDevice, g->stream));
}
extern "C" int h3_gpu_download(h3_gpu *g, const h3_gpu_tensor *t, size_t offset, void *host,
                               size_t count) {
    if (!g || !t || t->owner != g || !host || offset > t->bytes || count > t->bytes - offset) return 0;
    return cuda_ok(g, cudaMemcpyAsync(host, static_cast<const char *>(t->data) + offset, count,
                                      cudaMemcpyDeviceToHost, g->stream)) &&
           cuda_ok(g, cudaStreamSynchronize(g->stream));
}

// ======================= dense / rectangular attention =======================

// cuda/h3_gpu_cuda.cu:1109-1130. The reference allocates a logsumexp tensor per call and frees
// it right after the enqueue without ever reading it; the kernels here take NULL instead.
static int sdpa(h3_gpu *g, h3_gpu_tensor *y, const h3_gpu_tensor *q, const h3_gpu_tensor *k,
                const h3_gpu_tensor *v, unsigned batch, unsigned n, unsigned h, unsigned kh,
                unsigned d, float scale, bool causal, bool allow_flash3) {
    if (!g) return 0;
    if (!n || !h || !kh || h % kh || !d || !batch) return 0;
    if (d != 128) {
        set_error(g, "BF16 attention supports head dimension 128 only");
        return 0;
    }
    const size_t qn = (size_t)batch * n * h * d, kn = (size_t)batch * n * kh * d;
    if (!require_bf16(g, q, qn, "attention query") || !require_bf16(g, k, kn, "attention key") ||
        !require_bf16(g, v, kn, "attention value") || !require_bf16(g, y, qn, "attention output"))
        return 0;
    return cuda_ok(g, !causal && allow_flash3
                          ? h3_flash3_bf16(y->data, q->data, k->data, v->data, nullptr, batch, n, h,
                                           kh, scale, g->stream)
                          : h3_flash_bf16(y->data, q->data, k->data, v->data, nullptr, batch, n, h,
                                          kh, scale, causal, g->stream));
}
extern "C" int h3_gpu_sdpa_bf16(h3_gpu *g, h3_gpu_tensor *y, const h3_gpu_tensor *q,
                                const h3_gpu_tensor *k, const h3_gpu_tensor *v, uint32_t n,
                                uint32_t h, uint32_t d, float s) {
    return sdpa(g, y, q, k, v, 1, n, h, h, d, s, false, true);
}
extern "C" int h3_gpu_sdpa_fa2_bf16(h3_gpu *g, h3_gpu_tensor *y, const h3_gpu_tensor *q,
                                    const h3_gpu_tensor *k, const h3_gpu_tensor *v, uint32_t n,
                                    uint32_t h, uint32_t d, float s) {
    return sdpa(g, y, q, k, v, 1, n, h, h, d, s, false, false);
}
extern "C" int h3_gpu_gqa_causal_bf16(h3_gpu *g, h3_gpu_tensor *y, const h3_gpu_tensor *q,
                                      const h3_gpu_tensor *k, const h3_gpu_tensor *v, uint32_t n,
                                      uint32_t h, uint32_t kh, uint32_t d, float s) {
    return sdpa(g, y, q, k, v, 1, n, h, kh, d, s, true, true);
}
extern "C" int h3_gpu_sdpa_f16_d64(h3_gpu *g, h3_gpu_tensor *y, const h3_gpu_tensor *q,
                                   const h3_gpu_tensor *k, const h3_gpu_tensor *v, uint32_t n,
                                   uint32_t h, uint32_t d, float s) {
    if (!g) return 0;
    const size_t count = (size_t)n * h * d;
    if (d != 64 || !n || !h) {
        set_error(g, "FP16 attention supports head dimension 64 only");
        return 0;
    }
    const h3_gpu_tensor *all[] = {q, k, v, y};
    const char *names[] = {"FP16 attention query", "FP16 attention key", "FP16 attention value",
                           "FP16 attention output"};
    for (int i = 0; i < 4; i++) {
        if (!require_elements(g, all[i], count, names[i])) return 0;
        if (all[i]->dtype != H3_GPU_F16) {
            set_error(g, "expected FP16: %s", names[i]);
            return 0;
        }
    }
    return cuda_ok(g, h3_flash3_f16_d64(y->data, q->data, k->data, v->data, nullptr, 1, n, h, s,
                                        g->stream));
}
extern "C" int h3_gpu_cross_attention_bf16(h3_gpu *g, h3_gpu_tensor *y, size_t yo,
                                           const h3_gpu_tensor *q, size_t qo,
                                           const h3_gpu_tensor *k, const h3_gpu_tensor *v, size_t ko,
                                           uint32_t nq, uint32_t nk, uint32_t heads) {
    if (!g) return 0;
    const size_t width = (size_t)heads * 128;
    if (!nq || !nk || !heads || !require_elements(g, y, (yo + nq) * width, "live output") ||
        !require_elements(g, q, (qo + nq) * width, "live query") ||
        !require_elements(g, k, (ko + nk) * width, "live key") ||
        !require_elements(g, v, (ko + nk) * width, "live value"))
        return 0;
    for (auto *t : {static_cast<const h3_gpu_tensor *>(y), q, k, v})
        if (t->dtype != H3_GPU_BF16) {
            set_error(g, "live attention requires BF16");
            return 0;
        }
    return cuda_ok(g, h3_flash3_cross_bf16(static_cast<uint16_t *>(y->data) + yo * width,
                                           static_cast<const uint16_t *>(q->data) + qo * width,
                                           static_cast<const uint16_t *>(k->data) + ko * width,
                                           static_cast<const uint16_t *>(v->data) + ko * width,
                                           nullptr, nq, nk, heads, 1.0f / sqrtf(128.0f), g->stream));
}

// Live-mode attention without the per-layer concatenation copies (an addition; the reference
// builds text | sink | recent0 | recent1 | current by device copies first, h3_dit_live.inc:81-94):
// query rows attend the listed K/V row ranges as if they were one tensor. Every range is
// [>= kv_row[s] + kv_rows[s]][heads][128] bf16; at most six ranges; scale 1/sqrt(128) as in
// h3_gpu_cross_attention_bf16.
extern "C" int h3b_cross_attention_segments_bf16(h3_gpu *g, h3_gpu_tensor *y, size_t yo,
                                                 const h3_gpu_tensor *q, size_t qo, uint32_t nq,
                                                 uint32_t heads, uint32_t segments,
                                                 const h3_gpu_tensor *const *k,
                                                 const h3_gpu_tensor *const *v, const size_t *kv_row,
                                                 const uint32_t *kv_rows) {
    if (!g) return 0;
    const size_t width = (size_t)heads * 128;
    if (!nq || !heads || !segments || segments > 6 || !k || !v || !kv_row || !kv_rows) {
        set_error(g, "segmented live attention: 1 to 6 key/value ranges and a non-empty query");
        return 0;
    }
    if (!require_bf16(g, y, (yo + nq) * width, "live output") ||
        !require_bf16(g, q, (qo + nq) * width, "live query"))
        return 0;
    const void *kp[6], *vp[6];
    for (uint32_t s = 0; s < segments; s++) {
        if (!kv_rows[s]) {
            set_error(g, "segmented live attention: range %u is empty", s);
            return 0;
        }
        if (!require_bf16(g, k[s], (kv_row[s] + kv_rows[s]) * width, "live key") ||
            !require_bf16(g, v[s], (kv_row[s] + kv_rows[s]) * width, "live value"))
            return 0;
        kp[s] = static_cast<const uint16_t *>(k[s]->data) + kv_row[s] * width;
        vp[s] = static_cast<const uint16_t *>(v[s]->data) + kv_row[s] * width;
    }
    return cuda_ok(g, h3b::attn_segments_tc5(static_cast<uint16_t *>(y->data) + yo * width,
                                             static_cast<const uint16_t *>(q->data) + qo * width, kp, vp,
                                             kv_rows, segments, nq, heads, 1.0f / sqrtf(128.0f), g->stream));
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
    if (!cuda_ok(g, cudaStreamCreateWithFlags(&p.h2d, cudaStreamNonBlocking)) ||
        !cuda_ok(g, cudaStreamCreateWithFlags(&p.d2h, cudaStreamNonBlocking)))
        return 0;
    for (int s = 0; s < 2; s++) {
        if (!cuda_ok(g, cudaEventCreateWithFlags(&p.loaded[s], cudaEventDisableTiming)) ||
            !cuda_ok(g, cudaEventCreateWithFlags(&p.computed[s], cudaEventDisableTiming)) ||
            !cuda_ok(g, cudaEventCreateWithFlags(&p.stored[s], cudaEventDisableTiming)))
            return 0;
        for (int t = 0; t < 4; t++)
            if (!cuda_ok(g, cudaMalloc(&p.slot[s][t], slot_bytes))) return 0;
    }
    p.slot_bytes = slot_bytes;
    p.ready = true;
    return 1;
}
extern "C" int h3b_sdpa_bf16_host(h3_gpu *g, uint16_t *out, const uint16_t *q, const uint16_t *k,
                                  const uint16_t *v, uint32_t sequence, uint32_t heads,
                                  uint32_t head_dim, float scale, uint32_t head_groups) {
    if (!g) return 0;
    if (!out || !q || !k || !v || !sequence || !heads) {
        set_error(g, "host attention: null pointer or empty shape");
        return 0;
    }
    if (head_dim != 128) {
        set_error(g, "BF16 attention supports head dimension 128 only");
        return 0;
    }
    if (!head_groups || heads % head_groups) {
        set_error(g, "host attention: %u heads do not split into %u groups", heads, head_groups);
        return 0;
    }
    const uint32_t hg = heads / head_groups;
    const size_t pitch = (size_t)heads * 256;
    if (!pipeline_prepare(g, (size_t)hg * 256 * sequence)) return 0;
    host_pipeline &p = g->pipe;
    // The first and the last group are cut in two: the copy-in before the first kernel and the
    // copy-out after the last one are the only transfers nothing overlaps, so they are made short.
    uint32_t first_head[66], head_count[66];
    uint32_t chunks = 0;
    if (head_groups > 64) {
        set_error(g, "host attention: at most 64 head groups");
        return 0;
    }
    for (uint32_t group = 0; group < head_groups; group++) {
        const bool edge = (group == 0 || group + 1 == head_groups) && hg >= 2;
        const uint32_t parts = edge ? 2 : 1, base = group * hg;
        for (uint32_t part = 0; part < parts; part++) {
            first_head[chunks] = base + (part ? hg / 2 : 0);
            head_count[chunks++] = parts == 1 ? hg : part ? hg - hg / 2 : hg / 2;
        }
    }
    // everything already queued on the context's stream comes first
    if (!cuda_ok(g, cudaEventRecord(p.computed[0], g->stream)) ||
        !cuda_ok(g, cudaStreamWaitEvent(p.h2d, p.computed[0], 0)))
        return 0;
    for (uint32_t chunk = 0; chunk < chunks; chunk++) {
        const int s = chunk & 1;
        const uint32_t n = head_count[chunk];
        const size_t offset = (size_t)first_head[chunk] * 128;   // elements into a host row
        const size_t row_bytes = (size_t)n * 256;
        if (chunk >= 2) {
            // slot reuse: inputs after the kernel of chunk-2, output after its copy-out
            if (!cuda_ok(g, cudaStreamWaitEvent(p.h2d, p.computed[s], 0)) ||
                !cuda_ok(g, cudaStreamWaitEvent(g->stream, p.stored[s], 0)))
                return 0;
        }
        const uint16_t *src[3] = {q, k, v};
        for (int t = 0; t < 3; t++)
            if (!cuda_ok(g, cudaMemcpy2DAsync(p.slot[s][t], row_bytes, src[t] + offset, pitch,
                                              row_bytes, sequence, cudaMemcpyHostToDevice, p.h2d)))
                return 0;
        if (!cuda_ok(g, cudaEventRecord(p.loaded[s], p.h2d)) ||
            !cuda_ok(g, cudaStreamWaitEvent(g->stream, p.loaded[s], 0)) ||
            !cuda_ok(g, h3_flash3_bf16(p.slot[s][3], p.slot[s][0], p.slot[s][1], p.slot[s][2], nullptr,
                                       1, sequence, n, n, scale, g->stream)) ||
            !cuda_ok(g, cudaEventRecord(p.computed[s], g->stream)) ||
            !cuda_ok(g, cudaStreamWaitEvent(p.d2h, p.computed[s], 0)) ||
            !cuda_ok(g, cudaMemcpy2DAsync(out + offset, pitch, p.slot[s][3], row_bytes, row_bytes,
                                          sequence, cudaMemcpyDeviceToHost, p.d2h)) ||
            !cuda_ok(g, cudaEventRecord(p.stored[s], p.d2h)))
            return 0;
    }
    return cuda_ok(g, cudaStreamSynchronize(p.d2h)) && cuda_ok(g, cudaStreamSynchronize(g->stream));
}

// ======================= Q/K norm + rotary embedding (attention's producer) =======================

static int rope_input(h3_gpu *g, h3b::QkvRopeInput &in, const h3_gpu_tensor *qkv, const h3_gpu_tensor *qn,
                      const h3_gpu_tensor *kn, const h3_gpu_tensor *co, const h3_gpu_tensor *si,
                      uint32_t rows, uint32_t heads, uint32_t dim, uint32_t half, float eps, int grouped) {
    if (dim != 128 || half % 4 || half * 2 > dim || !rows || !heads) {
        set_error(g, "qkv_rope: head_dim %u / rope_half %u not supported (128; multiple of 4, <= 64)", dim, half);
        return 0;
    }
    const size_t inner = (size_t)heads * dim;
    if (!require_bf16(g, qkv, (size_t)rows * inner * 3, "QKV projection") ||
        !require_bf16(g, qn, dim, "query norm weight") || !require_bf16(g, kn, dim, "key norm weight") ||
        !require_bf16(g, co, (size_t)rows * half, "RoPE cosine") ||
        !require_bf16(g, si, (size_t)rows * half, "RoPE sine"))
        return 0;
    in = h3b::QkvRopeInput{qkv->data, qn->data, kn->data, co->data, si->data, rows, heads, half, grouped != 0, eps};
    return 1;
}
static int qkv_rope(h3_gpu *g, h3_gpu_tensor *q, h3_gpu_tensor *k, h3_gpu_tensor *v, const h3_gpu_tensor *x,
                    const h3_gpu_tensor *qn, const h3_gpu_tensor *kn, const h3_gpu_tensor *co,
                    const h3_gpu_tensor *si, uint32_t rows, uint32_t heads, uint32_t dim, uint32_t half,
                    float eps, int grouped) {
    if (!g) return 0;
    h3b::QkvRopeInput in{};
    if (!rope_input(g, in, x, qn, kn, co, si, rows, heads, dim, half, eps, grouped)) return 0;
    const size_t n = (size_t)rows * heads * dim;
    if (!require_bf16(g, q, n, "query") || !require_bf16(g, k, n, "key") || !require_bf16(g, v, n, "value"))
        return 0;
    return cuda_ok(g, h3b::qkv_rope_token_major(in, q->data, k->data, v->data, g->stream));
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

// ======================= video sparse attention =======================

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
    for (auto *t : {s->map, s->sizes, s->q, s->k, s->v, s->out, s->poolq, s->poolk, s->poolv,
                    s->scores, s->compression, s->indices, s->counts})
        h3_gpu_tensor_free(t);
    for (cudaEvent_t e : s->stage)
        if (e) cudaEventDestroy(e);
    delete s;
}

// Tile map of cuda/vsa.cuh:192-242: dense 64-row text and audio tiles, then 4x4x4 cubes of the
// (time, height, width) token grid in raster order with (dt, dy, dx) order inside a cube.
extern "C" h3_gpu_vsa *h3_gpu_vsa_new(h3_gpu *g, uint32_t text, uint32_t audio, uint32_t time,
                                      uint32_t height, uint32_t width, uint32_t heads) {
    if (!g || !text || !audio || !time || !height || !width || !heads) return nullptr;
    constexpr uint64_t MAX_TILES = 4096;
    const uint64_t blocks = ((uint64_t)text + 63) / 64 + ((uint64_t)audio + 63) / 64;
    const uint64_t nt = ((uint64_t)time + 3) / 4, nh = ((uint64_t)height + 3) / 4,
                   nw = ((uint64_t)width + 3) / 4;
    if (blocks >= MAX_TILES || nt > MAX_TILES || nh > MAX_TILES || nw > MAX_TILES ||
        blocks + nt * nh * nw > MAX_TILES || heads > 56) {
        set_error(g, "VSA requires at most %d tiles and 56 heads", (int)MAX_TILES);
        return nullptr;
    }
    std::vector<int> map, sizes;
    try {
        map.reserve((blocks + nt * nh * nw) * 64);
        sizes.reserve(blocks + nt * nh * nw);
    } catch (const std::bad_alloc &) {
        set_error(g, "out of host memory constructing VSA tiles");
        return nullptr;
    }
    int cursor = 0, prefix = 0;
    for (uint32_t count : {text, audio}) {
        for (uint32_t i = 0; i < count; i += 64, ++prefix) {
            const int valid = (int)std::min<uint32_t>(64, count - i);
            sizes.push_back(valid);
            for (int j = 0; j < 64; j++) map.push_back(j < valid ? cursor + (int)i + j : -1);
        }
        cursor += (int)count;
    }
    for (uint32_t t = 0; t < time; t += 4)
        for (uint32_t y = 0; y < height; y += 4)
            for (uint32_t x = 0; x < width; x += 4) {
                const size_t start = map.size();
                for (uint32_t dt = t; dt < std::min(time, t + 4); dt++)
                    for (uint32_t dy = y; dy < std::min(height, y + 4); dy++)
                        for (uint32_t dx = x; dx < std::min(width, x + 4); dx++)
                            map.push_back(cursor + (int)((dt * height + dy) * width + dx));
                sizes.push_back((int)(map.size() - start));
                map.resize(start + 64, -1);
            }
    auto *s = new (std::nothrow) h3_gpu_vsa{};
    if (!s) return nullptr;
    s->gpu = g;
    s->rows = cursor + (int)(time * height * width);
    s->heads = (int)heads;
    s->tiles = (int)sizes.size();
    s->prefix = prefix;
    s->keep = std::max(1, (s->tiles - prefix + 9) / 10);  // cuda/vsa.cuh:242
    const size_t n = map.size() * heads * 128, pool = sizes.size() * heads * 128;
    s->map = allocate(g, map.size(), H3_GPU_U32);
    s->sizes = allocate(g, sizes.size(), H3_GPU_U32);
    s->q = allocate(g, n, H3_GPU_BF16);
    s->k = allocate(g, n, H3_GPU_BF16);
    s->v = allocate(g, n, H3_GPU_BF16);
    s->out = allocate(g, n, H3_GPU_BF16);
    s->poolq = allocate(g, pool, H3_GPU_F32);
    s->poolk = allocate(g, pool, H3_GPU_F32);
    s->poolv = allocate(g, pool, H3_GPU_F32);
    s->compression = allocate(g, pool, H3_GPU_F32);
    s->indices = allocate(g, sizes.size() * sizes.size() * heads, H3_GPU_U32);
    s->counts = allocate(g, sizes.size() * heads, H3_GPU_U32);
    if (!s->map || !s->sizes || !s->q || !s->k || !s->v || !s->out || !s->poolq || !s->poolk ||
        !s->poolv || !s->compression || !s->indices || !s->counts ||
        !cuda_ok(g, cudaMemcpyAsync(s->map->data, map.data(), map.size() * sizeof(int),
                                    cudaMemcpyHostToDevice, g->stream)) ||
        !cuda_ok(g, cudaMemcpyAsync(s->sizes->data, sizes.data(), sizes.size() * sizeof(int),
                                    cudaMemcpyHostToDevice, g->stream)) ||
        !cuda_ok(g, cudaStreamSynchronize(g->stream))) {
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
        s->scores = allocate(s->gpu, (size_t)s->tiles * s->tiles * s->heads, H3_GPU_F32);
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
            if (!e && !cuda_ok(s->gpu, cudaEventCreate(&e))) return 0;
    s->time_stages = enable != 0;
    return 1;
}
// Milliseconds of the last call's four stages: pooling (or norm + RoPE + pooling), scores +
// selection + compression, block-sparse attention, merge. Waits for that call to finish.
extern "C" int h3b_vsa_stage_ms(h3_gpu_vsa *s, float *ms) {
    if (!s || !ms || !s->time_stages) return 0;
    if (!cuda_ok(s->gpu, cudaEventSynchronize(s->stage[4]))) return 0;
    for (int i = 0; i < 4; i++)
        if (!cuda_ok(s->gpu, cudaEventElapsedTime(&ms[i], s->stage[i], s->stage[i + 1]))) return 0;
    return 1;
}
extern "C" void *h3b_vsa_buffer(const h3_gpu_vsa *s, int which) {
    if (!s) return nullptr;
    const h3_gpu_tensor *all[] = {s->map, s->sizes, s->q, s->k, s->v, s->out, s->poolq, s->poolk,
                                  s->poolv, s->indices, s->counts, s->compression, s->scores};
    if (which < 0 || which >= (int)(sizeof all / sizeof all[0]) || !all[which]) return nullptr;
    return all[which]->data;
}

static int vsa_mark(h3_gpu_vsa *s, int which) {
    return !s->time_stages || cuda_ok(s->gpu, cudaEventRecord(s->stage[which], s->gpu->stream));
}

// Everything after the tiled copies and tile means exist: scores + selection + compression,
// the block-sparse kernel, merge back to token order (cuda/vsa.cuh:281-299).
static int vsa_after_tiling(h3_gpu_vsa *s, h3_gpu_tensor *out, const h3_gpu_tensor *gate) {
    h3_gpu *g = s->gpu;
    float *pooled[3] = {(float *)s->poolq->data, (float *)s->poolk->data, (float *)s->poolv->data};
    const int *map = (const int *)s->map->data;
    const float scale = 1.0f / sqrtf(128.0f);
    if (!vsa_mark(s, 1)) return 0;
    if (!cuda_ok(g, h3b::vsa_score_select_compress(
                        pooled[0], pooled[1], pooled[2],
                        s->trace_scores ? (float *)s->scores->data : nullptr,
                        (int *)s->indices->data, (int *)s->counts->data,
                        (float *)s->compression->data, s->tiles, s->prefix, s->keep, s->heads, scale,
                        g->stream)))
        return 0;
    if (!vsa_mark(s, 2)) return 0;
    if (!cuda_ok(g, h3_vsa_hopper(s->out->data, s->q->data, s->k->data, s->v->data, nullptr,
                                  (int *)s->indices->data, (int *)s->counts->data,
                                  (int *)s->sizes->data, s->tiles, s->heads, g->stream)))
        return 0;
    if (!vsa_mark(s, 3)) return 0;
    return cuda_ok(g, h3b::vsa_untile_merge(out->data, s->out->data, gate->data,
                                            (const float *)s->compression->data, map, s->tiles,
                                            s->heads, g->stream)) &&
           vsa_mark(s, 4);
}


// cuda/vsa.cuh:263-300, as three launches around the block-sparse kernel.
extern "C" int h3_gpu_vsa_bf16(h3_gpu_vsa *s, h3_gpu_tensor *out, const h3_gpu_tensor *q,
                               const h3_gpu_tensor *k, const h3_gpu_tensor *value,
                               const h3_gpu_tensor *gate) {
    if (!s) return 0;
    h3_gpu *g = s->gpu;
    const size_t elements = (size_t)s->rows * s->heads * 128;
    const h3_gpu_tensor *tensors[] = {out, q, k, value, gate};
    for (auto *t : tensors)
        if (!require_bf16(g, t, elements, "VSA input/output")) return 0;
    const void *src[3] = {q->data, k->data, value->data};
    void *tiled[3] = {s->q->data, s->k->data, s->v->data};
    float *pooled[3] = {(float *)s->poolq->data, (float *)s->poolk->data, (float *)s->poolv->data};
    const int *map = (const int *)s->map->data, *sizes = (const int *)s->sizes->data;
    if (!vsa_mark(s, 0)) return 0;
    if (!cuda_ok(g, h3b::vsa_tile_pool3(src, tiled, pooled, map, sizes, s->tiles, s->heads, 3,
                                        g->stream)))
        return 0;
    return vsa_after_tiling(s, out, gate);
}

// The same pipeline fed by the QKV projection output: norm + rotation write the tiled copies and
// the tile means themselves (csrc/qkv_rope.cu), then the shared remainder.
extern "C" int h3b_vsa_qkv_rope_bf16(h3_gpu_vsa *s, h3_gpu_tensor *out, const h3_gpu_tensor *qkv,
                                     const h3_gpu_tensor *qn, const h3_gpu_tensor *kn,
                                     const h3_gpu_tensor *co, const h3_gpu_tensor *si,
                                     const h3_gpu_tensor *gate, uint32_t rope_half, float eps, int grouped) {
    if (!s) return 0;
    h3_gpu *g = s->gpu;
    const size_t elements = (size_t)s->rows * s->heads * 128;
    if (!require_bf16(g, out, elements, "VSA output") || !require_bf16(g, gate, elements, "VSA gate")) return 0;
    h3b::QkvRopeInput in{};
    if (!rope_input(g, in, qkv, qn, kn, co, si, (uint32_t)s->rows, (uint32_t)s->heads, 128, rope_half, eps, grouped))
        return 0;
    void *tiled[3] = {s->q->data, s->k->data, s->v->data};
    float *pooled[3] = {(float *)s->poolq->data, (float *)s->poolk->data, (float *)s->poolv->data};
    if (!vsa_mark(s, 0)) return 0;
    if (!cuda_ok(g, h3b::qkv_rope_vsa_tiles(in, (const int *)s->map->data, (const int *)s->sizes->data,
                                            s->tiles, tiled, pooled, g->stream)))
        return 0;
    return vsa_after_tiling(s, out, gate);
}

// ======================= multi-GPU: communicators and Ulysses =======================

struct h3_gpu_comm {
    ncclComm_t comm;
    int rank;
    int size;
};
static int nccl_ok(h3_gpu *g, ncclResult_t r, const char *what) {
    if (r == ncclSuccess) return 1;
    set_error(g, "NCCL %s: %s", what, ncclGetErrorString(r));
    return 0;
}
extern "C" int h3_gpu_device_count(void) {
    int count = 0;
    return cudaGetDeviceCount(&count) == cudaSuccess ? count : 0;
}
extern "C" int h3_gpu_select_device(int device, char *error, size_t size) {
    cudaError_t e = cudaSetDevice(device);
    if (e == cudaSuccess) return 1;
    if (error && size)
        snprintf(error, size, "cannot select CUDA device %d: %s", device, cudaGetErrorString(e));
    return 0;
}
extern "C" int h3_gpu_comm_init_all(int count, h3_gpu_comm **comms, char *error, size_t size) {
    if (count < 1 || count > 64 || !comms) {
        if (error && size) snprintf(error, size, "invalid NCCL communicator count %d", count);
        return 0;
    }
    std::vector<ncclComm_t> raw(count);
    std::vector<int> devices(count);
    for (int i = 0; i < count; i++) devices[i] = i;
    ncclResult_t r = ncclCommInitAll(raw.data(), count, devices.data());
    if (r != ncclSuccess) {
        if (error && size) snprintf(error, size, "NCCL init: %s", ncclGetErrorString(r));
        return 0;
    }
    for (int i = 0; i < count; i++) comms[i] = new h3_gpu_comm{raw[i], i, count};
    return 1;
}
extern "C" int h3b_comm_unique_id(void *id128, char *error, size_t size) {
    static_assert(sizeof(ncclUniqueId) == 128, "unique id size");
    ncclUniqueId id;
    ncclResult_t r = id128 ? ncclGetUniqueId(&id) : ncclInvalidArgument;
    if (r != ncclSuccess) {
        if (error && size) snprintf(error, size, "NCCL unique id: %s", ncclGetErrorString(r));
        return 0;
    }
    memcpy(id128, &id, sizeof id);
    return 1;
}
extern "C" int h3b_comm_init_rank(const void *id128, int rank, int count, h3_gpu_comm **comm,
                                  char *error, size_t size) {
    if (!id128 || !comm || count < 1 || rank < 0 || rank >= count) {
        if (error && size) snprintf(error, size, "invalid NCCL rank %d of %d", rank, count);
        return 0;
    }
    ncclUniqueId id;
    memcpy(&id, id128, sizeof id);
    ncclComm_t raw;
    ncclResult_t r = ncclCommInitRank(&raw, count, id, rank);
    if (r != ncclSuccess) {
        if (error && size) snprintf(error, size, "NCCL init: %s", ncclGetErrorString(r));
        return 0;
    }
    *comm = new h3_gpu_comm{raw, rank, count};
    return 1;
}
extern "C" int h3b_comm_rank(const h3_gpu_comm *c) { return c ? c->rank : -1; }
extern "C" int h3b_comm_size(const h3_gpu_comm *c) { return c ? c->size : 0; }
extern "C" void h3_gpu_comm_free(h3_gpu_comm *c) {
    if (!c) return;
    if (c->comm) ncclCommDestroy(c->comm);
    delete c;
}
// Unblocks every rank waiting in a collective after one rank failed (cuda/parallel.cuh:60-65).
extern "C" void h3_gpu_comm_abort(h3_gpu_comm *c) {
    if (c && c->comm) ncclCommAbort(c->comm);
    if (c) c->comm = nullptr;
}

static int swap_leading_bf16(h3_gpu *g, void *out, const void *in, unsigned a, unsigned b,
                             size_t c_elements) {
    const size_t bytes = c_elements * 2;
    if (bytes % 16) {
        set_error(g, "Ulysses block of %zu bytes is not 16-byte aligned", bytes);
        return 0;
    }
    return cuda_ok(g, h3b::swap_leading_16b(out, in, a, b, bytes / 16, g->stream));
}
// Every rank sends block j of `send` to rank j and receives rank j's block into block j.
static int all_to_all(h3_gpu *g, h3_gpu_comm *c, void *recv, const void *send, size_t block_bytes) {
    if (!nccl_ok(g, ncclGroupStart(), "group start")) return 0;
    for (int peer = 0; peer < c->size; peer++) {
        ncclResult_t r = ncclSend((const char *)send + peer * block_bytes, block_bytes, ncclUint8,
                                  peer, c->comm, g->stream);
        if (r == ncclSuccess)
            r = ncclRecv((char *)recv + peer * block_bytes, block_bytes, ncclUint8, peer, c->comm,
                         g->stream);
        if (r != ncclSuccess) {
            ncclGroupEnd();
            return nccl_ok(g, r, "all-to-all");
        }
    }
    return nccl_ok(g, ncclGroupEnd(), "group end");
}
static int ulysses_check(h3_gpu *g, h3_gpu_comm *c, const h3_gpu_tensor *t,
                         const h3_gpu_tensor *scratch, unsigned rows, unsigned heads, unsigned dim) {
    const size_t count = (size_t)rows * heads * dim;
    if (!c || !c->comm || heads % c->size) {
        set_error(g, "Ulysses: %u heads do not split over %d ranks", heads, c ? c->size : 0);
        return 0;
    }
    return require_bf16(g, t, count, "Ulysses tensor") &&
           require_bf16(g, scratch, count, "Ulysses scratch");
}
// [rows][heads][dim] on each rank -> [ranks*rows][heads/ranks][dim] (cuda/parallel.cuh:125-133).
extern "C" int h3_gpu_ulysses_scatter_heads_bf16(h3_gpu *g, h3_gpu_comm *c, h3_gpu_tensor *t,
                                                 h3_gpu_tensor *scratch, uint32_t rows,
                                                 uint32_t heads, uint32_t dim) {
    if (!g || !ulysses_check(g, c, t, scratch, rows, heads, dim)) return 0;
    const size_t group = (size_t)(heads / c->size) * dim;
    return swap_leading_bf16(g, scratch->data, t->data, rows, c->size, group) &&
           all_to_all(g, c, t->data, scratch->data, (size_t)rows * group * 2);
}
// The inverse (cuda/parallel.cuh:135-143).
extern "C" int h3_gpu_ulysses_gather_heads_bf16(h3_gpu *g, h3_gpu_comm *c, h3_gpu_tensor *t,
                                                h3_gpu_tensor *scratch, uint32_t rows,
                                                uint32_t heads, uint32_t dim) {
    if (!g || !ulysses_check(g, c, t, scratch, rows, heads, dim)) return 0;
    const size_t group = (size_t)(heads / c->size) * dim;
    return all_to_all(g, c, scratch->data, t->data, (size_t)rows * group * 2) &&
           swap_leading_bf16(g, t->data, scratch->data, c->size, rows, group);
}
// output[rank * count + i] = input_of_rank[i] (cuda/parallel.cuh:146-153).
extern "C" int h3_gpu_all_gather_bf16(h3_gpu *g, h3_gpu_comm *c, h3_gpu_tensor *output,
                                      const h3_gpu_tensor *input, size_t count) {
    if (!g || !c || !c->comm || !require_bf16(g, input, count, "all-gather input") ||
        !require_bf16(g, output, count * c->size, "all-gather output"))
        return 0;
    return nccl_ok(g, ncclAllGather(input->data, output->data, count * 2, ncclUint8, c->comm,
                                    g->stream), "all-gather");
}

// ======================= fused Ulysses exchange over peer memory =======================
// One process per GPU: each rank owns a window (cudaMalloc, exported as a CUDA IPC handle) of
// `slots` tensors plus a flag array; after h3b_exchange_connect every rank holds mappings of
// all windows and an exchange is one kernel (csrc/ulysses.cu) instead of a transpose kernel
// plus NCCL send/recv. No counterpart in the reference, which exchanges through NCCL only.
struct h3b_exchange {
    h3_gpu *gpu{};
    int rank{}, ranks{}, slots{};
    size_t slot_elements{}, slot_bytes{}, flags_offset{};
    char *local{};                       // this rank's window
    char *mapped[16]{};                  // every rank's window as seen from here
    unsigned *done_counter{};            // in the local window, after the flags
    unsigned long long epoch{};
    bool connected{};
};

extern "C" void h3b_exchange_free(h3b_exchange *x) {
    if (!x) return;
    cudaStreamSynchronize(x->gpu->stream);
    for (int p = 0; p < x->ranks; p++)
        if (p != x->rank && x->mapped[p]) cudaIpcCloseMemHandle(x->mapped[p]);
    if (x->local) cudaFree(x->local);
    delete x;
}

extern "C" int h3b_exchange_create(h3_gpu *g, int rank, int ranks, size_t slot_elements, int slots,
                                   h3b_exchange **exchange, void *handle64) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    if (!g || !exchange || !handle64 || ranks < 1 || ranks > 16 || rank < 0 || rank >= ranks ||
        slots < 1 || !slot_elements) {
        set_error(g, "exchange: invalid rank %d of %d or empty window", rank, ranks);
        return 0;
    }
    auto *x = new (std::nothrow) h3b_exchange{};
    if (!x) return 0;
    x->gpu = g;
    x->rank = rank;
    x->ranks = ranks;
    x->slots = slots;
    x->slot_elements = slot_elements;
    x->slot_bytes = (slot_elements * 2 + 255) / 256 * 256;
    x->flags_offset = x->slot_bytes * slots;
    const size_t bytes = x->flags_offset + 16 * sizeof(unsigned long long) + 256;
    cudaIpcMemHandle_t handle;
    if (!cuda_ok(g, cudaMalloc(reinterpret_cast<void **>(&x->local), bytes)) ||
        !cuda_ok(g, cudaMemset(x->local, 0, bytes)) ||
        !cuda_ok(g, cudaIpcGetMemHandle(&handle, x->local))) {
        h3b_exchange_free(x);
        return 0;
    }
    x->done_counter = reinterpret_cast<unsigned *>(x->local + x->flags_offset + 16 * sizeof(unsigned long long));
    x->mapped[rank] = x->local;
    memcpy(handle64, &handle, 64);
    *exchange = x;
    return 1;
}

// handles: ranks x 64 bytes in rank order (every rank's handle64, gathered by any transport).
extern "C" int h3b_exchange_connect(h3b_exchange *x, const void *handles) {
    if (!x || !handles) return 0;
    h3_gpu *g = x->gpu;
    for (int p = 0; p < x->ranks; p++) {
        if (p == x->rank) continue;
        cudaIpcMemHandle_t handle;
        memcpy(&handle, static_cast<const char *>(handles) + 64 * p, 64);
        void *mapped = nullptr;
        if (!cuda_ok(g, cudaIpcOpenMemHandle(&mapped, handle, cudaIpcMemLazyEnablePeerAccess))) return 0;
        x->mapped[p] = static_cast<char *>(mapped);
    }
    x->connected = true;
    return 1;
}

// Non-owning tensor over slot `slot` of this rank's window (free it with h3_gpu_tensor_free).
extern "C" h3_gpu_tensor *h3b_exchange_slot(h3b_exchange *x, int slot) {
    if (!x || slot < 0 || slot >= x->slots) return nullptr;
    return h3b_tensor_wrap(x->gpu, x->local + x->slot_bytes * slot, x->slot_elements, H3_GPU_BF16);
}

static int exchange_run(h3b_exchange *x, bool gather, int slot, const h3_gpu_tensor *src, uint32_t rows,
                        uint32_t heads, uint32_t dim) {
    if (!x) return 0;
    h3_gpu *g = x->gpu;
    const size_t count = (size_t)rows * heads * dim;
    if (!x->connected || slot < 0 || slot >= x->slots || heads % x->ranks || count > x->slot_elements) {
        set_error(g, "exchange: not connected, bad slot, %u heads over %d ranks, or %zu elements exceed the slot",
                  heads, x->ranks, count);
        return 0;
    }
    if (!require_bf16(g, src, count, "exchange source")) return 0;
    void *window[16];
    unsigned long long *flags[16];
    for (int p = 0; p < x->ranks; p++) {
        window[p] = x->mapped[p] + x->slot_bytes * slot;
        flags[p] = reinterpret_cast<unsigned long long *>(x->mapped[p] + x->flags_offset);
    }
    int *status = nullptr;
    if (!cuda_ok(g, h3b::device_status_word(&status))) return 0;
    return cuda_ok(g, h3b::exchange_push(gather, src->data, window, flags, ++x->epoch, x->done_counter, status,
                                         x->rank, x->ranks, rows, heads, dim, g->stream));
}
// src [rows][heads][dim] on each rank -> slot of every rank: [ranks*rows][heads/ranks][dim].
extern "C" int h3b_exchange_scatter_heads_bf16(h3b_exchange *x, int slot, const h3_gpu_tensor *src,
                                               uint32_t rows, uint32_t heads, uint32_t dim) {
    return exchange_run(x, false, slot, src, rows, heads, dim);
}
// src [ranks*rows][heads/ranks][dim] on each rank -> slot of every rank: [rows][heads][dim].
extern "C" int h3b_exchange_gather_heads_bf16(h3b_exchange *x, int slot, const h3_gpu_tensor *src,
                                              uint32_t rows, uint32_t heads, uint32_t dim) {
    return exchange_run(x, true, slot, src, rows, heads, dim);
}

// Attention with the sequence-gather fused into its epilogue: every rank attends all
// `sequence` rows for its heads / ranks heads (q, k, v: [>= sequence][heads/ranks][128], e.g.
// the scatter slots) and each finished output row is stored straight into the row shard of the
// rank that owns it, slot `slot` of that rank's window laid out [rows][heads][128]. One
// attention launch plus a one-warp epoch handshake replace attention + gather kernel.
extern "C" int h3b_exchange_sdpa_gather_bf16(h3b_exchange *x, int slot, const h3_gpu_tensor *q,
                                             const h3_gpu_tensor *k, const h3_gpu_tensor *v,
                                             uint32_t sequence, uint32_t rows, uint32_t heads,
                                             float scale) {
    if (!x) return 0;
    h3_gpu *g = x->gpu;
    if (!x->connected || slot < 0 || slot >= x->slots || !heads || heads % x->ranks || !rows ||
        (size_t)rows * heads * 128 > x->slot_elements || (size_t)sequence > (size_t)rows * x->ranks) {
        set_error(g, "fused attention+gather: not connected, bad slot or shape (%u rows x %d ranks, %u heads)",
                  rows, x->ranks, heads);
        return 0;
    }
    const uint32_t local_heads = heads / x->ranks;
    const size_t need = (size_t)sequence * local_heads * 128;
    if (!require_bf16(g, q, need, "attention query") || !require_bf16(g, k, need, "attention key") ||
        !require_bf16(g, v, need, "attention value"))
        return 0;
    h3b::PeerOutput peer{};
    unsigned long long *flags[16];
    for (int p = 0; p < x->ranks; p++) {
        peer.base[p] = x->mapped[p] + x->slot_bytes * slot;
        flags[p] = reinterpret_cast<unsigned long long *>(x->mapped[p] + x->flags_offset);
    }
    peer.rows_per_rank = rows;
    peer.rank = (unsigned)x->rank;
    peer.total_heads = heads;
    int *status = nullptr;
    if (!cuda_ok(g, h3b::device_status_word(&status))) return 0;
    return cuda_ok(g, h3b::attn_dense_tc5(nullptr, q->data, k->data, v->data, nullptr, 1, sequence, sequence,
                                          local_heads, local_heads, scale, g->stream, &peer)) &&
           cuda_ok(g, h3b::exchange_handshake(flags, ++x->epoch, status, x->rank, x->ranks, g->stream));
}

// Producer fused with the head scatter: norm + rotation store each (row, head) vector of q, k
// and v into the owning rank's slots, then one epoch handshake for all three tensors.
extern "C" int h3b_exchange_qkv_rope_scatter_bf16(h3b_exchange *x, int slot_q, int slot_k, int slot_v,
                                                  const h3_gpu_tensor *qkv, const h3_gpu_tensor *qn,
                                                  const h3_gpu_tensor *kn, const h3_gpu_tensor *co,
                                                  const h3_gpu_tensor *si, uint32_t rows, uint32_t heads,
                                                  uint32_t rope_half, float eps, int grouped) {
    if (!x) return 0;
    h3_gpu *g = x->gpu;
    const int slots[3] = {slot_q, slot_k, slot_v};
    bool bad = !x->connected || !heads || heads % x->ranks || (size_t)rows * heads * 128 > x->slot_elements;
    for (int t = 0; t < 3; t++) {
        bad = bad || slots[t] < 0 || slots[t] >= x->slots;
        for (int o = 0; o < t; o++) bad = bad || slots[t] == slots[o];
    }
    if (bad) {
        set_error(g, "fused norm/RoPE scatter: not connected, bad slots or shape (%u rows, %u heads, %d ranks)",
                  rows, heads, x->ranks);
        return 0;
    }
    h3b::QkvRopeInput in{};
    if (!rope_input(g, in, qkv, qn, kn, co, si, rows, heads, 128, rope_half, eps, grouped)) return 0;
    void *window[3][16];
    unsigned long long *flags[16];
    for (int p = 0; p < x->ranks; p++) {
        for (int t = 0; t < 3; t++) window[t][p] = x->mapped[p] + x->slot_bytes * slots[t];
        flags[p] = reinterpret_cast<unsigned long long *>(x->mapped[p] + x->flags_offset);
    }
    int *status = nullptr;
    if (!cuda_ok(g, h3b::device_status_word(&status))) return 0;
    return cuda_ok(g, h3b::qkv_rope_head_shards(in, window[0], window[1], window[2], x->rank, x->ranks, g->stream)) &&
           cuda_ok(g, h3b::exchange_handshake(flags, ++x->epoch, status, x->rank, x->ranks, g->stream));
}
