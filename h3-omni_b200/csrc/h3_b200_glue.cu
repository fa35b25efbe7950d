// Glue translation unit: the reference's CUDA backend with its attention-adjacent stages replaced.
//
// The reference builds its whole backend as ONE translation unit (cuda/h3_gpu_cuda.cu pulls
// cuda/vsa.cuh and cuda/parallel.cuh in textually, cuda/h3_gpu_cuda.cu:1465-1480) and keeps
// struct h3_gpu and struct h3_gpu_tensor private to it (:29-47). Linking libh3b200_attn.so in place
// of the FlashAttention / ThunderKittens adapter objects already swaps the five kernel-adapter
// symbols, but the stages AROUND the kernels - tile pooling, the two cuBLAS score/compression GEMMs,
// the radix-sort selection, the pooled softmax, the merge, and the transpose + NCCL Ulysses
// exchange - would still be the reference's. This file swaps those too without editing or copying a
// single reference file: the reference's own definitions are renamed by the preprocessor while its
// translation unit is included from where it lies (-DH3_REF_BACKEND="<reference>/cuda/h3_gpu_cuda.cu"),
// and the public names are then defined below, inside the same translation unit, with access to
// g->stream, t->data and the h3_gpu_vsa work buffers. The reference's versions stay linked under
// h3_ref_* names (the fall-back of the Ulysses calls, and an A/B oracle on the same GPU).
//
// Build: h3-omni_b200/glue_build.py. The result, libh3_cuda_b200.so, exports the reference's
// complete h3_gpu.h / cuda/h3_cuda.h ABI.
#ifndef H3_REF_BACKEND
#error "compile with -DH3_REF_BACKEND=\"<reference root>/cuda/h3_gpu_cuda.cu\" (see glue_build.py)"
#endif

#define h3_gpu_vsa_bf16 h3_ref_vsa_bf16
#define h3_gpu_ulysses_scatter_heads_bf16 h3_ref_ulysses_scatter_heads_bf16
#define h3_gpu_ulysses_gather_heads_bf16 h3_ref_ulysses_gather_heads_bf16
#include H3_REF_BACKEND
#undef h3_gpu_vsa_bf16
#undef h3_gpu_ulysses_scatter_heads_bf16
#undef h3_gpu_ulysses_gather_heads_bf16

#include <mutex>

// The stage entry points of libh3b200_attn.so this file calls (include/h3b200_attn.h; that header
// cannot be included here because it declares the same ABI types as the reference's h3_gpu.h).
struct h3b_exchange;
extern "C" {
cudaError_t h3b_vsa_pool_raw(const void *const source[3], void *const tiled[3], float *const pooled[3],
                             const int *map, const int *sizes, unsigned tiles, unsigned heads, cudaStream_t stream);
cudaError_t h3b_vsa_select_raw(const float *pooled_q, const float *pooled_k, const float *pooled_v, float *scores,
                               int *indices, int *counts, float *compression, unsigned tiles, unsigned prefix,
                               unsigned keep, unsigned heads, cudaStream_t stream);
cudaError_t h3b_vsa_merge_raw(void *output, const void *tiled_sparse, const void *gate, const float *compression,
                              const int *map, unsigned tiles, unsigned heads, cudaStream_t stream);
void *h3b_exchange_slot_pointer(h3b_exchange *exchange, int slot);
cudaError_t h3b_exchange_scatter_raw(h3b_exchange *exchange, int count, const int *slots, const void *const *sources,
                                     uint32_t rows, uint32_t heads, uint32_t dim, cudaStream_t stream);
cudaError_t h3b_exchange_gather_raw(h3b_exchange *exchange, int slot, const void *source, uint32_t rows,
                                    uint32_t heads, uint32_t dim, cudaStream_t stream);
const char *h3b_exchange_error(const h3b_exchange *exchange);
}

// ---- video sparse attention: cuda/vsa.cuh:263-300 with this library's stages -------------------
// Same arguments, same checks and messages, same work buffers of the reference's h3_gpu_vsa object
// (its `scores` buffer is simply never written: the [heads][tiles][tiles] matrix is not
// materialised). Four launches: pooling of q, k and v; scores + selection + pooled softmax +
// compression; the block-sparse kernel (h3_vsa_hopper of this library); merge.
extern "C" int h3_gpu_vsa_bf16(h3_gpu_vsa *v, h3_gpu_tensor *out, const h3_gpu_tensor *q, const h3_gpu_tensor *k,
                               const h3_gpu_tensor *value, const h3_gpu_tensor *gate) {
    if (!v) return 0;
    h3_gpu *g = v->gpu;
    const size_t elements = (size_t)v->rows * v->heads * 128;
    for (const h3_gpu_tensor *t : {(const h3_gpu_tensor *)out, q, k, value, gate})
        if (!h3_gpu_require_bf16(g, t, elements, "VSA input/output")) return 0;
    const void *source[3] = {q->data, k->data, value->data};
    void *tiled[3] = {v->q->data, v->k->data, v->v->data};
    float *pooled[3] = {(float *)v->poolq->data, (float *)v->poolk->data, (float *)v->poolv->data};
    const int *map = (const int *)v->map->data, *sizes = (const int *)v->sizes->data;
    int *indices = (int *)v->indices->data, *counts = (int *)v->counts->data;
    return cuda_ok(g, h3b_vsa_pool_raw(source, tiled, pooled, map, sizes, v->tiles, v->heads, g->stream)) &&
           cuda_ok(g, h3b_vsa_select_raw(pooled[0], pooled[1], pooled[2], nullptr, indices, counts,
                                         (float *)v->compression->data, v->tiles, v->prefix, v->keep, v->heads,
                                         g->stream)) &&
           cuda_ok(g, h3_vsa_hopper(v->out->data, v->q->data, v->k->data, v->v->data, (float *)v->lse->data, indices,
                                    counts, (int *)sizes, v->tiles, v->heads, g->stream)) &&
           cuda_ok(g, h3b_vsa_merge_raw(out->data, v->out->data, gate->data, (const float *)v->compression->data, map,
                                        v->tiles, v->heads, g->stream));
}

// ---- Ulysses: cuda/parallel.cuh:125-143 through the fused peer-memory exchange --------------------
// A rank attaches an exchange window (h3b_exchange_create_raw + h3b_exchange_connect_local, one
// slot of at least rows*heads*dim elements) to its communicator once; from then on scatter and
// gather on that communicator are one push kernel into the peers' windows plus one device copy
// back into the caller's tensor (the ABI is in place; `scratch` is not needed and not touched).
// A communicator without a window runs the reference's own transpose + NCCL code.
namespace {
struct Attachment {
    h3_gpu_comm *comm;
    h3b_exchange *exchange;
};
std::mutex g_attach_lock;
Attachment g_attached[64];

h3b_exchange *attached(h3_gpu_comm *comm) {
    std::lock_guard<std::mutex> hold(g_attach_lock);
    for (const Attachment &a : g_attached)
        if (a.comm == comm && comm) return a.exchange;
    return nullptr;
}
int fused_exchange(h3_gpu *g, h3b_exchange *x, h3_gpu_tensor *t, uint32_t rows, uint32_t heads, uint32_t dim,
                   bool gather) {
    const size_t count = (size_t)rows * heads * dim;
    if (!h3_gpu_require_bf16(g, t, count, "Ulysses tensor")) return 0;
    const int slot = 0;
    const void *source = t->data;
    const cudaError_t e = gather ? h3b_exchange_gather_raw(x, slot, source, rows, heads, dim, g->stream)
                                 : h3b_exchange_scatter_raw(x, 1, &slot, &source, rows, heads, dim, g->stream);
    if (e != cudaSuccess) {
        h3_gpu_set_error(g, "%s", h3b_exchange_error(x));
        return 0;
    }
    return cuda_ok(g, cudaMemcpyAsync(t->data, h3b_exchange_slot_pointer(x, slot), count * 2, cudaMemcpyDeviceToDevice,
                                      g->stream));
}
}  // namespace

// exchange == NULL detaches. Returns 0 when the table is full.
extern "C" int h3b_glue_attach_exchange(h3_gpu_comm *comm, h3b_exchange *exchange) {
    if (!comm) return 0;
    std::lock_guard<std::mutex> hold(g_attach_lock);
    Attachment *free_entry = nullptr;
    for (Attachment &a : g_attached) {
        if (a.comm == comm) {
            a.exchange = exchange;
            if (!exchange) a.comm = nullptr;
            return 1;
        }
        if (!a.comm && !free_entry) free_entry = &a;
    }
    if (!exchange) return 1;
    if (!free_entry) return 0;
    *free_entry = Attachment{comm, exchange};
    return 1;
}
extern "C" int h3_gpu_ulysses_scatter_heads_bf16(h3_gpu *g, h3_gpu_comm *c, h3_gpu_tensor *t, h3_gpu_tensor *scratch,
                                                 uint32_t rows, uint32_t heads, uint32_t dim) {
    if (h3b_exchange *x = g ? attached(c) : nullptr) return fused_exchange(g, x, t, rows, heads, dim, false);
    return h3_ref_ulysses_scatter_heads_bf16(g, c, t, scratch, rows, heads, dim);
}
extern "C" int h3_gpu_ulysses_gather_heads_bf16(h3_gpu *g, h3_gpu_comm *c, h3_gpu_tensor *t, h3_gpu_tensor *scratch,
                                                uint32_t rows, uint32_t heads, uint32_t dim) {
    if (h3b_exchange *x = g ? attached(c) : nullptr) return fused_exchange(g, x, t, rows, heads, dim, true);
    return h3_ref_ulysses_gather_heads_bf16(g, c, t, scratch, rows, heads, dim);
}
