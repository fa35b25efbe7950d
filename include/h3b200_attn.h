/*
 * libh3b200_attn - B200 (sm_100a) attention engine for the H3-omni diffusion transformer.
 *
 * C ABI, three layers:
 *   1. The five kernel-adapter symbols the reference's CUDA backend links against
 *      (reference cuda/h3_flash.h:4-20 and cuda/vsa_hopper.h:4-6). Exporting these is what
 *      makes the library a drop-in for the reference's FlashAttention-2/3 and Hopper VSA
 *      adapter objects.
 *   2. A mirror of the reference's GPU primitive ABI for the attention path only
 *      (reference h3_gpu.h and cuda/h3_cuda.h): same names, argument meaning and error
 *      behaviour (return 1 = ok, 0 = failure with a message from h3_gpu_error()).
 *   3. Additions of this library (prefix h3b_), none of which the reference has.
 *
 * All device work is enqueued asynchronously on the context's stream; nothing here
 * synchronises the host except h3_gpu_submit, tensor reads and h3b_device_status.
 * A context and its tensors belong to one host thread and one device.
 */
#ifndef H3B200_ATTN_H
#define H3B200_ATTN_H

#include <cuda_runtime.h>
#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------------------
 * 1. Kernel-adapter symbols. Tensors are token-major [batch][sequence][heads][dim],
 *    16-bit elements; logsumexp (may be NULL here; the reference never reads it) is
 *    [batch][heads][sequence] f32 = max*scale + log(sum). Return a cudaError_t, never exit.
 * ------------------------------------------------------------------------------------ */

/* Replaces reference cuda/flash_attention.cu:29-67 (FlashAttention-2 adapter): bf16,
 * head dim 128, optional causal mask, grouped-query when kv_heads < heads. */
cudaError_t h3_flash_bf16(void *output, const void *query, const void *key, const void *value,
                          float *logsumexp, unsigned batch, unsigned sequence, unsigned heads,
                          unsigned kv_heads, float scale, bool causal, cudaStream_t stream);
/* Replaces reference cuda/flash3_attention.cu:74-79 (FlashAttention-3 adapter): bf16,
 * head dim 128, non-causal. This is the DiT joint video+audio self-attention. */
cudaError_t h3_flash3_bf16(void *output, const void *query, const void *key, const void *value,
                           float *logsumexp, unsigned batch, unsigned sequence, unsigned heads,
                           unsigned kv_heads, float scale, cudaStream_t stream);
/* Replaces reference cuda/flash3_attention.cu:81-87: fp16, head dim 64 (video VAE). */
cudaError_t h3_flash3_f16_d64(void *output, const void *query, const void *key, const void *value,
                              float *logsumexp, unsigned batch, unsigned sequence, unsigned heads,
                              float scale, cudaStream_t stream);
/* Replaces reference cuda/flash3_attention.cu:89-94: rectangular bf16 attention,
 * query_rows x key_rows, batch 1 (live mode: short query chunk against KV history). */
cudaError_t h3_flash3_cross_bf16(void *output, const void *query, const void *key,
                                 const void *value, float *logsumexp, unsigned query_rows,
                                 unsigned key_rows, unsigned heads, float scale,
                                 cudaStream_t stream);
/* Replaces reference cuda/vsa_hopper.cu:6-28: block-sparse attention over 64-row tiles.
 * out, q, k, v: [heads][tiles*64][128] bf16; lse [heads][tiles*64] f32 (may be NULL);
 * indices [heads][tiles][tiles] (first counts[h][q] entries valid, ascending),
 * counts [heads][tiles], sizes [tiles] = valid keys per tile. */
cudaError_t h3_vsa_hopper(void *out, const void *q, const void *k, const void *v, float *lse,
                          int *indices, int *counts, int *sizes, unsigned tiles, unsigned heads,
                          cudaStream_t stream);

/* ------------------------------------------------------------------------------------
 * 2. GPU primitive ABI, attention path only (reference h3_gpu.h / cuda/h3_cuda.h).
 * ------------------------------------------------------------------------------------ */
typedef struct h3_gpu h3_gpu;
typedef struct h3_gpu_tensor h3_gpu_tensor;
typedef struct h3_gpu_comm h3_gpu_comm;
typedef struct h3_gpu_vsa h3_gpu_vsa;

typedef enum { /* reference h3_gpu.h:10-16 */
    H3_GPU_F32 = 0,
    H3_GPU_BF16,
    H3_GPU_I8,
    H3_GPU_U32,
    H3_GPU_F16
} h3_gpu_dtype;

/* Context and tensors: reference h3_gpu.h:36-96, cuda/h3_gpu_cuda.cu:163-402. */
h3_gpu *h3_gpu_create(const char *shader_source_path, char *error, size_t error_size);
void h3_gpu_free(h3_gpu *gpu);
h3_gpu_tensor *h3_gpu_tensor_new_f32(h3_gpu *gpu, size_t elements);
h3_gpu_tensor *h3_gpu_tensor_new_bf16(h3_gpu *gpu, size_t elements);
h3_gpu_tensor *h3_gpu_tensor_from_f32(h3_gpu *gpu, const float *values, size_t elements);
h3_gpu_tensor *h3_gpu_tensor_from_bf16(h3_gpu *gpu, const uint16_t *values, size_t elements);
h3_gpu_tensor *h3_gpu_tensor_from_u32(h3_gpu *gpu, const uint32_t *values, size_t elements);
void h3_gpu_tensor_free(h3_gpu_tensor *tensor);
size_t h3_gpu_tensor_elements(const h3_gpu_tensor *tensor);
h3_gpu_dtype h3_gpu_tensor_dtype(const h3_gpu_tensor *tensor);
int h3_gpu_tensor_read_f32(const h3_gpu_tensor *tensor, float *values, size_t elements);
int h3_gpu_tensor_read_bf16(const h3_gpu_tensor *tensor, uint16_t *values, size_t elements);
int h3_gpu_tensor_write_f32(h3_gpu_tensor *tensor, const float *values, size_t elements);
int h3_gpu_tensor_write_bf16(h3_gpu_tensor *tensor, const uint16_t *values, size_t elements);
int h3_gpu_tensor_write_bf16_range(h3_gpu_tensor *tensor, size_t destination_offset,
                                   const uint16_t *values, size_t elements);
int h3_gpu_begin(h3_gpu *gpu);
int h3_gpu_continue(h3_gpu *gpu);
int h3_gpu_submit(h3_gpu *gpu);
const char *h3_gpu_error(const h3_gpu *gpu);
int h3_gpu_zero(h3_gpu *gpu, h3_gpu_tensor *tensor); /* cuda/parallel.cuh:155-157 */
int h3_gpu_copy_bf16(h3_gpu *gpu, h3_gpu_tensor *destination, size_t destination_offset,
                     const h3_gpu_tensor *source, size_t source_offset,
                     size_t elements); /* h3_gpu.h:132-135 */
int h3_gpu_download(h3_gpu *gpu, const h3_gpu_tensor *tensor, size_t offset, void *host,
                    size_t count); /* cuda/h3_cuda.h:55-56; offset and count in bytes */

/* Dense attention: reference h3_gpu.h:494-497 -> cuda/h3_gpu_cuda.cu:1109-1130,1216-1220.
 * Q, K, V, O are [sequence][heads][128] bf16; head_dim must be 128. */
int h3_gpu_sdpa_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *query,
                     const h3_gpu_tensor *key, const h3_gpu_tensor *value, uint32_t sequence,
                     uint32_t heads, uint32_t head_dim, float scale);
/* cuda/h3_cuda.h:78-81 -> cuda/h3_gpu_cuda.cu:1242-1246 (always the h3_flash_bf16 path). */
int h3_gpu_sdpa_fa2_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *query,
                         const h3_gpu_tensor *key, const h3_gpu_tensor *value, uint32_t tokens,
                         uint32_t heads, uint32_t head_dim, float scale);
/* h3_gpu.h:534-540: causal grouped-query attention (text encoder). */
int h3_gpu_gqa_causal_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *query,
                           const h3_gpu_tensor *key, const h3_gpu_tensor *value,
                           uint32_t sequence, uint32_t query_heads, uint32_t kv_heads,
                           uint32_t head_dim, float scale);
/* cuda/h3_cuda.h:202-205 -> cuda/vae_fp16.cuh:275-296: fp16, head dim 64. */
int h3_gpu_sdpa_f16_d64(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *query,
                        const h3_gpu_tensor *key, const h3_gpu_tensor *value, uint32_t tokens,
                        uint32_t heads, uint32_t head_dim, float scale);
/* cuda/h3_cuda.h:16-19 -> cuda/h3_gpu_cuda.cu:1221-1241: live-mode rectangular attention
 * over row slices; scale is fixed at 1/sqrt(128). */
int h3_gpu_cross_attention_bf16(h3_gpu *gpu, h3_gpu_tensor *out, size_t out_row,
                                const h3_gpu_tensor *q, size_t q_row, const h3_gpu_tensor *k,
                                const h3_gpu_tensor *v, size_t kv_row, uint32_t query_rows,
                                uint32_t key_rows, uint32_t heads);

/* Q/K RMS-norm + rotary embedding on the fused QKV projection output, the producer of the
 * attention inputs: h3_gpu.h:434-455 -> cuda/h3_gpu_cuda.cu:989-1031 (kernels
 * cuda/primitives.cuh:897-962, cuda/fast_primitives.cuh:184-265). qkv is [sequence][3][heads][128]
 * (grouped: [sequence][heads][3][128], the checkpoint's layout); q_norm, k_norm [128];
 * rope_cos, rope_sin [sequence][rope_half]; query, key, value [sequence][heads][128]; all bf16.
 * Results are bit-identical to the reference's kernels. head_dim must be 128 (the DiT's; the
 * reference's generic kernel also takes other sizes), rope_half a multiple of 4, <= 64. */
int h3_gpu_qkv_rope_bf16(h3_gpu *gpu, h3_gpu_tensor *query, h3_gpu_tensor *key, h3_gpu_tensor *value,
                         const h3_gpu_tensor *qkv, const h3_gpu_tensor *q_norm,
                         const h3_gpu_tensor *k_norm, const h3_gpu_tensor *rope_cos,
                         const h3_gpu_tensor *rope_sin, uint32_t sequence, uint32_t heads,
                         uint32_t head_dim, uint32_t rope_half, float epsilon);
int h3_gpu_grouped_qkv_rope_bf16(h3_gpu *gpu, h3_gpu_tensor *query, h3_gpu_tensor *key,
                                 h3_gpu_tensor *value, const h3_gpu_tensor *qkv,
                                 const h3_gpu_tensor *q_norm, const h3_gpu_tensor *k_norm,
                                 const h3_gpu_tensor *rope_cos, const h3_gpu_tensor *rope_sin,
                                 uint32_t sequence, uint32_t heads, uint32_t head_dim,
                                 uint32_t rope_half, float epsilon);

/* Video sparse attention: cuda/h3_cuda.h:70-76 -> cuda/vsa.cuh:192-300. */
h3_gpu_vsa *h3_gpu_vsa_new(h3_gpu *gpu, uint32_t text_rows, uint32_t audio_rows, uint32_t time,
                           uint32_t height, uint32_t width, uint32_t heads);
void h3_gpu_vsa_free(h3_gpu_vsa *vsa);
int h3_gpu_vsa_bf16(h3_gpu_vsa *vsa, h3_gpu_tensor *output, const h3_gpu_tensor *query,
                    const h3_gpu_tensor *key, const h3_gpu_tensor *value,
                    const h3_gpu_tensor *gate);

/* Multi-GPU, Ulysses sequence parallelism: cuda/h3_cuda.h:20-39 -> cuda/parallel.cuh:25-153. */
int h3_gpu_device_count(void);
int h3_gpu_select_device(int device, char *error, size_t error_size);
int h3_gpu_comm_init_all(int count, h3_gpu_comm **comms, char *error, size_t error_size);
void h3_gpu_comm_free(h3_gpu_comm *comm);
void h3_gpu_comm_abort(h3_gpu_comm *comm);
int h3_gpu_ulysses_scatter_heads_bf16(h3_gpu *gpu, h3_gpu_comm *comm, h3_gpu_tensor *tensor,
                                      h3_gpu_tensor *scratch, uint32_t rows, uint32_t heads,
                                      uint32_t dim);
int h3_gpu_ulysses_gather_heads_bf16(h3_gpu *gpu, h3_gpu_comm *comm, h3_gpu_tensor *tensor,
                                     h3_gpu_tensor *scratch, uint32_t rows, uint32_t heads,
                                     uint32_t dim);
int h3_gpu_all_gather_bf16(h3_gpu *gpu, h3_gpu_comm *comm, h3_gpu_tensor *output,
                           const h3_gpu_tensor *input, size_t count);

/* ------------------------------------------------------------------------------------
 * 3. Additions (no counterpart in the reference).
 * ------------------------------------------------------------------------------------ */

/* Device status word of the current device: 0 = ok, 1 = a bounded device-side wait gave
 * up, 2 = a device-side bounds check refused an access. Synchronises the device.
 * reset != 0 clears the word after reading. h3_gpu_submit reports a non-zero word as a failure
 * ("device-side wait timed out (status 1)" / "device-side bounds check failed (status 2)") once
 * and clears it; the word belongs to the device, so a failure raised through one context is
 * reported by whichever context of that device submits next. */
cudaError_t h3b_device_status(int *status, int reset);

/* Wrap device memory the caller owns (e.g. a framework tensor) as a non-owning
 * h3_gpu_tensor; h3_gpu_tensor_free releases only the handle. */
h3_gpu_tensor *h3b_tensor_wrap(h3_gpu *gpu, void *device_pointer, size_t elements,
                               h3_gpu_dtype dtype);
h3_gpu_tensor *h3b_tensor_new_f16(h3_gpu *gpu, size_t elements);
void *h3b_tensor_data(const h3_gpu_tensor *tensor);
/* Run the context on a caller-owned stream (NULL restores the context's own stream). */
int h3b_gpu_set_stream(h3_gpu *gpu, cudaStream_t stream);
cudaStream_t h3b_gpu_stream(const h3_gpu *gpu);

/* Live-mode attention over K/V given as up to six separate row ranges (text, sink, recent
 * chunks, current chunk ...) attended as if concatenated - without the concatenation copies the
 * reference makes per layer (h3_dit_live.inc:81-94). keys[s] / values[s] are
 * [>= kv_row[s] + kv_rows[s]][heads][128] bf16; rows kv_row[s] .. +kv_rows[s] of range s are used,
 * in range order. Scale is 1/sqrt(128) as in h3_gpu_cross_attention_bf16. */
int h3b_cross_attention_segments_bf16(h3_gpu *gpu, h3_gpu_tensor *out, size_t out_row,
                                      const h3_gpu_tensor *q, size_t q_row, uint32_t query_rows,
                                      uint32_t heads, uint32_t segments,
                                      const h3_gpu_tensor *const *keys,
                                      const h3_gpu_tensor *const *values, const size_t *kv_row,
                                      const uint32_t *kv_rows);

/* Live mode's KV history of one layer as a ring buffer (no counterpart as an object in the
 * reference, which keeps h3_live_kv tensor pairs that it allocates, copies and frees at every
 * chunk: h3_dit.c:77-80, live_pair_copy, and the commit at h3_dit.c:4451-4481). One allocation at
 * h3b_live_kv_new holds every slot; afterwards nothing is allocated or freed.
 *   stage       - the clean chunk's media K/V rows (first audio_rows of them audio) are copied in:
 *                 live_pair_copy;
 *   commit      - the staged chunk becomes the newest history chunk and the older of the two recent
 *                 chunks is dropped, by index rotation; the first commit also keeps the chunk's
 *                 video rows as the sink (h3_dit.c:4457-4481);
 *   clear_audio - the recent chunks are attended without their audio rows from now on (:4483-4486);
 *   attention   - query rows against  text | sink (from the third commit) | older | newer |
 *                 current media  as K/V row ranges, i.e. the second call of h3_dit_live.inc:95-99
 *                 without the concatenation copies of :81-94. key / value are the block's own
 *                 [sequence][heads][128] rows, text rows first. Scale 1/sqrt(128).
 * chunk_rows: the largest number of media rows a chunk can have. */
typedef struct h3b_live_kv h3b_live_kv;
h3b_live_kv *h3b_live_kv_new(h3_gpu *gpu, uint32_t chunk_rows, uint32_t heads);
void h3b_live_kv_free(h3b_live_kv *history);
void h3b_live_kv_reset(h3b_live_kv *history);
uint32_t h3b_live_kv_commits(const h3b_live_kv *history);
uint32_t h3b_live_kv_history_rows(const h3b_live_kv *history);
int h3b_live_kv_stage(h3b_live_kv *history, const h3_gpu_tensor *key, const h3_gpu_tensor *value,
                      size_t first_row, uint32_t rows, uint32_t audio_rows);
int h3b_live_kv_commit(h3b_live_kv *history);
int h3b_live_kv_clear_audio(h3b_live_kv *history);
int h3b_live_kv_attention_bf16(h3b_live_kv *history, h3_gpu_tensor *out, size_t out_row,
                               const h3_gpu_tensor *q, size_t q_row, uint32_t query_rows,
                               const h3_gpu_tensor *key, const h3_gpu_tensor *value, uint32_t text_rows,
                               uint32_t sequence);

/* What follows attention in every block, as one call (no counterpart as one call in the
 * reference, which runs h3_gpu_linear_bf16 (INNER -> HIDDEN) and h3_gpu_gate_adaln_bf16,
 * h3_dit.c:2573-2597, cuda/fast_primitives.cuh:50-124):
 *   y      = bf16(attention_heads . out_weight^T)      out_weight [hidden][inner], fp32 accumulate
 *   gated  = bf16(residual + bf16(y * gate_modulation[row_map[row]][gate_slot]))
 *   output = AdaLN(gated; norm_weight, modulation[row_map[row]][shift_slot / scale_slot], epsilon)
 * The projection is a tcgen05 GEMM whose epilogue applies gate and residual, so y is never written;
 * AdaLN follows the reference kernel's operation order (bit-identical to it on the same gated
 * rows). attention_heads may be an exchange slot (the rows the attention kernel gathered).
 * gated_residual may alias residual; output == NULL computes the gate only. inner % 64 == 0,
 * hidden % 8 == 0, hidden <= 8192. */
int h3b_attention_output_gate_adaln_bf16(
    h3_gpu *gpu, h3_gpu_tensor *gated_residual, h3_gpu_tensor *output, const h3_gpu_tensor *residual,
    const h3_gpu_tensor *attention_heads, const h3_gpu_tensor *out_weight, const h3_gpu_tensor *norm_weight,
    const h3_gpu_tensor *gate_modulation, const h3_gpu_tensor *modulation, const h3_gpu_tensor *row_map,
    uint32_t rows, uint32_t inner, uint32_t hidden, uint32_t slots, uint32_t gate_slot, uint32_t shift_slot,
    uint32_t scale_slot, float epsilon);

/* Dense attention from and to HOST memory, head dim 128: q, k, v, out are token-major
 * [sequence][heads][128] bf16 in host memory (pinned for full speed). The heads are cut into
 * chunks, and copy-in, kernel and copy-out of consecutive chunks overlap on three streams, so the
 * call costs about max(copy time, kernel time). head_groups > 0: that many equal groups
 * (heads % head_groups == 0, at most 64), the first and the last run as two halves to shorten the
 * two transfers nothing can overlap. head_groups == 0: the library chooses - two one-head chunks
 * at either end, inner chunks of at least two heads and about 24 MB per tensor (24 heads of 52,352
 * rows: 1 1 2 2 2 2 2 2 2 2 2 2 1 1). The kernels of consecutive chunks run on two streams and
 * overlap, so short chunks leave no SM idle. Synchronous: returns when `out` is complete.
 * h3b_sdpa_host_plan returns the number of chunks such a call uses and writes their head counts
 * (0: the heads do not split that way, or more than `capacity` chunks). */
uint32_t h3b_sdpa_host_plan(uint32_t sequence, uint32_t heads, uint32_t head_groups, uint32_t *head_count,
                            uint32_t capacity);
int h3b_sdpa_bf16_host(h3_gpu *gpu, uint16_t *out, const uint16_t *q, const uint16_t *k,
                       const uint16_t *v, uint32_t sequence, uint32_t heads, uint32_t head_dim,
                       float scale, uint32_t head_groups);

/* One-process-per-GPU communicator: rank 0 calls h3b_comm_unique_id, ships the 128 bytes
 * to the other ranks by any means, then every rank calls h3b_comm_init_rank. */
int h3b_comm_unique_id(void *id128, char *error, size_t error_size);
int h3b_comm_init_rank(const void *id128, int rank, int count, h3_gpu_comm **comm, char *error,
                       size_t error_size);
int h3b_comm_rank(const h3_gpu_comm *comm);
int h3b_comm_size(const h3_gpu_comm *comm);

/* Fused Ulysses exchange over peer memory, one process per GPU. Every rank creates a window of
 * `slots` bf16 tensors of slot_elements each and gets a 64-byte handle; the ranks all-gather the
 * handles by any transport and connect. A scatter or gather is then ONE kernel that reads the
 * local tensor once and stores each 16-byte unit into its final place in the owning rank's window
 * over NVLink, followed by a bounded epoch handshake (a timeout is reported through the device
 * status word, not a hang). The destination of both calls is slot `slot` of every rank's window:
 *   scatter: src [rows][heads][dim] per rank -> [ranks*rows][heads/ranks][dim] per rank
 *   gather : src [ranks*rows][heads/ranks][dim] per rank -> [rows][heads][dim] per rank
 * Calls must be made in the same order on every rank, each on its context's stream. Reusing a slot
 * is safe by construction: an exchange starts storing only after every rank has STARTED the same
 * exchange, and a rank starts it only after everything queued before it on its stream - the
 * readers of what earlier exchanges left in its window - has finished. So the one rule is: queue
 * the readers of a slot on the exchange's stream before the next exchange call of any kind.
 * After a timeout (status 1) nothing more is stored and the failure shows on every rank. */
typedef struct h3b_exchange h3b_exchange;
int h3b_exchange_create(h3_gpu *gpu, int rank, int ranks, size_t slot_elements, int slots,
                        h3b_exchange **exchange, void *handle64);
int h3b_exchange_connect(h3b_exchange *exchange, const void *handles);
/* The ranks as threads of ONE process (how the reference runs them, h3_dit.c:4066-4177): a CUDA IPC
 * handle cannot be opened by the process that made it, so the windows are joined by their device
 * pointers and peer access is switched on between the devices. all_ranks: every rank's exchange in
 * rank order. Each rank calls this for its own exchange with its own device current, after all
 * ranks have created theirs. */
int h3b_exchange_connect_local(h3b_exchange *exchange, h3b_exchange *const *all_ranks);
/* Bound of every device-side wait of this exchange's kernels, default 2000 ms. */
int h3b_exchange_set_wait_limit_ms(h3b_exchange *exchange, unsigned milliseconds);
const char *h3b_exchange_error(const h3b_exchange *exchange);
void h3b_exchange_free(h3b_exchange *exchange);
h3_gpu_tensor *h3b_exchange_slot(h3b_exchange *exchange, int slot);
int h3b_exchange_scatter_heads_bf16(h3b_exchange *exchange, int slot, const h3_gpu_tensor *src,
                                    uint32_t rows, uint32_t heads, uint32_t dim);
int h3b_exchange_gather_heads_bf16(h3b_exchange *exchange, int slot, const h3_gpu_tensor *src,
                                   uint32_t rows, uint32_t heads, uint32_t dim);
/* Up to four tensors of one shape (q, k, v, and the gate of video sparse attention) scattered by
 * ONE kernel with one pair of handshakes: sources[t] goes to slot slots[t]. Replaces the three or
 * four exchanges per block of h3_dit.c:2529-2538. */
int h3b_exchange_scatter_heads_multi_bf16(h3b_exchange *exchange, int count, const int *slots,
                                          const h3_gpu_tensor *const *sources, uint32_t rows,
                                          uint32_t heads, uint32_t dim);
/* The same exchange for a backend that keeps its own tensor and context objects: no h3_gpu, raw
 * device pointers, the stream given per call, cudaError_t results (text: h3b_exchange_error).
 * handle64 may be NULL when the ranks will be joined with h3b_exchange_connect_local. */
cudaError_t h3b_exchange_create_raw(int rank, int ranks, size_t slot_elements, int slots,
                                    h3b_exchange **exchange, void *handle64);
void *h3b_exchange_slot_pointer(h3b_exchange *exchange, int slot);
cudaError_t h3b_exchange_scatter_raw(h3b_exchange *exchange, int count, const int *slots,
                                     const void *const *sources, uint32_t rows, uint32_t heads,
                                     uint32_t dim, cudaStream_t stream);
cudaError_t h3b_exchange_gather_raw(h3b_exchange *exchange, int slot, const void *source, uint32_t rows,
                                    uint32_t heads, uint32_t dim, cudaStream_t stream);

/* Attention over this rank's heads/ranks heads with the sequence-gather fused into the kernel's
 * epilogue: q, k, v are [>= sequence][heads/ranks][128] (typically the scatter slots); each output
 * row is stored by the attention kernel itself into the row shard of the rank that owns the row -
 * slot `slot` of that rank's window, [rows][heads][128] - followed by the epoch handshake.
 * Rows >= sequence of the last shard are left untouched. */
int h3b_exchange_sdpa_gather_bf16(h3b_exchange *exchange, int slot, const h3_gpu_tensor *q,
                                  const h3_gpu_tensor *k, const h3_gpu_tensor *v, uint32_t sequence,
                                  uint32_t rows, uint32_t heads, float scale);

/* The producer fused with the head scatter (no counterpart in the reference, which runs
 * h3_gpu_grouped_qkv_rope_bf16 and then three h3_gpu_ulysses_scatter_heads_bf16 exchanges,
 * h3_dit.c:2459-2462,2529-2538): this rank's `rows` rows of the QKV projection are normalised,
 * rotated and stored directly into slots slot_q, slot_k, slot_v of the ranks that own each head,
 * laid out [ranks*rows][heads/ranks][128] as the scatter leaves them; one kernel and one epoch
 * handshake. rope_cos / rope_sin are this rank's [rows][rope_half] tables. */
int h3b_exchange_qkv_rope_scatter_bf16(h3b_exchange *exchange, int slot_q, int slot_k, int slot_v,
                                       const h3_gpu_tensor *qkv, const h3_gpu_tensor *q_norm,
                                       const h3_gpu_tensor *k_norm, const h3_gpu_tensor *rope_cos,
                                       const h3_gpu_tensor *rope_sin, uint32_t rows, uint32_t heads,
                                       uint32_t rope_half, float epsilon, int grouped);

/* VSA introspection for tests and tools: geometry, an override for the number of kept
 * video tiles (the reference fixes ceil(10 %)), and device pointers of the work buffers
 * of the last h3_gpu_vsa_bf16 call. which: 0 map, 1 sizes, 2-4 tiled q/k/v, 5 sparse out,
 * 6-8 pooled q/k/v, 9 indices, 10 counts, 11 compression, 12 scores (only when tracing). */
int h3b_vsa_info(const h3_gpu_vsa *vsa, int *rows, int *tiles, int *prefix, int *keep);
int h3b_vsa_set_keep(h3_gpu_vsa *vsa, int keep);
int h3b_vsa_trace_scores(h3_gpu_vsa *vsa, int enable);
void *h3b_vsa_buffer(const h3_gpu_vsa *vsa, int which);
/* Optional stage timing (CUDA events on the context's stream, off by default): after a call,
 * h3b_vsa_stage_ms waits for it and returns the milliseconds of its four stages: pooling (or
 * norm + RoPE + pooling), scores + selection + compression, block-sparse attention, merge. */
int h3b_vsa_time_stages(h3_gpu_vsa *vsa, int enable);
int h3b_vsa_stage_ms(h3_gpu_vsa *vsa, float *ms4);

/* The stages of h3_gpu_vsa_bf16 on raw device pointers, for a backend that keeps its own tensor
 * objects and adopts the stages one by one (they replace, in this order, the three tile_pool
 * launches of cuda/vsa.cuh:274-278; the score SGEMM, select_blocks, pooled_softmax and the
 * compression SGEMM of :281-294; untile_merge of :295-299; the block-sparse kernel between them is
 * h3_vsa_hopper). source / tiled / pooled hold q, k, v in this order; layouts as in the reference:
 * source and gate and output token-major [rows][heads][128] bf16, tiled [heads][tiles*64][128]
 * bf16, pooled and compression [heads][tiles][128] f32, indices [heads][tiles][tiles], counts
 * [heads][tiles], map [tiles*64], sizes [tiles] int32. scores ([heads][tiles][tiles] f32) may be
 * NULL: the score matrix is then never written. compression may be NULL (selection only). */
cudaError_t h3b_vsa_pool_raw(const void *const source[3], void *const tiled[3], float *const pooled[3],
                             const int *map, const int *sizes, unsigned tiles, unsigned heads,
                             cudaStream_t stream);
cudaError_t h3b_vsa_select_raw(const float *pooled_q, const float *pooled_k, const float *pooled_v,
                               float *scores, int *indices, int *counts, float *compression,
                               unsigned tiles, unsigned prefix, unsigned keep, unsigned heads,
                               cudaStream_t stream);
cudaError_t h3b_vsa_merge_raw(void *output, const void *tiled_sparse, const void *gate,
                              const float *compression, const int *map, unsigned tiles, unsigned heads,
                              cudaStream_t stream);
/* Q/K norm + RoPE on raw pointers (the arithmetic of h3_gpu_qkv_rope_bf16 / _grouped_). */
cudaError_t h3b_qkv_rope_raw(void *query, void *key, void *value, const void *qkv, const void *q_norm,
                             const void *k_norm, const void *rope_cos, const void *rope_sin,
                             unsigned sequence, unsigned heads, unsigned rope_half, float epsilon,
                             int grouped, cudaStream_t stream);

/* Video sparse attention fed by the QKV projection output instead of separate q, k, v
 * (no counterpart in the reference, which runs h3_gpu_grouped_qkv_rope_bf16 and then
 * h3_gpu_vsa_bf16): norm + rotation write q, k, v directly in tile order together with the
 * tile means, so the token-major q, k, v are never materialised. Output and every work buffer
 * equal those of h3_gpu_qkv_rope_bf16 followed by h3_gpu_vsa_bf16, bit for bit. */
int h3b_vsa_qkv_rope_bf16(h3_gpu_vsa *vsa, h3_gpu_tensor *output, const h3_gpu_tensor *qkv,
                          const h3_gpu_tensor *q_norm, const h3_gpu_tensor *k_norm,
                          const h3_gpu_tensor *rope_cos, const h3_gpu_tensor *rope_sin,
                          const h3_gpu_tensor *gate, uint32_t rope_half, float epsilon, int grouped);

/* Which kernel runs the block-sparse fine stage behind h3_vsa_hopper (process-wide; for A/B
 * measurement and tests). There are two: the persistent kernel, in which every query tile walks
 * its own list only, and the pair-walk kernel, in which a CTA takes two adjacent query tiles and
 * walks the union of their lists (per-row online softmax; cheaper per multiply-add, wasteful when
 * the two lists differ). 0 (default): a pre-pass gives every pair of tiles to the pair walk when
 * their lists mostly coincide (|A u B| < 0.7 (|A| + |B|)) and to the persistent kernel otherwise;
 * the rare tiles whose softmax sums leave the exponent range the persistent kernel covers are
 * recomputed by the pair walk. 1: pair-walk kernel only. 2: persistent kernel, then every tile
 * recomputed by the pair walk. 3: persistent kernel for every pair. */
void h3b_vsa_fine_mode(int mode);

/* Top-k tile selection of video sparse attention with no device allocation at all. It has no
 * counterpart in the reference: it is for callers that cannot allocate where they call from -
 * a host that gave this code a fixed memory arena at start-up, a memory-capped deployment
 * where a late cudaMalloc may fail, or a latency-critical loop that must not take the
 * allocator's lock. It computes the pooled means of query and key per tile and from them
 * indices [heads][tiles][tiles] and counts [heads][tiles], exactly as h3_gpu_vsa_bf16 does
 * internally, but keeps the pooled means in one 8 MiB device array that is part of the
 * library image (every GPU that loads the library holds it until the process exits).
 *   - Limit: heads * tiles <= 8192; larger shapes return cudaErrorInvalidValue and
 *     h3b_vsa_topk_static_error() says why. Nothing is launched in that case.
 *   - query, key: [rows][heads][128] bf16; map [tiles*64] and sizes [tiles] as built by
 *     h3_gpu_vsa_new (device pointers). counts is written in full; of each indices row the
 *     first counts[row] entries are written, the entries behind them keep the caller's bytes.
 *   - The first call on each device resolves the array's device address (a runtime query,
 *     no allocation); make that first call before starting any stream capture.
 *   - All calls share the one array and it keeps the previous call's contents. Every call
 *     rewrites the part it reads, so nothing needs clearing, but two calls whose kernels can
 *     overlap on the GPU (different streams, or different host threads) race on it: keep
 *     calls on one device ordered.
 * It calls no cudaMalloc, cudaFree or any allocating library routine. */
cudaError_t h3b_vsa_topk_static(const void *query, const void *key, const int *map,
                                const int *sizes, int *indices, int *counts, unsigned tiles,
                                unsigned prefix, unsigned keep, unsigned heads,
                                cudaStream_t stream);
const char *h3b_vsa_topk_static_error(void);

#ifdef __cplusplus
}
#endif
#endif /* H3B200_ATTN_H */
