// Internal launch interface between the C-ABI entry points and the kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

struct CUtensorMap_st;

namespace h3b {

// Address of this device's status word (0 = ok; see DeviceStatus in sm100_ptx.cuh).
cudaError_t device_status_word(int **word);

// Output redirection for the sequence-gather fused into the attention epilogue: query row r of
// local head h is stored to rank r / rows_per_rank, at [r % rows_per_rank][rank*local_heads + h]
// of that rank's [rows_per_rank][total_heads][128] tensor (plain peer stores over NVLink).
struct PeerOutput {
    void *base[16];
    unsigned rows_per_rank, rank, total_heads;
};

// tcgen05 kernels (attn_tc5.cu). Token-major [B][L][H][128] bf16. With `peer` (batch 1 only)
// `out` is ignored and the output goes to the owners' tensors.
cudaError_t attn_dense_tc5(void *out, const void *q, const void *k, const void *v, float *lse,
                           unsigned batch, unsigned lq, unsigned lk, unsigned heads,
                           unsigned kv_heads, float scale, cudaStream_t stream,
                           const PeerOutput *peer = nullptr);
// Two query tiles per CTA (attn_tc5_pair.cu); tensor maps as built by attn_dense_tc5.
cudaError_t attn_dense_tc5_pair(const ::CUtensorMap_st *mq, const ::CUtensorMap_st *mk,
                                const ::CUtensorMap_st *mv, void *out, float *lse, unsigned batch,
                                unsigned lq, unsigned lk, unsigned heads, unsigned kv_heads,
                                float scale, int *status, cudaStream_t stream,
                                const PeerOutput *peer = nullptr, unsigned segments = 0,
                                const unsigned *segment_rows = nullptr, unsigned split_tiles = 0);
// Split-KV (batch 1): with split_tiles > 0 the launch above cuts the keys into slices of
// split_tiles 128-row tiles on grid.z and writes per-slice outputs [slices][lq][heads][128] bf16 and
// logsumexp [slices][heads][lq] f32 (both required); this combines them.
cudaError_t attn_merge_splits(void *out, float *lse_out, const void *partial, const float *lse, unsigned splits,
                              unsigned lq, unsigned heads, cudaStream_t stream);
// Rectangular attention of lq query rows against the concatenation of `segments` (<= 6) K/V row
// ranges, each token-major [rows_s][heads][128], without concatenating them (batch 1).
cudaError_t attn_segments_tc5(void *out, const void *q, const void *const *k, const void *const *v,
                              const unsigned *segment_rows, unsigned segments, unsigned lq,
                              unsigned heads, float scale, cudaStream_t stream);
// Head-major tiled [H][tiles*64][128] bf16 with per-(head, query tile) KV tile lists.
cudaError_t attn_sparse_tc5(void *out, const void *q, const void *k, const void *v, float *lse,
                            const int *indices, const int *counts, const int *sizes,
                            unsigned tiles, unsigned heads, cudaStream_t stream);

// The persistent block-sparse kernel with the keys on the MMA's M axis (attn_sparse_t.cu), behind a
// pre-pass that assigns every pair of adjacent query tiles to it or to the pair-walk kernel.
// mq has a 64-row box; `ticket` (one zeroed word), `redo` and `elsewhere` ([heads][tiles] bytes
// each) are work memory the caller provides on `stream`. After the launch redo marks the tiles the
// pair-walk kernel has to compute: those assigned to it, and those whose row sums left the safe
// exponent range here. assign: -1 by list overlap, 0 all here, 1 all to the pair walk.
cudaError_t attn_sparse_t_launch(const ::CUtensorMap_st *mq, const ::CUtensorMap_st *mk,
                                 const ::CUtensorMap_st *mv, void *out, float *lse, const int *indices,
                                 const int *counts, const int *sizes, unsigned tiles, unsigned heads,
                                 unsigned *ticket, unsigned char *redo, unsigned char *elsewhere, int assign,
                                 bool force_redo, int *status, cudaStream_t stream);
// 0 (default): pairs of query tiles whose lists mostly coincide go to the pair-walk kernel, the
// others to the persistent kernel, whose out-of-range tiles are recomputed by the pair walk;
// 1: pair-walk kernel only; 2: persistent kernel for everything, then every tile recomputed;
// 3: persistent kernel for everything.
void attn_sparse_set_mode(int mode);

// Warp-level mma.sync kernel (attn_mma.cu): causal / GQA bf16 D=128 and fp16 D=64.
// elem: 0 = bf16 (dim 128), 1 = fp16 (dim 64).
cudaError_t attn_mma(void *out, const void *q, const void *k, const void *v, float *lse,
                     unsigned batch, unsigned lq, unsigned lk, unsigned heads, unsigned kv_heads,
                     float scale, bool causal, int elem, cudaStream_t stream);

// VSA coarse stage and merge (vsa_coarse.cu). `count` of the three tensors are pooled in
// one launch; scores / compression may be NULL (then not written / not computed).
cudaError_t vsa_tile_pool3(const void *const src[3], void *const tiled[3], float *const pooled[3],
                           const int *map, const int *sizes, int tiles, int heads, int count,
                           cudaStream_t stream);
cudaError_t vsa_score_select_compress(const float *poolq, const float *poolk, const float *poolv,
                                      float *scores, int *indices, int *counts,
                                      float *compression, int tiles, int prefix, int keep,
                                      int heads, float scale, cudaStream_t stream);
cudaError_t vsa_untile_merge(void *output, const void *tiled, const void *gate,
                             const float *compression, const int *map, int tiles, int heads,
                             cudaStream_t stream);

// Q/K RMS-norm + rotary embedding of the fused QKV projection output (qkv_rope.cu), head dim 128.
// qkv: [rows][3][heads][128] or, grouped, [rows][heads][3][128]; weights [128]; angles
// [rows][rope_half]; all bf16.
struct QkvRopeInput {
    const void *qkv, *q_weight, *k_weight, *rope_cos, *rope_sin;
    unsigned rows, heads, rope_half;
    bool grouped;
    float epsilon;
};
// q, k, v token-major [rows][heads][128].
cudaError_t qkv_rope_token_major(const QkvRopeInput &in, void *q, void *k, void *v, cudaStream_t stream);
// Straight into every rank's head shard [ranks*rows][heads/ranks][128] (window_x[p]: rank p's).
cudaError_t qkv_rope_head_shards(const QkvRopeInput &in, void *const window_q[], void *const window_k[],
                                 void *const window_v[], int rank, int ranks, cudaStream_t stream);
// Straight into VSA tile order [heads][tiles*64][128] plus FP32 tile means [heads][tiles][128].
cudaError_t qkv_rope_vsa_tiles(const QkvRopeInput &in, const int *map, const int *sizes, int tiles,
                               void *const tiled[3], float *const pooled[3], cudaStream_t stream);

// Attention output projection with gate + residual in the GEMM epilogue, and row-wise AdaLN
// (out_proj_gate.cu). weight [hidden][inner], modulation [mod rows][slots][hidden], all bf16.
cudaError_t out_proj_gate(void *gated, const void *residual, const void *attention_heads, const void *weight,
                          const void *modulation, const unsigned *row_map, unsigned rows, unsigned inner,
                          unsigned hidden, unsigned slots, unsigned gate_slot, cudaStream_t stream);
cudaError_t adaln_rows(void *output, const void *input, const void *norm_weight, const void *modulation,
                       const unsigned *row_map, unsigned rows, unsigned width, unsigned slots, unsigned shift_slot,
                       unsigned scale_slot, float epsilon, cudaStream_t stream);

// Ulysses block transpose (ulysses.cu): out[b][a][:] = in[a][b][:], rows of `row_units` 16-byte units.
cudaError_t transpose_rows_16b(void *out, const void *in, unsigned a, unsigned b, size_t row_units,
                               cudaStream_t stream);

// Fused exchange over peer memory (ulysses.cu). Every rank's window ends in one flag block.
constexpr int EXCHANGE_MAX_RANKS = 16, EXCHANGE_MAX_TENSORS = 4;
struct ExchangeFlags {
    unsigned long long done[EXCHANGE_MAX_RANKS];    // done[p]: last exchange whose data from rank p is complete here
    unsigned long long ready[EXCHANGE_MAX_RANKS];   // ready[p]: last exchange rank p has started
    unsigned counter;                               // CTAs of the running push kernel that have finished
    unsigned reserved[63];
};
struct ExchangeSync {
    ExchangeFlags *flags[EXCHANGE_MAX_RANKS];   // this process's mappings of every rank's flag block
    unsigned long long epoch;                   // number of this exchange, the same on every rank
    unsigned long long limit_ns;                // bound of every flag wait
    int *status;                                // device status word of this rank
    int rank, ranks;
};
// `tensors` (<= 4) tensors in one launch: src[t] goes to window[t][p] on rank p.
cudaError_t exchange_push(bool gather, int tensors, const void *const src[],
                          void *const window[][EXCHANGE_MAX_RANKS], const ExchangeSync &sync, unsigned rows,
                          unsigned heads, unsigned dim, cudaStream_t stream);
// Open / close around a kernel that stores into the peers' windows itself.
cudaError_t exchange_open(const ExchangeSync &sync, cudaStream_t stream);
cudaError_t exchange_close(const ExchangeSync &sync, cudaStream_t stream);

}  // namespace h3b
