// Dense attention forward, two query tiles per CTA (tcgen05 + TMEM + TMA), bf16, head dim 128.
//
// The single-tile kernel in attn_tc5.cu relies on two co-resident CTAs to overlap softmax
// with MMAs, but nothing keeps the two CTAs out of phase, and each loads K/V for itself.
// Here one CTA owns 256 query rows as two 128-row tiles A and B that share every K/V tile,
// and the MMA warp enforces the interleaving
//      PV_A(j)  QK_A(j+1)  PV_B(j)  QK_B(j+1)  ...
// so that while softmax warpgroup A works on S_A(j+1) the tensor pipe runs B's MMAs and vice
// versa. One CTA per SM: all 512 TMEM columns (S_A, S_B, O_A, O_B, 128 each), 64 KB of Q and a
// five-slot K/V ring in shared memory.
//   warps 0-3 / 4-7 : softmax warpgroups A / B (one thread per query row, the row's 128
//                     scores held in registers: one TMEM read pass)
//   warp 8          : TMA producer
//   warp 9          : MMA issuer      (warps 8-11 give most of their registers to the
//                                      softmax warpgroups with setmaxnreg)
//   warp 10         : watches the K/V ring for the issuer (see below)
// Whatever the issuing thread does between two batches of MMAs leaves the tensor pipe idle (its
// queue is short), and a probe of an mbarrier costs that thread 80-100 cycles even when the
// barrier is long complete. So the issuer waits on exactly two barriers per step, P_A and P_B:
// a thread of warp 10 waits for V_j and K_j+1 to land and adds its arrival to P_A's barrier; and
// the softmax threads need no "PV done" signal inside the loop because the commit that announces
// S(j) also covers PV(j-1), issued before it by the same thread. The ring has five slots: a tile
// takes 2000-3000 cycles from the request to shared memory when every SM asks at once, and with
// four slots (two steps of K/V) the request for step j+2 cannot leave before step j is over.
// P goes to the issuer in three pieces (keys 0-63, 64-95, 96-127), so six of a tile's eight PV
// MMAs run while the rest of its exponentials is still being taken; waits that are expected to be long park
// in hardware (mbar_wait_parked) - at the board's power limit a spinning warp costs clock.
// A fixed fraction of the exponentials is evaluated by a polynomial on the FMA pipe (see
// softmax_tc5.cuh) so the exponential unit is not the critical resource.
// Serves h3_flash3_bf16 / h3_flash3_cross_bf16 / non-causal h3_flash_bf16 whenever the call
// has more than one query tile (replacing the reference's cuda/flash3_attention.cu:18-94).
#include <cuda.h>

#include "attn_kernels.h"
#include "softmax_tc5.cuh"

namespace h3b {
namespace {

constexpr int PBM = 128, PBN = 128, PHD = 128;
constexpr int PAIR_THREADS = 384;                  // three warpgroups: softmax A, softmax B, {TMA, MMA}
constexpr int PAIR_STAGES = 5;                      // K0 V0 K1 V1 ... ring of 32 KB tiles
constexpr int PAIR_TILE_BYTES = PBN * PHD * 2;      // 32 KB
constexpr int PAIR_HALF_BYTES = PBN * 128;          // one 64-column half
constexpr int PAIR_Q_BYTES = 2 * PBM * PHD * 2;     // 64 KB
constexpr int PAIR_SMEM_BYTES = PAIR_Q_BYTES + PAIR_STAGES * PAIR_TILE_BYTES + 1024;
constexpr int PAIR_O_COL = 256;
constexpr float PAIR_RESCALE_LOG2 = 8.0f;
constexpr int PAIR_POLY_EVERY = 0x55;               // which groups of four columns take a pair of exponentials on the FMA pipe (25 %)

#ifdef H3B_TRACE
// Development aid, compiled only with -DH3B_TRACE: cycle counters of CTA (0,0,0).
__device__ long long g_pair_trace[32];
#define TRACE_T0() const long long trace_t0 = clock64()
#define TRACE_ADD(slot) g_pair_trace_local[slot] += clock64() - trace_t0
#else
#define TRACE_T0()
#define TRACE_ADD(slot)
#endif

constexpr int PAIR_MAX_SEGMENTS = 6;
// K/V may be given as up to six separate row ranges (live mode: text, sink, two recent chunks,
// current chunk ...) that are attended as if concatenated; every range has its own tensor maps
// and may end in a partial tile.
struct PairKvMaps {
    CUtensorMap k[PAIR_MAX_SEGMENTS], v[PAIR_MAX_SEGMENTS];
};

struct PairParams {
    int segments, seg_rows[PAIR_MAX_SEGMENTS];
    int lq, lk, heads, kv_heads;
    // Split-KV for short query blocks: when split_tiles > 0, blockIdx.z is not a batch but a
    // slice of split_tiles key tiles; the CTA writes its partial output and logsumexp as if
    // they were batch element blockIdx.z, and merge_splits_kernel combines the slices.
    int split_tiles;
    float scale, scale_log2;
    __nv_bfloat16 *out;
    float *lse;
    int *status;
    // sequence-gather fused into the epilogue (see PeerOutput); rows_per_rank == 0: off
    __nv_bfloat16 *peer_out[16];
    unsigned rows_per_rank, rank, total_heads;
};

__global__ void __launch_bounds__(PAIR_THREADS, 1)
attn_tc5_pair_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ PairKvMaps kv,
                     const PairParams p) {
    constexpr int ST = PAIR_STAGES;
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bars[1 + 2 * ST + 9];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_word;
    __shared__ int skip_launch;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_smem = smem_base;
    const uint32_t ring = q_smem + PAIR_Q_BYTES;

    const uint32_t bar0 = smem_u32(bars);
    const uint32_t bar_q_full = bar0;
    // tile number 2j is K_j, 2j+1 is V_j; tile i lives in slot i % ST and is that slot's use i / ST
    auto bar_full = [&](int s) { return bar0 + 8u * (1 + s); };
    auto bar_empty = [&](int s) { return bar0 + 8u * (1 + ST + s); };
    auto bar_s_full = [&](int t) { return bar0 + 8u * (1 + 2 * ST + t); };
    // P is handed over in three pieces (keys 0-63, 64-95, 96-127) so that PV MMAs run while the
    // later exponentials are still being taken
    auto bar_p_full = [&](int t, int piece) { return bar0 + 8u * (1 + 2 * ST + 2 + 3 * t + piece); };
    const uint32_t bar_pv_done = bar0 + 8u * (1 + 2 * ST + 8);   // the last PV of both tiles

    const int head = blockIdx.y, batch = p.split_tiles ? 0 : blockIdx.z, out_batch = blockIdx.z;
    const int kv_head = head / (p.heads / p.kv_heads);
    const int q_row0 = blockIdx.x * 2 * PBM;
    const int tile0 = p.split_tiles * (int)blockIdx.z;   // first key tile of this CTA's slice (0 without split)
    // key rows of range s as this CTA sees it (a split call has one range and takes a slice of it)
    const int slice_rows = p.split_tiles ? min(p.seg_rows[0] - tile0 * PBN, p.split_tiles * PBN) : 0;
    auto seg_rows = [&](int s) { return p.split_tiles ? slice_rows : p.seg_rows[s]; };
    int n_tiles = 0;   // key tiles over all segments
    for (int s = 0; s < p.segments; s++) n_tiles += (seg_rows(s) + PBN - 1) / PBN;

    if (tid == 0) {
        mbar_init(bar_q_full, 1);
        for (int s = 0; s < ST; s++) {
            mbar_init(bar_full(s), 1);
            mbar_init(bar_empty(s), 1);
        }
        for (int t = 0; t < 2; t++) mbar_init(bar_s_full(t), 1);
        mbar_init(bar_p_full(0, 0), 128 + 1);   // the softmax threads of tile A and the ring watcher
        mbar_init(bar_p_full(0, 1), 128);
        mbar_init(bar_p_full(0, 2), 128);
        mbar_init(bar_p_full(1, 0), 128);
        mbar_init(bar_p_full(1, 1), 128);
        mbar_init(bar_p_full(1, 2), 128);
        mbar_init(bar_pv_done, 1);
        mbar_fence_init();
        abort_word = 0;
        // A launch whose stream has already recorded a failure does nothing: when a protocol
        // error makes every CTA run into its wait limit, the CTAs that start later leave at once.
        skip_launch = *reinterpret_cast<volatile int *>(p.status) != STATUS_OK;
    }
    if (warp == 9) {
        tmem_alloc(smem_u32(&tmem_slot), 512);
        tmem_relinquish();
    }
    tc5_fence_before();
    __syncthreads();
    tc5_fence_after();
    const uint32_t tmem = tmem_slot;

    if (skip_launch) {
        // straight to the teardown
    } else if (warp >= 8) {
    warpgroup_reg_dec<88>();
    if (warp == 8) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&map_q);
            mbar_arrive_expect_tx(bar_q_full, PAIR_Q_BYTES);
            for (int t = 0; t < 2; t++) {
                const uint32_t dst = q_smem + t * (PAIR_Q_BYTES / 2);
                tma_load_4d(dst, &map_q, bar_q_full, 0, head, q_row0 + t * PBM, batch);
                tma_load_4d(dst + PAIR_HALF_BYTES, &map_q, bar_q_full, 64, head, q_row0 + t * PBM, batch);
            }
            int idx = 0;   // tile number: even = K, odd = V
            bool ok = true;
            for (int seg = 0; ok && seg < p.segments; seg++) {
                const int tiles = (seg_rows(seg) + PBN - 1) / PBN;
                for (int tile = 0; ok && tile < tiles; tile++) {
                    for (int which = 0; which < 2; which++, idx++) {
                        const int s = idx % ST, use = idx / ST;
                        if (use > 0 && !mbar_wait_parked(bar_empty(s), (use - 1) & 1, &abort_word)) {
                            ok = false;
                            break;
                        }
                        const uint32_t dst = ring + s * PAIR_TILE_BYTES;
                        const void *map = which ? (const void *)&kv.v[seg] : (const void *)&kv.k[seg];
                        mbar_arrive_expect_tx(bar_full(s), PAIR_TILE_BYTES);
                        tma_load_4d(dst, map, bar_full(s), 0, kv_head, (tile0 + tile) * PBN, batch);
                        tma_load_4d(dst + PAIR_HALF_BYTES, map, bar_full(s), 64, kv_head, (tile0 + tile) * PBN, batch);
                    }
                }
            }
        }
    } else if (warp == 9) {
        // ------------------------------- MMA issuer -------------------------------
        // The whole warp walks the loop and one elected lane issues: with the loop inside a
        // one-lane branch every descriptor word is per-thread data that has to be moved to a
        // uniform register in front of each MMA.
        {
            const bool leader = elect_one();
            constexpr uint32_t idesc_qk = mma_idesc(PBM, PBN, 1, 0);
            constexpr uint32_t idesc_pv = mma_idesc(PBM, PHD, 1, 1);
            // Descriptors are built once (Q) or once per stage (K, V); a K-step only adds to
            // the low word: +2 per 32 bytes inside a 64-column half, +1024 for the second half
            // (16 KB), +128 per 16 V rows (2 KB).
            uint32_t q_lo[2], q_hi[2];
            for (int t = 0; t < 2; t++) {
                const uint64_t d = smem_desc_sw128(q_smem + t * (PAIR_Q_BYTES / 2), 16, 1024);
                q_lo[t] = (uint32_t)d;
                q_hi[t] = (uint32_t)(d >> 32);
            }
            const uint64_t k_proto = smem_desc_sw128(ring, 16, 1024);
            const uint64_t v_proto = smem_desc_sw128(ring, PAIR_HALF_BYTES, 1024);
            const uint32_t k_hi = (uint32_t)(k_proto >> 32), v_hi = (uint32_t)(v_proto >> 32);
            const uint32_t k_ring_lo = (uint32_t)k_proto, v_ring_lo = (uint32_t)v_proto;  // LBO lives in the low word
            auto issue_qk = [&](int j, int t) {   // S_t = Q_t . K_j^T
                const uint32_t k_lo = k_ring_lo + ((2 * j) % ST) * (PAIR_TILE_BYTES >> 4);
                if (leader) {
#pragma unroll
                    for (int kk = 0; kk < PHD / 16; kk++) {
                        const uint32_t off = (kk / 4) * (PAIR_HALF_BYTES >> 4) + (kk % 4) * 2;
                        mma_ss_words(tmem + t * PBN, q_lo[t] + off, q_hi[t], k_lo + off, k_hi, idesc_qk,
                                     kk > 0);
                    }
                    mma_commit(bar_s_full(t));   // also tells the softmax threads that PV_t(j-1) is complete
                }
                __syncwarp();
            };
            auto issue_pv = [&](int j, int t, int piece) {   // O_t += P_t . V_j over keys 0-63, 64-95 or 96-127
                const uint32_t v_lo = v_ring_lo + ((2 * j + 1) % ST) * (PAIR_TILE_BYTES >> 4);
                const int first = piece == 0 ? 0 : piece == 1 ? 4 : 6, last = piece == 0 ? 4 : piece == 1 ? 6 : 8;
                if (leader) {
#pragma unroll
                    for (int kk = 0; kk < 8; kk++)
                        if (kk >= first && kk < last)
                            mma_ts_words(tmem + PAIR_O_COL + t * PHD, tmem + t * PBN + kk * 8,
                                         v_lo + kk * (2048 >> 4), v_hi, idesc_pv, (j > 0) || (kk > 0));
                }
                __syncwarp();
            };
#ifdef H3B_TRACE
            long long g_pair_trace_local[8] = {};
            const long long trace_begin = clock64();
#endif
            auto release = [&](int tile) {   // the slot may be refilled once the MMAs issued so far are done
                if (leader) mma_commit(bar_empty(tile % ST));
            };
            bool alive = mbar_wait_converged(bar_q_full, 0, &abort_word) &&
                         mbar_wait_converged(bar_full(0), 0, &abort_word);
            if (alive) {
                tc5_fence_after();
                issue_qk(0, 0);
                issue_qk(0, 1);
                release(0);
            }
            for (int j = 0; alive && j < n_tiles; j++) {
                const bool more = j + 1 < n_tiles;
                {
                    // P of tile A, and (through the ring watcher) V of this step and K of the next
                    TRACE_T0();
                    if (!mbar_wait_converged(bar_p_full(0, 0), j & 1, &abort_word)) break;
                    TRACE_ADD(0);
                }
                tc5_fence_after();
                {
                    TRACE_T0();
                    issue_pv(j, 0, 0);
                    if (!mbar_wait_converged(bar_p_full(0, 1), j & 1, &abort_word)) break;
                    tc5_fence_after();
                    issue_pv(j, 0, 1);
                    if (!mbar_wait_converged(bar_p_full(0, 2), j & 1, &abort_word)) break;
                    tc5_fence_after();
                    issue_pv(j, 0, 2);
                    TRACE_ADD(4);
                }
                if (more) {
                    TRACE_T0();
                    issue_qk(j + 1, 0);
                    TRACE_ADD(5);
                }
                {
                    TRACE_T0();
                    if (!mbar_wait_converged(bar_p_full(1, 0), j & 1, &abort_word)) break;
                    TRACE_ADD(3);
                }
                tc5_fence_after();
                {
                    TRACE_T0();
                    issue_pv(j, 1, 0);
                    if (!mbar_wait_converged(bar_p_full(1, 1), j & 1, &abort_word)) break;
                    tc5_fence_after();
                    issue_pv(j, 1, 1);
                    if (!mbar_wait_converged(bar_p_full(1, 2), j & 1, &abort_word)) break;
                    tc5_fence_after();
                    issue_pv(j, 1, 2);
                    release(2 * j + 1);
                    TRACE_ADD(6);
                }
                if (more) {
                    TRACE_T0();
                    issue_qk(j + 1, 1);
                    release(2 * j + 2);
                    TRACE_ADD(7);
                } else if (leader) {
                    mma_commit(bar_pv_done);      // both accumulators are final
                }
                __syncwarp();
            }
#ifdef H3B_TRACE
            if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && lane == 0) {
                g_pair_trace[0] = clock64() - trace_begin;   // MMA thread: whole walk
                g_pair_trace[1] = g_pair_trace_local[0];     // waiting for P of tile A
                g_pair_trace[2] = 0;
                g_pair_trace[3] = 0;
                g_pair_trace[4] = g_pair_trace_local[3];     // waiting for P of tile B
                g_pair_trace[5] = n_tiles;
                g_pair_trace[6] = g_pair_trace_local[4];     // thread time inside issue_pv(A)
                g_pair_trace[7] = g_pair_trace_local[5];     // thread time inside issue_qk(A)
                g_pair_trace[24] = g_pair_trace_local[6];    // the same for tile B: both PV halves with the wait between them
                g_pair_trace[25] = g_pair_trace_local[7];    // issue_qk(B) and the ring release
            }
#endif
        }
    } else if (warp == 10) {
        // ------------------------------- ring watcher -------------------------------
        if (lane == 0) {
            // One arrival per phase of P_A's barrier: the next tiles are often there before the
            // softmax threads are done, so wait for the phase to end before arriving again.
            for (int g = 0; g < n_tiles; g++) {
                const int v = 2 * g + 1, k = 2 * g + 2;
                if (!mbar_wait_parked(bar_full(v % ST), (v / ST) & 1, &abort_word)) break;
                if (g + 1 < n_tiles && !mbar_wait_parked(bar_full(k % ST), (k / ST) & 1, &abort_word)) break;
                mbar_arrive(bar_p_full(0, 0));
                if (!mbar_wait_parked(bar_p_full(0, 0), g & 1, &abort_word)) break;
            }
        }
    }
    } else {
        warpgroup_reg_inc<208>();
        // ------------------------------ online softmax ------------------------------
        const int t = warp >> 2;                // which query tile
        const int r = tid & 127;                // row inside the tile == TMEM lane
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t s_addr = tmem + lane_base + t * PBN;
        const uint32_t o_addr = tmem + lane_base + PAIR_O_COL + t * PHD;
        float m_ref = -INFINITY, l = 0.0f;
        bool alive = true;
#ifdef H3B_TRACE
        long long g_pair_trace_local[8] = {};
        const long long trace_begin = clock64();
#endif
        int seg = 0, seg_tile = 0;   // which segment, which tile of it, step j is
        for (int j = 0; j < n_tiles; j++) {
            while (seg_tile * PBN >= seg_rows(seg)) {
                seg++;
                seg_tile = 0;
            }
            const int nvalid = min(PBN, seg_rows(seg) - seg_tile * PBN);
            seg_tile++;
            {
                TRACE_T0();
                alive = __all_sync(0xffffffffu, mbar_wait_parked(bar_s_full(t), j & 1, &abort_word));
                TRACE_ADD(0);
            }
            if (!alive) break;
            tc5_fence_after();
#ifdef H3B_TRACE
            const long long trace_work = clock64();
#endif
            bool first_half_out = false, second_piece_out = false;
            if (nvalid >= PBN) {
                // the whole row of scores in registers: one TMEM read pass
                uint32_t s0[32], s1[32], s2[32], s3[32];
                tmem_ld32(s_addr, s0);
                tmem_ld32(s_addr + 32, s1);
                tmem_ld32(s_addr + 64, s2);
                tmem_ld32(s_addr + 96, s3);
                tmem_wait_ld();
                float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                max_chunk4(s0, mx);
                max_chunk4(s1, mx);
                max_chunk4(s2, mx);
                max_chunk4(s3, mx);
                const float m_new = fmaxf(max3(m_ref, mx[0], mx[1]), fmaxf(mx[2], mx[3]));
                const bool grow = (m_new - m_ref) * p.scale_log2 > PAIR_RESCALE_LOG2;
                if (__any_sync(0xffffffffu, grow)) {
                    const float alpha = grow ? fast_exp2((m_ref - m_new) * p.scale_log2) : 1.0f;
                    if (grow) m_ref = m_new;
                    l *= alpha;
                    if (j > 0) {   // PV(j-1) is complete: S(j)'s commit covered it
#pragma unroll
                        for (int c = 0; c < PHD / 32; c++) {
                            uint32_t v[32];
                            tmem_ld32(o_addr + c * 32, v);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; i++)
                                v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                            tmem_st32(o_addr + c * 32, v);
                        }
                        tmem_wait_st();
                    }
                }
                const float neg = -m_ref * p.scale_log2;
                const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
                const float2 neg2 = make_float2(neg, neg);
                float2 sum0 = make_float2(0.f, 0.f), sum1 = make_float2(0.f, 0.f);
                uint32_t packed[16];
                exp_chunk_mixed<PAIR_POLY_EVERY>(s0, packed, scale2, neg2, sum0, sum1);
                tmem_st16(s_addr, packed);
                exp_chunk_mixed<PAIR_POLY_EVERY>(s1, packed, scale2, neg2, sum0, sum1);
                tmem_st16(s_addr + 16, packed);
                tmem_wait_st();
                tc5_fence_before();
                mbar_arrive(bar_p_full(t, 0));
                first_half_out = true;
                exp_chunk_mixed<PAIR_POLY_EVERY>(s2, packed, scale2, neg2, sum0, sum1);
                tmem_st16(s_addr + 32, packed);
                tmem_wait_st();
                tc5_fence_before();
                mbar_arrive(bar_p_full(t, 1));
                second_piece_out = true;
                exp_chunk_mixed<PAIR_POLY_EVERY>(s3, packed, scale2, neg2, sum0, sum1);
                tmem_st16(s_addr + 48, packed);
                l += (sum0.x + sum0.y) + (sum1.x + sum1.y);
            } else {
                // ragged last tile: masked two-pass path
                const float mx = row_max_masked<PBN>(s_addr, nvalid);
                const float m_new = fmaxf(m_ref, mx);
                const bool grow = (m_new - m_ref) * p.scale_log2 > PAIR_RESCALE_LOG2;
                if (__any_sync(0xffffffffu, grow)) {
                    const float alpha = grow ? fast_exp2((m_ref - m_new) * p.scale_log2) : 1.0f;
                    if (grow) m_ref = m_new;
                    l *= alpha;
                    if (j > 0) {   // PV(j-1) is complete: S(j)'s commit covered it
#pragma unroll
                        for (int c = 0; c < PHD / 32; c++) {
                            uint32_t v[32];
                            tmem_ld32(o_addr + c * 32, v);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; i++)
                                v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                            tmem_st32(o_addr + c * 32, v);
                        }
                        tmem_wait_st();
                    }
                }
                l += exp_store_masked<PBN>(s_addr, s_addr, p.scale_log2, -m_ref * p.scale_log2, nvalid);
            }
            tmem_wait_st();
            tc5_fence_before();
            if (!first_half_out) mbar_arrive(bar_p_full(t, 0));
            if (!second_piece_out) mbar_arrive(bar_p_full(t, 1));
            mbar_arrive(bar_p_full(t, 2));
#ifdef H3B_TRACE
            g_pair_trace_local[1] += clock64() - trace_work;
#endif
        }
#ifdef H3B_TRACE
        if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (tid & 127) == 0) {
            g_pair_trace[8 + 4 * t] = clock64() - trace_begin;       // softmax warpgroup t: whole walk
            g_pair_trace[9 + 4 * t] = g_pair_trace_local[0];         // waiting for S
            g_pair_trace[10 + 4 * t] = g_pair_trace_local[1];        // S ready -> P delivered
        }
#endif

        // -------- epilogue: O / l -> bf16, straight to global memory --------
        if (alive) alive = __all_sync(0xffffffffu, mbar_wait(bar_pv_done, 0, &abort_word));
        if (alive) {
            tc5_fence_after();
            const float inv = 1.0f / l;
            const int row = q_row0 + t * PBM + r;
            const bool store = row < p.lq;
            __nv_bfloat16 *dst;
            if (p.rows_per_rank) {
                // this row belongs to another rank's row shard: store it there, in place
                const unsigned owner = (unsigned)row / p.rows_per_rank, local = (unsigned)row % p.rows_per_rank;
                dst = p.peer_out[store ? owner : 0] +
                      ((size_t)local * p.total_heads + (size_t)p.rank * p.heads + head) * PHD;
            } else {
                dst = p.out + (((size_t)out_batch * p.lq + row) * p.heads + head) * PHD;
            }
            if (store && p.lse)
                p.lse[((size_t)out_batch * p.heads + head) * p.lq + row] = m_ref * p.scale + __logf(l);
#pragma unroll
            for (int c = 0; c < PHD / 32; c++) {
                uint32_t v[32];
                tmem_ld32(o_addr + c * 32, v);
                tmem_wait_ld();
                if (store) {
                    uint4 *d4 = reinterpret_cast<uint4 *>(dst + c * 32);
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        uint4 w;
                        w.x = pack_bf16(__uint_as_float(v[i * 8 + 0]) * inv, __uint_as_float(v[i * 8 + 1]) * inv);
                        w.y = pack_bf16(__uint_as_float(v[i * 8 + 2]) * inv, __uint_as_float(v[i * 8 + 3]) * inv);
                        w.z = pack_bf16(__uint_as_float(v[i * 8 + 4]) * inv, __uint_as_float(v[i * 8 + 5]) * inv);
                        w.w = pack_bf16(__uint_as_float(v[i * 8 + 6]) * inv, __uint_as_float(v[i * 8 + 7]) * inv);
                        d4[i] = w;
                    }
                }
            }
        }
    }

    // ---------------------------------- teardown ----------------------------------
    tc5_fence_before();
    __syncthreads();
    if (abort_word) {
        if (tid == 0) atomicCAS(p.status, STATUS_OK, STATUS_WAIT_TIMEOUT);
        if (warp == 8) __nanosleep(1000000);   // let copies in flight land before smem is reused
        __syncthreads();
    }
    if (warp == 9) {
        tc5_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

// Combines the slices of a split-KV call: out[r][h][:] = sum_s w_s O_s[r][h][:] / sum_s w_s with
// w_s = exp(lse_s - max_s lse_s). One thread per (row, head, eight dims).
__global__ void __launch_bounds__(256)
merge_splits_kernel(__nv_bfloat16 *__restrict__ out, float *__restrict__ lse_out, const uint4 *__restrict__ partial,
                    const float *__restrict__ lse, int splits, int lq, int heads) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)lq * heads * (PHD / 8);
    if (i >= total) return;
    const int v = (int)(i % (PHD / 8)), head = (int)((i / (PHD / 8)) % heads), row = (int)(i / ((size_t)(PHD / 8) * heads));
    float top = -INFINITY;
    for (int s = 0; s < splits; s++) top = fmaxf(top, lse[((size_t)s * heads + head) * lq + row]);
    float acc[8] = {}, weight = 0.0f;
    for (int s = 0; s < splits; s++) {
        const float w = __expf(lse[((size_t)s * heads + head) * lq + row] - top);
        const uint4 x = partial[(((size_t)s * lq + row) * heads + head) * (PHD / 8) + v];
        const uint32_t words[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int k = 0; k < 4; k++) {
            acc[2 * k] = fmaf(w, __uint_as_float(words[k] << 16), acc[2 * k]);
            acc[2 * k + 1] = fmaf(w, __uint_as_float(words[k] & 0xffff0000u), acc[2 * k + 1]);
        }
        weight += w;
    }
    const float inv = 1.0f / weight;
    uint4 y;
    y.x = pack_bf16(acc[0] * inv, acc[1] * inv);
    y.y = pack_bf16(acc[2] * inv, acc[3] * inv);
    y.z = pack_bf16(acc[4] * inv, acc[5] * inv);
    y.w = pack_bf16(acc[6] * inv, acc[7] * inv);
    reinterpret_cast<uint4 *>(out)[i] = y;
    if (lse_out && v == 0) lse_out[(size_t)head * lq + row] = top + __logf(weight);
}

}  // namespace

cudaError_t attn_merge_splits(void *out, float *lse_out, const void *partial, const float *lse, unsigned splits,
                              unsigned lq, unsigned heads, cudaStream_t stream) {
    const size_t total = (size_t)lq * heads * (PHD / 8);
    merge_splits_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(
        static_cast<__nv_bfloat16 *>(out), lse_out, static_cast<const uint4 *>(partial), lse, (int)splits, (int)lq,
        (int)heads);
    return cudaGetLastError();
}

cudaError_t attn_dense_tc5_pair(const CUtensorMap_st *mq, const CUtensorMap_st *mk,
                                const CUtensorMap_st *mv, void *out, float *lse, unsigned batch,
                                unsigned lq, unsigned lk, unsigned heads, unsigned kv_heads,
                                float scale, int *status, cudaStream_t stream, const PeerOutput *peer,
                                unsigned segments, const unsigned *segment_rows, unsigned split_tiles) {
    static thread_local int configured_device = -1;
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    if (configured_device != device) {
        e = cudaFuncSetAttribute(attn_tc5_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 PAIR_SMEM_BYTES);
        if (e != cudaSuccess) return e;
        configured_device = device;
    }
    // mk / mv point to `segments` maps each; without a segment list: one range of lk rows
    if (segments > (unsigned)PAIR_MAX_SEGMENTS || (segments > 1 && batch != 1)) return cudaErrorInvalidValue;
    // split-KV: one key range, batch 1, no peer output; the slices ride on grid.z
    unsigned splits = 1;
    if (split_tiles) {
        if (segments > 1 || batch != 1 || peer || !lse) return cudaErrorInvalidValue;
        splits = ((lk + PBN - 1) / PBN + split_tiles - 1) / split_tiles;
    }
    PairKvMaps kv{};
    PairParams p{};
    p.segments = segments ? (int)segments : 1;
    for (int i = 0; i < p.segments; i++) {
        kv.k[i] = mk[i];
        kv.v[i] = mv[i];
        p.seg_rows[i] = segments ? (int)segment_rows[i] : (int)lk;
        if (p.seg_rows[i] <= 0) return cudaErrorInvalidValue;
    }
    p.lq = (int)lq;
    p.lk = (int)lk;
    p.heads = (int)heads;
    p.kv_heads = (int)kv_heads;
    p.scale = scale;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.out = static_cast<__nv_bfloat16 *>(out);
    p.lse = lse;
    p.status = status;
    p.split_tiles = (int)split_tiles;
    if (peer) {
        if (batch != 1 || !peer->rows_per_rank) return cudaErrorInvalidValue;
        for (int i = 0; i < 16; i++) p.peer_out[i] = static_cast<__nv_bfloat16 *>(peer->base[i]);
        p.rows_per_rank = peer->rows_per_rank;
        p.rank = peer->rank;
        p.total_heads = peer->total_heads;
    }
    dim3 grid((lq + 2 * PBM - 1) / (2 * PBM), heads, split_tiles ? splits : batch);
    attn_tc5_pair_kernel<<<grid, PAIR_THREADS, PAIR_SMEM_BYTES, stream>>>(*mq, kv, p);
    return cudaGetLastError();
}

}  // namespace h3b

#ifdef H3B_TRACE
extern "C" cudaError_t h3b_debug_pair_trace(long long *host32) {
    return cudaMemcpyFromSymbol(host32, h3b::g_pair_trace, sizeof(long long) * 32);
}
#endif
