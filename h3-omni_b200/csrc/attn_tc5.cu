// Attention forward on Blackwell tensor cores (tcgen05 + TMEM + TMA), bf16, head dim 128.
//
// One CTA owns one 128-row query tile and walks KV tiles of BN rows:
//   warp 4 (one lane)  : TMA producer - Q once, then K/V tiles into swizzled shared memory
//   warp 5 (one lane)  : MMA issuer   - S = Q.K^T into TMEM, later O += P.V with P read from TMEM
//   warps 0-3          : online softmax - one thread per query row; S is read from TMEM,
//                        P is written back over it as packed bf16; O stays in TMEM for the
//                        whole walk and is rescaled lazily (only when the running row
//                        maximum grows by more than 2^8).
// Two CTAs are resident per SM (96 KB shared memory and 256 TMEM columns each), so one CTA's
// softmax overlaps the other's MMAs.
//
// DENSE  (BN = 128): token-major [B][L][H][128] tensors, rectangular Lq x Lk, GQA.
//   Replaces the kernels behind h3_flash3_bf16 / h3_flash3_cross_bf16
//   (cuda/flash3_attention.cu:18-94 in the reference).
// SPARSE (BN = 64): head-major tiled [H][tiles*64][128] tensors; a CTA pairs two adjacent
//   64-row query tiles and walks the sorted union of their selected KV tiles, masking each
//   half against its own list and every KV tile against its valid length. (Two gathered KV
//   tiles per step, N = 128, was tried because an N = 64 MMA reaches only two thirds of the
//   tensor rate; it lost more by giving up the double-buffered S than it gained.) Replaces
//   fwd_attend_ker<128> (cuda/vendor/vsa_hopper_forward.cuh:68-270) behind h3_vsa_hopper.
#include <cuda.h>

#include <algorithm>

#include "attn_kernels.h"
#include "sm100_ptx.cuh"
#include "softmax_tc5.cuh"

namespace h3b {

namespace {

constexpr int BM = 128;          // query rows per CTA
constexpr int HD = 128;          // head dimension
constexpr int TC5_THREADS = 192;
constexpr int TMEM_COLS = 256;   // S/P buffers in [0,128), O in [128,256)
constexpr int O_COL = 128;
constexpr int Q_BYTES = BM * HD * 2;
constexpr float RESCALE_LOG2 = 8.0f;

struct Tc5Params {
    int lq, lk, heads, kv_heads;
    float scale, scale_log2;
    __nv_bfloat16 *out;
    float *lse;
    const int *indices, *counts, *sizes;
    const unsigned char *redo;   // sparse: when set, only query tiles marked here are computed
    int tiles;
    int *status;
};

template <int BN>
struct Tc5Config {
    static constexpr int S_BUFS = 128 / BN;        // S double-buffered when the tile is narrow
    static constexpr int STAGES = 128 / BN;        // K ring and V ring depth
    static constexpr int TILE_BYTES = BN * HD * 2; // one K or V tile
    static constexpr int HALF_BYTES = BN * 128;    // one 64-column half of a tile
    static constexpr int SMEM_BYTES = Q_BYTES + 2 * STAGES * TILE_BYTES + 1024;
};

template <int BN, bool SPARSE>
__global__ void __launch_bounds__(TC5_THREADS, 2)
attn_tc5_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const Tc5Params p) {
    using Cfg = Tc5Config<BN>;
    constexpr int SB = Cfg::S_BUFS, ST = Cfg::STAGES;

    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bars[1 + 4 * ST + 2 * SB + 1];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_word;
    __shared__ uint32_t bits_a[SPARSE ? 128 : 1], bits_b[SPARSE ? 128 : 1];
    __shared__ int union_count;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_smem = smem_base;
    const uint32_t k_smem = q_smem + Q_BYTES;
    const uint32_t v_smem = k_smem + ST * Cfg::TILE_BYTES;

    const uint32_t bar0 = smem_u32(bars);
    auto bar_q_full = [&]() { return bar0; };
    auto bar_k_full = [&](int s) { return bar0 + 8u * (1 + s); };
    auto bar_k_empty = [&](int s) { return bar0 + 8u * (1 + ST + s); };
    auto bar_v_full = [&](int s) { return bar0 + 8u * (1 + 2 * ST + s); };
    auto bar_v_empty = [&](int s) { return bar0 + 8u * (1 + 3 * ST + s); };
    auto bar_s_full = [&](int s) { return bar0 + 8u * (1 + 4 * ST + s); };
    auto bar_p_full = [&](int s) { return bar0 + 8u * (1 + 4 * ST + SB + s); };
    const uint32_t bar_pv_done = bar0 + 8u * (1 + 4 * ST + 2 * SB);

    const int head = blockIdx.y;
    const int batch = blockIdx.z;
    const int kv_head = SPARSE ? head : head / (p.heads / p.kv_heads);
    const int q_row0 = blockIdx.x * BM;  // dense: token row; sparse: padded tiled row

    if (SPARSE && p.redo) {
        // recomputation pass: leave at once unless one of this CTA's two query tiles is marked
        const size_t first = (size_t)head * p.tiles + blockIdx.x * 2;
        const bool second = blockIdx.x * 2 + 1 < p.tiles;
        if (!p.redo[first] && !(second && p.redo[first + 1])) return;
    }

    if (tid == 0) {
        mbar_init(bar_q_full(), 1);
        for (int s = 0; s < ST; s++) {
            mbar_init(bar_k_full(s), 1);
            mbar_init(bar_k_empty(s), 1);
            mbar_init(bar_v_full(s), 1);
            mbar_init(bar_v_empty(s), 1);
        }
        for (int s = 0; s < SB; s++) {
            mbar_init(bar_s_full(s), 1);
            mbar_init(bar_p_full(s), 128);
        }
        mbar_init(bar_pv_done, 1);
        mbar_fence_init();
        abort_word = 0;
        union_count = 0;
    }
    if (SPARSE && tid < 128) {
        bits_a[tid] = 0;
        bits_b[tid] = 0;
    }
    if (warp == 5) {
        tmem_alloc(smem_u32(&tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc5_fence_before();
    __syncthreads();
    tc5_fence_after();
    const uint32_t tmem = tmem_slot;

    int n_tiles;  // KV tiles this CTA walks
    if (SPARSE) {
        // Bitmaps of the KV tiles selected by query tile A (rows 0-63) and B (rows 64-127).
        const int qa = blockIdx.x * 2, qb = qa + 1;
        const size_t row_a = (size_t)head * p.tiles + qa;
        const int raw_a = p.counts[row_a], raw_b = qb < p.tiles ? p.counts[row_a + 1] : 0;
        // a count outside [0, tiles] is refused like a bad index; the list is clamped
        if (tid == 0 && (raw_a < 0 || raw_a > p.tiles || raw_b < 0 || raw_b > p.tiles))
            atomicCAS(p.status, STATUS_OK, STATUS_BAD_ARGUMENT);
        const int count_a = max(0, min(raw_a, p.tiles));
        const int count_b = max(0, min(raw_b, p.tiles));
        for (int i = tid; i < count_a + count_b; i += TC5_THREADS) {
            const bool is_a = i < count_a;
            const int kt = is_a ? p.indices[row_a * p.tiles + i]
                                : p.indices[(row_a + 1) * p.tiles + (i - count_a)];
            if (kt < 0 || kt >= p.tiles) {
                atomicCAS(p.status, STATUS_OK, STATUS_BAD_ARGUMENT);  // skip, never dereference
                continue;
            }
            atomicOr(is_a ? &bits_a[kt >> 5] : &bits_b[kt >> 5], 1u << (kt & 31));
        }
        __syncthreads();
        if (warp == 0) {
            int c = 0;
            for (int w = lane; w < 128; w += 32) c += __popc(bits_a[w] | bits_b[w]);
            for (int o = 16; o; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
            if (lane == 0) union_count = c;
        }
        __syncthreads();
        n_tiles = union_count;
    } else {
        n_tiles = (p.lk + BN - 1) / BN;
    }

    // Ordered walk over the union bitmap (sparse) or 0,1,2,... (dense).
    struct Walk {
        int word;
        uint32_t cur;
    };
    Walk walk{-1, 0u};
    auto next_tile = [&](int j, int &kt, int &flags) {
        if constexpr (!SPARSE) {
            kt = j;
            flags = 3;
        } else {
            while (walk.cur == 0u) {
                walk.word++;
                walk.cur = bits_a[walk.word] | bits_b[walk.word];
            }
            const int b = __ffs(walk.cur) - 1;
            walk.cur &= walk.cur - 1;
            kt = walk.word * 32 + b;
            flags = ((bits_a[walk.word] >> b) & 1u) | (((bits_b[walk.word] >> b) & 1u) << 1);
        }
    };

    if (warp == 4) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&map_q);
            tma_prefetch_desc(&map_k);
            tma_prefetch_desc(&map_v);
            mbar_arrive_expect_tx(bar_q_full(), Q_BYTES);
            if (SPARSE) {
                tma_load_4d(q_smem, &map_q, bar_q_full(), 0, q_row0, head, 0);
                tma_load_4d(q_smem + Q_BYTES / 2, &map_q, bar_q_full(), 64, q_row0, head, 0);
            } else {
                tma_load_4d(q_smem, &map_q, bar_q_full(), 0, head, q_row0, batch);
                tma_load_4d(q_smem + Q_BYTES / 2, &map_q, bar_q_full(), 64, head, q_row0, batch);
            }
            for (int j = 0; j < n_tiles; j++) {
                int kt, flags;
                next_tile(j, kt, flags);
                const int s = j % ST, use = j / ST;
                const int row = kt * BN;
                if (use > 0 && !mbar_wait(bar_k_empty(s), (use - 1) & 1, &abort_word)) break;
                const uint32_t kd = k_smem + s * Cfg::TILE_BYTES;
                mbar_arrive_expect_tx(bar_k_full(s), Cfg::TILE_BYTES);
                if (SPARSE) {
                    tma_load_4d(kd, &map_k, bar_k_full(s), 0, row, kv_head, 0);
                    tma_load_4d(kd + Cfg::HALF_BYTES, &map_k, bar_k_full(s), 64, row, kv_head, 0);
                } else {
                    tma_load_4d(kd, &map_k, bar_k_full(s), 0, kv_head, row, batch);
                    tma_load_4d(kd + Cfg::HALF_BYTES, &map_k, bar_k_full(s), 64, kv_head, row, batch);
                }
                if (use > 0 && !mbar_wait(bar_v_empty(s), (use - 1) & 1, &abort_word)) break;
                const uint32_t vd = v_smem + s * Cfg::TILE_BYTES;
                mbar_arrive_expect_tx(bar_v_full(s), Cfg::TILE_BYTES);
                if (SPARSE) {
                    tma_load_4d(vd, &map_v, bar_v_full(s), 0, row, kv_head, 0);
                    tma_load_4d(vd + Cfg::HALF_BYTES, &map_v, bar_v_full(s), 64, row, kv_head, 0);
                } else {
                    tma_load_4d(vd, &map_v, bar_v_full(s), 0, kv_head, row, batch);
                    tma_load_4d(vd + Cfg::HALF_BYTES, &map_v, bar_v_full(s), 64, kv_head, row, batch);
                }
            }
        }
    } else if (warp == 5) {
        // ------------------------------- MMA issuer -------------------------------
        if (lane == 0 && n_tiles > 0) {
            constexpr uint32_t idesc_qk = mma_idesc(BM, BN, 1, 0);
            constexpr uint32_t idesc_pv = mma_idesc(BM, HD, 1, 1);
            bool alive = mbar_wait(bar_q_full(), 0, &abort_word);
            // Descriptors once per kernel (Q) or per stage (K, V); each MMA then costs one add on
            // the low word: +2 per 32 bytes inside a 64-column half, +HALF_BYTES/16 for the second
            // half, +128 per 16 V rows. The issuing thread shares its scheduler with busy softmax
            // warps, so every instruction it saves keeps the tensor pipe fed.
            const uint64_t q_desc = smem_desc_sw128(q_smem, 16, 1024);
            const uint64_t k_proto = smem_desc_sw128(k_smem, 16, 1024);
            const uint64_t v_proto = smem_desc_sw128(v_smem, Cfg::HALF_BYTES, 1024);   // LBO lives in the low word
            const uint32_t q_lo = (uint32_t)q_desc, q_hi = (uint32_t)(q_desc >> 32);
            const uint32_t k_lo0 = (uint32_t)k_proto, k_hi = (uint32_t)(k_proto >> 32);
            const uint32_t v_lo0 = (uint32_t)v_proto, v_hi = (uint32_t)(v_proto >> 32);
            auto issue_qk = [&](int j) -> bool {
                const int s = j % ST, sb = j % SB;
                if (!mbar_wait(bar_k_full(s), (j / ST) & 1, &abort_word)) return false;
                const uint32_t k_lo = k_lo0 + s * (Cfg::TILE_BYTES >> 4);
#pragma unroll
                for (int kk = 0; kk < HD / 16; kk++)
                    mma_ss_words(tmem + sb * BN, q_lo + (kk / 4) * (Q_BYTES / 2 >> 4) + (kk % 4) * 2, q_hi,
                                 k_lo + (kk / 4) * (Cfg::HALF_BYTES >> 4) + (kk % 4) * 2, k_hi, idesc_qk,
                                 kk > 0);
                mma_commit(bar_s_full(sb));
                mma_commit(bar_k_empty(s));
                return true;
            };
            alive = alive && issue_qk(0);
            for (int j = 0; alive && j < n_tiles; j++) {
                if (SB == 2 && j + 1 < n_tiles && !issue_qk(j + 1)) break;
                const int s = j % ST, sb = j % SB;
                // V was requested long ago: probe it before P so the (normally immediate) wait
                // is off the path between P arriving and the PV issue
                if (!mbar_wait(bar_v_full(s), (j / ST) & 1, &abort_word)) break;
                if (!mbar_wait(bar_p_full(sb), (j / SB) & 1, &abort_word)) break;
                tc5_fence_after();
                // V tile [BN rows][128] is MN-major for this product: the two 64-column halves
                // are HALF_BYTES apart, 8-row groups 1024 bytes apart.
                const uint32_t v_lo = v_lo0 + s * (Cfg::TILE_BYTES >> 4);
                mma_ts_words(tmem + O_COL, tmem + sb * BN, v_lo, v_hi, idesc_pv, j > 0);
#pragma unroll
                for (int kk = 1; kk < BN / 16; kk++)
                    mma_ts_words(tmem + O_COL, tmem + sb * BN + kk * 8, v_lo + kk * (2048 >> 4), v_hi,
                                 idesc_pv, 1);
                mma_commit(bar_v_empty(s));
                mma_commit(bar_pv_done);
                if (SB == 1 && j + 1 < n_tiles && !issue_qk(j + 1)) break;
            }
        }
    } else {
        // ------------------------------ online softmax ------------------------------
        const int r = tid;  // query row inside the tile == TMEM lane
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        const int half = r >> 6;
        float m_ref = -INFINITY, l = 0.0f;
        bool alive = true;
        for (int j = 0; j < n_tiles; j++) {
            int kt, flags;
            next_tile(j, kt, flags);
            int nvalid;
            if (SPARSE) {
                nvalid = ((flags >> half) & 1) ? min(p.sizes[kt], BN) : 0;
            } else {
                nvalid = min(BN, p.lk - j * BN);
            }
            const int sb = j % SB;
            alive = __all_sync(0xffffffffu, mbar_wait(bar_s_full(sb), (j / SB) & 1, &abort_word));
            if (!alive) break;
            tc5_fence_after();
            const uint32_t s_addr = tmem + lane_base + sb * BN;

            // nvalid is the same for all rows of a warp (a warp never straddles the two
            // query tiles of a sparse pair); say so, the TMEM accesses below are warp-wide.
            nvalid = __shfl_sync(0xffffffffu, nvalid, 0);
            float mx = -INFINITY;
            if (nvalid >= BN) {
                mx = row_max_full<BN>(s_addr);
            } else if (nvalid > 0) {
                mx = row_max_masked<BN>(s_addr, nvalid);
            }
            const float m_new = fmaxf(m_ref, mx);
            const bool grow = (m_new - m_ref) * p.scale_log2 > RESCALE_LOG2;
            // Every thread observes every phase of pv_done exactly once and in order (phase
            // j-1 during iteration j), so a parity wait can never alias a phase two behind:
            // PV(j) cannot complete before this thread has delivered P(j).
            bool saw_prev_pv = (j == 0);
            if (__any_sync(0xffffffffu, grow)) {
                const float alpha = grow ? fast_exp2((m_ref - m_new) * p.scale_log2) : 1.0f;
                if (grow) m_ref = m_new;
                l *= alpha;
                if (j > 0) {
                    alive = __all_sync(0xffffffffu,
                                       mbar_wait(bar_pv_done, (j - 1) & 1, &abort_word));
                    if (!alive) break;
                    saw_prev_pv = true;
                    tc5_fence_after();
#pragma unroll
                    for (int c = 0; c < HD / 32; c++) {
                        uint32_t v[32];
                        tmem_ld32(tmem + lane_base + O_COL + c * 32, v);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; i++)
                            v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                        tmem_st32(tmem + lane_base + O_COL + c * 32, v);
                    }
                    tmem_wait_st();
                }
            }
            const float neg = (m_ref == -INFINITY) ? 0.0f : -m_ref * p.scale_log2;
            if (nvalid >= BN) {
                l += exp_store_full<BN>(s_addr, s_addr, p.scale_log2, neg);
            } else if (nvalid > 0) {
                l += exp_store_masked<BN>(s_addr, s_addr, p.scale_log2, neg, nvalid);
            } else {
                store_zero_p<BN>(s_addr);  // this half of the pair did not select the tile
            }
            if (!saw_prev_pv) {
                alive = __all_sync(0xffffffffu, mbar_wait(bar_pv_done, (j - 1) & 1, &abort_word));
                if (!alive) break;
            }
            tmem_wait_st();
            tc5_fence_before();
            mbar_arrive(bar_p_full(sb));
        }

        // -------- epilogue: O / l -> bf16, straight to global memory --------
        if (alive && n_tiles > 0) {
            alive = __all_sync(0xffffffffu,
                               mbar_wait(bar_pv_done, (n_tiles - 1) & 1, &abort_word));
        }
        if (SPARSE && alive && n_tiles == 0) {
            // neither query tile selected anything: defined result, zero rows
            const int padded = q_row0 + r;
            if (padded < p.tiles * 64) {
                uint4 *d4 = reinterpret_cast<uint4 *>(p.out + ((size_t)head * p.tiles * 64 + padded) * HD);
#pragma unroll
                for (int i = 0; i < HD / 8; i++) d4[i] = make_uint4(0u, 0u, 0u, 0u);
                if (p.lse) p.lse[(size_t)head * p.tiles * 64 + padded] = INFINITY;
            }
        }
        if (alive && n_tiles > 0) {
            tc5_fence_after();
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;   // a half with an empty list: zero rows
            bool store;
            __nv_bfloat16 *dst;
            if (SPARSE) {
                const int padded = q_row0 + r;
                store = padded < p.tiles * 64;
                dst = p.out + ((size_t)head * p.tiles * 64 + padded) * HD;
                if (store && p.lse)
                    p.lse[(size_t)head * p.tiles * 64 + padded] =
                        (__logf(l) + m_ref * p.scale_log2 * 0.69314718056f) * -11.313708499f;
            } else {
                const int row = q_row0 + r;
                store = row < p.lq;
                dst = p.out + (((size_t)batch * p.lq + row) * p.heads + head) * HD;
                if (store && p.lse)
                    p.lse[((size_t)batch * p.heads + head) * p.lq + row] =
                        m_ref * p.scale + __logf(l);
            }
#pragma unroll
            for (int c = 0; c < HD / 32; c++) {
                uint32_t v[32];
                tmem_ld32(tmem + lane_base + O_COL + c * 32, v);
                tmem_wait_ld();
                if (store) {
                    uint4 *d4 = reinterpret_cast<uint4 *>(dst + c * 32);
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        uint4 w;
                        w.x = pack_bf16(__uint_as_float(v[i * 8 + 0]) * inv,
                                        __uint_as_float(v[i * 8 + 1]) * inv);
                        w.y = pack_bf16(__uint_as_float(v[i * 8 + 2]) * inv,
                                        __uint_as_float(v[i * 8 + 3]) * inv);
                        w.z = pack_bf16(__uint_as_float(v[i * 8 + 4]) * inv,
                                        __uint_as_float(v[i * 8 + 5]) * inv);
                        w.w = pack_bf16(__uint_as_float(v[i * 8 + 6]) * inv,
                                        __uint_as_float(v[i * 8 + 7]) * inv);
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
        // Give copies that may still be in flight time to land before the CTA's
        // shared memory is handed to another CTA.
        if (warp == 4) __nanosleep(1000000);
        __syncthreads();
    }
    if (warp == 5) {
        tc5_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

// -------------------------------- host side ------------------------------------

using EncodeTiled = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                 const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                 const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
    static EncodeTiled fn = [] {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult query;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &query) !=
                cudaSuccess ||
            query != cudaDriverEntryPointSuccess)
            return (EncodeTiled) nullptr;
        return (EncodeTiled)sym;
    }();
    return fn;
}

// Rank-4 bf16 map with a 64-element (128-byte) swizzled inner box.
cudaError_t make_map(CUtensorMap *map, const void *base, const uint64_t dims[4],
                     const uint64_t strides_bytes[3], const uint32_t box[4]) {
    EncodeTiled fn = encode_fn();
    if (!fn) return cudaErrorNotSupported;
    const cuuint32_t ones[4] = {1, 1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(base), dims,
                    strides_bytes, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

template <int BN, bool SPARSE>
cudaError_t launch(const CUtensorMap &mq, const CUtensorMap &mk, const CUtensorMap &mv,
                   const Tc5Params &p, dim3 grid, cudaStream_t stream) {
    auto kernel = attn_tc5_kernel<BN, SPARSE>;
    static thread_local int configured_device = -1;
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    if (configured_device != device) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Tc5Config<BN>::SMEM_BYTES);
        if (e != cudaSuccess) return e;
        configured_device = device;
    }
    kernel<<<grid, TC5_THREADS, Tc5Config<BN>::SMEM_BYTES, stream>>>(mq, mk, mv, p);
    return cudaGetLastError();
}

}  // namespace

cudaError_t attn_dense_tc5(void *out, const void *q, const void *k, const void *v, float *lse,
                           unsigned batch, unsigned lq, unsigned lk, unsigned heads,
                           unsigned kv_heads, float scale, cudaStream_t stream, const PeerOutput *peer) {
    if (!batch || !lq || !lk || !heads || !kv_heads || heads % kv_heads) return cudaErrorInvalidValue;
    if (heads > 65535u || batch > 65535u) return cudaErrorInvalidValue;
    int *status = nullptr;
    cudaError_t e = device_status_word(&status);
    if (e != cudaSuccess) return e;
    CUtensorMap mq, mk, mv;
    const uint32_t box[4] = {64, 1, 128, 1};
    {
        const uint64_t dims[4] = {128, heads, lq, batch};
        const uint64_t strides[3] = {256, (uint64_t)heads * 256, (uint64_t)lq * heads * 256};
        if ((e = make_map(&mq, q, dims, strides, box)) != cudaSuccess) return e;
    }
    {
        const uint64_t dims[4] = {128, kv_heads, lk, batch};
        const uint64_t strides[3] = {256, (uint64_t)kv_heads * 256, (uint64_t)lk * kv_heads * 256};
        if ((e = make_map(&mk, k, dims, strides, box)) != cudaSuccess) return e;
        if ((e = make_map(&mv, v, dims, strides, box)) != cudaSuccess) return e;
    }
    Tc5Params p{};
    p.lq = (int)lq;
    p.lk = (int)lk;
    p.heads = (int)heads;
    p.kv_heads = (int)kv_heads;
    p.scale = scale;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.out = static_cast<__nv_bfloat16 *>(out);
    p.lse = lse;
    p.status = status;
    // A short query block against a long key range (live mode: the text rows of a chunk against
    // the whole KV history, h3_dit_live.inc:95) gives far fewer CTAs than the GPU has SMs, each
    // walking every key. Then the keys are cut into slices that run side by side and a small
    // kernel merges the slices by their logsumexp.
    if (!peer && batch == 1) {
        static thread_local int sms_device = -1, sms = 0;
        int device = 0;
        if ((e = cudaGetDevice(&device)) != cudaSuccess) return e;
        if (device != sms_device) {
            if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess) return e;
            sms_device = device;
        }
        const unsigned ctas = ((lq + 2 * BM - 1) / (2 * BM)) * heads, key_tiles = (lk + 127) / 128;
        if (ctas * 2 <= (unsigned)sms && key_tiles >= 32) {
            unsigned splits = std::min<unsigned>({16u, (unsigned)sms / ctas, key_tiles / 8});
            const unsigned split_tiles = (key_tiles + splits - 1) / splits;
            splits = (key_tiles + split_tiles - 1) / split_tiles;
            if (splits >= 2) {
                // work memory, stream-ordered like the logsumexp buffer of the reference's wrapper
                const size_t part_bytes = (size_t)splits * lq * heads * 256, lse_bytes = (size_t)splits * heads * lq * 4;
                char *work = nullptr;
                if ((e = cudaMallocAsync(reinterpret_cast<void **>(&work), part_bytes + lse_bytes, stream)) != cudaSuccess)
                    return e;
                float *part_lse = reinterpret_cast<float *>(work + part_bytes);
                e = attn_dense_tc5_pair(&mq, &mk, &mv, work, part_lse, 1, lq, lk, heads, kv_heads, scale, status,
                                        stream, nullptr, 0, nullptr, split_tiles);
                if (e == cudaSuccess) e = attn_merge_splits(out, lse, work, part_lse, splits, lq, heads, stream);
                const cudaError_t freed = cudaFreeAsync(work, stream);
                return e != cudaSuccess ? e : freed;
            }
        }
    }
    // More than one query tile: the two-tile-per-CTA kernel (attn_tc5_pair.cu).
    if (lq > (unsigned)BM || peer)
        return attn_dense_tc5_pair(&mq, &mk, &mv, out, lse, batch, lq, lk, heads, kv_heads, scale,
                                   status, stream, peer);
    dim3 grid((lq + BM - 1) / BM, heads, batch);
    return launch<128, false>(mq, mk, mv, p, grid, stream);
}

cudaError_t attn_segments_tc5(void *out, const void *q, const void *const *k, const void *const *v,
                              const unsigned *segment_rows, unsigned segments, unsigned lq,
                              unsigned heads, float scale, cudaStream_t stream) {
    if (!segments || segments > 6u || !lq || !heads || heads > 65535u) return cudaErrorInvalidValue;
    int *status = nullptr;
    cudaError_t e = device_status_word(&status);
    if (e != cudaSuccess) return e;
    CUtensorMap mq, mk[6], mv[6];
    const uint32_t box[4] = {64, 1, 128, 1};
    unsigned total = 0;
    {
        const uint64_t dims[4] = {128, heads, lq, 1};
        const uint64_t strides[3] = {256, (uint64_t)heads * 256, (uint64_t)lq * heads * 256};
        if ((e = make_map(&mq, q, dims, strides, box)) != cudaSuccess) return e;
    }
    for (unsigned s = 0; s < segments; s++) {
        if (!segment_rows[s] || !k[s] || !v[s]) return cudaErrorInvalidValue;
        const uint64_t dims[4] = {128, heads, segment_rows[s], 1};
        const uint64_t strides[3] = {256, (uint64_t)heads * 256, (uint64_t)segment_rows[s] * heads * 256};
        if ((e = make_map(&mk[s], k[s], dims, strides, box)) != cudaSuccess) return e;
        if ((e = make_map(&mv[s], v[s], dims, strides, box)) != cudaSuccess) return e;
        total += segment_rows[s];
    }
    return attn_dense_tc5_pair(&mq, mk, mv, out, nullptr, 1, lq, total, heads, heads, scale, status, stream,
                               nullptr, segments, segment_rows);
}

namespace {
int g_sparse_mode = 0;
}
void attn_sparse_set_mode(int mode) { g_sparse_mode = mode; }

cudaError_t attn_sparse_tc5(void *out, const void *q, const void *k, const void *v, float *lse,
                            const int *indices, const int *counts, const int *sizes,
                            unsigned tiles, unsigned heads, cudaStream_t stream) {
    if (!tiles || !heads || tiles > 4096u || heads > 65535u) return cudaErrorInvalidValue;
    int *status = nullptr;
    cudaError_t e = device_status_word(&status);
    if (e != cudaSuccess) return e;
    CUtensorMap mq, mq64, mk, mv;
    const uint64_t dims[4] = {128, (uint64_t)tiles * 64, heads, 1};
    const uint64_t strides[3] = {256, (uint64_t)tiles * 64 * 256, (uint64_t)heads * tiles * 64 * 256};
    const uint32_t box_q[4] = {64, 128, 1, 1}, box_kv[4] = {64, 64, 1, 1};
    if ((e = make_map(&mq, q, dims, strides, box_q)) != cudaSuccess) return e;
    if ((e = make_map(&mq64, q, dims, strides, box_kv)) != cudaSuccess) return e;
    if ((e = make_map(&mk, k, dims, strides, box_kv)) != cudaSuccess) return e;
    if ((e = make_map(&mv, v, dims, strides, box_kv)) != cudaSuccess) return e;
    Tc5Params p{};
    p.heads = p.kv_heads = (int)heads;
    p.scale = 0.08838834764831845f;  // 1/sqrt(128), fixed by the reference kernel
    p.scale_log2 = p.scale * 1.4426950408889634f;
    p.out = static_cast<__nv_bfloat16 *>(out);
    p.lse = lse;
    p.indices = indices;
    p.counts = counts;
    p.sizes = sizes;
    p.tiles = (int)tiles;
    p.status = status;
    dim3 grid((tiles + 1) / 2, heads, 1);
    const int mode = g_sparse_mode;
    if (mode == 1) return launch<64, true>(mq, mk, mv, p, grid, stream);
    // Work memory of the persistent kernel, stream-ordered like the logsumexp buffer the
    // reference's wrapper allocates per call (cuda/h3_gpu_cuda.cu:1115-1127): one ticket word
    // and two marks per query tile.
    unsigned char *work = nullptr;
    const size_t marks = ((size_t)tiles * heads + 255) / 256 * 256;
    const size_t work_bytes = 256 + 2 * marks;
    if ((e = cudaMallocAsync(reinterpret_cast<void **>(&work), work_bytes, stream)) != cudaSuccess) return e;
    e = cudaMemsetAsync(work, 0, 256, stream);
    if (e == cudaSuccess)
        e = attn_sparse_t_launch(&mq64, &mk, &mv, out, lse, indices, counts, sizes, tiles, heads,
                                 reinterpret_cast<unsigned *>(work), work + 256, work + 256 + marks,
                                 mode == 0 ? -1 : 0, mode == 2, status, stream);
    if (e == cudaSuccess) {
        // marked tiles (row sums outside the safe exponent range) are recomputed with per-row maxima
        p.redo = work + 256;
        e = launch<64, true>(mq, mk, mv, p, grid, stream);
    }
    const cudaError_t freed = cudaFreeAsync(work, stream);
    return e != cudaSuccess ? e : freed;
}

}  // namespace h3b
