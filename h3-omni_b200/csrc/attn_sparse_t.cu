// Block-sparse attention forward for video sparse attention (tcgen05 + TMEM + TMA), bf16, head
// dim 128: the fine stage behind h3_vsa_hopper (replaces fwd_attend_ker<128>,
// cuda/vendor/vsa_hopper_forward.cuh:68-270 of the reference).
//
// A 64-row query tile would halve the tensor rate if it sat on the M axis of the MMA (M = 64),
// and pairing two query tiles to reach M = 128 forces both to walk the union of their lists.
// So the roles are swapped: the KEYS sit on the M axis. One step of one query tile takes two
// KV tiles of its own list (128 key rows) and computes
//      S^T[128 keys x 64 queries] = K . Q^T         (A = K pair, B = Q tile, both from smem)
//      O^T[128 dims x 64 queries] += V^T . P^T      (A = V pair, MN-major; B = P^T from smem)
// Every MMA is M = 128, N = 64, K = 128 and every multiply-add belongs to a selected
// (query tile, KV tile) pair; nothing is computed for tiles a query tile did not select.
//
// Softmax with the keys on TMEM lanes: a thread owns one key row and sees 64 scores, one per
// query. Per-query maxima would need a cross-lane reduction per step, so the exponent
// reference is ONE value per query tile, the largest score of the tile's first step; any
// reference gives the exact softmax as long as nothing over- or underflows, and the row sums
// l[q] are kept per thread and reduced once per query tile. A query row whose sum leaves
// [2^-60, 2^100) (or is not finite) marks its tile in `redo`, and the launcher then
// recomputes marked tiles with the per-row online-softmax kernel of attn_tc5.cu. With
// attention logits inside about [-28, +69] nats of the first step's maximum nothing is marked.
//
// Persistent kernel, one CTA per SM, 16 warps:
//   warps 0-3 / 4-7 : softmax groups; group g takes the steps whose global number is g mod 2
//   warp 8          : TMA issue (Q tile per item; K pairs and V pairs in two rings of two slots)
//   warp 9 / 11     : MMA issue of the QK products / of the PV products (one thread cannot issue
//                     sixteen N = 64 MMAs per step and do the waits in the time the pipe needs)
//   warp 10         : scheduler: takes a ticket (head, query tile), checks and stages its list
//   warps 12-15     : epilogue: O^T / l -> bf16 rows in global memory, while the next item runs
// Items are double-buffered (Q, list, O^T accumulator), so consecutive query tiles overlap.
// Every wait is bounded and ends in the device status word.
#include <cuda.h>

#include "attn_kernels.h"
#include "sm100_ptx.cuh"

namespace h3b {
namespace {

constexpr int ST_THREADS = 512;
constexpr int ST_RING = 4;
constexpr int ST_SLOT = 128 * 128 * 2;     // K pair or V pair: two 64-dim halves of [128 rows][128 B]
constexpr int ST_HALF = 128 * 128;         // one half
constexpr int ST_TILE = 64 * 128;          // one 64-row tile inside a half
constexpr int ST_Q = 64 * 128 * 2;         // query tile: two halves of [64 rows][128 B]
constexpr int ST_QHALF = 64 * 128;
constexpr int ST_P = 128 * 64 * 2;         // P^T: [128 key rows][64 queries] bf16
constexpr int ST_MAX_STEPS = 2048;
constexpr int ST_OFF_Q = 0;
constexpr int ST_OFF_RING = ST_OFF_Q + 2 * ST_Q;
constexpr int ST_OFF_P = ST_OFF_RING + ST_RING * ST_SLOT;
constexpr int ST_OFF_PAIRS = ST_OFF_P + 2 * ST_P;
constexpr int ST_OFF_VALID = ST_OFF_PAIRS + 2 * ST_MAX_STEPS * 4;
constexpr int ST_OFF_LPART = ST_OFF_VALID + 2 * ST_MAX_STEPS * 2;
constexpr int ST_SMEM = ST_OFF_LPART + 2 * 8 * 64 * 4 + 1024;
constexpr int ST_S_COL = 0, ST_O_COL = 128;   // TMEM: S^T[2] at 0 / 64, O^T[2] at 128 / 192
constexpr int ST_TMEM_COLS = 256;
constexpr int ENC_NEG_INF = (int)0x807fffffu;   // encode(-inf)

#ifdef H3B_TRACE
// Development aid, compiled only with -DH3B_TRACE: cycle counters of CTA 0.
__device__ long long g_sparse_trace[64];
#define TR_DECL long long tr_acc[8] = {}; const long long tr_begin = clock64()
#define TR_T0 const long long tr_t0 = clock64()
#define TR_ADD(slot) tr_acc[slot] += clock64() - tr_t0
#define TR_OUT(base, n) if (blockIdx.x == 0) { g_sparse_trace[base] = clock64() - tr_begin; for (int x = 0; x < n; x++) g_sparse_trace[base + 1 + x] = tr_acc[x]; }
#else
#define TR_DECL
#define TR_T0
#define TR_ADD(slot)
#define TR_OUT(base, n)
#endif

struct SparseTParams {
    const int *indices, *counts, *sizes;
    __nv_bfloat16 *out;
    float *lse;
    unsigned *ticket;          // zero at launch
    unsigned char *redo;       // [heads][tiles], written for every item this kernel computes
    const unsigned char *elsewhere;   // [heads][tiles]: tiles left to the pair-walk kernel (skipped here)
    int *status;
    int tiles, heads, force_redo;
    float scale_log2;
};

struct Item {
    int head, qt, n, count;    // n = steps (pairs of KV tiles); n < 0: no more work
};

// Order-preserving int image of a float (so the maximum can be taken with integer atomics).
__device__ __forceinline__ int encode_ordered(float f) {
    const int b = __float_as_int(f);
    return b >= 0 ? b : b ^ 0x7fffffff;
}
__device__ __forceinline__ float decode_ordered(int e) {
    return __int_as_float(e >= 0 ? e : e ^ 0x7fffffff);
}
__device__ __forceinline__ void fence_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
// Instruction descriptor with both operand majors selectable (kind::f16, bf16 in, f32 out).
__host__ __device__ constexpr uint32_t idesc_bf16(uint32_t m, uint32_t n, uint32_t a_mn, uint32_t b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (a_mn << 15) | (b_mn << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// p = exp2(s * c + neg) for 32 queries of this thread's key row; the sums go to l2[0..15]
// (pairs of adjacent queries), the bf16 pairs to four 16-byte swizzled stores.
template <int HALF>
__device__ __forceinline__ void exp_half_row(const uint32_t (&s)[32], float2 (&l2)[32], float2 c2, float2 neg2,
                                             uint32_t row_addr, int row) {
#pragma unroll
    for (int c = 0; c < 4; c++) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int e = c * 8 + i * 2;
            const float2 x = __ffma2_rn(make_float2(__uint_as_float(s[e]), __uint_as_float(s[e + 1])), c2, neg2);
            w[i] = pack_bf16(fast_exp2(x.x), fast_exp2(x.y));
            // the row sums add the rounded weights, the ones the PV product really uses, so that
            // numerator and denominator agree (a row with a single key comes out exact)
            const float2 p = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
            l2[HALF * 16 + c * 4 + i] = __fadd2_rn(l2[HALF * 16 + c * 4 + i], p);
        }
        st_shared_v4(row_addr + (((HALF * 4 + c) ^ (row & 7)) << 4), w[0], w[1], w[2], w[3]);
    }
}

__global__ void __launch_bounds__(ST_THREADS, 1)
attn_sparse_t_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, const SparseTParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bars[26];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_word;
    __shared__ Item desc[2];
    __shared__ int mref[2];
    __shared__ float linv[64];
    __shared__ int bad_rows[2];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *const base_ptr = smem_raw + (base - smem_u32(smem_raw));
    uint32_t *const pairs = reinterpret_cast<uint32_t *>(base_ptr + ST_OFF_PAIRS);     // [2][MAX_STEPS]
    uint16_t *const valid = reinterpret_cast<uint16_t *>(base_ptr + ST_OFF_VALID);    // [2][MAX_STEPS]
    float *const lpart = reinterpret_cast<float *>(base_ptr + ST_OFF_LPART);          // [2][8][64]

    const uint32_t bar0 = smem_u32(bars);
    auto bar_item_ready = [&](int b) { return bar0 + 8u * (0 + b); };
    auto bar_item_free = [&](int b) { return bar0 + 8u * (2 + b); };
    auto bar_item_done = [&](int b) { return bar0 + 8u * (4 + b); };
    auto bar_q_full = [&](int b) { return bar0 + 8u * (6 + b); };
    auto bar_k_full = [&](int s) { return bar0 + 8u * (8 + s); };
    auto bar_v_full = [&](int s) { return bar0 + 8u * (10 + s); };
    auto bar_k_empty = [&](int s) { return bar0 + 8u * (12 + s); };
    auto bar_v_empty = [&](int s) { return bar0 + 8u * (14 + s); };
    auto bar_pv_done = [&](int k) { return bar0 + 8u * (23 + k); };
    auto bar_s_full = [&](int k) { return bar0 + 8u * (16 + k); };
    auto bar_p_full = [&](int k) { return bar0 + 8u * (18 + k); };
    auto bar_mref = [&](int b) { return bar0 + 8u * (20 + b); };
    const uint32_t bar_epi = bar0 + 8u * 22;

    if (tid == 0) {
        for (int b = 0; b < 2; b++) {
            mbar_init(bar_item_ready(b), 1);
            mbar_init(bar_item_free(b), 4);     // the four epilogue warps
            mbar_init(bar_item_done(b), 9);     // last PV (or the MMA thread itself) + eight softmax warps
            mbar_init(bar_q_full(b), 1);
            mbar_init(bar_s_full(b), 1);
            mbar_init(bar_p_full(b), 128);
            mbar_init(bar_mref(b), 4);
            mref[b] = ENC_NEG_INF;
        }
        mbar_init(bar_epi, 128);            // the epilogue warps among themselves
        for (int s = 0; s < 2; s++) {
            mbar_init(bar_k_full(s), 1);
            mbar_init(bar_v_full(s), 1);
            mbar_init(bar_k_empty(s), 1);
            mbar_init(bar_v_empty(s), 1);
            mbar_init(bar_pv_done(s), 1);
        }
        mbar_fence_init();
        abort_word = 0;
    }
    if (warp == 9) {
        tmem_alloc(smem_u32(&tmem_slot), ST_TMEM_COLS);
        tmem_relinquish();
    }
    tc5_fence_before();
    __syncthreads();
    tc5_fence_after();
    const uint32_t tmem = tmem_slot;
    const int total_items = p.tiles * p.heads;

    // Reads item `i`'s descriptor (waits until the scheduler has published it).
    auto fetch = [&](int i, Item &it) -> bool {
        if (!mbar_wait(bar_item_ready(i & 1), (i >> 1) & 1, &abort_word)) return false;
        it = desc[i & 1];
        return true;
    };
    // The same for a whole warp: lane 0 polls (fewer probes of shared memory, which the tensor
    // core is reading its operands from).
    auto fetch_warp = [&](int i, Item &it) -> bool {
        if (!mbar_wait_uniform(bar_item_ready(i & 1), (i >> 1) & 1, &abort_word)) return false;
        it = desc[i & 1];
        return true;
    };
    // the last step of an odd list holds one KV tile only
    auto single = [](const Item &it, int j) { return j == it.n - 1 && (it.count & 1); };

    if (warp >= 8 && warp < 12) {
        warpgroup_reg_dec<80>();
        if (warp == 10) {
            // ------------------------------ scheduler ------------------------------
            for (int i = 0;; i++) {
                const int b = i & 1;
                bool ok = true;
                if (i >= 2) ok = mbar_wait_warp(bar_item_free(b), ((i >> 1) - 1) & 1, &abort_word);
                if (!ok) break;
                unsigned ticket = 0;
                if (lane == 0) ticket = atomicAdd(p.ticket, 1u);
                ticket = __shfl_sync(0xffffffffu, ticket, 0);
                if (ticket >= (unsigned)total_items) {
                    if (lane == 0) {
                        desc[b] = Item{0, 0, -1, 0};
                        mbar_arrive(bar_item_ready(b));
                    }
                    break;
                }
                const int head = (int)ticket / p.tiles, qt = (int)ticket % p.tiles;
                const size_t row = (size_t)head * p.tiles + qt;
                if (p.elsewhere[row]) {   // this tile's pair goes to the pair-walk kernel
                    i--;
                    continue;
                }
                int count = p.counts[row];
                bool bad = count < 0 || count > p.tiles;
                count = max(0, min(count, p.tiles));
                const int n = (count + 1) >> 1;
                const int *list = p.indices + row * p.tiles;
                for (int s0 = 0; s0 < n; s0 += 32) {
                    const int s = s0 + lane;
                    if (s < n) {
                        int kx = list[2 * s], ky = 2 * s + 1 < count ? list[2 * s + 1] : -1;
                        int nx = 0, ny = 0;
                        if (kx < 0 || kx >= p.tiles) {
                            bad = true;
                            kx = 0;
                        } else {
                            nx = max(0, min(p.sizes[kx], 64));
                        }
                        if (ky >= p.tiles || (ky < 0 && 2 * s + 1 < count)) {
                            bad = true;
                            ky = 0;
                        } else if (ky >= 0) {
                            ny = max(0, min(p.sizes[ky], 64));
                        } else {
                            ky = 0;
                        }
                        pairs[b * ST_MAX_STEPS + s] = (uint32_t)kx | ((uint32_t)ky << 16);
                        valid[b * ST_MAX_STEPS + s] = (uint16_t)(nx | (ny << 8));
                    }
                }
                if (__any_sync(0xffffffffu, bad) && lane == 0)
                    atomicCAS(p.status, STATUS_OK, STATUS_BAD_ARGUMENT);   // refused entries count as masked tiles
                __syncwarp();
                if (lane == 0) {
                    desc[b] = Item{head, qt, n, count};
                    mbar_arrive(bar_item_ready(b));
                }
            }
        } else if (warp == 8 && lane == 0) {
            // ------------------------------ TMA issue ------------------------------
            // One thread feeds both rings. It never blocks on one ring while the other could
            // move: K loads may run ahead of V loads, but at most one item ahead, because the
            // scheduler can publish item i + 2 only after item i is finished, V loads included.
            tma_prefetch_desc(&map_q);
            tma_prefetch_desc(&map_k);
            tma_prefetch_desc(&map_v);
            TR_DECL;
            struct Cursor {
                Item it;
                int item, j, g;
                bool end;
            };
            Cursor kc{Item{0, 0, 0, 0}, -1, 0, 0, false}, vc{Item{0, 0, 0, 0}, -1, 0, 0, false};
            auto try_next_item = [&](Cursor &c, bool is_k) -> bool {   // true: the cursor moved
                const int next = c.item + 1;
                if (is_k && next > vc.item + 1 && !vc.end) return false;
                if (!mbar_try_wait(bar_item_ready(next & 1), (next >> 1) & 1)) return false;
                c.it = desc[next & 1];
                c.item = next;
                c.j = 0;
                if (c.it.n < 0) {
                    c.end = true;
                } else if (is_k && c.it.n > 0) {
                    const int b = next & 1;
                    const uint32_t dst = base + ST_OFF_Q + b * ST_Q;
                    mbar_arrive_expect_tx(bar_q_full(b), ST_Q);
                    tma_load_4d(dst, &map_q, bar_q_full(b), 0, c.it.qt * 64, c.it.head, 0);
                    tma_load_4d(dst + ST_QHALF, &map_q, bar_q_full(b), 64, c.it.qt * 64, c.it.head, 0);
                }
                return true;
            };
            auto try_load = [&](Cursor &c, const void *map, uint32_t ring, uint32_t full0, uint32_t empty0) -> bool {
                const int slot = c.g & 1, use = c.g >> 1;
                if (use > 0 && !mbar_try_wait(empty0 + 8u * slot, (use - 1) & 1)) return false;
                const uint32_t word = pairs[(c.item & 1) * ST_MAX_STEPS + c.j];
                const int kt[2] = {(int)(word & 0xffffu), (int)(word >> 16)};
                const int count = single(c.it, c.j) ? 1 : 2;
                const uint32_t dst = ring + slot * ST_SLOT, bar = full0 + 8u * slot;
                mbar_arrive_expect_tx(bar, count * 2 * ST_TILE);
                for (int t = 0; t < count; t++)
                    for (int h = 0; h < 2; h++)
                        tma_load_4d(dst + h * ST_HALF + t * ST_TILE, map, bar, 64 * h, kt[t] * 64, c.it.head, 0);
                c.g++;
                c.j++;
                return true;
            };
            unsigned long long idle_since = 0;
            while (!(kc.end && vc.end)) {
                bool moved = false;
                if (!kc.end) {
                    if (kc.j >= kc.it.n) moved |= try_next_item(kc, true);
                    else moved |= try_load(kc, &map_k, base + ST_OFF_RING, bar_k_full(0), bar_k_empty(0));
                }
                if (!vc.end) {
                    if (vc.j >= vc.it.n) moved |= try_next_item(vc, false);
                    else moved |= try_load(vc, &map_v, base + ST_OFF_RING + 2 * ST_SLOT, bar_v_full(0), bar_v_empty(0));
                }
                if (moved) {
                    idle_since = 0;
                } else {
                    // bounded like every other wait in this kernel
                    if (abort_word) break;
                    const unsigned long long now = global_timer_ns();
                    if (!idle_since) idle_since = now;
                    if (now - idle_since > WAIT_LIMIT_NS) {
                        abort_word = 1;
                        break;
                    }
                }
            }
            TR_OUT(0, 1);
        } else if (warp == 9) {
            // ------------------------------ QK issue: S^T[g & 1] = K pair . Q^T ------------------------------
            // The whole warp walks the loop and one elected lane issues: inside a one-lane branch
            // every descriptor word would be per-thread data that has to be moved to a uniform
            // register in front of each MMA.
            const bool leader = elect_one();
            constexpr uint32_t idesc_qk = idesc_bf16(128, 64, 0, 0);
            const uint64_t q_proto = smem_desc_sw128(base + ST_OFF_Q, 16, 1024);
            const uint64_t k_proto = smem_desc_sw128(base + ST_OFF_RING, 16, 1024);
            const uint32_t q_lo0 = (uint32_t)q_proto, q_hi = (uint32_t)(q_proto >> 32);
            const uint32_t k_lo0 = (uint32_t)k_proto, k_hi = (uint32_t)(k_proto >> 32);
            int g = 0, q_uses0 = 0, q_uses1 = 0;
            TR_DECL;
            for (int i = 0;; i++) {
                Item it;
                if (!fetch_warp(i, it) || it.n < 0) break;
                if (it.n == 0) continue;
                int &uses = (i & 1) ? q_uses1 : q_uses0;   // only items with a list load a query tile
                if (!mbar_wait_converged(bar_q_full(i & 1), (uses++) & 1, &abort_word)) break;
                const uint32_t b_lo = q_lo0 + (i & 1) * (ST_Q >> 4);
                bool ok = true;
                for (int j = 0; j < it.n; j++, g++) {
                    const int slot = g & 1;
                    {
                        TR_T0;
                        ok = mbar_wait_converged(bar_k_full(slot), (g >> 1) & 1, &abort_word) &&
                             // the softmax group has finished reading S^T of step g - 2
                             (g < 2 || mbar_wait_converged(bar_p_full(slot), ((g - 2) >> 1) & 1, &abort_word));
                        TR_ADD(0);
                    }
                    if (!ok) break;
                    TR_T0;
                    tc5_fence_after();
                    const uint32_t a_lo = k_lo0 + slot * (ST_SLOT >> 4), d_tmem = tmem + ST_S_COL + slot * 64;
                    if (leader) {
#pragma unroll
                        for (int kk = 0; kk < 8; kk++)
                            mma_ss_words(d_tmem, a_lo + (kk / 4) * (ST_HALF >> 4) + (kk % 4) * 2, k_hi,
                                         b_lo + (kk / 4) * (ST_QHALF >> 4) + (kk % 4) * 2, q_hi, idesc_qk, kk > 0);
                        mma_commit(bar_s_full(slot));
                        mma_commit(bar_k_empty(slot));
                    }
                    __syncwarp();
                    TR_ADD(1);
                }
                if (!ok) break;
            }
#ifdef H3B_TRACE
            tr_acc[2] = g;
#endif
            if (lane == 0) TR_OUT(8, 3);
        } else if (warp == 11) {
            // ------------------------------ PV issue: O^T[item & 1] += V pair^T . P^T[g & 1] ------------------------------
            const bool leader = elect_one();
            constexpr uint32_t idesc_pv = idesc_bf16(128, 64, 1, 1);
            const uint64_t v_proto = smem_desc_sw128(base + ST_OFF_RING + 2 * ST_SLOT, ST_HALF, 1024);
            const uint64_t p_proto = smem_desc_sw128(base + ST_OFF_P, ST_P, 1024);
            const uint32_t v_lo0 = (uint32_t)v_proto, v_hi = (uint32_t)(v_proto >> 32);
            const uint32_t p_lo0 = (uint32_t)p_proto, p_hi = (uint32_t)(p_proto >> 32);
            int g = 0;
            TR_DECL;
            for (int i = 0;; i++) {
                Item it;
                const int b = i & 1;
                if (!fetch_warp(i, it) || it.n < 0) break;
                // the accumulator (and the item_done phase) of item i - 2 must have been consumed
                if (i >= 2 && !mbar_wait_converged(bar_item_free(b), ((i >> 1) - 1) & 1, &abort_word)) break;
                if (it.n == 0) {   // empty list: nothing to multiply; the epilogue writes zero rows
                    if (leader) mbar_arrive(bar_item_done(b));
                    __syncwarp();
                    continue;
                }
                const uint32_t d_tmem = tmem + ST_O_COL + b * 64;
                bool ok = true;
                for (int j = 0; j < it.n; j++, g++) {
                    const int slot = g & 1;
                    {
                        TR_T0;
                        ok = mbar_wait_converged(bar_v_full(slot), (g >> 1) & 1, &abort_word) &&
                             mbar_wait_converged(bar_p_full(slot), (g >> 1) & 1, &abort_word);
                        TR_ADD(0);
                    }
                    if (!ok) break;
                    TR_T0;
                    tc5_fence_after();
                    const uint32_t a_lo = v_lo0 + slot * (ST_SLOT >> 4), b_lo = p_lo0 + slot * (ST_P >> 4);
                    if (leader) {
                        mma_ss_words(d_tmem, a_lo, v_hi, b_lo, p_hi, idesc_pv, j > 0);
#pragma unroll
                        for (int kk = 1; kk < 4; kk++)
                            mma_ss_words(d_tmem, a_lo + kk * (2048 >> 4), v_hi, b_lo + kk * (2048 >> 4), p_hi, idesc_pv, 1);
                        if (!single(it, j)) {   // never multiply rows of a tile that was not loaded
#pragma unroll
                            for (int kk = 4; kk < 8; kk++)
                                mma_ss_words(d_tmem, a_lo + kk * (2048 >> 4), v_hi, b_lo + kk * (2048 >> 4), p_hi,
                                             idesc_pv, 1);
                        }
                        mma_commit(bar_v_empty(slot));
                        mma_commit(bar_pv_done(slot));
                    }
                    __syncwarp();
                    TR_ADD(1);
                }
                if (!ok) break;
                if (leader) mma_commit(bar_item_done(b));
                __syncwarp();
            }
            if (lane == 0) TR_OUT(12, 2);
        }
    } else if (warp >= 12) {
        warpgroup_reg_dec<64>();
        // ------------------------------ epilogue ------------------------------
        const int d = tid - 384;   // head dimension this thread owns == TMEM lane
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        int epi_phase = 0;
        for (int i = 0;; i++) {
            const int b = i & 1;
            Item it;
            if (!fetch_warp(i, it) || it.n < 0) break;
            if (!mbar_wait_uniform(bar_item_done(b), (i >> 1) & 1, &abort_word)) break;
            tc5_fence_after();
            const float m_log2 = (mref[b] == ENC_NEG_INF ? 0.0f : decode_ordered(mref[b])) * p.scale_log2;
            const size_t out_row0 = ((size_t)it.head * p.tiles + it.qt) * 64;
            if (d < 64) {
                float l = 0.0f;
#pragma unroll
                for (int w = 0; w < 8; w++) l += lpart[(b * 8 + w) * 64 + d];
                const int real = max(0, min(p.sizes[it.qt], 64));
                // NaN, infinity, overflow and underflow of a real query row all fail this test
                const bool bad = it.n > 0 && d < real && !(l >= 0x1p-60f && l < 0x1p100f);
                const bool warp_bad = __any_sync(0xffffffffu, bad);
                if (lane == 0) bad_rows[warp - 12] = warp_bad ? 1 : 0;
                linv[d] = l > 0.0f ? 1.0f / l : 0.0f;
                if (p.lse) p.lse[out_row0 + d] = (__logf(l) + m_log2 * 0.69314718056f) * -11.313708499f;
            }
            // linv and bad_rows complete (an mbarrier, not bar.sync: a wait here must stay bounded)
            mbar_arrive(bar_epi);
            if (!mbar_wait_uniform(bar_epi, (epi_phase++) & 1, &abort_word)) break;
            if (d == 0) p.redo[(size_t)it.head * p.tiles + it.qt] = (bad_rows[0] | bad_rows[1] | p.force_redo) ? 1 : 0;
            __nv_bfloat16 *dst = p.out + out_row0 * 128 + d;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                uint32_t v[16];
                if (it.n > 0) {
                    tmem_ld16(tmem + lane_base + ST_O_COL + b * 64 + c * 16, v);
                    tmem_wait_ld();
                }
#pragma unroll
                for (int q = 0; q < 16; q++) {
                    const float o = it.n > 0 ? __uint_as_float(v[q]) * linv[c * 16 + q] : 0.0f;
                    dst[(size_t)(c * 16 + q) * 128] = __float2bfloat16_rn(o);
                }
            }
            tc5_fence_before();
            mbar_arrive(bar_epi);   // every thread is done with linv, bad_rows, lpart, mref and O^T[b]
            if (!mbar_wait_uniform(bar_epi, (epi_phase++) & 1, &abort_word)) break;
            if (d == 0) mref[b] = ENC_NEG_INF;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_item_free(b));
        }
    } else {
        warpgroup_reg_inc<184>();
        // ------------------------------ softmax ------------------------------
        const int k = warp >> 2;                       // this group takes global steps g with g % 2 == k
        const int row = tid & 127;                     // key row of the pair == TMEM lane
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        const uint32_t s_addr = tmem + lane_base + ST_S_COL + k * 64;
        const uint32_t p_row = base + ST_OFF_P + k * ST_P + row * 128;
        const float2 c2 = make_float2(p.scale_log2, p.scale_log2);
        float2 l2[32];
#pragma unroll
        for (int i = 0; i < 32; i++) l2[i] = make_float2(0.f, 0.f);
        int G = 0;   // global number of the current item's first step
        int ref_uses0 = 0, ref_uses1 = 0;   // items with a list seen so far, per buffer
        bool alive = true;
        TR_DECL;
        for (int i = 0; alive; i++) {
            const int b = i & 1;
            Item it;
            if (!fetch(i, it) || it.n < 0) break;
            float neg = 0.0f;
            bool have_ref = false;
            for (int j = (G & 1) == k ? 0 : 1; j < it.n; j += 2) {
                const int g = G + j;
                {
                    TR_T0;
                    alive = __all_sync(0xffffffffu, mbar_wait(bar_s_full(k), (g >> 1) & 1, &abort_word));
                    TR_ADD(0);
                }
                if (!alive) break;
                TR_T0;
                tc5_fence_after();
                uint32_t s0[32], s1[32];
                tmem_ld32(s_addr, s0);
                tmem_ld32(s_addr + 32, s1);
                tmem_wait_ld();
                const unsigned vw = valid[b * ST_MAX_STEPS + j];
                const int rows_here = row < 64 ? (int)(vw & 0xffu) : (int)(vw >> 8);
                const bool live = (row & 63) < rows_here;
                if (j == 0) {
                    // the tile's exponent reference: the largest score of its first step
                    float m = -INFINITY;
                    if (live) {
#pragma unroll
                        for (int e = 0; e < 32; e++)
                            m = fmaxf(m, fmaxf(__uint_as_float(s0[e]), __uint_as_float(s1[e])));
                    }
                    const int warp_max = __reduce_max_sync(0xffffffffu, encode_ordered(m));
                    if (lane == 0) {
                        atomicMax(&mref[b], warp_max);
                        mbar_arrive(bar_mref(b));
                    }
                }
                if (!have_ref) {
                    alive = __all_sync(0xffffffffu, mbar_wait(bar_mref(b), (b ? ref_uses1 : ref_uses0) & 1, &abort_word));
                    if (!alive) break;
                    const int e = *reinterpret_cast<volatile int *>(&mref[b]);
                    neg = e == ENC_NEG_INF ? 0.0f : -decode_ordered(e) * p.scale_log2;
                    have_ref = true;
                }
                // P^T[k] was last read by the PV product of step g - 2
                if (g >= 2) {
                    alive = __all_sync(0xffffffffu, mbar_wait(bar_pv_done(k), ((g - 2) >> 1) & 1, &abort_word));
                    if (!alive) break;
                }
                if (live) {
                    const float2 neg2 = make_float2(neg, neg);
                    exp_half_row<0>(s0, l2, c2, neg2, p_row, row);
                    exp_half_row<1>(s1, l2, c2, neg2, p_row, row);
                } else {
#pragma unroll
                    for (int c = 0; c < 8; c++) st_shared_v4(p_row + (c << 4), 0u, 0u, 0u, 0u);
                }
                tc5_fence_before();
                fence_async_smem();
                mbar_arrive(bar_p_full(k));
                TR_ADD(1);
            }
            if (!alive) break;
            TR_T0;
            // ---- item end: this warp's row sums, reduced over its 32 key rows in a fixed order ----
            if (i >= 2) {
                alive = __all_sync(0xffffffffu, mbar_wait(bar_item_free(b), ((i >> 1) - 1) & 1, &abort_word));
                if (!alive) break;
            }
            {
                auto l = [&](int x) { return (x & 1) ? l2[x >> 1].y : l2[x >> 1].x; };
                float a[32], bb[16], cc[8], dd[4], ee[2];
                const bool u16 = lane & 16, u8 = lane & 8, u4 = lane & 4, u2 = lane & 2, u1 = lane & 1;
#pragma unroll
                for (int x = 0; x < 32; x++) {
                    const float lo = l(x), hi = l(x + 32);
                    a[x] = (u16 ? hi : lo) + __shfl_xor_sync(0xffffffffu, u16 ? lo : hi, 16);
                }
#pragma unroll
                for (int x = 0; x < 16; x++) {
                    const float lo = a[x], hi = a[x + 16];
                    bb[x] = (u8 ? hi : lo) + __shfl_xor_sync(0xffffffffu, u8 ? lo : hi, 8);
                }
#pragma unroll
                for (int x = 0; x < 8; x++) {
                    const float lo = bb[x], hi = bb[x + 8];
                    cc[x] = (u4 ? hi : lo) + __shfl_xor_sync(0xffffffffu, u4 ? lo : hi, 4);
                }
#pragma unroll
                for (int x = 0; x < 4; x++) {
                    const float lo = cc[x], hi = cc[x + 4];
                    dd[x] = (u2 ? hi : lo) + __shfl_xor_sync(0xffffffffu, u2 ? lo : hi, 2);
                }
#pragma unroll
                for (int x = 0; x < 2; x++) {
                    const float lo = dd[x], hi = dd[x + 2];
                    ee[x] = (u1 ? hi : lo) + __shfl_xor_sync(0xffffffffu, u1 ? lo : hi, 1);
                }
                const int col = (u16 ? 32 : 0) + (u8 ? 16 : 0) + (u4 ? 8 : 0) + (u2 ? 4 : 0) + (u1 ? 2 : 0);
                // The partial sums are filed by the parity of the item's OWN step numbers (this group
                // took the even or the odd ones), not by the group's number: which group gets an
                // item's first step depends on what the CTA computed before, and the epilogue's
                // summation order - hence the result's last bit - must not.
                float *mine = lpart + (b * 8 + ((k ^ (G & 1)) * 4 + (warp & 3))) * 64;
                mine[col] = ee[0];
                mine[col + 1] = ee[1];
#pragma unroll
                for (int x = 0; x < 32; x++) l2[x] = make_float2(0.f, 0.f);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_item_done(b));
            G += it.n;
            if (it.n > 0) (b ? ref_uses1 : ref_uses0)++;
            TR_ADD(2);
        }
        if ((tid & 127) == 0) TR_OUT(16 + 8 * k, 3);
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
        tmem_dealloc(tmem, ST_TMEM_COLS);
    }
}

// Which kernel takes which pair of adjacent query tiles. The pair-walk kernel multiplies both
// tiles by every KV tile of the UNION of their lists with M = 128 MMAs that read less shared
// memory per multiply-add; this kernel multiplies each tile by its own list only. Measured cost:
// about 990 cycles per union tile there, 692 cycles per list entry here, so a pair goes to the
// pair walk when |A u B| < 0.7 (|A| + |B|) - lists that mostly coincide, as neighbouring cubes of
// real video tend to produce - and stays here otherwise (also when the union is longer than 256
// tiles). One warp per pair; both lists ascending.
__global__ void __launch_bounds__(256)
pair_choice_kernel(const int *__restrict__ indices, const int *__restrict__ counts, unsigned char *elsewhere,
                   unsigned char *redo, int tiles, int heads, int force) {
    __shared__ uint32_t bits[8][128];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pairs = (tiles + 1) / 2;
    const int pair = blockIdx.x * 8 + warp, head = blockIdx.y;
    if (pair >= pairs) return;
    const int qa = 2 * pair, qb = qa + 1;
    const size_t row = (size_t)head * tiles + qa;
    int choice = 0;
    if (force >= 0) {
        choice = force;
    } else if (qb < tiles) {
        const int na = max(0, min(counts[row], tiles)), nb = max(0, min(counts[row + 1], tiles));
        for (int w = lane; w < 128; w += 32) bits[warp][w] = 0u;
        __syncwarp();
        for (int i = lane; i < na; i += 32) {
            const int kt = indices[row * tiles + i];
            if (kt >= 0 && kt < tiles) atomicOr(&bits[warp][kt >> 5], 1u << (kt & 31));
        }
        __syncwarp();
        int common = 0;
        for (int i = lane; i < nb; i += 32) {
            const int kt = indices[(row + 1) * tiles + i];
            if (kt >= 0 && kt < tiles) common += (bits[warp][kt >> 5] >> (kt & 31)) & 1u;
        }
        common = __reduce_add_sync(0xffffffffu, common);
        // Long lists stay with the persistent kernel whatever their overlap: there they are one
        // ticket among thousands, while a pair-walk CTA walks its whole union alone (the prefix
        // tiles of a video - every query tile attends all 905 KV tiles - would leave 96 CTAs
        // running for a millisecond after everything else has finished).
        const int joined = na + nb - common;
        choice = (10 * joined < 7 * (na + nb) && joined <= 256) ? 1 : 0;
    }
    if (lane == 0) {
        elsewhere[row] = redo[row] = (unsigned char)choice;
        if (qb < tiles) elsewhere[row + 1] = redo[row + 1] = (unsigned char)choice;
    }
}

}  // namespace

#ifdef H3B_TRACE
extern "C" cudaError_t h3b_debug_sparse_trace(long long *host64) {
    return cudaMemcpyFromSymbol(host64, g_sparse_trace, sizeof(long long) * 64);
}
#endif

cudaError_t attn_sparse_t_launch(const CUtensorMap_st *mq, const CUtensorMap_st *mk, const CUtensorMap_st *mv,
                                 void *out, float *lse, const int *indices, const int *counts, const int *sizes,
                                 unsigned tiles, unsigned heads, unsigned *ticket, unsigned char *redo,
                                 unsigned char *elsewhere, int assign, bool force_redo, int *status,
                                 cudaStream_t stream) {
    static thread_local int configured_device = -1, sms = 0;
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    if (configured_device != device) {
        e = cudaFuncSetAttribute(attn_sparse_t_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ST_SMEM);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (e != cudaSuccess) return e;
        configured_device = device;
    }
    SparseTParams p{};
    p.indices = indices;
    p.counts = counts;
    p.sizes = sizes;
    p.out = static_cast<__nv_bfloat16 *>(out);
    p.lse = lse;
    p.ticket = ticket;
    p.redo = redo;
    p.elsewhere = elsewhere;
    p.status = status;
    p.tiles = (int)tiles;
    p.heads = (int)heads;
    p.force_redo = force_redo ? 1 : 0;
    p.scale_log2 = 0.08838834764831845f * 1.4426950408889634f;   // 1/sqrt(128), fixed by the reference kernel
    // assign: -1 = by list overlap, 0 = every pair to this kernel, 1 = every pair to the pair walk
    pair_choice_kernel<<<dim3(((tiles + 1) / 2 + 7) / 8, heads), 256, 0, stream>>>(indices, counts, elsewhere, redo,
                                                                                  (int)tiles, (int)heads, assign);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    const unsigned items = tiles * heads;
    const unsigned grid = items < (unsigned)sms ? items : (unsigned)sms;   // one persistent CTA per SM
    attn_sparse_t_kernel<<<grid, ST_THREADS, ST_SMEM, stream>>>(*mq, *mk, *mv, p);
    return cudaGetLastError();
}

}  // namespace h3b
