// Attention output projection with the gate and the residual in its epilogue, then AdaLN: the
// three launches that follow every attention call in the reference's block
// (h3_dit.c:2573-2597: h3_gpu_linear_bf16 INNER -> HIDDEN, then h3_gpu_gate_adaln_bf16 =
// cuda/fast_primitives.cuh:50-124) as two.
//
//   y      = bf16(attention_heads . W^T)                       W: [hidden][inner] bf16, fp32 accumulate
//   gated  = bf16(residual + bf16(y * gate[map[row]][gate_slot]))         (h3_gate_bf16)
//   output = bf16(bf16(bf16(gated * rsqrt(mean(gated^2) + eps) * norm_w) * bf16(1 + scale)) + shift)   (h3_adaln_bf16)
//
// Kernel 1 is a persistent tcgen05 GEMM (TMA-fed, 128 x 256 output tiles, two accumulators in
// TMEM so the epilogue of one tile runs under the MMAs of the next) whose epilogue applies gate and
// residual to the fp32 accumulators and writes `gated`; y is never written to memory. Kernel 2 is
// the row-wise AdaLN in the reference's own operation order (it needs the whole gated row for the
// RMS, so it cannot live in a tile epilogue). The A operand may be the window slot the attention
// kernel gathered its output into, so at N GPUs nothing is copied between attention and projection.
#include <cuda.h>

#include "attn_kernels.h"
#include "h3_gpu_internal.h"
#include "sm100_ptx.cuh"

namespace h3b {
namespace {

constexpr int GM = 128, GN = 256, GK = 64;          // CTA tile; GK = one 128-byte swizzle row
constexpr int G_STAGES = 4;
constexpr int G_A_BYTES = GM * GK * 2, G_B_BYTES = GN * GK * 2, G_STAGE = G_A_BYTES + G_B_BYTES;   // 16 + 32 KB
constexpr int G_SMEM = G_STAGES * G_STAGE + 1024;
constexpr int G_THREADS = 192;                       // warps 0-3 epilogue, 4 TMA, 5 MMA

struct OutProjParams {
    const __nv_bfloat16 *residual, *modulation;
    const unsigned *row_map;
    __nv_bfloat16 *gated;
    int rows, inner, hidden, slots, gate_slot;
    int tiles_m, tiles_n;
    int *status;
};

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void *map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}

__global__ void __launch_bounds__(G_THREADS, 1)
out_proj_gate_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     const OutProjParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bars[2 * G_STAGES + 4];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_word;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar0 = smem_u32(bars);
    auto bar_full = [&](int s) { return bar0 + 8u * s; };
    auto bar_empty = [&](int s) { return bar0 + 8u * (G_STAGES + s); };
    auto bar_acc_full = [&](int a) { return bar0 + 8u * (2 * G_STAGES + a); };
    auto bar_acc_empty = [&](int a) { return bar0 + 8u * (2 * G_STAGES + 2 + a); };
    if (tid == 0) {
        for (int s = 0; s < G_STAGES; s++) {
            mbar_init(bar_full(s), 1);
            mbar_init(bar_empty(s), 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(bar_acc_full(a), 1);
            mbar_init(bar_acc_empty(a), 128);
        }
        mbar_fence_init();
        abort_word = 0;
    }
    if (warp == 5) {
        tmem_alloc(smem_u32(&tmem_slot), 512);
        tmem_relinquish();
    }
    tc5_fence_before();
    __syncthreads();
    tc5_fence_after();
    const uint32_t tmem = tmem_slot;
    const int total = p.tiles_m * p.tiles_n, ksteps = p.inner / GK;
    // tile t of this CTA: consecutive tiles share the row block (its 128 x inner slice of A stays in L2)

    if (warp == 4) {
        if (lane == 0) {
            tma_prefetch_desc(&map_a);
            tma_prefetch_desc(&map_b);
            int fill = 0;
            for (int tile = blockIdx.x; tile < total; tile += gridDim.x) {
                const int m0 = (tile / p.tiles_n) * GM, n0 = (tile % p.tiles_n) * GN;
                bool ok = true;
                for (int k = 0; k < ksteps; k++, fill++) {
                    const int s = fill % G_STAGES, use = fill / G_STAGES;
                    if (use > 0 && !mbar_wait(bar_empty(s), (use - 1) & 1, &abort_word)) {
                        ok = false;
                        break;
                    }
                    const uint32_t dst = base + s * G_STAGE;
                    mbar_arrive_expect_tx(bar_full(s), G_STAGE);
                    tma_load_2d(dst, &map_a, bar_full(s), k * GK, m0);
                    tma_load_2d(dst + G_A_BYTES, &map_b, bar_full(s), k * GK, n0);
                }
                if (!ok) break;
            }
        }
    } else if (warp == 5) {
        // The whole warp walks the loop and one elected lane issues (descriptor arithmetic stays
        // in the uniform datapath; inside a one-lane branch it would be per-thread data).
        {
            const bool leader = elect_one();
            constexpr uint32_t idesc = mma_idesc(GM, GN, 1, 0);
            const uint64_t a_proto = smem_desc_sw128(base, 16, 1024), b_proto = smem_desc_sw128(base + G_A_BYTES, 16, 1024);
            const uint32_t a_lo0 = (uint32_t)a_proto, hi = (uint32_t)(a_proto >> 32), b_lo0 = (uint32_t)b_proto;
            int fill = 0, local = 0;
            for (int tile = blockIdx.x; tile < total; tile += gridDim.x, local++) {
                const int acc = local & 1;
                bool ok = local < 2 || mbar_wait_converged(bar_acc_empty(acc), ((local >> 1) - 1) & 1, &abort_word);
                tc5_fence_after();
                for (int k = 0; ok && k < ksteps; k++, fill++) {
                    const int s = fill % G_STAGES;
                    if (!mbar_wait_converged(bar_full(s), (fill / G_STAGES) & 1, &abort_word)) {
                        ok = false;
                        break;
                    }
                    tc5_fence_after();
                    const uint32_t a_lo = a_lo0 + s * (G_STAGE >> 4), b_lo = b_lo0 + s * (G_STAGE >> 4);
                    if (leader) {
#pragma unroll
                        for (int kk = 0; kk < GK / 16; kk++)
                            mma_ss_words(tmem + acc * GN, a_lo + kk * 2, hi, b_lo + kk * 2, hi, idesc, (k > 0) || (kk > 0));
                        mma_commit(bar_empty(s));
                    }
                    __syncwarp();
                }
                if (!ok) break;
                if (leader) mma_commit(bar_acc_full(acc));
                __syncwarp();
            }
        }
    } else {
        // ---- epilogue: one thread per output row of the tile ----
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        int local = 0;
        for (int tile = blockIdx.x; tile < total; tile += gridDim.x, local++) {
            const int acc = local & 1;
            const int m0 = (tile / p.tiles_n) * GM, n0 = (tile % p.tiles_n) * GN;
            if (!__all_sync(0xffffffffu, mbar_wait(bar_acc_full(acc), (local >> 1) & 1, &abort_word))) break;
            tc5_fence_after();
            const int row = m0 + tid;
            const bool live = row < p.rows;
            const __nv_bfloat16 *gate = nullptr, *res = nullptr;
            __nv_bfloat16 *dst = nullptr;
            if (live) {
                gate = p.modulation + ((size_t)p.row_map[row] * p.slots + p.gate_slot) * p.hidden;
                res = p.residual + (size_t)row * p.hidden;
                dst = p.gated + (size_t)row * p.hidden;
            }
#pragma unroll 1
            for (int c = 0; c < GN; c += 32) {
                uint32_t v[32];
                tmem_ld32(tmem + lane_base + acc * GN + c, v);
                tmem_wait_ld();
                const int col = n0 + c;
                if (live && col < p.hidden) {   // hidden is a multiple of 8: whole 16-byte vectors
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        if (col + i * 8 >= p.hidden) break;
                        const uint4 g4 = *reinterpret_cast<const uint4 *>(gate + col + i * 8);
                        const uint4 r4 = *reinterpret_cast<const uint4 *>(res + col + i * 8);
                        const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w}, rw[4] = {r4.x, r4.y, r4.z, r4.w};
                        uint32_t ow[4];
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            // y rounded to bf16 (the reference stores it), times gate rounded, plus residual, rounded
                            const float y0 = round_bf16(__uint_as_float(v[i * 8 + 2 * j]));
                            const float y1 = round_bf16(__uint_as_float(v[i * 8 + 2 * j + 1]));
                            const float o0 = __fadd_rn(bf16_lo(rw[j]), round_bf16(__fmul_rn(y0, bf16_lo(gw[j]))));
                            const float o1 = __fadd_rn(bf16_hi(rw[j]), round_bf16(__fmul_rn(y1, bf16_hi(gw[j]))));
                            ow[j] = pack_bf16(o0, o1);
                        }
                        *reinterpret_cast<uint4 *>(dst + col + i * 8) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                    }
                }
            }
            tc5_fence_before();
            mbar_arrive(bar_acc_empty(acc));
        }
    }
    tc5_fence_before();
    __syncthreads();
    if (abort_word) {
        if (tid == 0) atomicCAS(p.status, STATUS_OK, STATUS_WAIT_TIMEOUT);
        if (warp == 4) __nanosleep(1000000);
        __syncthreads();
    }
    if (warp == 5) {
        tc5_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

// AdaLN of a row in the operation order of the reference's kernel (cuda/fast_primitives.cuh:50-124
// with GATE = false; the reference builds with --fmad=false, hence the explicit roundings): thread
// t < 128 owns the 4-value groups at 4t + 512c, sums squares with fmaf in index order, shuffle-down
// tree, warp sums paired (0+2, 1+3), then (0+1).
template <int CHUNKS>
__global__ void __launch_bounds__(128)
adaln_rows_kernel(const uint16_t *__restrict__ input, const uint16_t *__restrict__ weight,
                  const uint16_t *__restrict__ modulation, const unsigned *__restrict__ row_map,
                  uint16_t *__restrict__ output, unsigned rows, unsigned width, unsigned slots, unsigned shift_slot,
                  unsigned scale_slot, float epsilon) {
    const unsigned row = blockIdx.x, tid = threadIdx.x;
    if (row >= rows) return;
    __shared__ float warp_sums[4];
    const uint16_t *x = input + (size_t)row * width;
    uint2 held[CHUNKS];
    float sum = 0.0f;
#pragma unroll
    for (int c = 0; c < CHUNKS; c++) {
        const unsigned start = 4 * tid + 512 * c;
        if (start < width) {
            held[c] = *reinterpret_cast<const uint2 *>(x + start);
            const float v[4] = {bf16_lo(held[c].x), bf16_hi(held[c].x), bf16_lo(held[c].y), bf16_hi(held[c].y)};
#pragma unroll
            for (int i = 0; i < 4; i++) sum = fmaf(v[i], v[i], sum);
        }
    }
    for (unsigned distance = 16; distance; distance >>= 1) sum = __fadd_rn(sum, __shfl_down_sync(0xffffffffu, sum, distance));
    if (tid % 32 == 0) warp_sums[tid / 32] = sum;
    __syncthreads();
    if (tid < 2) warp_sums[tid] = __fadd_rn(warp_sums[tid], warp_sums[tid + 2]);
    __syncthreads();
    if (tid == 0) warp_sums[0] = __fadd_rn(warp_sums[0], warp_sums[1]);
    __syncthreads();
    const float inverse = rsqrtf(__fadd_rn(__fdiv_rn(warp_sums[0], (float)width), epsilon));
    const size_t mod = (size_t)row_map[row] * slots * width;
#pragma unroll
    for (int c = 0; c < CHUNKS; c++) {
        const unsigned start = 4 * tid + 512 * c;
        if (start < width) {
            const uint2 w2 = *reinterpret_cast<const uint2 *>(weight + start);
            const uint2 sh = *reinterpret_cast<const uint2 *>(modulation + mod + (size_t)shift_slot * width + start);
            const uint2 sc = *reinterpret_cast<const uint2 *>(modulation + mod + (size_t)scale_slot * width + start);
            const float xv[4] = {bf16_lo(held[c].x), bf16_hi(held[c].x), bf16_lo(held[c].y), bf16_hi(held[c].y)};
            const float wv[4] = {bf16_lo(w2.x), bf16_hi(w2.x), bf16_lo(w2.y), bf16_hi(w2.y)};
            const float shv[4] = {bf16_lo(sh.x), bf16_hi(sh.x), bf16_lo(sh.y), bf16_hi(sh.y)};
            const float scv[4] = {bf16_lo(sc.x), bf16_hi(sc.x), bf16_lo(sc.y), bf16_hi(sc.y)};
            float o[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float normalized = __fmul_rn(__fmul_rn(xv[i], inverse), wv[i]);
                o[i] = __fadd_rn(round_bf16(__fmul_rn(round_bf16(normalized), round_bf16(__fadd_rn(1.0f, scv[i])))), shv[i]);
            }
            *reinterpret_cast<uint2 *>(output + (size_t)row * width + start) =
                make_uint2(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]));
        }
    }
}

using EncodeTiled = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                 const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
cudaError_t map_2d(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    static EncodeTiled fn = [] {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult query;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &query) != cudaSuccess ||
            query != cudaDriverEntryPointSuccess)
            return (EncodeTiled) nullptr;
        return (EncodeTiled)sym;
    }();
    if (!fn) return cudaErrorNotSupported;
    const cuuint64_t dims[2] = {cols, rows}, strides[1] = {cols * 2};
    const cuuint32_t box[2] = {GK, box_rows}, ones[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, ones,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

}  // namespace

cudaError_t out_proj_gate(void *gated, const void *residual, const void *attention_heads, const void *weight,
                          const void *modulation, const unsigned *row_map, unsigned rows, unsigned inner,
                          unsigned hidden, unsigned slots, unsigned gate_slot, cudaStream_t stream) {
    if (!rows || !inner || !hidden || inner % GK || hidden % 8 || gate_slot >= slots) return cudaErrorInvalidValue;
    for (const void *ptr : {(const void *)gated, residual, attention_heads, weight, modulation})
        if (!ptr || reinterpret_cast<uintptr_t>(ptr) % 16) return cudaErrorMisalignedAddress;
    static thread_local int configured_device = -1, sms = 0;
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    if (configured_device != device) {
        e = cudaFuncSetAttribute(out_proj_gate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, G_SMEM);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (e != cudaSuccess) return e;
        configured_device = device;
    }
    CUtensorMap map_a, map_b;
    if ((e = map_2d(&map_a, attention_heads, rows, inner, GM)) != cudaSuccess) return e;
    if ((e = map_2d(&map_b, weight, hidden, inner, GN)) != cudaSuccess) return e;
    OutProjParams p{};
    p.residual = static_cast<const __nv_bfloat16 *>(residual);
    p.modulation = static_cast<const __nv_bfloat16 *>(modulation);
    p.row_map = row_map;
    p.gated = static_cast<__nv_bfloat16 *>(gated);
    p.rows = (int)rows;
    p.inner = (int)inner;
    p.hidden = (int)hidden;
    p.slots = (int)slots;
    p.gate_slot = (int)gate_slot;
    p.tiles_m = (int)((rows + GM - 1) / GM);
    p.tiles_n = (int)((hidden + GN - 1) / GN);
    if ((e = device_status_word(&p.status)) != cudaSuccess) return e;
    const int total = p.tiles_m * p.tiles_n;
    out_proj_gate_kernel<<<total < sms ? total : sms, G_THREADS, G_SMEM, stream>>>(map_a, map_b, p);
    return cudaGetLastError();
}

cudaError_t adaln_rows(void *output, const void *input, const void *norm_weight, const void *modulation,
                       const unsigned *row_map, unsigned rows, unsigned width, unsigned slots, unsigned shift_slot,
                       unsigned scale_slot, float epsilon, cudaStream_t stream) {
    if (!rows || !width || width % 4 || shift_slot >= slots || scale_slot >= slots) return cudaErrorInvalidValue;
    const unsigned chunks = (width + 511) / 512;
    auto launch = [&](auto kernel) {
        kernel<<<rows, 128, 0, stream>>>(static_cast<const uint16_t *>(input), static_cast<const uint16_t *>(norm_weight),
                                         static_cast<const uint16_t *>(modulation), row_map,
                                         static_cast<uint16_t *>(output), rows, width, slots, shift_slot, scale_slot,
                                         epsilon);
        return cudaGetLastError();
    };
    if (chunks <= 4) return launch(adaln_rows_kernel<4>);
    if (chunks <= 8) return launch(adaln_rows_kernel<8>);
    if (chunks <= 11) return launch(adaln_rows_kernel<11>);
    if (chunks <= 16) return launch(adaln_rows_kernel<16>);
    return cudaErrorInvalidValue;   // rows wider than 8192 values are not needed on this path
}

}  // namespace h3b

// The three calls of the reference's block after attention (h3_dit.c:2573-2597) as one:
// h3_gpu_linear_bf16(attention_output, attention_heads, out_weight, NULL, rows, inner, hidden), then
// h3_gpu_gate_adaln_bf16(gated_residual, output, residual, attention_output, norm_weight,
// gate_modulation, modulation, row_map, rows, hidden, slots, gate_slot, shift_slot, scale_slot, eps).
// attention_output is never materialised. gated_residual may alias residual; output may be NULL
// (gate only, h3_gpu_gate_bf16). Same argument checks and messages as the two reference calls.
extern "C" int h3b_attention_output_gate_adaln_bf16(
    h3_gpu *g, h3_gpu_tensor *gated_residual, h3_gpu_tensor *output, const h3_gpu_tensor *residual,
    const h3_gpu_tensor *attention_heads, const h3_gpu_tensor *out_weight, const h3_gpu_tensor *norm_weight,
    const h3_gpu_tensor *gate_modulation, const h3_gpu_tensor *modulation, const h3_gpu_tensor *row_map, uint32_t rows,
    uint32_t inner, uint32_t hidden, uint32_t slots, uint32_t gate_slot, uint32_t shift_slot, uint32_t scale_slot,
    float epsilon) {
    using h3b::bf16;
    if (!g) return 0;
    if (!rows || !inner || !hidden || inner % 64 || hidden % 8 || gate_slot >= slots) {
        h3b::fail(g, "attention output projection: inner %u must be a multiple of 64, hidden %u of 8, gate slot %u < %u",
                  inner, hidden, gate_slot, slots);
        return 0;
    }
    const size_t count = (size_t)rows * hidden;
    if (!h3b::satisfied(g, {bf16(attention_heads, (size_t)rows * inner, "linear input"),
                            bf16(out_weight, (size_t)hidden * inner, "linear weight"), bf16(residual, count, "gate residual"),
                            bf16(gate_modulation, (size_t)slots * hidden, "gate modulation"),
                            h3b::Need{row_map, rows, "gate row map", H3_GPU_U32, false},
                            bf16(gated_residual, count, "gate output")}))
        return 0;
    if (!h3b::cuda_good(g, h3b::out_proj_gate(gated_residual->data, residual->data, attention_heads->data,
                                              out_weight->data, gate_modulation->data,
                                              static_cast<const unsigned *>(row_map->data), rows, inner, hidden, slots,
                                              gate_slot, g->stream)))
        return 0;
    if (!output) return 1;
    if (!h3b::satisfied(g, {bf16(output, count, "AdaLN output"), bf16(norm_weight, hidden, "AdaLN weight"),
                            bf16(modulation, (size_t)slots * hidden, "AdaLN modulation")}) ||
        shift_slot >= slots || scale_slot >= slots)
        return 0;
    return h3b::cuda_good(g, h3b::adaln_rows(output->data, gated_residual->data, norm_weight->data, modulation->data,
                                             static_cast<const unsigned *>(row_map->data), rows, hidden, slots, shift_slot,
                                             scale_slot, epsilon, g->stream));
}
