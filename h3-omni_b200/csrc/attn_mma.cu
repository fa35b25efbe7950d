// Warp-level (mma.sync m16n8k16) flash attention forward for the two link-completeness
// variants that are off the DiT hot path:
//   - bf16, head dim 128, causal and/or grouped-query (h3_flash_bf16; the reference's
//     FlashAttention-2 adapter, cuda/flash_attention.cu:29-67, used by its text and vision
//     encoders and by the FastH3 refiner), and
//   - fp16, head dim 64, non-causal (h3_flash3_f16_d64, cuda/flash3_attention.cu:81-87,
//     video VAE).
// Sequences there are short, so this kernel aims at correctness and portability of shapes
// (any Lq, Lk, batch, GQA ratio), not at tensor-core peak; the dense DiT path uses attn_tc5.cu.
//
// A CTA of 4 warps owns 64 query rows (16 per warp) and walks KV tiles of 64 rows staged in
// shared memory (K row-major, V transposed so both MMA B operands are 32-bit loads).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "attn_kernels.h"

namespace h3b {
namespace {

constexpr int MMA_BM = 64, MMA_BN = 64, MMA_THREADS = 128;

template <typename T>
struct Elem;
template <>
struct Elem<__nv_bfloat16> {
    static __device__ __forceinline__ uint32_t pack(float a, float b) {
        __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&v);
    }
    static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
            "{%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};
template <>
struct Elem<__half> {
    static __device__ __forceinline__ uint32_t pack(float a, float b) {
        __half2 v = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&v);
    }
    static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
            "{%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};

template <typename T, int D, bool CAUSAL>
__global__ void __launch_bounds__(MMA_THREADS)
attn_mma_kernel(T *__restrict__ out, const T *__restrict__ q, const T *__restrict__ k,
                const T *__restrict__ v, float *__restrict__ lse, int lq, int lk, int heads,
                int kv_heads, float scale) {
    constexpr int KS = D + 8;        // K tile row stride (elements), conflict-free 32-bit reads
    constexpr int VS = MMA_BN + 8;   // V^T tile row stride
    __shared__ __align__(16) T k_s[MMA_BN * KS];
    __shared__ __align__(16) T vt_s[D * VS];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int head = blockIdx.y, batch = blockIdx.z;
    const int kv_head = head / (heads / kv_heads);
    const int row0 = blockIdx.x * MMA_BM + warp * 16;  // this warp's first query row
    const float scale_log2 = scale * 1.4426950408889634f;

    // Q fragments (A operand), rows g and g+8 of the warp's 16.
    uint32_t qa[D / 16][4];
    {
        const int r0 = row0 + g, r1 = row0 + g + 8;
        const T *q0 = q + (((size_t)batch * lq + min(r0, lq - 1)) * heads + head) * D;
        const T *q1 = q + (((size_t)batch * lq + min(r1, lq - 1)) * heads + head) * D;
#pragma unroll
        for (int kk = 0; kk < D / 16; kk++) {
            qa[kk][0] = *reinterpret_cast<const uint32_t *>(q0 + kk * 16 + 2 * t);
            qa[kk][1] = *reinterpret_cast<const uint32_t *>(q1 + kk * 16 + 2 * t);
            qa[kk][2] = *reinterpret_cast<const uint32_t *>(q0 + kk * 16 + 8 + 2 * t);
            qa[kk][3] = *reinterpret_cast<const uint32_t *>(q1 + kk * 16 + 8 + 2 * t);
        }
    }

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;

    const int cta_last_row = min(blockIdx.x * MMA_BM + MMA_BM, lq) - 1;
    const int kv_end = CAUSAL ? min(lk, cta_last_row + 1) : lk;

    for (int j0 = 0; j0 < kv_end; j0 += MMA_BN) {
        __syncthreads();  // previous tile fully consumed
        // Stage K (row-major) and V (transposed); rows past lk read as zero.
        constexpr int VEC = 8;  // elements per 16-byte load
        for (int i = tid; i < MMA_BN * (D / VEC); i += MMA_THREADS) {
            const int r = i / (D / VEC), c = (i % (D / VEC)) * VEC;
            uint4 kvec = make_uint4(0, 0, 0, 0), vvec = make_uint4(0, 0, 0, 0);
            if (j0 + r < lk) {
                const size_t off = (((size_t)batch * lk + j0 + r) * kv_heads + kv_head) * D + c;
                kvec = *reinterpret_cast<const uint4 *>(k + off);
                vvec = *reinterpret_cast<const uint4 *>(v + off);
            }
            *reinterpret_cast<uint4 *>(&k_s[r * KS + c]) = kvec;
            const T *ve = reinterpret_cast<const T *>(&vvec);
#pragma unroll
            for (int e = 0; e < VEC; e++) vt_s[(c + e) * VS + r] = ve[e];
        }
        __syncthreads();

        // S = Q.K^T for this warp's 16 rows x 64 keys.
        float s[MMA_BN / 8][4];
#pragma unroll
        for (int nb = 0; nb < MMA_BN / 8; nb++) {
            s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.0f;
#pragma unroll
            for (int kk = 0; kk < D / 16; kk++) {
                const T *kr = &k_s[(nb * 8 + g) * KS + kk * 16 + 2 * t];
                Elem<T>::mma(s[nb], qa[kk], *reinterpret_cast<const uint32_t *>(kr),
                             *reinterpret_cast<const uint32_t *>(kr + 8));
            }
        }
        // Mask keys past lk and, for causal, keys after the query row.
        const int r0 = row0 + g, r1 = r0 + 8;
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nb = 0; nb < MMA_BN / 8; nb++) {
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int key = j0 + nb * 8 + 2 * t + e;
                const bool dead = key >= lk;
                if (dead || (CAUSAL && key > r0)) s[nb][e] = -INFINITY;
                if (dead || (CAUSAL && key > r1)) s[nb][2 + e] = -INFINITY;
                mx0 = fmaxf(mx0, s[nb][e]);
                mx1 = fmaxf(mx1, s[nb][2 + e]);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
        const float a0 = (n0 == -INFINITY) ? 1.0f : exp2f((m0 - n0) * scale_log2);
        const float a1 = (n1 == -INFINITY) ? 1.0f : exp2f((m1 - n1) * scale_log2);
        m0 = n0;
        m1 = n1;
        const float b0 = (m0 == -INFINITY) ? 0.0f : m0 * scale_log2;
        const float b1 = (m1 == -INFINITY) ? 0.0f : m1 * scale_log2;
        float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
        for (int nb = 0; nb < MMA_BN / 8; nb++) {
            s[nb][0] = exp2f(s[nb][0] * scale_log2 - b0);
            s[nb][1] = exp2f(s[nb][1] * scale_log2 - b0);
            s[nb][2] = exp2f(s[nb][2] * scale_log2 - b1);
            s[nb][3] = exp2f(s[nb][3] * scale_log2 - b1);
            sum0 += s[nb][0] + s[nb][1];
            sum1 += s[nb][2] + s[nb][3];
        }
        l0 = l0 * a0 + sum0;
        l1 = l1 * a1 + sum1;
#pragma unroll
        for (int i = 0; i < D / 8; i++) {
            o[i][0] *= a0;
            o[i][1] *= a0;
            o[i][2] *= a1;
            o[i][3] *= a1;
        }
        // O += P.V with P rounded to the element type (FlashAttention convention).
#pragma unroll
        for (int ks = 0; ks < MMA_BN / 16; ks++) {
            uint32_t pa[4];
            pa[0] = Elem<T>::pack(s[2 * ks][0], s[2 * ks][1]);
            pa[1] = Elem<T>::pack(s[2 * ks][2], s[2 * ks][3]);
            pa[2] = Elem<T>::pack(s[2 * ks + 1][0], s[2 * ks + 1][1]);
            pa[3] = Elem<T>::pack(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
            for (int nb = 0; nb < D / 8; nb++) {
                const T *vr = &vt_s[(nb * 8 + g) * VS + ks * 16 + 2 * t];
                Elem<T>::mma(o[nb], pa, *reinterpret_cast<const uint32_t *>(vr),
                             *reinterpret_cast<const uint32_t *>(vr + 8));
            }
        }
    }

    // Quad-reduce the row sums, normalise, store.
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = 1.0f / l0, i1 = 1.0f / l1;
    const int r0 = row0 + g, r1 = r0 + 8;
#pragma unroll
    for (int nb = 0; nb < D / 8; nb++) {
        if (r0 < lq) {
            T *dst = out + (((size_t)batch * lq + r0) * heads + head) * D + nb * 8 + 2 * t;
            *reinterpret_cast<uint32_t *>(dst) = Elem<T>::pack(o[nb][0] * i0, o[nb][1] * i0);
        }
        if (r1 < lq) {
            T *dst = out + (((size_t)batch * lq + r1) * heads + head) * D + nb * 8 + 2 * t;
            *reinterpret_cast<uint32_t *>(dst) = Elem<T>::pack(o[nb][2] * i1, o[nb][3] * i1);
        }
    }
    if (lse && t == 0) {
        if (r0 < lq) lse[((size_t)batch * heads + head) * lq + r0] = m0 * scale + logf(l0);
        if (r1 < lq) lse[((size_t)batch * heads + head) * lq + r1] = m1 * scale + logf(l1);
    }
}

template <typename T, int D>
cudaError_t launch_mma(void *out, const void *q, const void *k, const void *v, float *lse,
                       unsigned batch, unsigned lq, unsigned lk, unsigned heads,
                       unsigned kv_heads, float scale, bool causal, cudaStream_t stream) {
    dim3 grid((lq + MMA_BM - 1) / MMA_BM, heads, batch);
    if (causal)
        attn_mma_kernel<T, D, true><<<grid, MMA_THREADS, 0, stream>>>(
            (T *)out, (const T *)q, (const T *)k, (const T *)v, lse, (int)lq, (int)lk, (int)heads,
            (int)kv_heads, scale);
    else
        attn_mma_kernel<T, D, false><<<grid, MMA_THREADS, 0, stream>>>(
            (T *)out, (const T *)q, (const T *)k, (const T *)v, lse, (int)lq, (int)lk, (int)heads,
            (int)kv_heads, scale);
    return cudaGetLastError();
}

}  // namespace

cudaError_t attn_mma(void *out, const void *q, const void *k, const void *v, float *lse,
                     unsigned batch, unsigned lq, unsigned lk, unsigned heads, unsigned kv_heads,
                     float scale, bool causal, int elem, cudaStream_t stream) {
    if (!batch || !lq || !lk || !heads || !kv_heads || heads % kv_heads) return cudaErrorInvalidValue;
    if (heads > 65535u || batch > 65535u) return cudaErrorInvalidValue;
    if (elem == 0)
        return launch_mma<__nv_bfloat16, 128>(out, q, k, v, lse, batch, lq, lk, heads, kv_heads,
                                              scale, causal, stream);
    if (elem == 1)
        return launch_mma<__half, 64>(out, q, k, v, lse, batch, lq, lk, heads, kv_heads, scale,
                                      causal, stream);
    return cudaErrorInvalidValue;
}

}  // namespace h3b
