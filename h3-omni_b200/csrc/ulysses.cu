// Kernels of the Ulysses head-scatter / sequence-gather exchange.
//
// Library path (behind h3_gpu_ulysses_*): a local block transpose around an NCCL all-to-all, the
// data movement of the reference's cuda/parallel.cuh:67-143.
//
// Fused path (h3b_exchange_*): every rank owns a window in its own memory that all ranks can
// store into (plain peer stores over NVLink; no TMA, no multicast). One kernel reads the local
// tensors once and stores every 16-byte unit straight to its final place in the owning rank's
// window. Two flag arrays in every window order the ranks:
//   ready[p] = last exchange rank p has STARTED. A rank starts exchange E only after everything
//              queued before it on its stream has finished, so ready[p] >= E tells the others that
//              rank p no longer reads what earlier exchanges left in its window: they may overwrite.
//   done[p]  = last exchange whose data FROM rank p is complete in this window.
// Every wait on a flag is bounded; a wait that gives up records status 1 in the device status
// word, stores nothing more and does not publish, so the failure shows on every rank.
#include <algorithm>

#include "attn_kernels.h"

namespace h3b {
namespace {

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long *p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait until *word >= epoch.
__device__ __forceinline__ bool flag_reached(const unsigned long long *word, unsigned long long epoch,
                                             unsigned long long limit_ns) {
    if (ld_acquire_sys(word) >= epoch) return true;
    const unsigned long long start = timer_ns();
    for (unsigned spin = 1;; spin++) {
        if (ld_acquire_sys(word) >= epoch) return true;
        if ((spin & 63u) == 0u && timer_ns() - start > limit_ns) return false;
        __nanosleep(64);
    }
}
// Thread p < ranks: announce this rank's start of `epoch` to rank p, then wait for rank p's.
__device__ __forceinline__ bool open_with_peer(const ExchangeSync &s, int p) {
    st_release_sys(&s.flags[p]->ready[s.rank], s.epoch);
    return flag_reached(&s.flags[s.rank]->ready[p], s.epoch, s.limit_ns);
}
// Thread p < ranks: tell rank p that this rank's data of `epoch` is complete, wait for rank p's.
__device__ __forceinline__ bool close_with_peer(const ExchangeSync &s, int p) {
    st_release_sys(&s.flags[p]->done[s.rank], s.epoch);
    return flag_reached(&s.flags[s.rank]->done[p], s.epoch, s.limit_ns);
}

// ---- block transpose: out[b][a][:] = in[a][b][:] with rows of `units` 16-byte units --------------
// One warp moves one row; the rows of a warp's (a, b) walk are contiguous on the input side.
__global__ void __launch_bounds__(256)
transpose_rows_kernel(uint4 *__restrict__ out, const uint4 *__restrict__ in, unsigned a_count, unsigned b_count,
                      unsigned units) {
    const unsigned lane = threadIdx.x & 31;
    const size_t rows = (size_t)a_count * b_count;
    const size_t warps = (size_t)gridDim.x * (blockDim.x >> 5);
    for (size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += warps) {
        const size_t a = row / b_count, b = row % b_count;
        const uint4 *src = in + row * units;
        uint4 *dst = out + (b * a_count + a) * units;
        for (unsigned u = lane; u < units; u += 32) dst[u] = __ldg(src + u);
    }
}

// ---- fused exchange ------------------------------------------------------------------------------
struct PushArgs {
    ExchangeSync sync;
    const uint4 *src[EXCHANGE_MAX_TENSORS];
    uint4 *window[EXCHANGE_MAX_TENSORS][EXCHANGE_MAX_RANKS];   // slot base of tensor t in rank p's window
    int tensors;
    unsigned rows, heads, dim16;   // dim in 16-byte units
};

//   scatter: src [rows][heads][dim] -> window of rank p gets [ranks*rows][heads/ranks][dim]
//   gather : src [ranks*rows][heads/ranks][dim] -> window of rank p gets [rows][heads][dim]
template <bool GATHER>
__global__ void __launch_bounds__(256)
exchange_push_kernel(const PushArgs a) {
    __shared__ int opened, last;
    const ExchangeSync &s = a.sync;
    if (threadIdx.x == 0) opened = 1;
    __syncthreads();
    if ((int)threadIdx.x < s.ranks && !open_with_peer(s, threadIdx.x)) {
        opened = 0;
        atomicCAS(s.status, 0, 1);
    }
    __syncthreads();
    if (opened) {
        const unsigned hg = a.heads / s.ranks;
        const size_t per_tensor = (size_t)(GATHER ? s.ranks : 1) * a.rows * (GATHER ? hg : a.heads) * a.dim16;
        const size_t stride = (size_t)gridDim.x * blockDim.x;
        for (int t = 0; t < a.tensors; t++) {
            const uint4 *src = a.src[t];
            auto destination = [&](size_t i) -> uint4 * {
                const unsigned d = (unsigned)(i % a.dim16);
                const size_t rest = i / a.dim16;
                if (!GATHER) {
                    // (row, head): head group p goes to rank p, row block `rank` of its tensor
                    const unsigned head = (unsigned)(rest % a.heads), row = (unsigned)(rest / a.heads);
                    return a.window[t][head / hg] + (((size_t)s.rank * a.rows + row) * hg + head % hg) * a.dim16 + d;
                }
                // (global row, local head): the rows of rank p go to rank p, head block `rank`
                const unsigned head = (unsigned)(rest % hg);
                const size_t grow = rest / hg;
                return a.window[t][grow / a.rows] +
                       ((size_t)(grow % a.rows) * a.heads + (size_t)s.rank * hg + head) * a.dim16 + d;
            };
            // four independent 16-byte loads in flight per thread, then four (mostly remote) stores
            size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
            for (; i + 3 * stride < per_tensor; i += 4 * stride) {
                uint4 v[4];
#pragma unroll
                for (int u = 0; u < 4; u++) v[u] = __ldg(src + i + u * stride);
#pragma unroll
                for (int u = 0; u < 4; u++) *destination(i + u * stride) = v[u];
            }
            for (; i < per_tensor; i += stride) *destination(i) = __ldg(src + i);
        }
    }
    // completion: the last CTA to finish publishes this rank's epoch and waits for the peers'
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) last = atomicInc(&s.flags[s.rank]->counter, gridDim.x - 1) == gridDim.x - 1;   // wraps to 0
    __syncthreads();
    if (!last || *reinterpret_cast<volatile int *>(s.status) != 0) return;
    if ((int)threadIdx.x < s.ranks && !close_with_peer(s, threadIdx.x)) atomicCAS(s.status, 0, 1);
}

// Around a kernel that stores into the peers' windows itself (attention with the gather in its
// epilogue, norm + RoPE with the scatter in its stores): open before it, close after it.
__global__ void exchange_open_kernel(const ExchangeSync s) {
    if ((int)threadIdx.x < s.ranks && !open_with_peer(s, threadIdx.x)) atomicCAS(s.status, 0, 1);
}
__global__ void exchange_close_kernel(const ExchangeSync s) {
    __threadfence_system();
    if (*reinterpret_cast<volatile int *>(s.status) != 0) return;
    if ((int)threadIdx.x < s.ranks && !close_with_peer(s, threadIdx.x)) atomicCAS(s.status, 0, 1);
}

cudaError_t sm_count(int *sms) {
    static thread_local int cached_device = -1, cached = 0;
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e == cudaSuccess && device != cached_device) {
        e = cudaDeviceGetAttribute(&cached, cudaDevAttrMultiProcessorCount, device);
        if (e == cudaSuccess) cached_device = device;
    }
    *sms = cached;
    return e;
}

}  // namespace

cudaError_t transpose_rows_16b(void *out, const void *in, unsigned a, unsigned b, size_t row_units,
                               cudaStream_t stream) {
    const size_t rows = (size_t)a * b;
    if (!rows || !row_units) return cudaSuccess;
    if (row_units > 0xffffffffull) return cudaErrorInvalidValue;
    int sms = 0;
    cudaError_t e = sm_count(&sms);
    if (e != cudaSuccess) return e;
    const unsigned blocks = (unsigned)std::min<size_t>((rows + 7) / 8, (size_t)sms * 8);
    transpose_rows_kernel<<<blocks, 256, 0, stream>>>(static_cast<uint4 *>(out), static_cast<const uint4 *>(in), a,
                                                      b, (unsigned)row_units);
    return cudaGetLastError();
}

cudaError_t exchange_push(bool gather, int tensors, const void *const src[],
                          void *const window[][EXCHANGE_MAX_RANKS], const ExchangeSync &sync, unsigned rows,
                          unsigned heads, unsigned dim, cudaStream_t stream) {
    if (sync.ranks < 1 || sync.ranks > EXCHANGE_MAX_RANKS || tensors < 1 || tensors > EXCHANGE_MAX_TENSORS ||
        heads % sync.ranks || (dim * 2) % 16)
        return cudaErrorInvalidValue;
    PushArgs a{};
    a.sync = sync;
    a.tensors = tensors;
    for (int t = 0; t < tensors; t++) {
        a.src[t] = static_cast<const uint4 *>(src[t]);
        for (int p = 0; p < sync.ranks; p++) a.window[t][p] = static_cast<uint4 *>(window[t][p]);
    }
    a.rows = rows;
    a.heads = heads;
    a.dim16 = dim * 2 / 16;
    int sms = 0;
    cudaError_t e = sm_count(&sms);
    if (e != cudaSuccess) return e;
    const size_t total = (size_t)rows * heads * a.dim16 * tensors;
    const unsigned blocks = (unsigned)std::max<size_t>(1, std::min<size_t>((total + 1023) / 1024, (size_t)sms * 8));
    if (gather)
        exchange_push_kernel<true><<<blocks, 256, 0, stream>>>(a);
    else
        exchange_push_kernel<false><<<blocks, 256, 0, stream>>>(a);
    return cudaGetLastError();
}

cudaError_t exchange_open(const ExchangeSync &sync, cudaStream_t stream) {
    if (sync.ranks < 1 || sync.ranks > EXCHANGE_MAX_RANKS) return cudaErrorInvalidValue;
    exchange_open_kernel<<<1, 32, 0, stream>>>(sync);
    return cudaGetLastError();
}
cudaError_t exchange_close(const ExchangeSync &sync, cudaStream_t stream) {
    if (sync.ranks < 1 || sync.ranks > EXCHANGE_MAX_RANKS) return cudaErrorInvalidValue;
    exchange_close_kernel<<<1, 32, 0, stream>>>(sync);
    return cudaGetLastError();
}

}  // namespace h3b
