// Local transposes around the Ulysses all-to-all: out[b][a][c] = in[a][b][c] with c in
// 16-byte units (reference cuda/parallel.cuh:67-93). Pure byte movement, HBM-bound; the grid
// is a multiple of the SM count and walks the tensor grid-stride so every SM streams.
#include <algorithm>

#include "attn_kernels.h"

namespace h3b {
namespace {
__global__ void __launch_bounds__(256)
swap_leading_kernel(uint4 *__restrict__ out, const uint4 *__restrict__ in, unsigned a_count,
                    unsigned b_count, size_t c_count) {
    const size_t total = (size_t)a_count * b_count * c_count;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t c = i % c_count, ab = i / c_count;
        const size_t b = ab % b_count, a = ab / b_count;
        out[(b * a_count + a) * c_count + c] = in[i];
    }
}
}  // namespace

cudaError_t swap_leading_16b(void *out, const void *in, unsigned a, unsigned b, size_t c_units,
                             cudaStream_t stream) {
    const size_t total = (size_t)a * b * c_units;
    if (!total) return cudaSuccess;
    static thread_local int sms = 0;
    if (!sms) {
        int device = 0;
        cudaError_t e = cudaGetDevice(&device);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (e != cudaSuccess) return e;
    }
    const size_t wanted = (total + 255) / 256;
    const unsigned blocks = (unsigned)std::min<size_t>(wanted, (size_t)sms * 8);
    swap_leading_kernel<<<blocks, 256, 0, stream>>>(static_cast<uint4 *>(out),
                                                    static_cast<const uint4 *>(in), a, b, c_units);
    return cudaGetLastError();
}
}  // namespace h3b

// ---- fused exchange over peer memory -------------------------------------------------
// The NCCL path above is transpose kernel + grouped send/recv (+ the same in reverse): two
// passes over the tensor per exchange. Here one kernel reads the local tensor once and stores
// every 16-byte unit straight to its final place in the owning rank's window over NVLink
// (plain peer stores, no TMA), then the last CTA to finish publishes this rank's epoch to every
// peer and waits - bounded - until every peer's epoch has arrived here.
//   scatter: src [rows][heads][dim] -> window of rank p gets [ranks*rows][heads/ranks][dim]
//   gather : src [ranks*rows][heads/ranks][dim] -> window of rank p gets [rows][heads][dim]
namespace h3b {
namespace {

constexpr int MAX_RANKS = 16;
struct PushArgs {
    uint4 *window[MAX_RANKS];                 // slot base in every rank's window (peer pointers)
    unsigned long long *flags[MAX_RANKS];     // flag array [ranks] in every rank's window
    unsigned long long epoch;
    unsigned *done_counter;                   // local
    int *status;                              // local device status word
    int rank, ranks;
    unsigned rows, heads, dim16;              // dim in 16-byte units
};

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long *p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// Publish this rank's epoch in peer `peer`'s flag array, then wait (bounded, about 2 s) until
// that peer's epoch has arrived here: its data is then complete in our window.
__device__ __forceinline__ void epoch_handshake(unsigned long long *const *flags, unsigned long long epoch,
                                                int *status, int rank, int peer) {
    st_release_sys(flags[peer] + rank, epoch);
    const unsigned long long *mine = flags[rank] + peer;
    const unsigned long long start = clock64();
    for (unsigned spin = 0;; spin++) {
        if (ld_acquire_sys(mine) >= epoch) return;
        if ((spin & 1023u) == 1023u && clock64() - start > 4000000000ull) break;
        __nanosleep(100);
    }
    atomicCAS(status, 0, 1);   // timed out; the host sees status 1
}

template <bool GATHER>
__global__ void __launch_bounds__(256)
exchange_push_kernel(const uint4 *__restrict__ src, PushArgs a) {
    const unsigned hg = a.heads / a.ranks;
    const size_t total = (size_t)(GATHER ? a.ranks : 1) * a.rows * (GATHER ? hg : a.heads) * a.dim16;
    auto destination = [&](size_t i) -> uint4 * {
        const unsigned d = (unsigned)(i % a.dim16);
        const size_t rest = i / a.dim16;
        if (!GATHER) {
            // src (row, head): head group p goes to rank p at row rank*rows + row
            const unsigned head = (unsigned)(rest % a.heads), row = (unsigned)(rest / a.heads);
            return a.window[head / hg] + (((size_t)a.rank * a.rows + row) * hg + head % hg) * a.dim16 + d;
        }
        // src (global row, local head): rows of rank p go to rank p at head rank*hg + head
        const unsigned head = (unsigned)(rest % hg);
        const size_t grow = rest / hg;
        const unsigned row = (unsigned)(grow % a.rows);
        return a.window[grow / a.rows] + ((size_t)row * a.heads + (size_t)a.rank * hg + head) * a.dim16 + d;
    };
    // four independent 16-byte loads in flight per thread, then four (mostly remote) stores
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + 3 * stride < total; i += 4 * stride) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; u++) v[u] = __ldg(src + i + u * stride);
#pragma unroll
        for (int u = 0; u < 4; u++) *destination(i + u * stride) = v[u];
    }
    for (; i < total; i += stride) *destination(i) = __ldg(src + i);
    // completion: the last CTA publishes and waits
    __shared__ bool last;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(a.done_counter, 1u) == gridDim.x - 1;
    __syncthreads();
    if (!last) return;
    if (threadIdx.x == 0) *a.done_counter = 0;   // ready for the next exchange on this stream
    if ((int)threadIdx.x < a.ranks) epoch_handshake(a.flags, a.epoch, a.status, a.rank, threadIdx.x);
}

// One launch of `ranks` threads after a kernel that already stored into the peers' windows
// (stream order makes that kernel's stores precede the release below).
__global__ void exchange_handshake_kernel(PushArgs a) {
    __threadfence_system();
    if ((int)threadIdx.x < a.ranks) epoch_handshake(a.flags, a.epoch, a.status, a.rank, threadIdx.x);
}

}  // namespace

cudaError_t exchange_push(bool gather, const void *src, void *const window[], unsigned long long *const flags[],
                          unsigned long long epoch, unsigned *done_counter, int *status, int rank, int ranks,
                          unsigned rows, unsigned heads, unsigned dim, cudaStream_t stream) {
    if (ranks < 1 || ranks > MAX_RANKS || heads % ranks || (dim * 2) % 16) return cudaErrorInvalidValue;
    PushArgs a{};
    for (int p = 0; p < ranks; p++) {
        a.window[p] = static_cast<uint4 *>(window[p]);
        a.flags[p] = flags[p];
    }
    a.epoch = epoch;
    a.done_counter = done_counter;
    a.status = status;
    a.rank = rank;
    a.ranks = ranks;
    a.rows = rows;
    a.heads = heads;
    a.dim16 = dim * 2 / 16;
    static thread_local int sms = 0;
    if (!sms) {
        int device = 0;
        cudaError_t e = cudaGetDevice(&device);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (e != cudaSuccess) return e;
    }
    const size_t total = (size_t)rows * heads * a.dim16;
    const unsigned blocks = (unsigned)std::min<size_t>((total + 1023) / 1024, (size_t)sms * 8);
    if (gather)
        exchange_push_kernel<true><<<blocks, 256, 0, stream>>>(static_cast<const uint4 *>(src), a);
    else
        exchange_push_kernel<false><<<blocks, 256, 0, stream>>>(static_cast<const uint4 *>(src), a);
    return cudaGetLastError();
}

cudaError_t exchange_handshake(unsigned long long *const flags[], unsigned long long epoch, int *status,
                               int rank, int ranks, cudaStream_t stream) {
    if (ranks < 1 || ranks > MAX_RANKS) return cudaErrorInvalidValue;
    PushArgs a{};
    for (int p = 0; p < ranks; p++) a.flags[p] = flags[p];
    a.epoch = epoch;
    a.status = status;
    a.rank = rank;
    a.ranks = ranks;
    exchange_handshake_kernel<<<1, 32, 0, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace h3b
