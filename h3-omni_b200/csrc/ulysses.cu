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
