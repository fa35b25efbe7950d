// Host-side definitions shared by the translation units that implement the primitive ABI:
// the context and tensor objects, error recording and argument validation.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <initializer_list>

#include "../../include/h3b200_attn.h"

// Staging for h3b_sdpa_bf16_host: two slots of compact per-head-group device buffers,
// a stream for each copy direction and the events that order the three streams.
struct host_pipeline {
    void *slot[2][4]{};            // q, k, v, out per slot
    size_t slot_bytes{};
    cudaStream_t h2d{}, d2h{}, compute[2]{};   // kernels of consecutive chunks alternate between two streams
    cudaEvent_t loaded[2]{}, computed[2]{}, stored[2]{}, entry{};
    bool ready{};
};
struct h3_gpu {
    int device{};
    cudaStream_t own_stream{}, stream{};
    char error[512]{};
    host_pipeline pipe;
};
struct h3_gpu_tensor {
    void *data{};
    size_t elements{}, bytes{};
    h3_gpu_dtype dtype{};
    h3_gpu *owner{};
    bool owns{};
};

namespace h3b {

// Records a message in the context (what h3_gpu_error returns). A null context is ignored.
void fail(h3_gpu *g, const char *format, ...);
// true when e is cudaSuccess; otherwise records "CUDA: <text>" and returns false.
bool cuda_good(h3_gpu *g, cudaError_t e);

// One requirement on a tensor argument: it belongs to the context, holds at least `elements`
// elements and, unless any_dtype, has the given dtype. The messages are the reference backend's
// ("invalid tensor: <what> (need <n> elements)", "expected BF16: <what>").
struct Need {
    const h3_gpu_tensor *tensor;
    size_t elements;
    const char *what;
    h3_gpu_dtype dtype;
    bool any_dtype;
};
inline Need bf16(const h3_gpu_tensor *t, size_t n, const char *what) { return Need{t, n, what, H3_GPU_BF16, false}; }
inline Need sized(const h3_gpu_tensor *t, size_t n, const char *what) { return Need{t, n, what, H3_GPU_F32, true}; }
bool satisfied(h3_gpu *g, std::initializer_list<Need> needs);

size_t dtype_bytes(h3_gpu_dtype t);
// Stream-ordered allocation on the context's stream.
h3_gpu_tensor *new_tensor(h3_gpu *g, size_t elements, h3_gpu_dtype dtype);

}  // namespace h3b
