"""The allocation-free top-k entry point against the regular VSA path.

Some users of this library cannot allocate device memory at the call site (a fixed arena
handed out at start-up, a memory cap, a latency-critical loop). h3b_vsa_topk_static serves
them from a scratch array built into the library. This file checks that it returns exactly the
index lists and counts the regular entry point (h3_gpu_vsa_bf16) computes, on two calls in a
row that share the scratch array, and that shapes beyond its limit are refused.

Collected last on purpose (file name): a failure here cannot hide the other tests.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def regular_path(gpu, oracle, text, audio, shape, heads, seed):
    """indices/counts from h3_gpu_vsa_bf16's work buffers, plus what the new entry needs."""
    handle = gpu.call("vsa_new", text, audio, *shape, heads)
    info = [C.c_int() for _ in range(4)]
    assert gpu.lib.h3b_vsa_info(handle, *[C.byref(x) for x in info])
    rows, tiles, prefix, keep = (x.value for x in info)
    q, k, v = (oracle.normal_bf16((rows, heads, 128), seed + i) for i in range(3))
    gate = np.zeros((rows, heads, 128), dtype=np.uint16)
    out = gpu.tensor(np.zeros(q.shape, dtype=np.uint16))
    tq, tk = gpu.tensor(q), gpu.tensor(k)
    assert gpu.lib.h3_gpu_vsa_bf16(handle, out, tq, tk, gpu.tensor(v), gpu.tensor(gate)), gpu.error()
    buffer = gpu.lib.h3b_vsa_buffer
    indices = gpu.read_device(buffer(handle, 9), (heads, tiles, tiles), np.int32)
    counts = gpu.read_device(buffer(handle, 10), (heads, tiles), np.int32)
    return dict(handle=handle, tiles=tiles, prefix=prefix, keep=keep, heads=heads, q=tq, k=tk,
                map=buffer(handle, 0), sizes=buffer(handle, 1), indices=indices, counts=counts)


def static_path(gpu, case):
    heads, tiles = case["heads"], case["tiles"]
    indices = gpu.tensor(np.full((heads, tiles, tiles), -7, dtype=np.int32))
    counts = gpu.tensor(np.full((heads, tiles), -7, dtype=np.int32))
    data = gpu.lib.h3b_tensor_data
    code = gpu.lib.h3b_vsa_topk_static(data(case["q"]), data(case["k"]), case["map"], case["sizes"],
                                       data(indices), data(counts), tiles, case["prefix"],
                                       case["keep"], heads, gpu.lib.h3b_gpu_stream(gpu.gpu))
    assert code == 0, C.string_at(gpu.lib.h3b_vsa_topk_static_error()).decode()
    return (gpu.read(indices, (heads, tiles, tiles), np.int32),
            gpu.read(counts, (heads, tiles), np.int32))


def free_device_bytes():
    """Free device memory as the CUDA runtime reports it (after everything queued has run)."""
    from h3_omni_b200 import native
    rt = native._cudart()
    free, total = C.c_size_t(), C.c_size_t()
    assert rt.cudaDeviceSynchronize() == 0
    assert rt.cudaMemGetInfo(C.byref(free), C.byref(total)) == 0
    return free.value


def test_static_topk_leaves_device_memory_as_it_found_it(gpu, oracle):
    """The point of the entry point: a call allocates nothing. The tensors of the call are made
    first, one call runs to set the scratch address up, then the amount of free device memory is
    read before and after two more calls (on the stream, no tensor created in between)."""
    case = regular_path(gpu, oracle, 17, 30, (7, 8, 8), 3, 4400)
    try:
        heads, tiles = case["heads"], case["tiles"]
        indices = gpu.tensor(np.zeros((heads, tiles, tiles), dtype=np.int32))
        counts = gpu.tensor(np.zeros((heads, tiles), dtype=np.int32))
        data, stream = gpu.lib.h3b_tensor_data, gpu.lib.h3b_gpu_stream(gpu.gpu)

        def call():
            return gpu.lib.h3b_vsa_topk_static(data(case["q"]), data(case["k"]), case["map"], case["sizes"], data(indices),
                                               data(counts), tiles, case["prefix"], case["keep"], heads, stream)

        assert call() == 0
        before = free_device_bytes()
        assert call() == 0 and call() == 0
        assert free_device_bytes() == before
        same_lists(case, gpu.read(indices, (heads, tiles, tiles), np.int32), gpu.read(counts, (heads, tiles), np.int32))
    finally:
        gpu.lib.h3_gpu_vsa_free(case["handle"])


def same_lists(case, indices, counts):
    assert np.array_equal(counts, case["counts"])
    valid = np.arange(case["tiles"])[None, None, :] < counts[:, :, None]
    assert np.array_equal(indices[valid], case["indices"][valid])


def test_static_topk_matches_regular_path_twice(gpu, oracle):
    first = regular_path(gpu, oracle, 65, 67, (5, 7, 9), 4, 4100)
    second = regular_path(gpu, oracle, 17, 448, (37, 15, 27), 8, 4200)
    try:
        same_lists(first, *static_path(gpu, first))      # first call sets the scratch up
        same_lists(second, *static_path(gpu, second))    # second call reuses it, other shape
        same_lists(first, *static_path(gpu, first))      # and back: no stale contents leak
        assert gpu.device_status() == 0
    finally:
        gpu.lib.h3_gpu_vsa_free(first["handle"])
        gpu.lib.h3_gpu_vsa_free(second["handle"])


def test_static_topk_rejects_shapes_beyond_its_scratch(gpu, oracle):
    case = regular_path(gpu, oracle, 3, 11, (1, 2, 3), 2, 4300)
    try:
        data = gpu.lib.h3b_tensor_data
        sink = gpu.tensor(np.zeros(16, dtype=np.int32))
        # 56 heads x 288 tiles = 16128 rows of pooled means > 8192
        code = gpu.lib.h3b_vsa_topk_static(data(case["q"]), data(case["k"]), case["map"],
                                           case["sizes"], data(sink), data(sink), 288, 8, 28, 56, None)
        assert code != 0
        message = C.string_at(gpu.lib.h3b_vsa_topk_static_error()).decode()
        assert "exceeds the static scratch limit of 8192" in message
        assert gpu.lib.h3b_vsa_topk_static(None, None, None, None, None, None, 3, 2, 1, 2, None) != 0
        assert np.array_equal(gpu.read(sink, (16,), np.int32), np.zeros(16, dtype=np.int32))
    finally:
        gpu.lib.h3_gpu_vsa_free(case["handle"])
