"""Q/K RMS-norm + rotary embedding (the producer of the attention inputs) through the C ABI.

The reference pins this operator by demanding bit equality between its two kernels
(tests/serving/profile/elementwise_bench.cu:179-188); its model-level test
(tests/test_bf16.c:1551-1590) needs checkpoint fixtures that are not available. Here:
  - CPU: the oracle against a float64 restatement of the mathematics;
  - GPU: the CUDA kernel against the oracle (identical except where the GPU's approximate
    rsqrt decides a bf16 rounding: a small fraction of elements, by one rounding step, the
    copied V exact), and bit-exact against the reference's own kernel run on the same GPU;
  - the fused sinks (VSA tile order + tile means, Ulysses head shards) bit-exact against the
    unfused sequence of calls.
"""
import ctypes as C

import numpy as np
import pytest

from conftest import ROPE_HALF, assert_rope_close, rope_inputs
from refbackend import REF_LIB, Reference

HALF = ROPE_HALF
make_inputs = rope_inputs


def float64_restatement(oracle, qkv, qw, kw, co, si, heads, grouped):
    rows = qkv.shape[0]
    x = oracle.from_bf16(qkv).astype(np.float64)
    x = x.reshape(rows, heads, 3, 128) if grouped else x.reshape(rows, 3, heads, 128).transpose(0, 2, 1, 3)
    c, s = oracle.from_bf16(co)[:, None, :].astype(np.float64), oracle.from_bf16(si)[:, None, :].astype(np.float64)

    def one(v, w):
        n = v / np.sqrt((v * v).mean(-1, keepdims=True) + 1e-5) * oracle.from_bf16(w)
        out = n.copy()
        out[..., :HALF] = n[..., :HALF] * c - n[..., HALF:2 * HALF] * s
        out[..., HALF:2 * HALF] = n[..., HALF:2 * HALF] * c + n[..., :HALF] * s
        return out
    return one(x[:, :, 0], qw), one(x[:, :, 1], kw), x[:, :, 2]


@pytest.mark.parametrize("grouped", [True, False])
def test_oracle_matches_float64_mathematics(oracle, grouped):
    rows, heads = 37, 5
    qkv, qw, kw, co, si = make_inputs(oracle, rows, heads, 5)
    q, k, v = oracle.qkv_rope(qkv, qw, kw, co, si, heads, HALF, 1e-5, grouped)
    wq, wk, wv = float64_restatement(oracle, qkv, qw, kw, co, si, heads, grouped)
    # three bf16 roundings of values up to ~8: a few bf16 ulps of 8 (2^-5)
    assert np.abs(oracle.from_bf16(q) - wq).max() < 0.1
    assert np.abs(oracle.from_bf16(k) - wk).max() < 0.1
    assert np.array_equal(oracle.from_bf16(v).astype(np.float64), wv)
    # dimensions >= 2 * rope_half are not rotated: one rounding only
    assert np.abs(oracle.from_bf16(q)[..., 2 * HALF:] - wq[..., 2 * HALF:]).max() < 0.04


def run_ours(gpu, name, qkv, qw, kw, co, si, rows, heads):
    tensors = [gpu.tensor(x) for x in (qkv, qw, kw, co, si)]
    outs = [gpu.empty_bf16(rows * heads * 128) for _ in range(3)]
    gpu.call(name, *outs, *tensors, rows, heads, 128, HALF, 1e-5)
    result = [gpu.read(t, (rows, heads, 128)) for t in outs]
    for t in tensors + outs:
        gpu.free(t)
    return result


@pytest.mark.gpu
@pytest.mark.parametrize("rows,heads,grouped", [(1, 1, True), (37, 5, True), (37, 5, False), (1000, 24, True),
                                                (263, 56, True), (263, 56, False)])
def test_kernel_against_oracle(gpu, oracle, rows, heads, grouped):
    qkv, qw, kw, co, si = make_inputs(oracle, rows, heads, 40 + rows)
    name = "grouped_qkv_rope_bf16" if grouped else "qkv_rope_bf16"
    q, k, v = run_ours(gpu, name, qkv, qw, kw, co, si, rows, heads)
    wq, wk, wv = oracle.qkv_rope(qkv, qw, kw, co, si, heads, HALF, 1e-5, grouped)
    assert np.array_equal(v, wv)
    assert_rope_close(oracle, q, wq)
    assert_rope_close(oracle, k, wk)


@pytest.mark.gpu
def test_rejects_unsupported_shapes(gpu, oracle):
    qkv, qw, kw, co, si = make_inputs(oracle, 4, 2, 1)
    tensors = [gpu.tensor(x) for x in (qkv, qw, kw, co, si)]
    outs = [gpu.empty_bf16(4 * 2 * 128) for _ in range(3)]
    with pytest.raises(RuntimeError, match="not supported"):
        gpu.call("qkv_rope_bf16", *outs, *tensors, 4, 4, 64, 16, 1e-5)
    with pytest.raises(RuntimeError, match="not supported"):
        gpu.call("qkv_rope_bf16", *outs, *tensors, 4, 2, 128, 46, 1e-5)
    small = gpu.empty_bf16(16)
    with pytest.raises(RuntimeError, match="query"):
        gpu.call("qkv_rope_bf16", small, outs[1], outs[2], *tensors, 4, 2, 128, HALF, 1e-5)


@pytest.fixture(scope="module")
def ref(gpu):
    if not REF_LIB.exists():
        pytest.skip("oracle/_ref/libh3_ref_cuda.so not built (needs the reference tree at build time)")
    r = Reference()
    yield r
    r.close()


@pytest.mark.gpu
@pytest.mark.parametrize("rows,heads,grouped", [(37, 5, True), (37, 5, False), (1031, 24, True), (263, 56, True)])
def test_bit_exact_against_reference_kernel(gpu, ref, oracle, rows, heads, grouped):
    """The reference's h3_fast_qkv_rope_bf16 (cuda/fast_primitives.cuh:184-265), compiled from
    its own source, on the same GPU and inputs."""
    qkv, qw, kw, co, si = make_inputs(oracle, rows, heads, 90 + rows)
    name = "grouped_qkv_rope_bf16" if grouped else "qkv_rope_bf16"
    mine = run_ours(gpu, name, qkv, qw, kw, co, si, rows, heads)
    outs = [ref.empty(rows * heads * 128) for _ in range(3)]
    fn = getattr(ref.lib, "h3_gpu_" + name)
    fn.argtypes = [C.c_void_p] * 9 + [C.c_uint32] * 4 + [C.c_float]
    ref.check(fn(ref.gpu, *outs, *[ref.tensor(x) for x in (qkv, qw, kw, co, si)], rows, heads, 128, HALF, 1e-5),
              name)
    for got, t in zip(mine, outs):
        assert np.array_equal(got, ref.read(t, (rows, heads, 128)))


@pytest.mark.gpu
@pytest.mark.parametrize("text,audio,shape,heads", [(3, 11, (1, 2, 3), 2), (65, 67, (5, 7, 9), 5),
                                                    (17, 30, (7, 8, 8), 24)])
def test_vsa_fed_by_projection_equals_two_calls(gpu, oracle, text, audio, shape, heads):
    """h3b_vsa_qkv_rope_bf16 == h3_gpu_grouped_qkv_rope_bf16 + h3_gpu_vsa_bf16, bit for bit,
    in the output and in every work buffer."""
    handle = gpu.call("vsa_new", text, audio, *shape, heads)
    info = [C.c_int() for _ in range(4)]
    assert gpu.lib.h3b_vsa_info(handle, *[C.byref(x) for x in info])
    rows, tiles = info[0].value, info[1].value
    qkv, qw, kw, co, si = make_inputs(oracle, rows, heads, 7)
    gate = oracle.normal_bf16((rows, heads, 128), 8, 0.3)
    n = rows * heads * 128
    tin = [gpu.tensor(x) for x in (qkv, qw, kw, co, si)]
    tgate = gpu.tensor(gate)
    shapes = {2: ((heads, tiles * 64, 128), np.uint16), 3: ((heads, tiles * 64, 128), np.uint16),
              4: ((heads, tiles * 64, 128), np.uint16), 6: ((heads, tiles, 128), np.float32),
              7: ((heads, tiles, 128), np.float32), 8: ((heads, tiles, 128), np.float32),
              9: ((heads, tiles, tiles), np.int32), 10: ((heads, tiles), np.int32),
              11: ((heads, tiles, 128), np.float32)}

    def buffers():
        return {w: gpu.read_device(gpu.lib.h3b_vsa_buffer(handle, w), s, d) for w, (s, d) in shapes.items()}
    q, k, v, out_a, out_b = (gpu.empty_bf16(n) for _ in range(5))
    gpu.call("grouped_qkv_rope_bf16", q, k, v, *tin, rows, heads, 128, HALF, 1e-5)
    assert gpu.lib.h3_gpu_vsa_bf16(handle, out_a, q, k, v, tgate), gpu.error()
    want_out, want = gpu.read(out_a, (rows, heads, 128)), buffers()
    assert gpu.lib.h3b_vsa_qkv_rope_bf16(handle, out_b, *tin, tgate, HALF, C.c_float(1e-5), 1), gpu.error()
    got_out, got = gpu.read(out_b, (rows, heads, 128)), buffers()
    counts = want[10]
    for w in shapes:
        if w == 9:   # index lists are defined up to counts[h][q] entries
            for h in range(heads):
                for t in range(tiles):
                    c = counts[h, t]
                    assert np.array_equal(got[9][h, t, :c], want[9][h, t, :c])
        else:
            assert np.array_equal(got[w], want[w]), "work buffer %d differs" % w
    assert np.array_equal(got_out, want_out)
    assert gpu.device_status() == 0
    gpu.lib.h3_gpu_vsa_free(handle)
    for t in tin + [tgate, q, k, v, out_a, out_b]:
        gpu.free(t)


@pytest.mark.gpu
def test_single_rank_fused_scatter_is_token_major(gpu, oracle):
    """With one rank the head shard of every head is this rank's own slot, laid out like the
    token-major output."""
    rows, heads = 203, 6
    qkv, qw, kw, co, si = make_inputs(oracle, rows, heads, 17)
    want = run_ours(gpu, "grouped_qkv_rope_bf16", qkv, qw, kw, co, si, rows, heads)
    x, handle = C.c_void_p(), (C.c_ubyte * 64)()
    assert gpu.lib.h3b_exchange_create(gpu.gpu, 0, 1, rows * heads * 128, 3, C.byref(x), handle), gpu.error()
    assert gpu.lib.h3b_exchange_connect(x, bytes(handle)), gpu.error()
    tin = [gpu.tensor(a) for a in (qkv, qw, kw, co, si)]
    assert gpu.lib.h3b_exchange_qkv_rope_scatter_bf16(x, 2, 0, 1, *tin, rows, heads, HALF, C.c_float(1e-5), 1), \
        gpu.error()
    slots = [gpu.lib.h3b_exchange_slot(x, i) for i in range(3)]
    for slot, expect in zip((2, 0, 1), want):
        assert np.array_equal(gpu.read(slots[slot], (rows, heads, 128)), expect)
    assert not gpu.lib.h3b_exchange_qkv_rope_scatter_bf16(x, 0, 0, 1, *tin, rows, heads, HALF, C.c_float(1e-5), 1)
    assert gpu.device_status() == 0
    for t in slots:
        gpu.lib.h3_gpu_tensor_free(t)
    for t in tin:
        gpu.free(t)
    gpu.lib.h3b_exchange_free(x)
