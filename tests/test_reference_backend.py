"""The reference's own CUDA backend, built unmodified from its tree and linked against this
library (oracle/ref_build.py), as a live checker on the GPU box.

Two things are checked here that no CPU test can check:
  1. Drop-in: the reference's wrappers (h3_gpu_sdpa_bf16, h3_gpu_cross_attention_bf16,
     h3_gpu_vsa_bf16 of reference cuda/h3_gpu_cuda.cu and cuda/vsa.cuh) run on this library's
     kernels through the five kernel-adapter symbols and give correct results.
  2. Pinning: reference code that still runs on a B200 by itself - the FP32 fallback attention,
     tile pooling, cuBLAS pooled scores, block selection, pooled softmax, compression, merge -
     agrees with the CPU oracle and with this library's replacements for it.
"""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

from conftest import assert_attention_close, metrics
from refbackend import REF_LIB, Reference, ref_vsa_buffers

pytestmark = pytest.mark.gpu
SCALE = float(1.0 / np.sqrt(128.0))


@pytest.fixture(scope="module")
def ref(gpu):
    if not REF_LIB.exists():
        pytest.skip("oracle/_ref/libh3_ref_cuda.so not built (needs the reference tree at build time)")
    r = Reference()
    yield r
    r.close()


@pytest.mark.parametrize("L,H", [(7, 2), (263, 4), (1000, 8), (2048, 56)])
def test_reference_sdpa_wrapper_runs_on_our_kernel(ref, gpu, oracle, L, H):
    """reference h3_gpu_sdpa_bf16 -> sdpa() -> h3_flash3_bf16 (ours). Same bits as our own
    primitive layer, and within the acceptance limits of the FP32 oracle."""
    q, k, v = (oracle.normal_bf16((L, H, 128), 11 + i) for i in range(3))
    y = ref.empty(q.size)
    ref.check(ref.lib.h3_gpu_sdpa_bf16(ref.gpu, y, ref.tensor(q), ref.tensor(k), ref.tensor(v), L, H, 128, SCALE), "sdpa")
    got = ref.read(y, q.shape)
    want, _ = oracle.attention(q[None], k[None], v[None], SCALE)
    assert_attention_close(oracle.from_bf16(got), want[0])
    mine = gpu.empty_bf16(q.size)
    gpu.call("sdpa_bf16", mine, gpu.tensor(q), gpu.tensor(k), gpu.tensor(v), L, H, 128, SCALE)
    assert np.array_equal(gpu.read(mine, q.shape), got)
    y2 = ref.empty(q.size)
    ref.check(ref.lib.h3_gpu_sdpa_fa2_bf16(ref.gpu, y2, ref.tensor(q), ref.tensor(k), ref.tensor(v), L, H, 128, SCALE), "fa2")
    assert np.array_equal(ref.read(y2, q.shape), got)


def test_reference_live_wrapper_runs_on_our_kernel(ref, oracle):
    """reference h3_gpu_cross_attention_bf16 -> h3_flash3_cross_bf16 (ours), two-call pattern."""
    text, media, history, H = 33, 405, 1215, 7
    total_k = text + history + media
    q = oracle.normal_bf16((text + media, H, 128), 21)
    k = oracle.normal_bf16((total_k, H, 128), 22)
    v = oracle.normal_bf16((total_k, H, 128), 23)
    tq, tk, tv = ref.tensor(q), ref.tensor(k), ref.tensor(v)
    y = ref.tensor(np.zeros(q.shape, dtype=np.uint16))
    ref.check(ref.lib.h3_gpu_cross_attention_bf16(ref.gpu, y, 0, tq, 0, tk, tv, 0, text, text, H), "text")
    ref.check(ref.lib.h3_gpu_cross_attention_bf16(ref.gpu, y, text, tq, text, tk, tv, 0, media, total_k, H), "media")
    got = oracle.from_bf16(ref.read(y, q.shape))
    a, _ = oracle.attention(q[None, :text], k[None, :text], v[None, :text], SCALE)
    b, _ = oracle.attention(q[None, text:], k[None], v[None], SCALE)
    m = assert_attention_close(got, np.concatenate([a[0], b[0]]))
    assert m["rel_l2"] < 0.004


@pytest.mark.parametrize("L,H", [(65, 2), (300, 4), (700, 3)])
def test_reference_fp32_fallback_pins_the_cpu_oracle(ref, oracle, L, H):
    """reference h3_gpu_sdpa_f32 on F32 tensors takes its own FP32 path (cuBLAS SGEMM +
    softmax_rows, cuda/h3_gpu_cuda.cu:1131-1180) - the arithmetic the CPU oracle restates."""
    q, k, v = (oracle.normal_bf16((L, H, 128), 31 + i) for i in range(3))
    qf, kf, vf = (oracle.from_bf16(x) for x in (q, k, v))
    y = ref.empty(q.size, f32=True)
    ref.check(ref.lib.h3_gpu_sdpa_f32(ref.gpu, y, ref.tensor(qf), ref.tensor(kf), ref.tensor(vf), L, H, 128, SCALE), "sdpa_f32")
    got = ref.read(y, q.shape, f32=True)
    want, _ = oracle.attention(q[None], k[None], v[None], SCALE)
    assert np.abs(got - want[0]).max() < 5e-6
    assert metrics(got, want[0])["rel_l2"] < 2e-6


@pytest.mark.parametrize("text,audio,shape,heads", [(65, 67, (5, 7, 9), 4), (17, 30, (7, 8, 8), 56),
                                                     (17, 448, (37, 15, 27), 4)])
def test_reference_vsa_orchestration_against_ours(ref, gpu, oracle, text, audio, shape, heads):
    """reference h3_gpu_vsa_bf16: its own tile_pool, cuBLAS scores, select_blocks, pooled
    softmax, cuBLAS compression and untile_merge around OUR h3_vsa_hopper - compared stage by
    stage with this library's h3_gpu_vsa_bf16 on the same inputs."""
    vmap = oracle.VsaMap(text, audio, *shape)
    T = vmap.tiles
    q, k, v = (oracle.normal_bf16((vmap.rows, heads, 128), 700 + i) for i in range(3))
    gate = oracle.normal_bf16((vmap.rows, heads, 128), 703, 0.3)
    rh = ref.lib.h3_gpu_vsa_new(ref.gpu, text, audio, *shape, heads)
    ref.check(rh, "vsa_new")
    out = ref.tensor(np.zeros(q.shape, dtype=np.uint16))
    ref.check(ref.lib.h3_gpu_vsa_bf16(rh, out, ref.tensor(q), ref.tensor(k), ref.tensor(v), ref.tensor(gate)), "vsa")
    ref_out = ref.read(out, q.shape)
    dev = ref_vsa_buffers(ref, rh, heads, T)
    rd = gpu.read_device
    ref_map = rd(dev["map"], (T * 64,), np.int32)
    ref_sizes = rd(dev["sizes"], (T,), np.int32)
    ref_pool = [rd(dev[n], (heads, T, 128), np.float32) for n in ("poolq", "poolk", "poolv")]
    ref_tiled_q = rd(dev["q"], (heads, T * 64, 128), np.uint16)
    ref_counts = rd(dev["counts"], (heads, T), np.int32)
    ref_indices = rd(dev["indices"], (heads, T, T), np.int32)
    ref_prob = rd(dev["scores"], (heads, T, T), np.float32)      # softmax-ed in place by then
    ref_comp = rd(dev["compression"], (heads, T, 128), np.float32)
    ref.lib.h3_gpu_vsa_free(rh)

    # the tile map and the pooled means of the reference pin the CPU oracle bit for bit
    assert np.array_equal(ref_map, vmap.map) and np.array_equal(ref_sizes, vmap.sizes)
    stages = oracle.vsa_forward(q, k, v, gate, vmap)
    assert np.array_equal(ref_tiled_q, stages["tiled"][0])
    for i in range(3):
        assert np.array_equal(ref_pool[i].view(np.uint32), stages["pooled"][i].view(np.uint32))

    # selection: the reference sorts cuBLAS scores, we sort fixed-order fmaf scores; the lists
    # must agree except where the k-th and (k+1)-th scores are within FP32 rounding of each other
    assert np.array_equal(ref_counts, stages["counts"])
    valid = np.arange(T)[None, None, :] < ref_counts[:, :, None]
    differ = 0
    for h in range(heads):
        for qt in range(vmap.prefix, T):
            a = set(ref_indices[h, qt, :ref_counts[h, qt]])
            b = set(stages["indices"][h, qt, :stages["counts"][h, qt]])
            if a != b:
                differ += 1
                s = stages["scores"][h, qt]
                swapped = sorted(a ^ b)
                spread = max(s[swapped]) - min(s[swapped])
                assert spread <= 1e-5 * max(1.0, np.abs(s).max()), (h, qt, swapped, spread)
    assert differ <= max(1, heads * T // 200), differ

    # pooled softmax and compression of the reference pin the oracle's restatement
    assert np.abs(ref_prob - stages["prob"]).max() < 1e-6
    assert np.abs(ref_comp - stages["compression"]).max() < 2e-5

    # end to end: reference orchestration + our fine kernel vs this library's whole pipeline
    ours = gpu.call("vsa_new", text, audio, *shape, heads)
    try:
        y = gpu.tensor(np.zeros(q.shape, dtype=np.uint16))
        assert gpu.lib.h3_gpu_vsa_bf16(ours, y, gpu.tensor(q), gpu.tensor(k), gpu.tensor(v), gpu.tensor(gate)), gpu.error()
        mine = gpu.read(y, q.shape)
    finally:
        gpu.lib.h3_gpu_vsa_free(ours)
    a, b = oracle.from_bf16(ref_out).astype(np.float64), oracle.from_bf16(mine).astype(np.float64)
    if differ == 0:
        # same lists -> same fine-stage inputs; only the compression GEMM's summation order differs
        assert np.abs(a - b).max() <= 2 ** -6 * max(1.0, np.abs(a).max())
        assert (ref_out != mine).mean() < 0.02
    rel = np.linalg.norm(a - b) / np.linalg.norm(a)
    assert rel < 0.012 and np.abs(a - b).max() / np.abs(a).max() < 0.03
