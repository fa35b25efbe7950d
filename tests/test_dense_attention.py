"""Dense, rectangular, causal/GQA and fp16 attention through the C ABI against the CPU oracle.

Shapes follow the reference's own primitive tests (tests/pytorch/primitives.py:93-136: odd
lengths 7/128/263, GQA, causal) and its live-mode test (tests/live/attention.py:16-38: the
two-call text/media pattern with row offsets), plus tile-boundary lengths for the 128-row
tcgen05 tiles.
"""
import ctypes as C

import numpy as np
import pytest

from conftest import assert_attention_close

pytestmark = pytest.mark.gpu
SCALE = float(1.0 / np.sqrt(128.0))


def run_sdpa(gpu, oracle, L, H, seed, primitive="sdpa_bf16"):
    q, k, v = (oracle.normal_bf16((1, L, H, 128), seed + i) for i in range(3))
    ty = gpu.empty_bf16(q.size)
    tq, tk, tv = gpu.tensor(q), gpu.tensor(k), gpu.tensor(v)
    gpu.call(primitive, ty, tq, tk, tv, L, H, 128, SCALE)
    got = oracle.from_bf16(gpu.read(ty, q.shape))
    want, _ = oracle.attention(q, k, v, SCALE)
    for t in (ty, tq, tk, tv):
        gpu.free(t)
    return got, want


@pytest.mark.parametrize("L", [1, 7, 63, 64, 65, 127, 128, 129, 255, 256, 257, 263, 300, 1000])
def test_sdpa_bf16_lengths(gpu, oracle, L):
    got, want = run_sdpa(gpu, oracle, L, 3, 100 + L)
    assert_attention_close(got, want)
    assert gpu.device_status() == 0


@pytest.mark.parametrize("L,H", [(2048, 8), (1536, 56), (4096, 2)])
def test_sdpa_bf16_larger(gpu, oracle, L, H):
    got, want = run_sdpa(gpu, oracle, L, H, 7 * L + H)
    assert_attention_close(got, want)
    assert gpu.device_status() == 0


@pytest.mark.parametrize("nq,nk,heads", [(64, 9000, 4), (200, 16001, 3), (300, 33000, 2), (1, 5000, 24)])
def test_short_query_block_against_long_keys_split_kv(gpu, oracle, nq, nk, heads):
    """Live mode's text rows against the whole KV history (h3_dit_live.inc:95): too few query tiles
    to fill the GPU, so the keys are cut into slices computed side by side and merged by their
    logsumexp. Same limits as every dense call, ragged last slice included, and the kernel-adapter
    symbol's logsumexp output against the FP32 recomputation."""
    q = oracle.normal_bf16((1, nq, heads, 128), 31)
    k, v = (oracle.normal_bf16((1, nk, heads, 128), 32 + i) for i in range(2))
    tq, tk, tv = gpu.tensor(q), gpu.tensor(k), gpu.tensor(v)
    ty = gpu.tensor(np.full(q.shape, 0x7fc0, dtype=np.uint16))
    gpu.call("cross_attention_bf16", ty, 0, tq, 0, tk, tv, 0, nq, nk, heads)
    want, _, want_lse = oracle.attention(q, k, v, SCALE, want_lse=True)
    assert_attention_close(oracle.from_bf16(gpu.read(ty, q.shape)), want)
    tl = gpu.tensor(np.zeros((heads, nq), dtype=np.float32))
    d = gpu.lib.h3b_tensor_data
    gpu.raw("h3_flash3_cross_bf16", d(ty), d(tq), d(tk), d(tv), d(tl), nq, nk, heads, C.c_float(SCALE),
            gpu.lib.h3b_gpu_stream(gpu.gpu))
    assert np.abs(gpu.read(tl, (heads, nq), np.float32) - want_lse.reshape(heads, nq)).max() <= 2e-3
    assert gpu.device_status() == 0


def test_c1_dense_l4096_h8(gpu, oracle):
    """Benchmark configuration 1 exactly: Q, K, V bf16 [1, 8, 4096, 128] from N(0, 1), seed 1001,
    scale 1/sqrt(128), no mask; max-abs <= 1e-2 and cosine >= 0.9999 against the FP32
    recomputation (the whole output, every row)."""
    got, want = run_sdpa(gpu, oracle, 4096, 8, 1001)
    m = assert_attention_close(got, want)
    assert m["rel_l2"] <= 0.004   # the level the reference's own kernel is held to on live shapes
    assert gpu.device_status() == 0


def test_sdpa_fa2_entry_matches_flash3_entry(gpu, oracle):
    """h3_gpu_sdpa_fa2_bf16 (FlashAttention-2 adapter path) and h3_gpu_sdpa_bf16 agree."""
    a, want = run_sdpa(gpu, oracle, 263, 4, 5, "sdpa_bf16")
    b, _ = run_sdpa(gpu, oracle, 263, 4, 5, "sdpa_fa2_bf16")
    assert_attention_close(b, want)
    assert np.array_equal(a, b)


def test_sdpa_uniform_distribution(gpu, oracle):
    """Second input distribution of the reference's attention microbenchmark
    (tests/serving/profile/attn_bench.cu:95-98): Q, K ~ U(-2, 2), V ~ U(-1, 1)."""
    rng = np.random.default_rng(99)
    L, H = 700, 4
    q = oracle.to_bf16(rng.uniform(-2, 2, (1, L, H, 128)))
    k = oracle.to_bf16(rng.uniform(-2, 2, (1, L, H, 128)))
    v = oracle.to_bf16(rng.uniform(-1, 1, (1, L, H, 128)))
    ty = gpu.empty_bf16(q.size)
    gpu.call("sdpa_bf16", ty, gpu.tensor(q), gpu.tensor(k), gpu.tensor(v), L, H, 128, SCALE)
    got = oracle.from_bf16(gpu.read(ty, q.shape))
    want, _ = oracle.attention(q, k, v, SCALE)
    assert_attention_close(got, want)


def test_sdpa_large_logits_rescale(gpu, oracle):
    """Rows whose maximum keeps growing exercise the lazy accumulator rescale."""
    L, H = 640, 2
    q = oracle.normal_bf16((1, L, H, 128), 41, 3.0)
    k = oracle.from_bf16(oracle.normal_bf16((1, L, H, 128), 42, 1.0))
    k *= np.linspace(0.2, 4.0, L, dtype=np.float32)[None, :, None, None]  # later keys larger
    k = oracle.to_bf16(k)
    v = oracle.normal_bf16((1, L, H, 128), 43)
    ty = gpu.empty_bf16(q.size)
    gpu.call("sdpa_bf16", ty, gpu.tensor(q), gpu.tensor(k), gpu.tensor(v), L, H, 128, SCALE)
    got = oracle.from_bf16(gpu.read(ty, q.shape))
    want, _ = oracle.attention(q, k, v, SCALE)
    assert_attention_close(got, want, max_abs=2e-2)


@pytest.mark.parametrize("L,H,KH", [(7, 8, 2), (128, 8, 2), (263, 8, 4), (263, 6, 1)])
@pytest.mark.parametrize("causal", [False, True])
def test_flash_bf16_gqa_causal(gpu, oracle, L, H, KH, causal):
    """h3_flash_bf16 directly: causal and grouped-query, batch 2, with logsumexp."""
    B = 2
    q = oracle.normal_bf16((B, L, H, 128), 1000 + L)
    k = oracle.normal_bf16((B, L, KH, 128), 2000 + L)
    v = oracle.normal_bf16((B, L, KH, 128), 3000 + L)
    ty = gpu.empty_bf16(q.size)
    tq, tk, tv = gpu.tensor(q), gpu.tensor(k), gpu.tensor(v)
    tl = gpu.tensor(np.zeros((B, H, L), dtype=np.float32))
    data = gpu.lib.h3b_tensor_data
    gpu.raw("h3_flash_bf16", data(ty), data(tq), data(tk), data(tv), data(tl), B, L, H, KH, SCALE,
            causal, gpu.lib.h3b_gpu_stream(gpu.gpu))
    got = oracle.from_bf16(gpu.read(ty, q.shape))
    lse = gpu.read(tl, (B, H, L), np.float32)
    want, _, want_lse = oracle.attention(q, k, v, SCALE, causal=causal, want_lse=True)
    assert_attention_close(got, want)
    assert np.abs(lse - want_lse).max() < 2e-3
    assert gpu.device_status() == 0


def test_gqa_causal_primitive(gpu, oracle):
    """h3_gpu_gqa_causal_bf16 (reference h3_gpu.h:534-540), the text-encoder call."""
    L, H, KH = 150, 16, 2
    q = oracle.normal_bf16((1, L, H, 128), 1)
    k = oracle.normal_bf16((1, L, KH, 128), 2)
    v = oracle.normal_bf16((1, L, KH, 128), 3)
    ty = gpu.empty_bf16(q.size)
    gpu.call("gqa_causal_bf16", ty, gpu.tensor(q), gpu.tensor(k), gpu.tensor(v), L, H, KH, 128, SCALE)
    got = oracle.from_bf16(gpu.read(ty, q.shape))
    want, _ = oracle.attention(q, k, v, SCALE, causal=True)
    assert_attention_close(got, want)


@pytest.mark.parametrize("L,H", [(7, 2), (64, 3), (263, 4), (1030, 2)])
def test_sdpa_f16_d64(gpu, oracle, L, H):
    """h3_gpu_sdpa_f16_d64: fp16, head dim 64 (video VAE call, reference cuda/vae_fp16.cuh:275-296)."""
    from h3_omni_b200 import native
    rng = np.random.default_rng(L)
    q, k, v = (oracle.to_f16(rng.standard_normal((1, L, H, 64))) for _ in range(3))
    ty = gpu.empty_f16(q.size)
    gpu.call("sdpa_f16_d64", ty, gpu.tensor(q, native.F16), gpu.tensor(k, native.F16),
             gpu.tensor(v, native.F16), L, H, 64, 0.125)
    got = oracle.from_f16(gpu.read(ty, q.shape))
    want, _ = oracle.attention(q, k, v, 0.125, elem="f16")
    assert_attention_close(got, want, max_abs=5e-3, rel_l2=0.004)


def test_sdpa_rejects_bad_arguments(gpu, oracle):
    """Error behaviour of the primitive layer: 0 + message, no launch."""
    q = gpu.tensor(oracle.normal_bf16((4, 2, 128), 1))
    f = gpu.tensor(np.zeros(4 * 2 * 128, dtype=np.float32))
    y = gpu.empty_bf16(4 * 2 * 128)
    with pytest.raises(RuntimeError, match="need 2048 elements"):
        gpu.call("sdpa_bf16", y, q, q, q, 8, 2, 128, SCALE)
    with pytest.raises(RuntimeError, match="expected BF16"):
        gpu.call("sdpa_bf16", y, f, q, q, 4, 2, 128, SCALE)
    with pytest.raises(RuntimeError, match="head dimension 128"):
        gpu.call("sdpa_bf16", y, q, q, q, 4, 4, 64, SCALE)
    assert gpu.lib.h3_flash3_bf16(None, None, None, None, None, 1, 4, 2, 2, SCALE, None) != 0
    assert gpu.lib.h3_flash3_bf16(gpu.lib.h3b_tensor_data(y), gpu.lib.h3b_tensor_data(q),
                                  gpu.lib.h3b_tensor_data(q), gpu.lib.h3b_tensor_data(q), None, 1,
                                  4, 3, 2, SCALE, None) != 0  # 3 heads do not group over 2


def live_case(gpu, oracle, text, media, history, H, seed):
    """Two-call live pattern (reference h3_dit_live.inc:88-99, tests/live/attention.py:16-38):
    K/V rows are [text | history | current media]; text queries attend text only, media
    queries attend everything."""
    total_q = text + media
    total_k = text + history + media
    q = oracle.normal_bf16((total_q, H, 128), seed)
    k = oracle.normal_bf16((total_k, H, 128), seed + 1)
    v = oracle.normal_bf16((total_k, H, 128), seed + 2)
    tq, tk, tv = gpu.tensor(q), gpu.tensor(k), gpu.tensor(v)
    ty = gpu.tensor(np.zeros(q.shape, dtype=np.uint16))
    gpu.call("cross_attention_bf16", ty, 0, tq, 0, tk, tv, 0, text, text, H)
    gpu.call("cross_attention_bf16", ty, text, tq, text, tk, tv, 0, media, total_k, H)
    got = oracle.from_bf16(gpu.read(ty, q.shape))
    want_text, _ = oracle.attention(q[None, :text], k[None, :text], v[None, :text], SCALE)
    want_media, _ = oracle.attention(q[None, text:], k[None], v[None], SCALE)
    want = np.concatenate([want_text[0], want_media[0]])
    return got, want


@pytest.mark.parametrize("text,media,history,H", [(17, 100, 0, 4), (77, 300, 500, 4),
                                                   (128, 405, 1215, 7), (5, 64, 3000, 2)])
def test_live_cross_attention(gpu, oracle, text, media, history, H):
    got, want = live_case(gpu, oracle, text, media, history, H, text + media)
    m = assert_attention_close(got, want)
    assert m["rel_l2"] < 0.004  # the reference's own limit, tests/live/attention.py:38
    assert gpu.device_status() == 0


def test_cross_attention_row_offsets_leave_other_rows(gpu, oracle):
    """Output rows outside [out_row, out_row + query_rows) are not touched."""
    H = 2
    q = oracle.normal_bf16((300, H, 128), 5)
    k = oracle.normal_bf16((400, H, 128), 6)
    v = oracle.normal_bf16((400, H, 128), 7)
    sentinel = np.full((300, H, 128), 0x7fc0, dtype=np.uint16)
    ty = gpu.tensor(sentinel)
    gpu.call("cross_attention_bf16", ty, 50, gpu.tensor(q), 20, gpu.tensor(k), gpu.tensor(v), 100,
             130, 250, H)
    out = gpu.read(ty, q.shape)
    assert np.array_equal(out[:50], sentinel[:50]) and np.array_equal(out[180:], sentinel[180:])
    want, _ = oracle.attention(q[None, 20:150], k[None, 100:350], v[None, 100:350], SCALE)
    assert_attention_close(oracle.from_bf16(out[50:180]), want[0])


def test_head_split_is_bit_exact(gpu, oracle):
    """Attention over all heads equals the concatenation of per-half calls bit for bit
    (reference tests/live/sharding.py:38-46): no cross-head arithmetic anywhere."""
    L, H = 333, 8
    q, k, v = (oracle.normal_bf16((L, H, 128), 70 + i) for i in range(3))
    ty = gpu.empty_bf16(q.size)
    gpu.call("sdpa_bf16", ty, gpu.tensor(q), gpu.tensor(k), gpu.tensor(v), L, H, 128, SCALE)
    full = gpu.read(ty, q.shape)
    halves = []
    for lo in (0, H // 2):
        sl = slice(lo, lo + H // 2)
        th = gpu.empty_bf16(L * (H // 2) * 128)
        gpu.call("sdpa_bf16", th, gpu.tensor(q[:, sl]), gpu.tensor(k[:, sl]), gpu.tensor(v[:, sl]),
                 L, H // 2, 128, SCALE)
        halves.append(gpu.read(th, (L, H // 2, 128)))
    assert np.array_equal(full, np.concatenate(halves, axis=1))


def test_run_twice_is_deterministic(gpu, oracle):
    L, H = 517, 3
    q, k, v = (oracle.normal_bf16((L, H, 128), 80 + i) for i in range(3))
    tq, tk, tv = gpu.tensor(q), gpu.tensor(k), gpu.tensor(v)
    outs = []
    for _ in range(2):
        ty = gpu.empty_bf16(q.size)
        gpu.call("sdpa_bf16", ty, tq, tk, tv, L, H, 128, SCALE)
        outs.append(gpu.read(ty, q.shape))
    assert np.array_equal(outs[0], outs[1])


@pytest.mark.parametrize("groups", [0, 1, 2, 4])
def test_host_buffer_attention_matches_device_path(gpu, oracle, groups):
    """h3b_sdpa_bf16_host (head groups pipelined over copy and compute streams, pageable host
    memory here) gives the same bits as the device-tensor primitive: grouping heads changes
    nothing per head. A second call reuses the staging slots."""
    L, H = 700, 8
    q, k, v = (oracle.normal_bf16((L, H, 128), 90 + i) for i in range(3))
    ty = gpu.empty_bf16(q.size)
    gpu.call("sdpa_bf16", ty, gpu.tensor(q), gpu.tensor(k), gpu.tensor(v), L, H, 128, SCALE)
    want = gpu.read(ty, q.shape)
    for _ in range(2):
        out = np.zeros(q.shape, dtype=np.uint16)
        ok = gpu.lib.h3b_sdpa_bf16_host(gpu.gpu, out.ctypes.data_as(C.c_void_p), q.ctypes.data_as(C.c_void_p),
                                        k.ctypes.data_as(C.c_void_p), v.ctypes.data_as(C.c_void_p), L, H,
                                        128, SCALE, groups)
        assert ok, gpu.error()
        assert np.array_equal(out, want)
    assert not gpu.lib.h3b_sdpa_bf16_host(gpu.gpu, out.ctypes.data_as(C.c_void_p), q.ctypes.data_as(C.c_void_p),
                                          k.ctypes.data_as(C.c_void_p), v.ctypes.data_as(C.c_void_p), L, H,
                                          128, SCALE, 3)
    assert "do not split into 3 groups" in gpu.error()
    assert gpu.device_status() == 0


@pytest.mark.parametrize("nq,ranges,H", [(300, [77, 405, 1000, 128, 300], 4), (64, [5], 2),
                                          (405, [129, 1, 127, 256, 33, 700], 7)])
def test_segmented_live_attention_equals_concatenated(gpu, oracle, nq, ranges, H):
    """h3b_cross_attention_segments_bf16 over separate K/V ranges == h3_gpu_cross_attention_bf16
    over their concatenation (the reference's live path, h3_dit_live.inc:81-99). Ranges that
    are multiples of 128 rows give the same bits; ragged ones regroup the key tiles, so those
    are compared by tolerance and against the oracle."""
    q = oracle.normal_bf16((nq + 9, H, 128), 500)
    ks = [oracle.normal_bf16((r + 3, H, 128), 510 + i) for i, r in enumerate(ranges)]
    vs = [oracle.normal_bf16((r + 3, H, 128), 520 + i) for i, r in enumerate(ranges)]
    kcat = np.concatenate([x[3:] for x in ks])
    vcat = np.concatenate([x[3:] for x in vs])
    tq = gpu.tensor(q)
    want_t = gpu.tensor(np.zeros((nq, H, 128), dtype=np.uint16))
    gpu.call("cross_attention_bf16", want_t, 0, tq, 9, gpu.tensor(kcat), gpu.tensor(vcat), 0, nq, len(kcat), H)
    concat = gpu.read(want_t, (nq, H, 128))
    n = len(ranges)
    tk = (C.c_void_p * n)(*[gpu.tensor(x) for x in ks])
    tv = (C.c_void_p * n)(*[gpu.tensor(x) for x in vs])
    rows = (C.c_uint32 * n)(*ranges)
    offs = (C.c_size_t * n)(*([3] * n))
    out = gpu.tensor(np.zeros((nq + 2, H, 128), dtype=np.uint16))
    ok = gpu.lib.h3b_cross_attention_segments_bf16(gpu.gpu, out, 2, tq, 9, nq, H, n, tk, tv, offs, rows)
    assert ok, gpu.error()
    got = gpu.read(out, (nq + 2, H, 128))
    assert not got[:2].any()
    want, _ = oracle.attention(q[None, 9:], kcat[None], vcat[None], SCALE)
    assert_attention_close(oracle.from_bf16(got[2:]), want[0])
    if all(r % 128 == 0 for r in ranges) or n == 1:
        assert np.array_equal(got[2:], concat)
    else:
        assert np.abs(oracle.from_bf16(got[2:]) - oracle.from_bf16(concat)).max() <= 4e-3
    assert gpu.device_status() == 0
    assert not gpu.lib.h3b_cross_attention_segments_bf16(gpu.gpu, out, 2, tq, 9, nq, H, 7, tk, tv, offs, rows)


@pytest.mark.parametrize("seed", range(12))
def test_random_shapes_against_oracle(gpu, oracle, seed):
    """Seeded random shapes around the tile boundaries of both tcgen05 kernels (128-row query
    tiles, 256-row CTA pairs, 128-row key tiles): a dense call, a rectangular call with row
    offsets, a causal/GQA call and a segmented call per seed, each against the oracle."""
    rng = np.random.default_rng(1000 + seed)
    near = lambda: int(rng.choice([1, 64, 127, 128, 129, 255, 256, 257, 383, 384, 385, 511, 640]) + rng.integers(0, 3))
    H = int(rng.choice([1, 2, 3, 5]))
    # dense
    L = near()
    got, want = run_sdpa(gpu, oracle, L, H, 3000 + seed)
    assert_attention_close(got, want[0])
    # rectangular with offsets
    nq, nk, qo, ko, oo = near(), near(), int(rng.integers(0, 5)), int(rng.integers(0, 5)), int(rng.integers(0, 5))
    q = oracle.normal_bf16((nq + qo, H, 128), 3100 + seed)
    k = oracle.normal_bf16((nk + ko, H, 128), 3200 + seed)
    v = oracle.normal_bf16((nk + ko, H, 128), 3300 + seed)
    out = gpu.tensor(np.zeros((nq + oo, H, 128), dtype=np.uint16))
    tq, tk, tv = gpu.tensor(q), gpu.tensor(k), gpu.tensor(v)
    gpu.call("cross_attention_bf16", out, oo, tq, qo, tk, tv, ko, nq, nk, H)
    got = gpu.read(out, (nq + oo, H, 128))
    assert not got[:oo].any()
    want, _ = oracle.attention(q[None, qo:], k[None, ko:], v[None, ko:], SCALE)
    assert_attention_close(oracle.from_bf16(got[oo:]), want[0])
    for t in (out, tq, tk, tv):
        gpu.free(t)
    # causal / grouped-query (the FlashAttention-2 adapter)
    KH = int(rng.choice([1, 2]))
    Hq = KH * int(rng.choice([1, 2, 3]))
    causal = bool(rng.integers(0, 2))
    Lc = near()
    q = oracle.normal_bf16((1, Lc, Hq, 128), 3400 + seed)
    k = oracle.normal_bf16((1, Lc, KH, 128), 3500 + seed)
    v = oracle.normal_bf16((1, Lc, KH, 128), 3600 + seed)
    ty, tq, tk, tv = gpu.empty_bf16(q.size), gpu.tensor(q), gpu.tensor(k), gpu.tensor(v)
    data = gpu.lib.h3b_tensor_data
    gpu.raw("h3_flash_bf16", data(ty), data(tq), data(tk), data(tv), None, 1, Lc, Hq, KH, SCALE, causal,
            gpu.lib.h3b_gpu_stream(gpu.gpu))
    want, _ = oracle.attention(q, k, v, SCALE, causal=causal)
    assert_attention_close(oracle.from_bf16(gpu.read(ty, q.shape)), want)
    for t in (ty, tq, tk, tv):
        gpu.free(t)
    # segmented keys
    n = int(rng.integers(1, 7))
    ranges = [near() for _ in range(n)]
    nq = near()
    q = oracle.normal_bf16((nq, H, 128), 3700 + seed)
    ks = [oracle.normal_bf16((r, H, 128), 3800 + 10 * seed + i) for i, r in enumerate(ranges)]
    vs = [oracle.normal_bf16((r, H, 128), 3900 + 10 * seed + i) for i, r in enumerate(ranges)]
    tensors = [gpu.tensor(x) for x in ks + vs]
    tk = (C.c_void_p * n)(*tensors[:n])
    tv = (C.c_void_p * n)(*tensors[n:])
    rows = (C.c_uint32 * n)(*ranges)
    offs = (C.c_size_t * n)(*([0] * n))
    tq, out = gpu.tensor(q), gpu.tensor(np.zeros((nq, H, 128), dtype=np.uint16))
    assert gpu.lib.h3b_cross_attention_segments_bf16(gpu.gpu, out, 0, tq, 0, nq, H, n, tk, tv, offs, rows), gpu.error()
    want, _ = oracle.attention(q[None], np.concatenate(ks)[None], np.concatenate(vs)[None], SCALE)
    assert_attention_close(oracle.from_bf16(gpu.read(out, (nq, H, 128))), want[0])
    for t in tensors + [tq, out]:
        gpu.free(t)
    assert gpu.device_status() == 0
