"""CPU checks of the oracle itself: it must agree with independent numpy float64 math and
with the structural facts the reference documents (tile counts, keep rule, selection
semantics, exchange algebra). The reference ships no golden tensors for attention, so these
are the oracle's anchors on CPU; on the GPU box it is checked again against the reference's
own CUDA code where that still runs (tests/test_reference_backend.py).
"""
import numpy as np
import pytest


def numpy_attention(q, k, v, scale, causal=False):
    """[L,H,D] float64 softmax(QK^T)V per head."""
    out = np.empty(q.shape, dtype=np.float64)
    for h in range(q.shape[1]):
        kh = h // (q.shape[1] // k.shape[1])
        s = (q[:, h].astype(np.float64) @ k[:, kh].astype(np.float64).T) * scale
        if causal:
            s = np.where(np.arange(k.shape[0])[None, :] > np.arange(q.shape[0])[:, None], -np.inf, s)
        s -= s.max(axis=1, keepdims=True)
        p = np.exp(s)
        out[:, h] = (p / p.sum(axis=1, keepdims=True)) @ v[:, kh].astype(np.float64)
    return out


def test_bf16_round_trip_and_rounding(oracle):
    x = np.array([1.0, 1.00390625, 1.01171875, -3.140625, 0.0, 65504.0, 1e-40], dtype=np.float32)
    b = oracle.to_bf16(x)
    assert np.array_equal(oracle.to_bf16(oracle.from_bf16(b)), b)
    # 1 + 2^-8 is a tie between 1.0 and 1 + 2^-7: round to even -> 1.0; 1 + 3*2^-8 -> 1 + 2^-6
    assert oracle.from_bf16(b)[1] == 1.0 and oracle.from_bf16(b)[2] == 1.015625
    assert np.isnan(oracle.from_bf16(oracle.to_bf16(np.array([np.nan], dtype=np.float32)))).all()


def test_seeded_generator_is_deterministic_and_normal(oracle):
    a = oracle.normal_bf16((1000, 128), 7)
    b = oracle.normal_bf16((1000, 128), 7)
    c = oracle.normal_bf16((1000, 128), 8)
    assert np.array_equal(a, b) and not np.array_equal(a, c)
    x = oracle.from_bf16(a).astype(np.float64)
    assert abs(x.mean()) < 0.01 and abs(x.std() - 1.0) < 0.01
    # counter-based: a prefix of a longer stream is the shorter stream
    assert np.array_equal(oracle.normal_bf16((100,), 7), a.ravel()[:100])


@pytest.mark.parametrize("L,H,KH,causal", [(7, 2, 2, False), (65, 4, 2, False), (130, 4, 1, True),
                                           (263, 3, 3, True)])
def test_attention_matches_numpy_float64(oracle, L, H, KH, causal):
    scale = 1.0 / np.sqrt(128.0)
    q = oracle.normal_bf16((1, L, H, 128), 1)
    k = oracle.normal_bf16((1, L, KH, 128), 2)
    v = oracle.normal_bf16((1, L, KH, 128), 3)
    out32, out16, lse = oracle.attention(q, k, v, scale, causal=causal, want_lse=True)
    want = numpy_attention(oracle.from_bf16(q[0]), oracle.from_bf16(k[0]), oracle.from_bf16(v[0]),
                           scale, causal)
    assert np.abs(out32[0] - want).max() < 2e-5
    assert np.array_equal(out16, oracle.to_bf16(out32))
    assert np.isfinite(lse).all()


def test_rectangular_and_sampled_rows(oracle):
    scale = 1.0 / np.sqrt(128.0)
    q = oracle.normal_bf16((1, 40, 2, 128), 4)
    k = oracle.normal_bf16((1, 333, 2, 128), 5)
    v = oracle.normal_bf16((1, 333, 2, 128), 6)
    out32, _ = oracle.attention(q, k, v, scale)
    want = numpy_attention(oracle.from_bf16(q[0]), oracle.from_bf16(k[0]), oracle.from_bf16(v[0]), scale)
    assert np.abs(out32[0] - want).max() < 2e-5
    rows = np.array([0, 13, 39], dtype=np.int32)
    sampled = oracle.attention_rows_f64(rows, q[0], k[0], v[0], scale)
    assert np.abs(sampled - want[rows]).max() < 1e-6


def test_f16_d64_attention(oracle):
    rng = np.random.default_rng(3)
    q, k, v = (oracle.to_f16(rng.standard_normal((1, 50, 2, 64))) for _ in range(3))
    out32, out16 = oracle.attention(q, k, v, 0.125, elem="f16")
    want = numpy_attention(oracle.from_f16(q[0]), oracle.from_f16(k[0]), oracle.from_f16(v[0]), 0.125)
    assert np.abs(out32[0] - want).max() < 2e-5


def test_vsa_map_geometry(oracle):
    """Tile counts the reference documents: 864x480 5 s = 37x15x27 tokens -> 280 video tiles,
    288 with 17 text + 448 audio rows (cuda/FASTH3.md:136); keep = ceil(10 %) (cuda/vsa.cuh:242)."""
    m = oracle.VsaMap(17, 448, 37, 15, 27)
    assert (m.tiles, m.prefix, m.keep) == (288, 8, 28)
    assert m.rows == 17 + 448 + 37 * 15 * 27
    assert m.sizes[0] == 17 and list(m.sizes[1:8]) == [64] * 7
    valid = m.map[m.map >= 0]
    assert np.array_equal(np.sort(valid), np.arange(m.rows))          # every token exactly once
    assert np.array_equal((m.map.reshape(-1, 64) >= 0).sum(1), m.sizes)
    # first video cube: (dt, dy, dx) order over a 4x4x4 corner of the 37x15x27 grid
    base = 17 + 448
    cube = m.map[8 * 64:9 * 64]
    want = [base + (dt * 15 + dy) * 27 + dx for dt in range(4) for dy in range(4) for dx in range(4)]
    assert list(cube) == want
    # edge cubes are partial: 15 = 3*4 + 3, 27 = 6*4 + 3, 37 = 9*4 + 1
    assert m.sizes.min() == 1 * 3 * 3 and m.sizes[8:].max() == 64
    b = oracle.VsaMap(64, 512, 32, 30, 54)
    assert (b.tiles, b.prefix) == (8 * 8 * 14 + 9, 9)
    with pytest.raises(ValueError):
        oracle.VsaMap(3, 11, 4, 4, 4 * 4096)


def test_vsa_pool_matches_float64_mean(oracle):
    m = oracle.VsaMap(3, 11, 5, 7, 9)
    x = oracle.normal_bf16((m.rows, 2, 128), 9)
    tiled, pooled = oracle.vsa_tile_pool(x, m)
    xf = oracle.from_bf16(x).astype(np.float64)
    for t in (0, 1, 2, m.tiles - 1):
        rows = m.map[t * 64:(t + 1) * 64]
        want = xf[rows[rows >= 0]].sum(0) / m.sizes[t]
        assert np.abs(pooled[:, t] - want).max() < 1e-5
        got_rows = tiled[:, t * 64:(t + 1) * 64]
        assert np.array_equal(got_rows[:, :m.sizes[t]].transpose(1, 0, 2), x[rows[rows >= 0]])
        assert not got_rows[:, m.sizes[t]:].any()


def test_vsa_select_semantics(oracle):
    rng = np.random.default_rng(5)
    tiles, prefix, keep, heads = 40, 3, 5, 2
    scores = rng.standard_normal((heads, tiles, tiles)).astype(np.float32)
    scores[0, 10, 20:30] = 7.0  # a ten-way tie at the top: the five lowest indices win
    indices, counts = oracle.vsa_select(scores, prefix, keep)
    assert (counts[:, :prefix] == tiles).all() and (counts[:, prefix:] == prefix + keep).all()
    assert list(indices[0, 10, :counts[0, 10]]) == [0, 1, 2, 20, 21, 22, 23, 24]
    for h in range(heads):
        for qt in range(prefix, tiles):
            got = indices[h, qt, :counts[h, qt]]
            assert (np.diff(got) > 0).all() and list(got[:prefix]) == list(range(prefix))
            if (h, qt) != (0, 10):
                order = np.argsort(-scores[h, qt, prefix:], kind="stable")[:keep] + prefix
                assert set(got[prefix:]) == set(order)


def test_vsa_softmax_and_compress_match_numpy(oracle):
    rng = np.random.default_rng(6)
    for tiles in (9, 40, 300):
        scores = rng.standard_normal((2, tiles, tiles)).astype(np.float32) * 3
        prob = oracle.vsa_pooled_softmax(scores)
        s = scores.astype(np.float64)
        want = np.exp(s - s.max(-1, keepdims=True))
        want /= want.sum(-1, keepdims=True)
        assert np.abs(prob - want).max() < 1e-6
        poolv = rng.standard_normal((2, tiles, 128)).astype(np.float32)
        comp = oracle.vsa_compress(prob, poolv)
        assert np.abs(comp - prob.astype(np.float64) @ poolv).max() < 1e-5


def dense_masked_vsa(oracle, q, k, v, gate, m, keep):
    """Independent float64 restatement of the whole VSA forward through a dense token mask,
    the way the reference's own math oracle is built (tests/fasth3/vsa.py:67-95)."""
    heads = q.shape[1]
    scale = 1.0 / np.sqrt(128.0)
    qf, kf, vf, gf = (oracle.from_bf16(x).astype(np.float64) for x in (q, k, v, gate))
    tile_rows = [m.map[t * 64:(t + 1) * 64][:m.sizes[t]] for t in range(m.tiles)]
    out = np.zeros(q.shape, dtype=np.float64)
    for h in range(heads):
        pq = np.stack([qf[r, h].mean(0) for r in tile_rows])
        pk = np.stack([kf[r, h].mean(0) for r in tile_rows])
        pv = np.stack([vf[r, h].mean(0) for r in tile_rows])
        scores = pq @ pk.T * scale
        p = np.exp(scores - scores.max(-1, keepdims=True))
        comp = (p / p.sum(-1, keepdims=True)) @ pv
        for qt in range(m.tiles):
            if qt < m.prefix:
                chosen = list(range(m.tiles))
            else:
                top = np.argsort(-scores[qt, m.prefix:], kind="stable")[:keep] + m.prefix
                chosen = list(range(m.prefix)) + sorted(top)
            keys = np.concatenate([tile_rows[t] for t in chosen])
            s = qf[tile_rows[qt], h] @ kf[keys, h].T * scale
            w = np.exp(s - s.max(-1, keepdims=True))
            sparse = (w / w.sum(-1, keepdims=True)) @ vf[keys, h]
            c16 = oracle.from_bf16(oracle.to_bf16(comp[qt].astype(np.float32))).astype(np.float64)
            s16 = oracle.from_bf16(oracle.to_bf16(sparse.astype(np.float32))).astype(np.float64)
            out[tile_rows[qt], h] = s16 + c16 * gf[tile_rows[qt], h]
    return out


@pytest.mark.parametrize("text,audio,shape,heads", [(3, 11, (1, 2, 3), 2), (65, 67, (5, 7, 9), 2)])
@pytest.mark.parametrize("gate_scale", [0.0, 0.3])
def test_vsa_pipeline_matches_dense_mask_math(oracle, text, audio, shape, heads, gate_scale):
    """Cases and limits of the reference's VSA math test (tests/fasth3/vsa.py:109-131)."""
    m = oracle.VsaMap(text, audio, *shape)
    q, k, v = (oracle.normal_bf16((m.rows, heads, 128), 50 + i) for i in range(3))
    gate = oracle.normal_bf16((m.rows, heads, 128), 53, gate_scale) if gate_scale else \
        np.zeros((m.rows, heads, 128), dtype=np.uint16)
    stages = oracle.vsa_forward(q, k, v, gate, m)
    got = oracle.from_bf16(stages["out"]).astype(np.float64)
    want = dense_masked_vsa(oracle, q, k, v, gate, m, m.keep)
    rel = np.linalg.norm(got - want) / np.linalg.norm(want)
    norm_max = np.abs(got - want).max() / np.abs(want).max()
    assert rel < 0.012 and norm_max < 0.03, (rel, norm_max)


def test_ulysses_algebra(oracle):
    """scatter then gather is the identity; scatter gives every rank all rows of its heads
    (reference cuda/parallel.cuh:25-30,125-143)."""
    ranks, rows, heads, dim = 4, 5, 8, 16
    x = np.arange(ranks * rows * heads * dim, dtype=np.uint16).reshape(ranks, rows, heads, dim)
    y = oracle.ulysses(x)
    full = x.reshape(ranks * rows, heads, dim)
    for r in range(ranks):
        assert np.array_equal(y[r], full[:, r * 2:(r + 1) * 2])
    assert np.array_equal(oracle.ulysses(y, inverse=True), x)
