"""Video sparse attention through the C ABI: every stage of h3_gpu_vsa_bf16 against the oracle.

Cases are those of the reference's VSA test (tests/fasth3/vsa.py:109-112), including the
864x480 5 s grid (37, 15, 27) and the 2051-tile case that switches the pooled softmax to its
block reduction order. Integer and order-pinned stages (tile gather, pooled means, pooled
scores, top-k indices and counts) must be bit-exact; the floating-point stages meet the
reference's limits (relative L2 < 0.012, normalised max < 0.03, tests/fasth3/vsa.py:131).
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

CASES = [(3, 11, (1, 2, 3), 2), (65, 67, (5, 7, 9), 4), (17, 30, (7, 8, 8), 56),
         (5, 13, (4, 4, 44), 4), (17, 448, (37, 15, 27), 4)]


class Vsa:
    def __init__(self, gpu, text, audio, shape, heads):
        self.gpu = gpu
        self.handle = gpu.call("vsa_new", text, audio, *shape, heads)
        info = [C.c_int() for _ in range(4)]
        assert gpu.lib.h3b_vsa_info(self.handle, *[C.byref(x) for x in info])
        self.rows, self.tiles, self.prefix, self.keep = (x.value for x in info)
        self.heads = heads

    def buffer(self, which, shape, dtype):
        return self.gpu.read_device(self.gpu.lib.h3b_vsa_buffer(self.handle, which), shape, dtype)

    def run(self, q, k, v, gate):
        gpu = self.gpu
        out = gpu.tensor(np.zeros(q.shape, dtype=np.uint16))
        tensors = [gpu.tensor(x) for x in (q, k, v, gate)]
        if not gpu.lib.h3_gpu_vsa_bf16(self.handle, out, *tensors):
            raise RuntimeError(gpu.error())
        result = gpu.read(out, q.shape)
        for t in [out] + tensors:
            gpu.free(t)
        return result

    def close(self):
        self.gpu.lib.h3_gpu_vsa_free(self.handle)


def inputs(oracle, rows, heads, seed, gate_scale):
    q, k, v = (oracle.normal_bf16((rows, heads, 128), seed + i) for i in range(3))
    gate = oracle.normal_bf16((rows, heads, 128), seed + 3, gate_scale) if gate_scale else \
        np.zeros((rows, heads, 128), dtype=np.uint16)
    return q, k, v, gate


def check_stages(gpu, oracle, vsa, vmap, q, k, v, gate, got, keep):
    T, H = vsa.tiles, vsa.heads
    stages = oracle.vsa_forward(q, k, v, gate, vmap, keep=keep)
    # geometry
    assert np.array_equal(vsa.buffer(0, (T * 64,), np.int32), vmap.map)
    assert np.array_equal(vsa.buffer(1, (T,), np.int32), vmap.sizes)
    # gather + pooled means: bit-exact (summation order of reference cuda/vsa.cuh:22-42)
    for i in range(3):
        assert np.array_equal(vsa.buffer(2 + i, (H, T * 64, 128), np.uint16), stages["tiled"][i])
        pooled = vsa.buffer(6 + i, (H, T, 128), np.float32)
        assert np.array_equal(pooled.view(np.uint32), stages["pooled"][i].view(np.uint32))
    # pooled scores: bit-exact against the oracle's fixed fmaf order
    scores = vsa.buffer(12, (H, T, T), np.float32)
    assert np.array_equal(scores.view(np.uint32), stages["scores"].view(np.uint32))
    # top-k: counts and index lists bit-exact
    counts = vsa.buffer(10, (H, T), np.int32)
    indices = vsa.buffer(9, (H, T, T), np.int32)
    assert np.array_equal(counts, stages["counts"])
    valid = np.arange(T)[None, None, :] < counts[:, :, None]
    assert np.array_equal(indices[valid], stages["indices"][valid])
    # fine stage on the same lists
    sparse = oracle.from_bf16(vsa.buffer(5, (H, T * 64, 128), np.uint16))
    real = np.repeat((vmap.map >= 0)[None, :], H, axis=0)
    diff = (sparse - stages["sparse_f32"])[real]
    assert np.isfinite(sparse[real]).all()
    assert np.abs(diff).max() <= 1e-2
    a, b = sparse[real].ravel().astype(np.float64), stages["sparse_f32"][real].ravel().astype(np.float64)
    assert a @ b / (np.linalg.norm(a) * np.linalg.norm(b)) >= 0.9999
    # compression branch (expf on device vs host may differ in the last place)
    comp = vsa.buffer(11, (H, T, 128), np.float32)
    assert np.abs(comp - stages["compression"]).max() <= 1e-5 * max(1.0, np.abs(stages["compression"]).max())
    # merged output: the reference's limits, and near-identity with the oracle's output
    want = oracle.from_bf16(stages["out"]).astype(np.float64)
    g = oracle.from_bf16(got).astype(np.float64)
    rel = np.linalg.norm(g - want) / np.linalg.norm(want)
    norm_max = np.abs(g - want).max() / np.abs(want).max()
    assert np.isfinite(g).all() and rel < 0.012 and norm_max < 0.03, (rel, norm_max)
    return rel


@pytest.mark.parametrize("text,audio,shape,heads", CASES)
@pytest.mark.parametrize("gate_scale", [0.0, 0.3])
def test_vsa_stages(gpu, oracle, text, audio, shape, heads, gate_scale):
    vmap = oracle.VsaMap(text, audio, *shape)
    vsa = Vsa(gpu, text, audio, shape, heads)
    try:
        assert (vsa.rows, vsa.tiles, vsa.prefix, vsa.keep) == (vmap.rows, vmap.tiles, vmap.prefix, vmap.keep)
        assert gpu.lib.h3b_vsa_trace_scores(vsa.handle, 1)
        q, k, v, gate = inputs(oracle, vsa.rows, heads, 1234 + heads, gate_scale)
        got = vsa.run(q, k, v, gate)
        check_stages(gpu, oracle, vsa, vmap, q, k, v, gate, got, vmap.keep)
        assert gpu.device_status() == 0
    finally:
        vsa.close()


def test_vsa_keep_override_and_ties(gpu, oracle):
    """12.5 % keep (the benchmark's setting) and exact score ties: duplicated key cubes give
    identical pooled keys, so ties are exact and must resolve to the lower tile index."""
    text, audio, shape, heads = 64, 128, (8, 8, 16), 2
    vmap = oracle.VsaMap(text, audio, *shape)
    vsa = Vsa(gpu, text, audio, shape, heads)
    try:
        keep = (vsa.tiles - vsa.prefix) // 8
        assert gpu.lib.h3b_vsa_set_keep(vsa.handle, keep)
        assert not gpu.lib.h3b_vsa_set_keep(vsa.handle, 0)
        assert gpu.lib.h3b_vsa_trace_scores(vsa.handle, 1)
        q, k, v, gate = inputs(oracle, vsa.rows, heads, 77, 0.3)
        # make video cubes 10..13 exact copies of cube 5 in K (same rows order inside a cube)
        src_rows = vmap.map[(vsa.prefix + 5) * 64:(vsa.prefix + 6) * 64]
        for t in range(10, 14):
            k[vmap.map[(vsa.prefix + t) * 64:(vsa.prefix + t + 1) * 64]] = k[src_rows]
        got = vsa.run(q, k, v, gate)
        check_stages(gpu, oracle, vsa, vmap, q, k, v, gate, got, keep)
        scores = vsa.buffer(12, (heads, vsa.tiles, vsa.tiles), np.float32)
        assert np.array_equal(scores[:, :, vsa.prefix + 5], scores[:, :, vsa.prefix + 12])
    finally:
        vsa.close()


def test_vsa_head_split_is_bit_exact(gpu, oracle):
    """Heads are independent: the same call on a subset of the heads gives the same bits for those
    heads (the property the reference checks for its head-sharded attention,
    tests/live/sharding.py:38-46). The persistent fine-stage kernel hands query tiles to CTAs
    dynamically, so this also pins that a tile's result does not depend on what its CTA computed
    before it."""
    text, audio, shape, heads = 64, 64, (16, 16, 32), 6
    whole = Vsa(gpu, text, audio, shape, heads)
    part = Vsa(gpu, text, audio, shape, 3)
    try:
        q, k, v, gate = inputs(oracle, whole.rows, heads, 2024, 0.3)
        for mode in (0, 3):
            gpu.lib.h3b_vsa_fine_mode(mode)
            all_heads = whole.run(q, k, v, gate)
            for lo in (0, 3):
                some = part.run(*[np.ascontiguousarray(a[:, lo:lo + 3]) for a in (q, k, v, gate)])
                assert np.array_equal(some, all_heads[:, lo:lo + 3]), (mode, lo)
            again = whole.run(q, k, v, gate)
            assert np.array_equal(again, all_heads), mode
        assert gpu.device_status() == 0
    finally:
        gpu.lib.h3b_vsa_fine_mode(0)
        whole.close()
        part.close()


def test_vsa_block_softmax_order_2051_tiles(gpu, oracle):
    """Above 2048 tiles the pooled softmax uses the 1024-thread reduction order
    (reference cuda/vsa.cuh:108-156; case (3, 11, (4, 4, 8193), 1) of tests/fasth3/vsa.py:112)."""
    text, audio, shape, heads = 3, 11, (4, 4, 8193), 1
    vmap = oracle.VsaMap(text, audio, *shape)
    assert vmap.tiles == 2051
    vsa = Vsa(gpu, text, audio, shape, heads)
    try:
        assert gpu.lib.h3b_vsa_trace_scores(vsa.handle, 1)
        q, k, v, gate = inputs(oracle, vsa.rows, heads, 4321, 0.3)
        got = vsa.run(q, k, v, gate)
        check_stages(gpu, oracle, vsa, vmap, q, k, v, gate, got, vmap.keep)
    finally:
        vsa.close()


def test_vsa_hopper_symbol_direct(gpu, oracle):
    """h3_vsa_hopper on hand-made lists: odd tile count (last query pair half empty), a query
    tile with a single KV tile, unsorted-free ascending lists, partial tiles, and lse."""
    rng = np.random.default_rng(8)
    tiles, heads = 7, 3
    sizes = np.array([64, 17, 64, 1, 64, 33, 64], dtype=np.int32)
    q, k, v = (oracle.normal_bf16((heads, tiles * 64, 128), 900 + i) for i in range(3))
    indices = np.zeros((heads, tiles, tiles), dtype=np.int32)
    counts = np.zeros((heads, tiles), dtype=np.int32)
    for h in range(heads):
        for t in range(tiles):
            n = 1 if (h, t) == (0, 2) else int(rng.integers(1, tiles + 1))
            chosen = np.sort(rng.choice(tiles, n, replace=False))
            indices[h, t, :n] = chosen
            counts[h, t] = n
    d = gpu.lib.h3b_tensor_data
    tq, tk, tv = gpu.tensor(q), gpu.tensor(k), gpu.tensor(v)
    to = gpu.tensor(np.zeros(q.shape, dtype=np.uint16))
    tl = gpu.tensor(np.zeros((heads, tiles * 64), dtype=np.float32))
    ti, tc, ts = gpu.tensor(indices), gpu.tensor(counts), gpu.tensor(sizes)
    gpu.raw("h3_vsa_hopper", d(to), d(tq), d(tk), d(tv), d(tl), d(ti), d(tc), d(ts), tiles, heads,
            gpu.lib.h3b_gpu_stream(gpu.gpu))
    got = oracle.from_bf16(gpu.read(to, q.shape))
    lse = gpu.read(tl, (heads, tiles * 64), np.float32)
    _, want, want_lse = oracle.vsa_fine(q, k, v, indices, counts, sizes)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= 1e-2
    # lse is scaled by sqrt(128) in this kernel's convention; its row sum is taken over the bf16-rounded
    # weights (the ones the PV product uses), so it carries their rounding: up to 2^-8 relative,
    # 0.0039 * sqrt(128) = 0.044 here. Nothing in the reference reads lse.
    assert np.abs(lse - want_lse).max() <= 5e-2
    assert gpu.device_status() == 0


def _fine_direct(gpu, q, k, v, indices, counts, sizes, want_lse=False, expect_status=0):
    """h3_vsa_hopper on explicit lists; returns (bf16 bits, lse or None). The device status word
    is read (and cleared) right after the call and must equal expect_status."""
    heads, padded, _ = q.shape
    tiles = padded // 64
    d = gpu.lib.h3b_tensor_data
    tensors = [gpu.tensor(x) for x in (q, k, v, indices, counts, sizes)]
    to = gpu.tensor(np.full(q.shape, 0x7fc0, dtype=np.uint16))   # NaN pattern: every row must be written
    tl = gpu.tensor(np.zeros((heads, padded), dtype=np.float32)) if want_lse else None
    gpu.raw("h3_vsa_hopper", d(to), *[d(t) for t in tensors[:3]], d(tl) if tl else None,
            *[d(t) for t in tensors[3:]], tiles, heads, gpu.lib.h3b_gpu_stream(gpu.gpu))
    assert gpu.device_status() == expect_status
    out = gpu.read(to, q.shape)
    lse = gpu.read(tl, (heads, padded), np.float32) if tl else None
    for t in tensors + [to] + ([tl] if tl else []):
        gpu.free(t)
    return out, lse


def _random_lists(rng, tiles, heads, low=1):
    indices = np.zeros((heads, tiles, tiles), dtype=np.int32)
    counts = np.zeros((heads, tiles), dtype=np.int32)
    for h in range(heads):
        for t in range(tiles):
            n = int(rng.integers(low, tiles + 1))
            indices[h, t, :n] = np.sort(rng.choice(tiles, n, replace=False))
            counts[h, t] = n
    return indices, counts


def test_vsa_fine_pairs_go_to_the_cheaper_kernel(gpu, oracle):
    """Default mode: pairs of adjacent query tiles with (nearly) the same list are computed by the
    pair-walk kernel, pairs with different lists by the persistent kernel. With identical lists in
    every pair the result is the pair-walk kernel's bit for bit; with disjoint lists the
    persistent kernel's."""
    tiles, heads = 16, 2
    sizes = np.full(tiles, 64, dtype=np.int32)
    q, k, v = (oracle.normal_bf16((heads, tiles * 64, 128), 40 + i) for i in range(3))
    same = np.zeros((heads, tiles, tiles), dtype=np.int32)
    apart = np.zeros((heads, tiles, tiles), dtype=np.int32)
    counts = np.full((heads, tiles), 6, dtype=np.int32)
    for t in range(tiles):
        same[:, t, :6] = np.arange(6) + 2 * (t // 2) % 8            # both tiles of a pair: one list
        apart[:, t, :6] = np.arange(6) * 2 + (t & 1)                  # even tiles / odd tiles: disjoint
    try:
        for lists, twin in ((same, 1), (apart, 3)):
            got = {}
            for mode in (0, twin):
                gpu.lib.h3b_vsa_fine_mode(mode)
                got[mode], _ = _fine_direct(gpu, q, k, v, lists, counts, sizes)
            assert np.array_equal(got[0], got[twin])
            _, want, _ = oracle.vsa_fine(q, k, v, lists, counts, sizes)
            assert np.abs(oracle.from_bf16(got[0]) - want).max() <= 1e-2
    finally:
        gpu.lib.h3b_vsa_fine_mode(0)


def test_vsa_fine_kernels_agree(gpu, oracle):
    """The fine-stage modes on the same lists (odd and even list lengths, partial tiles):
    the persistent kernel and the pair-walk kernel both meet the oracle; with every tile marked
    for recomputation the result is the pair-walk kernel's, bit for bit."""
    rng = np.random.default_rng(21)
    tiles, heads = 23, 5
    sizes = rng.integers(1, 65, tiles).astype(np.int32)
    sizes[::3] = 64
    q, k, v = (oracle.normal_bf16((heads, tiles * 64, 128), 300 + i) for i in range(3))
    indices, counts = _random_lists(rng, tiles, heads)
    _, want, want_lse = oracle.vsa_fine(q, k, v, indices, counts, sizes)
    got = {}
    try:
        for mode in (0, 1, 2, 3):
            gpu.lib.h3b_vsa_fine_mode(mode)
            bits, lse = _fine_direct(gpu, q, k, v, indices, counts, sizes, want_lse=True)
            out = oracle.from_bf16(bits)
            assert np.isfinite(out).all(), mode
            assert np.abs(out - want).max() <= 1e-2, mode
            real = (np.arange(64)[None, :] < sizes[:, None]).ravel()
            assert np.abs(lse - want_lse)[:, real].max() <= 5e-2, mode
            got[mode] = bits
    finally:
        gpu.lib.h3b_vsa_fine_mode(0)
    assert np.array_equal(got[1], got[2])


@pytest.mark.parametrize("mode", [0, 1])
def test_vsa_fine_empty_lists(gpu, oracle, mode):
    """A query tile with an empty list gives zero rows (never stale memory or NaN), also when
    only one tile of a pair is empty; the reference's selection never emits such lists
    (cuda/vsa.cuh:52-75 keeps the prefix tiles), so this pins behaviour outside its contract.
    A count above the tile count is refused with status 2."""
    rng = np.random.default_rng(5)
    tiles, heads = 9, 2
    sizes = np.full(tiles, 64, dtype=np.int32)
    q, k, v = (oracle.normal_bf16((heads, tiles * 64, 128), 500 + i) for i in range(3))
    indices, counts = _random_lists(rng, tiles, heads)
    empty = [(0, 0), (0, 1), (0, 4), (1, 3), (1, 8)]          # a whole pair, single halves, the odd last tile
    for h, t in empty:
        counts[h, t] = 0
    _, want, _ = oracle.vsa_fine(q, k, v, indices, np.maximum(counts, 1), sizes)
    try:
        gpu.lib.h3b_vsa_fine_mode(mode)
        bits, _ = _fine_direct(gpu, q, k, v, indices, counts, sizes)
        out = oracle.from_bf16(bits).reshape(heads, tiles, 64, 128)
        want = want.reshape(heads, tiles, 64, 128)
        for h in range(heads):
            for t in range(tiles):
                if (h, t) in empty:
                    assert not bits.reshape(heads, tiles, 64, 128)[h, t].any()
                else:
                    assert np.abs(out[h, t] - want[h, t]).max() <= 1e-2
        too_many = counts.copy()
        too_many[1, 2] = tiles + 1
        bits, _ = _fine_direct(gpu, q, k, v, indices, too_many, sizes, expect_status=2)
        assert np.isfinite(oracle.from_bf16(bits)).all()
    finally:
        gpu.lib.h3b_vsa_fine_mode(0)


def test_vsa_fine_extreme_logits_are_recomputed(gpu, oracle):
    """Query rows whose logits lie hundreds of nats apart inside one tile leave the exponent range
    the persistent kernel covers with one reference per tile; those tiles are recomputed with
    per-row maxima and the result still meets the oracle."""
    rng = np.random.default_rng(9)
    tiles, heads = 6, 2
    sizes = np.full(tiles, 64, dtype=np.int32)
    qf = rng.standard_normal((heads, tiles * 64, 128)).astype(np.float32)
    qf[:, 0::4] *= 64.0          # logits of these rows reach +-250 nats
    qf[:, 1::4] *= 0.0           # these rows see logit 0 for every key
    q = oracle.to_bf16(qf)
    k, v = (oracle.normal_bf16((heads, tiles * 64, 128), 700 + i) for i in range(2))
    indices, counts = _random_lists(rng, tiles, heads, low=2)
    _, want, _ = oracle.vsa_fine(q, k, v, indices, counts, sizes)
    bits, _ = _fine_direct(gpu, q, k, v, indices, counts, sizes)
    out = oracle.from_bf16(bits)
    assert np.isfinite(out).all()
    # near one-hot rows: a bf16 rounding of P can move weight between two close keys
    a, b = out.ravel().astype(np.float64), want.ravel().astype(np.float64)
    assert a @ b / (np.linalg.norm(a) * np.linalg.norm(b)) >= 0.999
    mild = np.ones(q.shape[1], dtype=bool)
    mild[0::4] = False
    assert np.abs(out - want)[:, mild].max() <= 1e-2


def test_vsa_hopper_rejects_bad_lists(gpu, oracle):
    """An out-of-range tile index is refused on the device (status 2), never dereferenced."""
    tiles, heads = 4, 1
    q = oracle.normal_bf16((heads, tiles * 64, 128), 1)
    indices = np.zeros((heads, tiles, tiles), dtype=np.int32)
    indices[0, 1, 0] = 99
    counts = np.ones((heads, tiles), dtype=np.int32)
    sizes = np.full(tiles, 64, dtype=np.int32)
    d = gpu.lib.h3b_tensor_data
    tq = gpu.tensor(q)
    to = gpu.tensor(np.zeros(q.shape, dtype=np.uint16))
    gpu.raw("h3_vsa_hopper", d(to), d(tq), d(tq), d(tq), None, d(gpu.tensor(indices)),
            d(gpu.tensor(counts)), d(gpu.tensor(sizes)), tiles, heads, gpu.lib.h3b_gpu_stream(gpu.gpu))
    assert gpu.device_status() == 2
    assert gpu.device_status() == 0  # cleared by the read
    assert gpu.lib.h3_vsa_hopper(d(to), d(tq), d(tq), d(tq), None, None, None, None, tiles, heads, None) != 0


def test_vsa_new_limits(gpu):
    """Constructor limits of reference cuda/vsa.cuh:195-205."""
    assert not gpu.lib.h3_gpu_vsa_new(gpu.gpu, 0, 11, 1, 2, 3, 2)
    assert not gpu.lib.h3_gpu_vsa_new(gpu.gpu, 3, 11, 1, 2, 3, 57)
    assert not gpu.lib.h3_gpu_vsa_new(gpu.gpu, 3, 11, 4, 4, 4 * 4096, 1)
    assert "at most 4096 tiles" in gpu.error()
