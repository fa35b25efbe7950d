"""The CPU oracle against golden outputs of the reference's own CUDA code.

tests/golden/reference_*.npz were produced on a B200 by tests/golden/make_reference_fixtures.py
from the reference's unmodified cuda/h3_gpu_cuda.cu (FP32 fallback attention, tile_pool, cuBLAS
pooled scores + pooled_softmax, select_blocks, cuBLAS compression, Q/K norm + RoPE). They pin the restatement in
oracle/h3_attention_oracle.c: integer and order-pinned stages bit for bit, cuBLAS-ordered
floating-point stages to FP32 rounding.
"""
from pathlib import Path

import numpy as np
import pytest

from conftest import ROPE_HALF, assert_rope_close, bf16_step_distance, out_proj_inputs, rope_inputs

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("name,grouped", [("qkv_rope_bf16", False), ("grouped_qkv_rope_bf16", True)])
def test_qkv_rope_matches_reference_kernel(oracle, name, grouped):
    """The reference computes the inverse root mean square with the GPU's approximate rsqrt, the
    oracle with 1/sqrtf: equal except where that last bit decides a bf16 rounding."""
    g = np.load(GOLDEN / "reference_qkv_rope.npz")
    rows, heads, seed = int(g["rows"]), int(g["heads"]), int(g["seed"])
    q, k, v = oracle.qkv_rope(*rope_inputs(oracle, rows, heads, seed), heads, ROPE_HALF, 1e-5, grouped)
    assert np.array_equal(v, g[name + "_v"])
    assert_rope_close(oracle, q, g[name + "_q"])
    assert_rope_close(oracle, k, g[name + "_k"])


def test_fp32_attention_matches_reference_fallback(oracle):
    g = np.load(GOLDEN / "reference_sdpa_f32.npz")
    L, H, seed = int(g["L"]), int(g["H"]), int(g["seed"])
    q, k, v = (oracle.normal_bf16((1, L, H, 128), seed + i) for i in range(3))
    want, _ = oracle.attention(q, k, v, float(1.0 / np.sqrt(128.0)))
    assert np.abs(want[0] - g["out"]).max() < 5e-6


@pytest.mark.parametrize("n", [0, 1, 2])
def test_vsa_coarse_stage_matches_reference(oracle, n):
    g = np.load(GOLDEN / ("reference_vsa_%d.npz" % n))
    heads, seed = int(g["heads"]), int(g["seed"])
    vmap = oracle.VsaMap(int(g["text"]), int(g["audio"]), *[int(x) for x in g["shape"]])
    assert np.array_equal(vmap.map, g["map"]) and np.array_equal(vmap.sizes, g["sizes"])
    q, k, v = (oracle.normal_bf16((vmap.rows, heads, 128), seed + i) for i in range(3))
    gate = np.zeros((vmap.rows, heads, 128), dtype=np.uint16)
    s = oracle.vsa_forward(q, k, v, gate, vmap)
    # gather and pooled means: bit-exact
    assert np.array_equal(s["tiled"][0], g["tiled_q"])
    for mine, name in zip(s["pooled"], ("poolq", "poolk", "poolv")):
        assert np.array_equal(mine.view(np.uint32), g[name].view(np.uint32))
    # selection: identical counts; identical lists except where the reference's cuBLAS-ordered
    # scores and the oracle's fmaf-ordered scores break a near-tie differently
    assert np.array_equal(s["counts"], g["counts"])
    T = vmap.tiles
    mismatched = 0
    for h in range(heads):
        for qt in range(T):
            n_kept = g["counts"][h, qt]
            a, b = g["indices"][h, qt, :n_kept], s["indices"][h, qt, :n_kept]
            if not np.array_equal(a, b):
                mismatched += 1
                swapped = sorted(set(a) ^ set(b))
                sc = s["scores"][h, qt]
                assert max(sc[swapped]) - min(sc[swapped]) <= 1e-5 * max(1.0, np.abs(sc).max())
    assert mismatched <= 1
    # pooled softmax and compression: FP32 rounding of a different summation order
    assert np.abs(s["prob"] - g["prob"]).max() < 1e-6
    assert np.abs(s["compression"] - g["compression"]).max() < 2e-5


def test_out_projection_gate_adaln_matches_reference(oracle):
    """h3_gpu_linear_bf16 (cuBLAS) + h3_gpu_gate_adaln_bf16 of the reference against the oracle's
    restatement: the projection sums in another order (a bf16 rounding flips now and then), gate
    and AdaLN follow the reference kernel's operation order."""
    g = np.load(GOLDEN / "reference_out_proj.npz")
    c = {k: int(g[k]) for k in ("rows", "inner", "hidden", "seed", "slots", "gate", "shift", "scale")}
    x, w, residual, norm_weight, modulation, row_map = out_proj_inputs(oracle, c["rows"], c["inner"], c["hidden"], c["seed"])
    gated, out = oracle.out_proj_gate_adaln(residual, x, w, norm_weight, modulation, modulation, row_map, c["slots"],
                                            c["gate"], c["shift"], c["scale"])
    for mine, name in ((gated, "gated"), (out, "out")):
        d = bf16_step_distance(mine, g[name])
        assert (d != 0).mean() < 0.01, name
        assert np.abs(oracle.from_bf16(mine) - oracle.from_bf16(g[name])).max() <= 2.0 ** -5, name
    # AdaLN on the reference's own gated rows: only 1/sqrtf against the GPU's approximate rsqrtf remains
    _, exact = oracle.out_proj_gate_adaln(g["gated"], x, np.zeros_like(w), norm_weight, np.zeros_like(modulation),
                                          modulation, row_map, c["slots"], c["gate"], c["shift"], c["scale"])
    assert (exact != g["out"]).mean() < 0.005
