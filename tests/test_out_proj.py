"""Attention output projection + gate + AdaLN (h3b_attention_output_gate_adaln_bf16): the tcgen05
GEMM with gate and residual in its epilogue and the row-wise AdaLN, against the CPU oracle and
against the reference's own h3_gpu_linear_bf16 + h3_gpu_gate_adaln_bf16 running on the same GPU."""
import ctypes as C

import numpy as np
import pytest

from conftest import bf16_step_distance, out_proj_inputs
from refbackend import REF_LIB, Reference

pytestmark = pytest.mark.gpu
SLOTS, GATE, SHIFT, SCALE_SLOT = 6, 2, 3, 4      # the slots h3_dit.c:2590-2596 uses
CASES = [(70, 256, 1024), (300, 3072, 5376), (129, 7168, 5376), (1, 64, 8), (515, 128, 2056)]


def run_ours(gpu, x, w, residual, norm_weight, modulation, row_map, adaln=True, in_place=False):
    rows, inner = x.shape
    hidden = w.shape[0]
    t = [gpu.tensor(a) for a in (residual, x, w, norm_weight, modulation, modulation, row_map)]
    gated = t[0] if in_place else gpu.empty_bf16(rows * hidden)
    out = gpu.empty_bf16(rows * hidden) if adaln else None
    ok = gpu.lib.h3b_attention_output_gate_adaln_bf16(gpu.gpu, gated, out, *t, rows, inner, hidden, SLOTS, GATE, SHIFT,
                                                      SCALE_SLOT, C.c_float(1e-5))
    assert ok, gpu.error()
    return gpu.read(gated, (rows, hidden)), gpu.read(out, (rows, hidden)) if adaln else None


def close_to(oracle, got, want, what):
    """Two results of the chain that differ only in the summation order of the projection: the
    projected value differs by FP32 rounding, which now and then decides a bf16 rounding."""
    d = bf16_step_distance(got, want)
    assert (d != 0).mean() < 0.02, what
    a, b = oracle.from_bf16(got).astype(np.float64), oracle.from_bf16(want).astype(np.float64)
    assert np.linalg.norm(a - b) / np.linalg.norm(b) < 0.004, what      # half of the reference's bf16 limit (acceptance.json:5-8)
    assert np.abs(a - b).max() <= 2.0 ** -4, what


@pytest.mark.parametrize("rows,inner,hidden", CASES)
def test_against_the_oracle(gpu, oracle, rows, inner, hidden):
    inputs = out_proj_inputs(oracle, rows, inner, hidden, 900 + rows)
    x, w, residual, norm_weight, modulation, row_map = inputs
    gated, out = run_ours(gpu, *inputs)
    want_gated, want_out = oracle.out_proj_gate_adaln(residual, x, w, norm_weight, modulation, modulation, row_map, SLOTS,
                                                      GATE, SHIFT, SCALE_SLOT)
    close_to(oracle, gated, want_gated, "gated residual")
    close_to(oracle, out, want_out, "AdaLN output")
    # AdaLN alone, on the GPU's own gated rows: only the approximate rsqrt separates it from the oracle
    _, exact_out = oracle.out_proj_gate_adaln(gated, x, np.zeros_like(w), norm_weight, np.zeros_like(modulation), modulation,
                                              row_map, SLOTS, GATE, SHIFT, SCALE_SLOT)
    # (a flipped rounding of the normalised value is scaled and shifted afterwards, so a few
    # elements land more than one bf16 step away)
    assert (out != exact_out).mean() < 0.01
    assert np.abs(oracle.from_bf16(out) - oracle.from_bf16(exact_out)).max() <= 2.0 ** -5
    # gate only, and in place over the residual stream
    only_gate, none = run_ours(gpu, *inputs, adaln=False)
    assert none is None and np.array_equal(only_gate, gated)
    in_place, _ = run_ours(gpu, *inputs, in_place=True)
    assert np.array_equal(in_place, gated)
    assert gpu.device_status() == 0


def test_argument_checks(gpu, oracle):
    x, w, residual, norm_weight, modulation, row_map = out_proj_inputs(oracle, 8, 64, 64, 1)
    t = [gpu.tensor(a) for a in (residual, x, w, norm_weight, modulation, modulation, row_map)]
    out = gpu.empty_bf16(8 * 64)
    call = gpu.lib.h3b_attention_output_gate_adaln_bf16
    assert not call(gpu.gpu, out, out, *t, 8, 60, 64, SLOTS, GATE, SHIFT, SCALE_SLOT, C.c_float(1e-5))
    assert "multiple of 64" in gpu.error()
    assert not call(gpu.gpu, out, out, *t, 8, 64, 64, SLOTS, SLOTS, SHIFT, SCALE_SLOT, C.c_float(1e-5))
    small = gpu.empty_bf16(4)
    assert not call(gpu.gpu, small, out, *t, 8, 64, 64, SLOTS, GATE, SHIFT, SCALE_SLOT, C.c_float(1e-5))
    assert "gate output" in gpu.error()


@pytest.mark.parametrize("rows,inner,hidden", [(70, 256, 1024), (300, 3072, 5376)])
def test_against_the_reference_kernels(gpu, oracle, rows, inner, hidden):
    """h3_gpu_linear_bf16 + h3_gpu_gate_adaln_bf16 of the reference's own backend on this GPU: the
    gated rows agree up to the summation order of the projection (cuBLAS there); AdaLN on the same
    gated rows is bit-identical."""
    if not REF_LIB.exists():
        pytest.skip("oracle/_ref/libh3_ref_cuda.so not built (needs the reference tree at build time)")
    ref = Reference()
    try:
        L = ref.lib
        L.h3_gpu_tensor_from_u32.restype = C.c_void_p
        L.h3_gpu_tensor_from_u32.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        L.h3_gpu_linear_bf16.argtypes = [C.c_void_p] * 5 + [C.c_uint32] * 3
        L.h3_gpu_gate_adaln_bf16.argtypes = [C.c_void_p] * 9 + [C.c_uint32] * 6 + [C.c_float]
        L.h3_gpu_adaln_bf16.argtypes = [C.c_void_p] * 6 + [C.c_uint32] * 5 + [C.c_float]
        inputs = out_proj_inputs(oracle, rows, inner, hidden, 900 + rows)
        x, w, residual, norm_weight, modulation, row_map = inputs
        gated, out = run_ours(gpu, *inputs)
        tx, tw, tres, tnorm, tmod = (ref.tensor(a) for a in (x, w, residual, norm_weight, modulation))
        tmap = L.h3_gpu_tensor_from_u32(ref.gpu, row_map.ctypes.data_as(C.c_void_p), row_map.size)
        y, their_gated, their_out = ref.empty(rows * hidden), ref.empty(rows * hidden), ref.empty(rows * hidden)
        ref.check(L.h3_gpu_linear_bf16(ref.gpu, y, tx, tw, None, rows, inner, hidden), "linear")
        ref.check(L.h3_gpu_gate_adaln_bf16(ref.gpu, their_gated, their_out, tres, y, tnorm, tmod, tmod, tmap, rows, hidden,
                                           SLOTS, GATE, SHIFT, SCALE_SLOT, 1e-5), "gate_adaln")
        close_to(oracle, gated, ref.read(their_gated, (rows, hidden)), "gated residual vs reference")
        close_to(oracle, out, ref.read(their_out, (rows, hidden)), "AdaLN output vs reference")
        same_rows = ref.tensor(gated)
        exact = ref.empty(rows * hidden)
        ref.check(L.h3_gpu_adaln_bf16(ref.gpu, exact, same_rows, tnorm, tmod, tmap, rows, hidden, SLOTS, SHIFT, SCALE_SLOT,
                                      1e-5), "adaln")
        assert np.array_equal(ref.read(exact, (rows, hidden)), out)
        L.h3_gpu_tensor_free(tmap)
    finally:
        ref.close()
