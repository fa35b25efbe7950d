"""Generates tests/golden/reference_*.npz ON A GPU BOX from the reference's own CUDA code.

    python tests/golden/make_reference_fixtures.py OUTPUT_DIR

Uses oracle/_ref/libh3_ref_cuda.so (the reference's cuda/h3_gpu_cuda.cu compiled unmodified,
see oracle/ref_build.py). Everything stored here is computed by REFERENCE code:
  reference_sdpa_f32.npz : FP32 fallback attention (cuda/h3_gpu_cuda.cu:1131-1180) on F32 tensors
  reference_qkv_rope.npz : Q/K norm + RoPE (cuda/fast_primitives.cuh:184-265), both input layouts
  reference_vsa_*.npz    : tile map, sizes, tiled Q, pooled means (tile_pool), pooled scores after
                           the in-place softmax (cuBLAS SGEMM + pooled_softmax), index lists and
                           counts (select_blocks), compression (cuBLAS SGEMM)
  reference_out_proj.npz : attention output projection (h3_gpu_linear_bf16, cuBLAS), gate + AdaLN
                           (h3_gpu_gate_adaln_bf16, cuda/fast_primitives.cuh:50-124)
The merged VSA output is NOT stored: its fine stage runs this repository's kernel.
Inputs are regenerated from seeds by the oracle's generator, so only outputs are stored.
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))
import __graft_entry__ as entry  # noqa: E402
import ctypes as C  # noqa: E402

from conftest import ROPE_HALF, out_proj_inputs, rope_inputs  # noqa: E402
from refbackend import Reference, ref_vsa_buffers  # noqa: E402

SDPA_CASE = dict(L=130, H=2, seed=31)
ROPE_CASE = dict(rows=37, heads=5, seed=61)
OUT_PROJ_CASE = dict(rows=37, inner=192, hidden=1024, seed=81, slots=6, gate=2, shift=3, scale=4)
VSA_CASES = [dict(text=3, audio=11, shape=(1, 2, 3), heads=2, seed=700),
             dict(text=65, audio=67, shape=(5, 7, 9), heads=2, seed=710),
             dict(text=17, audio=30, shape=(7, 8, 8), heads=3, seed=720)]


def main(out_dir):
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    entry.load_package()
    from h3_omni_b200 import native
    oracle = entry.load_oracle()
    ours = native.Native()   # only used to copy device buffers back
    ref = Reference()
    scale = float(1.0 / np.sqrt(128.0))
    c = SDPA_CASE
    q, k, v = (oracle.from_bf16(oracle.normal_bf16((c["L"], c["H"], 128), c["seed"] + i)) for i in range(3))
    y = ref.empty(q.size, f32=True)
    ref.check(ref.lib.h3_gpu_sdpa_f32(ref.gpu, y, ref.tensor(q), ref.tensor(k), ref.tensor(v), c["L"], c["H"], 128, scale), "sdpa_f32")
    np.savez_compressed(out_dir / "reference_sdpa_f32.npz", out=ref.read(y, q.shape, f32=True), **c)
    c = ROPE_CASE
    inputs = rope_inputs(oracle, c["rows"], c["heads"], c["seed"])
    stored = dict(c)
    for name in ("qkv_rope_bf16", "grouped_qkv_rope_bf16"):
        outs = [ref.empty(c["rows"] * c["heads"] * 128) for _ in range(3)]
        fn = getattr(ref.lib, "h3_gpu_" + name)
        fn.argtypes = [C.c_void_p] * 9 + [C.c_uint32] * 4 + [C.c_float]
        ref.check(fn(ref.gpu, *outs, *[ref.tensor(x) for x in inputs], c["rows"], c["heads"], 128, ROPE_HALF, 1e-5), name)
        for which, t in zip("qkv", outs):
            stored[name + "_" + which] = ref.read(t, (c["rows"], c["heads"], 128))
    np.savez_compressed(out_dir / "reference_qkv_rope.npz", **stored)
    c = OUT_PROJ_CASE
    x, w, residual, norm_weight, modulation, row_map = out_proj_inputs(oracle, c["rows"], c["inner"], c["hidden"], c["seed"])
    L = ref.lib
    L.h3_gpu_tensor_from_u32.restype = C.c_void_p
    L.h3_gpu_tensor_from_u32.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
    L.h3_gpu_linear_bf16.argtypes = [C.c_void_p] * 5 + [C.c_uint32] * 3
    L.h3_gpu_gate_adaln_bf16.argtypes = [C.c_void_p] * 9 + [C.c_uint32] * 6 + [C.c_float]
    tmap = L.h3_gpu_tensor_from_u32(ref.gpu, row_map.ctypes.data_as(C.c_void_p), row_map.size)
    n = c["rows"] * c["hidden"]
    y, gated, out = ref.empty(n), ref.empty(n), ref.empty(n)
    tmod = ref.tensor(modulation)
    ref.check(L.h3_gpu_linear_bf16(ref.gpu, y, ref.tensor(x), ref.tensor(w), None, c["rows"], c["inner"], c["hidden"]), "linear")
    ref.check(L.h3_gpu_gate_adaln_bf16(ref.gpu, gated, out, ref.tensor(residual), y, ref.tensor(norm_weight), tmod, tmod, tmap,
                                       c["rows"], c["hidden"], c["slots"], c["gate"], c["shift"], c["scale"], 1e-5), "gate_adaln")
    shape = (c["rows"], c["hidden"])
    np.savez_compressed(out_dir / "reference_out_proj.npz", y=ref.read(y, shape), gated=ref.read(gated, shape),
                        out=ref.read(out, shape), **c)
    for n, c in enumerate(VSA_CASES):
        vmap = oracle.VsaMap(c["text"], c["audio"], *c["shape"])
        T, H = vmap.tiles, c["heads"]
        q, k, v = (oracle.normal_bf16((vmap.rows, H, 128), c["seed"] + i) for i in range(3))
        gate = np.zeros((vmap.rows, H, 128), dtype=np.uint16)
        handle = ref.lib.h3_gpu_vsa_new(ref.gpu, c["text"], c["audio"], *c["shape"], H)
        ref.check(handle, "vsa_new")
        out = ref.tensor(np.zeros(q.shape, dtype=np.uint16))
        ref.check(ref.lib.h3_gpu_vsa_bf16(handle, out, ref.tensor(q), ref.tensor(k), ref.tensor(v), ref.tensor(gate)), "vsa")
        dev = ref_vsa_buffers(ref, handle, H, T)
        rd = ours.read_device
        np.savez_compressed(
            out_dir / ("reference_vsa_%d.npz" % n), text=c["text"], audio=c["audio"], shape=c["shape"],
            heads=H, seed=c["seed"], map=rd(dev["map"], (T * 64,), np.int32),
            sizes=rd(dev["sizes"], (T,), np.int32), tiled_q=rd(dev["q"], (H, T * 64, 128), np.uint16),
            poolq=rd(dev["poolq"], (H, T, 128), np.float32), poolk=rd(dev["poolk"], (H, T, 128), np.float32),
            poolv=rd(dev["poolv"], (H, T, 128), np.float32), prob=rd(dev["scores"], (H, T, T), np.float32),
            indices=rd(dev["indices"], (H, T, T), np.int32), counts=rd(dev["counts"], (H, T), np.int32),
            compression=rd(dev["compression"], (H, T, 128), np.float32))
        ref.lib.h3_gpu_vsa_free(handle)
    ref.close()
    ours.close()
    print("wrote fixtures to", out_dir)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else str(ROOT / "tests" / "golden"))
