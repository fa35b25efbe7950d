"""ctypes binding of the CPU oracle (oracle/h3_attention_oracle.c).

Test infrastructure: imported by tests/, the smoke check and the benchmark's
CPU-baseline leg only. The library under test never imports this module.
All tensors are numpy arrays; 16-bit floats travel as uint16 bit patterns.
"""
import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_LIB = None


def build():
    """Compile the C oracle with the committed Makefile (idempotent)."""
    subprocess.run(["make", "-s", "-C", str(HERE)], check=True)
    return HERE / "libh3_oracle.so"


def lib():
    global _LIB
    if _LIB is None:
        path = HERE / "libh3_oracle.so"
        if not path.exists():
            build()
        _LIB = C.CDLL(str(path))
        _LIB.oracle_time_attention.restype = C.c_double
        _LIB.oracle_vsa_map.restype = C.c_int
    return _LIB


def _p(a):
    """Pointer to a C-contiguous array (the C side indexes raw memory)."""
    if a is None:
        return None
    if not a.flags["C_CONTIGUOUS"]:
        raise ValueError("oracle arrays must be C-contiguous")
    return a.ctypes.data_as(C.c_void_p)


def _c(*arrays):
    return [np.ascontiguousarray(a) for a in arrays]


def to_bf16(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().oracle_f32_to_bf16(_p(x), _p(out), C.c_size_t(x.size))
    return out


def from_bf16(x):
    x = np.ascontiguousarray(x, dtype=np.uint16)
    return (x.astype(np.uint32) << 16).view(np.float32)


def to_f16(x):
    return np.ascontiguousarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def from_f16(x):
    return np.ascontiguousarray(x, dtype=np.uint16).view(np.float16).astype(np.float32)


def normal_bf16(shape, seed, sigma=1.0):
    """Seeded N(0, sigma) bf16 tensor from the oracle's counter-based generator."""
    out = np.empty(shape, dtype=np.uint16)
    lib().oracle_fill_normal_bf16(_p(out), C.c_size_t(out.size), C.c_uint64(seed), C.c_float(sigma))
    return out


def attention(q, k, v, scale, causal=False, elem="bf16", want_lse=False):
    """q: [B, Lq, H, D], k/v: [B, Lk, KH, D] uint16. Returns (out_f32, out_16[, lse])."""
    q, k, v = _c(q, k, v)
    b, lq, h, d = q.shape
    lk, kh = k.shape[1], k.shape[2]
    out32 = np.empty(q.shape, dtype=np.float32)
    out16 = np.empty(q.shape, dtype=np.uint16)
    lse = np.empty((b, h, lq), dtype=np.float32) if want_lse else None
    lib().oracle_attention(_p(out32), _p(out16), _p(lse), _p(q), _p(k), _p(v), b, lq, lk, h, kh, d,
                           C.c_float(scale), int(causal), 1 if elem == "f16" else 0)
    return (out32, out16, lse) if want_lse else (out32, out16)


def attention_rows_f64(rows, q, k, v, scale):
    """q: [Lq, H, D]; rows: int array. Returns [len(rows), H, D] f32 (FP64 accumulation)."""
    q, k, v = _c(q, k, v)
    lq, h, d = q.shape
    lk, kh = k.shape[0], k.shape[1]
    rows = np.ascontiguousarray(rows, dtype=np.int32)
    out = np.empty((len(rows), h, d), dtype=np.float32)
    lib().oracle_attention_rows_f64(_p(out), _p(rows), len(rows), _p(q), _p(k), _p(v), lq, lk, h,
                                    kh, d, C.c_float(scale))
    return out


class VsaMap:
    """Tile map of h3_gpu_vsa_new: map [tiles*64], sizes [tiles], rows, prefix, keep."""

    def __init__(self, text, audio, time, height, width, heads=1):
        info = np.zeros(4, dtype=np.int32)
        tiles = lib().oracle_vsa_map(None, None, _p(info), text, audio, time, height, width, heads)
        if tiles < 0:
            raise ValueError("VSA requires at most 4096 tiles and 56 heads")
        self.map = np.empty(tiles * 64, dtype=np.int32)
        self.sizes = np.empty(tiles, dtype=np.int32)
        lib().oracle_vsa_map(_p(self.map), _p(self.sizes), _p(info), text, audio, time, height,
                             width, heads)
        self.rows, self.tiles, self.prefix, self.keep = (int(x) for x in info)


def vsa_tile_pool(src, vmap, want_tiled=True):
    src, = _c(src)
    rows, heads, d = src.shape
    tiled = np.empty((heads, vmap.tiles * 64, d), dtype=np.uint16) if want_tiled else None
    pooled = np.empty((heads, vmap.tiles, d), dtype=np.float32)
    lib().oracle_vsa_tile_pool(_p(src), _p(tiled), _p(pooled), _p(vmap.map), _p(vmap.sizes),
                               vmap.tiles, heads)
    return tiled, pooled


def vsa_scores(poolq, poolk, scale):
    poolq, poolk = _c(poolq, poolk)
    heads, tiles, _ = poolq.shape
    scores = np.empty((heads, tiles, tiles), dtype=np.float32)
    lib().oracle_vsa_scores(_p(scores), _p(poolq), _p(poolk), tiles, heads, C.c_float(scale))
    return scores


def vsa_select(scores, prefix, keep):
    scores, = _c(scores)
    heads, tiles, _ = scores.shape
    indices = np.full((heads, tiles, tiles), -1, dtype=np.int32)
    counts = np.empty((heads, tiles), dtype=np.int32)
    lib().oracle_vsa_select(_p(scores), _p(indices), _p(counts), tiles, prefix, keep, heads)
    return indices, counts


def vsa_fine(q, k, v, indices, counts, sizes, round_p=True):
    q, k, v, indices, counts, sizes = _c(q, k, v, indices, counts, sizes)
    heads, padded, d = q.shape
    tiles = padded // 64
    out = np.empty(q.shape, dtype=np.uint16)
    out32 = np.empty(q.shape, dtype=np.float32)
    lse = np.empty((heads, padded), dtype=np.float32)
    lib().oracle_vsa_fine(_p(out), _p(out32), _p(lse), _p(q), _p(k), _p(v), _p(indices),
                          _p(counts), _p(sizes), tiles, heads, int(round_p))
    return out, out32, lse


def vsa_pooled_softmax(scores):
    heads, tiles, _ = scores.shape
    prob = np.ascontiguousarray(scores, dtype=np.float32).copy()
    lib().oracle_vsa_pooled_softmax(_p(prob), tiles, heads * tiles)
    return prob


def vsa_compress(prob, poolv):
    prob, poolv = _c(prob, poolv)
    heads, tiles, d = poolv.shape
    out = np.empty((heads, tiles, d), dtype=np.float32)
    lib().oracle_vsa_compress(_p(out), _p(prob), _p(poolv), tiles, heads)
    return out


def vsa_untile_merge(tiled, gate, compression, vmap, out=None):
    tiled, gate, compression = _c(tiled, gate, compression)
    rows, heads, d = gate.shape
    if out is None:
        out = np.zeros((rows, heads, d), dtype=np.uint16)
    lib().oracle_vsa_untile_merge(_p(out), _p(tiled), _p(gate), _p(compression), _p(vmap.map),
                                  vmap.tiles, heads)
    return out


def vsa_forward(q, k, v, gate, vmap, keep=None, round_p=True):
    """Whole h3_gpu_vsa_bf16 pipeline (cuda/vsa.cuh:263-300). Returns a dict of every stage."""
    keep = vmap.keep if keep is None else keep
    scale = np.float32(1.0) / np.sqrt(np.float32(128.0))
    tq, pq = vsa_tile_pool(q, vmap)
    tk, pk = vsa_tile_pool(k, vmap)
    tv, pv = vsa_tile_pool(v, vmap)
    scores = vsa_scores(pq, pk, scale)
    indices, counts = vsa_select(scores, vmap.prefix, keep)
    sparse, sparse32, lse = vsa_fine(tq, tk, tv, indices, counts, vmap.sizes, round_p)
    prob = vsa_pooled_softmax(scores)
    comp = vsa_compress(prob, pv)
    out = vsa_untile_merge(sparse, gate, comp, vmap)
    return dict(tiled=(tq, tk, tv), pooled=(pq, pk, pv), scores=scores, indices=indices,
                counts=counts, sparse=sparse, sparse_f32=sparse32, lse=lse, prob=prob,
                compression=comp, out=out)


def qkv_rope(qkv, q_weight, k_weight, rope_cos, rope_sin, heads, rope_half, epsilon=1e-5, grouped=True):
    """qkv: [rows, 3*heads*128] uint16 (bf16 bits). Returns q, k, v [rows, heads, 128]."""
    qkv, q_weight, k_weight, rope_cos, rope_sin = _c(qkv, q_weight, k_weight, rope_cos, rope_sin)
    rows = qkv.shape[0]
    q, k, v = (np.empty((rows, heads, 128), dtype=np.uint16) for _ in range(3))
    lib().oracle_qkv_rope(_p(q), _p(k), _p(v), _p(qkv), _p(q_weight), _p(k_weight), _p(rope_cos),
                          _p(rope_sin), rows, heads, rope_half, C.c_float(epsilon), int(grouped))
    return q, k, v


def ulysses(x, inverse=False):
    """x: [ranks, rows, heads, dim] -> [ranks, ranks*rows, heads/ranks, dim] (or back)."""
    if not inverse:
        ranks, rows, heads, dim = x.shape
        out = np.empty((ranks, ranks * rows, heads // ranks, dim), dtype=np.uint16)
    else:
        ranks, total, hg, dim = x.shape
        rows, heads = total // ranks, hg * ranks
        out = np.empty((ranks, rows, heads, dim), dtype=np.uint16)
    lib().oracle_ulysses(_p(out), _p(np.ascontiguousarray(x)), ranks, rows, heads, dim,
                         int(inverse))
    return out


def out_proj_gate_adaln(residual, x, w, norm_weight, gate_mod, mod, row_map, slots, gate_slot, shift_slot,
                        scale_slot, epsilon=1e-5, adaln=True):
    """x [rows, inner], w [hidden, inner], residual [rows, hidden], gate_mod / mod [mod rows, slots, hidden]
    bf16 bit patterns; row_map uint32 [rows]. Returns (gated, output or None)."""
    residual, x, w, norm_weight, gate_mod, mod = _c(residual, x, w, norm_weight, gate_mod, mod)
    row_map = np.ascontiguousarray(row_map, dtype=np.uint32)
    rows, inner = x.shape
    hidden = w.shape[0]
    gated = np.empty((rows, hidden), dtype=np.uint16)
    out = np.empty((rows, hidden), dtype=np.uint16) if adaln else None
    lib().oracle_out_proj_gate_adaln(_p(gated), _p(out) if adaln else None, _p(residual), _p(x), _p(w),
                                     _p(norm_weight), _p(gate_mod), _p(mod), _p(row_map), rows, inner, hidden,
                                     slots, gate_slot, shift_slot, scale_slot, C.c_float(epsilon))
    return gated, out


def set_threads(threads):
    """Use `threads` OpenMP threads from now on; returns the count in effect."""
    lib().oracle_set_threads(int(threads))
    return int(lib().oracle_threads())


def threads():
    return int(lib().oracle_threads())


def time_attention(q, k, v, scale):
    """Seconds for one bf16 dense attention pass on all OpenMP threads. q: [Lq,H,D]."""
    q, k, v = _c(q, k, v)
    lq, h, d = q.shape
    out = np.empty(q.shape, dtype=np.uint16)
    return lib().oracle_time_attention(_p(out), _p(q), _p(k), _p(v), lq, k.shape[0], h, d,
                                       C.c_float(scale))
