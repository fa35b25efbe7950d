"""One rank of the full-size Ulysses parity check (benchmark config: 10 s clip, L = 62*1620 + 1024 =
101,464 rows, H = 24, sequence sharded by rank).

usage: long_clip_worker.py RANK WORLD RENDEZVOUS_DIR
Every rank generates the seeded full tensors, keeps its row shard on the GPU, runs the three fused
head scatters and the attention with the gather fused into its epilogue, and checks sampled rows
of its own output shard against the FP64 recomputation of the reference's microbenchmark
(tests/serving/profile/attn_bench.cu:23-55). Prints "OK" on success.
"""
import ctypes as C
import os
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402


def main():
    rank, world, rdv = int(sys.argv[1]), int(sys.argv[2]), Path(sys.argv[3])
    entry.load_package()
    from h3_omni_b200 import native, ulysses
    oracle = entry.load_oracle()
    lib = native.load_library()
    err = C.create_string_buffer(256)
    assert lib.h3_gpu_select_device(rank, err, 256), err.value
    gpu = native.Native()
    L, H, D = 62 * 1620 + 1024, 24, 128
    scale = float(1 / np.sqrt(128.0))
    plan = ulysses.plan(L, H, world)
    rows = plan.shard_rows
    full = [oracle.normal_bf16((L, H, D), 1004 + i) for i in range(3)]
    lo, hi = rank * rows, min(L, (rank + 1) * rows)

    x, handle = C.c_void_p(), (C.c_ubyte * 64)()
    assert lib.h3b_exchange_create(gpu.gpu, rank, world, rows * H * D, 4, C.byref(x), handle), gpu.error()
    tmp = rdv / ("ipc_%d.tmp" % rank)
    tmp.write_bytes(bytes(handle))
    tmp.rename(rdv / ("ipc_%d" % rank))
    deadline = time.time() + 600
    while not all((rdv / ("ipc_%d" % r)).exists() for r in range(world)):
        if time.time() > deadline:
            raise SystemExit("handle rendezvous timed out")
        time.sleep(0.1)
    assert lib.h3b_exchange_connect(x, b"".join((rdv / ("ipc_%d" % r)).read_bytes() for r in range(world))), \
        gpu.error()
    slots = [lib.h3b_exchange_slot(x, i) for i in range(4)]
    for i, t in enumerate(full):
        shard = np.zeros((rows, H, D), dtype=np.uint16)
        shard[:hi - lo] = t[lo:hi]
        src = gpu.tensor(shard)
        assert lib.h3b_exchange_scatter_heads_bf16(x, i, src, rows, H, D), gpu.error()
        gpu.submit()
        gpu.free(src)
    assert lib.h3b_exchange_sdpa_gather_bf16(x, 3, slots[0], slots[1], slots[2], L, rows, H, scale), gpu.error()
    out = gpu.read(slots[3], (rows, H, D))
    assert gpu.device_status() == 0
    rng = np.random.default_rng(rank)
    local = np.unique(np.concatenate([[0, 127, 128, hi - lo - 1], rng.integers(0, hi - lo, 12)])).astype(np.int32)
    want = oracle.attention_rows_f64(local + lo, *full, scale)
    got = oracle.from_bf16(out[local]).astype(np.float64)
    diff = got - want
    max_abs = float(np.abs(diff).max())
    cosine = float((got * want).sum() / (np.linalg.norm(got) * np.linalg.norm(want)))
    rel = float(np.linalg.norm(diff) / np.linalg.norm(want))
    assert max_abs <= 1e-2 and cosine >= 0.9999 and rel <= 0.008, (max_abs, cosine, rel)
    for t in slots:
        lib.h3_gpu_tensor_free(t)
    lib.h3b_exchange_free(x)
    gpu.close()
    print("OK rank %d max-abs %.2e rel-L2 %.2e" % (rank, max_abs, rel), flush=True)


if __name__ == "__main__":
    main()
