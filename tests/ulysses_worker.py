"""One rank of the multi-GPU Ulysses test (run as a child process per GPU).

usage: ulysses_worker.py RANK WORLD RENDEZVOUS_DIR
Scatters row shards of Q, K, V, runs attention on this rank's heads over the whole sequence,
gathers the output, and checks every step against the CPU oracle. Prints "OK" on success.
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
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    entry.load_package()
    from h3_omni_b200 import native, ulysses
    oracle = entry.load_oracle()
    lib = native.load_library()
    err = C.create_string_buffer(256)
    assert lib.h3_gpu_select_device(rank, err, 256), err.value
    gpu = native.Native()
    ident = rdv / "nccl_id"
    if rank == 0:
        buf = (C.c_ubyte * 128)()
        assert lib.h3b_comm_unique_id(buf, err, 256), err.value
        tmp = rdv / "nccl_id.tmp"
        tmp.write_bytes(bytes(buf))
        tmp.rename(ident)
    deadline = time.time() + 120
    while not ident.exists():
        if time.time() > deadline:
            raise SystemExit("rendezvous timed out")
        time.sleep(0.05)
    comm = C.c_void_p()
    assert lib.h3b_comm_init_rank(ident.read_bytes(), rank, world, C.byref(comm), err, 256), err.value
    assert lib.h3b_comm_rank(comm) == rank and lib.h3b_comm_size(comm) == world

    L, H, D = 8 * world * 37 + 5, 8, 128   # not a multiple of the rank count: padded tail
    scale = float(1 / np.sqrt(128.0))
    plan = ulysses.plan(L, H, world)
    rows = plan.shard_rows
    full = [oracle.normal_bf16((plan.padded_rows, H, D), 300 + i) for i in range(3)]
    for x in full:
        x[L:] = 0
    shards = [x.reshape(world, rows, H, D) for x in full]
    scratch = gpu.empty_bf16(rows * H * D)
    tensors = [gpu.tensor(s[rank]) for s in shards]
    for t, s in zip(tensors, shards):
        gpu.call("ulysses_scatter_heads_bf16", comm, t, scratch, rows, H, D)
        got = gpu.read(t, (world * rows, H // world, D))
        assert np.array_equal(got, oracle.ulysses(s)[rank]), "scatter mismatch"
    out = gpu.empty_bf16(rows * H * D)
    gpu.call("zero", out)
    gpu.call("sdpa_bf16", out, *tensors, L, plan.local_heads, D, scale)
    local = gpu.read(out, (world * rows, H // world, D)).copy()
    hs = slice(rank * plan.local_heads, (rank + 1) * plan.local_heads)
    want, _ = oracle.attention(full[0][None, :L, hs], full[1][None, :L, hs], full[2][None, :L, hs], scale)
    err_max = np.abs(oracle.from_bf16(local[:L]) - want[0]).max()
    assert err_max <= 1e-2, err_max
    gpu.call("ulysses_gather_heads_bf16", comm, out, scratch, rows, H, D)
    gathered = gpu.read(out, (rows, H, D))
    # every rank's heads of my rows: recompute with the oracle on my valid rows
    mine = slice(rank * rows, min(L, (rank + 1) * rows))
    n = mine.stop - mine.start
    if n > 0:
        want_rows, _ = oracle.attention(full[0][None, mine], full[1][None, :L], full[2][None, :L], scale)
        assert np.abs(oracle.from_bf16(gathered[:n]) - want_rows[0]).max() <= 1e-2
    # all-gather of a row shard
    total = gpu.empty_bf16(world * rows * H * D)
    src = gpu.tensor(shards[0][rank])
    gpu.call("all_gather_bf16", comm, total, src, rows * H * D)
    assert np.array_equal(gpu.read(total, (world, rows, H, D)), shards[0])
    assert gpu.device_status() == 0

    # ---- the fused exchange over peer memory must move the same bytes as the NCCL path ----
    x = C.c_void_p()
    handle = (C.c_ubyte * 64)()
    assert lib.h3b_exchange_create(gpu.gpu, rank, world, rows * H * D, 4, C.byref(x), handle), gpu.error()
    tmp = rdv / ("ipc_%d.tmp" % rank)
    tmp.write_bytes(bytes(handle))
    tmp.rename(rdv / ("ipc_%d" % rank))
    deadline = time.time() + 120
    while not all((rdv / ("ipc_%d" % r)).exists() for r in range(world)):
        if time.time() > deadline:
            raise SystemExit("handle rendezvous timed out")
        time.sleep(0.05)
    handles = b"".join((rdv / ("ipc_%d" % r)).read_bytes() for r in range(world))
    assert lib.h3b_exchange_connect(x, handles), gpu.error()
    slots = [lib.h3b_exchange_slot(x, i) for i in range(4)]
    for epoch in range(2):   # twice: the epoch handshake must hold across repeated exchanges
        for i, sh in enumerate(shards):
            src = gpu.tensor(sh[rank])
            assert lib.h3b_exchange_scatter_heads_bf16(x, i, src, rows, H, D), gpu.error()
            got = gpu.read(slots[i], (world * rows, H // world, D))
            assert np.array_equal(got, oracle.ulysses(sh)[rank]), "fused scatter mismatch"
        out2 = gpu.empty_bf16(rows * H * D)
        gpu.call("zero", out2)
        gpu.call("sdpa_bf16", out2, slots[0], slots[1], slots[2], L, plan.local_heads, D, scale)
        assert np.array_equal(gpu.read(out2, (world * rows, H // world, D))[:L], local[:L])
        assert lib.h3b_exchange_gather_heads_bf16(x, 3, out2, rows, H, D), gpu.error()
        fused = gpu.read(slots[3], (rows, H, D))
        assert np.array_equal(fused[:n], gathered[:n]), "fused gather differs from the NCCL gather"
        # attention with the gather fused into its epilogue: same bits, one launch less
        gpu.call("zero", slots[3])
        assert lib.h3b_exchange_sdpa_gather_bf16(x, 3, slots[0], slots[1], slots[2], L, rows, H, scale), gpu.error()
        fused2 = gpu.read(slots[3], (rows, H, D))
        assert np.array_equal(fused2[:n], gathered[:n]), "attention with fused gather differs"
        assert gpu.device_status() == 0
    # ---- q, k and v scattered by ONE kernel: the same bytes as three single scatters ----
    singles = [oracle.ulysses(sh)[rank] for sh in shards]
    for i in range(3):
        gpu.call("zero", slots[i])
    srcs = [gpu.tensor(sh[rank]) for sh in shards]
    order = (C.c_int * 3)(2, 0, 1)                      # any distinct slots
    assert lib.h3b_exchange_scatter_heads_multi_bf16(x, 3, order, (C.c_void_p * 3)(*srcs), rows, H, D), gpu.error()
    for i, slot in enumerate(order):
        assert np.array_equal(gpu.read(slots[slot], (world * rows, H // world, D)), singles[i]), "multi scatter"
    assert not lib.h3b_exchange_scatter_heads_multi_bf16(x, 2, (C.c_int * 2)(1, 1), (C.c_void_p * 2)(*srcs[:2]), rows, H, D)
    # ---- one slot reused back to back with a reader in between (no other exchange between them):
    # the second scatter may overwrite the slot only after every rank's reader has run ----
    keep = gpu.empty_bf16(rows * H * D)
    for round_ in range(6):
        a, b = srcs[round_ % 3], srcs[(round_ + 1) % 3]
        assert lib.h3b_exchange_scatter_heads_bf16(x, 0, a, rows, H, D), gpu.error()
        gpu.call("copy_bf16", keep, 0, slots[0], 0, rows * H * D)          # the reader, queued on the stream
        assert lib.h3b_exchange_scatter_heads_bf16(x, 0, b, rows, H, D), gpu.error()
        assert np.array_equal(gpu.read(keep, (world * rows, H // world, D)), singles[round_ % 3]), "reader saw the next exchange"
        assert np.array_equal(gpu.read(slots[0], (world * rows, H // world, D)), singles[(round_ + 1) % 3])
    assert gpu.device_status() == 0
    # ---- norm + RoPE fused with the scatter: same bits as norm + RoPE followed by three scatters ----
    half = 48
    qkv = oracle.normal_bf16((world, rows, 3 * H * D), 77, 1.5)   # every rank's rows of the projection
    rng = np.random.default_rng(5)
    qw, kw = (oracle.to_bf16(1.0 + 0.2 * rng.standard_normal(D).astype(np.float32)) for _ in range(2))
    angle = rng.uniform(0.0, 6.28, (world, rows, half)).astype(np.float32)
    tin = [gpu.tensor(a) for a in (qkv[rank], qw, kw, oracle.to_bf16(np.cos(angle[rank])),
                                   oracle.to_bf16(np.sin(angle[rank])))]
    parts = [gpu.empty_bf16(rows * H * D) for _ in range(3)]
    gpu.call("grouped_qkv_rope_bf16", *parts, *tin, rows, H, D, half, 1e-5)
    unfused = []
    for i, part in enumerate(parts):
        assert lib.h3b_exchange_scatter_heads_bf16(x, i, part, rows, H, D), gpu.error()
        unfused.append(gpu.read(slots[i], (world * rows, H // world, D)).copy())
    for i in range(3):
        gpu.call("zero", slots[i])
    # every rank must have cleared its slots before any peer stores into them again
    assert lib.h3b_exchange_gather_heads_bf16(x, 3, out2, rows, H, D), gpu.error()
    gpu.submit()
    assert lib.h3b_exchange_qkv_rope_scatter_bf16(x, 0, 1, 2, *tin, rows, H, half, C.c_float(1e-5), 1), gpu.error()
    for i in range(3):
        assert np.array_equal(gpu.read(slots[i], (world * rows, H // world, D)), unfused[i]), \
            "fused norm/RoPE scatter differs (tensor %d)" % i
    assert gpu.device_status() == 0
    for t in slots:
        lib.h3_gpu_tensor_free(t)
    lib.h3b_exchange_free(x)

    # ---- video sparse attention under Ulysses (reference h3_dit.c:2496-2525: scatter q, k, v and
    # the gate, VSA on this rank's heads over the whole sequence, gather): bit-identical to the
    # same call with all heads on one GPU ----
    text, audio, grid = 21, 64, (4, 8, 16)
    Lv = text + audio + grid[0] * grid[1] * grid[2]
    vplan = ulysses.plan(Lv, H, world)
    vrows = vplan.shard_rows
    vfull = [oracle.normal_bf16((vplan.padded_rows, H, D), 900 + i, 0.3 if i == 3 else 1.0) for i in range(4)]
    for t in vfull:
        t[Lv:] = 0
    x2, handle2 = C.c_void_p(), (C.c_ubyte * 64)()
    assert lib.h3b_exchange_create(gpu.gpu, rank, world, vrows * H * D, 5, C.byref(x2), handle2), gpu.error()
    tmp = rdv / ("ipcv_%d.tmp" % rank)
    tmp.write_bytes(bytes(handle2))
    tmp.rename(rdv / ("ipcv_%d" % rank))
    deadline = time.time() + 120
    while not all((rdv / ("ipcv_%d" % r)).exists() for r in range(world)):
        if time.time() > deadline:
            raise SystemExit("handle rendezvous timed out")
        time.sleep(0.05)
    assert lib.h3b_exchange_connect(x2, b"".join((rdv / ("ipcv_%d" % r)).read_bytes() for r in range(world))), \
        gpu.error()
    vslots = [lib.h3b_exchange_slot(x2, i) for i in range(5)]
    for i, t in enumerate(vfull):
        shard = gpu.tensor(t.reshape(world, vrows, H, D)[rank])
        assert lib.h3b_exchange_scatter_heads_bf16(x2, i, shard, vrows, H, D), gpu.error()
    local_vsa = gpu.call("vsa_new", text, audio, *grid, H // world)
    local_out = gpu.empty_bf16(world * vrows * (H // world) * D)
    gpu.call("zero", local_out)
    assert lib.h3_gpu_vsa_bf16(local_vsa, local_out, *vslots[:4]), gpu.error()
    assert lib.h3b_exchange_gather_heads_bf16(x2, 4, local_out, vrows, H, D), gpu.error()
    sharded = gpu.read(vslots[4], (vrows, H, D))
    whole_vsa = gpu.call("vsa_new", text, audio, *grid, H)
    whole_out = gpu.empty_bf16(Lv * H * D)
    assert lib.h3_gpu_vsa_bf16(whole_vsa, whole_out, *[gpu.tensor(t[:Lv]) for t in vfull]), gpu.error()
    whole = gpu.read(whole_out, (Lv, H, D))
    lo, hi = rank * vrows, min(Lv, (rank + 1) * vrows)
    assert np.array_equal(sharded[:hi - lo], whole[lo:hi]), "VSA over head shards differs from one GPU"
    stages = oracle.vsa_forward(*[t[:Lv] for t in vfull], oracle.VsaMap(text, audio, *grid))
    want = oracle.from_bf16(stages["out"][lo:hi]).astype(np.float64)
    got = oracle.from_bf16(sharded[:hi - lo]).astype(np.float64)
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 0.012   # reference tests/fasth3/vsa.py:131
    assert gpu.device_status() == 0
    lib.h3_gpu_vsa_free(local_vsa)
    lib.h3_gpu_vsa_free(whole_vsa)
    for t in vslots:
        lib.h3_gpu_tensor_free(t)
    lib.h3b_exchange_free(x2)
    lib.h3_gpu_comm_free(comm)
    gpu.close()
    print("OK rank %d" % rank, flush=True)


if __name__ == "__main__":
    main()
