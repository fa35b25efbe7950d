"""Ulysses sequence parallelism: host plan and exchange algebra on CPU (gloo, world size 2),
the in-place scatter/gather primitives on one GPU, and the full multi-rank path on real GPUs
when the box has more than one."""
import ctypes as C
import os
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]


def test_plan_matches_reference_sharding(package):
    from h3_omni_b200 import ulysses
    p = ulysses.plan(101464, 24, 8)          # 10 s clip: no padding at 2, 4, 8 ranks
    assert (p.shard_rows, p.local_heads, p.padded_rows) == (12683, 3, 101464)
    p = ulysses.plan(15400, 56, 7)           # reference-true heads split over 7 ranks
    assert (p.shard_rows, p.local_heads) == (2200, 8)
    p = ulysses.plan(1001, 8, 4)             # padded tail lives on the last rank
    assert p.shard_rows == 251 and [p.valid_rows(r) for r in range(4)] == [251, 251, 251, 248]
    assert p.exchange_bytes() == 251 * 8 * 128 * 2 * 3 // 4
    with pytest.raises(ValueError):
        ulysses.plan(100, 24, 5)


def _gloo_rank(rank, world, port, rows, heads, dim, result):
    """Block transpose + all-to-all exactly as the library orders them, on gloo."""
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    full = torch.arange(world * rows * heads * dim, dtype=torch.int32).reshape(world, rows, heads, dim)
    mine = full[rank].clone()
    group = heads // world
    # scatter: [rows][ranks][group*dim] -> [ranks][rows][group*dim]; block j to rank j
    send = mine.reshape(rows, world, group * dim).transpose(0, 1).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send)
    scattered = recv.reshape(world * rows, group, dim)
    # gather: blocks back, then [ranks][rows][group*dim] -> [rows][ranks][group*dim]
    back = torch.empty_like(recv)
    dist.all_to_all_single(back, recv)
    restored = back.transpose(0, 1).contiguous().reshape(rows, heads, dim)
    result.put((rank, scattered.numpy().copy(), restored.numpy().copy()))
    dist.destroy_process_group()


def test_exchange_algebra_gloo_world2(oracle):
    import torch.multiprocessing as mp
    world, rows, heads, dim = 2, 5, 4, 8
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_gloo_rank, args=(r, world, port, rows, heads, dim, result)) for r in range(world)]
    for p in procs:
        p.start()
    got = sorted(result.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    full = np.arange(world * rows * heads * dim, dtype=np.int32).reshape(world, rows, heads, dim)
    want = oracle.ulysses(full.astype(np.uint16))
    for rank, scattered, restored in got:
        assert np.array_equal(scattered.astype(np.uint16), want[rank])
        assert np.array_equal(restored, full[rank])


@pytest.mark.gpu
def test_single_rank_exchange_is_identity(gpu, oracle):
    comms = (C.c_void_p * 1)()
    err = C.create_string_buffer(256)
    assert gpu.lib.h3_gpu_comm_init_all(1, comms, err, 256), err.value
    comm = C.c_void_p(comms[0])
    try:
        rows, heads = 300, 6
        x = oracle.normal_bf16((rows, heads, 128), 3)
        t, scratch = gpu.tensor(x), gpu.empty_bf16(x.size)
        gpu.call("ulysses_scatter_heads_bf16", comm, t, scratch, rows, heads, 128)
        assert np.array_equal(gpu.read(t, x.shape), x)
        gpu.call("ulysses_gather_heads_bf16", comm, t, scratch, rows, heads, 128)
        assert np.array_equal(gpu.read(t, x.shape), x)
        small = gpu.empty_bf16(16)
        with pytest.raises(RuntimeError, match="Ulysses scratch"):
            gpu.call("ulysses_scatter_heads_bf16", comm, t, small, rows, heads, 128)
    finally:
        gpu.lib.h3_gpu_comm_free(comm)
    bad = C.c_void_p()
    assert not gpu.lib.h3_gpu_comm_init_all(0, None, err, 256)
    with pytest.raises(RuntimeError, match="do not split"):
        gpu.call("ulysses_scatter_heads_bf16", None, t, scratch, rows, heads, 128)


@pytest.mark.gpu
def test_multi_rank_scatter_attention_gather(gpu):
    """One child process per GPU; skipped on a single-GPU box."""
    count = gpu.lib.h3_gpu_device_count()
    if count < 2:
        pytest.skip("needs 2 or more GPUs")
    world = 4 if count >= 4 else 2
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    with tempfile.TemporaryDirectory() as rdv:
        procs = [subprocess.Popen([sys.executable, str(ROOT / "tests" / "ulysses_worker.py"), str(r),
                                   str(world), rdv], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                  text=True, env=env) for r in range(world)]
        outputs = []
        for p in procs:
            try:
                out, _ = p.communicate(timeout=300)
            except subprocess.TimeoutExpired:
                p.kill()
                out, _ = p.communicate()
            outputs.append(out)
        for r, (p, out) in enumerate(zip(procs, outputs)):
            assert p.returncode == 0 and "OK rank %d" % r in out, out[-2000:]


@pytest.mark.gpu
def test_one_process_thread_per_device(gpu, oracle):
    """The reference's own arrangement (h3_dit.c:4031-4185): one process, h3_gpu_comm_init_all,
    one host thread and one h3_gpu context per device. Scatter and gather of a row shard per
    thread against the oracle's index algebra. Run in a child process (its CUDA contexts on
    several devices should not outlive the test); skipped on a single-GPU box."""
    if gpu.lib.h3_gpu_device_count() < 2:
        pytest.skip("needs 2 or more GPUs")
    code = r'''
import ctypes as C, sys, threading
import numpy as np
sys.path.insert(0, %r)
import __graft_entry__ as entry
entry.load_package()
from h3_omni_b200 import native
oracle = entry.load_oracle()
lib = native.load_library()
world, rows, H, D = 2, 77, 6, 128
comms = (C.c_void_p * world)()
err = C.create_string_buffer(256)
assert lib.h3_gpu_comm_init_all(world, comms, err, 256), err.value
shards = oracle.normal_bf16((world, rows, H, D), 41)
want = oracle.ulysses(shards)
failures = []
def run(rank):
    try:
        assert lib.h3_gpu_select_device(rank, err, 256), err.value
        g = native.Native()
        comm = C.c_void_p(comms[rank])
        assert lib.h3b_comm_rank(comm) == rank and lib.h3b_comm_size(comm) == world
        t, scratch = g.tensor(shards[rank]), g.empty_bf16(rows * H * D)
        g.call("ulysses_scatter_heads_bf16", comm, t, scratch, rows, H, D)
        assert np.array_equal(g.read(t, (world * rows, H // world, D)), want[rank]), "scatter"
        g.call("ulysses_gather_heads_bf16", comm, t, scratch, rows, H, D)
        assert np.array_equal(g.read(t, (rows, H, D)), shards[rank]), "gather"
        assert g.device_status() == 0
        g.close()
    except BaseException as e:   # reported by the main thread
        failures.append("rank %%d: %%r" %% (rank, e))
threads = [threading.Thread(target=run, args=(r,)) for r in range(world)]
for t in threads: t.start()
for t in threads: t.join(120)
assert not failures and not any(t.is_alive() for t in threads), failures
for r in range(world): lib.h3_gpu_comm_free(C.c_void_p(comms[r]))
print("OK threads")
''' % str(ROOT)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    p = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300, env=env)
    assert p.returncode == 0 and "OK threads" in p.stdout, (p.stdout + p.stderr)[-3000:]


@pytest.mark.gpu
def test_fused_exchange_between_threads_of_one_process(gpu, oracle):
    """The fused exchange in the reference's own arrangement - one process, one host thread and
    one context per device: windows joined with h3b_exchange_connect_local (a CUDA IPC handle
    cannot be opened by the process that made it). Scatter of q, k, v in one kernel, attention with
    the gather fused into its epilogue, against the oracle. Child process; needs 2 GPUs."""
    if gpu.lib.h3_gpu_device_count() < 2:
        pytest.skip("needs 2 or more GPUs")
    code = r'''
import ctypes as C, sys, threading
import numpy as np
sys.path.insert(0, %r)
import __graft_entry__ as entry
entry.load_package()
from h3_omni_b200 import native, ulysses
oracle = entry.load_oracle()
lib = native.load_library()
world, H, D = 2, 4, 128
L = 2 * 211 + 1
plan = ulysses.plan(L, H, world)
rows = plan.shard_rows
scale = float(1 / np.sqrt(128.0))
full = [oracle.normal_bf16((plan.padded_rows, H, D), 500 + i) for i in range(3)]
for x in full: x[L:] = 0
want, _ = oracle.attention(*[x[None, :L] for x in full], scale)
err = C.create_string_buffer(256)
exchanges = (C.c_void_p * world)()
created, connected = threading.Barrier(world), threading.Barrier(world)
failures = []
def run(rank):
    try:
        assert lib.h3_gpu_select_device(rank, err, 256), err.value
        g = native.Native()
        x = C.c_void_p()
        assert lib.h3b_exchange_create(g.gpu, rank, world, rows * H * D, 4, C.byref(x), (C.c_ubyte * 64)()), g.error()
        exchanges[rank] = x
        created.wait(60)
        assert lib.h3b_exchange_connect_local(x, exchanges), g.error()
        connected.wait(60)
        srcs = [g.tensor(t.reshape(world, rows, H, D)[rank]) for t in full]
        slots = [lib.h3b_exchange_slot(x, i) for i in range(4)]
        for _ in range(2):
            assert lib.h3b_exchange_scatter_heads_multi_bf16(x, 3, (C.c_int * 3)(0, 1, 2), (C.c_void_p * 3)(*srcs), rows, H, D), g.error()
            assert lib.h3b_exchange_sdpa_gather_bf16(x, 3, slots[0], slots[1], slots[2], L, rows, H, scale), g.error()
            got = oracle.from_bf16(g.read(slots[3], (rows, H, D)))
            n = plan.valid_rows(rank)
            assert np.abs(got[:n] - want[0, rank * rows: rank * rows + n]).max() <= 1e-2
        assert g.device_status() == 0
        connected.wait(60)          # nobody frees a window a peer may still store into
        lib.h3b_exchange_free(x)
        g.close()
    except BaseException as e:
        failures.append("rank %%d: %%r" %% (rank, e))
        created.abort(); connected.abort()
threads = [threading.Thread(target=run, args=(r,)) for r in range(world)]
for t in threads: t.start()
for t in threads: t.join(180)
assert not failures and not any(t.is_alive() for t in threads), failures
print("OK local exchange")
''' % str(ROOT)
    p = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=400)
    assert p.returncode == 0 and "OK local exchange" in p.stdout, (p.stdout + p.stderr)[-3000:]


@pytest.mark.gpu
def test_full_size_ten_second_clip_over_ranks(gpu):
    """Benchmark config 4 (L = 101,464, H = 24) over 2 GPUs (4 when the box has them): fused scatters,
    attention with fused gather, sampled rows against the FP64 recomputation. One child process
    per GPU; skipped on a single-GPU box."""
    count = gpu.lib.h3_gpu_device_count()
    if count < 2:
        pytest.skip("needs 2 or more GPUs")
    world = 4 if count >= 4 else 2
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    with tempfile.TemporaryDirectory() as rdv:
        procs = [subprocess.Popen([sys.executable, str(ROOT / "tests" / "long_clip_worker.py"), str(r), str(world), rdv],
                                  stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
                 for r in range(world)]
        outputs = []
        for p in procs:
            try:
                out, _ = p.communicate(timeout=900)
            except subprocess.TimeoutExpired:
                p.kill()
                out, _ = p.communicate()
            outputs.append(out)
        for r, (p, out) in enumerate(zip(procs, outputs)):
            assert p.returncode == 0 and "OK rank %d" % r in out, out[-2000:]
