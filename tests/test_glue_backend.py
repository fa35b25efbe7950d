"""The reference's CUDA backend with its attention stages replaced (libh3_cuda_b200.so, built by
h3-omni_b200/glue_build.py from the reference tree through csrc/h3_b200_glue.cu): the reference's
own h3_gpu_create / h3_gpu_vsa_new / tensors, and behind the unchanged h3_gpu_vsa_bf16 and
h3_gpu_ulysses_* names this library's pooling, selection, block-sparse, merge and exchange kernels."""
import ctypes as C
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from refbackend import GLUE_LIB, Reference, ref_vsa_buffers

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def glue(gpu):
    if not GLUE_LIB.exists():
        pytest.skip("libh3_cuda_b200.so not built (needs the reference tree at build time)")
    r = Reference(GLUE_LIB)
    r.lib.h3_ref_vsa_bf16.argtypes = [C.c_void_p] * 6
    yield r
    r.close()


@pytest.mark.parametrize("text,audio,shape,heads", [(17, 30, (7, 8, 8), 4), (17, 448, (37, 15, 27), 2)])
def test_vsa_same_bits_as_the_library(glue, gpu, oracle, text, audio, shape, heads):
    """h3_gpu_vsa_bf16 of the glue build - the reference's object and buffers, this library's
    stages - gives the bits of the library's own h3_gpu_vsa_bf16, lists and pooled means
    included; and the reference's own stages (kept as h3_ref_vsa_bf16: tile_pool, two cuBLAS
    GEMMs, radix-sort selection, pooled softmax, merge around the same block-sparse kernel) agree
    with it to the reference's tolerance."""
    vmap = oracle.VsaMap(text, audio, *shape)
    rows, tiles = vmap.rows, vmap.tiles
    q, k, v = (oracle.normal_bf16((rows, heads, 128), 70 + i) for i in range(3))
    gate = oracle.normal_bf16((rows, heads, 128), 73, 0.3)
    handle = glue.lib.h3_gpu_vsa_new(glue.gpu, text, audio, *shape, heads)
    assert handle
    try:
        ins = [glue.tensor(x) for x in (q, k, v, gate)]
        out = glue.tensor(np.zeros(q.shape, dtype=np.uint16))
        glue.check(glue.lib.h3_gpu_vsa_bf16(handle, out, *ins), "glue vsa")
        got = glue.read(out, q.shape)
        buffers = ref_vsa_buffers(glue, handle, heads, tiles)

        mine = gpu.call("vsa_new", text, audio, *shape, heads)
        try:
            mine_out = gpu.tensor(np.zeros(q.shape, dtype=np.uint16))
            assert gpu.lib.h3_gpu_vsa_bf16(mine, mine_out, *[gpu.tensor(x) for x in (q, k, v, gate)]), gpu.error()
            assert np.array_equal(gpu.read(mine_out, q.shape), got)
            counts = gpu.read_device(gpu.lib.h3b_vsa_buffer(mine, 10), (heads, tiles), np.int32)
            indices = gpu.read_device(gpu.lib.h3b_vsa_buffer(mine, 9), (heads, tiles, tiles), np.int32)
            their_counts = gpu.read_device(buffers["counts"], (heads, tiles), np.int32)
            their_indices = gpu.read_device(buffers["indices"], (heads, tiles, tiles), np.int32)
            assert np.array_equal(counts, their_counts)
            valid = np.arange(tiles)[None, None, :] < counts[:, :, None]
            assert np.array_equal(indices[valid], their_indices[valid])
            for which, name in ((6, "poolq"), (7, "poolk"), (8, "poolv")):
                a = gpu.read_device(gpu.lib.h3b_vsa_buffer(mine, which), (heads, tiles, 128), np.uint32)
                assert np.array_equal(a, gpu.read_device(buffers[name], (heads, tiles, 128), np.uint32)), name
        finally:
            gpu.lib.h3_gpu_vsa_free(mine)

        # the reference's own stages on the same object and inputs
        out_ref = glue.tensor(np.zeros(q.shape, dtype=np.uint16))
        glue.check(glue.lib.h3_ref_vsa_bf16(handle, out_ref, *ins), "reference vsa")
        want = oracle.from_bf16(glue.read(out_ref, q.shape)).astype(np.float64)
        mine_f = oracle.from_bf16(got).astype(np.float64)
        assert np.linalg.norm(mine_f - want) / np.linalg.norm(want) < 0.012     # reference tests/fasth3/vsa.py:131
        assert np.abs(mine_f - want).max() / np.abs(want).max() < 0.03
    finally:
        glue.lib.h3_gpu_vsa_free(handle)


def test_vsa_argument_checks_are_the_references(glue, oracle):
    handle = glue.lib.h3_gpu_vsa_new(glue.gpu, 3, 11, 1, 2, 3, 2)
    assert handle
    try:
        small = glue.empty(16)
        assert not glue.lib.h3_gpu_vsa_bf16(handle, small, small, small, small, small)
        assert b"VSA input/output" in C.string_at(glue.lib.h3_gpu_error(glue.gpu))
        assert not glue.lib.h3_gpu_vsa_bf16(None, small, small, small, small, small)
    finally:
        glue.lib.h3_gpu_vsa_free(handle)


def test_ulysses_through_an_attached_window(gpu, oracle):
    """Two rank threads in one process, the reference's h3_gpu_comm_init_all and contexts: with an
    exchange window attached to each communicator, h3_gpu_ulysses_scatter/gather_heads_bf16 of the
    glue build move the data through this library's push kernel; detached, through the reference's
    own transpose + NCCL code. Both against the oracle's index algebra. Child process, 2 GPUs."""
    if not GLUE_LIB.exists():
        pytest.skip("libh3_cuda_b200.so not built (needs the reference tree at build time)")
    if gpu.lib.h3_gpu_device_count() < 2:
        pytest.skip("needs 2 GPUs")
    code = r'''
import ctypes as C, sys, threading
import numpy as np
sys.path.insert(0, %r); sys.path.insert(0, %r)
import __graft_entry__ as entry
from refbackend import GLUE_LIB, Reference
oracle = entry.load_oracle()
world, rows, H, D = 2, 91, 4, 128
shards = oracle.normal_bf16((world, rows, H, D), 17)
want = oracle.ulysses(shards)
lib = C.CDLL(str(GLUE_LIB))
lib.h3_gpu_comm_init_all.argtypes = [C.c_int, C.c_void_p, C.c_char_p, C.c_size_t]
lib.h3_gpu_select_device.argtypes = [C.c_int, C.c_char_p, C.c_size_t]
for name in ("h3_gpu_ulysses_scatter_heads_bf16", "h3_gpu_ulysses_gather_heads_bf16"):
    getattr(lib, name).argtypes = [C.c_void_p] * 4 + [C.c_uint32] * 3
lib.h3b_glue_attach_exchange.argtypes = [C.c_void_p, C.c_void_p]
core = C.CDLL(str(GLUE_LIB.parent / "libh3b200_attn.so"))
core.h3b_exchange_create_raw.argtypes = [C.c_int, C.c_int, C.c_size_t, C.c_int, C.c_void_p, C.c_void_p]
core.h3b_exchange_connect_local.argtypes = [C.c_void_p, C.c_void_p]
core.h3b_exchange_free.argtypes = [C.c_void_p]
comms = (C.c_void_p * world)()
err = C.create_string_buffer(256)
assert lib.h3_gpu_comm_init_all(world, comms, err, 256), err.value
exchanges = (C.c_void_p * world)()
step = threading.Barrier(world)
failures = []
def run(rank):
    try:
        assert lib.h3_gpu_select_device(rank, err, 256), err.value
        ref = Reference(GLUE_LIB)
        x = C.c_void_p()
        assert core.h3b_exchange_create_raw(rank, world, rows * H * D, 1, C.byref(x), None) == 0
        exchanges[rank] = x
        step.wait(60)
        assert core.h3b_exchange_connect_local(x, exchanges)
        step.wait(60)
        for attach in (True, False):
            assert lib.h3b_glue_attach_exchange(C.c_void_p(comms[rank]), x if attach else None)
            t, scratch = ref.tensor(shards[rank]), ref.empty(rows * H * D)
            ref.check(lib.h3_gpu_ulysses_scatter_heads_bf16(ref.gpu, C.c_void_p(comms[rank]), t, scratch, rows, H, D), "scatter")
            assert np.array_equal(ref.read(t, (world * rows, H // world, D)), want[rank]), ("scatter", attach)
            ref.check(lib.h3_gpu_ulysses_gather_heads_bf16(ref.gpu, C.c_void_p(comms[rank]), t, scratch, rows, H, D), "gather")
            assert np.array_equal(ref.read(t, (rows, H, D)), shards[rank]), ("gather", attach)
            step.wait(60)
        core.h3b_exchange_free(x)
        ref.close()
    except BaseException as e:
        failures.append("rank %%d: %%r" %% (rank, e))
        step.abort()
threads = [threading.Thread(target=run, args=(r,)) for r in range(world)]
for t in threads: t.start()
for t in threads: t.join(180)
assert not failures and not any(t.is_alive() for t in threads), failures
print("OK glue ulysses")
''' % (str(ROOT), str(ROOT / "tests"))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    p = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=400, env=env)
    assert p.returncode == 0 and "OK glue ulysses" in p.stdout, (p.stdout + p.stderr)[-3000:]
