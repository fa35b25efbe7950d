"""Failure paths without faulting anything: a bounded device-side wait that runs out, an aborted
communicator, a context used with the wrong device current. Nothing here hangs, traps or
faults a GPU: the waits are short, and the failures are made on the host or by a flag that
nobody sets."""
import ctypes as C
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _exchange_pair(gpu, elements, slots=2):
    """Two exchange objects - ranks 0 and 1 of 2 - in this process on this device, joined by their
    plain pointers (what h3b_exchange_connect_local is for)."""
    xs = (C.c_void_p * 2)()
    for rank in range(2):
        x = C.c_void_p()
        assert gpu.lib.h3b_exchange_create(gpu.gpu, rank, 2, elements, slots, C.byref(x), (C.c_ubyte * 64)()), gpu.error()
        xs[rank] = x
    for rank in range(2):
        assert gpu.lib.h3b_exchange_connect_local(C.c_void_p(xs[rank]), xs), gpu.error()
    return xs


def test_bounded_wait_runs_out_and_is_reported(gpu, oracle):
    """Rank 0 starts an exchange that rank 1 never joins: the flag it waits for is never set. The
    wait gives up after its limit (200 ms here), the kernel stores nothing and returns, the next
    submit fails with the time-out message, and the context works again after that."""
    rows, heads = 64, 4
    x = oracle.normal_bf16((rows, heads, 128), 5)
    xs = _exchange_pair(gpu, x.size)
    try:
        assert gpu.lib.h3b_exchange_set_wait_limit_ms(C.c_void_p(xs[0]), 200)
        src = gpu.tensor(x)
        assert gpu.device_status() == 0
        start = time.monotonic()
        assert gpu.lib.h3b_exchange_scatter_heads_bf16(C.c_void_p(xs[0]), 0, src, rows, heads, 128), gpu.error()
        assert not gpu.lib.h3_gpu_submit(gpu.gpu)
        elapsed = time.monotonic() - start
        assert "device-side wait timed out" in gpu.error()
        assert 0.15 < elapsed < 5.0, elapsed
        # reported once: the word was cleared by that submit
        assert gpu.lib.h3_gpu_submit(gpu.gpu), gpu.error()
        assert gpu.device_status() == 0
        # nothing was stored into the peer's window (its slot is still zero) ...
        peer_slot = gpu.lib.h3b_exchange_slot_pointer(C.c_void_p(xs[1]), 0)
        assert not gpu.read_device(peer_slot, (x.size,), np.uint16).any()
        # ... and the context computes as before
        q, k, v = (oracle.normal_bf16((1, 200, 2, 128), 6 + i) for i in range(3))
        tq, tk, tv, ty = gpu.tensor(q), gpu.tensor(k), gpu.tensor(v), gpu.empty_bf16(q.size)
        gpu.call("sdpa_bf16", ty, tq, tk, tv, 200, 2, 128, float(1 / np.sqrt(128)))
        want, _ = oracle.attention(q, k, v, float(1 / np.sqrt(128)))
        assert np.abs(oracle.from_bf16(gpu.read(ty, q.shape)) - want).max() <= 1e-2
    finally:
        for rank in range(2):
            gpu.lib.h3b_exchange_free(C.c_void_p(xs[rank]))


def test_unconnected_and_mismatched_exchange_is_refused(gpu, oracle):
    x = C.c_void_p()
    assert gpu.lib.h3b_exchange_create(gpu.gpu, 0, 2, 1024, 1, C.byref(x), (C.c_ubyte * 64)()), gpu.error()
    try:
        src = gpu.empty_bf16(1024)
        assert not gpu.lib.h3b_exchange_scatter_heads_bf16(x, 0, src, 4, 2, 128)
        assert "not connected" in gpu.error()
        assert not gpu.lib.h3b_exchange_connect_local(x, (C.c_void_p * 2)(x, x))   # rank 1 is missing
        assert "does not match" in gpu.error()
        assert not gpu.lib.h3b_exchange_set_wait_limit_ms(x, 0)
    finally:
        gpu.lib.h3b_exchange_free(x)


def test_aborted_communicator_fails_cleanly(gpu, oracle):
    """h3_gpu_comm_abort (reference cuda/parallel.cuh:60-65; the rank group calls it when one rank
    has failed, h3_dit.c:4054-4071) on a communicator no kernel is using: later collectives on
    it are refused with a message instead of touching the dead communicator, and freeing it is
    still fine."""
    comms = (C.c_void_p * 1)()
    err = C.create_string_buffer(256)
    assert gpu.lib.h3_gpu_comm_init_all(1, comms, err, 256), err.value
    comm = C.c_void_p(comms[0])
    rows, heads = 50, 2
    x = oracle.normal_bf16((rows, heads, 128), 8)
    t, scratch = gpu.tensor(x), gpu.empty_bf16(x.size)
    gpu.call("ulysses_scatter_heads_bf16", comm, t, scratch, rows, heads, 128)
    gpu.submit()
    gpu.lib.h3_gpu_comm_abort(comm)
    with pytest.raises(RuntimeError, match="do not split"):
        gpu.call("ulysses_scatter_heads_bf16", comm, t, scratch, rows, heads, 128)
    assert not gpu.lib.h3_gpu_all_gather_bf16(gpu.gpu, comm, scratch, t, 16)
    gpu.lib.h3_gpu_comm_abort(comm)      # a second abort is a no-op
    gpu.lib.h3_gpu_comm_abort(None)
    gpu.lib.h3_gpu_comm_free(comm)
    assert np.array_equal(gpu.read(t, x.shape), x)
    assert gpu.device_status() == 0


def test_attention_output_may_alias_the_exchange_scratch(gpu, oracle):
    """The reference's buffer plan (h3_dit.c:1647-1650, 2529-2546): the QKV projection buffer is
    the scratch of the three scatters, attention then writes its output INTO that buffer
    (attention_heads aliases qkv) while reading q, k, v, and the gather uses the query tensor
    as its scratch. Same sequence here through the NCCL-path primitives on one rank."""
    comms = (C.c_void_p * 1)()
    err = C.create_string_buffer(256)
    assert gpu.lib.h3_gpu_comm_init_all(1, comms, err, 256), err.value
    comm = C.c_void_p(comms[0])
    try:
        rows, heads = 333, 4
        scale = float(1 / np.sqrt(128))
        q, k, v = (oracle.normal_bf16((1, rows, heads, 128), 60 + i) for i in range(3))
        tq, tk, tv = gpu.tensor(q), gpu.tensor(k), gpu.tensor(v)
        qkv = gpu.tensor(oracle.normal_bf16((rows, 3 * heads * 128), 63))     # holds the projection, then scratch
        for t in (tq, tk, tv):
            gpu.call("ulysses_scatter_heads_bf16", comm, t, qkv, rows, heads, 128)
        gpu.call("sdpa_bf16", qkv, tq, tk, tv, rows, heads, 128, scale)       # output aliases the scratch
        gpu.call("ulysses_gather_heads_bf16", comm, qkv, tq, rows, heads, 128)  # the query is scratch now
        flat = gpu.read(qkv, (rows * 3 * heads * 128,))
        got = oracle.from_bf16(flat[:rows * heads * 128].reshape(1, rows, heads, 128))
        want, _ = oracle.attention(q, k, v, scale)
        assert np.abs(got - want).max() <= 1e-2
        assert gpu.device_status() == 0
    finally:
        gpu.lib.h3_gpu_comm_free(comm)


def test_submit_refuses_a_context_of_another_device(gpu):
    if gpu.lib.h3_gpu_device_count() < 2:
        pytest.skip("needs 2 GPUs")
    err = C.create_string_buffer(256)
    assert gpu.lib.h3_gpu_select_device(1, err, 256), err.value
    try:
        assert not gpu.lib.h3_gpu_submit(gpu.gpu)
        assert "is current" in gpu.error()
    finally:
        assert gpu.lib.h3_gpu_select_device(0, err, 256), err.value


def test_launches_after_a_recorded_failure_do_nothing_until_it_is_reported(gpu, oracle):
    """Once the device status word holds a failure, the dense attention kernel's CTAs leave at
    once (so a protocol error cannot make thousands of CTAs run into their wait limits one wave
    after the other): the output keeps what was in it. The failure is reported by the next submit,
    which clears the word, and the same launch then computes."""
    d = gpu.lib.h3b_tensor_data
    stream = gpu.lib.h3b_gpu_stream(gpu.gpu)
    # a refused index list (a count beyond the number of tiles) records status 2 without any fault
    tiles, heads = 4, 1
    fq, fk, fv = (oracle.normal_bf16((heads, tiles * 64, 128), 70 + i) for i in range(3))
    indices = np.tile(np.arange(tiles, dtype=np.int32), (heads, tiles, 1))
    counts = np.full((heads, tiles), tiles + 1, dtype=np.int32)
    sizes = np.full(tiles, 64, dtype=np.int32)
    ft = [gpu.tensor(x) for x in (fq, fk, fv, indices, counts, sizes)]
    fo = gpu.empty_bf16(fq.size)
    gpu.raw("h3_vsa_hopper", d(fo), d(ft[0]), d(ft[1]), d(ft[2]), None, d(ft[3]), d(ft[4]), d(ft[5]), tiles, heads,
            stream)
    # dense attention with more than one query tile, into an output that holds a marker
    L, H = 300, 2
    q, k, v = (oracle.normal_bf16((1, L, H, 128), 80 + i) for i in range(3))
    tq, tk, tv = gpu.tensor(q), gpu.tensor(k), gpu.tensor(v)
    marker = np.full(q.shape, 0x1234, dtype=np.uint16)
    ty = gpu.tensor(marker)
    scale = C.c_float(float(1 / np.sqrt(128)))
    gpu.raw("h3_flash3_bf16", d(ty), d(tq), d(tk), d(tv), None, 1, L, H, H, scale, stream)
    assert not gpu.lib.h3_gpu_submit(gpu.gpu)
    assert "bounds check failed" in gpu.error()
    assert gpu.lib.h3_gpu_submit(gpu.gpu), gpu.error()
    assert np.array_equal(gpu.read(ty, q.shape), marker)
    gpu.raw("h3_flash3_bf16", d(ty), d(tq), d(tk), d(tv), None, 1, L, H, H, scale, stream)
    want, _ = oracle.attention(q, k, v, float(1 / np.sqrt(128)))
    assert np.abs(oracle.from_bf16(gpu.read(ty, q.shape)) - want).max() <= 1e-2
    for t in ft + [fo, tq, tk, tv, ty]:
        gpu.free(t)
