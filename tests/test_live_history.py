"""Live mode's KV history as a ring buffer (h3b_live_kv_*) against the reference's allocate-copy-
rotate bookkeeping (h3_dit.c:4451-4489, h3_dit_live.inc:56-109), restated here on the host: over
twelve chunks the ring must present exactly the rows the reference would concatenate."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
SCALE = float(1.0 / np.sqrt(128.0))


class CopyRotate:
    """The reference's state per layer: pending, recent[0], recent[1], sink; each (K, V, audio, skip)."""

    def __init__(self):
        self.pending, self.recent, self.sink, self.commits = None, [None, None], None, 0

    def stage(self, k, v, text, audio):
        self.pending = dict(k=k[text:].copy(), v=v[text:].copy(), audio=audio, skip=0)

    def commit(self):
        if not self.commits:
            p = self.pending
            self.sink = dict(k=p["k"][p["audio"]:].copy(), v=p["v"][p["audio"]:].copy())
        self.recent = [self.recent[1], self.pending]
        self.pending = None
        self.commits += 1

    def clear_audio(self):
        for r in self.recent:
            if r:
                r["skip"] = r["audio"]

    def ranges(self, k, v, text):
        """[(K rows, V rows)] in the order live_attention concatenates them."""
        out = [(k[:text], v[:text])]
        history = []
        if self.commits > 2:
            history.append((self.sink["k"], self.sink["v"]))
        if self.commits > 1:
            history.append((self.recent[0]["k"][self.recent[0]["skip"]:], self.recent[0]["v"][self.recent[0]["skip"]:]))
        if self.commits:
            history.append((self.recent[1]["k"][self.recent[1]["skip"]:], self.recent[1]["v"][self.recent[1]["skip"]:]))
        return out + history + [(k[text:], v[text:])]


def test_ring_history_equals_copy_rotate_over_twelve_chunks(gpu, oracle):
    heads, text, chunk_rows = 3, 20, 260
    ring = gpu.lib.h3b_live_kv_new(gpu.gpu, chunk_rows, heads)
    assert ring
    ref = CopyRotate()
    rng = np.random.default_rng(12)
    try:
        for chunk in range(12):
            audio, video = int(rng.integers(0, 40)), int(rng.integers(100, 220))
            sequence = text + audio + video
            q, k, v = (oracle.normal_bf16((sequence, heads, 128), 1000 + 3 * chunk + i) for i in range(3))
            tq, tk, tv = gpu.tensor(q), gpu.tensor(k), gpu.tensor(v)
            # media rows of this block against text | history | current media
            out = gpu.tensor(np.zeros(q.shape, dtype=np.uint16))
            media = sequence - text
            assert gpu.lib.h3b_live_kv_attention_bf16(ring, out, text, tq, text, media, tk, tv, text, sequence), gpu.error()
            got = gpu.read(out, q.shape)[text:]
            ranges = [r for r in ref.ranges(k, v, text) if len(r[0])]
            assert gpu.lib.h3b_live_kv_history_rows(ring) == sum(len(r[0]) for r in ranges) - sequence
            # (a) the segmented kernel on the reference's tensors, range by range: bit-identical
            keys = [gpu.tensor(r[0]) for r in ranges]
            values = [gpu.tensor(r[1]) for r in ranges]
            n = len(ranges)
            out2 = gpu.tensor(np.zeros(q.shape, dtype=np.uint16))
            assert gpu.lib.h3b_cross_attention_segments_bf16(
                gpu.gpu, out2, text, tq, text, media, heads, n, (C.c_void_p * n)(*keys), (C.c_void_p * n)(*values),
                (C.c_size_t * n)(*([0] * n)), (C.c_uint32 * n)(*[len(r[0]) for r in ranges])), gpu.error()
            assert np.array_equal(gpu.read(out2, q.shape)[text:], got), chunk
            # (b) the reference's way: concatenate, then one rectangular call; (c) the FP32 oracle
            kc, vc = np.concatenate([r[0] for r in ranges]), np.concatenate([r[1] for r in ranges])
            out3 = gpu.tensor(np.zeros(q.shape, dtype=np.uint16))
            gpu.call("cross_attention_bf16", out3, text, tq, text, gpu.tensor(kc), gpu.tensor(vc), 0, media, len(kc), heads)
            want, _ = oracle.attention(q[None, text:], kc[None], vc[None], SCALE)
            got32 = oracle.from_bf16(got)
            assert np.abs(got32 - want[0]).max() <= 1e-2
            assert np.abs(got32 - oracle.from_bf16(gpu.read(out3, q.shape)[text:])).max() <= 1e-2
            # stage and commit this chunk on both sides
            assert gpu.lib.h3b_live_kv_stage(ring, tk, tv, text, media, audio), gpu.error()
            ref.stage(k, v, text, audio)
            assert gpu.lib.h3b_live_kv_commit(ring), gpu.error()
            ref.commit()
            assert gpu.lib.h3b_live_kv_commits(ring) == ref.commits
            if chunk in (4, 9):
                assert gpu.lib.h3b_live_kv_clear_audio(ring)
                ref.clear_audio()
            for t in keys + values + [tq, tk, tv, out, out2, out3]:
                gpu.free(t)
        assert gpu.device_status() == 0
        # a commit without a staged chunk, a chunk that does not fit, a reset
        assert not gpu.lib.h3b_live_kv_commit(ring)
        assert "incomplete live clean commit" in gpu.error()
        big = gpu.empty_bf16((chunk_rows + 1) * heads * 128)
        assert not gpu.lib.h3b_live_kv_stage(ring, big, big, 0, chunk_rows + 1, 0)
        gpu.lib.h3b_live_kv_reset(ring)
        assert gpu.lib.h3b_live_kv_commits(ring) == 0 and gpu.lib.h3b_live_kv_history_rows(ring) == 0
    finally:
        gpu.lib.h3b_live_kv_free(ring)
