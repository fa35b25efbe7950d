"""The C-ABI shared library without a GPU: it builds, loads, and exports every function
include/h3b200_attn.h declares - among them the five kernel-adapter symbols the reference's CUDA
backend links against (cuda/h3_flash.h:4-20, cuda/vsa_hopper.h:4-6). No compute call is made."""
import ctypes as C

import pytest

ADAPTERS = ["h3_flash_bf16", "h3_flash3_bf16", "h3_flash3_f16_d64", "h3_flash3_cross_bf16", "h3_vsa_hopper"]


@pytest.fixture(scope="module")
def library(package):
    package.build()
    from h3_omni_b200 import native
    return native, native.load_library()


def test_every_declared_function_is_exported(library):
    native, lib = library
    names = [name for _, name, _ in native.declarations()]
    assert len(names) == len(set(names)), "a function is declared twice"
    assert len(names) >= 60
    for name in names:
        assert hasattr(lib, name), name + " is declared but not exported"
    for name in ADAPTERS:
        assert name in names


def test_reference_signatures_of_the_adapters(library):
    """Argument counts of the reference's declarations (pointers, sizes, scale, flags, stream)."""
    native, _ = library
    arity = {name: len(args) for _, name, args in native.declarations()}
    assert arity["h3_flash_bf16"] == 12       # out q k v lse batch seq heads kv_heads scale causal stream
    assert arity["h3_flash3_bf16"] == 11      # the same without the causal flag
    assert arity["h3_flash3_f16_d64"] == 10   # out q k v lse batch seq heads scale stream
    assert arity["h3_flash3_cross_bf16"] == 10
    assert arity["h3_vsa_hopper"] == 11       # out q k v lse indices counts sizes tiles heads stream
    assert arity["h3_gpu_sdpa_bf16"] == 9 and arity["h3_gpu_cross_attention_bf16"] == 11
    assert arity["h3_gpu_qkv_rope_bf16"] == 14 and arity["h3_gpu_grouped_qkv_rope_bf16"] == 14


def test_no_oracle_in_the_library(library):
    """The product never links or loads the CPU oracle."""
    _, lib = library
    for name in ("oracle_attention", "oracle_vsa_select", "oracle_qkv_rope"):
        with pytest.raises(AttributeError):
            getattr(lib, name)


def test_calls_without_a_context_fail_cleanly(library):
    _, lib = library
    assert lib.h3_gpu_sdpa_bf16(None, None, None, None, None, 1, 1, 128, C.c_float(1.0)) == 0
    assert lib.h3_gpu_vsa_bf16(None, None, None, None, None, None) == 0
    assert lib.h3b_vsa_info(None, None, None, None, None) == 0
    assert lib.h3b_comm_rank(None) == -1 and lib.h3b_comm_size(None) == 0
    assert lib.h3_gpu_tensor_elements(None) == 0
    assert C.string_at(lib.h3_gpu_error(None)) == b"no GPU context"


def test_host_call_plans_its_head_chunks(library):
    """h3b_sdpa_host_plan is host arithmetic: equal groups with the outer two halved, or, asked
    to choose, two one-head chunks at either end and inner chunks of at least two heads and
    about 24 MB per tensor."""
    _, lib = library
    lib.h3b_sdpa_host_plan.restype = C.c_uint32
    counts = (C.c_uint32 * 66)()

    def plan(sequence, heads, groups, capacity=66):
        return list(counts[:lib.h3b_sdpa_host_plan(sequence, heads, groups, counts, capacity)])

    assert plan(52352, 24, 6) == [2, 2, 4, 4, 4, 4, 2, 2]
    assert plan(52352, 24, 0) == [1, 1] + [2] * 10 + [1, 1]
    assert plan(16384, 24, 0) == [1, 1, 5, 5, 5, 5, 1, 1] and plan(16384, 11, 0) == [1, 1, 4, 3, 1, 1]
    assert len(plan(101464, 200, 0)) <= 64
    assert plan(700, 8, 1) == [4, 4] and plan(700, 8, 4) == [1, 1, 2, 2, 1, 1]
    assert plan(700, 8, 3) == [] and plan(700, 0, 0) == [] and plan(52352, 24, 6, capacity=4) == []
    for heads in range(1, 65):
        for sequence in (1, 700, 16384, 101464):
            chunks = plan(sequence, heads, 0)
            assert sum(chunks) == heads and all(chunks), (heads, sequence, chunks)
