"""ctypes driver of the reference's own CUDA backend (oracle/_ref/libh3_ref_cuda.so, built by
oracle/ref_build.py from the reference tree and linked against this library). Test infrastructure."""
import ctypes as C
from pathlib import Path

import numpy as np

REF_LIB = Path(__file__).resolve().parents[1] / "oracle" / "_ref" / "libh3_ref_cuda.so"
# the same backend with its attention stages replaced by this library's (h3-omni_b200/glue_build.py)
GLUE_LIB = Path(__file__).resolve().parents[1] / "h3-omni_b200" / "libh3_cuda_b200.so"


class Reference:
    """Minimal ctypes driver of the reference backend (its public h3_gpu.h / h3_cuda.h calls)."""

    def __init__(self, library=REF_LIB):
        self.lib = C.CDLL(str(library))
        L = self.lib
        for name in ("h3_gpu_create", "h3_gpu_tensor_from_bf16", "h3_gpu_tensor_from_f32",
                     "h3_gpu_tensor_new_bf16", "h3_gpu_tensor_new_f32", "h3_gpu_vsa_new", "h3_gpu_error"):
            getattr(L, name).restype = C.c_void_p
        L.h3_gpu_create.argtypes = [C.c_char_p, C.c_char_p, C.c_size_t]
        for name in ("h3_gpu_tensor_from_bf16", "h3_gpu_tensor_from_f32"):
            getattr(L, name).argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        for name in ("h3_gpu_tensor_new_bf16", "h3_gpu_tensor_new_f32"):
            getattr(L, name).argtypes = [C.c_void_p, C.c_size_t]
        for name in ("h3_gpu_tensor_read_bf16", "h3_gpu_tensor_read_f32"):
            getattr(L, name).argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        L.h3_gpu_submit.argtypes = [C.c_void_p]
        L.h3_gpu_free.argtypes = [C.c_void_p]
        L.h3_gpu_tensor_free.argtypes = [C.c_void_p]
        L.h3_gpu_error.argtypes = [C.c_void_p]
        sd = [C.c_void_p] * 5 + [C.c_uint32, C.c_uint32, C.c_uint32, C.c_float]
        L.h3_gpu_sdpa_bf16.argtypes = sd
        L.h3_gpu_sdpa_f32.argtypes = sd
        L.h3_gpu_sdpa_fa2_bf16.argtypes = sd
        L.h3_gpu_cross_attention_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p,
                                                  C.c_size_t, C.c_void_p, C.c_void_p, C.c_size_t,
                                                  C.c_uint32, C.c_uint32, C.c_uint32]
        L.h3_gpu_vsa_new.argtypes = [C.c_void_p] + [C.c_uint32] * 6
        L.h3_gpu_vsa_free.argtypes = [C.c_void_p]
        L.h3_gpu_vsa_bf16.argtypes = [C.c_void_p] * 6
        error = C.create_string_buffer(512)
        self.gpu = L.h3_gpu_create(None, error, 512)
        if not self.gpu:
            raise RuntimeError(error.value.decode())
        self.owned = []

    def check(self, ok, what):
        if not ok:
            raise RuntimeError(what + ": " + C.string_at(self.lib.h3_gpu_error(self.gpu)).decode())

    def tensor(self, x):
        x = np.ascontiguousarray(x)
        fn = self.lib.h3_gpu_tensor_from_f32 if x.dtype == np.float32 else self.lib.h3_gpu_tensor_from_bf16
        t = fn(self.gpu, x.ctypes.data_as(C.c_void_p), x.size)
        self.check(t, "tensor")
        self.owned.append(t)
        return t

    def empty(self, elements, f32=False):
        t = (self.lib.h3_gpu_tensor_new_f32 if f32 else self.lib.h3_gpu_tensor_new_bf16)(self.gpu, elements)
        self.check(t, "tensor")
        self.owned.append(t)
        return t

    def read(self, t, shape, f32=False):
        self.check(self.lib.h3_gpu_submit(self.gpu), "submit")
        x = np.empty(shape, dtype=np.float32 if f32 else np.uint16)
        fn = self.lib.h3_gpu_tensor_read_f32 if f32 else self.lib.h3_gpu_tensor_read_bf16
        self.check(fn(t, x.ctypes.data_as(C.c_void_p), x.size), "read")
        return x

    def close(self):
        for t in self.owned:
            self.lib.h3_gpu_tensor_free(t)
        self.lib.h3_gpu_free(self.gpu)


def ref_vsa_buffers(ref, handle, heads, tiles):
    """Work buffers of the reference's private h3_gpu_vsa object (reference cuda/vsa.cuh:7-13:
    a context pointer, five ints, then tensor pointers map, sizes, q, k, v, out, lse, poolq,
    poolk, poolv, scores, compression, indices, counts; each tensor starts with its device
    pointer, cuda/h3_gpu_cuda.cu:41-47)."""
    names = ["map", "sizes", "q", "k", "v", "out", "lse", "poolq", "poolk", "poolv", "scores",
             "compression", "indices", "counts"]
    base = handle + 8 + 24
    pointers = (C.c_void_p * len(names)).from_address(base)
    device = {n: C.c_void_p.from_address(pointers[i]).value for i, n in enumerate(names)}
    ref.check(ref.lib.h3_gpu_submit(ref.gpu), "submit")
    return device


