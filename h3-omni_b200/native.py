"""ctypes access to libh3b200_attn through its public C header.

Mirrors the way the reference drives its own backend from Python
(reference tests/pytorch/native.py:11-60): signatures are read from the header, a context is
created with h3_gpu_create, primitives are called by name and failures raise with the text of
h3_gpu_error. Host data are numpy arrays; 16-bit floats travel as uint16 bit patterns.
"""
import ctypes as C
import re
from pathlib import Path

import numpy as np

from .build import LIB

HEADER = Path(__file__).resolve().parents[1] / "include" / "h3b200_attn.h"
F32, BF16, I8, U32, F16 = range(5)
_CTYPES = {
    "int": C.c_int, "unsigned": C.c_uint, "float": C.c_float, "size_t": C.c_size_t,
    "uint32_t": C.c_uint32, "uint64_t": C.c_uint64, "bool": C.c_bool, "void": None,
    "h3_gpu_dtype": C.c_int, "cudaError_t": C.c_int, "cudaStream_t": C.c_void_p,
}


def declarations():
    """[(return type, name, [argument types])] for every function the header declares."""
    source = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    source = re.sub(r"^\s*#.*$", "", source, flags=re.M)
    source = re.sub(r"typedef\s+enum\s*\{.*?\}\s*\w+;", "", source, flags=re.S)
    out = []
    for result, name, args in re.findall(r"([\w ]+?\s*\*?)\s*\b(h3b?_\w+)\s*\(([^;{}]*)\)\s*;", source):
        parts = [a.strip() for a in args.split(",") if a.strip() and a.strip() != "void"]
        out.append((result.strip(), name, parts))
    return out


def _ctype(text, is_argument):
    text = text.replace("const", "").strip()
    if "*" in text:
        return C.c_void_p
    base = text.rsplit(" ", 1)[0].strip() if is_argument and " " in text else text
    return _CTYPES[base]


def _preload_bundled_nccl():
    """One NCCL per process: when a Python-packaged NCCL is installed (the one torch is built
    against), load it first so that this library binds to it whether torch is imported before or
    after; with the system NCCL loaded first, a later `import torch` fails to resolve symbols."""
    import importlib.util
    spec = importlib.util.find_spec("nvidia.nccl")
    for root in (spec.submodule_search_locations if spec else []):
        path = Path(root) / "lib" / "libnccl.so.2"
        if path.exists():
            C.CDLL(str(path), mode=C.RTLD_GLOBAL)
            return


def load_library():
    """Load the shared library and type every declared function. Raises if it is missing."""
    if not LIB.exists():
        raise RuntimeError("libh3b200_attn.so is not built; run `python h3-omni_b200/build.py`")
    _preload_bundled_nccl()
    lib = C.CDLL(str(LIB))
    for result, name, args in declarations():
        fn = getattr(lib, name)
        fn.restype = _ctype(result, False)
        fn.argtypes = [_ctype(a, True) for a in args]
    return lib


class Native:
    """One h3_gpu context on the current CUDA device."""

    def __init__(self):
        self.lib = load_library()
        error = C.create_string_buffer(512)
        self.gpu = self.lib.h3_gpu_create(None, error, len(error))
        if not self.gpu:
            raise RuntimeError(error.value.decode())
        self.owned = []

    def close(self):
        for t in self.owned:
            self.lib.h3_gpu_tensor_free(t)
        self.owned = []
        if self.gpu:
            self.lib.h3_gpu_free(self.gpu)
            self.gpu = None

    def error(self):
        return C.string_at(self.lib.h3_gpu_error(self.gpu)).decode()

    def call(self, name, *args):
        """h3_gpu_<name>(gpu, *args); raises RuntimeError with h3_gpu_error on failure."""
        result = getattr(self.lib, "h3_gpu_" + name)(self.gpu, *args)
        if not result:
            raise RuntimeError(name + ": " + self.error())
        return result

    def raw(self, name, *args):
        """A kernel-adapter symbol (returns cudaError_t); raises on a non-zero code."""
        code = getattr(self.lib, name)(*args)
        if code:
            raise RuntimeError("%s returned cudaError %d" % (name, code))

    def tensor(self, x, dtype=None):
        """Upload a numpy array. uint16 arrays are bf16 unless dtype=F16."""
        x = np.ascontiguousarray(x)
        ptr = x.ctypes.data_as(C.c_void_p)
        if x.dtype == np.float32:
            t = self.call("tensor_from_f32", ptr, x.size)
        elif x.dtype in (np.int32, np.uint32):
            t = self.call("tensor_from_u32", ptr, x.size)
        elif x.dtype == np.uint16 and dtype == F16:
            t = self.lib.h3b_tensor_new_f16(self.gpu, x.size)
            if not t:
                raise RuntimeError("tensor_new_f16: " + self.error())
            self._upload_raw(t, x)
        elif x.dtype == np.uint16:
            t = self.call("tensor_from_bf16", ptr, x.size)
        else:
            raise TypeError(x.dtype)
        self.owned.append(t)
        return t

    def _upload_raw(self, t, x):
        self.submit()
        code = _cudart().cudaMemcpy(C.c_void_p(self.lib.h3b_tensor_data(t)), x.ctypes.data_as(C.c_void_p),
                             C.c_size_t(x.nbytes), 1)
        if code:
            raise RuntimeError("cudaMemcpy failed: %d" % code)

    def empty_bf16(self, elements):
        t = self.call("tensor_new_bf16", elements)
        self.owned.append(t)
        return t

    def empty_f16(self, elements):
        t = self.lib.h3b_tensor_new_f16(self.gpu, elements)
        if not t:
            raise RuntimeError("tensor_new_f16: " + self.error())
        self.owned.append(t)
        return t

    def wrap(self, device_pointer, elements, dtype=BF16):
        """Non-owning tensor over caller-owned device memory (e.g. torch data_ptr())."""
        t = self.lib.h3b_tensor_wrap(self.gpu, C.c_void_p(device_pointer), elements, dtype)
        if not t:
            raise RuntimeError("tensor_wrap failed")
        self.owned.append(t)
        return t

    def free(self, t):
        self.owned.remove(t)
        self.lib.h3_gpu_tensor_free(t)

    def submit(self):
        self.call("submit")

    def read(self, t, shape, dtype=np.uint16):
        """Synchronise and download a tensor as numpy (uint16 for bf16/fp16, float32, int32)."""
        self.submit()
        x = np.empty(shape, dtype=dtype)
        if not self.lib.h3_gpu_download(self.gpu, t, 0, x.ctypes.data_as(C.c_void_p), x.nbytes):
            raise RuntimeError("download: " + self.error())
        return x

    def read_device(self, pointer, shape, dtype):
        """Download from a raw device pointer (VSA work buffers)."""
        self.submit()
        x = np.empty(shape, dtype=dtype)
        code = _cudart().cudaMemcpy(x.ctypes.data_as(C.c_void_p), C.c_void_p(pointer),
                                    C.c_size_t(x.nbytes), 2)
        if code:
            raise RuntimeError("cudaMemcpy failed: %d" % code)
        return x

    def device_status(self, reset=True):
        status = C.c_int(0)
        code = self.lib.h3b_device_status(C.byref(status), int(reset))
        if code:
            raise RuntimeError("h3b_device_status: cudaError %d" % code)
        return status.value


_CUDART = None


def _cudart():
    """The CUDA runtime the library itself linked against (already loaded with it)."""
    global _CUDART
    if _CUDART is None:
        for name in ("libcudart.so.12", "libcudart.so"):
            try:
                _CUDART = C.CDLL(name)
                break
            except OSError:
                continue
        if _CUDART is None:
            raise RuntimeError("libcudart not found")
        _CUDART.cudaMemcpy.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]
        _CUDART.cudaMemcpy.restype = C.c_int
    return _CUDART
