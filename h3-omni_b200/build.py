"""Builds libh3b200_attn.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libh3b200_attn.so"
SOURCES = ["attn_tc5.cu", "attn_sparse_t.cu", "attn_tc5_pair.cu", "attn_mma.cu", "vsa_coarse.cu", "qkv_rope.cu", "ulysses.cu", "h3_gpu_b200.cu", "vsa_object.cu", "multi_gpu.cu", "live_kv.cu", "out_proj_gate.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def nvcc():
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(path).exists():
        raise RuntimeError("nvcc not found; the library cannot be built")
    return path


def stale():
    if not LIB.exists():
        return True
    built = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    deps.append(HERE.parent / "include" / "h3b200_attn.h")
    return any(p.stat().st_mtime > built for p in deps)


def build(force=False, verbose=False):
    """Compile every CUDA source and link the shared library. Returns its path."""
    if not force and not stale():
        return LIB
    objdir = HERE / "build"
    objdir.mkdir(exist_ok=True)
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(name):
        obj = objdir / (Path(name).stem + ".o")
        cmd = [nvcc(), *NVCC_FLAGS, *extra, "-c", str(CSRC / name), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s" % (name, r.stderr))
        if verbose:
            sys.stderr.write(r.stderr)
        return str(obj)

    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 1)) as pool:
        objects = list(pool.map(compile_one, SOURCES))
    # -Bsymbolic: calls between this library's own exported functions never bind to another
    # library that exports the same reference ABI names in the same process.
    link = [nvcc(), "-shared", "-o", str(LIB), *objects, "-lnccl", "-lcudart", "-Xlinker", "-Bsymbolic"]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + r.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
