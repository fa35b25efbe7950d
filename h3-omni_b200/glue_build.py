"""Builds libh3_cuda_b200.so: the reference's CUDA backend with its attention stages replaced.

The reference's cuda/h3_gpu_cuda.cu is compiled for sm_100a from where it lies in the reference
tree, through csrc/h3_b200_glue.cu (which includes it and redefines h3_gpu_vsa_bf16 and the two
Ulysses exchanges on this library's stages), and linked against libh3b200_attn.so, which supplies
the five kernel-adapter symbols and the stage entry points. Nothing of the reference is copied
or edited; its own build system is not run. The reference tree is found through H3_REF_ROOT
(or the first argument); without it the build is skipped and a previously built library is kept.

    H3_REF_ROOT=/path/to/H3-omni python h3-omni_b200/glue_build.py
"""
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
GLUE = HERE / "csrc" / "h3_b200_glue.cu"
PRODUCT = HERE / "libh3b200_attn.so"
OUT = HERE / "libh3_cuda_b200.so"


def reference_root(argument=None):
    root = argument or os.environ.get("H3_REF_ROOT")
    return Path(root) if root else None


def build_if_possible(root=None, force=False):
    """Returns the library path, or None when it cannot be built here and was not built before."""
    root = reference_root(root)
    source = root / "cuda" / "h3_gpu_cuda.cu" if root else None
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not source or not source.exists() or not Path(nvcc).exists() or not PRODUCT.exists():
        return OUT if OUT.exists() else None
    newest = max(p.stat().st_mtime for p in (source, GLUE, PRODUCT))
    if OUT.exists() and not force and OUT.stat().st_mtime >= newest:
        return OUT
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "--fmad=false", "-w", "-DH3_VSA",
           '-DH3_REF_BACKEND="%s"' % source, "-Xcompiler", "-fPIC", "-shared", "-o", str(OUT), str(GLUE),
           "-I", str(root), "-I", str(root / "cuda"), "-L", str(HERE), "-lh3b200_attn", "-lcublas", "-lcublasLt",
           "-lcudnn", "-lnccl", "-Xlinker", "-Bsymbolic", "-Xlinker", "-rpath=$ORIGIN"]
    result = subprocess.run(cmd, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError("glue build failed:\n" + result.stderr[-4000:])
    return OUT


if __name__ == "__main__":
    print(build_if_possible(sys.argv[1] if len(sys.argv) > 1 else None, force=True))
