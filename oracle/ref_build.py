"""Builds the reference's own CUDA backend as a checker library, oracle/_ref/libh3_ref_cuda.so.

Test infrastructure. The reference's `cuda/h3_gpu_cuda.cu` (one translation unit that textually
includes its primitive, VSA and Ulysses sources) is compiled for sm_100a from where it lies in
the reference tree - nothing is copied - and linked against libh3b200_attn.so, which supplies the
five kernel-adapter symbols the reference normally gets from FlashAttention / ThunderKittens
objects. The result serves two purposes on the GPU box:
  * the reference's unmodified wrappers and VSA orchestration run on this repository's kernels
    (the drop-in claim, exercised end to end), and
  * the reference code that still runs on a B200 by itself - FP32 fallback attention, tile
    pooling, cuBLAS pooled scores, block selection, pooled softmax, compression, merge, the
    Ulysses exchange - becomes a live oracle for the CPU restatement and for our kernels.
The reference's own build system (Makefile, prepare_*.py, network fetches) is not run.
"""
import os
import shutil
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
OUT = HERE / "_ref" / "libh3_ref_cuda.so"
PRODUCT = ROOT / "h3-omni_b200" / "libh3b200_attn.so"


def reference_root(argument=None):
    """The reference tree: the argument, else H3_REF_ROOT; None when neither is given."""
    root = argument or os.environ.get("H3_REF_ROOT")
    return Path(root) if root else None


def build_if_possible(root=None, force=False):
    """Returns the library path, or None when the reference tree or nvcc is not available
    (on the GPU box the prebuilt file travels with the repository instead)."""
    ref = reference_root(root)
    source = ref / "cuda" / "h3_gpu_cuda.cu" if ref else Path("/nonexistent")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not source.exists() or not Path(nvcc).exists() or not PRODUCT.exists():
        return OUT if OUT.exists() else None
    if OUT.exists() and not force and OUT.stat().st_mtime >= max(source.stat().st_mtime,
                                                                  PRODUCT.stat().st_mtime):
        return OUT
    OUT.parent.mkdir(exist_ok=True)
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "--fmad=false", "-w", "-DH3_VSA",
           "-Xcompiler", "-fPIC", "-shared", "-o", str(OUT), str(source), "-I", str(ref),
           "-I", str(ref / "cuda"), "-L", str(PRODUCT.parent), "-lh3b200_attn", "-lcublas",
           "-lcublasLt", "-lcudnn", "-lnccl", "-Xlinker", "-Bsymbolic", "-Xlinker",
           "-rpath=$ORIGIN/../../h3-omni_b200"]
    result = subprocess.run(cmd, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError("reference backend did not build:\n" + result.stderr[-4000:])
    return OUT


if __name__ == "__main__":
    import sys
    print(build_if_possible(sys.argv[1] if len(sys.argv) > 1 else None, force=True))
