"""Build libfastbb_b200.so in-tree with nvcc for sm_100a: `python -m fastbb_b200.build`.

The counterpart of the reference's `build_prebuilt` (fastbb/kernels.py:51-63), which ships one fatbin for seven
architectures; this library targets B200 only and is a regular shared object loaded with ctypes.CDLL.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc", "fastbb_b200.cu")
OUT = os.path.join(HERE, "libfastbb_b200.so")
FLASH_SRC = os.path.join(HERE, "csrc", "fastbb_flash64.cu")   # attention kernel + its entry points only
FLASH_OUT = os.path.join(HERE, "libfastbb_flash64.so")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC"]


def sources():
    d = os.path.join(HERE, "csrc")
    return [os.path.join(d, f) for f in sorted(os.listdir(d))] + [os.path.join(HERE, "..", "include", "fastbb_b200.h")]


def up_to_date(out=OUT):
    return os.path.exists(out) and all(os.path.getmtime(out) >= os.path.getmtime(s) for s in sources())


def build(force=False, verbose=False, flash_only=False):
    """Compile csrc/fastbb_b200.cu (which includes the other .cu files) into libfastbb_b200.so, or, with flash_only,
    csrc/fastbb_flash64.cu into libfastbb_flash64.so (what `attention.py` + `_lib.py` need on their own). Returns the path."""
    src, out = (FLASH_SRC, FLASH_OUT) if flash_only else (SRC, OUT)
    if not force and up_to_date(out):
        return out
    nvcc = shutil.which("nvcc") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    cmd = [nvcc, *FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", out + ".tmp", src]
    subprocess.run(cmd, check=True)
    os.replace(out + ".tmp", out)
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, flash_only="--flash-only" in sys.argv))
