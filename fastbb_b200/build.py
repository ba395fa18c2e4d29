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
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC"]


def sources():
    d = os.path.join(HERE, "csrc")
    return [os.path.join(d, f) for f in sorted(os.listdir(d))] + [os.path.join(HERE, "..", "include", "fastbb_b200.h")]


def up_to_date():
    return os.path.exists(OUT) and all(os.path.getmtime(OUT) >= os.path.getmtime(s) for s in sources())


def build(force=False, verbose=False):
    """Compile csrc/fastbb_b200.cu (which includes the other .cu files) into libfastbb_b200.so. Returns the path."""
    if not force and up_to_date():
        return OUT
    nvcc = shutil.which("nvcc") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    cmd = [nvcc, *FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", OUT + ".tmp", SRC]
    subprocess.run(cmd, check=True)
    os.replace(OUT + ".tmp", OUT)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
