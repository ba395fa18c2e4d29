"""Install the reference package (fastforks/fastbb) into oracle/_ref/, which is git-ignored: build output, never history.

    python oracle/make_ref.py [/path/to/reference]          (default: $FASTBB_REFERENCE, then the build container's checkout)

TEST / BENCH INFRASTRUCTURE ONLY. What lands in oracle/_ref/ is the reference's own, unmodified `fastbb` package; only
bench.py's reference legs (`--impl reference`, `cpu_baseline`) and tests may import it: to time and check the reference's
friendly fp32 tier (FastViT(attn="sdpa", gacc=False, dtype=float32), fastbb/vit.py:42,108-150) on the host cores and,
in the `--impl reference` arm on a machine with a GPU, to time its own GPU tiers beside that for context.
Nothing under fastbb_b200/ imports it. The reference checkout itself does not travel to the GPU machine; this folder,
like the built .so files, does.

The install is a plain `pip install --no-deps --no-build-isolation --target oracle/_ref` of a temporary copy of the
checkout (the checkout is read-only and setuptools writes into the source tree). If pip is unavailable the package
directory is copied instead; either way the result is the same Python files.
"""
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
DEFAULT_SRC = os.environ.get("FASTBB_REFERENCE", os.path.join(os.sep, "root", "reference"))


def available():
    return os.path.exists(os.path.join(DEST, "fastbb", "vit.py"))


def make(src=DEFAULT_SRC, force=False):
    """Returns DEST if the reference is (now) installed there, None if there is no checkout to install from."""
    if available() and not force:
        make_kernels()
        return DEST
    if not os.path.exists(os.path.join(src, "fastbb", "vit.py")):
        return None
    if os.path.isdir(DEST):
        shutil.rmtree(DEST)
    os.makedirs(DEST)
    with tempfile.TemporaryDirectory() as tmp:
        copy = os.path.join(tmp, "reference")
        shutil.copytree(src, copy, ignore=shutil.ignore_patterns(".git", "*.fatbin", "__pycache__"))
        cmd = [sys.executable, "-m", "pip", "install", "--quiet", "--no-index", "--no-deps", "--no-build-isolation", "--target", DEST, copy]
        ok = subprocess.run(cmd, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL).returncode == 0 and available()
        if not ok:
            shutil.copytree(os.path.join(copy, "fastbb"), os.path.join(DEST, "fastbb"), dirs_exist_ok=True)
    if available():
        make_kernels()
    return DEST if available() else None


def make_kernels(arch="sm_100"):
    """Compile the reference's own kernel file for the GPU machine's architecture with the reference's own recipe
    (fastbb/kernels.py:84-94: `nvcc -cubin -O3 -std=c++17 --expt-relaxed-constexpr -arch=sm_XY`) into
    oracle/_ref/fastbb/prebuilt/, under the file name its loader looks for (source hash + architecture), so that its GPU
    tiers (`fh-g0`, `hh-g1`: mma.sync kernels, recompiled) can be timed on the same GPU as this library
    (`bench.py --impl reference`: gpu_tiers_ms_per_image) without a compile on that machine. Returns the path, or None without nvcc."""
    import hashlib
    src = os.path.join(DEST, "fastbb", "fastbb_kernels.cu")
    nvcc = shutil.which("nvcc") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if not (os.path.exists(src) and os.path.exists(nvcc)):
        return None
    tag = hashlib.sha1(open(src, "rb").read() + arch.encode()).hexdigest()[:16]
    out = os.path.join(DEST, "fastbb", "prebuilt", f"fastbb_kernels_{tag}.cubin")
    if not os.path.exists(out):
        os.makedirs(os.path.dirname(out), exist_ok=True)
        cuda_home = os.path.dirname(os.path.dirname(nvcc))
        cmd = [nvcc, "-cubin", "-O3", "-std=c++17", "--expt-relaxed-constexpr", f"-arch={arch}", f"-I{cuda_home}/include", "-o", out + ".tmp", src]
        if subprocess.run(cmd, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL).returncode != 0:
            return None
        os.replace(out + ".tmp", out)
    return out


if __name__ == "__main__":
    out = make(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_SRC, force=True)
    print(out or "no reference checkout found: oracle/_ref not made")
