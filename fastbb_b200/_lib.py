"""ctypes loader for libfastbb_b200.so, the C-ABI shared library holding the sm_100a kernels.

Plays the role of the reference's driver-API loader (fastbb/kernels.py:71-133 `Kernels`): the host code stays
Python/PyTorch and crosses one thin FFI boundary per operator. Differences: the boundary is a C ABI with one
entry point per operator instead of a kernel-name + signature-string table; a non-zero status becomes a Python
exception; nothing is cached per device in Python, so several GPUs can be used from one process.
There is no CPU or PyTorch fallback: if the library is missing, importing an operator raises.

Attention on its own: `attention.py` + this file + `libfastbb_flash64.so` (`python -m fastbb_b200.build --flash-only`) are
all a project needs that vendors only the attention API, as several forks do with the reference's
attention.py + kernels.py. When the full library is absent, load() falls back to that one and sets up only the
entry points it exports.
"""
import contextlib
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfastbb_b200.so")
FLASH_LIB_PATH = os.path.join(_HERE, "libfastbb_flash64.so")   # attention kernel and its entry points only

FBB_OK = 0
DTYPE_CODE = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}
EPI_NONE, EPI_GELU, EPI_SWIGLU = 0, 1, 2
ACC_F32, ACC_F16 = 0, 1
FLASH_VARIANT = {"ff": 0, "fh": 1, "hh": 2}

_vp, _i32, _i64, _f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float


def on(device):
    """Context manager that makes `device` current for the enclosed C calls (a no-op when it already is)."""
    return torch.cuda.device(device) if device.index != torch.cuda.current_device() else contextlib.nullcontext()


class BlockDesc(ctypes.Structure):
    """fbb_block_desc of include/fastbb_b200.h: weight pointers and shapes of one transformer block."""
    _fields_ = ([(n, _vp) for n in ("ln1_w", "ln1_b", "qkv_w", "qkv_b", "proj_w", "proj_b", "gamma1", "ln2_w", "ln2_b",
                                    "fc1_w", "fc1_b", "fc2_w", "fc2_b", "gamma2")]
                + [(n, _i32) for n in ("C", "heads", "hidden", "mlp", "acc_main", "acc_fc2", "flash_variant")]
                + [(n, _f32) for n in ("eps1", "eps2", "scale")])


MLP_GELU, MLP_SWIGLU = 0, 1
_bdp = ctypes.POINTER(BlockDesc)

# name -> (restype, argtypes); mirrors include/fastbb_b200.h one to one.
PROTOTYPES = {
    "fbb_version": (_i32, []),
    "fbb_status_string": (ctypes.c_char_p, [_i32]),
    "fbb_last_error": (ctypes.c_char_p, []),
    "fbb_device_status": (_i32, [ctypes.POINTER(ctypes.c_uint * 4)]),
    "fbb_diag_wait_timeout": (_i32, [ctypes.c_uint64, ctypes.c_uint, _vp]),
    "fbb_diag_sm_clock_mhz": (_i32, [_vp, _i64, _vp]),
    "fbb_linear_max_cta_pairs": (_i32, [_i32]),
    "fbb_layernorm_f16": (_i32, [_vp, _vp, _vp, _vp, _i64, _i32, _i64, _i64, _f32, _i32, _i32, _vp]),
    "fbb_layernorm_split_f16": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _f32, _i32, _i32, _vp]),
    "fbb_linear_f16": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i64, _i64, _i64, _i64, _i32, _i32, _vp]),
    "fbb_linear_layernorm_f16": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i64, _i64, _i64, _i64, _i32, _i32, _vp, _vp, _f32, _vp, _i64,
                                        _vp, _vp]),
    "fbb_linear_layernorm_launches": (_i32, [_i64, _i32, _i32, _i32]),
    "fbb_flash64_f16": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i32] + [_i64] * 12 + [_f32, _i32, _vp]),
    "fbb_flash64_workspace_bytes": (_i64, [_i32, _i32, _i32]),
    "fbb_flash64_launches": (_i32, [_i32, _i32, _i32, _i32]),
    "fbb_flash64_f16_ws": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i32] + [_i64] * 12 + [_f32, _i32, _vp, _i64, _vp]),
    "fbb_flash64_f16_static": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i32] + [_i64] * 12 + [_f32, _i32, _vp]),
    "fbb_stack_scratch_bytes": (_i64, [_bdp, _i32, _i64]),
    "fbb_stack_launches": (_i32, [_bdp, _i32, _i64]),
    "fbb_stack_forward_f16": (_i32, [_bdp, _i32, _vp, _i32, _i32, _vp, _i64, _vp, _i64, _vp]),
    "fbb_block_forward_f16": (_i32, [_bdp, _vp, _i32, _i32, _vp, _i64, _vp, _i64, _vp]),
}


class FastbbError(RuntimeError):
    """A non-zero status from libfastbb_b200.so (negative: rejected arguments; positive: a CUDA error code)."""

    def __init__(self, status, message):
        super().__init__(f"fastbb_b200 status {status}: {message}")
        self.status = status


_LIB = None
LAUNCHES = 0  # kernels enqueued through this module since import (each operator call is exactly one launch)


def launched(n=1):
    global LAUNCHES
    LAUNCHES += n


# what libfastbb_flash64.so exports (the other prototypes are skipped when that library is the one loaded)
FLASH_ONLY_SYMBOLS = ("fbb_version", "fbb_status_string", "fbb_last_error", "fbb_device_status", "fbb_diag_wait_timeout",
                      "fbb_diag_sm_clock_mhz", "fbb_flash64_f16",
                      "fbb_flash64_workspace_bytes", "fbb_flash64_launches", "fbb_flash64_f16_ws", "fbb_flash64_f16_static")


def load(path=None):
    """Load (once) and return the ctypes handle with every prototype set. Without `path`: the full library, or, if only
    the attention-only library has been built, that one. Raises OSError if neither exists."""
    global _LIB
    if _LIB is None or path is not None:
        p = path or (LIB_PATH if os.path.exists(LIB_PATH) or not os.path.exists(FLASH_LIB_PATH) else FLASH_LIB_PATH)
        if not os.path.exists(p):
            raise OSError(f"{p} not found: build it with `python -m fastbb_b200.build` (needs nvcc with sm_100a support); "
                          "there is no fallback path")
        lib = ctypes.CDLL(p)
        lib.flash_only = not hasattr(lib, "fbb_linear_f16")
        for name, (res, args) in PROTOTYPES.items():
            if lib.flash_only and name not in FLASH_ONLY_SYMBOLS:
                continue
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        if path is not None:
            return lib
        _LIB = lib
    return _LIB


def check(status):
    if status != FBB_OK:
        lib = load()
        msg = lib.fbb_last_error().decode() or lib.fbb_status_string(status).decode()
        raise FastbbError(status, msg)


def stream_ptr(device=None):
    """cudaStream_t of torch's current stream on `device` as an integer (0 = legacy default stream)."""
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t):
    return t.data_ptr() if t is not None else None


def device_status():
    """Synchronise the current device and raise FastbbError if any kernel gave up a bounded wait."""
    out = (ctypes.c_uint * 4)()
    check(load().fbb_device_status(ctypes.byref(out)))
    return tuple(out)
