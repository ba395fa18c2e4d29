"""Flash attention for head_dim 64 on the tcgen05 tensor cores (kernel: csrc/flash64.cu).

Same call signature as the reference's fastbb/attention.py:31 `attention`:

attention(q, k, v, scale=None, out=None, variant="hh")
    q, k, v: [B, N, H, 64] fp16 views (d contiguous, other strides multiples of 8 elements; e.g. the unbound packed qkv
    GEMM output [B, N, 3, H, 64]); returns O as [B, N, H, 64] (contiguous -> .view(B, N, H*64), no transpose).
variant: the reference's "hh" / "fh" / "ff" (accumulate types of QK^T and PV in its kernels) are all accepted; on B200
both products accumulate in fp32 for every variant (an f16 tensor-memory accumulator is no faster and costs a conversion).
Small inputs run the same kernel with one 128-query tile per CTA instead of the reference's SDPA fallback
(fastbb/vit.py:146-150); anything the kernel does not cover (other head dims, dtypes, strides, CPU tensors,
scale <= 0) raises instead of falling back to torch (fastbb/attention.py:38-48).

When the query tiles do not fill the SMs evenly (ViT-L/14 at 896x1344: 400 CTAs of work on 148 SMs) the kernel runs in
its split form, which needs ~11 MB of scratch memory, handed to fbb_flash64_f16_ws. Calls that may overlap on the GPU
must not share that memory, so where it comes from depends on the caller:
  * `workspace=<uint8 CUDA tensor>` lends a caller-owned (zeroed) one; `workspace=False` selects the plain
    one-CTA-per-tile form, which needs none;
  * inside `with use_workspaces(owner):` (what FastViT.run and graphs.Graphed do) it comes from `owner`, a
    `Workspaces` object: one buffer per device, created and zeroed OUTSIDE any stream capture (the warm-up call before a
    capture creates it), so that a captured graph bakes in memory its owner keeps alive and no other graph uses;
  * otherwise (plain eager calls) from a small per-(device, stream) table of this module, oldest entry evicted first.
"""
import collections
import contextlib
import threading

import torch

from . import _lib


def _ok(t):
    return (t.is_cuda and t.dtype == torch.float16 and t.dim() == 4 and t.shape[-1] == 64 and t.stride(-1) == 1
            and all(s % 8 == 0 for s in t.stride()[:3]) and t.data_ptr() % 16 == 0)


class Workspaces:
    """Split-form scratch memory owned by one caller (a FastViT, a Graphed): one zeroed uint8 buffer per device. An owner's
    calls are expected to be ordered on one stream at a time (a model instance is not re-entrant); two owners never share."""

    def __init__(self):
        self._by_device = {}
        self._counters = {}

    def counter(self, device):
        """A zeroed 4-byte counter on `device` for fbb_linear_layernorm_f16 (every launch leaves it zero again)."""
        idx = device.index if device.index is not None else torch.cuda.current_device()
        c = self._counters.get(idx)
        if c is None:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("the counter must exist before a stream capture starts: run the same call once outside the capture first")
            c = self._counters[idx] = torch.zeros(64, device=device, dtype=torch.int32)
        return c

    def get(self, device, need):
        idx = device.index if device.index is not None else torch.cuda.current_device()
        ws = self._by_device.get(idx)
        if ws is None or ws.numel() < need:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("the attention workspace must exist before a stream capture starts: run the same call once "
                                   "outside the capture first (FastViT.run_graphed and graphs.Graphed do)")
            ws = self._by_device[idx] = torch.zeros(need, device=device, dtype=torch.uint8)
        return ws


_ACTIVE = threading.local()                 # .owner: the Workspaces of the innermost use_workspaces() block of this thread
_EAGER = collections.OrderedDict()          # (device index, stream handle) -> uint8 tensor, for calls outside any owner
_EAGER_MAX = 8


@contextlib.contextmanager
def use_workspaces(owner):
    """Attention calls made inside the block (by this thread) take their scratch memory from `owner` (a Workspaces)."""
    prev = getattr(_ACTIVE, "owner", None)
    _ACTIVE.owner = owner
    try:
        yield owner
    finally:
        _ACTIVE.owner = prev


_EAGER_OWNERS = collections.OrderedDict()   # (device index, stream handle) -> Workspaces, only for its counter


def _counter(device):
    """Counter for fbb_linear_layernorm_f16 from the active owner, or from a per-(device, stream) table for plain eager calls."""
    owner = getattr(_ACTIVE, "owner", None)
    if owner is None:
        key = (device.index if device.index is not None else torch.cuda.current_device(), torch.cuda.current_stream(device).cuda_stream)
        owner = _EAGER_OWNERS.get(key)
        if owner is None:
            owner = _EAGER_OWNERS[key] = Workspaces()
            while len(_EAGER_OWNERS) > _EAGER_MAX:
                _EAGER_OWNERS.popitem(last=False)
        _EAGER_OWNERS.move_to_end(key)
    return owner.counter(device)


def _workspace(device, need):
    owner = getattr(_ACTIVE, "owner", None)
    if owner is not None:
        return owner.get(device, need)
    key = (device.index if device.index is not None else torch.cuda.current_device(), torch.cuda.current_stream(device).cuda_stream)
    ws = _EAGER.get(key)
    if ws is None or ws.numel() < need:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("attention() inside a stream capture needs a workspace that outlives the graph: wrap the call in "
                               "use_workspaces(...) with one made before the capture, or pass workspace=")
        ws = _EAGER[key] = torch.zeros(need, device=device, dtype=torch.uint8)
        while len(_EAGER) > _EAGER_MAX:
            _EAGER.popitem(last=False)
    _EAGER.move_to_end(key)
    return ws


def attention(q, k, v, scale=None, out=None, variant="hh", rows=None, workspace=None):
    """q, k, v [B, N, H, 64] -> [B, N, H, 64]. `rows` (the reference's CTA-height override) is accepted and ignored."""
    B, N, H, D = q.shape
    if out is not None and (out.shape != (*q.shape[:-1], v.shape[-1]) or out.device != q.device or out.dtype != q.dtype):
        raise ValueError("out must match the attention output shape, dtype and device")
    if variant not in _lib.FLASH_VARIANT:
        raise ValueError(f"unsupported variant: {variant}")
    if scale is None:
        scale = D ** -0.5
    if not scale > 0:
        raise ValueError("scale must be > 0")
    if not (_ok(q) and _ok(k) and _ok(v) and k.shape == q.shape and v.shape == q.shape and k.device == q.device == v.device
            and (out is None or _ok(out))):
        raise ValueError("attention needs CUDA fp16 [B, N, H, 64] tensors with a contiguous last dim, strides that are "
                         "multiples of 8 elements and 16-byte aligned storage (there is no fallback path)")
    if out is None:
        out = torch.empty((B, N, H, D), device=q.device, dtype=q.dtype)
    if B == 0 or N == 0 or H == 0:
        return out
    with _lib.on(q.device):
        lib = _lib.load()
        ws_ptr, ws_bytes = None, 0
        if workspace is not False:
            need = lib.fbb_flash64_workspace_bytes(B, N, H)
            if need > 0:
                ws = _workspace(q.device, need) if workspace is None else workspace
                if not (ws.is_cuda and ws.device == q.device and ws.dtype == torch.uint8 and ws.is_contiguous() and ws.numel() >= need):
                    raise ValueError(f"workspace must be a contiguous uint8 tensor of >= {need} bytes on {q.device}")
                ws_ptr, ws_bytes = ws.data_ptr(), ws.numel()
        _lib.check(lib.fbb_flash64_f16_ws(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, N, H,
            q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
            v.stride(0), v.stride(1), v.stride(2), out.stride(0), out.stride(1), out.stride(2),
            float(scale), _lib.FLASH_VARIANT[variant], ws_ptr, ws_bytes, _lib.stream_ptr(q.device)))
        _lib.launched(lib.fbb_flash64_launches(B, N, H, int(ws_ptr is not None)))
    return out


def attention_bhnd(q, k, v, scale=None, variant="hh", workspace=None):
    """SDPA-layout drop-in: q, k, v [B, H, N, 64] -> [B, H, N, 64] (strided views, no copies)."""
    return attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), scale=scale, variant=variant,
                     workspace=workspace).transpose(1, 2)
