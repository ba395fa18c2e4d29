"""F.linear on the tcgen05 tensor cores with fused epilogues (kernel: csrc/gemm.cu).

Same call signature as the reference's fastbb/gemm.py:30 `linear`:

    y = linear(x, fc1.weight, fc1.bias, act="gelu")                 # x [..., K] fp16
    x = linear(h, fc2.weight, fc2.bias, res=x, gamma=ls2.gamma)     # out = res + gamma * y (new tensor)

variant: "f32", "c1", "c2" (default), "c4" -> fp32 tensor-memory accumulator (the reference's chunked fp16
accumulation exists to approach fp32 error at GeForce fp16 rate; on B200 the fp32 accumulator runs at the same rate,
so all of them map to it); "h" -> fp16 accumulator. act: None | "none" | "gelu" (exact erf), plus "swiglu" (w holds
w12; the output has N/2 columns, out = silu(x1) * x2, fastbb/vit.py:139-141), which the reference runs as three kernels.
Unsupported inputs raise (the reference falls back to torch instead, fastbb/gemm.py:36-51).
"""
import torch

from . import _lib
from .layernorm import _on

_ACT = {None: _lib.EPI_NONE, "none": _lib.EPI_NONE, "gelu": _lib.EPI_GELU, "swiglu": _lib.EPI_SWIGLU}
_ACC = {"f32": _lib.ACC_F32, "c1": _lib.ACC_F32, "c2": _lib.ACC_F32, "c4": _lib.ACC_F32, "h": _lib.ACC_F16}


def linear(x, w, b=None, act=None, res=None, gamma=None, variant="c2", out=None, bn_pref=None):
    if act not in _ACT:
        raise ValueError(f"unsupported activation: {act}")
    if variant not in _ACC:
        raise ValueError(f"unsupported variant: {variant}")
    if not x.is_cuda:
        raise ValueError("fastbb_b200.linear needs CUDA tensors (there is no CPU path)")
    if x.dtype != torch.float16 or w.dtype != torch.float16:
        raise ValueError("x and w must be fp16")
    K, N = x.shape[-1], w.shape[0]
    if w.dim() != 2 or w.shape[1] != K or w.device != x.device:
        raise ValueError("w must be [N, K] on the input's device")
    n_out = N // 2 if act == "swiglu" else N
    oshape = (*x.shape[:-1], n_out)
    if out is not None and (out.shape != oshape or out.device != x.device or out.dtype != x.dtype or not out.is_contiguous()
                            or out.data_ptr() % 16):
        raise ValueError("out must be contiguous with the output shape, input dtype and device")
    for t, n in ((b, N), (gamma, n_out)):
        if t is not None and (t.device != x.device or t.dtype != x.dtype or not t.is_contiguous() or t.numel() != n):
            raise ValueError("bias / gamma must be contiguous fp16 vectors of the output width on the input's device")
    if res is not None and (res.device != x.device or res.dtype != torch.float16 or res.shape != oshape):
        raise ValueError("res must be fp16 with the output shape on the input's device")
    if gamma is not None and res is None:
        raise ValueError("gamma is the LayerScale of the residual epilogue: it needs res")
    x2 = x.reshape(-1, K)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    if w.stride(-1) != 1:
        w = w.contiguous()
    M = x2.shape[0]
    r2 = None
    if res is not None:
        r2 = res.reshape(-1, n_out)
        if r2.stride(-1) != 1:
            r2 = r2.contiguous()
    if out is None:
        out = torch.empty(oshape, device=x.device, dtype=torch.float16)
    if M == 0:
        return out
    with _on(x.device):
        _lib.check(_lib.load().fbb_linear_f16(
            x2.data_ptr(), w.data_ptr(), out.data_ptr(), _lib.ptr(b), _lib.ptr(r2), _lib.ptr(gamma), M, N, K,
            x2.stride(0) if M > 1 else K, w.stride(0) if N > 1 else K, n_out, (r2.stride(0) if M > 1 else n_out) if r2 is not None else 0,
            _ACT[act], _ACC[variant], _lib.stream_ptr(x.device)))
    _lib.launched()
    return out


def linear_layer_norm(x, w, b=None, act=None, res=None, gamma=None, variant="c2", ln_weight=None, ln_bias=None, eps=1e-6, out=None):
    """(out, y): out = linear(x, w, b, act, res, gamma) as above (act None or "gelu") and y = LayerNorm(out) * ln_weight +
    ln_bias over the last dimension, through fbb_linear_layernorm_f16: ONE launch when the shape allows (what a
    transformer block's proj + norm2, and fc2 + the next block's norm1, become), otherwise the two kernels one after
    the other. x must be 2-D or 3-D contiguous; out may be `res` itself (in place on the residual stream)."""
    from .attention import _counter
    if act not in (None, "none", "gelu"):
        raise ValueError(f"unsupported activation for the fused form: {act}")
    if variant not in _ACC:
        raise ValueError(f"unsupported variant: {variant}")
    if not (x.is_cuda and x.dtype == torch.float16 and w.dtype == torch.float16 and x.is_contiguous() and w.is_contiguous()):
        raise ValueError("linear_layer_norm needs contiguous CUDA fp16 x and w (there is no CPU path)")
    K, N = x.shape[-1], w.shape[0]
    if w.dim() != 2 or w.shape[1] != K or w.device != x.device:
        raise ValueError("w must be [N, K] on the input's device")
    oshape = (*x.shape[:-1], N)
    for t in (b, gamma, ln_weight, ln_bias):
        if t is not None and (t.device != x.device or t.dtype != torch.float16 or not t.is_contiguous() or t.numel() != N):
            raise ValueError("bias / gamma / LayerNorm parameters must be contiguous fp16 vectors of the output width on the input's device")
    if res is not None and (res.device != x.device or res.dtype != torch.float16 or res.shape != oshape or not res.is_contiguous()):
        raise ValueError("res must be contiguous fp16 with the output shape on the input's device")
    if gamma is not None and res is None:
        raise ValueError("gamma is the LayerScale of the residual epilogue: it needs res")
    if out is None:
        out = torch.empty(oshape, device=x.device, dtype=torch.float16)
    elif out.shape != oshape or out.device != x.device or out.dtype != torch.float16 or not out.is_contiguous():
        raise ValueError("out must be contiguous fp16 with the output shape on the input's device")
    y = torch.empty(oshape, device=x.device, dtype=torch.float16)
    M = x.numel() // K if K else 0
    if M == 0:
        return out, y
    with _on(x.device):
        lib = _lib.load()
        counter = _counter(x.device)
        _lib.check(lib.fbb_linear_layernorm_f16(
            x.data_ptr(), w.data_ptr(), out.data_ptr(), _lib.ptr(b), _lib.ptr(res), _lib.ptr(gamma), M, N, K, K, K, N, N if res is not None else 0,
            _ACT[act], _ACC[variant], _lib.ptr(ln_weight), _lib.ptr(ln_bias), float(eps), y.data_ptr(), N, counter.data_ptr(),
            _lib.stream_ptr(x.device)))
        _lib.launched(lib.fbb_linear_layernorm_launches(M, N, _ACT[act], 1))
    return out, y
