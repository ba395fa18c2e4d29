"""LayerNorm over the last dimension fused with the cast to fp16 (kernel: csrc/layernorm.cu).

Stands in for the `b.norm1(x)`, `b.norm2(x)` and `vit.norm(t)` module calls of the reference's block
(fastbb/vit.py:114,126,130,139,159,166,170,184,241), which run aten's native_layer_norm.
"""
import torch

from . import _lib


_on = _lib.on


def layer_norm(x, weight=None, bias=None, eps=1e-6, out=None):
    """x [..., C] (fp16, bf16 or fp32, last dim contiguous) -> fp16 [..., C]. Statistics in fp32."""
    if not x.is_cuda:
        raise ValueError("fastbb_b200.layer_norm needs a CUDA tensor (there is no CPU path)")
    if x.dtype not in _lib.DTYPE_CODE:
        raise ValueError(f"unsupported input dtype {x.dtype}")
    C = x.shape[-1]
    x2 = x.reshape(-1, C)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    M = x2.shape[0]
    if out is None:
        out = torch.empty(x.shape, device=x.device, dtype=torch.float16)
    elif out.shape != x.shape or out.dtype != torch.float16 or out.device != x.device or not out.is_contiguous():
        raise ValueError("out must be a contiguous fp16 tensor of the input's shape on the input's device")
    pd = torch.float16
    for p in (weight, bias):
        if p is not None:
            if p.numel() != C or not p.is_contiguous() or p.device != x.device or p.dtype not in _lib.DTYPE_CODE:
                raise ValueError("weight / bias must be contiguous [C] tensors on the input's device")
            pd = p.dtype
    if weight is not None and bias is not None and weight.dtype != bias.dtype:
        raise ValueError("weight and bias must share a dtype")
    if M == 0:
        return out
    with _on(x.device):
        _lib.check(_lib.load().fbb_layernorm_f16(
            x2.data_ptr(), out.data_ptr(), _lib.ptr(weight), _lib.ptr(bias), M, C, x2.stride(0) if M > 1 else C, C, float(eps),
            _lib.DTYPE_CODE[x.dtype], _lib.DTYPE_CODE[pd], _lib.stream_ptr(x.device)))
    _lib.launched()
    return out


def module_norm(norm, x, out=None):
    """Apply an nn.LayerNorm module's parameters through the fused kernel."""
    if tuple(norm.normalized_shape) != (x.shape[-1],):
        raise ValueError("only LayerNorm over the last dimension is supported")
    return layer_norm(x, norm.weight, norm.bias, norm.eps, out=out)
