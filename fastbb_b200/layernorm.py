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


def layer_norm_split(x, weight=None, bias=None, eps=1e-6, n_prefix=1, grid=None, norm=True):
    """The final norm of a ViT with its outputs split as get_intermediate_layers returns them, in one launch
    (kernel: layernorm_split_f16_kernel; replaces vit.norm + cls split + register drop + the permute / contiguous copy of
    reshape=True, fastbb/vit.py:184,225-232).

    x [B, N, C] fp16 contiguous, rows 0 .. n_prefix-1 of an image = cls + register tokens. Returns (patches, cls, regs):
    patches [B, N - n_prefix, C], or [B, C, h, w] when grid=(h, w) is given; cls [B, C]; regs [B, n_prefix - 1, C] (None
    without registers). norm=False copies the rows unnormalised."""
    if not (x.is_cuda and x.dtype == torch.float16 and x.dim() == 3 and x.is_contiguous()):
        raise ValueError("layer_norm_split needs a contiguous CUDA fp16 [B, N, C] tensor")
    B, N, C = x.shape
    HW = N - n_prefix
    if grid is not None and grid[0] * grid[1] != HW:
        raise ValueError(f"grid {tuple(grid)} does not match the {HW} patch tokens")
    for p in (weight, bias):
        if p is not None and not (p.numel() == C and p.is_contiguous() and p.device == x.device and p.dtype == torch.float16):
            raise ValueError("weight / bias must be contiguous fp16 [C] tensors on the input's device")
    patches = torch.empty((B, C, *grid) if grid is not None else (B, HW, C), device=x.device, dtype=torch.float16)
    cls = torch.empty((B, C), device=x.device, dtype=torch.float16)
    regs = torch.empty((B, n_prefix - 1, C), device=x.device, dtype=torch.float16) if n_prefix > 1 else None
    if B == 0 or N == 0:
        return patches, cls, regs
    with _on(x.device):
        _lib.check(_lib.load().fbb_layernorm_split_f16(
            x.data_ptr(), _lib.ptr(weight), _lib.ptr(bias), patches.data_ptr(), cls.data_ptr(), _lib.ptr(regs), B, N, C, n_prefix,
            float(eps), 1 if norm else 0, 1 if grid is not None else 0, _lib.stream_ptr(x.device)))
    _lib.launched()
    return patches, cls, regs
