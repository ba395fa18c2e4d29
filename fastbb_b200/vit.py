"""Host orchestration of the ViT fast path on B200: a drop-in for `get_intermediate_layers` of DINOv2-style ViTs and a
per-block forward patch for any pre-LN ViT (timm VisionTransformer, official DINOv2, Depth-Anything-V2 copies).

Public surface and behaviour follow the reference's fastbb/vit.py (FastViT :41-255, install_vit_blocks :311-328): fp16
weights and activations, autocast disabled inside, the packed qkv GEMM output read in place by the attention kernel,
position-embedding interpolation in fp32 cached per grid and invalidated when the parameter is reloaded, optional CUDA
graphs per input shape. What differs is below the operator calls: one block is

    LayerNorm kernel -> qkv GEMM (+bias) -> flash attention -> proj GEMM (+bias, LayerScale, residual)
    LayerNorm kernel -> fc1 GEMM (+bias, GELU) | w12 GEMM (+bias, SwiGLU) -> fc2 | w3 GEMM (+bias, LayerScale, residual)

seven launches of this package's own sm_100a kernels (eight where the attention hands the cls / register rows to its side
launch), with no torch fallback for small inputs or unsupported layouts
(the reference switches to SDPA below 2.2e5 elements, fastbb/vit.py:37,146; here the attention kernel has its own
small-input configuration). The process-global cuBLAS fp16-accumulation flag the reference flips around a run
(fastbb/vit.py:27-34) is never touched: the accumulate mode is an argument of each GEMM.
"""
import ctypes
import math
import os
import weakref

import torch
import torch.nn.functional as F

from . import _lib
from .attention import Workspaces, _workspace, attention, use_workspaces
from .gemm import linear, linear_layer_norm
from .layernorm import layer_norm, layer_norm_split

HEAD_DIM = 64


def _gemm_variants(gacc):
    """(variant for qkv/proj/fc1/w12, variant for fc2/w3) for a parsed spec value."""
    if gacc is True:
        return "h", "h"
    if gacc == "nofc2":
        return "h", "f32"
    if gacc is False or gacc == "chunk":
        return "f32", "f32"
    raise ValueError(f"unknown GEMM accumulate mode {gacc!r}")


def _norm(mod, x):
    """LayerNorm modules run through the fused kernel; any other norm module is the model's own code."""
    if isinstance(mod, torch.nn.LayerNorm) and len(mod.normalized_shape) == 1:
        return layer_norm(x, mod.weight, mod.bias, mod.eps)
    return mod(x)


def _gamma(block, name):
    return getattr(getattr(block, name, None), "gamma", None)


def _is_erf_gelu(act):
    return act is None or (isinstance(act, torch.nn.GELU) and act.approximate == "none")


def run_block(block, x, attn_variant, gacc):
    """One pre-LN transformer block on x [B, N, C] fp16 (contiguous); returns a new tensor, x is not modified.
    Block math as in fastbb/vit.py:108-143 (eval mode, no drop path)."""
    v_main, v_fc2 = _gemm_variants(gacc)
    a, m = block.attn, block.mlp
    B, N, C = x.shape
    H = a.num_heads
    if C != H * HEAD_DIM:
        raise NotImplementedError(f"the attention kernel covers head_dim {HEAD_DIM} only (embed {C}, heads {H})")
    qkv = linear(_norm(block.norm1, x), a.qkv.weight, a.qkv.bias, variant=v_main).view(B, N, 3, H, HEAD_DIM)
    q, k, v = qkv.unbind(2)
    o = attention(q, k, v, scale=getattr(a, "scale", None), variant="ff" if attn_variant == "sdpa" else attn_variant)
    g1 = _gamma(block, "ls1")
    x = linear(o.view(B, N, C), a.proj.weight, a.proj.bias, res=x, gamma=g1, variant=v_main)
    y = _norm(block.norm2, x)
    g2 = _gamma(block, "ls2")
    if hasattr(m, "fc1"):
        act = getattr(m, "act", None)
        if _is_erf_gelu(act):
            h = linear(y, m.fc1.weight, m.fc1.bias, act="gelu", variant=v_main)
        else:
            h = act(linear(y, m.fc1.weight, m.fc1.bias, variant=v_main))
        return linear(h, m.fc2.weight, m.fc2.bias, res=x, gamma=g2, variant=v_fc2)
    h = linear(y, m.w12.weight, m.w12.bias, act="swiglu", variant=v_main)  # DINOv2 SwiGLU FFN (ViT-g)
    return linear(h, m.w3.weight, m.w3.bias, res=x, gamma=g2, variant=v_fc2)


def _plain_ln(mod, C):
    """A LayerNorm over the last dimension with fp16 (or absent) contiguous parameters: what the fused kernels can apply."""
    return (isinstance(mod, torch.nn.LayerNorm) and tuple(mod.normalized_shape) == (C,)
            and all(p is None or (p.is_cuda and p.dtype == torch.float16 and p.is_contiguous()) for p in (mod.weight, mod.bias)))


def run_blocks_chained(blocks, x, attn_variant, gacc):
    """The per-operator path over a run of blocks with the same launches as the C stack runner: each residual GEMM carries
    the LayerNorm that follows it (proj + norm2; fc2 + the next block's norm1) through linear_layer_norm, which is one
    launch where the shape allows. Same results, bit for bit, as run_stack. x [B, N, C] fp16 contiguous CUDA; returns the
    new x (the input is not modified). Blocks the fused call does not cover go through run_block."""
    y = None  # LayerNorm-1 output of the next block, when the previous fc2 launch already produced it
    for i, block in enumerate(blocks):
        a, m = block.attn, block.mlp
        B, N, C = x.shape
        nxt = blocks[i + 1] if i + 1 < len(blocks) else None
        fusable = (hasattr(m, "fc1") or hasattr(m, "w12")) and C == a.num_heads * HEAD_DIM and _plain_ln(block.norm2, C)
        if not fusable:
            x, y = run_block(block, x, attn_variant, gacc), None
            continue
        v_main, v_fc2 = _gemm_variants(gacc)
        H = a.num_heads
        y1 = y if y is not None else _norm(block.norm1, x)
        qkv = linear(y1, a.qkv.weight, a.qkv.bias, variant=v_main).view(B, N, 3, H, HEAD_DIM)
        q, k, v = qkv.unbind(2)
        o = attention(q, k, v, scale=getattr(a, "scale", None), variant="ff" if attn_variant == "sdpa" else attn_variant)
        n2 = block.norm2
        x, y2 = linear_layer_norm(o.view(B, N, C), a.proj.weight, a.proj.bias, res=x, gamma=_gamma(block, "ls1"), variant=v_main,
                                  ln_weight=n2.weight, ln_bias=n2.bias, eps=n2.eps)
        if hasattr(m, "fc1"):
            act = getattr(m, "act", None)
            h = linear(y2, m.fc1.weight, m.fc1.bias, act="gelu", variant=v_main) if _is_erf_gelu(act) else act(linear(y2, m.fc1.weight, m.fc1.bias, variant=v_main))
            fc2 = m.fc2
        else:
            h = linear(y2, m.w12.weight, m.w12.bias, act="swiglu", variant=v_main)
            fc2 = m.w3
        g2 = _gamma(block, "ls2")
        if nxt is not None and _plain_ln(getattr(nxt, "norm1", None), C) and h.is_contiguous():
            n1 = nxt.norm1
            x, y = linear_layer_norm(h, fc2.weight, fc2.bias, res=x, gamma=g2, variant=v_fc2, ln_weight=n1.weight, ln_bias=n1.bias, eps=n1.eps)
        else:
            x, y = linear(h, fc2.weight, fc2.bias, res=x, gamma=g2, variant=v_fc2), None
    return x


def _dev_f16(t, numel=None):
    """Device pointer of an fp16 CUDA parameter the C block runner can read as is, None if absent; raises LookupError
    for anything else (strided, other dtype): the caller then takes the per-operator path, which handles those."""
    if t is None:
        return None
    if not (t.is_cuda and t.dtype == torch.float16 and t.is_contiguous() and t.data_ptr() % 16 == 0 and (numel is None or t.numel() == numel)):
        raise LookupError
    return t.data_ptr()


def _ln_params(mod, C):
    if not (isinstance(mod, torch.nn.LayerNorm) and tuple(mod.normalized_shape) == (C,)):
        raise LookupError
    return _dev_f16(mod.weight, C), _dev_f16(mod.bias, C), float(mod.eps)


def _fill_block_desc(d, block, attn_variant, gacc):
    """Weight pointers and shapes of `block` into the fbb_block_desc `d`; raises LookupError if the block is not of the
    form fbb_stack_forward_f16 covers (LayerNorm norms, fp16 contiguous weights, erf-GELU or SwiGLU MLP, head dim 64)."""
    a, m = block.attn, block.mlp
    C = a.qkv.weight.shape[1]
    H = a.num_heads
    if C != H * HEAD_DIM or tuple(a.qkv.weight.shape) != (3 * C, C) or tuple(a.proj.weight.shape) != (C, C):
        raise LookupError
    v_main, v_fc2 = _gemm_variants(gacc)
    d.ln1_w, d.ln1_b, d.eps1 = _ln_params(block.norm1, C)
    d.ln2_w, d.ln2_b, d.eps2 = _ln_params(block.norm2, C)
    d.qkv_w, d.qkv_b = _dev_f16(a.qkv.weight), _dev_f16(a.qkv.bias, 3 * C)
    d.proj_w, d.proj_b = _dev_f16(a.proj.weight), _dev_f16(a.proj.bias, C)
    d.gamma1, d.gamma2 = _dev_f16(_gamma(block, "ls1"), C), _dev_f16(_gamma(block, "ls2"), C)
    if hasattr(m, "fc1"):
        if not _is_erf_gelu(getattr(m, "act", None)):
            raise LookupError
        fc1, fc2, hidden, d.mlp = m.fc1, m.fc2, m.fc1.weight.shape[0], _lib.MLP_GELU
        rows1 = hidden
    else:
        fc1, fc2, hidden, d.mlp = m.w12, m.w3, m.w12.weight.shape[0] // 2, _lib.MLP_SWIGLU
        rows1 = 2 * hidden
    if tuple(fc1.weight.shape) != (rows1, C) or tuple(fc2.weight.shape) != (C, hidden) or hidden % 8:
        raise LookupError
    d.fc1_w, d.fc1_b = _dev_f16(fc1.weight), _dev_f16(fc1.bias, rows1)
    d.fc2_w, d.fc2_b = _dev_f16(fc2.weight), _dev_f16(fc2.bias, C)
    d.C, d.heads, d.hidden = C, H, hidden
    d.acc_main, d.acc_fc2 = _ACC[v_main], _ACC[v_fc2]
    d.flash_variant = _lib.FLASH_VARIANT["ff" if attn_variant == "sdpa" else attn_variant]
    scale = getattr(a, "scale", None)
    d.scale = float(HEAD_DIM ** -0.5 if scale is None else scale)
    if not d.scale > 0:
        raise LookupError


_ACC = {"f32": _lib.ACC_F32, "h": _lib.ACC_F16}


class _CachedDesc:
    """A filled fbb_block_desc of one block with what it was read from, so that a later call can tell cheaply whether it
    still describes the block: the submodules and parameter tensors (by identity and device address) and the plain
    attributes that went into it. Reading a block afresh costs ~20 us of Python (module attribute lookups); at ViT-S
    sizes that was a third of an eager forward pass."""
    __slots__ = ("desc", "mods", "params", "attrs", "cfg", "serial")
    _count = 0

    @staticmethod
    def _attrs(block):
        a, act = block.attn, getattr(block.mlp, "act", None)
        return (a.num_heads, getattr(a, "scale", None), block.norm1.eps, block.norm2.eps, type(act), getattr(act, "approximate", None))

    def __init__(self, block, attn_variant, gacc):
        self.desc = _lib.BlockDesc()
        _fill_block_desc(self.desc, block, attn_variant, gacc)
        self.cfg = (attn_variant, gacc)
        a, m = block.attn, block.mlp
        # (parent, name, child) with parent None standing for the block itself: this object is the value of a weak-keyed
        # table whose key is the block, so it must not hold the block (its submodules do not point back to it)
        leaves = [(None, n) for n in ("norm1", "norm2", "ls1", "ls2")] + [(a, "qkv"), (a, "proj")]
        leaves += [(m, n) for n in (("fc1", "fc2", "act") if hasattr(m, "fc1") else ("w12", "w3"))]
        self.mods = [(None, "attn", a), (None, "mlp", m)] + [(parent, n, (block if parent is None else parent)._modules.get(n)) for parent, n in leaves]
        self.params = [(leaf, n, t, None if t is None else t.data_ptr())
                       for _, _, leaf in self.mods[2:] if leaf is not None for n, t in leaf._parameters.items()]
        self.attrs = self._attrs(block)
        _CachedDesc._count += 1
        self.serial = _CachedDesc._count  # names this reading of the block in other tables without keeping it alive

    def valid(self, block, attn_variant, gacc):
        if self.cfg != (attn_variant, gacc):
            return False
        for parent, n, child in self.mods:
            if (block if parent is None else parent)._modules.get(n) is not child:
                return False
        for leaf, n, t, ptr in self.params:
            if leaf._parameters.get(n) is not t or (t is not None and t.data_ptr() != ptr):
                return False
        return self.attrs == self._attrs(block)


def _block_desc(block, attn_variant, gacc):
    """The block's fbb_block_desc, read afresh only when the block changed since the last call (raises like
    _fill_block_desc)."""
    return _block_entry(block, attn_variant, gacc).desc


def _block_entry(block, attn_variant, gacc):
    ent = _DESCS.get(block)
    if ent is None or not ent.valid(block, attn_variant, gacc):
        ent = _DESCS[block] = _CachedDesc(block, attn_variant, gacc)
    return ent


_DESCS = weakref.WeakKeyDictionary()  # block module -> _CachedDesc (kept outside the module: nothing to copy or pickle)
_STACK_SIZES = {}                    # see run_stack


def run_stack(blocks, x, attn_variant, gacc):
    """blocks[...] applied IN PLACE to x [B, N, C] (fp16, contiguous, CUDA) through ONE call of the C stack runner
    (fbb_stack_forward_f16: 7 or 8 launches per block, the same kernels in the same order as run_block). Returns False
    without touching x if some block is outside what the runner covers; the caller then uses run_block."""
    n = len(blocks)
    descs = (_lib.BlockDesc * n)()
    try:
        ents = [_block_entry(b, attn_variant, gacc) for b in blocks]
    except (LookupError, AttributeError):
        return False
    for i, e in enumerate(ents):
        descs[i] = e.desc
    if not (x.is_cuda and x.dtype == torch.float16 and x.is_contiguous() and x.dim() == 3 and x.shape[2] == descs[0].C):
        return False
    B, N, _ = x.shape
    if B == 0 or N == 0 or n == 0:
        return True
    lib = _lib.load()
    with _lib.on(x.device):
        # scratch size, attention workspace size and launch count of this run of blocks at this shape: three C calls,
        # remembered per (descriptors, shape, device) - they are a tenth of the host time of a ViT-S forward pass
        key = (tuple(e.serial for e in ents), B, N, x.device.index)
        sizes = _STACK_SIZES.get(key)
        if sizes is None:
            need = lib.fbb_flash64_workspace_bytes(B, N, descs[0].heads)
            launches = lib.fbb_stack_launches(descs, n, B * N) + n * (lib.fbb_flash64_launches(B, N, descs[0].heads, int(need > 0)) - 1)
            if len(_STACK_SIZES) >= 256:
                _STACK_SIZES.clear()
            sizes = _STACK_SIZES[key] = (lib.fbb_stack_scratch_bytes(descs, n, B * N), need, launches)
        scratch = torch.empty(sizes[0], device=x.device, dtype=torch.uint8)
        ws = _workspace(x.device, sizes[1]) if sizes[1] > 0 else None
        _lib.check(lib.fbb_stack_forward_f16(descs, n, x.data_ptr(), B, N, scratch.data_ptr(), scratch.numel(),
                                             ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
                                             _lib.stream_ptr(x.device)))
    _lib.launched(sizes[2])
    return True


def _param_version(parameters):
    """Identity + mutation counters of parameters: changes when weights are reloaded or moved."""
    try:
        return tuple((id(p), p._version, p.device, p.dtype) for p in parameters)
    except RuntimeError:  # inference tensors do not track mutations
        return None


def _flatten_blocks(blocks):
    out = []
    for b in blocks:
        if isinstance(b, torch.nn.ModuleList) or type(b).__name__ == "BlockChunk":
            out.extend(list(b))
        else:
            out.append(b)
    return [b for b in out if not isinstance(b, torch.nn.Identity)]


class FastViT:
    """Wraps a DINOv2-style module tree (`pos_embed, patch_size, blocks, patch_embed, cls_token, norm`, optional
    `num_register_tokens, register_tokens, interpolate_offset, interpolate_antialias`) and runs its block stack on the
    B200 kernels. Constructor arguments as in fastbb/vit.py:42."""

    def __init__(self, vit, attn="fh", gacc=True, dtype=torch.float16, out_dtype=None, graphs=False, graph_noclone=False):
        if dtype != torch.float16:
            raise ValueError("the B200 kernels compute in fp16 storage; dtype must be torch.float16")
        _gemm_variants(gacc)
        # the official code interpolates the fp32 table, so keep it before the module is cast
        self.pos_fp32 = vit.pos_embed.detach().float().clone()
        self.vit = vit.to(dtype).eval()
        self.dtype, self.attn, self.gacc, self.out_dtype = dtype, attn, gacc, out_dtype
        ps = vit.patch_size
        self.ps = ps if isinstance(ps, int) else ps[0]
        self.nreg = getattr(vit, "num_register_tokens", 0) or 0
        self.blocks = _flatten_blocks(vit.blocks)
        self._pos = {}
        self._pos_version = _param_version((vit.pos_embed,))
        self.graphs, self.graph_noclone = graphs, graph_noclone
        self._graphs, self._pool, self._graph_version = {}, None, None
        self._orig = {}
        self._patch_w, self._patch_w_version = None, None
        self._workspaces = Workspaces()  # this instance's attention scratch memory (never shared with another model or graph)

    _version = staticmethod(_param_version)

    # ------------------------------------------------------------------ tokens
    def _refresh_pos(self):
        """Drop cached tables (and graphs that baked them in) when pos_embed was reloaded, moved or re-cast."""
        now = _param_version((self.vit.pos_embed,))
        if now is not None and now == self._pos_version:
            return
        same_storage = (now is not None and self._pos_version is not None and now[0][:2] == self._pos_version[0][:2])
        if same_storage:  # only moved / cast: the fp32 master copy is still right
            self.pos_fp32 = self.pos_fp32.to(self.vit.pos_embed.device)
        else:
            self.pos_fp32 = self.vit.pos_embed.detach().float().clone()
        self._pos.clear()
        self._graphs.clear()
        self._pool = None
        self._pos_version = now

    def pos_embed(self, h0, w0):
        """Position table for an h0 x w0 patch grid, fp16 [1, 1 + h0*w0, C] (upstream DINOv2 interpolation rule)."""
        self._refresh_pos()
        table = self._pos.get((h0, w0))
        if table is None:
            pe = self.pos_fp32
            n = pe.shape[1] - 1
            side = int(math.sqrt(n))
            if n == h0 * w0 and h0 == w0:
                table = pe
            else:
                off = getattr(self.vit, "interpolate_offset", 0.1)
                size_kw = {"scale_factor": ((h0 + off) / side, (w0 + off) / side)} if off else {"size": (h0, w0)}
                grid = pe[:, 1:].reshape(1, side, side, -1).permute(0, 3, 1, 2)
                grid = F.interpolate(grid, mode="bicubic", antialias=getattr(self.vit, "interpolate_antialias", False), **size_kw)
                if grid.shape[-2:] != (h0, w0):
                    raise RuntimeError(f"position grid came out as {tuple(grid.shape[-2:])}, wanted {(h0, w0)}")
                table = torch.cat([pe[:, :1], grid.permute(0, 2, 3, 1).flatten(1, 2)], 1)
            table = self._pos[(h0, w0)] = table.to(self.dtype)
        return table

    def _patch_gemm_weight(self):
        """[C, 4*ps*ps] fp16 view of a plain patch-embedding convolution (kernel = stride = patch, 3 input channels, no norm)
        with a zero fourth input channel, so that the reduction length is a multiple of 8; None when the model's patch
        embedding is anything else (then its own forward is used). Cached until the weight is reloaded."""
        pe = getattr(self.vit, "patch_embed", None)
        proj = getattr(pe, "proj", None)
        ps = self.ps
        plain = (isinstance(proj, torch.nn.Conv2d) and proj.kernel_size == (ps, ps) and proj.stride == (ps, ps)
                 and proj.padding == (0, 0) and proj.dilation == (1, 1) and proj.groups == 1 and proj.in_channels == 3
                 and _ident(getattr(pe, "norm", None)) and (4 * ps * ps) % 8 == 0 and proj.weight.is_cuda
                 and proj.weight.dtype == self.dtype and getattr(pe, "flatten", True) is not False)
        if not plain:
            return None, None
        version = _param_version((proj.weight,))
        if version is None or version != self._patch_w_version:
            w = proj.weight.detach()
            w4 = torch.zeros(w.shape[0], 4, ps, ps, dtype=w.dtype, device=w.device)
            w4[:, :3] = w
            self._patch_w, self._patch_w_version = w4.reshape(w.shape[0], 4 * ps * ps), version
        return self._patch_w, proj.bias

    def tokens(self, x):
        """Image batch [B, 3, H, W] -> tokens [B, 1 + nreg + hw, C] (fastbb/vit.py:97-105): patch embedding, cls token,
        position table, registers after cls. A plain patch-embedding convolution runs as one GEMM per image on the
        linear kernel, with the bias and the position table fused into its epilogue and the result written straight
        into the token buffer; any other patch-embedding module runs as the model's own code."""
        vit = self.vit
        B, _, h, w = x.shape
        h0, w0 = h // self.ps, w // self.ps
        pos = self.pos_embed(h0, w0)
        w4, bias = self._patch_gemm_weight() if (x.is_cuda and h % self.ps == 0 and w % self.ps == 0) else (None, None)
        if w4 is None:
            t = vit.patch_embed(x.to(self.dtype))
            t = torch.cat([vit.cls_token.to(self.dtype).expand(B, -1, -1), t], 1)
            t = t + pos
            if self.nreg:
                t = torch.cat([t[:, :1], vit.register_tokens.to(self.dtype).expand(B, -1, -1), t[:, 1:]], 1)
            return t
        ps, C, nreg = self.ps, w4.shape[0], self.nreg
        # unfold into [B, h0*w0, 4*ps*ps] (one strided copy that also casts to fp16; the fourth channel is zero)
        patches = torch.empty(B, h0, w0, 4, ps, ps, dtype=self.dtype, device=x.device)
        patches[:, :, :, :3].copy_(x.reshape(B, 3, h0, ps, w0, ps).permute(0, 2, 4, 1, 3, 5))
        patches[:, :, :, 3].zero_()
        patches = patches.view(B, h0 * w0, 4 * ps * ps)
        t = torch.empty(B, 1 + nreg + h0 * w0, C, dtype=self.dtype, device=x.device)
        t[:, 0] = vit.cls_token.to(self.dtype)[0, 0] + pos[0, 0]
        if nreg:
            t[:, 1:1 + nreg] = vit.register_tokens.to(self.dtype)
        pos_patches = pos[0, 1:]
        for b in range(B):
            linear(patches[b], w4, bias, res=pos_patches, variant="f32", out=t[b, 1 + nreg:])
        return t

    # ------------------------------------------------------------------ block
    def block(self, b, x):
        return run_block(b, x, self.attn, self.gacc)

    # ------------------------------------------------------------------ API
    def run(self, x, layers, norm=True, split=False):
        """-> list of tokens [B, 1 + nreg + HW, C] after the blocks in `layers` (normed with vit.norm if norm).
        split=True (what get_intermediate_layers(reshape=True) uses): a list of (patches [B, C, h, w], cls [B, C], registers)
        instead, written by ONE launch per selected layer (final norm + cls split + register drop + channel-major store)
        when vit.norm is a plain LayerNorm; otherwise the same tuple built with torch ops."""
        out = []
        layers = sorted(l for l in set(layers) if 0 <= l < len(self.blocks))  # as the reference's loop: others never match
        if not layers:
            return out
        last = layers[-1]
        with torch.autocast("cuda", enabled=False), use_workspaces(self._workspaces):
            t = self.tokens(x).contiguous()
            # One C call per run of blocks between two selected layers (t is this function's own buffer, updated in
            # place); blocks the C runner does not cover, or FBB_NO_RUNNER=1, take the per-operator path.
            use_runner = os.environ.get("FBB_NO_RUNNER") != "1"
            i = 0
            while i <= last:
                j = min(l for l in layers if l >= i)  # next selected layer
                if not (use_runner and run_stack(self.blocks[i:j + 1], t, self.attn, self.gacc)):
                    use_runner = False
                    if t.is_cuda:
                        t = run_blocks_chained(self.blocks[i:j + 1], t, self.attn, self.gacc)
                    else:
                        for b in self.blocks[i:j + 1]:
                            t = run_block(b, t, self.attn, self.gacc)
                out.append(self._split_outputs(t, x, norm) if split else (_norm(self.vit.norm, t) if norm else t.clone()))
                i = j + 1
        if os.environ.get("FBB_CHECK_STATUS") == "1" and not torch.cuda.is_current_stream_capturing():
            _lib.device_status()  # debugging aid (synchronises): raises if a kernel of this run gave up a bounded wait
        return out

    def _split_outputs(self, t, x, norm):
        """(patches [B, C, h, w], cls, registers) of the token tensor t for an input image batch x."""
        B, _, h, w = x.shape
        grid, n_prefix, nm = (h // self.ps, w // self.ps), 1 + self.nreg, self.vit.norm
        plain = (t.is_cuda and isinstance(nm, torch.nn.LayerNorm) and tuple(nm.normalized_shape) == (t.shape[-1],) and t.shape[-1] <= 2048
                 and n_prefix <= 32 and all(p is None or (p.dtype == torch.float16 and p.is_contiguous()) for p in (nm.weight, nm.bias)))
        if plain:
            return layer_norm_split(t, nm.weight, nm.bias, nm.eps, n_prefix=n_prefix, grid=grid, norm=norm)
        o = _norm(nm, t) if norm else t
        patches = o[:, n_prefix:].reshape(B, grid[0], grid[1], -1).permute(0, 3, 1, 2).contiguous()
        return patches, o[:, 0].clone(), (o[:, 1:n_prefix].clone() if self.nreg else None)

    def run_graphed(self, x, layers, norm=True, split=False):
        """graphs=True: one CUDA graph per (input shape, layers), captured on first use after one warm-up run; outputs
        are the graph's static buffers (cloned unless graph_noclone). Falls back to run() for inference tensors."""
        self._refresh_pos()
        version = _param_version(self.vit.parameters())
        if version is None:
            return self.run(x, layers, norm, split)
        if version != self._graph_version:
            self._graphs.clear()
            self._pool = None
            self._graph_version = version
        key = (tuple(x.shape), x.dtype, x.device, tuple(sorted(layers)), norm, split)
        entry = self._graphs.get(key)
        if entry is None:
            static_in = x.clone()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self.run(static_in, layers, norm, split)  # warm-up: position cache, kernel attributes, attention workspace
            torch.cuda.current_stream().wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, pool=self._pool):
                static_out = self.run(static_in, layers, norm, split)
            self._pool = graph.pool()
            entry = self._graphs[key] = (graph, static_in, static_out)
        graph, static_in, static_out = entry
        static_in.copy_(x)
        graph.replay()
        if self.graph_noclone:
            return static_out
        return [tuple(None if e is None else e.clone() for e in o) if isinstance(o, tuple) else o.clone() for o in static_out]

    def _run(self, x, layers, norm, split=False):
        return (self.run_graphed if self.graphs else self.run)(x, layers, norm, split)

    def get_intermediate_layers(self, x, n=1, reshape=False, return_class_token=False, norm=True):
        """Same contract as DinoVisionTransformer.get_intermediate_layers (fastbb/vit.py:220-235)."""
        nb = len(self.blocks)
        layers = list(range(nb - n, nb)) if isinstance(n, int) else list(n)
        cast = self.out_dtype is not None and self.out_dtype != self.dtype
        if reshape:  # [B, C, h, w] patches: one launch per layer does the norm, the cls split and the channel-major store
            triples = self._run(x, set(layers), norm, split=True)
            outs = [p.to(self.out_dtype) if cast else p for p, _, _ in triples]
            cls = [c.to(self.out_dtype) if cast else c for _, c, _ in triples]
        else:
            outs = self._run(x, set(layers), norm)
            if cast:
                outs = [o.to(self.out_dtype) for o in outs]
            cls = [o[:, 0] for o in outs]
            outs = [o[:, 1 + self.nreg:] for o in outs]
        return tuple(zip(outs, cls)) if return_class_token else tuple(outs)

    def forward_features(self, x):
        """Same keys as the official DinoVisionTransformer.forward_features (eval, no masks)."""
        t = self._run(x, {len(self.blocks) - 1}, norm=False)[0]
        with torch.autocast("cuda", enabled=False):
            n = _norm(self.vit.norm, t)
        r = 1 + self.nreg
        return {"x_norm_clstoken": n[:, 0], "x_norm_regtokens": n[:, 1:r], "x_norm_patchtokens": n[:, r:],
                "x_prenorm": t, "masks": None}

    def __call__(self, x):
        """= official forward in eval mode with an Identity head: the normed cls token."""
        return self.forward_features(x)["x_norm_clstoken"]

    def install(self):
        """Make the wrapped module's `get_intermediate_layers` (an instance attribute) call this object."""
        self._orig["get_intermediate_layers"] = self.vit.__dict__.get("get_intermediate_layers")
        self.vit.get_intermediate_layers = self.get_intermediate_layers
        self.vit._fastbb = self
        return self


# ==================================================================== block-level drop-in (any ViT-style model)
class _BlockCfg:
    """Spec of a patched block (attention variant, GEMM accumulate mode)."""

    def __init__(self, attn, gacc, workspaces=None):
        _gemm_variants(gacc)
        self.attn, self.gacc = attn, gacc
        # attention scratch memory shared by the blocks patched in one install_vit_blocks call (they run one after another)
        self.workspaces = workspaces if workspaces is not None else Workspaces()

    def block(self, b, x, own=False):
        """One block on x [B, N, C] fp16 contiguous -> new tensor. `own`: x is a private copy the call may overwrite.
        One C call (fbb_block_forward_f16's table form) when the block is of the form the runner covers, else seven."""
        if x.dim() == 3 and os.environ.get("FBB_NO_RUNNER") != "1":
            t = x if own else x.clone()
            if run_stack([b], t, self.attn, self.gacc):
                return t
        return run_block(b, x, self.attn, self.gacc)


def _ident(m):
    return m is None or isinstance(m, (torch.nn.Identity, torch.nn.Dropout))


def _block_supported(b):
    """True for a pre-norm block norm1 -> attn(packed qkv, proj) -> ls1 -> +x; norm2 -> mlp(fc1, act, fc2 | w12, w3) ->
    ls2 -> +x with 64-wide heads. q/k norms, gates, rope, separate qkv biases and unknown drop-path modules are not
    (the structural test of fastbb/vit.py:273-294, plus the head-dim rule, because there is no SDPA path here)."""
    a, m = getattr(b, "attn", None), getattr(b, "mlp", None)
    if a is None or m is None or not (hasattr(b, "norm1") and hasattr(b, "norm2")):
        return False
    qkv, proj = getattr(a, "qkv", None), getattr(a, "proj", None)
    if not (isinstance(qkv, torch.nn.Linear) and isinstance(proj, torch.nn.Linear)):
        return False
    heads = getattr(a, "num_heads", None)
    if not isinstance(heads, int) or qkv.in_features != heads * HEAD_DIM:
        return False
    if any(not _ident(getattr(a, n, None)) for n in ("q_norm", "k_norm", "norm")) or getattr(a, "gate", None) is not None:
        return False
    if getattr(a, "qkv_bias_separate", False) or getattr(a, "rope", None) is not None:
        return False
    for n in ("drop_path", "drop_path1", "drop_path2"):
        d = getattr(b, n, None)
        if hasattr(b, n) and not _ident(d) and type(d).__name__ != "DropPath":
            return False
    for n in ("ls1", "ls2"):
        ls = getattr(b, n, None)
        if not (_ident(ls) or hasattr(ls, "gamma")):
            return False
    if hasattr(m, "fc1"):
        return _ident(getattr(m, "norm", None)) and isinstance(m.fc1, torch.nn.Linear) and isinstance(m.fc2, torch.nn.Linear)
    return hasattr(m, "w12") and hasattr(m, "w3")


def _fast_block_forward(self, x, *args, **kw):
    """Replacement for block.forward: masks, attention biases, causal attention and training mode go to the block's
    original forward; everything else runs on the B200 kernels and comes back in the caller's dtype."""
    masked = (args and args[0] is not None) or kw.get("attn_mask") is not None or kw.get("attn_bias") is not None
    if masked or kw.get("is_causal") or self.training:
        return type(self).forward(self, x, *args, **kw)
    cfg = self._fbb_cfg
    caller_dtype = x.dtype
    with torch.autocast("cuda", enabled=False), use_workspaces(cfg.workspaces):
        wd = self.attn.qkv.weight.dtype
        xc = x.to(wd).contiguous()
        y = cfg.block(self, xc, own=xc.data_ptr() != x.data_ptr())  # a cast or compaction made a private copy already
    return y if caller_dtype == wd else y.to(caller_dtype)


def install_vit_blocks(model, spec="fh-g0", convert=True):
    """Patch every supported transformer block in `model` (forward -> B200 kernels). Tokenizer, position embedding and
    heads stay the model's own code. convert=True: model.half(). Idempotent; returns the number of newly patched blocks."""
    from . import parse_vit_spec
    attn, gacc = parse_vit_spec(spec)
    if convert:
        model.half()
    n = 0
    workspaces = Workspaces()
    for b in model.modules():
        if b is model and not hasattr(b, "norm1"):
            continue
        if "_fbb_cfg" not in b.__dict__ and _block_supported(b):
            b._fbb_cfg = _BlockCfg(attn, gacc, workspaces)
            b.forward = _fast_block_forward.__get__(b)
            n += 1
    return n
