"""CPU oracle for the ViT block fast path: an fp32 restatement of what the reference computes.

TEST INFRASTRUCTURE ONLY. Nothing in the product package may import this module; it is used by tests/, by
__graft_entry__.smoke() and by bench.py's cpu_baseline / reference arm as the checker and the timed CPU baseline.

Each function restates one piece of the reference (paths relative to the reference repository) in plain fp32
PyTorch-on-CPU tensor algebra (matmul, exp, mean: no fused library operator such as scaled_dot_product_attention,
F.layer_norm or F.gelu on the checked path). It is pinned against the reference itself: tests/golden/make_golden.py
imports the reference, runs its friendly fp32 tier (FastViT(attn="sdpa", gacc=False, dtype=float32), plus
gemm.linear and attention.attention on CPU tensors) on the seeded inputs made here, and commits the outputs under
tests/golden/; tests/test_oracle.py checks this file against those vectors. The reference's own tests hold no golden
vector or known-answer test for this path (its one ViT test, tests/test_fastbb.py:75-86, only covers the
position-embedding cache, mirrored in tests/test_host_api.py).

Model parameters are a plain dict of fp32 tensors keyed by the official DINOv2 names
(fastbb/models/dinov2.py:64-81): patch_embed.proj.{weight,bias}, cls_token, pos_embed, register_tokens, mask_token,
blocks.N.{norm1,norm2}.{weight,bias}, blocks.N.attn.{qkv,proj}.{weight,bias}, blocks.N.{ls1,ls2}.gamma,
blocks.N.mlp.{fc1,fc2}|{w12,w3}.{weight,bias}, norm.{weight,bias}.
"""
import math

import torch

# name -> (embed_dim, depth, heads, ffn)                                       fastbb/models/dinov2.py:15-18
ARCH = {
    "vits14": (384, 12, 6, "mlp"), "vitb14": (768, 12, 12, "mlp"), "vitl14": (1024, 24, 16, "mlp"),
    "vitg14": (1536, 40, 24, "swiglu"),
    # timm ViT-B/16 stand-in (no LayerScale, patch 16): block stack only, used through install_vit_blocks
    "vitb16_timm": (768, 12, 12, "mlp"),
}


def swiglu_hidden(d):
    """Hidden width of the DINOv2 SwiGLU FFN (fastbb/models/dinov2.py:52)."""
    return (int(4 * d * 2 / 3) + 7) // 8 * 8


# ------------------------------------------------------------------------------------------------ synthetic weights
def make_params(arch, seed=0, img_size=518, patch_size=14, num_register_tokens=0, layerscale=True, depth=None):
    """Seeded random-init parameters of the benchmark configs: weights, cls, pos-embed, patch-embed trunc-normal
    (std 0.02, cut at 2 sigma); biases 0; LayerNorm (1, 0); LayerScale gamma ~ U(0.05, 0.2)."""
    d, full_depth, heads, ffn = ARCH[arch]
    depth = full_depth if depth is None else depth
    g = torch.Generator().manual_seed(seed)

    def tn(*shape):
        t = torch.empty(*shape)
        torch.nn.init.trunc_normal_(t, std=0.02, a=-0.04, b=0.04, generator=g)
        return t

    p = {
        "patch_embed.proj.weight": tn(d, 3, patch_size, patch_size), "patch_embed.proj.bias": torch.zeros(d),
        "cls_token": tn(1, 1, d), "pos_embed": tn(1, (img_size // patch_size) ** 2 + 1, d), "mask_token": torch.zeros(1, d),
        "norm.weight": torch.ones(d), "norm.bias": torch.zeros(d),
    }
    if num_register_tokens:
        p["register_tokens"] = tn(1, num_register_tokens, d)
    for i in range(depth):
        b = f"blocks.{i}."
        for n in ("norm1", "norm2"):
            p[b + n + ".weight"], p[b + n + ".bias"] = torch.ones(d), torch.zeros(d)
        p[b + "attn.qkv.weight"], p[b + "attn.qkv.bias"] = tn(3 * d, d), torch.zeros(3 * d)
        p[b + "attn.proj.weight"], p[b + "attn.proj.bias"] = tn(d, d), torch.zeros(d)
        if layerscale:
            p[b + "ls1.gamma"] = torch.empty(d).uniform_(0.05, 0.2, generator=g)
            p[b + "ls2.gamma"] = torch.empty(d).uniform_(0.05, 0.2, generator=g)
        if ffn == "mlp":
            p[b + "mlp.fc1.weight"], p[b + "mlp.fc1.bias"] = tn(4 * d, d), torch.zeros(4 * d)
            p[b + "mlp.fc2.weight"], p[b + "mlp.fc2.bias"] = tn(d, 4 * d), torch.zeros(d)
        else:
            h = swiglu_hidden(d)
            p[b + "mlp.w12.weight"], p[b + "mlp.w12.bias"] = tn(2 * h, d), torch.zeros(2 * h)
            p[b + "mlp.w3.weight"], p[b + "mlp.w3.bias"] = tn(d, h), torch.zeros(d)
    return p


def make_image(batch, height, width, seed=1):
    """Seeded N(0,1) image batch [B, 3, H, W] of the benchmark configs."""
    return torch.randn(batch, 3, height, width, generator=torch.Generator().manual_seed(seed))


def depth_of(params):
    return 1 + max(int(k.split(".")[1]) for k in params if k.startswith("blocks."))


# ------------------------------------------------------------------------------------------------ operators
def layer_norm(x, w, b, eps=1e-6):
    """nn.LayerNorm over the last dim (call sites fastbb/vit.py:114,126,184; eps fastbb/models/dinov2.py:49,80)."""
    x = x.float()
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    y = (x - mu) / torch.sqrt(var + eps)
    if w is not None:
        y = y * w.float()
    if b is not None:
        y = y + b.float()
    return y


def gelu_erf(x):
    return 0.5 * x * (1.0 + torch.erf(x * (1.0 / math.sqrt(2.0))))


def silu(x):
    return x / (1.0 + torch.exp(-x))


def linear(x, w, b=None, act=None, res=None, gamma=None):
    """fastbb/gemm.py:18-24 `_ref` (bias -> act -> res + gamma*y, the epilogue order of fastbb_kernels.cu:418-427),
    plus act="swiglu": y = silu(x1) * x2 with x1, x2 = chunk(2) (fastbb/vit.py:139-141)."""
    y = x.float() @ w.float().t()
    if b is not None:
        y = y + b.float()
    if act == "gelu":
        y = gelu_erf(y)
    elif act == "swiglu":
        x1, x2 = y.chunk(2, dim=-1)
        y = silu(x1) * x2
    elif act not in (None, "none"):
        raise ValueError(f"unsupported activation: {act}")
    if res is not None:
        y = res.float() + (gamma.float() * y if gamma is not None else y)
    return y


def attention(q, k, v, scale=None):
    """softmax(scale * q k^T) v with q, k, v [B, N, H, D] -> [B, N, H, D] (fastbb/attention.py:31-60: no mask, default
    scale D**-0.5; fastbb_kernels.cu:58-299 computes the same in 64-key blocks with a running maximum)."""
    q, k, v = q.float(), k.float(), v.float()
    if scale is None:
        scale = q.shape[-1] ** -0.5
    s = torch.einsum("bnhd,bmhd->bhnm", q, k) * scale
    s = s - s.amax(-1, keepdim=True)
    p = torch.exp(s)
    p = p / p.sum(-1, keepdim=True)
    return torch.einsum("bhnm,bmhd->bnhd", p, v)


# ------------------------------------------------------------------------------------------------ block and stack
def block(params, i, x, heads):
    """One pre-LN block (fastbb/vit.py:108-143): x + g1*proj(attn(qkv(LN1 x))), then x + g2*mlp(LN2 x)."""
    p = lambda n: params.get(f"blocks.{i}.{n}")  # noqa: E731
    B, N, C = x.shape
    qkv = linear(layer_norm(x, p("norm1.weight"), p("norm1.bias")), p("attn.qkv.weight"), p("attn.qkv.bias"))
    q, k, v = qkv.view(B, N, 3, heads, C // heads).unbind(2)
    o = attention(q, k, v).reshape(B, N, C)
    x = linear(o, p("attn.proj.weight"), p("attn.proj.bias"), res=x, gamma=p("ls1.gamma"))
    y = layer_norm(x, p("norm2.weight"), p("norm2.bias"))
    if p("mlp.fc1.weight") is not None:
        h = linear(y, p("mlp.fc1.weight"), p("mlp.fc1.bias"), act="gelu")
        return linear(h, p("mlp.fc2.weight"), p("mlp.fc2.bias"), res=x, gamma=p("ls2.gamma"))
    h = linear(y, p("mlp.w12.weight"), p("mlp.w12.bias"), act="swiglu")
    return linear(h, p("mlp.w3.weight"), p("mlp.w3.bias"), res=x, gamma=p("ls2.gamma"))


def _cubic_weights(t, A=-0.75):
    """Keys cubic-convolution weights for taps at -1, 0, 1, 2 around floor(x) (bicubic, A = -0.75 as in aten)."""
    w0 = ((A * (t + 1) - 5 * A) * (t + 1) + 8 * A) * (t + 1) - 4 * A
    w1 = ((A + 2) * t - (A + 3)) * t * t + 1
    w2 = ((A + 2) * (1 - t) - (A + 3)) * (1 - t) * (1 - t) + 1
    w3 = ((A * (2 - t) - 5 * A) * (2 - t) + 8 * A) * (2 - t) - 4 * A
    return torch.stack([w0, w1, w2, w3], -1)


def _bicubic_axis(src, out_size, scale):
    """Resample the first axis of src [M, ...] to out_size with align_corners=False and an explicit scale factor
    (source coordinate (i + 0.5) / scale - 0.5, border taps clamped), no antialiasing."""
    M = src.shape[0]
    i = torch.arange(out_size, dtype=torch.float32)
    x = (i + 0.5) / scale - 0.5
    x0 = torch.floor(x)
    w = _cubic_weights(x - x0)                                       # [out, 4]
    idx = (x0.long()[:, None] + torch.arange(-1, 3)[None, :]).clamp(0, M - 1)  # [out, 4]
    g = src[idx]                                                      # [out, 4, ...]
    return (g * w.view(out_size, 4, *([1] * (src.dim() - 1)))).sum(1)


def pos_embed(params, h0, w0, interpolate_offset=0.1):
    """Position table for an h0 x w0 patch grid (fastbb/vit.py:78-95): identity when the grid matches the square
    table, else bicubic interpolation of the patch part in fp32 with the upstream `interpolate_offset` rule
    (scale factor (h0 + off) / M when off != 0, otherwise target size). Antialiased resampling (register-token
    checkpoints) is not restated here."""
    pe = params["pos_embed"].float()
    N = pe.shape[1] - 1
    M = int(math.sqrt(N))
    if N == h0 * w0 and h0 == w0:
        return pe
    grid = pe[0, 1:].reshape(M, M, -1)
    sh = (h0 + interpolate_offset) / M if interpolate_offset else h0 / M
    sw = (w0 + interpolate_offset) / M if interpolate_offset else w0 / M
    t = _bicubic_axis(grid, h0, sh)                       # [h0, M, C]
    t = _bicubic_axis(t.transpose(0, 1), w0, sw)          # [w0, h0, C]
    t = t.transpose(0, 1).reshape(1, h0 * w0, -1)
    return torch.cat([pe[:, :1], t], 1)


def tokens(params, x, patch_size=14, interpolate_offset=0.1):
    """Patch embedding (stride = kernel = patch conv as a matmul over unfolded patches), cls token, position
    embedding, register tokens after cls (fastbb/vit.py:97-105)."""
    B, _, H, W = x.shape
    ps = patch_size
    w = params["patch_embed.proj.weight"].float()
    d = w.shape[0]
    h0, w0 = H // ps, W // ps
    patches = x.float().reshape(B, 3, h0, ps, w0, ps).permute(0, 2, 4, 1, 3, 5).reshape(B, h0 * w0, 3 * ps * ps)
    t = patches @ w.reshape(d, -1).t() + params["patch_embed.proj.bias"].float()
    t = torch.cat([params["cls_token"].float().expand(B, -1, -1), t], 1)
    t = t + pos_embed(params, h0, w0, interpolate_offset)
    if "register_tokens" in params:
        t = torch.cat([t[:, :1], params["register_tokens"].float().expand(B, -1, -1), t[:, 1:]], 1)
    return t


def run(params, x, layers, heads, norm=True, patch_size=14, interpolate_offset=0.1):
    """Tokens after the blocks in `layers`, normed with the final LayerNorm if `norm` (fastbb/vit.py:175-187)."""
    out = []
    last = max(layers)
    t = tokens(params, x, patch_size, interpolate_offset)
    for i in range(depth_of(params)):
        t = block(params, i, t, heads)
        if i in layers:
            out.append(layer_norm(t, params["norm.weight"], params["norm.bias"]) if norm else t.clone())
        if i >= last:
            break
    return out


def get_intermediate_layers(params, x, n, heads, return_class_token=False, norm=True, patch_size=14, interpolate_offset=0.1):
    """fastbb/vit.py:220-235 without the reshape option: tuple of patch tokens (or (patch, cls) pairs)."""
    nb = depth_of(params)
    layers = list(range(nb - n, nb)) if isinstance(n, int) else list(n)
    nreg = params["register_tokens"].shape[1] if "register_tokens" in params else 0
    outs = run(params, x, set(layers), heads, norm, patch_size, interpolate_offset)
    cls = [o[:, 0] for o in outs]
    outs = [o[:, 1 + nreg:] for o in outs]
    return tuple(zip(outs, cls)) if return_class_token else tuple(outs)


def block_stack(params, x, heads):
    """All blocks applied to ready-made tokens x [B, N, C]: what install_vit_blocks accelerates (fastbb/vit.py:311-328)."""
    for i in range(depth_of(params)):
        x = block(params, i, x, heads)
    return x


def rel_l2(a, b):
    """Relative L2 error of a against the reference b: the reference's parity measure (README.md:12)."""
    a, b = a.detach().double(), b.detach().double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))
