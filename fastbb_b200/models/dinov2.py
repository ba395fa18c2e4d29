"""DINOv2 ViT-S/B/L/g (with or without 4 register tokens) as a standalone feature extractor on the B200 kernels.

    from fastbb_b200.models.dinov2 import dinov2
    m = dinov2("vitl14", "dinov2_vitl14_pretrain.pth", spec="hh-g1-graph")      # -> FastViT (fp16, CUDA)
    feats = m.get_intermediate_layers(img, n=[4, 11, 17, 23], reshape=True, return_class_token=True)
    out = m.forward_features(img)      # x_norm_clstoken, x_norm_regtokens, x_norm_patchtokens, x_prenorm

Counterpart of the reference's fastbb/models/dinov2.py: the module tree below only carries parameters under the
official names (strict state-dict match with the facebookresearch/dinov2 checkpoints); the forward pass is
fastbb_b200.vit.FastViT. `weights` may be a checkpoint path or an already loaded state dict.
"""
import torch
import torch.nn as nn

# name -> (embed_dim, depth, heads, ffn)
ARCH = {
    "vits14": (384, 12, 6, "mlp"),
    "vitb14": (768, 12, 12, "mlp"),
    "vitl14": (1024, 24, 16, "mlp"),
    "vitg14": (1536, 40, 24, "swiglu"),
}


def swiglu_hidden(d):
    """Hidden width of the DINOv2 SwiGLU FFN: 2/3 of 4d rounded up to a multiple of 8 (4096 for d = 1536)."""
    return (int(4 * d * 2 / 3) + 7) // 8 * 8


class _LayerScale(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.gamma = nn.Parameter(torch.empty(d))


class _Mlp(nn.Module):
    def __init__(self, d, hidden):
        super().__init__()
        self.fc1 = nn.Linear(d, hidden)
        self.fc2 = nn.Linear(hidden, d)


class _SwiGLU(nn.Module):
    def __init__(self, d, hidden):
        super().__init__()
        self.w12 = nn.Linear(d, 2 * hidden)
        self.w3 = nn.Linear(hidden, d)


class _Attention(nn.Module):
    def __init__(self, d, heads):
        super().__init__()
        self.num_heads = heads
        self.scale = (d // heads) ** -0.5
        self.qkv = nn.Linear(d, 3 * d)
        self.proj = nn.Linear(d, d)


class _Block(nn.Module):
    def __init__(self, d, heads, ffn):
        super().__init__()
        self.norm1 = nn.LayerNorm(d, eps=1e-6)
        self.attn = _Attention(d, heads)
        self.ls1 = _LayerScale(d)
        self.norm2 = nn.LayerNorm(d, eps=1e-6)
        self.mlp = _Mlp(d, 4 * d) if ffn == "mlp" else _SwiGLU(d, swiglu_hidden(d))
        self.ls2 = _LayerScale(d)


class _PatchEmbed(nn.Module):
    def __init__(self, d, patch):
        super().__init__()
        self.proj = nn.Conv2d(3, d, patch, patch)

    def forward(self, x):
        return self.proj(x).flatten(2).transpose(1, 2)


class DinoV2Params(nn.Module):
    """Parameter container with the official names: patch_embed.proj, cls_token, pos_embed, register_tokens, mask_token,
    blocks.N.{norm1, attn.qkv, attn.proj, ls1.gamma, norm2, mlp.*, ls2.gamma}, norm."""

    def __init__(self, arch, num_register_tokens=0, img_size=518, patch_size=14, depth=None):
        super().__init__()
        d, full_depth, heads, ffn = ARCH[arch]
        depth = full_depth if depth is None else depth  # truncated stacks are used by tests and benchmarks
        self.embed_dim, self.patch_size, self.num_register_tokens = d, patch_size, num_register_tokens
        # hub configuration of the register-token checkpoints: antialiased interpolation without the 0.1 offset
        self.interpolate_antialias = num_register_tokens > 0
        self.interpolate_offset = 0.0 if num_register_tokens else 0.1
        self.patch_embed = _PatchEmbed(d, patch_size)
        self.cls_token = nn.Parameter(torch.empty(1, 1, d))
        self.pos_embed = nn.Parameter(torch.empty(1, (img_size // patch_size) ** 2 + 1, d))
        self.register_tokens = nn.Parameter(torch.empty(1, num_register_tokens, d)) if num_register_tokens else None
        self.mask_token = nn.Parameter(torch.empty(1, d))
        self.blocks = nn.ModuleList([_Block(d, heads, ffn) for _ in range(depth)])
        self.norm = nn.LayerNorm(d, eps=1e-6)
        self.head = nn.Identity()


def from_state_dict(arch, sd, device="cuda", dtype=torch.float16):
    """Build DinoV2Params for `arch` on `device` holding `sd` (official names). Weights are cast to `dtype` on the CPU
    and assigned, so the device only ever holds the fp16 copy; pos_embed stays fp32 (it is interpolated in fp32)."""
    nreg = sd["register_tokens"].shape[1] if "register_tokens" in sd else 0
    side = int(round((sd["pos_embed"].shape[1] - 1) ** 0.5))
    patch = sd["patch_embed.proj.weight"].shape[-1]
    depth = 1 + max(int(k.split(".")[1]) for k in sd if k.startswith("blocks."))
    with torch.device("meta"):
        m = DinoV2Params(arch.replace("_reg", ""), num_register_tokens=nreg, img_size=side * patch, patch_size=patch, depth=depth)
    sd = {k: v.to(torch.float32 if k == "pos_embed" else dtype).to(device) for k, v in sd.items()}
    m.load_state_dict(sd, strict=True, assign=True)
    return m.eval()


def dinov2(arch, weights, spec=None, device="cuda", dtype=torch.float16, graphs=False):
    """DINOv2 `arch` (vits14 | vitb14 | vitl14 | vitg14; a '_reg' suffix or a checkpoint with register tokens -> 4
    registers) as a FastViT. `spec` as in fastbb_b200.install_vit, including the '-graph' suffix."""
    from .. import DEFAULT_VIT, parse_vit_spec, split_graph_suffix
    from ..vit import FastViT
    if isinstance(weights, (str, bytes)) or hasattr(weights, "__fspath__"):
        weights = torch.load(weights, map_location="cpu", weights_only=True, mmap=True)
    m = from_state_dict(arch, weights, device=device, dtype=dtype)
    spec, want_graph = split_graph_suffix(spec or DEFAULT_VIT)
    attn, gacc = parse_vit_spec(spec)
    return FastViT(m, attn=attn, gacc=gacc, dtype=dtype, graphs=graphs or want_graph)
