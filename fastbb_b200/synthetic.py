"""Seeded synthetic weights and images for benchmarks and demos (no checkpoint or dataset is needed to run the path).

The benchmark configurations use random-init models: weights, cls token, position table and patch embedding
trunc-normal (std 0.02, cut at two sigma), biases 0, LayerNorm (1, 0), LayerScale gamma ~ U(0.05, 0.2); images N(0,1).
State dicts use the official DINOv2 parameter names, so they load into models.dinov2.DinoV2Params and into the
reference's own container alike.
"""
import torch

from .models.dinov2 import ARCH, swiglu_hidden


def make_params(arch, seed=0, img_size=518, patch_size=14, num_register_tokens=0, layerscale=True, depth=None):
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
    return torch.randn(batch, 3, height, width, generator=torch.Generator().manual_seed(seed))
