"""Generate the golden vectors under tests/golden/ by running the REFERENCE itself (its friendly fp32 CPU tier).

    python tests/golden/make_golden.py /path/to/reference [fixture ...]     (a checkout of fastforks/fastbb; or $FASTBB_REFERENCE)

Without fixture names every fixture is regenerated (the results are deterministic: same seeds, same bits); with names
(c0_vits14_224, c1_vitl14_896x1344, c3_vitg14_518, c3_vitg14_518_b4, c2_vitb16_blocks_1025, c2_vitb16_blocks_4097_b8, ops)
only those.

The reference is a Python package whose fp32 tier needs no GPU: FastViT(attn="sdpa", gacc=False, dtype=float32)
(fastbb/vit.py:42,108-150), install_vit_blocks(model, "sdpa-g0", convert=False) (fastbb/vit.py:311-328), gemm.linear
and attention.attention on CPU tensors (both take their torch branch there, fastbb/gemm.py:36-51,
fastbb/attention.py:44-48). Inputs are the seeded synthetic weights and images of oracle/vit_oracle.py, so a fixture
stores only the reference's OUTPUTS (subsampled where they are large) plus checksums of the inputs, which the tests use
to detect a change of the random generator. The reference cannot travel to the GPU machine; these files can.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import vit_oracle as O  # noqa: E402

# (fixture name, arch, image H, W, batch, layers, token stride of the stored subsample)
STACKS = [
    ("c0_vits14_224", "vits14", 224, 224, 1, [2, 5, 8, 11], 2),
    ("c1_vitl14_896x1344", "vitl14", 896, 1344, 1, [4, 11, 17, 23], 128),
    ("c3_vitg14_518", "vitg14", 518, 518, 1, [9, 19, 29, 39], 32),
    ("c3_vitg14_518_b4", "vitg14", 518, 518, 4, [9, 19, 29, 39], 64),   # the per-GPU share of batch 32 on eight GPUs
]
PARAM_SEED, IMAGE_SEED = 0, 1
OP_STRIDE = 4  # operator outputs are stored every 4th row / token


def checksum(t):
    return float(t.double().sum()), float(t.double().abs().sum())


def timm_like_stack(ref_dinov2, depth=12, d=768, heads=12):
    """Stand-in for timm's ViT-B/16 block stack: the attribute names fastbb/vit.py:273-294 checks, no LayerScale."""
    import torch.nn as nn

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.norm1, self.norm2 = nn.LayerNorm(d, eps=1e-6), nn.LayerNorm(d, eps=1e-6)
            self.attn = ref_dinov2._Attn(d, heads)
            self.ls1, self.ls2 = nn.Identity(), nn.Identity()
            self.mlp = ref_dinov2._Mlp(d, 4 * d)
            self.mlp.act = nn.GELU()

        def forward(self, x):
            raise RuntimeError("the original forward must not run in this fixture")

    class Stack(nn.Module):
        def __init__(self):
            super().__init__()
            self.blocks = nn.ModuleList([Block() for _ in range(depth)])

        def forward(self, x):
            for b in self.blocks:
                x = b(x)
            return x

    return Stack()


def main(ref_root, only=()):
    want = lambda name: not only or name in only  # noqa: E731
    sys.path.insert(0, ref_root)
    import fastbb  # the reference
    from fastbb import attention as ref_attention
    from fastbb import gemm as ref_gemm
    from fastbb.models import dinov2 as ref_dinov2
    from fastbb.vit import FastViT as RefFastViT

    torch.manual_seed(0)
    for name, arch, H, W, B, layers, stride in STACKS:
        if not want(name):
            continue
        params = O.make_params(arch, seed=PARAM_SEED)
        x = O.make_image(B, H, W, seed=IMAGE_SEED)
        m = ref_dinov2.DinoV2Params(arch)
        m.load_state_dict(params, strict=True)
        fv = RefFastViT(m, attn="sdpa", gacc=False, dtype=torch.float32)
        with torch.no_grad():
            outs = fv.get_intermediate_layers(x, n=layers, return_class_token=True)
        rec = {"layers": np.array(layers), "token_stride": np.array(stride),
               "image_checksum": np.array(checksum(x)),
               "qkv0_checksum": np.array(checksum(params["blocks.0.attn.qkv.weight"])),
               "gamma_checksum": np.array(checksum(params["blocks.0.ls1.gamma"]))}
        for i, (patch, cls) in zip(layers, outs):
            rec[f"patch_{i}"] = patch[:, ::stride].numpy().astype(np.float32)
            rec[f"cls_{i}"] = cls.numpy().astype(np.float32)
            rec[f"patch_norm_{i}"] = np.array(float(patch.double().norm()))
            if B > 1:
                rec[f"patch_norm_per_image_{i}"] = patch.double().flatten(1).norm(dim=1).numpy()
        np.savez(os.path.join(HERE, name + ".npz"), **rec)
        print(name, {k: getattr(v, "shape", None) for k, v in rec.items() if k.startswith("patch_") and "norm" not in k})

    # ---- c2: timm-style ViT-B/16 block stack through the reference's install_vit_blocks (fp32, no conversion)
    params = O.make_params("vitb16_timm", seed=PARAM_SEED, layerscale=False, patch_size=16, img_size=224)
    stack = timm_like_stack(ref_dinov2)
    sd = {k: v for k, v in params.items() if k.startswith("blocks.")}
    stack.load_state_dict(sd, strict=True)
    stack.eval()
    n = fastbb.install_vit_blocks(stack, "sdpa-g0", convert=False)
    assert n == 12, n
    if want("c2_vitb16_blocks_1025"):
        tokens = torch.randn(1, 1025, 768, generator=torch.Generator().manual_seed(IMAGE_SEED))  # 512x512 / 16 + cls
        with torch.no_grad():
            y = stack(tokens)
        np.savez(os.path.join(HERE, "c2_vitb16_blocks_1025.npz"), out=y[:, ::16].numpy().astype(np.float32),
                 out_norm=np.array(float(y.double().norm())), token_stride=np.array(16), tokens_checksum=np.array(checksum(tokens)))
        print("c2_vitb16_blocks_1025", tuple(y.shape))
    if want("c2_vitb16_blocks_4097_b8"):
        # the configuration as stated: 1024x1024 / 16 + cls = 4097 tokens, batch 8 (batch 1 = its first image)
        tokens = torch.randn(8, 4097, 768, generator=torch.Generator().manual_seed(IMAGE_SEED))
        with torch.no_grad():
            y = torch.cat([stack(tokens[i:i + 1]) for i in range(8)])
        np.savez(os.path.join(HERE, "c2_vitb16_blocks_4097_b8.npz"), out=y[:, ::128].numpy().astype(np.float32),
                 out_norm_per_image=y.double().flatten(1).norm(dim=1).numpy(), token_stride=np.array(128),
                 tokens_checksum=np.array(checksum(tokens)))
        print("c2_vitb16_blocks_4097_b8", tuple(y.shape))
    if not want("ops"):
        return

    # ---- operators: the reference's gemm.linear and attention.attention on CPU tensors
    g = torch.Generator().manual_seed(7)
    rec = {"op_stride": np.array(OP_STRIDE)}
    for tag, (M, N, K, act, has_res) in {"plain": (257, 1152, 384, None, False), "gelu": (257, 1536, 384, "gelu", False),
                                          "res": (257, 384, 1536, None, True), "odd": (63, 200, 72, "gelu", True)}.items():
        xx, ww = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g) * 0.05
        bb = torch.randn(N, generator=g) * 0.1
        res = torch.randn(M, N, generator=g) if has_res else None
        gam = torch.rand(N, generator=g) * 0.15 + 0.05 if has_res else None
        with torch.no_grad():
            yy = ref_gemm.linear(xx, ww, bb, act=act, res=res, gamma=gam)
        rec[f"linear_{tag}_out"] = yy[::OP_STRIDE].numpy()
        rec[f"linear_{tag}_in_checksum"] = np.array(checksum(xx) + checksum(ww))
    for N, H in ((257, 6), (400, 16)):
        q, k, v = (torch.randn(1, N, H, 64, generator=g) for _ in range(3))
        with torch.no_grad():
            o = ref_attention.attention(q, k, v, scale=0.125)
        rec[f"attention_{N}_out"] = o[:, ::OP_STRIDE].numpy()
        rec[f"attention_{N}_in_checksum"] = np.array(checksum(q) + checksum(v))
    # position-embedding interpolation of the reference (bicubic with the 0.1 offset rule), 37x37 table -> 64x96 grid
    params = O.make_params("vits14", seed=PARAM_SEED)
    m = ref_dinov2.DinoV2Params("vits14")
    m.load_state_dict(params, strict=True)
    pe = RefFastViT(m, attn="sdpa", gacc=False, dtype=torch.float32).pos_embed(64, 96)
    rec["pos_embed_64x96"] = pe[:, ::16].detach().numpy()
    np.savez(os.path.join(HERE, "ops.npz"), **rec)
    print("ops", sorted(rec))


if __name__ == "__main__":
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FASTBB_REFERENCE")
    if not ref:
        sys.exit("usage: make_golden.py /path/to/reference  (a checkout of fastforks/fastbb)")
    main(ref, tuple(sys.argv[2:]))
