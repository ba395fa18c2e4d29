"""Host-side logic of FastViT / install_vit / install_vit_blocks on CPU. The kernels cannot run here, so the block
function is replaced by an fp32 stand-in built on the oracle: these tests check orchestration (layer selection, cls /
register split, reshape, out_dtype, caches, patching rules), not numerics."""
import pytest
import torch
import torch.nn as nn

import fastbb_b200 as fb
from fastbb_b200 import vit as fvit
from fastbb_b200.models.dinov2 import ARCH, DinoV2Params, from_state_dict, swiglu_hidden


def test_vit_position_cache_reloads_weights():
    # same scenario as the reference's only ViT test (tests/test_fastbb.py:75-86)
    vit = nn.Module()
    vit.pos_embed = nn.Parameter(torch.zeros(1, 5, 8))
    vit.patch_size = 2
    vit.blocks = nn.ModuleList()
    fast = fvit.FastViT(vit, attn="sdpa", gacc=False)
    assert torch.equal(fast.pos_embed(2, 2), torch.zeros(1, 5, 8, dtype=torch.float16))
    vit.load_state_dict({"pos_embed": torch.ones(1, 5, 8)})
    assert torch.equal(fast.pos_embed(2, 2), torch.ones(1, 5, 8, dtype=torch.float16))


def test_pos_embed_interpolation_matches_oracle(oracle):
    params = oracle.make_params("vits14", seed=0)
    m = from_state_dict("vits14", params, device="cpu")
    fast = fvit.FastViT(m, attn="fh", gacc=False)
    got = fast.pos_embed(16, 24).float()
    want = oracle.pos_embed(params, 16, 24)
    assert got.shape == (1, 16 * 24 + 1, 384)
    assert oracle.rel_l2(got, want) < 1e-3  # fp16 rounding of the cached table
    assert fast.pos_embed(16, 24) is fast.pos_embed(16, 24)  # cached per grid


def _oracle_block(oracle, params_by_block):
    def run_block(block, x, attn_variant, gacc):
        i = params_by_block[id(block)]
        return oracle.block(params_by_block["params"], i, x.float(), block.attn.num_heads).to(x.dtype)
    return run_block


def _build(oracle, monkeypatch, depth=4, nreg=0):
    params = oracle.make_params("vits14", seed=0, depth=depth, num_register_tokens=nreg)
    with torch.device("meta"):
        m = DinoV2Params("vits14", num_register_tokens=nreg)
    m.blocks = nn.ModuleList(list(m.blocks)[:depth])
    m.load_state_dict({k: v.clone() for k, v in params.items()}, strict=True, assign=True)
    fast = fvit.FastViT(m.eval(), attn="fh", gacc=False)
    index = {id(b): i for i, b in enumerate(fast.blocks)}
    index["params"] = params
    monkeypatch.setattr(fvit, "run_block", _oracle_block(oracle, index))
    monkeypatch.setattr(fvit, "_norm", lambda mod, x: torch.nn.functional.layer_norm(x.float(), mod.normalized_shape, mod.weight.float(), mod.bias.float(), mod.eps).to(x.dtype))
    return params, m, fast


def test_get_intermediate_layers_contract(oracle, monkeypatch):
    params, m, fast = _build(oracle, monkeypatch)
    x = oracle.make_image(2, 56, 70, seed=3)
    outs = fast.get_intermediate_layers(x, n=[1, 3], return_class_token=True)
    want = oracle.get_intermediate_layers(params, x, [1, 3], 6, return_class_token=True)
    assert len(outs) == 2
    for (p, c), (wp, wc) in zip(outs, want):
        assert p.shape == (2, 4 * 5, 384) and c.shape == (2, 384) and p.dtype == torch.float16
        assert oracle.rel_l2(p.float(), wp) < 5e-3 and oracle.rel_l2(c.float(), wc) < 5e-3
    # n as an int = last n blocks; reshape gives [B, C, h, w]; out_dtype casts
    last2 = fast.get_intermediate_layers(x, n=2, reshape=True)
    assert [t.shape for t in last2] == [(2, 384, 4, 5)] * 2 and last2[0].is_contiguous()
    fast.out_dtype = torch.float32
    assert fast.get_intermediate_layers(x, n=1)[0].dtype == torch.float32
    fast.out_dtype = None
    # norm=False returns the raw residual stream
    raw = fast.get_intermediate_layers(x, n=[3], norm=False)[0]
    want_raw = oracle.get_intermediate_layers(params, x, [3], 6, norm=False)[0]
    assert oracle.rel_l2(raw.float(), want_raw) < 5e-3
    # the caller's input is not modified and the module was cast in place
    assert x.dtype == torch.float32 and m.blocks[0].attn.qkv.weight.dtype == torch.float16


def test_forward_features_and_registers(oracle, monkeypatch):
    params, m, fast = _build(oracle, monkeypatch, depth=2, nreg=4)
    assert fast.nreg == 4 and m.interpolate_antialias and m.interpolate_offset == 0.0
    x = oracle.make_image(1, 42, 42, seed=4)
    ff = fast.forward_features(x)
    assert set(ff) == {"x_norm_clstoken", "x_norm_regtokens", "x_norm_patchtokens", "x_prenorm", "masks"}
    assert ff["x_norm_regtokens"].shape == (1, 4, 384) and ff["x_norm_patchtokens"].shape == (1, 9, 384)
    assert ff["x_prenorm"].shape == (1, 1 + 4 + 9, 384) and ff["masks"] is None
    assert torch.equal(fast(x), ff["x_norm_clstoken"])
    # patch tokens exclude cls and registers
    assert fast.get_intermediate_layers(x, n=1)[0].shape == (1, 9, 384)


def test_install_routes_the_instance_attribute(oracle, monkeypatch):
    params, m, fast = _build(oracle, monkeypatch, depth=1)
    assert fast.install() is fast
    assert m.__dict__["get_intermediate_layers"] == fast.get_intermediate_layers and m._fastbb is fast


def test_block_flattening_handles_chunks_and_identity():
    class BlockChunk(nn.ModuleList):
        pass
    a, b, c = nn.Linear(1, 1), nn.Linear(1, 1), nn.Linear(1, 1)
    blocks = nn.ModuleList([BlockChunk([nn.Identity(), a]), nn.ModuleList([b]), c])
    assert fvit._flatten_blocks(blocks) == [a, b, c]


def test_fastvit_rejects_other_dtypes_and_modes():
    vit = nn.Module()
    vit.pos_embed = nn.Parameter(torch.zeros(1, 5, 8))
    vit.patch_size = (2, 2)
    vit.blocks = nn.ModuleList()
    with pytest.raises(ValueError):
        fvit.FastViT(vit, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        fvit.FastViT(vit, gacc="bogus")
    assert fvit.FastViT(vit).ps == 2


# ---------------------------------------------------------------- install_vit_blocks
class TimmLikeBlock(nn.Module):
    """The attributes timm's Block exposes (what the structural test reads), no LayerScale."""

    def __init__(self, d=128, heads=2):
        super().__init__()
        self.norm1, self.norm2 = nn.LayerNorm(d, eps=1e-6), nn.LayerNorm(d, eps=1e-6)
        self.attn = nn.Module()
        self.attn.num_heads, self.attn.qkv, self.attn.proj = heads, nn.Linear(d, 3 * d), nn.Linear(d, d)
        self.attn.q_norm, self.attn.k_norm = nn.Identity(), nn.Identity()
        self.ls1, self.ls2, self.drop_path1, self.drop_path2 = nn.Identity(), nn.Identity(), nn.Identity(), nn.Identity()
        self.mlp = nn.Module()
        self.mlp.fc1, self.mlp.act, self.mlp.fc2, self.mlp.norm = nn.Linear(d, 4 * d), nn.GELU(), nn.Linear(4 * d, d), nn.Identity()
        self.calls = 0

    def forward(self, x, attn_mask=None):
        self.calls += 1
        return x


def test_block_supported_rules():
    ok = TimmLikeBlock()
    assert fvit._block_supported(ok)
    b = TimmLikeBlock(); b.attn.q_norm = nn.LayerNorm(64); assert not fvit._block_supported(b)
    b = TimmLikeBlock(); b.attn.rope = object(); assert not fvit._block_supported(b)
    b = TimmLikeBlock(); b.attn.gate = nn.Linear(1, 1); assert not fvit._block_supported(b)
    b = TimmLikeBlock(); b.attn.qkv_bias_separate = True; assert not fvit._block_supported(b)
    b = TimmLikeBlock(); b.mlp.norm = nn.LayerNorm(512); assert not fvit._block_supported(b)
    b = TimmLikeBlock(d=96, heads=2); assert not fvit._block_supported(b)      # head_dim 48: no kernel, so not patched
    b = TimmLikeBlock(); b.ls1 = nn.Linear(1, 1); assert not fvit._block_supported(b)
    b = TimmLikeBlock(); del b.mlp.fc1; assert not fvit._block_supported(b)
    b = TimmLikeBlock(); del b.mlp.fc1; b.mlp.w12, b.mlp.w3 = nn.Linear(128, 512), nn.Linear(256, 128); assert fvit._block_supported(b)
    assert not fvit._block_supported(nn.Linear(2, 2))


def test_install_vit_blocks_patches_once_and_keeps_fallbacks(monkeypatch):
    model = nn.Sequential(TimmLikeBlock(), TimmLikeBlock(), nn.Linear(128, 128))
    assert fb.install_vit_blocks(model, "fh-g1", convert=True) == 2
    assert fb.install_vit_blocks(model, "fh-g1") == 0                      # idempotent
    assert model[0].attn.qkv.weight.dtype == torch.float16
    cfg = model[0]._fbb_cfg
    assert (cfg.attn, cfg.gacc) == ("fh", True)
    seen = []
    monkeypatch.setattr(fvit, "run_block", lambda blk, x, a, g: (seen.append((x.dtype, a, g)), x + 1)[1])
    model.eval()
    x = torch.zeros(1, 3, 128)                                             # fp32 caller
    y = model[0](x)
    assert y.dtype == torch.float32 and torch.all(y == 1) and seen == [(torch.float16, "fh", True)]
    # masks, attention biases, causal attention and training mode use the original forward
    assert model[0](x, attn_mask=torch.ones(1)) is x and model[0].calls == 1
    model[0].train()
    assert model[0](x) is x and model[0].calls == 2
    assert len(seen) == 1


def test_arch_table_and_swiglu_width():
    assert ARCH["vitl14"] == (1024, 24, 16, "mlp") and ARCH["vitg14"] == (1536, 40, 24, "swiglu")
    assert swiglu_hidden(1536) == 4096
    with torch.device("meta"):
        g = DinoV2Params("vitg14")
    assert g.blocks[0].mlp.w12.weight.shape == (8192, 1536) and g.blocks[0].mlp.w3.weight.shape == (1536, 4096)
    assert g.pos_embed.shape == (1, 37 * 37 + 1, 1536)


def test_synthetic_generator_matches_the_oracles(oracle):
    """The package ships its own seeded generator for benchmarks; it must make the tensors the golden fixtures assume."""
    from fastbb_b200 import synthetic
    a, b = synthetic.make_params("vits14", seed=0, depth=2), oracle.make_params("vits14", seed=0, depth=2)
    assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a)
    a, b = synthetic.make_params("vitg14", seed=3, depth=1, num_register_tokens=4), oracle.make_params("vitg14", seed=3, depth=1, num_register_tokens=4)
    assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a)
    assert torch.equal(synthetic.make_image(2, 28, 42, seed=5), oracle.make_image(2, 28, 42, seed=5))


def test_block_descriptor_cache_does_not_keep_the_block_alive(monkeypatch):
    """The C runner's per-block descriptor cache is a weak-keyed table: an entry follows the block (same object while the
    block is unchanged, re-read after a change) and goes away with it - neither the block nor its weights may be held by
    the cache. (The descriptor fill itself needs CUDA tensors and is replaced here.)"""
    import gc
    import weakref
    monkeypatch.setattr(fvit, "_fill_block_desc", lambda d, block, attn, gacc: None)

    class Attn(nn.Module):
        def __init__(self):
            super().__init__()
            self.num_heads, self.qkv, self.proj = 2, nn.Linear(128, 384), nn.Linear(128, 128)

    class Mlp(nn.Module):
        def __init__(self):
            super().__init__()
            self.fc1, self.act, self.fc2 = nn.Linear(128, 512), nn.GELU(), nn.Linear(512, 128)

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.norm1, self.norm2, self.attn, self.mlp = nn.LayerNorm(128), nn.LayerNorm(128), Attn(), Mlp()
            self.ls1, self.ls2 = nn.Identity(), nn.Identity()

    b = Block()
    e = fvit._block_entry(b, "fh", False)
    assert fvit._block_entry(b, "fh", False) is e and e.valid(b, "fh", False)
    b.norm1.eps = 1e-3
    assert not e.valid(b, "fh", False) and fvit._block_entry(b, "fh", False) is not e
    b.mlp.fc2 = nn.Linear(512, 128)
    assert not fvit._DESCS[b].valid(b, "fh", False)
    rb, rw = weakref.ref(b), weakref.ref(b.attn.qkv.weight)
    del b, e
    gc.collect()
    assert rb() is None and rw() is None
