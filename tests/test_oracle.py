"""The CPU oracle against the reference's own outputs (tests/golden/*.npz, made by tests/golden/make_golden.py by running
the reference's fp32 tier) and against naive float64 restatements. Tolerances are fp32 round-off: the oracle and the
reference compute the same formulas with different summation orders."""
import os

import numpy as np
import pytest
import torch

from conftest import assert_same_inputs, load_golden

FP32_TOL = 2e-5


def _stack_case(oracle, name, arch, H, W, heads):
    g = load_golden(name)
    params = oracle.make_params(arch, seed=0)
    x = oracle.make_image(1, H, W, seed=1)
    assert_same_inputs(g["image_checksum"], x, "image")
    assert_same_inputs(g["qkv0_checksum"], params["blocks.0.attn.qkv.weight"], "qkv weight")
    assert_same_inputs(g["gamma_checksum"], params["blocks.0.ls1.gamma"], "LayerScale gamma")
    layers = [int(i) for i in g["layers"]]
    stride = int(g["token_stride"])
    outs = oracle.get_intermediate_layers(params, x, layers, heads, return_class_token=True)
    for i, (patch, cls) in zip(layers, outs):
        assert oracle.rel_l2(patch[:, ::stride], torch.from_numpy(g[f"patch_{i}"])) < FP32_TOL, f"{name} layer {i} patch"
        assert oracle.rel_l2(cls, torch.from_numpy(g[f"cls_{i}"])) < FP32_TOL, f"{name} layer {i} cls"
        assert abs(float(patch.double().norm()) / float(g[f"patch_norm_{i}"]) - 1) < 1e-5


def test_stack_c0_vits14_224(oracle):
    _stack_case(oracle, "c0_vits14_224", "vits14", 224, 224, 6)


def test_stack_c1_vitl14_896x1344(oracle):
    _stack_case(oracle, "c1_vitl14_896x1344", "vitl14", 896, 1344, 16)


def test_stack_c3_vitg14_518_swiglu(oracle):
    _stack_case(oracle, "c3_vitg14_518", "vitg14", 518, 518, 24)


def test_block_stack_c2_timm_like(oracle):
    g = load_golden("c2_vitb16_blocks_1025")
    params = oracle.make_params("vitb16_timm", seed=0, layerscale=False, patch_size=16, img_size=224)
    tokens = torch.randn(1, 1025, 768, generator=torch.Generator().manual_seed(1))
    assert_same_inputs(g["tokens_checksum"], tokens, "tokens")
    y = oracle.block_stack(params, tokens, 12)
    assert oracle.rel_l2(y[:, ::int(g["token_stride"])], torch.from_numpy(g["out"])) < FP32_TOL
    assert abs(float(y.double().norm()) / float(g["out_norm"]) - 1) < 1e-5


def test_block_stack_c2_at_4097_tokens_one_image_of_the_batch_fixture(oracle):
    """The full-size c2 fixture (4097 tokens, batch 8) also pins the oracle: image 5 of the batch, run on its own."""
    g = load_golden("c2_vitb16_blocks_4097_b8")
    params = oracle.make_params("vitb16_timm", seed=0, layerscale=False, patch_size=16, img_size=224)
    tokens = torch.randn(8, 4097, 768, generator=torch.Generator().manual_seed(1))
    assert_same_inputs(g["tokens_checksum"], tokens, "tokens")
    y = oracle.block_stack(params, tokens[5:6], 12)
    assert oracle.rel_l2(y[:, ::int(g["token_stride"])], torch.from_numpy(g["out"][5:6])) < FP32_TOL
    assert abs(float(y.double().norm()) / float(g["out_norm_per_image"][5]) - 1) < 1e-5


def test_stack_c3_batch4_fixture_one_image(oracle):
    """The batch-4 c3 fixture against the oracle on image 2 of the batch (the images of a batch are independent)."""
    g = load_golden("c3_vitg14_518_b4")
    params = oracle.make_params("vitg14", seed=0)
    x = oracle.make_image(4, 518, 518, seed=1)
    assert_same_inputs(g["image_checksum"], x, "image")
    layers = [int(i) for i in g["layers"]]
    stride = int(g["token_stride"])
    outs = oracle.get_intermediate_layers(params, x[2:3], layers, 24, return_class_token=True)
    for i, (patch, cls) in zip(layers, outs):
        assert oracle.rel_l2(patch[:, ::stride], torch.from_numpy(g[f"patch_{i}"][2:3])) < FP32_TOL
        assert oracle.rel_l2(cls, torch.from_numpy(g[f"cls_{i}"][2:3])) < FP32_TOL
        assert abs(float(patch.double().norm()) / float(g[f"patch_norm_per_image_{i}"][2]) - 1) < 1e-5


def _op_inputs():
    """Same generator sequence as make_golden.py."""
    g = torch.Generator().manual_seed(7)
    lin = {}
    for tag, (M, N, K, act, has_res) in {"plain": (257, 1152, 384, None, False), "gelu": (257, 1536, 384, "gelu", False),
                                          "res": (257, 384, 1536, None, True), "odd": (63, 200, 72, "gelu", True)}.items():
        x, w = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g) * 0.05
        b = torch.randn(N, generator=g) * 0.1
        res = torch.randn(M, N, generator=g) if has_res else None
        gam = torch.rand(N, generator=g) * 0.15 + 0.05 if has_res else None
        lin[tag] = (x, w, b, act, res, gam)
    att = {}
    for N, H in ((257, 6), (400, 16)):
        att[N] = tuple(torch.randn(1, N, H, 64, generator=g) for _ in range(3))
    return lin, att


def test_operators_against_reference_outputs(oracle):
    g = load_golden("ops")
    s = int(g["op_stride"])
    lin, att = _op_inputs()
    for tag, (x, w, b, act, res, gam) in lin.items():
        assert np.allclose(g[f"linear_{tag}_in_checksum"], (*_cs(x), *_cs(w)), rtol=1e-9), "generator drift"
        y = oracle.linear(x, w, b, act=act, res=res, gamma=gam)
        assert oracle.rel_l2(y[::s], torch.from_numpy(g[f"linear_{tag}_out"])) < FP32_TOL, tag
    for N, (q, k, v) in att.items():
        assert np.allclose(g[f"attention_{N}_in_checksum"], (*_cs(q), *_cs(v)), rtol=1e-9), "generator drift"
        o = oracle.attention(q, k, v, scale=0.125)
        assert oracle.rel_l2(o[:, ::s], torch.from_numpy(g[f"attention_{N}_out"])) < FP32_TOL, N


def _cs(t):
    return float(t.double().sum()), float(t.double().abs().sum())


def test_pos_embed_bicubic_against_reference(oracle):
    g = load_golden("ops")
    params = oracle.make_params("vits14", seed=0)
    pe = oracle.pos_embed(params, 64, 96)
    assert pe.shape == (1, 64 * 96 + 1, 384)
    assert oracle.rel_l2(pe[:, ::16], torch.from_numpy(g["pos_embed_64x96"])) < FP32_TOL
    # identity when the grid equals the table
    assert torch.equal(oracle.pos_embed(params, 37, 37), params["pos_embed"])


# ---------------------------------------------------------------- naive float64 cross-checks (independent of torch kernels)
def test_layer_norm_naive():
    from oracle import vit_oracle as O
    rng = np.random.default_rng(0)
    x = rng.standard_normal((5, 24)) * 3 + 1
    w, b = rng.standard_normal(24), rng.standard_normal(24)
    want = np.empty_like(x)
    for r in range(5):
        mu = sum(x[r]) / 24
        var = sum((x[r] - mu) ** 2) / 24
        want[r] = (x[r] - mu) / np.sqrt(var + 1e-6) * w + b
    got = O.layer_norm(torch.tensor(x, dtype=torch.float32), torch.tensor(w, dtype=torch.float32), torch.tensor(b, dtype=torch.float32))
    assert np.allclose(got.numpy(), want, atol=1e-5)


def test_attention_naive():
    from oracle import vit_oracle as O
    rng = np.random.default_rng(1)
    B, N, H, D = 1, 7, 2, 64
    q, k, v = (rng.standard_normal((B, N, H, D)) for _ in range(3))
    want = np.zeros((B, N, H, D))
    for h in range(H):
        for i in range(N):
            s = np.array([q[0, i, h] @ k[0, j, h] for j in range(N)]) * 0.125
            p = np.exp(s - s.max())
            p /= p.sum()
            want[0, i, h] = sum(p[j] * v[0, j, h] for j in range(N))
    got = O.attention(*(torch.tensor(t, dtype=torch.float32) for t in (q, k, v)))
    assert np.allclose(got.numpy(), want, atol=1e-5)


def test_linear_epilogue_order_naive():
    from oracle import vit_oracle as O
    import math
    rng = np.random.default_rng(2)
    x, w, b = rng.standard_normal((3, 8)), rng.standard_normal((4, 8)), rng.standard_normal(4)
    res, gam = rng.standard_normal((3, 4)), rng.random(4)
    want = np.empty((3, 4))
    for i in range(3):
        for j in range(4):
            v = x[i] @ w[j] + b[j]
            v = 0.5 * v * (1 + math.erf(v / math.sqrt(2)))
            want[i, j] = res[i, j] + gam[j] * v
    t = lambda a: torch.tensor(a, dtype=torch.float32)  # noqa: E731
    got = O.linear(t(x), t(w), t(b), act="gelu", res=t(res), gamma=t(gam))
    assert np.allclose(got.numpy(), want, atol=1e-5)
    # swiglu: silu(x1) * x2 over the two halves of the output
    y = x @ w.T + b
    want2 = (y[:, :2] / (1 + np.exp(-y[:, :2]))) * y[:, 2:]
    assert np.allclose(O.linear(t(x), t(w), t(b), act="swiglu").numpy(), want2, atol=1e-5)
    with pytest.raises(ValueError):
        O.linear(t(x), t(w), act="relu")


def test_reference_package_and_its_gpu_kernels_build_into_oracle_ref():
    """oracle/make_ref.py where a checkout (or an earlier install) of the reference is at hand: the package lands in
    oracle/_ref and its kernel file compiles for sm_100 under the very file name the reference's loader looks for
    (sha1 of the source + architecture, fastbb/kernels.py:84-87), so the GPU machine needs no compiler run."""
    import hashlib
    import shutil
    from oracle import make_ref
    dest = make_ref.make()
    if dest is None:
        pytest.skip("no reference checkout and no oracle/_ref here")
    assert make_ref.available()
    if shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"):
        pytest.skip("no nvcc")
    out = make_ref.make_kernels()
    src = os.path.join(dest, "fastbb", "fastbb_kernels.cu")
    tag = hashlib.sha1(open(src, "rb").read() + b"sm_100").hexdigest()[:16]
    assert out == os.path.join(dest, "fastbb", "prebuilt", f"fastbb_kernels_{tag}.cubin") and os.path.getsize(out) > 100_000
