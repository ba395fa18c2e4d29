"""Parity of the three CUDA operators, called through the C ABI (ctypes), against the CPU oracle on seeded inputs,
against the reference's own outputs (tests/golden/ops.npz), and through size-independent properties at the benchmark's
full sizes. Outputs sit inside canary-padded buffers so a write outside the logical tensor is caught.

Tolerances (relative L2 against the fp32 oracle evaluated on the same fp16-rounded inputs): one fp16 rounding of the
output is 2.1e-4 rms; fp32-accumulate paths must stay below 1e-3, fp16-accumulate paths below 1e-2 (the reference's
own criterion for its fastest tier, README.md:12)."""
import numpy as np
import pytest
import torch

from conftest import load_golden

pytestmark = pytest.mark.gpu

TOL_F32, TOL_F16 = 1e-3, 1e-2
CANARY = 1234.0


def dev():
    return torch.device("cuda:0")


def padded(shape, pad=64):
    """A contiguous [rows, cols] view in the middle of a canary-filled buffer; returns (view, check())."""
    rows, cols = int(np.prod(shape[:-1])), shape[-1]
    buf = torch.full((rows * cols + 2 * pad,), CANARY, dtype=torch.float16, device=dev())
    view = buf[pad:pad + rows * cols].view(*shape)

    def check():
        assert torch.all(buf[:pad] == CANARY) and torch.all(buf[pad + rows * cols:] == CANARY), "kernel wrote outside its output"
    return view, check


def status_ok():
    from fastbb_b200 import _lib
    assert _lib.device_status() == (0, 0, 0, 0)


# ------------------------------------------------------------------------------------------------ LayerNorm
@pytest.mark.parametrize("M,C,dtype", [(1, 384, torch.float16), (257, 384, torch.float16), (6145, 1024, torch.float16),
                                       (1370, 1536, torch.float32), (33, 4096, torch.bfloat16), (5, 8, torch.float16),
                                       (129, 2048, torch.float16), (64, 768, torch.float32)])
def test_layernorm_matches_oracle(oracle, M, C, dtype):
    from fastbb_b200.layernorm import layer_norm
    g = torch.Generator().manual_seed(M * 131 + C)
    x = (torch.randn(M, C, generator=g) * 2 + 0.5).to(dtype)
    w, b = (1 + 0.1 * torch.randn(C, generator=g)).half(), (0.1 * torch.randn(C, generator=g)).half()
    out, check = padded((M, C), pad=max(64, 16 - (M * C) % 8))
    y = layer_norm(x.to(dev()), w.to(dev()), b.to(dev()), 1e-6, out=out)
    want = oracle.layer_norm(x, w, b, 1e-6)
    assert oracle.rel_l2(y.cpu().float(), want) < TOL_F32
    check()
    status_ok()


def test_layernorm_large_mean_and_no_affine(oracle):
    from fastbb_b200.layernorm import layer_norm
    x = (torch.randn(64, 1024, generator=torch.Generator().manual_seed(3)) + 300.0).half()  # mean >> std: no E[x^2]-E[x]^2
    y = layer_norm(x.to(dev()), None, None, 1e-6)
    assert oracle.rel_l2(y.cpu().float(), oracle.layer_norm(x, None, None, 1e-6)) < 2e-3
    # idempotence without affine: normalising a normalised row changes nothing beyond fp16 rounding
    assert oracle.rel_l2(layer_norm(y, None, None, 1e-6).cpu().float(), y.cpu().float()) < 1e-3


def test_layernorm_strided_rows_and_errors(oracle):
    from fastbb_b200 import _lib
    from fastbb_b200.layernorm import layer_norm
    base = torch.randn(40, 512, generator=torch.Generator().manual_seed(4)).half().to(dev())
    x = base[:, :384]                                           # row stride 512, C = 384
    y = layer_norm(x, None, None, 1e-6)
    assert oracle.rel_l2(y.cpu().float(), oracle.layer_norm(x.cpu(), None, None, 1e-6)) < TOL_F32
    with pytest.raises(_lib.FastbbError):
        layer_norm(torch.zeros(4, 12, dtype=torch.float16, device=dev()))      # C % 8 != 0
    assert layer_norm(torch.zeros(0, 64, dtype=torch.float16, device=dev())).shape == (0, 64)


@pytest.mark.parametrize("norm", [True, False])
@pytest.mark.parametrize("B,N,C,n_prefix,grid", [(2, 257, 384, 1, (16, 16)), (1, 6145, 1024, 1, (64, 96)), (2, 105, 384, 5, (10, 10)),
                                                 (3, 1370, 1536, 1, (37, 37)), (1, 40, 2048, 3, (1, 37)), (2, 2, 64, 1, (1, 1))])
def test_layernorm_split_matches_oracle_in_both_layouts(oracle, B, N, C, n_prefix, grid, norm):
    """The final norm with split outputs: cls rows, register rows and patch rows (token-major, and channel-major =
    [B, C, h, w]) against the oracle's LayerNorm of the same rows; the channel-major tensor is the token-major one
    transposed, bit for bit, and both equal the plain LayerNorm kernel's output (bit for bit where that kernel uses the
    same arithmetic)."""
    from fastbb_b200.layernorm import layer_norm, layer_norm_split
    g = torch.Generator().manual_seed(B * 7 + N + C)
    x = (torch.randn(B, N, C, generator=g) * 1.5 + 0.3).half()
    w, b = (1 + 0.1 * torch.randn(C, generator=g)).half(), (0.1 * torch.randn(C, generator=g)).half()
    xd, wd, bd = x.to(dev()), w.to(dev()), b.to(dev())
    p_tok, cls, regs = layer_norm_split(xd, wd, bd, 1e-6, n_prefix=n_prefix, norm=norm)
    p_chw, cls2, regs2 = layer_norm_split(xd, wd, bd, 1e-6, n_prefix=n_prefix, grid=grid, norm=norm)
    want = oracle.layer_norm(x, w, b, 1e-6) if norm else x.float()
    assert p_tok.shape == (B, N - n_prefix, C) and p_chw.shape == (B, C, *grid) and p_chw.is_contiguous()
    assert oracle.rel_l2(p_tok.cpu().float(), want[:, n_prefix:]) < TOL_F32
    assert oracle.rel_l2(cls.cpu().float(), want[:, 0]) < TOL_F32
    assert torch.equal(p_chw.flatten(2).transpose(1, 2), p_tok) and torch.equal(cls, cls2)
    if n_prefix > 1:
        assert regs.shape == (B, n_prefix - 1, C) and torch.equal(regs, regs2)
        assert oracle.rel_l2(regs.cpu().float(), want[:, 1:n_prefix]) < TOL_F32
    else:
        assert regs is None
    full = layer_norm(xd, wd, bd, 1e-6) if norm else xd
    if C <= 1536:  # rows this short take the two-rows-per-warp kernel, whose arithmetic the split kernel repeats exactly
        assert torch.equal(p_tok, full[:, n_prefix:]) and torch.equal(cls, full[:, 0])
    else:
        assert oracle.rel_l2(p_tok.float(), full[:, n_prefix:].float()) < 3e-4
    status_ok()


def test_layernorm_split_rejects_what_it_does_not_cover():
    from fastbb_b200 import _lib
    from fastbb_b200.layernorm import layer_norm_split
    x = torch.zeros(1, 50, 64, dtype=torch.float16, device=dev())
    with pytest.raises(ValueError):
        layer_norm_split(x, grid=(7, 8))                      # 56 != 49 patch tokens
    with pytest.raises(_lib.FastbbError):
        layer_norm_split(x, n_prefix=40)                      # more prefix rows than the kernel's one prefix tile holds
    with pytest.raises(ValueError):
        layer_norm_split(x.float())
    assert layer_norm_split(x[:0])[0].shape == (0, 49, 64)


# ------------------------------------------------------------------------------------------------ linear
LINEAR_CASES = [
    # M, N, K, act, bias, res, variant
    (128, 256, 64, None, False, False, "f32"),
    (1, 1024, 1024, None, True, False, "f32"),
    (63, 200, 72, "gelu", True, True, "f32"),
    (64, 8, 8, None, False, False, "f32"),
    (65, 136, 40, None, True, True, "c2"),
    (127, 128, 1024, "gelu", True, False, "f32"),
    (129, 264, 96, None, True, True, "f32"),
    (257, 1152, 384, None, True, False, "f32"),
    (257, 384, 1536, None, True, True, "f32"),
    (400, 3072, 768, "gelu", True, False, "c4"),
    (1370, 1536, 1536, None, True, True, "f32"),
    (257, 1536, 384, "gelu", True, False, "h"),
    (1370, 4608, 1536, None, True, False, "h"),
    (300, 272, 64, "swiglu", True, False, "f32"),
    (1370, 8192, 1536, "swiglu", True, False, "f32"),
    (1370, 8192, 1536, "swiglu", True, False, "h"),
]


@pytest.mark.parametrize("M,N,K,act,has_bias,has_res,variant", LINEAR_CASES)
def test_linear_matches_oracle(oracle, M, N, K, act, has_bias, has_res, variant):
    from fastbb_b200.gemm import linear
    g = torch.Generator().manual_seed(M * 7 + N * 3 + K)
    x = torch.randn(M, K, generator=g).half()
    w = (torch.randn(N, K, generator=g) / K ** 0.5).half()
    b = (0.1 * torch.randn(N, generator=g)).half() if has_bias else None
    n_out = N // 2 if act == "swiglu" else N
    res = torch.randn(M, n_out, generator=g).half() if has_res else None
    gam = (0.05 + 0.15 * torch.rand(n_out, generator=g)).half() if has_res else None
    out, check = padded((M, n_out))
    d = lambda t: None if t is None else t.to(dev())  # noqa: E731
    y = linear(d(x), d(w), d(b), act=act, res=d(res), gamma=d(gam), variant=variant, out=out)
    want = oracle.linear(x, w, b, act=act, res=res, gamma=gam)
    assert y.shape == (M, n_out)
    assert oracle.rel_l2(y.cpu().float(), want) < (TOL_F16 if variant == "h" else TOL_F32)
    check()
    status_ok()


@pytest.mark.parametrize("form", ["s256", "s128", "p256", "p128", "w32", "w96", "w256", "w288", "w352", "w512"])
def test_linear_every_tile_form_matches_oracle(oracle, form, monkeypatch):
    """The kernel has several forms (one CTA or a CTA pair per tile, 256- or 128-column tiles; wide pair items of 32 to
    512 columns over two accumulators, with the rows beyond the last full 256-row tile computed by the epilogue warps)
    and picks one by a cost model; this forces each of them on tail-heavy shapes, including the SwiGLU (which never
    takes the wide form and falls through to the default choice) and fp16-accumulate epilogues."""
    from fastbb_b200 import _lib
    from fastbb_b200.gemm import linear
    monkeypatch.setenv("FBB_GEMM_FORCE", form)
    if form[0] == "p" and _lib.load().fbb_linear_max_cta_pairs(256) == 0:
        pytest.skip("this device cannot co-schedule CTA pairs")
    g = torch.Generator().manual_seed(99)
    for M, N, K, act, variant in [(513, 1160, 200, "gelu", "f32"), (257, 384, 1536, None, "f32"), (1370, 1024, 264, "swiglu", "f32"),
                                  (300, 520, 72, None, "h"), (1, 256, 64, None, "f32"), (264, 200, 136, "gelu", "h"), (776, 72, 64, None, "f32"), (1032, 528, 72, "swiglu", "f32")]:
        x = torch.randn(M, K, generator=g).half()
        w = (torch.randn(N, K, generator=g) / K ** 0.5).half()
        b = (0.1 * torch.randn(N, generator=g)).half()
        n_out = N // 2 if act == "swiglu" else N
        res = torch.randn(M, n_out, generator=g).half() if act is None else None
        gam = (0.05 + 0.15 * torch.rand(n_out, generator=g)).half() if act is None else None
        out, check = padded((M, n_out))
        d = lambda t: None if t is None else t.to(dev())  # noqa: E731
        y = linear(d(x), d(w), d(b), act=act, res=d(res), gamma=d(gam), variant=variant, out=out)
        want = oracle.linear(x, w, b, act=act, res=res, gamma=gam)
        assert oracle.rel_l2(y.cpu().float(), want) < (TOL_F16 if variant == "h" else TOL_F32), (form, M, N, K, act)
        check()
    status_ok()


@pytest.mark.parametrize("M,N,K,act,variant", [(2561, 2000, 136, "gelu", "f32"), (2561, 1848, 72, None, "h"), (6145, 1024, 64, None, "f32"),
                                                (2600, 2048, 200, None, "f32")])
def test_linear_last_wave_in_slices_equals_whole_tiles(oracle, M, N, K, act, variant, monkeypatch):
    """The persistent 256-column form cuts the tiles of a partly filled second wave into 128- or 64-column slices (168
    to 196 tiles on 148 SMs here, with ragged last rows and columns, and slices that lie wholly beyond N). Each width, and the rule's own choice, must give the oracle's result and, element for element, the bits
    of the launch without slices (every output element sees the same K loop)."""
    from fastbb_b200.gemm import linear
    monkeypatch.setenv("FBB_GEMM_FORCE", "s256")
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).half()
    w = (torch.randn(N, K, generator=g) / K ** 0.5).half()
    b = (0.1 * torch.randn(N, generator=g)).half()
    res = torch.randn(M, N, generator=g).half() if act is None else None
    gam = (0.05 + 0.15 * torch.rand(N, generator=g)).half() if act is None else None
    want = oracle.linear(x, w, b, act=act, res=res, gamma=gam)
    d = lambda t: None if t is None else t.to(dev())  # noqa: E731
    xd, wd, bd, rd, gd = d(x), d(w), d(b), d(res), d(gam)
    outs = {}
    for width in ["0", "64", "128", None]:
        if width is None:
            monkeypatch.delenv("FBB_GEMM_NARROW", raising=False)
        else:
            monkeypatch.setenv("FBB_GEMM_NARROW", width)
        out, check = padded((M, N))
        outs[width] = linear(xd, wd, bd, act=act, res=rd, gamma=gd, variant=variant, out=out).clone()
        check()
        assert oracle.rel_l2(outs[width].cpu().float(), want) < (TOL_F16 if variant == "h" else TOL_F32), width
    for width in ["64", "128", None]:
        assert torch.equal(outs[width], outs["0"]), width
    status_ok()


def test_linear_against_reference_outputs(oracle):
    """Same seeded inputs as tests/golden/make_golden.py; the stored outputs come from the reference's gemm.linear."""
    from fastbb_b200.gemm import linear
    from test_oracle import _op_inputs
    g = load_golden("ops")
    s = int(g["op_stride"])
    lin, _ = _op_inputs()
    d = lambda t: None if t is None else t.half().to(dev())  # noqa: E731
    for tag, (x, w, b, act, res, gam) in lin.items():
        y = linear(d(x), d(w), d(b), act=act, res=d(res), gamma=d(gam), variant="f32")
        # inputs were rounded to fp16 for the kernel: 2e-3 covers that rounding on K <= 1536 dot products
        assert oracle.rel_l2(y.cpu().float()[::s], torch.from_numpy(g[f"linear_{tag}_out"])) < 2e-3, tag


def test_linear_residual_without_gamma_batched_input_and_aliasing(oracle):
    from fastbb_b200.gemm import linear
    g = torch.Generator().manual_seed(11)
    x = torch.randn(2, 130, 256, generator=g).half()
    w = (torch.randn(256, 256, generator=g) / 16).half()
    res = torch.randn(2, 130, 256, generator=g).half()
    want = oracle.linear(x, w, None, res=res)
    xd, wd, rd = x.to(dev()), w.to(dev()), res.to(dev())
    y = linear(xd, wd, None, res=rd)
    assert y.shape == (2, 130, 256) and y.data_ptr() != rd.data_ptr()
    assert oracle.rel_l2(y.cpu().float(), want) < TOL_F32
    assert torch.equal(rd.cpu(), res)                       # res untouched: a new tensor is returned
    y2 = linear(xd, wd, None, res=rd, out=rd)               # in place on the residual stream is allowed
    assert y2.data_ptr() == rd.data_ptr() and torch.equal(y2, y)


def test_linear_large_magnitude_and_fp16_overflow_to_inf(oracle):
    from fastbb_b200.gemm import linear
    x = torch.full((128, 64), 60.0).half()
    w = torch.full((8, 64), 20.0).half()                    # 64 * 1200 = 76800 > fp16 max: fp32 accumulate, inf on store
    y = linear(x.to(dev()), w.to(dev())).cpu()
    assert torch.isinf(y).all()
    w2 = torch.full((8, 64), 10.0).half()                   # 38400 fits
    y2 = linear(x.to(dev()), w2.to(dev())).cpu().float()
    assert torch.allclose(y2, torch.full_like(y2, 38400.0), rtol=1e-3)


def test_linear_rejects_what_the_kernel_does_not_cover():
    from fastbb_b200 import _lib
    from fastbb_b200.gemm import linear
    x = torch.zeros(8, 12, dtype=torch.float16, device=dev())
    with pytest.raises(_lib.FastbbError):
        linear(x, torch.zeros(16, 12, dtype=torch.float16, device=dev()))              # K % 8
    x = torch.zeros(8, 16, dtype=torch.float16, device=dev())
    with pytest.raises(ValueError):
        linear(x, torch.zeros(16, 16, dtype=torch.float32, device=dev()))
    with pytest.raises(ValueError):
        linear(x, torch.zeros(16, 16, dtype=torch.float16, device=dev()), out=torch.zeros(8, 8, dtype=torch.float16, device=dev()))
    with pytest.raises(ValueError):
        linear(x, torch.zeros(16, 16, dtype=torch.float16, device=dev()), gamma=torch.zeros(16, dtype=torch.float16, device=dev()))


@pytest.mark.parametrize("M,N,K", [(6145, 3072, 1024), (6145, 4096, 1024), (6145, 1024, 4096), (32768, 1024, 1024)])
def test_linear_full_size_linearity_and_column_sums(M, N, K):
    """Benchmark-size GEMMs, checked without an M*N*K CPU product: (a) y(x1 + x2) = y(x1) + y(x2) - y(0) (the bias
    cancels), (b) the sum over output columns equals x . (sum of W rows) + sum(bias), a matrix-vector product the CPU
    does in milliseconds."""
    from fastbb_b200.gemm import linear
    g = torch.Generator(device="cuda").manual_seed(M + N)
    x1 = torch.randn(M, K, device=dev(), generator=g).half()
    x2 = torch.randn(M, K, device=dev(), generator=g).half()
    w = (torch.randn(N, K, device=dev(), generator=g) * 0.02).half()
    b = (torch.randn(N, device=dev(), generator=g) * 0.1).half()
    y1, y2 = linear(x1, w, b, variant="f32").float(), linear(x2, w, b, variant="f32").float()
    xs = (x1.float() + x2.float()).half()
    exact = xs.float() == x1.float() + x2.float()           # rows where the fp16 sum is exact
    y12 = linear(xs, w, b, variant="f32").float()
    rows = exact.all(dim=1)
    assert rows.sum() >= 0
    diff = (y12 - (y1 + y2 - b.float()))
    assert diff.norm() / y12.norm() < 5e-3
    colsum = y1.double().sum(dim=1).cpu()
    want = (x1.cpu().double() @ w.cpu().double().sum(dim=0)) + b.cpu().double().sum()
    assert ((colsum - want).norm() / want.norm()) < 2e-3
    status_ok()


LINEAR_LN_CASES = [
    # M, N, K, act, variant
    (6145, 1024, 1024, None, "f32"), (6145, 1024, 4096, None, "h"), (4097, 768, 768, None, "f32"), (5480, 1536, 1536, None, "f32"),
    (257, 384, 384, None, "f32"), (1370, 1024, 1024, None, "f32"), (520, 384, 1536, "gelu", "f32"), (300, 200, 64, None, "f32"),
    (2056, 2048, 256, None, "f32"), (1, 64, 64, None, "f32"),
]


@pytest.mark.parametrize("M,N,K,act,variant", LINEAR_LN_CASES)
def test_linear_layer_norm_matches_oracle(oracle, M, N, K, act, variant, monkeypatch):
    """GEMM with the LayerScale + residual epilogue followed by the LayerNorm of its output rows, as one call: the GEMM
    output against the oracle, the normalised rows against the oracle's LayerNorm of the fp16 output (what the separate
    kernel would read), the one-launch form against the two-launch form, and the counter left at zero. Shapes cover the
    fused form with one to four column chunks per row tile, remainder rows (M = 256 k + 1, + 8), and shapes that cannot
    fuse (N not a multiple of 32, too many row tiles)."""
    from fastbb_b200 import _lib
    from fastbb_b200.attention import _counter
    from fastbb_b200.gemm import linear_layer_norm
    monkeypatch.setenv("FBB_LN_FUSION", "1")                    # the one-launch form is off by default (it measured slower)
    g = torch.Generator().manual_seed(M + 3 * N + K)
    x = torch.randn(M, K, generator=g).half()
    w = (torch.randn(N, K, generator=g) / K ** 0.5).half()
    b = (0.1 * torch.randn(N, generator=g)).half()
    res = (torch.randn(M, N, generator=g) + 0.5).half()
    gam = (0.05 + 0.15 * torch.rand(N, generator=g)).half()
    lw, lb = (1 + 0.1 * torch.randn(N, generator=g)).half(), (0.1 * torch.randn(N, generator=g)).half()
    d = lambda t: t.to(dev())  # noqa: E731
    out, y = linear_layer_norm(d(x), d(w), d(b), act=act, res=d(res), gamma=d(gam), variant=variant, ln_weight=d(lw), ln_bias=d(lb), eps=1e-6)
    want = oracle.linear(x, w, b, act=act, res=res, gamma=gam)
    tol = TOL_F16 if variant == "h" else TOL_F32
    assert oracle.rel_l2(out.cpu().float(), want) < tol
    assert oracle.rel_l2(y.cpu().float(), oracle.layer_norm(out.cpu(), lw, lb, 1e-6)) < TOL_F32   # LayerNorm of the fp16 rows the call wrote
    assert int(_counter(dev())[0]) == 0
    fused = _lib.load().fbb_linear_layernorm_launches(M, N, 1 if act == "gelu" else 0, 1) == 1
    assert fused == (N % 32 == 0 and N <= 2048 and M < 74 * 256)
    out_b, y_b = linear_layer_norm(d(x), d(w), d(b), act=act, res=d(res), gamma=d(gam), variant=variant, ln_weight=d(lw), ln_bias=d(lb), eps=1e-6)
    assert torch.equal(out_b, out) and torch.equal(y_b, y)      # again, same counter: identical
    monkeypatch.setenv("FBB_GEMM_FORCE", "s256")                # a forced tile form also selects the two-launch path
    out2, y2 = linear_layer_norm(d(x), d(w), d(b), act=act, res=d(res), gamma=d(gam), variant=variant, ln_weight=d(lw), ln_bias=d(lb), eps=1e-6)
    assert oracle.rel_l2(out2.cpu().float(), out.cpu().float()) < 3e-4 and oracle.rel_l2(y2.cpu().float(), y.cpu().float()) < 1e-3
    status_ok()


@pytest.mark.parametrize("fusion", ["1", "0"])
def test_linear_layer_norm_in_place_large_mean_and_no_affine(oracle, fusion, monkeypatch):
    """In place on the residual stream (out is res), rows whose mean dwarfs their spread (the statistics are merged
    chunk by chunk from two-pass partials, not taken from E[x^2] - E[x]^2), no LayerNorm parameters."""
    from fastbb_b200.gemm import linear_layer_norm
    monkeypatch.setenv("FBB_LN_FUSION", fusion)
    g = torch.Generator().manual_seed(8)
    M, N, K = 1281, 1024, 256
    x = torch.randn(M, K, generator=g).half()
    w = (torch.randn(N, K, generator=g) / 16).half()
    res = (torch.randn(M, N, generator=g) + 300.0).half()
    rd = res.to(dev())
    out, y = linear_layer_norm(x.to(dev()), w.to(dev()), None, res=rd, ln_weight=None, ln_bias=None, eps=1e-6, out=rd)
    assert out.data_ptr() == rd.data_ptr()
    want = oracle.linear(x, w, None, res=res)
    assert oracle.rel_l2(out.cpu().float(), want) < TOL_F32
    assert oracle.rel_l2(y.cpu().float(), oracle.layer_norm(out.cpu(), None, None, 1e-6)) < 2e-3
    status_ok()


def _sample_rows(M, tile=128, n_random=24, seed=0):
    """First and last rows, both sides of a few tile boundaries, the ragged last tile, and some seeded random rows."""
    rows = {0, 1, tile - 1, tile, 2 * tile - 1, 2 * tile, M // 2, M - 1, M - 2, (M - 1) // tile * tile, (M - 1) // tile * tile - 1,
            (M - 1) // (2 * tile) * (2 * tile), (M - 1) // (2 * tile) * (2 * tile) - 1}
    g = torch.Generator().manual_seed(seed)
    rows |= set(int(i) for i in torch.randint(0, M, (n_random,), generator=g))
    return sorted(r for r in rows if 0 <= r < M)


@pytest.mark.parametrize("variant", ["f32", "h"])
@pytest.mark.parametrize("M", [6145, 32768])
@pytest.mark.parametrize("K,N,act,has_res", [(1024, 3072, None, False), (1024, 1024, None, True), (1024, 4096, "gelu", False),
                                             (4096, 1024, None, True), (1024, 4096, "swiglu", False)])
def test_linear_full_size_sampled_rows_match_oracle(oracle, M, K, N, act, has_res, variant):
    """Benchmark-size GEMMs against the oracle on a sample of output rows (every column of each): real values, not only
    invariants, at the sizes where the tile forms, tail waves and the remainder rows differ from the small cases."""
    from fastbb_b200.gemm import linear
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    x = torch.randn(M, K, device=dev(), generator=g).half()
    w = (torch.randn(N, K, device=dev(), generator=g) * 0.02).half()
    b = (torch.randn(N, device=dev(), generator=g) * 0.1).half()
    n_out = N // 2 if act == "swiglu" else N
    res = torch.randn(M, n_out, device=dev(), generator=g).half() if has_res else None
    gam = (0.05 + 0.15 * torch.rand(n_out, device=dev(), generator=g)).half() if has_res else None
    out, check = padded((M, n_out))
    y = linear(x, w, b, act=act, res=res, gamma=gam, variant=variant, out=out)
    rows = _sample_rows(M, seed=N)
    want = oracle.linear(x[rows].cpu(), w.cpu(), b.cpu(), act=act, res=None if res is None else res[rows].cpu(),
                         gamma=None if gam is None else gam.cpu())
    assert oracle.rel_l2(y[rows].cpu().float(), want) < (TOL_F16 if variant == "h" else TOL_F32)
    check()
    status_ok()


# ------------------------------------------------------------------------------------------------ flash attention
FLASH_SHAPES = [(1, 1, 1), (1, 63, 2), (1, 64, 2), (1, 65, 1), (1, 127, 3), (1, 128, 1), (1, 129, 2), (1, 257, 6), (2, 400, 16),
                (1, 1370, 16), (3, 255, 5)]


@pytest.mark.parametrize("variant", ["ff", "fh", "hh"])
@pytest.mark.parametrize("B,N,H", FLASH_SHAPES)
def test_flash_matches_oracle(oracle, variant, B, N, H):
    from fastbb_b200.attention import attention
    g = torch.Generator().manual_seed(B * 1000 + N * 10 + H)
    qkv = torch.randn(B, N, 3, H, 64, generator=g).half()
    qd, kd, vd = qkv.to(dev()).unbind(2)                     # strided views of the packed buffer, as in the block
    out, check = padded((B, N, H, 64))
    o = attention(qd, kd, vd, scale=0.125, variant=variant, out=out)
    q, k, v = qkv.unbind(2)
    want = oracle.attention(q, k, v, scale=0.125)
    assert oracle.rel_l2(o.cpu().float(), want) < TOL_F32   # every variant accumulates in fp32 on this part
    assert not torch.isnan(o).any()
    check()
    status_ok()


def test_flash_against_reference_outputs(oracle):
    from fastbb_b200.attention import attention
    from test_oracle import _op_inputs
    g = load_golden("ops")
    s = int(g["op_stride"])
    _, att = _op_inputs()
    for N, (q, k, v) in att.items():
        o = attention(*(t.half().to(dev()) for t in (q, k, v)), scale=0.125, variant="ff")
        assert oracle.rel_l2(o.cpu().float()[:, ::s], torch.from_numpy(g[f"attention_{N}_out"])) < 2e-3, N


@pytest.mark.parametrize("variant", ["ff", "fh", "hh"])
def test_flash_peaked_rows_default_scale_and_bhnd_layout(oracle, variant):
    from fastbb_b200.attention import attention_bhnd
    g = torch.Generator().manual_seed(5)
    q, k = (3 * torch.randn(1, 4, 300, 64, generator=g)).half(), (3 * torch.randn(1, 4, 300, 64, generator=g)).half()
    v = torch.randn(1, 4, 300, 64, generator=g).half()
    o = attention_bhnd(q.to(dev()), k.to(dev()), v.to(dev()), variant=variant)
    want = oracle.attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2)
    assert o.shape == (1, 4, 300, 64)
    assert oracle.rel_l2(o.cpu().float(), want) < 2e-3


@pytest.mark.parametrize("variant", ["ff", "fh", "hh"])
@pytest.mark.parametrize("N", [4097, 6145, 16385])
def test_flash_full_size_properties(variant, N):
    """Benchmark-size sequences without an N^2 CPU softmax: (a) rows of P sum to one, so V = const gives O = const;
    (b) permuting the keys (with their values) leaves O unchanged; (c) with identical keys, O is the mean of V."""
    from fastbb_b200.attention import attention
    H = 16
    g = torch.Generator(device="cuda").manual_seed(N)
    q = torch.randn(1, N, H, 64, device=dev(), generator=g).half()
    k = torch.randn(1, N, H, 64, device=dev(), generator=g).half()
    v = torch.randn(1, N, H, 64, device=dev(), generator=g).half()
    ones = torch.full_like(v, 0.5)
    o = attention(q, k, ones, scale=0.125, variant=variant).float()
    assert (o - 0.5).abs().max() < 1.5e-3
    perm = torch.randperm(N, device=dev(), generator=g)
    o1 = attention(q, k, v, scale=0.125, variant=variant).float()
    o2 = attention(q, k[:, perm], v[:, perm], scale=0.125, variant=variant).float()
    assert (o1 - o2).norm() / o1.norm() < 2e-3
    same_k = k[:, :1].expand(1, N, H, 64).contiguous()
    o3 = attention(q, same_k, v, scale=0.125, variant=variant).float()
    mean_v = v.float().mean(dim=1, keepdim=True)
    assert (o3 - mean_v).abs().max() < 5e-3
    status_ok()


@pytest.mark.parametrize("variant", ["ff", "fh", "hh"])
@pytest.mark.parametrize("B,N,H", [(1, 4097, 16), (1, 6145, 16), (1, 16385, 16), (8, 4097, 12), (4, 1370, 24)])
def test_flash_full_size_sampled_rows_match_oracle(oracle, variant, B, N, H):
    """Benchmark-size sequences against the oracle on a sample of query rows against ALL keys (first and last rows, tile
    boundaries, the ragged last tile, random rows): pins real values where the invariants above would let a
    permutation-invariant, row-sum-preserving error through."""
    from fastbb_b200.attention import attention
    g = torch.Generator(device="cuda").manual_seed(N + H)
    qkv = torch.randn(B, N, 3, H, 64, device=dev(), generator=g).half()
    q, k, v = qkv.unbind(2)
    out, check = padded((B, N, H, 64))
    o = attention(q, k, v, scale=0.125, variant=variant, out=out)
    rows = _sample_rows(N, seed=H)
    want = oracle.attention(q[:, rows].cpu(), k.cpu(), v.cpu(), scale=0.125)
    assert oracle.rel_l2(o[:, rows].cpu().float(), want) < TOL_F32
    check()
    status_ok()


@pytest.mark.parametrize("variant", ["ff", "hh"])
@pytest.mark.parametrize("B,N,H", [(2, 2500, 11), (1, 4097, 12), (20, 300, 16), (1, 6145, 16), (5, 1370, 16)])
def test_flash_split_form_matches_one_cta_per_group(oracle, variant, B, N, H):
    """More query-tile groups than SMs and not a multiple of them: the persistent form splits some groups' keys over two
    CTAs and merges them through the workspace. It must agree with the plain form (one CTA per group) up to rounding,
    with the oracle where that is cheap, leave the workspace's flags cleared, and give the same answer when called again."""
    from fastbb_b200 import _lib
    from fastbb_b200.attention import attention
    need = _lib.load().fbb_flash64_workspace_bytes(B, N, H)
    if need == 0:
        pytest.skip("this device's SM count divides the number of tile groups: nothing is split")
    g = torch.Generator().manual_seed(B * 1000 + N * 10 + H)
    qkv = torch.randn(B, N, 3, H, 64, generator=g).half()
    qd, kd, vd = qkv.to(dev()).unbind(2)
    ws = torch.zeros(need + 64, dtype=torch.uint8, device=dev())
    plain = attention(qd, kd, vd, scale=0.125, variant=variant, workspace=False)
    out, check = padded((B, N, H, 64))
    split = attention(qd, kd, vd, scale=0.125, variant=variant, out=out, workspace=ws)
    torch.cuda.synchronize()
    sms = torch.cuda.get_device_properties(dev()).multi_processor_count
    assert int(ws[:68 * sms].count_nonzero()) == 0                        # the flag words and row counters (68 bytes per SM) are clear again
    assert oracle.rel_l2(split.float().cpu(), plain.float().cpu()) < 3e-4
    check()
    again = attention(qd, kd, vd, scale=0.125, variant=variant, workspace=ws)
    assert torch.equal(again, split)
    default = attention(qd, kd, vd, scale=0.125, variant=variant)      # the module's own per-stream workspace
    assert torch.equal(default, split)
    if B * H * N * N <= 2 * 11 * 2500 * 2500:
        q, k, v = qkv.unbind(2)
        assert oracle.rel_l2(split.cpu().float(), oracle.attention(q, k, v, scale=0.125)) < TOL_F32
    with pytest.raises(_lib.FastbbError):                                # a workspace that is too small is rejected, not ignored
        _lib.check(_lib.load().fbb_flash64_f16_ws(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), out.data_ptr(), B, N, H,
                                                  *qd.stride()[:3], *kd.stride()[:3], *vd.stride()[:3], *out.stride()[:3],
                                                  0.125, 0, ws.data_ptr(), 1024, None))
    status_ok()


@pytest.mark.parametrize("B,N,H,side", [(1, 6145, 16, True), (1, 4097, 12, True), (1, 3329, 16, True), (1, 6146, 8, True),
                                         (1, 32776, 2, True), (1, 2561, 16, False), (1, 6149, 16, False), (1, 6153, 16, False),
                                         (10, 513, 16, False), (2, 1281, 32, False)])
def test_flash_leftover_rows_by_the_side_launch(oracle, B, N, H, side):
    """A few query rows beyond the last full 256-row group (cls token, registers) are computed by a second, small launch
    on the CUDA cores instead of a tile group per head - when a workspace is lent, they are at most 8 per head and 18
    in all, the sequence has at least 3072 tokens, and the rest still fills the SMs with two-tile CTAs in a persistent form. Those rows must match the oracle and the tiled
    path, every other row must be what the tiled path gives, and the row counters must be zero again afterwards."""
    from fastbb_b200 import _lib
    from fastbb_b200.attention import attention
    lib = _lib.load()
    sms = torch.cuda.get_device_properties(dev()).multi_processor_count
    if sms != 148:
        pytest.skip("the shapes of this test are chosen for 148 SMs")
    assert lib.fbb_flash64_launches(B, N, H, 1) == (2 if side else 1) and lib.fbb_flash64_launches(B, N, H, 0) == 1
    need = lib.fbb_flash64_workspace_bytes(B, N, H)
    assert need > 0 or not side
    g = torch.Generator().manual_seed(B * 1000 + N * 10 + H)
    qkv = torch.randn(B, N, 3, H, 64, generator=g).half()
    qkv[:, -3:, 0] *= 3.0                                                   # peaked rows among the leftover ones
    qd, kd, vd = qkv.to(dev()).unbind(2)
    ws = torch.zeros(max(need, 16) + 64, dtype=torch.uint8, device=dev())
    tiled = attention(qd, kd, vd, scale=0.125, variant="fh", workspace=False)
    out, check = padded((B, N, H, 64))
    before = _lib.LAUNCHES
    got = attention(qd, kd, vd, scale=0.125, variant="fh", out=out, workspace=ws if need > 0 else None)
    assert _lib.LAUNCHES - before == (2 if side else 1)
    torch.cuda.synchronize()
    check()
    assert int(ws[:68 * sms].count_nonzero()) == 0
    r = N % 256
    rows = list(range(N - max(r, 1) - 2, N))
    q, k, v = qkv.unbind(2)
    want = oracle.attention(q[:, rows], k, v, scale=0.125)
    assert oracle.rel_l2(got[:, rows].cpu().float(), want) < TOL_F32
    assert oracle.rel_l2(got.cpu().float(), tiled.cpu().float()) < 3e-4
    assert (got[:, rows].float() - tiled[:, rows].float()).abs().max() < 2e-3
    again = attention(qd, kd, vd, scale=0.125, variant="fh", workspace=ws if need > 0 else None)
    assert torch.equal(again, got)
    status_ok()


def test_flash_rejects_what_the_kernel_does_not_cover():
    from fastbb_b200.attention import attention
    q = torch.zeros(1, 8, 2, 32, dtype=torch.float16, device=dev())
    with pytest.raises(ValueError):
        attention(q, q, q)                                   # head_dim 32
    q = torch.zeros(1, 8, 2, 64, dtype=torch.float16, device=dev())
    with pytest.raises(ValueError):
        attention(q, q, q, scale=0.0)
    with pytest.raises(ValueError):
        attention(q, q, q, variant="xx")
    with pytest.raises(ValueError):
        attention(q.float(), q.float(), q.float())
    assert attention(q[:, :0], q[:, :0], q[:, :0]).shape == (1, 0, 2, 64)


def test_a_wait_that_runs_out_is_reported_and_leaves_the_device_usable(oracle):
    """Every pipeline wait in the kernels is bounded: when one runs out, the kernel records a code in the device status
    word and returns. fbb_diag_wait_timeout runs exactly that wait (same function, a 1 ms limit) on a barrier nothing
    arrives on; the kernel gives up and returns normally, fbb_device_status reports FBB_ERR_DEVICE_WAIT with the code and
    detail, clears the word, and the next kernels run clean. Nothing faults, traps or spins past the limit."""
    import ctypes
    from fastbb_b200 import _lib
    from fastbb_b200.layernorm import layer_norm
    lib = _lib.load()
    assert _lib.device_status() == (0, 0, 0, 0)             # a clean device reports zeros
    _lib.check(lib.fbb_diag_wait_timeout(1_000_000, 77, _lib.stream_ptr(dev())))
    out = (ctypes.c_uint * 4)()
    rc = lib.fbb_device_status(ctypes.byref(out))
    assert rc == -6 and tuple(out) == (5, 77, 0, 1)          # FBB_ERR_DEVICE_WAIT: other wait, detail, block 0, one report
    assert b"device wait ran out" in lib.fbb_last_error()
    with pytest.raises(_lib.FastbbError):
        _lib.check(lib.fbb_diag_wait_timeout(1_000_000, 78, _lib.stream_ptr(dev())))
        _lib.device_status()                                 # the Python wrapper turns the status into an exception
    assert _lib.device_status() == (0, 0, 0, 0)             # cleared by the read
    x = torch.randn(64, 384, generator=torch.Generator().manual_seed(1)).half()
    y = layer_norm(x.to(dev()), None, None, 1e-6)            # the context is intact: the next kernel runs and is right
    assert oracle.rel_l2(y.cpu().float(), oracle.layer_norm(x, None, None, 1e-6)) < TOL_F32
    with pytest.raises(_lib.FastbbError):
        _lib.check(lib.fbb_diag_wait_timeout(0, 0, None))    # limits outside (0, 100 ms] are rejected on the host
    assert _lib.device_status() == (0, 0, 0, 0)


def test_sm_clock_probe_reads_a_plausible_clock():
    from fastbb_b200 import _lib
    buf = torch.zeros(1, dtype=torch.float32, device=dev())
    _lib.check(_lib.load().fbb_diag_sm_clock_mhz(buf.data_ptr(), 1 << 16, _lib.stream_ptr(dev())))
    torch.cuda.synchronize()
    assert 100.0 < float(buf[0]) < 3000.0
