#!/usr/bin/env python
"""Per-kernel sweep on one B200 (the kernel-level configuration of the benchmark plan): flash attention, linear layers
and LayerNorm at the shapes the ViT configs produce, timed with CUDA events and reported against the roofline.

    python bench_kernels.py                                   # whole sweep, one JSON line per case
    python bench_kernels.py --only flash --n 6145 --variant ff --iters 1 --warmup 0     # one case (e.g. under ncu)
    python bench_kernels.py --only linear --m 6145 --k 1024 --nn 4096 --act gelu
    python bench_kernels.py --only layernorm

(a) flash attention: fp16 Q/K/V ~ N(0,1), head dim 64, 16 heads, batch 1, N in {257, 400, 1370, 4097, 6145, 16385},
    scale 1/8; FLOPs = 4 N^2 H 64.
(b) linear: M in {257, 1370, 6145, 32768} x (K, N) in {(1024,3072), (1024,1024), (1024,4096), (4096,1024)}, weights
    ~ N(0, 0.02), activations ~ N(0,1), both accumulate modes; FLOPs = 2 M N K.
(c) LayerNorm: hidden 1024, M = 6145; bytes = M C (2 + 2).
Between timed launches a 256 MB buffer is overwritten when --flush-l2 is given (default: inputs stay L2-resident, as
they are inside the block stack where each kernel reads what the previous one just wrote).
--torch adds, for every case, the PyTorch library path for the same operator on the same tensors in the same process
(what the reference's friendly tier launches, fastbb/vit.py:114-143): F.linear followed by the separate F.gelu and
addcmul passes the fused epilogues replace (`torch_gemm_us` is the F.linear call alone), F.scaled_dot_product_attention,
F.layer_norm; the line then carries `torch_us` and `ratio` = torch_us / us.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return p["bf16_tflops"], p["hbm_gbs"], "measured"
    except (OSError, KeyError, ValueError):
        return 1590.0, 6650.0, "fallback"


def main():
    import torch
    from fastbb_b200.attention import Workspaces, attention, use_workspaces
    from fastbb_b200.gemm import linear
    from fastbb_b200.layernorm import layer_norm

    ap = argparse.ArgumentParser()
    ap.add_argument("--only", choices=["flash", "linear", "layernorm"])
    ap.add_argument("--n", type=int)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--variant", default=None)
    ap.add_argument("--m", type=int)
    ap.add_argument("--k", type=int)
    ap.add_argument("--nn", type=int)
    ap.add_argument("--act", default=None)
    ap.add_argument("--res", action="store_true", help="linear: with the LayerScale + residual epilogue (res + gamma * y)")
    ap.add_argument("--acc", default=None)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--flush-l2", action="store_true")
    ap.add_argument("--torch", action="store_true", help="also time the PyTorch library operators on the same tensors")
    args = ap.parse_args()
    import torch.nn.functional as F

    dev = torch.device("cuda:0")
    tf_peak, gb_peak, src = peaks()
    g = torch.Generator(device=dev).manual_seed(0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if args.flush_l2 else None

    owner = Workspaces()  # attention scratch memory of this script: made by the warm-up calls, before any capture

    def timed(fn):
        with use_workspaces(owner):
            return timed_(fn)

    def timed_(fn):
        """Mean device time of one launch in ms. Without --flush-l2 the launches are replayed back to back from a CUDA
        graph, so host launch overhead (several us per call) does not hide inside the number; with it, every launch
        is timed on its own after the flush."""
        for _ in range(max(args.warmup, 1)):
            fn()
        torch.cuda.synchronize()
        if flush is None and args.iters > 1:
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side), torch.cuda.graph(graph, stream=side):
                for _ in range(args.iters):
                    fn()
            torch.cuda.current_stream().wait_stream(side)
            graph.replay()
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            graph.replay()
            e.record()
            torch.cuda.synchronize()
            return s.elapsed_time(e) / args.iters
        total = 0.0
        for _ in range(args.iters):
            if flush is not None:
                flush.fill_(1)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            total += s.elapsed_time(e)
        return total / args.iters  # ms

    def emit(**kw):
        kw.update(peak_source=src, l2="flushed" if flush is not None else "resident", iters=args.iters)
        print(json.dumps(kw), flush=True)

    if args.only in (None, "flash"):
        for N in ([args.n] if args.n else [257, 400, 1370, 4097, 6145, 16385]):
            qkv = torch.randn(args.batch, N, 3, args.heads, 64, device=dev, generator=g).half()
            q, k, v = qkv.unbind(2)
            out = torch.empty(args.batch, N, args.heads, 64, device=dev, dtype=torch.float16)
            for variant in ([args.variant] if args.variant else ["ff", "fh", "hh"]):
                ms = timed(lambda: attention(q, k, v, scale=0.125, variant=variant, out=out))
                tf = 4.0 * args.batch * N * N * args.heads * 64 / (ms * 1e-3) / 1e12
                extra = {}
                if args.torch:
                    qt, kt, vt = (t.transpose(1, 2) for t in (q, k, v))   # [B, H, N, 64] views, as the reference's SDPA path passes them
                    tms = timed(lambda: F.scaled_dot_product_attention(qt, kt, vt, scale=0.125))
                    extra = dict(torch_us=tms * 1e3, ratio=tms / ms, torch_what="F.scaled_dot_product_attention")
                emit(kernel="flash64", variant=variant, B=args.batch, N=N, H=args.heads, us=ms * 1e3, tflops=tf,
                     frac_of_measured_burst=tf / tf_peak, frac_of_nominal_2250=tf / 2250.0, **extra)
    if args.only in (None, "linear"):
        shapes = [(args.k, args.nn)] if args.k and args.nn else [(1024, 3072), (1024, 1024), (1024, 4096), (4096, 1024)]
        for M in ([args.m] if args.m else [257, 1370, 6145, 32768]):
            for K, N in shapes:
                x = torch.randn(M, K, device=dev, generator=g).half()
                w = (torch.randn(N, K, device=dev, generator=g) * 0.02).half()
                b = torch.zeros(N, device=dev, dtype=torch.float16)
                n_out = N // 2 if args.act == "swiglu" else N
                out = torch.empty(M, n_out, device=dev, dtype=torch.float16)
                res = torch.randn(M, n_out, device=dev, generator=g).half() if args.res else None
                gam = (0.05 + 0.15 * torch.rand(n_out, device=dev, generator=g)).half() if args.res else None
                extra = {}
                if args.torch:
                    def torch_path():
                        y = F.linear(x, w, b)
                        if args.act == "gelu":
                            y = F.gelu(y)
                        elif args.act == "swiglu":
                            x1, x2 = y.chunk(2, dim=-1)
                            y = F.silu(x1).mul_(x2)
                        return torch.addcmul(res, y, gam) if res is not None else y
                    tms, gms = timed(torch_path), timed(lambda: F.linear(x, w, b))
                    extra = dict(torch_us=tms * 1e3, torch_gemm_us=gms * 1e3, torch_what="F.linear + separate activation / addcmul passes")
                for acc in ([args.acc] if args.acc else ["f32", "h"]):
                    ms = timed(lambda: linear(x, w, b, act=args.act, res=res, gamma=gam, variant=acc, out=out))
                    tf = 2.0 * M * N * K / (ms * 1e-3) / 1e12
                    if extra:
                        extra["ratio"] = extra["torch_us"] / (ms * 1e3)
                    emit(kernel="linear", acc=acc, act=args.act, res=bool(args.res), M=M, N=N, K=K, us=ms * 1e3, tflops=tf,
                         frac_of_measured_burst=tf / tf_peak, frac_of_nominal_2250=tf / 2250.0, **extra)
    if args.only in (None, "layernorm"):
        M, C = args.m or 6145, args.k or 1024
        x = torch.randn(M, C, device=dev, generator=g).half()
        w, b = torch.ones(C, device=dev, dtype=torch.float16), torch.zeros(C, device=dev, dtype=torch.float16)
        out = torch.empty_like(x)
        ms = timed(lambda: layer_norm(x, w, b, 1e-6, out=out))
        gbs = M * C * 4.0 / (ms * 1e-3) / 1e9
        extra = {}
        if args.torch:
            tms = timed(lambda: F.layer_norm(x, (C,), w, b, 1e-6))
            extra = dict(torch_us=tms * 1e3, ratio=tms / ms, torch_what="F.layer_norm")
        emit(kernel="layernorm", M=M, C=C, us=ms * 1e3, gbs=gbs, frac_of_measured_copy=gbs / gb_peak, frac_of_nominal_8000=gbs / 8000.0,
             bytes=M * C * 4, **extra)


if __name__ == "__main__":
    main()
