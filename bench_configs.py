#!/usr/bin/env python
"""Throughput of the other benchmark configurations (bench.py covers the headline one and imports the functions below
for its batched-split record): images/s, ms per batch and TFLOP/s for

  c0  DINOv2 ViT-S/14, 224x224, batch 1                          (257 tokens: the small-token path)
  c2  timm-style ViT-B/16 block stack, 1024x1024 (4097 tokens), batch 1 and 8, install_vit_blocks(..., "fh-g1")
  c3  DINOv2 ViT-g/14 (SwiGLU), 518x518 (1370 tokens), global batch 32, spec hh-g1
  c1-torch  (--torch) the headline workload on the SAME GPU through plain PyTorch operators in fp16 (F.linear, SDPA,
      F.layer_norm, F.gelu, addcmul), the operator sequence of the reference's friendly tier (fastbb/vit.py:108-150)
      written out here. This is the library bar on this machine: cuBLAS / cuDNN / aten kernels, none of this
      repository's. (The reference package itself, CPU and GPU tiers, is timed by `bench.py --impl reference`.)

    python bench_configs.py [--only c3] [--steps 20] [--torch]
    python -m torch.distributed.run --nproc-per-node 8 ... bench_configs.py --only c3      # batch sharded 4 per GPU

Under torchrun the global batch of c2 (8) and c3 (32) is split contiguously over the ranks (one replica per GPU, no
collective on the forward path); each rank times its own slice with CUDA events and the slowest rank sets the time.
A single process runs the per-GPU share of an 8-GPU job (c3: 4 images, c2: batch 1 and 8) unless --batch is given.
Weights and inputs are seeded synthetic tensors; timm is not required (c2 uses a stand-in block with timm's attribute
names). One JSON line per case on rank 0.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def stack_flops(tokens_per_image, batch, C, depth, swiglu_hidden=None):
    T = tokens_per_image * batch
    if swiglu_hidden is None:
        gemm = 24.0 * T * C * C
    else:
        gemm = 2.0 * T * C * (3 * C + C + 2 * swiglu_hidden + swiglu_hidden)
    return depth * (gemm + 4.0 * batch * tokens_per_image ** 2 * C)


def timed(fn, dev, steps, warmup):
    """ms per call: CUDA events around `steps` calls after >= 3 warm-ups, barrier on both sides, max over ranks."""
    import torch
    from fastbb_b200 import replicas
    for _ in range(max(warmup, 3)):
        fn()
    torch.cuda.synchronize()
    replicas.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(steps):
        fn()
    e.record()
    torch.cuda.synchronize()
    replicas.barrier()
    return replicas.max_over_ranks(s.elapsed_time(e), dev) / steps


def timed_e2e(fn, x_host, dev, steps):
    """ms per batch from a pinned host batch to pinned host outputs through HostPipeline (copies inside the timing)."""
    import torch
    from fastbb_b200 import replicas
    from fastbb_b200.pipeline import HostPipeline
    pipe = HostPipeline(fn, device=dev, depth=3)
    for _ in range(8):  # enough submissions for the allocator to hold every buffer the steady state keeps in flight
        pipe.submit(x_host)
    pipe.drain()
    torch.cuda.synchronize()
    replicas.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(steps):
        pipe.submit(x_host)
    pipe.drain()
    e.record()
    torch.cuda.synchronize()
    replicas.barrier()
    return replicas.max_over_ranks(s.elapsed_time(e), dev) / steps, pipe.h2d_bytes, pipe.d2h_bytes


def record(name, spec, world, global_batch, local_batch, ms, flops_local, steps, e2e=None, note=None):
    r = {"config": name, "spec": spec, "n_gpus": world, "global_batch": global_batch, "batch_per_gpu": local_batch, "ms_per_batch": ms,
         "images_per_s": global_batch / (ms * 1e-3), "tflops_per_gpu": flops_local / (ms * 1e-3) / 1e12, "steps": steps, "data": "synthetic"}
    if e2e is not None:
        ms_e2e, h2d, d2h = e2e
        r.update(e2e_ms_per_batch=ms_e2e, e2e_images_per_s=global_batch / (ms_e2e * 1e-3), h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h)
    if note:
        r["note"] = note
    return r


def run_c0(dev, rank, world, steps, warmup):
    from fastbb_b200 import synthetic
    from fastbb_b200.models.dinov2 import dinov2
    fast = dinov2("vits14", synthetic.make_params("vits14", seed=0), spec="fh-g0-graph", device=dev)
    x = synthetic.make_image(1, 224, 224, seed=1).to(dev)
    ms = timed(lambda: fast.get_intermediate_layers(x, n=4, return_class_token=True), dev, steps, warmup)
    return record("c0 ViT-S/14 224x224 b1 per GPU", "fh-g0-graph", world, world, 1, ms, stack_flops(257, 1, 384, 12), steps)


def timm_like_stack(dev, depth=12, d=768, heads=12):
    """Block stack with the attribute names of timm.models.vision_transformer.Block (no LayerScale), seeded init."""
    import torch
    import torch.nn as nn

    class Attn(nn.Module):
        def __init__(self):
            super().__init__()
            self.num_heads, self.scale = heads, (d // heads) ** -0.5
            self.qkv, self.proj = nn.Linear(d, 3 * d), nn.Linear(d, d)

    class Mlp(nn.Module):
        def __init__(self):
            super().__init__()
            self.fc1, self.act, self.fc2 = nn.Linear(d, 4 * d), nn.GELU(), nn.Linear(4 * d, d)

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.norm1, self.norm2 = nn.LayerNorm(d, eps=1e-6), nn.LayerNorm(d, eps=1e-6)
            self.attn, self.mlp, self.ls1, self.ls2 = Attn(), Mlp(), nn.Identity(), nn.Identity()

        def forward(self, x):
            raise RuntimeError("original forward reached")

    torch.manual_seed(0)
    stack = nn.Sequential(*[Block() for _ in range(depth)]).to(dev).eval()
    for p in stack.parameters():
        if p.dim() > 1:
            nn.init.trunc_normal_(p, std=0.02)
    return stack


def run_c2(dev, rank, world, steps, warmup, global_batch, e2e=False, stack=None):
    """ViT-B/16 block stack at 4097 tokens through install_vit_blocks(..., "fh-g1"); the global batch is split over the ranks
    (a batch smaller than the world runs as one replica of it per rank, reported as such)."""
    import torch
    import fastbb_b200 as fb
    from fastbb_b200 import replicas
    if stack is None:
        stack = timm_like_stack(dev)
        assert fb.install_vit_blocks(stack, "fh-g1") == 12
    gb = global_batch
    lo, hi = replicas.shard_bounds(gb, rank, world) if gb >= world else (0, gb)
    lb = max(hi - lo, 1)
    x = torch.randn(lb, 4097, 768, device=dev, dtype=torch.float16)
    with torch.no_grad():
        ms = timed(lambda: stack(x), dev, steps, warmup)
        ee = None
        if e2e:
            x_host = torch.randn(lb, 4097, 768, dtype=torch.float16).pin_memory()
            ee = timed_e2e(lambda t: stack(t), x_host, dev, steps)
    total = gb if gb >= world else gb * world
    return record("c2 ViT-B/16 block stack 1024x1024 (4097 tokens)", "fh-g1 via install_vit_blocks", world, total, lb, ms,
                  stack_flops(4097, lb, 768, 12), steps, ee, None if gb >= world else f"batch {gb} does not split over {world} GPUs: one replica per GPU")


def run_c3(dev, rank, world, steps, warmup, global_batch, e2e=False, fast=None):
    """ViT-g/14 518x518, hh-g1-graph, global batch split contiguously over the ranks."""
    from fastbb_b200 import replicas, synthetic
    from fastbb_b200.models.dinov2 import dinov2, swiglu_hidden
    lo, hi = replicas.shard_bounds(global_batch, rank, world)
    lb = hi - lo
    if fast is None:
        fast = dinov2("vitg14", synthetic.make_params("vitg14", seed=0), spec="hh-g1-graph", device=dev)
    x_host = synthetic.make_image(lb, 518, 518, seed=1 + rank).half().pin_memory()
    x = x_host.to(dev)
    fn = lambda t: fast.get_intermediate_layers(t, n=[9, 19, 29, 39], return_class_token=True)  # noqa: E731
    ms = timed(lambda: fn(x), dev, steps, warmup)
    ee = timed_e2e(fn, x_host, dev, steps) if e2e else None
    return record("c3 ViT-g/14 518x518 (1370 tokens)", "hh-g1-graph", world, global_batch, lb, ms,
                  stack_flops(1370, lb, 1536, 40, swiglu_hidden(1536)), steps, ee)


def torch_friendly_c1(dev, steps, warmup):
    """The headline workload (ViT-L/14, 896x1344, layers 4/11/17/23) through plain PyTorch fp16 operators on this GPU."""
    import torch
    import torch.nn.functional as F
    from fastbb_b200 import synthetic
    params = synthetic.make_params("vitl14", seed=0)
    x = synthetic.make_image(1, 896, 1344, seed=1).to(dev)
    layers = [4, 11, 17, 23]
    from fastbb_b200.models.dinov2 import dinov2
    fast = dinov2("vitl14", params, spec="fh-g0", device=dev)   # only for its tokenizer and module tree
    vit = fast.vit

    def fn():
        t = fast.tokens(x)
        out = []
        for i, b in enumerate(fast.blocks):
            B, N, C = t.shape
            qkv = F.linear(b.norm1(t), b.attn.qkv.weight, b.attn.qkv.bias).view(B, N, 3, 16, 64)
            q, k, v = (u.transpose(1, 2) for u in qkv.unbind(2))
            o = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, N, C)
            t = torch.addcmul(t, F.linear(o, b.attn.proj.weight, b.attn.proj.bias), b.ls1.gamma)
            h = F.gelu(F.linear(b.norm2(t), b.mlp.fc1.weight, b.mlp.fc1.bias))
            t = t.addcmul(F.linear(h, b.mlp.fc2.weight, b.mlp.fc2.bias), b.ls2.gamma)
            if i in layers:
                out.append(vit.norm(t))
        return out
    kind = "plain PyTorch fp16 operators, written out as the reference's friendly tier runs them: F.linear, SDPA, nn.LayerNorm, F.gelu, addcmul"
    with torch.no_grad():
        ms = timed(fn, dev, steps, warmup)
    r = record("c1 ViT-L/14 896x1344 (6145 tokens) b1, library operators", "torch fp16 eager", 1, 1, 1, ms, stack_flops(6145, 1, 1024, 24), steps)
    r["what"] = kind
    return r


def main():
    import torch
    from fastbb_b200 import replicas

    ap = argparse.ArgumentParser()
    ap.add_argument("--only", choices=["c0", "c2", "c3"])
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, help="global batch (default: the config's)")
    ap.add_argument("--e2e", action="store_true", help="also time host-to-host through HostPipeline")
    ap.add_argument("--torch", action="store_true", help="only the library-operator line for the headline workload")
    args = ap.parse_args()
    rank, local_rank, world = replicas.init_process_group()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)

    def emit(r):
        if rank == 0:
            print(json.dumps(r), flush=True)

    if args.torch:
        if rank == 0:
            emit(torch_friendly_c1(dev, args.steps, args.warmup))
    else:
        if args.only in (None, "c0"):
            emit(run_c0(dev, rank, world, args.steps, args.warmup))
        if args.only in (None, "c2"):
            import fastbb_b200 as fb
            stack = timm_like_stack(dev)
            assert fb.install_vit_blocks(stack, "fh-g1") == 12
            for gb in ([args.batch] if args.batch else [1, 8]):
                emit(run_c2(dev, rank, world, args.steps, args.warmup, gb, args.e2e, stack))
        if args.only in (None, "c3"):
            emit(run_c3(dev, rank, world, args.steps, args.warmup, args.batch or (32 if world > 1 else 4), args.e2e))

    import torch.distributed as dist
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
