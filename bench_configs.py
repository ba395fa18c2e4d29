#!/usr/bin/env python
"""Throughput of the other benchmark configurations (bench.py covers the headline one): images/s, ms per batch and
TFLOP/s for

  c0  DINOv2 ViT-S/14, 224x224, batch 1                          (257 tokens: the small-token path)
  c2  timm-style ViT-B/16 block stack, 1024x1024 (4097 tokens), batch 1 and 8, install_vit_blocks(..., "fh-g1")
  c3  DINOv2 ViT-g/14 (SwiGLU), 518x518 (1370 tokens), global batch 32, spec hh-g1

    python bench_configs.py [--only c3] [--steps 20]
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


def main():
    import torch
    import torch.nn as nn
    import fastbb_b200 as fb
    from fastbb_b200 import replicas, synthetic
    from fastbb_b200.models.dinov2 import dinov2, swiglu_hidden

    ap = argparse.ArgumentParser()
    ap.add_argument("--only", choices=["c0", "c2", "c3"])
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, help="global batch (default: the config's)")
    args = ap.parse_args()
    rank, local_rank, world = replicas.init_process_group()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)

    def timed(fn):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        replicas.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(args.steps):
            fn()
        e.record()
        torch.cuda.synchronize()
        replicas.barrier()
        return replicas.max_over_ranks(s.elapsed_time(e), dev) / args.steps

    def emit(name, spec, global_batch, local_batch, ms, flops_local):
        if rank == 0:
            print(json.dumps({"config": name, "spec": spec, "n_gpus": world, "global_batch": global_batch, "batch_per_gpu": local_batch,
                              "ms_per_batch": ms, "images_per_s": global_batch / (ms * 1e-3), "tflops_per_gpu": flops_local / (ms * 1e-3) / 1e12,
                              "steps": args.steps, "data": "synthetic"}), flush=True)

    if args.only in (None, "c0"):
        fast = dinov2("vits14", synthetic.make_params("vits14", seed=0), spec="fh-g0-graph", device=dev)
        x = synthetic.make_image(1, 224, 224, seed=1).to(dev)
        ms = timed(lambda: fast.get_intermediate_layers(x, n=4, return_class_token=True))
        emit("c0 ViT-S/14 224x224 b1 per GPU", "fh-g0-graph", world, 1, ms, stack_flops(257, 1, 384, 12))
        del fast

    if args.only in (None, "c2"):
        class Attn(nn.Module):
            def __init__(self, d, heads):
                super().__init__()
                self.num_heads, self.scale = heads, (d // heads) ** -0.5
                self.qkv, self.proj = nn.Linear(d, 3 * d), nn.Linear(d, d)

        class Mlp(nn.Module):
            def __init__(self, d):
                super().__init__()
                self.fc1, self.act, self.fc2 = nn.Linear(d, 4 * d), nn.GELU(), nn.Linear(4 * d, d)

        class Block(nn.Module):  # attribute names of timm.models.vision_transformer.Block, no LayerScale
            def __init__(self, d=768, heads=12):
                super().__init__()
                self.norm1, self.norm2 = nn.LayerNorm(d, eps=1e-6), nn.LayerNorm(d, eps=1e-6)
                self.attn, self.mlp, self.ls1, self.ls2 = Attn(d, heads), Mlp(d), nn.Identity(), nn.Identity()

            def forward(self, x):
                raise RuntimeError("original forward reached")

        torch.manual_seed(0)
        stack = nn.Sequential(*[Block() for _ in range(12)]).to(dev).eval()
        for p in stack.parameters():
            if p.dim() > 1:
                nn.init.trunc_normal_(p, std=0.02)
        assert fb.install_vit_blocks(stack, "fh-g1") == 12
        for gb in ([args.batch] if args.batch else [1, 8]):
            lo, hi = replicas.shard_bounds(gb, rank, world) if gb >= world else (0, gb)
            lb = hi - lo
            x = torch.randn(max(lb, 1), 4097, 768, device=dev, dtype=torch.float16)
            with torch.no_grad():
                ms = timed(lambda: stack(x))
            total = gb if gb >= world else gb * world
            emit("c2 ViT-B/16 block stack 1024x1024 (4097 tokens)", "fh-g1 via install_vit_blocks", total, max(lb, 1), ms,
                 stack_flops(4097, max(lb, 1), 768, 12))
        del stack

    if args.only in (None, "c3"):
        gb = args.batch or (32 if world > 1 else 4)
        lo, hi = replicas.shard_bounds(gb, rank, world)
        lb = hi - lo
        fast = dinov2("vitg14", synthetic.make_params("vitg14", seed=0), spec="hh-g1-graph", device=dev)
        x = synthetic.make_image(lb, 518, 518, seed=1 + rank).to(dev)
        ms = timed(lambda: fast.get_intermediate_layers(x, n=[9, 19, 29, 39], return_class_token=True))
        emit("c3 ViT-g/14 518x518 (1370 tokens)", "hh-g1-graph", gb, lb, ms, stack_flops(1370, lb, 1536, 40, swiglu_hidden(1536)))

    import torch.distributed as dist
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
