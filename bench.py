#!/usr/bin/env python
"""Headline benchmark: DINOv2 ViT-L/14, 896x1344 input (6145 tokens), fp16, batch 1,
get_intermediate_layers(n=[4, 11, 17, 23], return_class_token=True) -- images/s and ms/image on N B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--spec fh-g0-graph] [--impl ours|reference]

N > 1 is launched by torchrun, one rank per GPU. The batch-1 workload does not shard, so every rank runs an
independent replica on its own GPU (weak scaling, no collective on the forward path); only the timing scalar is
reduced (MAX over ranks). Prints ONE JSON line on rank 0.

  value     images/s with the input image already resident in HBM (CUDA events around exactly K steps)
  e2e       the same through the public API (fastbb_b200.pipeline.HostPipeline) from a pinned host image to pinned host
            outputs: every step uploads its image and downloads its features inside the timed region, on copy streams
            overlapped with compute
  roofline  the dominant kernel (flash attention): algorithmic FLOPs per launch / mean launch time, timed live with
            CUDA events around each of its launches in a separate instrumented pass over the same K steps
  cpu_baseline / --impl reference
            the CPU restatement of the reference's fp32 tier (oracle/), timed on the host cores on a bounded sample

Inputs are synthetic: seeded N(0,1) image, trunc-normal(0.02) weights, LayerScale gamma ~ U(0.05, 0.2).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ARCH, IMG_H, IMG_W, LAYERS, HEADS = "vitl14", 896, 1344, [4, 11, 17, 23], 16
TOKENS, EMBED, DEPTH = (IMG_H // 14) * (IMG_W // 14) + 1, 1024, 24
FLOPS_ATTN_PER_LAUNCH = 4.0 * TOKENS * TOKENS * EMBED                      # QK^T + PV of one block, all heads
FLOPS_PER_IMAGE = DEPTH * (24.0 * TOKENS * EMBED * EMBED + FLOPS_ATTN_PER_LAUNCH)
NOMINAL_FP16_TFLOPS = 2250.0


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"tflops_burst": p["bf16_tflops"], "tflops_sustained": p["bf16_tflops_sustained"], "hbm_gbs": p["hbm_gbs"],
                "source": "measured"}
    except (OSError, KeyError, ValueError):
        return {"tflops_burst": 1590.0, "tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU during the timed region: one `nvidia-smi -lms 100` child
    process, started before and terminated after (reading settings only; nothing on the GPU is changed)."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.lines, self.proc, self.reader = index, [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE, text=True)
        except OSError:
            return
        self.reader = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
        self.reader.start()
        time.sleep(0.25)  # first sample lands before the timed region starts

    def summary(self):
        if self.proc is not None:
            self.proc.terminate()
            self.proc.wait(timeout=5)
            self.reader.join(timeout=5)
        rows = [[c.strip() for c in ln.split(",")] for ln in self.lines if ln.count(",") >= 5]
        rows = rows[1:] if len(rows) > 2 else rows  # the first row predates the load
        mhz = [float(r[0]) for r in rows if r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in rows if r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in rows for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(rows)}


def oracle_cpu_sample(steps, warmup, blocks=3):
    """Reference fp32 tier restated on the CPU (oracle/), bounded sample: tokenizer + `blocks` of the 24 blocks of one
    896x1344 image per step; the block time is scaled to 24 blocks (all blocks cost the same). Returns (img/s, info)."""
    import torch
    from oracle import vit_oracle as O
    try:  # torchrun exports OMP_NUM_THREADS=1; the CPU baseline uses every core this process may run on
        torch.set_num_threads(len(os.sched_getaffinity(0)))
    except (AttributeError, RuntimeError):
        pass
    params = O.make_params(ARCH, seed=0, depth=blocks)
    x = O.make_image(1, IMG_H, IMG_W, seed=1)
    times = []
    with torch.no_grad():
        for i in range(warmup + steps):
            t0 = time.perf_counter()
            t = O.tokens(params, x)
            t1 = time.perf_counter()
            for b in range(blocks):
                t = O.block(params, b, t, HEADS)
            t2 = time.perf_counter()
            if i >= warmup:
                times.append((t1 - t0) + (t2 - t1) * DEPTH / blocks)
    sec = statistics.median(times)
    return 1.0 / sec, {"cores": torch.get_num_threads(), "kind": "port",
                       "sample": f"tokenizer + {blocks} of {DEPTH} blocks of one {IMG_H}x{IMG_W} image per step, block time x{DEPTH}/{blocks}; "
                                 f"median of {steps} steps"}


def run_reference(args, rank, world):
    if rank != 0:
        return
    value, info = oracle_cpu_sample(max(1, min(args.steps, 3)), 1)
    line = {"impl": "reference", "metric": "images_per_s", "value": value, "unit": "img/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 / value, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": workload_config("reference fp32 friendly tier restated on CPU"),
            "cpu_baseline": {"value": value, "unit": "img/s", **info},
            "e2e": {"value": value, "unit": "img/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def workload_config(spec):
    return {"workload": f"DINOv2 ViT-L/14 {IMG_H}x{IMG_W} ({TOKENS} tokens) fp16 batch 1 per GPU, get_intermediate_layers n={LAYERS} + cls tokens",
            "spec": spec, "flops_per_image": FLOPS_PER_IMAGE,
            "l2": "no explicit flush: each step streams 604 MB of weights plus ~100 MB activations per block through the 126 MB L2"}


def run_ours(args, rank, local_rank, world):
    import torch
    from fastbb_b200 import _lib, attention as attn_mod, replicas
    from fastbb_b200 import vit as vit_mod
    from fastbb_b200.models.dinov2 import dinov2
    from fastbb_b200 import synthetic as O

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU path")
    _lib.load()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    params = O.make_params(ARCH, seed=0)
    fast = dinov2(ARCH, params, spec=args.spec, device=dev)
    del params
    x_host = O.make_image(1, IMG_H, IMG_W, seed=1).pin_memory()
    x_dev = x_host.to(dev)

    def step(x):
        return fast.get_intermediate_layers(x, n=LAYERS, return_class_token=True)

    # launches per step, counted on an eager pass (a graph replay launches the same kernels)
    graphs, fast.graphs = fast.graphs, False
    before = _lib.LAUNCHES
    outs = step(x_dev)
    launches_per_step = _lib.LAUNCHES - before
    fast.graphs = graphs
    for _ in range(max(args.warmup, 3)):
        step(x_dev)
    torch.cuda.synchronize()
    replicas.barrier()

    # ---------------- timed region: exactly K steps, inputs resident in HBM
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    replicas.barrier()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        step(x_dev)
    e1.record()
    torch.cuda.synchronize()
    replicas.barrier()
    ms_total = replicas.max_over_ranks(e0.elapsed_time(e1), dev)
    clocks = sampler.summary()

    # ---------------- end to end: pinned host image in, pinned host features out, every step's copies inside the timing.
    # Through the package's HostPipeline: uploads and downloads run on side streams, overlapped with the next / previous
    # step's compute (each step still uploads its own image and downloads its own features).
    from fastbb_b200.pipeline import HostPipeline
    pipe = HostPipeline(step, device=dev, depth=2)
    for _ in range(3):
        pipe.submit(x_host)
    pipe.drain()
    torch.cuda.synchronize()
    replicas.barrier()
    e0.record()
    for _ in range(args.steps):
        pipe.submit(x_host)
    pipe.drain()
    e1.record()
    torch.cuda.synchronize()
    replicas.barrier()
    ms_e2e = replicas.max_over_ranks(e0.elapsed_time(e1), dev)
    host_check = pipe.result(pipe.drain())
    assert all(torch.isfinite(p.float()).all() for p, _ in host_check), "non-finite features in the end-to-end pass"
    h2d, d2h = pipe.h2d_bytes, pipe.d2h_bytes

    # ---------------- roofline of the dominant kernel: events around every flash-attention launch, eager pass
    variant = "ff" if fast.attn == "sdpa" else fast.attn
    marks = []
    real_attention = attn_mod.attention

    def timed_attention(*a, **kw):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        o = real_attention(*a, **kw)
        e.record()
        marks.append((s, e))
        return o
    fast.graphs = False
    vit_mod.attention = timed_attention
    # the per-operator host path (same kernels, same order as the C stack runner) so that each launch can be bracketed
    runner_env = os.environ.get("FBB_NO_RUNNER")
    os.environ["FBB_NO_RUNNER"] = "1"
    try:
        for _ in range(args.steps):
            step(x_dev)
        torch.cuda.synchronize()
    finally:
        vit_mod.attention = real_attention
        fast.graphs = graphs
        if runner_env is None:
            del os.environ["FBB_NO_RUNNER"]
        else:
            os.environ["FBB_NO_RUNNER"] = runner_env
    assert len(marks) == DEPTH * args.steps, "the instrumented pass did not see every attention launch"
    attn_ms = [s.elapsed_time(e) for s, e in marks]
    attn_mean_ms = sum(attn_ms) / len(attn_ms)
    peaks = measured_peaks()
    achieved = FLOPS_ATTN_PER_LAUNCH / (attn_mean_ms * 1e-3) / 1e12

    if rank == 0:
        ms_step = ms_total / args.steps
        value = world * args.steps / (ms_total * 1e-3)
        line = {
            "metric": "images_per_s", "value": value, "unit": "img/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "ms_per_image": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp16", "data": "synthetic", "config": workload_config(args.spec),
            "tensor_frac": {"tflops": FLOPS_PER_IMAGE / (ms_step * 1e-3) / 1e12,
                            "of_nominal_2250": FLOPS_PER_IMAGE / (ms_step * 1e-3) / 1e12 / NOMINAL_FP16_TFLOPS,
                            "of_measured_sustained": FLOPS_PER_IMAGE / (ms_step * 1e-3) / 1e12 / peaks["tflops_sustained"]},
            "clocks": clocks,
            "e2e": {"value": world * args.steps / (ms_e2e * 1e-3), "unit": "img/s", "ms_per_image": ms_e2e / args.steps,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches_per_step * args.steps,
            "roofline": {"kernel": f"flash64_umma_kernel ({variant})", "bound": "tensor", "achieved": achieved,
                         "peak": peaks["tflops_sustained"], "unit": "TFLOP/s", "frac": achieved / peaks["tflops_sustained"],
                         "peak_source": f"{peaks['source']} cuBLAS bf16 sustained", "frac_of_nominal_2250": achieved / NOMINAL_FP16_TFLOPS,
                         "launch_ms": attn_mean_ms, "launches_timed": len(attn_ms), "flops_per_launch": FLOPS_ATTN_PER_LAUNCH,
                         "share_of_step": attn_mean_ms * DEPTH / ms_step, "traffic": ATTN_DRAM_TRAFFIC_BYTES},
        }
        if world == 1 and not args.no_cpu_baseline:
            v, info = oracle_cpu_sample(1, 1)
            line["cpu_baseline"] = {"value": v, "unit": "img/s", **info}
        print(json.dumps(line), flush=True)


# dram__bytes_read.sum + dram__bytes_write.sum of one flash-attention launch at this workload, from the ncu capture
# summarised in profiles/flash64_fh_N6145_H16.md (37.86 MB read, 0.64 MB written: the inputs once; the output and the
# split groups' partial results stay in L2).
ATTN_DRAM_TRAFFIC_BYTES = 37862912 + 637184


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--spec", default="fh-g0-graph")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank, local_rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    from fastbb_b200 import replicas
    replicas.init_process_group()
    try:
        run_ours(args, rank, local_rank, world)
    finally:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
