#!/usr/bin/env python
"""Headline benchmark: DINOv2 ViT-L/14, 896x1344 input (6145 tokens), fp16, batch 1,
get_intermediate_layers(n=[4, 11, 17, 23], return_class_token=True) -- images/s and ms/image on N B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--spec fh-g0-graph] [--impl ours|reference]

N > 1 is launched by torchrun, one rank per GPU. The batch-1 workload does not shard, so every rank runs an
independent replica on its own GPU (weak scaling, no collective on the forward path); only timing scalars cross ranks.
Prints ONE JSON line on rank 0.

  value      images/s with the input image already resident in HBM (CUDA events around exactly K steps)
  e2e        the same through the public API (fastbb_b200.pipeline.HostPipeline) from a pinned host image (fp16, as a
             caller that decodes to half precision hands it over) to pinned host outputs: every step uploads its image and
             downloads its features inside the timed region, on copy streams overlapped with compute; with the per-rank
             times and, for context, each rank's pinned-copy bandwidth measured with all ranks copying at once
  roofline   the dominant kernel (flash attention): algorithmic FLOPs per launch / mean launch time, timed live with CUDA
             events around each of its launches in a separate instrumented pass (the per-operator path captured into a
             graph and replayed back to back), against the measured BURST cuBLAS rate; beside it the SM clock the launches
             ran at (an on-device probe) and the same launch timed alone in this process, so that a difference between
             the two is explained by the clock or not
  kernel_ms  the instrumented pass's per-step time in each kernel class and what a step spends outside them (gap_ms)
  configs    the batched configurations split over the ranks (ViT-g/14 batch 32, ViT-B/16 batch 8; at N = 1 their
             eight-GPU share), device-resident and end to end
  cpu_baseline / --impl reference
             the reference's own friendly fp32 tier on the host cores (its package under oracle/_ref when present, else
             the CPU restatement under oracle/), whole forward passes of the same workload, actually timed

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
# dram__bytes_read.sum + dram__bytes_write.sum of one flash-attention launch at this workload, from one ncu capture of the
# kernel (37.86 MB read, 0.64 MB written: the inputs once; the output and the split groups' partial results stay in L2).
ATTN_DRAM_TRAFFIC_BYTES = 37862912 + 637184
CPU_SECONDS_LIMIT = 75.0   # the reference arm stops adding timed passes once this much CPU time has been spent


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


# ------------------------------------------------------------------------------------------------ the CPU arm
def cpu_forward():
    """-> (fn, kind, what): fn() runs one whole forward pass of the headline workload in fp32 on the host cores."""
    import torch
    from oracle import vit_oracle as O
    try:  # torchrun exports OMP_NUM_THREADS=1; the CPU arm uses every core this process may run on
        torch.set_num_threads(len(os.sched_getaffinity(0)))
    except (AttributeError, RuntimeError):
        pass
    params = O.make_params(ARCH, seed=0)
    x = O.make_image(1, IMG_H, IMG_W, seed=1)
    ref_dir = os.path.join(ROOT, "oracle", "_ref")
    if os.path.exists(os.path.join(ref_dir, "fastbb", "vit.py")):
        sys.path.insert(0, ref_dir)
        from fastbb.models.dinov2 import DinoV2Params
        from fastbb.vit import FastViT as RefFastViT
        m = DinoV2Params(ARCH)
        m.load_state_dict(params, strict=True)
        ref = RefFastViT(m, attn="sdpa", gacc=False, dtype=torch.float32)
        return (lambda: ref.get_intermediate_layers(x, n=LAYERS, return_class_token=True), "reference",
                "the reference package itself (oracle/_ref): FastViT(attn='sdpa', gacc=False, dtype=float32), its friendly tier")
    return (lambda: O.get_intermediate_layers(params, x, LAYERS, HEADS, return_class_token=True), "port",
            "CPU restatement of the reference's fp32 tier (oracle/vit_oracle.py); the reference package is not installed under oracle/_ref")


def cpu_timed(steps, warmup, limit_s):
    """Whole forward passes, each actually timed: `warmup` untimed (at most one), then up to `steps`, stopping early once
    the limit is reached. Returns (seconds per pass, passes timed, passes warmed, kind, what, cores)."""
    import torch
    fn, kind, what = cpu_forward()
    spent = 0.0
    warmed = 0
    with torch.no_grad():
        if warmup > 0:
            t0 = time.perf_counter()
            fn()
            spent += time.perf_counter() - t0
            warmed = 1
        times = []
        while len(times) < max(1, steps) and (not times or spent + times[-1] <= limit_s):
            t0 = time.perf_counter()
            fn()
            times.append(time.perf_counter() - t0)
            spent += times[-1]
    return sum(times) / len(times), len(times), warmed, kind, what, torch.get_num_threads()


def workload_config():
    """The same dictionary in both arms: it names the workload, not the implementation (see the line's "arm" key)."""
    return {"workload": f"DINOv2 ViT-L/14 {IMG_H}x{IMG_W} ({TOKENS} tokens) batch 1 per GPU, get_intermediate_layers n={LAYERS} + cls tokens",
            "flops_per_image": FLOPS_PER_IMAGE,
            "l2": "no explicit flush: each step streams 604 MB of weights plus ~100 MB activations per block through the 126 MB L2"}


def reference_gpu_tiers(steps=5, warmup=3):
    """For context beside the CPU figure, when this machine has a GPU: the same workload through the reference's own GPU
    tiers, unmodified, from oracle/_ref - `fh-g0` (its flash64_* mma.sync kernel, recompiled for this architecture by
    oracle/make_ref.py: make_kernels, cuBLAS GEMMs) and `sdpa-g0` in fp16 (its friendly tier: PyTorch operators). ms per
    image, CUDA events around `steps` calls. Nothing of this repository's library is on that path."""
    import torch
    ref_dir = os.path.join(ROOT, "oracle", "_ref")
    if not torch.cuda.is_available():
        return {"unavailable": "no CUDA device"}
    if not os.path.exists(os.path.join(ref_dir, "fastbb", "vit.py")):
        return {"unavailable": "oracle/_ref not built (python oracle/make_ref.py)"}
    from oracle import vit_oracle as O
    sys.path.insert(0, ref_dir)
    from fastbb import parse_vit_spec
    from fastbb.models.dinov2 import DinoV2Params
    from fastbb.vit import FastViT as RefFastViT
    dev = torch.device("cuda", 0)
    params = O.make_params(ARCH, seed=0)
    x = O.make_image(1, IMG_H, IMG_W, seed=1).to(dev)
    out = {"what": "the reference package (oracle/_ref) on cuda:0, fp16: ms per image", "steps": steps}
    for spec in ("fh-g0", "sdpa-g0"):
        try:
            attn, gacc = parse_vit_spec(spec)
            m = DinoV2Params(ARCH)
            m.load_state_dict(params, strict=True)
            ref = RefFastViT(m.to(dev), attn=attn, gacc=gacc, dtype=torch.float16)
            with torch.no_grad():
                for _ in range(warmup):
                    ref.get_intermediate_layers(x, n=LAYERS, return_class_token=True)
                torch.cuda.synchronize()
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                for _ in range(steps):
                    ref.get_intermediate_layers(x, n=LAYERS, return_class_token=True)
                e.record()
                torch.cuda.synchronize()
            out[spec] = s.elapsed_time(e) / steps
            del ref, m
            torch.cuda.empty_cache()
        except Exception as err:  # a loader or driver refusal on this machine is a result, not a failure of the arm
            out[spec] = {"unavailable": f"{type(err).__name__}: {err}"[:300]}
    return out


def run_reference(args, rank, world):
    if rank != 0:
        return
    sec, timed, warmed, kind, what, cores = cpu_timed(args.steps, min(args.warmup, 1), CPU_SECONDS_LIMIT)
    value = 1.0 / sec
    sample = (f"{timed} whole forward pass(es) of one {IMG_H}x{IMG_W} image, each timed ({warmed} untimed before); the command asked for "
              f"{args.steps} steps / {args.warmup} warm-up, the CPU arm stops at {CPU_SECONDS_LIMIT:.0f} s of CPU time")
    line = {"impl": "reference", "metric": "images_per_s", "value": value, "unit": "img/s", "n_gpus": args.gpus, "steps": timed,
            "warmup": warmed, "steps_requested": args.steps, "warmup_requested": args.warmup, "ms_per_step": 1e3 * sec,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(), "arm": what,
            "cpu_baseline": {"value": value, "unit": "img/s", "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": "img/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    if not args.no_reference_gpu:
        line["gpu_tiers_ms_per_image"] = reference_gpu_tiers()
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------ this repository's arm
def copy_bandwidth(dev, nbytes=64 << 20, reps=5):
    """Pinned host <-> device copy rate of this rank in GB/s, (h2d, d2h), all ranks copying at the same time."""
    import torch
    from fastbb_b200 import replicas
    host = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    devbuf = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    out = []
    for src, dst in ((host, devbuf), (devbuf, host)):
        dst.copy_(src, non_blocking=True)
        torch.cuda.synchronize()
        replicas.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(reps):
            dst.copy_(src, non_blocking=True)
        e.record()
        torch.cuda.synchronize()
        out.append(nbytes * reps / (s.elapsed_time(e) * 1e-3) / 1e9)
    return out


def run_ours(args, rank, local_rank, world):
    import torch
    from fastbb_b200 import _lib, replicas
    from fastbb_b200 import vit as vit_mod
    from fastbb_b200.attention import Workspaces, attention, use_workspaces
    from fastbb_b200.models.dinov2 import dinov2
    from fastbb_b200 import synthetic as O

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU path")
    lib = _lib.load()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    params = O.make_params(ARCH, seed=0)
    fast = dinov2(ARCH, params, spec=args.spec, device=dev)
    del params
    x_host = O.make_image(1, IMG_H, IMG_W, seed=1).half().pin_memory()   # the host hands over a half-precision image
    x_dev = x_host.to(dev)
    mhz = torch.zeros(256, dtype=torch.float32, device=dev)

    def probe(slot, spin=1 << 15):
        _lib.check(lib.fbb_diag_sm_clock_mhz(mhz[slot:].data_ptr(), spin, _lib.stream_ptr(dev)))

    def step(x):
        return fast.get_intermediate_layers(x, n=LAYERS, return_class_token=True)

    # launches per step, counted on an eager pass (a graph replay launches the same kernels)
    graphs, fast.graphs = fast.graphs, False
    before = _lib.LAUNCHES
    step(x_dev)
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
    probe(0, 1 << 16)          # after the closing event: the SM clock the last steps ran at
    torch.cuda.synchronize()
    replicas.barrier()
    ms_total_ranks = replicas.gather_over_ranks(e0.elapsed_time(e1), dev)
    ms_total = max(ms_total_ranks)
    clocks = sampler.summary()
    clocks["sm_mhz_on_device_after_timed_steps"] = round(float(mhz[0]), 1)
    if world > 1:  # every rank's own GPU: a GPU that the machine slows down shows here, not in rank 0's sampler
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        code = sum(1 << i for i, n in enumerate(names) if n in clocks["reasons"])
        codes = replicas.gather_over_ranks(code, dev)
        clocks["per_rank"] = {"ms_per_step": [round(t / args.steps, 3) for t in ms_total_ranks],
                              "sm_mhz_sampled": [round(v) for v in replicas.gather_over_ranks(clocks["sm_mhz"] or 0.0, dev)],
                              "sm_mhz_on_device_after_timed_steps": [round(v) for v in replicas.gather_over_ranks(float(mhz[0]), dev)],
                              "reasons": [[n for i, n in enumerate(names) if int(c) >> i & 1] for c in codes]}
        clocks["reasons"] = sorted({n for r in clocks["per_rank"]["reasons"] for n in r})

    # ---------------- end to end: pinned host image in, pinned host features out, every step's copies inside the timing.
    # Through the package's HostPipeline: uploads and downloads run on side streams, overlapped with the next / previous
    # step's compute (each step still uploads its own image and downloads its own features).
    from fastbb_b200.pipeline import HostPipeline
    pipe = HostPipeline(step, device=dev, depth=3)
    for _ in range(8):  # enough submissions for the allocator to hold every buffer the steady state keeps in flight
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
    ms_e2e_mine = e0.elapsed_time(e1)
    ms_e2e_ranks = replicas.gather_over_ranks(ms_e2e_mine, dev)
    ms_e2e = max(ms_e2e_ranks)
    host_check = pipe.result(pipe.drain())
    assert all(torch.isfinite(p.float()).all() for p, _ in host_check), "non-finite features in the end-to-end pass"
    h2d, d2h = pipe.h2d_bytes, pipe.d2h_bytes
    bw_h2d, bw_d2h = copy_bandwidth(dev)
    bw_h2d_ranks, bw_d2h_ranks = replicas.gather_over_ranks(bw_h2d, dev), replicas.gather_over_ranks(bw_d2h, dev)

    # ---------------- instrumented pass: events around every launch of the three kernel classes, the SM clock after every
    # fourth attention launch. The per-operator host path (same kernels, same order as the C stack runner) is captured into
    # one CUDA graph with an (external) event on either side of each launch, and that graph is replayed back to back like
    # the timed steps: the times are device times without host gaps, in the clock regime the timed steps run in. The
    # event nodes keep a kernel's set-up from overlapping the previous kernel's tail, so the per-class sums are upper
    # bounds (gap_ms comes out near zero or slightly negative). Where external events are not available the same
    # brackets are taken in eager mode, which adds launch latency to every launch.
    variant = "ff" if fast.attn == "sdpa" else fast.attn
    marks = {"flash": [], "linear": [], "layernorm": []}
    real = {"attention": vit_mod.attention, "linear": vit_mod.linear, "layer_norm": vit_mod.layer_norm, "split": vit_mod.layer_norm_split,
            "linear_ln": vit_mod.linear_layer_norm}
    probes_used = [1]
    try:
        torch.cuda.Event(enable_timing=True, external=True)
        ev_kw, inst_mode = {"external": True}, "graph"
    except TypeError:
        ev_kw, inst_mode = {}, "eager"

    def bracket(kind, fn, clock_every=0):
        def wrapped(*a, **kw):
            s, e = torch.cuda.Event(enable_timing=True, **ev_kw), torch.cuda.Event(enable_timing=True, **ev_kw)
            s.record()
            o = fn(*a, **kw)
            e.record()
            marks[kind].append((s, e))
            if clock_every and len(marks[kind]) % clock_every == 0 and probes_used[0] < mhz.numel():
                probe(probes_used[0], 1 << 14)
                probes_used[0] += 1
            return o
        return wrapped

    inst_replays = max(3, min(args.steps, 10))
    fast.graphs = False
    runner_env = os.environ.get("FBB_NO_RUNNER")
    os.environ["FBB_NO_RUNNER"] = "1"
    ei0, ei1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    try:
        step(x_dev)            # untimed: the per-operator path's own first-use costs
        torch.cuda.synchronize()
        vit_mod.attention = bracket("flash", real["attention"], clock_every=4)
        vit_mod.linear = bracket("linear", real["linear"])
        vit_mod.linear_layer_norm = bracket("linear", real["linear_ln"])   # a residual GEMM with the LayerNorm after it in its launch
        vit_mod.layer_norm = bracket("layernorm", real["layer_norm"])
        vit_mod.layer_norm_split = bracket("layernorm", real["split"])
        if inst_mode == "graph":
            ig = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side), torch.cuda.graph(ig, stream=side):
                step(x_dev)
            torch.cuda.current_stream().wait_stream(side)
            for _ in range(inst_replays - 1):
                ig.replay()
            ei0.record()
            ig.replay()            # the events hold the times of this last replay
            ei1.record()
            inst_steps = 1
        else:
            inst_steps = inst_replays
            ei0.record()
            for _ in range(inst_steps):
                step(x_dev)
            ei1.record()
        torch.cuda.synchronize()
    finally:
        vit_mod.attention, vit_mod.linear, vit_mod.linear_layer_norm = real["attention"], real["linear"], real["linear_ln"]
        vit_mod.layer_norm, vit_mod.layer_norm_split = real["layer_norm"], real["split"]
        fast.graphs = graphs
        if runner_env is None:
            del os.environ["FBB_NO_RUNNER"]
        else:
            os.environ["FBB_NO_RUNNER"] = runner_env
    assert len(marks["flash"]) == DEPTH * inst_steps, "the instrumented pass did not see every attention launch"
    per_step = {k: sum(s.elapsed_time(e) for s, e in v) / inst_steps for k, v in marks.items()}
    attn_ms = [s.elapsed_time(e) for s, e in marks["flash"]]
    attn_mean_ms = sum(attn_ms) / len(attn_ms)
    inst_mhz = [float(v) for v in mhz[1:probes_used[0]].tolist() if v > 0]
    inst_mhz_med = statistics.median(inst_mhz) if inst_mhz else None

    # ---------------- the same attention launch alone (back to back from a graph), with its own clock reading
    qkv = torch.randn(1, TOKENS, 3, HEADS, 64, device=dev, dtype=torch.float16)
    q, k, v = qkv.unbind(2)
    o = torch.empty(1, TOKENS, HEADS, 64, device=dev, dtype=torch.float16)
    alone_ws = Workspaces()   # this graph's own attention scratch memory, made by the warm-up calls below
    with use_workspaces(alone_ws):
        for _ in range(3):
            attention(q, k, v, variant=variant, out=o)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side), torch.cuda.graph(g, stream=side), use_workspaces(alone_ws):
        for _ in range(10):
            attention(q, k, v, variant=variant, out=o)
    torch.cuda.current_stream().wait_stream(side)
    g.replay()
    torch.cuda.synchronize()
    e0.record()
    g.replay()
    e1.record()
    probe(0)
    torch.cuda.synchronize()
    alone_ms, alone_mhz = e0.elapsed_time(e1) / 10, float(mhz[0])

    peaks = measured_peaks()
    achieved = FLOPS_ATTN_PER_LAUNCH / (attn_mean_ms * 1e-3) / 1e12

    # ---------------- the batched configurations, split over the ranks
    configs = None
    if not args.no_configs:
        import bench_configs as BC
        cs = max(3, min(args.steps, 10))
        c3 = BC.run_c3(dev, rank, world, cs, 3, 32 if world > 1 else 4, e2e=True)
        c2 = BC.run_c2(dev, rank, world, cs, 3, 8 if world > 1 else 1, e2e=True)
        if world == 1:
            c3["note"] = "one GPU: the eight-GPU share of batch 32 (4 images)"
            c2["note"] = "one GPU: the eight-GPU share of batch 8 (1 image)"
        configs = {"c3_b32": c3, "c2_b8": c2, "scaling": "strong (fixed global batch split over the ranks)" if world > 1 else "n/a at one GPU"}

    if rank == 0:
        ms_step = ms_total / args.steps
        value = world * args.steps / (ms_total * 1e-3)
        tflops = FLOPS_PER_IMAGE / (ms_step * 1e-3) / 1e12
        kernel_ms = {"flash": per_step["flash"], "linear": per_step["linear"], "layernorm": per_step["layernorm"]}
        # what the eager instrumented step spends outside the three classes: torch's patch-row layout kernels, host gaps
        kernel_ms["other"] = max(0.0, ei0.elapsed_time(ei1) / inst_steps - sum(kernel_ms.values()))
        kernel_ms["instrumented_step_ms"] = ei0.elapsed_time(ei1) / inst_steps
        line = {
            "metric": "images_per_s", "value": value, "unit": "img/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "ms_per_image": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp16", "data": "synthetic", "config": workload_config(), "arm": f"fastbb_b200 spec {args.spec}",
            "tensor_frac": {"tflops": tflops, "of_nominal_2250": tflops / NOMINAL_FP16_TFLOPS,
                            "of_measured_burst": tflops / peaks["tflops_burst"], "of_measured_sustained": tflops / peaks["tflops_sustained"]},
            "clocks": clocks,
            "e2e": {"value": world * args.steps / (ms_e2e * 1e-3), "unit": "img/s", "ms_per_image": ms_e2e / args.steps,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "input": "fp16 pinned host image", "pipeline_depth": 3,
                    "ms_per_image_per_rank": {"min": min(ms_e2e_ranks) / args.steps, "median": statistics.median(ms_e2e_ranks) / args.steps,
                                              "max": max(ms_e2e_ranks) / args.steps},
                    "copy_gbs_needed_per_rank": (h2d + d2h) / (ms_step * 1e-3) / 1e9,
                    "pinned_copy_gbs_per_rank_all_ranks_at_once": {"h2d": [round(b, 1) for b in bw_h2d_ranks], "d2h": [round(b, 1) for b in bw_d2h_ranks]}},
            "gpu_launches": launches_per_step * args.steps,
            "kernel_ms": {**kernel_ms, "how": (f"events around every launch of the per-operator path, captured into one graph; the last of {inst_replays} back-to-back replays"
                                               if inst_mode == "graph" else f"events around every launch, eager per-operator pass of {inst_steps} step(s); per step"),
                          "gap_ms": ms_step - (kernel_ms["flash"] + kernel_ms["linear"] + kernel_ms["layernorm"])},
            "roofline": {"kernel": f"flash64_umma_kernel ({variant})", "bound": "tensor", "achieved": achieved,
                         "peak": peaks["tflops_burst"], "unit": "TFLOP/s", "frac": achieved / peaks["tflops_burst"],
                         "peak_source": f"{peaks['source']} cuBLAS bf16 burst (a kernel timed on its own; the sustained and nominal fractions are beside it)",
                         "frac_of_measured_sustained": achieved / peaks["tflops_sustained"], "frac_of_nominal_2250": achieved / NOMINAL_FP16_TFLOPS,
                         "launch_ms": attn_mean_ms, "launches_timed": len(attn_ms), "flops_per_launch": FLOPS_ATTN_PER_LAUNCH,
                         "share_of_step": per_step["flash"] / ms_step, "traffic": ATTN_DRAM_TRAFFIC_BYTES,
                         "sm_mhz_in_model": inst_mhz_med, "launch_us_x_mhz_in_model": attn_mean_ms * 1e3 * inst_mhz_med if inst_mhz_med else None,
                         "alone": {"launch_ms": alone_ms, "sm_mhz": alone_mhz, "launch_us_x_mhz": alone_ms * 1e3 * alone_mhz,
                                   "tflops": FLOPS_ATTN_PER_LAUNCH / (alone_ms * 1e-3) / 1e12}},
        }
        if configs is not None:
            line["configs"] = configs
        if world == 1 and not args.no_cpu_baseline:
            sec, timed, warmed, kind, what, cores = cpu_timed(1, 1, 45.0)
            line["cpu_baseline"] = {"value": 1.0 / sec, "unit": "img/s", "cores": cores, "kind": kind,
                                    "sample": f"{timed} whole forward pass of one {IMG_H}x{IMG_W} image, timed after {warmed} untimed pass; {what}"}
        print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--spec", default="fh-g0-graph")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="skip the batched configurations (ViT-g/14, ViT-B/16)")
    ap.add_argument("--no-reference-gpu", action="store_true", help="reference arm: skip the reference's own GPU tiers (timed after the CPU passes, for context)")
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
