#!/usr/bin/env python
"""Decode-attention benchmark: factorized-K + RoPE GQA decode with dense V (the qAB_rope
configuration: batch 16, 32 query / 8 KV heads, head_dim 128, context 16384, rank 512, bf16).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one decode-attention call over the whole batch (one new token per sequence, one
layer).  Prints ONE JSON line (rank 0).  `value` is tokens/s with inputs resident in HBM;
`e2e` is the same call through the public Python API with every input copied from pinned host
memory and the output read back inside the timed region.  With N > 1 (torchrun, one rank per
GPU) every rank holds its own batch shard of the same size (weak scaling) and the step ends
with an NCCL all-gather of the outputs.

--impl reference times the reference's eager CPU math (the oracle port; the reference itself is
Python that is not present on the GPU box) on the host cores, on a bounded sample of the batch.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode_attn_tokens_per_s"
UNIT = "tokens/s"


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


def cpu_reference_throughput(cfg, rows: int, reps: int, warmup: int):
    """The reference's eager path (oracle port) on the host cores: tokens/s on `rows` batch rows
    at full context, in the configuration dtype and in fp32; the faster of the two is reported."""
    from kernel_collections_b200 import synthetic
    from oracle import xkv_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    A, B, q, V = synthetic.recon_rope_inputs(cfg, seed=0, batch_rows=rows)
    B4 = B.view(cfg.rank, cfg.num_kv_heads, cfg.head_dim).permute(1, 0, 2)[None].expand(rows, -1, -1, -1)
    qr = O.rope_query(q, cfg.theta, cfg.kv_len)
    Vt = V.transpose(1, 2)
    best = {}
    for dt in (cfg.dtype, torch.float32):
        ts = []
        for i in range(warmup + reps):
            t0 = time.perf_counter()
            O.recon_rope_decode(qr, A, B4, Vt, cfg.theta, compute_dtype=dt)
            dtm = time.perf_counter() - t0
            if i >= warmup:
                ts.append(dtm)
        best[str(dt).replace("torch.", "")] = rows / statistics.median(ts)
    name = max(best, key=best.get)
    return best[name], name, best


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-rows", type=int, default=4, help="batch rows of the CPU-baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--small", action="store_true", help="context 4096 (profiling-sized case, 0.2 GB of inputs)")
    ap.add_argument("--force-generic", action="store_true")
    ap.add_argument("--workload", default="c2", choices=["c2", "c5"],
                    help="c2: the headline configuration (default).  c5: one GPU's 16-row shard of the long-context "
                         "sweep (64 query heads, rank 1024, context 131072); inputs drawn on the device, no e2e leg")
    args = ap.parse_args()

    from kernel_collections_b200 import synthetic
    cfg = synthetic.ReconRopeConfig()
    if args.workload == "c5":
        cfg = cfg.scaled(name="c5_shard_b16_of_128_L131072_R1024_H64", batch=16, num_heads=64, kv_len=131072, rank=1024)
    if args.small:
        cfg = cfg.scaled(kv_len=4096, name="c2_small_L4096")
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    config = {"workload": cfg.name, "batch_per_gpu": cfg.batch, "global_batch": cfg.batch * world,
              "num_heads": cfg.num_heads, "num_kv_heads": cfg.num_kv_heads, "head_dim": cfg.head_dim,
              "kv_len": cfg.kv_len, "rank": cfg.rank, "rope_theta": cfg.theta, "value": "dense",
              "parallelism": f"batch-shard x{world}" + (" + NCCL all-gather of outputs" if world > 1 else ""),
              "l2_policy": f"inputs ({cfg.algorithmic_bytes() / 1e9:.2f} GB per GPU) exceed the 126 MB L2"}

    if args.impl == "reference":
        if rank != 0:
            return
        rows = max(1, args.cpu_rows)
        warm = min(args.warmup, 1)
        reps = max(1, min(args.steps, 3))
        v, name, both = cpu_reference_throughput(cfg, rows, reps, warm)
        cores = torch.get_num_threads()
        line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus,
                "steps": reps, "warmup": warm, "ms_per_step": 1e3 * rows / v, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": name, "data": "synthetic", "config": config,
                "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                                 "sample": f"{rows} of {cfg.batch} batch rows at full context, median of {reps}",
                                 "by_dtype": both},
                "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    import kernel_collections_b200 as K
    from kernel_collections_b200 import _C, dist as xdist
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    big = args.workload == "c5"          # tens of GB: drawn on the device, e2e leg skipped
    if big:
        g = torch.Generator(device=dev).manual_seed(rank)
        KD = cfg.num_kv_heads * cfg.head_dim
        dA = torch.randn(cfg.batch, cfg.kv_len, cfg.rank, generator=g, device=dev, dtype=cfg.dtype)
        dB = (torch.randn(cfg.rank, KD, generator=g, device=dev) / cfg.rank ** 0.5).to(cfg.dtype)
        dV = torch.randn(cfg.batch, cfg.kv_len, cfg.num_kv_heads, cfg.head_dim, generator=g, device=dev, dtype=cfg.dtype)
        dq = K.rope_query(torch.randn(cfg.batch, cfg.num_heads, 1, cfg.head_dim, generator=g, device=dev).to(cfg.dtype),
                          cfg.theta, cfg.kv_len)
        h2d = d2h = 0
    else:
        A, B, q, V = synthetic.recon_rope_inputs(cfg, seed=rank)
        hA, hB, hq, hV = (t.pin_memory() for t in (A, B, q, V))
        dA, dB, dV = hA.to(dev), hB.to(dev), hV.to(dev)
        dq = K.rope_query(hq.to(dev), cfg.theta, cfg.kv_len)
        hq = dq.cpu().pin_memory()          # the rotated query is what a caller hands over each step
        h2d = sum(t.numel() * t.element_size() for t in (hA, hB, hq, hV))
        out_host = torch.empty((cfg.batch * world, cfg.num_heads, 1, cfg.head_dim), dtype=cfg.dtype).pin_memory()
        d2h = out_host.numel() * out_host.element_size()

    def step(a, b_, qq, v):
        o = K.recon_rope_decode(qq, a, b_, v.transpose(1, 2), theta=cfg.theta, force_generic=args.force_generic)
        if world > 1:
            o = xdist.all_gather_outputs(o, cfg.batch * world)
        return o

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    from kernel_collections_b200 import ops as _ops, attention as _att
    plan = _ops.plan(score_mode=_C.SCORE_RECON_ROPE, value_mode=_C.VALUE_DENSE, q=dq[:, :, 0],
                                k=dA, k_proj=_att.as_key_proj(dB, cfg.head_dim), v=dV,
                                sm_scale=cfg.head_dim ** -0.5, theta=cfg.theta, force_generic=args.force_generic)
    launches_per_step = 3 + (1 if world > 1 else 0)

    # ---- device-resident timing ---------------------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        step(dA, dB, dq, dV)
    barrier()
    sampler = ClockSampler(local_rank)
    stream = torch.cuda.current_stream()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    ev[0].record(stream)
    for i in range(args.steps):
        step(dA, dB, dq, dV)
        ev[i + 1].record(stream)
    barrier()
    clocks = sampler.stop()
    per_step = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]
    total_ms = ev[0].elapsed_time(ev[-1])

    # ---- end to end: pinned host -> device, call, result -> host ---------------------------------
    e2e_steps = max(3, min(args.steps, 10))
    e2e_ms = float("nan")
    if not big:
        bufs = [torch.empty_like(t, device=dev) for t in (hA, hB, hq, hV)]

        def e2e_step():
            for dst, src in zip(bufs, (hA, hB, hq, hV)):
                dst.copy_(src, non_blocking=True)
            o = step(*bufs)
            out_host.copy_(o, non_blocking=True)

        e2e_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(e2e_steps):
            e2e_step()
        e1.record(stream)
        barrier()
        e2e_ms = e0.elapsed_time(e1)

    t = torch.tensor([total_ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    total_ms, e2e_ms = t.tolist()
    if rank != 0:
        if world > 1:
            torch.distributed.destroy_process_group()
        return

    ms_per_step = total_ms / args.steps
    tokens = cfg.batch * world
    value = tokens / (ms_per_step * 1e-3)
    peaks = load_peaks()
    kern_ms = statistics.mean(per_step)      # whole step (all launches) charged to the dominant kernel
    tflops = cfg.algorithmic_flops() / (kern_ms * 1e-3) / 1e12
    gbs = cfg.algorithmic_bytes() / (kern_ms * 1e-3) / 1e9
    t_hbm = cfg.algorithmic_bytes() / (peaks["hbm_gbs"] * 1e9)
    t_tc = cfg.algorithmic_flops() / (peaks["bf16_tflops"] * 1e12)
    bound = "tensor" if t_tc >= t_hbm else "hbm"
    roof = {"bound": bound, "kernel": plan,
            "achieved": tflops if bound == "tensor" else gbs,
            "peak": peaks["bf16_tflops"] if bound == "tensor" else peaks["hbm_gbs"],
            "unit": "TFLOP/s" if bound == "tensor" else "GB/s",
            "frac": (tflops / peaks["bf16_tflops"]) if bound == "tensor" else gbs / peaks["hbm_gbs"],
            "traffic": None, "peak_source": peaks["source"] + " (burst)",
            "hbm_gbs": gbs, "hbm_frac": gbs / peaks["hbm_gbs"], "tensor_tflops": tflops,
            "tensor_frac": tflops / peaks["bf16_tflops"],
            "latent_stream_gbs": cfg.latent_bytes() / (kern_ms * 1e-3) / 1e9,
            "algorithmic_bytes": cfg.algorithmic_bytes(), "algorithmic_flops": cfg.algorithmic_flops(),
            "timed": "CUDA events around each step on the launching stream; step time charged to the dominant kernel"}
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": str(cfg.dtype).replace("torch.", ""),
            "data": "synthetic", "config": config, "clocks": clocks,
            "e2e": {"value": None if big else tokens / (e2e_ms / e2e_steps * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "note": "all inputs (latent, B, q, dense V) copied from pinned host memory every step"},
            "gpu_launches": launches_per_step * args.steps, "roofline": roof}
    if world == 1 and not args.no_cpu_baseline and not big:
        v, name, both = cpu_reference_throughput(cfg, max(1, args.cpu_rows), 5, 1)
        line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                                "dtype": name, "by_dtype": both,
                                "sample": f"{args.cpu_rows} of {cfg.batch} batch rows at full context, median of 5"}
    print(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
