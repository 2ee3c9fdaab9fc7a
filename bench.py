#!/usr/bin/env python
"""Prefill throughput of the 24-layer 606M Jarvis model (B=8 x T=2048 per GPU) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One JSON line on stdout (rank 0).  A step is one full prefill forward of the hot path over one
batch of synthetic token ids (uniform over the vocabulary) with random-init, absmean-quantised
2-bit packed weights.  `value` is whole-job tokens/s with the ids resident in HBM; `e2e` is the same
through the public module API (`Jarvis.forward`) with the ids copied from pinned host memory and the
last-position logits copied back every step.  `roofline` describes the dominant kernel (the tcgen05
ternary GEMM) from CUDA events recorded around every one of its launches inside the timed region.
`cpu_baseline` / `--impl reference` time the CPU oracle (the reference algorithm restated in torch
fp32, weights re-quantised per call as the reference does) on a bounded sample of the same workload.
Multi-GPU: sequences are data-parallel, one independent B=8 batch per GPU (weak scaling); the block
has no cross-sequence exchange apart from the per-call LSF decay, which stays per batch.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(vocab=50257, d_model=1024, n_layers=24, n_heads=16, n_experts=4, top_k=2, B=8, T=2048)


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of each of the four GEMM shapes of a layer, from ncu
# captures of the same kernel (profiles/ternary_gemm_kernel_qkv_and_w2.md): q/k/v 80.9 MB, out-proj + residual
# 111.5 MB, expert w1 + GELU 152.5 MB, expert w2 174.8 MB.  Below the algorithmic bytes (135 / 168 / 203 / 203 MB)
# because part of every output is still in L2 when the kernel ends.
GEMM_DRAM_BYTES_PER_LAUNCH = (80.9e6 + 111.5e6 + 152.5e6 + 174.8e6) / 4


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks = [int(s[0]) for s in self.samples if s[0].isdigit()]
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower() == "active" for s in self.samples)]
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(clocks)}


# --------------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------------
def build_model(device, seed=0):
    import jarvis_b200
    from jarvis_b200 import modules as jm

    with torch.device(device):
        model = jm.Jarvis(vocab_size=CFG["vocab"], d_model=CFG["d_model"], n_layers=CFG["n_layers"],
                          n_heads=CFG["n_heads"], num_experts=CFG["n_experts"], top_k=CFG["top_k"],
                          max_seq_len=CFG["T"])
    gen = torch.Generator(device=device).manual_seed(seed)
    with torch.no_grad():
        for m in model.modules():
            if isinstance(m, jm.TernaryLinear):
                m.weight.copy_(torch.randn(m.weight.shape, generator=gen, device=device) * 0.02)
        for blk in model.blocks:
            blk.attn.gamma_raw.copy_(torch.logit(torch.rand(CFG["n_heads"], generator=gen, device=device) * 0.099 + 0.9))
    return model.eval()


class GemmTimer:
    """Wraps ops.ternary_linear / ternary_linear_grouped to bracket every launch with CUDA events on
    the launching stream and to add up the algorithmic flops (2*M*N*K; for the grouped form M is the
    number of dispatched rows)."""

    def __init__(self, ops):
        self.ops = ops
        self.events = []
        self.flops = 0.0
        self.enabled = False
        self._lin, self._grp = ops.ternary_linear, ops.ternary_linear_grouped

    def install(self):
        def lin(x, packed, alpha, **kw):
            if not self.enabled:
                return self._lin(x, packed, alpha, **kw)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            out = self._lin(x, packed, alpha, **kw)
            b.record()
            self.events.append((a, b))
            self.flops += 2.0 * x.shape[0] * x.shape[1] * packed.shape[0]
            return out

        def grp(x, packed, alpha, offs, **kw):
            if not self.enabled:
                return self._grp(x, packed, alpha, offs, **kw)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            out = self._grp(x, packed, alpha, offs, **kw)
            b.record()
            self.events.append((a, b))
            self.flops += 2.0 * x.shape[0] * x.shape[1] * packed.shape[1]
            return out

        self.ops.ternary_linear, self.ops.ternary_linear_grouped = lin, grp

    def summary(self):
        ms = sum(a.elapsed_time(b) for a, b in self.events)
        return len(self.events), ms, self.flops


def run_ours(args, rank, world, local_rank):
    import jarvis_b200
    from jarvis_b200 import _lib, ops

    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    model = build_model(device, seed=0)
    B, T = CFG["B"], CFG["T"]
    if args.batch_split and world > 1:
        assert B % world == 0, "--batch-split needs a world size that divides the batch of 8"
        model.set_batch_split(torch.distributed.group.WORLD, global_tokens=B * T)
        B //= world
    gen = torch.Generator(device=device).manual_seed(1000 + rank)
    idx_dev = torch.randint(0, CFG["vocab"], (B, T), generator=gen, device=device)
    idx_host = idx_dev.cpu().pin_memory()
    last_host = torch.empty((B, CFG["vocab"]), dtype=torch.bfloat16).pin_memory()
    timer = GemmTimer(ops)
    timer.install()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            torch.distributed.barrier()
            torch.cuda.synchronize()

    def step_device():
        return model(idx_dev)[0]

    def step_e2e():
        idx = idx_host.to(device, non_blocking=True)
        logits = model(idx)[0]
        last_host.copy_(logits[:, -1, :], non_blocking=True)
        return logits

    for _ in range(max(args.warmup, 3)):
        step_device()
    barrier()
    assert _lib.device_status() == 0, "a bounded wait ran out during warm-up"

    # ---- device-resident throughput ------------------------------------------------------------
    sampler = ClockSampler(local_rank)
    sampler.start()
    _lib.kernel_launches(reset=True)
    timer.enabled = True
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step_device()
    e1.record()
    barrier()
    timer.enabled = False
    launches = _lib.kernel_launches(reset=True)
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    n_gemm, gemm_ms, gemm_flops = timer.summary()

    # ---- end to end through the module API with host buffers ----------------------------------
    for _ in range(2):
        step_e2e()
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(args.steps):
        step_e2e()
    f1.record()
    barrier()
    ms_e2e = f0.elapsed_time(f1)
    status = _lib.device_status()

    t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=device)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    ms, ms_e2e = float(t[0]), float(t[1])
    if rank != 0:
        return None
    peaks = measured_peaks()
    tokens = world * B * T * args.steps
    achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    peak_tf = peaks["bf16_tflops_sustained"]
    out = {
        "metric": "prefill tok/s (606M, B=8xT=2048)", "value": tokens / (ms * 1e-3), "unit": "tok/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "strong" if (args.batch_split and world > 1) else "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "24-layer 606M Jarvis prefill, vocab 50257, B=8 x T=2048 per GPU, 2-bit packed "
                               "ternary weights (seeded Gaussian init, absmean), token ids uniform over the vocab",
                   "per_gpu_batch": B, "seq_len": T, "parallelism": (f"dp{world}, one batch of 8 split over the ranks, per-layer all-reduce of the MoE statistics"
                                   if (args.batch_split and world > 1) else f"dp{world} (independent batches, no collective)"),
                   "l2": "activations per step (>2 GB incl. logits) exceed the 126 MB L2; no explicit flush"},
        "e2e": {"value": tokens / (ms_e2e * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": idx_host.numel() * 8,
                "d2h_bytes_per_step": last_host.numel() * 2,
                "result": "last-position logits of every sequence (bf16), read back to pinned host memory"},
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "ternary_gemm_kernel (tcgen05)", "achieved": achieved,
                     "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf,
                     "peak_source": f"bf16_tflops_sustained of {peaks['source']}",
                     "traffic": GEMM_DRAM_BYTES_PER_LAUNCH, "traffic_unit": "bytes per launch (mean of the 4 shapes, ncu)",
                     "launches": n_gemm, "flops_per_step": gemm_flops / args.steps,
                     "avg_launch_ms": gemm_ms / max(n_gemm, 1), "gemm_share_of_step": gemm_ms / ms},
        "device_status": status,
    }
    return out


# --------------------------------------------------------------------------------------------
# CPU oracle arm (reference algorithm on the host cores)
# --------------------------------------------------------------------------------------------
def cpu_state_dict(seed=0):
    """fp32 CPU weights with the benchmark's recipe (values differ from the GPU arm's draw; the CPU
    arm is timed, not compared)."""
    g = torch.Generator().manual_seed(seed)
    C, E = CFG["d_model"], CFG["n_experts"]
    sd = {"tok_emb.weight": torch.randn(CFG["vocab"], C, generator=g), "final_norm.weight": torch.ones(C),
          "lm_head.weight": torch.randn(CFG["vocab"], C, generator=g) * 0.02}
    for i in range(CFG["n_layers"]):
        p = f"blocks.{i}."
        for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
            sd[p + f"attn.{n}.weight"] = torch.randn(C, C, generator=g) * 0.02
        sd[p + "attn.gamma_raw"] = torch.logit(torch.rand(CFG["n_heads"], generator=g) * 0.099 + 0.9)
        sd[p + "norm1.weight"] = torch.ones(C)
        sd[p + "norm2.weight"] = torch.ones(C)
        sd[p + "moe.router.weight"] = (torch.rand(E, C, generator=g) * 2 - 1) / C ** 0.5
        for e in range(E):
            sd[p + f"moe.w1.{e}.weight"] = torch.randn(2 * C, C, generator=g) * 0.02
            sd[p + f"moe.w2.{e}.weight"] = torch.randn(C, 2 * C, generator=g) * 0.02
        sd[p + "liquid.var_scale"] = torch.tensor(1.0)
    return sd


def time_cpu_oracle(steps, warmup, limit_s):
    """Times oracle.model_forward on (1, T_s) token ids; T_s is the largest of 2048/1024/512/256 whose
    projected total stays within limit_s.  Returns (tok/s, seconds per step, T_s, cores)."""
    from oracle import jarvis_oracle as orc

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    sd = cpu_state_dict()
    g = torch.Generator().manual_seed(7)

    def run(T):
        idx = torch.randint(0, CFG["vocab"], (1, T), generator=g)
        t0 = time.perf_counter()
        with torch.no_grad():
            orc.model_forward(idx, sd, CFG["n_layers"], CFG["n_heads"])
        return time.perf_counter() - t0

    probe = run(256)
    T_s = 256
    for cand in (2048, 1024, 512):
        if probe * (cand / 256) * 1.3 * (steps + warmup) <= limit_s:   # ~linear in T with a T^2 LSF term
            T_s = cand
            break
    for _ in range(warmup):
        run(T_s)
    times = [run(T_s) for _ in range(steps)]
    sec = statistics.median(times)
    return T_s / sec, sec, T_s, cores


def run_reference(args, rank, world):
    if rank != 0:
        return None
    tps, sec, T_s, cores = time_cpu_oracle(args.steps, args.warmup, limit_s=200.0)
    sample = f"1 of the 8 sequences, first {T_s} of 2048 positions, all 24 layers + lm_head, fp32, per step"
    return {
        "impl": "reference", "metric": "prefill tok/s (606M, B=8xT=2048)", "value": tps, "unit": "tok/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "24-layer 606M Jarvis prefill, vocab 50257 (CPU: bounded sample per step)",
                   "sample": sample},
        "cpu_baseline": {"value": tps, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU oracle leg of the default run")
    ap.add_argument("--batch-split", action="store_true",
                    help="strong scaling: ONE B=8 batch split over the ranks, MoE statistics all-reduced per layer")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        out = run_reference(args, rank, world)
        if out is not None:
            print(json.dumps(out), flush=True)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the sm_100a path has no CPU fallback (use --impl reference)")
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    out = run_ours(args, rank, world, local_rank)
    if out is not None:
        if world == 1 and not args.no_cpu_baseline:
            tps, sec, T_s, cores = time_cpu_oracle(steps=1, warmup=0, limit_s=40.0)
            out["cpu_baseline"] = {
                "value": tps, "unit": "tok/s", "cores": cores, "kind": "port",
                "sample": f"1 of the 8 sequences, first {T_s} of 2048 positions, all 24 layers + lm_head, fp32, "
                          f"one pass ({sec:.1f} s)"}
        print(json.dumps(out), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
