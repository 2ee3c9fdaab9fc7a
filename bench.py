#!/usr/bin/env python
"""Prefill throughput of the 24-layer 606M Jarvis model (B=8 x T=2048 per GPU) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One JSON line on stdout (rank 0).  A step is one full prefill forward of the hot path over one
batch of synthetic token ids (uniform over the vocabulary) with random-init, absmean-quantised
2-bit packed weights.  `value` is whole-job tokens/s with the ids resident in HBM (nothing but the
forward inside the timed loop); `e2e` is the same through the public module API (`Jarvis.forward`)
with the ids copied from pinned host memory and the last-position logits copied back every step.

After the two timed loops a separate pass of a few steps brackets every launch of the three kernel
classes of the metric with CUDA events on the launching stream: `roofline` describes the dominant
kernel (the tcgen05 ternary GEMM, against the bf16 tensor peak: the burst figure when the SM clock
sampled during the timed loop stayed near its maximum, else the sustained one; both fractions are
given), `roofline_scans` the attention scan and the LSF scan against the HBM copy peak.

`cpu_baseline` / `--impl reference` time the CPU oracle (the reference algorithm restated in torch
fp32, weights re-quantised per call as the reference does) on a bounded sample of the same workload.

Multi-GPU: the headline line is data parallel over sequences, one independent B=8 batch per GPU
(weak scaling, no data-path collective: the block has no cross-sequence exchange apart from the
per-call LSF decay, which stays per batch).  With N > 1 the forms of the path that DO communicate are
timed afterwards and reported under `multi_gpu`:
  strong  ONE B=8 batch split over the ranks; every layer all-reduces its MoE statistics
  ep      the ternary top-2 MoE layer alone on 65,536 tokens, experts spread over the ranks, token rows
          exchanged over NVLink (Zipf(1.2)-skewed and balanced routing), against one GPU doing all of it
  cp      B=2 x T=65,536 hidden states with every sequence cut across the ranks (context parallel:
          per-layer all-gather of the scans' end states)
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
# captures of the same kernel: q/k/v 80.9 MB, out-proj + residual 111.5 MB, expert w1 + GELU 152.5 MB, expert w2
# 174.8 MB.  Below the algorithmic bytes (135 / 168 / 203 / 203 MB) because part of every output is still in L2
# when the kernel ends.
GEMM_DRAM_BYTES_PER_LAUNCH = (80.9e6 + 111.5e6 + 152.5e6 + 174.8e6) / 4
# the same two counters for one launch of the attention pipeline kernel (B=8 x T=2048: 136.3 MB algorithmic) and
# of the LSF scan with the fused f32 residual (167.8 MB algorithmic)
ATTN_DRAM_BYTES_PER_LAUNCH = 114.5e6
LSF_DRAM_BYTES_PER_LAUNCH = 112.4e6


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
                self.samples.append((time.time(), parts))

    def stop(self, t0=None, t1=None):
        """Summary of the samples read between the host times t0 and t1 (the timed region).  nvidia-smi needs a
        few hundred ms to deliver its first line, so the sampler is started before the warm-up steps; a timed
        region shorter than the sampling period takes the samples up to 0.3 s either side of it (the same
        workload runs there: warm-up before, the end-to-end steps after)."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = [s for t, s in self.samples if t0 is None or t0 <= t <= t1]
        window = "timed region"
        if not rows and t0 is not None:
            rows = [s for t, s in self.samples if t0 - 0.3 <= t <= t1 + 0.3]
            window = "timed region +- 0.3 s"
        clocks = [int(s[0]) for s in rows if s[0].isdigit()]
        mx = [int(s[1]) for s in rows if s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower() == "active" for s in rows)]
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(clocks), "window": window}


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


class KernelTimers:
    """Wraps the ops entry points of the three kernel classes of the metric (ternary GEMMs, attention scan,
    LSF scan) to bracket every launch with CUDA events on the launching stream and to add up the algorithmic
    work: 2*M*N*K flops per GEMM (grouped form: M = dispatched rows), 512 B per token-head (+ the f32 state
    written) per attention scan, bytes read + written per LSF scan (2 B per bf16 element in, 8 B per element
    for the fused f32 residual read-modify-write, or the output's element size)."""

    def __init__(self, ops):
        self.ops = ops
        self.enabled = False
        self.ev = {"gemm": [], "attn": [], "lsf": []}
        self.work = {"gemm": 0.0, "attn": 0.0, "lsf": 0.0}
        self._orig = (ops.ternary_linear, ops.ternary_linear_grouped, ops.attn_scan, ops.lsf_scan)

    def _timed(self, kind, work, fn, *a, **kw):
        if not self.enabled:
            return fn(*a, **kw)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn(*a, **kw)
        e1.record()
        self.ev[kind].append((e0, e1))
        self.work[kind] += work
        return out

    def install(self):
        lin, grp, attn, lsf = self._orig

        def t_lin(x, packed, alpha, **kw):
            return self._timed("gemm", 2.0 * x.shape[0] * x.shape[1] * packed.shape[0], lin, x, packed, alpha, **kw)

        def t_grp(x, packed, alpha, offs, **kw):
            return self._timed("gemm", 2.0 * x.shape[0] * x.shape[1] * packed.shape[1], grp, x, packed, alpha, offs, **kw)

        def t_attn(q, k, v, gamma, cos, sin, B, T, H, **kw):
            work = 512.0 * B * T * H + (B * H * 64 * 64 * 4 if kw.get("want_state") or kw.get("state_out") is not None else 0)
            return self._timed("attn", work, attn, q, k, v, gamma, cos, sin, B, T, H, **kw)

        def t_lsf(m, **kw):
            n = m.numel()
            work = float(n * m.element_size())
            if kw.get("resid") is not None:
                work += 8.0 * n
            if kw.get("want_out", True):
                work += float(n * (4 if kw.get("out_dtype") == torch.float32 else m.element_size()))
            return self._timed("lsf", work, lsf, m, **kw)

        self.ops.ternary_linear, self.ops.ternary_linear_grouped = t_lin, t_grp
        self.ops.attn_scan, self.ops.lsf_scan = t_attn, t_lsf

    def uninstall(self):
        (self.ops.ternary_linear, self.ops.ternary_linear_grouped, self.ops.attn_scan, self.ops.lsf_scan) = self._orig

    def summary(self, kind):
        ms = sum(a.elapsed_time(b) for a, b in self.ev[kind])
        return len(self.ev[kind]), ms, self.work[kind]


def _max_over_ranks(values, device, world):
    t = torch.tensor(values, dtype=torch.float64, device=device)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return [float(v) for v in t]


def _time_steps(fn, n, barrier):
    """CUDA-event time of n calls of fn in ms, bracketed by barriers."""
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    barrier()
    return e0.elapsed_time(e1)


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

    sampler = ClockSampler(local_rank)      # started here: its first line takes a few hundred ms
    sampler.start()
    for _ in range(max(args.warmup, 3)):
        step_device()
    barrier()
    assert _lib.device_status() == 0, "a bounded wait ran out during warm-up"

    # ---- device-resident throughput: nothing but the forward inside the timed loop ---------------
    _lib.kernel_launches(reset=True)
    t_begin = time.time()
    ms = _time_steps(step_device, args.steps, barrier)
    t_end = time.time()
    launches = _lib.kernel_launches(reset=True)

    # ---- end to end through the module API with host buffers ----------------------------------
    for _ in range(2):
        step_e2e()
    ms_e2e = _time_steps(step_e2e, args.steps, barrier)
    clocks = sampler.stop(t_begin, t_end)

    # ---- per-kernel pass: events around every GEMM / attention-scan / LSF-scan launch ------------
    timers = KernelTimers(ops)
    timers.install()
    timers.enabled = True
    n_prof = min(3, args.steps)
    ms_prof = _time_steps(step_device, n_prof, barrier)
    timers.enabled = False
    timers.uninstall()
    status = _lib.device_status()

    ms, ms_e2e = _max_over_ranks([ms, ms_e2e], device, world)
    peaks = measured_peaks()
    tokens = world * B * T * args.steps
    n_gemm, gemm_ms, gemm_flops = timers.summary("gemm")
    achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    # the burst peak is the honest denominator while the SM clock stays near its maximum for the whole (short)
    # timed region; under the power cap the sustained figure applies
    near_max = bool(clocks.get("sm_mhz") and clocks.get("sm_max_mhz") and clocks["sm_mhz"] >= 0.9 * clocks["sm_max_mhz"])
    peak_tf = peaks["bf16_tflops"] if near_max else peaks["bf16_tflops_sustained"]
    scans = {}
    for kind, name, traffic in (("attn", "attn_scan_pipe_kernel (+ attn_state_pass_kernel)", ATTN_DRAM_BYTES_PER_LAUNCH),
                                ("lsf", "lsf_tma_kernel (fused f32 residual)", LSF_DRAM_BYTES_PER_LAUNCH)):
        n_k, k_ms, k_bytes = timers.summary(kind)
        gbs = k_bytes / (k_ms * 1e-3) / 1e9 if k_ms > 0 else 0.0
        scans[kind + "_scan"] = {"bound": "hbm", "kernel": name, "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                 "frac": gbs / peaks["hbm_gbs"], "peak_source": f"hbm_gbs of {peaks['source']}",
                                 "traffic": traffic, "launches": n_k, "algorithmic_bytes_per_launch": k_bytes / max(n_k, 1),
                                 "avg_launch_ms": k_ms / max(n_k, 1), "share_of_step": k_ms / ms_prof}
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
                     "peak_source": f"{'bf16_tflops (burst)' if near_max else 'bf16_tflops_sustained'} of {peaks['source']}: "
                                    f"median SM clock {clocks.get('sm_mhz')} of {clocks.get('sm_max_mhz')} MHz in the timed loop",
                     "frac_burst": achieved / peaks["bf16_tflops"], "frac_sustained": achieved / peaks["bf16_tflops_sustained"],
                     "traffic": GEMM_DRAM_BYTES_PER_LAUNCH, "traffic_unit": "bytes per launch (mean of the 4 shapes, ncu)",
                     "launches": n_gemm, "flops_per_step": gemm_flops / n_prof,
                     "avg_launch_ms": gemm_ms / max(n_gemm, 1), "gemm_share_of_step": gemm_ms / ms_prof,
                     "measured_in": f"a separate pass of {n_prof} steps with events around every launch ({ms_prof / n_prof:.2f} ms per step)"},
        "roofline_scans": scans,
        "device_status": status,
    }
    if world > 1 and not args.batch_split and not args.no_multi_gpu_records:
        # The headline numbers are final at this point.  Should one of the communicating forms below stall (a rank
        # lost, a collective that never completes), the watchdog prints the line without them and ends the process
        # instead of leaving the launcher to its own time limit.
        def bail():
            if rank == 0:
                out["multi_gpu"] = {"error": f"no result within {args.multi_gpu_limit_s} s"}
                print(json.dumps(out), flush=True)
            os._exit(0)

        dog = threading.Timer(args.multi_gpu_limit_s, bail)
        dog.daemon = True
        dog.start()
        sub = multi_gpu_records(model, device, rank, world, barrier)
        dog.cancel()
        out["multi_gpu"] = sub
    return out if rank == 0 else None


# --------------------------------------------------------------------------------------------
# N > 1: the forms of the path that communicate (timed after the headline loop)
# --------------------------------------------------------------------------------------------
def multi_gpu_records(model, device, rank, world, barrier):
    """-> {"strong": ..., "ep": ..., "cp": ...}; every rank takes part, rank 0 keeps the numbers.  Each record is
    independent: an exception inside one is caught on every rank alike (the code paths do not depend on the
    rank) and reported in its place."""
    import torch.distributed as dist
    from jarvis_b200 import modules as jm, parallel as par, synthetic

    out = {}
    B, T = CFG["B"], CFG["T"]

    # ---- strong scaling: one B=8 batch split over the ranks -------------------------------------------
    try:
        if B % world:
            raise ValueError(f"world size {world} does not divide the batch of {B}")
        whole = torch.randint(0, CFG["vocab"], (B, T), generator=torch.Generator().manual_seed(77)).to(device)
        per = B // world
        mine = whole[rank * per:(rank + 1) * per].contiguous()
        strong_mine, strong_tokens = mine, B * T
        model.set_batch_split(dist.group.WORLD, global_tokens=B * T)
        for _ in range(2):
            model(mine)
        n = 5
        ms = _max_over_ranks([_time_steps(lambda: model(mine), n, barrier)], device, world)[0] / n
        model.set_batch_split(None)
        out["strong"] = {"workload": "ONE batch of B=8 x T=2048 split over the ranks (per-layer NCCL all-reduce of the MoE "
                                     "statistics keeps the LSF decay that of the unsplit batch)",
                         "ms_per_step": ms, "tok_per_s": B * T / (ms * 1e-3), "sequences_per_gpu": per}
    except Exception as exc:  # noqa: BLE001
        model.set_batch_split(None)
        out["strong"] = {"error": f"{type(exc).__name__}: {exc}"}

    # ---- expert parallel: the MoE layer alone on 65,536 tokens --------------------------------------------
    try:
        N, C, E = 65536, CFG["d_model"], CFG["n_experts"]
        if N % world or (world > E and world % E) or (world <= E and E % world):
            raise ValueError(f"world size {world} does not fit 65,536 tokens / {E} experts")
        torch.manual_seed(0)
        moe = synthetic.gaussian_ternary_(jm.SparseMoELayer(C), seed=0).to(device).eval()
        peer = (world <= E and E % world == 0) or (world > E and world % E == 0)
        ep = par.PeerExpertParallelMoE(moe, max_tokens=N // world) if peer else par.ExpertParallelMoE(moe)
        rec = {"workload": "ternary top-2 MoE layer alone, 65,536 tokens x 1024 bf16, experts 1024->2048->1024, tokens "
                           "data parallel, experts spread over the ranks, rows " +
                           ("pulled over NVLink by the gather / combine kernels (peer loads); with more ranks than experts "
                            "every expert is served by world/4 ranks" if peer
                            else "exchanged with NCCL all-to-all (uneven splits)"),
               "cases": {}}
        for case in ("zipf_1.2", "balanced"):
            if case == "zipf_1.2":
                x, w_r, shares = synthetic.zipf_router_inputs(N, C, E, seed=0)
            else:
                g = torch.Generator().manual_seed(5)
                x = torch.randn(N, C, generator=g).to(torch.bfloat16)
                w_r = (torch.rand(E, C, generator=g) * 2 - 1) / C ** 0.5
                shares = None
            with torch.no_grad():
                moe.router.weight.copy_(w_r.to(device))
            x = x.to(device)
            n_loc = N // world
            x_loc = x[rank * n_loc:(rank + 1) * n_loc].contiguous()
            if peer:
                # as in the model, where the fused norm + router kernel leaves the rows in the exchange's own buffer
                ep.ex.xn[:n_loc].copy_(x_loc)
                x_loc = ep.ex.xn[:n_loc]
            got, _ = ep.run_rows(x_loc)
            ref, _ = moe.run_rows(x_loc)
            err = float((got.float() - ref.float()).norm() / ref.float().norm())
            n = 10
            for _ in range(2):
                ep.run_rows(x_loc)
            ms = _max_over_ranks([_time_steps(lambda: ep.run_rows(x_loc), n, barrier)], device, world)[0] / n
            # one GPU doing the whole layer, timed on every rank at once (same work everywhere)
            for _ in range(2):
                moe.run_rows(x)
            ms_one = _max_over_ranks([_time_steps(lambda: moe.run_rows(x), n, barrier)], device, world)[0] / n
            recv = (ep.seg[-1:].to(torch.int64) if peer
                    else torch.tensor([sum(sum(r) for r in ep.last_recv_counts)], device=device))
            allrecv = [torch.zeros_like(recv) for _ in range(world)]
            dist.all_gather(allrecv, recv)
            rows = [int(v) for v in allrecv]
            rec["cases"][case] = {"ms": ms, "ms_one_gpu": ms_one, "speedup_vs_one_gpu": ms_one / ms,
                                  "tokens_per_s": N / (ms * 1e-3), "rows_received_per_rank": rows,
                                  "load_imbalance": max(rows) / (sum(rows) / world),
                                  "top1_shares": None if shares is None else [round(float(v), 4) for v in shares],
                                  "rel_l2_vs_single_gpu_layer": _max_over_ranks([err], device, world)[0]}
        if peer:
            ep.close()
        out["ep"] = rec
    except Exception as exc:  # noqa: BLE001
        out["ep"] = {"error": f"{type(exc).__name__}: {exc}"}

    # ---- context parallel: B=2 x T=65,536 hidden states ---------------------------------------------------
    try:
        Bc, Tc = 2, 65536
        if Tc % world:
            raise ValueError(f"world size {world} does not divide T={Tc}")
        idx = torch.randint(0, CFG["vocab"], (Bc, Tc), generator=torch.Generator().manual_seed(78)).to(device)
        tl = Tc // world
        mine = idx[:, rank * tl:(rank + 1) * tl].contiguous()
        model.set_context_parallel(dist.group.WORLD)
        for _ in range(2):
            model.hidden_rows(mine)
        n = 3
        ms = _max_over_ranks([_time_steps(lambda: model.hidden_rows(mine), n, barrier)], device, world)[0] / n
        model.set_context_parallel(None)
        out["cp"] = {"workload": "24 layers, hidden states, B=2 x T=65,536, every sequence cut into equal slices over the ranks "
                                 "(per layer: NCCL all-gather of the attention and LSF end states, all-reduce of the MoE statistics)",
                     "ms": ms, "tok_per_s": Bc * Tc / (ms * 1e-3), "tokens_per_gpu": Bc * tl}
    except Exception as exc:  # noqa: BLE001
        model.set_context_parallel(None)
        out["cp"] = {"error": f"{type(exc).__name__}: {exc}"}

    # ---- ragged state-carrying decode: 256 sequences, one token per step, sequences data parallel ----------------
    # Every rank keeps 256 / world sequences with their carried states (attention state (H, 64, 64) f32 and LSF
    # membrane per layer, prior lengths ~ U[1, 4096]); the step is one CUDA graph per rank, the per-layer all-reduce
    # of the MoE statistics inside it keeps the LSF decay that of the whole batch of 256.
    try:
        Bd = 256
        if Bd % world:
            raise ValueError(f"world size {world} does not divide {Bd} sequences")
        H, Cm, L = CFG["n_heads"], CFG["d_model"], len(model.blocks)

        def decode_ms(n_seq, seed, split):
            g = torch.Generator(device=device).manual_seed(seed)
            pos = torch.randint(1, 4097, (n_seq,), generator=g, device=device, dtype=torch.int32)
            state = {"h": [torch.randn(n_seq, Cm, generator=g, device=device) for _ in range(L)],
                     "S": [torch.randn(n_seq, H, 64, 64, generator=g, device=device) for _ in range(L)]}
            toks = torch.randint(0, CFG["vocab"], (4, n_seq, 1), generator=g, device=device)
            model.set_batch_split(dist.group.WORLD if split else None, global_tokens=Bd if split else None)
            sess = jm.DecodeSession(model, state, pos, max_position=4096 + 64).capture()
            for i in range(2):
                sess.step(toks[i])
            n = 16
            ms = _max_over_ranks([_time_steps(lambda: sess.step(toks[0]), n, barrier)], device, world)[0] / n
            model.set_batch_split(None)
            del sess, state
            torch.cuda.empty_cache()
            return ms

        ms = decode_ms(Bd // world, 900 + rank, True)
        ms_one = decode_ms(Bd, 900, False)        # one GPU holding all 256 sequences, timed on every rank at once
        out["decode"] = {"workload": "606M model, 256 sequences x 1 token per step, carried f32 state, ragged positions, "
                                     "sequences split over the ranks (CUDA-graphed step, per-layer NCCL all-reduce of the "
                                     "MoE statistics inside the graph)",
                         "ms_per_step": ms, "tok_per_s": Bd / (ms * 1e-3), "sequences_per_gpu": Bd // world,
                         "ms_per_step_one_gpu": ms_one, "speedup_vs_one_gpu": ms_one / ms}
    except Exception as exc:  # noqa: BLE001
        model.set_batch_split(None)
        out["decode"] = {"error": f"{type(exc).__name__}: {exc}"}

    # ---- strong scaling again, the split forward captured in a CUDA graph (last: a failed capture ends the records) --
    # From Python the ~340 launches of a forward cost several ms of host time, which a 14 ms step hides and a split
    # batch does not; a replay is one launch (the per-layer NCCL all-reduce is captured with it).
    if "ms_per_step" in out.get("strong", {}):
        try:
            model.set_batch_split(dist.group.WORLD, global_tokens=strong_tokens)
            sess = jm.PrefillSession(model, strong_mine.shape[0], strong_mine.shape[1], device).capture()
            for _ in range(2):
                sess(strong_mine)
            n = 5
            ms = _max_over_ranks([_time_steps(lambda: sess(strong_mine), n, barrier)], device, world)[0] / n
            out["strong"]["ms_per_step_cuda_graph"] = ms
            out["strong"]["tok_per_s_cuda_graph"] = strong_tokens / (ms * 1e-3)
        except Exception as exc:  # noqa: BLE001
            out["strong"]["cuda_graph_error"] = f"{type(exc).__name__}: {exc}"
        model.set_batch_split(None)
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
    ap.add_argument("--no-multi-gpu-records", action="store_true",
                    help="N > 1: skip the strong-scaling / expert-parallel / context-parallel records")
    ap.add_argument("--multi-gpu-limit-s", type=float, default=240.0,
                    help="N > 1: time limit of those records; past it the line is printed without them")
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
