#!/usr/bin/env python
"""Per-kernel timing against the measured roofline (one kernel class per invocation).

    python jarvis-q1.58-500m_b200/kernel_bench.py gemm --M 16384 --N 3072 --K 1024 [--groups 4] [--epilogue 0]
    python jarvis-q1.58-500m_b200/kernel_bench.py attn --B 32 --H 16 --T 2048
    python jarvis-q1.58-500m_b200/kernel_bench.py lsf  --B 32 --T 2048 --C 1024 [--resid]
    python jarvis-q1.58-500m_b200/kernel_bench.py moe  --N 65536 [--zipf 1.2]

Prints one JSON line: average launch time from CUDA events on the launching stream (3 warm-up
launches, L2 flushed between timed launches by writing a 256 MiB buffer), algorithmic bytes or flops
per launch and the fraction of the peak measured on this machine class (a JSON file of copy bandwidth and
bf16 GEMM throughput at the repository root; without it 6650 GB/s and 1590 TFLOP/s, and the line says "fallback").
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import jarvis_b200  # noqa: E402
from jarvis_b200 import _lib, ops  # noqa: E402


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def timeit(fn, iters, flush=True):
    # L2 flush: a 256 MiB buffer is written twice before every timed launch (~90 us of device work, so the host has
    # queued the launch, with its allocations, tensor maps and ctypes call, before the device gets there)
    scratch = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush:
            scratch.fill_(1)
            scratch.fill_(2)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    assert _lib.device_status() == 0
    return total / iters


def report(name, ms, *, bytes_=None, flops=None, extra=None):
    hbm, tf, src = peaks()
    out = {"kernel": name, "ms": ms}
    if bytes_ is not None:
        out.update(bound="hbm", achieved=bytes_ / ms / 1e6, peak=hbm, unit="GB/s", algorithmic_bytes=bytes_)
    else:
        out.update(bound="tensor", achieved=flops / ms / 1e9, peak=tf, unit="TFLOP/s", algorithmic_flops=flops)
    out["frac"] = out["achieved"] / out["peak"]
    out["peak_source"] = src + (" burst bf16" if flops is not None else " copy")
    out.update(extra or {})
    print(json.dumps(out), flush=True)


def case_gemm(a):
    g = torch.Generator(device="cuda").manual_seed(0)
    G = a.groups
    x = torch.randn(a.M, a.K, generator=g, device="cuda").bfloat16()
    codes = torch.randint(0, 3, (G, a.N, a.K // 4, 4), generator=g, device="cuda", dtype=torch.uint8)
    packed = (codes[..., 0] | (codes[..., 1] << 2) | (codes[..., 2] << 4) | (codes[..., 3] << 6)).contiguous()
    if a.prepared:
        packed = ops.prepare_weights(packed)
    alpha = torch.full((G,), 0.016, device="cuda")
    epi = a.epilogue
    odt = torch.bfloat16 if epi in (0, 1) else torch.float32
    out = torch.zeros(a.M, a.N, dtype=odt, device="cuda")
    if G == 1:
        fn = lambda: ops.ternary_linear(x, packed[0], alpha, epilogue=epi, out=out, token_tile=a.tile,
                                        prepared=a.prepared)  # noqa: E731
    else:
        cuts = torch.linspace(0, a.M, G + 1).round().to(torch.int32).cuda()
        fn = lambda: ops.ternary_linear_grouped(x, packed, alpha, cuts, epilogue=epi, out=out, token_tile=a.tile,
                                                prepared=a.prepared)  # noqa: E731
    ms = timeit(fn, a.iters)
    report("ternary_gemm_kernel", ms, flops=2.0 * a.M * a.N * a.K, extra={"M": a.M, "N": a.N, "K": a.K, "groups": G,
                                                                         "epilogue": epi, "token_tile": a.tile,
                                                                         "prepared_layout": bool(a.prepared)})


def case_attn(a):
    g = torch.Generator(device="cuda").manual_seed(0)
    C = a.H * 64
    qkv = torch.randn(a.B * a.T, 3 * C, generator=g, device="cuda").bfloat16()
    gamma = torch.rand(a.H, generator=g, device="cuda") * 0.099 + 0.9
    t = torch.arange(a.T, dtype=torch.float32, device="cuda")
    inv = 1.0 / (10000.0 ** (torch.arange(0, 64, 2, device="cuda").float() / 64))
    fr = torch.outer(t, inv)
    cos, sin = fr.cos().contiguous(), fr.sin().contiguous()
    o = torch.empty(a.B * a.T, C, dtype=torch.bfloat16, device="cuda")
    if a.T == 1:
        # the decode step: carried f32 state (B, H, 64, 64) updated in place, ragged positions
        S = torch.randn(a.B, a.H, 64, 64, generator=g, device="cuda")
        pos = torch.randint(0, 4096, (a.B,), generator=g, device="cuda", dtype=torch.int32)
        t = torch.arange(4097, dtype=torch.float32, device="cuda")
        fr = torch.outer(t, inv)
        cos, sin = fr.cos().contiguous(), fr.sin().contiguous()
        fn = lambda: ops.attn_scan(qkv[:, :C], qkv[:, C:2 * C], qkv[:, 2 * C:], gamma, cos, sin, a.B, 1, a.H,  # noqa: E731
                                   start_pos=pos, state_in=S, want_state=True, state_out=S, out=o)
        ms = timeit(fn, a.iters)
        report("attn_decode_stream_kernel" if a.B * a.H >= 64 else "attn_decode_kernel", ms,
               bytes_=2.0 * a.B * a.H * 64 * 64 * 4 + 512.0 * a.B * a.H, extra={"B": a.B, "H": a.H, "T": 1})
        return
    fn = lambda: ops.attn_scan(qkv[:, :C], qkv[:, C:2 * C], qkv[:, 2 * C:], gamma, cos, sin, a.B, a.T, a.H,  # noqa: E731
                               want_state=True, out=o)
    ms = timeit(fn, a.iters)
    by = 512.0 * a.B * a.H * a.T + a.B * a.H * 64 * 64 * 4
    report("attn_scan_kernel", ms, bytes_=by, extra={"B": a.B, "H": a.H, "T": a.T,
                                                     "tflops_side": 32768.0 * a.B * a.H * a.T / ms / 1e9})


def case_lsf(a):
    g = torch.Generator(device="cuda").manual_seed(0)
    m = torch.randn(a.B, a.T, a.C, generator=g, device="cuda").bfloat16()
    al = torch.tensor([0.95], device="cuda")
    if a.resid:
        r = torch.randn(a.B, a.T, a.C, generator=g, device="cuda")
        fn = lambda: ops.lsf_scan(m, alpha_scalar=al, resid=r, want_out=False)  # noqa: E731
        by = 10.0 * m.numel()
    else:
        fn = lambda: ops.lsf_scan(m, alpha_scalar=al)  # noqa: E731
        by = 4.0 * m.numel()
    ms = timeit(fn, a.iters)
    report("lsf_scan_kernel", ms, bytes_=by, extra={"B": a.B, "T": a.T, "C": a.C, "fused_residual": bool(a.resid)})


def case_moe(a):
    """Config 4: one ternary top-2 MoE layer on N tokens, top-1 loads skewed Zipf(s) by a constant
    input feature with per-expert router offsets."""
    from jarvis_b200 import modules as jm
    torch.manual_seed(0)
    C = 1024
    moe = jm.ternary_init_(jm.SparseMoELayer(C)).cuda().eval()
    x = torch.randn(a.N, C, device="cuda")
    x[:, 0] = 1.0
    if a.zipf > 0:
        w = torch.tensor([1.0 / (i + 1) ** a.zipf for i in range(4)])
        with torch.no_grad():
            moe.router.weight[:, 0] = (torch.log(w / w.sum()) * 1.6).cuda()
    xb = x.bfloat16()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world == 1:
        fn = lambda: moe.run_rows(xb)  # noqa: E731
        ms = timeit(fn, a.iters)
        counts = moe.last_routing[2][0].cpu().tolist()
        report("moe_layer (router..combine)", ms, flops=2.0 * 2 * a.N * (2 * C * C) * 2,
               extra={"N": a.N, "slot_counts": counts, "tokens_per_s": a.N / ms * 1e3})
        return
    # expert parallel: tokens data-parallel (contiguous ranges), experts spread over the ranks,
    # NCCL all-to-all for dispatch and return; time = max over ranks of the CUDA-event time
    import torch.distributed as dist
    from jarvis_b200 import parallel as par
    rank = dist.get_rank()
    n_loc = a.N // world
    x_loc = xb[rank * n_loc:(rank + 1) * n_loc].contiguous()
    ep = par.PeerExpertParallelMoE(moe, max_tokens=n_loc) if a.peer else par.ExpertParallelMoE(moe)
    out, _ = ep.run_rows(x_loc)
    ref, _ = moe.run_rows(x_loc)
    err = float((out.float() - ref.float()).norm() / ref.float().norm())
    assert err < 1e-6, f"expert-parallel result differs from the single-GPU layer: {err}"
    dist.barrier()
    ms = timeit(lambda: ep.run_rows(x_loc), a.iters)
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if a.peer:
        recv = ep.seg[-1:].to(torch.int64)          # rows this rank's experts received (device count)
    else:
        recv = torch.tensor([sum(r) for r in ep.last_recv_counts], device="cuda").sum().reshape(1)
    allrecv = [torch.zeros_like(recv) for _ in range(world)]
    dist.all_gather(allrecv, recv)
    if rank == 0:
        ms = float(t[0])
        name = ("moe_layer expert-parallel over peer memory (router, pull-gather, experts, pull-combine)" if a.peer
                else "moe_layer expert-parallel (router, all-to-all, experts, all-to-all, combine)")
        report(name, ms,
               flops=2.0 * 2 * a.N * (2 * C * C) * 2,
               extra={"N": a.N, "n_gpus": world, "tokens_per_s": a.N / ms * 1e3, "rel_l2_vs_single_gpu": err,
                      "rows_received_per_rank": [int(v) for v in allrecv]})
    if a.peer:
        ep.close()


def case_router(a):
    """norm2 + top-2 router fused (rmsnorm_router_kernel) and the plain RMSNorm on N tokens x 1024 channels."""
    g = torch.Generator(device="cuda").manual_seed(0)
    N, C, E = a.N, 1024, 4
    x = torch.randn(N, C, generator=g, device="cuda")
    wn = torch.rand(C, generator=g, device="cuda") + 0.5
    wr = torch.randn(E, C, generator=g, device="cuda") * 0.05
    ms = timeit(lambda: ops.rmsnorm_router(x, wn, 1e-6, wr), a.iters)
    report("rmsnorm_router_kernel", ms, bytes_=6.0 * N * C, extra={"N": N})
    ms = timeit(lambda: ops.rmsnorm(x, wn, 1e-6), a.iters)
    report("rmsnorm_kernel", ms, bytes_=6.0 * N * C, extra={"N": N})


def case_decode(a):
    """Config 5: ragged state-carrying decode on the 606M model: B sequences, one token per step,
    positions ~ U[1, 4096], carried attention state (B, H, 64, 64) f32 and LSF membrane per layer."""
    from jarvis_b200 import modules as jm
    dev = torch.device("cuda")
    with torch.device(dev):
        model = jm.Jarvis(max_seq_len=4096 + a.steps + 8)
    gen = torch.Generator(device=dev).manual_seed(0)
    with torch.no_grad():
        for mod in model.modules():
            if isinstance(mod, jm.TernaryLinear):
                mod.weight.copy_(torch.randn(mod.weight.shape, generator=gen, device=dev) * 0.02)
    model.eval()
    B, L, H = a.B, len(model.blocks), 16
    pos = torch.randint(1, 4097, (B,), generator=gen, device=dev, dtype=torch.int32)
    state = {"h": [torch.randn(B, 1024, generator=gen, device=dev) for _ in range(L)],
             "S": [torch.randn(B, H, 64, 64, generator=gen, device=dev) for _ in range(L)]}
    idx = torch.randint(0, 50257, (a.steps, B, 1), generator=gen, device=dev)
    sess = jm.DecodeSession(model, state, pos, max_position=4096 + a.steps + 8)
    if not a.eager:
        sess.capture()
    else:
        for w in range(3):
            sess.step(idx[w % a.steps])
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for sidx in range(a.steps):
        sess.step(idx[sidx])
    e1.record()
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    ms = e0.elapsed_time(e1) / a.steps
    by = L * (2.0 * B * H * 64 * 64 * 4 + 5 * 2 ** 20) + 2.0 * 1024 * 50304
    report("decode step (606M, all kernels + lm_head)", ms, bytes_=by,
           extra={"B": B, "steps": a.steps, "tokens_per_s": B / ms * 1e3, "state_dtype": "f32",
                  "cuda_graph": not a.eager})


def case_serve(a):
    """Continuous batching on the 606M model: `--requests` requests with prompts ~ U[16, 256] tokens and
    16..64 new tokens each through `--slots` slots (serving.build_scheduler: admission by prefill, one
    CUDA-graphed batched step + sampling kernel per iteration).  Wall-clock, host work included."""
    import time
    from jarvis_b200 import modules as jm, serving
    dev = torch.device("cuda")
    with torch.device(dev):
        model = jm.Jarvis(max_seq_len=1024)
    gen = torch.Generator(device=dev).manual_seed(0)
    with torch.no_grad():
        for mod in model.modules():
            if isinstance(mod, jm.TernaryLinear):
                mod.weight.copy_(torch.randn(mod.weight.shape, generator=gen, device=dev) * 0.02)
    model.eval()
    sched = serving.build_scheduler(model, max_batch_size=a.slots, max_position=1024, temperature=0.7, top_k=50,
                                    top_p=0.9, seed=0)
    g = torch.Generator().manual_seed(1)
    n_prompt = 0
    for i in range(a.requests):
        plen = int(torch.randint(16, 257, (1,), generator=g))
        n_prompt += plen
        sched.add_request(serving.Request(i, torch.randint(0, 50257, (plen,), generator=g).tolist(),
                                          int(torch.randint(16, 65, (1,), generator=g))))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    iters = sched.run()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert _lib.device_status() == 0
    n_new = sum(len(r.generated_tokens) for r in sched.completed)
    print(json.dumps({"kernel": "continuous batching (606M)", "requests": a.requests, "slots": a.slots, "iterations": iters,
                      "prompt_tokens": n_prompt, "generated_tokens": n_new, "seconds": dt,
                      "generated_tok_per_s": n_new / dt, "ms_per_iteration": dt / iters * 1e3}), flush=True)


def case_context(a):
    """Long-sequence prefill of the 606M model with the sequences cut across the ranks (context parallelism):
    B sequences of T tokens, rank r holding tokens [r*T/W, (r+1)*T/W) of each; hidden states only (no lm_head).
    Under torchrun; with one process it times the whole sequence on one GPU (the figure to compare with)."""
    import torch.distributed as dist
    from jarvis_b200 import modules as jm
    dev = torch.device("cuda")
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    with torch.device(dev):
        model = jm.Jarvis(max_seq_len=a.T)
    gen = torch.Generator(device=dev).manual_seed(0)
    with torch.no_grad():
        for mod in model.modules():
            if isinstance(mod, jm.TernaryLinear):
                mod.weight.copy_(torch.randn(mod.weight.shape, generator=gen, device=dev) * 0.02)
    model.eval()
    idx = torch.randint(0, 50257, (a.B, a.T), generator=torch.Generator().manual_seed(1)).to(dev)
    tl = a.T // world
    if world > 1:
        model.set_context_parallel(dist.group.WORLD)
    mine = idx[:, rank * tl:(rank + 1) * tl].contiguous()
    for _ in range(3):
        model.hidden_rows(mine)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
        model.hidden_rows(mine)
    e1.record()
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    t = torch.tensor([e0.elapsed_time(e1) / a.iters], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t)
    if rank == 0:
        report("context-parallel prefill (606M, 24 layers, hidden states)", ms, flops=a.B * a.T * 603.98e6 / world,
               extra={"B": a.B, "T": a.T, "n_gpus": world, "tokens_per_s": a.B * a.T / ms * 1e3,
                      "note": "achieved = per-GPU ternary-GEMM rate; tokens_per_s = whole job"})
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="case", required=True)
    s = sub.add_parser("gemm")
    s.add_argument("--M", type=int, default=16384); s.add_argument("--N", type=int, default=3072)
    s.add_argument("--K", type=int, default=1024); s.add_argument("--groups", type=int, default=1)
    s.add_argument("--epilogue", type=int, default=0); s.add_argument("--tile", type=int, default=0)
    s.add_argument("--canonical", dest="prepared", action="store_false", help="decode the weight_packing.py layout in-kernel")
    s = sub.add_parser("attn")
    s.add_argument("--B", type=int, default=32); s.add_argument("--H", type=int, default=16)
    s.add_argument("--T", type=int, default=2048)
    s = sub.add_parser("lsf")
    s.add_argument("--B", type=int, default=32); s.add_argument("--T", type=int, default=2048)
    s.add_argument("--C", type=int, default=1024); s.add_argument("--resid", action="store_true")
    s = sub.add_parser("moe")
    s.add_argument("--N", type=int, default=65536); s.add_argument("--zipf", type=float, default=1.2)
    s.add_argument("--peer", action="store_true", help="expert parallel: exchange rows by peer-memory loads, not NCCL all-to-all")
    s = sub.add_parser("decode")
    s.add_argument("--B", type=int, default=256); s.add_argument("--steps", type=int, default=64)
    s.add_argument("--eager", action="store_true", help="launch every kernel from Python instead of replaying a CUDA graph")
    s = sub.add_parser("router")
    s.add_argument("--N", type=int, default=16384)
    s = sub.add_parser("serve")
    s.add_argument("--slots", type=int, default=64); s.add_argument("--requests", type=int, default=256)
    s = sub.add_parser("context")
    s.add_argument("--B", type=int, default=2); s.add_argument("--T", type=int, default=16384)
    for p in sub.choices.values():
        p.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        import torch.distributed as dist
        lr = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(lr)
        dist.init_process_group("nccl", device_id=torch.device("cuda", lr))
    {"gemm": case_gemm, "attn": case_attn, "lsf": case_lsf, "moe": case_moe, "decode": case_decode,
     "context": case_context, "serve": case_serve, "router": case_router}[a.case](a)
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
