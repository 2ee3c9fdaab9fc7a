"""Generates tests/golden/*.npz by running the REFERENCE's own modules on CPU (fp32).

Run where the reference tree is mounted:
    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference   (or JARVIS_REFERENCE=...)
The fixtures are committed; the tests never need the reference tree.  Inputs are seeded
synthetic tensors; every stored output was produced by reference code, never by this repo.
Every golden_* function seeds the global RNG itself, so each .npz regenerates bit for bit whatever
ran before it; the one varying byte range is the `created_at` time stamp that the reference's exporter
writes into the manifest of tiny.jarvis-tbin.
"""
import os
import sys

import numpy as np
import torch

sys.dont_write_bytecode = True
_REPO = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
REF = sys.argv[1] if len(sys.argv) > 1 else (os.environ.get("JARVIS_REFERENCE") or os.path.join(os.path.dirname(_REPO), "reference"))
for sub in ("jarvis_engine", "runtime", "associative_attention_cuda", "sparse_model_cuda", "liquid_fusion_cuda"):
    sys.path.insert(0, os.path.join(REF, sub))

import jarvis_model as jm  # noqa: E402
import weight_packing as wp  # noqa: E402
from utils.ternary_ops import TernaryQuantizeSTE  # noqa: E402
import associative_attention as aa  # noqa: E402  (CPU fallbacks of the CUDA drop-in)
import sparse_model as sm  # noqa: E402
import liquid_state_fusion as lsf_ext  # noqa: E402
import validate_liquid_state_fusion as lsf_val  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))
torch.set_grad_enabled(False)


def npy(t):
    return t.detach().cpu().numpy()


GRID = 0.02 / 32.0  # ternary-layer weights live on an int8 grid so the fixtures stay small


def save(name, **arrays):
    """Weights whose key ends in `weight` and that sit on the int8 grid are stored as int8 under
    `<key>__i8` (tests/golden/loader.py multiplies them back by GRID, bit for bit)."""
    packed = {}
    for k, v in arrays.items():
        a = npy(v) if torch.is_tensor(v) else np.asarray(v)
        if a.dtype == np.float32 and a.ndim == 2 and a.size >= 4096:
            i8 = np.rint(a / np.float32(GRID))
            if np.abs(i8).max() <= 127 and np.array_equal(i8.astype(np.float32) * np.float32(GRID), a):
                packed[k + "__i8"] = i8.astype(np.int8)
                continue
        packed[k] = a
    np.savez_compressed(os.path.join(OUT, name + ".npz"), **packed)
    print(name, len(packed), "arrays", os.path.getsize(os.path.join(OUT, name + ".npz")) // 1024, "KiB")


def grid_randn(shape, gen):
    """N(0, 0.02^2) rounded onto the int8 grid (|w| <= 127 * GRID ~ 4 sigma)."""
    return torch.clamp(torch.round(torch.randn(shape, generator=gen) * 32.0), -127, 127) * GRID


def ternary_init(module, gen):
    """Every ternary matrix (q/k/v/out projections, expert w1 / w2) gets grid weights; names are matched with a
    leading dot so that a bare SparseMoELayer (`w1.0.weight`) is covered like a block (`moe.w1.0.weight`)."""
    for name, p in module.named_parameters():
        dotted = "." + name
        if name.endswith("proj.weight") or ".w1." in dotted or ".w2." in dotted:
            p.copy_(grid_randn(p.shape, gen))


# ---- 1. ternary quantisation + packing --------------------------------------------------
def golden_pack():
    torch.manual_seed(101)   # constructors below draw from the global RNG
    gen = torch.Generator().manual_seed(1)
    w = torch.randn(96, 64, generator=gen) * 0.02
    w[0, :6] = torch.tensor([0.0, 1e-9, -1.0, 1.0, 0.5, -0.5])
    wq = TernaryQuantizeSTE.apply(w)                      # alpha * q
    alpha = w.abs().mean().clamp(min=1e-8)
    q = torch.round(torch.clamp(w / alpha, -1.0, 1.0))
    assert torch.equal(wq, q * alpha)
    packed, shape = wp.pack_ternary_tensor(q)
    unpacked = wp.unpack_ternary_tensor(packed, shape, dtype=torch.float32, device="cpu")
    pats = torch.stack([torch.zeros(8, 16), torch.ones(8, 16), -torch.ones(8, 16),
                        torch.tensor([-1.0, 0.0, 1.0, 0.0]).repeat(8, 4)])
    pat_packed = torch.stack([wp.pack_ternary_tensor(p)[0] for p in pats])
    x = torch.randn(10, 64, generator=gen)
    y = torch.nn.functional.linear(x, wq)
    save("pack", w=w, alpha=alpha, q=q, packed=packed, unpacked=unpacked, patterns=pats, patterns_packed=pat_packed,
         x=x, y=y)


# ---- 2. attention ---------------------------------------------------------------------
def golden_attention():
    torch.manual_seed(102)   # constructors below draw from the global RNG
    d_model, H = 128, 2
    out = {}
    gen = torch.Generator().manual_seed(42)
    m = jm.AssociativeLinearAttention(d_model, H).eval()
    ternary_init(m, gen)
    m.gamma_raw.copy_(torch.logit(torch.rand(H, generator=gen) * 0.099 + 0.9))
    for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
        out[f"{n}.weight"] = getattr(m, n).weight
    out["gamma_raw"] = m.gamma_raw.clone()
    for T in (1, 17, 64, 37, 123, 192):
        x = torch.randn(2 if T < 64 else 1, T, d_model, generator=gen)
        sp = 0 if T != 37 else 128
        out[f"T{T}_x"] = x
        out[f"T{T}_y"] = m(x, start_pos=sp)
        out[f"T{T}_start_pos"] = sp
    # extreme decays (validate_attention.py uses gamma ~0.01 and ~0.99)
    for tag, g in (("lo", 0.01), ("hi", 0.99)):
        m.gamma_raw.fill_(float(torch.logit(torch.tensor(g))))
        x = torch.randn(1, 100, d_model, generator=gen)
        out[f"g{tag}_x"], out[f"g{tag}_y"] = x, m(x)
        out[f"g{tag}_gamma_raw"] = m.gamma_raw.clone()
    save("attention", **out)

    # carried state: the CUDA drop-in's CPU fallback accepts h_prev (Path A for T%64==0, else Path B)
    out = {}
    gen = torch.Generator().manual_seed(900)
    m = aa.CUDAAssociativeLinearAttention(d_model, H).eval()
    ternary_init(m, gen)
    m.gamma_raw.copy_(torch.logit(torch.rand(H, generator=gen) * 0.099 + 0.9))
    for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
        out[f"{n}.weight"] = getattr(m, n).weight
    out["gamma_raw"] = m.gamma_raw.clone()
    for T in (64, 128, 50):
        x = torch.randn(1, T, d_model, generator=gen)
        S0 = torch.randn(1, H, 64, 64, generator=gen)
        out[f"T{T}_x"], out[f"T{T}_S0"] = x, S0
        out[f"T{T}_y"] = m(x, start_pos=5, h_prev=S0)
    # feature map + RoPE and the chunk-state scan as stand-alone functions
    gen = torch.Generator().manual_seed(5)
    q = torch.randn(1, 2, 70, 64, generator=gen)
    k = torch.randn(1, 2, 70, 64, generator=gen)
    rot = jm.RotaryEmbedding(64, max_seq_len=256)
    cos, sin = rot.cos_cached[3:73], rot.sin_cached[3:73]
    qr, kr = aa.FusedRoPEELUFunction.apply(q, k, cos, sin)
    out.update(rope_q=q, rope_k=k, rope_q_out=qr, rope_k_out=kr, rope_start=3)
    dS = torch.randn(1, 2, 3, 64, 64, generator=gen)
    gc = torch.rand(2, generator=gen)
    h0 = torch.randn(1, 2, 64, 64, generator=gen)
    all_states, h_last = aa.RecurrentChunkStateScanFunction.apply(dS, gc, h0)
    out.update(scan_dS=dS, scan_gc=gc, scan_h0=h0, scan_all=all_states, scan_last=h_last)
    save("attention_state", **out)


# ---- 3. MoE ---------------------------------------------------------------------------
def golden_moe():
    torch.manual_seed(103)   # constructors below draw from the global RNG
    d_model = 128
    out = {}
    cases = [("b1t16", 1, 16, None), ("b2t64", 2, 64, None), ("all_e0", 2, 32, "all0"), ("e0_empty", 2, 32, "empty0"),
             ("imbalanced", 2, 64, "imb")]
    gen = torch.Generator().manual_seed(42)
    m = jm.SparseMoELayer(d_model).eval()
    ternary_init(m, gen)
    for e in range(4):
        out[f"w1.{e}.weight"] = m.w1[e].weight
        out[f"w2.{e}.weight"] = m.w2[e].weight
    for tag, B, T, force in cases:
        m.router.weight.copy_(torch.randn(4, d_model, generator=gen) * 0.05)
        x = torch.randn(B, T, d_model, generator=gen)
        if force == "all0":      # expert 0 always first
            x[..., 0] = 1.0
            m.router.weight[:, 0] = torch.tensor([40.0, 0.0, -10.0, -20.0])
        elif force == "empty0":  # expert 0 never chosen
            x[..., 0] = 1.0
            m.router.weight[:, 0] = torch.tensor([-40.0, 0.0, 0.0, 0.0])
        elif force == "imb":
            x[..., 0] = 1.0
            m.router.weight[:, 0] = torch.tensor([3.0, 1.0, 0.0, -1.0])
        y, lb, am, av = m(x)
        xf = x.view(-1, d_model)
        probs = torch.softmax(m.router(xf), dim=-1)
        tp, ti = probs.topk(2, dim=-1)
        # dispatch order of the PyTorch path: boolean masks over the flattened (N*K) list
        flat = ti.reshape(-1)
        order = torch.cat([(flat == e).nonzero(as_tuple=True)[0] for e in range(4)])
        # the CUDA drop-in's CPU fallback must agree with the pure module
        m2 = sm.CUDASparseMoELayer(d_model).eval()
        m2.load_state_dict(m.state_dict())
        y2 = m2(x)[0]
        assert torch.allclose(y, y2, atol=1e-6)
        out.update({f"{tag}_x": x, f"{tag}_y": y, f"{tag}_l_balance": lb, f"{tag}_act_mean": am, f"{tag}_act_var": av,
                    f"{tag}_router": m.router.weight.clone(), f"{tag}_topk_idx": ti, f"{tag}_topk_probs": tp,
                    f"{tag}_probs": probs, f"{tag}_order": order})
    save("moe", **out)


# ---- 4. LSF ---------------------------------------------------------------------------
def golden_lsf():
    torch.manual_seed(104)   # constructors below draw from the global RNG
    out = {}
    gen = torch.Generator().manual_seed(3)
    m = jm.LiquidStateFusion(32).eval()
    m.var_scale.fill_(1.3)
    for tag, T, var, hp in (("t1", 1, 0.5, True), ("t65", 65, 0.02, True), ("t200", 200, 3.0, False)):
        x = torch.randn(2, T, 32, generator=gen)
        h_prev = torch.randn(2, 32, generator=gen) if hp else None
        av = torch.tensor(var)
        h_out, h_last = m(x, av, h_prev)
        out.update({f"{tag}_x": x, f"{tag}_act_var": av, f"{tag}_h_out": h_out, f"{tag}_h_last": h_last})
        if hp:
            out[f"{tag}_h_prev"] = h_prev
    out["var_scale"] = m.var_scale
    # extension API: per-element alpha (validate_liquid_state_fusion.py shapes: B=2, D=8)
    for T in (1, 15, 65, 127, 129, 256):
        alpha = torch.rand(2, T, 8, generator=gen) * 0.98 + 0.01
        M = torch.randn(2, T, 8, generator=gen)
        h0 = torch.randn(2, 8, generator=gen)
        H_seq, _ = lsf_val.sequential_baseline(alpha, M, h0)
        H_fn = lsf_ext.LiquidStateFusionFunction.apply(alpha, M, h0)
        assert torch.allclose(H_seq, H_fn, atol=1e-5)
        out.update({f"ext{T}_alpha": alpha, f"ext{T}_M": M, f"ext{T}_h0": h0, f"ext{T}_H": H_seq})
    save("lsf", **out)


# ---- 5. block and a tiny model -----------------------------------------------------------
def golden_block_model():
    torch.manual_seed(105)   # constructors below draw from the global RNG
    gen = torch.Generator().manual_seed(0)
    blk = jm.JarvisBlock(128, 2, 4, 2, use_cuda_attn=False, use_cuda_moe=False).eval()
    ternary_init(blk, gen)
    blk.attn.gamma_raw.copy_(torch.logit(torch.rand(2, generator=gen) * 0.099 + 0.9))
    x = torch.randn(2, 100, 128, generator=gen)
    h_prev = torch.randn(2, 128, generator=gen)
    xo, hl, lb, lr = blk(x, h_prev, start_pos=9)
    out = {"x": x, "h_prev": h_prev, "start_pos": 9, "x_out": xo, "h_last": hl, "l_balance": lb, "l_reflect": lr}
    out.update({"sd_" + k: v for k, v in blk.state_dict().items()})
    save("block", **out)

    gen = torch.Generator().manual_seed(1337)
    model = jm.Jarvis(vocab_size=256, d_model=128, n_layers=2, n_heads=2, max_seq_len=256,
                      use_cuda_attn=False, use_cuda_moe=False).eval()
    ternary_init(model, gen)
    idx = torch.randint(0, 256, (2, 96), generator=gen)
    logits, _ = model(idx)
    model.reset_state()   # forward() stores the membrane states even when persist_state is False
    logits2, _ = model(idx[:, :32], persist_state=True)
    logits3, _ = model(idx[:, 32:64], persist_state=True)
    out = {"idx": idx, "logits": logits, "persist_logits_a": logits2, "persist_logits_b": logits3,
           "n_state_keys": len(model.state_dict())}
    out.update({"sd_" + k: v for k, v in model.state_dict().items()})
    save("model", **out)


# ---- 6. the .jarvis-tbin container, written and re-read by the reference's own code ---------------
def golden_tbin():
    torch.manual_seed(106)   # constructors below draw from the global RNG
    sys.path.insert(0, os.path.join(REF, "experiments", "architecture_matrix", "ternary_packed"))
    import jarvis_tbin_format as tb
    gen = torch.Generator().manual_seed(77)
    model = jm.Jarvis(vocab_size=64, d_model=128, n_layers=1, n_heads=2, max_seq_len=64,
                      use_cuda_attn=False, use_cuda_moe=False).eval()
    ternary_init(model, gen)
    path = os.path.join(OUT, "tiny.jarvis-tbin")
    tb.export_to_jarvis_tbin(model, path, {"note": "golden"})
    twin = jm.Jarvis(vocab_size=64, d_model=128, n_layers=1, n_heads=2, max_seq_len=64,
                     use_cuda_attn=False, use_cuda_moe=False).eval()
    tb.load_from_jarvis_tbin(twin, path, device="cpu")
    sd = twin.state_dict()                      # effective weights alpha * q, dense tensors through bf16
    idx = torch.randint(0, 64, (2, 40), generator=gen)
    save("tbin", idx=idx, logits=twin(idx)[0],
         **{"sd_" + k: sd[k] for k in ("blocks.0.attn.q_proj.weight", "blocks.0.moe.w2.3.weight", "tok_emb.weight",
                                       "blocks.0.moe.router.weight", "blocks.0.attn.gamma_raw")})


# ---- 7. decode driver: the reference's sampling filter and its continuous-batching slot policy -----------
def _reference_defs(path, names):
    """exec only the named top-level classes / functions of a reference script (its module level parses
    arguments and imports tokenisers, which the fixtures do not need)."""
    import ast
    import collections
    import time
    import typing
    src = open(path).read()
    tree = ast.parse(src)
    body = [n for n in tree.body if isinstance(n, (ast.FunctionDef, ast.ClassDef)) and n.name in names]
    ns = {"torch": torch, "F": torch.nn.functional, "collections": collections, "time": time,
          "List": typing.List, "Dict": typing.Dict, "Optional": typing.Optional}
    exec(compile(ast.Module(body=body, type_ignores=[]), path, "exec"), ns)
    return ns


def golden_sampling():
    torch.manual_seed(107)   # constructors below draw from the global RNG
    ns = _reference_defs(os.path.join(REF, "jarvis_engine", "evaluate_jarvis.py"), {"sample_next_token"})
    gen = torch.Generator().manual_seed(2024)
    B, V = 6, 512
    logits = torch.randn(B, V, generator=gen) * 3.0
    logits[1, 100:140] = logits[1, 100]          # a plateau of equal logits around the top-k boundary
    logits[2] = torch.round(logits[2])            # many exact ties
    captured = {}
    real_multinomial = torch.multinomial

    def fake_multinomial(probs, num_samples=1):
        captured["probs"] = probs.clone()
        return probs.argmax(dim=-1, keepdim=True)

    out = {"logits": logits}
    settings = [(0.7, 50, 0.9), (1.0, 5, 0.5), (1.3, 200, 0.95), (0.7, 50, 1.0), (0.25, 1024, 0.3)]
    torch.multinomial = fake_multinomial
    try:
        for i, (t, k, p) in enumerate(settings):
            ns["sample_next_token"](logits.clone(), temperature=t, top_k=k, top_p=p)
            out[f"probs_{i}"] = captured["probs"]
    finally:
        torch.multinomial = real_multinomial
    out["settings"] = torch.tensor(settings, dtype=torch.float64)
    out["greedy"] = ns["sample_next_token"](logits.clone(), temperature=0.0)
    save("sampling", **out)


def golden_scheduler():
    torch.manual_seed(108)   # constructors below draw from the global RNG
    ns = _reference_defs(os.path.join(REF, "experiments", "exp_batching_continuous.py"),
                         {"Request", "ContinuousBatchingScheduler"})
    sched = ns["ContinuousBatchingScheduler"](max_batch_size=4, device="cpu")
    reqs = [ns["Request"](req_id=i, prompt_tokens=[10, 20, 30], max_new_tokens=(i % 4 + 2)) for i in range(10)]
    for r in reqs:
        sched.add_request(r)
    trace, finish_iter = [], [-1] * len(reqs)
    it = 0
    while sched.active_slots or sched.waiting_queue:
        stepped = sched.step()
        it += 1
        slots = [sched.active_slots[s].req_id if s in sched.active_slots else -1 for s in range(4)]
        for r in reqs:
            if r.is_finished and finish_iter[r.req_id] < 0:
                finish_iter[r.req_id] = it
        trace.append([stepped, len(sched.waiting_queue)] + slots)
    save("scheduler", trace=torch.tensor(trace), finish_iter=torch.tensor(finish_iter),
         n_generated=torch.tensor([len(r.generated_tokens) for r in reqs]))


if __name__ == "__main__":
    golden_pack()
    golden_attention()
    golden_moe()
    golden_lsf()
    golden_block_model()
    golden_sampling()
    golden_scheduler()
    golden_tbin()
