"""GPU parity against the CPU oracle AT THE SHAPES OF THE BENCHMARK CONFIGURATIONS (d_model 1024, 16 heads x 64,
4 experts 1024 -> 2048 -> 1024, vocabulary 50257), not at shrunken stand-ins:

  1. one block, B=1 x T=512, seed 0: output, LSF membrane, routing, dispatch maps, final attention state, l_balance
  2. the model at B=2 x T=2048 with 2 layers, and one whole 24-layer sequence
  3. the scan sweep at B=32, H=16, T in {512, 2048, 8192, 32768} (oracle on a subset of the sequences), LSF at C=1024
  4. the MoE layer alone on 65,536 tokens with Zipf(1.2) top-1 loads
  5. ragged state-carrying decode: prior lengths ~ U[1, 4096], 64 single-token steps, drift of the carried state

Tolerances: integer / index results bit-exact; floating point rel-L2 <= 1e-2 against the fp32 oracle per stage
(bf16 compute), model-level logits rel-L2 <= 3e-2 and cosine > 0.999 (the reference's own model gate,
tests/test_correctness_gate.py:79).
"""
import pytest
import torch

import jarvis_b200  # noqa: F401
from jarvis_b200 import _lib, modules as jm, ops, synthetic
from oracle import jarvis_oracle as orc

pytestmark = pytest.mark.gpu
TOL = 1e-2
C, H, E, V = 1024, 16, 4, 50257


def rel_l2(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def cosine(a, b):
    a, b = a.double().cpu().reshape(-1), b.double().cpu().reshape(-1)
    return float(a @ b / (a.norm() * b.norm()))


def margins(probs):
    srt = probs.sort(dim=-1, descending=True).values
    return torch.minimum(srt[:, 0] - srt[:, 1], srt[:, 1] - srt[:, 2])


# ---------------------------------------------------------------------------------------------- config 1
def test_config1_single_block_fp32_reference_shape():
    torch.manual_seed(0)
    blk = synthetic.gaussian_ternary_(jm.JarvisBlock(C, H, E, 2), seed=0).eval()
    sd = {k: v.clone() for k, v in blk.state_dict().items()}
    x = torch.randn(1, 512, C)
    ref = orc.block_forward(x, sd, H)
    blk = blk.cuda()
    rows = x.reshape(512, C).clone().cuda()
    h_last, sc, S = blk.forward_rows(rows, 1, 512, want_attn_state=True)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert rel_l2(rows, ref["x"].reshape(512, C)) <= TOL
    assert rel_l2(S, ref["attn_state"]) <= TOL
    assert rel_l2(h_last, ref["h_last"]) <= 2e-2           # one token's membrane: 1024 values
    assert abs(float(sc[0]) - float(ref["l_balance"])) <= 2e-2 * abs(float(ref["l_balance"]))
    assert abs(float(sc[2]) - float(ref["act_var"])) <= 3e-2 * float(ref["act_var"])
    # routing: the router sees activations that differ from the oracle's by bf16 rounding, so indices must
    # agree wherever the oracle's probabilities are not nearly tied
    idx, gates, meta = blk.moe.last_routing
    clear = margins(ref["probs"]) > 5e-3
    assert clear.float().mean() > 0.9
    assert torch.equal(idx.cpu()[clear], ref["idx"][clear])
    assert (idx.cpu() != ref["idx"]).any(dim=-1).float().mean() < 0.02
    assert torch.allclose(gates.cpu()[clear], ref["gates"][clear], atol=2e-2)
    # the five dispatch maps are a pure function of the indices: bit-exact
    for got, want in zip(meta, orc.moe_metadata(idx.cpu(), E)):
        assert torch.equal(got.cpu(), want)
    # and on the oracle's own router input (rounded to bf16 on both sides) the indices are bit-exact
    xo = ref["x"].reshape(512, C) - orc.lsf_model(ref["moe_out"], ref["act_var"], sd["liquid.var_scale"])[0].reshape(512, C)
    xn = orc.rmsnorm(xo, sd["norm2.weight"]).bfloat16()
    i_ref, g_ref, p_ref = orc.router_top2(xn.float(), sd["moe.router.weight"])
    i_gpu, g_gpu, _ = ops.router_top2(xn.cuda(), sd["moe.router.weight"].cuda())
    ok = margins(p_ref) > 1e-5
    assert ok.float().mean() > 0.99 and torch.equal(i_gpu.cpu()[ok], i_ref[ok])
    assert torch.allclose(g_gpu.cpu()[ok], g_ref[ok], atol=1e-5)


# ---------------------------------------------------------------------------------------------- config 2
def _model(n_layers, seed, max_seq_len=2048):
    torch.manual_seed(seed)
    model = synthetic.gaussian_ternary_(jm.Jarvis(V, C, n_layers, H, E, 2, max_seq_len=max_seq_len), seed=seed).eval()
    return model, {k: v.clone() for k, v in model.state_dict().items()}


def _check_logits(model, sd, idx, n_layers, rows_step):
    with torch.no_grad():
        hidden_ref, _ = orc.model_forward(idx, sd, n_layers, H, return_hidden=True)
    model = model.cuda()
    logits, _ = model(idx.cuda())
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    B, T = idx.shape
    sel = torch.arange(0, B * T, rows_step)
    ref = hidden_ref.reshape(B * T, C)[sel] @ sd["lm_head.weight"].t()          # fp32 logits of the sampled rows
    got = logits.reshape(B * T, V)[sel.cuda()].float()
    return rel_l2(got, ref), cosine(got, ref)


def test_config2_two_layers_at_the_prefill_shape():
    model, sd = _model(2, seed=0)
    idx = torch.randint(0, V, (2, 2048), generator=torch.Generator().manual_seed(1))
    err, cos = _check_logits(model, sd, idx, 2, rows_step=16)
    assert err <= 1.5e-2 and cos > 0.9995, (err, cos)


def test_config2_all_24_layers_one_sequence():
    model, sd = _model(24, seed=0)
    idx = torch.randint(0, V, (1, 2048), generator=torch.Generator().manual_seed(2))
    err, cos = _check_logits(model, sd, idx, 24, rows_step=8)
    print(f"24 layers, T=2048: logits rel-L2 {err:.3e}, cosine {cos:.6f}")
    assert err <= 3e-2 and cos > 0.999, (err, cos)


# ---------------------------------------------------------------------------------------------- config 3
def _rope_tabs(n_pos):
    cos, sin = orc.rope_tables(n_pos, 64)
    return cos[:, :32].contiguous().cuda(), sin[:, :32].contiguous().cuda()


@pytest.mark.parametrize("T,check", [(512, (0, 13, 31)), (2048, (0, 31)), (8192, (5, 31)), (32768, (31,))])
def test_config3_attention_scan_sweep(T, check):
    """B=32, H=16: the whole batch runs on the GPU; output rows and final state of the sequences in `check` are
    compared with the fp64 token-by-token recurrence."""
    B = 32
    g = torch.Generator(device="cuda").manual_seed(T)
    qkv = torch.randn(B * T, 3 * C, generator=g, device="cuda").bfloat16()
    gamma = torch.rand(H, generator=g, device="cuda") * 0.099 + 0.9
    cos, sin = _rope_tabs(T)
    o, S = ops.attn_scan(qkv[:, :C], qkv[:, C:2 * C], qkv[:, 2 * C:], gamma, cos, sin, B, T, H, want_state=True)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    for b in check:
        rows = qkv[b * T:(b + 1) * T].float().cpu()

        def heads(t):
            return t.reshape(1, T, H, 64).transpose(1, 2)

        qf, kf = orc.feature_map_rope(heads(rows[:, :C]), heads(rows[:, C:2 * C]), 0)
        o_ref, S_ref = orc.attn_scan_recurrent(qf, kf, heads(rows[:, 2 * C:]), gamma.cpu())
        got = o[b * T:(b + 1) * T].float().cpu().reshape(1, T, H, 64).transpose(1, 2)
        eo, es = rel_l2(got, o_ref), rel_l2(S[b:b + 1], S_ref)
        # per head as well: a wrong head -> decay or head -> column mapping would hide in the global norm
        eh = max(rel_l2(got[:, h], o_ref[:, h]) for h in range(H))
        assert eo <= TOL and es <= TOL and eh <= 1.5e-2, (T, b, eo, es, eh)


@pytest.mark.parametrize("T", [512, 2048, 8192, 32768])
def test_config3_lsf_scan_sweep(T):
    B = 32
    g = torch.Generator(device="cuda").manual_seed(T + 1)
    m = torch.randn(B, T, C, generator=g, device="cuda").bfloat16()
    h0 = torch.randn(B, C, generator=g, device="cuda")
    al = torch.tensor([0.97], device="cuda")
    out, last = ops.lsf_scan(m, alpha_scalar=al, h0=h0)
    resid = torch.zeros(B, T, C, device="cuda") if T <= 8192 else None
    if resid is not None:
        ops.lsf_scan(m, alpha_scalar=al, h0=h0, resid=resid, want_out=False)
    torch.cuda.synchronize()
    for b in (0, 31):
        ref = orc.lsf_scan(m[b:b + 1].float().cpu(), 0.97, h0[b:b + 1].cpu())
        assert rel_l2(out[b:b + 1].float(), ref) <= 4e-3          # bf16 rounding of the stored result only
        assert rel_l2(last[b:b + 1], ref[:, -1]) <= 1e-5
        if resid is not None:
            assert rel_l2(resid[b:b + 1], ref) <= 1e-5            # fused residual form: f32 accumulate into zeros


# ---------------------------------------------------------------------------------------------- config 4
def test_config4_zipf_moe_layer_65536_tokens():
    N = 65536
    x, w_r, shares = synthetic.zipf_router_inputs(N, C, E, seed=0)
    target = synthetic.zipf_shares(E)
    assert torch.allclose(target, torch.tensor([0.528, 0.230, 0.141, 0.100]), atol=1.5e-3)
    assert float((shares - target).abs().max()) < 5e-3, shares
    # router + dispatch order, bit-exact against the oracle on the same bf16 inputs
    i_ref, g_ref, p_ref = orc.router_top2(x.float(), w_r)
    top1 = torch.bincount(i_ref[:, 0], minlength=E).float() / N
    assert float((top1 - target).abs().max()) < 5e-3
    xd = x.cuda()
    i_gpu, g_gpu, _ = ops.router_top2(xd, w_r.cuda())
    ok = margins(p_ref) > 1e-5
    assert ok.float().mean() > 0.995
    assert torch.equal(i_gpu.cpu()[ok], i_ref[ok])
    assert torch.allclose(g_gpu.cpu()[ok], g_ref[ok], atol=1e-5)
    meta = ops.moe_metadata(i_gpu, E)
    for got, want in zip(meta, orc.moe_metadata(i_gpu.cpu(), E)):
        assert torch.equal(got.cpu(), want)
    if bool(ok.all()):
        for got, want in zip(meta, orc.moe_metadata(i_ref, E)):
            assert torch.equal(got.cpu(), want)
    # the whole layer through the module; the oracle runs the first 4096 tokens (tokens are routed independently)
    torch.manual_seed(0)
    moe = synthetic.gaussian_ternary_(jm.SparseMoELayer(C), seed=0).eval()
    with torch.no_grad():
        moe.router.weight.copy_(w_r)
    w1 = [m.weight.detach().clone() for m in moe.w1]
    w2 = [m.weight.detach().clone() for m in moe.w2]
    moe = moe.cuda()
    out, sc = moe.run_rows(xd, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    n_ref = 4096
    ref_out, _, _, _, aux = orc.moe_forward(x[:n_ref].float().reshape(1, n_ref, C), w_r, w1, w2)
    same = (moe.last_routing[0][:n_ref].cpu() == aux["idx"]).all(dim=-1)
    assert same.float().mean() > 0.995
    assert rel_l2(out[:n_ref].cpu()[same], ref_out.reshape(n_ref, C)[same]) <= TOL
    assert abs(float(sc[2]) - float(out.var())) <= 1e-4 * float(out.var())
    counts = meta[0].cpu()
    assert int(counts.sum()) == 2 * N and int(counts.max()) <= N


# ---------------------------------------------------------------------------------------------- config 5
def test_config5_ragged_decode_64_steps_state_drift():
    """8 sequences, prior lengths ~ U[1, 4096] prefilled one by one (both sides make the same calls), then 64
    single-token steps of the whole ragged batch with the state handed from step to step."""
    n_layers, B, steps = 2, 8, 64
    model, sd = _model(n_layers, seed=3, max_seq_len=4096 + steps + 8)
    model = model.cuda()
    lens = synthetic.ragged_prior_lengths(B, 4096, seed=5)
    sd_prefill = dict(sd, **{"lm_head.weight": sd["lm_head.weight"][:8]})    # the prompts' logits are not compared
    g = torch.Generator().manual_seed(6)
    h_ref = [[] for _ in range(n_layers)]
    S_ref = [[] for _ in range(n_layers)]
    h_gpu = [[] for _ in range(n_layers)]
    S_gpu = [[] for _ in range(n_layers)]
    with torch.no_grad():
        for b in range(B):
            prompt = torch.randint(0, V, (1, int(lens[b])), generator=g)
            _, hr, sr = orc.model_step(prompt, sd_prefill, n_layers, H)
            _, st = model.step(prompt.cuda())
            for layer in range(n_layers):
                h_ref[layer].append(hr[layer]); S_ref[layer].append(sr[layer])
                h_gpu[layer].append(st["h"][layer]); S_gpu[layer].append(st["S"][layer])
    h_ref = [torch.cat(t) for t in h_ref]
    S_ref = [torch.cat(t) for t in S_ref]
    state = {"h": [torch.cat(t) for t in h_gpu], "S": [torch.cat(t) for t in S_gpu]}
    prefill_err = max(rel_l2(a, b) for a, b in zip(state["S"], S_ref))
    assert prefill_err <= TOL, prefill_err
    pos = lens.to(torch.int32)
    drift = []
    with torch.no_grad():
        for step in range(steps):
            tok = torch.randint(0, V, (B, 1), generator=g)
            logits, state = model.step(tok.cuda(), (pos + step).cuda(), state, max_position=4096 + steps + 8)
            ref, h_ref, S_ref = orc.model_step(tok, sd, n_layers, H, h_ref, S_ref, pos + step)
            drift.append(max(rel_l2(a, b) for a, b in zip(state["S"], S_ref)))
            assert rel_l2(logits.float(), ref) <= 2e-2, (step, rel_l2(logits.float(), ref))
            assert drift[-1] <= TOL, (step, drift[-1])
    assert _lib.device_status() == 0
    print(f"carried-state rel-L2 vs oracle: after prefill {prefill_err:.2e}, step 1 {drift[0]:.2e}, step 64 {drift[-1]:.2e}")
