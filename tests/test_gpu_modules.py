"""GPU parity of the drop-in modules against outputs of the reference's own modules (golden
fixtures) and the CPU oracle: block, tiny model, persistence semantics, state-dict contract."""
import pytest
import torch

import jarvis_b200
from jarvis_b200 import _lib, modules as jm
from oracle import jarvis_oracle as orc
from tests.golden.loader import load

pytestmark = pytest.mark.gpu
TOL = 1e-2   # rel-L2 of bf16 compute against the fp32 reference


def rel_l2(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def test_block_fixture():
    g = load("block")
    sd = {k[3:]: v for k, v in g.items() if k.startswith("sd_")}
    blk = jm.JarvisBlock(128, 2, 4, 2).eval()
    assert set(blk.state_dict().keys()) == set(sd.keys()) and len(sd) == 23
    blk.load_state_dict(sd)
    blk = blk.cuda()
    x, h_last, l_bal, l_ref = blk(g["x"].cuda(), g["h_prev"].cuda(), start_pos=int(g["start_pos"]))
    assert _lib.device_status() == 0
    assert rel_l2(x, g["x_out"]) <= TOL
    assert rel_l2(h_last, g["h_last"]) <= 2e-2   # last-token membrane alone: few elements, same bf16 inputs
    assert abs(float(l_bal) - float(g["l_balance"])) <= 2e-2 * abs(float(g["l_balance"]))
    assert abs(float(l_ref) - float(g["l_reflect"])) <= 5e-2 * abs(float(g["l_reflect"])) + 1e-6


def test_model_fixture_and_persistence():
    g = load("model")
    sd = {k[3:]: v for k, v in g.items() if k.startswith("sd_")}
    model = jm.Jarvis(vocab_size=256, d_model=128, n_layers=2, n_heads=2, max_seq_len=256).eval()
    assert set(model.state_dict().keys()) == set(sd.keys())
    model.load_state_dict(sd)
    model = model.cuda()
    idx = g["idx"].cuda()
    logits, loss = model(idx)
    assert loss is None and logits.shape == (2, 96, 256)
    assert rel_l2(logits.float(), g["logits"]) <= 1.5e-2   # + bf16 lm_head and bf16 logits
    st = model.get_backend_status()
    assert st["attn_backend"] == "cuda" and st["moe_backend"] == "cuda" and st["attn_cuda_blocks"] == "2/2"
    # persist_state: LSF membrane + RoPE offset carried (reference semantics), then reset
    model.reset_state()
    la, _ = model(idx[:, :32], persist_state=True)
    assert model._token_pos == 32 and all(h is not None and h.shape == (2, 128) for h in model._h_states)
    lb, _ = model(idx[:, 32:64], persist_state=True)
    assert model._token_pos == 64
    assert rel_l2(la.float(), g["persist_logits_a"]) <= 1.5e-2
    assert rel_l2(lb.float(), g["persist_logits_b"]) <= 1.5e-2
    model.reset_state()
    assert model._token_pos == 0 and all(h is None for h in model._h_states)
    # targets -> loss is finite and includes the aux terms
    _, loss = model(idx, targets=idx)
    assert torch.isfinite(loss)


def test_model_fixture_with_the_prologue_fused_into_the_projection():
    """Same fixtures with the attention feature map + RoPE done by the q/k/v GEMM's epilogue (off by default)."""
    g = load("model")
    sd = {k[3:]: v for k, v in g.items() if k.startswith("sd_")}
    model = jm.Jarvis(vocab_size=256, d_model=128, n_layers=2, n_heads=2, max_seq_len=256).eval()
    model.load_state_dict(sd)
    model = model.cuda()
    for blk in model.blocks:
        blk.attn.fuse_prologue = True
    idx = g["idx"].cuda()
    logits, _ = model(idx)
    assert rel_l2(logits.float(), g["logits"]) <= 1.5e-2
    model.reset_state()
    la, _ = model(idx[:, :32], persist_state=True)
    lb, _ = model(idx[:, 32:64], persist_state=True)          # start_pos = 32 goes through the epilogue's positions
    assert rel_l2(la.float(), g["persist_logits_a"]) <= 1.5e-2
    assert rel_l2(lb.float(), g["persist_logits_b"]) <= 1.5e-2
    # state-carrying chunked prefill: the state leaves and re-enters the scan in the natural (D_v, D_k) order
    a, st = model.step(idx[:, :64])
    b, _ = model.step(idx[:, 64:], positions=64, state=st)
    for blk in model.blocks:
        blk.attn.fuse_prologue = False
    a2, st2 = model.step(idx[:, :64])
    b2, _ = model.step(idx[:, 64:], positions=64, state=st2)
    assert rel_l2(a.float(), a2.float()) <= 1e-2 and rel_l2(b.float(), b2.float()) <= 1e-2
    for x, y in zip(st["S"], st2["S"]):
        assert rel_l2(x, y) <= 1e-2
    assert _lib.device_status() == 0


def test_ragged_state_carrying_decode_matches_oracle():
    """Prefill of ragged lengths is emulated by random carried states and per-sequence positions; then
    T=1 steps with the state handed from step to step, against the oracle stepped the same way."""
    g = load("model")
    sd = {k[3:]: v for k, v in g.items() if k.startswith("sd_")}
    model = jm.Jarvis(vocab_size=256, d_model=128, n_layers=2, n_heads=2, max_seq_len=256).eval()
    model.load_state_dict(sd)
    model = model.cuda()
    gen = torch.Generator().manual_seed(3)
    B = 5
    pos = torch.tensor([1, 40, 7, 300, 4095], dtype=torch.int32)
    state = {"h": [torch.randn(B, 128, generator=gen) for _ in range(2)],
             "S": [torch.randn(B, 2, 64, 64, generator=gen) * 3 for _ in range(2)]}
    st_gpu = {k: [t.cuda() for t in v] for k, v in state.items()}
    h_ref, S_ref = state["h"], state["S"]
    for step in range(3):
        idx = torch.randint(0, 256, (B, 1), generator=gen)
        logits, st_gpu = model.step(idx.cuda(), (pos + step).cuda(), st_gpu, max_position=4200)
        ref, h_ref, S_ref = orc.model_step(idx, sd, 2, 2, h_ref, S_ref, pos + step)
        assert rel_l2(logits.float(), ref) <= 1.5e-2, step
        for layer in range(2):
            assert rel_l2(st_gpu["S"][layer], S_ref[layer]) <= TOL
            assert rel_l2(st_gpu["h"][layer], h_ref[layer]) <= 2e-2
    assert _lib.device_status() == 0
    # chunked prefill through step() equals one call of the attention-carrying path
    idx = torch.randint(0, 256, (2, 96), generator=gen).cuda()
    full, _ = model.step(idx)
    a, st = model.step(idx[:, :64])
    b, _ = model.step(idx[:, 64:], positions=64, state=st)
    # (the LSF decay is per call, so only the first chunk is comparable bit-for-bit in spirit)
    assert rel_l2(a.float(), full[:, :64].float()) < 5e-2


def test_decode_session_graph_replay_matches_eager_steps():
    torch.manual_seed(5)
    model = jm.ternary_init_(jm.Jarvis(vocab_size=256, d_model=128, n_layers=2, n_heads=2, max_seq_len=512)).cuda().eval()
    B = 4
    gen = torch.Generator(device="cuda").manual_seed(1)
    pos = torch.tensor([3, 50, 9, 200], dtype=torch.int32, device="cuda")
    state = {"h": [torch.randn(B, 128, generator=gen, device="cuda") for _ in range(2)],
             "S": [torch.randn(B, 2, 64, 64, generator=gen, device="cuda") for _ in range(2)]}
    ref_state = {k: [t.clone() for t in v] for k, v in state.items()}
    sess = jm.DecodeSession(model, state, pos, max_position=400).capture()
    sess.load_state(ref_state, pos)                      # capture advanced the buffers: reset them
    toks = torch.randint(0, 256, (3, B, 1), generator=gen, device="cuda")
    for i in range(3):
        got = sess.step(toks[i]).clone()
        want, ref_state = model.step(toks[i], pos + i, ref_state, max_position=400)
        assert torch.equal(got, want), i                 # same kernels, same order: bit-identical
    for a, b in zip(sess.state["S"], ref_state["S"]):
        assert torch.equal(a, b)
    assert torch.equal(sess.positions, pos + 3)


def test_dependent_launch_on_and_off_give_the_same_results():
    """The kernels of the chain start while their predecessor is still running and wait before they touch memory
    (programmatic dependent launch): a prefill forward, eager decode steps and a captured decode graph must give
    what fully serialised launches give (the only run-to-run freedom is the order of the fp64 atomics behind
    act_var, far below the comparison's resolution)."""
    torch.manual_seed(6)
    model = jm.ternary_init_(jm.Jarvis(vocab_size=256, d_model=128, n_layers=3, n_heads=2, max_seq_len=512)).cuda().eval()
    gen = torch.Generator(device="cuda").manual_seed(2)
    idx = torch.randint(0, 256, (3, 300), generator=gen, device="cuda")
    B = 6
    pos = torch.randint(1, 300, (B,), generator=gen, device="cuda", dtype=torch.int32)
    state0 = {"h": [torch.randn(B, 128, generator=gen, device="cuda") for _ in range(3)],
              "S": [torch.randn(B, 2, 64, 64, generator=gen, device="cuda") for _ in range(3)]}
    toks = torch.randint(0, 256, (4, B, 1), generator=gen, device="cuda")
    results = {}
    before = _lib.set_dependent_launch(True)                # on unless JB200_DEPENDENT_LAUNCH=0 started the process
    try:
        for on in (False, True):
            _lib.set_dependent_launch(on)
            with torch.no_grad():
                logits = model(idx)[0].float().clone()
            st = {k: [t.clone() for t in v] for k, v in state0.items()}
            steps = []
            for i in range(4):
                out, st = model.step(toks[i], pos + i, st, max_position=400)
                steps.append(out.float().clone())
            sess = jm.DecodeSession(model, {k: [t.clone() for t in v] for k, v in state0.items()}, pos.clone(),
                                    max_position=400).capture()
            sess.load_state(state0, pos)
            graph_steps = [sess.step(toks[i]).float().clone() for i in range(4)]
            torch.cuda.synchronize()
            results[on] = (logits, steps, graph_steps, [t.clone() for t in st["S"]])
    finally:
        _lib.set_dependent_launch(before)
    assert _lib.device_status() == 0
    off, on = results[False], results[True]
    assert rel_l2(on[0], off[0]) < 1e-5
    for a, b, c in zip(on[1], off[1], on[2]):
        assert rel_l2(a, b) < 1e-5 and rel_l2(c, b) < 1e-5
    for a, b in zip(on[3], off[3]):
        assert rel_l2(a, b) < 1e-6


def test_prefill_session_graph_replay_matches_the_eager_forward():
    torch.manual_seed(9)
    model = jm.ternary_init_(jm.Jarvis(vocab_size=256, d_model=128, n_layers=2, n_heads=2, max_seq_len=512)).cuda().eval()
    gen = torch.Generator(device="cuda").manual_seed(3)
    sess = jm.PrefillSession(model, 3, 200).capture()
    for _ in range(2):
        idx = torch.randint(0, 256, (3, 200), generator=gen, device="cuda")
        got = sess(idx).float().clone()
        with torch.no_grad():
            want = model(idx)[0].float()
        assert rel_l2(got, want) < 1e-5
    assert _lib.device_status() == 0


def test_attention_state_handoff_matches_single_call():
    """Beyond the reference: carrying S makes prefill(T1) + prefill(T2) equal one prefill of the
    attention stage (the LSF decay stays per call, so the comparison is at the attention module)."""
    torch.manual_seed(0)
    attn = jm.ternary_init_(jm.AssociativeLinearAttention(256, 4)).cuda().eval()
    x = torch.randn(2, 192, 256, device="cuda")
    y_full = attn(x)
    y_a, S = attn.forward_with_state(x[:, :128])
    y_b, _ = attn.forward_with_state(x[:, 128:], start_pos=128, h_prev=S)
    assert rel_l2(torch.cat((y_a, y_b), 1), y_full) < 5e-3
    # oracle with the same carried state
    ref = orc.attention_forward(x.cpu(), attn.q_proj.weight.cpu(), attn.k_proj.weight.cpu(), attn.v_proj.weight.cpu(),
                                attn.out_proj.weight.cpu(), attn.gamma_raw.detach().cpu(), 4)
    assert rel_l2(y_full, ref) <= TOL


def test_moe_module_matches_oracle_with_own_routing():
    torch.manual_seed(1)
    moe = jm.ternary_init_(jm.SparseMoELayer(256)).cuda().eval()
    x = torch.randn(2, 300, 256, device="cuda").bfloat16().float()
    out, l_bal, act_mean, act_var = moe(x)
    ref_out, ref_lb, ref_mean, ref_var, aux = orc.moe_forward(
        x.cpu(), moe.router.weight.detach().cpu(), [m.weight.detach().cpu() for m in moe.w1],
        [m.weight.detach().cpu() for m in moe.w2])
    idx = moe.last_routing[0].cpu()
    same = (idx == aux["idx"]).all(dim=-1)
    assert same.float().mean() > 0.995          # near-ties may resolve differently
    o, r = out.view(-1, 256).cpu()[same], ref_out.view(-1, 256)[same]
    assert rel_l2(o, r) <= TOL
    assert abs(float(l_bal) - float(ref_lb)) < 1e-4
    assert abs(float(act_var) - float(ref_var)) <= 3e-2 * float(ref_var)


def test_lsf_ext_module_persistence():
    ext = jm.LiquidStateFusionExt(persistent=True)
    a = torch.rand(2, 40, 8, device="cuda") * 0.98 + 0.01
    m = torch.randn(2, 40, 8, device="cuda")
    H = ext(a, m)
    H2 = ext(a, m)                       # continues from the stored last state
    ref = orc.lsf_scan(m.cpu(), a.cpu(), H[:, -1].cpu())
    assert torch.allclose(H2.cpu(), ref, atol=1e-5)
    ext.reset_state()
    assert torch.allclose(ext(a, m), H, atol=0)


def test_packed_checkpoint_round_trip():
    """Export in the reference exporter's key format, load into a fresh model: same logits bit for bit,
    and the packed bytes equal the oracle's packing of the oracle's quantisation."""
    from jarvis_b200 import checkpoint as ck
    torch.manual_seed(11)
    a = jm.ternary_init_(jm.Jarvis(vocab_size=256, d_model=128, n_layers=2, n_heads=2, max_seq_len=128)).cuda().eval()
    sd = {("_orig_mod." + k if i % 2 else k): v for i, (k, v) in enumerate(a.state_dict().items())}
    packed, meta = ck.export_packed_state_dict(sd)
    assert "blocks.0.attn.q_proj.weight.packed_weight" in packed and "blocks.1.moe.w2.3.weight.alpha" in packed
    assert packed["tok_emb.weight"].dtype == torch.bfloat16 and len(meta) == 2 * 12
    w = a.state_dict()["blocks.0.moe.w1.2.weight"].cpu()
    alpha, q = orc.absmean_quantize(w)
    assert abs(float(packed["blocks.0.moe.w1.2.weight.alpha"]) - alpha) <= 1e-6 * alpha
    assert (packed["blocks.0.moe.w1.2.weight.packed_weight"] != orc.pack_ternary(q)).sum() <= 2
    b = jm.Jarvis(vocab_size=256, d_model=128, n_layers=2, n_heads=2, max_seq_len=128).cuda().eval()
    ck.load_packed_state_dict(b, packed)
    # the non-ternary tensors went through bf16: give model a the same rounding before comparing
    with torch.no_grad():
        for k, v in a.state_dict().items():
            if not ck.is_ternary_key(k, v) and v.is_floating_point():
                v.copy_(v.to(torch.bfloat16).float())
    idx = torch.randint(0, 256, (2, 64), device="cuda")
    assert torch.equal(a(idx)[0], b(idx)[0])


def test_tbin_container_runs_and_round_trips(tmp_path):
    import os
    from jarvis_b200 import checkpoint as ck
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "tiny.jarvis-tbin")
    g = load("tbin")
    packed, _ = ck.read_tbin(path)
    model = jm.Jarvis(vocab_size=64, d_model=128, n_layers=1, n_heads=2, max_seq_len=64).cuda().eval()
    ck.load_packed_state_dict(model, packed)
    logits, _ = model(g["idx"].cuda())
    assert rel_l2(logits.float(), g["logits"]) <= 1.5e-2          # the reference ran the same container on CPU
    out = tmp_path / "again.jarvis-tbin"
    ck.write_tbin(model.state_dict(), str(out))
    again, meta = ck.read_tbin(str(out))
    assert set(again) == set(packed) and len(meta["tensors"]) == 26
    for k in packed:
        if k.endswith(".packed_weight"):
            assert torch.equal(again[k], packed[k]), k          # alpha * q re-quantises to the same codes
        elif not k.endswith(".alpha"):
            assert torch.equal(again[k], packed[k]), k


def test_cpu_tensors_are_rejected():
    lin = jm.TernaryLinear(64, 128)
    with pytest.raises(RuntimeError, match="no CPU fallback|CUDA"):
        lin(torch.randn(2, 64))
