"""Pins the CPU oracle against fixtures produced by the reference's own modules
(tests/golden/make_golden.py).  CPU only."""
import torch

from oracle import jarvis_oracle as orc
from tests.golden.loader import load

FP32_TOL = 2e-5


def close(a, b, tol=FP32_TOL):
    """fp32 agreement up to summation order: max error relative to the tensor's own scale (the
    scan has no normaliser, so intermediate values are ~100x the outputs and absolute
    differences of 1e-4 between two fp32 evaluations are rounding noise)."""
    scale = max(float(b.abs().max()), 1e-6)
    return float((a - b).abs().max()) <= tol * scale * 10 and float((a - b).norm()) <= tol * max(float(b.norm()), 1e-6) * 10


def test_pack_fixture():
    g = load("pack")
    alpha, q = orc.absmean_quantize(g["w"])
    assert alpha == float(g["alpha"])
    assert torch.equal(q, g["q"])
    assert torch.equal(orc.pack_ternary(q), g["packed"])
    assert torch.equal(orc.unpack_ternary(g["packed"], q.shape), g["unpacked"])
    for pat, packed in zip(g["patterns"], g["patterns_packed"]):
        assert torch.equal(orc.pack_ternary(pat), packed)
        assert torch.equal(orc.unpack_ternary(packed, pat.shape), pat)
    assert torch.equal(orc.ternary_linear(g["x"], q, alpha), g["y"])


def _attn_weights(g):
    return [g[f"{n}.weight"] for n in ("q_proj", "k_proj", "v_proj", "out_proj")]


def test_attention_fixture():
    g = load("attention")
    w = _attn_weights(g)
    for T in (1, 17, 64, 37, 123, 192):
        y = orc.attention_forward(g[f"T{T}_x"], *w, g["gamma_raw"], 2, int(g[f"T{T}_start_pos"]))
        assert close(y, g[f"T{T}_y"]), T
    for tag in ("lo", "hi"):
        y = orc.attention_forward(g[f"g{tag}_x"], *w, g[f"g{tag}_gamma_raw"], 2)
        assert close(y, g[f"g{tag}_y"]), tag


def test_attention_carried_state_fixture():
    g = load("attention_state")
    w = _attn_weights(g)
    for T in (64, 128, 50):
        y = orc.attention_forward(g[f"T{T}_x"], *w, g["gamma_raw"], 2, 5, g[f"T{T}_S0"])
        assert close(y, g[f"T{T}_y"], 1e-4), T
    qr, kr = orc.feature_map_rope(g["rope_q"], g["rope_k"], int(g["rope_start"]))
    assert close(qr, g["rope_q_out"]) and close(kr, g["rope_k_out"])
    # chunk-state scan: S_{k+1} = gamma^c S_k + dS_k, all entering states + the last one
    S = g["scan_h0"].clone()
    for kk in range(g["scan_dS"].shape[2]):
        assert close(S, g["scan_all"][:, :, kk])
        S = g["scan_gc"].view(1, -1, 1, 1) * S + g["scan_dS"][:, :, kk]
    assert close(S, g["scan_last"])


def test_chunked_scan_equals_token_recurrence():
    gen = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(1, 2, 150, 64, generator=gen) for _ in range(3))
    q, k = orc.feature_map_rope(q, k, 0)
    gamma = torch.tensor([0.9, 0.999])
    S0 = torch.randn(1, 2, 64, 64, generator=gen)
    o, S = orc.attn_scan_chunked(q, k, v, gamma, S0)
    o64, S64 = orc.attn_scan_recurrent(q, k, v, gamma, S0)
    assert float((o - o64).norm() / o64.norm()) < 1e-5
    assert float((S - S64).norm() / S64.norm()) < 1e-5
    # splitting the sequence and carrying the state reproduces the one-shot result
    o_a, S_a = orc.attn_scan_chunked(q[:, :, :70], k[:, :, :70], v[:, :, :70], gamma, S0)
    o_b, S_b = orc.attn_scan_chunked(q[:, :, 70:], k[:, :, 70:], v[:, :, 70:], gamma, S_a)
    assert float((torch.cat((o_a, o_b), 2) - o64).norm() / o64.norm()) < 1e-5
    assert float((S_b - S64).norm() / S64.norm()) < 1e-5


def test_moe_fixture():
    g = load("moe")
    w1 = [g[f"w1.{e}.weight"] for e in range(4)]
    w2 = [g[f"w2.{e}.weight"] for e in range(4)]
    for tag in ("b1t16", "b2t64", "all_e0", "e0_empty", "imbalanced"):
        out, lb, am, av, aux = orc.moe_forward(g[f"{tag}_x"], g[f"{tag}_router"], w1, w2)
        assert torch.equal(aux["idx"], g[f"{tag}_topk_idx"]), tag
        assert close(aux["probs"], g[f"{tag}_probs"])
        assert close(out, g[f"{tag}_y"]), tag
        assert abs(float(lb) - float(g[f"{tag}_l_balance"])) < 1e-6
        assert abs(float(am) - float(g[f"{tag}_act_mean"])) < 1e-6
        assert abs(float(av) - float(g[f"{tag}_act_var"])) < 1e-6
        counts, offsets, scatter, gather, gate_idx = orc.moe_metadata(aux["idx"], 4)
        order = g[f"{tag}_order"]            # slot -> flattened assignment m, per the boolean masks
        assert torch.equal(gather.long() * 2 + gate_idx.long(), order), tag
        assert torch.equal(scatter.reshape(-1).long()[order], torch.arange(order.numel()))
        assert int(offsets[-1]) == order.numel() and torch.equal(offsets[1:] - offsets[:-1], counts)
    assert int(orc.moe_metadata(g["e0_empty_topk_idx"], 4)[0][0]) == 0


def test_lsf_fixture():
    g = load("lsf")
    for tag in ("t1", "t65", "t200"):
        h_out, h_last = orc.lsf_model(g[f"{tag}_x"], g[f"{tag}_act_var"], g["var_scale"], g.get(f"{tag}_h_prev"))
        assert close(h_out, g[f"{tag}_h_out"]) and close(h_last, g[f"{tag}_h_last"])
        # the closed form equals the sequential scan with the same scalar alpha
        alpha = orc.lsf_alpha(g[f"{tag}_act_var"], g["var_scale"])
        assert close(orc.lsf_scan(g[f"{tag}_x"], alpha, g.get(f"{tag}_h_prev")), g[f"{tag}_h_out"], 1e-4)
    for T in (1, 15, 65, 127, 129, 256):
        H = orc.lsf_scan(g[f"ext{T}_M"], g[f"ext{T}_alpha"], g[f"ext{T}_h0"])
        assert close(H, g[f"ext{T}_H"], 1e-6), T


def test_block_fixture():
    g = load("block")
    p = {k[3:]: v for k, v in g.items() if k.startswith("sd_")}
    r = orc.block_forward(g["x"], p, 2, g["h_prev"], int(g["start_pos"]))
    assert close(r["x"], g["x_out"]) and close(r["h_last"], g["h_last"])
    assert abs(float(r["l_balance"]) - float(g["l_balance"])) < 1e-6
    assert abs(float(r["l_reflect"]) - float(g["l_reflect"])) < 1e-6


def test_model_fixture():
    g = load("model")
    sd = {k[3:]: v for k, v in g.items() if k.startswith("sd_")}
    assert len(sd) == int(g["n_state_keys"]) == 2 * 23 + 3
    logits, _ = orc.model_forward(g["idx"], sd, 2, 2)
    assert close(logits, g["logits"], 1e-4)
    # persist_state=True: LSF membrane and RoPE offset carried across calls, attention state not
    la, h = orc.model_forward(g["idx"][:, :32], sd, 2, 2)
    lb, _ = orc.model_forward(g["idx"][:, 32:64], sd, 2, 2, h_prevs=h, start_pos=32)
    assert close(la, g["persist_logits_a"], 1e-4) and close(lb, g["persist_logits_b"], 1e-4)
