"""GPU parity of the non-GEMM stages against the CPU oracle and the reference-generated golden
fixtures: attention scan (+ carried state), router, dispatch order, gather/combine, LSF, RMSNorm.
Integer / index results must be bit-exact; floating-point results are compared with
rel-L2 <= 1e-2 against the fp32 oracle (bf16 compute), tighter where the kernel runs in fp32."""
import pytest
import torch

import jarvis_b200  # noqa: F401
from jarvis_b200 import _lib, ops
from oracle import jarvis_oracle as orc
from tests.golden.loader import load

pytestmark = pytest.mark.gpu
TOL_BF16 = 1e-2


def rel_l2(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def rope_tabs(n_pos):
    cos, sin = orc.rope_tables(n_pos, 64)
    return cos[:, :32].contiguous().cuda(), sin[:, :32].contiguous().cuda()


# ------------------------------------------------------------------ rmsnorm / embedding
@pytest.mark.parametrize("C", [128, 1024, 2048])
def test_rmsnorm(C):
    g = torch.Generator().manual_seed(C)
    x = torch.randn(37, C, generator=g)
    w = torch.rand(C, generator=g) + 0.5
    ref = orc.rmsnorm(x, w)
    assert rel_l2(ops.rmsnorm(x.cuda(), w.cuda(), out_dtype=torch.float32), ref) < 1e-6
    assert rel_l2(ops.rmsnorm(x.cuda(), w.cuda()).float(), ref) < 4e-3
    xb = x.bfloat16()
    assert rel_l2(ops.rmsnorm(xb.cuda(), w.cuda(), out_dtype=torch.float32), orc.rmsnorm(xb.float(), w)) < 1e-6


def test_embedding():
    g = torch.Generator().manual_seed(0)
    table = torch.randn(1000, 128, generator=g)
    idx = torch.randint(0, 1000, (3, 50), generator=g)
    assert torch.equal(ops.embedding(idx.cuda(), table.cuda()).cpu(), table[idx])


# ------------------------------------------------------------------ attention scan
def _scan_case(B, H, T, seed, start_pos=0, with_state=False, gammas=None):
    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(B, T, H * 64, generator=g).bfloat16() for _ in range(3))
    gamma = torch.rand(H, generator=g) * 0.099 + 0.9 if gammas is None else torch.tensor(gammas)
    S0 = torch.randn(B, H, 64, 64, generator=g) if with_state else None

    def heads(t):
        return t.float().view(B, T, H, 64).transpose(1, 2)

    per_seq = torch.is_tensor(start_pos)
    o_ref = torch.empty(B, H, T, 64, dtype=torch.float64)
    S_ref = torch.empty(B, H, 64, 64, dtype=torch.float64)
    for b in range(B):
        sp = int(start_pos[b]) if per_seq else start_pos
        qf, kf = orc.feature_map_rope(heads(q)[b:b + 1], heads(k)[b:b + 1], sp)
        o_ref[b:b + 1], S_ref[b:b + 1] = orc.attn_scan_recurrent(qf, kf, heads(v)[b:b + 1], gamma,
                                                                 None if S0 is None else S0[b:b + 1])
    n_pos = (int(start_pos.max()) if per_seq else start_pos) + T
    cos, sin = rope_tabs(n_pos)
    qkv = torch.cat((q, k, v), dim=-1).reshape(B * T, 3 * H * 64).cuda()   # fused projection layout
    o, S = ops.attn_scan(qkv[:, :H * 64], qkv[:, H * 64:2 * H * 64], qkv[:, 2 * H * 64:], gamma.cuda(), cos, sin,
                         B, T, H, start_pos=start_pos.cuda() if per_seq else start_pos,
                         state_in=None if S0 is None else S0.cuda(), want_state=True)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    o = o.float().cpu().view(B, T, H, 64).transpose(1, 2)
    return rel_l2(o, o_ref), rel_l2(S, S_ref)


@pytest.mark.parametrize("T", [1, 17, 63, 64, 65, 127, 128, 289, 512])
def test_attn_scan_lengths(T):
    eo, es = _scan_case(2, 2, T, seed=42 + T)
    assert eo <= TOL_BF16 and es <= TOL_BF16, (eo, es)


def test_attn_scan_carried_state_and_positions():
    eo, es = _scan_case(2, 3, 200, seed=1, start_pos=128, with_state=True)
    assert eo <= TOL_BF16 and es <= TOL_BF16, (eo, es)
    eo, es = _scan_case(3, 2, 70, seed=2, start_pos=torch.tensor([0, 5, 1000], dtype=torch.int32), with_state=True)
    assert eo <= TOL_BF16 and es <= TOL_BF16, (eo, es)


@pytest.mark.parametrize("B,H,T", [(10, 16, 1100), (19, 8, 1025), (38, 4, 1500)])
def test_attn_scan_balanced_launch_cuts_sequences_in_two(B, H, T):
    """A few more sequence-heads than SMs (a last wave at most half full): that many are cut in two inside ONE
    launch, the second part starting from the state the first part's CTA leaves behind.  Same results as any
    other launch: outputs and final state against the fp64 recurrence, with a carried state and ragged positions;
    and bit-identical to the call without scratch memory (which never cuts)."""
    props = torch.cuda.get_device_properties(0)
    U, sms = B * H, props.multi_processor_count
    pos = torch.randint(0, 500, (B,), generator=torch.Generator().manual_seed(B), dtype=torch.int32)
    eo, es = _scan_case(B, H, T, seed=B + T, start_pos=pos, with_state=True)
    assert eo <= TOL_BF16 and es <= TOL_BF16, (eo, es)
    g = torch.Generator(device="cuda").manual_seed(T)
    C = H * 64
    qkv = torch.randn(B * T, 3 * C, generator=g, device="cuda").bfloat16()
    gamma = torch.rand(H, generator=g, device="cuda") * 0.099 + 0.9
    cos, sin = rope_tabs(T)
    args = (qkv[:, :C], qkv[:, C:2 * C], qkv[:, 2 * C:], gamma, cos, sin, B, T, H)
    o1, S1 = ops.attn_scan(*args, want_state=True)
    o2, S2 = ops.attn_scan(*args, want_state=True, segmented=False)
    assert torch.equal(o1, o2) and torch.equal(S1, S2)
    if sms == 148:
        assert U > sms and 0 < U % sms <= sms // 2      # the shapes above are meant to take the balanced launch
    assert _lib.device_status() == 0


@pytest.mark.parametrize("B,H", [(3, 2), (40, 4), (301, 16)])
def test_attn_single_token_steps_with_carried_state(B, H):
    """T = 1 with a carried state and ragged positions: a handful of (sequence, head) pairs take the per-pair
    kernel, 64 pairs or more stream the state tiles through shared memory; in place and out of place."""
    pos = torch.randint(0, 3000, (B,), generator=torch.Generator().manual_seed(B), dtype=torch.int32)
    eo, es = _scan_case(B, H, 1, seed=7 * B + H, start_pos=pos, with_state=True)
    assert eo <= TOL_BF16 and es <= 1e-5, (eo, es)
    # in place == out of place, bit for bit, and two different batch sizes of the same rows agree
    g = torch.Generator(device="cuda").manual_seed(B)
    qkv = torch.randn(B, 3 * H * 64, generator=g, device="cuda").bfloat16()
    gamma = torch.rand(H, generator=g, device="cuda") * 0.099 + 0.9
    S0 = torch.randn(B, H, 64, 64, generator=g, device="cuda")
    cos, sin = rope_tabs(3001)
    C = H * 64
    args = (qkv[:, :C], qkv[:, C:2 * C], qkv[:, 2 * C:], gamma, cos, sin)
    o1, S1 = ops.attn_scan(*args, B, 1, H, start_pos=pos.cuda(), state_in=S0, want_state=True)
    S2 = S0.clone()
    o2, S2r = ops.attn_scan(*args, B, 1, H, start_pos=pos.cuda(), state_in=S2, want_state=True, state_out=S2)
    assert S2r.data_ptr() == S2.data_ptr() and torch.equal(S1, S2) and torch.equal(o1, o2)
    # the first sequences alone (fewer pairs: possibly the other kernel): same state bits
    nb = min(B, 3)
    sub = tuple(a[:nb] for a in args[:3]) + args[3:]
    _, S3 = ops.attn_scan(*sub, nb, 1, H, start_pos=pos[:nb].cuda(), state_in=S0[:nb].contiguous(), want_state=True)
    assert torch.equal(S3, S1[:nb])
    assert _lib.device_status() == 0


@pytest.mark.parametrize("T", [1000, 2048])
def test_attn_scan_segmented_long_sequences(T):
    """Long sequences are cut into parallel segments (state pre-pass + fold); result must match the
    oracle and the unsegmented kernel, with and without an incoming state."""
    eo, es = _scan_case(1, 2, T, seed=T, start_pos=7, with_state=True)
    assert eo <= TOL_BF16 and es <= TOL_BF16, (eo, es)
    g = torch.Generator().manual_seed(T + 1)
    B, H = 2, 2
    qkv = torch.randn(B * T, 3 * H * 64, generator=g).bfloat16().cuda()
    gamma = (torch.rand(H, generator=g) * 0.099 + 0.9).cuda()
    S0 = torch.randn(B, H, 64, 64, generator=g).cuda()
    cos, sin = rope_tabs(T)
    args = (qkv[:, :H * 64], qkv[:, H * 64:2 * H * 64], qkv[:, 2 * H * 64:], gamma, cos, sin, B, T, H)
    o1, S1 = ops.attn_scan(*args, state_in=S0, want_state=True, segmented=True)
    o2, S2 = ops.attn_scan(*args, state_in=S0, want_state=True, segmented=False)
    assert rel_l2(o1.float(), o2.float()) < 3e-3 and rel_l2(S1, S2) < 1e-5


def test_attn_scan_extreme_decay():
    eo, es = _scan_case(1, 2, 150, seed=3, gammas=[0.01, 0.99])
    assert eo <= TOL_BF16 and es <= TOL_BF16, (eo, es)


def test_attn_scan_split_equals_one_shot():
    """prefill(T1) then prefill(T2) with the handed-off state == prefill(T1 + T2)."""
    g = torch.Generator().manual_seed(9)
    B, H, T = 2, 4, 192
    qkv = torch.randn(B, T, 3 * H * 64, generator=g).bfloat16().cuda()
    gamma = (torch.rand(H, generator=g) * 0.099 + 0.9).cuda()
    cos, sin = rope_tabs(T)

    def run(x, t, **kw):
        flat = x.reshape(B * t, 3 * H * 64)
        return ops.attn_scan(flat[:, :H * 64], flat[:, H * 64:2 * H * 64], flat[:, 2 * H * 64:], gamma, cos, sin, B, t,
                             H, want_state=True, **kw)

    o_full, S_full = run(qkv, T)
    o_a, S_a = run(qkv[:, :128].contiguous(), 128)
    o_b, S_b = run(qkv[:, 128:].contiguous(), 64, start_pos=128, state_in=S_a)
    o_split = torch.cat((o_a.view(B, 128, -1), o_b.view(B, 64, -1)), dim=1).reshape(B * T, -1)
    assert rel_l2(o_split.float(), o_full.float()) < 3e-3   # chunk boundaries coincide: only bf16 mirror rounding differs
    assert rel_l2(S_b, S_full) < 1e-5


def test_attention_module_fixture():
    """End to end against the reference module's outputs: projections -> scan -> out_proj."""
    gf = load("attention")
    H = 2
    packs = {}
    for n in ("q_proj", "k_proj", "v_proj", "out_proj"):
        packs[n] = ops.pack_ternary(gf[f"{n}.weight"].cuda())
    w_qkv = torch.cat([packs[n][0] for n in ("q_proj", "k_proj", "v_proj")])
    a_qkv = torch.cat([packs[n][1] for n in ("q_proj", "k_proj", "v_proj")])
    gamma = torch.sigmoid(gf["gamma_raw"]).cuda()
    cos, sin = rope_tabs(512)
    for T in (1, 17, 64, 37, 123, 192):
        x = gf[f"T{T}_x"]
        B = x.shape[0]
        xb = x.reshape(B * T, 128).bfloat16().cuda()
        qkv = ops.ternary_linear(xb, w_qkv, a_qkv, alpha_rows=128)
        o, _ = ops.attn_scan(qkv[:, :128], qkv[:, 128:256], qkv[:, 256:], gamma, cos, sin, B, T, H,
                             start_pos=int(gf[f"T{T}_start_pos"]))
        y = ops.ternary_linear(o, *packs["out_proj"], epilogue=ops.EPI_F32)
        assert rel_l2(y.view(B, T, 128), gf[f"T{T}_y"]) <= TOL_BF16, T


# ------------------------------------------------------------------ router / metadata / gather / combine
def test_router_bit_exact_on_tie_free_rows():
    g = torch.Generator().manual_seed(4)
    N, C, E = 5000, 1024, 4
    x = torch.randn(N, C, generator=g).bfloat16()
    w = torch.randn(E, C, generator=g) * 0.03
    idx_ref, gates_ref, probs_ref = orc.router_top2(x.float(), w)
    idx, gates, probs = ops.router_top2(x.cuda(), w.cuda(), want_probs=True)
    srt = probs_ref.sort(dim=-1, descending=True).values
    margin = torch.minimum(srt[:, 0] - srt[:, 1], srt[:, 1] - srt[:, 2])
    clear = margin > 1e-5
    assert clear.float().mean() > 0.99
    assert torch.equal(idx.cpu()[clear], idx_ref[clear])
    assert (idx.cpu() != idx_ref).any(dim=-1).sum().item() <= (~clear).sum().item()
    assert torch.allclose(probs.cpu(), probs_ref, atol=2e-6)
    assert torch.allclose(gates.cpu()[clear], gates_ref[clear], atol=1e-5)


def test_fused_rmsnorm_router_is_bit_identical_to_the_two_kernels():
    g = torch.Generator().manual_seed(8)
    for N, C in ((3000, 1024), (100, 256), (5000, 128)):
        x = torch.randn(N, C, generator=g).cuda() * 3
        wn = (torch.rand(C, generator=g) + 0.5).cuda()
        wr = (torch.randn(4, C, generator=g) * 0.05).cuda()
        ps1 = torch.zeros(4, dtype=torch.float64, device="cuda")
        h1 = torch.zeros(4, dtype=torch.int32, device="cuda")
        ps2, h2 = torch.zeros_like(ps1), torch.zeros_like(h1)
        xn1 = ops.rmsnorm(x, wn, 1e-6)
        idx1, gates1, _ = ops.router_top2(xn1, wr, probs_sum=ps1, top1_hist=h1)
        xn2, idx2, gates2 = ops.rmsnorm_router(x, wn, 1e-6, wr, probs_sum=ps2, top1_hist=h2)
        assert torch.equal(xn1, xn2) and torch.equal(idx1, idx2) and torch.equal(gates1, gates2)
        # P_e is summed per warp in f32 before the f64 atomics: the two kernels group the tokens differently
        assert torch.equal(h1, h2) and torch.allclose(ps1, ps2, rtol=1e-6)


def test_router_ties_go_to_lower_expert():
    x = torch.zeros(64, 256, dtype=torch.bfloat16)
    w = torch.randn(4, 256)
    idx, gates, _ = ops.router_top2(x.cuda(), w.cuda())
    assert torch.equal(idx.cpu(), torch.tensor([[0, 1]]).repeat(64, 1))
    assert torch.allclose(gates.cpu(), torch.full((64, 2), 0.5), atol=1e-6)


@pytest.mark.parametrize("N,K,E", [(1, 2, 4), (3, 2, 4), (127, 2, 4), (128, 2, 4), (129, 2, 4), (5000, 2, 4),
                                   (65536, 2, 4), (1000, 1, 8), (777, 3, 16)])
def test_metadata_bit_exact(N, K, E):
    g = torch.Generator().manual_seed(N + K + E)
    idx = torch.randint(0, E, (N, K), generator=g)
    if N >= 100:
        idx[: N // 2] = idx[: N // 2].clamp(max=1)        # skew
    ref = orc.moe_metadata(idx, E)
    got = ops.moe_metadata(idx.cuda(), E)
    for r, t in zip(ref, got):
        assert torch.equal(t.cpu(), r)


def test_metadata_forced_routings_from_fixture():
    gf = load("moe")
    for tag in ("all_e0", "e0_empty", "imbalanced", "b2t64"):
        idx = gf[f"{tag}_topk_idx"]
        counts, offsets, scatter, gather, gate_idx = (t.cpu() for t in ops.moe_metadata(idx.cuda(), 4))
        assert torch.equal(gather.long() * 2 + gate_idx.long(), gf[f"{tag}_order"]), tag
        assert torch.equal(counts.long(), torch.bincount(idx.reshape(-1), minlength=4))


def test_gather_and_combine():
    g = torch.Generator().manual_seed(6)
    N, C, E = 1000, 1024, 4
    x = torch.randn(N, C, generator=g).bfloat16()
    idx = torch.stack([torch.randperm(E, generator=g)[:2] for _ in range(N)])
    gates = torch.rand(N, 2, generator=g)
    counts, offsets, scatter, gather, gate_idx = ops.moe_metadata(idx.cuda(), E)
    disp = ops.dispatch_gather(x.cuda(), gather)
    assert torch.equal(disp.cpu(), x[gather.cpu().long()])
    y = torch.randn(2 * N, C, generator=g).bfloat16()
    stats = torch.zeros(2, dtype=torch.float64, device="cuda")
    out = ops.scatter_combine(y.cuda(), gates.cuda(), scatter, out_dtype=torch.float32, stats=stats)
    ref = (gates[:, :, None] * y.float()[scatter.cpu().long()]).sum(dim=1)
    assert rel_l2(out, ref) < 1e-6
    sc = ops.moe_finalize(stats, None, None, E, N, N * C, 0.01).cpu()
    assert abs(float(sc[1]) - float(ref.mean())) < 1e-6 and abs(float(sc[2]) - float(ref.var())) < 1e-5 * float(ref.var())
    out_bf = ops.scatter_combine(y.cuda(), gates.cuda(), scatter)
    assert rel_l2(out_bf.float(), ref) < 4e-3


def test_moe_layer_fixture():
    """Whole MoE layer against the reference module's outputs, forced routings included."""
    gf = load("moe")
    E, C = 4, 128
    w1 = [ops.pack_ternary(gf[f"w1.{e}.weight"].cuda()) for e in range(E)]
    w2 = [ops.pack_ternary(gf[f"w2.{e}.weight"].cuda()) for e in range(E)]
    p1, a1 = torch.stack([w[0] for w in w1]), torch.cat([w[1] for w in w1])
    p2, a2 = torch.stack([w[0] for w in w2]), torch.cat([w[1] for w in w2])
    for tag in ("b1t16", "b2t64", "all_e0", "e0_empty", "imbalanced"):
        x = gf[f"{tag}_x"].reshape(-1, C)
        N = x.shape[0]
        idx = gf[f"{tag}_topk_idx"].cuda()     # the reference's routing: isolates the expert path
        gates = (gf[f"{tag}_topk_probs"] / (gf[f"{tag}_topk_probs"].sum(-1, keepdim=True) + 1e-8)).cuda()
        counts, offsets, scatter, gather, gate_idx = ops.moe_metadata(idx, E)
        disp = ops.dispatch_gather(x.bfloat16().cuda(), gather)
        hid = ops.ternary_linear_grouped(disp, p1, a1, offsets, epilogue=ops.EPI_GELU_BF16)
        yd = ops.ternary_linear_grouped(hid, p2, a2, offsets, epilogue=ops.EPI_BF16)
        stats = torch.zeros(2, dtype=torch.float64, device="cuda")
        out = ops.scatter_combine(yd, gates, scatter, out_dtype=torch.float32, stats=stats)
        assert rel_l2(out.view_as(gf[f"{tag}_y"]), gf[f"{tag}_y"]) <= TOL_BF16, tag
        sc = ops.moe_finalize(stats, None, None, E, N, N * C, 0.01).cpu()
        assert abs(float(sc[2]) - float(gf[f"{tag}_act_var"])) <= 3e-2 * float(gf[f"{tag}_act_var"])
        assert _lib.device_status() == 0


def test_router_balance_loss_fixture():
    gf = load("moe")
    # the fixture's d_model (128) is below the router kernel's 256-column step: embed it in 256 columns
    for tag in ("b2t64", "imbalanced"):
        x = torch.zeros(gf[f"{tag}_x"].numel() // 128, 256)
        x[:, :128] = gf[f"{tag}_x"].reshape(-1, 128)
        w = torch.zeros(4, 256)
        w[:, :128] = gf[f"{tag}_router"]
        xb = x.bfloat16()
        idx_ref, _, probs_ref = orc.router_top2(xb.float(), w)
        psum = torch.zeros(4, dtype=torch.float64, device="cuda")
        hist = torch.zeros(4, dtype=torch.int32, device="cuda")
        idx, gates, _ = ops.router_top2(xb.cuda(), w.cuda(), probs_sum=psum, top1_hist=hist)
        sc = ops.moe_finalize(None, psum, hist, 4, x.shape[0], 1, 0.01).cpu()
        f = torch.nn.functional.one_hot(idx_ref[:, 0], 4).float().mean(0)
        lb = 0.01 * 4 * (f * probs_ref.mean(0)).sum()
        assert abs(float(sc[0]) - float(lb)) < 1e-6
        assert abs(float(lb) - float(gf[f"{tag}_l_balance"])) < 2e-4   # bf16 rounding of x only


# ------------------------------------------------------------------ LSF
def test_lsf_model_fixture():
    gf = load("lsf")
    vs = gf["var_scale"].reshape(1).cuda()
    for tag in ("t1", "t65", "t200"):
        x = gf[f"{tag}_x"].cuda()
        h0 = gf.get(f"{tag}_h_prev")
        out, last = ops.lsf_scan(x, act_var=gf[f"{tag}_act_var"].reshape(1).cuda(), var_scale=vs,
                                 h0=None if h0 is None else h0.cuda())
        assert rel_l2(out, gf[f"{tag}_h_out"]) < 2e-5, tag
        assert rel_l2(last, gf[f"{tag}_h_last"]) < 2e-5, tag


@pytest.mark.parametrize("T", [1, 15, 65, 127, 129, 256])
def test_lsf_extension_fixture(T):
    gf = load("lsf")
    out, _ = ops.lsf_scan(gf[f"ext{T}_M"].cuda(), alpha_tensor=gf[f"ext{T}_alpha"].cuda(), h0=gf[f"ext{T}_h0"].cuda())
    assert float((out.cpu() - gf[f"ext{T}_H"]).abs().max()) < 1e-5       # the reference's fp32 tolerance
    outb, _ = ops.lsf_scan(gf[f"ext{T}_M"].bfloat16().cuda(), alpha_tensor=gf[f"ext{T}_alpha"].bfloat16().cuda(),
                           h0=gf[f"ext{T}_h0"].cuda())
    assert float((outb.float().cpu() - gf[f"ext{T}_H"]).abs().max()) < 8e-2  # the reference's bf16 tolerance


@pytest.mark.parametrize("B,T,D", [(2, 1000, 192), (1, 2048, 1024), (3, 300, 66)])
def test_lsf_scan_bf16_with_residual(B, T, D):
    g = torch.Generator().manual_seed(T)
    m = torch.randn(B, T, D, generator=g).bfloat16()
    h0 = torch.randn(B, D, generator=g)
    resid = torch.randn(B, T, D, generator=g)
    alpha = torch.tensor([0.93])
    ref = orc.lsf_scan(m.float(), float(alpha), h0)
    r = resid.clone().cuda()
    out, last = ops.lsf_scan(m.cuda(), alpha_scalar=alpha.cuda(), h0=h0.cuda(), resid=r, out_dtype=torch.float32)
    assert rel_l2(out, ref) < 1e-5 and rel_l2(last, ref[:, -1]) < 1e-5
    assert rel_l2(r, resid + ref) < 1e-6
    outb, _ = ops.lsf_scan(m.cuda(), alpha_scalar=alpha.cuda(), h0=h0.cuda())
    assert rel_l2(outb.float(), ref) < 4e-3


@pytest.mark.parametrize("B,C,with_h,with_norm", [(5, 128, True, True), (256, 1024, True, True), (3, 1024, False, True),
                                                   (9, 520, True, False)])
def test_fused_single_token_tail_is_bit_identical_to_the_three_kernels(B, C, with_h, with_norm):
    """moe_finalize + the T = 1 LSF step with the fused residual + the RMSNorm that follows, in one launch."""
    gen = torch.Generator(device="cuda").manual_seed(B * 7 + C)
    m = (torch.randn(B, C, generator=gen, device="cuda") * 0.3).bfloat16()
    x = torch.randn(B, C, generator=gen, device="cuda")
    h = torch.randn(B, C, generator=gen, device="cuda") if with_h else None
    w = torch.rand(C, generator=gen, device="cuda") + 0.5
    E, n_tok = 4, B
    stats = torch.stack([m.double().sum(), (m.double() ** 2).sum()])
    probs = torch.rand(E, generator=gen, device="cuda", dtype=torch.float64) * n_tok
    hist = torch.tensor([B - 2, 1, 1, 0], dtype=torch.int32, device="cuda")
    vs = torch.tensor([1.3], device="cuda")
    # the three kernels
    sc_ref = ops.moe_finalize(stats, probs, hist, E, n_tok, n_tok * C, 0.01)
    x_ref = x.clone()
    _, h_ref = ops.lsf_scan(m.view(B, 1, C), act_var=sc_ref[2:3], var_scale=vs, alpha_min=0.1, alpha_max=0.99, h0=h,
                            resid=x_ref.view(B, 1, C), want_out=False)
    xn_ref = ops.rmsnorm(x_ref, w, 1e-6) if with_norm else None
    # one launch
    sc = torch.zeros(3, device="cuda")
    x_got = x.clone()
    xn, h_got = ops.lsf_step_norm(m, stats, probs, hist, E, n_tok, n_tok * C, 0.01, sc, vs, 0.1, 0.99, h, x_got,
                                  norm=(w, 1e-6) if with_norm else None)
    assert torch.equal(sc, sc_ref) and torch.equal(h_got, h_ref) and torch.equal(x_got, x_ref)
    assert (xn is None and xn_ref is None) or torch.equal(xn, xn_ref)
    # against the oracle's formulas
    alpha = 0.1 + 0.89 * torch.sigmoid(-vs.cpu() * sc_ref[2].cpu())
    h_want = alpha * (h.cpu() if with_h else 0.0) + (1 - alpha) * m.float().cpu()
    assert rel_l2(h_got, h_want) < 2e-6 and rel_l2(x_got, x.cpu() + h_want) < 2e-6
    if with_norm:
        assert rel_l2(xn.float(), orc.rmsnorm(x_got.cpu(), w.cpu())) < 4e-3
    # in place on the membrane
    if with_h:
        h2, x2 = h.clone(), x.clone()
        _, out = ops.lsf_step_norm(m, stats, probs, hist, E, n_tok, n_tok * C, 0.01, sc, vs, 0.1, 0.99, h2, x2, h_out=h2)
        assert out is h2 and torch.equal(h2, h_ref)
    assert _lib.device_status() == 0


def test_lsf_segmented_matches_single_pass_and_oracle():
    g = torch.Generator().manual_seed(77)
    B, T, D = 2, 3000, 192
    m = torch.randn(B, T, D, generator=g)
    a = torch.rand(B, T, D, generator=g) * 0.5 + 0.49
    h0 = torch.randn(B, D, generator=g)
    ref = orc.lsf_scan(m, a, h0)
    seg, last = ops.lsf_scan(m.cuda(), alpha_tensor=a.cuda(), h0=h0.cuda(), segmented=True)
    one, _ = ops.lsf_scan(m.cuda(), alpha_tensor=a.cuda(), h0=h0.cuda(), segmented=False)
    assert rel_l2(seg, ref) < 1e-5 and rel_l2(one, ref) < 1e-5 and rel_l2(last, ref[:, -1]) < 1e-5
    al = torch.tensor([0.985])
    ref_s = orc.lsf_scan(m, float(al), h0)
    seg_s, last_s = ops.lsf_scan(m.cuda(), alpha_scalar=al.cuda(), h0=h0.cuda(), segmented=True)
    one_s, _ = ops.lsf_scan(m.cuda(), alpha_scalar=al.cuda(), h0=h0.cuda(), segmented=False)
    assert rel_l2(seg_s, ref_s) < 1e-5 and rel_l2(one_s, ref_s) < 1e-5 and rel_l2(last_s, ref_s[:, -1]) < 1e-5


def test_lsf_linearity_large():
    """Size-independent property at a full-size shape: scan(a*x + y) == a*scan(x) + scan(y)."""
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(8, 2048, 1024, generator=g, device="cuda")
    y = torch.randn(8, 2048, 1024, generator=g, device="cuda")
    al = torch.tensor([0.97], device="cuda")
    sx, _ = ops.lsf_scan(x, alpha_scalar=al)
    sy, _ = ops.lsf_scan(y, alpha_scalar=al)
    sxy, _ = ops.lsf_scan(2.0 * x + y, alpha_scalar=al)
    assert rel_l2(sxy, 2.0 * sx + sy) < 1e-5


# ------------------------------------------------------------------ full-size properties (BASELINE shapes)
def test_gemm_linearity_at_prefill_size():
    """16384 x 3072 x 1024 (the q/k/v projection of the B=8 x T=2048 prefill): W(x1 + x2) == W x1 + W x2 up
    to the bf16 rounding of the outputs, and rows are independent of the batch they sit in."""
    g = torch.Generator(device="cuda").manual_seed(0)
    M, K, N = 16384, 1024, 3072
    x1 = torch.randint(-8, 9, (M, K), generator=g, device="cuda").float()
    x2 = torch.randint(-8, 9, (M, K), generator=g, device="cuda").float()
    q = torch.randint(-1, 2, (N, K), generator=g, device="cuda").float()
    packed = ops.prepare_weights(ops.pack_codes(q))
    one = torch.ones(1, device="cuda")
    f = lambda x: ops.ternary_linear(x.bfloat16(), packed, one, epilogue=ops.EPI_F32, prepared=True)  # noqa: E731
    y1, y2, y12 = f(x1), f(x2), f(x1 + x2)
    assert torch.equal(y12, y1 + y2)                     # integers: exact
    sub = f(x1[5000:5300].contiguous())
    assert torch.equal(sub, y1[5000:5300])
    # checksum against fp64 on a slice
    ref = (x1[:64].double() @ q.double().t()).float()
    assert torch.equal(y1[:64], ref)


def test_attn_scan_split_equals_one_shot_at_prefill_size():
    g = torch.Generator(device="cuda").manual_seed(1)
    B, H, T = 8, 16, 2048
    qkv = torch.randn(B, T, 3 * H * 64, generator=g, device="cuda").bfloat16()
    gamma = torch.rand(H, generator=g, device="cuda") * 0.099 + 0.9
    cos, sin = rope_tabs(T)
    C = H * 64

    def run(x, t, **kw):
        flat = x.reshape(B * t, 3 * C)
        return ops.attn_scan(flat[:, :C], flat[:, C:2 * C], flat[:, 2 * C:], gamma, cos, sin, B, t, H,
                             want_state=True, **kw)

    o_full, S_full = run(qkv, T)
    o_a, S_a = run(qkv[:, :1024].contiguous(), 1024)
    o_b, S_b = run(qkv[:, 1024:].contiguous(), 1024, start_pos=1024, state_in=S_a)
    o_split = torch.cat((o_a.view(B, 1024, C), o_b.view(B, 1024, C)), dim=1).reshape(B * T, C)
    assert rel_l2(o_split.float(), o_full.float()) < 3e-3
    assert rel_l2(S_b, S_full) < 1e-5
    assert _lib.device_status() == 0


def test_dispatch_round_trip_at_moe_bench_size():
    """65,536 tokens (the MoE-alone configuration): gather then combine with unit gates on one slot
    returns the input; the maps are a permutation."""
    g = torch.Generator(device="cuda").manual_seed(2)
    N, C, E = 65536, 1024, 4
    x = torch.randn(N, C, generator=g, device="cuda").bfloat16()
    idx = torch.stack((torch.randint(0, 2, (N,), generator=g, device="cuda"),
                       torch.randint(2, 4, (N,), generator=g, device="cuda")), dim=1)
    counts, offsets, scatter, gather, gate_idx = ops.moe_metadata(idx, E)
    assert int(offsets[-1]) == 2 * N and torch.equal(torch.sort(scatter.reshape(-1)).values.long(),
                                                     torch.arange(2 * N, device="cuda"))
    disp = ops.dispatch_gather(x, gather)
    gates = torch.tensor([[1.0, 0.0]], device="cuda").repeat(N, 1)
    back = ops.scatter_combine(disp, gates, scatter)
    assert torch.equal(back, x)


# ------------------------------------------------------------------ fused prologue (q/k/v GEMM epilogue + prepared scan)
def _fused_case(B, H, T, seed, start_pos=0, with_state=False):
    """x -> q|k|v projection with the attention prologue in its epilogue -> scan with prepared q/k, against the
    oracle's projection + feature map + RoPE + recurrent scan."""
    g = torch.Generator().manual_seed(seed)
    C = H * 64
    x = (torch.randn(B * T, C, generator=g) * 0.5).bfloat16()
    qs = [torch.randint(-1, 2, (C, C), generator=g).float() for _ in range(3)]
    alphas = torch.tensor([0.05, 0.04, 0.06])
    gamma = torch.rand(H, generator=g) * 0.099 + 0.9
    S0 = torch.randn(B, H, 64, 64, generator=g) if with_state else None
    per_seq = torch.is_tensor(start_pos)
    proj = [a * (x.float() @ w.t()) for a, w in zip(alphas, qs)]

    def heads(t):
        return t.view(B, T, H, 64).transpose(1, 2)

    o_ref = torch.empty(B, H, T, 64, dtype=torch.float64)
    S_ref = torch.empty(B, H, 64, 64, dtype=torch.float64)
    qk_ref = []
    for b in range(B):
        sp = int(start_pos[b]) if per_seq else start_pos
        qf, kf = orc.feature_map_rope(heads(proj[0])[b:b + 1], heads(proj[1])[b:b + 1], sp)
        qk_ref.append((qf, kf))
        o_ref[b:b + 1], S_ref[b:b + 1] = orc.attn_scan_recurrent(qf, kf, heads(proj[2])[b:b + 1], gamma,
                                                                 None if S0 is None else S0[b:b + 1])
    n_pos = (int(start_pos.max()) if per_seq else start_pos) + T
    cos, sin = rope_tabs(n_pos)
    canon = [orc.pack_ternary(w).cuda() for w in qs]
    rows = torch.cat([ops.interleave_head_rows(canon[0], H), ops.interleave_head_rows(canon[1], H), canon[2]])
    sp_dev = start_pos.cuda() if per_seq else start_pos
    outs = []
    for prepared in (False, True):
        pk = ops.prepare_weights(rows) if prepared else rows
        qkv = ops.qkv_linear_rope(x.cuda(), pk, alphas.cuda(), cos, sin, T, 2 * C, start_pos=sp_dev, alpha_rows=C,
                                  prepared=prepared)
        outs.append(qkv)
    assert torch.equal(outs[0], outs[1])
    qkv = outs[1]
    # the epilogue's q', k' (undo the head-dim interleave; q' is stored without the 1/8)
    un = torch.empty(64, dtype=torch.long)
    un[torch.arange(32)] = 2 * torch.arange(32)
    un[32 + torch.arange(32)] = 2 * torch.arange(32) + 1
    qp = qkv[:, :C].float().cpu().view(B, T, H, 64)[..., un].transpose(1, 2) * 0.125
    kp = qkv[:, C:2 * C].float().cpu().view(B, T, H, 64)[..., un].transpose(1, 2)
    q_want = torch.cat([a for a, _ in qk_ref]); k_want = torch.cat([b for _, b in qk_ref])
    assert rel_l2(qp, q_want) <= 4e-3 and rel_l2(kp, k_want) <= 4e-3          # one bf16 rounding
    assert rel_l2(qkv[:, 2 * C:].float().cpu(), proj[2]) <= 4e-3
    o, S = ops.attn_scan(qkv[:, :C], qkv[:, C:2 * C], qkv[:, 2 * C:], gamma.cuda(), cos, sin, B, T, H, start_pos=sp_dev,
                         state_in=None if S0 is None else S0.cuda(), want_state=True, qk_prepared=True)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    o = o.float().cpu().view(B, T, H, 64).transpose(1, 2)
    return rel_l2(o, o_ref), rel_l2(S, S_ref)


@pytest.mark.parametrize("T", [2, 17, 64, 65, 289, 1000])
def test_fused_prologue_lengths(T):
    eo, es = _fused_case(2, 2, T, seed=T)
    assert eo <= 1e-2 and es <= 1e-2


def test_fused_prologue_state_positions_and_segments():
    eo, es = _fused_case(2, 4, 130, seed=5, start_pos=torch.tensor([7, 300], dtype=torch.int32), with_state=True)
    assert eo <= 1e-2 and es <= 1e-2
    eo, es = _fused_case(1, 2, 2048, seed=6, start_pos=11, with_state=True)      # cut into segments
    assert eo <= 1e-2 and es <= 1e-2
    eo, es = _fused_case(3, 2, 48, seed=7)      # 32-token epilogue chunks straddle sequence boundaries (T % 32 != 0)
    assert eo <= 1e-2 and es <= 1e-2


def test_fused_prologue_argument_errors():
    x = torch.zeros(64, 128, dtype=torch.bfloat16, device="cuda")
    pk = torch.zeros(384, 32, dtype=torch.uint8, device="cuda")
    cos, sin = rope_tabs(64)
    with pytest.raises(RuntimeError, match="multiple of the sequence length"):
        ops.qkv_linear_rope(x, pk, torch.ones(3, device="cuda"), cos, sin, 48, 256, alpha_rows=128)
    with pytest.raises(RuntimeError, match="whole 64-wide heads"):
        ops.qkv_linear_rope(x, pk, torch.ones(3, device="cuda"), cos, sin, 32, 200, alpha_rows=128)
    with pytest.raises(RuntimeError, match="needs its tables"):
        ops.ternary_linear(x, pk, torch.ones(3, device="cuda"), epilogue=4, alpha_rows=128)


@pytest.mark.parametrize("T", [2, 65, 1000, 2048])
def test_attn_state_only_call_matches_the_full_scan(T):
    """o == NULL: only the k/v half runs, every piece in parallel; the end state must be the full call's (same
    bf16 products, another summation order), with and without an incoming state, and against the oracle."""
    g = torch.Generator().manual_seed(T)
    B, H = 2, 3
    q, k, v = (torch.randn(B * T, H * 64, generator=g).bfloat16().cuda() for _ in range(3))
    gamma = (torch.rand(H, generator=g) * 0.099 + 0.9).cuda()
    cos, sin = rope_tabs(T + 9)
    S0 = torch.randn(B, H, 64, 64, generator=g).cuda()
    for s_in in (None, S0):
        _, S_full = ops.attn_scan(q, k, v, gamma, cos, sin, B, T, H, start_pos=9, state_in=s_in, want_state=True)
        none, S_only = ops.attn_scan(q, k, v, gamma, cos, sin, B, T, H, start_pos=9, state_in=s_in, want_out=False)
        assert none is None
        assert rel_l2(S_only, S_full) <= 2e-3
    assert _lib.device_status() == 0

    def heads(t):
        return t.float().cpu().view(B, T, H, 64).transpose(1, 2)

    qf, kf = orc.feature_map_rope(heads(q), heads(k), 9)
    _, S_ref = orc.attn_scan_recurrent(qf, kf, heads(v), gamma.cpu(), S0.cpu())
    assert rel_l2(S_only, S_ref) <= 1e-2


def test_empty_inputs_are_accepted_everywhere():
    """Zero tokens / zero sequences: every entry point returns empty results without launching on nothing."""
    dev = "cuda"
    C, H, E = 128, 2, 4
    x0 = torch.empty(0, C, dtype=torch.bfloat16, device=dev)
    q = torch.randint(-1, 2, (128, C)).float()
    pk = orc.pack_ternary(q).cuda()
    y = ops.ternary_linear(x0, pk, torch.ones(1, device=dev))
    assert tuple(y.shape) == (0, 128)
    offs = torch.zeros(E + 1, dtype=torch.int32, device=dev)
    yg = ops.ternary_linear_grouped(x0, orc.pack_ternary(torch.zeros(E, 128, C)).cuda(), torch.ones(E, device=dev), offs)
    assert tuple(yg.shape) == (0, 128)
    assert tuple(ops.rmsnorm(torch.empty(0, C, device=dev), torch.ones(C, device=dev)).shape) == (0, C)
    idx, gates, _ = ops.router_top2(x0, torch.randn(E, C, device=dev))
    assert tuple(idx.shape) == (0, 2) and tuple(gates.shape) == (0, 2)
    counts, offsets, scatter, gather, gate_idx = ops.moe_metadata(idx, E)
    assert counts.tolist() == [0] * E and offsets.tolist() == [0] * (E + 1) and gather.numel() == 0
    disp = ops.dispatch_gather(x0, gather)
    assert tuple(disp.shape) == (0, C)
    out = ops.scatter_combine(disp, gates, scatter)
    assert tuple(out.shape) == (0, C)
    cos, sin = rope_tabs(8)
    qkv = torch.empty(0, 3 * H * 64, dtype=torch.bfloat16, device=dev)
    o, S = ops.attn_scan(qkv[:, :H * 64], qkv[:, H * 64:2 * H * 64], qkv[:, 2 * H * 64:], torch.full((H,), 0.9, device=dev),
                         cos, sin, 0, 4, H)
    assert o.shape[0] == 0
    h, last = ops.lsf_scan(torch.empty(0, 4, C, dtype=torch.bfloat16, device=dev), alpha_scalar=torch.full((1,), 0.5, device=dev))
    assert h.shape[0] == 0
    tok = ops.sample(torch.empty(0, 50, device=dev), torch.empty(0, device=dev), temperature=1.0, top_k=5, top_p=0.9)
    assert tuple(tok.shape) == (0, 1)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
