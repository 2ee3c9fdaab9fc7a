"""GPU tests of the decode driver: the sampling kernel against the oracle's restatement of the reference's
filter, and continuous batching on real slots (reference slot policy; logits of every step against the
CPU oracle stepped with the same inputs)."""
import pytest
import torch

import jarvis_b200  # noqa: F401
from jarvis_b200 import _lib, modules as jm, ops, serving
from oracle import jarvis_oracle as orc
from tests.golden.loader import load

pytestmark = pytest.mark.gpu


def rel_l2(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


@pytest.mark.parametrize("setting", [(0.7, 50, 0.9), (1.0, 5, 0.5), (1.3, 200, 0.95), (0.7, 50, 1.0), (0.25, 1024, 0.3)])
def test_sampling_kernel_matches_oracle(setting):
    t, k, p = setting
    g = load("sampling")
    logits = g["logits"]
    gen = torch.Generator().manual_seed(int(k))
    for trial in range(8):
        u = torch.rand(logits.shape[0], generator=gen)
        if trial == 0:
            u.zero_()
        want_tok, want_prob = orc.sample_inverse_cdf(logits, u, t, k, p)
        tok, prob = ops.sample(logits.cuda(), u.cuda(), temperature=t, top_k=k, top_p=p, want_prob=True)
        assert torch.equal(tok.cpu(), want_tok), trial
        assert torch.allclose(prob.cpu(), want_prob, rtol=1e-4, atol=1e-7)


def test_sampling_kernel_greedy_strided_bf16_rows():
    gen = torch.Generator().manual_seed(9)
    V, ld = 50257, 50304
    buf = torch.randn(3, ld, generator=gen).bfloat16().cuda()
    rows = buf[:, :V]
    assert rows.stride(0) == ld
    tok = ops.sample(rows, None, temperature=0.0)
    want, _ = orc.sample_inverse_cdf(rows.float().cpu(), torch.zeros(3), temperature=0.0)
    assert torch.equal(tok.cpu(), want)
    # sampled path on the full vocabulary: the draw must be one of the oracle's kept tokens with its probability
    u = torch.rand(3, generator=gen)
    tok, prob = ops.sample(rows, u.cuda(), temperature=0.8, top_k=40, top_p=0.95, want_prob=True)
    want_tok, want_prob = orc.sample_inverse_cdf(rows.float().cpu(), u, 0.8, 40, 0.95)
    assert torch.equal(tok.cpu(), want_tok)
    assert torch.allclose(prob.cpu(), want_prob, rtol=1e-4)
    assert _lib.device_status() == 0


def test_sampling_kernel_frequencies_follow_the_filtered_distribution():
    g = load("sampling")
    row = g["logits"][:1]
    n = 8192
    gen = torch.Generator().manual_seed(1)
    u = torch.rand(n, generator=gen).cuda()
    tok = ops.sample(row.expand(n, -1).contiguous().cuda(), u, temperature=1.0, top_k=8, top_p=0.9)
    freq = torch.bincount(tok.view(-1).cpu(), minlength=row.shape[1]).float() / n
    want = orc.sample_filtered_probs(row, 1.0, 8, 0.9)[0]
    assert torch.equal(freq > 0, want > 0)
    assert (freq - want).abs().max() < 0.02


def test_sampling_long_runs_of_equal_logits_keep_the_largest_and_stay_deterministic():
    """More equal values at the k-th rank than the kernel's candidate buffer holds (a constant row with one
    larger entry): the larger entry must survive, the equal ones are taken in ascending token id, and the same
    (logits, u) always gives the same token."""
    V = 6000
    row = torch.zeros(4, V)
    row[0, 4321] = 5.0          # argmax hidden behind thousands of ties
    row[1, 17] = 1.0
    row[2, V - 1] = 2.0
    # row 3: all equal
    u = torch.tensor([0.0, 0.999, 0.5, 0.25])
    dev = row.cuda()
    first = ops.sample(dev, u.cuda(), temperature=1.0, top_k=50, top_p=1.0)
    for _ in range(5):
        assert torch.equal(ops.sample(dev, u.cuda(), temperature=1.0, top_k=50, top_p=1.0), first)
    assert int(first[0]) == 4321                                   # u = 0 picks the most probable token
    tok, prob = ops.sample(dev, torch.zeros(4).cuda(), temperature=1.0, top_k=50, top_p=1.0, want_prob=True)
    assert tok.view(-1).tolist()[:3] == [4321, 17, V - 1] and int(tok[3]) == 0
    # kept set = the larger value + the first 2047 equal tokens by id: u close to 1 lands on the last kept id
    last = ops.sample(dev, torch.full((4,), 0.999999).cuda(), temperature=1.0, top_k=50, top_p=1.0).view(-1).tolist()
    assert last[3] == 2047 and last[1] in (2046, 2047) and last[0] == 2046
    # greedy path for comparison
    assert ops.sample(dev, None, temperature=0.0).view(-1).tolist() == [4321, 17, V - 1, 0]
    assert _lib.device_status() == 0


def test_sampling_argument_errors():
    x = torch.zeros(2, 100, device="cuda")
    with pytest.raises(RuntimeError, match="top_k"):
        ops.sample(x, torch.zeros(2, device="cuda"), temperature=1.0, top_k=0, top_p=0.9)
    with pytest.raises(RuntimeError, match="uniform"):
        ops.sample(x, None, temperature=1.0, top_k=5, top_p=0.9)


def _tiny_model():
    g = load("model")
    sd = {k[3:]: v for k, v in g.items() if k.startswith("sd_")}
    model = jm.Jarvis(vocab_size=256, d_model=128, n_layers=2, n_heads=2, max_seq_len=256).eval()
    model.load_state_dict(sd)
    return model.cuda(), sd


@pytest.mark.parametrize("use_graph", [False, True])
def test_continuous_batching_on_real_slots(use_graph):
    """Ten requests through four slots: the slot trace is the reference scheduler's, and every iteration's
    logits equal the CPU oracle stepped with the same tokens, positions and carried states (idle slots
    included, since the LSF decay is a function of the whole batch)."""
    model, sd = _tiny_model()
    g = load("scheduler")
    eng = serving.CudaDecodeEngine(model, max_batch_size=4, max_position=512, temperature=0.0, pad_token=0,
                                   use_cuda_graph=use_graph, record=True)
    sched = serving.ContinuousBatchingScheduler(eng, max_batch_size=4)
    gen = torch.Generator().manual_seed(4)
    reqs = [serving.Request(i, torch.randint(1, 256, (int(torch.randint(1, 40, (1,), generator=gen)),),
                                             generator=gen).tolist(), max_new_tokens=(i % 4 + 2)) for i in range(10)]
    for r in reqs:
        sched.add_request(r)
    trace = []
    while sched.active_slots or sched.waiting_queue:
        stepped = sched.step()
        trace.append([stepped, len(sched.waiting_queue)] +
                     [sched.active_slots[s].req_id if s in sched.active_slots else -1 for s in range(4)])
    assert torch.equal(torch.tensor(trace), g["trace"])
    assert [len(r.generated_tokens) for r in reqs] == g["n_generated"].tolist()
    assert _lib.device_status() == 0
    # replay every recorded iteration in the oracle
    for it, rec in enumerate(eng.record):
        ref, _, _ = orc.model_step(rec["idx"].cpu(), sd, 2, 2, [t.cpu() for t in rec["h"]], [t.cpu() for t in rec["S"]],
                                   rec["positions"].cpu())
        assert rel_l2(rec["logits"], ref[:, 0, :]) <= 2e-2, it
    # the state a freshly admitted slot starts from is the prefill of its prompt minus the last token
    first = eng.record[0]
    for slot in range(4):
        prompt = reqs[slot].prompt_tokens
        assert int(first["idx"][slot, 0]) == prompt[-1]
        assert int(first["positions"][slot]) == len(prompt) - 1
        if len(prompt) > 1:
            _, h_ref, S_ref = orc.model_step(torch.tensor([prompt[:-1]]), sd, 2, 2)
            for layer in range(2):
                assert rel_l2(first["S"][layer][slot], S_ref[layer][0]) <= 1e-2
                assert rel_l2(first["h"][layer][slot], h_ref[layer][0]) <= 2e-2
    # greedy tokens: each generated token is the argmax of its recorded logits row
    for rec in eng.record:
        assert torch.equal(rec["tokens"].view(-1).cpu(), rec["logits"].argmax(dim=-1).cpu())


def test_sampled_generation_is_reproducible_by_seed():
    model, _ = _tiny_model()
    outs = []
    for _ in range(2):
        sched = serving.build_scheduler(model, max_batch_size=2, max_position=128, temperature=0.9, top_k=20, top_p=0.9,
                                        seed=123, use_cuda_graph=False)
        for i in range(3):
            sched.add_request(serving.Request(i, [5, 6, 7 + i], max_new_tokens=6))
        sched.run()
        outs.append([r.generated_tokens for r in sorted(sched.completed, key=lambda r: r.req_id)])
    assert outs[0] == outs[1]
    assert all(len(t) == 6 for t in outs[0])


def test_evaluate_cli_pieces_on_a_tiny_model(tmp_path):
    """Corpus loss through evaluate_corpus equals calling the model window by window, and sits on the oracle's
    cross-entropy; greedy generation by re-running the window equals stateful decode for a prompt that fits
    one window... up to the LSF decay, which is per call: so only the first generated token is compared."""
    from jarvis_b200 import checkpoint, evaluate
    model, sd = _tiny_model()
    path = tmp_path / "tiny.pt"
    torch.save({"model_state_dict": {"_orig_mod." + k: v for k, v in sd.items()}, "step": 7}, path)
    loaded, step = evaluate.load_model(str(path), vocab=256, d_model=128, n_layers=2, n_heads=2)
    assert step == 7
    gen = torch.Generator().manual_seed(8)
    toks = torch.randint(0, 256, (400,), generator=gen)
    rep = evaluate.evaluate_corpus(loaded, toks, num_windows=4, seq_len=64, seed=1)
    starts = evaluate.window_starts(400, 4, 64, 1)
    losses, ce_ref = [], []
    for s in starts:
        x, y = toks[s:s + 64][None].cuda(), toks[s + 1:s + 65][None].cuda()
        losses.append(float(model(x, targets=y)[1]))
        ref_logits, _ = orc.model_forward(x.cpu(), sd, 2, 2)
        ce_ref.append(float(torch.nn.functional.cross_entropy(ref_logits.view(-1, 256), y.cpu().view(-1))))
    assert abs(rep["mean_loss"] - sum(losses) / 4) < 1e-5
    assert abs(rep["mean_loss"] - sum(ce_ref) / 4) < 0.05 * abs(sum(ce_ref) / 4) + 0.05   # loss = CE + small aux terms
    # packed container round trip through the loader
    tb = tmp_path / "tiny.jarvis-tbin"
    checkpoint.write_tbin(sd, str(tb))
    from_tbin, _ = evaluate.load_model(str(tb), vocab=256, d_model=128, n_layers=2, n_heads=2)
    x = toks[:48][None].cuda()
    assert rel_l2(from_tbin(x)[0].float(), model(x)[0].float()) < 2e-2
    # generation
    prompt = toks[:20].tolist()
    a = evaluate.generate(model, prompt, max_new_tokens=5, temperature=0.0)
    b = evaluate.generate(model, prompt, max_new_tokens=5, temperature=0.0, stateful=True)
    assert len(a) == 5 and len(b) == 5 and a[0] == b[0]
    first = int(model(torch.tensor([prompt]).cuda())[0][0, -1].float().argmax())
    assert a[0] == first
    c = evaluate.generate(model, prompt, max_new_tokens=5, temperature=0.8, top_k=10, top_p=0.9, seed=5)
    d = evaluate.generate(model, prompt, max_new_tokens=5, temperature=0.8, top_k=10, top_p=0.9, seed=5)
    assert c == d
