"""CPU tests of the decode driver's host logic: the oracle's sampling filter against the distribution the
reference's sample_next_token builds (golden fixture), and the slot policy against the trace of the
reference's ContinuousBatchingScheduler."""
import pytest
import torch

import jarvis_b200  # noqa: F401  (alias of the package directory)
from jarvis_b200 import serving
from oracle import jarvis_oracle as orc
from tests.golden.loader import load


def test_oracle_sampling_filter_matches_reference_distribution():
    g = load("sampling")
    logits = g["logits"]
    for i, (t, k, p) in enumerate(g["settings"].tolist()):
        want = g[f"probs_{i}"]
        got = orc.sample_filtered_probs(logits, t, int(k), p)
        # the same probabilities, as a multiset: which of several EQUAL logits survive the nucleus cut depends
        # on the tie order of the reference's unstable sort (the oracle orders ties by token id)
        assert torch.allclose(got.sort(dim=-1).values, want.sort(dim=-1).values, rtol=1e-6, atol=1e-9), i
        for b in range(logits.shape[0]):
            kept, dropped = logits[b][want[b] > 0], logits[b][want[b] == 0]
            if kept.min() > dropped.max():                # no tie across the cut: the kept set itself is pinned
                assert torch.equal(got[b] > 0, want[b] > 0), (i, b)
                assert torch.allclose(got[b], want[b], rtol=1e-6, atol=1e-9), (i, b)
    tok, _ = orc.sample_inverse_cdf(logits, torch.zeros(logits.shape[0]), temperature=0.0)
    assert torch.equal(tok, g["greedy"])


def test_oracle_inverse_cdf_draw():
    g = load("sampling")
    logits = g["logits"]
    p = orc.sample_filtered_probs(logits, 0.7, 50, 0.9)
    # u = 0 takes the most probable token; u just below 1 takes the least probable kept token
    tok0, pr0 = orc.sample_inverse_cdf(logits, torch.zeros(6), 0.7, 50, 0.9)
    assert torch.equal(tok0.view(-1), p.argmax(dim=-1))
    assert torch.allclose(pr0, p.max(dim=-1).values)
    tok1, pr1 = orc.sample_inverse_cdf(logits, torch.full((6,), 0.9999999), 0.7, 50, 0.9)
    for b in range(6):
        kept = p[b][p[b] > 0]
        assert float(pr1[b]) == float(kept.min())
    # empirical frequencies follow the filtered distribution
    gen = torch.Generator().manual_seed(0)
    u = torch.rand(4000, generator=gen)
    row = logits[:1].expand(4000, -1)
    toks, _ = orc.sample_inverse_cdf(row, u, 1.0, 5, 1.0)
    freq = torch.bincount(toks.view(-1), minlength=logits.shape[1]).float() / 4000
    want = orc.sample_filtered_probs(logits[:1], 1.0, 5, 1.0)[0]
    assert (freq - want).abs().max() < 0.03


class _FakeEngine:
    """Stands in for the CUDA engine: every active slot gets token 42, like the reference's simulation."""

    def __init__(self, limit=None):
        self.admitted, self.released = [], []
        self.limit = limit

    def admit(self, slot, prompt_tokens, max_new_tokens=0):
        if self.limit is not None and len(prompt_tokens) + max_new_tokens > self.limit:
            raise ValueError("too long")
        self.admitted.append((slot, tuple(prompt_tokens)))

    def release(self, slot):
        self.released.append(slot)

    def step(self, active_slots):
        return {s: 42 for s in active_slots}


def test_slot_policy_matches_reference_scheduler_trace():
    g = load("scheduler")
    eng = _FakeEngine()
    sched = serving.ContinuousBatchingScheduler(eng, max_batch_size=4)
    reqs = [serving.Request(req_id=i, prompt_tokens=[10, 20, 30], max_new_tokens=(i % 4 + 2)) for i in range(10)]
    for r in reqs:
        sched.add_request(r)
    trace, finish_iter, it = [], [-1] * 10, 0
    while sched.active_slots or sched.waiting_queue:
        stepped = sched.step()
        it += 1
        slots = [sched.active_slots[s].req_id if s in sched.active_slots else -1 for s in range(4)]
        for r in reqs:
            if r.is_finished and finish_iter[r.req_id] < 0:
                finish_iter[r.req_id] = it
        trace.append([stepped, len(sched.waiting_queue)] + slots)
    assert torch.equal(torch.tensor(trace), g["trace"])
    assert torch.equal(torch.tensor(finish_iter), g["finish_iter"])
    assert [len(r.generated_tokens) for r in reqs] == g["n_generated"].tolist()
    assert all(r.generated_tokens == [42] * len(r.generated_tokens) for r in reqs)
    assert len(eng.admitted) == 10 and sorted(eng.released) == sorted(s for s, _ in eng.admitted)
    assert sched.step() == 0      # idle


def test_requests_that_would_outrun_the_position_table_are_refused():
    """prompt + max_new_tokens beyond the engine's limit: retired unfinished with an error, the slot is reused."""
    eng = _FakeEngine(limit=8)
    sched = serving.ContinuousBatchingScheduler(eng, max_batch_size=1)
    sched.add_request(serving.Request(0, [1, 2, 3], max_new_tokens=6))      # 9 > 8: refused
    sched.add_request(serving.Request(1, [1, 2, 3], max_new_tokens=5))      # 8: fits
    sched.run()
    by_id = {r.req_id: r for r in sched.completed}
    assert by_id[0].error is not None and not by_id[0].is_finished and by_id[0].generated_tokens == []
    assert by_id[1].error is None and by_id[1].is_finished and len(by_id[1].generated_tokens) == 5
    assert eng.admitted == [(0, (1, 2, 3))]


def test_cuda_engine_admit_checks_prompt_plus_new_tokens():
    """CudaDecodeEngine.admit refuses before touching the device (no GPU needed to check the rule)."""
    eng = serving.CudaDecodeEngine.__new__(serving.CudaDecodeEngine)
    eng.max_position = 16
    with pytest.raises(ValueError, match="exceeds max_position"):
        eng.admit(0, list(range(10)), max_new_tokens=7)
    with pytest.raises(ValueError, match="exceeds max_position"):
        eng.admit(0, list(range(17)))


def test_eos_token_retires_early():
    eng = _FakeEngine()
    sched = serving.ContinuousBatchingScheduler(eng, max_batch_size=2, eos_token=42)
    sched.add_request(serving.Request(0, [1], max_new_tokens=10))
    assert sched.run() == 1
    assert sched.completed[0].generated_tokens == [42] and sched.completed[0].is_finished


def test_evaluate_window_selection_follows_the_reference_rule():
    from jarvis_b200 import evaluate
    # long corpus: back-to-back windows
    assert evaluate.window_starts(10 * 9, num_windows=10, seq_len=8, seed=1) == [i * 8 for i in range(10)]
    # short corpus: seeded random starts, the same numbers torch draws for the reference (evaluate_jarvis.py:343-345)
    g = torch.Generator(device="cpu").manual_seed(42)
    want = torch.randint(0, 50 - 8 - 1, (10,), generator=g).tolist()
    assert evaluate.window_starts(50, num_windows=10, seq_len=8, seed=42) == want
    import pytest
    with pytest.raises(ValueError):
        evaluate.window_starts(8, 1, 8, 0)


def test_evaluate_corpus_statistics_with_a_stub_model():
    from jarvis_b200 import evaluate

    class Stub(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.tok_emb = torch.nn.Embedding(16, 4)

        def forward(self, x, targets=None, persist_state=False):
            assert not persist_state and x.shape == targets.shape
            assert torch.equal(x[0, 1:], targets[0, :-1])          # y is x shifted by one token
            return None, x.float().mean() / 10.0

    toks = torch.arange(0, 200) % 16
    r = evaluate.evaluate_corpus(Stub(), toks, num_windows=5, seq_len=8, seed=3)
    want = [float((toks[i * 8:i * 8 + 8].float().mean()) / 10.0) for i in range(5)]
    assert abs(r["mean_loss"] - sum(want) / 5) < 1e-6
    import math
    import statistics
    assert abs(r["std_loss"] - statistics.stdev(want)) < 1e-6
    assert abs(r["perplexity"] - math.exp(r["mean_loss"])) < 1e-9
    assert r["windows_evaluated"] == 5 and r["tokens_evaluated"] == 40 and not r["has_nan_inf"]


def test_evaluate_token_files(tmp_path):
    from jarvis_b200 import evaluate
    import numpy as np
    np.save(tmp_path / "c.npy", np.arange(7))
    (tmp_path / "c.ids").write_text("3 1 4 1 5")
    enc = evaluate.IdTokenizer()
    assert evaluate.load_token_file(str(tmp_path / "c.npy"), enc).tolist() == list(range(7))
    assert evaluate.load_token_file(str(tmp_path / "c.ids"), enc).tolist() == [3, 1, 4, 1, 5]
    import pytest
    with pytest.raises(FileNotFoundError):
        evaluate.load_token_file(str(tmp_path / "missing.txt"), enc)
    a = evaluate.parse_args(["--prompt", "1 2 3", "--temperature", "0", "--stateful"])
    assert a.prompt == "1 2 3" and a.temperature == 0 and a.stateful and a.top_k == 50 and a.num_windows == 200
