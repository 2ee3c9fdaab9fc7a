"""Multi-GPU checks (skipped on a single-GPU box): expert-parallel MoE against the single-GPU layer
and the data-parallel prefill bench line, each as torchrun child processes on 2 GPUs with NVLS off."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torchrun(n, script_args, timeout=600):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", "29517", *script_args]
    return subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_moe_two_gpus():
    res = _torchrun(2, ["jarvis-q1.58-500m_b200/kernel_bench.py", "moe", "--N", "8192", "--iters", "2"])
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["n_gpus"] == 2 and line["rel_l2_vs_single_gpu"] < 1e-6
    assert sum(line["rows_received_per_rank"]) == 2 * 8192


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_over_peer_memory_two_gpus():
    """Same layer with the exchanges done by kernels reading the other GPU's memory (plain loads, no multimem)."""
    res = _torchrun(2, ["jarvis-q1.58-500m_b200/kernel_bench.py", "moe", "--N", "8192", "--iters", "2", "--peer"])
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads([ln for ln in res.stdout.strip().splitlines() if ln.startswith("{")][-1])
    assert line["n_gpus"] == 2 and line["rel_l2_vs_single_gpu"] < 1e-6
    assert sum(line["rows_received_per_rank"]) == 2 * 8192


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_data_parallel_bench_two_gpus():
    res = _torchrun(2, ["bench.py", "--gpus", "2", "--steps", "2", "--warmup", "3"], timeout=900)
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["n_gpus"] == 2 and line["scaling"] == "weak" and line["value"] > 0


_SPLIT_SCRIPT = """
import os, sys, json, torch, torch.distributed as dist
sys.path.insert(0, os.getcwd())
import jarvis_b200
from jarvis_b200 import modules as jm
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
torch.manual_seed(0)
model = jm.ternary_init_(jm.Jarvis(vocab_size=512, d_model=256, n_layers=3, n_heads=4, max_seq_len=256)).cuda().eval()
idx = torch.randint(0, 512, (4, 192), generator=torch.Generator().manual_seed(1)).cuda()
full, _ = model(idx)                                   # the whole batch on every rank: the reference result
model.set_batch_split(dist.group.WORLD, global_tokens=idx.numel())
per = idx.shape[0] // world
part, _ = model(idx[rank * per:(rank + 1) * per])      # this rank's slice, statistics all-reduced per layer
err = float((part.float() - full[rank * per:(rank + 1) * per].float()).norm() / full.float().norm())
model.set_batch_split(None)
alone, _ = model(idx[rank * per:(rank + 1) * per])     # independent call: a different decay, a different result
diff = float((alone.float() - full[rank * per:(rank + 1) * per].float()).norm() / full.float().norm())
t = torch.tensor([err, diff], device="cuda"); dist.all_reduce(t, op=dist.ReduceOp.MAX)
if rank == 0: print(json.dumps({"err": float(t[0]), "independent_diff": float(t[1])}))
dist.destroy_process_group()
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_batch_split_over_two_gpus_reproduces_the_unsplit_batch(tmp_path):
    script = tmp_path / "split.py"
    script.write_text(_SPLIT_SCRIPT)
    res = _torchrun(2, [str(script)])
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["err"] < 2e-3            # same kernels; only the summation order of the statistics differs
    assert line["independent_diff"] > line["err"]


_CONTEXT_SCRIPT = """
import os, sys, json, torch, torch.distributed as dist
sys.path.insert(0, os.getcwd())
import jarvis_b200
from jarvis_b200 import modules as jm
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
torch.manual_seed(0)
model = jm.ternary_init_(jm.Jarvis(vocab_size=512, d_model=256, n_layers=3, n_heads=4, max_seq_len=1024)).cuda().eval()
idx = torch.randint(0, 512, (2, 640), generator=torch.Generator().manual_seed(2)).cuda()
full, _ = model(idx)                                        # whole sequences on every rank: the reference result
model.reset_state()
model.carry_attention_state = True
full_a, _ = model(idx[:, :384], persist_state=True)         # two persisted calls on one GPU
full_b, _ = model(idx[:, 384:], persist_state=True)
h_ref = [h.clone() for h in model._h_states]; s_ref = [s.clone() for s in model._attn_states]
model.reset_state(); model.carry_attention_state = False
model.set_context_parallel(dist.group.WORLD)
tl = idx.shape[1] // world
part, _ = model(idx[:, rank * tl:(rank + 1) * tl])          # this rank's slice of every sequence
want = full[:, rank * tl:(rank + 1) * tl]
err = float((part.float() - want.float()).norm() / want.float().norm())
# persisted calls: states after call a (whole-sequence end states on every rank) feed call b
model.reset_state(); model.carry_attention_state = True
ta, tb = 384 // world, 256 // world
pa, _ = model(idx[:, rank * ta:(rank + 1) * ta], persist_state=True)
pb, _ = model(idx[:, 384 + rank * tb:384 + (rank + 1) * tb], persist_state=True)
wa, wb = full_a[:, rank * ta:(rank + 1) * ta], full_b[:, rank * tb:(rank + 1) * tb]
err_a = float((pa.float() - wa.float()).norm() / wa.float().norm())
err_b = float((pb.float() - wb.float()).norm() / wb.float().norm())
err_h = max(float((a - b).norm() / b.norm()) for a, b in zip(model._h_states, h_ref))
err_s = max(float((a - b).norm() / b.norm()) for a, b in zip(model._attn_states, s_ref))
pos = model._token_pos
t = torch.tensor([err, err_a, err_b, err_h, err_s], device="cuda"); dist.all_reduce(t, op=dist.ReduceOp.MAX)
if rank == 0: print(json.dumps({"err": float(t[0]), "err_a": float(t[1]), "err_b": float(t[2]), "err_h": float(t[3]),
                                "err_s": float(t[4]), "token_pos": pos}))
dist.destroy_process_group()
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_context_parallel_over_two_gpus_reproduces_the_whole_sequence(tmp_path):
    script = tmp_path / "context.py"
    script.write_text(_CONTEXT_SCRIPT)
    res = _torchrun(2, [str(script)])
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    # same kernels on the same tokens; the carried states cross ranks in f32 and the MoE statistics are summed
    # in another order
    assert line["err"] < 5e-3 and line["err_a"] < 5e-3 and line["err_b"] < 5e-3
    assert line["err_h"] < 5e-3 and line["err_s"] < 5e-3
    assert line["token_pos"] == 640


_EP_MODEL_SCRIPT = """
import os, sys, json, torch, torch.distributed as dist
sys.path.insert(0, os.getcwd())
import jarvis_b200
from jarvis_b200 import modules as jm
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
torch.manual_seed(0)
model = jm.ternary_init_(jm.Jarvis(vocab_size=512, d_model=256, n_layers=3, n_heads=4, max_seq_len=256)).cuda().eval()
idx = torch.randint(0, 512, (4, 192), generator=torch.Generator().manual_seed(1)).cuda()
full, _ = model(idx)                                   # the whole batch with local experts: the reference result
per = idx.shape[0] // world
model.set_expert_parallel(dist.group.WORLD, max_tokens=per * idx.shape[1], global_tokens=idx.numel())
part, _ = model(idx[rank * per:(rank + 1) * per])      # this rank's sequences, experts spread over the ranks
err = float((part.float() - full[rank * per:(rank + 1) * per].float()).norm() / full.float().norm())
again, _ = model(idx[rank * per:(rank + 1) * per])     # the exchange buffers are reused call after call
same = bool(torch.equal(part, again))
model.set_expert_parallel(None)
local, _ = model(idx)
back = bool(torch.equal(local, full))
t = torch.tensor([err, 0.0 if same else 1.0, 0.0 if back else 1.0], device="cuda"); dist.all_reduce(t, op=dist.ReduceOp.MAX)
if rank == 0: print(json.dumps({"err": float(t[0]), "repeatable": float(t[1]) == 0.0, "restored": float(t[2]) == 0.0}))
dist.destroy_process_group()
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_model_with_experts_spread_over_two_gpus(tmp_path):
    """Jarvis.set_expert_parallel: every MoE layer's experts on different GPUs, rows exchanged by peer-memory
    loads, statistics all-reduced; logits equal those of the whole batch on one GPU up to the summation order of
    the statistics (as with set_batch_split)."""
    script = tmp_path / "ep_model.py"
    script.write_text(_EP_MODEL_SCRIPT)
    res = _torchrun(2, [str(script)])
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["err"] < 5e-3 and line["repeatable"] and line["restored"]
