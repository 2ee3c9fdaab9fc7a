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
def test_data_parallel_bench_two_gpus():
    res = _torchrun(2, ["bench.py", "--gpus", "2", "--steps", "2", "--warmup", "3"], timeout=900)
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["n_gpus"] == 2 and line["scaling"] == "weak" and line["value"] > 0
