"""Expert-parallel and column-parallel paths on real GPUs over NCCL, as child processes (one per GPU).  Skipped on a
single-GPU box; the host-side logic is covered on CPU by test_sharding_cpu.py."""
import json
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _torchrun(nproc, args):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port())] + args
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    return [json.loads(line) for line in r.stdout.splitlines() if line.startswith("{")]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_expert_parallel_matches_single_gpu():
    lines = _torchrun(2, ["-m", "quactlize_b200.bench_ep", "--tokens", "300", "--experts", "8", "--hidden", "512", "--ffn", "768",
                          "--steps", "2", "--warmup", "1", "--check"])
    assert any(l.get("ok") is True for l in lines)
    assert any("TFLOPs_aggregate" in l for l in lines)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_bench_column_parallel_two_gpus():
    lines = _torchrun(2, ["bench.py", "--gpus", "2", "--steps", "3", "--warmup", "3", "--no-cpu"])
    line = lines[-1]
    assert line["n_gpus"] == 2 and line["scaling"] == "weak" and line["value"] > 0 and line["gpu_launches"] > 0
