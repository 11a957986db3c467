"""Fused tensor-parallel kernels and the tensor-parallel Llama on 2+ GPUs (skipped on a single-GPU box)."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_fused_tp_kernels_and_llama_tp_match_single_gpu():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29621", os.path.join(HERE, "tp_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    line = [l for l in p.stdout.splitlines() if l.startswith("TP_RESULT ")]
    assert line, p.stdout[-3000:] + p.stderr[-3000:]
    res = json.loads(line[0][len("TP_RESULT "):])
    assert res["ok"], res


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 4, reason="needs >= 4 GPUs")
def test_llama_on_a_2x2_mesh_with_a_shared_kv_head_matches_single_gpu():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr",
           "127.0.0.1", "--master-port", "29623", os.path.join(HERE, "tp_worker.py"), "mesh2d"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    line = [l for l in p.stdout.splitlines() if l.startswith("TP_RESULT ")]
    assert line, p.stdout[-3000:] + p.stderr[-3000:]
    res = json.loads(line[0][len("TP_RESULT "):])
    assert res["ok"], res
