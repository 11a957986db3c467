"""Fused data-parallel reducer on 2+ GPUs (skipped on a single-GPU box)."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_fused_dp_matches_nccl_baseline():
    n = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29611", os.path.join(HERE, "dp_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    line = [l for l in p.stdout.splitlines() if l.startswith("DP_RESULT ")]
    assert p.returncode == 0 and line, p.stdout[-2000:] + p.stderr[-2000:]
    res = json.loads(line[0][len("DP_RESULT "):])
    assert res["ok"], res
    assert res["multimem"] is False


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
@pytest.mark.parametrize("buffers", ["shadow", "shadow,stage", "grad,shadow"])
def test_fused_dp_over_nvswitch_multicast_matches_nccl_baseline(buffers):
    """The same worker with NVLS left on.  ``shadow``: the parameter buffer is bound to a multicast object and the new
    weights leave through multimem.st; ``stage``: each gradient bucket is also copied into a multicast-bound buffer and
    reduced in the switch with multimem.ld_reduce; ``grad``: the gradient buffer itself is bound.  No rank leaves."""
    n = min(torch.cuda.device_count(), 4)
    env = {k: v for k, v in os.environ.items() if k != "NCCL_NVLS_ENABLE"}
    env["INCIN_TEST_EXPECT_MULTIMEM"] = "1"
    env["INCIN_MULTIMEM_BUFFERS"] = buffers
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29641", os.path.join(HERE, "dp_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    line = [l for l in p.stdout.splitlines() if l.startswith("DP_RESULT ")]
    assert p.returncode == 0 and line, p.stdout[-2000:] + p.stderr[-2000:]
    res = json.loads(line[0][len("DP_RESULT "):])
    assert res["ok"] and res["multimem"], res
