"""Stand-alone peer-memory collectives, pipeline channels and a two-stage pipeline step on 2+ GPUs."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_peer_collectives_and_pipeline():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29623", os.path.join(HERE, "coll_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    lines = [l for l in p.stdout.splitlines() if l.startswith("COLL_RESULT ")]
    assert lines, p.stdout[-3000:] + p.stderr[-3000:]
    per_rank = json.loads(lines[0].split(" ", 1)[1])
    assert len(per_rank) == 2
    for res in per_rank:
        bad = [k for k, v in res.items() if v is False]
        assert not bad, (bad, res)
    assert per_rank[0]["timeout_reported"] and per_rank[0]["context_alive"]
