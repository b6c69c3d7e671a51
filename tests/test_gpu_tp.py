"""Tensor-parallel decoder on 2 GPUs (skipped on a single-GPU box): token ids and
logits shards against the oracle, through the peer-memory exchange."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("mode", ["sum", "pull", "single_cta"])
def test_two_rank_decoder_matches_oracle(mode):
    """Two ranks on two GPUs against the oracle, with the exchange consumed by the multi-CTA
    packet sum + the next projection's fused add+norm (the default), inside the next
    projection's prologue (TLB_TP_PULL_MAX=4), and by the older single-CTA add+norm kernel
    (TLB_TP_SUM=0)."""
    extra = {"sum": {}, "pull": {"TLB_TP_PULL_MAX": "4"}, "single_cta": {"TLB_TP_SUM": "0"}}[mode]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", **extra)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29611", os.path.join(HERE, "tp_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert "TP_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
