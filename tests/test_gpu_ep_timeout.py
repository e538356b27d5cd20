"""A peer that stays out of an expert-parallel step must not hang the others: the bounded host wait
(ATENIA_MOE_EP_TIMEOUT_S) ends with ATENIA_ERR_NCCL and the layer is left in a state that answers.
Needs 2 GPUs.  The failure is made on the host (a rank that does not call); NVLS is off."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("layout", ["sharded", "replicated", "flags"])
def test_missing_peer_ends_with_an_error_status(layout):
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", ATENIA_MOE_EP_TIMEOUT_S="4")
    if layout == "flags":
        env.update(ATENIA_MOE_EP_FLAGS="1", ATENIA_MOE_EP_FLAG_TIMEOUT_MS="1500")
    port = 29691 + {"sharded": 0, "replicated": 5, "flags": 9}[layout]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "ep_timeout_worker.py"), layout]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "ok=True" in r.stdout
