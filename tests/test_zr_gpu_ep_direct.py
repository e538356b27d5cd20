"""Direct (peer-store) expert-parallel exchange on real GPUs: an N-rank run equals the single-GPU run
(needs >= 2 GPUs with peer access)."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("flags", [0, 1])
@pytest.mark.parametrize("name,port", [("mixtral", 29671), ("deepseek_v2_lite", 29678)])
def test_direct_exchange_equals_single_gpu(name, port, flags):
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    world = min(n, int(os.environ.get("ATENIA_EP_TEST_WORLD", "2")))
    # flags = 1: counts and completion epochs through the peers' memory instead of three collectives
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", ATENIA_MOE_EP_FLAGS=str(flags))
    port += 3 * flags
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "ep_worker.py"),
           name, "301", "direct"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "equal=True" in r.stdout
