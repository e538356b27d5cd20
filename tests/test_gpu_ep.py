"""Expert parallelism on real GPUs: an N-rank run equals the single-GPU run (needs >= 2 GPUs)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("name", ["mixtral", "deepseek_v2_lite"])
def test_expert_parallel_equals_single_gpu(name):
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    # two ranks by default; ATENIA_EP_TEST_WORLD=4 (or 8) widens the group on a box that has the GPUs
    world = min(n, int(os.environ.get("ATENIA_EP_TEST_WORLD", "2")))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", ATENIA_MOE_EP_TIMEOUT_S="30")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29611 + (0 if name == "mixtral" else 7)), os.path.join(ROOT, "tests", "ep_worker.py"),
           name, "301"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "equal=True" in r.stdout
