"""Replicated-token expert parallelism (decode) on real GPUs: every rank returns the bytes of the
single-GPU result, for one layer and for a CUDA-graph-replayed stack (needs >= 2 GPUs)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("name,tokens,port", [("mixtral_int8", 8, 29641), ("mixtral", 64, 29648),
                                               ("deepseek_v2_lite", 33, 29655)])
def test_replicated_tokens_equal_single_gpu(name, tokens, port):
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    world = min(n, int(os.environ.get("ATENIA_EP_TEST_WORLD", "2")))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(ROOT, "tests", "ep_replicated_worker.py"), name, str(tokens)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "equal=True" in r.stdout
