"""execute_real_moe_layer in sub-batches with the copies overlapped: pinned sub-batch sizes
(ATENIA_MOE_EXEC_CHUNK) and the default schedule of large batches (a short piece at each end)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("chunk,tokens", [(64, 64), (64, 65), (100, 1000), (256, 777), (4096, 300), (None, 2048),
                                          (None, 2777)])
def test_chunked_execute_matches_one_forward(chunk, tokens):
    env = dict(os.environ)
    env.pop("ATENIA_MOE_EXEC_CHUNK", None)
    if chunk is not None:
        env["ATENIA_MOE_EXEC_CHUNK"] = str(chunk)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "exec_chunk_worker.py"), str(tokens)],
                       capture_output=True, text=True, timeout=240, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "ok=True" in r.stdout
