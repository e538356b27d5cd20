"""ATENIA_MOE_EXEC_CHUNK: execute_real_moe_layer in sub-batches with the copies overlapped."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Opt-in in the library and here until it has run on hardware: ATENIA_TEST_EXEC_CHUNK=1.
pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(os.environ.get("ATENIA_TEST_EXEC_CHUNK", "0") != "1",
                                 reason="opt-in path: set ATENIA_TEST_EXEC_CHUNK=1")]


@pytest.mark.parametrize("chunk,tokens", [(64, 64), (64, 65), (100, 1000), (256, 777), (4096, 300)])
def test_chunked_execute_matches_one_forward(chunk, tokens):
    env = dict(os.environ, ATENIA_MOE_EXEC_CHUNK=str(chunk))
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "exec_chunk_worker.py"), str(tokens)],
                       capture_output=True, text=True, timeout=240, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "ok=True" in r.stdout
