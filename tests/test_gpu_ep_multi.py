"""Expert parallelism across real GPUs (needs >= 2 devices; skipped otherwise)."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("balanced,hot", [(False, 0), (True, 0), (True, 4)])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_matches_single_gpu(world, balanced, hot):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(ROOT, "tests", "ep_multi_worker.py")]
    env = dict(os.environ, QS3_TEST_BALANCED="1" if balanced else "0", QS3_TEST_HOT=str(hot))
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "EP_MULTI_OK" in r.stdout
    print(r.stdout[-300:])
