"""Multi-GPU tests (peer-memory collectives, bounded waits, TP modes): one child process per GPU."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(which, n):
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29533", os.path.join(here, "multigpu_worker.py"), which]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + "\n" + r.stderr[-3000:]
    assert "multigpu worker ok" in r.stdout


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("which", ["collectives", "fused", "ring", "wait", "model", "nvls"])
def test_multi_gpu(which, world):
    """Every case at 2, 4 and 8 ranks (own-row epilogue with up to 7 peers, rank-rotated tile order,
    half-GPU co-residency of the fused kernels); a box with fewer GPUs skips the larger worlds."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    if which == "wait" and world > 2:
        pytest.skip("the bounded-wait probe involves no peer; covered at 2 ranks")
    if which == "nvls" and world not in (2, 8):
        pytest.skip("switch multicast is checked at 2 ranks and on the whole box")
    _run(which, world)
