"""Real multi-GPU tests (2 GPUs by default): child processes under torch.distributed.run, NVLS
off, plain peer loads / stores.  See tests/mp_worker.py for what is checked."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(n, what, port, nvls="0"):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MOONEP_B200_NVLS=nvls)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(ROOT, "tests", "mp_worker.py"), what]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert res.returncode == 0 and f"MULTIGPU_OK R={n}" in res.stdout, \
        f"worker failed:\n{res.stdout[-3000:]}\n{res.stderr[-3000:]}"


@pytest.mark.parametrize("what,port", [("comm", 29611), ("symm", 29619), ("layer", 29612), ("fused", 29617), ("decoder", 29615), ("leave", 29616)])
def test_two_gpus(what, port):
    _run(2, what, port)


def test_two_gpus_nvls_overlay():
    """The NVSwitch multicast overlay: create, add, bind, map, a multimem.st broadcast that every
    rank reads back from its own copy, orderly teardown.  The only test that binds memory to a
    multicast object; no rank leaves while it is bound."""
    _run(2, "nvls", 29618, nvls="1")


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_four_gpus():
    _run(4, "all", 29613)


@pytest.mark.skipif(torch.cuda.device_count() < 8, reason="needs 8 GPUs")
def test_eight_gpus():
    _run(8, "all", 29614)
