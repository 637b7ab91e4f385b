"""GPU, needs at least two devices (skipped otherwise): the push all-reduce across real ranks."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("engine", ["tiled", "slot"])
def test_push_allreduce_two_ranks(engine):
    """Both decode kernels carry the tensor-parallel exchanges; the worker checks them against NCCL and against the
    unsharded layers."""
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29533", os.path.join(here, "tp_push_worker.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    if engine == "slot":
        env["UNIQL_B200_DECODE_ENGINE"] = "slot"
    else:
        env.pop("UNIQL_B200_DECODE_ENGINE", None)
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert "PUSH_ALLREDUCE_OK" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]
