"""GPU, needs at least two devices (skipped otherwise): the push all-reduce across real ranks."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_push_allreduce_two_ranks():
    """The push all-reduce and the exchanges inside the decode kernel (sum of a row-parallel shard, feature gather of a
    column shard, Hadamard of the gathered row), checked by the worker against NCCL and the unsharded layers."""
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29533", os.path.join(here, "tp_push_worker.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    env.pop("UNIQL_B200_DECODE_ENGINE", None)
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert "PUSH_ALLREDUCE_OK" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]
