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


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_one_thread_drives_two_devices():
    """Function attributes (the raised dynamic shared-memory limit) are per device: the same host thread runs the
    decode linear, a grouped launch and a 14336-point Hadamard first on device 0, then on device 1."""
    import numpy as np

    from helpers import linear_tolerance_check, make_acts, quantized_layer
    from oracle import uniql_oracle as orc
    from uniql_b200 import ops
    layer = quantized_layer(7, 4096, 14336)
    x = make_acts(3, 2, 14336)
    want = orc.linear_ref(orc.hadamard_transform(x.double().numpy()).astype(np.float16), None, None, None, 4096,
                          w_deq=layer["w_deq"])
    xr = make_acts(4, 300, 14336)
    want_rows = orc.hadamard_transform(xr[:4].double().numpy())
    for dev in (0, 1):
        d = torch.device("cuda", dev)
        p, s = torch.from_numpy(layer["packed"]).to(d), torch.from_numpy(layer["scales"]).to(d)
        y = ops.w4a16_linear(x.to(d), p, s, None, 4096, hadamard_dim=14336)
        linear_tolerance_check(y.cpu().numpy(), want)
        (y2,) = ops.w4a16_linear_group(x.to(d), [(p, s, None, 4096)], hadamard_dim=14336)
        assert torch.equal(y, y2)
        h = ops.hadamard(xr.to(d), 14336 ** -0.5)                     # many rows: tensor-core kernel, > 48 KB shared memory
        assert np.abs(h[:4].double().cpu().numpy() - want_rows).max() <= 2e-3 * np.abs(want_rows).max()
        hf = ops.hadamard(xr.float().to(d), 14336 ** -0.5)            # fp32 rows: the 32-element kernel
        assert np.abs(hf[:4].double().cpu().numpy() - want_rows).max() <= 2e-5 * np.abs(want_rows).max()
        assert ops.read_and_clear_status(d) == 0
