"""GPU: the tensor-parallel launches on a communicator of world size 1.

Every cross-GPU exchange of the decode path is a store of epoch-tagged words into the consumer's block followed by a
bounded wait on the consumer's side; with one rank the consumer's block is this GPU's own, so the same kernels, epoch
counters, parities, feature area and feature-area Hadamard kernel run here exactly as in a tensor-parallel layer, and the
results must equal the plain single-GPU launches.  (Two or more ranks are covered by tests/tp_push_worker.py and by the
tp_parity check of `bench.py --gpus N`.)"""
import numpy as np
import pytest
import torch

from helpers import linear_tolerance_check, make_acts, quantized_layer
from oracle import uniql_oracle as orc

pytestmark = pytest.mark.gpu


def _dev(layer):
    b = torch.from_numpy(layer["bias"]).cuda() if layer["bias"] is not None else None
    return torch.from_numpy(layer["packed"]).cuda(), torch.from_numpy(layer["scales"]).cuda(), b


@pytest.fixture(scope="module")
def comm():
    from uniql_b200 import tp
    c = tp.PushAllReduce.single_rank(max_elems=16 * 16384)
    yield c
    c.close()


def test_push_all_reduce_of_one_rank_is_a_copy(comm):
    for n in (8, 4096, 16 * 4096, 16 * 16384):
        t = torch.randn(n, device="cuda").half()
        want = t.clone()
        for _ in range(3):                                    # both parities, advancing epochs
            comm.all_reduce(t)
        torch.cuda.synchronize()
        assert torch.equal(t, want)


@pytest.mark.parametrize("m", [1, 3, 8, 16])
def test_row_parallel_linear_with_the_sum_in_its_epilogue(comm, m):
    """UNIQL_TP_REDUCE: shapes alternate on one communicator (every 64-column block keeps its own epoch); bias and
    residual are added after the sum; the plain launch's values up to the fp16 rounding of the exchanged partial."""
    from uniql_b200 import ops
    shapes = [(4096, 4096, False), (4096, 14336, True), (1024, 512, False), (4096, 4096, False), (3584, 18944, True)]
    layers = [(quantized_layer(n + k, n, k, bias=b), n, k) for n, k, b in shapes]     # same layers for every m
    for rep in range(2):
        for layer, n, k in layers:
            p, s, b = _dev(layer)
            x = make_acts(m + rep, m, k).cuda()
            res = make_acts(m + 40 + rep, m, n, outliers=False).cuda()
            got = comm.linear_all_reduce(x, p, s, b, n, residual=res)
            (want,) = ops.w4a16_linear_group(x, [(p, s, b, n)], residual=res)
            torch.cuda.synchronize()
            # the partial crosses the exchange as fp16 before bias and residual are added: one more rounding than the
            # plain launch, never more than a couple of fp16 steps of the result
            assert torch.allclose(got.float(), want.float(), rtol=2e-3, atol=2e-3 * float(want.float().abs().max()))
            linear_tolerance_check((got.float() - res.float()).cpu().numpy(),
                                   orc.linear_ref(x.cpu().numpy(), None, None, layer["bias"], n, w_deq=layer["w_deq"]))
    assert ops.read_and_clear_status("cuda") == 0


@pytest.mark.parametrize("hidden,inter,m", [(4096, 14336, 1), (4096, 14336, 4), (4096, 14336, 16), (4096, 8192, 2),
                                            (512, 16384, 1)])
def test_gathered_mlp_chain_equals_the_single_gpu_launches(comm, hidden, inter, m):
    """gate+up+SwiGLU whose epilogue also fills the feature area, then the Hadamard kernel that reads the row from
    there and the down projection that sums in its epilogue: same values as the plain grouped launches, and inside
    the tolerance of the oracle."""
    from uniql_b200 import ops
    gate, up, down = quantized_layer(1, inter, hidden), quantized_layer(2, inter, hidden), quantized_layer(3, hidden, inter)
    gp, gs, _ = _dev(gate)
    up_, us, _ = _dev(up)
    dp, ds, _ = _dev(down)
    for rep in range(3):                                     # both parities of the feature area
        x = make_acts(10 + rep, m, hidden).cuda()
        res = make_acts(20 + rep, m, hidden, outliers=False).cuda()
        h = comm.gate_up_gather(x, (gp, gs, None, inter), (up_, us, None, inter), 0)
        y = comm.down_gather_reduce(m, (dp, ds, None, hidden), inter, 0, residual=res)
        (h0,) = ops.w4a16_linear_group(x, [(gp, gs, None, inter), (up_, us, None, inter)], epilogue="swiglu")
        (y0,) = ops.w4a16_linear_group(h0, [(dp, ds, None, hidden)], residual=res, hadamard_dim=inter)
        torch.cuda.synchronize()
        assert torch.equal(h, h0)
        assert torch.allclose(y.float(), y0.float(), rtol=2e-2, atol=2e-2 * float(y0.float().abs().max()))
    hh = orc.hadamard_transform(h0.double().cpu().numpy()).astype(np.float16)
    lin = orc.linear_ref(hh, None, None, None, hidden, w_deq=down["w_deq"])
    linear_tolerance_check((y.float() - res.float()).cpu().numpy(), lin)
    assert ops.read_and_clear_status("cuda") == 0


def test_tensor_parallel_launches_replay_from_a_cuda_graph(comm):
    """Epoch counters live on the device: a captured chain replays any number of times."""
    from uniql_b200 import ops
    hidden, inter, m = 4096, 14336, 2
    gate, up, down = quantized_layer(4, inter, hidden), quantized_layer(5, inter, hidden), quantized_layer(6, hidden, inter)
    gp, gs, _ = _dev(gate)
    up_, us, _ = _dev(up)
    dp, ds, _ = _dev(down)
    x = make_acts(1, m, hidden).cuda()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        def chain():
            comm.gate_up_gather(x, (gp, gs, None, inter), (up_, us, None, inter), 0)
            return comm.down_gather_reduce(m, (dp, ds, None, hidden), inter, 0, residual=x)
        want = chain().clone()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            y = chain()
        for _ in range(5):
            graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(y, want)
    assert ops.read_and_clear_status("cuda") == 0
