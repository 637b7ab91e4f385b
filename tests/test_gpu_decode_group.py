"""GPU: grouped decode launches through the C ABI (uniql_w4a16_linear_group) against the oracle.

What the reference's blocks run as separate launches -- gate_proj, up_proj and act_fn(gate) * up
(modeling/llama/llama_qblocks.py:48-51), q/k/v (:104-106), the residual add, the Hadamard module in front of
down_proj -- is one launch here; the expected values are built from the oracle's fp32 linear of the same
dequantised weights with the same elementwise maths on top."""
import numpy as np
import pytest
import torch

from helpers import linear_tolerance_check, make_acts, quantized_layer
from oracle import uniql_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["tiled", "slot"], autouse=True)
def engine(request, monkeypatch):
    """Both decode kernels take every grouped launch: the CTA-tiled one (the default, and the only one tensor-parallel
    launches use) and the slot-balanced one (single GPU; UNIQL_B200_DECODE_ENGINE=slot selects it here)."""
    if request.param == "slot":
        monkeypatch.setenv("UNIQL_B200_DECODE_ENGINE", "slot")
    else:
        monkeypatch.delenv("UNIQL_B200_DECODE_ENGINE", raising=False)
    return request.param


def _dev(layer):
    b = torch.from_numpy(layer["bias"]).cuda() if layer["bias"] is not None else None
    return (torch.from_numpy(layer["packed"]).cuda(), torch.from_numpy(layer["scales"]).cuda(), b, layer["n"])


def _ref(layer, x):
    return orc.linear_ref(np.asarray(x), None, None, layer["bias"], layer["n"], w_deq=layer["w_deq"])


def _silu(v):
    v = v.astype(np.float64)
    return (v / (1.0 + np.exp(-v))).astype(np.float32)


@pytest.mark.parametrize("n,k,m,bias", [(256, 256, 1, False), (192, 384, 3, True), (1024, 1536, 2, False),
                                        (14336, 4096, 1, False), (14336, 4096, 4, False), (12160, 4096, 16, False),
                                        (18944, 3584, 8, False), (1792, 4096, 1, False)])
def test_gate_up_swiglu_matches_separate_modules(n, k, m, bias):
    from uniql_b200 import ops
    gate = quantized_layer(2 * n + k, n, k, bias=bias)
    up = quantized_layer(2 * n + k + 1, n, k, bias=bias)
    x = make_acts(m + 3, m, k)
    (h,) = ops.w4a16_linear_group(x.cuda(), [_dev(gate), _dev(up)], epilogue="swiglu")
    torch.cuda.synchronize()
    want = _silu(_ref(gate, x.numpy())) * _ref(up, x.numpy())
    linear_tolerance_check(h.cpu().numpy(), want)
    # and against the unfused chain of this library: same kernel arithmetic, roundings in the same places
    g16 = ops.w4a16_linear(x.cuda(), *_dev(gate)[:3], n)
    u16 = ops.w4a16_linear(x.cuda(), *_dev(up)[:3], n)
    chain = (torch.nn.functional.silu(g16.float()).half().float() * u16.float()).half()
    diff = (h.float() - chain.float()).abs().max().item()
    assert diff <= 2e-3 * max(1.0, chain.float().abs().max().item())


@pytest.mark.parametrize("shapes,k,m", [([(4096, False), (1024, False), (1024, False)], 4096, 1),
                                        ([(3584, True), (512, True), (512, True)], 3584, 8),
                                        ([(3584, False), (896, False), (896, False)], 4096, 16),
                                        ([(256, True), (64, False)], 256, 5),
                                        ([(128, False), (128, True), (64, False), (192, False)], 384, 2)])
def test_qkv_group_matches_single_launches(shapes, k, m):
    from uniql_b200 import ops
    layers = [quantized_layer(17 * i + n + k, n, k, bias=b) for i, (n, b) in enumerate(shapes)]
    x = make_acts(m + 9, m, k)
    outs = ops.w4a16_linear_group(x.cuda(), [_dev(l) for l in layers])
    torch.cuda.synchronize()
    assert len(outs) == len(layers)
    for layer, y in zip(layers, outs):
        assert y.shape == (m, layer["n"])
        linear_tolerance_check(y.cpu().numpy(), _ref(layer, x.numpy()))
        single = ops.w4a16_linear(x.cuda(), *_dev(layer)[:3], layer["n"])
        linear_tolerance_check(y.cpu().numpy(), single.float().cpu().numpy())


@pytest.mark.parametrize("n,k,m", [(4096, 4096, 1), (200, 384, 4), (4096, 14336, 2)])
def test_residual_add_in_the_epilogue(n, k, m):
    from uniql_b200 import ops
    layer = quantized_layer(n + k + 5, n, k, bias=True)
    x = make_acts(m, m, k)
    res = make_acts(m + 50, m, n, outliers=False)
    (y,) = ops.w4a16_linear_group(x.cuda(), [_dev(layer)], residual=res.cuda())
    torch.cuda.synchronize()
    lin = _ref(layer, x.numpy())
    want = lin.astype(np.float16).astype(np.float32) + res.float().numpy()
    got = y.cpu().numpy().astype(np.float32)
    # the linear part is inside its tolerance; the add itself is one fp16 rounding
    rms = float(np.sqrt(np.mean(lin.astype(np.float64) ** 2)))
    assert np.all(np.abs(got - want) <= 1e-2 * np.abs(lin) + 1e-2 * rms + 2e-3 * np.abs(want) + 1e-3)
    # in place: the residual buffer is also the output
    buf = res.cuda().clone()
    ops.w4a16_linear_group(x.cuda(), [_dev(layer)], residual=buf, outs=[buf])
    torch.cuda.synchronize()
    assert torch.equal(buf, y)


@pytest.mark.parametrize("n,k,m", [(4096, 14336, 1), (4096, 14336, 2), (4096, 14336, 4), (4096, 8192, 1),
                                   (4096, 8192, 3), (1024, 3584, 2), (256, 4096, 1), (512, 1536, 4), (128, 20480, 1),
                                   (256, 5120, 2), (4096, 14336, 8), (4096, 8192, 16)])
def test_hadamard_in_the_prologue(n, k, m):
    """hadamard_dim = k: rows are transformed (fp32 arithmetic, rounded to fp16 as the separate module does) by a
    transform kernel chained in front of the linear; the slot-balanced kernel does it in its own prologue for m <= 4."""
    from uniql_b200 import ops
    layer = quantized_layer(n + k + m, n, k)
    x = make_acts(m + 2, m, k)
    y = ops.w4a16_linear(x.cuda(), *_dev(layer)[:3], n, hadamard_dim=k)
    torch.cuda.synchronize()
    xh = orc.hadamard_transform(x.double().numpy()).astype(np.float16)
    linear_tolerance_check(y.cpu().numpy(), _ref(layer, xh))
    # the separate module followed by the plain linear gives nearly the same bits
    xh_dev = ops.hadamard(x.cuda(), k ** -0.5)
    y2 = ops.w4a16_linear(xh_dev, *_dev(layer)[:3], n)
    linear_tolerance_check(y.cpu().numpy(), y2.float().cpu().numpy())


def test_swiglu_then_hadamard_down_is_the_mlp():
    """The two launches of a decode MLP: h = silu(gate x) * (up x), y = down(H h) + residual."""
    from uniql_b200 import ops
    hidden, inter, m = 1024, 3584, 2
    gate = quantized_layer(1, inter, hidden)
    up = quantized_layer(2, inter, hidden)
    down = quantized_layer(3, hidden, inter)
    x = make_acts(4, m, hidden)
    res = make_acts(5, m, hidden, outliers=False)
    (h,) = ops.w4a16_linear_group(x.cuda(), [_dev(gate), _dev(up)], epilogue="swiglu")
    (y,) = ops.w4a16_linear_group(h, [_dev(down)], residual=res.cuda(), hadamard_dim=inter)
    torch.cuda.synchronize()
    h_ref = (_silu(_ref(gate, x.numpy())) * _ref(up, x.numpy())).astype(np.float16)
    hh = orc.hadamard_transform(h_ref.astype(np.float64)).astype(np.float16)
    lin = _ref(down, hh)
    want = lin.astype(np.float16).astype(np.float32) + res.float().numpy()
    rms = float(np.sqrt(np.mean(lin.astype(np.float64) ** 2)))
    got = y.cpu().numpy().astype(np.float32)
    assert np.all(np.abs(got - want) <= 2e-2 * np.abs(lin) + 2e-2 * rms + 2e-3 * np.abs(want) + 1e-3)


def test_grouped_launches_are_deterministic_and_share_scratch():
    from uniql_b200 import ops
    gate = quantized_layer(21, 4096, 4096)
    up = quantized_layer(22, 4096, 4096)
    down = quantized_layer(23, 512, 14336)
    x = make_acts(1, 1, 4096)
    xd = make_acts(2, 4, 14336)
    first = None
    for _ in range(3):
        (h,) = ops.w4a16_linear_group(x.cuda(), [_dev(gate), _dev(up)], epilogue="swiglu")
        y = ops.w4a16_linear(xd.cuda(), *_dev(down)[:3], 512, hadamard_dim=14336)      # different geometry in between
        torch.cuda.synchronize()
        if first is None:
            first = (h.clone(), y.clone())
        assert torch.equal(h, first[0]) and torch.equal(y, first[1])
    assert ops.read_and_clear_status("cuda") == 0


def test_group_argument_errors():
    from uniql_b200 import UniqlError, ops
    a = quantized_layer(1, 128, 256)
    b = quantized_layer(2, 192, 256)
    x = make_acts(1, 2, 256).cuda()
    with pytest.raises(UniqlError):                      # SwiGLU needs two projections of the same width
        ops.w4a16_linear_group(x, [_dev(a), _dev(b)], epilogue="swiglu")
    with pytest.raises(UniqlError):                      # the residual belongs to a single output
        ops.w4a16_linear_group(x, [_dev(a), _dev(b)], residual=torch.zeros(2, 128, dtype=torch.float16, device="cuda"))
    with pytest.raises(UniqlError):                      # above 16 rows: plain outputs only ...
        ops.w4a16_linear_group(make_acts(1, 17, 256).cuda(), [_dev(a)], residual=torch.zeros(17, 128, dtype=torch.float16, device="cuda"))
    with pytest.raises(UniqlError):                      # ... and at most 128 rows
        ops.w4a16_linear_group(make_acts(1, 129, 256).cuda(), [_dev(a)])
    with pytest.raises(RuntimeError):
        ops.w4a16_linear_group(x, [_dev(a)], epilogue="gelu")


@pytest.mark.parametrize("shapes,k,m", [([(4096, False), (1024, False), (1024, False)], 4096, 64),
                                        ([(3584, True), (512, True), (512, True)], 3584, 17),
                                        ([(14336, False), (14336, False)], 4096, 64),
                                        ([(18944, False), (18944, False)], 3584, 128),
                                        ([(256, True), (192, False)], 256, 33),
                                        ([(128, False), (128, True), (320, False), (192, False)], 384, 100)])
def test_mid_batch_group_runs_on_the_tensor_core_kernel(shapes, k, m):
    """17..128 rows: the projections of a grouped call share one launch of the operand-swapped tcgen05 kernel (one tile
    list over all of them, cluster split along k when there are few tiles); every output agrees with the single launch."""
    from uniql_b200 import ops
    layers = [quantized_layer(19 * i + n + k, n, k, bias=b) for i, (n, b) in enumerate(shapes)]
    x = make_acts(m + 5, m, k)
    outs = ops.w4a16_linear_group(x.cuda(), [_dev(l) for l in layers])
    torch.cuda.synchronize()
    assert len(outs) == len(layers)
    for layer, y in zip(layers, outs):
        assert y.shape == (m, layer["n"])
        single = ops.w4a16_linear(x.cuda(), *_dev(layer)[:3], layer["n"])
        # same kernel; the split over k (and with it the order of the fp32 sums) depends on the launch's tile count
        linear_tolerance_check(y.cpu().numpy(), single.float().cpu().numpy())
        assert float((y.float() - single.float()).abs().max()) <= 2e-3 * float(single.float().abs().max()) + 1e-3
    if layers[0]["n"] <= 4096:
        for layer, y in zip(layers, outs):
            linear_tolerance_check(y.cpu().numpy(), _ref(layer, x.numpy()))
    assert ops.read_and_clear_status("cuda") == 0
