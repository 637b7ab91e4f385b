"""The torch binding (uniql_b200/_torch_ext.so, csrc/torch_binding.cpp) against the ctypes path: both call the same
C ABI, so their results are equal bit for bit; the modules' forward uses the binding."""
import numpy as np
import pytest
import torch

from helpers import linear_tolerance_check, make_acts, quantized_layer
from oracle import uniql_oracle as orc


def _ext():
    from uniql_b200._lib import torch_ext
    ext = torch_ext()
    assert ext is not None, "uniql_b200/_torch_ext.so is not built or failed to load"
    return ext


def test_binding_loads_and_refuses_cpu_tensors(built_lib):
    ext = _ext()
    from uniql_b200 import lib
    assert ext.abi_version() == lib().uniql_abi_version()
    w = torch.zeros(8, 512, dtype=torch.int32)
    s = torch.zeros(1, 256, dtype=torch.float16)
    with pytest.raises(RuntimeError):
        ext.linear(torch.zeros(1, 128, dtype=torch.float16), w, s, None, 256, 0, False)
    with pytest.raises(RuntimeError):
        ext.hadamard(torch.zeros(4, 64), 1.0)
    with pytest.raises(RuntimeError):
        ext.embedding(torch.zeros(3, dtype=torch.int64), torch.zeros(4, 8, dtype=torch.int32), torch.zeros(4, dtype=torch.float16))
    with pytest.raises(RuntimeError):
        ext.linear_group(torch.zeros(1, 128, dtype=torch.float16), [w], [s], [None], [256], 0, None, 0, False)


def _dev(layer):
    b = torch.from_numpy(layer["bias"]).cuda() if layer["bias"] is not None else None
    return torch.from_numpy(layer["packed"]).cuda(), torch.from_numpy(layer["scales"]).cuda(), b


@pytest.mark.gpu
@pytest.mark.parametrize("n,k,bias", [(256, 256, True), (200, 384, False), (4096, 4096, False), (1000, 1024, True)])
@pytest.mark.parametrize("m", [1, 5, 16, 40, 300])
def test_linear_equals_ctypes_path(n, k, m, bias):
    from uniql_b200 import ops
    ext = _ext()
    layer = quantized_layer(n + k + m, n, k, bias=bias)
    p, s, b = _dev(layer)
    x = make_acts(m, m, k).cuda()
    want = ops.w4a16_linear(x, p, s, b, n)
    got = ext.linear(x, p, s, b, n, 0, False)
    assert got.shape == (m, n) and torch.equal(got, want)
    linear_tolerance_check(got.cpu().numpy(), orc.linear_ref(x.cpu().numpy(), None, None, layer["bias"], n, w_deq=layer["w_deq"]))
    # leading dimensions are kept, strided rows are accepted
    x3 = x.reshape(1, m, k)
    assert ext.linear(x3, p, s, b, n, 0, False).shape == (1, m, n)
    wide = torch.zeros(m, k + 8, dtype=torch.float16, device="cuda")
    wide[:, :k] = x
    assert torch.equal(ext.linear(wide[:, :k], p, s, b, n, 0, False), want)


@pytest.mark.gpu
def test_modules_run_through_the_binding_with_padding_and_hadamard():
    from uniql_b200 import ops
    from uniql_b200.quantize.quant_linear_layers import W4A16B16O16HadLinear, W4A16B16O16Linear
    lin = torch.nn.Linear(200, 300, bias=True).half().cuda()            # in_features padded to 256, out to 512
    q = W4A16B16O16Linear.from_fp16(lin)
    x = make_acts(3, 2 * 7, 200).reshape(2, 7, 200).cuda()
    y = q(x)
    assert y.shape == (2, 7, 300)
    x2 = torch.nn.functional.pad(x.reshape(-1, 200), (0, 56))
    assert torch.equal(y.reshape(-1, 300), ops.w4a16_linear(x2, q.weight, q.scale, q.bias, 300))
    from uniql_b200.quantize import quantize_helpers as qh
    w_deq = qh.w4a16_dequantize(q.weight.cpu(), q.scale.cpu())[:200, :300].float()
    want = x.reshape(-1, 200).float().cpu() @ w_deq + lin.bias.detach().float().cpu()
    linear_tolerance_check(y.reshape(-1, 300).cpu().numpy(), want.numpy())
    layer = quantized_layer(5, 512, 3584)
    h = W4A16B16O16HadLinear(3584, 512, device="cuda")
    h.weight, h.scale = _dev(layer)[:2]
    for m in (1, 4, 16, 33):
        xa = make_acts(m, m, 3584).cuda()
        assert torch.equal(h(xa), ops.w4a16_linear(xa, h.weight, h.scale, None, 512, hadamard_dim=3584))
    assert ops.read_and_clear_status("cuda") == 0


@pytest.mark.gpu
def test_grouped_launches_embedding_and_hadamard_equal_ctypes_path():
    from uniql_b200 import fused as fz
    from uniql_b200 import ops
    from uniql_b200.quantize.quant_linear_layers import W4A16B16O16HadLinear, W4A16B16O16Linear
    ext = _ext()

    def mod(seed, n, k, bias=False, cls=W4A16B16O16Linear):
        layer = quantized_layer(seed, n, k, bias=bias)
        m = cls(k, n, bias=bias, device="cuda")
        m.weight, m.scale, b = _dev(layer)
        if bias:
            m.bias = torch.nn.Parameter(b, requires_grad=False)
        return m

    gate, up, down = mod(1, 3584, 1024), mod(2, 3584, 1024), mod(3, 1024, 3584, cls=W4A16B16O16HadLinear)
    q, k_, v = mod(4, 1024, 1024, True), mod(5, 256, 1024, True), mod(6, 256, 1024, True)
    for m in (1, 3, 16):
        x = make_acts(m, m, 1024).cuda()
        h = fz.gate_up_swiglu(gate, up, x)
        (h0,) = ops.w4a16_linear_group(x, [(gate.weight, gate.scale, None, 3584), (up.weight, up.scale, None, 3584)],
                                       epilogue="swiglu")
        assert torch.equal(h, h0)
        y = fz.linear_residual(down, h, x)
        (y0,) = ops.w4a16_linear_group(h0, [(down.weight, down.scale, None, 1024)], residual=x, hadamard_dim=3584)
        assert torch.equal(y, y0)
        outs = fz.qkv_proj(q, k_, v, x.reshape(1, m, 1024))
        outs0 = ops.w4a16_linear_group(x, [(t.weight, t.scale, t.bias, t.out_features) for t in (q, k_, v)])
        assert all(o.shape == (1, m, o0.shape[1]) and torch.equal(o[0], o0) for o, o0 in zip(outs, outs0))
    # 17..128 rows: gate and up share one tensor-core launch, SiLU and the product stay in PyTorch; beyond that the
    # separate modules run -- the same values either way (the split over k may order the fp32 sums differently)
    for rows in (40, 128, 200):
        xb = make_acts(9, rows, 1024).cuda()
        got = fz.gate_up_swiglu(gate, up, xb).float()
        want = (torch.nn.functional.silu(gate(xb)) * up(xb)).float()
        assert got.shape == (rows, 3584)
        assert float((got - want).abs().max()) <= 4e-3 * float(want.abs().max()) + 1e-3
        qo = fz.qkv_proj(q, k_, v, xb)
        for o, mod in zip(qo, (q, k_, v)):
            w = mod(xb).float()
            assert o.shape == w.shape and float((o.float() - w).abs().max()) <= 2e-3 * float(w.abs().max()) + 1e-3
    xb = make_acts(9, 40, 1024).cuda()
    with pytest.raises(RuntimeError):
        ext.linear_group(make_acts(9, 130, 1024).cuda(), [gate.weight], [gate.scale], [None], [3584], 0, None, 0, False)  # > 128 rows
    with pytest.raises(RuntimeError):
        ext.linear_group(xb, [gate.weight, up.weight], [gate.scale, up.scale], [None, None], [3584, 3584], 1, None, 0, False)  # SwiGLU above 16 rows
    with pytest.raises(RuntimeError):
        ext.linear_group(xb[:2], [gate.weight, q.weight], [gate.scale, q.scale], [None, None], [3584, 1024], 1, None, 0, False)
    # embedding and Hadamard
    table = (torch.randn(300, 256, generator=torch.Generator().manual_seed(1)) * 0.02).half().numpy()
    ep, es = orc.embedding_quantize(table)
    ids = torch.randint(0, 300, (2, 9), generator=torch.Generator().manual_seed(2)).cuda()
    got = ext.embedding(ids, torch.from_numpy(ep).cuda(), torch.from_numpy(es).cuda())
    assert got.shape == (2, 9, 256)
    assert torch.equal(got, ops.w4_embedding(ids, torch.from_numpy(ep).cuda(), torch.from_numpy(es).cuda()))
    for dim, rows, dt in ((14336, 3, torch.float16), (8192, 100, torch.bfloat16), (768, 5, torch.float32)):
        xh = torch.randn(rows, dim, device="cuda").to(dt)
        assert torch.equal(ext.hadamard(xh, dim ** -0.5), ops.hadamard(xh, dim ** -0.5))
    assert ops.read_and_clear_status("cuda") == 0
    # the diagnostics word is the same tensor on both paths
    assert ext.status_tensor(0).data_ptr() == ops.status_word(torch.device("cuda", 0)).data_ptr()


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(17, 3584), (64, 14336), (2, 5, 256), (300, 18944), (1, 8)])
def test_silu_mul_one_pass_equals_the_two_pytorch_ops(shape):
    """uniql_silu_mul: fp16 SiLU, fp16 product -- the values PyTorch's silu followed by mul give (one fp16 step of
    slack for a differently rounded exponential), through both bindings, for strided inputs too."""
    from uniql_b200 import ops
    ext = _ext()
    gen = torch.Generator().manual_seed(sum(shape))
    g = (torch.randn(*shape, generator=gen) * 3).half().cuda()
    u = (torch.randn(*shape, generator=gen) * 2).half().cuda()
    want = torch.nn.functional.silu(g) * u
    for got in (ops.silu_mul(g, u), ext.silu_mul(g, u)):
        assert got.shape == want.shape and got.dtype == torch.float16
        diff = (got.float() - want.float()).abs()
        assert bool((diff <= 2.0 ** -9 * want.float().abs() + 1e-6).all())
        assert float((got.float() != want.float()).float().mean()) < 0.01      # nearly always the same bits
    wide = torch.zeros(*shape[:-1], shape[-1] + 8, dtype=torch.float16, device="cuda")
    wide[..., :shape[-1]] = g
    assert torch.equal(ext.silu_mul(wide[..., :shape[-1]], u), ext.silu_mul(g, u))
    with pytest.raises(RuntimeError):
        ext.silu_mul(g, u[..., :-1] if shape[-1] > 8 else u.float())
