"""GPU: the scratch-free entry point `uniql_w4a16_linear_static`, called through the C ABI.

Some callers cannot give this library device scratch: they run inside a memory plan they do not own, or in a
loop where allocator calls are forbidden after start-up.  For them the decode kernel can use a fixed array
built into the library.  This test drives that entry point with raw pointers, twice in a row (the array is
shared and keeps the previous call's contents), and checks the results against the regular entry point, which
runs the same kernel with caller-supplied scratch.  It is collected last on purpose.
"""
import numpy as np
import pytest
import torch

from helpers import linear_tolerance_check, make_acts, quantized_layer
from oracle import uniql_oracle as orc

pytestmark = pytest.mark.gpu


def _static_call(x, packed, scales, bias, n_out):
    from uniql_b200._lib import check, lib
    m, k = x.shape
    n = scales.shape[1]
    out = torch.empty((m, n_out), dtype=torch.float16, device=x.device)
    stream = torch.cuda.current_stream().cuda_stream
    code = lib().uniql_w4a16_linear_static(
        x.data_ptr(), x.stride(0), packed.data_ptr(), scales.data_ptr(), bias.data_ptr() if bias is not None else None,
        out.data_ptr(), out.stride(0), m, n, n_out, k, 128, None, stream)
    check(code, "uniql_w4a16_linear_static")
    return out


@pytest.mark.parametrize("n,k,m", [(4096, 4096, 1), (1024, 1536, 5), (14336, 4096, 4), (4096, 12160, 4),
                                   (512, 14336, 4)])
def test_static_scratch_matches_regular_entry_point(n, k, m):
    from uniql_b200 import ops
    from uniql_b200._lib import lib
    layer = quantized_layer(n + k + m, n, k, bias=True)
    packed = torch.from_numpy(layer["packed"]).cuda()
    scales = torch.from_numpy(layer["scales"]).cuda()
    bias = torch.from_numpy(layer["bias"]).cuda()
    # the kernel keeps its per-block tickets AND its partial tiles in the array: every shape here needs more than the
    # ticket region, so a wrong device address or stale contents would show in the result
    assert lib().uniql_w4a16_scratch_bytes(m, n, k, 0) > 16384
    # a layer of another width run in between: its tiles and tickets land on the same bytes of the array
    other = quantized_layer(7, 768, 2304, bias=False)
    o_packed, o_scales = torch.from_numpy(other["packed"]).cuda(), torch.from_numpy(other["scales"]).cuda()
    ref = None
    for call in range(2):                      # two calls in a row share the built-in array
        x = make_acts(100 * call + m, m, k).cuda()
        got = _static_call(x, packed, scales, bias, n)
        xo = make_acts(call, 3, 2304).cuda()
        got_o = _static_call(xo, o_packed, o_scales, None, 768)
        want = ops.w4a16_linear(x, packed, scales, bias, n)
        want_o = ops.w4a16_linear(xo, o_packed, o_scales, None, 768)
        torch.cuda.synchronize()
        # same kernel, same split: identical bits, and inside the oracle tolerance used by the other linear tests
        assert torch.equal(got, want)
        assert torch.equal(got_o, want_o)
        ref = orc.linear_ref(x.cpu().numpy(), None, None, layer["bias"], n, w_deq=layer["w_deq"])
        linear_tolerance_check(got.cpu().numpy(), ref)
    assert ref is not None


def test_static_scratch_limits_are_reported():
    from uniql_b200._lib import lib
    L = lib()
    x = torch.zeros(17, 256, dtype=torch.float16, device="cuda")
    w = torch.zeros(16, 512, dtype=torch.int32, device="cuda")
    s = torch.zeros(2, 256, dtype=torch.float16, device="cuda")
    out = torch.zeros(17, 256, dtype=torch.float16, device="cuda")
    args = (w.data_ptr(), s.data_ptr(), None, out.data_ptr(), 256)
    assert L.uniql_w4a16_linear_static(x.data_ptr(), 256, *args, 17, 256, 256, 256, 128, None, None) == -3   # m > 16
    assert L.uniql_w4a16_linear_static(x.data_ptr(), 256, *args, 1, 256, 256, 256, -1, None, None) == -2    # per-channel
    # a problem whose scratch need is beyond the built-in array is refused, nothing is launched.  The buffers are real
    # and large enough all the same: this call must never be able to touch memory it does not own.
    big_n, big_k, big_m = 65536, 8192, 16
    assert L.uniql_w4a16_scratch_bytes(big_m, big_n, big_k, 0) > 8 * 1024 * 1024
    xb = torch.zeros(big_m, big_k, dtype=torch.float16, device="cuda")
    wb = torch.zeros(big_k // 16, 2 * big_n, dtype=torch.int32, device="cuda")
    sb = torch.zeros(big_k // 128, big_n, dtype=torch.float16, device="cuda")
    ob = torch.zeros(big_m, big_n, dtype=torch.float16, device="cuda")
    assert L.uniql_w4a16_linear_static(xb.data_ptr(), big_k, wb.data_ptr(), sb.data_ptr(), None, ob.data_ptr(), big_n,
                                       big_m, big_n, big_n, big_k, 128, None, None) == -7
    torch.cuda.synchronize()
    assert b"built-in scratch" in L.uniql_strerror(-7)
