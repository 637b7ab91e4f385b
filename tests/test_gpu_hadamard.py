"""GPU: Hadamard transform (power-of-two and 12N/20N/28N/40N) and the fused Hadamard + linear.
Power-of-two sizes follow the unambiguous Sylvester definition.  For 12N/20N/28N/40N the reference's
third-party matrices are unavailable, so parity there is against this build's own (Paley) matrices."""
import numpy as np
import pytest
import torch

from helpers import linear_tolerance_check, make_acts, quantized_layer
from oracle import uniql_oracle as orc

pytestmark = pytest.mark.gpu

DIMS = [8, 64, 256, 512, 4096, 8192, 32768, 96, 768, 1536, 640, 5120, 224, 3584, 14336, 320, 10240, 40960]


@pytest.mark.parametrize("dim", DIMS)
@pytest.mark.parametrize("rows", [1, 5])
def test_transform_fp32(dim, rows):
    from uniql_b200 import ops
    rng = np.random.default_rng(dim + rows)
    x = rng.standard_normal((rows, dim)).astype(np.float32)
    y = ops.hadamard(torch.from_numpy(x).cuda(), 1.0 / np.sqrt(dim)).cpu().numpy()
    want = orc.hadamard_transform(x.astype(np.float64))
    assert np.abs(y - want).max() <= 2e-5 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("dim", [4096, 14336, 8192, 3584])
def test_transform_16bit(dim, dtype):
    from uniql_b200 import ops
    x = make_acts(dim, 3, dim).to(dtype)
    y = ops.hadamard(x.cuda(), 1.0 / np.sqrt(dim)).cpu()
    want = orc.hadamard_transform(x.double().numpy())
    eps = 2.0 ** -10 if dtype == torch.float16 else 2.0 ** -7
    assert np.abs(y.double().numpy() - want).max() <= eps * np.abs(want).max() + 1e-6
    assert y.dtype == dtype


@pytest.mark.parametrize("rows,dim", [(4801, 1024), (4801, 512), (1301, 4096), (1301, 3584), (700, 14336),
                                      (2400, 96), (1200, 8192)])
def test_many_rows_row_kernel(rows, dim):
    """More than 16 rows take the one-CTA-per-row-group kernel; short rows share a CTA (the odd row counts leave a
    partly filled last CTA); a handful of rows are compared with the oracle, all rows with the first/last pattern."""
    from uniql_b200 import ops
    rng = np.random.default_rng(rows + dim)
    x = rng.standard_normal((rows, dim)).astype(np.float32)
    x[-1] = x[0]                                           # same input in the first and the last row
    y = ops.hadamard(torch.from_numpy(x).cuda(), 1.0 / np.sqrt(dim)).cpu().numpy()
    pick = np.unique(np.concatenate([np.arange(0, 9), rng.integers(0, rows, 16), [rows - 2, rows - 1]]))
    want = orc.hadamard_transform(x[pick].astype(np.float64))
    assert np.abs(y[pick] - want).max() <= 2e-5 * max(1.0, np.abs(want).max())
    assert np.array_equal(y[0], y[-1])
    # involution up to the scale: H (H x) / dim = x for symmetric H; for the Paley bases H H^T = dim I is checked
    # through the energy instead
    assert np.allclose((y.astype(np.float64) ** 2).sum(1), (x.astype(np.float64) ** 2).sum(1), rtol=1e-4)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("dim", [2048, 4096, 8192, 16384, 1536, 3072, 6144, 3584, 7168, 14336, 5120, 10240, 20480])
def test_many_rows_16bit_tensor_core_kernel(dim, dtype):
    """16-bit rows with 128 <= dim / base <= 512 (power-of-two sizes count 16 or 32 as their base) apply the base matrix
    with mma.sync on the raw inputs; every (m-tile count, segment length) variant is covered.  Oracle on sampled rows,
    first row == last row, and the in-place call gives the same bits."""
    from uniql_b200 import ops
    from uniql_b200._lib import check, lib
    rows = 333
    x = make_acts(dim + 1, rows, dim).to(dtype)
    x[-1] = x[0]
    xd = x.cuda()
    y = ops.hadamard(xd, dim ** -0.5)
    torch.cuda.synchronize()
    pick = [0, 1, 2, 100, 331, 332]
    want = orc.hadamard_transform(x[pick].double().numpy())
    eps = 2.0 ** -10 if dtype == torch.float16 else 2.0 ** -7
    got = y[pick].double().cpu().numpy()
    assert np.abs(got - want).max() <= eps * np.abs(want).max() + 1e-6
    # away from the largest values the error stays at fp32 accumulation + one rounding of the result
    assert (np.abs(got - want) <= eps * np.abs(want) + 2e-5 * np.abs(want).max()).all()
    assert torch.equal(y[0], y[-1])
    code = lib().uniql_hadamard(xd.data_ptr(), xd.data_ptr(), rows, dim, float(dim ** -0.5),
                                0 if dtype == torch.float16 else 1, torch.cuda.current_stream().cuda_stream)
    check(code, "uniql_hadamard")
    torch.cuda.synchronize()
    assert torch.equal(xd, y)


def test_many_rows_in_place_fp16():
    from uniql_b200._lib import check, lib
    rows, dim = 3000, 2048
    x = make_acts(7, rows, dim).cuda()
    want = ops_hadamard_copy(x, dim)
    code = lib().uniql_hadamard(x.data_ptr(), x.data_ptr(), rows, dim, float(dim ** -0.5), 0,
                                torch.cuda.current_stream().cuda_stream)
    check(code, "uniql_hadamard")
    torch.cuda.synchronize()
    assert torch.equal(x, want)


def ops_hadamard_copy(x, dim):
    from uniql_b200 import ops
    return ops.hadamard(x.clone(), dim ** -0.5)


def test_module_and_helpers_follow_reference_dispatch():
    from uniql_b200.quantize.hadamard_helpers import get_had_fn, had_transform
    from uniql_b200.quantize.quant_hadamard_layers import Hadamard
    assert get_had_fn(14336)[1] == 28 and get_had_fn(8192)[1] == 2 and get_had_fn(5120)[1] == 40
    with pytest.raises(AssertionError):
        get_had_fn(12160)
    had = Hadamard(3584).to("cuda")
    x = make_acts(1, 6, 3584).cuda().reshape(2, 3, 3584)
    y = had(x)
    assert y.shape == x.shape and y.data_ptr() != x.data_ptr()
    want = orc.hadamard_transform(x.double().cpu().numpy())
    assert np.abs(y.double().cpu().numpy() - want).max() <= 2e-3 * np.abs(want).max()
    w = torch.randn(16, 512, device="cuda", dtype=torch.float16)
    assert torch.allclose(had_transform(had_transform(w)).float(), w.float(), atol=2e-2)


@pytest.mark.parametrize("n,k", [(4096, 14336), (4096, 8192), (256, 3584), (512, 1536)])
@pytest.mark.parametrize("m", [1, 4, 16, 40])
def test_fused_hadamard_linear(n, k, m):
    """linear(Hadamard(x)) with the transformed activations rounded to fp16 in between."""
    from uniql_b200 import ops
    layer = quantized_layer(n + k + 1, n, k)
    x = make_acts(m, m, k)
    y = ops.w4a16_linear(x.cuda(), torch.from_numpy(layer["packed"]).cuda(), torch.from_numpy(layer["scales"]).cuda(),
                         None, n, hadamard_dim=k).cpu().numpy()
    xh = orc.hadamard_transform(x.double().numpy()).astype(np.float16)
    want = orc.linear_ref(xh, None, None, None, n, w_deq=layer["w_deq"])
    linear_tolerance_check(y, want)
    # and it agrees with the two-step module composition (the slot-balanced kernel transforms inside the linear with
    # its fp32 sums in another order, so a transformed value may round to the neighbouring fp16 now and then)
    xh_gpu = ops.hadamard(x.cuda(), 1.0 / np.sqrt(k))
    y2 = ops.w4a16_linear(xh_gpu, torch.from_numpy(layer["packed"]).cuda(), torch.from_numpy(layer["scales"]).cuda(),
                          None, n).cpu().numpy()
    linear_tolerance_check(y, y2.astype(np.float32))


@pytest.mark.parametrize("n,k,m", [(4096, 14336, 1024), (4096, 14336, 4096), (4096, 8192, 2048)])
def test_fused_hadamard_linear_prefill_sampled_rows(n, k, m):
    """down_proj / out_proj with their online transform at prefill sizes: full-size launch, 40 seeded rows against the
    oracle (transform in float64, rounded to fp16, then the fp32 linear), the other rows through the column-sum
    identity sum_rows(y) = (sum_rows(fp16(H x))) W."""
    from uniql_b200 import ops
    layer = quantized_layer(n + k + 3, n, k)
    x = make_acts(m + 11, m, k)
    packed, scales = torch.from_numpy(layer["packed"]).cuda(), torch.from_numpy(layer["scales"]).cuda()
    y = ops.w4a16_linear(x.cuda(), packed, scales, None, n, hadamard_dim=k)
    torch.cuda.synchronize()
    y = y.cpu().numpy()
    rng = np.random.default_rng(m + k)
    rows = np.sort(rng.choice(m, size=40, replace=False))
    rows[0], rows[-1] = 0, m - 1
    xh = orc.hadamard_transform(x.double().numpy()[rows]).astype(np.float16)
    linear_tolerance_check(y[rows], orc.linear_ref(xh, None, None, None, n, w_deq=layer["w_deq"]))
    xh_all = ops.hadamard(x.cuda(), 1.0 / np.sqrt(k)).float().sum(0, keepdim=True).cpu().numpy()
    col_ref = orc.linear_ref(xh_all, None, None, None, n, w_deq=layer["w_deq"])
    col_sum = y.astype(np.float64).sum(0, keepdims=True)
    tol = 2.0 ** -10 * np.abs(y).astype(np.float64).sum(0, keepdims=True) + 1e-3
    assert (np.abs(col_sum - col_ref) <= tol).all()
    assert ops.read_and_clear_status("cuda") == 0


def test_had_linear_offline_rotation_matches_online():
    """HadLinear folds H into the weight; y = x W^T must equal (xH)(WH)^T."""
    from uniql_b200.quantize.quant_linear_layers import HadLinear
    lin = torch.nn.Linear(512, 64, bias=False).half().cuda()
    had = HadLinear(lin, input_transform=True, output_transform=False, fuse_had=True)
    from uniql_b200 import ops
    x = torch.randn(4, 512, device="cuda", dtype=torch.float16)
    y = had(ops.hadamard(x, 1.0 / np.sqrt(512)))
    assert torch.allclose(y.float(), (x.float() @ lin.weight.float().t()), atol=3e-2)


@pytest.mark.parametrize("dim", [12 * 512, 20 * 256, 28 * 512, 40 * 256, 28 * 64, 12 * 8])
def test_replaced_base_matrix_is_used_by_every_path(dim):
    """uniql_hadamard_set_base_matrix: with another Hadamard matrix of the same order installed, the few-row kernel,
    the many-row kernel, the fused linear (both decode kernels) and the exported matrix all follow it; results
    against the oracle fed the same matrix.  The built-in matrix is restored afterwards."""
    from uniql_b200 import ops
    base = orc.had_factor(dim)
    h0 = orc.base_matrix(base)
    rng = np.random.default_rng(dim)
    h1 = h0[rng.permutation(base)][:, rng.permutation(base)] * rng.choice([-1, 1], size=(base, 1)) * rng.choice([-1, 1], size=(1, base))
    assert not np.array_equal(h0, h1)
    try:
        ops.hadamard_set_base_matrix(base, h1)
        for rows, dtype in ((1, torch.float16), (5, torch.float32), (16, torch.float16), (70, torch.float32), (300, torch.bfloat16)):
            x = torch.randn(rows, dim, generator=torch.Generator().manual_seed(rows)).to(dtype)
            y = ops.hadamard(x.cuda(), dim ** -0.5)
            want = orc.hadamard_transform(x.double().numpy(), base_h=h1)
            tol = {torch.float32: 2e-5, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}[dtype]
            assert np.abs(y.double().cpu().numpy() - want).max() <= tol * max(1.0, np.abs(want).max())
            wrong = orc.hadamard_transform(x.double().numpy())
            assert np.abs(y.double().cpu().numpy() - wrong).max() > 0.05       # and it is not the built-in transform
        if dim >= 1024:
            import os
            n, layer = 256, quantized_layer(dim, 256, dim)
            packed, scales = torch.from_numpy(layer["packed"]).cuda(), torch.from_numpy(layer["scales"]).cuda()
            for m in (1, 4, 16, 40):
                x = make_acts(m, m, dim)
                xh = orc.hadamard_transform(x.double().numpy(), base_h=h1).astype(np.float16)
                want = orc.linear_ref(xh, None, None, None, n, w_deq=layer["w_deq"])
                for engine in ("tiled", "slot"):
                    os.environ["UNIQL_B200_DECODE_ENGINE"] = engine
                    try:
                        y = ops.w4a16_linear(x.cuda(), packed, scales, None, n, hadamard_dim=dim).cpu().numpy()
                    finally:
                        del os.environ["UNIQL_B200_DECODE_ENGINE"]
                    linear_tolerance_check(y, want)
    finally:
        ops.hadamard_set_base_matrix(base, None)
    x = torch.randn(3, dim, generator=torch.Generator().manual_seed(3))
    y = ops.hadamard(x.cuda(), dim ** -0.5)
    assert np.abs(y.double().cpu().numpy() - orc.hadamard_transform(x.double().numpy())).max() <= 2e-5 * 4
