"""GPU: W4A16 linear against the oracle (fp32 accumulation of the same dequantised weights), through the C ABI.
Tolerance (stated by the task): max-normalised error <= 1e-2 and |y - y_ref| <= 1e-2|y_ref| + 1e-2 rms(y_ref)."""
import os

import numpy as np
import pytest
import torch

from helpers import linear_tolerance_check, make_acts, quantized_layer
from oracle import uniql_oracle as orc

pytestmark = pytest.mark.gpu


def _run(layer, x, n_out=None, hadamard=False):
    from uniql_b200 import ops
    n_out = layer["n"] if n_out is None else n_out
    b = torch.from_numpy(layer["bias"]).cuda() if layer["bias"] is not None else None
    y = ops.w4a16_linear(x.cuda(), torch.from_numpy(layer["packed"]).cuda(), torch.from_numpy(layer["scales"]).cuda(),
                         b, n_out, hadamard_dim=layer["k"] if hadamard else 0)
    torch.cuda.synchronize()
    return y.cpu().numpy()


def _ref(layer, x, n_out=None):
    n_out = layer["n"] if n_out is None else n_out
    return orc.linear_ref(x.numpy(), None, None, layer["bias"], n_out, w_deq=layer["w_deq"])


SMALL_SHAPES = [(64, 128), (256, 256), (200, 384), (896, 512), (1024, 1536), (448, 2304)]


@pytest.mark.parametrize("n,k", SMALL_SHAPES)
@pytest.mark.parametrize("m", [1, 2, 3, 8, 9, 15, 16])
def test_decode_small_shapes(n, k, m):
    layer = quantized_layer(n * 7 + k, n, k, bias=(n % 128 == 0))
    x = make_acts(m, m, k)
    linear_tolerance_check(_run(layer, x), _ref(layer, x))


@pytest.mark.parametrize("m", [17, 33, 63, 64, 65])
def test_rows_beyond_16(m):
    layer = quantized_layer(11, 512, 1024, bias=True)
    x = make_acts(m, m, 1024)
    linear_tolerance_check(_run(layer, x), _ref(layer, x))


@pytest.mark.parametrize("n,k", [(4096, 4096), (6144, 4096), (14336, 4096), (4096, 14336), (12160, 4096),
                                 (4096, 12160), (5632, 4096), (4096, 3584), (3584, 18944), (18560, 4096), (4096, 8192)])
@pytest.mark.parametrize("m", [1, 4, 16])
def test_baseline_shapes_decode(n, k, m):
    layer = quantized_layer(n + k, n, k)
    x = make_acts(m + 1, m, k)
    linear_tolerance_check(_run(layer, x), _ref(layer, x))


def test_padded_output_columns_and_full_width():
    layer = quantized_layer(5, 200, 384, bias=True)
    x = make_acts(2, 4, 384)
    # the stand-in for quant_linear_cuda returns the full stored width; padded columns are zero
    from uniql_b200.compat import quant_linear_cuda
    ws = torch.zeros(64, dtype=torch.int32, device="cuda")
    y = quant_linear_cuda.w4a16o16_gemm(x.cuda(), torch.from_numpy(layer["packed"]).cuda(),
                                        torch.from_numpy(layer["scales"]).cuda(), ws, 4, 256, 384, False, -1, -1, -1, 16)
    assert y.shape == (4, 256)
    y = y.cpu().numpy()
    assert (y[:, 200:] == 0).all()
    nobias = dict(layer, bias=None)
    linear_tolerance_check(y[:, :200], _ref(nobias, x))
    assert int(ws.abs().sum()) == 0


def test_deterministic_and_scratch_reuse():
    layer = quantized_layer(3, 4096, 4096)
    x = make_acts(9, 1, 4096)
    a = _run(layer, x)
    for _ in range(3):
        assert np.array_equal(a.view(np.uint16), _run(layer, x).view(np.uint16))
    small = quantized_layer(4, 256, 256)
    xs = make_acts(1, 3, 256)
    linear_tolerance_check(_run(small, xs), _ref(small, xs))
    assert np.array_equal(a.view(np.uint16), _run(layer, x).view(np.uint16))


def test_strided_activations_and_batch_dims():
    from uniql_b200.quantize.quant_linear_layers import W4A16B16O16Linear
    lin = torch.nn.Linear(384, 200, bias=True).half()
    q = W4A16B16O16Linear.from_fp16(lin).cuda()
    x = make_acts(1, 6, 768).cuda()[:, :384].reshape(2, 3, 384)      # row stride 768
    y = q(x)
    assert y.shape == (2, 3, 200) and y.is_contiguous()
    w_deq = orc.dequantize(q.weight.cpu().numpy(), q.scale.cpu().numpy())
    want = orc.linear_ref(x.reshape(6, 384).cpu().numpy(), None, None, lin.bias.data.numpy(), 200, w_deq=w_deq)
    linear_tolerance_check(y.reshape(6, 200).cpu().numpy(), want)


def test_reference_checkpoint_loads_and_runs(golden_dir):
    """State dict produced by the reference's from_fp16 (K padded 200 -> 256 is not in this fixture;
    N padded 200 -> 256 is)."""
    from uniql_b200.quantize.quant_linear_layers import W4A16B16O16Linear
    g = np.load(os.path.join(golden_dir, "linear_module.npz"))
    q = W4A16B16O16Linear(384, 200, bias=True)
    q.load_state_dict({k[3:]: torch.from_numpy(g[k]) for k in g.files if k.startswith("sd_")}, strict=True)
    q = q.to("cuda").to(torch.float16)
    x = make_acts(3, 5, 384)
    y = q(x.cuda()).cpu().numpy()
    w = torch.from_numpy(g["fp16_weight"]).float()
    # against the *unquantised* layer the error is the quantisation error: loose sanity bound
    y_fp = x.float() @ w.t() + torch.from_numpy(g["fp16_bias"]).float()
    assert np.abs(y - y_fp.numpy()).max() < 0.2 * np.abs(y_fp.numpy()).max()
    w_deq = orc.dequantize(g["sd_weight"], g["sd_scale"])
    linear_tolerance_check(y, orc.linear_ref(x.numpy(), None, None, g["fp16_bias"], 200, w_deq=w_deq))


def test_k_padding_path():
    from uniql_b200.quantize.quant_linear_layers import W4A16B16O16Linear
    lin = torch.nn.Linear(200, 192, bias=False).half()
    q = W4A16B16O16Linear.from_fp16(lin).cuda()
    assert q.pad_in == 56 and q.size_k == 256
    x = make_acts(8, 3, 200, outliers=False)
    y = q(x.cuda()).cpu().numpy()
    w_deq = orc.dequantize(q.weight.cpu().numpy(), q.scale.cpu().numpy())
    xp = np.pad(x.numpy(), ((0, 0), (0, 56)))
    linear_tolerance_check(y, orc.linear_ref(xp, None, None, None, 192, w_deq=w_deq))


def test_error_codes():
    from uniql_b200 import UniqlError, ops
    x = torch.zeros(1, 256, dtype=torch.float16, device="cuda")
    w = torch.zeros(16, 128, dtype=torch.int32, device="cuda")
    with pytest.raises(UniqlError) as e:       # a single scale row = the reference's per-channel mode
        ops.w4a16_linear(x, w, torch.zeros(1, 64, dtype=torch.float16, device="cuda"), None, 64)
    assert e.value.code == -2
    with pytest.raises(RuntimeError):
        ops.w4a16_linear(x.float(), w, torch.zeros(2, 64, dtype=torch.float16, device="cuda"), None, 64)
    with pytest.raises(RuntimeError):
        ops.w4a16_linear(x[:, :128], w, torch.zeros(2, 64, dtype=torch.float16, device="cuda"), None, 64)


def test_linearity_property_full_size():
    """Size-independent property at a BASELINE shape: f(x1 + x2) = f(x1) + f(x2) up to fp16 rounding,
    and f(e_k) reproduces a dequantised weight row exactly."""
    layer = quantized_layer(77, 14336, 4096)
    x1, x2 = make_acts(1, 4, 4096, outliers=False), make_acts(2, 4, 4096, outliers=False)
    y1, y2, y12 = _run(layer, x1), _run(layer, x2), _run(layer, (x1.float() + x2.float()).half())
    ref12 = _ref(layer, (x1.float() + x2.float()).half())
    linear_tolerance_check(y1.astype(np.float32) + y2.astype(np.float32), ref12)
    linear_tolerance_check(y12, ref12)
    e = torch.zeros(3, 4096, dtype=torch.float16)
    rows = [0, 2049, 4095]
    for i, r in enumerate(rows):
        e[i, r] = 1
    y = _run(layer, e)
    assert np.array_equal(y, layer["w_deq"][rows][:, :14336])


# ---------------------------------------------------------------------------------------------
# prefill regime (m > 16): tcgen05 tensor-core kernel
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("n,k", [(256, 128), (384, 256), (200, 384), (1792, 1024), (448, 512), (128, 4096)])
@pytest.mark.parametrize("m", [17, 64, 127, 128, 129, 300])
def test_prefill_small_shapes(n, k, m):
    layer = quantized_layer(n * 3 + k + m, n, k, bias=(n % 256 == 0))
    x = make_acts(m, m, k)
    linear_tolerance_check(_run(layer, x), _ref(layer, x))


@pytest.mark.parametrize("n,k", [(4096, 4096), (14336, 4096), (4096, 14336), (12160, 4096), (4096, 12160),
                                 (5632, 4096), (4096, 3584), (18560, 4096), (4096, 8192)])
@pytest.mark.parametrize("m", [1024, 4096])
def test_baseline_shapes_prefill_sampled_rows(n, k, m):
    """Full-size launch; 48 seeded rows of the output are compared with the oracle (the rest of the rows are
    covered by the checksum below: column sums of y equal (sum of rows of x) @ W within fp16 accumulation noise)."""
    layer = quantized_layer(n + k + 5, n, k)
    x = make_acts(m + 3, m, k)
    y = _run(layer, x)
    rng = np.random.default_rng(m + n)
    rows = np.sort(rng.choice(m, size=48, replace=False))
    rows[0], rows[-1] = 0, m - 1
    ref = orc.linear_ref(x.numpy()[rows], None, None, None, n, w_deq=layer["w_deq"])
    linear_tolerance_check(y[rows], ref)
    col_ref = orc.linear_ref(x.float().sum(0, keepdim=True).numpy(), None, None, None, n, w_deq=layer["w_deq"])
    col_sum = y.astype(np.float64).sum(0, keepdims=True)
    # each y element carries at most half an fp16 ulp of rounding; the sum of m of them stays far below this
    tol = 2.0 ** -10 * np.abs(y).astype(np.float64).sum(0, keepdims=True) + 1e-3
    assert (np.abs(col_sum - col_ref) <= tol).all()


@pytest.mark.parametrize("n,k", [(12160, 4096), (4096, 12160), (3584, 4096), (4096, 3584), (896, 4096)])
def test_sliced_llama_shapes_at_2048_rows(n, k):
    """The 85 % Llama-3.1-8B layers (intermediate 12160, head_dim 112) at the 2048-row prefill of that configuration:
    sampled rows against the oracle, all rows through the column-sum identity."""
    m = 2048
    layer = quantized_layer(n + k + 85, n, k)
    x = make_acts(m + 5, m, k)
    y = _run(layer, x)
    rng = np.random.default_rng(n * 3 + k)
    rows = np.sort(rng.choice(m, size=48, replace=False))
    rows[0], rows[-1] = 0, m - 1
    linear_tolerance_check(y[rows], orc.linear_ref(x.numpy()[rows], None, None, None, n, w_deq=layer["w_deq"]))
    col_ref = orc.linear_ref(x.float().sum(0, keepdim=True).numpy(), None, None, None, n, w_deq=layer["w_deq"])
    col_sum = y.astype(np.float64).sum(0, keepdims=True)
    tol = 2.0 ** -10 * np.abs(y).astype(np.float64).sum(0, keepdims=True) + 1e-3
    assert (np.abs(col_sum - col_ref) <= tol).all()


# ---------------------------------------------------------------------------------------------
# batches of 17..128 rows: operand-swapped tcgen05 kernel, with a cluster split over k when there are few column tiles
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("n,k", [(4096, 4096), (14336, 4096), (4096, 14336), (1024, 4096), (6144, 4096), (18944, 3584),
                                 (3584, 18944), (512, 2048), (192, 640)])
@pytest.mark.parametrize("m", [17, 48, 64, 100, 128])
def test_baseline_shapes_mid_batch(n, k, m):
    layer = quantized_layer(n + k + 1, n, k, bias=(n == 1024))      # one layer per shape, reused for every m
    x = make_acts(m + 7, m, k)
    linear_tolerance_check(_run(layer, x), _ref(layer, x))


def test_mid_batch_deterministic():
    layer = quantized_layer(23, 1024, 4096)          # 8 column tiles -> split over k inside a cluster
    x = make_acts(6, 96, 4096)
    a = _run(layer, x)
    for _ in range(2):
        assert np.array_equal(a.view(np.uint16), _run(layer, x).view(np.uint16))


def test_prefill_strided_input_bias_and_batch_dims():
    from uniql_b200.quantize.quant_linear_layers import W4A16B16O16Linear
    lin = torch.nn.Linear(512, 328, bias=True).half()
    q = W4A16B16O16Linear.from_fp16(lin).cuda()
    x = make_acts(4, 96, 1024).cuda()[:, 256:768].reshape(4, 24, 512)
    y = q(x)
    assert y.shape == (4, 24, 328)
    w_deq = orc.dequantize(q.weight.cpu().numpy(), q.scale.cpu().numpy())
    want = orc.linear_ref(x.reshape(96, 512).cpu().numpy(), None, None, lin.bias.data.numpy(), 328, w_deq=w_deq)
    linear_tolerance_check(y.reshape(96, 328).cpu().numpy(), want)


def test_prefill_deterministic():
    layer = quantized_layer(21, 1024, 2048)
    x = make_acts(5, 200, 2048)
    a = _run(layer, x)
    for _ in range(2):
        assert np.array_equal(a.view(np.uint16), _run(layer, x).view(np.uint16))
