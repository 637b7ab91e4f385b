"""GPU: shapes of the remaining benchmark configurations (Qwen2.5-7B stack, Mamba2 block, UniQL-sliced Llama)
that the other files do not already cover."""
import numpy as np
import pytest
import torch

from helpers import linear_tolerance_check, make_acts, quantized_layer
from oracle import uniql_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,k", [(3584, 3584), (512, 3584), (18944, 3584)])
@pytest.mark.parametrize("m", [1, 8, 64])
def test_qwen_projections_with_bias(n, k, m):
    from uniql_b200 import ops
    layer = quantized_layer(n + 3 * k + m, n, k, bias=True)
    x = make_acts(m + 11, m, k)
    y = ops.w4a16_linear(x.cuda(), torch.from_numpy(layer["packed"]).cuda(), torch.from_numpy(layer["scales"]).cuda(),
                         torch.from_numpy(layer["bias"]).cuda(), n).cpu().numpy()
    linear_tolerance_check(y, orc.linear_ref(x.numpy(), None, None, layer["bias"], n, w_deq=layer["w_deq"]))


@pytest.mark.parametrize("m", [1, 8, 64])
def test_qwen_lm_head_full_width_checked_on_column_slices(m):
    """152064 x 3584 with random codes; the oracle dequantises three 256-column slices (plain slices of the packed
    layout) and the matching output columns are compared."""
    from uniql_b200 import ops
    n, k = 152064, 3584
    g = torch.Generator(device="cuda").manual_seed(3)
    packed = torch.randint(-2 ** 31, 2 ** 31 - 1, (k // 16, 2 * n), dtype=torch.int64, device="cuda", generator=g).to(torch.int32)
    scales = (torch.rand(k // 128, n, device="cuda", generator=g) * 0.01 + 0.002).half()
    x = make_acts(m + 5, m, k)
    y = ops.w4a16_linear(x.cuda(), packed, scales, None, n).cpu().numpy()
    assert np.isfinite(y).all()
    for n0 in (0, 75776, n - 256):
        w = orc.dequantize(packed[:, 2 * n0:2 * n0 + 512].cpu().numpy(), scales[:, n0:n0 + 256].cpu().numpy())
        linear_tolerance_check(y[:, n0:n0 + 256], orc.linear_ref(x.numpy(), None, None, None, 256, w_deq=w))


@pytest.mark.parametrize("m", [1, 16, 300])
def test_mamba_out_proj_with_8192_point_hadamard(m):
    from uniql_b200.quantize.quant_linear_layers import W4A16B16O16HadLinear
    lin = torch.nn.Linear(8192, 4096, bias=False).half()
    q = W4A16B16O16HadLinear.from_fp16(lin).cuda()
    assert isinstance(q, W4A16B16O16HadLinear)
    x = make_acts(m + 1, m, 8192)
    y = q(x.cuda()).cpu().numpy()
    xh = orc.hadamard_transform(x.double().numpy()).astype(np.float16)
    w = orc.dequantize(q.weight.cpu().numpy(), q.scale.cpu().numpy())
    linear_tolerance_check(y, orc.linear_ref(xh, None, None, None, 4096, w_deq=w))


@pytest.mark.parametrize("m", [16, 2048])
def test_mamba_in_proj_padded_width(m):
    from uniql_b200 import ops
    layer = quantized_layer(4, 18560, 4096)
    assert layer["n_pad"] == 18688
    x = make_acts(m, m, 4096)
    y = ops.w4a16_linear(x.cuda(), torch.from_numpy(layer["packed"]).cuda(), torch.from_numpy(layer["scales"]).cuda(),
                         None, 18560).cpu().numpy()
    rows = np.unique(np.linspace(0, m - 1, 24).astype(int))
    linear_tolerance_check(y[rows], orc.linear_ref(x.numpy()[rows], None, None, None, 18560, w_deq=layer["w_deq"]))


def test_uniql_sliced_llama_head_dim_shapes():
    """UniQL prunes head_dim (128 -> 112): q 3584, k/v 896 (stored 1024), o 4096 x 3584."""
    from uniql_b200 import ops
    for n, k, m in [(896, 4096, 1), (896, 4096, 16), (896, 4096, 2048), (4096, 3584, 2048)]:
        layer = quantized_layer(n + k, n, k)
        x = make_acts(m + 2, m, k)
        y = ops.w4a16_linear(x.cuda(), torch.from_numpy(layer["packed"]).cuda(),
                             torch.from_numpy(layer["scales"]).cuda(), None, n).cpu().numpy()
        rows = np.unique(np.linspace(0, m - 1, 16).astype(int))
        linear_tolerance_check(y[rows], orc.linear_ref(x.numpy()[rows], None, None, None, n, w_deq=layer["w_deq"]))


def test_tensor_parallel_shards_on_one_gpu_reproduce_the_full_layer():
    """All ranks' shards evaluated on one device: concatenated column shards and summed row shards equal the
    unsharded result (8 ranks, Qwen's uneven 148-group down projection)."""
    from uniql_b200 import tp
    from uniql_b200.quantize.quant_linear_layers import W4A16B16O16Linear
    world = 8
    up = W4A16B16O16Linear.from_fp16(torch.nn.Linear(512, 18944, bias=True).half()).cuda()
    down = W4A16B16O16Linear.from_fp16(torch.nn.Linear(18944, 512, bias=True).half()).cuda()
    x = make_acts(9, 4, 512).cuda()
    h_full = up(x)
    y_full = down(h_full)
    cols = [tp.ColumnParallelW4A16Linear(up, r, world) for r in range(world)]
    h = torch.cat([c(x) for c in cols], dim=-1)
    assert torch.equal(h, h_full)
    parts = []
    for r in range(world):
        rp = tp.RowParallelW4A16Linear(down, r, world)
        parts.append(rp.local(h_full[:, rp.k0:rp.k1]).float())      # the partial sum, before any collective
    y = torch.stack(parts).sum(0) + down.bias.float()
    assert torch.allclose(y, y_full.float(), rtol=2e-2, atol=2e-2 * float(y_full.float().abs().max()))
