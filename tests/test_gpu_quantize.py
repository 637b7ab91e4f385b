"""GPU: RTN group-128 quantiser + packer, bit-exact against the oracle and the host path, through the C ABI."""
import numpy as np
import pytest
import torch

from oracle import uniql_oracle as orc

pytestmark = pytest.mark.gpu


def _weight(seed, n_out, k_in, std=0.02):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(n_out, k_in, generator=g) * std).to(torch.float16)


def _gpu(w, group_scale=None, n_pad=None, want_ref=True):
    from uniql_b200 import ops
    out = ops.w4a16_quantize(w, group_scale, n_pad=n_pad, want_ref=want_ref)
    torch.cuda.synchronize()
    return [None if t is None else t.cpu().numpy() for t in out]


def _bits(a):
    return np.ascontiguousarray(a).view(np.uint16)


@pytest.mark.parametrize("n_out,k_in", [(256, 256), (200, 384), (64, 200), (1000, 1024), (328, 512), (4096, 1024),
                                        (192, 129), (512, 4096)])
def test_rtn_bit_exact_against_oracle(n_out, k_in):
    w = _weight(n_out * 3 + k_in, n_out, k_in)
    w[5 % n_out, :] = 0                                   # an all-zero column: scale 0, code 0 in every group
    if k_in > 128:
        w[:, 128:256][7 % n_out] = 0                      # one all-zero group in another column
    pad_out = (256 - n_out % 256) % 256
    ref, packed, scales = orc.w4a16_quantize(np.ascontiguousarray(w.numpy().T), pad_out)
    got_ref, got_packed, got_scales = _gpu(w.cuda())
    assert got_packed.shape == packed.shape and np.array_equal(got_packed, packed)
    assert got_scales.shape == scales.shape and np.array_equal(_bits(got_scales), _bits(scales))
    assert got_ref.shape == ref.shape and np.array_equal(_bits(got_ref), _bits(ref))


def test_strided_rows_other_dtype_and_no_reference_output():
    big = _weight(3, 300, 1000)
    w = big[:, 8:648]                                      # row stride 1000, first element 16 bytes into the row
    pad_out = (256 - 300 % 256) % 256
    _, packed, scales = orc.w4a16_quantize(np.ascontiguousarray(w.numpy().T), pad_out)
    ref, got_packed, got_scales = _gpu(big.cuda()[:, 8:648], want_ref=False)
    assert ref is None
    assert np.array_equal(got_packed, packed) and np.array_equal(_bits(got_scales), _bits(scales))
    # rows starting 2 bytes off a 16-byte boundary take the element-wise loads
    w2 = big[:, 1:513]
    _, packed2, scales2 = orc.w4a16_quantize(np.ascontiguousarray(w2.numpy().T), pad_out)
    _, got2, gs2 = _gpu(big.cuda()[:, 1:513], want_ref=False)
    assert np.array_equal(got2, packed2) and np.array_equal(_bits(gs2), _bits(scales2))
    # fp32 input is rounded to fp16 first, as from_fp16 does
    _, got3, gs3 = _gpu(w.float().cuda(), want_ref=False)
    assert np.array_equal(got3, packed) and np.array_equal(_bits(gs3), _bits(scales))


@pytest.mark.parametrize("n_out,k_in", [(256, 512), (200, 384)])
def test_given_scales_match_the_host_path(n_out, k_in):
    """The GPTQ hand-over: weights already on the grid of the supplied scales (quantize_helpers.py:205-218)."""
    from uniql_b200.quantize import quantize_helpers as qh
    w = _weight(n_out + k_in, n_out, k_in)
    w_ref, _, scale_nat = orc.rtn_quantize_g128(np.ascontiguousarray(w.numpy().T))
    w_fake = torch.from_numpy(np.ascontiguousarray(w_ref[:k_in].T))          # [n_out, k_in], on the grid
    gscale = torch.from_numpy(scale_nat)                                     # [groups, n_out]
    pad_out = (256 - n_out % 256) % 256
    want_ref, want_packed, want_scales = qh.w4a16_quantize(w_fake.t().contiguous(), 4, 128, gscale, pad_out=pad_out)
    got_ref, got_packed, got_scales = _gpu(w_fake.cuda(), gscale.cuda())
    assert np.array_equal(got_packed, want_packed.numpy())
    assert np.array_equal(_bits(got_scales), _bits(want_scales.numpy()))
    assert np.array_equal(_bits(got_ref), _bits(want_ref.numpy()))


def test_from_fp16_on_the_gpu_equals_the_host_path_and_runs():
    from uniql_b200.quantize.quant_linear_layers import W4A16B16O16Linear
    lin = torch.nn.Linear(640, 328, bias=True).half()
    q_cpu = W4A16B16O16Linear.from_fp16(lin)
    q_gpu = W4A16B16O16Linear.from_fp16(lin.cuda())
    assert (q_gpu.size_k, q_gpu.size_n, q_gpu.pad_in, q_gpu.pad_out) == (q_cpu.size_k, q_cpu.size_n, q_cpu.pad_in,
                                                                        q_cpu.pad_out)
    assert torch.equal(q_gpu.weight.cpu(), q_cpu.weight) and torch.equal(q_gpu.scale.cpu(), q_cpu.scale)
    x = torch.randn(3, 640).half().cuda()
    y = q_gpu(x)
    y2 = q_cpu.cuda()(x)
    assert torch.equal(y, y2)


def test_bad_arguments_are_refused():
    from uniql_b200 import ops
    from uniql_b200._lib import UniqlError
    w = _weight(1, 128, 256).cuda()
    with pytest.raises(UniqlError):
        ops.w4a16_quantize(w, n_pad=100)                   # not a multiple of 64
    with pytest.raises(UniqlError):
        ops.w4a16_quantize(w, n_pad=64)                    # smaller than out_features
    with pytest.raises(RuntimeError):
        ops.w4a16_quantize(w, torch.zeros(3, 128, device="cuda", dtype=torch.float16))   # wrong scale shape


def test_full_size_gate_projection_properties():
    """14336 x 4096 (the bench's gate projection): properties that need no CPU-sized oracle run.  Every weight lies
    within half a quantisation step of its dequantised value, scales follow max|w| * 2/15, and a decode-size product
    through the linear kernel agrees with the fp16 weights within the quantisation noise."""
    from uniql_b200 import ops
    from uniql_b200.quantize import quantize_helpers as qh
    n, k = 14336, 4096
    g = torch.Generator(device="cuda").manual_seed(5)
    w = (torch.randn(n, k, generator=g, device="cuda") * 0.02).to(torch.float16)
    w_ref, packed, scales = ops.w4a16_quantize(w, n_pad=n)
    assert packed.shape == (k // 16, 2 * n) and scales.shape == (k // 128, n) and w_ref.shape == (k, n)
    nat = qh.unpermute_group_scales(scales)                                       # [groups, n]
    want = (w.t().reshape(k // 128, 128, n).abs().amax(dim=1).float() * (2.0 / 15.0)).to(torch.float16)
    assert torch.equal(nat, want)
    step = nat.float().repeat_interleave(128, dim=0)                              # [k, n]
    err = (w_ref.float() - w.t().float()).abs()
    # half a step, plus the fp16 roundings of w / s (|w / s| <= 7.5) and of w_ref itself
    assert bool((err <= 0.52 * step + 1e-8).all())
    codes = torch.round(w_ref.float() / step.clamp_min(1e-30)) + 8
    assert float(codes.min()) >= 0 and float(codes.max()) <= 15
    # the packed buffers drive the linear kernel to the same result as the reference weights
    x = (torch.randn(4, k, generator=g, device="cuda")).to(torch.float16)
    y = ops.w4a16_linear(x, packed, scales, None, n)
    y_ref = x.float() @ w_ref.float()
    assert float((y.float() - y_ref).abs().max() / y_ref.abs().max()) <= 1e-2    # the linear path's tolerance
