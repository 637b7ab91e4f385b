"""Load-time slicing of packed layers (uniql_b200.modeling_helpers) against fixtures made by running the reference's
own functions (tests/golden/make_golden.py, make_slicing) on the same seeded layers.  CPU; bit-exact."""
import os

import numpy as np
import pytest
import torch

from uniql_b200 import modeling_helpers as mh
from uniql_b200.quantize import quantize_helpers as qh


@pytest.fixture(scope="module")
def gold(golden_dir):
    return np.load(os.path.join(golden_dir, "slicing.npz"))


ORDER = ["up", "down", "qk", "v", "o", "in", "out"]
HIDDEN, INTER, RED = 256, 384, 320
NHEADS, HD, RHD = 3, 64, 48
NG, NH, INTER2, STATE, LINTER, LSTATE = 2, 4, 256, 32, 192, 24


def _layer(gold, tag):
    seed, out_f, in_f = (int(v) for v in gold["inputs_seed_out_in"][ORDER.index(tag)])
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(out_f, in_f, generator=g) * 0.02).to(torch.float16)
    assert int(w.numpy().view(np.uint16).astype(np.int64).sum()) == int(gold[tag + "_w_sum"]), \
        "the seeded generator no longer reproduces the fixture's input"
    pad_out = (256 - out_f % 256) % 256
    _, packed, scale = qh.w4a16_quantize(w.t().contiguous(), 4, 128, None, pad_out)
    ws = torch.zeros((out_f + pad_out) // 64 * 16, dtype=torch.int32)
    return packed, scale, ws


def _same(got, want):
    got = got.cpu().numpy()
    assert got.shape == want.shape and got.dtype == want.dtype
    if got.dtype == np.float16:
        assert np.array_equal(got.view(np.uint16), want.view(np.uint16))
    else:
        assert np.array_equal(got, want)


def _run(tag, packed, scale, ws, gold=None):
    if tag == "up":
        return mh.slice_w4a16_up_gate_proj(packed, scale, ws, HIDDEN, INTER, RED, packed.shape)
    if tag == "down":
        return mh.slice_w4a16_down_proj(packed, scale, ws, HIDDEN, INTER, RED, packed.shape)
    if tag == "qk":
        bias = torch.from_numpy(gold["qk_bias_in"]).to(packed.device)
        p, b, s, w = mh.slice_w4a16_qk_proj(packed, bias, scale, ws, HIDDEN, NHEADS, HD, RHD, packed.shape)
        return p, s, w, b
    if tag == "v":
        return mh.slice_w4a16_v_proj(packed, scale, ws, HIDDEN, NHEADS, HD, RHD, packed.shape)
    if tag == "o":
        return mh.slice_w4a16_o_proj(packed, scale, ws, HIDDEN, NHEADS, HD, RHD, packed.shape)
    if tag == "in":
        return mh.slice_w4a16_in_proj(packed, scale, ws, HIDDEN, NG, NH, INTER2, STATE, LINTER, LSTATE, packed.shape)
    return mh.slice_w4a16_out_proj(packed, scale, ws, HIDDEN, NG, NH, INTER2, LINTER, packed.shape)


@pytest.mark.parametrize("tag", ORDER)
def test_slicers_match_reference(gold, tag):
    packed, scale, ws = _layer(gold, tag)
    out = _run(tag, packed, scale, ws, gold)
    _same(out[0], gold[tag + "_packed"])
    _same(out[1], gold[tag + "_scale"])
    _same(out[2], gold[tag + "_ws"])
    if tag == "qk":
        _same(out[3], gold["qk_bias"])


def test_index_helpers_match_reference(gold):
    idx = torch.arange(NHEADS * HD).reshape(NHEADS, HD)
    _same(mh.slice_indices(idx, HD, RHD), gold["slice_indices"])
    _same(mh.get_topk_head_indices(NG, NH, INTER2 // NH, LINTER // NH), gold["topk_head"])
    _same(mh.get_topk_ssm_state_indices(NG, STATE, LSTATE), gold["topk_state"])


def test_conv1d_and_norm_slicers_match_reference(gold):
    conv_ch = INTER2 + 2 * NG * STATE
    g = torch.Generator().manual_seed(28)
    conv_w = (torch.randn(conv_ch, 4, generator=g) * 0.02).to(torch.float16).reshape(conv_ch, 1, 4)
    conv_b = torch.linspace(-1, 1, conv_ch).to(torch.float16)
    cw, cb = mh.slice_conv1d(conv_w, conv_b, NG, NH, INTER2, STATE, LINTER, LSTATE)
    _same(cw, gold["conv_w_out"])
    _same(cb, gold["conv_b_out"])
    _same(mh.slice_norm(torch.linspace(0, 1, INTER2).to(torch.float16), NG, NH, INTER2, LINTER), gold["norm_out"])


def test_sliced_layer_computes_the_sliced_product(gold):
    """A sliced v_proj gives, per head, the first RHD channels of the full layer's output (dequantised weights)."""
    packed, scale, ws = _layer(gold, "v")
    p2, s2, _ = mh.slice_w4a16_v_proj(packed, scale, ws, HIDDEN, NHEADS, HD, RHD, packed.shape)
    full = qh.w4a16_dequantize(packed, scale)[:HIDDEN, :NHEADS * HD].float()
    part = qh.w4a16_dequantize(p2, s2)[:HIDDEN, :NHEADS * RHD].float()
    want = full.reshape(HIDDEN, NHEADS, HD)[:, :, :RHD].reshape(HIDDEN, -1)
    assert torch.equal(part, want)


@pytest.mark.gpu
@pytest.mark.parametrize("tag", ORDER)
def test_slicers_on_the_gpu_match_reference(gold, tag):
    """Same functions with the tensors on the GPU (o / out re-quantise through uniql_w4a16_quantize)."""
    packed, scale, ws = _layer(gold, tag)
    out = _run(tag, packed.cuda(), scale.cuda(), ws.cuda(), gold)
    assert out[0].is_cuda and out[1].is_cuda
    _same(out[0], gold[tag + "_packed"])
    _same(out[1], gold[tag + "_scale"])
    _same(out[2], gold[tag + "_ws"])


@pytest.mark.gpu
@pytest.mark.parametrize("n,k,keep", [(320, 256, 200), (1000, 384, 777), (4096, 1024, 2500)])
def test_gather_and_dequantize_kernels_against_the_host_path(n, k, keep):
    """The two CUDA primitives on random index lists, against the unpack -> index -> repack path on the CPU."""
    from uniql_b200 import ops
    g = torch.Generator().manual_seed(n + k)
    w = (torch.randn(n, k, generator=g) * 0.02).to(torch.float16)
    _, packed, scale = qh.w4a16_quantize(w.t().contiguous(), 4, 128, None, (256 - n % 256) % 256)
    idx = torch.randperm(n, generator=g)[:keep]
    zero_from = k - 37
    want_p, want_s, n_pad = mh._select_columns(packed, scale, k, zero_from, idx, True)
    got_p, got_s = ops.w4a16_gather_columns(packed.cuda(), scale.cuda(), idx, n_pad, zero_from)
    assert torch.equal(got_p.cpu(), want_p) and torch.equal(got_s.cpu().view(torch.int16), want_s.view(torch.int16))
    holes = idx.clone()
    holes[::7] = -1                                            # negative entries give zero columns
    got_p2, got_s2 = ops.w4a16_gather_columns(packed.cuda(), scale.cuda(), holes, n_pad)
    codes = qh.unpack_w4a16_permute_weights(got_p2.cpu(), k, n_pad, 4, qh.get_w4a16_weight_perms(), 128)
    assert int(codes[:, :keep][:, ::7].abs().max()) == 0
    assert float(qh.unpermute_group_scales(got_s2.cpu())[:, :keep][:, ::7].abs().max()) == 0.0
    rows = torch.randperm(k, generator=g)[:k // 2 + 3]
    deq = qh.w4a16_dequantize(packed, scale)[:, :n]            # [Kp, n]
    want = deq[rows].t().contiguous()
    got = ops.w4a16_dequantize_rows(packed.cuda(), scale.cuda(), rows, n)
    assert torch.equal(got.cpu().view(torch.int16), want.view(torch.int16))


@pytest.mark.gpu
def test_out_of_range_indices_are_refused_and_flagged():
    """An index outside the source layer never reads out of bounds: the wrapper raises, and the kernels themselves
    (called through the C ABI without the wrapper's check) write zeros and raise a status bit."""
    from uniql_b200 import ops
    from uniql_b200._lib import lib
    n, k = 320, 256
    g = torch.Generator().manual_seed(1)
    w = (torch.randn(n, k, generator=g) * 0.02).to(torch.float16)
    _, packed, scale = qh.w4a16_quantize(w.t().contiguous(), 4, 128, None, (256 - n % 256) % 256)
    packed, scale = packed.cuda(), scale.cuda()
    n_src = scale.shape[1]
    with pytest.raises(RuntimeError):
        ops.w4a16_gather_columns(packed, scale, torch.tensor([0, n_src, 3]), 64)
    with pytest.raises(RuntimeError):
        ops.w4a16_dequantize_rows(packed, scale, torch.tensor([0, k, 3]), n)
    ops.read_and_clear_status("cuda")
    st = ops.status_word(torch.device("cuda", 0))
    idx = torch.tensor([5, n_src + 7, 9], dtype=torch.int32, device="cuda")
    out_p = torch.full((k // 16, 128), -1, dtype=torch.int32, device="cuda")
    out_s = torch.ones((k // 128, 64), dtype=torch.float16, device="cuda")
    assert lib().uniql_w4a16_gather_columns(packed.data_ptr(), scale.data_ptr(), k, n_src, idx.data_ptr(), 3, k,
                                            out_p.data_ptr(), out_s.data_ptr(), 64, st.data_ptr(), None) == 0
    assert ops.read_and_clear_status("cuda") == 4
    codes = qh.unpack_w4a16_permute_weights(out_p.cpu(), k, 64, 4, qh.get_w4a16_weight_perms(), 128)
    want = qh.unpack_w4a16_permute_weights(packed.cpu(), k, n_src, 4, qh.get_w4a16_weight_perms(), 128)
    assert torch.equal(codes[:, 0], want[:, 5]) and torch.equal(codes[:, 2], want[:, 9]) and int(codes[:, 1].abs().max()) == 0
    rows = torch.tensor([3, -2, k + 100, 7], dtype=torch.int32, device="cuda")
    deq = torch.full((n, 4), 9.0, dtype=torch.float16, device="cuda")
    assert lib().uniql_w4a16_dequantize_rows(packed.data_ptr(), scale.data_ptr(), k, n_src, rows.data_ptr(), 4, n,
                                             deq.data_ptr(), 4, st.data_ptr(), None) == 0
    assert ops.read_and_clear_status("cuda") == 4
    full = qh.w4a16_dequantize(packed.cpu(), scale.cpu())[:, :n]
    assert torch.equal(deq[:, 0].cpu(), full[3]) and torch.equal(deq[:, 3].cpu(), full[7])
    assert float(deq[:, 1:3].abs().max()) == 0.0


def test_host_path_raises_on_out_of_range_columns():
    g = torch.Generator().manual_seed(2)
    w = (torch.randn(192, 256, generator=g) * 0.02).to(torch.float16)
    _, packed, scale = qh.w4a16_quantize(w.t().contiguous(), 4, 128, None, 64)
    with pytest.raises(IndexError):
        mh._select_columns(packed, scale, 256, 256, torch.tensor([0, 999]), True)


def test_checkpoint_walker_applies_every_slicer(gold):
    """slice_quantized_weights (modeling/modeling_helpers.py:235-358) over a one-layer state dict with an MLP block and
    an attention block: every entry equals what the reference's slicers returned for that layer."""
    from types import SimpleNamespace as NS

    class UniqlMLP:            # stand-ins for the reference's quantised block classes: only names and sizes matter
        pass

    class UniqlAttention:
        pass

    def shaped(t):
        return NS(weight=NS(shape=t.shape))

    layers_in = {tag: _layer(gold, tag) for tag in ("up", "down", "qk", "v", "o")}
    mlp, attn = UniqlMLP(), UniqlAttention()
    mlp.intermediate_size = RED
    mlp.up_proj, mlp.gate_proj, mlp.down_proj = shaped(layers_in["up"][0]), shaped(layers_in["up"][0]), shaped(layers_in["down"][0])
    attn.head_dim = RHD
    attn.q_proj = attn.k_proj = shaped(layers_in["qk"][0])
    attn.v_proj, attn.o_proj = shaped(layers_in["v"][0]), shaped(layers_in["o"][0])
    layer = NS(named_children=lambda: [("mlp", mlp), ("self_attn", attn)])
    model = NS(config=NS(hidden_size=HIDDEN, intermediate_size=INTER, num_attention_heads=NHEADS,
                         num_key_value_heads=NHEADS, head_dim=HD))
    helper = NS(get_layers=lambda m: [layer], mlp_w4a16_uniql_class_name="UniqlMLP",
                attn_w4a16_uniql_class_name="UniqlAttention", mamba_w4a16_uniql_class_name="UniqlMamba",
                get_mlp_key=lambda i: f"model.layers.{i}.mlp", get_attn_key=lambda i: f"model.layers.{i}.self_attn")
    sd = {}
    for name, tag in (("mlp.up_proj", "up"), ("mlp.gate_proj", "up"), ("mlp.down_proj", "down"), ("self_attn.q_proj", "qk"),
                      ("self_attn.k_proj", "qk"), ("self_attn.v_proj", "v"), ("self_attn.o_proj", "o")):
        for part, t in zip(("weight", "scale", "workspace"), layers_in[tag]):
            sd[f"model.layers.0.{name}.{part}"] = t.clone()
    sd["model.layers.0.self_attn.q_proj.bias"] = torch.from_numpy(gold["qk_bias_in"])
    idx = torch.arange(NHEADS * HD, dtype=torch.int64).reshape(NHEADS, HD)
    sd["model.layers.0.self_attn.indices"] = idx.clone()
    out = mh.slice_quantized_weights(model, helper, sd)
    assert out is sd
    for name, tag in (("mlp.up_proj", "up"), ("mlp.gate_proj", "up"), ("mlp.down_proj", "down"), ("self_attn.q_proj", "qk"),
                      ("self_attn.k_proj", "qk"), ("self_attn.v_proj", "v"), ("self_attn.o_proj", "o")):
        _same(sd[f"model.layers.0.{name}.weight"], gold[tag + "_packed"])
        _same(sd[f"model.layers.0.{name}.scale"], gold[tag + "_scale"])
        _same(sd[f"model.layers.0.{name}.workspace"], gold[tag + "_ws"])
    _same(sd["model.layers.0.self_attn.q_proj.bias"], gold["qk_bias"])
    assert "model.layers.0.self_attn.k_proj.bias" not in sd
    assert torch.equal(sd["model.layers.0.self_attn.indices"], mh.slice_indices(idx, HD, RHD))


@pytest.mark.gpu
def test_llama_8b_sized_layers_sliced_on_the_gpu_keep_their_weights():
    """Llama-3.1-8B layers cut to the 85 % model (intermediate 14336 -> 12160, head_dim 128 -> 112), on the GPU.  At this
    size the CPU re-pack takes minutes, so the check is a property that holds at any size: dequantising a sliced layer
    gives, bit for bit, the kept rows and columns of the dequantised original (column slices keep codes and scales;
    the row slice of o_proj re-quantises, so there the sliced layer is compared with a second quantisation of the kept
    rows and its checksum with the checksum of the device-side quantiser run directly)."""
    from uniql_b200 import ops
    hidden, inter, red, nheads, nkv, hd, rhd = 4096, 14336, 12160, 32, 8, 128, 112
    gen = torch.Generator(device="cuda").manual_seed(85)

    def layer(n, k):
        w = (torch.randn(n, k, generator=gen, device="cuda") * 0.02).half()
        _, packed, scale = ops.w4a16_quantize(w, want_ref=False)
        return packed, scale, torch.zeros(packed.shape[1] // 2 // 64 * 16, dtype=torch.int32, device="cuda")

    def deq(packed, scale, n):
        k = packed.shape[0] * 16
        return ops.w4a16_dequantize_rows(packed, scale, torch.arange(k), n)          # fp16 [n, k]

    def same(a, b):
        return torch.equal(a.view(torch.int16), b.view(torch.int16))

    # gate / up: column prefix
    p, s, ws = layer(inter, hidden)
    p2, s2, ws2 = mh.slice_w4a16_up_gate_proj(p, s, ws, hidden, inter, red, p.shape)
    width = (red + 255) // 256 * 256                            # stored widths are multiples of 256
    assert p2.shape == (hidden // 16, 2 * width) and s2.shape == (hidden // 128, width) and ws2.numel() == width // 64 * 16
    assert same(deq(p2, s2, red), deq(p, s, inter)[:red])
    assert float(deq(p2, s2, width)[red:].abs().max()) == 0.0   # columns between 12160 and 12288: zero scales
    # down: row prefix
    p, s, ws = layer(hidden, inter)
    p2, s2, _ = mh.slice_w4a16_down_proj(p, s, ws, hidden, inter, red, p.shape)
    assert p2.shape == (red // 16, 2 * hidden) and s2.shape == (red // 128, hidden)
    assert same(deq(p2, s2, hidden), deq(p, s, hidden)[:, :red])
    # q (32 heads) and k (8 heads): leading channels of both rotary halves of every head
    for heads in (nheads, nkv):
        p, s, ws = layer(heads * hd, hidden)
        bias = torch.arange(heads * hd, device="cuda", dtype=torch.float16)
        p2, b2, s2, ws2 = mh.slice_w4a16_qk_proj(p, bias, s, ws, hidden, heads, hd, rhd, p.shape)
        idx = mh._rotary_half_indices(heads, hd, rhd).cuda()
        n_keep = heads * rhd
        n_pad = (n_keep + 255) // 256 * 256
        assert p2.shape == (hidden // 16, 2 * n_pad) and ws2.numel() == n_pad // 64 * 16
        assert same(deq(p2, s2, n_keep), deq(p, s, heads * hd)[idx]) and torch.equal(b2, bias[idx])
        if n_pad > n_keep:                                       # padded columns carry zero scales
            assert float(deq(p2, s2, n_pad)[n_keep:].abs().max()) == 0.0
    # v: first 112 channels of every head
    p, s, ws = layer(nkv * hd, hidden)
    p2, s2, _ = mh.slice_w4a16_v_proj(p, s, ws, hidden, nkv, hd, rhd, p.shape)
    idx = mh.get_topk_head_indices(1, nkv, hd, rhd).cuda()
    assert same(deq(p2, s2, nkv * rhd), deq(p, s, nkv * hd)[idx])
    # o: keep 112 of 128 input rows per head -> groups change -> dequantise, quantise again
    p, s, ws = layer(hidden, nheads * hd)
    p2, s2, _ = mh.slice_w4a16_o_proj(p, s, ws, hidden, nheads, hd, rhd, p.shape)
    idx = mh.get_topk_head_indices(1, nheads, hd, rhd).cuda()
    kept = deq(p, s, hidden)[:, idx].contiguous()                                    # fp16 [4096, 3584]
    _, want_p, want_s = ops.w4a16_quantize(kept, want_ref=False)
    assert p2.shape == (nheads * rhd // 16, 2 * hidden) and torch.equal(p2, want_p) and same(s2, want_s)
    assert int(p2.long().sum()) == int(want_p.long().sum())
    # re-quantising moves every weight by at most half a step of its new group scale (plus the fp16 roundings of the
    # scale and of w / scale: the group maximum sits at 7.5 steps and is clamped to 7)
    step = ops.w4a16_dequantize_rows(torch.full_like(p2, 0x99999999 - (1 << 32)), s2, torch.arange(nheads * rhd), hidden)
    assert bool(((deq(p2, s2, hidden).float() - kept.float()).abs() <= 0.52 * step.float().abs() + 1e-5).all())
    assert ops.read_and_clear_status("cuda") == 0
