"""Load-time slicing of packed W4A16 layers for UniQL's elastic (pruned) checkpoints.

Same function names, arguments and results as modeling/modeling_helpers.py:361-867 of the reference
(`slice_w4a16_{up_gate,down,qk,v,o,in,out}_proj`, `slice_indices`, `get_topk_head_indices`,
`get_topk_ssm_state_indices`).  The reference writes each of them as unpack -> slice -> repack with Python loops on the
CPU; here they reduce to two primitives that run wherever the tensors live:

* `_select_columns`: keep a list of output columns of a packed layer (codes and scales), re-pad to the kernel's
  column granularity.  A column prefix on a 64-column boundary is a plain slice of the packed buffers.
* `_requantize_rows`: dequantise, keep a list of input rows, quantise again with fresh RTN scales (the reference does
  exactly this for o_proj / out_proj, :632-650 and :845-862).
On a GPU both are hand-written kernels working on the packed buffers (`uniql_w4a16_gather_columns`,
`uniql_w4a16_dequantize_rows` + `uniql_w4a16_quantize`); on the CPU they use the host packers.

Results are bit-identical to the reference's (tests/test_slicing.py against fixtures made by running the reference).
"""
from __future__ import annotations

import math

import torch

from .quantize.quantize_helpers import (MARLIN_QQQ_MAX_PARALLEL, MARLIN_QQQ_MIN_THREAD_N, get_w4a16_permute_weights,
                                        get_w4a16_weight_perms, permute_group_scales,
                                        unpack_w4a16_permute_weights, unpermute_group_scales, w4a16_quantize)

GROUP = 128


def _round_up(v: int, m: int) -> int:
    return (v + m - 1) // m * m


def _check(num_bits, group_size):
    assert num_bits == 4, "Only support 4-bit quantization for now"
    assert group_size in [-1, 128], "Only support group_size of -1 or 128 for now"


# ----------------------------------------------------------------------------------------------- index helpers
def get_topk_head_indices(n_groups, num_heads, head_dim, topk_head_dim):
    """First `topk_head_dim` channels of every head, heads in group-major order (modeling_helpers.py:124-130)."""
    heads = torch.arange(num_heads) * head_dim
    return (heads.unsqueeze(-1) + torch.arange(topk_head_dim).unsqueeze(0)).reshape(-1)


def get_topk_ssm_state_indices(n_groups, ssm_state_size, topk_ssm_state):
    """First `topk_ssm_state` states of every group (modeling_helpers.py:132-137)."""
    base = torch.arange(n_groups) * ssm_state_size
    return (base.unsqueeze(-1) + torch.arange(topk_ssm_state).unsqueeze(0)).reshape(-1)


def _rotary_half_indices(nheads, head_dim, reduced_head_dim):
    """Per head, the first reduced/2 channels of each rotary half (modeling_helpers.py:481-485)."""
    half, hd_half = head_dim // 2, reduced_head_dim // 2
    within = torch.cat([torch.arange(hd_half), half + torch.arange(hd_half)])
    return (torch.arange(nheads).unsqueeze(-1) * head_dim + within.unsqueeze(0)).reshape(-1)


def slice_indices(indices, head_dim, reduced_head_dim):
    """modeling_helpers.py:658-662."""
    half, hd_half = head_dim // 2, reduced_head_dim // 2
    return torch.cat([indices[:, :hd_half], indices[:, half:half + hd_half]], dim=-1).to(torch.uint8)


def _workspace(workspace, size_n):
    return workspace[:(size_n // MARLIN_QQQ_MIN_THREAD_N) * MARLIN_QQQ_MAX_PARALLEL].contiguous()


# ----------------------------------------------------------------------------------------------- primitives
def _codes(weight, size_k, size_n):
    return unpack_w4a16_permute_weights(weight, size_k, size_n, 4, get_w4a16_weight_perms(), GROUP)


def _pack(q_w):
    size_k, size_n = q_w.shape
    return get_w4a16_permute_weights(q_w, size_k, size_n, 4, get_w4a16_weight_perms(), GROUP).contiguous()


def _select_columns(weight, scale, size_k, real_k, col_index, zero_rows_past_real_k):
    """Packed layer [size_k, *] -> packed layer with the columns `col_index` (a 1-D long tensor of source columns),
    zero-padded to a multiple of 256 columns.  Rows >= real_k become code 0 when `zero_rows_past_real_k` (the
    reference strips the k padding before slicing and pads with zeros afterwards)."""
    dev = weight.device
    n_src = weight.shape[1] // 2
    n_new = col_index.numel()
    n_pad = _round_up(n_new, 256)
    if weight.is_cuda:
        from . import ops
        packed, new_scale = ops.w4a16_gather_columns(weight, scale, col_index, n_pad,
                                                     real_k if zero_rows_past_real_k else None)
        return packed, new_scale, n_pad
    col_index = col_index.to(dev)
    q = _codes(weight, size_k, n_src)[:, col_index]
    if zero_rows_past_real_k and real_k < size_k:
        q = q.clone()
        q[real_k:] = 0
    q = torch.nn.functional.pad(q, (0, n_pad - n_new), "constant", 0)
    s = unpermute_group_scales(scale)[:, col_index]
    s = torch.nn.functional.pad(s, (0, n_pad - n_new), "constant", 0)
    return _pack(q.contiguous()), permute_group_scales(s.contiguous()).contiguous(), n_pad


def _requantize_rows(weight, scale, size_k, hidden_size, row_index, pad_n):
    """Dequantise, keep the input rows `row_index`, quantise again with new RTN scales (fp16 arithmetic as in
    modeling_helpers.py:632-650)."""
    dev = weight.device
    n_src = weight.shape[1] // 2
    if weight.is_cuda:
        from . import ops
        w_nk = ops.w4a16_dequantize_rows(weight, scale, row_index, hidden_size)      # [hidden, rows kept]
        _, packed, new_scale = ops.w4a16_quantize(w_nk, None, n_pad=hidden_size + pad_n, want_ref=False)
        return packed, new_scale
    q = _codes(weight, size_k, n_src)[:, :hidden_size]
    s = unpermute_group_scales(scale)[:, :hidden_size]
    w = (q.to(s.dtype) - 8).reshape(s.shape[0], GROUP, hidden_size) * s.unsqueeze(1)
    w = w.reshape(-1, hidden_size)[row_index.to(dev)].contiguous()          # [rows kept, hidden]
    _, packed, new_scale = w4a16_quantize(w, 4, GROUP, None, pad_out=pad_n)
    return packed, new_scale


# ----------------------------------------------------------------------------------------------- the slicers
def slice_w4a16_up_gate_proj(weight, scale, workspace, hidden_size, intermediate_size, reduced_intermediate_size,
                             load_shape, num_bits=4, group_size=128):
    """modeling_helpers.py:361-408: keep the first `reduced` output columns.  The kept width is a multiple of 256,
    so the packed buffers are sliced in place; the scales of the columns between `reduced` and the padded width are
    zeroed (their codes are kept, as in the reference)."""
    _check(num_bits, group_size)
    assert load_shape[0] == weight.shape[0], "hidden_size dimension mismatch"
    width = _round_up(reduced_intermediate_size, 256)
    assert weight.shape[1] // 2 >= width, "Reduced size shape exceeds recovered weight"
    packed = weight[:, :2 * width].contiguous()
    s = unpermute_group_scales(scale[:, :width].contiguous())
    s[:, reduced_intermediate_size:] = 0
    return packed, permute_group_scales(s).contiguous(), _workspace(workspace, width)


def slice_w4a16_down_proj(weight, scale, workspace, hidden_size, intermediate_size, reduced_intermediate_size,
                          load_shape, num_bits=4, group_size=128):
    """modeling_helpers.py:411-448: keep the first `reduced` input rows, rounded up to whole groups — a plain slice
    of packed rows (16 k per row) and scale rows (128 k per row)."""
    _check(num_bits, group_size)
    assert load_shape[1] == weight.shape[1], "hidden_size dimension mismatch"
    rows = _round_up(reduced_intermediate_size, GROUP)
    assert weight.shape[0] * 16 >= rows, "Reduced size shape exceeds recovered weight"
    return (weight[:rows // 16].contiguous(), scale[:int(math.ceil(reduced_intermediate_size / 128))].contiguous(),
            workspace)


def slice_w4a16_qk_proj(weight, bias, scale, workspace, hidden_size, nheads, head_dim, reduced_head_dim, load_shape,
                        num_bits=4, group_size=128):
    """modeling_helpers.py:451-530: per head keep the leading channels of both rotary halves."""
    _check(num_bits, group_size)
    assert load_shape[0] == weight.shape[0], "hidden_size dimension mismatch"
    idx = _rotary_half_indices(nheads, head_dim, reduced_head_dim)
    size_k = _round_up(hidden_size, GROUP)
    packed, new_scale, n_pad = _select_columns(weight, scale, size_k, hidden_size, idx, True)
    new_bias = bias[idx.to(bias.device)] if bias is not None else None
    return packed, new_bias, new_scale, _workspace(workspace, n_pad)


def slice_w4a16_v_proj(weight, scale, workspace, hidden_size, nheads, head_dim, reduced_head_dim, load_shape,
                       num_bits=4, group_size=128):
    """modeling_helpers.py:533-596: per head keep the first `reduced_head_dim` channels."""
    _check(num_bits, group_size)
    assert load_shape[0] == weight.shape[0], "hidden_size dimension mismatch"
    idx = get_topk_head_indices(1, nheads, head_dim, reduced_head_dim)
    size_k = _round_up(hidden_size, GROUP)
    packed, new_scale, n_pad = _select_columns(weight, scale, size_k, hidden_size, idx, True)
    return packed, new_scale, _workspace(workspace, n_pad)


def slice_w4a16_o_proj(weight, scale, workspace, hidden_size, nheads, head_dim, reduced_head_dim, load_shape,
                       num_bits=4, group_size=128):
    """modeling_helpers.py:600-655: per head keep the first `reduced_head_dim` input rows; the groups of 128 rows
    change, so the layer is dequantised and quantised again."""
    _check(num_bits, group_size)
    assert load_shape[1] == weight.shape[1], "hidden_size dimension mismatch"
    size_k = _round_up(nheads * head_dim, GROUP)
    pad_n = _round_up(hidden_size, 256) - hidden_size
    idx = get_topk_head_indices(1, nheads, head_dim, reduced_head_dim)
    packed, new_scale = _requantize_rows(weight, scale, size_k, hidden_size, idx, pad_n)
    return packed, new_scale, workspace


def slice_w4a16_in_proj(weight, scale, workspace, hidden_size, n_groups, num_heads, intermediate_size, ssm_state_size,
                        load_intermediate_size, load_ssm_state_size, load_shape, num_bits=4, group_size=128):
    """modeling_helpers.py:665-767 (Mamba2 in_proj = z | x | B | C | dt): leading channels of every head for z and
    x, leading states of every group for B and C, dt whole."""
    _check(num_bits, group_size)
    assert load_shape[0] == weight.shape[0], "hidden_size dimension mismatch"
    head_dim = intermediate_size // num_heads
    heads = get_topk_head_indices(n_groups, num_heads, head_dim, load_intermediate_size // num_heads)
    states = get_topk_ssm_state_indices(n_groups, ssm_state_size, load_ssm_state_size)
    x0 = intermediate_size
    b0 = 2 * intermediate_size
    c0 = b0 + n_groups * ssm_state_size
    dt0 = c0 + n_groups * ssm_state_size
    idx = torch.cat([heads, x0 + heads, b0 + states, c0 + states, dt0 + torch.arange(num_heads)])
    size_k = _round_up(hidden_size, GROUP)
    packed, new_scale, n_pad = _select_columns(weight, scale, size_k, hidden_size, idx, True)
    return packed, new_scale, _workspace(workspace, n_pad)


def slice_w4a16_out_proj(weight, scale, workspace, hidden_size, n_groups, num_heads, intermediate_size,
                         load_intermediate_size, load_shape, num_bits=4, group_size=128):
    """modeling_helpers.py:809-867 (Mamba2 out_proj): leading channels of every head on the input side,
    dequantise and quantise again."""
    _check(num_bits, group_size)
    assert load_shape[1] == weight.shape[1], "hidden_size dimension mismatch"
    size_k = _round_up(intermediate_size, GROUP)
    pad_n = _round_up(hidden_size, 256) - hidden_size
    head_dim = intermediate_size // num_heads
    idx = get_topk_head_indices(n_groups, num_heads, head_dim, load_intermediate_size // num_heads)
    packed, new_scale = _requantize_rows(weight, scale, size_k, hidden_size, idx, pad_n)
    return packed, new_scale, workspace


def slice_conv1d(weight, bias, n_groups, num_heads, intermediate_size, ssm_state_size, load_intermediate_size,
                 load_ssm_state_size):
    """modeling_helpers.py:770-797 (Mamba2 conv1d over x | B | C): the channels that in_proj keeps."""
    head_dim = intermediate_size // num_heads
    heads = get_topk_head_indices(n_groups, num_heads, head_dim, load_intermediate_size // num_heads)
    states = get_topk_ssm_state_indices(n_groups, ssm_state_size, load_ssm_state_size)
    b0 = intermediate_size
    c0 = b0 + n_groups * ssm_state_size
    idx = torch.cat([heads, b0 + states, c0 + states]).to(weight.device)
    return weight[idx].contiguous(), bias[idx].contiguous()


def slice_norm(weight, n_groups, num_heads, intermediate_size, load_intermediate_size):
    """modeling_helpers.py:800-806 (gated RMSNorm weight): the channels that in_proj keeps."""
    head_dim = intermediate_size // num_heads
    idx = get_topk_head_indices(n_groups, num_heads, head_dim, load_intermediate_size // num_heads)
    return weight[idx.to(weight.device)].contiguous()


# ----------------------------------------------------------------------------------------------- checkpoint walker
def _put(loaded, key, names, values):
    for name, value in zip(names, values):
        if value is not None:
            loaded[f"{key}.{name}"] = value


def slice_quantized_weights(model, model_helper, loaded_model):
    """Applies the slicers above to a loaded full-size state dict, layer by layer, so that it fits an elastic
    (reduced-width) model -- the walker of modeling/modeling_helpers.py:235-358, same arguments and result.

    `model_helper` names the quantised block classes (`mlp_w4a16_uniql_class_name`, `attn_w4a16_uniql_class_name`,
    `mamba_w4a16_uniql_class_name`) and the state-dict prefixes (`get_mlp_key`, `get_attn_key`, `get_mamba_key`,
    `get_layers`); the reduced sizes are read from the model's own modules.  `loaded_model` is modified in place and
    returned; tensors stay on the device they are on (GPU tensors are sliced by the CUDA kernels)."""
    cfg = model.config
    wsw = ("weight", "scale", "workspace")
    for layer_idx, layer in enumerate(model_helper.get_layers(model)):
        for _, module in layer.named_children():
            cls = module.__class__.__name__
            if cls == model_helper.mlp_w4a16_uniql_class_name:
                key = model_helper.get_mlp_key(layer_idx)
                for name in ("up_proj", "gate_proj"):
                    k = f"{key}.{name}"
                    if k + ".weight" not in loaded_model:        # blocks without a gate projection
                        continue
                    _put(loaded_model, k, wsw, slice_w4a16_up_gate_proj(
                        *(loaded_model[f"{k}.{n}"] for n in wsw), cfg.hidden_size, cfg.intermediate_size,
                        module.intermediate_size, getattr(module, name).weight.shape))
                k = f"{key}.down_proj"
                _put(loaded_model, k, wsw, slice_w4a16_down_proj(
                    *(loaded_model[f"{k}.{n}"] for n in wsw), cfg.hidden_size, cfg.intermediate_size,
                    module.intermediate_size, module.down_proj.weight.shape))
            elif cls == model_helper.attn_w4a16_uniql_class_name:
                key = model_helper.get_attn_key(layer_idx)
                head_dim = getattr(cfg, "head_dim", cfg.hidden_size // cfg.num_attention_heads)
                for name, heads in (("q_proj", cfg.num_attention_heads), ("k_proj", cfg.num_key_value_heads)):
                    k = f"{key}.{name}"
                    w, b, s, ws = slice_w4a16_qk_proj(
                        loaded_model[k + ".weight"], loaded_model.get(k + ".bias"), loaded_model[k + ".scale"],
                        loaded_model[k + ".workspace"], cfg.hidden_size, heads, head_dim, module.head_dim,
                        getattr(module, name).weight.shape)
                    _put(loaded_model, k, ("weight", "bias", "scale", "workspace"), (w, b, s, ws))
                k = f"{key}.v_proj"
                _put(loaded_model, k, wsw, slice_w4a16_v_proj(
                    *(loaded_model[f"{k}.{n}"] for n in wsw), cfg.hidden_size, cfg.num_key_value_heads, head_dim,
                    module.head_dim, module.v_proj.weight.shape))
                k = f"{key}.o_proj"
                _put(loaded_model, k, wsw, slice_w4a16_o_proj(
                    *(loaded_model[f"{k}.{n}"] for n in wsw), cfg.hidden_size, cfg.num_attention_heads, head_dim,
                    module.head_dim, module.o_proj.weight.shape))
                if f"{key}.indices" in loaded_model:
                    loaded_model[f"{key}.indices"] = slice_indices(loaded_model[f"{key}.indices"], head_dim, module.head_dim)
            elif cls == model_helper.mamba_w4a16_uniql_class_name:
                key = model_helper.get_mamba_key(layer_idx)
                full_inter = model_helper.get_mamba_full_intermediate_size
                full_state = model_helper.get_mamba_full_ssm_state_size
                k = f"{key}.in_proj"
                _put(loaded_model, k, wsw, slice_w4a16_in_proj(
                    *(loaded_model[f"{k}.{n}"] for n in wsw), hidden_size=cfg.hidden_size, n_groups=module.n_groups,
                    num_heads=module.num_heads, intermediate_size=full_inter, ssm_state_size=full_state,
                    load_intermediate_size=module.intermediate_size, load_ssm_state_size=module.ssm_state_size,
                    load_shape=module.in_proj.weight.shape))
                k = f"{key}.conv1d"
                _put(loaded_model, k, ("weight", "bias"), slice_conv1d(
                    loaded_model[k + ".weight"], loaded_model[k + ".bias"], module.n_groups, module.num_heads, full_inter,
                    full_state, module.intermediate_size, module.ssm_state_size))
                k = f"{key}.norm"
                loaded_model[k + ".weight"] = slice_norm(loaded_model[k + ".weight"], module.n_groups, module.num_heads,
                                                         full_inter, module.intermediate_size)
                k = f"{key}.out_proj"
                _put(loaded_model, k, wsw, slice_w4a16_out_proj(
                    *(loaded_model[f"{k}.{n}"] for n in wsw), hidden_size=cfg.hidden_size, n_groups=module.n_groups,
                    num_heads=module.num_heads, intermediate_size=full_inter,
                    load_intermediate_size=module.intermediate_size, load_shape=module.out_proj.weight.shape))
    return loaded_model
