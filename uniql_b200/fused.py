"""Block-level entry points that run what UniQL's decoder blocks issue as several launches in one.

The reference's blocks call their quantized linears one by one and glue them with elementwise kernels:
`down_proj(act_fn(gate_proj(x)) * up_proj(x))` (modeling/llama/llama_qblocks.py:48-51), three q/k/v linears
(:104-106), `residual + o_proj(...)`.  At decode sizes every one of those launches costs more than the bytes it
moves, so for up to 16 rows the functions below issue one grouped kernel (uniql_w4a16_linear_group) per step; up
to 128 rows the projections still share one launch (plain outputs, the elementwise maths in PyTorch); larger batches
run the same modules one after the other on the tensor-core kernels, exactly as the reference does it.  All take and return the tensors the reference's code would.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import ops

DECODE_ROWS = 16         # the decode kernel: SwiGLU, residual and Hadamard inside the launch
GROUP_ROWS = 128         # plain outputs of several projections in one launch (tensor-core kernel above 16 rows)


def _layer(mod):
    return (mod.weight, mod.scale, mod.bias, mod.out_features)


def _rows(x):
    return x.numel() // x.shape[-1] if x.shape[-1] else 0


def _flat(x, mod):
    x2 = x.reshape(-1, x.shape[-1])
    if mod.pad_in:
        x2 = F.pad(x2, (0, mod.pad_in), "constant", 0)
    return x2


def gate_up_swiglu(gate_proj, up_proj, x):
    """silu(gate_proj(x)) * up_proj(x) for two W4A16B16O16Linear modules of the same shape."""
    ext = ops.torch_ext()
    if ext is not None and _rows(x) <= GROUP_ROWS:
        fused_act = _rows(x) <= DECODE_ROWS
        out = ext.linear_group(x, [gate_proj.weight, up_proj.weight], [gate_proj.scale, up_proj.scale],
                               [gate_proj.bias, up_proj.bias], [gate_proj.out_features, up_proj.out_features],
                               1 if fused_act else 0, None, gate_proj.pad_in, False)
        return out[0] if fused_act else ext.silu_mul(out[0], out[1])
    x2 = _flat(x, gate_proj)
    if x2.shape[0] <= DECODE_ROWS:
        (h,) = ops.w4a16_linear_group(x2, [_layer(gate_proj), _layer(up_proj)], epilogue="swiglu")
    elif x2.shape[0] <= GROUP_ROWS:
        g, u = ops.w4a16_linear_group(x2, [_layer(gate_proj), _layer(up_proj)])
        h = ops.silu_mul(g, u)
    else:
        h = ops.silu_mul(gate_proj(x2), up_proj(x2))
    return h.view(*x.shape[:-1], gate_proj.out_features)


def qkv_proj(q_proj, k_proj, v_proj, x):
    """(q_proj(x), k_proj(x), v_proj(x)) for three W4A16B16O16Linear modules with the same in_features."""
    mods = (q_proj, k_proj, v_proj)
    ext = ops.torch_ext()
    if ext is not None and _rows(x) <= GROUP_ROWS:
        return tuple(ext.linear_group(x, [m.weight for m in mods], [m.scale for m in mods], [m.bias for m in mods],
                                      [m.out_features for m in mods], 0, None, q_proj.pad_in, False))
    x2 = _flat(x, q_proj)
    if x2.shape[0] <= GROUP_ROWS:
        outs = ops.w4a16_linear_group(x2, [_layer(m) for m in mods])
    else:
        outs = [m(x2) for m in mods]
    return tuple(o.view(*x.shape[:-1], m.out_features) for o, m in zip(outs, mods))


def linear_residual(proj, x, residual):
    """residual + proj(x) (o_proj / down_proj / out_proj with the block's skip connection); when `proj` is a
    W4A16B16O16HadLinear its Hadamard transform of x is part of the same call."""
    ext = ops.torch_ext()
    if ext is not None and _rows(x) <= DECODE_ROWS:
        return ext.linear_group(x, [proj.weight], [proj.scale], [proj.bias], [proj.out_features], 0, residual,
                                proj.pad_in, bool(getattr(proj, "hadamard_dim", 0)))[0].view(
                                    *residual.shape[:-1], proj.out_features)
    x2 = _flat(x, proj)
    r2 = residual.reshape(-1, residual.shape[-1])
    had = proj.size_k if getattr(proj, "hadamard_dim", 0) else 0
    if x2.shape[0] <= DECODE_ROWS and r2.stride(-1) == 1:
        (y,) = ops.w4a16_linear_group(x2, [_layer(proj)], residual=r2, hadamard_dim=had)
    else:
        y = r2 + proj(x2)
    return y.view(*residual.shape[:-1], proj.out_features)


class W4A16GateUp(torch.nn.Module):
    """Holds a block's gate_proj and up_proj and returns act_fn(gate) * up in one launch at decode sizes."""

    def __init__(self, gate_proj, up_proj):
        super().__init__()
        self.gate_proj, self.up_proj = gate_proj, up_proj

    def forward(self, x):
        return gate_up_swiglu(self.gate_proj, self.up_proj, x)


class W4A16QKV(torch.nn.Module):
    """Holds a block's q/k/v projections and returns the three results of one launch at decode sizes."""

    def __init__(self, q_proj, k_proj, v_proj):
        super().__init__()
        self.q_proj, self.k_proj, self.v_proj = q_proj, k_proj, v_proj

    def forward(self, x):
        return qkv_proj(self.q_proj, self.k_proj, self.v_proj, x)
