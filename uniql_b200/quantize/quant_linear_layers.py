"""W4A16 linear modules with the constructor, buffers and state-dict layout of UniQL's
quantize/quant_linear_layers.py, running on this package's sm_100a kernels.

`W4A16B16O16Linear` is the drop-in.  `W4A16B16O16HadLinear` is the same layer with the online
Hadamard transform of its input (a `Hadamard(in_features)` module placed in front of it) fused into
the kernel call.  `HadLinear` is the offline fp16 helper the quantisation driver uses.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .hadamard_helpers import get_had_fn
from .quantize_helpers import MARLIN_QQQ_MAX_PARALLEL, MARLIN_QQQ_MIN_THREAD_N, w4a16_quantize


class W4A16B16O16Linear(torch.nn.Module):
    """fp16 activations x int4 group-128 weights -> fp16 (quant_linear_layers.py:11-119)."""

    hadamard_dim = 0

    def __init__(self, in_features, out_features, bias=False, group_size=128, device=None, **kwargs):
        factory_kwargs = {"device": device}
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.size_n, self.size_k = out_features, in_features
        self.pad_out = (256 - self.size_n % 256) % 256       # stored width is a multiple of 256
        self.size_n += self.pad_out
        self.pad_in = (group_size - self.size_k % group_size) % group_size
        self.size_k += self.pad_in
        self.max_par = 16
        # Kept for state-dict compatibility; the reference uses it as inter-CTA locks, these kernels do not.
        self.register_buffer("workspace", torch.zeros(
            (self.size_n // MARLIN_QQQ_MIN_THREAD_N) * MARLIN_QQQ_MAX_PARALLEL, dtype=torch.int32, **factory_kwargs))
        self.register_buffer("weight", torch.empty(
            (self.size_k // 16, self.size_n * 16 // 8), dtype=torch.int32, **factory_kwargs))
        self.register_buffer("scale", torch.empty(
            (self.size_k // group_size, self.size_n), dtype=torch.float16, **factory_kwargs))
        if bias:
            self.register_parameter("bias", nn.Parameter(torch.empty(
                out_features, dtype=torch.float16, **factory_kwargs)))
        else:
            self.bias = None

    @classmethod
    def from_fp16(cls, originalLayer: nn.Linear):
        """RTN (or GPTQ-provided scales) -> packed buffers (quant_linear_layers.py:50-89)."""
        bits = 4
        group_size = 128 if originalLayer.in_features > 128 else -1
        group_scale = None
        if getattr(originalLayer, "apply_gptq", False):
            bits = originalLayer.bits
            group_size = originalLayer.group_size
            group_scale = originalLayer.group_scale.to(torch.float16)     # [n_groups, out_dim]
        assert bits == 4, "Only support 4-bit quantization"
        if group_size not in [-1, 128]:
            raise ValueError("Only groupsize -1 and 128 are supported.")
        if group_size == -1:
            raise ValueError("per-channel W4A16 (in_features <= 128) is not supported by the uniql_b200 kernels")

        device = originalLayer.weight.device
        qlinear = cls(originalLayer.in_features, originalLayer.out_features, device=device)
        w = originalLayer.weight
        pad_out = (256 - w.shape[0] % 256) % 256
        if w.is_cuda:
            # on the GPU in one pass over the [Dout, Din] weight, same bits as the host path below
            gs = group_scale.to(device) if group_scale is not None else None
            _, q_w, scale = ops.w4a16_quantize(w, gs, n_pad=w.shape[0] + pad_out, want_ref=False)
            size_k, size_n = q_w.shape[0] * 16, q_w.shape[1] // 2
        else:
            w_t = w.detach().to(torch.float16).t().contiguous()           # [Din, Dout]
            w_ref, q_w, scale = w4a16_quantize(w_t, bits, group_size, group_scale, pad_out=pad_out)
            size_k, size_n = w_ref.shape
        qlinear.pad_out = pad_out
        qlinear.size_k, qlinear.size_n = size_k, size_n
        qlinear.pad_in = size_k - w.shape[1]
        qlinear.max_par = 16
        qlinear.weight = q_w.to(device)
        qlinear.scale = scale.to(device)
        if originalLayer.bias is not None:
            qlinear.bias = nn.Parameter(originalLayer.bias.data.clone().to(torch.float16), requires_grad=False)
        return qlinear

    def forward(self, x):
        ext = ops.torch_ext()
        if ext is not None:       # the binding records nothing for autograd: no no_grad context needed around it
            return ext.linear(x, self.weight, self.scale, self.bias, self.out_features, self.pad_in,
                              bool(self.hadamard_dim))
        return self._forward_ctypes(x)

    @torch.no_grad()
    def _forward_ctypes(self, x):
        x_shape = x.shape
        x2 = x.reshape(-1, x_shape[-1])
        if self.pad_in != 0:
            x2 = F.pad(x2, (0, self.pad_in), "constant", 0)
        # bias add and the removal of padded output columns happen inside the kernel epilogue
        y = ops.w4a16_linear(x2, self.weight, self.scale, self.bias, self.out_features,
                             hadamard_dim=self.hadamard_dim and self.size_k)
        return y.view(*x_shape[:-1], self.out_features)

    def __repr__(self):
        return (f"{type(self).__name__}(in_features={self.in_features}, out_features={self.out_features}, "
                f"bias={self.bias is not None})")


class W4A16B16O16HadLinear(W4A16B16O16Linear):
    """`Hadamard(in_features)` followed by `W4A16B16O16Linear`, as one fused kernel call.

    Equivalent to  linear(Hadamard(in_features)(x))  with the transformed activations rounded to fp16
    in between, exactly as the two separate modules would do.  in_features must be a size the reference's
    get_had_fn accepts (a power of two times 1, 12, 20, 28 or 40) and a multiple of 128."""

    hadamard_dim = 1

    def __init__(self, in_features, out_features, bias=False, group_size=128, device=None, **kwargs):
        super().__init__(in_features, out_features, bias=bias, group_size=group_size, device=device, **kwargs)
        assert self.pad_in == 0, "the fused Hadamard needs in_features to be a multiple of the group size"
        get_had_fn(in_features)     # validates the size the same way the reference does


class HadLinear(torch.nn.Linear):
    """fp16 linear whose weight is (or will be) rotated by Hadamard matrices on its input and/or output
    side; used offline before quantisation (quant_linear_layers.py:122-181)."""

    def __init__(self, originalLayer: nn.Linear, input_transform=True, output_transform=False, fuse_had=False):
        assert originalLayer.weight.is_cuda, "Hadamard transform must be on CUDA"
        super().__init__(originalLayer.in_features, originalLayer.out_features,
                         originalLayer.bias is not None, originalLayer.weight.device, originalLayer.weight.dtype)
        self.input_transform = input_transform
        if input_transform:
            self.input_transform_fn, self.Nin, self.had_scale_in = get_had_fn(originalLayer.in_features)
        self.output_transform = output_transform
        if output_transform:
            self.output_transform_fn, self.Nout, self.had_scale_out = get_had_fn(originalLayer.out_features)
        self.weight.data = originalLayer.weight.data
        if originalLayer.bias is not None:
            assert self.output_transform is False, "Bias is not supported for output_transform"
            self.bias.data = originalLayer.bias.data
        self.fuse_had = fuse_had
        if self.fuse_had:
            self.fuse_hadamard()

    def _rotated(self, w):
        if self.input_transform:
            w = self.input_transform_fn(w, self.had_scale_in)
        if self.output_transform:
            w = self.output_transform_fn(w.t(), self.had_scale_out).t()
        return w

    def fuse_hadamard(self):
        self.weight.data = self._rotated(self.weight.data.clone()).contiguous()
        self.fuse_had = True

    def forward(self, x):
        w = self.weight if self.fuse_had else self._rotated(self.weight.clone())
        return F.linear(x, w, self.bias)

    def __repr__(self):
        return (f"HadLinear(in_features={self.in_features}, out_features={self.out_features}, "
                f"bias={self.bias is not None}, input_transform={self.input_transform}, "
                f"output_transform={self.output_transform}, fuse_had={self.fuse_had})")
