"""`fast_hadamard_transform_cuda` stand-in: the five entry points UniQL calls
(quantize/hadamard_helpers.py:20-35).  Each returns a new tensor H x * scale over the last axis."""
from .. import ops


def _checked(base):
    def fn(x, scale):
        dim = x.shape[-1]
        if base == 1:
            ok = dim > 0 and (dim & (dim - 1)) == 0
        else:
            p = dim // base
            ok = dim % base == 0 and p > 0 and (p & (p - 1)) == 0
        if not ok:
            raise RuntimeError(f"dim {dim} is not {'a power of two' if base == 1 else f'{base} times a power of two'}")
        ext = ops.torch_ext()
        if ext is not None:
            return ext.hadamard(x, float(scale))
        return ops.hadamard(x, scale)
    return fn


fast_hadamard_transform = _checked(1)
fast_hadamard_transform_12N = _checked(12)
fast_hadamard_transform_20N = _checked(20)
fast_hadamard_transform_28N = _checked(28)
fast_hadamard_transform_40N = _checked(40)
