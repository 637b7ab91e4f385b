"""Hadamard size dispatch with the reference's names (quantize/hadamard_helpers.py:18-48)."""
import math

from ..compat import fast_hadamard_transform_cuda


def is_pow2(n):
    return (n & (n - 1) == 0) and (n > 0)


def next_power_of_two(x):
    """Smallest power of two >= x."""
    return 1 if x == 0 else 2 ** (x - 1).bit_length()


def prev_power_of_two(x):
    """Largest power of two <= x (0 for x < 1)."""
    if x < 1:
        return 0
    return 2 ** (x.bit_length() - 1)


def get_had_fn(dim):
    """(transform_fn, base, 1/sqrt(dim)); bases are tried in the order 40, 28, 20, 12, power of two."""
    had_scale = 1.0 / math.sqrt(dim)
    for base in (40, 28, 20, 12):
        if dim % base == 0 and is_pow2(dim // base):
            return getattr(fast_hadamard_transform_cuda, f"fast_hadamard_transform_{base}N"), base, had_scale
    assert is_pow2(dim), f"Invalid dim: {dim}. dim must be a power of 2."
    return fast_hadamard_transform_cuda.fast_hadamard_transform, 2, had_scale


def had_transform(w):
    """Transform the last axis of w (any leading shape); returns a new tensor."""
    saved_shape = w.shape
    dim = saved_shape[-1]
    transform_fn, _, had_scale = get_had_fn(dim)
    w_h = transform_fn(w.reshape(-1, dim), had_scale)
    return w_h.reshape(saved_shape)
