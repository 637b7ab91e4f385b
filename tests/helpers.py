"""Shared input generators for the parity tests (seeded, synthetic)."""
import functools

import numpy as np
import torch

from oracle import uniql_oracle as orc


def make_weights(seed, n, k, std=0.02):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(n, k, generator=g) * std).to(torch.float16)


def make_acts(seed, m, k, outliers=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g)
    if outliers:
        idx = torch.randperm(k, generator=g)[: max(1, k // 100)]
        x[:, idx] *= 20
    return x.to(torch.float16)


@functools.lru_cache(maxsize=16)
def quantized_layer(seed, n, k, bias=False):
    """Returns dict with packed/scales (numpy), w_deq fp16 [k, n_padded], n_pad, bias.  The last few layers are kept:
    parametrised tests ask for the same (seed, shape) several times and quantising a large layer on the CPU takes
    seconds; callers treat the arrays as read-only."""
    w = make_weights(seed, n, k)
    pad_out = (256 - n % 256) % 256
    w_ref, packed, scales = orc.w4a16_quantize(np.ascontiguousarray(w.numpy().T), pad_out)
    b = None
    if bias:
        g = torch.Generator().manual_seed(seed + 999)
        b = (torch.randn(n, generator=g) * 0.5).to(torch.float16).numpy()
    return dict(packed=packed, scales=scales, w_deq=w_ref, n=n, n_pad=n + pad_out, k=w_ref.shape[0], bias=b)


def linear_tolerance_check(y, y_ref):
    """The parity gate for the fp16-output linear: max-normalised error <= 1e-2 and
    |y - y_ref| <= 1e-2 |y_ref| + 1e-2 rms(y_ref) elementwise."""
    y = np.asarray(y, dtype=np.float32)
    y_ref = np.asarray(y_ref, dtype=np.float32)
    assert y.shape == y_ref.shape
    assert np.isfinite(y).all()
    denom = max(float(np.abs(y_ref).max()), 1e-6)
    max_rel = float(np.abs(y - y_ref).max()) / denom
    rms = float(np.sqrt(np.mean(y_ref.astype(np.float64) ** 2)))
    bound = 1e-2 * np.abs(y_ref) + 1e-2 * rms + 1e-6
    worst = float((np.abs(y - y_ref) / bound).max())
    assert max_rel <= 1e-2, f"max-normalised error {max_rel:.3e} > 1e-2"
    assert worst <= 1.0, f"elementwise bound exceeded by factor {worst:.3f}"
    return max_rel
