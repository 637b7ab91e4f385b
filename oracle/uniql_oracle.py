"""CPU oracle for the UniQL W4A16 quantized-linear hot path (TEST INFRASTRUCTURE ONLY).

This file restates, in plain numpy, the arithmetic of the reference's W4A16
linear, 4-bit embedding and Hadamard path.  It is the checker the parity tests
compare the CUDA kernels against; nothing in the product package imports it.
Only tests, the smoke check and the benchmark's CPU-baseline leg may use it.

Pinning:
  * linear quantise / pack / unpack / dequantise and the embedding quantiser are
    pinned bit-for-bit against the reference's own Python helpers, executed on
    the CPU, through the fixtures in tests/golden/ (made by
    tests/golden/make_golden.py).
  * power-of-two Hadamard: the Sylvester construction is unambiguous.
  * 12N/20N/28N/40N Hadamard: PARITY UNPINNED.  The reference delegates to the
    third-party package fast-hadamard-transform (git submodule, not vendored, no
    commit pin visible), whose base matrices are not available.  The matrices
    here are Paley constructions; the CUDA kernels use the same ones.

Reference citations are paths inside the UniQL project.
"""
from __future__ import annotations

import math

import numpy as np

GROUP = 128          # quantize/quant_linear_layers.py:13 (group_size=128)
TILE = 16            # quantize/quantize_helpers.py:13 (GPTQ_MARLIN_TILE)
_INTERLEAVE = np.array([0, 2, 4, 6, 1, 3, 5, 7])


# --------------------------------------------------------------------------
# RTN quantiser  (quantize/quantize_helpers.py:88-141, group branch :99-122)
# --------------------------------------------------------------------------
def _f16_mul_scalar(a16: np.ndarray, scalar: float) -> np.ndarray:
    """fp16 tensor times a Python scalar the way torch does it on CPU:
    operands widened to fp32, one multiply, one rounding back to fp16."""
    return (a16.astype(np.float32) * np.float32(scalar)).astype(np.float16)


def rtn_quantize_g128(w_kn: np.ndarray, group: int = GROUP):
    """w_kn: fp16 [K, N] (already transposed: in-features first).

    Returns (w_ref fp16 [Kp,N], q int32 [Kp,N] in 0..15, scale fp16 [Kp/group,N]).
    K is zero-padded up to a multiple of `group` (quantize_helpers.py:101-103).
    """
    assert w_kn.dtype == np.float16 and w_kn.ndim == 2
    k, n = w_kn.shape
    pad_k = (group - k % group) % group
    if pad_k:
        w_kn = np.concatenate([w_kn, np.zeros((pad_k, n), np.float16)], 0)
    w = w_kn.reshape(-1, group, n)
    scale = np.abs(w).max(axis=1, keepdims=True)                 # :109
    scale = _f16_mul_scalar(scale, 2 / 15)                       # :110
    with np.errstate(divide="ignore", invalid="ignore"):
        ratio = (w.astype(np.float32) / scale.astype(np.float32)).astype(np.float16)
    ratio = np.where(np.isnan(ratio), np.float16(0), ratio)      # all-zero group: torch's
    # NaN->int conversion saturates and the clamp below maps it to 0 as well.
    nan_mask = (scale == 0)
    q = np.rint(ratio.astype(np.float32)).astype(np.int64) + 8   # :113-114 (round half to even)
    q = np.clip(q, 0, 15).astype(np.int32)                       # :115
    q = np.where(np.broadcast_to(nan_mask, q.shape), 0, q).astype(np.int32)
    w_ref = ((q - 8).astype(np.float32) * scale.astype(np.float32)).astype(np.float16)  # :117
    return (w_ref.reshape(-1, n), q.reshape(-1, n), scale.reshape(-1, n))


# --------------------------------------------------------------------------
# Weight permutation + nibble packing
# (quantize_helpers.py:145-165 perm, :38-50 tiling, :67-84 pack)
# --------------------------------------------------------------------------
def weight_perm() -> np.ndarray:
    """The 1024-entry permutation of quantize_helpers.py:145-165."""
    perm = []
    for i in range(32):
        col = i // 4
        perm1 = []
        for block in (0, 1):
            for row in (2 * (i % 4), 2 * (i % 4) + 1, 2 * (i % 4 + 4), 2 * (i % 4 + 4) + 1):
                perm1.append(16 * row + col + 8 * block)
        for j in range(4):
            perm.extend(p + 256 * j for p in perm1)
    perm = np.array(perm).reshape(-1, 8)[:, _INTERLEAVE].ravel()
    return perm


def pack_weights(q_kn: np.ndarray) -> np.ndarray:
    """q int32 [K,N] (0..15) -> packed int32 [K/16, 2N] in the kernel's order."""
    k, n = q_kn.shape
    assert k % TILE == 0 and n % 64 == 0
    t = q_kn.reshape(k // TILE, TILE, n // TILE, TILE).transpose(0, 2, 1, 3)
    t = t.reshape(k // TILE, n * TILE)                           # :44-46
    perm = weight_perm()
    t = t.reshape(-1, perm.size)[:, perm].reshape(t.shape)       # :48
    t = t.astype(np.uint32)
    packed = np.zeros((t.shape[0], t.shape[1] // 8), np.uint32)
    for i in range(8):                                           # :79-80
        packed |= t[:, i::8] << np.uint32(4 * i)
    return packed.view(np.int32)


def unpack_weights(packed: np.ndarray, k: int, n: int) -> np.ndarray:
    """Inverse of pack_weights (quantize_helpers.py:279-328)."""
    p = packed.view(np.uint32)
    assert p.shape == (k // TILE, 2 * n)
    t = np.zeros((p.shape[0], p.shape[1] * 8), np.uint32)
    for i in range(8):
        t[:, i::8] = (p >> np.uint32(4 * i)) & np.uint32(0xF)
    perm = weight_perm()
    inv = np.empty_like(perm)
    inv[perm] = np.arange(perm.size)
    t = t.reshape(-1, perm.size)[:, inv].reshape(k // TILE, n * TILE)
    t = t.reshape(k // TILE, n // TILE, TILE, TILE).transpose(0, 2, 1, 3)
    return np.ascontiguousarray(t.reshape(k, n)).astype(np.int32)


def scale_perm() -> np.ndarray:
    """quantize_helpers.py:54-57 (group mode, 64 wide)."""
    return np.array([i + 8 * j for i in range(8) for j in range(8)])


def permute_scales(scale_gn: np.ndarray) -> np.ndarray:
    """quantize_helpers.py:169-180, group mode."""
    g, n = scale_gn.shape
    assert n % 64 == 0
    return np.ascontiguousarray(scale_gn.reshape(-1, 64)[:, scale_perm()].reshape(g, n))


def unpermute_scales(scale_perm_gn: np.ndarray) -> np.ndarray:
    """quantize_helpers.py:245-275, group mode."""
    g, n = scale_perm_gn.shape
    inv = np.argsort(scale_perm())
    return np.ascontiguousarray(scale_perm_gn.reshape(-1, 64)[:, inv].reshape(g, n))


def w4a16_quantize(w_kn: np.ndarray, pad_out: int = 0):
    """quantize_helpers.py:184-241 with num_bits=4, group_size=128, scale=None.

    Returns (w_ref fp16 [Kp,Np], packed int32 [Kp/16, 2Np], scales fp16 [Kp/128, Np])."""
    w_ref, q, scale = rtn_quantize_g128(w_kn)
    if pad_out:                                                  # :219-222
        w_ref = np.pad(w_ref, ((0, 0), (0, pad_out)))
        q = np.pad(q, ((0, 0), (0, pad_out)))
        scale = np.pad(scale, ((0, 0), (0, pad_out)))
    return w_ref, pack_weights(q), permute_scales(scale)


def dequantize(packed: np.ndarray, scales_perm: np.ndarray) -> np.ndarray:
    """Packed buffers -> fp16 [K,N]: w = fp16((q-8) * s).

    Same arithmetic as the GEMM kernel's per-element dequant
    (csrc/linear/marlin_gemm_kernel.cuh:118-146) and as the reference's own
    host-side dequantise (modeling/modeling_helpers.py:632-640)."""
    kt, n2 = packed.shape
    k, n = kt * TILE, n2 // 2
    q = unpack_weights(packed, k, n)
    s = unpermute_scales(scales_perm)
    assert s.shape == (k // GROUP, n)
    qc = (q - 8).astype(np.float32).reshape(k // GROUP, GROUP, n)
    w = (qc * s.astype(np.float32)[:, None, :]).astype(np.float16)
    return w.reshape(k, n)


def linear_ref(x: np.ndarray, packed: np.ndarray, scales_perm: np.ndarray,
               bias: np.ndarray | None = None, n_out: int | None = None,
               w_deq: np.ndarray | None = None) -> np.ndarray:
    """fp32 reference of W4A16B16O16Linear.forward (quant_linear_layers.py:91-116):
    y = x @ W_deq accumulated in fp32 (+ bias), first n_out columns."""
    if w_deq is None:
        w_deq = dequantize(packed, scales_perm)
    y = x.astype(np.float32) @ w_deq.astype(np.float32)
    if n_out is not None:
        y = y[:, :n_out]
    if bias is not None:
        y = y + bias.astype(np.float32)[None, :]
    return y


# --------------------------------------------------------------------------
# 4-bit embedding (quantize/quant_embedding_layers.py:25-47,
#                  csrc/embedding/quant_embedding_kernel.cuh:47-76, 96-112)
# --------------------------------------------------------------------------
def embedding_quantize(w_vd: np.ndarray):
    """fp16 [V,D] -> (packed int32 [V, D/8], scales fp16 [V]).

    quant_embedding_layers.py:36-43: s = amax/8, q = clamp(round(w/s + 8), 0, 15)
    computed in the table's dtype (fp16), groups of 8 interleaved then packed."""
    assert w_vd.dtype == np.float16
    v, d = w_vd.shape
    assert d % 8 == 0
    amax = np.abs(w_vd).max(axis=1, keepdims=True)
    scales = (amax.astype(np.float32) / np.float32(8)).astype(np.float16)
    with np.errstate(divide="ignore", invalid="ignore"):
        r = (w_vd.astype(np.float32) / scales.astype(np.float32)).astype(np.float16)
    r = (r.astype(np.float32) + np.float32(8)).astype(np.float16)
    q = np.clip(np.rint(r.astype(np.float32)), 0, 15)
    q = np.where(np.isnan(q), 0, q).astype(np.uint32)
    q = q.reshape(v, -1, 8)[:, :, _INTERLEAVE].reshape(v, -1)
    packed = np.zeros((v, d // 8), np.uint32)
    for i in range(8):
        packed |= (q[:, i::8] & np.uint32(0xF)) << np.uint32(4 * i)
    return packed.view(np.int32), scales.reshape(-1)


def embedding_unpack(packed_vw: np.ndarray) -> np.ndarray:
    """int32 [V, D/8] -> uint8 [V, D] nibbles in natural element order.
    Output element o of a word comes from nibble [0,4,1,5,2,6,3,7][o]
    (quant_embedding_kernel.cuh:104-110)."""
    p = packed_vw.view(np.uint32)
    v, w = p.shape
    src = np.array([0, 4, 1, 5, 2, 6, 3, 7])
    out = np.empty((v, w, 8), np.uint8)
    for o in range(8):
        out[:, :, o] = (p >> np.uint32(4 * src[o])) & np.uint32(0xF)
    return out.reshape(v, w * 8)


def embedding_lookup(ids: np.ndarray, packed_vw: np.ndarray, scales_v: np.ndarray) -> np.ndarray:
    """out[t, :] = fp16((q-8) * s[id]) — a single rounding to fp16
    (quant_embedding_kernel.cuh:47-76: exact q-8 in fp16, then one __hmul2)."""
    flat = ids.reshape(-1)
    if flat.size == 0:
        return np.zeros((*ids.shape, packed_vw.shape[1] * 8), np.float16)
    rows = embedding_unpack(packed_vw[flat])
    qc = rows.astype(np.float32) - np.float32(8)
    s = scales_v[flat].astype(np.float32)[:, None]
    out = (qc * s).astype(np.float16)
    return out.reshape(*ids.shape, -1)


# --------------------------------------------------------------------------
# Hadamard  (quantize/hadamard_helpers.py:18-48, quant_hadamard_layers.py:16-18)
# --------------------------------------------------------------------------
def is_pow2(n: int) -> bool:
    return n > 0 and (n & (n - 1)) == 0


def had_factor(dim: int) -> int:
    """Base-matrix order the reference dispatches on (hadamard_helpers.py:18-36):
    40, 28, 20, 12 tried in that order, else a power of two (returns 1)."""
    for base in (40, 28, 20, 12):
        if dim % base == 0 and is_pow2(dim // base):
            return base
    assert is_pow2(dim), f"Invalid dim: {dim}. dim must be a power of 2."
    return 1


def _legendre(a: int, q: int) -> int:
    a %= q
    if a == 0:
        return 0
    return 1 if pow(a, (q - 1) // 2, q) == 1 else -1


def _jacobsthal(q: int) -> np.ndarray:
    return np.array([[_legendre(j - i, q) for j in range(q)] for i in range(q)], np.int64)


def paley1(q: int) -> np.ndarray:
    """Paley construction I, q prime, q % 4 == 3 -> Hadamard matrix of order q+1."""
    assert q % 4 == 3
    n = q + 1
    qm = _jacobsthal(q)
    s = np.zeros((n, n), np.int64)
    s[0, 1:] = 1
    s[1:, 0] = -1
    s[1:, 1:] = qm
    return s + np.eye(n, dtype=np.int64)


def paley2(q: int) -> np.ndarray:
    """Paley construction II, q prime, q % 4 == 1 -> Hadamard matrix of order 2(q+1)."""
    assert q % 4 == 1
    n = q + 1
    c = np.zeros((n, n), np.int64)
    c[0, 1:] = 1
    c[1:, 0] = 1
    c[1:, 1:] = _jacobsthal(q)
    h = np.zeros((2 * n, 2 * n), np.int64)
    blk_p = np.array([[1, -1], [-1, -1]])
    blk_z = np.array([[1, 1], [1, -1]])
    for i in range(n):
        for j in range(n):
            if c[i, j] == 0:
                h[2 * i:2 * i + 2, 2 * j:2 * j + 2] = blk_z
            else:
                h[2 * i:2 * i + 2, 2 * j:2 * j + 2] = c[i, j] * blk_p
    return h


def base_matrix(base: int) -> np.ndarray:
    """±1 Hadamard matrix of order 12, 20, 28 or 40 (this build's choice)."""
    if base == 12:
        h = paley1(11)
    elif base == 20:
        h = paley1(19)
    elif base == 28:
        h = paley2(13)
    elif base == 40:
        h20 = paley1(19)
        h = np.kron(np.array([[1, 1], [1, -1]]), h20)
    else:
        raise ValueError(base)
    assert np.array_equal(h @ h.T, base * np.eye(base, dtype=np.int64))
    return h


def fwht(x: np.ndarray) -> np.ndarray:
    """Unnormalised Sylvester-ordered Walsh-Hadamard transform along the last axis."""
    n = x.shape[-1]
    assert is_pow2(n)
    y = x.astype(np.float64).copy()
    h = 1
    while h < n:
        y = y.reshape(*x.shape[:-1], n // (2 * h), 2, h)
        a = y[..., 0, :] + y[..., 1, :]
        b = y[..., 0, :] - y[..., 1, :]
        y = np.stack([a, b], axis=-2)
        h *= 2
    return y.reshape(x.shape)


def hadamard_transform(x: np.ndarray, scale: float | None = None, base_h: np.ndarray | None = None) -> np.ndarray:
    """y = (H_base (x) H_{2^k}) x * scale along the last axis, float64 result.  `base_h` replaces this build's
    choice of base matrix (for a caller who holds the third-party package's tables).

    The index splits as i = a * 2^k + b with a the base-matrix index (slow) and
    b the Sylvester index (fast).  scale defaults to 1/sqrt(dim)
    (hadamard_helpers.py:19)."""
    dim = x.shape[-1]
    base = had_factor(dim)
    if scale is None:
        scale = 1.0 / math.sqrt(dim)
    if base == 1:
        return fwht(x) * scale
    p = dim // base
    y = fwht(x.reshape(*x.shape[:-1], base, p))
    hb = (base_matrix(base) if base_h is None else np.asarray(base_h)).astype(np.float64)
    assert hb.shape == (base, base)
    y = np.einsum("ij,...jp->...ip", hb, y)
    return y.reshape(x.shape) * scale
