"""Host-side packing helpers with the same names and semantics as UniQL's quantize/quantize_helpers.py.

Everything here is plain torch, runs on whatever device its inputs live on, and is vectorised: the
weight order is generated from its closed form instead of a 1024-entry lookup applied tile by tile, and
nibble packing is a shift-and-sum rather than a numpy loop.  Results are bit-identical to the reference
helpers (checked against fixtures produced by the reference itself).

Layout (reference: quantize_helpers.py:145-165 + :38-50 + :67-84).  For a [K, N] int4 matrix the packed
tensor is int32 [K/16, 2N].  Word w of packed row kt:  blk = w // 128, lane = (w % 128) // 4, j = w % 4,
g = lane // 4, c = lane % 4.  It holds the eight values
    W[16kt + r, 64blk + 16j + g + 8b]   for (r, b) in
    nibble 0..7 = (2c,0) (2c+8,0) (2c,1) (2c+8,1) (2c+1,0) (2c+9,0) (2c+1,1) (2c+9,1).
Scales (reference :54-62, :169-180): inside every 64-column block, stored[8i + j] = natural[i + 8j].
"""
from __future__ import annotations

import functools

import torch

MARLIN_QQQ_TILE = 16
MARLIN_QQQ_MIN_THREAD_N = 64
MARLIN_QQQ_MIN_THREAD_K = 128
MARLIN_QQQ_MAX_PARALLEL = 16
GPTQ_MARLIN_TILE = 16

SUPPORTED_NUM_BITS = [4]
SUPPORTED_GROUP_SIZES = [-1, 128]


class MarlinWorkspace:
    """Zeroed int32 ticket buffer, sized as the reference sizes it (quantize_helpers.py:19-32)."""

    def __init__(self, out_features, min_thread_n, max_parallel):
        assert out_features % min_thread_n == 0, (
            f"out_features = {out_features} is undivisible by min_thread_n = {min_thread_n}")
        self.scratch = torch.zeros((out_features // min_thread_n) * max_parallel, dtype=torch.int, device="cuda")


def get_pack_factor(num_bits):
    assert 32 % num_bits == 0, f"Unsupported num_bits = {num_bits}"
    return 32 // num_bits


@functools.lru_cache(maxsize=None)
def _word_maps():
    """(row[128, 8], col[128, 8]): source coordinates, inside a 16 x 64 tile block, of nibble p of word r."""
    r = torch.arange(128)
    lane, j = r // 4, r % 4
    g, c = lane // 4, lane % 4
    # nibble p -> logical element e = [0,2,4,6,1,3,5,7][p]; e = 4*b + 2*hi + odd
    e = torch.tensor([0, 2, 4, 6, 1, 3, 5, 7])
    b, hi, odd = e // 4, (e // 2) % 2, e % 2
    row = 2 * c[:, None] + odd[None, :] + 8 * hi[None, :]
    col = 16 * j[:, None] + g[:, None] + 8 * b[None, :]
    return row.contiguous(), col.contiguous()


@torch.no_grad()
def get_w4a16_weight_perms():
    """The reference's 1024-entry tile permutation (quantize_helpers.py:145-165), from the closed form."""
    row, col = _word_maps()
    # a tile row of the reference's intermediate layout is 4 tiles of 16x16, each flattened row-major
    tile, incol = col // 16, col % 16
    return (256 * tile + 16 * row + incol).reshape(-1)


@torch.no_grad()
def get_scale_perms():
    scale_perm = [i + 8 * j for i in range(8) for j in range(8)]
    scale_perm_single = [2 * i + j for i in range(4) for j in (0, 1, 8, 9, 16, 17, 24, 25)]
    return scale_perm, scale_perm_single


def _to_int32_bits(v: torch.Tensor) -> torch.Tensor:
    """int64 values in [0, 2^32) -> int32 with the same bit pattern."""
    return torch.where(v >= 2 ** 31, v - 2 ** 32, v).to(torch.int32)


@torch.no_grad()
def pack_w4a16(q_w: torch.Tensor, rows_per_chunk: int = 256) -> torch.Tensor:
    """int [K, N] with values 0..15 -> packed int32 [K/16, 2N]."""
    size_k, size_n = q_w.shape
    assert size_k % 16 == 0 and size_n % 64 == 0, f"size_k = {size_k}, size_n = {size_n}"
    row, col = _word_maps()
    row, col = row.to(q_w.device), col.to(q_w.device)
    shifts = (4 * torch.arange(8, device=q_w.device)).to(torch.int64)
    kt, nblk = size_k // 16, size_n // 64
    out = torch.empty((kt, nblk * 128), dtype=torch.int32, device=q_w.device)
    for k0 in range(0, kt, rows_per_chunk):
        k1 = min(kt, k0 + rows_per_chunk)
        t = q_w[16 * k0:16 * k1].reshape(k1 - k0, 16, nblk, 64).to(torch.int64) & 0xF
        vals = t[:, row, :, col]                        # [128, 8, kt_chunk, nblk]
        word = (vals << shifts.view(1, 8, 1, 1)).sum(dim=1)        # [128, kt_chunk, nblk]
        out[k0:k1] = _to_int32_bits(word.permute(1, 2, 0).reshape(k1 - k0, nblk * 128))
    return out


@torch.no_grad()
def unpack_w4a16(q_packed: torch.Tensor, rows_per_chunk: int = 256) -> torch.Tensor:
    """packed int32 [K/16, 2N] -> int32 [K, N] with values 0..15."""
    kt, w2 = q_packed.shape
    assert w2 % 128 == 0
    nblk = w2 // 128
    row, col = _word_maps()
    row, col = row.to(q_packed.device), col.to(q_packed.device)
    shifts = (4 * torch.arange(8, device=q_packed.device)).to(torch.int64)
    out = torch.empty((kt * 16, nblk * 64), dtype=torch.int32, device=q_packed.device)
    flat_idx = (row * 64 + col).reshape(-1)             # position inside a 16 x 64 block, per (word, nibble)
    for k0 in range(0, kt, rows_per_chunk):
        k1 = min(kt, k0 + rows_per_chunk)
        w = q_packed[k0:k1].to(torch.int64) & 0xFFFFFFFF
        nib = (w.reshape(k1 - k0, nblk, 128, 1) >> shifts.view(1, 1, 1, 8)) & 0xF     # [kt, nblk, 128, 8]
        blockv = torch.empty((k1 - k0, nblk, 1024), dtype=torch.int32, device=q_packed.device)
        blockv[:, :, flat_idx] = nib.reshape(k1 - k0, nblk, 1024).to(torch.int32)
        out[16 * k0:16 * k1] = blockv.reshape(k1 - k0, nblk, 16, 64).permute(0, 2, 1, 3).reshape(-1, nblk * 64)
    return out


@torch.no_grad()
def permute_weights(q_w, size_k, size_n, perm, tile=GPTQ_MARLIN_TILE):
    """Re-order to the reference's pre-packing layout [K/16, 16N] (quantize_helpers.py:38-50)."""
    assert size_k % tile == 0, f"size_k = {size_k}, tile = {tile}"
    assert size_n % tile == 0, f"size_n = {size_n}, tile = {tile}"
    t = q_w.reshape(size_k // tile, tile, size_n // tile, tile).permute(0, 2, 1, 3)
    t = t.reshape(size_k // tile, size_n * tile)
    return t.reshape(-1, perm.numel())[:, perm.to(t.device)].reshape(t.shape)


@torch.no_grad()
def unpermute_weights(q_w, size_k, size_n, perm, tile=GPTQ_MARLIN_TILE):
    """Inverse of permute_weights (quantize_helpers.py:279-300)."""
    perm = perm.to(q_w.device)
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(perm.numel(), device=perm.device)
    t = q_w.reshape(-1, perm.numel())[:, inv].reshape(size_k // tile, size_n // tile, tile, tile)
    return t.permute(0, 2, 1, 3).reshape(size_k, size_n).contiguous()


@torch.no_grad()
def get_w4a16_permute_weights(q_w, size_k, size_n, num_bits, perm, group_size):
    """Permute + pack (quantize_helpers.py:67-84).  `perm` is accepted for signature compatibility."""
    assert num_bits == 4
    assert q_w.shape == (size_k, size_n)
    return pack_w4a16(q_w)


@torch.no_grad()
def unpack_w4a16_permute_weights(q_packed, size_k, size_n, num_bits, perm, group_size):
    """Unpack + un-permute (quantize_helpers.py:304-328)."""
    assert num_bits == 4
    q = unpack_w4a16(q_packed)
    assert q.shape == (size_k, size_n)
    return q


@torch.no_grad()
def get_fake_quantize_weights(w: torch.Tensor, num_bits: int, group_size: int = -1):
    """RTN quantiser (quantize_helpers.py:88-141).  w: float [K, N].  Returns (w_ref, q_w, scale)."""
    size_k, size_n = w.shape
    assert w.is_floating_point(), "w must be float"
    if group_size == -1:
        group_size = size_k
    assert group_size <= size_k
    if group_size < size_k:
        padding_k = (group_size - (size_k % group_size)) % group_size
        if padding_k > 0:
            w = torch.nn.functional.pad(w, (0, 0, 0, padding_k), mode="constant", value=0)
        w = w.reshape((-1, group_size, size_n))
        max_q_val = 2 ** num_bits - 1
        half_q_val = (max_q_val + 1) // 2
        scale = w.abs().amax(dim=1, keepdim=True)
        scale = scale * (2 / max_q_val)
        q_w = torch.round(w / scale)
        q_w = torch.nan_to_num(q_w, nan=-float(half_q_val)).int()      # all-zero group -> code 0
        q_w = torch.clamp(q_w + half_q_val, 0, max_q_val)
        w_ref = (q_w - half_q_val) * scale
        q_w = q_w.reshape((-1, size_n)).contiguous()
        w_ref = w_ref.reshape((-1, size_n)).contiguous()
        scale = scale.reshape((-1, size_n)).contiguous()
    else:
        # Per-channel codes are signed in the reference while its packer and kernel assume offset-8 codes;
        # that mode never round-trips there and no kernel here accepts it.
        raise ValueError("per-channel (group_size == size_k) quantisation is not supported; use group_size=128")
    return w_ref, q_w, scale


@torch.no_grad()
def w4a16_permute_scales(scale, size_k, size_n, group_size):
    scale_perm, scale_perm_single = get_scale_perms()
    if group_size < size_k and group_size != -1:
        assert group_size == 128, "Only group_size 128 is supported for per-group quantization"
        scale = scale.reshape((-1, len(scale_perm)))[:, scale_perm]
    else:
        assert group_size == size_k
        scale = scale.reshape((-1, len(scale_perm_single)))[:, scale_perm_single]
    return scale.reshape((-1, size_n)).contiguous()


@torch.no_grad()
def w4a16_unpermute_scales(permuted_scale, size_k, size_n, group_size):
    scale_perm_group, scale_perm_single = get_scale_perms()
    if group_size < size_k and group_size != -1:
        assert group_size == 128, "Only group_size 128 is supported for per-group quantization"
        perm = scale_perm_group
    else:
        assert group_size == size_k
        perm = scale_perm_single
    inv = torch.argsort(torch.tensor(perm)).to(permuted_scale.device)
    return permuted_scale.reshape(-1, len(perm))[:, inv].reshape(-1, size_n).contiguous()


@torch.no_grad()
def w4a16_quantize(w: torch.Tensor, num_bits: int, group_size: int = -1, scale: torch.Tensor = None,
                   pad_out: int = 0):
    """[K, N] float -> [w_ref, packed int32 [Kp/16, 2Np], permuted scales] (quantize_helpers.py:184-241)."""
    size_k, size_n = w.shape
    if group_size == -1:
        group_size = size_k
    assert group_size <= size_k
    assert num_bits in SUPPORTED_NUM_BITS, f"Unsupported num_bits = {num_bits}"
    assert group_size in SUPPORTED_GROUP_SIZES + [size_k], f"Unsupported groupsize = {group_size}"

    if scale is None:
        w_ref, q_w, scale = get_fake_quantize_weights(w, num_bits, group_size)
    else:
        # w is already fake-quantised with the given [n_groups, N] scales: recover the integer codes
        max_q_val = 2 ** num_bits - 1
        half_q_val = (max_q_val + 1) // 2
        padding_k = (group_size - (size_k % group_size)) % group_size
        if padding_k > 0:
            w = torch.nn.functional.pad(w, (0, 0, 0, padding_k), "constant", 0)
        w_ref = w.clone()
        q_w = ((w.reshape((-1, group_size, size_n)) / scale.unsqueeze(1)) + half_q_val).round()
        q_w = torch.nan_to_num(q_w, nan=0.0).int()
        q_w = torch.clamp(q_w, 0, max_q_val).reshape((size_k + padding_k, size_n)).contiguous()

    if pad_out != 0:
        w_ref = torch.nn.functional.pad(w_ref, (0, pad_out, 0, 0), "constant", 0)
        q_w = torch.nn.functional.pad(q_w, (0, pad_out, 0, 0), "constant", 0)
        scale = torch.nn.functional.pad(scale, (0, pad_out), "constant", 0)

    size_k, size_n = w_ref.shape
    packed = pack_w4a16(q_w)
    marlin_scale = w4a16_permute_scales(scale, size_k, size_n, group_size)
    return [w_ref.to(w.device), packed.to(w.device), marlin_scale.to(w.device)]


@torch.no_grad()
def unpermute_group_scales(permuted_scale: torch.Tensor) -> torch.Tensor:
    """Group-128 scale rows back to natural column order, whatever the number of rows (the name-compatible
    w4a16_unpermute_scales switches to the per-channel order when there is a single group)."""
    inv = torch.argsort(torch.tensor(get_scale_perms()[0])).to(permuted_scale.device)
    return permuted_scale.reshape(-1, 64)[:, inv].reshape(permuted_scale.shape).contiguous()


@torch.no_grad()
def permute_group_scales(scale: torch.Tensor) -> torch.Tensor:
    """Inverse of unpermute_group_scales."""
    perm = torch.tensor(get_scale_perms()[0], device=scale.device)
    return scale.reshape(-1, 64)[:, perm].reshape(scale.shape).contiguous()


@torch.no_grad()
def w4a16_dequantize(q_packed: torch.Tensor, permuted_scale: torch.Tensor, group_size: int = 128) -> torch.Tensor:
    """Packed buffers -> fp16 [K, N], w = fp16((q - 8) * s): the inverse the reference applies when it
    re-slices weights at load time (modeling/modeling_helpers.py:632-640)."""
    size_k, size_n = q_packed.shape[0] * 16, q_packed.shape[1] // 2
    q = unpack_w4a16(q_packed).to(permuted_scale.dtype) - 8
    s = unpermute_group_scales(permuted_scale)
    return (q.reshape(-1, group_size, size_n) * s.unsqueeze(1)).reshape(size_k, size_n)
