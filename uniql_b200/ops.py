"""Torch-facing wrappers over the C ABI: allocate outputs/scratch with torch, pass raw pointers.

These functions are what the drop-in modules and the `quant_linear_cuda` / `quant_embedding_cuda` /
`fast_hadamard_transform_cuda` stand-ins call.  All of them require CUDA tensors; there is no fallback.
"""
from __future__ import annotations

import torch

import ctypes

from ._lib import Prefetch, Proj, check, lib, torch_ext

_DTYPE_CODE = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}

_scratch: dict = {}      # (device index, stream handle) -> uint8 tensor whose counter region is zero
_status: dict = {}       # device index -> int32[1] status word


def _stream_handle(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def status_word(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        ext = torch_ext()
        # one word per device, shared with the torch binding when that is loaded
        t = ext.status_tensor(idx) if ext is not None else torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = t
    return t


def read_and_clear_status(device) -> int:
    """Synchronising read of the kernel diagnostics word (bit 0: an embedding id was out of range; bit 1: a bounded
    wait gave up; bit 2: a slicing index was outside the source layer)."""
    t = status_word(torch.device(device))
    v = int(t.item())
    t.zero_()
    return v


def _scratch_for(device: torch.device, nbytes: int) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (idx, _stream_handle(device))
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        size = max(nbytes, 1 << 20)
        size = (size + (1 << 20) - 1) >> 20 << 20
        buf = torch.zeros(size, dtype=torch.uint8, device=torch.device("cuda", idx))
        _scratch[key] = buf
    return buf


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (uniql_b200 has no CPU path)")


_need_cache: dict = {}   # (m, n, k, hadamard_dim) -> scratch bytes


def w4a16_linear(x: torch.Tensor, weight: torch.Tensor, scale: torch.Tensor, bias: torch.Tensor | None,
                 n_out: int, hadamard_dim: int = 0, out: torch.Tensor | None = None, comm=None) -> torch.Tensor:
    """y[m, n_out] = x[m, k] @ dequant(weight, scale)[:, :n_out] (+ bias); x fp16 2-D, row-major.
    With `comm` (a communicator handle from uniql_comm_create) the result is summed over the ranks inside the
    kernel (row-parallel linear, m <= 16)."""
    if not (x.is_cuda and weight.is_cuda and scale.is_cuda):
        raise RuntimeError("x, weight and scale must be CUDA tensors (uniql_b200 has no CPU path)")
    if x.dtype != torch.float16 or x.dim() != 2:
        raise RuntimeError("x must be a 2-D float16 tensor")
    if weight.dtype != torch.int32 or scale.dtype != torch.float16:
        raise RuntimeError("weight must be int32 and scale float16")
    if x.stride(1) != 1:
        x = x.contiguous()
    m, k = x.shape
    kt, n2 = weight.shape
    if kt * 16 != k:
        raise RuntimeError(f"size_k mismatch: x has {k} columns, packed weight covers {kt * 16}")
    n = n2 // 2
    groups = scale.shape[0]
    if groups == 1 and k != 128:
        groupsize = -1
    else:
        if k % groups != 0:
            raise RuntimeError("scale rows do not divide k")
        groupsize = k // groups
    if scale.shape[1] != n:
        raise RuntimeError("scale width does not match the packed weight")
    if not weight.is_contiguous() or not scale.is_contiguous():
        raise RuntimeError("weight and scale must be contiguous")
    bias_ptr = None
    if bias is not None:
        if bias.dtype != torch.float16 or bias.numel() < n_out or not bias.is_contiguous():
            raise RuntimeError("bias must be a contiguous float16 tensor with at least n_out elements")
        bias_ptr = bias.data_ptr()
    if (m > 1 and x.stride(0) % 8 != 0) or x.data_ptr() % 16 != 0:
        x = x.clone(memory_format=torch.contiguous_format)
    lda = x.stride(0) if m > 1 else k
    dev = x.device
    idx = dev.index
    switch = torch.cuda.current_device() != idx
    if switch:
        prev = torch.cuda.current_device()
        torch.cuda.set_device(idx)
    try:
        if out is None:
            out = torch.empty((m, n_out), dtype=torch.float16, device=dev)
        L = lib()
        key = (m, n, k, hadamard_dim)
        nbytes = _need_cache.get(key)
        if nbytes is None:
            nbytes = _need_cache[key] = L.uniql_w4a16_scratch_bytes(m, n, k, hadamard_dim)
        stream = torch._C._cuda_getCurrentRawStream(idx)
        skey = (idx, stream)
        scratch = _scratch.get(skey)
        if scratch is None or scratch.numel() < nbytes:
            scratch = _scratch_for(dev, nbytes)
        st = _status.get(idx)
        if st is None:
            st = status_word(dev)
        if comm is not None:
            code = L.uniql_w4a16_linear_allreduce(
                comm, x.data_ptr(), lda, weight.data_ptr(), scale.data_ptr(), bias_ptr,
                out.data_ptr(), out.stride(0), m, n, n_out, k, groupsize,
                scratch.data_ptr(), scratch.numel(), st.data_ptr(), stream)
        else:
            code = L.uniql_w4a16_linear(
                x.data_ptr(), lda, weight.data_ptr(), scale.data_ptr(), bias_ptr,
                out.data_ptr(), out.stride(0), m, n, n_out, k, groupsize, hadamard_dim,
                scratch.data_ptr(), scratch.numel(), st.data_ptr(), stream)
    finally:
        if switch:
            torch.cuda.set_device(prev)
    if code != 0:
        check(code, "uniql_w4a16_linear")
    return out


_EPILOGUES = {"none": 0, "swiglu": 1}
TP_REDUCE, TP_GATHER_OUT, TP_GATHER_IN = 1, 2, 4
_group_need_cache: dict = {}


def w4a16_linear_group(x: torch.Tensor | None, layers, epilogue: str = "none", residual: torch.Tensor | None = None,
                       hadamard_dim: int = 0, outs=None, comm=None, tp_flags: int = 0, col_offset: int = 0,
                       k_offset: int = 0, m: int | None = None, prefetch=None):
    """One launch for up to four projections that read the same activations: the decode kernel for m <= 16 (all
    options below), the operand-swapped tensor-core kernel for 17 <= m <= 128 (plain outputs only).

    layers: sequence of (weight int32 [k/16, 2n], scale fp16 [k/128, n], bias fp16 or None, n_out).
    epilogue "swiglu": two layers (gate, up) -> one output silu(gate) * up.  residual: fp16 [m, n_out] added to the
    result (single layer or swiglu).  hadamard_dim: size of the Hadamard transform applied to the rows of x first.
    With `comm` (communicator handle) and tp_flags (TP_REDUCE / TP_GATHER_OUT / TP_GATHER_IN) the launch is a step of a
    tensor-parallel layer; with TP_GATHER_IN x may be None and m must be given.
    prefetch: up to four tensors (or (tensor, bytes) pairs) -- the packed weights the following launches will stream --
    that the kernel asks L2 for when its own stream ends.
    Returns the list of outputs (one tensor for swiglu)."""
    if epilogue not in _EPILOGUES:
        raise RuntimeError(f"unknown epilogue {epilogue!r}")
    layers = list(layers)
    w0 = layers[0][0]
    if not w0.is_cuda:
        raise RuntimeError("weights must be CUDA tensors (uniql_b200 has no CPU path)")
    dev = w0.device
    k = w0.shape[0] * 16
    if x is not None:
        if not x.is_cuda or x.dtype != torch.float16 or x.dim() != 2:
            raise RuntimeError("x must be a 2-D float16 CUDA tensor")
        if x.stride(1) != 1 or (x.shape[0] > 1 and x.stride(0) % 8 != 0) or x.data_ptr() % 16 != 0:
            x = x.contiguous() if x.stride(1) != 1 else x.clone(memory_format=torch.contiguous_format)
        m = x.shape[0]
        if x.shape[1] != k:
            raise RuntimeError(f"size_k mismatch: x has {x.shape[1]} columns, packed weight covers {k}")
        lda = x.stride(0) if m > 1 else k
        x_ptr = x.data_ptr()
    else:
        if not (tp_flags & TP_GATHER_IN) or m is None:
            raise RuntimeError("x may only be omitted for a TP_GATHER_IN launch with m given")
        lda, x_ptr = k, None
    n_outputs = 1 if epilogue == "swiglu" else len(layers)
    if outs is None:
        outs = [torch.empty((m, layers[i][3]), dtype=torch.float16, device=dev) for i in range(n_outputs)]
    arr = (Proj * len(layers))()
    ns = (ctypes.c_int64 * len(layers))()
    for i, (w, s, b, n_out) in enumerate(layers):
        if w.dtype != torch.int32 or s.dtype != torch.float16 or not w.is_contiguous() or not s.is_contiguous():
            raise RuntimeError("weight must be contiguous int32 and scale contiguous float16")
        if w.shape[0] * 16 != k or s.shape[0] * 128 != k or s.shape[1] * 2 != w.shape[1]:
            raise RuntimeError("projections of one launch must share k, with group-128 scales")
        if b is not None and (b.dtype != torch.float16 or b.numel() < n_out or not b.is_contiguous()):
            raise RuntimeError("bias must be a contiguous float16 tensor with at least n_out elements")
        d = outs[min(i, n_outputs - 1)]
        arr[i].B, arr[i].s = w.data_ptr(), s.data_ptr()
        arr[i].bias = b.data_ptr() if b is not None else None
        arr[i].D, arr[i].ldd = d.data_ptr(), d.stride(0)
        arr[i].n, arr[i].n_out = s.shape[1], n_out
        ns[i] = s.shape[1]
    res_ptr, ldr = None, 0
    if residual is not None:
        if residual.dtype != torch.float16 or residual.dim() != 2 or residual.stride(1) != 1:
            raise RuntimeError("residual must be a 2-D float16 tensor with unit column stride")
        res_ptr, ldr = residual.data_ptr(), residual.stride(0)
    pf_arr, npf = None, 0
    if prefetch:
        pf_arr = (Prefetch * 4)()
        for item in prefetch:
            t, nb = item if isinstance(item, tuple) else (item, item.numel() * item.element_size())
            if npf < 4 and nb >= 128:
                pf_arr[npf].ptr, pf_arr[npf].bytes = t.data_ptr(), min(nb, t.numel() * t.element_size())
                npf += 1
    idx = dev.index
    L = lib()
    with torch.cuda.device(dev):
        key = (m, k, tuple(ns), _EPILOGUES[epilogue], hadamard_dim)
        nbytes = _group_need_cache.get(key)
        if nbytes is None:
            nbytes = _group_need_cache[key] = L.uniql_w4a16_group_scratch_bytes(m, k, ns, len(layers), _EPILOGUES[epilogue],
                                                                                 hadamard_dim)
        scratch = _scratch_for(dev, nbytes)
        st = status_word(dev)
        stream = torch._C._cuda_getCurrentRawStream(idx)
        if comm is not None:
            code = L.uniql_w4a16_linear_group_tp(comm, tp_flags, col_offset, k_offset, x_ptr, lda, m, k, arr, len(layers),
                                                 _EPILOGUES[epilogue], res_ptr, ldr, hadamard_dim, pf_arr, npf,
                                                 scratch.data_ptr(), scratch.numel(), st.data_ptr(), stream)
        else:
            code = L.uniql_w4a16_linear_group(x_ptr, lda, m, k, arr, len(layers), _EPILOGUES[epilogue], res_ptr, ldr,
                                              hadamard_dim, pf_arr, npf, scratch.data_ptr(), scratch.numel(),
                                              st.data_ptr(), stream)
    if code != 0:
        check(code, "uniql_w4a16_linear_group")
    return outs


def w4_embedding(ids: torch.Tensor, weight: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """out[..., :] = dequantised rows of the 4-bit table for int64 ids of shape [T] or [B, T]."""
    _require_cuda(ids, "input"); _require_cuda(weight, "weight"); _require_cuda(scales, "scale")
    if weight.dim() != 2 or weight.dtype != torch.int32:
        raise RuntimeError("weight must be a 2-D int32 tensor")
    if scales.dim() != 1 or scales.dtype != torch.float16 or scales.numel() != weight.shape[0]:
        raise RuntimeError("scale must be a 1-D float16 tensor with one entry per table row")
    if ids.dim() not in (1, 2) or ids.dtype != torch.int64:
        raise RuntimeError("input must be a 1-D or 2-D int64 tensor")
    ids_c = ids.contiguous()
    weight = weight.contiguous()
    vocab, words = weight.shape
    dim = words * 8
    out = torch.empty((*ids.shape, dim), dtype=torch.float16, device=ids.device)
    with torch.cuda.device(ids.device):
        code = lib().uniql_w4_embedding(
            ids_c.data_ptr(), ids_c.numel(), weight.data_ptr(), scales.contiguous().data_ptr(), out.data_ptr(),
            vocab, dim, status_word(ids.device).data_ptr(), _stream_handle(ids.device))
    check(code, "uniql_w4_embedding")
    return out


def hadamard(x: torch.Tensor, scale: float) -> torch.Tensor:
    """New tensor y = H x * scale along the last axis (x is made contiguous first)."""
    _require_cuda(x, "x")
    if x.dtype not in _DTYPE_CODE:
        raise RuntimeError(f"unsupported dtype {x.dtype}")
    xc = x.contiguous()
    dim = xc.shape[-1]
    rows = xc.numel() // dim if dim else 0
    y = torch.empty_like(xc)
    with torch.cuda.device(x.device):
        code = lib().uniql_hadamard(xc.data_ptr(), y.data_ptr(), rows, dim, float(scale), _DTYPE_CODE[x.dtype],
                                    _stream_handle(x.device))
    check(code, "uniql_hadamard")
    return y


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up for fp16 CUDA tensors of the same shape, one pass (fp16 SiLU, fp16 product, as the two PyTorch
    ops would round)."""
    _require_cuda(gate, "gate"); _require_cuda(up, "up")
    if gate.dtype != torch.float16 or up.dtype != torch.float16 or gate.shape != up.shape:
        raise RuntimeError("gate and up must be float16 tensors of the same shape")
    cols = gate.shape[-1]
    g2, u2 = gate.reshape(-1, cols), up.reshape(-1, cols)
    if g2.stride(1) != 1 or g2.stride(0) % 8 or g2.data_ptr() % 16:
        g2 = g2.contiguous()
    if u2.stride(1) != 1 or u2.stride(0) % 8 or u2.data_ptr() % 16:
        u2 = u2.contiguous()
    out = torch.empty(g2.shape, dtype=torch.float16, device=gate.device)
    with torch.cuda.device(gate.device):
        code = lib().uniql_silu_mul(g2.data_ptr(), g2.stride(0), u2.data_ptr(), u2.stride(0), out.data_ptr(), cols,
                                    g2.shape[0], cols, _stream_handle(gate.device))
    check(code, "uniql_silu_mul")
    return out.view(gate.shape)


def hadamard_base_matrix(base: int) -> torch.Tensor:
    """The int8 [base, base] matrix of +1 / -1 the library applies for orders 12, 20, 28 and 40 right now."""
    import ctypes
    buf = (ctypes.c_int8 * (base * base))()
    check(lib().uniql_hadamard_base_matrix(int(base), buf), "uniql_hadamard_base_matrix")
    return torch.tensor(list(buf), dtype=torch.int8).reshape(base, base)


def hadamard_set_base_matrix(base: int, matrix=None) -> None:
    """Replace the order-`base` Hadamard matrix (12, 20, 28, 40) for every transform launched afterwards in this
    process; `matrix` is a [base, base] array of +1 / -1 with orthogonal rows, None restores the built-in one.  The
    reference's transforms come from the third-party fast_hadamard_transform package (quantize/hadamard_helpers.py:18-36):
    passing that package's tables here makes this library reproduce them."""
    import ctypes
    if matrix is None:
        check(lib().uniql_hadamard_set_base_matrix(int(base), None), "uniql_hadamard_set_base_matrix")
        return
    m = torch.as_tensor(matrix).to(torch.int8).contiguous().cpu()
    if tuple(m.shape) != (base, base):
        raise RuntimeError(f"matrix must be [{base}, {base}]")
    buf = (ctypes.c_int8 * (base * base))(*m.reshape(-1).tolist())
    check(lib().uniql_hadamard_set_base_matrix(int(base), buf), "uniql_hadamard_set_base_matrix")


def w4a16_quantize(weight: torch.Tensor, group_scale: torch.Tensor | None = None, n_pad: int | None = None,
                   want_ref: bool = True):
    """Quantise and pack an nn.Linear weight [out, in] (fp16, CUDA) on the GPU.

    Returns (w_ref fp16 [Kp, n_pad] or None, packed int32 [Kp/16, 2*n_pad], scales fp16 [Kp/128, n_pad]) with the
    values of the reference's w4a16_quantize(weight.T, 4, 128, group_scale, pad_out) (quantize_helpers.py:184-241);
    n_pad defaults to `out` rounded up to 256 as in W4A16B16O16Linear.from_fp16 (quant_linear_layers.py:65-66)."""
    _require_cuda(weight, "weight")
    if weight.dim() != 2:
        raise RuntimeError("weight must be [out_features, in_features]")
    w = weight.detach()
    if w.dtype != torch.float16:
        w = w.to(torch.float16)
    if w.stride(1) != 1:
        w = w.contiguous()
    n_out, k_in = w.shape
    if n_pad is None:
        n_pad = (n_out + 255) // 256 * 256
    kp = (k_in + 127) // 128 * 128
    gs = None
    if group_scale is not None:
        _require_cuda(group_scale, "group_scale")
        gs = group_scale.detach().to(torch.float16).contiguous()
        if tuple(gs.shape) != (kp // 128, n_out):
            raise RuntimeError(f"group_scale must be [{kp // 128}, {n_out}], got {tuple(gs.shape)}")
    dev = w.device
    packed = torch.empty((kp // 16, 2 * n_pad), dtype=torch.int32, device=dev)
    scales = torch.empty((kp // 128, n_pad), dtype=torch.float16, device=dev)
    w_ref = torch.empty((kp, n_pad), dtype=torch.float16, device=dev) if want_ref else None
    with torch.cuda.device(dev):
        code = lib().uniql_w4a16_quantize(w.data_ptr(), w.stride(0), n_out, k_in,
                                          gs.data_ptr() if gs is not None else None,
                                          packed.data_ptr(), scales.data_ptr(),
                                          w_ref.data_ptr() if w_ref is not None else None, n_pad,
                                          _stream_handle(dev))
    check(code, "uniql_w4a16_quantize")
    return w_ref, packed, scales


def w4a16_gather_columns(weight: torch.Tensor, scale: torch.Tensor, col_index: torch.Tensor, n_out_pad: int,
                         zero_rows_from: int | None = None):
    """New packed layer with output column c = source column col_index[c], zero-padded to n_out_pad columns; rows from
    `zero_rows_from` on get code 0.  Returns (packed int32 [K/16, 2*n_out_pad], scales fp16 [K/128, n_out_pad])."""
    _require_cuda(weight, "weight")
    _require_cuda(scale, "scale")
    dev = weight.device
    size_k, n_src_pad = weight.shape[0] * 16, weight.shape[1] // 2
    idx = col_index.to(device=dev, dtype=torch.int32).contiguous()
    # load-time call: a synchronising range check is affordable, and the CPU path would raise IndexError here too
    # (negative entries are allowed: they produce zero columns)
    if idx.numel() and int(idx.max()) >= n_src_pad:
        raise RuntimeError("col_index out of range")
    weight, scale = weight.contiguous(), scale.contiguous()
    packed = torch.empty((size_k // 16, 2 * n_out_pad), dtype=torch.int32, device=dev)
    scales = torch.empty((size_k // 128, n_out_pad), dtype=torch.float16, device=dev)
    with torch.cuda.device(dev):
        code = lib().uniql_w4a16_gather_columns(weight.data_ptr(), scale.data_ptr(), size_k, n_src_pad, idx.data_ptr(),
                                                idx.numel(), size_k if zero_rows_from is None else zero_rows_from,
                                                packed.data_ptr(), scales.data_ptr(), n_out_pad,
                                                status_word(dev).data_ptr(), _stream_handle(dev))
    check(code, "uniql_w4a16_gather_columns")
    return packed, scales


def w4a16_dequantize_rows(weight: torch.Tensor, scale: torch.Tensor, row_index: torch.Tensor, n_real: int) -> torch.Tensor:
    """fp16 [n_real, len(row_index)]: dequantised weights of the chosen input rows in nn.Linear layout."""
    _require_cuda(weight, "weight")
    _require_cuda(scale, "scale")
    dev = weight.device
    size_k, n_src_pad = weight.shape[0] * 16, weight.shape[1] // 2
    idx = row_index.to(device=dev, dtype=torch.int32).contiguous()
    if idx.numel() and (int(idx.min()) < 0 or int(idx.max()) >= size_k):
        raise RuntimeError("row_index out of range")
    weight, scale = weight.contiguous(), scale.contiguous()
    out = torch.empty((n_real, idx.numel()), dtype=torch.float16, device=dev)
    with torch.cuda.device(dev):
        code = lib().uniql_w4a16_dequantize_rows(weight.data_ptr(), scale.data_ptr(), size_k, n_src_pad, idx.data_ptr(),
                                                 idx.numel(), n_real, out.data_ptr(), idx.numel(),
                                                 status_word(dev).data_ptr(), _stream_handle(dev))
    check(code, "uniql_w4a16_dequantize_rows")
    return out
