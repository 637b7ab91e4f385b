"""Tensor-parallel sharding of W4A16 linears across the GPUs of one node (one process per GPU).

The reference has no distributed layer; this is the Megatron-style split its packed layout permits:

* column-parallel (q/k/v, gate/up, in_proj, lm_head): shard the output features N.  The packed weight
  permutes values only inside 16-row x 64-column blocks and the scales only inside 64-column blocks
  (quantize/quantize_helpers.py:38-62, 145-180 in UniQL), so a shard that starts and ends on a multiple of
  64 columns is a plain slice ``weight[:, 2*n0:2*n1]``, ``scale[:, n0:n1]``.  Other boundaries go through
  unpack -> gather -> repack (the recipe of modeling/modeling_helpers.py:665-767).
* row-parallel (o_proj, down_proj, out_proj): shard the input features K on multiples of 128
  (8 packed rows = 1 scale row): ``weight[kt0:kt1]``, ``scale[g0:g1]``; every rank produces a partial
  [M, N] that is summed with an all-reduce; the bias is added once, after the reduction.
* an online Hadamard in front of a row-parallel linear mixes the whole K axis: the column-parallel
  producers' shards are all-gathered, each rank transforms the full row and keeps its K slice.

Collectives go through torch.distributed (NCCL on GPUs, gloo in CPU tests).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from .quantize import quantize_helpers as qh
from .quantize.quant_linear_layers import W4A16B16O16Linear


def balanced_splits(units: int, world: int):
    """[(start, end)] * world: contiguous, sizes differ by at most one unit."""
    return [(units * r // world, units * (r + 1) // world) for r in range(world)]


def column_bounds(n_stored: int, world: int, unit: int = 64):
    """Column ranges (multiples of `unit`, default one 64-column packing block) for each rank."""
    assert n_stored % unit == 0
    return [(a * unit, b * unit) for a, b in balanced_splits(n_stored // unit, world)]


def row_bounds(k_stored: int, world: int, unit: int = 128):
    """Input-feature ranges (multiples of one quantisation group) for each rank."""
    assert k_stored % unit == 0
    return [(a * unit, b * unit) for a, b in balanced_splits(k_stored // unit, world)]


def shard_columns(weight: torch.Tensor, scale: torch.Tensor, n0: int, n1: int):
    """Packed buffers restricted to output columns [n0, n1); both multiples of 64."""
    assert n0 % 64 == 0 and n1 % 64 == 0 and 0 <= n0 < n1 <= scale.shape[1]
    return weight[:, 2 * n0:2 * n1].contiguous(), scale[:, n0:n1].contiguous()


def shard_rows(weight: torch.Tensor, scale: torch.Tensor, k0: int, k1: int):
    """Packed buffers restricted to input features [k0, k1); both multiples of 128."""
    assert k0 % 128 == 0 and k1 % 128 == 0 and 0 <= k0 < k1 <= weight.shape[0] * 16
    return weight[k0 // 16:k1 // 16].contiguous(), scale[k0 // 128:k1 // 128].contiguous()


def gather_columns(weight: torch.Tensor, scale: torch.Tensor, cols: torch.Tensor):
    """Arbitrary output-column selection (e.g. head or segment boundaries that are not multiples of 64):
    unpack, gather, pad the width up to a multiple of 64 with zero codes/scales, repack."""
    q = qh.unpack_w4a16(weight)[:, cols]
    s = qh.unpermute_group_scales(scale)[:, cols]
    pad = (-q.shape[1]) % 64
    if pad:
        q = torch.nn.functional.pad(q, (0, pad))
        s = torch.nn.functional.pad(s, (0, pad))
    return qh.pack_w4a16(q), qh.permute_group_scales(s)


def _local_linear(weight, scale, bias, in_features, out_features, cls=W4A16B16O16Linear):
    lin = cls(in_features, out_features, bias=bias is not None, device="meta")
    lin.size_k, lin.size_n = weight.shape[0] * 16, weight.shape[1] // 2
    lin.pad_in = lin.size_k - in_features
    lin.pad_out = lin.size_n - out_features
    lin._buffers["weight"] = weight
    lin._buffers["scale"] = scale
    lin._buffers["workspace"] = torch.zeros(lin.size_n // 64 * 16, dtype=torch.int32, device=weight.device)
    if bias is not None:
        lin.bias = nn.Parameter(bias, requires_grad=False)
    return lin


class ColumnParallelW4A16Linear(nn.Module):
    """This rank's slice of the output features of a W4A16 linear; the output stays sharded."""

    def __init__(self, full: W4A16B16O16Linear, rank: int, world: int, bounds=None):
        super().__init__()
        bounds = bounds or column_bounds(full.size_n, world)
        n0, n1 = bounds[rank]
        w, s = shard_columns(full.weight, full.scale, n0, n1)
        n_real = max(0, min(n1, full.out_features) - n0)       # columns of this shard that are not padding
        b = full.bias.data[n0:n0 + n_real].contiguous() if full.bias is not None else None
        self.n0, self.n1, self.out_features_local = n0, n1, n_real
        self.local = _local_linear(w, s, b, full.in_features, n_real, type(full))

    def forward(self, x):
        return self.local(x)


class RowParallelW4A16Linear(nn.Module):
    """This rank's slice of the input features; partial outputs are summed over the process group."""

    def __init__(self, full: W4A16B16O16Linear, rank: int, world: int, group=None, bounds=None, fused=None):
        """fused: a PushAllReduce; when given, decode-size calls (m <= 16) do the cross-GPU sum inside the linear
        kernel instead of a separate collective."""
        super().__init__()
        self.fused = fused
        bounds = bounds or row_bounds(full.size_k, world)
        k0, k1 = bounds[rank]
        w, s = shard_rows(full.weight, full.scale, k0, k1)
        self.k0, self.k1 = k0, k1
        self.group, self.world = group, world
        self.bias = full.bias                                   # added once, after the reduction
        self.local = _local_linear(w, s, None, k1 - k0, full.out_features)

    def forward(self, x_local):
        if self.world > 1 and self.fused is not None:
            x2 = x_local.reshape(-1, x_local.shape[-1])
            if self.fused.fits_fused(x2.shape[0], self.local.size_n):
                b = self.bias.data if self.bias is not None else None
                y = self.fused.linear_all_reduce(x2, self.local.weight, self.local.scale, b, self.local.out_features)
                return y.view(*x_local.shape[:-1], self.local.out_features)
        y = self.local(x_local)
        if self.world > 1:
            dist.all_reduce(y, group=self.group)
        if self.bias is not None:
            y = y + self.bias
        return y


def all_gather_features(x_local: torch.Tensor, sizes, group=None) -> torch.Tensor:
    """Concatenate column shards [.., sizes[r]] of every rank along the last axis (uneven sizes allowed)."""
    world = len(sizes)
    if world == 1:
        return x_local
    width = max(sizes)
    padded = x_local if x_local.shape[-1] == width else torch.nn.functional.pad(x_local, (0, width - x_local.shape[-1]))
    out = torch.empty((world, *padded.shape), dtype=padded.dtype, device=padded.device)
    dist.all_gather([out[r] for r in range(world)], padded.contiguous(), group=group)
    return torch.cat([out[r][..., :sizes[r]] for r in range(world)], dim=-1)


class PushAllReduce:
    """Latency-optimised all-reduce (sum) of fp16 tensors for decode-size messages, backed by
    `uniql_allreduce_push`: every rank stores its partial into each peer's staging buffer over NVLink and sums
    locally.  Set-up exchanges CUDA IPC handles through the (host side of the) process group.  Messages that
    do not fit (or are not fp16 / not a multiple of 8 elements) go through `dist.all_reduce`."""

    def __init__(self, group=None, max_elems: int = 16 * 16384, device=None):
        import ctypes

        from ._lib import check, lib
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.max_elems = max_elems
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self._lib = lib()
        self._comm = ctypes.c_void_p()
        nbytes = self._lib.uniql_comm_handle_bytes()
        handle = ctypes.create_string_buffer(nbytes)
        with torch.cuda.device(self.device):
            check(self._lib.uniql_comm_create(self.rank, self.world, max_elems, ctypes.byref(self._comm), handle),
                  "uniql_comm_create")
            handles = [None] * self.world
            dist.all_gather_object(handles, handle.raw, group=group)
            blob = ctypes.create_string_buffer(b"".join(handles), nbytes * self.world)
            check(self._lib.uniql_comm_connect(self._comm, blob), "uniql_comm_connect")
        dist.barrier(group=group)
        from . import ops
        self._status = ops.status_word(self.device)

    @classmethod
    def single_rank(cls, max_elems: int = 16 * 16384, device=None):
        """A communicator of world size 1 that needs no process group: the exchanges of the tensor-parallel launches
        (epoch-tagged words, parities, feature area) then run against this GPU's own block.  For tests and for code
        that is written against the tensor-parallel calls but runs on one GPU."""
        import ctypes

        from ._lib import check, lib
        self = cls.__new__(cls)
        self.group, self.rank, self.world, self.max_elems = None, 0, 1, max_elems
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self._lib = lib()
        self._comm = ctypes.c_void_p()
        nbytes = self._lib.uniql_comm_handle_bytes()
        handle = ctypes.create_string_buffer(nbytes)
        with torch.cuda.device(self.device):
            check(self._lib.uniql_comm_create(0, 1, max_elems, ctypes.byref(self._comm), handle), "uniql_comm_create")
            check(self._lib.uniql_comm_connect(self._comm, handle), "uniql_comm_connect")
        from . import ops
        self._status = ops.status_word(self.device)
        return self

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        """In-place sum over the group; returns t."""
        n = t.numel()
        if (t.dtype != torch.float16 or not t.is_contiguous() or n % 8 != 0 or n > self.max_elems
                or t.data_ptr() % 16 != 0):
            if self.world > 1:
                dist.all_reduce(t, group=self.group)
            return t
        from ._lib import check
        code = self._lib.uniql_allreduce_push(self._comm, t.data_ptr(), t.data_ptr(), n, self._status.data_ptr(),
                                              torch._C._cuda_getCurrentRawStream(self.device.index))
        check(code, "uniql_allreduce_push")
        return t

    def all_gather_features(self, x_local: torch.Tensor, sizes) -> torch.Tensor:
        """Concatenation of the ranks' column shards, done as a sum of zero-padded rows (one push all-reduce)."""
        offs = [0]
        for s in sizes:
            offs.append(offs[-1] + s)
        full = torch.zeros((*x_local.shape[:-1], offs[-1]), dtype=x_local.dtype, device=x_local.device)
        full[..., offs[self.rank]:offs[self.rank + 1]] = x_local
        return self.all_reduce(full)

    def fits_fused(self, m: int, n_stored: int) -> bool:
        """The fused exchanges hold 16 batch rows of up to max_elems / 16 columns."""
        return m <= 16 and 16 * n_stored <= self.max_elems

    def linear_all_reduce(self, x, weight, scale, bias, n_out, residual=None):
        """Row-parallel W4A16 linear + sum over ranks (+ bias, + residual) in one kernel launch.  Calls of different
        shapes may share the communicator (staging is addressed per 64-column block, each with its own epoch)."""
        from . import ops
        return ops.w4a16_linear_group(x, [(weight, scale, bias, n_out)], residual=residual, comm=self._comm,
                                      tp_flags=ops.TP_REDUCE)[0]

    def gate_up_gather(self, x, gate, up, col_offset: int):
        """Column-parallel gate/up shard: h = silu(gate x) * (up x) in one launch whose epilogue also stores the
        result columns, from feature index col_offset on, into every rank's feature area.  gate / up are
        (weight, scale, bias, n_out).  Returns this rank's shard of h."""
        from . import ops
        return ops.w4a16_linear_group(x, [gate, up], epilogue="swiglu", comm=self._comm, tp_flags=ops.TP_GATHER_OUT,
                                      col_offset=col_offset)[0]

    def down_gather_reduce(self, m: int, down, hadamard_dim: int, k_offset: int, residual=None):
        """Row-parallel down/out projection of the row gathered by the preceding gate_up_gather: every rank
        transforms the full row (Hadamard of hadamard_dim points, a few-row kernel that reads the words straight from
        this rank's feature area and waits, bounded, for those that have not arrived), multiplies its own k slice
        (from feature k_offset on) and the partial results are summed over the ranks in the linear's epilogue.  The two
        launches are chained by programmatic dependent launch; no collective call, no host step in between."""
        from . import ops
        return ops.w4a16_linear_group(None, [down], residual=residual, hadamard_dim=hadamard_dim, comm=self._comm,
                                      tp_flags=ops.TP_GATHER_IN | ops.TP_REDUCE, k_offset=k_offset, m=m)[0]

    def close(self):
        if self._comm:
            self._lib.uniql_comm_destroy(self._comm)
            self._comm = None
