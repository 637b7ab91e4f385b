"""CPU, world_size 2 over gloo: tensor-parallel shard arithmetic and the reductions around it.
The per-rank matmul is done by the oracle (there is no CPU kernel); what is under test is the sharding of the
packed buffers, the uneven splits, the all-reduce of row-parallel partials and the feature all-gather."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import uniql_oracle as orc
from uniql_b200 import tp
from uniql_b200.quantize.quant_linear_layers import W4A16B16O16Linear


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        hidden, inter, m = 256, 640, 3                     # 640 = 5 groups of 128 / 10 blocks of 64: uneven over 2 ranks
        up = W4A16B16O16Linear.from_fp16(torch.nn.Linear(hidden, inter, bias=True).half())
        down = W4A16B16O16Linear.from_fp16(torch.nn.Linear(inter, hidden, bias=True).half())
        x = torch.randn(m, hidden).half()

        def deq(mod):
            return orc.dequantize(mod.weight.numpy(), mod.scale.numpy()).astype(np.float32)

        # full (unsharded) result
        h_full = x.float().numpy() @ deq(up)[:, :inter] + up.bias.data.float().numpy()
        h_full16 = h_full.astype(np.float16)
        y_full = h_full16.astype(np.float32) @ deq(down)[:, :hidden] + down.bias.data.float().numpy()

        # column-parallel `up`: boundaries chosen so that they match the row split of `down`
        rows = tp.row_bounds(down.size_k, world)
        col = tp.ColumnParallelW4A16Linear(up, rank, world, bounds=[(a, b) for a, b in rows[:-1]] + [(rows[-1][0], up.size_n)])
        row = tp.RowParallelW4A16Linear(down, rank, world)
        assert (col.n0, min(col.n1, inter)) == (row.k0, row.k1)
        h_local = x.float().numpy() @ deq(col.local)[:, :col.out_features_local]
        h_local = (h_local + col.local.bias.data.float().numpy()).astype(np.float16)
        assert np.array_equal(h_local, h_full16[:, col.n0:col.n0 + col.out_features_local])

        # feature all-gather with uneven shard widths
        sizes = [min(b, inter) - a for a, b in rows]
        gathered = tp.all_gather_features(torch.from_numpy(h_local), sizes)
        assert np.array_equal(gathered.numpy(), h_full16)

        # row-parallel `down`: partial sums, all-reduce, bias once
        part = torch.from_numpy(h_local.astype(np.float32) @ deq(row.local)[:, :hidden])
        dist.all_reduce(part)
        y = part.numpy() + down.bias.data.float().numpy()
        assert np.allclose(y, y_full, rtol=1e-4, atol=1e-4)
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_column_row_parallel_pair_world2():
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {0: "ok", 1: "ok"}


@pytest.mark.parametrize("units,world", [(148, 8), (32, 8), (7, 4), (3, 8)])
def test_balanced_splits(units, world):
    s = tp.balanced_splits(units, world)
    assert s[0][0] == 0 and s[-1][1] == units
    sizes = [b - a for a, b in s]
    assert all(a[1] == b[0] for a, b in zip(s, s[1:])) and max(sizes) - min(sizes) <= 1


def test_shards_are_plain_slices_of_the_packed_layout():
    from uniql_b200.quantize import quantize_helpers as qh
    q = W4A16B16O16Linear.from_fp16(torch.nn.Linear(512, 320, bias=False).half())
    w = qh.w4a16_dequantize(q.weight, q.scale)
    for world in (2, 3, 4):
        for r in range(world):
            c = tp.ColumnParallelW4A16Linear(q, r, world)
            assert torch.equal(qh.w4a16_dequantize(c.local.weight, c.local.scale), w[:, c.n0:c.n1])
            rr = tp.RowParallelW4A16Linear(q, r, world)
            assert torch.equal(qh.w4a16_dequantize(rr.local.weight, rr.local.scale), w[rr.k0:rr.k1])
    w2, s2 = tp.gather_columns(q.weight, q.scale, torch.arange(10, 100))
    assert torch.equal(qh.w4a16_dequantize(w2, s2)[:, :90], w[:, 10:100])
