"""Worker for the multi-GPU push all-reduce check; launched by tests/test_gpu_tp_multi.py or by hand:
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 tests/tp_push_worker.py"""
import datetime
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
    from uniql_b200 import ops, tp
    ar = tp.PushAllReduce(max_elems=16 * 16384)
    ok = True
    fails = []

    def check(cond, what):
        nonlocal ok
        if not bool(cond):
            ok = False
            fails.append(what)

    for it, n in enumerate([4096, 8, 16 * 4096, 14336, 4096, 4096, 16 * 16384]):
        g = torch.Generator(device=dev).manual_seed(100 * it + rank)
        x = torch.randn(n, device=dev, generator=g).half()
        want = x.clone()
        dist.all_reduce(want)
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x)
        exact = torch.stack(parts).float().sum(0).half()        # rank-order fp32 sum, one rounding
        got = ar.all_reduce(x.clone())
        torch.cuda.synchronize()
        ok &= bool(torch.equal(got, exact))
        ok &= bool(torch.allclose(got.float(), want.float(), rtol=2e-3, atol=2e-3))
    # CUDA-graph replay keeps working because the epoch lives on the device
    x = torch.ones(4096, device=dev).half() * (rank + 1)
    buf = x.clone()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        ar.all_reduce(buf.clone())
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            buf.copy_(x)
            ar.all_reduce(buf)
        for _ in range(5):
            graph.replay()
        torch.cuda.synchronize()
    ok &= bool((buf == world * (world + 1) / 2).all())
    sizes = [3, 5] if world == 2 else [2] * world
    sizes = [8 * s for s in sizes]
    shard = torch.full((2, sizes[rank]), float(rank + 1), device=dev).half()
    gathered = ar.all_gather_features(shard, sizes)
    torch.cuda.synchronize()
    off = 0
    for r, sz in enumerate(sizes):
        ok &= bool((gathered[:, off:off + sz] == r + 1).all())
        off += sz
    # ---- fused row-parallel linear + all-reduce equals linear followed by the stand-alone push all-reduce.
    # ONE communicator serves every shape, and the shapes alternate call by call: the staging words are addressed per
    # 64-column block with per-block epochs, so a change of width must not pick up words of an earlier call ----
    from uniql_b200.quantize.quant_linear_layers import W4A16B16O16HadLinear, W4A16B16O16Linear
    torch.manual_seed(5)                                    # same full layers on every rank
    chan = tp.PushAllReduce(max_elems=16 * 16384)
    cases = []
    for n, k, m in [(4096, 4096, 1), (1024, 2048, 16), (4096, 14336, 4), (512, 1024, 2)]:
        full = W4A16B16O16Linear.from_fp16(torch.nn.Linear(k, n, bias=True).half()).to(dev)
        cases.append((full, tp.RowParallelW4A16Linear(full, rank, world, fused=chan),
                      tp.RowParallelW4A16Linear(full, rank, world), m, k))
    for call in range(3):
        for full, row_fused, row_plain, m, k in cases:
            xfull = torch.randn(m, k, device=dev, generator=torch.Generator(device=dev).manual_seed(77 + call)).half()
            xin = xfull[:, row_plain.k0:row_plain.k1]
            y_f = row_fused(xin)
            part = row_plain.local(xin)
            y_p = ar.all_reduce(part.clone().view(-1)).view_as(part)
            torch.cuda.synchronize()
            check(torch.allclose(y_f.float(), (y_p.float() + full.bias.float()), rtol=2e-3, atol=2e-3 * max(1.0, float(y_p.float().abs().max()))), f"fused vs push m={m} k={k} call {call}")
            y_full = full(xfull)
            check(torch.allclose(y_f.float(), y_full.float(), rtol=2e-2, atol=2e-2 * float(y_full.float().abs().max())), f"fused vs unsharded m={m} k={k} call {call}")
    # ---- the decode MLP of a tensor-parallel layer in two launches: gate/up shard with SwiGLU whose epilogue stores
    # the activated columns into every rank's feature area, then the down shard that reads the full row there,
    # transforms it (Hadamard kernel reading the feature area), multiplies its k slice and sums over the ranks in its epilogue ----
    from uniql_b200 import fused as fz
    # (the gather path transforms in 256-point segments or longer: 14336 = 28 x 512, 8192 = 16 x 512)
    for hidden, inter, m in [(4096, 14336, 16), (4096, 14336, 1), (4096, 14336, 4), (4096, 8192, 2)]:
        if (inter // 64) % world or (inter // 128) % world:
            continue
        gate = W4A16B16O16Linear.from_fp16(torch.nn.Linear(hidden, inter, bias=False).half()).to(dev)
        up = W4A16B16O16Linear.from_fp16(torch.nn.Linear(hidden, inter, bias=False).half()).to(dev)
        down = W4A16B16O16HadLinear.from_fp16(torch.nn.Linear(inter, hidden, bias=False).half()).to(dev)
        c0, c1 = tp.column_bounds(inter, world)[rank]
        k0, k1 = tp.row_bounds(inter, world)[rank]
        assert (c0, c1) == (k0, k1)
        gw, gs = tp.shard_columns(gate.weight, gate.scale, c0, c1)
        uw, us = tp.shard_columns(up.weight, up.scale, c0, c1)
        dw, ds = tp.shard_rows(down.weight, down.scale, k0, k1)
        for call in range(3):
            x = torch.randn(m, hidden, device=dev, generator=torch.Generator(device=dev).manual_seed(9 + call)).half()
            res = torch.randn(m, hidden, device=dev, generator=torch.Generator(device=dev).manual_seed(19 + call)).half()
            h_loc = chan.gate_up_gather(x, (gw, gs, None, c1 - c0), (uw, us, None, c1 - c0), c0)
            y = chan.down_gather_reduce(m, (dw, ds, None, hidden), inter, k0, residual=res)
            torch.cuda.synchronize()
            h_full = fz.gate_up_swiglu(gate, up, x)
            # the shard comes from the kernel with the cross-GPU epilogue, the full row from the single-GPU kernel: same
            # arithmetic, another order of the fp32 sums
            check(torch.allclose(h_loc.float(), h_full[:, c0:c1].float(), rtol=1e-2, atol=1e-2 * float(h_full.float().abs().max())), f"gate_up shard {hidden}x{inter} m={m}")
            y_full = fz.linear_residual(down, h_full, res)
            lin = (y_full.float() - res.float())
            check(torch.allclose(y.float(), y_full.float(), rtol=2e-2, atol=2e-2 * float(lin.abs().max())), f"down gather+reduce {hidden}x{inter} m={m} call {call}")
    check(ops.read_and_clear_status(dev) == 0, "status word")
    if fails:
        print(f"rank {rank} failures: {fails[:8]}", flush=True)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("PUSH_ALLREDUCE_OK" if int(flag.item()) == 1 else "PUSH_ALLREDUCE_FAILED", flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
