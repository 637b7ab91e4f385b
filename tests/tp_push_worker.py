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
    # ---- fused row-parallel linear + all-reduce equals linear followed by the stand-alone push all-reduce ----
    from uniql_b200.quantize.quant_linear_layers import W4A16B16O16Linear
    torch.manual_seed(5)                                    # same full layer on every rank
    for n, k, m in [(4096, 4096, 1), (1024, 2048, 16), (4096, 14336, 4)]:
        full = W4A16B16O16Linear.from_fp16(torch.nn.Linear(k, n, bias=True).half()).to(dev)
        chan = tp.PushAllReduce(max_elems=16 * 4096)          # one channel per call-site shape
        row_fused = tp.RowParallelW4A16Linear(full, rank, world, fused=chan)
        row_plain = tp.RowParallelW4A16Linear(full, rank, world)
        g = torch.Generator(device=dev).manual_seed(77)
        xin = torch.randn(m, k, device=dev, generator=g).half()[:, row_plain.k0:row_plain.k1]
        for call in range(3):
            y_f = row_fused(xin * (call + 1))
            part = row_plain.local(xin * (call + 1))
            y_p = ar.all_reduce(part.clone().view(-1)).view_as(part)
            torch.cuda.synchronize()
            ok &= bool(torch.allclose(y_f.float(), (y_p.float() + full.bias.float()), rtol=2e-3, atol=2e-3))
            y_full = full(torch.randn(m, k, device=dev, generator=torch.Generator(device=dev).manual_seed(77)).half() * (call + 1))
            ok &= bool(torch.allclose(y_f.float(), y_full.float(), rtol=2e-2, atol=2e-2 * float(y_full.float().abs().max())))
    ok &= ops.read_and_clear_status(dev) == 0
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("PUSH_ALLREDUCE_OK" if int(flag.item()) == 1 else "PUSH_ALLREDUCE_FAILED", flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
