#!/usr/bin/env python
"""Benchmark of the W4A16 hot path on the Llama-3.1-8B decoder projection set (synthetic weights).

    python bench.py --gpus N --steps K --warmup W            # this build (CUDA kernels)
    python bench.py --impl reference --steps K --warmup W     # CPU dequantise + matmul (the reference's math)

One step = one pass over the 32-layer stack of projections (qkv 6144x4096, o 4096x4096, gate and up
14336x4096 as one launch with the SwiGLU product in its epilogue, down 4096x14336 with a 14336-point online
Hadamard on its input) at decode batch M, replayed from a CUDA graph.
With N > 1 the linears are tensor-parallel (column-parallel qkv/gate/up, row-parallel o/down; the cross-GPU sums and
the feature gather run inside the linears' own launches) and the sharded result is checked against the unsharded layer
before anything is timed (`tp_parity`; a failure exits with code 4).
Prints ONE JSON line on rank 0: the headline (`value`, `roofline`, `e2e`, `cpu_baseline`, `clocks`, `gpu_launches`)
plus extra keys -- step percentiles, the same stack at 16 and 64 rows, the tensor-core kernels at 64 and 4096 rows,
the Qwen2.5-7B and Mamba2-8B legs and the auxiliary kernels (one GPU only).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HIDDEN, INTER, QKV, LAYERS = 4096, 14336, 6144, 32
SHAPES = {"qkv": (QKV, HIDDEN), "o": (HIDDEN, HIDDEN), "gate": (INTER, HIDDEN), "up": (INTER, HIDDEN),
          "down": (HIDDEN, INTER)}
FALLBACK_HBM_GBS = 6650.0        # HBM copy bandwidth of a B200 (GB/s), used only if MEASURED_PEAKS.json is absent
# DRAM bytes read + written by one fused gate+up launch (two 14336x4096 projections, m = 1) as counted by the
# profiler (dram__bytes_read.sum + dram__bytes_write.sum = 60,643,072 + 201,472) in one capture of that launch
NCU_TRAFFIC_GATE_UP_M1 = 60844544


def linear_bytes(n, k, m):
    """Algorithmic bytes of one W4A16 linear: packed weights + group scales + activations in + out."""
    return k * n // 2 + (k // 128) * n * 2 + m * k * 2 + m * n * 2


def gate_up_bytes(n, k, m):
    """Algorithmic bytes of the fused gate+up launch: two packed weights + scales, activations in, one result out."""
    return 2 * (k * n // 2 + (k // 128) * n * 2) + m * k * 2 + m * n * 2


def step_bytes(m):
    return LAYERS * sum(linear_bytes(n, k, m) for n, k in SHAPES.values())


def step_flops(m):
    return LAYERS * sum(2 * m * n * k for n, k in SHAPES.values())


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured", d
    return FALLBACK_HBM_GBS, "fallback", {}


class ClockSampler:
    """Samples SM clock and throttle reasons beside the timed region (read-only NVML queries in a thread)."""
    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = None
        self._thread = None

    def start(self):
        import threading
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = self.gpu_index
            if visible:
                try:
                    idx = int(visible.split(",")[self.gpu_index])
                except (ValueError, IndexError):
                    idx = self.gpu_index
            handle = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            return
        self._stop = threading.Event()

        def loop():
            while not self._stop.is_set():
                try:
                    self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)))
                    mask = pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle)
                    for name, bit in self.REASONS.items():
                        if mask & bit:
                            self.reasons.add(name)
                except Exception:
                    pass
                time.sleep(0.002)

        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()

    def stop(self):
        if self._thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable"]}
        self._stop.set()
        self._thread.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ----------------------------------------------------------------------------------------- CPU arm
def cpu_linear_sample(m, threads, budget_s):
    """Time the reference's CPU path (unpack + un-permute + (q-8)*s dequantise, then matmul) on a bounded
    sample of the workload.  Returns (bytes_processed, seconds_dequant, seconds_matmul, description)."""
    import numpy as np
    import torch

    from oracle import uniql_oracle as orc
    torch.set_num_threads(threads)
    rng = np.random.default_rng(0)
    # probe with one o_proj-sized linear, then decide how much of a layer fits the budget
    def one(n, k):
        packed = rng.integers(-2 ** 31, 2 ** 31 - 1, size=(k // 16, 2 * n), dtype=np.int64).astype(np.int32)
        scales = (rng.random((k // 128, n), dtype=np.float32) * 0.01 + 0.001).astype(np.float16)
        x = torch.from_numpy(rng.standard_normal((m, k), dtype=np.float32).astype(np.float16))
        t0 = time.perf_counter()
        w = orc.dequantize(packed, scales)
        t1 = time.perf_counter()
        wt = torch.from_numpy(w)
        y = x.float() @ wt.float()
        t2 = time.perf_counter()
        return t1 - t0, t2 - t1, float(y[0, 0])

    td, tm, _ = one(HIDDEN, HIDDEN)
    nbytes = linear_bytes(HIDDEN, HIDDEN, m)
    desc = "o_proj 4096x4096"
    per_weight = (td + tm) / (HIDDEN * HIDDEN)
    layer_weights = sum(n * k for n, k in SHAPES.values())
    if per_weight * layer_weights < budget_s:
        td = tm = 0.0
        nbytes = 0
        for name, (n, k) in SHAPES.items():
            a, b, _ = one(n, k)
            td += a; tm += b
            nbytes += linear_bytes(n, k, m)
        desc = "one decoder layer (qkv, o, gate, up, down; Hadamard not included)"
    return nbytes, td, tm, desc


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    m = args.batch
    total = max(1, args.steps + args.warmup)
    budget = max(2.0, 150.0 / total)
    times, nbytes, desc, td_last, tm_last = [], 0, "", 0.0, 0.0
    for i in range(total):
        nbytes, td, tm, desc = cpu_linear_sample(m, threads, budget)
        if i >= args.warmup:
            times.append(td + tm)
            td_last, tm_last = td, tm
    t = sum(times) / len(times)
    gbs = nbytes / t / 1e9
    line = {
        "impl": "reference", "metric": "w4a16_linear_m1_hbm_gbs", "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16xint4->f32acc",
        "data": "synthetic",
        "config": {"workload": "Llama-3.1-8B decoder projection set, W4A16 g128, decode batch %d" % m,
                   "sample_per_step": desc},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": desc,
                         "dequant_s": td_last, "matmul_s": tm_last},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "decode_tok_s": m / (t * step_bytes(m) / nbytes),
    }
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------- GPU arm
def aux_kernels(device, stream, peak):
    """The other kernels of the path on DRAM-sized inputs (N=1 only): embedding gather, Hadamard, quantise + pack.
    Each entry: CUDA-event time per launch, algorithmic GB/s and its fraction of the HBM peak used for `roofline`."""
    import torch

    from uniql_b200 import ops

    def timed(fn, reps=5):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / reps

    def entry(us, nbytes, what):
        gbs = nbytes / (us * 1e-6) / 1e9
        return {"us_per_launch": us, "bytes": nbytes, "gbs": gbs, "frac_of_hbm_peak": gbs / peak, "workload": what}

    out = {}
    g = torch.Generator(device=device).manual_seed(7)
    # embedding: Qwen2.5-7B table (152064 x 3584, 4-bit, one fp16 scale per row), 32768 random token ids
    vocab, dim, tokens = 152064, 3584, 32768
    table = torch.randint(-2 ** 31, 2 ** 31 - 1, (vocab, dim // 8), generator=g, device=device, dtype=torch.int64).to(torch.int32)
    scales = (torch.rand(vocab, generator=g, device=device) * 0.01 + 0.001).to(torch.float16)
    ids = torch.randint(0, vocab, (tokens,), generator=g, device=device, dtype=torch.int64)
    us = timed(lambda: ops.w4_embedding(ids, table, scales))
    out["w4_embedding"] = entry(us, tokens * (dim // 2 + 2 + 8 + 2 * dim), f"{tokens} ids into a {vocab}x{dim} table")
    del table, scales, ids
    # Hadamard 14336 = 28 x 512 (down_proj input): 16384 rows (prefill) and 1 row (decode latency)
    rows, hd = 16384, 14336
    x = torch.randn(rows, hd, generator=g, device=device).to(torch.float16)
    us = timed(lambda: ops.hadamard(x, hd ** -0.5))
    out["hadamard_14336_rows16384"] = entry(us, 2 * rows * hd * 2, f"{rows} x {hd} fp16 in and out")
    x1 = x[:1].contiguous()
    us = timed(lambda: ops.hadamard(x1, hd ** -0.5), reps=20)
    out["hadamard_14336_rows1"] = entry(us, 2 * hd * 2, "1 row: launch and latency bound, not a bandwidth figure")
    del x, x1
    # RTN quantise + pack of one gate projection (no w_ref output); two weights in turn
    n, k = SHAPES["gate"]
    ws = [(torch.randn(n, k, generator=g, device=device) * 0.02).to(torch.float16) for _ in range(2)]
    state = {"i": 0}

    def quant():
        state["i"] ^= 1
        ops.w4a16_quantize(ws[state["i"]], n_pad=n, want_ref=False)

    us = timed(quant, reps=6)
    out["w4a16_quantize"] = entry(us, n * k * 2 + n * k // 2 + (k // 128) * n * 2,
                                  f"{n}x{k} fp16 weight -> packed int4 + scales (includes the output allocation)")
    return out


def build_stack(m, rank, world, device, layers):
    """Synthetic RTN-quantised layers (seeded), sharded for this rank."""
    import torch

    from uniql_b200 import ops, tp
    from uniql_b200.quantize.quant_linear_layers import W4A16B16O16HadLinear, W4A16B16O16Linear

    def quantised(seed, n, k, cls, col=None, row=None):
        g = torch.Generator(device=device).manual_seed(seed)
        w = (torch.randn(n, k, generator=g, device=device) * 0.02).to(torch.float16)
        if col is not None:
            w = w[col[0]:col[1]]
        if row is not None:
            w = w[:, row[0]:row[1]]
        # RTN group-128 quantise + pack on the GPU (same bits as qh.w4a16_quantize(w.t(), 4, 128, None, 0))
        _, packed, scale = ops.w4a16_quantize(w, n_pad=w.shape[0], want_ref=False)
        lin = cls(w.shape[1], w.shape[0], device="meta")
        lin._buffers["weight"], lin._buffers["scale"] = packed, scale
        lin._buffers["workspace"] = torch.zeros(lin.size_n // 64 * 16, dtype=torch.int32, device=device)
        return lin

    stack = []
    for l in range(layers):
        mods = {}
        for j, (name, (n, k)) in enumerate(SHAPES.items()):
            seed = 1000 * l + j
            if name in ("qkv", "gate", "up"):
                mods[name] = quantised(seed, n, k, W4A16B16O16Linear, col=tp.column_bounds(n, world)[rank])
            elif name == "o":
                mods[name] = quantised(seed, n, k, W4A16B16O16Linear, row=tp.row_bounds(k, world)[rank])
            else:
                cls = W4A16B16O16HadLinear if world == 1 else W4A16B16O16Linear
                mods[name] = quantised(seed, n, k, cls, row=tp.row_bounds(k, world)[rank])
        stack.append(mods)
    return stack


def _triple(mod):
    return (mod.weight, mod.scale, mod.bias, mod.out_features)


def make_step(stack, world, rank, group, mode="none", comm=None, taps=None):
    """Returns step(x) -> y running the projections of every layer: qkv -> o -> [gate, up, SwiGLU] -> Hadamard -> down
    (no attention maths: the q shard stands in for the attention output).  Five launches per layer at decode sizes
    (qkv, o, gate+up with SwiGLU, Hadamard, down).
    mode (world > 1): "fused" = cross-GPU sums and the feature gather inside the decode kernels, "push" = separate
    push all-reduce kernels, "nccl" = torch.distributed collectives.  taps: list that receives the two row-parallel
    outputs (o_proj, down_proj) of every layer."""
    import torch.distributed as dist

    from uniql_b200 import fused as fz
    from uniql_b200 import ops, tp
    o_rows = tp.row_bounds(HIDDEN, world)[rank]
    d_rows = tp.row_bounds(INTER, world)[rank]
    sizes = [b - a for a, b in tp.column_bounds(INTER, world)]
    had_scale = 1.0 / (INTER ** 0.5)

    def reduce_(t):
        if mode == "push" and comm is not None:
            comm.all_reduce(t)
        else:
            dist.all_reduce(t, group=group)

    def step(x):
        m = x.shape[0]
        for mods in stack:
            qkv = mods["qkv"](x)
            att = qkv[:, :o_rows[1] - o_rows[0]]
            if world == 1:
                y = mods["o"](att)
                h = fz.gate_up_swiglu(mods["gate"], mods["up"], y)
                x = mods["down"](h)                        # Hadamard kernel + linear, chained by dependent launch
            elif mode == "fused" and m <= 16:
                o, d = mods["o"], mods["down"]
                y = comm.linear_all_reduce(att, o.weight, o.scale, None, o.out_features)
                comm.gate_up_gather(y, _triple(mods["gate"]), _triple(mods["up"]), d_rows[0])
                x = comm.down_gather_reduce(m, _triple(d), INTER, d_rows[0])
            else:
                y = mods["o"](att)
                reduce_(y)
                hl = fz.gate_up_swiglu(mods["gate"], mods["up"], y)
                if mode == "push" and comm is not None and m * INTER <= comm.max_elems:
                    h = comm.all_gather_features(hl, sizes)
                else:
                    h = tp.all_gather_features(hl, sizes, group)
                h = ops.hadamard(h, had_scale)
                x = mods["down"](h[:, d_rows[0]:d_rows[1]])
                reduce_(x)
            if taps is not None:
                taps.append((y, x))
        return x
    return step


def parity_numbers(y, y_ref):
    """The linear parity rule: max-normalised error, and the worst ratio of |y - y_ref| to
    1e-2 |y_ref| + 1e-2 rms(y_ref).  Passing means max_rel <= 1e-2 and worst <= 1."""
    import torch
    y, y_ref = y.float(), y_ref.float()
    denom = max(float(y_ref.abs().max()), 1e-6)
    max_rel = float((y - y_ref).abs().max()) / denom
    rms = float(y_ref.double().pow(2).mean().sqrt())
    worst = float(((y - y_ref).abs() / (1e-2 * y_ref.abs() + 1e-2 * rms + 1e-6)).max())
    finite = bool(torch.isfinite(y).all())
    return max_rel, worst, finite


def tp_parity(stack, world, rank, group, comm, x_dev, device):
    """Layer 0 through the fused exchanges and through NCCL on the same input, both compared on rank 0 with the
    unsharded layer built from the same seeds.  Returns the dict printed as "tp_parity" (rank 0) or None."""
    import torch

    from uniql_b200 import fused as fz
    m = x_dev.shape[0]
    got = {}
    for mode in ("fused", "nccl"):
        taps = []
        make_step(stack[:1], world, rank, group, mode=mode, comm=comm, taps=taps)(x_dev)
        torch.cuda.synchronize()
        got[mode] = [t.clone() for t in taps[0]]
    if rank != 0:
        return None
    full = build_stack(m, 0, 1, device, 1)[0]
    qkv = full["qkv"](x_dev)
    qw, aw = QKV // world, HIDDEN // world
    att = torch.cat([qkv[:, r * qw:r * qw + aw] for r in range(world)], dim=1)
    y_ref = full["o"](att)
    out = {"vs": "unsharded layer 0 (same seeds) on rank 0, rule of the linear parity tests", "ok": True}
    for mode in ("fused", "nccl"):
        # each row-parallel output is compared with the unsharded linear applied to the same (gathered) input
        y = got[mode][0]
        h = fz.gate_up_swiglu(full["gate"], full["up"], y)
        x_ref = full["down"](h)
        r0 = parity_numbers(y, y_ref)
        r1 = parity_numbers(got[mode][1], x_ref)
        out[mode] = {"o_proj_max_rel": r0[0], "o_proj_worst": r0[1], "down_proj_max_rel": r1[0], "down_proj_worst": r1[1]}
        if not (r0[2] and r1[2] and r0[0] <= 1e-2 and r0[1] <= 1.0 and r1[0] <= 1e-2 and r1[1] <= 1.0):
            out["ok"] = False
    out["max_rel"] = max(out["fused"]["o_proj_max_rel"], out["fused"]["down_proj_max_rel"])
    return out


def _log(msg):
    if os.environ.get("UNIQL_BENCH_VERBOSE"):
        print(f"[bench rank {os.environ.get('RANK', '0')} {time.strftime('%H:%M:%S')}] {msg}", file=sys.stderr, flush=True)


def _arm_deadline(seconds):
    """Hard stop for a run that stopped making progress (a collective that never completes): the process exits
    by itself instead of sitting on the GPUs until an outer limit kills it."""
    import threading

    def fire():
        print(f"bench.py: no result after {seconds} s, giving up", file=sys.stderr, flush=True)
        os._exit(3)

    t = threading.Timer(seconds, fire)
    t.daemon = True
    t.start()
    return t


def _graph_of(fn, stream):
    """Capture fn() into a CUDA graph on `stream` (after one eager call) and return the graph."""
    import torch
    fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        fn()
    return g


def _time_replays(graph, stream, reps, warm=3):
    """CUDA-event time of `reps` back-to-back replays, in microseconds per replay."""
    import torch
    for _ in range(warm):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(reps):
        graph.replay()
    e1.record(stream)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps


def _random_layer(gen, n, k, device, bias=False):
    """A packed layer with random codes and plausible scales (timing only: no quantiser run, no checkpoint)."""
    import torch

    from uniql_b200.quantize.quant_linear_layers import W4A16B16O16Linear
    lin = W4A16B16O16Linear(k, n, bias=bias, device="meta")
    lin._buffers["weight"] = torch.randint(-2 ** 31, 2 ** 31 - 1, (lin.size_k // 16, 2 * lin.size_n), generator=gen,
                                           device=device, dtype=torch.int64).to(torch.int32)
    lin._buffers["scale"] = (torch.rand(lin.size_k // 128, lin.size_n, generator=gen, device=device) * 0.004 + 0.001).half()
    lin._buffers["workspace"] = torch.zeros(lin.size_n // 64 * 16, dtype=torch.int32, device=device)
    if bias:
        lin.bias = torch.nn.Parameter((torch.randn(n, generator=gen, device=device) * 0.1).half(), requires_grad=False)
    return lin


def qwen_decode_leg(device, stream, peak, batches=(1, 8, 64)):
    """BASELINE configuration 4 on one GPU: 4-bit embedding gather -> 28 Qwen2.5-7B layers (q/k/v with bias, o, gate, up,
    down; no attention maths) -> lm_head 152064 x 3584, one CUDA graph per decode batch, random packed weights."""
    import torch

    from uniql_b200 import fused as fz
    from uniql_b200 import ops
    hidden, inter, kv, vocab, nlayers = 3584, 18944, 512, 152064, 28
    gen = torch.Generator(device=device).manual_seed(11)
    table = torch.randint(-2 ** 31, 2 ** 31 - 1, (vocab, hidden // 8), generator=gen, device=device, dtype=torch.int64).to(torch.int32)
    tscale = (torch.rand(vocab, generator=gen, device=device) * 0.01 + 0.001).half()
    layers = []
    for _ in range(nlayers):
        layers.append({"q": _random_layer(gen, hidden, hidden, device, True), "k": _random_layer(gen, kv, hidden, device, True),
                       "v": _random_layer(gen, kv, hidden, device, True), "o": _random_layer(gen, hidden, hidden, device),
                       "gate": _random_layer(gen, inter, hidden, device), "up": _random_layer(gen, inter, hidden, device),
                       "down": _random_layer(gen, hidden, inter, device)})
    head = _random_layer(gen, vocab, hidden, device)

    def lin_bytes(mod, m):
        return mod.size_k * mod.size_n // 2 + (mod.size_k // 128) * mod.size_n * 2 + m * mod.size_k * 2 + m * mod.out_features * 2

    out = {}
    for b in batches:
        ids = torch.randint(0, vocab, (b,), generator=gen, device=device, dtype=torch.int64)

        def step():
            x = ops.w4_embedding(ids, table, tscale)
            for L in layers:
                q, _, _ = fz.qkv_proj(L["q"], L["k"], L["v"], x)
                x = fz.linear_residual(L["o"], q, x)
                h = fz.gate_up_swiglu(L["gate"], L["up"], x)
                x = fz.linear_residual(L["down"], h, x)
            return head(x)

        g = _graph_of(step, stream)
        us = _time_replays(g, stream, 10)
        nbytes = b * (hidden // 2 + 2 + 8 + 2 * hidden) + lin_bytes(head, b) + sum(lin_bytes(mod, b) for L in layers for mod in L.values())
        out[f"batch{b}"] = {"ms_per_step": us / 1e3, "decode_tok_s": b / (us * 1e-6), "gbs": nbytes / (us * 1e-6) / 1e9,
                            "frac_of_hbm_peak": nbytes / (us * 1e-6) / 1e9 / peak,
                            "launches_per_step": 2 + 4 * nlayers if b <= 16 else None}
        del g
    out["workload"] = ("Qwen2.5-7B W4A16 linear stack: embedding gather, 28 x (q/k/v+bias, o+residual, gate/up SwiGLU, "
                       "down+residual), lm_head 152064x3584; random packed weights, seeded uniform token ids, 1 GPU")
    return out


def mamba_decode_leg(device, stream, peak, batches=(1, 16)):
    """BASELINE configuration 5 on one GPU: 56 x (in_proj 18560 x 4096, out_proj 4096 x 8192 with its 8192-point online
    Hadamard); the first 8192 columns of in_proj's output stand in for the SSM output."""
    import torch

    from uniql_b200.quantize.quant_linear_layers import W4A16B16O16HadLinear
    d_model, d_inner, d_in, nlayers = 4096, 8192, 18560, 56
    gen = torch.Generator(device=device).manual_seed(13)
    layers = []
    for _ in range(nlayers):
        out_proj = _random_layer(gen, d_model, d_inner, device)
        out_proj.__class__ = W4A16B16O16HadLinear
        layers.append((_random_layer(gen, d_in, d_model, device), out_proj))
    out = {}
    for b in batches:
        x0 = torch.randn(b, d_model, generator=gen, device=device).half()

        def step():
            x = x0
            for in_proj, out_proj in layers:
                z = in_proj(x)
                x = out_proj(z[:, :d_inner])
            return x

        g = _graph_of(step, stream)
        us = _time_replays(g, stream, 10)
        nbytes = sum(mod.size_k * mod.size_n // 2 + (mod.size_k // 128) * mod.size_n * 2 + b * mod.size_k * 2 +
                     b * mod.out_features * 2 for pair in layers for mod in pair)
        out[f"batch{b}"] = {"ms_per_step": us / 1e3, "decode_tok_s": b / (us * 1e-6), "gbs": nbytes / (us * 1e-6) / 1e9,
                            "frac_of_hbm_peak": nbytes / (us * 1e-6) / 1e9 / peak}
        del g
    out["workload"] = "Mamba2-8b block linears x56 (in_proj 18560x4096, out_proj 4096x8192 + 8192-pt Hadamard), random packed weights, 1 GPU"
    return out


def run_ours(args):
    _arm_deadline(args.deadline)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        # whole-step CUDA-graph capture of NCCL collectives needs the process group's asynchronous error
        # handling (a watchdog thread that polls CUDA events) switched off before the group is created
        os.environ.setdefault("TORCH_NCCL_ASYNC_ERROR_HANDLING", "0")
        os.environ.setdefault("NCCL_ASYNC_ERROR_HANDLING", "0")
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: uniql_b200 has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    group = None
    if world > 1:
        import datetime
        dist.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(seconds=180))
        group = dist.group.WORLD
    import uniql_b200  # noqa: F401  (fails loudly if the library is missing)
    from uniql_b200 import fused as fz
    from uniql_b200 import ops

    m = args.batch
    layers = args.layers
    peak, peak_kind, peaks = measured_peaks()
    _log("process group up, building the synthetic stack")
    stack = build_stack(m, rank, world, device, layers)
    _log("stack built")
    comm, collective = None, "none"
    if world > 1:
        collective = os.environ.get("UNIQL_TP_COLLECTIVE", "fused")
        if collective in ("push", "fused"):
            from uniql_b200 import tp
            # 16 batch rows of the widest activation row (the 14336 intermediate features)
            comm = tp.PushAllReduce(group, max_elems=16 * 16384, device=device)
        _log(f"collective: {collective}")
    step = make_step(stack, world, rank, group, collective, comm)
    gen = torch.Generator(device=device).manual_seed(7)
    x_dev = (torch.randn(m, HIDDEN, generator=gen, device=device) * 0.05).to(torch.float16)
    x_host = x_dev.cpu().pin_memory()
    y_host = torch.empty((m, HIDDEN), dtype=torch.float16).pin_memory()
    stream = torch.cuda.Stream(device=device)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # qkv, o, gate+up (SwiGLU in the epilogue), Hadamard, down: the cross-GPU sums and the feature gather ride in the
    # linears' epilogues, the Hadamard kernel of a tensor-parallel layer reads the gathered row directly
    # (17..128 rows: qkv, o, gate+up as one tensor-core launch, Hadamard, down; beyond that gate and up are separate
    # launches; SiLU * up is PyTorch's above 16 rows)
    launches_per_layer = 5 if m <= 128 else 6
    parity = None
    with torch.cuda.stream(stream):
        # ---- tensor parallel: check the sharded result before timing anything ----
        if world > 1 and collective == "fused" and m <= 16:
            parity = tp_parity(stack, world, rank, group, comm, x_dev, device)
            ok = torch.tensor([1 if (parity is None or parity["ok"]) else 0], device=device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok.item()) == 0:
                if rank == 0:
                    print(json.dumps({"tp_parity": parity, "error": "tensor-parallel result differs from the unsharded layer"}))
                sys.stdout.flush()
                os._exit(4)
            _log("tp parity ok")
        for _ in range(2):
            y = step(x_dev)
        torch.cuda.synchronize()
        _log("eager warm-up done")
        # ---- device-resident throughput: the step replayed from a CUDA graph (the reference's own
        # profiling harness replays decode from a graph as well) ----
        graph, mode = None, "cuda_graph"
        use_graph = os.environ.get("UNIQL_BENCH_GRAPH", "1") != "0"
        try:
            if not use_graph:
                raise RuntimeError("graph replay disabled by UNIQL_BENCH_GRAPH=0")
            graph = torch.cuda.CUDAGraph()
            static_x = x_dev.clone()
            with torch.cuda.graph(graph, stream=stream):
                static_y = step(static_x)
        except Exception as e:  # pragma: no cover - depends on NCCL capture support
            graph, mode = None, f"eager ({type(e).__name__})"
            torch.cuda.synchronize()
        if world > 1:      # every rank must take the same path
            flag = torch.tensor([1 if graph is not None else 0], device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if int(flag.item()) == 0 and graph is not None:
                graph, mode = None, "eager (capture failed on another rank)"

        def run_step():
            if graph is not None:
                graph.replay()
            else:
                step(x_dev)

        _log(f"launch mode: {mode}")
        for _ in range(max(3, args.warmup)):
            run_step()
        barrier()
        _log("warm-up done")
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        for _ in range(args.steps):
            run_step()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        _log(f"timed region done: {ms / args.steps:.3f} ms/step")

        # ---- spread of single steps: 200 replays, one event pair each ----
        pct = None
        if graph is not None:
            evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(200)]
            barrier()
            for a, b in evs:
                a.record(stream)
                graph.replay()
                b.record(stream)
            barrier()
            ts = sorted(a.elapsed_time(b) for a, b in evs)
            pct = {"p10_ms": ts[20], "p50_ms": ts[100], "p90_ms": ts[180], "replays": 200}

        # ---- end to end through the module API with host buffers (eager calls) ----
        def e2e_step():
            x_in = x_host.to(device, non_blocking=True)
            y_out = step(x_in)
            y_host.copy_(y_out, non_blocking=True)

        for _ in range(3):
            e2e_step()
        barrier()
        e2e_steps = max(1, min(args.steps, 20))
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record(stream)
        for _ in range(e2e_steps):
            e2e_step()
        f1.record(stream)
        barrier()
        ms_e2e = f0.elapsed_time(f1)
        # same, with the step replayed from the captured graph between the two copies
        ms_e2e_graph = None
        if graph is not None:
            f0.record(stream)
            for _ in range(e2e_steps):
                static_x.copy_(x_host, non_blocking=True)
                graph.replay()
                y_host.copy_(static_y, non_blocking=True)
            f1.record(stream)
            barrier()
            ms_e2e_graph = f0.elapsed_time(f1)
        clocks = sampler.stop() if rank == 0 else None
        _log("e2e done")

        # ---- the same stack at decode batches 16 and 64 (extra keys; the headline stays batch `m`) ----
        batch_curve = {}
        for bm in (16, 64):
            if bm == m or os.environ.get("UNIQL_BENCH_NO_LEGS"):     # profiling runs of the aux kernels skip these too
                continue
            xb = (torch.randn(bm, HIDDEN, generator=gen, device=device) * 0.05).to(torch.float16)
            bmode = collective if (bm <= 16 or collective != "fused") else "push"
            bstep = make_step(stack, world, rank, group, bmode, comm)
            try:
                gb = _graph_of(lambda: bstep(xb), stream)
                us = _time_replays(gb, stream, 5)
            except Exception as e:  # pragma: no cover
                gb, us = None, None
                torch.cuda.synchronize()
                batch_curve[f"batch{bm}"] = {"error": type(e).__name__}
            if world > 1:
                barrier()
            if us is not None:
                batch_curve[f"batch{bm}"] = {"ms_per_step": us / 1e3, "decode_tok_s": bm / (us * 1e-6) * (layers / LAYERS)}
            del gb

        # ---- dominant kernel alone: the fused gate+up launch (2 x 14336/world x 4096 + SwiGLU), one launch per layer so
        # every launch streams different weights (L2-cold), timed with CUDA events on the launching stream ----
        pairs = [(mods["gate"], mods["up"]) for mods in stack]
        xg = (torch.randn(m, HIDDEN, generator=gen, device=device) * 0.05).to(torch.float16)
        n_gate_local = pairs[0][0].out_features
        og = torch.empty((m, n_gate_local), dtype=torch.float16, device=device)

        def pair_pass():
            for g, u in pairs:
                if m <= 16:
                    ops.w4a16_linear_group(xg, [_triple(g), _triple(u)], epilogue="swiglu", outs=[og])
                else:
                    fz.gate_up_swiglu(g, u, xg)

        ggraph = _graph_of(pair_pass, stream)
        pair_us = _time_replays(ggraph, stream, 10) / len(pairs)
        # a single projection of the same pair, for comparison with the unfused launch
        gate_mods = [mods["gate"] for mods in stack]
        og1 = torch.empty((m, n_gate_local), dtype=torch.float16, device=device)

        def gate_pass():
            for g in gate_mods:
                ops.w4a16_linear(xg, g.weight, g.scale, None, g.out_features, out=og1)

        g1 = _graph_of(gate_pass, stream)
        gate_us = _time_replays(g1, stream, 10) / len(gate_mods)
        del ggraph, g1

        # ---- prefill regime: the gate projection at m = 4096 through the tcgen05 kernel ----
        mp = 4096
        xp = torch.randn(mp, HIDDEN, generator=gen, device=device).to(torch.float16)
        op = torch.empty((mp, gate_mods[0].out_features), dtype=torch.float16, device=device)
        for g in gate_mods[:3]:
            ops.w4a16_linear(xp, g.weight, g.scale, None, g.out_features, out=op)
        torch.cuda.synchronize()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record(stream)
        for g in gate_mods:
            ops.w4a16_linear(xp, g.weight, g.scale, None, g.out_features, out=op)
        p1.record(stream)
        torch.cuda.synchronize()
        prefill_us = p0.elapsed_time(p1) * 1e3 / len(gate_mods)
        # the same projection at batch 64 (small-batch tcgen05 kernel), one launch per distinct weight set
        x64 = torch.randn(64, HIDDEN, generator=gen, device=device).to(torch.float16)
        o64 = torch.empty((64, gate_mods[0].out_features), dtype=torch.float16, device=device)

        def pass64():
            for g in gate_mods:
                ops.w4a16_linear(x64, g.weight, g.scale, None, g.out_features, out=o64)

        g64 = _graph_of(pass64, stream)
        m64_us = _time_replays(g64, stream, 3, warm=1) / len(gate_mods)
        del xp, op, g64
        aux = qwen = mamba = None
        if world == 1 and not os.environ.get("UNIQL_BENCH_NO_AUX"):
            aux = aux_kernels(device, stream, peak)
            torch.cuda.empty_cache()
            if not os.environ.get("UNIQL_BENCH_NO_LEGS"):       # profiling runs of the aux kernels skip the model legs
                qwen = qwen_decode_leg(device, stream, peak)
                torch.cuda.empty_cache()
                mamba = mamba_decode_leg(device, stream, peak)

    def rank_max(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ms = rank_max(ms)
    ms_e2e = rank_max(ms_e2e)
    if ms_e2e_graph is not None:
        ms_e2e_graph = rank_max(ms_e2e_graph)
    pair_us = rank_max(pair_us)
    gate_us = rank_max(gate_us)
    prefill_us = rank_max(prefill_us)
    m64_us = rank_max(m64_us)
    status = ops.read_and_clear_status(device)

    if rank == 0:
        t_step = ms / args.steps * 1e-3
        scale_l = LAYERS / layers
        nbytes = step_bytes(m) / scale_l
        n_gate = SHAPES["gate"][0] // world
        pair_bytes = gate_up_bytes(n_gate, HIDDEN, m)
        achieved = pair_bytes / (pair_us * 1e-6) / 1e9
        t_e2e = ms_e2e / e2e_steps * 1e-3
        line = {
            "metric": "w4a16_linear_m1_hbm_gbs", "value": nbytes / t_step / 1e9, "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": t_step * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16xint4->f32acc", "data": "synthetic",
            "config": {"workload": f"Llama-3.1-8B decoder projection set x{layers} layers, W4A16 g128, "
                                   f"decode batch {m}: qkv, o, gate+up with SwiGLU, 14336-pt online Hadamard + down",
                       "parallelism": f"tp{world}", "launch": mode,
                       "launches_per_layer": launches_per_layer,
                       "collective": {"fused": "row-parallel sums and the feature gather inside the decode kernels "
                                               "(peer stores over NVLink, epoch-tagged words; no separate collective launch)",
                                      "push": "uniql_allreduce_push (peer stores over NVLink, one kernel)",
                                      "nccl": "NCCL all_reduce / all_gather", "none": "none"}[collective],
                       "l2": "each step streams %.2f GB of distinct weights per GPU (> 126 MB L2): no flush needed"
                             % (nbytes / world / 1e9)},
            "decode_tok_s": m / (t_step * scale_l),
            "pct_of_hbm_peak": {"of_measured_%.0f" % peak: nbytes / world / t_step / 1e9 / peak,
                                "of_nominal_8000": nbytes / world / t_step / 1e9 / 8000.0},
            "roofline": {"bound": "hbm",
                         "kernel": f"w4a16_gemv_kernel, gate+up 2x{n_gate}x{HIDDEN} with SwiGLU epilogue, m={m}",
                         "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                         "frac": achieved / peak, "us_per_launch": pair_us, "bytes_per_launch": pair_bytes,
                         "traffic": NCU_TRAFFIC_GATE_UP_M1 if (world == 1 and m == 1) else None},
            "single_projection": {"kernel": f"w4a16_gemv_kernel, gate {n_gate}x{HIDDEN}, m={m}", "us_per_launch": gate_us,
                                  "gbs": linear_bytes(n_gate, HIDDEN, m) / (gate_us * 1e-6) / 1e9,
                                  "frac_of_hbm_peak": linear_bytes(n_gate, HIDDEN, m) / (gate_us * 1e-6) / 1e9 / peak},
            "step_percentiles": pct,
            "e2e": None,
            "m4096_tflops": {"value": world * 2.0 * 4096 * n_gate * HIDDEN / (prefill_us * 1e-6) / 1e12,
                             "kernel": f"w4a16_gemm_tc_kernel {n_gate}x{HIDDEN} m=4096 per GPU", "us_per_launch": prefill_us,
                             "frac_of_measured_bf16_burst": (2.0 * 4096 * n_gate * HIDDEN / (prefill_us * 1e-6) / 1e12)
                             / float(peaks.get("bf16_tflops", 1590.0)),
                             "frac_of_nominal_2250": (2.0 * 4096 * n_gate * HIDDEN / (prefill_us * 1e-6) / 1e12) / 2250.0},
            "m64_us": {"value": m64_us, "kernel": f"w4a16_gemm_tc_swap_kernel {n_gate}x{HIDDEN} m=64 per GPU",
                       "weight_gbs": (n_gate * HIDDEN / 2 + n_gate * HIDDEN / 64) / (m64_us * 1e-6) / 1e9},
            "batch_curve": batch_curve,
            "aux_kernels": aux,
            "qwen25_7b_decode": qwen,
            "mamba2_8b_decode": mamba,
            "tp_parity": parity,
            "gpu_launches": (launches_per_layer or 0) * layers * args.steps,
            "clocks": clocks,
            "kernel_status_word": status,
        }
        eager = {"value": nbytes / t_e2e / 1e9, "unit": "GB/s", "h2d_bytes_per_step": m * HIDDEN * 2,
                 "d2h_bytes_per_step": m * HIDDEN * 2, "ms_per_step": t_e2e * 1e3,
                 "how": "pinned host x -> device, eager Python module calls, result -> pinned host"}
        if ms_e2e_graph is not None:
            # headline end-to-end number: host input copied in, the module stack replayed from its CUDA graph
            # (how the reference's own decode profiling runs, profile_model.py:540-553), result copied out
            tg = ms_e2e_graph / e2e_steps * 1e-3
            line["e2e"] = {"value": nbytes / tg / 1e9, "unit": "GB/s", "h2d_bytes_per_step": m * HIDDEN * 2,
                           "d2h_bytes_per_step": m * HIDDEN * 2, "ms_per_step": tg * 1e3,
                           "how": "pinned host x -> device, module stack replayed from a CUDA graph, result -> pinned host"}
            line["e2e_eager_module_calls"] = eager
        else:
            line["e2e"] = eager
        if world == 1:
            cb, td, tm, desc = cpu_linear_sample(m, os.cpu_count() or 1, 25.0)
            line["cpu_baseline"] = {"value": cb / (td + tm) / 1e9, "unit": "GB/s", "cores": os.cpu_count() or 1,
                                    "kind": "port", "sample": desc, "dequant_s": td, "matmul_s": tm}
        print(json.dumps(line))
    if world > 1:
        # Leave without tearing the communicator down: destroying a process group whose collectives live in
        # instantiated CUDA graphs was seen to block; every rank has finished its GPU work at this point.
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=1, help="decode batch M")
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--deadline", type=int, default=900, help="seconds after which a stuck run exits by itself")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
