"""CPU: the decode kernel's work split, replayed on the host by the library itself (uniql_w4a16_plan_selftest).

Every (64-column block, quantisation group) slot must be streamed by exactly one warp, every run of slots must own a
partial tile below the reserved count and the per-block tickets must add up to what the finishing warp waits for --
for single, grouped and SwiGLU launches, with and without the Hadamard prologue, and for tensor-parallel k slices."""
import ctypes

import pytest

CASES = [
    # (m, k, [n...], epilogue, hadamard_dim, k_offset, fused prologue expected)
    (1, 4096, [4096], 0, 0, 0, 0),
    (1, 4096, [14336], 0, 0, 0, 0),
    (1, 4096, [14336, 14336], 1, 0, 0, 0),
    (4, 4096, [12288, 12288], 1, 0, 0, 0),
    (1, 4096, [4096, 1024, 1024], 0, 0, 0, 0),
    (8, 3584, [3584, 512, 512], 0, 0, 0, 0),
    (16, 3584, [152064], 0, 0, 0, 0),
    (1, 14336, [4096], 0, 14336, 0, 1),
    (4, 14336, [4096], 0, 14336, 0, 1),
    (8, 14336, [4096], 0, 14336, 0, 0),            # more than 4 rows: transform kernel in front
    (2, 8192, [4096], 0, 8192, 0, 1),
    (1, 3584, [1024], 0, 3584, 0, 1),
    (1, 1792, [4096], 0, 14336, 1792 * 3, 1),      # rank 3 of 8: k slice starts inside a 512-point segment
    (1, 7168, [4096], 0, 14336, 7168, 1),
    (2, 1024, [4096], 0, 8192, 3072, 1),
    (4, 40960, [256], 0, 40960, 0, 1),
    (1, 128, [64], 0, 0, 0, 0),
    (1, 256, [256], 0, 0, 0, 0),                   # fewer slots than warps
    (3, 12160, [4096], 0, 0, 0, 0),
    (1, 18944, [3584], 0, 0, 0, 0),
]


@pytest.mark.parametrize("m,k,ns,epilogue,had,koff,fused", CASES)
def test_every_slot_once_and_tickets_add_up(built_lib, m, k, ns, epilogue, had, koff, fused):
    from uniql_b200._lib import lib
    arr = (ctypes.c_int64 * len(ns))(*ns)
    flag = ctypes.c_int(-1)
    assert lib().uniql_w4a16_plan_selftest(m, k, arr, len(ns), epilogue, had, koff, ctypes.byref(flag)) == 0
    assert flag.value == fused


def test_geometries_the_kernel_refuses(built_lib):
    from uniql_b200._lib import lib
    L = lib()

    def run(m, k, ns, epilogue=0, had=0, koff=0):
        arr = (ctypes.c_int64 * len(ns))(*ns)
        return L.uniql_w4a16_plan_selftest(m, k, arr, len(ns), epilogue, had, koff, None)

    assert run(17, 256, [256]) == -3               # decode kernel only
    assert run(1, 200, [256]) == -3                # k not a multiple of the group size
    assert run(1, 256, [100]) == -3                # n not a multiple of 64
    assert run(1, 256, [256, 128], epilogue=1) == -1   # SwiGLU pair of different widths
    assert run(1, 12160, [4096], had=12160) == -3  # no Hadamard of that size exists
    assert run(1, 1792, [4096], had=14336, koff=13000) == -3   # slice not on a group boundary / past the row


def _tiled_plan(m, k, widths, epilogue=0):
    import ctypes

    from uniql_b200._lib import lib
    n = (ctypes.c_int64 * len(widths))(*widths)
    out = (ctypes.c_int64 * 5)()
    code = lib().uniql_w4a16_gemv_plan_check(m, k, n, len(widths), epilogue, out)
    return code, list(out)


def _pad(n, unit=256):
    return (n + unit - 1) // unit * unit


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("m", [1, 2, 4, 8, 9, 16])
def test_tiled_kernel_plans_hold_for_every_benchmarked_shard(built_lib, world, m):
    """uniql_w4a16_gemv_plan_check (host only): the plans of the CTA-tiled decode kernel for the Llama-3.1-8B,
    Qwen2.5-7B and Mamba2-8B projections, whole and sharded over 2, 4 and 8 ranks the way uniql_b200.tp shards them
    (columns on 64-column blocks, rows on 128-row groups, uneven splits included)."""
    from uniql_b200 import tp
    cases = []
    for hidden, inter, qkv in ((4096, 14336, 6144), (3584, 18944, 4608), (4096, 12160, 6144)):
        col = [b - a for a, b in tp.column_bounds(_pad(inter), world)]
        qcol = [b - a for a, b in tp.column_bounds(_pad(qkv), world)]
        krow_o = [b - a for a, b in tp.row_bounds(_pad(hidden, 128), world)]
        krow_d = [b - a for a, b in tp.row_bounds(_pad(inter, 128), world)]
        for r in range(world):
            cases.append((hidden, [qcol[r]], 0))                       # qkv shard
            cases.append((krow_o[r], [_pad(hidden)], 0))               # o shard (row-parallel)
            cases.append((hidden, [col[r], col[r]], 1))                # gate + up with SwiGLU
            cases.append((hidden, [col[r]], 0))
            cases.append((krow_d[r], [_pad(hidden)], 0))               # down shard (row-parallel)
    cases += [(4096, [18688], 0), (8192, [4096], 0), (3584, [152064], 0), (4096, [4096, 1024, 1024], 0),
              (3584, [3584, 512, 512], 0), (256, [256], 0), (128, [64], 0), (384, [128, 128, 64, 192], 0)]
    seen = set()
    for k, widths, epi in cases:
        key = (k, tuple(widths), epi)
        if key in seen or k <= 0 or min(widths) <= 0:
            continue
        seen.add(key)
        code, (wn, s, cluster, smem, partial) = _tiled_plan(m, k, widths, epi)
        assert code == 0, f"check {code} failed for m={m} k={k} n={widths} epilogue={epi}: WN={wn} S={s} smem={smem}"
        assert wn in (1, 2, 4, 8) and 1 <= s <= 64 and (epi == 0 or wn >= 2)
        assert (partial == 0) == (s == 1 or cluster == 1)


def test_tiled_kernel_plan_check_refuses_bad_shapes(built_lib):
    assert _tiled_plan(17, 4096, [4096])[0] == 1          # decode kernel: at most 16 rows
    assert _tiled_plan(1, 4000, [4096])[0] == 1           # k must be a multiple of 128
    assert _tiled_plan(1, 4096, [4096, 2048], 1)[0] == 2  # SwiGLU needs two equal widths
    assert _tiled_plan(1, 4096, [100])[0] == 3            # widths are multiples of 64
