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
