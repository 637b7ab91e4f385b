"""CPU: host-side mirror of the reference interface (packing helpers, module constructors, state dicts)."""
import os
import re

import numpy as np
import pytest
import torch

from uniql_b200.quantize import quantize_helpers as qh
from uniql_b200.quantize.quant_embedding_layers import W4O16Embedding
from uniql_b200.quantize.quant_linear_layers import W4A16B16O16HadLinear, W4A16B16O16Linear


@pytest.fixture(scope="module")
def gq(golden_dir):
    return np.load(os.path.join(golden_dir, "w4a16_quantize.npz"))


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_helpers_bit_exact(gq, tag):
    w = torch.from_numpy(gq[tag + "_w"])
    pad = int(gq[tag + "_pad_out"])
    w_ref, packed, scale = qh.w4a16_quantize(w.t().contiguous(), 4, 128, None, pad)
    assert torch.equal(w_ref, torch.from_numpy(gq[tag + "_w_ref"]))
    assert torch.equal(packed, torch.from_numpy(gq[tag + "_packed"]))
    assert torch.equal(scale, torch.from_numpy(gq[tag + "_scale"]))
    k, n = w_ref.shape
    perm = qh.get_w4a16_weight_perms()
    assert torch.equal(perm, torch.from_numpy(gq["weight_perm"]))
    q = qh.unpack_w4a16_permute_weights(packed, k, n, 4, perm, 128)
    assert torch.equal(q, torch.from_numpy(gq[tag + "_q"]).int())
    assert torch.equal(qh.get_w4a16_permute_weights(q, k, n, 4, perm, 128), packed)
    assert torch.equal(qh.w4a16_unpermute_scales(scale, k, n, 128), torch.from_numpy(gq[tag + "_scale_unperm"]))
    assert torch.equal(qh.w4a16_dequantize(packed, scale), w_ref)
    # the reference's tile permutation helpers invert each other
    t = qh.permute_weights(q, k, n, perm)
    assert torch.equal(qh.unpermute_weights(t, k, n, perm), q)


def test_gptq_mode_recovers_codes(gq):
    w_ref = torch.from_numpy(gq["a_w_ref"])
    s = torch.from_numpy(gq["a_scale_unperm"])
    out = qh.w4a16_quantize(w_ref, 4, 128, s, 0)
    assert torch.equal(out[1], torch.from_numpy(gq["a_packed"]))


def test_per_channel_rejected():
    with pytest.raises(ValueError):
        qh.get_fake_quantize_weights(torch.randn(64, 64).half(), 4, -1)
    lin = torch.nn.Linear(64, 256).half()
    with pytest.raises(ValueError):
        W4A16B16O16Linear.from_fp16(lin)


def test_linear_module_matches_reference_state_dict(golden_dir):
    g = np.load(os.path.join(golden_dir, "linear_module.npz"))
    lin = torch.nn.Linear(384, 200, bias=True).half()
    lin.weight.data = torch.from_numpy(g["fp16_weight"])
    lin.bias.data = torch.from_numpy(g["fp16_bias"])
    q = W4A16B16O16Linear.from_fp16(lin)
    assert (q.pad_in, q.pad_out, q.size_k, q.size_n) == tuple(int(g[k]) for k in ("pad_in", "pad_out", "size_k", "size_n"))
    sd = q.state_dict()
    ref_keys = sorted(k[3:] for k in g.files if k.startswith("sd_"))
    assert sorted(sd.keys()) == ref_keys
    for k in ref_keys:
        assert sd[k].dtype == torch.from_numpy(g["sd_" + k]).dtype
        assert torch.equal(sd[k], torch.from_numpy(g["sd_" + k])), k
    # a freshly constructed module loads the reference's checkpoint tensors strictly
    fresh = W4A16B16O16Linear(384, 200, bias=True)
    fresh.load_state_dict({k: torch.from_numpy(g["sd_" + k]) for k in ref_keys}, strict=True)
    fresh = fresh.to(torch.float16)            # reference models call .to(float16) after loading
    assert fresh.weight.dtype == torch.int32 and fresh.workspace.dtype == torch.int32


@pytest.mark.parametrize("n,k,stored", [(4096, 4096, 4096), (896, 4096, 1024), (12160, 4096, 12288),
                                        (18560, 4096, 18688), (152064, 3584, 152064), (4096, 200, 4096)])
def test_linear_buffer_shapes(n, k, stored):
    m = W4A16B16O16Linear(k, n, device="meta")
    kp = (k + 127) // 128 * 128
    assert m.size_n == stored and m.size_k == kp
    assert tuple(m.weight.shape) == (kp // 16, stored * 2) and m.weight.dtype == torch.int32
    assert tuple(m.scale.shape) == (kp // 128, stored) and m.scale.dtype == torch.float16
    assert tuple(m.workspace.shape) == (stored // 64 * 16,)


def test_had_linear_validates_size():
    W4A16B16O16HadLinear(14336, 256, device="meta")
    W4A16B16O16HadLinear(8192, 256, device="meta")
    with pytest.raises(AssertionError):
        W4A16B16O16HadLinear(12160, 256, device="meta")


def test_embedding_module_matches_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "embedding_module.npz"))
    emb = torch.nn.Embedding(96, 160).half()
    emb.weight.data = torch.from_numpy(g["fp16_weight"])
    q = W4O16Embedding.from_fp16(emb)
    assert torch.equal(q.weight.data, torch.from_numpy(g["sd_weight"]))
    assert torch.equal(q.scales, torch.from_numpy(g["sd_scales"]))
    assert isinstance(q.weight, torch.nn.Parameter) and not q.weight.requires_grad
    fresh = W4O16Embedding(96, 160)
    fresh.load_state_dict({"weight": torch.from_numpy(g["sd_weight"]), "scales": torch.from_numpy(g["sd_scales"])},
                          strict=True)


def test_ops_refuse_cpu_tensors():
    from uniql_b200 import ops
    with pytest.raises(RuntimeError):
        ops.w4a16_linear(torch.zeros(1, 128).half(), torch.zeros(8, 128, dtype=torch.int32),
                         torch.zeros(1, 64).half(), None, 64)
    with pytest.raises(RuntimeError):
        ops.w4_embedding(torch.zeros(1, dtype=torch.int64), torch.zeros(4, 4, dtype=torch.int32), torch.zeros(4).half())
    with pytest.raises(RuntimeError):
        ops.hadamard(torch.zeros(1, 64), 1.0)


def test_compat_install_registers_reference_names():
    import sys
    from uniql_b200 import compat
    saved = {n: sys.modules.pop(n, None) for n in ("quant_linear_cuda", "quant_embedding_cuda", "fast_hadamard_transform_cuda")}
    try:
        compat.install()
        import fast_hadamard_transform_cuda as f
        import quant_embedding_cuda as e
        import quant_linear_cuda as l
        assert callable(l.w4a16o16_gemm) and callable(e.w4a16_embedding_lookup)
        for name in ("", "_12N", "_20N", "_28N", "_40N"):
            assert callable(getattr(f, "fast_hadamard_transform" + name))
    finally:
        for n, m in saved.items():
            sys.modules.pop(n, None)
            if m is not None:
                sys.modules[n] = m


def test_c_abi_exports_every_declared_symbol(built_lib):
    import ctypes
    from uniql_b200 import _lib
    header = open(os.path.join(os.path.dirname(os.path.dirname(built_lib)), "include", "uniql_b200.h")).read()
    declared = set(re.findall(r"\b(uniql_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    handle = ctypes.CDLL(built_lib)
    for name in declared:
        assert hasattr(handle, name), f"{name} declared in the header but not exported"
    assert declared == set(_lib.SYMBOLS), "ctypes table and header disagree"
    assert _lib.lib().uniql_abi_version() == 2
    assert b"groupsize" in _lib.lib().uniql_strerror(-2)


def test_c_abi_argument_validation_without_gpu(built_lib):
    """Argument checks run before any CUDA call, so they can be exercised on a CPU-only host."""
    L = __import__("uniql_b200")._lib.lib()
    assert L.uniql_w4a16_linear(None, 128, None, None, None, None, 64, 1, 64, 64, 128, -1, 0, None, 0, None, None) == -2
    assert L.uniql_w4a16_linear(None, 128, None, None, None, None, 64, 1, 65, 64, 128, 128, 0, None, 0, None, None) == -3
    assert L.uniql_w4a16_linear(None, 100, None, None, None, None, 64, 1, 64, 64, 100, 128, 0, None, 0, None, None) == -3
    assert L.uniql_w4a16_linear(None, 128, None, None, None, None, 64, 0, 64, 64, 128, 128, 0, None, 0, None, None) == 0
    assert L.uniql_w4a16_linear(None, 128, None, None, None, None, 64, 1, 64, 64, 128, 128, 0, None, 0, None, None) == -1
    assert L.uniql_w4_embedding(None, 0, None, None, None, 10, 64, None, None) == 0
    assert L.uniql_w4_embedding(None, 1, None, None, None, 10, 60, None, None) == -3
    assert L.uniql_w4_embedding(None, 1, None, None, None, 10, 64, None, None) == -1
    assert L.uniql_hadamard(None, None, 1, 12160, 1.0, 0, None) == -3
    assert L.uniql_hadamard(None, None, 1, 64, 1.0, 7, None) == -6
    assert L.uniql_hadamard(None, None, 0, 64, 1.0, 0, None) == 0
    # uniql_w4a16_quantize(W, ldw, n_out, k_in, group_scale, packed, scales, w_ref, n_pad, stream)
    assert L.uniql_w4a16_quantize(None, 256, 128, 256, None, None, None, None, 100, None) == -3    # n_pad % 64
    assert L.uniql_w4a16_quantize(None, 256, 128, 256, None, None, None, None, 64, None) == -3     # n_pad < n_out
    assert L.uniql_w4a16_quantize(None, 100, 128, 256, None, None, None, None, 128, None) == -1    # ldw < k_in
    assert L.uniql_w4a16_quantize(None, 256, 0, 256, None, None, None, None, 128, None) == -1      # empty
    assert L.uniql_w4a16_quantize(None, 256, 128, 256, None, None, None, None, 128, None) == -1    # null pointers


@pytest.mark.parametrize("base", [12, 20, 28, 40])
def test_library_base_matrix_equals_oracle(built_lib, base):
    import ctypes
    from oracle import uniql_oracle as orc
    from uniql_b200._lib import lib
    buf = (ctypes.c_int8 * (base * base))()
    assert lib().uniql_hadamard_base_matrix(base, buf) == 0
    got = np.frombuffer(buf, dtype=np.int8).reshape(base, base)
    assert np.array_equal(got, orc.base_matrix(base))
    assert lib().uniql_hadamard_base_matrix(16, buf) == -3


def test_base_matrix_can_be_replaced_and_is_validated(built_lib):
    """uniql_hadamard_set_base_matrix: a row/column-permuted, sign-flipped copy is still a Hadamard matrix and is
    accepted; broken ones are refused and leave the current matrix in place; NULL restores the built-in one."""
    from oracle import uniql_oracle as orc
    from uniql_b200 import UniqlError, ops
    for base in (12, 20, 28, 40):
        h0 = orc.base_matrix(base)
        rng = np.random.default_rng(base)
        h1 = h0[rng.permutation(base)][:, rng.permutation(base)] * rng.choice([-1, 1], size=(base, 1)) * rng.choice([-1, 1], size=(1, base))
        try:
            ops.hadamard_set_base_matrix(base, h1)
            assert np.array_equal(ops.hadamard_base_matrix(base).numpy(), h1)
            bad = h1.copy()
            bad[1, 2] = -bad[1, 2]
            with pytest.raises(UniqlError):
                ops.hadamard_set_base_matrix(base, bad)                       # rows no longer orthogonal
            zero = h1.copy()
            zero[0, 0] = 0
            with pytest.raises(UniqlError):
                ops.hadamard_set_base_matrix(base, zero)                      # entries must be +1 / -1
            assert np.array_equal(ops.hadamard_base_matrix(base).numpy(), h1)  # refused calls change nothing
        finally:
            ops.hadamard_set_base_matrix(base, None)
        assert np.array_equal(ops.hadamard_base_matrix(base).numpy(), h0)
    with pytest.raises(UniqlError):
        ops.hadamard_set_base_matrix(16, np.ones((16, 16)))
    with pytest.raises(RuntimeError):
        ops.hadamard_set_base_matrix(12, np.ones((11, 12)))
