"""CPU: the oracle restatement against fixtures produced by the reference's own Python helpers."""
import os

import numpy as np
import pytest

from oracle import uniql_oracle as orc


@pytest.fixture(scope="module")
def gq(golden_dir):
    return np.load(os.path.join(golden_dir, "w4a16_quantize.npz"))


def bits(a):
    return a.view(np.uint16)


def test_permutation_tables(gq):
    assert np.array_equal(orc.weight_perm(), gq["weight_perm"])
    assert np.array_equal(orc.scale_perm(), gq["scale_perm"])


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_quantize_pack_bit_exact(gq, tag):
    w = gq[tag + "_w"]
    w_ref, packed, scale = orc.w4a16_quantize(np.ascontiguousarray(w.T), int(gq[tag + "_pad_out"]))
    assert np.array_equal(bits(w_ref), bits(gq[tag + "_w_ref"]))
    assert np.array_equal(packed, gq[tag + "_packed"])
    assert np.array_equal(bits(scale), bits(gq[tag + "_scale"]))


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_unpack_dequantize(gq, tag):
    k, n = gq[tag + "_w_ref"].shape
    assert np.array_equal(orc.unpack_weights(gq[tag + "_packed"], k, n), gq[tag + "_q"])
    assert np.array_equal(bits(orc.unpermute_scales(gq[tag + "_scale"])), bits(gq[tag + "_scale_unperm"]))
    # value equality: padded columns dequantise to -0.0 where the reference's w_ref holds +0.0
    assert np.array_equal(orc.dequantize(gq[tag + "_packed"], gq[tag + "_scale"]), gq[tag + "_w_ref"])


def test_pack_roundtrip_random():
    rng = np.random.default_rng(0)
    q = rng.integers(0, 16, size=(64, 192), dtype=np.int32)
    assert np.array_equal(orc.unpack_weights(orc.pack_weights(q), 64, 192), q)
    s = rng.standard_normal((3, 192)).astype(np.float16)
    assert np.array_equal(orc.unpermute_scales(orc.permute_scales(s)), s)


def test_embedding_against_reference(golden_dir):
    e = np.load(os.path.join(golden_dir, "embedding_module.npz"))
    packed, scales = orc.embedding_quantize(e["fp16_weight"])
    assert np.array_equal(packed, e["sd_weight"])
    assert np.array_equal(bits(scales), bits(e["sd_scales"]))
    ids = np.arange(e["fp16_weight"].shape[0])
    out = orc.embedding_lookup(ids, packed, scales)
    # dequantised rows stay within one quantisation step of the source (code +8 clamps to 15);
    # row 3 has a sub-normal fp16 scale and is only checked for bit-equality on the GPU
    err = np.abs(out.astype(np.float32) - e["fp16_weight"].astype(np.float32))
    ok = err <= 1.01 * scales.astype(np.float32)[:, None] + 1e-7
    ok[3] = True
    assert ok.all()
    assert orc.embedding_lookup(np.zeros((2, 3), np.int64), packed, scales).shape == (2, 3, 160)
    assert orc.embedding_lookup(np.zeros((0,), np.int64), packed, scales).shape == (0, 160)


def test_hadamard_dispatch_matches_reference(golden_dir):
    d = np.load(os.path.join(golden_dir, "hadamard_dispatch.npz"))
    for dim, base, scale in zip(d["dims"], d["base"], d["scale"]):
        mine = orc.had_factor(int(dim))
        assert (mine if mine != 1 else 2) == int(base)      # the reference reports N=2 for powers of two
        assert abs(1.0 / np.sqrt(dim) - scale) < 1e-12
    with pytest.raises(AssertionError):
        orc.had_factor(12160)                               # no transform exists for this size


@pytest.mark.parametrize("base", [12, 20, 28, 40])
def test_base_matrices_are_hadamard(base):
    h = orc.base_matrix(base)
    assert set(np.unique(h)) == {-1, 1}
    assert np.array_equal(h @ h.T, base * np.eye(base, dtype=np.int64))


@pytest.mark.parametrize("dim", [8, 64, 96, 160, 224, 320, 1024])
def test_hadamard_is_orthogonal_involution_up_to_transpose(dim):
    rng = np.random.default_rng(dim)
    x = rng.standard_normal((3, dim))
    y = orc.hadamard_transform(x)
    assert np.allclose((y ** 2).sum(-1), (x ** 2).sum(-1))
    # explicit matrix check
    eye = np.eye(dim)
    hmat = orc.hadamard_transform(eye) * np.sqrt(dim)       # rows of H^T
    assert np.allclose(hmat @ hmat.T, dim * eye)
    assert np.allclose(y, x @ hmat / np.sqrt(dim))
