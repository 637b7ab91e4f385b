"""Generate the golden fixtures in this directory from the UNMODIFIED UniQL sources.

Usage (needs a checkout of the reference project; CPU only):

    python tests/golden/make_golden.py /path/to/UniQL

The reference's CUDA extension modules (quant_linear_cuda, quant_embedding_cuda,
fast_hadamard_transform_cuda) are replaced by empty stand-ins so that the pure
Python/CPU parts of the reference — the RTN quantiser, the weight/scale
permutation and packing helpers, their inverses, the module constructors and
their from_fp16 class methods, the load-time slicing functions — can be imported and executed as they are.
Outputs are small .npz files holding the seeded inputs and the reference's outputs.
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _import_reference(root):
    for name in ("quant_linear_cuda", "quant_embedding_cuda", "fast_hadamard_transform_cuda"):
        sys.modules[name] = types.ModuleType(name)
    for fn in ("fast_hadamard_transform", "fast_hadamard_transform_12N", "fast_hadamard_transform_20N",
               "fast_hadamard_transform_28N", "fast_hadamard_transform_40N"):
        setattr(sys.modules["fast_hadamard_transform_cuda"], fn, lambda x, s: (_ for _ in ()).throw(RuntimeError))
    sys.path.insert(0, root)
    import quantize.quantize_helpers as qh
    import quantize.quant_linear_layers as qll
    import quantize.quant_embedding_layers as qel
    import quantize.hadamard_helpers as hh
    return qh, qll, qel, hh


def _weights(seed, out_f, in_f, std=0.02):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(out_f, in_f, generator=g) * std).to(torch.float16)


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <path to a checkout of enyac-group/UniQL>")
    root = sys.argv[1]
    qh, qll, qel, hh = _import_reference(root)

    # ---- 1. w4a16_quantize on a few shapes (incl. N padding and K padding) ----
    cases = {"a": (256, 256, 0), "b": (320, 384, 64), "c": (192, 200, 64)}   # (out, in, pad_out)
    blob = {}
    for tag, (out_f, in_f, pad_out) in cases.items():
        w = _weights(100 + len(blob), out_f, in_f)
        if tag == "b":
            w[5, 128:256] = 0          # an all-zero quantisation group
            w[7, 3] = 0.5              # an outlier
        w_t = w.t().contiguous()
        w_ref, packed, scale = qh.w4a16_quantize(w_t, 4, 128, None, pad_out)
        size_k, size_n = w_ref.shape
        # inverse helpers of the reference
        q_rec = qh.unpack_w4a16_permute_weights(packed, size_k, size_n, 4, qh.get_w4a16_weight_perms(), 128)
        s_rec = qh.w4a16_unpermute_scales(scale, size_k, size_n, 128)
        # dequantise the way modeling/modeling_helpers.py:632-640 does
        wq = q_rec.to(s_rec.dtype) - 8
        w_deq = (wq.reshape(-1, 128, size_n) * s_rec.unsqueeze(1)).reshape(size_k, size_n)
        assert torch.equal(w_deq, w_ref)
        blob[f"{tag}_w"] = w.numpy()
        blob[f"{tag}_pad_out"] = np.int64(pad_out)
        blob[f"{tag}_w_ref"] = w_ref.numpy()
        blob[f"{tag}_packed"] = packed.numpy()
        blob[f"{tag}_scale"] = scale.numpy()
        blob[f"{tag}_q"] = q_rec.numpy().astype(np.uint8)
        blob[f"{tag}_scale_unperm"] = s_rec.numpy()
    blob["weight_perm"] = qh.get_w4a16_weight_perms().numpy()
    blob["scale_perm"] = np.array(qh.get_scale_perms()[0])
    np.savez_compressed(os.path.join(HERE, "w4a16_quantize.npz"), **blob)

    # ---- 2. module state dicts made by the reference's from_fp16 ----
    lin = torch.nn.Linear(384, 200, bias=True)
    lin.weight.data = _weights(7, 200, 384).float()
    lin.bias.data = torch.linspace(-1, 1, 200)
    lin = lin.to(torch.float16)
    qlin = qll.W4A16B16O16Linear.from_fp16(lin)
    sd = {k: v.numpy() for k, v in qlin.state_dict().items()}
    np.savez_compressed(os.path.join(HERE, "linear_module.npz"),
                        fp16_weight=lin.weight.data.numpy(), fp16_bias=lin.bias.data.numpy(),
                        pad_in=np.int64(qlin.pad_in), pad_out=np.int64(qlin.pad_out),
                        size_k=np.int64(qlin.size_k), size_n=np.int64(qlin.size_n),
                        **{"sd_" + k: v for k, v in sd.items()})

    emb = torch.nn.Embedding(96, 160)
    emb.weight.data = _weights(11, 96, 160).float()
    emb.weight.data[3] *= 1e-4          # a row whose scale is sub-normal in fp16
    emb.weight.data[4, 0] = 0.3         # hits nibble 15 after clamping
    emb = emb.to(torch.float16)
    qemb = qel.W4O16Embedding.from_fp16(emb)
    np.savez_compressed(os.path.join(HERE, "embedding_module.npz"),
                        fp16_weight=emb.weight.data.numpy(),
                        sd_weight=qemb.weight.data.numpy(), sd_scales=qemb.scales.numpy())

    # ---- 3. Hadamard size dispatch (get_had_fn only picks the function) ----
    dims = [64, 4096, 8192, 14336, 3584, 1536, 5120, 2560, 768, 10240]
    picks = []
    for d in dims:
        fn, n, sc = hh.get_had_fn(d)
        picks.append((d, n, sc))
    np.savez_compressed(os.path.join(HERE, "hadamard_dispatch.npz"),
                        dims=np.array([p[0] for p in picks]), base=np.array([p[1] for p in picks]),
                        scale=np.array([p[2] for p in picks]))
    make_slicing(root, qh)
    print("wrote fixtures to", HERE)


def make_slicing(root, qh):
    """The load-time slicing functions of modeling/modeling_helpers.py:361-867, run unmodified on small seeded
    layers (shapes with and without k / n padding).  Inputs are regenerated by the test from the stored fp16 weights;
    stored per case: the reference's packed weight, scale (and bias / workspace length)."""
    import modeling.modeling_helpers as mh

    seeds = {}

    def quantised(seed, out_f, in_f):
        seeds[len(seeds)] = (seed, out_f, in_f)
        w = _weights(seed, out_f, in_f)
        pad_out = (256 - out_f % 256) % 256
        _, packed, scale = qh.w4a16_quantize(w.t().contiguous(), 4, 128, None, pad_out)
        ws = torch.zeros((out_f + pad_out) // 64 * 16, dtype=torch.int32)
        return w, packed, scale, ws

    blob = {}

    def put(tag, w, outs, names):
        # the fp16 input is regenerated by the test from (seed, shape) with the same generator call as _weights();
        # a checksum of its bits guards against a change of the generator
        blob[tag + "_w_sum"] = np.int64(w.numpy().view(np.uint16).astype(np.int64).sum())
        for n, o in zip(names, outs):
            if o is not None:
                blob[f"{tag}_{n}"] = o.numpy()

    # Llama-style MLP: hidden 256 (the reference's column slicers assume an unpadded hidden size), intermediate
    # 384 -> 320 (320 needs 192 columns / 64 rows of padding)
    hidden, inter, red = 256, 384, 320
    w, packed, scale, ws = quantised(21, inter, hidden)
    put("up", w, mh.slice_w4a16_up_gate_proj(packed, scale, ws, hidden, inter, red, packed.shape), ("packed", "scale", "ws"))
    w, packed, scale, ws = quantised(22, hidden, inter)
    put("down", w, mh.slice_w4a16_down_proj(packed, scale, ws, hidden, inter, red, packed.shape), ("packed", "scale", "ws"))
    # attention: 3 heads x 64 -> 48 (q/k keep the first halves of both rotary halves, v/o the leading dims)
    nheads, hd, rhd = 3, 64, 48
    w, packed, scale, ws = quantised(23, nheads * hd, hidden)
    bias = torch.linspace(-1, 1, nheads * hd).to(torch.float16)
    blob["qk_bias_in"] = bias.numpy()
    put("qk", w, mh.slice_w4a16_qk_proj(packed, bias, scale, ws, hidden, nheads, hd, rhd, packed.shape),
        ("packed", "bias", "scale", "ws"))
    w, packed, scale, ws = quantised(24, nheads * hd, hidden)
    put("v", w, mh.slice_w4a16_v_proj(packed, scale, ws, hidden, nheads, hd, rhd, packed.shape), ("packed", "scale", "ws"))
    w, packed, scale, ws = quantised(25, hidden, nheads * hd)
    put("o", w, mh.slice_w4a16_o_proj(packed, scale, ws, hidden, nheads, hd, rhd, packed.shape), ("packed", "scale", "ws"))
    # Mamba2-style mixer: 2 groups, 4 heads, intermediate 256 -> 192, state 32 -> 24
    ng, nh, inter2, state, linter, lstate = 2, 4, 256, 32, 192, 24
    proj = 2 * inter2 + 2 * ng * state + nh
    w, packed, scale, ws = quantised(26, proj, hidden)
    put("in", w, mh.slice_w4a16_in_proj(packed, scale, ws, hidden, ng, nh, inter2, state, linter, lstate, packed.shape),
        ("packed", "scale", "ws"))
    w, packed, scale, ws = quantised(27, hidden, inter2)
    put("out", w, mh.slice_w4a16_out_proj(packed, scale, ws, hidden, ng, nh, inter2, linter, packed.shape),
        ("packed", "scale", "ws"))
    idx = torch.arange(nheads * hd).reshape(nheads, hd)
    blob["slice_indices"] = mh.slice_indices(idx, hd, rhd).numpy()
    blob["topk_head"] = mh.get_topk_head_indices(ng, nh, inter2 // nh, linter // nh).numpy()
    blob["topk_state"] = mh.get_topk_ssm_state_indices(ng, state, lstate).numpy()
    conv_ch = inter2 + 2 * ng * state
    conv_w = _weights(28, conv_ch, 4).reshape(conv_ch, 1, 4)
    conv_b = torch.linspace(-1, 1, conv_ch).to(torch.float16)
    cw, cb = mh.slice_conv1d(conv_w, conv_b, ng, nh, inter2, state, linter, lstate)
    blob["conv_w_out"], blob["conv_b_out"] = cw.numpy(), cb.numpy()
    blob["norm_out"] = mh.slice_norm(torch.linspace(0, 1, inter2).to(torch.float16), ng, nh, inter2, linter).numpy()
    blob["inputs_seed_out_in"] = np.array([seeds[i] for i in range(len(seeds))], dtype=np.int64)   # order: up, down, qk, v, o, in, out
    np.savez_compressed(os.path.join(HERE, "slicing.npz"), **blob)


if __name__ == "__main__":
    main()
