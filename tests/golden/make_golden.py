"""Generate the golden fixtures in this directory from the UNMODIFIED UniQL sources.

Usage (needs a checkout of the reference project; CPU only):

    python tests/golden/make_golden.py /path/to/UniQL

The reference's CUDA extension modules (quant_linear_cuda, quant_embedding_cuda,
fast_hadamard_transform_cuda) are replaced by empty stand-ins so that the pure
Python/CPU parts of the reference — the RTN quantiser, the weight/scale
permutation and packing helpers, their inverses, the module constructors and
their from_fp16 class methods — can be imported and executed as they are.
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
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    main()
