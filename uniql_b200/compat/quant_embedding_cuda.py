"""`quant_embedding_cuda` stand-in (reference binding: csrc/embedding/quant_embedding.cpp:3-8)."""
from .. import ops


def w4a16_embedding_lookup(input, weight, scale):
    """int64 ids [T] or [B, T] -> fp16 [T, D] / [B, T, D]; D = 8 * weight.shape[1]."""
    ext = ops.torch_ext()
    if ext is not None:
        return ext.embedding(input, weight, scale)
    return ops.w4_embedding(input, weight, scale)
