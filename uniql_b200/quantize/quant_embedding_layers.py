"""4-bit embedding module with the constructor, parameters and packing of UniQL's
quantize/quant_embedding_layers.py:8-54; the gather runs in this package's CUDA kernel."""
import torch
import torch.nn as nn

from ..compat import quant_embedding_cuda


class W4O16Embedding(nn.Module):
    def __init__(self, num_embeddings, embedding_dim, device=None, **kwargs):
        factory_kwargs = {"device": device}
        super().__init__()
        self.num_embeddings = num_embeddings
        self.embedding_dim = embedding_dim
        self.num_bits = 4
        self.pack_factor = 32 // self.num_bits
        # a Parameter (not a buffer) so that next(model.parameters()) keeps working, as in the reference
        self.register_parameter("weight", nn.Parameter(
            torch.empty((num_embeddings, embedding_dim // self.pack_factor), dtype=torch.int32, **factory_kwargs),
            requires_grad=False))
        self.register_buffer("scales", torch.empty((num_embeddings,), dtype=torch.float16, **factory_kwargs))

    @classmethod
    def from_fp16(cls, originalLayer: nn.Embedding):
        """Per-row symmetric RTN: s = amax/8, q = clamp(round(w/s + 8), 0, 15); each run of 8 codes is
        stored with code o in nibble [0,4,1,5,2,6,3,7][o] (quant_embedding_layers.py:25-47)."""
        device = originalLayer.weight.device
        qembed = cls(originalLayer.num_embeddings, originalLayer.embedding_dim, device=device)
        w = originalLayer.weight.data
        with torch.no_grad():
            scales = w.abs().amax(dim=-1, keepdim=True) / 8
            q = torch.round((w / scales) + 8).clamp(0, 15)
            q = torch.nan_to_num(q, nan=0.0).to(torch.int64).reshape(w.shape[0], -1, 8)
            nib_of_elem = torch.tensor([0, 4, 1, 5, 2, 6, 3, 7], device=q.device)
            word = (q << (4 * nib_of_elem)).sum(dim=-1)
            word = torch.where(word >= 2 ** 31, word - 2 ** 32, word).to(torch.int32)
        qembed.scales = scales.flatten().to(torch.float16).to(device)
        qembed.weight.data = word.to(device)
        return qembed

    @torch.no_grad()
    def forward(self, x):
        return quant_embedding_cuda.w4a16_embedding_lookup(x, self.weight, self.scales)

    def __repr__(self):
        return f"W4O16Embedding(num_embeddings={self.num_embeddings}, embedding_dim={self.embedding_dim})"
