"""Rotary position encoding with the half-split pairing (i, i + head_dim/2).

The table cos/sin[position, head_dim/2] is computed once on the host: inverse frequencies
theta^(-2i/head_dim) and angles position * frequency in float64, then rounded to float32
(adarsh-sgh/edgelm src/kernels_ref.cpp:11-21).  The rotation itself runs in float32 inside the
kernel that also appends the rotated keys and the raw values to the cache
(src/kernels_ref.cpp:82-98, 112-118).
"""
import torch

from ..csrc import ops
from .base import Part
from .registry import register_positions


@register_positions("rope")
class RotaryPositions(Part):
    graph_safe = True
    def __init__(self, spec, env):
        self.head_dim, self.theta, self.max_positions = spec["head_dim"], float(spec["theta"]), spec["max_positions"]
        self.cos = self.sin = None

    def sizes(self):
        return {"rope_theta": self.theta}

    def load(self, tensors, prefix, device):
        if self.cos is not None and self.cos.device == torch.device(device):
            return
        i = torch.arange(0, self.head_dim, 2, dtype=torch.float64)
        inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -(i / self.head_dim))
        ang = torch.arange(self.max_positions, dtype=torch.float64)[:, None] * inv[None, :]
        self.cos = torch.cos(ang).to(torch.float32).to(device).contiguous()
        self.sin = torch.sin(ang).to(torch.float32).to(device).contiguous()

    def rotation_tables(self):
        """(cos, sin) [positions, head_dim/2] float32: a mixer whose decode kernel rotates and appends
        by itself asks for these instead of calling encode_and_append."""
        return self.cos, self.sin

    def project_encode_append(self, ctx, h, w_qkv, qkv, cache, n_heads, n_kv_heads):
        """The stacked projection, the rotation and the append as ONE kernel, where that kernel exists: a prompt step
        in bfloat16 with a head size the tensor-core product's epilogue rotates (its threads hold a head's two halves
        after reading the accumulator).  True if done: `qkv` then holds the rotated queries (its key and value
        columns are not written; attention reads the cache).  False: the caller runs the product and then
        `encode_and_append`.  (adarsh-sgh/edgelm fuses the rotation into its attention op, src/passes.cpp:115-135.)"""
        from . import linear
        if h.shape[0] <= linear.FEW_ROWS or qkv.dtype != torch.bfloat16 or self.head_dim not in (64, 128):
            return False
        h = linear.as_tensor(h)
        if not ops.gemm_tc_rope_takes(h, w_qkv, qkv, cache.k, cache.v, self.cos, self.sin, self.head_dim):
            return False
        ops.gemm_tc_rope(h, w_qkv, qkv, ctx.tok_pos, ctx.tok_seq, ctx.seq_index, ctx.page_table(cache.group), self.cos, self.sin,
                         cache.k, cache.v, n_heads, n_kv_heads, self.head_dim, ctx.err)
        return True

    def encode_and_append(self, ctx, qkv, cache, n_heads, n_kv_heads):
        """Rotate the query and key heads of qkv[T, (nh + 2 nkv) hd] in place at each token's
        position; write the rotated keys and the values into the cache entry's pages."""
        ops.rope_kv_append(qkv, ctx.tok_pos, ctx.tok_seq, ctx.seq_index, ctx.page_table(cache.group), self.cos, self.sin,
                           cache.k, cache.v, n_heads, n_kv_heads, self.head_dim, ctx.err)
