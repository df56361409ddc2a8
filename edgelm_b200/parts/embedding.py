"""Token embedding: x[t] = E[id_t] (adarsh-sgh/edgelm src/kernels_ref.cpp:41-46), no scaling."""
from ..csrc import ops
from .base import Part, as_matrix
from .registry import register_embedding


@register_embedding("embedding")
class Embedding(Part):
    graph_safe = True
    def __init__(self, spec, env):
        self.vocab_size, self.dim, self.name = spec["vocab_size"], spec["dim"], spec["name"]
        self.dtype = env.dtype
        self.table = None

    def sizes(self):
        return {"vocab": self.vocab_size, "hidden": self.dim}

    def weight_shapes(self, prefix=""):
        return {self.name: (self.vocab_size, self.dim)}

    def load(self, tensors, prefix, device):
        self.table = as_matrix(tensors[self.name], self.dtype, device)

    def forward(self, ctx, x):
        ops.embed_gather(ctx.token_ids, self.table, x, ctx.err)
