"""RMSNorm: y = x * (1 / sqrt(mean(x^2) + eps)) * w, statistics in float32
(adarsh-sgh/edgelm src/kernels_ref.cpp:48-56); the weight is used as stored (no +1)."""
from ..csrc import ops
from .base import Part, as_vector
from .registry import register_norm


@register_norm("rmsnorm")
class RMSNorm(Part):
    graph_safe = True
    fusable = True  # a few-rows matrix product can compute this norm in its prologue (weight, eps)

    def __init__(self, spec, env):
        self.dim, self.eps, self.name = spec["dim"], float(spec["eps"]), spec["name"]
        self.weight = None

    def sizes(self):
        return {"rms_norm_eps": self.eps}

    def weight_shapes(self, prefix):
        return {prefix + self.name: (self.dim,)}

    def load(self, tensors, prefix, device):
        self.weight = as_vector(tensors[prefix + self.name], device)

    def forward(self, ctx, x, out, rows=None):
        ops.rmsnorm(x, self.weight, self.eps, out, rows_idx=rows)
