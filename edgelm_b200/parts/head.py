"""Output head: logits = norm(x[wanted rows]) H^T in float32, H the embedding table when tied
(adarsh-sgh/edgelm tools/elm.py:154-160).  The final norm is applied by the model before this
part; here is the matrix product alone."""
from . import linear
from .base import Part, as_matrix
from .registry import register_head


@register_head("lm_head")
class LMHead(Part):
    graph_safe = True
    def __init__(self, spec, env):
        self.vocab_size, self.dim, self.name, self.tied_to = spec["vocab_size"], spec["dim"], spec["name"], spec["tied_to"]
        self.dtype = env.dtype
        self.weight = None

    def sizes(self):
        return {"vocab": self.vocab_size, "tied": bool(self.tied_to)}

    def flops(self, n_rows, attended=0):
        return 2.0 * n_rows * self.dim * self.vocab_size

    def weight_shapes(self, prefix=""):
        return {} if self.tied_to else {self.name: (self.vocab_size, self.dim)}

    def ignorable(self):
        """Names that a file may hold without their being used: a tied model's stored copy of the head."""
        return (self.name,) if self.tied_to else ()

    def load(self, tensors, prefix, device, tied_table=None):
        self.weight = tied_table if self.tied_to else as_matrix(tensors[self.name], self.dtype, device)

    def forward(self, ctx, xn, logits):
        linear.matmul(ctx, xn, self.weight, logits)
