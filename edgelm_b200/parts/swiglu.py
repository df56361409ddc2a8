"""SwiGLU feed-forward: x += (silu(h Wg^T) * (h Wu^T)) Wd^T, silu(z) = z / (1 + exp(-z)), no bias
(adarsh-sgh/edgelm src/kernels_ref.cpp:143-160, tools/elm.py:140-152).  Gate and up never reach
memory: the activation is the epilogue of their matrix product, the residual sum that of the
down projection."""
from . import linear
from .base import Part, as_matrix, nbytes
from .registry import register_ffn


@register_ffn("swiglu")
class SwiGLU(Part):
    graph_safe = True
    takes_normed_input = True

    def __init__(self, spec, env):
        self.hidden, self.inter = spec["hidden_size"], spec["intermediate_size"]
        self.names = dict(spec["names"])
        self.dtype = env.dtype
        self.w_gate = self.w_up = self.w_down = None

    def sizes(self):
        return {"intermediate": self.inter}

    def flops(self, n_tokens, attended):
        return 6.0 * n_tokens * self.hidden * self.inter

    def weight_shapes(self, prefix):
        n = self.names
        return {prefix + n["gate"]: (self.inter, self.hidden), prefix + n["up"]: (self.inter, self.hidden),
                prefix + n["down"]: (self.hidden, self.inter)}

    def load(self, tensors, prefix, device):
        n = self.names
        self.w_gate = as_matrix(tensors[prefix + n["gate"]], self.dtype, device)
        self.w_up = as_matrix(tensors[prefix + n["up"]], self.dtype, device)
        self.w_down = as_matrix(tensors[prefix + n["down"]], self.dtype, device)

    def workspace_bytes(self, n_tokens, n_seqs):
        return nbytes((n_tokens, self.inter), self.dtype) + nbytes((n_tokens, self.hidden), self.dtype)

    def first_weights(self):
        return (self.w_gate, self.w_up)

    def forward(self, ctx, h, x):
        mid = ctx.ws.alloc((h.shape[0], self.inter), self.dtype)
        with ctx.prof("gate_up_swiglu"):
            linear.matmul(ctx, h, self.w_gate, mid, epilogue=linear.EPI_SWIGLU, w2=self.w_up, prefetch=(self.w_down,))
        with ctx.prof("down_proj_residual"):
            linear.matmul(ctx, mid, self.w_down, x, epilogue=linear.EPI_RESIDUAL, residual=x, prefetch=ctx.weights_after)
