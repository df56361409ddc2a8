"""Arrangement of one layer's parts.  "prenorm": x += mixer(norm1(x)); x += ffn(norm2(x))
(adarsh-sgh/edgelm tools/elm.py:122-153)."""
from . import linear
from .base import Part, nbytes
from .registry import register_block


@register_block("prenorm")
class PreNormBlock(Part):
    def __init__(self, layer_spec, env):
        self.prefix = layer_spec.prefix
        self.dtype = env.dtype
        self.mixer_norm = env.build("norm", layer_spec.mixer_norm)
        self.mixer = env.build("mixer", layer_spec.mixer)
        self.ffn_norm = env.build("norm", layer_spec.ffn_norm)
        self.ffn = env.build("ffn", layer_spec.ffn)
        self.parts = (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)
        self.hidden = layer_spec.mixer_norm["dim"]

    def weight_shapes(self, prefix=None):
        out = {}
        for p in self.parts:
            out.update(p.weight_shapes(self.prefix))
        return out

    def load(self, tensors, prefix, device):
        for p in self.parts:
            p.load(tensors, self.prefix, device)

    def cache_need(self):
        return self.mixer.cache_need()

    def sizes(self):
        out = {}
        for p in (self.mixer, self.ffn, self.mixer_norm):
            out.update(p.sizes())
        return out

    def flops(self, n_tokens, attended):
        return sum(p.flops(n_tokens, attended) for p in self.parts)

    def describe(self):
        return f"{self.kind}: {self.mixer_norm.describe()} -> {self.mixer.describe()}; {self.ffn_norm.describe()} -> {self.ffn.describe()}"

    def tile_sizes(self):
        return tuple(self.mixer.tile_sizes())

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts)

    def workspace_bytes(self, n_tokens, n_seqs):
        return nbytes((n_tokens, self.hidden), self.dtype) + max(self.mixer.workspace_bytes(n_tokens, n_seqs),
                                                                  self.ffn.workspace_bytes(n_tokens, n_seqs))

    def _normed(self, ctx, x, norm, part):
        """The part's input: lazily normalised if both the norm and the part can work that way
        (the part's first matrix product then computes the norm itself when the step is small)."""
        if getattr(part, "takes_normed_input", False) and getattr(norm, "fusable", False):
            return linear.NormedInput(ctx, x, norm, self.dtype)
        h = ctx.ws.alloc((x.shape[0], self.hidden), self.dtype)
        with ctx.prof("norm"):
            norm.forward(ctx, x, h)
        return h

    def first_weights(self):
        return self.mixer.first_weights()

    def forward(self, ctx, x, cache):
        # `ctx.weights_after`: what the step reads once the running part is done (a part's last product may start
        # it on its way into L2): after the mixer the feed-forward's first weights, after that whatever the caller
        # named as coming after this layer
        after_layer = ctx.weights_after
        ctx.weights_after = self.ffn.first_weights()
        with ctx.ws.frame():
            self.mixer.forward(ctx, self._normed(ctx, x, self.mixer_norm, self.mixer), x, cache)
        ctx.weights_after = after_layer
        with ctx.ws.frame():
            self.ffn.forward(ctx, self._normed(ctx, x, self.ffn_norm, self.ffn), x)
