"""The generic decoder: a ModelPlan turned into parts, and one forward over a step's tokens.

Nothing here names an architecture.  The plan says which parts each layer has and in which
order layers run; this class builds them through the part registries, hands each its tensors
by name, gives each schedule entry its cache entry, and runs: embedding, the scheduled
layers on the float32 residual stream, the final norm on the wanted rows, the head.
"""
import torch

from ..config.base import ConfigError, ModelPlan
from ..parts import registry as part_registry
from ..parts.base import nbytes


class DecoderModel:
    def __init__(self, plan: ModelPlan, dtype=torch.bfloat16):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ConfigError(f"compute dtype {dtype}: the engine computes in float32 or bfloat16")
        self.plan, self.dtype = plan.validate(), dtype
        env = part_registry.BuildEnv(dtype=dtype)
        self.embedding = env.build("embedding", plan.embedding)
        self.layers = []
        for spec in plan.layers:
            if spec.block not in part_registry.BLOCKS:
                raise ConfigError(f"no block arrangement '{spec.block}' is registered; registered: {', '.join(sorted(part_registry.BLOCKS))}")
            self.layers.append(part_registry.BLOCKS[spec.block](spec, env))
        self.final_norm = env.build("norm", plan.final_norm)
        self.head = env.build("head", plan.head)
        self.schedule = plan.schedule
        self.device = None
        for i, e in enumerate(self.schedule):
            need = self.layers[e.layer].cache_need()
            if e.reads_cache_of is not None and need is not None and not getattr(self.layers[e.layer].mixer, "reads_foreign_cache", False):
                raise ConfigError(f"schedule entry {i} reads another entry's cache, but its mixer keeps one of its own")

    # ------------------------------------------------------------------ weights
    def expected_weights(self):
        """name -> shape of every tensor the model wants from the weights files."""
        out = dict(self.embedding.weight_shapes(""))
        for layer in self.layers:
            out.update(layer.weight_shapes())
        out.update(self.final_norm.weight_shapes(""))
        out.update(self.head.weight_shapes(""))
        return out

    def ignorable_weights(self):
        return tuple(self.head.ignorable()) if hasattr(self.head, "ignorable") else ()

    def load(self, tensors, device):
        """Take the tensors (name -> tensor in the stored dtype); each part keeps what it computes with."""
        self.device = torch.device(device)
        self.embedding.load(tensors, "", device)
        for layer in self.layers:
            layer.load(tensors, None, device)
        self.final_norm.load(tensors, "", device)
        tied = getattr(self.head, "tied_to", None)
        if tied:
            if tied != getattr(self.embedding, "name", None):
                raise ConfigError(f"the head is tied to '{tied}', which is not the embedding's table")
            self.head.load(tensors, "", device, tied_table=self.embedding.table)
        else:
            self.head.load(tensors, "", device)
        return self

    # ------------------------------------------------------------------ cache and workspace
    def cache_needs(self):
        """One need (or None) per schedule entry, in schedule order."""
        return [None if e.reads_cache_of is not None else self.layers[e.layer].cache_need() for e in self.schedule]

    @property
    def graph_safe(self):
        """Whether every part allows its steps to be replayed from a CUDA graph."""
        return all(p.graph_safe for p in [self.embedding, self.final_norm, self.head] + self.layers)

    def tile_sizes(self):
        """Every attention tile size a layer will ask the step for."""
        return sorted({t for l in self.layers for t in l.tile_sizes()})

    def workspace_bytes(self, n_tokens, n_seqs, n_want):
        d = self.plan.hidden_size
        x = nbytes((n_tokens, d), torch.float32)
        layers = max(l.workspace_bytes(n_tokens, n_seqs) for l in self.layers)
        head = nbytes((n_want, d), self.dtype)
        return x + max(layers, head) + 4096

    def flops(self, n_tokens, attended, n_logit_rows):
        """Floating-point operations of one step, added up from the parts in schedule order: `n_tokens` new tokens,
        `attended` (query, key) pairs scored per attention layer, logits for `n_logit_rows` rows."""
        layers = sum(self.layers[e.layer].flops(n_tokens, attended) for e in self.schedule)
        return layers + self.head.flops(n_logit_rows)

    def sizes(self):
        """The model's sizes under plain names, from the parts themselves: the width, the vocabulary, the number of
        layer runs, and the sizes of the first layer's parts (`layer_kinds` says how many distinct layers there are)."""
        out = {"layers": len(self.schedule), "hidden": self.plan.hidden_size}
        out.update(self.layers[0].sizes())
        out.update(self.head.sizes())
        out["layer_kinds"] = len({l.describe() for l in self.layers})
        return out

    def describe(self):
        """Lines for people: what the model is made of, from the parts' own descriptions."""
        kinds = {}
        for e in self.schedule:
            d = self.layers[e.layer].describe()
            kinds[d] = kinds.get(d, 0) + 1
        lines = [f"{str(self.dtype).replace('torch.', '')} weights, {self.weight_bytes() / 1e6:.1f} MB; width {self.plan.hidden_size}, "
                 f"{len(self.schedule)} layer runs over {len(self.layers)} layers, up to {self.plan.max_positions} positions",
                 f"  {self.embedding.describe()}"]
        lines += [f"  {n} x {d}" for d, n in kinds.items()]
        lines += [f"  {self.final_norm.describe()} -> {self.head.describe()}"]
        return lines

    def weight_bytes(self):
        """Bytes of every distinct device tensor the parts hold (a tied head counts once)."""
        seen, total = set(), 0

        def visit(obj):
            nonlocal total
            for v in vars(obj).values():
                if isinstance(v, torch.Tensor) and v.is_cuda and v.data_ptr() not in seen:
                    seen.add(v.data_ptr())
                    total += v.numel() * v.element_size()
                elif hasattr(v, "weight_shapes") and id(v) not in seen:
                    seen.add(id(v))
                    visit(v)
        for p in [self.embedding, self.final_norm, self.head] + self.layers:
            visit(p)
        return total

    # ------------------------------------------------------------------ forward
    def forward(self, ctx, cache, logits):
        """Run the step's tokens; write float32 logits of ctx.want_rows into `logits` [R, vocab]."""
        T, R = ctx.n_tokens, logits.shape[0]
        ws = ctx.ws
        ws.reset()
        x = ws.alloc((T, self.plan.hidden_size), torch.float32)
        with ctx.prof("embedding"):
            self.embedding.forward(ctx, x)
        for i, e in enumerate(self.schedule):
            entry = cache.entries[e.reads_cache_of if e.reads_cache_of is not None else i]
            nxt = self.schedule[i + 1].layer if i + 1 < len(self.schedule) else None
            ctx.weights_after = self.layers[nxt].first_weights() if nxt is not None else ()
            self.layers[e.layer].forward(ctx, x, entry)
        ctx.weights_after = ()
        if R:
            with ws.frame():
                xn = ws.alloc((R, self.plan.hidden_size), self.dtype)
                with ctx.prof("final_norm"):
                    self.final_norm.forward(ctx, x, xn, rows=ctx.want_rows)
                with ctx.prof("lm_head"):
                    self.head.forward(ctx, xn, logits)
        return logits


def expected_weights(plan, dtype=torch.float32):
    """The tensor names and shapes of a plan, without touching a device."""
    return DecoderModel(plan, dtype).expected_weights()
