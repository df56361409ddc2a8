"""The interface of a part.

Every part, whatever its role, answers four questions:

  weight_shapes(prefix) -> {tensor name: shape}   which tensors it wants from the weights file
  load(tensors, prefix, device)                   take them (name -> CPU tensor in the stored dtype)
  workspace_bytes(n_tokens, n_seqs) -> int        scratch it takes from the step's workspace
  cache_need() -> KVNeed | StateNeed | None       what it keeps per sequence between steps (mixers)

two about itself, which the command line and the benchmark add up instead of reading any
architecture's configuration fields:

  sizes() -> {name: value}                        its sizes and constants under plain names
  flops(n_tokens, attended) -> float              floating-point operations of a step of `n_tokens` tokens in which
                                                  `attended` (query, key) pairs are scored (matrix products count 2 per
                                                  multiply-add; norms, rotations and activations are left out)

and has one `forward`, whose signature depends on the role:

  embedding   forward(ctx, x)                     x[T, D] float32 <- rows of the table for ctx.token_ids
  norm        forward(ctx, x, out, rows=None)     out <- norm(x[rows]) in the compute dtype
  mixer       forward(ctx, h, x, cache)           x += mix(h)          (cache: its entry, or None)
  ffn         forward(ctx, h, x)                  x += feed_forward(h)
  block       forward(ctx, x, cache)              one whole layer on the residual stream x
  head        forward(ctx, x, rows, logits)       logits[R, V] float32 for the wanted rows of x
  positions   encode_and_append(...)              position-encode q and k, append k and v to the cache

x is the residual stream, float32 [tokens, hidden] in both precisions; h is the normalised
input in the compute dtype.  Mixers and feed-forwards ADD into x, so that the residual sum can
be fused into their last matrix product.  `ctx` is the step's StepContext: positions, sequence
boundaries, page tables, workspace; tokens of all sequences are packed along the first axis.
"""
from dataclasses import dataclass
from typing import Tuple

import torch


@dataclass(frozen=True)
class KVNeed:
    """Keys and values for every position (`window` None) or for the last `window` positions."""
    n_kv_heads: int
    head_dim: int
    window: int = None


@dataclass(frozen=True)
class StateNeed:
    """A state of fixed size per sequence: a float32 tensor of this shape, zero when a sequence starts."""
    shape: Tuple[int, ...]


class Part:
    kind = "?"
    # True if `forward` only launches work on the current stream from fixed-address buffers (no host
    # reads of device data, no allocation): then steps through it may be replayed from a CUDA graph.
    graph_safe = False

    def weight_shapes(self, prefix):
        return {}

    def load(self, tensors, prefix, device):
        pass

    def workspace_bytes(self, n_tokens, n_seqs):
        return 0

    def cache_need(self):
        return None

    def sizes(self):
        return {}

    def flops(self, n_tokens, attended):
        return 0.0

    def describe(self):
        """One line: the kind and the sizes."""
        inner = ", ".join(f"{k} {v}" for k, v in self.sizes().items())
        return f"{self.kind}({inner})"

    def first_weights(self):
        """The weight tensors that this part's `forward` reads first (at most two): whoever runs before it may
        start them on their way into the L2 cache.  Default: none."""
        return ()

    def tile_sizes(self):
        """Sizes of attention tiles (`ctx.tiles(n)`) this part will ask for: the engine lays them out
        with the step's metadata, which is what lets a whole step be replayed from a CUDA graph."""
        return ()


def as_matrix(t, dtype, device):
    """A 2-D weight on the device in the compute dtype (bfloat16 rounding is to nearest even)."""
    return t.to(device=device, dtype=dtype).contiguous()


def as_vector(t, device):
    """A 1-D weight on the device; vectors are computed with in float32 in both precisions."""
    return t.to(device=device, dtype=torch.float32).contiguous()


def align_up(n, a=256):
    return (n + a - 1) // a * a


def nbytes(shape, dtype):
    n = 1
    for s in shape:
        n *= int(s)
    return align_up(n * torch.empty(0, dtype=dtype).element_size())
