"""Grouped-query causal attention over the paged cache.

q, k, v = h Wq^T, h Wk^T, h Wv^T (no bias; one matrix product over the three weights stacked);
rotary positions on q and k; k and v appended to the cache; for query head h and key head
h // (heads / kv_heads): softmax((q . K_j) / sqrt(head_dim)) over j <= the token's position,
times V; then x += a Wo^T (adarsh-sgh/edgelm src/kernels_ref.cpp:100-141, tools/elm.py:126-139).
"""
import math

import torch

from ..config.base import ConfigError
from ..csrc import ops
from . import linear
from .base import KVNeed, Part, as_matrix, nbytes
from .registry import register_mixer


@register_mixer("attention")
class Attention(Part):
    graph_safe = True
    takes_normed_input = True

    def __init__(self, spec, env):
        self.hidden = spec["hidden_size"]
        self.nh, self.nkv, self.hd = spec["num_heads"], spec["num_kv_heads"], spec["head_dim"]
        if self.nh <= 0 or self.nkv <= 0 or self.nh % self.nkv:
            raise ConfigError(f"attention: {self.nh} query heads are not a multiple of {self.nkv} key/value heads")
        if not (16 <= self.hd <= 256 and self.hd % 16 == 0):
            raise ConfigError(f"attention: head_dim {self.hd} is not taken by the attention kernels (16 to 256 in steps of 16)")
        self.names = dict(spec["names"])
        self.dtype = env.dtype
        self.positions = env.build_shared("positions", spec["positions"])
        # `window`: a token sees the last so many keys only, its own included (None: every key).  Nothing in the Llama
        # decoder sets it; a model with windowed layers names it in the spec of those layers' mixers.
        self.window = spec.get("window")
        if self.window is not None and int(self.window) < 1:
            raise ConfigError(f"attention: a window of {self.window} keys")
        self.window = int(self.window) if self.window is not None else None
        self.scale = 1.0 / math.sqrt(self.hd)
        self.group = self.nh // self.nkv
        self.tile_tokens = max(1, 32 // self.group)  # tokens whose heads fill one block of the prefill kernel
        self.w_qkv = self.w_o = None
        self._mma = None  # whether the mma.sync prefill kernel takes this head size (asked once a device is there)
        self._tc = None   # whether the tcgen05 prefill kernel does

    def sizes(self):
        out = {"heads": self.nh, "kv_heads": self.nkv, "head_dim": self.hd, **self.positions.sizes()}
        if self.window is not None:
            out["window"] = self.window
        return out

    def flops(self, n_tokens, attended):
        proj = 2.0 * n_tokens * self.hidden * (2 * self.nh + 2 * self.nkv) * self.hd    # q, k, v and the output projection
        if self.window is not None:
            attended = min(attended, n_tokens * self.window)
        return proj + 4.0 * attended * self.nh * self.hd                                # scores and weighted values

    def weight_shapes(self, prefix):
        n = self.names
        return {prefix + n["q"]: (self.nh * self.hd, self.hidden), prefix + n["k"]: (self.nkv * self.hd, self.hidden),
                prefix + n["v"]: (self.nkv * self.hd, self.hidden), prefix + n["o"]: (self.hidden, self.nh * self.hd)}

    def load(self, tensors, prefix, device):
        n = self.names
        # the three projections share their input: stacked once here, they are one matrix product per step
        self.w_qkv = torch.cat([as_matrix(tensors[prefix + n[k]], self.dtype, device) for k in ("q", "k", "v")], dim=0).contiguous()
        self.w_o = as_matrix(tensors[prefix + n["o"]], self.dtype, device)
        self.positions.load(tensors, prefix, device)

    def _decode_resident(self):
        """Blocks of the tensor-core decode attention kernel that an SM holds (its shared memory: the staged
        queries and four warps' key and value tiles of 64 padded rows), or None where that kernel does not run."""
        if self.dtype != torch.bfloat16 or self.hd not in (32, 64, 96, 128) or self.window is not None:
            return None
        head = (16 * (self.hd + 8) * 2 + 2 * self.hd * 2 + 4 * 8 + 127) // 128 * 128
        block = head + 4 * 2 * 64 * (self.hd + 8) * 2
        return max(1, (227 * 1024) // (block + 1024))

    def first_weights(self):
        return (self.w_qkv,)

    def cache_need(self):
        return KVNeed(self.nkv, self.hd, self.window)

    # Steps whose longest sequence brings fewer new tokens than this stay on the mma.sync kernel (tiles of 64 rows):
    # measured at 9 heads of 64 (32 heads): 128 new tokens 4.6 (5.0) us against 5.7 (5.8) us on tcgen05, 256 tokens
    # 7.0 (7.4) against 6.4 (6.7), 2,048 tokens 44.6 (104.5) against 17.6 (50.1).
    TC_PREFILL_MIN_TOKENS = 256

    def tile_sizes(self):
        sizes = ()
        if self._tc_prefill():
            sizes += (ops.TC_PREFILL_TILE,)
        return sizes + ((ops.MMA_PREFILL_TILE,) if self._mma_prefill() else (self.tile_tokens,))

    def _mma_prefill(self):
        if self._mma is None:   # (the tensor-core kernels have no lower key bound: a windowed mixer stays on the CUDA cores)
            self._mma = self.window is None and ops.attn_prefill_mma_takes(self.dtype, self.hd)
        return self._mma

    def _tc_prefill(self):
        if self._tc is None:
            self._tc = self.window is None and ops.attn_prefill_tc_takes(self.dtype, self.hd)
        return self._tc

    def workspace_bytes(self, n_tokens, n_seqs):
        qkv = nbytes((n_tokens, (self.nh + 2 * self.nkv) * self.hd), self.dtype)
        out = nbytes((n_tokens, self.nh * self.hd), self.dtype)
        h = nbytes((n_tokens, self.hidden), self.dtype)  # the normalised input, when it is written out
        # split partials of decoding: sequences x heads x splits cells; (sequences x kv heads) x splits is at most
        # 2 SMs + (sequences x kv heads), or three waves of resident blocks (`decode_splits`); up to 256 SMs
        cells = self.group * max(2 * 256 + n_seqs * self.nkv, 3 * 256 * (self._decode_resident() or 0))
        part = nbytes((cells * self.hd,), torch.float32) + nbytes((cells * 2,), torch.float32)
        return qkv + out + h + part

    def _attend_decode(self, ctx, qkv, a, cache, table, tables):
        """One new token per sequence.  `tables`: the rotation tables if rotation and cache append are this kernel's
        to do (then `qkv` holds the raw projections), else None."""
        ws = ctx.ws
        cos, sin = tables if tables is not None else (None, None)
        splits = ctx.decode_splits(self.nkv, self._decode_resident())
        part_o = part_ml = None
        if splits > 1:
            part_o = ws.alloc((ctx.n_seqs * self.nh * splits * self.hd,), torch.float32)
            part_ml = ws.alloc((ctx.n_seqs * self.nh * splits * 2,), torch.float32)
        ready = getattr(ctx, "metadata_precedes_kernels", False)
        with ctx.prof("attn_decode"):
            if tables is not None:
                ops.attn_decode_rope(qkv, a, cache.k, cache.v, table, ctx.seq_index, ctx.seq_pos, cos, sin, ctx.n_seqs, self.nh,
                                     self.nkv, self.hd, self.scale, splits, part_o, part_ml, err=ctx.err, window=self.window,
                                     meta_ready=ready)
            else:
                ops.attn_decode(qkv, a, cache.k, cache.v, table, ctx.seq_index, ctx.seq_pos, ctx.n_seqs, self.nh, self.nkv,
                                self.hd, self.scale, splits, part_o, part_ml, err=ctx.err, window=self.window, meta_ready=ready)

    def forward(self, ctx, h, x, cache):
        T = h.shape[0]
        ws = ctx.ws
        qkv = ws.alloc((T, (self.nh + 2 * self.nkv) * self.hd), self.dtype)
        a = ws.alloc((T, self.nh * self.hd), self.dtype)
        table = ctx.page_table(cache.group)
        tables = self.positions.rotation_tables() if hasattr(self.positions, "rotation_tables") else None
        encoded = False
        if not ctx.all_single and hasattr(self.positions, "project_encode_append"):
            # a prompt step: the position encoding may know a kernel that projects, encodes and appends in one
            with ctx.prof("qkv_proj_rope_append"):
                encoded = self.positions.project_encode_append(ctx, h, self.w_qkv, qkv, cache, self.nh, self.nkv)
        if not encoded:
            with ctx.prof("qkv_proj"):
                linear.matmul(ctx, h, self.w_qkv, qkv, prefetch=(self.w_o,))
        if ctx.all_single and tables is not None:
            # one token per sequence: rotation, append and attention in one kernel
            self._attend_decode(ctx, qkv, a, cache, table, tables)
            with ctx.prof("o_proj_residual"):
                linear.matmul(ctx, a, self.w_o, x, epilogue=linear.EPI_RESIDUAL, residual=x, prefetch=ctx.weights_after)
            return
        if not encoded:
            with ctx.prof("rope_kv_append"):
                self.positions.encode_and_append(ctx, qkv, cache, self.nh, self.nkv)
        if ctx.all_single:
            self._attend_decode(ctx, qkv, a, cache, table, None)
        elif self._tc_prefill() and max(ctx.seq_lengths) >= self.TC_PREFILL_MIN_TOKENS:
            tiles = ctx.tiles(ops.TC_PREFILL_TILE)
            with ctx.prof("attn_prefill"):
                ops.attn_prefill_tc(qkv, a, cache.k, cache.v, table, ctx.seq_index, tiles.seq, tiles.tok0, tiles.ntok, tiles.pos0,
                                    tiles.count, self.nh, self.nkv, self.hd, self.scale, ctx.err)
        elif self._mma_prefill():
            tiles = ctx.tiles(ops.MMA_PREFILL_TILE)
            with ctx.prof("attn_prefill"):
                ops.attn_prefill_mma(qkv, a, cache.k, cache.v, table, ctx.seq_index, tiles.seq, tiles.tok0, tiles.ntok,
                                     tiles.pos0, tiles.count, self.nh, self.nkv, self.hd, self.scale,
                                     max_keys=max(p + n for p, n in zip(ctx.seq_first_positions, ctx.seq_lengths)))
        else:
            tiles = ctx.tiles(self.tile_tokens)
            with ctx.prof("attn_prefill"):
                ops.attn_prefill(qkv, a, cache.k, cache.v, table, ctx.seq_index, tiles.seq, tiles.tok0, tiles.ntok,
                                 tiles.pos0, tiles.count, self.tile_tokens, self.nh, self.nkv, self.hd, self.scale, window=self.window)
        with ctx.prof("o_proj_residual"):
            linear.matmul(ctx, a, self.w_o, x, epilogue=linear.EPI_RESIDUAL, residual=x, prefetch=ctx.weights_after)
