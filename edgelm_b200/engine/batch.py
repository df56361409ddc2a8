"""A step's batch: which sequences bring which tokens, and everything the kernels need to know
about it, packed into one host buffer that goes to the device in one copy.

Tokens of all sequences are packed along one axis.  Per token: its id, its absolute position
and its sequence's index in the batch.  Per sequence: the position of its last new token, and
its row of each cache group's page table.  For steps with more than one token per sequence
there are also attention tiles (runs of at most `tile_tokens` consecutive tokens of one
sequence).  Nothing here is padded: a kernel sees exactly the tokens the step brings.
"""
from dataclasses import dataclass

import numpy as np
import torch

from .profiler import NULL_PROFILER


@dataclass
class Tiles:
    seq: torch.Tensor
    tok0: torch.Tensor
    ntok: torch.Tensor
    pos0: torch.Tensor
    count: int


# Splits of a sequence's pages in the decode attention, at most: with up to 16 the fold of the splits takes one trip to
# memory (it requests every split's values at once), and a step of one to four sequences of a small model has fewer
# blocks to launch (measured against 64: one sequence of 8,100 tokens at 135M sizes 0.741 -> 0.624 ms a step, four
# sequences of 128 to 2,300 tokens 0.644 -> 0.580; 32 splits are no better than 64).
MAX_SPLITS = 16


def make_tiles(seq_ntok, seq_pos0, tile_tokens):
    """Host lists (seq, first packed token, token count, first position) of the attention tiles."""
    seq, tok0, ntok, pos0 = [], [], [], []
    t0 = 0
    for s, (n, p0) in enumerate(zip(seq_ntok, seq_pos0)):
        for a in range(0, n, tile_tokens):
            seq.append(s)
            tok0.append(t0 + a)
            ntok.append(min(tile_tokens, n - a))
            pos0.append(p0 + a)
        t0 += n
    return seq, tok0, ntok, pos0


class StepContext:
    """What parts see of a step.  Built by the engine; parts read it.  The one thing written on the way is
    `weights_after` (by the model's loop and the block arrangement): the weight tensors that the step reads
    once the running part is done."""

    def __init__(self, ws, err, device, n_sms, profiler=None):
        self.ws, self.err, self.device, self.n_sms = ws, err, device, n_sms
        self.prof = profiler or NULL_PROFILER
        self.n_tokens = self.n_seqs = 0
        self.all_single = False
        self.weights_after = ()
        self.token_ids = self.tok_pos = self.tok_seq = self.seq_index = self.seq_pos = self.want_rows = None
        self.seq_slots = None          # real slot of each sequence (int32 device tensor): state groups, sampler streams
        self._tables = {}              # cache group id -> device page-table rows [n_seqs, stride]
        self._tiles = {}
        self._seq_ntok = self._seq_pos0 = None
        self._fixed_splits = None
        # positions, slots and page tables reach the device in one copy at the step's start, before its first kernel,
        # and the step's first kernels are the embedding's and a product's: a later kernel launched as a programmatic
        # dependent may read them before it waits for the kernel ahead of it
        self.metadata_precedes_kernels = True

    def page_table(self, group):
        """Device page-table rows [n_seqs, pages] of a key/value cache group, one row per sequence of the batch."""
        return self._tables[group.id]

    @property
    def seq_lengths(self):
        """Host list: how many tokens each sequence brings in this step (packed in this order)."""
        return list(self._seq_ntok)

    @property
    def seq_first_positions(self):
        """Host list: the absolute position of each sequence's first token of this step."""
        return list(self._seq_pos0)

    def decode_splits(self, n_kv_heads, resident=None):
        """Blocks per (sequence, kv head) of the decode attention: enough to fill the device, about two an SM.
        `resident`: how many of the kernel's blocks an SM holds at a time, if the caller knows.  With at least as
        many (sequence, kv head) pairs as SMs what counts is how full the last wave of blocks is: then the splits
        that fill one, two or three whole waves, the first of these that is at least 2 (measured at 32 kv heads,
        3 blocks an SM, steps of 8 sequences: 3 splits 2.00 ms against 2.03 with 2 and 2.21 with 1; of 16
        sequences: 2 splits 3.03 ms against 3.22 with 1)."""
        if self._fixed_splits is not None:
            return self._fixed_splits
        blocks = max(1, self.n_seqs * n_kv_heads)
        splits = int(min(MAX_SPLITS, max(1, (2 * self.n_sms + blocks - 1) // blocks)))
        if resident and blocks >= self.n_sms:
            for waves in (1, 2, 3):
                s = waves * resident * self.n_sms // blocks
                if s >= 2:
                    return int(min(MAX_SPLITS, s))
        return splits

    def tiles(self, tile_tokens):
        """Attention tiles of at most `tile_tokens` consecutive tokens of one sequence.  Sizes that
        the model's parts announced (`tile_sizes`) lie in the step's metadata already; any other
        size is built and copied now (which a replayed CUDA graph could not do)."""
        if tile_tokens not in self._tiles:
            seq, tok0, ntok, pos0 = make_tiles(self._seq_ntok, self._seq_pos0, tile_tokens)
            n = len(seq)
            host = torch.tensor(seq + tok0 + ntok + pos0, dtype=torch.int32).pin_memory()
            d = host.to(self.device, non_blocking=True)
            self._tiles[tile_tokens] = Tiles(d[:n], d[n:2 * n], d[2 * n:3 * n], d[3 * n:], n)
        return self._tiles[tile_tokens]


class BatchBuffers:
    """Pinned host staging and its device twin for the per-step metadata, sized once for the
    largest step; `fill` lays a step out and issues the single host-to-device copy."""

    def __init__(self, max_tokens, max_seqs, kv_groups, max_want, device, tile_sizes=()):
        self.device = device
        self.max_tokens, self.max_seqs, self.max_want = max_tokens, max_seqs, max_want
        self.groups = list(kv_groups)
        self.stride = {g.id: g.table.shape[1] for g in self.groups}
        self.tile_sizes = sorted(set(int(t) for t in tile_sizes))
        n = 3 * max_tokens + 4 * max_seqs + max_want + sum(max_seqs * s for s in self.stride.values())
        n += sum(4 * (max_tokens // t + max_seqs) for t in self.tile_sizes)
        self.host = torch.zeros(n, dtype=torch.int32).pin_memory()
        self.host_np = self.host.numpy()
        self.dev = torch.zeros(n, dtype=torch.int32, device=device)
        self.seq_index_full = torch.arange(max_seqs, dtype=torch.int32, device=device)
        self.last_bytes = 0
        self._copied = torch.cuda.Event()
        self._decode = None   # layout of the last step if it was one token per sequence: lets the next one be patched in place
        self._tile_cols = {}  # (tokens per sequence, first positions, tile size) -> the tiles' four columns: shapes come back

    def fill(self, ctx, token_ids, seq_slots, seq_ntok, seq_pos0, want_rows, cache):
        """Lay out the step and copy it; sets every tensor of `ctx` (views of the device buffer)."""
        T, B, R = len(token_ids), len(seq_slots), len(want_rows)
        if T > self.max_tokens or B > self.max_seqs or R > self.max_want:
            raise ValueError(f"a step of {T} tokens, {B} sequences and {R} wanted rows exceeds the buffers "
                             f"({self.max_tokens}, {self.max_seqs}, {self.max_want})")
        self._copied.synchronize()  # the previous step's copy has read the staging buffer
        h = self.host_np
        ntok = np.asarray(seq_ntok, dtype=np.int64)
        pos0 = np.asarray(seq_pos0, dtype=np.int64)
        o = 0
        views = {}

        def put(name, arr, n):
            nonlocal o
            h[o:o + n] = arr
            views[name] = (o, n)
            o += n

        put("token_ids", np.asarray(token_ids, dtype=np.int32), T)
        seq_of_tok = np.repeat(np.arange(B, dtype=np.int32), ntok)
        starts = np.concatenate([[0], np.cumsum(ntok)[:-1]])
        put("tok_pos", (np.arange(T, dtype=np.int64) - np.repeat(starts, ntok) + np.repeat(pos0, ntok)).astype(np.int32), T)
        put("tok_seq", seq_of_tok, T)
        put("seq_pos", (pos0 + ntok - 1).astype(np.int32), B)
        put("want_rows", np.asarray(want_rows, dtype=np.int32), R)
        slots = np.asarray(seq_slots, dtype=np.int64)
        put("seq_slots", slots.astype(np.int32), B)
        for g in self.groups:
            s = self.stride[g.id]
            put(("table", g.id), g.table[slots].reshape(-1), B * s)
        tile_counts = {}
        if T != B:  # steps of one token per sequence use no tiles
            shape = (tuple(int(v) for v in ntok), tuple(int(v) for v in pos0))
            for ts in self.tile_sizes:
                cols = self._tile_cols.get(shape + (ts,))
                if cols is None:
                    if len(self._tile_cols) >= 64:
                        self._tile_cols.clear()
                    cols = [np.asarray(col, dtype=np.int32) for col in make_tiles(list(shape[0]), list(shape[1]), ts)]
                    self._tile_cols[shape + (ts,)] = cols
                tile_counts[ts] = len(cols[0])
                for j, col in enumerate(cols):
                    put(("tiles", ts, j), col, len(col))
        self.dev[:o].copy_(self.host[:o], non_blocking=True)
        self._copied.record()
        self.last_bytes = o * 4

        def view(name):
            a, n = views[name]
            return self.dev[a:a + n]

        ctx.n_tokens, ctx.n_seqs = T, B
        ctx.all_single = bool(T == B and T > 0)
        ctx.token_ids, ctx.tok_pos, ctx.tok_seq = view("token_ids"), view("tok_pos"), view("tok_seq")
        ctx.seq_pos, ctx.want_rows = view("seq_pos"), view("want_rows")
        ctx.seq_index = self.seq_index_full[:B]
        ctx._tables = {g.id: view(("table", g.id)).view(B, self.stride[g.id]) for g in self.groups}
        ctx._tiles = {ts: Tiles(view(("tiles", ts, 0)), view(("tiles", ts, 1)), view(("tiles", ts, 2)), view(("tiles", ts, 3)), n)
                      for ts, n in tile_counts.items()}
        ctx._seq_ntok, ctx._seq_pos0 = [int(x) for x in ntok], [int(x) for x in pos0]
        ctx.seq_slots = view("seq_slots")
        self._decode = None
        if T == B and R == B:
            self._decode = {"slots": list(seq_slots), "pos": [int(x) for x in pos0], "views": views, "words": o,
                            "version": {g.id: g.version for g in self.groups}, "slot_index": slots}
        return ctx

    def refill_next_token(self, ctx, token_ids, seq_slots, seq_pos0):
        """The step after a step of one token per sequence, for the same sequences one position further: the
        staging buffer is patched in place (ids, positions, rows of the page tables that gained a page) instead of
        being laid out again, and copied.  `ctx` keeps its views.  False if the step is not of that kind."""
        d = self._decode
        if d is None or d["slots"] != seq_slots or len(token_ids) != len(seq_slots) or any(p != q + 1 for p, q in zip(seq_pos0, d["pos"])):
            return False
        B = len(seq_slots)
        self._copied.synchronize()  # the previous step's copy has read the staging buffer
        h, views = self.host_np, d["views"]
        a = views["token_ids"][0]
        h[a:a + B] = token_ids
        a = views["tok_pos"][0]
        h[a:a + B] += 1
        a = views["seq_pos"][0]
        h[a:a + B] += 1
        for g in self.groups:
            if g.version != d["version"][g.id]:    # a page was taken or given back since the rows were laid out
                s = self.stride[g.id]
                a = views[("table", g.id)][0]
                h[a:a + B * s] = g.table[d["slot_index"]].reshape(-1)
                d["version"][g.id] = g.version
        o = d["words"]
        if "copy" not in d:
            d["copy"] = (self.dev[:o], self.host[:o])   # (the two views, made once for the steps of this layout)
        d["copy"][0].copy_(d["copy"][1], non_blocking=True)
        self._copied.record()
        self.last_bytes = o * 4
        d["pos"] = list(seq_pos0)
        ctx._seq_pos0 = list(seq_pos0)
        return True
