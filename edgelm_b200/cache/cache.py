"""The cache of a model: what its mixers keep per sequence between steps.

A sequence holds a *slot* while it lives.  Each schedule entry whose mixer keeps something has
a *cache entry*; entries with the same need form a *group* with storage of its own:

  KV group     keys and values in pages of 64 positions, [entry][page][kv_head][64][head_dim]
               twice (K and V), one pool of pages and one page table [slot][page index] for
               the whole group, since all its entries grow together.  A sequence takes pages as
               it grows and gives them back when it ends; a reused page is not cleared, because
               no kernel reads a position beyond a sequence's length.
  state group  a float32 tensor of fixed shape per (entry, slot), zeroed when the slot is
               taken.  The Llama decoder has none; a mixer with a recurrent state would.

Lengths are per slot and shared by all groups.  Everything a step needs on the device about
the cache (the batch's rows of the page tables) is packed by the engine into the step's
metadata; this class owns the storage and the bookkeeping.
"""
import numpy as np
import torch

from ..parts.base import KVNeed, StateNeed
from .slots import CacheError, FreeList

PAGE = 64


def pages_for(n_tokens):
    return (int(n_tokens) + PAGE - 1) // PAGE


class CacheEntry:
    """What a mixer receives: its own layer of a group's storage."""

    def __init__(self, group, index):
        self.group, self.index = group, index

    @property
    def k(self):
        return self.group.k[self.index]

    @property
    def v(self):
        return self.group.v[self.index]

    @property
    def state(self):
        return self.group.state[self.index]


class KVGroup:
    def __init__(self, gid, need, n_entries, n_pages, n_slots, max_pages_per_seq, dtype, device):
        self.id, self.need, self.n_entries = gid, need, n_entries
        self.pool = FreeList(n_pages, f"page of cache group {gid}")
        self.table = np.full((n_slots, max_pages_per_seq), -1, dtype=np.int32)  # host copy; rows go to the device per step
        self.n_held = np.zeros(n_slots, dtype=np.int32)
        self.k = self.v = None
        if device is not None:
            shape = (n_entries, n_pages, need.n_kv_heads, PAGE, need.head_dim)
            self.k = torch.zeros(shape, dtype=dtype, device=device)
            self.v = torch.zeros(shape, dtype=dtype, device=device)

    def bytes_per_token(self, itemsize):
        return 2 * self.n_entries * self.need.n_kv_heads * self.need.head_dim * itemsize

    def ensure(self, slot, length):
        want = pages_for(length)
        if want > self.table.shape[1]:
            raise CacheError(f"a sequence of {length} tokens needs {want} pages; the table has {self.table.shape[1]} per sequence")
        have = int(self.n_held[slot])
        if want - have > self.pool.available():
            raise CacheError(f"the cache is full: {want - have} more pages of {PAGE} tokens are needed, {self.pool.available()} are free")
        for i in range(have, want):
            self.table[slot, i] = self.pool.take()
        self.n_held[slot] = max(have, want)

    def release(self, slot):
        for i in range(int(self.n_held[slot])):
            self.pool.give(int(self.table[slot, i]))
            self.table[slot, i] = -1
        self.n_held[slot] = 0


class StateGroup:
    def __init__(self, gid, need, n_entries, n_slots, device):
        self.id, self.need, self.n_entries = gid, need, n_entries
        self.state = None
        if device is not None:
            self.state = torch.zeros((n_entries, n_slots) + tuple(need.shape), dtype=torch.float32, device=device)

    def reset(self, slot):
        if self.state is not None:
            self.state[:, slot].zero_()


class SequenceCache:
    """`needs`: one KVNeed, StateNeed or None per schedule entry (None: keeps nothing, or reads
    another entry's cache).  `max_tokens` sizes every KV group: the most tokens that live
    sequences hold at one time, each sequence's count rounded up to whole pages."""

    def __init__(self, needs, max_tokens, max_positions, dtype=torch.float32, device=None, max_seqs=None):
        n_pages = pages_for(max_tokens)
        if n_pages <= 0:
            raise CacheError("the cache needs room for at least one page of tokens")
        self.max_positions = int(max_positions)
        self.n_pages = n_pages
        self.n_slots = min(n_pages, int(max_seqs)) if max_seqs else n_pages
        self.max_pages_per_seq = min(n_pages, pages_for(max_positions))
        self.slots = FreeList(self.n_slots, "slot")
        self.length = np.zeros(self.n_slots, dtype=np.int64)
        self.dtype, self.device = dtype, device
        self.groups, self.entries = [], []
        by_need = {}
        for i, need in enumerate(needs):
            if need is not None:
                by_need.setdefault(need, []).append(i)
        where = {}
        for need, idxs in by_need.items():
            gid = len(self.groups)
            if isinstance(need, KVNeed):
                if need.window is not None:
                    raise CacheError("a windowed key/value group has no storage class yet")
                g = KVGroup(gid, need, len(idxs), n_pages, self.n_slots, self.max_pages_per_seq, dtype, device)
            elif isinstance(need, StateNeed):
                g = StateGroup(gid, need, len(idxs), self.n_slots, device)
            else:
                raise CacheError(f"unknown cache need {need!r}")
            self.groups.append(g)
            for j, i in enumerate(idxs):
                where[i] = CacheEntry(g, j)
        self.entries = [where.get(i) for i in range(len(needs))]
        self.kv_groups = [g for g in self.groups if isinstance(g, KVGroup)]
        self.state_groups = [g for g in self.groups if isinstance(g, StateGroup)]

    # ------------------------------------------------------------------ sequences
    def open(self):
        """A slot for a new sequence of length 0."""
        slot = self.slots.take()
        self.length[slot] = 0
        for g in self.state_groups:
            g.reset(slot)
        return slot

    def _held(self, slot):
        if slot not in self.slots._held:
            raise CacheError(f"slot {slot} is not held by a live sequence")

    def reserve(self, slot, n_new):
        """Room for `n_new` more tokens of the sequence; all or nothing per group."""
        self._held(slot)
        new_len = int(self.length[slot]) + int(n_new)
        if new_len > self.max_positions:
            raise CacheError(f"a sequence of {new_len} tokens is longer than the {self.max_positions} positions the model has")
        for g in self.kv_groups:
            g.ensure(slot, new_len)

    def advance(self, slot, n_new):
        """The step that wrote `n_new` tokens is issued: they count from now on."""
        self._held(slot)
        self.length[slot] += int(n_new)

    def close(self, slot):
        """The sequence is over: its pages and its slot go back."""
        self._held(slot)
        for g in self.kv_groups:
            g.release(slot)
        self.length[slot] = 0
        self.slots.give(slot)

    def footprint(self, length):
        """Tokens of room, in whole pages, that one sequence of `length` tokens takes from the fullest key/value
        group; 0 for a model whose mixers keep states of fixed size only (such a model is bound by slots alone)."""
        return max((pages_for(length) * PAGE for _ in self.kv_groups), default=0)

    @property
    def capacity_tokens(self):
        """Tokens of room for live sequences, each counted by `footprint`; None: no bound but the slots."""
        return self.n_pages * PAGE if self.kv_groups else None

    def storage_bytes(self):
        total = 0
        for g in self.groups:
            for t in (getattr(g, "k", None), getattr(g, "v", None), getattr(g, "state", None)):
                if t is not None:
                    total += t.numel() * t.element_size()
        return total

    def describe(self):
        """Lines for people: slots, and each group's storage as the group accounts for it."""
        lines = [f"{self.n_slots} slots, {self.storage_bytes() / 1e6:.2f} MB"]
        for g in self.kv_groups:
            lines.append(f"  keys/values of {g.n_entries} layer run(s): {g.need.n_kv_heads} heads of {g.need.head_dim}, {self.n_pages} pages "
                         f"of {PAGE} tokens, {g.bytes_per_token(torch.empty(0, dtype=self.dtype).element_size())} B a token")
        for g in self.state_groups:
            lines.append(f"  fixed-size state of {g.n_entries} layer run(s): float32 {list(g.need.shape)} a sequence")
        return lines

    def tokens_held(self):
        """Tokens of room that live sequences hold, in whole pages."""
        return max((int(g.n_held.sum()) * PAGE for g in self.kv_groups), default=0)

    def bytes_per_token(self):
        item = torch.empty(0, dtype=self.dtype).element_size()
        return sum(g.bytes_per_token(item) for g in self.kv_groups)

    def check(self):
        """No slot or page lost, held twice, or held by a dead sequence."""
        self.slots.check()
        for g in self.kv_groups:
            g.pool.check()
            seen = set()
            for s in range(self.n_slots):
                row = [int(p) for p in g.table[s] if p >= 0]
                assert len(row) == int(g.n_held[s]), "a page table row and its count disagree"
                if s not in self.slots._held:
                    assert not row, "a free slot holds pages"
                assert int(g.n_held[s]) >= pages_for(self.length[s]), "a sequence is longer than its pages"
                for p in row:
                    assert p not in seen, "a page is held twice"
                    seen.add(p)
            assert seen == g.pool.held(), "the page tables and the page pool disagree"
