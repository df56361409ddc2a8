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
    """Keys and values of the schedule entries with one need.  With `need.window` the group keeps, per sequence, only
    the pages that the next token can still see: `trim` gives back the pages that fell out of the window, and the
    pool is sized for what sequences hold at one time (the window plus the tokens of one piece of a step), not for
    whole sequences.  The page table stays indexed by position // 64; entries of pages given back are -1, and the
    attention kernels of a windowed mixer never look before the window."""

    def __init__(self, gid, need, n_entries, n_pages, n_slots, max_pages_per_seq, dtype, device, piece_tokens=None):
        self.id, self.need, self.n_entries = gid, need, n_entries
        self.window = need.window
        self.pages_per_seq = max_pages_per_seq
        if self.window is not None:
            self.pages_per_seq = min(max_pages_per_seq, pages_for(self.window - 1 + int(piece_tokens)) + 1)
            n_pages = min(n_pages, n_slots * self.pages_per_seq)
        self.n_pages = n_pages
        self.pool = FreeList(n_pages, f"page of cache group {gid}")
        self.table = np.full((n_slots, max_pages_per_seq), -1, dtype=np.int32)  # host copy; rows go to the device per step
        self.n_held = np.zeros(n_slots, dtype=np.int32)
        self.low = np.zeros(n_slots, dtype=np.int32)      # a sequence holds the pages low .. low + n_held - 1
        self.version = 0                                  # counts changes of the table (a step's metadata is patched when it moved)
        self.k = self.v = None
        if device is not None:
            shape = (n_entries, n_pages, need.n_kv_heads, PAGE, need.head_dim)
            self.k = torch.zeros(shape, dtype=dtype, device=device)
            self.v = torch.zeros(shape, dtype=dtype, device=device)

    def bytes_per_token(self, itemsize):
        return 2 * self.n_entries * self.need.n_kv_heads * self.need.head_dim * itemsize

    def first_page(self, position):
        """The first page that the token at `position` sees a key of."""
        return 0 if self.window is None else max(0, int(position) - self.window + 1) // PAGE

    def pages_of(self, length):
        """Pages that a sequence of `length` tokens holds at most at one time."""
        return min(pages_for(length), self.pages_per_seq)

    def ensure(self, slot, old_length, new_length):
        """Pages for the tokens old_length .. new_length - 1 and for every key they see."""
        want_hi = pages_for(new_length)
        if want_hi > self.table.shape[1]:
            raise CacheError(f"a sequence of {new_length} tokens needs {want_hi} pages; the table has {self.table.shape[1]} per sequence")
        if self.n_held[slot] == 0:
            self.low[slot] = self.first_page(old_length)
        have_hi = int(self.low[slot]) + int(self.n_held[slot])
        if want_hi - have_hi > self.pool.available():
            raise CacheError(f"the cache is full: {want_hi - have_hi} more pages of {PAGE} tokens are needed, {self.pool.available()} are free")
        for i in range(have_hi, want_hi):
            self.table[slot, i] = self.pool.take()
        if want_hi > have_hi:
            self.n_held[slot] += want_hi - have_hi
            self.version += 1

    def trim(self, slot, length):
        """The sequence now has `length` tokens: pages that its next token no longer sees go back (windowed groups)."""
        if self.window is None:
            return
        new_low = self.first_page(length)
        low, n = int(self.low[slot]), int(self.n_held[slot])
        gone = max(0, min(new_low, low + n) - low)
        for i in range(low, low + gone):
            self.pool.give(int(self.table[slot, i]))
            self.table[slot, i] = -1
        if gone:
            self.n_held[slot] = n - gone
            self.low[slot] = low + gone
            self.version += 1

    def release(self, slot):
        low, n = int(self.low[slot]), int(self.n_held[slot])
        for i in range(low, low + n):
            self.pool.give(int(self.table[slot, i]))
            self.table[slot, i] = -1
        self.n_held[slot] = 0
        self.low[slot] = 0
        if n:
            self.version += 1


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

    PIECE_TOKENS = 256   # a sequence of a model with windowed groups brings at most so many tokens to one micro-step

    def __init__(self, needs, max_tokens, max_positions, dtype=torch.float32, device=None, max_seqs=None, piece_tokens=None):
        n_pages = pages_for(max_tokens)
        if n_pages <= 0:
            raise CacheError("the cache needs room for at least one page of tokens")
        self.max_positions = int(max_positions)
        self.n_pages = n_pages
        self.n_slots = min(n_pages, int(max_seqs)) if max_seqs else n_pages
        self.max_pages_per_seq = min(n_pages, pages_for(max_positions))
        self.slots = FreeList(self.n_slots, "slot")
        self._quiet = None   # [slots, their indices, steps]: so many further one-token steps of exactly these sequences need no look at the pages
        self.length = np.zeros(self.n_slots, dtype=np.int64)
        self.dtype, self.device = dtype, device
        self.groups, self.entries = [], []
        windowed = any(isinstance(n, KVNeed) and n.window is not None for n in needs)
        # with a windowed group, steps are cut so that a sequence brings at most `piece_tokens` tokens at a time: what
        # such a group must hold per sequence is then the window and one piece, whatever the prompt's length
        self.piece_tokens = int(piece_tokens or self.PIECE_TOKENS) if windowed else None
        by_need = {}
        for i, need in enumerate(needs):
            if need is not None:
                by_need.setdefault(need, []).append(i)
        where = {}
        for need, idxs in by_need.items():
            gid = len(self.groups)
            if isinstance(need, KVNeed):
                if need.window is not None and need.window < 1:
                    raise CacheError(f"a window of {need.window} keys")
                g = KVGroup(gid, need, len(idxs), n_pages, self.n_slots, self.max_pages_per_seq, dtype, device, self.piece_tokens)
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
        self._quiet = None
        slot = self.slots.take()
        self.length[slot] = 0
        for g in self.state_groups:
            g.reset(slot)
        return slot

    def _held(self, slot):
        if slot not in self.slots._held:
            raise CacheError(f"slot {slot} is not held by a live sequence")

    def reserve(self, slot, n_new):
        """Room for `n_new` more tokens of the sequence; all or nothing per group.  A windowed group reserves for the
        first piece only (at most `piece_tokens` tokens): the engine asks again before each later piece, after
        `advance` gave back what the earlier ones no longer need."""
        self._held(slot)
        self._quiet = None
        old_len = int(self.length[slot])
        new_len = old_len + int(n_new)
        if new_len > self.max_positions:
            raise CacheError(f"a sequence of {new_len} tokens is longer than the {self.max_positions} positions the model has")
        for g in self.kv_groups:
            g.ensure(slot, old_len, new_len if g.window is None else min(new_len, old_len + self.piece_tokens))

    def advance(self, slot, n_new):
        """The step that wrote `n_new` tokens is issued: they count from now on."""
        self._held(slot)
        self._quiet = None
        self.length[slot] += int(n_new)
        for g in self.kv_groups:
            g.trim(slot, int(self.length[slot]))

    def reserve_next(self, slots):
        """`reserve(slot, 1)` for every slot of a step of one token each (distinct slots), with the same outcome; the
        pages are looked at for the sequences that cross into a new page only, which is one step in 64."""
        q = self._quiet
        if q is not None and q[2] > 0 and q[0] == tuple(slots):
            q[2] -= 1     # (nothing else touched the cache since these sequences' last step, and no page edge is near)
            return
        self._quiet = None
        held = self.slots._held
        for s in slots:
            if s not in held:
                raise CacheError(f"slot {s} is not held by a live sequence")
        idx = np.asarray(slots, dtype=np.int64)
        new_len = self.length[idx] + 1
        if int(new_len.max()) > self.max_positions:
            raise CacheError(f"a sequence of {int(new_len.max())} tokens is longer than the {self.max_positions} positions the model has")
        want = (new_len + (PAGE - 1)) // PAGE
        for g in self.kv_groups:
            short = want > g.low[idx] + g.n_held[idx]
            if short.any():
                for s in idx[short]:
                    g.ensure(int(s), int(self.length[s]), int(self.length[s]) + 1)
        if self.kv_groups and all(g.window is None for g in self.kv_groups):
            # how many further steps of these sequences need nothing: none reaches a page edge or the last position
            room = self.max_positions - new_len
            for g in self.kv_groups:
                room = np.minimum(room, (g.low[idx] + g.n_held[idx]) * PAGE - new_len)
            self._quiet = [tuple(slots), idx, int(room.min())]

    def advance_next(self, slots):
        """`advance(slot, 1)` for every slot that `reserve_next` was called with."""
        q = self._quiet
        idx = q[1] if q is not None and q[0] == tuple(slots) else np.asarray(slots, dtype=np.int64)
        self.length[idx] += 1
        for g in self.kv_groups:
            if g.window is not None:
                for s in slots:
                    g.trim(s, int(self.length[s]))

    def close(self, slot):
        """The sequence is over: its pages and its slot go back."""
        self._held(slot)
        self._quiet = None
        for g in self.kv_groups:
            g.release(slot)
        self.length[slot] = 0
        self.slots.give(slot)

    def footprint(self, length):
        """Tokens of room, in whole pages, that one sequence of `length` tokens takes from the fullest key/value
        group; 0 for a model whose mixers keep states of fixed size only (such a model is bound by slots alone)."""
        # (each group has a pool of its own; in units of the largest pool a batch fits if the sum of its sequences'
        # footprints stays within `capacity_tokens`)
        return max((-(-g.pages_of(length) * self.n_pages // g.n_pages) * PAGE for g in self.kv_groups), default=0)

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
            win = f", the last {g.window} keys of a sequence" if g.window is not None else ""
            lines.append(f"  keys/values of {g.n_entries} layer run(s): {g.need.n_kv_heads} heads of {g.need.head_dim}{win}, {g.n_pages} pages "
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
                low, n = int(g.low[s]), int(g.n_held[s])
                assert len(row) == n and all(g.table[s, i] >= 0 for i in range(low, low + n)), "a page table row and its range disagree"
                if s not in self.slots._held:
                    assert not row, "a free slot holds pages"
                assert low + n >= pages_for(self.length[s]), "a sequence is longer than its pages"
                assert low <= g.first_page(self.length[s]) or n == 0, "a page that the next token sees was given back"
                assert g.window is None or n <= g.pages_per_seq, "a windowed group holds more than its window and one piece"
                for p in row:
                    assert p not in seen, "a page is held twice"
                    seen.add(p)
            assert seen == g.pool.held(), "the page tables and the page pool disagree"
