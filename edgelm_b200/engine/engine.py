"""The engine: a model, its cache, and the one step function.

`step(entries)` is the only way tokens reach the model.  Each entry names a live sequence,
brings its next tokens (a whole prompt, a piece of one, or one decoded token) and says at which
of these tokens logits are wanted.  The step runs exactly the tokens it is given, as one packed
batch, on top of what earlier steps left in the cache, and returns float32 logits [wanted,
vocab] in the order of the entries and of their wanted places.  Sequences of any lengths share
a step; nothing is padded.  A step larger than `max_step_tokens` is cut into consecutive
smaller ones, which gives the same logits, since every token attends through the cache.

Decoding one token per sequence can be replayed from a CUDA graph (`decode_sampled`): the
graph holds the forward pass and the sampler; per step the host copies the batch's metadata
in (one copy) and the sampled tokens out (one copy).
"""
from dataclasses import dataclass
from typing import List, Sequence

import numpy as np
import torch

from ..cache import SequenceCache
from ..config import read_config
from ..csrc import ops
from ..sampling.device import DeviceSampler
from ..weights import load_checked
from .arena import Workspace
from .batch import BatchBuffers, StepContext
from .model import DecoderModel
from .profiler import Profiler

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
          "f32": torch.float32}


class EngineError(RuntimeError):
    pass


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


def load_model(model_dir, dtype="bfloat16", device="cuda:0"):
    """Model folder (config.json + *.safetensors) -> DecoderModel on the device.  The model
    class comes from config.json through the architecture registry."""
    ops.require_device()
    torch_dtype = DTYPES[dtype] if isinstance(dtype, str) else dtype
    config = read_config(model_dir)
    model = DecoderModel(config.plan(), torch_dtype)
    tensors = load_checked(model_dir, model.expected_weights(), model.ignorable_weights())
    model.load(tensors, device)
    model.config = config
    return model


class Engine:
    def __init__(self, model: DecoderModel, max_tokens, max_step_tokens=8192, max_seqs=None, profile=False,
                 use_graphs=True):
        ops.require_device()
        if model.device is None:
            raise EngineError("the model has no weights yet (load them first)")
        self.model, self.device = model, model.device
        self.plan = model.plan
        self.cache = SequenceCache(model.cache_needs(), max_tokens, self.plan.max_positions, dtype=model.dtype,
                                   device=self.device, max_seqs=max_seqs)
        self.max_step_tokens = int(min(max_step_tokens, max(64, self.cache.n_pages * 64)))
        self.max_step_seqs = min(self.cache.n_slots, self.max_step_tokens)
        props = torch.cuda.get_device_properties(self.device)
        self.n_sms = props.multi_processor_count
        ws_bytes = model.workspace_bytes(self.max_step_tokens, self.max_step_seqs, self.max_step_tokens)
        self.ws = Workspace(ws_bytes, self.device)
        # the device error word: kernels OR a bit into it for bad input (a token id, a position, a page) and for a
        # bounded wait that ran out; every call that hands results to the host reads it with them
        # (the tokens that a graph-replayed decode step samples lie right behind it, so that one copy brings both)
        self._result = torch.zeros(1 + self.max_step_seqs, dtype=torch.int32, device=self.device)
        self._result_host = torch.zeros(1 + self.max_step_seqs, dtype=torch.int32).pin_memory()
        self._result_np = self._result_host.numpy()
        self.err = self._result[:1]
        self._err_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._err_copied = torch.cuda.Event()
        self._err_pending = False
        self.buffers = BatchBuffers(self.max_step_tokens, self.max_step_seqs, self.cache.kv_groups, self.max_step_tokens,
                                    self.device, tile_sizes=model.tile_sizes())
        self.profiler = Profiler() if profile else None
        self.ctx = StepContext(self.ws, self.err, self.device, self.n_sms, self.profiler)
        self.sampler = DeviceSampler(self.cache.n_slots, self.device)
        self.use_graphs = bool(use_graphs) and not profile and model.graph_safe
        self._graphs = {}
        self._step_graphs = {}     # shape of a step (tokens per sequence, wanted rows) -> captured forward
        self._step_seen = {}
        self.steps_run = 0
        self.h2d_bytes_last = 0
        self.kernel_launches_last = 0

    @classmethod
    def from_dir(cls, model_dir, dtype="bfloat16", max_tokens=4096, device="cuda:0", **kw):
        return cls(load_model(model_dir, dtype, device), max_tokens, **kw)

    # ------------------------------------------------------------------ sequences
    def open(self, n=1):
        """Slots for `n` new sequences."""
        return [self.cache.open() for _ in range(n)]

    def close(self, slots):
        """The sequences are finished: what they hold is given back."""
        for s in slots:
            self.cache.close(s)
        self._raise_pending()

    def length(self, slot):
        return int(self.cache.length[slot])

    @property
    def capacity_tokens(self):
        """Room for live sequences in tokens as the cache counts them (`footprint`); None: the slots are the only bound."""
        return self.cache.capacity_tokens

    @property
    def max_seqs(self):
        return self.cache.n_slots

    def footprint(self, length):
        """Tokens of the cache's room that one sequence of `length` tokens takes."""
        return self.cache.footprint(length)

    @property
    def max_positions(self):
        return self.plan.max_positions

    def seed(self, slots, params, first_request_index=0):
        """Start the sampler streams of new sequences (request i of a call draws from seed + i)."""
        self.sampler.seed(slots, params, first_request_index)

    # ------------------------------------------------------------------ the step
    def _validate(self, entries):
        seen = set()
        vocab = self.plan.vocab_size
        for e in entries:
            if e.slot in seen:
                raise EngineError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            ids = np.asarray(e.tokens, dtype=np.int64)     # one pass in NumPy: a prompt of thousands of ids is checked in microseconds
            n = ids.size
            if n == 0:
                raise EngineError(f"slot {e.slot} brings no token")
            if ids.ndim != 1:
                raise EngineError(f"slot {e.slot}: tokens must be a flat list of ids")
            lo, hi = int(ids.min()), int(ids.max())
            if lo < 0 or hi >= vocab:
                raise EngineError(f"token id {lo if lo < 0 else hi} is outside the vocabulary of {vocab}")
            e.tokens = ids
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise EngineError(f"slot {e.slot} wants logits at place {w} of {n} tokens")

    def step(self, entries: List[StepEntry]):
        """Run the entries' tokens; return float32 logits [total wanted, vocab] on the device.  The step is not
        waited for; what its kernels report to the error word is read, without a wait of its own, by the next call
        to the engine (or at once by `check_device_errors`), which raises `ops.KernelError`."""
        self._raise_pending()
        entries = [StepEntry(e.slot, e.tokens, e.want) if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        self._validate(entries)
        for e in entries:  # room for every token before anything runs
            self.cache.reserve(e.slot, len(e.tokens))
        n_want = sum(len(e.want) for e in entries)
        logits = torch.empty((n_want, self.plan.vocab_size), dtype=torch.float32, device=self.device)
        # cut into micro-steps of at most max_step_tokens tokens and max_step_seqs sequences
        micro, cur, cur_tokens = [], [], 0
        for e in entries:
            start = 0
            n = len(e.tokens)
            while start < n:
                room = self.max_step_tokens - cur_tokens
                if room == 0 or len(cur) == self.max_step_seqs or (cur and cur[-1][0] is e):   # (a sequence takes part in a micro-step once)
                    micro.append(cur)
                    cur, cur_tokens = [], 0
                    room = self.max_step_tokens
                take = min(room, n - start, self.cache.piece_tokens or n)
                cur.append((e, start, take))
                cur_tokens += take
                start += take
        if cur:
            micro.append(cur)
        # global row of every wanted place, in the order of the entries and of their `want` lists
        base, row_of = 0, {}
        for e in entries:
            for j, w in enumerate(e.want):
                row_of.setdefault((id(e), int(w)), []).append(base + j)
            base += len(e.want)
        order = []
        row0 = 0
        for pieces in micro:
            row0 += self._run_pieces(pieces, logits, row0, row_of, order)
        if order != list(range(n_want)):  # a cut sequence with unsorted wants: put the rows where they belong
            dest = torch.tensor(order, dtype=torch.int64, device=self.device)
            logits = torch.empty_like(logits).index_copy_(0, dest, logits)
        self._err_host.copy_(self.err, non_blocking=True)
        self._err_copied.record()
        self._err_pending = True
        return logits

    def _run_pieces(self, pieces, logits, row0, row_of, order):
        token_ids, slots, ntok, pos0, want_rows = [], [], [], [], []
        t0 = 0
        if self.cache.piece_tokens:     # windowed groups reserve piece by piece (what earlier pieces no longer need went back)
            for e, start, take in pieces:
                self.cache.reserve(e.slot, take)
        for e, start, take in pieces:
            token_ids.append(e.tokens[start:start + take])
            slots.append(e.slot)
            ntok.append(take)
            pos0.append(int(self.cache.length[e.slot]))
            for w in e.want:
                if start <= int(w) < start + take:
                    want_rows.append(t0 + int(w) - start)
                    order.append(row_of[(id(e), int(w))].pop(0))
            t0 += take
        ctx = self.buffers.fill(self.ctx, np.concatenate(token_ids), slots, ntok, pos0, want_rows, self.cache)
        self.h2d_bytes_last = self.buffers.last_bytes
        out = logits[row0:row0 + len(want_rows)]
        if self.profiler is not None:
            self.profiler.begin_step("decode" if ctx.all_single else "prefill", ctx.n_tokens, ctx.n_seqs, min(pos0))
        if not self._replay_step(ctx, tuple(ntok), len(want_rows), out):
            self.model.forward(ctx, self.cache, out)
        if self.profiler is not None:
            self.profiler.end_step()
        for s, n in zip(slots, ntok):
            self.cache.advance(s, n)
        self.steps_run += 1
        return len(want_rows)

    # A step's launches depend on its shape only (tokens per sequence, number of wanted rows): ids,
    # positions, page tables, tiles and wanted rows are data in the fixed metadata buffer.  So a
    # shape that comes back is replayed from a CUDA graph, which removes the host's launch work
    # (a prompt step is otherwise bound by it).  Captured at a shape's second appearance; the
    # graph writes logits into a buffer of its own, copied out after the replay.
    STEP_GRAPH_MIN_TOKENS = 32
    STEP_GRAPH_MAX_LOGIT_BYTES = 64 << 20
    STEP_GRAPH_LIMIT = 12

    def _replay_step(self, ctx, shape, n_want, out):
        if not self.use_graphs or ctx.n_tokens < self.STEP_GRAPH_MIN_TOKENS or ctx.all_single:
            return False
        if n_want * self.plan.vocab_size * 4 > self.STEP_GRAPH_MAX_LOGIT_BYTES:
            return False
        if any(t not in ctx._tiles for t in self.buffers.tile_sizes):   # (the model's own list, taken when the buffers were made)
            return False
        key = (shape, n_want)
        g = self._step_graphs.get(key)
        if g is None:
            self._step_seen[key] = self._step_seen.get(key, 0) + 1
            if self._step_seen[key] < 2:
                return False
            if len(self._step_graphs) >= self.STEP_GRAPH_LIMIT:
                self._step_graphs.pop(next(iter(self._step_graphs)))
            buf = torch.empty((n_want, self.plan.vocab_size), dtype=torch.float32, device=self.device)
            states = self._save_states(ctx)
            self.model.forward(ctx, self.cache, buf)   # once eagerly: kernel attributes are set outside the capture
            torch.cuda.synchronize()
            self._restore_states(ctx, states)
            graph = torch.cuda.CUDAGraph()
            before = ops.LAUNCHES
            with torch.cuda.graph(graph):
                self.model.forward(ctx, self.cache, buf)
            launches = ops.LAUNCHES - before
            ops.count_launches(-launches)
            g = {"graph": graph, "logits": buf, "launches": launches}
            self._step_graphs[key] = g
        g["graph"].replay()
        ops.count_launches(g["launches"])
        if n_want:
            out.copy_(g["logits"])
        return True

    def _save_states(self, ctx):
        """Copies of the batch's rows of every fixed-size state group: a step that is run once eagerly and then
        replayed from its fresh capture must advance such a state once, not twice."""
        if not self.cache.state_groups:
            return None
        idx = ctx.seq_slots.to(torch.int64)
        return idx, [g.state.index_select(1, idx) for g in self.cache.state_groups]

    def _restore_states(self, ctx, saved):
        if saved is not None:
            idx, rows = saved
            for g, r in zip(self.cache.state_groups, rows):
                g.state.index_copy_(1, idx, r)

    def check_device_errors(self):
        """Raise if a kernel flagged bad input or a wait that ran out since the last check (synchronises)."""
        self._err_pending = False
        self._flagged(int(self.err.item()))

    def _flagged(self, word):
        """`word`: the error word as the host read it.  Non-zero: the word is put right again, the captured graphs
        stay valid, and the call raises; the logits and tokens of the steps since the last reading are not to be used."""
        if word:
            self.err.zero_()
            what = [m for b, m in ops.ERR_BITS.items() if word & b]
            raise ops.KernelError("a kernel reported: " + "; ".join(what or [f"error word {word:#x}"]))

    def _raise_pending(self):
        """Read the error word that the last `step` copied out, once that copy has landed."""
        if self._err_pending:
            self._err_pending = False
            self._err_copied.synchronize()
            self._flagged(int(self._err_host[0]))

    # ------------------------------------------------------------------ sampled steps (generation)
    def prefill_sampled(self, slots, prompts, params):
        """Prompts of sequences that start together, in one step; returns a sampled token per sequence."""
        entries = [StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)]
        logits = self.step(entries)
        tokens = torch.empty(len(slots), dtype=torch.int32, device=self.device)
        self.sampler.sample(logits, params, self.ctx.seq_slots if len(slots) == self.ctx.n_seqs else
                            torch.tensor(slots, dtype=torch.int32, device=self.device), tokens)
        out = tokens.tolist()
        self.check_device_errors()
        return out

    def decode_sampled(self, slots, last_tokens, params):
        """One token per sequence, sampled on the device; from a CUDA graph when enabled.
        Host token ids in, host token ids out."""
        B = len(slots)
        if not self.use_graphs or B > self.max_step_seqs:
            logits = self.step([StepEntry(s, [t], [0]) for s, t in zip(slots, last_tokens)])
            tokens = torch.empty(B, dtype=torch.int32, device=self.device)
            self.sampler.sample(logits, params, self.ctx.seq_slots, tokens)
            out = tokens.tolist()
            self.check_device_errors()
            return out
        self.decode_launch(slots, last_tokens, params)
        self._result_host[:1 + B].copy_(self._result[:1 + B], non_blocking=True)   # the error word and the tokens: one copy, one wait
        torch.cuda.current_stream().synchronize()
        out = self._result_np[:1 + B].tolist()
        self._flagged(out[0])
        return out[1:]

    def decode_launch(self, slots, last_tokens, params):
        """Issue one decode step (metadata copy + graph replay) without waiting for it; the
        sampled tokens land in the returned record's device tensor `tokens`."""
        self._raise_pending()
        B = len(slots)
        vocab = self.plan.vocab_size
        if min(last_tokens) < 0 or max(last_tokens) >= vocab:
            raise EngineError(f"token id {min(last_tokens) if min(last_tokens) < 0 else max(last_tokens)} is outside the vocabulary of {vocab}")
        self.cache.reserve_next(slots)
        pos0 = self.cache.length[list(slots)].tolist()
        ctx = self.ctx
        if not self.buffers.refill_next_token(ctx, list(last_tokens), list(slots), pos0):
            ctx = self.buffers.fill(self.ctx, list(last_tokens), list(slots), [1] * B, pos0, list(range(B)), self.cache)
        self.h2d_bytes_last = self.buffers.last_bytes
        key = (B, params.key())
        g = self._graphs.get(key)
        if g is None:
            g = self._capture_decode(ctx, B, params)
            self._graphs[key] = g
        g["graph"].replay()
        ops.count_launches(g["launches"])
        self.cache.advance_next(slots)
        self.steps_run += 1
        return g

    def _capture_decode(self, ctx, B, params):
        """Capture forward + sampling for a batch of B single tokens.  The views of `ctx` have
        the same addresses for every step of B sequences, so the graph reads each step's fresh
        metadata; the number of attention splits is frozen with the graph."""
        logits = torch.empty((B, self.plan.vocab_size), dtype=torch.float32, device=self.device)
        tokens = self._result[1:1 + B]
        ops.lib()  # library loaded and kernels' attributes set before capture
        # one eager run first: it sets kernel attributes (shared-memory sizes) outside of the capture.  It writes
        # the same cache rows as the replay that follows; what it advances (the sampler's streams, the fixed-size
        # states of mixers that keep one) is put back.
        saved = self.sampler.state.clone()
        states = self._save_states(ctx)
        self.model.forward(ctx, self.cache, logits)
        self.sampler.sample(logits, params, ctx.seq_slots, tokens)
        torch.cuda.synchronize()
        self.sampler.state.copy_(saved)
        self._restore_states(ctx, states)
        graph = torch.cuda.CUDAGraph()
        before = ops.LAUNCHES
        with torch.cuda.graph(graph):
            self.model.forward(ctx, self.cache, logits)
            self.sampler.sample(logits, params, ctx.seq_slots, tokens)
        launches = ops.LAUNCHES - before
        ops.count_launches(-launches)  # captured, not run
        return {"graph": graph, "logits": logits, "tokens": tokens, "launches": launches}
