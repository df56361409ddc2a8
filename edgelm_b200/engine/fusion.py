"""Fusion of runs of layers for decode steps.

The parts of a layer each launch their own kernels, which is what a prompt wants.  With one new
token per sequence and few sequences a layer is five short kernels, and a step is bound by their
launches.  This pass looks at the schedule once the weights are there and finds runs of
consecutive entries whose blocks can describe themselves to the persistent decode kernel
(`Part.decode_fusion()`); each run becomes a `DecodeStack` that runs all its layers in one
launch.  Entries that cannot (another mixer, a layer that reads another's cache, sizes the kernel
does not take) keep running part by part, and so does every step that is not a small decode step.
The same idea as the graph passes of adarsh-sgh/edgelm that merge ops with a shared input, SwiGLU,
the residual add and rotation + attention (tools/elm.py:60-118), one level up.
"""
import struct

import torch

from ..csrc import ops

RECORD = struct.Struct("<12Q6i3fi")  # StackLayer of decode_stack.cu
KIND = "prenorm_attention_swiglu"


class DecodeStack:
    """A run of schedule entries as one kernel launch per decode step."""

    def __init__(self, schedule_indices, fusions, hidden, device):
        self.indices = list(schedule_indices)
        self.fusions = list(fusions)
        self.hidden, self.device = hidden, device
        f0 = self.fusions[0]
        self.hd = f0["head_dim"]
        self.max_qkv = max((f["num_heads"] + 2 * f["num_kv_heads"]) * self.hd for f in self.fusions)
        self.max_att = max(f["num_heads"] * self.hd for f in self.fusions)
        self.max_inter = max(f["inter"] for f in self.fusions)
        self.max_heads = max(f["num_heads"] for f in self.fusions)
        self.max_kv_heads = max(f["num_kv_heads"] for f in self.fusions)
        self.max_k = max(hidden, self.max_att, self.max_inter)
        # pages of an attention unit: fewer with more than 8 sequences (their activations take more shared memory)
        self.chunk_pages = min(ops.decode_stack_chunk_pages(self.hd, self.max_k, n) for n in (8, ops.DECODE_STACK_MAX_SEQS))
        rows = ops.DECODE_STACK_MAX_SEQS
        self.qkv = torch.empty((rows, self.max_qkv), dtype=torch.bfloat16, device=device)
        self.mid = torch.empty((rows, self.max_inter), dtype=torch.bfloat16, device=device)
        self.sync = torch.zeros(2, dtype=torch.int32, device=device)
        self.max_chunks = 0
        self.part_o = self.part_ml = None
        self.layer_bytes = sum(f[k].numel() * f[k].element_size() for f in self.fusions
                               for k in ("w_qkv", "w_o", "w_gate", "w_up", "w_down")) // len(self.fusions)
        self.force = False   # True: run fused whatever the sizes (tests, measurements)
        self.trace = None    # int64 [layers, 10] when phase stamps are wanted (see ops.decode_stack)
        self._records = {}   # addresses of tables and cache -> packed records on the device (kept: graphs read them)

    # Measured on a B200 (decode steps of SmolLM2-shaped models, contexts of 128 to 2300 tokens, device time per
    # step, fused against the parts' own kernels, whose few-rows products start under the tail of the kernel before
    # them): 7 MB of weights a layer: 0.774 against 0.816 ms at 1 sequence, 0.826 against 0.887 at 2, 0.843 against
    # 0.866 at 3, 0.875 against 0.853 at 4, 0.951 against 0.870 at 8; 20 MB a layer: 1.016 against 1.028 at 1 sequence,
    # 1.086 against 1.017 at 2; 100 MB a layer: slower at every batch.  A phase of the fused kernel costs about the
    # same whatever it computes (round trips through L2 and a grid barrier); the separate kernels have more blocks
    # and more bytes in flight, which wins as soon as a phase has real work.
    MAX_LAYER_BYTES = 24 << 20
    MAX_LAYER_BYTES_TIMES_SEQS = 24 << 20

    def takes(self, ctx):
        if not (ctx.all_single and 1 <= ctx.n_seqs <= ops.DECODE_STACK_MAX_SEQS):
            return False
        return self.force or (self.layer_bytes <= self.MAX_LAYER_BYTES and
                              self.layer_bytes * ctx.n_seqs <= self.MAX_LAYER_BYTES_TIMES_SEQS)

    def _room_for(self, stride):
        chunks = -(-stride // self.chunk_pages)
        if chunks > self.max_chunks:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("the fused decode kernel's partial results must be sized before a capture")
            rows = ops.DECODE_STACK_MAX_SEQS
            self.part_o = torch.empty(rows * self.max_heads * chunks * self.hd, dtype=torch.float32, device=self.device)
            self.part_ml = torch.empty(rows * self.max_heads * chunks * 2, dtype=torch.float32, device=self.device)
            self.max_chunks = chunks
            self._records.clear()

    def _records_for(self, ctx, cache):
        entries = [cache.entries[i] for i in self.indices]
        tables = [ctx.page_table(e.group) for e in entries]
        key = tuple((t.data_ptr(), e.k.data_ptr()) for t, e in zip(tables, entries))
        rec = self._records.get(key)
        if rec is None:
            blob = bytearray()
            for f, e, t in zip(self.fusions, entries, tables):
                k, v = e.k, e.v
                blob += RECORD.pack(f["w_qkv"].data_ptr(), f["w_o"].data_ptr(), f["w_gate"].data_ptr(), f["w_up"].data_ptr(),
                                    f["w_down"].data_ptr(), f["norm1"].data_ptr(), f["norm2"].data_ptr(), f["cos"].data_ptr(),
                                    f["sin"].data_ptr(), k.data_ptr(), v.data_ptr(), t.data_ptr(), f["num_heads"],
                                    f["num_kv_heads"], f["inter"], t.stride(0), f["cos"].shape[0], k.shape[0], f["eps1"],
                                    f["eps2"], f["scale"], 0)
            rec = torch.frombuffer(blob, dtype=torch.uint8).to(self.device)
            self._records[key] = rec
        return rec

    def run(self, ctx, cache, x):
        entries = [cache.entries[i] for i in self.indices]
        self._room_for(max(ctx.page_table(e.group).stride(0) for e in entries))
        rec = self._records_for(ctx, cache)
        with ctx.prof("decode_stack"):
            ops.decode_stack(rec, len(self.indices), x, self.hd, self.max_k, ctx.seq_index, ctx.seq_pos, self.qkv,
                             self.mid, self.part_o, self.part_ml, self.max_chunks, self.sync, ctx.err, self.trace)

    def reset(self):
        """After a device-side wait ran out the kernel leaves its barrier words as they were."""
        self.sync.zero_()


def _fusable(block, entry, dtype, hidden):
    if dtype != torch.bfloat16 or entry.reads_cache_of is not None or not hasattr(block, "decode_fusion"):
        return None
    f = block.decode_fusion()
    if f is None or f.get("kind") != KIND:
        return None
    hd, nh, nkv = f["head_dim"], f["num_heads"], f["num_kv_heads"]
    widest = max(hidden, nh * hd, f["inter"])
    ok = (ops.decode_stack_chunk_pages(hd, widest, ops.DECODE_STACK_MAX_SEQS) > 0 and nh % nkv == 0 and nh // nkv <= 16 and hidden % 8 == 0
          and f["inter"] % 8 == 0 and f["cos"].shape[1] == hd // 2)
    return f if ok else None


def plan_decode_runs(model):
    """[(DecodeStack | None, [schedule indices])]: the schedule cut into fused runs and single entries."""
    runs, cur, cur_f = [], [], []
    hidden = model.plan.hidden_size

    def close():
        nonlocal cur, cur_f
        if cur:
            runs.append((DecodeStack(cur, cur_f, hidden, model.device), cur))
        cur, cur_f = [], []

    for i, e in enumerate(model.schedule):
        f = _fusable(model.layers[e.layer], e, model.dtype, hidden)
        if f is not None and cur_f and f["head_dim"] != cur_f[0]["head_dim"]:
            close()
        if f is None:
            close()
            runs.append((None, [i]))
        else:
            cur.append(i)
            cur_f.append(f)
    close()
    return runs
