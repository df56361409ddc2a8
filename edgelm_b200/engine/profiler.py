"""Per-part profiler that writes Chrome traces.

Same event shape as adarsh-sgh/edgelm's (include/edgelm/profiler.hpp:13-34,
src/profiler.cpp:22-40): one complete event ("ph": "X", microseconds) per executed part with
its name, phase, token count and first position, plus one span per step; `stats()` groups by
phase and part name, sorted by time (src/profiler.cpp:42-78).  Durations are device times from
CUDA event pairs around each part; they are resolved when the trace is written, so profiling
adds no synchronisation to the step itself.  Profiled steps run eagerly, never from a CUDA graph.
"""
import contextlib
import json

import torch


class _Null:
    enabled = False

    @contextlib.contextmanager
    def __call__(self, name):
        yield

    def begin_step(self, *a, **k):
        pass

    def end_step(self):
        pass


NULL_PROFILER = _Null()


class Profiler:
    enabled = True

    def __init__(self):
        self.pending = []   # (name, phase, T, B, pos0, start event, end event)
        self.events = []    # resolved: dicts with ts_us, dur_us
        self._phase, self._T, self._B, self._pos0 = "step", 0, 0, 0
        self._origin = None
        self._step = None

    def begin_step(self, phase, n_tokens, n_seqs, pos0):
        self._phase, self._T, self._B, self._pos0 = phase, n_tokens, n_seqs, pos0
        s = torch.cuda.Event(enable_timing=True)
        s.record()
        if self._origin is None:
            self._origin = s
        self._step = s

    def end_step(self):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self.pending.append((self._phase, "phase", self._T, self._B, self._pos0, self._step, e))

    @contextlib.contextmanager
    def __call__(self, name):
        s = torch.cuda.Event(enable_timing=True)
        e = torch.cuda.Event(enable_timing=True)
        s.record()
        try:
            yield
        finally:
            e.record()
            self.pending.append((name, self._phase, self._T, self._B, self._pos0, s, e))

    def resolve(self):
        if self.pending:
            torch.cuda.synchronize()
        for name, phase, T, B, pos0, s, e in self.pending:
            self.events.append({"name": name, "phase": phase, "T": T, "B": B, "pos0": pos0,
                                "ts_us": self._origin.elapsed_time(s) * 1e3, "dur_us": s.elapsed_time(e) * 1e3})
        self.pending = []
        return self.events

    def write_trace(self, path):
        """Chrome trace JSON (open in ui.perfetto.dev or chrome://tracing)."""
        ev = [{"name": "thread_name", "ph": "M", "pid": 1, "tid": 1, "args": {"name": "edgelm_b200 cuda:0"}}]
        for e in self.resolve():
            tid = 2 if e["phase"] == "phase" else 1
            ev.append({"name": e["name"], "cat": e["phase"], "ph": "X", "pid": 1, "tid": tid, "ts": round(e["ts_us"], 3),
                       "dur": round(e["dur_us"], 3), "args": {"T": e["T"], "B": e["B"], "pos0": e["pos0"]}})
        with open(path, "w") as f:
            json.dump({"traceEvents": ev, "displayTimeUnit": "ms"}, f)
        return len(ev) - 1

    def stats(self):
        """Text table: per phase, time by part name."""
        rows = {}
        for e in self.resolve():
            if e["phase"] == "phase":
                continue
            k = (e["phase"], e["name"])
            c = rows.setdefault(k, [0, 0.0])
            c[0] += 1
            c[1] += e["dur_us"]
        out = []
        for phase in sorted({k[0] for k in rows}):
            total = sum(v[1] for k, v in rows.items() if k[0] == phase)
            out.append(f"{phase}: {total / 1e3:.3f} ms in parts")
            for (ph, name), (n, us) in sorted(rows.items(), key=lambda kv: -kv[1][1]):
                if ph == phase:
                    out.append(f"  {name:<22} {n:6d} calls {us / 1e3:10.3f} ms {100 * us / max(total, 1e-9):5.1f} %")
        return "\n".join(out) + "\n"
