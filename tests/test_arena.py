"""The step's workspace (a stack arena): nesting, reuse, the overflow error, equal steps at equal
addresses; and the declared sizes of the model's parts against what a step really takes.
adarsh-sgh/edgelm checks its arena plan the same way: no two live buffers overlap, and an
overlapping plan is refused (src/passes.cpp:210-223, tests/test_graph.cpp:82-130)."""
import random

import pytest
import torch

from edgelm_b200.engine.arena import ALIGN, Workspace, WorkspaceError


def _span(t):
    return t.data_ptr(), t.data_ptr() + t.numel() * t.element_size()


def test_frames_nest_and_give_back():
    ws = Workspace(64 * 1024, "cpu")
    a = ws.alloc((100,), torch.float32)
    top_a = ws.top
    with ws.frame():
        b = ws.alloc((3, 50), torch.bfloat16)
        with ws.frame():
            c = ws.alloc((7,), torch.float32)
            assert _span(b)[1] <= _span(c)[0]
        d = ws.alloc((7,), torch.float32)          # the inner frame is gone: its room is used again
        assert d.data_ptr() == c.data_ptr()
        assert _span(a)[1] <= _span(b)[0]
    assert ws.top == top_a
    e = ws.alloc((3, 50), torch.bfloat16)
    assert e.data_ptr() == b.data_ptr()
    assert all(t.data_ptr() % ALIGN == ws.buffer.data_ptr() % ALIGN for t in (a, b, c, e))
    assert ws.peak >= ws.top and ws.peak <= ws.capacity
    ws.reset()
    assert ws.top == 0 and ws.alloc((100,), torch.float32).data_ptr() == a.data_ptr()


def test_a_frame_is_left_even_when_its_body_raises():
    ws = Workspace(4096, "cpu")
    ws.alloc((10,), torch.float32)
    mark = ws.top
    with pytest.raises(RuntimeError, match="inside"):
        with ws.frame():
            ws.alloc((10,), torch.float32)
            raise RuntimeError("inside")
    assert ws.top == mark


def test_overflow_names_the_buffer():
    ws = Workspace(1024, "cpu")
    ws.alloc((128,), torch.float32)
    with pytest.raises(WorkspaceError, match=r"shape \(200, 2\).*does not fit"):
        ws.alloc((200, 2), torch.float32)
    assert ws.top == 512          # the failed request took nothing
    ws.alloc((128,), torch.float32)


def test_live_buffers_never_overlap_and_equal_steps_get_equal_addresses():
    """Random nested programs of allocations: whatever is live at one time is disjoint; running the
    same program twice gives the same addresses (what a replayed CUDA graph relies on)."""
    rng = random.Random(7)
    for trial in range(50):
        ws = Workspace(1 << 20, "cpu")
        program = []

        def make(depth):
            for _ in range(rng.randint(1, 4)):
                if depth < 3 and rng.random() < 0.4:
                    program.append("push")
                    make(depth + 1)
                    program.append("pop")
                else:
                    program.append((rng.randint(1, 3000), rng.choice([torch.float32, torch.bfloat16, torch.uint8])))
        make(0)

        def run():
            ws.reset()
            live, stack, addresses = [], [], []
            frames = []
            for op in program:
                if op == "push":
                    f = ws.frame()
                    f.__enter__()
                    frames.append(f)
                    stack.append(len(live))
                elif op == "pop":
                    frames.pop().__exit__(None, None, None)
                    del live[stack.pop():]
                else:
                    t = ws.alloc((op[0],), op[1])
                    lo, hi = _span(t)
                    for a, b in live:
                        assert hi <= a or b <= lo, "two live buffers overlap"
                    live.append((lo, hi))
                    addresses.append(lo)
            return addresses
        assert run() == run(), trial
