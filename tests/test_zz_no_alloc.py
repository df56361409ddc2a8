"""The entry point that allocates nothing (edgelm_b200/csrc/no_alloc.h), called through its
exported C symbol and compared with the regular decode-attention entry point.

Who calls it: code that cannot allocate device memory where it runs: a plugin inside another
runtime's pre-sized region, a loop that forbids allocator calls, a process with a frozen memory
pool.  The regular entry point wants two scratch buffers from its caller; this one keeps the
scratch in a device array inside the library.  This file is collected last, so that a run which
stops at the first failure has already run every other test; it passes alone in a fresh process
and after the other tests.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

SCRATCH_FLOATS = 1 << 20  # EDGELM_NOALLOC_SCRATCH_FLOATS


def _case(o, dtype, lengths, nh, nkv, hd, seed):
    """Sequences in a paged cache with pages in scrambled order; rows past a sequence's end hold NaN."""
    P = o.PAGE
    g = torch.Generator().manual_seed(seed)
    need = [(n + P - 1) // P for n in lengths]
    n_pages = sum(need) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((len(lengths), max(need)), -1, dtype=torch.int32)
    kc = torch.full((n_pages, nkv, P, hd), float("nan"))
    vc = torch.full((n_pages, nkv, P, hd), float("nan"))
    it = iter(perm)
    keys, values = [], []   # per sequence [n, nkv, hd], as the cache's dtype holds them
    for s, n in enumerate(lengths):
        ks, vs = [], []
        for pg in range(need[s]):
            page = next(it)
            table[s, pg] = page
            rows = min(n, (pg + 1) * P) - pg * P
            kc[page, :, :rows] = torch.randn(nkv, rows, hd, generator=g)
            vc[page, :, :rows] = torch.randn(nkv, rows, hd, generator=g)
            ks.append(kc[page, :, :rows].transpose(0, 1))
            vs.append(vc[page, :, :rows].transpose(0, 1))
        keys.append(torch.cat(ks).to(dtype).double())
        values.append(torch.cat(vs).to(dtype).double())
    d = torch.device("cuda:0")
    qkv = torch.randn(len(lengths), (nh + 2 * nkv) * hd, generator=g).to(dtype).to(d)
    return dict(qkv=qkv, k=kc.to(dtype).to(d), v=vc.to(dtype).to(d), table=table.to(d), keys=keys, values=values,
                seq=torch.arange(len(lengths), dtype=torch.int32, device=d),
                pos=torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=d))


def _plain(c, nh, nkv, hd):
    """softmax(q . K / sqrt(hd)) V of every sequence's one query row over all its keys, in float64: written here from
    the formula, sharing nothing with the library."""
    out = torch.zeros(len(c["keys"]), nh * hd, dtype=torch.float64)
    q = c["qkv"][:, :nh * hd].double().cpu().reshape(-1, nh, hd)
    for s, (k, v) in enumerate(zip(c["keys"], c["values"])):
        for h in range(nh):
            p = torch.softmax((k[:, h // (nh // nkv)] @ q[s, h]) / math.sqrt(hd), dim=0)
            out[s, h * hd:(h + 1) * hd] = p @ v[:, h // (nh // nkv)]
    return out


def _noalloc(o, c, out, nh, nkv, hd, splits):
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    fn = o.lib().edgelm_attn_decode_noalloc
    return fn(p(c["qkv"]), c["qkv"].stride(0), p(out), out.stride(0), p(c["k"]), p(c["v"]), o.BF16 if out.dtype == torch.bfloat16 else o.F32,
              p(c["table"]), c["table"].stride(0), p(c["seq"]), p(c["pos"]), c["qkv"].shape[0], nh, nkv, hd,
              ctypes.c_float(1.0 / math.sqrt(hd)), splits, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_no_alloc_matches_regular_entry_point_twice(dtype):
    from edgelm_b200.csrc import ops as o
    o.require_device()
    tol = 1e-5 if dtype == torch.float32 else 1e-2  # the kernel tests' tolerances; the two paths run the same kernels
    # two calls in a row with different shapes: the second finds the first one's leftovers in the scratch
    for call, (lengths, nh, nkv, hd, splits) in enumerate([([700, 65, 1, 300], 9, 3, 64, 5), ([64, 129, 1000], 4, 2, 32, 7)]):
        c = _case(o, dtype, lengths, nh, nkv, hd, seed=11 + call)
        B = len(lengths)
        want = torch.zeros(B, nh * hd, dtype=dtype, device="cuda:0")
        po = torch.zeros(B * nh * splits * hd, device="cuda:0")
        pm = torch.zeros(B * nh * splits * 2, device="cuda:0")
        o.attn_decode(c["qkv"], want, c["k"], c["v"], c["table"], c["seq"], c["pos"], B, nh, nkv, hd, 1.0 / math.sqrt(hd), splits, po, pm)
        got = torch.full_like(want, float("nan"))
        if call == 0:   # set-up: the first call on a device may load the library's module and looks up the array's address
            assert _noalloc(o, c, got, nh, nkv, hd, splits) == 0, o.lib().edgelm_last_error().decode()
            got.fill_(float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]   # the device's own count: an allocation by anyone in the process would show
        rc = _noalloc(o, c, got, nh, nkv, hd, splits)
        assert rc == 0, o.lib().edgelm_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"
        assert torch.isfinite(got.float()).all()
        err = float((got.double() - want.double()).abs().max() / max(1.0, float(want.double().abs().max())))
        assert err < tol, (call, err)
        plain = _plain(c, nh, nkv, hd)     # and against the formula itself, not only against the other entry point
        err = float((got.double().cpu() - plain).abs().max() / max(1.0, float(plain.abs().max())))
        assert err < tol, (call, err)


def test_no_alloc_refuses_what_does_not_fit():
    from edgelm_b200.csrc import ops as o
    o.require_device()
    c = _case(o, torch.float32, [10, 20], 8, 8, 64, seed=3)
    out = torch.zeros(2, 8 * 64, device="cuda:0")
    splits = SCRATCH_FLOATS // (2 * 8 * 66) + 1  # one split too many for the built-in array
    assert _noalloc(o, c, out, 8, 8, 64, splits) != 0
    msg = o.lib().edgelm_last_error().decode()
    assert "scratch" in msg and str(SCRATCH_FLOATS) in msg
    assert _noalloc(o, c, out, 8, 8, 24, 2) != 0 and "head size" in o.lib().edgelm_last_error().decode()
    assert _noalloc(o, c, out, 8, 8, 64, splits - 1) == 0  # the largest that fits runs
    torch.cuda.synchronize()
