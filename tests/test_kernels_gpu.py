"""Each CUDA kernel alone against a plain float64/float32 restatement of its formula, at sizes
that the tiny models do not use (odd widths, head sizes 16..256, ragged tails)."""
import math

import numpy as np
import pytest
import torch

import plain_llama as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def ops():
    from edgelm_b200.csrc import ops as o
    o.require_device()
    return o


def dev():
    return torch.device("cuda:0")


def tol(dtype):
    return 2e-5 if dtype == torch.float32 else 1.6e-2


def rel_err(a, b):
    a = a.double().cpu()
    b = b.double().cpu()
    return float((a - b).abs().max() / max(1.0, float(b.abs().max())))


def rnd(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(dev())


# ----------------------------------------------------------------------------- embedding
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab,dim", [(397, 96), (1000, 576), (50, 20)])
def test_embed_gather(dtype, vocab, dim):
    o = ops()
    table = rnd((vocab, dim), dtype, 1)
    ids = torch.tensor([0, vocab - 1, 3, 3, vocab // 2], dtype=torch.int32, device=dev())
    x = torch.empty(ids.numel(), dim, dtype=torch.float32, device=dev())
    err = torch.zeros(1, dtype=torch.int32, device=dev())
    o.embed_gather(ids, table, x, err)
    assert torch.equal(x, table[ids.long()].float())
    assert int(err.item()) == 0
    bad = torch.tensor([1, vocab, -1], dtype=torch.int32, device=dev())
    o.embed_gather(bad, table, x[:3], err)
    assert int(err.item()) & 1
    with pytest.raises(o.KernelError):
        o.read_error_word(err)
    assert int(err.item()) == 0


# ----------------------------------------------------------------------------- RMSNorm
@pytest.mark.parametrize("out_dtype", DTYPES)
@pytest.mark.parametrize("rows,dim,eps", [(5, 96, 1e-6), (33, 576, 1e-5), (1, 2048, 1e-5), (7, 250, 1e-3)])
def test_rmsnorm(out_dtype, rows, dim, eps):
    o = ops()
    x = rnd((rows, dim), torch.float32, 2, 3.0)
    w = 1 + rnd((dim,), torch.float32, 3, 0.1)
    out = torch.empty(rows, dim, dtype=out_dtype, device=dev())
    o.rmsnorm(x, w, eps, out)
    want = torch.from_numpy(plain.rmsnorm(x.cpu().numpy(), w.cpu().numpy(), eps))
    assert rel_err(out, want) < (2e-6 if out_dtype == torch.float32 else 8e-3)
    idx = torch.tensor([rows - 1, 0, rows // 2], dtype=torch.int32, device=dev())
    out2 = torch.empty(3, dim, dtype=out_dtype, device=dev())
    o.rmsnorm(x, w, eps, out2, rows_idx=idx)
    assert torch.equal(out2, out[idx.long()])


# ----------------------------------------------------------------------------- GEMM (CUDA cores)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 48, 64), (3, 37, 96), (17, 130, 160), (5, 397, 200), (70, 200, 96),
                                     (129, 65, 33), (16, 256, 576), (9, 31, 7)])
@pytest.mark.parametrize("force", [1, 2])
def test_gemm_simt_store_and_residual(dtype, M, N, K, force):
    o = ops()
    a = rnd((M, K), dtype, 4)
    w = rnd((N, K), dtype, 5, 0.2)
    want = a.double().cpu() @ w.double().cpu().T
    out = torch.empty(M, N, dtype=dtype, device=dev())
    o.gemm_simt(a, w, out, force_kernel=force)
    assert rel_err(out, want) < tol(dtype)
    if dtype == torch.bfloat16:  # logits: bfloat16 operands, float32 result
        out32 = torch.empty(M, N, dtype=torch.float32, device=dev())
        o.gemm_simt(a, w, out32, force_kernel=force)
        assert rel_err(out32, want) < 2e-5
    res = rnd((M, N), torch.float32, 6)
    res0 = res.clone()
    o.gemm_simt(a, w, res, epilogue=o.EPI_RESIDUAL, residual=res, force_kernel=force)  # in place on the residual stream
    assert rel_err(res, res0.double().cpu() + want) < 2e-5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(2, 200, 96), (40, 130, 64), (1, 1536, 576), (67, 77, 50)])
def test_gemm_simt_swiglu(dtype, M, N, K):
    o = ops()
    a = rnd((M, K), dtype, 7)
    wg = rnd((N, K), dtype, 8, 0.3)
    wu = rnd((N, K), dtype, 9, 0.3)
    g = a.double().cpu() @ wg.double().cpu().T
    u = a.double().cpu() @ wu.double().cpu().T
    want = g / (1 + torch.exp(-g)) * u
    for force in (1, 2):
        out = torch.empty(M, N, dtype=dtype, device=dev())
        o.gemm_simt(a, wg, out, epilogue=o.EPI_SWIGLU, w2=wu, force_kernel=force)
        assert rel_err(out, want) < tol(dtype)


def test_gemm_row_independent_of_batch():
    """A row's result is the same bits whether it is computed alone or among others."""
    o = ops()
    a = rnd((40, 96), torch.float32, 10)
    w = rnd((50, 96), torch.float32, 11)
    full = torch.empty(40, 50, device=dev())
    o.gemm_simt(a, w, full, force_kernel=2)
    part = torch.empty(3, 50, device=dev())
    o.gemm_simt(a[5:8], w, part, force_kernel=2)
    assert torch.equal(part, full[5:8])
    o.gemm_simt(a[5:8], w, part, force_kernel=1)
    full1 = torch.empty(40, 50, device=dev())
    o.gemm_simt(a, w, full1, force_kernel=1)
    assert torch.equal(part, full1[5:8])


# ----------------------------------------------------------------------------- paged cache helpers
class PagedCase:
    """Sequences with keys/values in a paged cache whose pages are dealt in a scrambled order."""

    def __init__(self, o, dtype, lengths, nkv, hd, seed, extra_pages=3):
        self.o, self.dtype, self.lengths, self.nkv, self.hd = o, dtype, lengths, nkv, hd
        P = o.PAGE
        need = [(n + P - 1) // P for n in lengths]
        n_pages = sum(need) + extra_pages
        g = torch.Generator().manual_seed(seed)
        perm = torch.randperm(n_pages, generator=g).tolist()
        self.max_pages = max(need) + 1
        self.n_slots = len(lengths) + 2
        slots = torch.randperm(self.n_slots, generator=g).tolist()[:len(lengths)]
        table = torch.full((self.n_slots, self.max_pages), -1, dtype=torch.int32)
        self.k = [torch.randn(n, nkv, hd, generator=g) for n in lengths]
        self.v = [torch.randn(n, nkv, hd, generator=g) for n in lengths]
        # unused rows hold huge values: reading them would show
        kc = torch.full((n_pages, nkv, P, hd), 1e4)
        vc = torch.full((n_pages, nkv, P, hd), float("nan"))
        it = iter(perm)
        for s, n in enumerate(lengths):
            for pg in range(need[s]):
                page = next(it)
                table[slots[s], pg] = page
                lo, hi = pg * P, min(n, (pg + 1) * P)
                kc[page, :, :hi - lo] = self.k[s][lo:hi].transpose(0, 1)
                vc[page, :, :hi - lo] = self.v[s][lo:hi].transpose(0, 1)
        self.k = [t.to(dtype).float() for t in self.k]
        self.v = [t.to(dtype).float() for t in self.v]
        self.kcache = kc.to(dtype).to(dev())
        self.vcache = vc.to(dtype).to(dev())
        self.table = table.to(dev())
        self.seq_slot = torch.tensor(slots, dtype=torch.int32, device=dev())


def attention_rows(q, k, v, pos0, nh, nkv, hd, window=None):
    """Plain causal attention of new rows at positions pos0.. over keys 0..pos0+t (float64); with `window` over the
    last `window` of them only."""
    T = q.shape[0]
    q = q.double().reshape(T, nh, hd)
    k = k.double()
    v = v.double()
    g = nh // nkv
    out = torch.zeros(T, nh, hd, dtype=torch.float64)
    for t in range(T):
        n = pos0 + t + 1
        lo = max(0, n - window) if window else 0
        for h in range(nh):
            s = (k[lo:n, h // g] @ q[t, h]) / math.sqrt(hd)
            p = torch.softmax(s, dim=0)
            out[t, h] = p @ v[lo:n, h // g]
    return out.reshape(T, nh * hd)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 16), (3, 1, 32), (9, 3, 64), (2, 2, 48), (8, 1, 128), (40, 1, 16), (2, 1, 256), (5, 5, 80)])
def test_attn_prefill(dtype, nh, nkv, hd):
    o = ops()
    # (cached length before the step, new tokens): whole prompts, continued prompts, single tokens
    seqs = [(0, 5), (0, 70), (64, 1), (100, 29), (63, 2), (0, 1)]
    lengths = [a + b for a, b in seqs]
    case = PagedCase(o, dtype, lengths, nkv, hd, seed=nh * 100 + hd)
    g = nh // nkv
    T = sum(b for _, b in seqs)
    width = (nh + 2 * nkv) * hd
    qkv = rnd((T, width), dtype, 20)
    tq = max(1, 32 // g)
    tile_seq, tile_tok0, tile_ntok, tile_pos0 = [], [], [], []
    t0 = 0
    for s, (p0, n) in enumerate(seqs):
        for a in range(0, n, tq):
            tile_seq.append(s)
            tile_tok0.append(t0 + a)
            tile_ntok.append(min(tq, n - a))
            tile_pos0.append(p0 + a)
        t0 += n
    mk = lambda x: torch.tensor(x, dtype=torch.int32, device=dev())
    out = torch.zeros(T, nh * hd, dtype=dtype, device=dev())
    o.attn_prefill(qkv, out, case.kcache, case.vcache, case.table, case.seq_slot, mk(tile_seq), mk(tile_tok0),
                   mk(tile_ntok), mk(tile_pos0), len(tile_seq), tq, nh, nkv, hd, 1.0 / math.sqrt(hd))
    t0 = 0
    for s, (p0, n) in enumerate(seqs):
        want = attention_rows(qkv[t0:t0 + n, :nh * hd].float().cpu(), case.k[s], case.v[s], p0, nh, nkv, hd)
        assert rel_err(out[t0:t0 + n], want) < (1e-5 if dtype == torch.float32 else 1e-2), (s, p0, n)
        t0 += n


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 16), (3, 1, 32), (9, 3, 64), (32, 32, 64), (6, 1, 96), (2, 1, 256)])
@pytest.mark.parametrize("n_splits", [1, 3, 16])
def test_attn_decode(dtype, nh, nkv, hd, n_splits):
    o = ops()
    lengths = [1, 64, 65, 700, 128, 37]
    case = PagedCase(o, dtype, lengths, nkv, hd, seed=nh + hd + n_splits)
    B = len(lengths)
    qkv = rnd((B, (nh + 2 * nkv) * hd), dtype, 21)
    seq_pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=dev())
    out = torch.zeros(B, nh * hd, dtype=dtype, device=dev())
    part_o = torch.full((B * nh * n_splits * hd,), float("nan"), device=dev())
    part_ml = torch.full((B * nh * n_splits * 2,), float("nan"), device=dev())
    o.attn_decode(qkv, out, case.kcache, case.vcache, case.table, case.seq_slot, seq_pos, B, nh, nkv, hd,
                  1.0 / math.sqrt(hd), n_splits, part_o, part_ml)
    for s, n in enumerate(lengths):
        want = attention_rows(qkv[s:s + 1, :nh * hd].float().cpu(), case.k[s], case.v[s], n - 1, nh, nkv, hd)
        assert rel_err(out[s:s + 1], want) < (1e-5 if dtype == torch.float32 else 1e-2), (s, n)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 16, 40), (9, 3, 64, 100), (2, 1, 128, 64), (3, 3, 48, 1), (6, 2, 32, 200)])
def test_attention_with_a_window(dtype, nh, nkv, hd, window):
    """The last `window` keys only, in prompt steps (whole, continued, single tokens) and in decode steps (1, 3 and 16
    splits).  The pages before a sequence's window hold poison (1e4 keys, NaN values) as pages that were given back
    may: a kernel that looked there would show."""
    o = ops()
    seqs = [(0, 5), (0, 150), (64, 1), (100, 129), (63, 2), (300, 70)]
    lengths = [a + b for a, b in seqs]
    case = PagedCase(o, dtype, lengths, nkv, hd, seed=nh * 10 + hd)
    P = o.PAGE
    for s_, (p0, n) in enumerate(seqs):      # poison the pages that no token of this step sees
        slot = int(case.seq_slot[s_])
        for pg in range(0, max(0, p0 - window + 1) // P):
            page = int(case.table[slot, pg])
            case.kcache[page] = 1e4
            case.vcache[page] = float("nan")
    g = nh // nkv
    T = sum(b for _, b in seqs)
    qkv = rnd((T, (nh + 2 * nkv) * hd), dtype, 22)
    tq = max(1, 32 // g)
    cols = [[], [], [], []]
    t0 = 0
    for s_, (p0, n) in enumerate(seqs):
        for a in range(0, n, tq):
            for c, v in zip(cols, (s_, t0 + a, min(tq, n - a), p0 + a)):
                c.append(v)
        t0 += n
    mk = lambda x: torch.tensor(x, dtype=torch.int32, device=dev())
    out = torch.zeros(T, nh * hd, dtype=dtype, device=dev())
    o.attn_prefill(qkv, out, case.kcache, case.vcache, case.table, case.seq_slot, *[mk(c) for c in cols], len(cols[0]), tq, nh, nkv, hd,
                   1.0 / math.sqrt(hd), window=window)
    t0 = 0
    for s_, (p0, n) in enumerate(seqs):
        want = attention_rows(qkv[t0:t0 + n, :nh * hd].float().cpu(), case.k[s_], case.v[s_], p0, nh, nkv, hd, window)
        assert rel_err(out[t0:t0 + n], want) < (1e-5 if dtype == torch.float32 else 1e-2), (s_, p0, n)
        t0 += n
    # decoding: the new token is the last of each sequence
    B = len(lengths)
    for s_, n in enumerate(lengths):
        slot = int(case.seq_slot[s_])
        for pg in range(0, max(0, n - window) // P):
            page = int(case.table[slot, pg])
            case.kcache[page] = 1e4
            case.vcache[page] = float("nan")
    q1 = rnd((B, (nh + 2 * nkv) * hd), dtype, 23)
    seq_pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=dev())
    for n_splits in (1, 3, 16):
        out = torch.zeros(B, nh * hd, dtype=dtype, device=dev())
        po = torch.full((B * nh * n_splits * hd,), float("nan"), device=dev())
        pm = torch.full((B * nh * n_splits * 2,), float("nan"), device=dev())
        o.attn_decode(q1, out, case.kcache, case.vcache, case.table, case.seq_slot, seq_pos, B, nh, nkv, hd, 1.0 / math.sqrt(hd),
                      n_splits, po, pm, window=window)
        for s_, n in enumerate(lengths):
            want = attention_rows(q1[s_:s_ + 1, :nh * hd].float().cpu(), case.k[s_], case.v[s_], n - 1, nh, nkv, hd, window)
            assert rel_err(out[s_:s_ + 1], want) < (1e-5 if dtype == torch.float32 else 1e-2), (n_splits, s_, n)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_windows_edge_stands_out(dtype):
    """One key is made to dominate every query.  Placed on the window's first key the output is its value; placed one
    key earlier it must leave no trace."""
    o = ops()
    nh, nkv, hd, n, window = 2, 1, 32, 700, 130
    for where, inside in ((n - window, True), (n - window - 1, False)):
        case = PagedCase(o, dtype, [n], nkv, hd, seed=9)
        qkv = rnd((1, (nh + 2 * nkv) * hd), dtype, 24)
        qkv[:, :nh * hd] = 0
        qkv[:, 0] = 30.0
        qkv[:, hd] = 30.0           # both heads look along dim 0
        page = int(case.table[int(case.seq_slot[0]), where // o.PAGE])
        case.kcache[page, 0, where % o.PAGE] = 0
        case.kcache[page, 0, where % o.PAGE, 0] = 30.0
        case.k[0][where] = 0
        case.k[0][where, 0, 0] = 30.0
        seq_pos = torch.tensor([n - 1], dtype=torch.int32, device=dev())
        out = torch.zeros(1, nh * hd, dtype=dtype, device=dev())
        po, pm = torch.empty(nh * 4 * hd, device=dev()), torch.empty(nh * 4 * 2, device=dev())
        o.attn_decode(qkv, out, case.kcache, case.vcache, case.table, case.seq_slot, seq_pos, 1, nh, nkv, hd, 1.0 / math.sqrt(hd), 4, po, pm,
                      window=window)
        tiles = [torch.tensor([v], dtype=torch.int32, device=dev()) for v in (0, 0, 1, n - 1)]
        out2 = torch.zeros(1, nh * hd, dtype=dtype, device=dev())
        o.attn_prefill(qkv, out2, case.kcache, case.vcache, case.table, case.seq_slot, *tiles, 1, 16, nh, nkv, hd, 1.0 / math.sqrt(hd), window=window)
        want = attention_rows(qkv[:, :nh * hd].float().cpu(), case.k[0], case.v[0], n - 1, nh, nkv, hd, window)
        for got in (out, out2):
            assert rel_err(got, want) < (1e-5 if dtype == torch.float32 else 1e-2)
            close = rel_err(got[:, :hd], case.v[0][where, 0][None]) < 5e-2
            assert close == inside, (where, inside)


def test_attention_far_key_stands_out():
    """One early key among hundreds is made to dominate: the output must be its value."""
    o = ops()
    nh, nkv, hd, n = 2, 1, 32, 900
    case = PagedCase(o, torch.float32, [n], nkv, hd, seed=5)
    q = torch.zeros(1, (nh + 2 * nkv) * hd)
    q[0, :hd] = 8.0 * case.k[0][3, 0]          # head 0 looks at key 3
    q[0, hd:2 * hd] = 8.0 * case.k[0][n - 1, 0]  # head 1 looks at the newest key
    qkv = q.to(dev())
    seq_pos = torch.tensor([n - 1], dtype=torch.int32, device=dev())
    for splits in (1, 4):
        out = torch.zeros(1, nh * hd, device=dev())
        po = torch.zeros(nh * splits * hd, device=dev())
        pm = torch.zeros(nh * splits * 2, device=dev())
        o.attn_decode(qkv, out, case.kcache, case.vcache, case.table, case.seq_slot, seq_pos, 1, nh, nkv, hd,
                      1.0 / math.sqrt(hd), splits, po, pm)
        want = attention_rows(q[:, :nh * hd], case.k[0], case.v[0], n - 1, nh, nkv, hd)
        assert rel_err(out, want) < 1e-5
        assert rel_err(out[0, :hd], case.v[0][3, 0]) < 1e-2
        assert rel_err(out[0, hd:], case.v[0][n - 1, 0]) < 1e-2


def test_attention_refuses_sizes():
    o = ops()
    t = torch.zeros(1, 4 * 24, device=dev())
    i = torch.zeros(1, 1, dtype=torch.int32, device=dev())
    c = torch.zeros(1, 1, 64, 24, device=dev())
    with pytest.raises(o.KernelError, match="head size"):
        o.attn_decode(t, t[:, :48], c, c, i, i[0], i[0], 1, 2, 1, 24, 1.0)
    with pytest.raises(o.KernelError, match="multiple"):
        o.attn_decode(t, t[:, :48], c, c, i, i[0], i[0], 1, 3, 2, 16, 1.0)


# ----------------------------------------------------------------------------- RoPE + cache append
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,theta", [(4, 2, 16, 1e4), (3, 1, 32, 1e5), (9, 3, 64, 1e5), (2, 2, 48, 500.0)])
def test_rope_kv_append(dtype, nh, nkv, hd, theta):
    o = ops()
    max_pos = 300
    cos, sin = plain.rope_angles(np.arange(max_pos), hd, theta)
    cos_t, sin_t = torch.from_numpy(cos).to(dev()), torch.from_numpy(sin).to(dev())
    seqs = [(0, 5), (62, 4), (130, 1)]  # (first position, new tokens); the second crosses a page edge
    T = sum(n for _, n in seqs)
    n_pages, n_slots, max_pages = 9, 4, 5
    table = torch.full((n_slots, max_pages), -1, dtype=torch.int32)
    slots = [2, 0, 3]
    table[2, 0] = 7
    table[0, 0], table[0, 1] = 1, 4
    table[3, 2] = 0
    tok_pos, tok_seq = [], []
    for s, (p0, n) in enumerate(seqs):
        tok_pos += list(range(p0, p0 + n))
        tok_seq += [s] * n
    mk = lambda x: torch.tensor(x, dtype=torch.int32, device=dev())
    qkv = rnd((T, (nh + 2 * nkv) * hd), dtype, 30)
    orig = qkv.clone().float().cpu().numpy()
    kc = torch.zeros(n_pages, nkv, o.PAGE, hd, dtype=dtype, device=dev())
    vc = torch.zeros_like(kc)
    err = torch.zeros(1, dtype=torch.int32, device=dev())
    o.rope_kv_append(qkv, mk(tok_pos), mk(tok_seq), mk(slots), table.to(dev()), cos_t, sin_t, kc, vc, nh, nkv, hd, err)
    assert int(err.item()) == 0
    q_want = plain.rope(orig[:, :nh * hd], tok_pos, nh, hd, theta)
    k_want = plain.rope(orig[:, nh * hd:(nh + nkv) * hd], tok_pos, nkv, hd, theta)
    v_want = orig[:, (nh + nkv) * hd:]
    t = 2e-6 if dtype == torch.float32 else 8e-3
    assert rel_err(qkv[:, :nh * hd], torch.from_numpy(q_want)) < t
    written = 0
    for i, (p, s) in enumerate(zip(tok_pos, tok_seq)):
        page = int(table[slots[s], p // o.PAGE])
        krow = kc[page, :, p % o.PAGE].reshape(-1)
        vrow = vc[page, :, p % o.PAGE].reshape(-1)
        assert rel_err(krow, torch.from_numpy(k_want[i])) < t
        assert torch.equal(vrow.float().cpu(), torch.from_numpy(v_want[i]))
        written += 1
    assert int((kc.float().abs().sum(dim=(1, 3)) > 0).sum()) == written  # nothing else was touched
    bad = mk([max_pos])
    o.rope_kv_append(qkv[:1], bad, mk([0]), mk(slots), table.to(dev()), cos_t, sin_t, kc, vc, nh, nkv, hd, err)
    assert int(err.item()) & 2
    err.zero_()


# ----------------------------------------------------------------------------- sampling
@pytest.mark.parametrize("vocab", [256, 397, 49152, 1000])
def test_argmax_first_maximum(vocab):
    o = ops()
    x = rnd((6, vocab), torch.float32, 40)
    x[1, 17] = x[1, vocab - 5] = 50.0
    x[2, :] = 1.0
    x[3, vocab - 1] = 60.0
    out = torch.zeros(6, dtype=torch.int32, device=dev())
    o.argmax_rows(x, out)
    want = [plain.argmax(r) for r in x.cpu().numpy()]
    assert out.tolist() == want
    assert out[1] == 17 and out[2] == 0 and out[3] == vocab - 1


@pytest.mark.parametrize("vocab,temp,k,seed", [(397, 0.8, 20, 7), (256, 1.0, 40, 42), (100, 0.5, 0, 3), (64, 1.3, 1000, 9),
                                                 (49152, 0.9, 40, 1), (5000, 2.0, -1, 12), (1000, 0.3, 2, 5),
                                                 (49152, 0.7, 0, 2), (3001, 1.1, 1024, 4), (3001, 1.1, 1025, 4),   # ranked list up to 1,024 kept tokens, radix descent beyond
                                                 (60000, 0.8, 50, 6)])                                           # a row too long for shared memory
def test_sample_topk_matches_plain(vocab, temp, k, seed):
    o = ops()
    import golden_models as gm
    rows = 6
    steps = 8
    state = [(s * 0x9E3779B97F4A7C15 + 1) & plain.MASK64 for s in range(seed, seed + rows)]
    st = torch.tensor([s - (1 << 64) if s >= (1 << 63) else s for s in state], dtype=torch.int64, device=dev())
    samplers = [plain.Sampler(temp, k, s) for s in range(seed, seed + rows)]
    out = torch.zeros(rows, dtype=torch.int32, device=dev())
    scratch = torch.zeros(rows, dtype=torch.int32, device=dev())
    for step in range(steps):
        if step % 2 == 0:
            x = torch.from_numpy(gm.sampler_logits(rows, vocab, step))  # coarse grid: many exact ties
        else:
            x = torch.randn(rows, vocab, generator=torch.Generator().manual_seed(step)) * 3
        xd = x.to(dev())
        # odd steps with the scratch (the fast kernel where it applies), even steps without (the general kernel)
        o.sample_topk(xd, temp, k, st, out, scratch=scratch if step % 4 < 2 else None)
        want = [s.sample(r) for s, r in zip(samplers, x.numpy())]
        assert out.tolist() == want, (step,)
    assert [v & plain.MASK64 for v in st.tolist()] == [s.state for s in samplers]


# ----------------------------------------------------------------------------- GEMM (tcgen05 tensor cores)
TC_SHAPES = [(128, 128, 64), (17, 64, 72), (129, 192, 576), (300, 100, 200), (256, 960, 576), (2048, 576, 1536),
             (64, 397, 96), (130, 49, 8), (1000, 130, 136), (2048, 2048, 256), (1920, 2050, 200),
             (64, 2048, 8192), (64, 576, 1536), (100, 397, 1032), (129, 200, 4096)]  # few tiles and long K: split-K


@pytest.mark.parametrize("M,N,K", TC_SHAPES)
def test_gemm_tc_store_and_residual(M, N, K):
    o = ops()
    a = rnd((M, K), torch.bfloat16, 50)
    w = rnd((N, K), torch.bfloat16, 51, 0.2)
    err = torch.zeros(1, dtype=torch.int32, device=dev())
    assert o.gemm_tc_takes(a, w, None)
    want = a.double().cpu() @ w.double().cpu().T
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev())
    o.gemm_tc(a, w, out, err)
    assert int(err.item()) == 0
    assert rel_err(out, want) < 1.6e-2
    out32 = torch.full((M, N), float("nan"), dtype=torch.float32, device=dev())
    o.gemm_tc(a, w, out32, err)
    assert rel_err(out32, want) < 2e-5
    res = rnd((M, N), torch.float32, 52)
    res0 = res.clone()
    o.gemm_tc(a, w, res, err, epilogue=o.EPI_RESIDUAL, residual=res)
    assert rel_err(res, res0.double().cpu() + want) < 2e-5
    assert int(err.item()) == 0
    # the same numbers as the CUDA-core kernel up to the order of float32 sums
    simt = torch.empty(M, N, dtype=torch.float32, device=dev())
    o.gemm_simt(a, w, simt)
    assert rel_err(out32, simt) < 2e-5


@pytest.mark.parametrize("M,N,K", [(128, 64, 64), (200, 200, 96), (2048, 1536, 576), (33, 130, 40), (64, 520, 1024), (40, 1536, 2048)])
def test_gemm_tc_swiglu(M, N, K):
    o = ops()
    a = rnd((M, K), torch.bfloat16, 53)
    wg = rnd((N, K), torch.bfloat16, 54, 0.3)
    wu = rnd((N, K), torch.bfloat16, 55, 0.3)
    err = torch.zeros(1, dtype=torch.int32, device=dev())
    g = a.double().cpu() @ wg.double().cpu().T
    u = a.double().cpu() @ wu.double().cpu().T
    want = g / (1 + torch.exp(-g)) * u
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev())
    o.gemm_tc(a, wg, out, err, epilogue=o.EPI_SWIGLU, w2=wu)
    assert int(err.item()) == 0
    assert rel_err(out, want) < 1.6e-2


# Products that the dispatch gives to the 128 x 256 tiles (128 x 2 x 128 for SwiGLU): at least 120 of them, N and K
# at least 1,024.  Without a residual they run on the persistent kernel (a block walks several tiles, two accumulator
# stages), with one as one wide tile a block.  Ragged M, N and K tails, a last wave that is not full, and a row count
# whose last tile holds one row.  Every case asserts which kernel ran.
TC_WIDE = [(2048, 6144, 2048), (1985, 2050, 1032), (3000, 1544, 1096), (2049, 4096, 1024)]
TC_WIDE_RESIDUAL = [(2048, 2048, 8192), (1920, 2050, 1032), (1985, 3080, 1096)]
TC_WIDE_SWIGLU = [(2048, 8192, 2048), (1100, 2050, 1096), (1985, 1536, 1032)]


def _products(a, w):
    """Float64 product on the device (the CPU would take seconds at these sizes)."""
    return (a.double() @ w.double().T).cpu()


@pytest.mark.parametrize("M,N,K", TC_WIDE)
def test_gemm_tc_wide_persistent_store(M, N, K):
    o = ops()
    a = rnd((M, K), torch.bfloat16, 150)
    w = rnd((N, K), torch.bfloat16, 151, 0.2)
    err = torch.zeros(1, dtype=torch.int32, device=dev())
    want = _products(a, w)
    for dt, tol_ in ((torch.bfloat16, 1.6e-2), (torch.float32, 2e-5)):
        out = torch.full((M, N), float("nan"), dtype=dt, device=dev())
        o.gemm_tc(a, w, out, err)
        k = o.gemm_tc_last_kernel()
        assert k["tile_columns"] == 256 and k["persistent"], k
        assert int(err.item()) == 0
        assert rel_err(out, want) < tol_
        # every element, not only the largest: a tile written to the wrong place shows as an error of order 1
        assert (out.double().cpu() - want).abs().max() < (0.3 if dt == torch.bfloat16 else 2e-3)


@pytest.mark.parametrize("M,N,K", TC_WIDE_RESIDUAL)
def test_gemm_tc_wide_residual(M, N, K):
    o = ops()
    a = rnd((M, K), torch.bfloat16, 152)
    w = rnd((N, K), torch.bfloat16, 153, 0.2)
    err = torch.zeros(1, dtype=torch.int32, device=dev())
    res = rnd((M, N), torch.float32, 154)
    want = res.double().cpu() + _products(a, w)
    o.gemm_tc(a, w, res, err, epilogue=o.EPI_RESIDUAL, residual=res)
    k = o.gemm_tc_last_kernel()
    assert k["tile_columns"] == 256 and not k["persistent"] and k["k_splits"] == 1, k
    assert int(err.item()) == 0
    assert rel_err(res, want) < 2e-5


@pytest.mark.parametrize("M,N,K", TC_WIDE_SWIGLU)
def test_gemm_tc_wide_persistent_swiglu(M, N, K):
    o = ops()
    a = rnd((M, K), torch.bfloat16, 155, 0.5)
    wg = rnd((N, K), torch.bfloat16, 156, 0.1)
    wu = rnd((N, K), torch.bfloat16, 157, 0.1)
    err = torch.zeros(1, dtype=torch.int32, device=dev())
    g, u = _products(a, wg), _products(a, wu)
    want = g / (1 + torch.exp(-g)) * u
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev())
    o.gemm_tc(a, wg, out, err, epilogue=o.EPI_SWIGLU, w2=wu)
    k = o.gemm_tc_last_kernel()
    assert k["tile_columns"] == 128 and k["persistent"], k
    assert int(err.item()) == 0
    assert rel_err(out, want) < 1.6e-2


def test_gemm_tc_dispatch_names_its_kernel():
    """The other branches of the dispatch, each on a product that should reach it."""
    o = ops()
    err = torch.zeros(1, dtype=torch.int32, device=dev())
    for (M, N, K), want in (((2048, 576, 576), dict(tile_columns=64, persistent=False, k_splits=1)),
                            ((2048, 2048, 256), dict(tile_columns=128, persistent=False, k_splits=1)),
                            ((256, 960, 576), dict(tile_columns=64, persistent=False)),
                            ((64, 576, 576), dict(tile_columns=32, persistent=False, k_splits=1)),
                            ((64, 2048, 2048), dict(tile_columns=128, persistent=False)),     # 4 Mi weights: not small enough for tiles of 32
                            ((64, 2048, 8192), dict(tile_columns=128, persistent=False))):
        a = rnd((M, K), torch.bfloat16, 158)
        w = rnd((N, K), torch.bfloat16, 159, 0.2)
        out = torch.empty((M, N), dtype=torch.bfloat16, device=dev())
        o.gemm_tc(a, w, out, err)
        k = o.gemm_tc_last_kernel()
        assert all(k[key] == v for key, v in want.items()), ((M, N, K), k)
        assert rel_err(out, _products(a, w)) < 1.6e-2
    k = o.gemm_tc_last_kernel()
    assert k["k_splits"] > 1, k   # 64 rows, N 2048, K 8192: sixteen tiles, split over K


@pytest.mark.parametrize("M,N,K", [(17, 576, 576), (64, 960, 576), (128, 1536, 576), (64, 576, 1536), (33, 100, 200), (64, 4704, 96),
                                     (100, 2040, 2048)])
def test_gemm_tc_tiles_of_32_columns_when_all_rows_are_one_tile(M, N, K):
    """Decode steps of 17 to 128 sequences: one tile of rows, and weights so small that wider tiles would come to a
    handful of blocks: tiles of 32 columns, every epilogue, with and without K split over the grid, a ragged last
    tile; against float64 and against the same product on wider tiles."""
    o = ops()
    a = rnd((M, K), torch.bfloat16, 160, 0.5)
    w = rnd((N, K), torch.bfloat16, 161, 0.2)
    w2 = rnd((N, K), torch.bfloat16, 162, 0.2)
    res0 = rnd((M, N), torch.float32, 163)
    err = torch.zeros(1, dtype=torch.int32, device=dev())
    want = _products(a, w)
    u = _products(a, w2)

    def run():
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev())
        o.gemm_tc(a, w, out, err)
        cols = o.gemm_tc_last_kernel()["tile_columns"]
        out32 = torch.full((M, N), float("nan"), dtype=torch.float32, device=dev())
        o.gemm_tc(a, w, out32, err)
        res = res0.clone()
        o.gemm_tc(a, w, res, err, epilogue=o.EPI_RESIDUAL, residual=res)
        sw = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev())
        o.gemm_tc(a, w, sw, err, epilogue=o.EPI_SWIGLU, w2=w2)
        torch.cuda.synchronize()
        return cols, out, out32, res, sw

    cols, out, out32, res, sw = run()
    assert cols == 32 and int(err.item()) == 0
    assert rel_err(out, want) < 1.6e-2 and rel_err(out32, want) < 2e-5 and rel_err(res, res0.double().cpu() + want) < 2e-5
    assert rel_err(sw, want / (1 + torch.exp(-want)) * u) < 1.6e-2
    o.lib().edgelm_gemm_tc_tiny(0)
    try:
        wider = run()
    finally:
        o.lib().edgelm_gemm_tc_tiny(1)
    assert wider[0] > 32
    assert rel_err(out32, wider[2].double().cpu()) < 1e-5 and rel_err(res, wider[3].double().cpu()) < 1e-5


def test_gemm_tc_strided_rows_and_refusals():
    o = ops()
    big = rnd((70, 3 * 64), torch.bfloat16, 56)
    a = big[:, 64:128]  # row pitch 192, a view as the attention output's columns would be
    w = rnd((40, 64), torch.bfloat16, 57)
    err = torch.zeros(1, dtype=torch.int32, device=dev())
    out = torch.zeros(70, 40, dtype=torch.float32, device=dev())
    o.gemm_tc(a, w, out, err)
    assert rel_err(out, a.double().cpu() @ w.double().cpu().T) < 2e-5
    assert not o.gemm_tc_takes(rnd((4, 12), torch.bfloat16, 1), rnd((4, 12), torch.bfloat16, 2), None)  # K = 12: pitch of 24 bytes
    with pytest.raises(o.KernelError, match="multiples of 8"):
        o.gemm_tc(rnd((4, 12), torch.bfloat16, 1), rnd((4, 12), torch.bfloat16, 2), torch.zeros(4, 4, device=dev()), err)


# ----------------------------------------------------------------------------- few-rows kernel (decode)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 576, 576), (8, 960, 576), (3, 37, 96), (9, 130, 160), (16, 49152, 64), (5, 397, 200),
                                     (8, 100, 8192), (2, 3000, 2048)])
def test_gemv_epilogues(dtype, M, N, K):
    o = ops()
    a = rnd((M, K), dtype, 60)
    w = rnd((N, K), dtype, 61, 0.2)
    w2 = rnd((N, K), dtype, 62, 0.2)
    assert o.gemv_takes(a, w, w2)
    want = a.double().cpu() @ w.double().cpu().T
    out = torch.full((M, N), float("nan"), dtype=dtype, device=dev())
    o.gemv(a, w, out)
    assert rel_err(out, want) < tol(dtype)
    out32 = torch.full((M, N), float("nan"), dtype=torch.float32, device=dev())
    o.gemv(a, w, out32)
    assert rel_err(out32, want) < 2e-5
    ref = torch.empty(M, N, dtype=torch.float32, device=dev())
    o.gemm_simt(a, w, ref, force_kernel=1)
    assert torch.equal(out32, ref)  # the same order of sums as the scalar kernel: the same bits
    res = rnd((M, N), torch.float32, 63)
    res0 = res.clone()
    o.gemv(a, w, res, epilogue=o.EPI_RESIDUAL, residual=res)
    assert rel_err(res, res0.double().cpu() + want) < 2e-5
    u = a.double().cpu() @ w2.double().cpu().T
    sw = torch.full((M, N), float("nan"), dtype=dtype, device=dev())
    o.gemv(a, w, sw, epilogue=o.EPI_SWIGLU, w2=w2)
    assert rel_err(sw, want / (1 + torch.exp(-want)) * u) < tol(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K,eps", [(8, 960, 576, 1e-5), (1, 200, 96, 1e-6), (12, 64, 2048, 1e-5), (3, 50, 8200, 1e-3)])
def test_gemv_with_norm_prologue(dtype, M, N, K, eps):
    o = ops()
    x = rnd((M, K), torch.float32, 64, 2.0)
    nw = 1 + rnd((K,), torch.float32, 65, 0.1)
    w = rnd((N, K), dtype, 66, 0.2)
    assert o.gemv_takes(x, w, None, normed=True)
    h = torch.empty(M, K, dtype=dtype, device=dev())
    o.rmsnorm(x, nw, eps, h)
    want = torch.empty(M, N, dtype=torch.float32, device=dev())
    o.gemv(h, w, want)
    got = torch.full((M, N), float("nan"), dtype=torch.float32, device=dev())
    o.gemv(x, w, got, norm_weight=nw, eps=eps)
    assert rel_err(got, want) < (2e-6 if dtype == torch.float32 else 4e-3)  # the norm's sum runs in another order
    plain_h = torch.from_numpy(plain.rmsnorm(x.cpu().numpy(), nw.cpu().numpy(), eps)).double()
    assert rel_err(got, plain_h @ w.double().cpu().T) < tol(dtype)


def test_gemv_refuses_unaligned():
    o = ops()
    assert not o.gemv_takes(rnd((2, 12), torch.bfloat16, 1), rnd((4, 12), torch.bfloat16, 2))
    assert not o.gemv_takes(rnd((2, 6), torch.float32, 1), rnd((4, 6), torch.float32, 2))
    with pytest.raises(o.KernelError, match="16-byte"):
        o.gemv(rnd((2, 12), torch.bfloat16, 1), rnd((4, 12), torch.bfloat16, 2), torch.zeros(2, 4, device=dev()))


# ----------------------------------------------------------------------------- few-rows kernel on mma.sync (bfloat16 decode)
@pytest.mark.parametrize("M,N,K", [(1, 576, 576), (8, 960, 576), (3, 37, 96), (9, 130, 160), (16, 4000, 64), (5, 397, 200),
                                     (8, 100, 6144), (2, 3000, 2048), (7, 16, 8), (13, 31, 40), (8, 64, 8192), (11, 40, 9000)])
def test_gemv_mma_epilogues(M, N, K):
    o = ops()
    a = rnd((M, K), torch.bfloat16, 70)
    w = rnd((N, K), torch.bfloat16, 71, 0.2)
    w2 = rnd((N, K), torch.bfloat16, 72, 0.2)
    assert o.gemv_mma_takes(a, w, w2)
    want = a.double().cpu() @ w.double().cpu().T
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev())
    o.gemv_mma(a, w, out)
    assert rel_err(out, want) < 1.6e-2
    out32 = torch.full((M, N), float("nan"), dtype=torch.float32, device=dev())
    o.gemv_mma(a, w, out32)
    assert rel_err(out32, want) < 2e-5
    res = rnd((M, N), torch.float32, 73)
    res0 = res.clone()
    o.gemv_mma(a, w, res, epilogue=o.EPI_RESIDUAL, residual=res)
    assert rel_err(res, res0.double().cpu() + want) < 2e-5
    u = a.double().cpu() @ w2.double().cpu().T
    sw = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev())
    o.gemv_mma(a, w, sw, epilogue=o.EPI_SWIGLU, w2=w2)
    assert rel_err(sw, want / (1 + torch.exp(-want)) * u) < 1.6e-2


@pytest.mark.parametrize("M,N,K,eps", [(8, 960, 576, 1e-5), (1, 200, 96, 1e-6), (12, 64, 2048, 1e-5), (3, 50, 4104, 1e-3), (5, 48, 8200, 1e-5)])
def test_gemv_mma_with_norm_prologue(M, N, K, eps):
    o = ops()
    x = rnd((M, K), torch.float32, 74, 2.0)
    nw = 1 + rnd((K,), torch.float32, 75, 0.1)
    w = rnd((N, K), torch.bfloat16, 76, 0.2)
    assert o.gemv_mma_takes(x, w, None, normed=True)
    h = torch.empty(M, K, dtype=torch.bfloat16, device=dev())
    o.rmsnorm(x, nw, eps, h)
    want = torch.empty(M, N, dtype=torch.float32, device=dev())
    o.gemv_mma(h, w, want)
    got = torch.full((M, N), float("nan"), dtype=torch.float32, device=dev())
    o.gemv_mma(x, w, got, norm_weight=nw, eps=eps)
    assert rel_err(got, want) < 4e-3  # the norm's sum runs in another order: a last-bit difference before rounding
    plain_h = torch.from_numpy(plain.rmsnorm(x.cpu().numpy(), nw.cpu().numpy(), eps)).double()
    assert rel_err(got, plain_h @ w.double().cpu().T) < 1.6e-2


def test_gemv_mma_row_independent_of_batch_and_refusals():
    o = ops()
    a = rnd((16, 96), torch.bfloat16, 77)
    w = rnd((50, 96), torch.bfloat16, 78)
    full = torch.empty(16, 50, device=dev())
    o.gemv_mma(a, w, full)
    one = torch.empty(1, 50, device=dev())
    o.gemv_mma(a[11:12], w, one)
    assert torch.equal(one, full[11:12])
    assert not o.gemv_mma_takes(rnd((17, 96), torch.bfloat16, 1), w)
    assert not o.gemv_mma_takes(rnd((2, 12), torch.bfloat16, 1), rnd((4, 12), torch.bfloat16, 2))
    assert not o.gemv_mma_takes(rnd((2, 96), torch.float32, 1), rnd((4, 96), torch.float32, 2))
    with pytest.raises(o.KernelError, match="M <= 16"):
        o.gemv_mma(rnd((17, 96), torch.bfloat16, 1), w, torch.zeros(17, 50, device=dev()))


@pytest.mark.parametrize("M,N,K", [(8, 6144, 2048), (3, 4744, 1032), (16, 8192, 2048), (1, 49152, 1024), (12, 5000, 4096), (5, 4736, 576)])
def test_gemv_mma_wide_outputs_on_the_walking_kernel(M, N, K):
    """Outputs wide enough for the kernel whose blocks walk several groups of 16 columns: a ragged last group, one and
    two tiles of rows, one and several rounds of K, K that is no multiple of 32; against float64 and against the kernel
    of one block a group."""
    o = ops()
    a = rnd((M, K), torch.bfloat16, 83)
    w = rnd((N, K), torch.bfloat16, 84, 0.2)
    w2 = rnd((N, K), torch.bfloat16, 85, 0.2)
    want = a.double().cpu() @ w.double().cpu().T
    u = a.double().cpu() @ w2.double().cpu().T
    got = {}
    for walk in (True, False):
        o.gemv_mma_walk(walk)
        try:
            out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev())
            o.gemv_mma(a, w, out)
            out32 = torch.full((M, N), float("nan"), dtype=torch.float32, device=dev())
            o.gemv_mma(a, w, out32, prefetch=(w2,))
            sw = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev())
            o.gemv_mma(a, w, sw, epilogue=o.EPI_SWIGLU, w2=w2)
            torch.cuda.synchronize()
        finally:
            o.gemv_mma_walk(True)
        assert rel_err(out, want) < 1.6e-2 and rel_err(out32, want) < 2e-5
        assert rel_err(sw, want / (1 + torch.exp(-want)) * u) < 1.6e-2
        got[walk] = (out32, sw)
    assert rel_err(got[True][0], got[False][0].double().cpu()) < 1e-5   # (the warps may share K differently: last bits)


def test_gemv_mma_prefetch_of_the_next_weights_changes_no_result():
    """The hint that starts other tensors on their way into L2: odd sizes (not a multiple of the blocks' slices),
    one and two regions, more blocks than 16-byte pieces; the product is the same bit for bit and the regions are
    untouched.  Misaligned regions are refused."""
    o = ops()
    a = rnd((5, 576), torch.bfloat16, 79)
    w = rnd((960, 576), torch.bfloat16, 80, 0.2)
    want = torch.empty(5, 960, device=dev())
    o.gemv_mma(a, w, want)
    big = rnd((1536, 577 * 8), torch.bfloat16, 81)        # 14 MB, rows of an odd number of 16-byte pieces
    small = rnd((3, 8), torch.bfloat16, 82)               # 48 bytes: fewer pieces than blocks
    big0, small0 = big.clone(), small.clone()
    for regions in ((big,), (small,), (big, small), (small, big)):
        got = torch.full((5, 960), float("nan"), device=dev())
        o.gemv_mma(a, w, got, prefetch=regions)
        assert torch.equal(got, want)
    got = torch.full((5, 960), float("nan"), device=dev())
    o.gemv_mma(a, w, got)                                  # (the hint is used up by the launch after it)
    torch.cuda.synchronize()
    assert torch.equal(got, want) and torch.equal(big, big0) and torch.equal(small, small0)
    with pytest.raises(o.KernelError, match="16-byte aligned"):
        o.gemv_mma(a, w, got, prefetch=(big.view(-1)[4:4 + 1024],))
    o.gemv_mma(a, w, got)
    assert torch.equal(got, want)


# ----------------------------------------------------------------------------- prefill attention on mma.sync (bfloat16)
@pytest.mark.parametrize("groups", [0, 1, 2, 4])
@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 32), (9, 3, 64), (3, 1, 96), (4, 4, 128), (8, 1, 64)])
def test_attn_prefill_mma(nh, nkv, hd, groups):
    o = ops()
    assert o.attn_prefill_mma_takes(torch.bfloat16, hd) and not o.attn_prefill_mma_takes(torch.bfloat16, 48)
    assert not o.attn_prefill_mma_takes(torch.float32, hd)
    seqs = [(0, 5), (0, 70), (64, 1), (100, 129), (63, 2), (0, 64), (30, 200)]  # (cached before, new tokens)
    lengths = [a + b for a, b in seqs]
    case = PagedCase(o, torch.bfloat16, lengths, nkv, hd, seed=nh * 10 + hd)
    T = sum(b for _, b in seqs)
    qkv = rnd((T, (nh + 2 * nkv) * hd), torch.bfloat16, 80)
    tq = o.MMA_PREFILL_TILE
    tile_seq, tile_tok0, tile_ntok, tile_pos0 = [], [], [], []
    t0 = 0
    for s, (p0, n) in enumerate(seqs):
        for a in range(0, n, tq):
            tile_seq.append(s)
            tile_tok0.append(t0 + a)
            tile_ntok.append(min(tq, n - a))
            tile_pos0.append(p0 + a)
        t0 += n
    mk = lambda x: torch.tensor(x, dtype=torch.int32, device=dev())
    out = torch.full((T, nh * hd), float("nan"), dtype=torch.bfloat16, device=dev())
    o.attn_prefill_mma(qkv, out, case.kcache, case.vcache, case.table, case.seq_slot, mk(tile_seq), mk(tile_tok0),
                       mk(tile_ntok), mk(tile_pos0), len(tile_seq), nh, nkv, hd, 1.0 / math.sqrt(hd),
                       max_keys=max(lengths), force_groups=groups)
    t0 = 0
    for s, (p0, n) in enumerate(seqs):
        want = attention_rows(qkv[t0:t0 + n, :nh * hd].float().cpu(), case.k[s], case.v[s], p0, nh, nkv, hd)
        assert rel_err(out[t0:t0 + n], want) < 1.2e-2, (s, p0, n)
        t0 += n


def test_attn_prefill_mma_far_key_and_diagonal():
    """Scaled queries make one early key, or the token's own key, dominate: a wrong mask or page shows."""
    o = ops()
    nh, nkv, hd, p0, n = 2, 1, 64, 130, 150
    case = PagedCase(o, torch.bfloat16, [p0 + n], nkv, hd, seed=8)
    q = torch.zeros(n, (nh + 2 * nkv) * hd)
    for t in range(n):
        q[t, :hd] = 12.0 * case.k[0][3, 0]                 # head 0: key 3, far back
        q[t, hd:2 * hd] = 12.0 * case.k[0][p0 + t, 0]      # head 1: its own position, the last it may see
    qkv = q.to(torch.bfloat16).to(dev())
    tq = o.MMA_PREFILL_TILE
    tiles = [(0, a, min(tq, n - a), p0 + a) for a in range(0, n, tq)]
    mk = lambda x: torch.tensor(x, dtype=torch.int32, device=dev())
    out = torch.zeros(n, nh * hd, dtype=torch.bfloat16, device=dev())
    o.attn_prefill_mma(qkv, out, case.kcache, case.vcache, case.table, case.seq_slot, mk([t[0] for t in tiles]),
                       mk([t[1] for t in tiles]), mk([t[2] for t in tiles]), mk([t[3] for t in tiles]), len(tiles), nh, nkv,
                       hd, 1.0 / math.sqrt(hd))
    want = attention_rows(qkv[:, :nh * hd].float().cpu(), case.k[0], case.v[0], p0, nh, nkv, hd)
    assert rel_err(out, want) < 1.2e-2
    assert rel_err(out[:, :hd], case.v[0][3, 0].expand(n, hd)) < 5e-2
    assert rel_err(out[:, hd:], case.v[0][p0:p0 + n, 0]) < 5e-2


# ----------------------------------------------------------------------------- prefill attention on tcgen05 (bfloat16, head size 64)
def _tc_tiles(seqs, tq):
    cols = [[], [], [], []]
    t0 = 0
    for s, (p0, n) in enumerate(seqs):
        for a in range(0, n, tq):
            for c, v in zip(cols, (s, t0 + a, min(tq, n - a), p0 + a)):
                c.append(v)
        t0 += n
    return [torch.tensor(c, dtype=torch.int32, device=dev()) for c in cols]


@pytest.mark.parametrize("nh,nkv", [(9, 3), (4, 4), (8, 1), (2, 1)])
def test_attn_prefill_tc(nh, nkv):
    o = ops()
    hd = 64
    assert o.attn_prefill_tc_takes(torch.bfloat16, 64) and not o.attn_prefill_tc_takes(torch.bfloat16, 128)
    assert not o.attn_prefill_tc_takes(torch.float32, 64)
    # (cached before, new tokens): page and block edges on both sides, a tile that spans two diagonal blocks,
    # a second page that does not exist, several tiles of one sequence
    seqs = [(0, 5), (0, 70), (64, 1), (100, 129), (63, 2), (0, 64), (30, 200), (0, 128), (127, 130), (0, 600)]
    lengths = [a + b for a, b in seqs]
    case = PagedCase(o, torch.bfloat16, lengths, nkv, hd, seed=nh * 10 + nkv)
    T = sum(b for _, b in seqs)
    qkv = rnd((T, (nh + 2 * nkv) * hd), torch.bfloat16, 81)
    tiles = _tc_tiles(seqs, o.TC_PREFILL_TILE)
    err = torch.zeros(1, dtype=torch.int32, device=dev())
    out = torch.full((T, nh * hd), float("nan"), dtype=torch.bfloat16, device=dev())
    o.attn_prefill_tc(qkv, out, case.kcache, case.vcache, case.table, case.seq_slot, *tiles, tiles[0].numel(), nh, nkv, hd,
                      1.0 / math.sqrt(hd), err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    t0 = 0
    for s, (p0, n) in enumerate(seqs):
        want = attention_rows(qkv[t0:t0 + n, :nh * hd].float().cpu(), case.k[s], case.v[s], p0, nh, nkv, hd)
        assert rel_err(out[t0:t0 + n], want) < 1.2e-2, (s, p0, n)
        t0 += n


def test_attn_prefill_tc_far_key_and_diagonal():
    """Scaled queries make one early key, or the token's own key, dominate: a wrong mask, page or value layout shows."""
    o = ops()
    nh, nkv, hd, p0, n = 2, 1, 64, 130, 300
    case = PagedCase(o, torch.bfloat16, [p0 + n], nkv, hd, seed=8)
    q = torch.zeros(n, (nh + 2 * nkv) * hd)
    for t in range(n):
        q[t, :hd] = 12.0 * case.k[0][3, 0]                 # head 0: key 3, far back
        q[t, hd:2 * hd] = 12.0 * case.k[0][p0 + t, 0]      # head 1: its own position, the last it may see
    qkv = q.to(torch.bfloat16).to(dev())
    tiles = _tc_tiles([(p0, n)], o.TC_PREFILL_TILE)
    err = torch.zeros(1, dtype=torch.int32, device=dev())
    out = torch.zeros(n, nh * hd, dtype=torch.bfloat16, device=dev())
    o.attn_prefill_tc(qkv, out, case.kcache, case.vcache, case.table, case.seq_slot, *tiles, tiles[0].numel(), nh, nkv, hd,
                      1.0 / math.sqrt(hd), err)
    want = attention_rows(qkv[:, :nh * hd].float().cpu(), case.k[0], case.v[0], p0, nh, nkv, hd)
    assert int(err.item()) == 0
    assert rel_err(out, want) < 1.2e-2
    assert rel_err(out[:, :hd], case.v[0][3, 0].expand(n, hd)) < 5e-2
    assert rel_err(out[:, hd:], case.v[0][p0:p0 + n, 0]) < 5e-2


# ----------------------------------------------------------------------------- q, k, v projection with RoPE and append in its epilogue
@pytest.mark.parametrize("nh,nkv,hd,K,lens,kernel", [
    (9, 3, 64, 576, [(0, 300)], dict(tile_columns=64)),                                   # one head a tile
    (15, 5, 64, 960, [(0, 1500), (64, 1), (100, 447), (63, 100)], dict(tile_columns=128)),     # continued prompts, 2,048 tokens
    (32, 32, 64, 2048, [(0, 2048), (10, 37)], dict(tile_columns=256, persistent=True)),   # the persistent kernel, ragged last tile
    (4, 2, 128, 256, [(0, 130), (5, 70)], dict(tile_columns=128)),                        # head size 128: a head is a whole tile
    (6, 1, 128, 1096, [(0, 3100), (3, 900)], dict(tile_columns=256, persistent=True)),
])
def test_gemm_tc_rope_append_epilogue(nh, nkv, hd, K, lens, kernel):
    """Against the plain implementation (product, rotation of q and k at each token's position, k and v at their
    places in the pages), and bit for bit against the separate kernels (product, then rotate + append)."""
    o = ops()
    seqs = lens
    T = sum(n for _, n in seqs)
    width = (nh + 2 * nkv) * hd
    theta, max_pos = 30000.0, max(p + n for p, n in seqs) + 5
    cos, sin = plain.rope_angles(np.arange(max_pos), hd, theta)
    cos_t, sin_t = torch.from_numpy(cos).to(dev()), torch.from_numpy(sin).to(dev())
    a = rnd((T, K), torch.bfloat16, 170, 0.5)
    w = rnd((width, K), torch.bfloat16, 171, 0.1)
    lengths = [p + n for p, n in seqs]
    ca = PagedCase(o, torch.bfloat16, lengths, nkv, hd, seed=nh + K)
    cb = PagedCase(o, torch.bfloat16, lengths, nkv, hd, seed=nh + K)
    tok_pos = torch.tensor([p + i for p, n in seqs for i in range(n)], dtype=torch.int32, device=dev())
    tok_seq = torch.tensor([s for s, (p, n) in enumerate(seqs) for _ in range(n)], dtype=torch.int32, device=dev())
    err = torch.zeros(1, dtype=torch.int32, device=dev())
    # separate kernels
    q1 = torch.empty(T, width, dtype=torch.bfloat16, device=dev())
    o.gemm_tc(a, w, q1, err)
    o.rope_kv_append(q1, tok_pos, tok_seq, ca.seq_slot, ca.table, cos_t, sin_t, ca.kcache, ca.vcache, nh, nkv, hd, err)
    # one kernel
    q2 = torch.full((T, width), 7.0, dtype=torch.bfloat16, device=dev())
    assert o.gemm_tc_rope_takes(a, w, q2, cb.kcache, cb.vcache, cos_t, sin_t, hd)
    o.gemm_tc_rope(a, w, q2, tok_pos, tok_seq, cb.seq_slot, cb.table, cos_t, sin_t, cb.kcache, cb.vcache, nh, nkv, hd, err)
    k = o.gemm_tc_last_kernel()
    assert all(k[key] == v for key, v in kernel.items()) and k["k_splits"] == 1, k
    assert int(err.item()) == 0
    assert torch.equal(q2[:, :nh * hd], q1[:, :nh * hd])
    assert bool((q2[:, nh * hd:] == 7.0).all())                     # the k and v columns are not written
    same = lambda x, y: bool(((x == y) | (torch.isnan(x) & torch.isnan(y))).all())
    assert same(cb.kcache, ca.kcache) and same(cb.vcache, ca.vcache)  # every row of every page, written or not
    # the plain implementation
    y = (a.double() @ w.double().T).float().cpu().to(torch.bfloat16).float().numpy()
    pos = tok_pos.cpu().numpy()
    qr = plain.rope(y[:, :nh * hd], pos, nh, hd, theta)
    kr = plain.rope(y[:, nh * hd:(nh + nkv) * hd], pos, nkv, hd, theta).reshape(T, nkv, hd)
    vr = y[:, (nh + nkv) * hd:].reshape(T, nkv, hd)
    assert rel_err(q2[:, :nh * hd], torch.from_numpy(qr)) < 1.6e-2
    t0 = 0
    for s, (p0, n) in enumerate(seqs):
        slot = int(cb.seq_slot[s])
        for t in (0, n // 2, n - 1):
            page = int(cb.table[slot, (p0 + t) // o.PAGE])
            assert rel_err(cb.kcache[page, :, (p0 + t) % o.PAGE], torch.from_numpy(kr[t0 + t])) < 1.6e-2
            assert rel_err(cb.vcache[page, :, (p0 + t) % o.PAGE], torch.from_numpy(vr[t0 + t])) < 1.6e-2
        t0 += n


def test_gemm_tc_rope_reports_bad_positions_and_pages():
    o = ops()
    nh, nkv, hd, K, T = 2, 1, 64, 64, 40
    cos, sin = plain.rope_angles(np.arange(64), hd, 1e4)
    cos_t, sin_t = torch.from_numpy(cos).to(dev()), torch.from_numpy(sin).to(dev())
    a, w = rnd((T, K), torch.bfloat16, 1), rnd(((nh + 2 * nkv) * hd, K), torch.bfloat16, 2)
    case = PagedCase(o, torch.bfloat16, [64], nkv, hd, seed=3)
    qkv = torch.zeros(T, (nh + 2 * nkv) * hd, dtype=torch.bfloat16, device=dev())
    tok_seq = torch.zeros(T, dtype=torch.int32, device=dev())
    for bad, bit in ((torch.arange(30, 30 + T), 2), (torch.arange(0, T), 4)):
        err = torch.zeros(1, dtype=torch.int32, device=dev())
        table = case.table.clone()
        if bit == 4:
            table[:] = -1
        o.gemm_tc_rope(a, w, qkv, bad.to(torch.int32).to(dev()), tok_seq, case.seq_slot, table, cos_t, sin_t, case.kcache, case.vcache,
                       nh, nkv, hd, err)
        assert int(err.item()) == bit
    assert not o.gemm_tc_rope_takes(a, w, qkv, case.kcache, case.vcache, cos_t, sin_t, 32)


# ----------------------------------------------------------------------------- decode attention with RoPE and append fused
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 16), (9, 3, 64), (3, 1, 32), (12, 2, 128), (2, 2, 48)])
@pytest.mark.parametrize("n_splits", [1, 5])
def test_attn_decode_rope_equals_separate_kernels(dtype, nh, nkv, hd, n_splits):
    o = ops()
    lengths = [1, 64, 65, 300, 128, 37]          # the new token is the last of each: page edges on both sides
    B = len(lengths)
    max_pos = 400
    cos, sin = plain.rope_angles(np.arange(max_pos), hd, 5000.0)
    cos_t, sin_t = torch.from_numpy(cos).to(dev()), torch.from_numpy(sin).to(dev())
    a = PagedCase(o, dtype, lengths, nkv, hd, seed=nh + hd)
    b = PagedCase(o, dtype, lengths, nkv, hd, seed=nh + hd)   # the same cache twice
    raw = rnd((B, (nh + 2 * nkv) * hd), dtype, 90)
    seq_pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=dev())
    tok_seq = torch.arange(B, dtype=torch.int32, device=dev())
    err = torch.zeros(1, dtype=torch.int32, device=dev())
    mk = lambda: (torch.full((B * nh * n_splits * hd,), float("nan"), device=dev()), torch.full((B * nh * n_splits * 2,), float("nan"), device=dev()))
    # separate kernels: rotate + append, then attend
    q1 = raw.clone()
    o.rope_kv_append(q1, seq_pos, tok_seq, a.seq_slot, a.table, cos_t, sin_t, a.kcache, a.vcache, nh, nkv, hd, err)
    want = torch.zeros(B, nh * hd, dtype=dtype, device=dev())
    po, pm = mk()
    o.attn_decode(q1, want, a.kcache, a.vcache, a.table, a.seq_slot, seq_pos, B, nh, nkv, hd, 1.0 / math.sqrt(hd), n_splits, po, pm)
    # fused
    got = torch.full_like(want, float("nan"))
    po, pm = mk()
    o.attn_decode_rope(raw.clone(), got, b.kcache, b.vcache, b.table, b.seq_slot, seq_pos, cos_t, sin_t, B, nh, nkv, hd,
                       1.0 / math.sqrt(hd), n_splits, po, pm)
    assert int(err.item()) == 0
    assert rel_err(got, want) < (1e-6 if dtype == torch.float32 else 4e-3)
    # and against the plain implementation: rotate the new token's q and k, put k and v at the end, attend
    for s, n in enumerate(lengths):
        row = raw[s].float().cpu().numpy()
        vh = row[(nh + nkv) * hd:].reshape(1, nkv, hd)
        qr = torch.from_numpy(plain.rope(row[None, :nh * hd], [n - 1], nh, hd, 5000.0)).to(dtype).float()
        kr = torch.from_numpy(plain.rope(row[None, nh * hd:(nh + nkv) * hd], [n - 1], nkv, hd, 5000.0)).to(dtype).float().reshape(1, nkv, hd)
        keys = torch.cat([a.k[s][:n - 1], kr], dim=0)
        vals = torch.cat([a.v[s][:n - 1], torch.from_numpy(vh).to(dtype).float()], dim=0)
        ref = attention_rows(qr, keys, vals, n - 1, nh, nkv, hd)
        assert rel_err(got[s:s + 1], ref) < (1e-5 if dtype == torch.float32 else 1.2e-2), (s, n)
    for s, n in enumerate(lengths):   # the appended rows are the same, nothing else changed
        for cache_a, cache_b in ((a.kcache, b.kcache), (a.vcache, b.vcache)):
            page = int(a.table[int(a.seq_slot[s]), (n - 1) // o.PAGE])
            assert rel_err(cache_b[page, :, (n - 1) % o.PAGE], cache_a[page, :, (n - 1) % o.PAGE]) < (1e-6 if dtype == torch.float32 else 8e-3)
    same = torch.isclose(a.kcache.float(), b.kcache.float(), rtol=1e-2, atol=1e-2, equal_nan=True)
    assert bool(same.all())
