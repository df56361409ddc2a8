"""Python face of the kernel library: torch tensors in, kernel launches on the current stream.

Each function checks dtypes, shapes and contiguity, passes raw device pointers through
ctypes, and raises `KernelError` with the library's message when a size is refused or a
launch fails.  Nothing here computes on the host or falls back to another implementation:
without the library, or without a device of compute capability 10.x, importing the ops
raises.
"""
import ctypes
import os
import threading

import torch

from . import build as _build

F32, BF16 = 0, 1
EPI_STORE, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2
PAGE = 64  # tokens per cache page, as in common.cuh

ERR_BITS = {1: "a token id outside the vocabulary", 2: "a position beyond the position table",
            4: "a page id outside the cache", 8: "a device-side wait ran out"}


class KernelError(RuntimeError):
    pass


_lib = None
_lock = threading.Lock()


def lib():
    """The loaded kernel library (built at the first call if needed)."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                path = _build.library_path()
                try:
                    loaded = ctypes.CDLL(path)
                except OSError as e:  # pragma: no cover
                    raise KernelError(f"edgelm_b200: cannot load the kernel library {path}: {e}") from e
                loaded.edgelm_last_error.restype = ctypes.c_char_p
                if os.environ.get("EDGELM_PDL") is not None:
                    loaded.edgelm_set_pdl(int(os.environ["EDGELM_PDL"]))
                _lib = loaded
    return _lib


def require_device():
    """Fail loudly unless a Blackwell-class CUDA device is current; there is no other path."""
    if not torch.cuda.is_available():
        raise KernelError("edgelm_b200 runs on a CUDA device (sm_100a) only; torch sees none")
    arch = lib().edgelm_device_arch()
    if arch // 10 != 10:
        raise KernelError(f"edgelm_b200's kernels are built for sm_100a; the current device reports sm_{arch}")


LAUNCHES = 0  # kernels launched through this module since import (a graph replay counts what it captured)


def count_launches(n):
    global LAUNCHES
    LAUNCHES += n


def _check(rc, launches=1):
    if rc != 0:
        raise KernelError(lib().edgelm_last_error().decode())
    count_launches(launches)


def _dt(t):
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported dtype {t.dtype}")


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(cond, msg):
    if not cond:
        raise KernelError(msg)


def _i32(t, name):
    _need(t.dtype == torch.int32 and t.is_cuda and t.is_contiguous(), f"{name} must be a contiguous int32 CUDA tensor")


def embed_gather(ids, table, x, err):
    """x[t, :] = table[ids[t], :] as float32; ids outside the table set bit 1 of `err`."""
    _i32(ids, "ids")
    _need(table.dim() == 2 and table.is_contiguous() and x.dtype == torch.float32 and x.is_contiguous(), "embed_gather: layout")
    _need(x.shape == (ids.numel(), table.shape[1]), "embed_gather: x has the wrong shape")
    _check(lib().edgelm_embed_gather(_p(ids), _p(table), _dt(table), _p(x), ids.numel(), table.shape[1], table.shape[0],
                                     _p(err), _stream()))


def rmsnorm(x, w, eps, out, rows_idx=None):
    """out[r] = x[rows_idx[r] or r] * rsqrt(mean(x^2) + eps) * w; x and w float32, out float32 or bfloat16."""
    _need(x.dtype == torch.float32 and w.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous(), "rmsnorm: layout")
    rows = out.shape[0]
    dim = x.shape[1]
    _need(out.shape[1] == dim and w.numel() == dim, "rmsnorm: widths differ")
    if rows_idx is not None:
        _i32(rows_idx, "rows_idx")
        _need(rows_idx.numel() == rows, "rmsnorm: one source row per output row")
    else:
        _need(x.shape[0] == rows, "rmsnorm: row counts differ")
    _check(lib().edgelm_rmsnorm(_p(x), _p(w), _p(out), _dt(out), _p(rows_idx), rows, dim, ctypes.c_float(eps), _stream()))


def gemm_simt(a, w, out, epilogue=EPI_STORE, w2=None, residual=None, force_kernel=0):
    """out = a @ w.T (+ epilogue) with float32 accumulation on the CUDA cores."""
    _need(a.dim() == 2 and w.dim() == 2 and out.dim() == 2, "gemm: 2-D operands")
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N), f"gemm: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    _need(a.stride(1) == 1 and out.stride(1) == 1 and w.is_contiguous(), "gemm: rows must be contiguous")
    _need(a.dtype == w.dtype and (w2 is None or (w2.dtype == w.dtype and w2.shape == w.shape and w2.is_contiguous())), "gemm: weight dtypes")
    if residual is not None:
        _need(residual.dtype == torch.float32 and residual.shape == out.shape and residual.stride() == out.stride(), "gemm: residual layout")
    _check(lib().edgelm_gemm_simt(_p(a), a.stride(0), _p(w), _p(w2), _p(out), out.stride(0), _p(residual), M, N, K,
                                  _dt(a), _dt(out), epilogue, force_kernel, _stream()))


def gemv_takes(a, w, w2=None, normed=False):
    """Whether the vector few-rows kernel takes these operands (K a multiple of a 16-byte vector, aligned rows).
    With `normed`, `a` is the float32 residual stream and the weights give the compute dtype."""
    if not w.is_contiguous() or a.stride(1) != 1:
        return False
    if normed and (a.dtype != torch.float32 or not a.is_contiguous()):
        return False
    if not normed and a.dtype != w.dtype:
        return False
    return bool(lib().edgelm_gemv_takes(_p(a), a.stride(0), _p(w), _p(w2), a.shape[1], _dt(w), 1 if normed else 0))


def gemv(a, w, out, epilogue=EPI_STORE, w2=None, residual=None, norm_weight=None, eps=0.0, n_sms=0):
    """out = act @ w.T (+ epilogue) for a few rows.  act = a, or RMSNorm(a) * norm_weight rounded to
    w's dtype when norm_weight is given (a is then the float32 residual stream)."""
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N), f"gemv: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    _need(out.stride(1) == 1 and w.is_contiguous(), "gemv: rows must be contiguous")
    _need(w2 is None or (w2.dtype == w.dtype and w2.shape == w.shape and w2.is_contiguous()), "gemv: second weight")
    if norm_weight is not None:
        _need(a.dtype == torch.float32 and a.is_contiguous() and norm_weight.dtype == torch.float32 and norm_weight.numel() == K, "gemv: norm operands")
    else:
        _need(a.dtype == w.dtype and a.stride(1) == 1, "gemv: activation dtype")
    if residual is not None:
        _need(residual.dtype == torch.float32 and residual.shape == out.shape and residual.stride() == out.stride(), "gemv: residual layout")
    _check(lib().edgelm_gemv(_p(a), a.stride(0), _p(norm_weight), ctypes.c_float(eps), _p(w), _p(w2), _p(out), out.stride(0),
                             _p(residual), M, N, K, _dt(w), _dt(out), epilogue, int(n_sms), _stream()))


def gemv_mma_takes(a, w, w2=None, normed=False):
    """Whether the tensor-core few-rows kernel takes these operands: bfloat16 weights, at most 16 rows,
    K a multiple of 8, aligned rows.  With `normed`, `a` is the float32 residual stream."""
    if w.dtype != torch.bfloat16 or not w.is_contiguous() or a.stride(1) != 1:
        return False
    if normed and (a.dtype != torch.float32 or not a.is_contiguous()):
        return False
    if not normed and a.dtype != torch.bfloat16:
        return False
    return bool(lib().edgelm_gemv_mma_takes(_p(a), a.stride(0), _p(w), _p(w2), a.shape[0], a.shape[1], 1 if normed else 0))


def gemv_mma(a, w, out, epilogue=EPI_STORE, w2=None, residual=None, norm_weight=None, eps=0.0, prefetch=()):
    """out = act @ w.T (+ epilogue) for at most 16 rows on mma.sync tensor cores; act = a, or
    RMSNorm(a) * norm_weight rounded to bfloat16 when norm_weight is given.  `prefetch`: up to two
    contiguous tensors (the weights the step reads next) that the kernel's blocks ask the L2 cache for."""
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N), f"gemv_mma: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    _need(out.stride(1) == 1 and w.is_contiguous() and w.dtype == torch.bfloat16, "gemv_mma: weight layout")
    _need(w2 is None or (w2.dtype == w.dtype and w2.shape == w.shape and w2.is_contiguous()), "gemv_mma: second weight")
    if norm_weight is not None:
        _need(a.dtype == torch.float32 and a.is_contiguous() and norm_weight.dtype == torch.float32 and norm_weight.numel() == K, "gemv_mma: norm operands")
    else:
        _need(a.dtype == torch.bfloat16 and a.stride(1) == 1, "gemv_mma: activation dtype")
    if residual is not None:
        _need(residual.dtype == torch.float32 and residual.shape == out.shape and residual.stride() == out.stride(), "gemv_mma: residual layout")
    if prefetch:
        _need(len(prefetch) <= 2 and all(t.is_contiguous() for t in prefetch), "gemv_mma: prefetch takes up to two contiguous tensors")
        regions = [(_p(t), ctypes.c_ulonglong(t.numel() * t.element_size())) for t in prefetch] + [(ctypes.c_void_p(0), ctypes.c_ulonglong(0))]
        _check(lib().edgelm_gemv_mma_prefetch_next(regions[0][0], regions[0][1], regions[1][0], regions[1][1]), launches=0)
    _check(lib().edgelm_gemv_mma(_p(a), a.stride(0), _p(norm_weight), ctypes.c_float(eps), _p(w), _p(w2), _p(out), out.stride(0),
                                 _p(residual), M, N, K, _dt(out), epilogue, _stream()))


def gemv_mma_walk(on):
    """Whether few-rows products with wide outputs (at least 296 groups of 16 columns, K up to 4,096) run on the
    kernel whose blocks walk several column groups (default) or on the one of a block per group."""
    lib().edgelm_gemv_mma_walk(int(bool(on)))


def gemm_tc_takes(a, w, out, w2=None):
    """Whether the tensor-core kernel takes these operands: bfloat16, K a multiple of 8, 16-byte aligned rows."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.stride(1) != 1 or not w.is_contiguous():
        return False
    return bool(lib().edgelm_gemm_tc_takes(_p(a), a.stride(0), _p(w), _p(w2), a.shape[1]))


SPLITK_SCRATCH_BYTES = 32 << 20
_splitk_scratch = None


def _splitk_ready():
    """The scratch that lets products of few tiles and long K spread over the device (split-K): allocated once, at
    the first product outside of a graph capture, and handed to the library."""
    global _splitk_scratch
    if _splitk_scratch is None and not torch.cuda.is_current_stream_capturing():
        _splitk_scratch = torch.empty(SPLITK_SCRATCH_BYTES // 4, dtype=torch.float32, device="cuda")
        lib().edgelm_gemm_tc_splitk.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
        lib().edgelm_gemm_tc_splitk(_p(_splitk_scratch), SPLITK_SCRATCH_BYTES, 1)


def gemm_tc(a, w, out, err, epilogue=EPI_STORE, w2=None, residual=None):
    """out = a @ w.T (+ epilogue) on the tcgen05 tensor cores: bfloat16 operands, float32 accumulation."""
    _splitk_ready()
    _need(a.dim() == 2 and w.dim() == 2 and out.dim() == 2, "gemm_tc: 2-D operands")
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N), f"gemm_tc: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    _need(a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "gemm_tc: bfloat16 operands")
    _need(a.stride(1) == 1 and out.stride(1) == 1 and w.is_contiguous(), "gemm_tc: rows must be contiguous")
    _need(w2 is None or (w2.dtype == w.dtype and w2.shape == w.shape and w2.is_contiguous()), "gemm_tc: second weight")
    if residual is not None:
        _need(residual.dtype == torch.float32 and residual.shape == out.shape and residual.stride() == out.stride(), "gemm_tc: residual layout")
    _check(lib().edgelm_gemm_tc(_p(a), a.stride(0), _p(w), _p(w2), _p(out), out.stride(0), _p(residual), M, N, K, _dt(out),
                                epilogue, _p(err), _stream()), launches=0)
    count_launches(lib().edgelm_gemm_tc_last_launches())


def gemm_tc_rope_takes(a, w, qkv, kcache, vcache, cos, sin, hd):
    """Whether the stacked q, k, v projection can rotate and append in its epilogue (`gemm_tc_rope`)."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or qkv.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16:
        return False
    if a.stride(1) != 1 or qkv.stride(1) != 1 or not w.is_contiguous() or not (kcache.is_contiguous() and vcache.is_contiguous()):
        return False
    return bool(lib().edgelm_gemm_tc_rope_takes(_p(a), a.stride(0), _p(w), _p(qkv), qkv.stride(0), a.shape[1], int(hd),
                                                _p(kcache), _p(vcache), _p(cos), _p(sin)))


def gemm_tc_rope(a, w, qkv, tok_pos, tok_seq, seq_slot, page_table, cos, sin, kcache, vcache, nh, nkv, hd, err):
    """The stacked q, k, v projection of a prompt step with rotation and cache append in its epilogue:
    qkv[:, :nh hd] = rotated query heads of a @ w.T; the rotated keys and the values go to each token's place in the
    cache pages.  The k and v columns of `qkv` are left as they were."""
    _splitk_ready()
    M, K = a.shape
    _need(w.shape == ((nh + 2 * nkv) * hd, K) and qkv.shape == (M, (nh + 2 * nkv) * hd), "gemm_tc_rope: shapes")
    _need(gemm_tc_rope_takes(a, w, qkv, kcache, vcache, cos, sin, hd), "gemm_tc_rope: these operands are not taken (bfloat16, head size 64 or 128, aligned)")
    _need(kcache.shape[1:] == (nkv, PAGE, hd) and vcache.shape == kcache.shape, "gemm_tc_rope: cache layout")
    _need(cos.dtype == torch.float32 and cos.shape[1] == hd // 2 and cos.is_contiguous() and sin.shape == cos.shape and sin.is_contiguous(), "gemm_tc_rope: table layout")
    for t, n in ((tok_pos, "tok_pos"), (tok_seq, "tok_seq"), (seq_slot, "seq_slot"), (page_table, "page_table")):
        _i32(t, n)
    _need(tok_pos.numel() == M and tok_seq.numel() == M, "gemm_tc_rope: one position and one sequence index per token")
    _check(lib().edgelm_gemm_tc_rope(_p(a), a.stride(0), _p(w), _p(qkv), qkv.stride(0), M, K, _p(tok_pos), _p(tok_seq), _p(seq_slot),
                                     _p(page_table), page_table.stride(0), kcache.shape[0], _p(cos), _p(sin), cos.shape[0],
                                     _p(kcache), _p(vcache), nh, nkv, hd, _p(err), _stream()), launches=0)
    count_launches(lib().edgelm_gemm_tc_last_launches())


def gemm_tc_last_kernel():
    """Which kernel the last `gemm_tc` call took: {"tile_columns", "persistent", "deep_ring", "k_splits"}."""
    v = int(lib().edgelm_gemm_tc_last_kernel())
    return {"tile_columns": v & 0xFFF, "persistent": bool(v >> 12 & 1), "deep_ring": bool(v >> 13 & 1), "k_splits": v >> 16}


def rope_kv_append(qkv, tok_pos, tok_seq, seq_slot, page_table, cos, sin, kcache, vcache, nh, nkv, hd, err):
    """Rotate q and k of the fused projection output in float32; write k and v into their pages."""
    T = qkv.shape[0]
    _need(qkv.is_contiguous() and qkv.shape[1] == (nh + 2 * nkv) * hd, "rope_kv_append: qkv layout")
    _need(kcache.dtype == qkv.dtype and vcache.dtype == qkv.dtype and kcache.is_contiguous() and vcache.is_contiguous(), "rope_kv_append: cache dtype")
    _need(kcache.shape[1:] == (nkv, PAGE, hd) and vcache.shape == kcache.shape, "rope_kv_append: cache shape")
    _need(cos.dtype == torch.float32 and cos.shape[1] == hd // 2 and cos.is_contiguous() and sin.shape == cos.shape and sin.is_contiguous(), "rope_kv_append: table layout")
    for t, n in ((tok_pos, "tok_pos"), (tok_seq, "tok_seq"), (seq_slot, "seq_slot"), (page_table, "page_table")):
        _i32(t, n)
    _need(tok_pos.numel() >= T and tok_seq.numel() >= T, "rope_kv_append: one position per token")
    _check(lib().edgelm_rope_kv_append(_p(qkv), _dt(qkv), _p(tok_pos), _p(tok_seq), _p(seq_slot), _p(page_table),
                                       page_table.stride(0), kcache.shape[0], _p(cos), _p(sin), cos.shape[0], _p(kcache),
                                       _p(vcache), T, nh, nkv, hd, _p(err), _stream()))


def attn_prefill(qkv, out, kcache, vcache, page_table, seq_slot, tile_seq, tile_tok0, tile_ntok, tile_pos0, n_tiles,
                 max_tile_tokens, nh, nkv, hd, scale, window=0):
    """Causal attention of new tokens (any number per sequence) over the paged cache.  `window` > 0: a token sees
    the last `window` keys only, its own included."""
    _need(qkv.dtype == out.dtype == kcache.dtype and qkv.stride(1) == 1 and out.stride(1) == 1, "attn_prefill: layout")
    for t, n in ((page_table, "page_table"), (seq_slot, "seq_slot"), (tile_seq, "tile_seq"), (tile_tok0, "tile_tok0"),
                 (tile_ntok, "tile_ntok"), (tile_pos0, "tile_pos0")):
        _i32(t, n)
    _check(lib().edgelm_attn_prefill(_p(qkv), qkv.stride(0), _p(out), out.stride(0), _p(kcache), _p(vcache), _dt(qkv),
                                     _p(page_table), page_table.stride(0), _p(seq_slot), _p(tile_seq), _p(tile_tok0),
                                     _p(tile_ntok), _p(tile_pos0), n_tiles, max_tile_tokens, nh, nkv, hd,
                                     ctypes.c_float(scale), int(window or 0), _stream()))


MMA_PREFILL_TILE = 64  # new tokens per tile of the tensor-core prefill kernel (PM_ROWS in attention_mma.cu)


def attn_prefill_mma_takes(dtype, hd):
    """Whether the tensor-core prefill attention takes this dtype and head size (bfloat16; 32, 64, 96, 128)."""
    return dtype == torch.bfloat16 and bool(lib().edgelm_attn_prefill_mma_takes(int(hd)))


def attn_prefill_mma(qkv, out, kcache, vcache, page_table, seq_slot, tile_seq, tile_tok0, tile_ntok, tile_pos0, n_tiles,
                     nh, nkv, hd, scale, max_keys=0, force_groups=0):
    """Causal attention of new tokens over the paged cache on mma.sync tensor cores; tiles of at most 64 tokens."""
    _need(qkv.dtype == out.dtype == kcache.dtype == torch.bfloat16 and qkv.stride(1) == 1 and out.stride(1) == 1, "attn_prefill_mma: layout")
    for t, n in ((page_table, "page_table"), (seq_slot, "seq_slot"), (tile_seq, "tile_seq"), (tile_tok0, "tile_tok0"),
                 (tile_ntok, "tile_ntok"), (tile_pos0, "tile_pos0")):
        _i32(t, n)
    _check(lib().edgelm_attn_prefill_mma(_p(qkv), qkv.stride(0), _p(out), out.stride(0), _p(kcache), _p(vcache),
                                         _p(page_table), page_table.stride(0), _p(seq_slot), _p(tile_seq), _p(tile_tok0),
                                         _p(tile_ntok), _p(tile_pos0), n_tiles, nh, nkv, hd, ctypes.c_float(scale), int(max_keys),
                                         int(force_groups), _stream()))


TC_PREFILL_TILE = 128  # new tokens per tile of the tcgen05 prefill kernel (AT_ROWS in attention_tc.cu)


def attn_prefill_tc_takes(dtype, hd):
    """Whether the tcgen05 prefill attention takes this dtype and head size (bfloat16, 64)."""
    return dtype == torch.bfloat16 and bool(lib().edgelm_attn_prefill_tc_takes(int(hd)))


def attn_prefill_tc(qkv, out, kcache, vcache, page_table, seq_slot, tile_seq, tile_tok0, tile_ntok, tile_pos0, n_tiles,
                    nh, nkv, hd, scale, err):
    """Causal attention of new tokens over the paged cache on tcgen05 tensor cores; tiles of at most 128 tokens."""
    _need(qkv.dtype == out.dtype == kcache.dtype == torch.bfloat16 and qkv.stride(1) == 1 and out.stride(1) == 1, "attn_prefill_tc: layout")
    _need(kcache.is_contiguous() and vcache.is_contiguous() and kcache.shape[1:] == (nkv, PAGE, hd) and vcache.shape == kcache.shape, "attn_prefill_tc: cache layout")
    for t, n in ((page_table, "page_table"), (seq_slot, "seq_slot"), (tile_seq, "tile_seq"), (tile_tok0, "tile_tok0"),
                 (tile_ntok, "tile_ntok"), (tile_pos0, "tile_pos0")):
        _i32(t, n)
    _check(lib().edgelm_attn_prefill_tc(_p(qkv), qkv.stride(0), qkv.shape[0], _p(out), out.stride(0), _p(kcache), _p(vcache),
                                        kcache.shape[0], _p(page_table), page_table.stride(0), _p(seq_slot), _p(tile_seq),
                                        _p(tile_tok0), _p(tile_ntok), _p(tile_pos0), n_tiles, nh, nkv, hd, ctypes.c_float(scale),
                                        _p(err), _stream()))


ATTN_PREFILL_TC_TRACE_SHAPE = (2 * 64 + 1, 8)


def attn_prefill_tc_trace(buffer):
    """The next launches of the tcgen05 prefill attention stamp the clock of one softmax warp per group of the
    grid's first block into `buffer` (int64, ATTN_PREFILL_TC_TRACE_SHAPE: [group * 64 + block][before / after the
    wait for the scores, after the exponentials, after the wait for the last P V, after a rescaling, after the
    arrival], and a last row for the block as a whole: entry, tensor memory there, the kernel before done, key
    blocks done, accumulator read, row stored, block done); None stops it."""
    if buffer is not None:
        _need(buffer.dtype == torch.int64 and buffer.is_contiguous() and tuple(buffer.shape) == ATTN_PREFILL_TC_TRACE_SHAPE, "attn_prefill_tc_trace: buffer")
    lib().edgelm_attn_prefill_tc_trace(_p(buffer))


def attn_decode(qkv, out, kcache, vcache, page_table, seq_slot, seq_pos, n_seqs, nh, nkv, hd, scale, n_splits=1,
                part_o=None, part_ml=None, err=None, window=0, meta_ready=False):
    """Attention of one new token per sequence over the paged cache, pages dealt to `n_splits` blocks.
    `err`: the device error word that a copy which never arrives is reported to.  `window` > 0: the token sees the
    last `window` keys only (the CUDA-core kernel then, whatever the dtype).  `meta_ready`: the caller vouches that
    positions, slots and page table were complete before the kernel that precedes this call on the stream started."""
    _need(qkv.dtype == out.dtype == kcache.dtype and qkv.stride(1) == 1 and out.stride(1) == 1, "attn_decode: layout")
    for t, n in ((page_table, "page_table"), (seq_slot, "seq_slot"), (seq_pos, "seq_pos")):
        _i32(t, n)
    if n_splits > 1:
        _need(part_o is not None and part_o.dtype == torch.float32 and part_o.numel() >= n_seqs * nh * n_splits * hd, "attn_decode: part_o too small")
        _need(part_ml is not None and part_ml.dtype == torch.float32 and part_ml.numel() >= n_seqs * nh * n_splits * 2, "attn_decode: part_ml too small")
    _check(lib().edgelm_attn_decode(_p(qkv), qkv.stride(0), _p(out), out.stride(0), _p(kcache), _p(vcache), _dt(qkv),
                                    _p(page_table), page_table.stride(0), _p(seq_slot), _p(seq_pos), n_seqs, nh, nkv, hd,
                                    ctypes.c_float(scale), n_splits, _p(part_o), _p(part_ml), int(window or 0), 1 if meta_ready else 0,
                                    _p(err), _stream()),
           launches=0)
    count_launches(lib().edgelm_attn_decode_last_launches())


def attn_decode_rope(qkv, out, kcache, vcache, page_table, seq_slot, seq_pos, cos, sin, n_seqs, nh, nkv, hd, scale,
                     n_splits=1, part_o=None, part_ml=None, err=None, window=0, meta_ready=False):
    """Decode attention with RoPE and the cache append fused in: `qkv` holds the raw projections of one
    new token per sequence; the rotated keys and the values are written into the cache pages."""
    _need(qkv.dtype == out.dtype == kcache.dtype and qkv.stride(1) == 1 and out.stride(1) == 1, "attn_decode_rope: layout")
    _need(qkv.shape[1] == (nh + 2 * nkv) * hd and kcache.shape[1:] == (nkv, PAGE, hd) and vcache.shape == kcache.shape, "attn_decode_rope: shapes")
    _need(cos.dtype == torch.float32 and cos.shape[1] == hd // 2 and cos.is_contiguous() and sin.shape == cos.shape and sin.is_contiguous(), "attn_decode_rope: table layout")
    for t, n in ((page_table, "page_table"), (seq_slot, "seq_slot"), (seq_pos, "seq_pos")):
        _i32(t, n)
    if n_splits > 1:
        _need(part_o is not None and part_o.dtype == torch.float32 and part_o.numel() >= n_seqs * nh * n_splits * hd, "attn_decode_rope: part_o too small")
        _need(part_ml is not None and part_ml.dtype == torch.float32 and part_ml.numel() >= n_seqs * nh * n_splits * 2, "attn_decode_rope: part_ml too small")
    _check(lib().edgelm_attn_decode_rope(_p(qkv), qkv.stride(0), _p(out), out.stride(0), _p(kcache), _p(vcache), _dt(qkv),
                                         _p(page_table), page_table.stride(0), _p(seq_slot), _p(seq_pos), _p(cos), _p(sin),
                                         cos.shape[0], n_seqs, nh, nkv, hd, ctypes.c_float(scale), n_splits, _p(part_o),
                                         _p(part_ml), int(window or 0), 1 if meta_ready else 0, _p(err), _stream()),
           launches=0)
    count_launches(lib().edgelm_attn_decode_last_launches())


def attn_set_error_word(err):
    """The device int32 that decode attention calls which name no error word of their own (the entry point that
    allocates nothing) report a copy that never arrived to (bit 8)."""
    _check(lib().edgelm_attn_set_error_word(_p(err)), launches=0)


def argmax_rows(logits, out):
    """out[r] = index of the first maximum of logits[r]."""
    _need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1, "argmax_rows: float32 rows")
    _i32(out, "out")
    _check(lib().edgelm_argmax_rows(_p(logits), logits.stride(0), logits.shape[0], logits.shape[1], _p(out), _stream()))


def sample_topk(logits, temperature, top_k, rng_state, out, state_index=None, scratch=None):
    """Temperature + top-k draw per row; rng_state (int64 xorshift64 states) advances by one draw.
    Row r uses state state_index[r] when given (a sequence's slot), else state r.  `scratch` (int32, a word per
    row) lets rows with at most 1,024 kept tokens and a vocabulary of at most 49,152 take the fast kernel (the row
    in registers, no histograms); without it every row takes the general one.  Same choices either way."""
    if scratch is not None:
        _i32(scratch, "scratch")
        _need(scratch.numel() >= logits.shape[0], "sample_topk: a scratch word per row")
    _need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1, "sample_topk: float32 rows")
    _need(rng_state.dtype == torch.int64 and rng_state.is_contiguous(), "sample_topk: rng_state")
    if state_index is None:
        _need(rng_state.numel() >= logits.shape[0], "sample_topk: one state per row")
    else:
        _i32(state_index, "state_index")
    _i32(out, "out")
    _check(lib().edgelm_sample_topk(_p(logits), logits.stride(0), logits.shape[0], logits.shape[1],
                                    ctypes.c_float(temperature), int(top_k), _p(rng_state), _p(state_index), _p(out),
                                    _p(scratch), _stream()), launches=1 if scratch is None else 2)


def read_error_word(err):
    """Host-side reading of the device error word; raises when a kernel reported bad input."""
    v = int(err.item())
    if v:
        what = [m for b, m in ERR_BITS.items() if v & b]
        err.zero_()
        raise KernelError("a kernel reported: " + "; ".join(what))

