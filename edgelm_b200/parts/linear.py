"""out = a . W^T with an epilogue, on the kernel that fits the sizes.

  rows <= 16        the few-rows kernels: weights streamed once, activations in shared memory, the
                    preceding RMSNorm computed in the prologue (`NormedInput`).  bfloat16 runs
                    on mma.sync tensor cores (gemv_mma.cu), float32 on the CUDA cores (gemv.cu);
  bfloat16, more    the tcgen05 tensor-core kernel (gemm_tc.cu): operands by TMA, accumulator in
                    tensor memory;
  anything else     the CUDA-core kernels of gemm_simt.cu: the whole float32 path for many rows,
                    and every size the other two do not take (K not a multiple of 8, unaligned rows).
"""
import os

import torch

from ..csrc import ops

EPI_STORE, EPI_RESIDUAL, EPI_SWIGLU = ops.EPI_STORE, ops.EPI_RESIDUAL, ops.EPI_SWIGLU

FEW_ROWS = 16  # up to here one pass over the weights with all rows in shared memory is bandwidth-bound already
MMA_MIN_ROWS = 1        # rows from which the tensor-core few-rows kernel is used (measured: never slower)
FUSE_NORM_MAX_WIDTH = 1024  # every block of a few-rows product recomputes a fused norm: worth it for narrow models only
MMA_WIDE_COLUMNS = 8192  # from here on (the vocabulary) the tensor-core kernel wins at any row count


def _few_rows_on_mma(rows, n_cols):
    return rows >= MMA_MIN_ROWS or n_cols >= MMA_WIDE_COLUMNS


class NormedInput:
    """A normalised input that may never be written out: `x` (the float32 residual stream) and the
    RMSNorm to apply.  A matrix product of few rows computes the norm in its own prologue; any
    other consumer calls `tensor()`, which runs the norm kernel once into the step's workspace."""

    def __init__(self, ctx, x, norm, dtype):
        self.ctx, self.x, self.norm, self.dtype = ctx, x, norm, dtype
        self._t = None
        self.shape = x.shape

    def tensor(self):
        if self._t is None:
            self._t = self.ctx.ws.alloc(tuple(self.x.shape), self.dtype)
            with self.ctx.prof("norm"):
                self.norm.forward(self.ctx, self.x, self._t)
        return self._t


def as_tensor(a):
    return a.tensor() if isinstance(a, NormedInput) else a


# Few-rows tensor-core products ask L2 for the weights the step reads next (EDGELM_PREFETCH_NEXT=0: not, for
# comparisons), if those are small: then the next product is a matter of latencies and finds its weights on the chip
# (decode steps of 8 sequences, 135M sizes: 0.877 -> 0.854 ms; 360M: 1.077 -> 1.070); weights of tens of megabytes
# are a matter of bandwidth, which the prefetch only takes from the running product (1.7B sizes: 2.01 -> 2.04 ms).
PREFETCH_NEXT = os.environ.get("EDGELM_PREFETCH_NEXT", "1") != "0"
PREFETCH_MAX_BYTES = 8 << 20


def matmul(ctx, a, w, out, epilogue=EPI_STORE, w2=None, residual=None, prefetch=()):
    """`a`: a tensor in the compute dtype or a NormedInput.  `ctx` gives the device error word that
    the tensor-core kernel's bounded waits report to.  `prefetch`: the weights that the step reads after
    this product (up to two tensors); the few-rows tensor-core kernel starts their way into L2, the other
    kernels ignore them."""
    prefetch = tuple(prefetch)[:2] if PREFETCH_NEXT and prefetch else ()
    if sum(t.numel() * t.element_size() for t in prefetch) > PREFETCH_MAX_BYTES:
        prefetch = ()
    rows = a.shape[0]
    if isinstance(a, NormedInput):
        if rows <= FEW_ROWS and a._t is None and a.x.shape[1] <= FUSE_NORM_MAX_WIDTH:
            if _few_rows_on_mma(rows, w.shape[0]) and ops.gemv_mma_takes(a.x, w, w2, normed=True):
                ops.gemv_mma(a.x, w, out, epilogue=epilogue, w2=w2, residual=residual, norm_weight=a.norm.weight, eps=a.norm.eps,
                             prefetch=prefetch)
                return
            if ops.gemv_takes(a.x, w, w2, normed=True):
                ops.gemv(a.x, w, out, epilogue=epilogue, w2=w2, residual=residual, norm_weight=a.norm.weight, eps=a.norm.eps,
                         n_sms=ctx.n_sms)
                return
        a = a.tensor()
    if rows <= FEW_ROWS and _few_rows_on_mma(rows, w.shape[0]) and ops.gemv_mma_takes(a, w, w2):
        ops.gemv_mma(a, w, out, epilogue=epilogue, w2=w2, residual=residual, prefetch=prefetch)
    elif rows <= FEW_ROWS and ops.gemv_takes(a, w, w2):
        ops.gemv(a, w, out, epilogue=epilogue, w2=w2, residual=residual, n_sms=ctx.n_sms)
    elif a.dtype == torch.bfloat16 and rows > FEW_ROWS and ops.gemm_tc_takes(a, w, out, w2):
        ops.gemm_tc(a, w, out, ctx.err, epilogue=epilogue, w2=w2, residual=residual)
    else:
        ops.gemm_simt(a, w, out, epilogue=epilogue, w2=w2, residual=residual)
