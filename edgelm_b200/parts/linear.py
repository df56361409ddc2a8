"""out = a . W^T with an epilogue, on the kernel that fits the sizes.

bfloat16 with enough rows goes to the tcgen05 tensor-core kernel (operands by TMA, accumulator
in tensor memory); everything else, and the whole float32 path, to the CUDA-core kernels.
Both take any M, N; the tensor-core kernel needs K to be a multiple of 8 (a TMA row pitch of
16 bytes) and falls back, not fails, when it is not.
"""
import torch

from ..csrc import ops

EPI_STORE, EPI_RESIDUAL, EPI_SWIGLU = ops.EPI_STORE, ops.EPI_RESIDUAL, ops.EPI_SWIGLU

TENSOR_CORE_MIN_ROWS = 17  # fewer rows: one pass over the weights on the CUDA cores is bandwidth-bound already


def matmul(ctx, a, w, out, epilogue=EPI_STORE, w2=None, residual=None):
    """`ctx` gives the device error word that the tensor-core kernel's bounded waits report to."""
    if a.dtype == torch.bfloat16 and a.shape[0] >= TENSOR_CORE_MIN_ROWS and ops.gemm_tc_takes(a, w, out, w2):
        ops.gemm_tc(a, w, out, ctx.err, epilogue=epilogue, w2=w2, residual=residual)
    else:
        ops.gemm_simt(a, w, out, epilogue=epilogue, w2=w2, residual=residual)
