"""`quant_linear_cuda` stand-in: same function name and argument list as the reference binding
(csrc/linear/quant_linear.cpp:6-24)."""
import torch

from .. import ops


def w4a16o16_gemm(A, B, s, workspace, size_m, size_n, size_k, output_transpose=False,
                  thread_k=-1, thread_n=-1, sms=-1, max_par=8):
    """Returns fp16 [size_m, size_n] = A[size_m, size_k] @ dequant(B, s).

    `workspace`, `thread_k`, `thread_n`, `sms` and `max_par` tuned the reference kernel's tiling and
    locking; they are accepted and ignored.  Error behaviour follows the reference host wrapper
    (csrc/linear/marlin_gemm_kernel.cuh:1008-1012, 1048-1050): RuntimeError on shape problems."""
    if output_transpose:
        raise RuntimeError("output_transpose=True is not supported (the reference's Python layer never sets it)")
    if A.dim() != 2 or A.shape[0] != size_m or A.shape[1] != size_k:
        raise RuntimeError(f"A must be [size_m={size_m}, size_k={size_k}], got {tuple(A.shape)}")
    if B.shape[0] * 16 != size_k or B.shape[1] != size_n * 2:
        raise RuntimeError(f"B must be [size_k/16={size_k // 16}, size_n*2={size_n * 2}], got {tuple(B.shape)}")
    if s.shape[1] != size_n:
        raise RuntimeError("s must have size_n columns")
    if workspace is not None and workspace.numel() < size_n // 128 * max_par:
        raise RuntimeError(f"workspace must be of size at least {size_n // 128 * max_par}")
    return ops.w4a16_linear(A, B, s, None, size_n)
