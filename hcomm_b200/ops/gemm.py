"""bf16 GEMM on the hand-written tcgen05 / TMEM / TMA kernel (``csrc/device/gemm_sm100.cu``).

``gemm_bf16(a, b)`` computes ``a @ b.T`` for row-major ``a [M, K]`` and ``b [N, K]`` (the layout of a
``torch.nn.Linear`` weight), accumulating in fp32 and returning bf16.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _lib


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    if not (a.is_cuda and b.is_cuda):
        raise RuntimeError("gemm_bf16 runs on a CUDA device; the tcgen05 kernel has no CPU path")
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("gemm_bf16 expects bfloat16 operands")
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[1]:
        raise ValueError(f"shapes {tuple(a.shape)} x {tuple(b.shape)}^T do not match")
    if a.stride(1) != 1 or b.stride(1) != 1:
        raise ValueError("the K dimension must be contiguous in both operands")
    m, k = a.shape
    n = b.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
    lib = _lib.load()
    stream = torch.cuda.current_stream(a.device).cuda_stream
    with torch.cuda.device(a.device):
        rc = lib.HcommGemmBf16(ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(b.data_ptr()), ctypes.c_void_p(out.data_ptr()), m, n, k,
                               a.stride(0), b.stride(0), out.stride(0), ctypes.c_void_p(stream))
    _lib.check(rc, "HcommGemmBf16")
    return out


def take_kernel_error() -> int:
    """Non-zero when a bounded wait inside a GEMM kernel expired since the last call (clears the flag)."""
    return int(_lib.load().HcommGemmTakeError())
