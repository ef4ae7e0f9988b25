"""Tensor-parallel GEMMs fused with their collective (``csrc/device/fused_gemm.cu``), and the unfused
cuBLAS + NCCL forms they are measured against.

    gemm_reduce_scatter(comm, a, b)   row-parallel linear:  rows r of  sum_q a_q @ b_q.T   on rank r
    all_gather_gemm(comm, x, w)       column-parallel linear:  concat_q(x_q) @ w.T
"""
from __future__ import annotations

import ctypes

import torch

from .. import _lib
from ..comm import Communicator


def _ptr(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr())


def _check(t: torch.Tensor, name: str):
    if not t.is_cuda or t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be a 2-D bfloat16 CUDA tensor with a contiguous last dimension")


def gemm_reduce_scatter(comm: Communicator, a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """a: [M, K_local], b: [N, K_local] (this rank's K slice).  Returns this rank's [M/size, N] rows of the summed product."""
    _check(a, "a"); _check(b, "b")
    m, k = a.shape
    n = b.shape[0]
    if b.shape[1] != k or m % comm.size:
        raise ValueError("shape mismatch")
    if out is None:
        out = torch.empty((m // comm.size, n), dtype=torch.bfloat16, device=a.device)
    stream = torch.cuda.current_stream(a.device).cuda_stream
    rc = _lib.load().HcommFusedGemmReduceScatterBf16(ctypes.c_void_p(comm.handle), _ptr(a), _ptr(b), _ptr(out), m, n, k, a.stride(0), b.stride(0),
                                                     out.stride(0), ctypes.c_void_p(stream))
    _lib.check(rc, "HcommFusedGemmReduceScatterBf16")
    return out


def all_gather_gemm(comm: Communicator, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """x: [M/size, K] (this rank's rows), w: [N_local, K].  Returns [M, N_local] = all_gather(x) @ w.T."""
    _check(x, "x"); _check(w, "w")
    ms, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or not x.is_contiguous():
        raise ValueError("shape mismatch or non-contiguous shard")
    if out is None:
        out = torch.empty((ms * comm.size, n), dtype=torch.bfloat16, device=x.device)
    stream = torch.cuda.current_stream(x.device).cuda_stream
    rc = _lib.load().HcommFusedAllGatherGemmBf16(ctypes.c_void_p(comm.handle), _ptr(x), _ptr(w), _ptr(out), ms, n, k, x.stride(0), w.stride(0),
                                                 out.stride(0), ctypes.c_void_p(stream))
    _lib.check(rc, "HcommFusedAllGatherGemmBf16")
    return out


# ---------------------------------------------------------------- unfused baselines (cuBLAS + NCCL)

def gemm_reduce_scatter_unfused(a: torch.Tensor, b: torch.Tensor, group=None) -> torch.Tensor:
    import torch.distributed as dist
    world = dist.get_world_size(group)
    full = torch.matmul(a, b.t())
    out = torch.empty((a.shape[0] // world, b.shape[0]), dtype=a.dtype, device=a.device)
    dist.reduce_scatter_tensor(out, full, group=group)
    return out


def all_gather_gemm_unfused(x: torch.Tensor, w: torch.Tensor, group=None) -> torch.Tensor:
    import torch.distributed as dist
    world = dist.get_world_size(group)
    full = torch.empty((x.shape[0] * world, x.shape[1]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(full, x, group=group)
    return torch.matmul(full, w.t())
