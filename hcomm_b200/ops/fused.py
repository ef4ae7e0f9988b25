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


MODES = {"auto": 0, "fused": 1, "split": 2}


def gemm_reduce_scatter(comm: Communicator, a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, mode: str = "auto") -> torch.Tensor:
    """a: [M, K_local], b: [N, K_local] (this rank's K slice).  Returns this rank's [M/size, N] rows of the summed product.

    mode: "fused" = one kernel, "split" = the library's GEMM followed by its reduce-scatter kernel, "auto" = the library's choice."""
    _check(a, "a"); _check(b, "b")
    m, k = a.shape
    n = b.shape[0]
    if b.shape[1] != k or m % comm.size:
        raise ValueError("shape mismatch")
    if out is None:
        out = torch.empty((m // comm.size, n), dtype=torch.bfloat16, device=a.device)
    stream = torch.cuda.current_stream(a.device).cuda_stream
    rc = _lib.load().HcommFusedGemmReduceScatterBf16Mode(ctypes.c_void_p(comm.handle), _ptr(a), _ptr(b), _ptr(out), m, n, k, a.stride(0), b.stride(0),
                                                         out.stride(0), ctypes.c_void_p(stream), MODES[mode])
    _lib.check(rc, "HcommFusedGemmReduceScatterBf16")
    return out


def all_gather_gemm(comm: Communicator, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None, mode: str = "auto") -> torch.Tensor:
    """x: [M/size, K] (this rank's rows), w: [N_local, K].  Returns [M, N_local] = all_gather(x) @ w.T.

    mode: "fused" = one kernel, "split" = a push kernel on the whole GPU followed by the GEMM, "auto" = the library's choice."""
    _check(x, "x"); _check(w, "w")
    ms, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or not x.is_contiguous():
        raise ValueError("shape mismatch or non-contiguous shard")
    if out is None:
        out = torch.empty((ms * comm.size, n), dtype=torch.bfloat16, device=x.device)
    stream = torch.cuda.current_stream(x.device).cuda_stream
    rc = _lib.load().HcommFusedAllGatherGemmBf16Mode(ctypes.c_void_p(comm.handle), _ptr(x), _ptr(w), _ptr(out), ms, n, k, x.stride(0), w.stride(0),
                                                     out.stride(0), ctypes.c_void_p(stream), MODES[mode])
    _lib.check(rc, "HcommFusedAllGatherGemmBf16")
    return out


PHASES = ("start", "end", "gate_wait", "acc_wait", "tile_wait", "push_busy", "push_end", "signal")


def set_phase_clocks(comm: Communicator, on: bool = True) -> None:
    """Makes the CTA-pair fused kernels record per-CTA phase clocks (see ``include/hcomm_fused.h``)."""
    _lib.check(_lib.load().HcommFusedSetPhaseClocks(ctypes.c_void_p(comm.handle), int(on)), "HcommFusedSetPhaseClocks")


def phase_clocks(comm: Communicator) -> dict:
    """Summary, in microseconds, of the phase clocks of the most recent fused call (synchronise its stream first):
    kernel span over all CTAs and, per waiting / working phase, the minimum, median and maximum over CTAs."""
    import numpy as np
    words = np.zeros((320, len(PHASES)), dtype=np.uint64)
    ctas = ctypes.c_int(0)
    _lib.check(_lib.load().HcommFusedGetPhaseClocks(ctypes.c_void_p(comm.handle), words.ctypes.data_as(ctypes.c_void_p), words.shape[0], ctypes.byref(ctas)),
               "HcommFusedGetPhaseClocks")
    w = words[:ctas.value].astype(np.int64)
    if not len(w):
        return {}
    t0 = int(w[:, 0].min())
    out = {"ctas": int(ctas.value), "span_us": (int(w[:, 1].max()) - t0) / 1e3, "first_cta_end_us": (int(w[:, 1].min()) - t0) / 1e3,
           "start_skew_us": (int(w[:, 0].max()) - t0) / 1e3}
    for i, name in enumerate(PHASES[2:], start=2):
        col = w[:, i]
        if name == "push_end":
            col = np.where(col > 0, col - t0, 0)
        out[name + "_us"] = {"min": float(col.min()) / 1e3, "median": float(np.median(col)) / 1e3, "max": float(col.max()) / 1e3}
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
