"""Small, self-terminating workloads for kernel profilers (one GPU, one process).

    python -m hcomm_b200.utils.profile_cases gemm            tcgen05 GEMM 8192^3 bf16 (operands larger than L2)
    python -m hcomm_b200.utils.profile_cases gemm_up         the benchmark's up projection 8192 x 28672 x 8192: this library's GEMM twice, then cuBLAS twice
    python -m hcomm_b200.utils.profile_cases gemm_raster      both benchmark projections once per (tile width 512 / 256, rasterisation group) pair, for counter sweeps
    python -m hcomm_b200.utils.profile_cases fused           GEMM->ReduceScatter and AllGather->GEMM, two ranks sharing the GPU
    python -m hcomm_b200.utils.profile_cases allreduce       one-shot, two-shot all-reduce and all-gather kernels, two ranks sharing the GPU
    python -m hcomm_b200.utils.profile_cases fused_pair      the CTA-pair variants of the two fused kernels on a one-rank communicator
    python -m hcomm_b200.utils.profile_cases moe             MoE dispatch + combine, one rank (256 experts, top-8, hidden 7168)

Ranks that share the GPU run inside ONE cooperative launch (kernels that wait for each other are never separate
launches on a GPU), so each case is a single process a profiler can wrap.  A few launches per kernel, a few hundred
MB on the device at most.
"""
from __future__ import annotations

import sys
import threading

import torch


def _ranks(n, fn):
    errs = []

    def wrap(r):
        try:
            torch.cuda.set_device(0)
            fn(r)
        except BaseException as e:  # noqa: BLE001
            errs.append(e)
    ts = [threading.Thread(target=wrap, args=(r,)) for r in range(n)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    if errs:
        raise errs[0]


def case_gemm(reps=3):
    from ..ops.gemm import gemm_bf16, take_kernel_error
    a = torch.randn(8192, 8192, device="cuda").to(torch.bfloat16)
    w = (torch.randn(8192, 8192, device="cuda") * 0.02).to(torch.bfloat16)
    out = torch.empty(8192, 8192, device="cuda", dtype=torch.bfloat16)
    for _ in range(reps):
        gemm_bf16(a, w, out)
    torch.cuda.synchronize()
    assert take_kernel_error() == 0


def case_gemm_up(reps=2):
    """1.1 GB of operands and result.  The tile width and group come from HCOMM_GEMM_BN / HCOMM_GEMM_GM or the model."""
    from ..ops.gemm import gemm_bf16, take_kernel_error
    a = torch.randn(8192, 8192, device="cuda").to(torch.bfloat16)
    w = (torch.randn(28672, 8192, device="cuda") * 0.02).to(torch.bfloat16)
    out = torch.empty(8192, 28672, device="cuda", dtype=torch.bfloat16)
    for _ in range(reps):
        gemm_bf16(a, w, out)
    for _ in range(reps):
        torch.matmul(a, w.t(), out=out)
    torch.cuda.synchronize()
    assert take_kernel_error() == 0


GEMM_RASTER_WIDTHS, GEMM_RASTER_GROUPS = (512, 256), (4, 6, 8, 12, 16, 24)


def case_gemm_raster():
    """One launch per (shape, tile width, group): 2 shapes x 2 widths x 6 groups = 24 launches of the CTA-pair kernels, in the
    order of the loops below, so that a profiler's per-launch counters (DRAM bytes, cycles) can be read as a table."""
    from .. import _lib
    from ..ops.gemm import gemm_bf16, take_kernel_error
    lib = _lib.load()
    for (m, n, k) in ((8192, 28672, 8192), (8192, 8192, 28672)):
        a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
        w = (torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16)
        out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        for bn in GEMM_RASTER_WIDTHS:
            for gm in GEMM_RASTER_GROUPS:
                lib.HcommGemmSetTuning(gm, bn)
                gemm_bf16(a, w, out)
        torch.cuda.synchronize()
        del a, w, out
    lib.HcommGemmSetTuning(0, 0)
    assert take_kernel_error() == 0


def _comms(n, buffer_mb):
    import hcomm_b200 as hb
    info = hb.get_root_info()
    comms = [None] * n
    _ranks(n, lambda r: comms.__setitem__(r, hb.Communicator(n, info, r, buffer_mb=buffer_mb)))
    return comms


def case_fused(reps=2):
    from ..ops.fused import all_gather_gemm, gemm_reduce_scatter
    from ..ops.gemm import take_kernel_error
    n, m, nn, k = 2, 4096, 4096, 4096
    comms = _comms(n, 96)
    a = [torch.randn(m, k, device="cuda").to(torch.bfloat16) for _ in range(n)]
    b = [(torch.randn(nn, k, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(n)]
    x = [torch.randn(m // n, k, device="cuda").to(torch.bfloat16) for _ in range(n)]

    def op(r):
        for _ in range(reps):
            gemm_reduce_scatter(comms[r], a[r], b[r])
            all_gather_gemm(comms[r], x[r], b[r])
        torch.cuda.synchronize()
    _ranks(n, op)
    assert take_kernel_error() == 0
    _ranks(n, lambda r: comms[r].destroy())


def case_fused_pair(reps=2):
    """One rank: every tile is the rank's own, nothing crosses NVLink; shows the tensor-core side of the pair kernels
    (ranks that share a GPU use the single-CTA variants, so the two-rank case above cannot show them)."""
    import hcomm_b200 as hb
    from ..ops.fused import all_gather_gemm, gemm_reduce_scatter
    from ..ops.gemm import take_kernel_error
    comm = hb.Communicator(1, hb.get_root_info(), 0, buffer_mb=160)
    m, nn, k = 8192, 4096, 8192
    a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    b = (torch.randn(nn, k, device="cuda") * 0.02).to(torch.bfloat16)
    for _ in range(reps):
        gemm_reduce_scatter(comm, a, b)
        all_gather_gemm(comm, a, b)
    torch.cuda.synchronize()
    assert take_kernel_error() == 0
    comm.destroy()


def case_allreduce(reps=2):
    n = 2
    comms = _comms(n, 64)
    small = [torch.randn(16 << 10, device="cuda").to(torch.bfloat16) for _ in range(n)]       # 32 KB: flag-in-data kernel
    big = [torch.randn(32 << 20, device="cuda").to(torch.bfloat16) for _ in range(n)]         # 64 MB: two-shot
    outs = [torch.empty_like(big[r]) for r in range(n)]
    gathered = [torch.empty(n * (16 << 20), device="cuda", dtype=torch.bfloat16) for _ in range(n)]

    def op(r):
        for _ in range(reps):
            comms[r].all_reduce(small[r], outs[r][: small[r].numel()])
            comms[r].all_reduce(big[r], outs[r])
            comms[r].all_gather(big[r][: 16 << 20], gathered[r])
        torch.cuda.synchronize()
    _ranks(n, op)
    _ranks(n, lambda r: comms[r].destroy())


def case_moe(reps=2):
    import hcomm_b200 as hb
    from ..ops.moe import MoeExchange
    comm = hb.Communicator(1, hb.get_root_info(), 0, buffer_mb=8)
    e, k, h, t = 256, 8, 7168, 4096
    moe = MoeExchange(comm, e, k, h, t)
    x = torch.randn(t, h, device="cuda").to(torch.bfloat16)
    top = torch.randn(t, e, device="cuda").topk(k, dim=1)
    idx, gates = top.indices.to(torch.int32).contiguous(), torch.softmax(top.values, 1).float().contiguous()
    for _ in range(reps):
        rec = moe.dispatch(x, idx)
        torch.cuda.synchronize()
        y = torch.zeros(rec.num_rows, h, device="cuda", dtype=torch.bfloat16)
        moe.combine(y, gates)
    torch.cuda.synchronize()
    assert moe.overflow() == 0
    moe.destroy()
    comm.destroy()


def main():
    torch.cuda.set_device(0)
    which = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    {"gemm": case_gemm, "gemm_up": case_gemm_up, "gemm_raster": case_gemm_raster, "fused": case_fused, "fused_pair": case_fused_pair, "allreduce": case_allreduce, "moe": case_moe}[which]()
    print(f"profile case {which}: done", flush=True)


if __name__ == "__main__":
    main()
