"""Times the tcgen05 bf16 GEMM against cuBLAS (``torch.matmul``) on one GPU.

    python -m hcomm_b200.utils.gemm_bench [--shapes 8192x28672x8192,8192x8192x28672] [--rounds 5] [--iters 5]

C[M, N] = A[M, K] * B[N, K]^T.  The two implementations take turns (``rounds`` rounds of ``iters`` back-to-back calls
each, CUDA events around every round), so a clock that drifts under the power cap touches both alike; the figure per
implementation is the median of its rounds.  With HCOMM_GEMM_AUTOTUNE=1 the first, untimed call lets the library measure
and pick its tile width and rasterisation group for the shape and the choice is printed (0 / 0 otherwise: the model
decided).  Operands of the default shapes exceed the L2.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import statistics
import time

import torch

DEFAULT = "8192x28672x8192,8192x8192x28672,8192x8192x8192,8192x14336x8192,8192x8192x14336,8192x7168x8192,8192x8192x7168,8192x3584x8192,8192x8192x3584"


def main():
    from .. import _lib
    from ..ops.gemm import gemm_bf16, take_kernel_error
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default=DEFAULT)
    ap.add_argument("--rounds", type=int, default=5)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--prespin", type=float, default=1.0)
    a = ap.parse_args()
    lib = _lib.load()
    torch.cuda.set_device(0)
    w = torch.randn(4096, 4096, device="cuda", dtype=torch.bfloat16)
    t0 = time.time()
    while time.time() - t0 < a.prespin:
        for _ in range(20):
            w @ w
        torch.cuda.synchronize()

    def timed(fn):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(a.iters):
            fn()
        e.record()
        e.synchronize()
        return s.elapsed_time(e) / a.iters

    for spec in a.shapes.split(","):
        m, n, k = (int(v) for v in spec.split("x"))
        x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
        wt = (torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16)
        c_ours = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        c_ref = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        ours = lambda: gemm_bf16(x, wt, c_ours)
        ref = lambda: torch.matmul(x, wt.t(), out=c_ref)
        ours(); ref()                                  # the library's measurement at first use, cuBLAS' heuristics
        torch.cuda.synchronize()
        bn, gm = ctypes.c_int(0), ctypes.c_int(0)
        lib.HcommGemmGetTuned(m, n, k, ctypes.byref(bn), ctypes.byref(gm))
        err = (c_ours.float() - c_ref.float()).abs().max().item()
        t_ours, t_ref = [], []
        for _ in range(a.rounds):
            t_ref.append(timed(ref))
            t_ours.append(timed(ours))
        mo, mr = statistics.median(t_ours), statistics.median(t_ref)
        fl = 2.0 * m * n * k
        print(json.dumps({"shape": [m, n, k], "ours_ms": round(mo, 4), "cublas_ms": round(mr, 4), "ours_tflops": round(fl / mo / 1e9, 1),
                          "cublas_tflops": round(fl / mr / 1e9, 1), "speedup_vs_cublas": round(mr / mo, 3), "tile_width": bn.value, "group_rows": gm.value,
                          "max_abs_diff": err}), flush=True)
        del x, wt, c_ours, c_ref
    assert take_kernel_error() == 0


if __name__ == "__main__":
    main()
