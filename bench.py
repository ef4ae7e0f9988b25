#!/usr/bin/env python
"""Headline benchmark.

    python bench.py --gpus N --steps K --warmup W          (N > 1: launched once per GPU by torch.distributed.run)
    python bench.py --impl reference ...                     prints why the reference cannot run here

Step = the tensor-parallel Llama-3-70B MLP of the task description (8192 tokens, hidden 8192, intermediate
28672, bf16, TP = N): a column-parallel up projection fused with its all-gather followed by a row-parallel
down projection fused with its reduce-scatter, both on the library's own tcgen05 kernels with the collective
moving over NVLink peer memory inside the kernel.  With N = 1 the same two GEMMs run without communication.
Total work is fixed as N grows (strong scaling).  The JSON line also carries, for N > 1, the unfused
cuBLAS + NCCL time of the same step and an all-reduce bus-bandwidth table against NCCL.

Timing: W >= 3 warm-up steps; every timed step is bracketed by CUDA events on the launching stream, an L2
flush (192 MB write) and a barrier sit between steps outside the events; the K step times are summed and the
maximum over ranks is reported.  The end-to-end figure repeats the measurement through the public API with the
step's input copied from pinned host memory and a scalar of the result read back every step.
"""
import argparse
import json
import os
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))

TOKENS, HIDDEN, INTER = 8192, 8192, 28672


def reference_arm():
    if int(os.environ.get("RANK", "0")) != 0:      # launched once per GPU: one line for the whole job
        return 0
    print(json.dumps({"impl": "reference", "unavailable": "the reference is an Ascend CANN C++/AscendC project without setup.py or pyproject.toml: "
                      "pip cannot install it and it cannot build for CUDA"}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--no-collectives", action="store_true", help="skip the all-reduce table")
    a = ap.parse_args()
    if a.impl == "reference":
        return reference_arm()
    a.warmup = max(3, a.warmup)

    os.environ.setdefault("HCCL_EXEC_TIMEOUT", "120")      # a wait that cannot complete ends the run instead of stalling it
    import torch
    import torch.distributed as dist
    import hcomm_b200 as hb
    from hcomm_b200.ops.gemm import take_kernel_error
    from hcomm_b200.parallel.tp import TensorParallelMlp
    from hcomm_b200.utils.timing import ClockSampler, l2_flush

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world != a.gpus:
        if world == 1 and a.gpus > 1:
            print(f"bench.py --gpus {a.gpus} must be launched with torch.distributed.run --nproc-per-node {a.gpus}", file=sys.stderr)
            return 2
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        box = [hb.get_root_info() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        info = box[0]
    else:
        info = hb.get_root_info()
    comm = hb.Communicator(world, info, rank, buffer_mb=512)
    mlp = TensorParallelMlp(comm, HIDDEN, INTER, device=dev, seed=1)
    rows = TOKENS // world
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    x = torch.randn(rows, HIDDEN, device=dev, generator=g).to(torch.bfloat16)

    def barrier():
        if world > 1:
            dist.barrier()

    def timed(step_fn, steps, warmup):
        for _ in range(warmup):
            step_fn()
        torch.cuda.synchronize()
        total_ms = 0.0
        for _ in range(steps):
            torch.cuda.synchronize()
            barrier()
            l2_flush(dev)        # cold L2 for the step; also keeps the GPU busy while the host enqueues the step
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            step_fn()
            e.record()
            e.synchronize()
            total_ms += s.elapsed_time(e)
        torch.cuda.synchronize()
        barrier()
        t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    # ---- device-timed: inputs resident on the GPU
    def step_device():
        return mlp(x)

    clocks = ClockSampler(local, period_ms=50)
    clocks.__enter__()
    total_ms = timed(step_device, a.steps, a.warmup)
    ms_per_step = total_ms / a.steps
    tokens_per_s = TOKENS / (ms_per_step * 1e-3)
    flops = 2.0 * TOKENS * HIDDEN * INTER * 2
    if take_kernel_error() != 0 or comm.async_error() != 0:
        print("a bounded wait expired inside a kernel; the measurement is void", file=sys.stderr)
        return 3

    # ---- end to end: input from pinned host memory every step, one scalar of the result back
    x_host = torch.empty(rows, HIDDEN, dtype=torch.bfloat16).pin_memory()
    x_host.copy_(x.cpu())
    result = torch.zeros(1, dtype=torch.float32).pin_memory()
    # Two device buffers: while step i computes, the input of step i+1 travels from pinned host memory on a copy
    # stream.  Every step issues one full host->device copy inside its timed window and reads one scalar back.
    copy_stream = torch.cuda.Stream(device=dev)
    x_slots = [torch.empty_like(x), torch.empty_like(x)]
    landed = [torch.cuda.Event(), torch.cuda.Event()]
    state = {"step": 0, "primed": False}

    def prefetch(slot):
        copy_stream.wait_stream(torch.cuda.current_stream(dev))     # the slot's previous reader has been queued before
        with torch.cuda.stream(copy_stream):
            x_slots[slot].copy_(x_host, non_blocking=True)
            landed[slot].record(copy_stream)

    def step_e2e():
        slot = state["step"] & 1
        if not state["primed"]:
            prefetch(slot)
            state["primed"] = True
        torch.cuda.current_stream(dev).wait_event(landed[slot])
        y = mlp(x_slots[slot])
        prefetch(slot ^ 1)
        result.copy_(y[:, :64].float().abs().mean().reshape(1), non_blocking=True)
        torch.cuda.current_stream(dev).synchronize()
        state["step"] += 1
        return float(result[0])

    e2e_ms = timed(step_e2e, a.steps, a.warmup) / a.steps
    clocks.__exit__(None, None, None)     # sampled through both timed regions of this library's step

    # ---- unfused baseline of the same step (cuBLAS + NCCL), same timing rules
    extra = {}
    if world > 1:
        from hcomm_b200.ops.fused import all_gather_gemm_unfused, gemm_reduce_scatter_unfused
        w_up, w_down = mlp.up.weight, mlp.down.weight
        unfused_ms = timed(lambda: gemm_reduce_scatter_unfused(all_gather_gemm_unfused(x, w_up), w_down), a.steps, a.warmup) / a.steps
        extra["unfused_cublas_nccl_ms_per_step"] = unfused_ms
        extra["fused_speedup_vs_unfused"] = unfused_ms / ms_per_step
        # roofline: slower of FLOPs at the measured GEMM peak and bytes over NVLink at 770 GB/s measured per direction
        peaks = {}
        try:
            peaks = json.loads((Path(__file__).resolve().parent / "MEASURED_PEAKS.json").read_text())
        except Exception:
            pass
        tflops = peaks.get("bf16_tflops_sustained", 1400.0)
        t_compute = flops / world / (tflops * 1e12) * 1e3
        link_bytes = 2 * (world - 1) / world * TOKENS * HIDDEN * 2 / world * world / world   # per rank, AG in + RS out
        t_link = ((world - 1) / world * TOKENS * HIDDEN * 2) / 770e9 * 1e3
        extra["roofline_ms"] = max(t_compute, t_link)
        extra["fraction_of_roofline"] = max(t_compute, t_link) / ms_per_step
        extra["roofline_basis"] = f"{tflops} TFLOP/s measured sustained cuBLAS bf16, 770 GB/s measured NVLink per direction"
        if not a.no_collectives:
            from hcomm_b200.utils.coll_bench import run_sweep
            sizes = [8, 4096, 262144, 4 << 20, 64 << 20, 256 << 20]
            rows_ar = run_sweep(comm, ["allreduce"], sizes, torch.bfloat16, iters=5, warmup=3, with_nccl=True) if rank >= 0 else []
            extra["allreduce_vs_nccl"] = [{"bytes": r["bytes"], "ours_busbw_gbs": round(r["ours_busbw_gbs"], 2), "nccl_busbw_gbs": round(r["nccl_busbw_gbs"], 2),
                                           "speedup": round(r["speedup_vs_nccl"], 3)} for r in rows_ar]
    else:
        unfused = timed(lambda: torch.matmul(torch.matmul(x, mlp.up.weight.t()), mlp.down.weight.t()), a.steps, a.warmup) / a.steps
        extra["cublas_ms_per_step"] = unfused
        extra["speedup_vs_cublas"] = unfused / ms_per_step

    if rank == 0:
        out = {
            "metric": "tp_mlp_fused_tokens_per_s", "value": tokens_per_s, "unit": "tokens/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "tflops_per_gpu": flops / world / (ms_per_step * 1e-3) / 1e12,
            "config": {"model": "Llama-3-70B MLP (hidden 8192, intermediate 28672): AllGather->GEMM then GEMM->ReduceScatter", "global_batch": TOKENS,
                       "seq_len": TOKENS, "parallelism": f"tp{world}", "l2_flush_between_steps": True, "weights": "random-init N(0,0.02)",
                       "activations": "N(0,1) seeded per rank"},
            "clocks": clocks.summary(),
            "e2e": {"value": TOKENS / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": rows * HIDDEN * 2, "d2h_bytes_per_step": 4,
                    "note": "input of step i+1 is copied from pinned host memory on a copy stream while step i computes; one scalar of the result is read back every step"},
            "gpu_launches": 2 * a.steps,
        }
        out.update(extra)
        print(json.dumps(out))
    comm.destroy()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
