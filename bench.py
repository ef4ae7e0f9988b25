#!/usr/bin/env python
"""Headline benchmark.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched once per GPU by torch.distributed.run)
    python bench.py --impl reference --gpus N ...             the same step on cuBLAS + NCCL only (see below)

Step = the tensor-parallel Llama-3-70B MLP of the task description (8192 tokens, hidden 8192, intermediate
28672, bf16, TP = N): a column-parallel up projection fused with its all-gather followed by a row-parallel
down projection fused with its reduce-scatter, both on the library's own tcgen05 kernels with the collective
moving over NVLink peer memory inside the kernel.  With N = 1 the same two GEMMs run without communication.
Total work is fixed as N grows (strong scaling).

`--impl reference`: the reference library (HCOMM) is an Ascend CANN C++ / AscendC project with neither a Python
package nor a CUDA back end, so it cannot be installed or run on this hardware.  The baseline the task names for
this metric is the same step on cuBLAS (torch.matmul) + NCCL (all_gather_into_tensor / reduce_scatter_tensor); that
is what this arm runs, in a process that imports nothing from this repository's package and loads none of its
libraries, and it says so in its "impl" field.

Timing (both arms alike): a time-based pre-spin of GEMMs brings the clocks up; W >= 3 warm-up steps; then K steps
back to back between two CUDA events on the launching stream, bracketed by a barrier and a device synchronisation
on both sides; the maximum over ranks is reported.  Every step touches more bytes than the 126 MB L2 holds (weights,
activations and staging of one step exceed 400 MB per GPU at every N), so consecutive steps do not find their
operands cached.  The end-to-end figure runs the same K steps through the public API with each step's input copied
from pinned host memory and each step's whole result copied back to pinned host memory, both on copy streams that
overlap the next / previous step's compute.  SM clocks and throttle reasons are sampled through NVML while the timed
regions run.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))

TOKENS, HIDDEN, INTER = 8192, 8192, 28672
REFERENCE_WHY = ("the reference is an Ascend CANN C++/AscendC project without setup.py or pyproject.toml: pip cannot install it and it "
                 "cannot build for CUDA")


class ClockSampler:
    """Samples this GPU's SM clock, power and clock-event reasons through NVML (in-process, ~20 us per sample)."""

    def __init__(self, torch_device_index: int, period_ms: int = 10):
        self.rows, self.period, self._stop, self._thread, self._h, self._nv = [], period_ms / 1e3, threading.Event(), None, None, None
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            props = torch.cuda.get_device_properties(torch_device_index)
            try:
                bus = "%08x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
                self._h = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
            except Exception:
                self._h = pynvml.nvmlDeviceGetHandleByIndex(torch_device_index)
            self._nv = pynvml
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._h = None

    def _loop(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.rows.append((nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM), nv.nvmlDeviceGetPowerUsage(self._h) / 1e3,
                                  nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)))
            except Exception:
                pass
            self._stop.wait(self.period)

    def start(self):
        if self._h is not None:
            self._stop.clear()
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def stop(self):
        if self._thread:
            self._stop.set()
            self._thread.join(timeout=2)
            self._thread = None

    def summary(self) -> dict:
        if self._h is None or not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        nv = self._nv
        names = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown, "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                 "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown, "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap,
                 "hw_power_brake": nv.nvmlClocksEventReasonHwPowerBrakeSlowdown}
        # "under load" = samples drawing clearly more than idle power
        pmax = max(r[1] for r in self.rows)
        load = [r for r in self.rows if r[1] >= 0.5 * pmax] or self.rows
        seen = set()
        for _, _, mask in load:
            for k, bit in names.items():
                if mask & bit:
                    seen.add(k)
        return {"sm_mhz": statistics.median(r[0] for r in load), "sm_max_mhz": float(self.max_mhz), "reasons": sorted(seen), "samples": len(self.rows),
                "samples_under_load": len(load), "power_w_max": round(pmax, 1)}


def bind_near_gpu(local):
    """Runs this process on the CPUs NVML names as closest to its GPU (both arms do), so that the pinned buffers of the
    end-to-end step are allocated on that GPU's side of the host.  Returns the number of CPUs kept, 0 when nothing changed."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(local)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        near = {64 * i + b for i, w in enumerate(mask) for b in range(64) if (w >> b) & 1}
        allowed = os.sched_getaffinity(0)
        keep = near & allowed
        if keep and keep != allowed:
            os.sched_setaffinity(0, keep)
            return len(keep)
    except Exception:
        pass
    return 0


def setup_dist(torch, dist, a):
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world != a.gpus and world == 1:
        print(f"bench.py --gpus {a.gpus} must be launched with torch.distributed.run --nproc-per-node {a.gpus}", file=sys.stderr)
        sys.exit(2)
    a.cpus_bound = 0 if a.no_bind else bind_near_gpu(local)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    return rank, world, local, dev


def make_inputs(torch, dev, rank, world):
    """Seeded synthetic data of the benchmark's shape: this rank's activation rows and weight shards."""
    rows = TOKENS // world
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    x = torch.randn(rows, HIDDEN, device=dev, generator=g).to(torch.bfloat16)
    gw = torch.Generator(device=dev).manual_seed(1 + 1000 * rank)
    w_up = (torch.randn(INTER // world, HIDDEN, device=dev, generator=gw) * 0.02).to(torch.bfloat16)
    w_down = (torch.randn(HIDDEN, INTER // world, device=dev, generator=gw) * 0.02).to(torch.bfloat16)
    return x, w_up, w_down


def prespin(torch, dev, seconds):
    """GEMMs for `seconds` of wall time so that the timed region starts at working clocks."""
    a = torch.randn(4096, 4096, device=dev, dtype=torch.bfloat16)
    t0 = time.time()
    n = 0
    while time.time() - t0 < seconds:
        for _ in range(20):
            torch.matmul(a, a)
        torch.cuda.synchronize()
        n += 20
    return time.time() - t0


def timed_region(torch, dist, dev, world, step_fn, steps, warmup, finish=None):
    """K steps back to back between two events; returns the maximum over ranks of the elapsed milliseconds."""
    for _ in range(warmup):
        step_fn()
    if finish:
        finish()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(steps):
        step_fn()
    if finish:
        finish()
    e.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t = torch.tensor([s.elapsed_time(e)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


class EndToEnd:
    """A step through `compute(x) -> y` with the input arriving from pinned host memory and the whole result returning to
    pinned host memory every step.  Two device input slots and two host result slots: the input of step i+1 travels on
    the upload stream while step i computes, the result of step i travels back on the download stream while step i+1
    computes.  finish() waits for the last result."""

    def __init__(self, torch, dev, x, compute):
        self.torch, self.dev, self.compute = torch, dev, compute
        self.x_host = torch.empty(x.shape, dtype=x.dtype).pin_memory()
        self.x_host.copy_(x.cpu())
        self.up, self.down = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        self.x_slots = [torch.empty_like(x), torch.empty_like(x)]
        self.landed = [torch.cuda.Event(), torch.cuda.Event()]
        self.y_host, self.y_dev, self.y_free = None, [None, None], [torch.cuda.Event(), torch.cuda.Event()]
        self.read_done = [None, None]
        self.step_no, self.primed = 0, False

    def _prefetch(self, slot):
        if self.read_done[slot] is not None:
            self.up.wait_event(self.read_done[slot])                      # the step that last read this slot has finished
        with self.torch.cuda.stream(self.up):
            self.x_slots[slot].copy_(self.x_host, non_blocking=True)
            self.landed[slot].record(self.up)

    def step(self):
        torch, slot = self.torch, self.step_no & 1
        cur = torch.cuda.current_stream(self.dev)
        if not self.primed:
            self._prefetch(slot)
            self.primed = True
        cur.wait_event(self.landed[slot])
        self._prefetch(slot ^ 1)                                          # travels while this step computes
        if self.y_dev[slot] is not None:
            cur.wait_event(self.y_free[slot])                             # the download of step i-2 has read this buffer
        y = self.compute(self.x_slots[slot], self.y_dev[slot])
        self.y_dev[slot] = y
        if self.read_done[slot] is None:
            self.read_done[slot] = torch.cuda.Event()
        self.read_done[slot].record(cur)
        if self.y_host is None:
            self.y_host = [torch.empty(y.shape, dtype=y.dtype).pin_memory() for _ in range(2)]
        self.down.wait_stream(cur)
        with torch.cuda.stream(self.down):
            self.y_host[slot].copy_(y, non_blocking=True)
            self.y_free[slot].record(self.down)
        self.step_no += 1

    def finish(self):
        self.torch.cuda.current_stream(self.dev).wait_stream(self.down)

    def bytes_per_step(self):
        return self.x_host.numel() * self.x_host.element_size(), self.y_host[0].numel() * self.y_host[0].element_size()


def roofline_ms(world):
    """Sum over the two operators of max(FLOPs / measured cuBLAS burst peak, bytes over NVLink / 900 GB/s per direction)."""
    peaks = {}
    try:
        peaks = json.loads((Path(__file__).resolve().parent / "MEASURED_PEAKS.json").read_text())
    except Exception:
        pass
    tflops = peaks.get("bf16_tflops", 1590.0)
    basis = ("%.1f TFLOP/s measured cuBLAS bf16 burst" % tflops) if "bf16_tflops" in peaks else "1590 TFLOP/s fallback cuBLAS bf16 burst"
    t_gemm = 2.0 * TOKENS * HIDDEN * INTER / world / (tflops * 1e12) * 1e3          # each of the two GEMMs, per rank
    t_link = (world - 1) / world * TOKENS * HIDDEN * 2 / 900e9 * 1e3                 # gathered rows in / partial rows out, per rank and direction
    return 2 * max(t_gemm, t_link), basis + ", 900 GB/s NVLink per direction", t_gemm, t_link


def config_block(world):
    return {"model": "Llama-3-70B MLP (hidden 8192, intermediate 28672): AllGather->GEMM then GEMM->ReduceScatter", "global_batch": TOKENS,
            "seq_len": TOKENS, "parallelism": f"tp{world}", "l2": "no flush: one step touches >400 MB per GPU, more than the 126 MB L2",
            "weights": "random-init N(0,0.02)", "activations": "N(0,1) seeded per rank", "timing": "K steps back to back between two CUDA events, max over ranks"}


def reference_arm(a):
    """cuBLAS + NCCL, nothing from this repository."""
    import torch
    import torch.distributed as dist
    a.warmup = max(3, a.warmup)
    rank, world, local, dev = setup_dist(torch, dist, a)
    x, w_up, w_down = make_inputs(torch, dev, rank, world)
    rows = TOKENS // world
    full = torch.empty(TOKENS, HIDDEN, dtype=torch.bfloat16, device=dev)
    h = torch.empty(TOKENS, INTER // world, dtype=torch.bfloat16, device=dev)
    yfull = torch.empty(TOKENS, HIDDEN, dtype=torch.bfloat16, device=dev)

    def compute(xin, out=None):
        if out is None:
            out = torch.empty(rows, HIDDEN, dtype=torch.bfloat16, device=dev)
        if world > 1:
            dist.all_gather_into_tensor(full, xin)
            torch.matmul(full, w_up.t(), out=h)
            torch.matmul(h, w_down.t(), out=yfull)
            dist.reduce_scatter_tensor(out, yfull)
        else:
            torch.matmul(xin, w_up.t(), out=h)
            torch.matmul(h, w_down.t(), out=out)
        return out

    spin_s = prespin(torch, dev, a.prespin)
    clocks = ClockSampler(local).start()
    ybuf = torch.empty(rows, HIDDEN, dtype=torch.bfloat16, device=dev)
    ms = timed_region(torch, dist, dev, world, lambda: compute(x, ybuf), a.steps, a.warmup) / a.steps
    e2e = EndToEnd(torch, dev, x, compute)
    e2e_ms = timed_region(torch, dist, dev, world, e2e.step, a.steps, a.warmup, e2e.finish) / a.steps
    clocks.stop()
    if rank == 0:
        bi, bo = e2e.bytes_per_step()
        roof, basis, _, _ = roofline_ms(world)
        print(json.dumps({
            "impl": "nccl+cublas (reference is Ascend-only)", "reference_unavailable": REFERENCE_WHY,
            "metric": "tp_mlp_fused_tokens_per_s", "value": TOKENS / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_block(world), "clocks": clocks.summary(), "prespin_s": round(spin_s, 2), "cpus_bound_near_gpu": a.cpus_bound,
            "e2e": {"value": TOKENS / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": bi, "d2h_bytes_per_step": bo},
            "gpu_launches": 0, "roofline_ms": roof, "fraction_of_roofline": roof / ms, "roofline_basis": basis}))
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--prespin", type=float, default=1.5, help="seconds of GEMMs before the warm-up steps")
    ap.add_argument("--no-collectives", action="store_true", help="skip the all-reduce table")
    ap.add_argument("--no-bind", action="store_true", help="leave the process on whatever CPUs it was started on")
    ap.add_argument("--mode", default="auto", choices=["auto", "fused", "split"], help="how the GEMM + collective operators run")
    ap.add_argument("--phases", default="", help="write the fused kernels' per-CTA phase clocks of one step to this JSON file (rank 0)")
    a = ap.parse_args()
    if a.impl == "reference":
        return reference_arm(a)
    a.warmup = max(3, a.warmup)

    os.environ.setdefault("HCCL_EXEC_TIMEOUT", "120")      # a wait that cannot complete ends the run instead of stalling it
    import torch
    import torch.distributed as dist
    import hcomm_b200 as hb
    from hcomm_b200.ops import fused
    from hcomm_b200.ops.gemm import take_kernel_error
    from hcomm_b200.parallel.tp import TensorParallelMlp

    rank, world, local, dev = setup_dist(torch, dist, a)
    if world > 1:
        box = [hb.get_root_info() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        info = box[0]
    else:
        info = hb.get_root_info()
    comm = hb.Communicator(world, info, rank, buffer_mb=512)
    x, w_up, w_down = make_inputs(torch, dev, rank, world)
    mlp = TensorParallelMlp(comm, HIDDEN, INTER, device=dev, w_up=w_up, w_down=w_down, mode=a.mode)
    rows = TOKENS // world
    flops = 2.0 * TOKENS * HIDDEN * INTER * 2

    # ---- one step checked against cuBLAS (+ NCCL) before anything is timed
    y = mlp(x)
    if world > 1:
        ref = fused.gemm_reduce_scatter_unfused(fused.all_gather_gemm_unfused(x, w_up), w_down)
    else:
        ref = torch.matmul(torch.matmul(x, w_up.t()), w_down.t())
    torch.cuda.synchronize()
    max_err = (y.float() - ref.float()).abs().max().item()
    ref_scale = ref.float().abs().max().item()
    err_t = torch.tensor([max_err, ref_scale], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(err_t, op=dist.ReduceOp.MAX)
    max_err, ref_scale = err_t.tolist()
    del ref
    if not max_err <= 3e-2 * max(1.0, ref_scale):
        print(f"the fused step differs from cuBLAS + NCCL: max |err| {max_err} at scale {ref_scale}", file=sys.stderr)
        return 4

    spin_s = prespin(torch, dev, a.prespin)
    clocks = ClockSampler(local).start()
    ybuf = torch.empty(rows, HIDDEN, dtype=torch.bfloat16, device=dev)
    total_ms = timed_region(torch, dist, dev, world, lambda: mlp(x, ybuf), a.steps, a.warmup)
    ms_per_step = total_ms / a.steps
    if take_kernel_error() != 0 or comm.async_error() != 0:
        print("a bounded wait expired inside a kernel; the measurement is void", file=sys.stderr)
        return 3

    # ---- end to end through the public API
    e2e = EndToEnd(torch, dev, x, lambda xin, out=None: mlp(xin, out))
    e2e_ms = timed_region(torch, dist, dev, world, e2e.step, a.steps, a.warmup, e2e.finish) / a.steps
    clocks.stop()
    bi, bo = e2e.bytes_per_step()

    extra = {}
    # ---- the same step on cuBLAS (+ NCCL) in this process, same timing rules (the driver's comparison is the reference arm)
    if world > 1:
        full = torch.empty(TOKENS, HIDDEN, dtype=torch.bfloat16, device=dev)
        h = torch.empty(TOKENS, INTER // world, dtype=torch.bfloat16, device=dev)
        yfull = torch.empty(TOKENS, HIDDEN, dtype=torch.bfloat16, device=dev)

        def unfused():
            dist.all_gather_into_tensor(full, x)
            torch.matmul(full, w_up.t(), out=h)
            torch.matmul(h, w_down.t(), out=yfull)
            dist.reduce_scatter_tensor(ybuf, yfull)
        unfused_ms = timed_region(torch, dist, dev, world, unfused, a.steps, a.warmup) / a.steps
        del full, h, yfull
        extra["unfused_cublas_nccl_ms_per_step"] = unfused_ms
        extra["fused_speedup_vs_unfused"] = unfused_ms / ms_per_step
    else:
        h = torch.empty(TOKENS, INTER, dtype=torch.bfloat16, device=dev)
        cublas_ms = timed_region(torch, dist, dev, world, lambda: torch.matmul(torch.matmul(x, w_up.t(), out=h), w_down.t(), out=ybuf), a.steps, a.warmup) / a.steps
        del h
        extra["cublas_ms_per_step"] = cublas_ms
        extra["speedup_vs_cublas"] = cublas_ms / ms_per_step
        # what the library's measurement at first use kept for the two GEMM shapes (tile width, rasterisation group)
        import ctypes
        from hcomm_b200 import _lib
        tuned = {}
        for name, (m, n, k) in (("up", (TOKENS, INTER, HIDDEN)), ("down", (TOKENS, HIDDEN, INTER))):
            bn, gm = ctypes.c_int(0), ctypes.c_int(0)
            _lib.load().HcommGemmGetTuned(m, n, k, ctypes.byref(bn), ctypes.byref(gm))
            tuned[name] = {"tile_width": bn.value, "group_rows": gm.value}
        extra["gemm_tuning"] = tuned
    roof, basis, t_gemm, t_link = roofline_ms(world)
    extra["roofline_ms"] = roof
    extra["fraction_of_roofline"] = roof / ms_per_step
    extra["roofline_basis"] = basis
    extra["roofline_terms_ms"] = {"gemm_each": t_gemm, "link_each": t_link}

    if a.phases:
        fused.set_phase_clocks(comm, True)
        ph = {}
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        hmid = mlp.up(x, mlp._h)
        torch.cuda.synchronize()
        ph["all_gather_gemm"] = fused.phase_clocks(comm) if world > 1 else {}
        if world > 1:
            dist.barrier()
        mlp.down(hmid, ybuf)
        torch.cuda.synchronize()
        ph["gemm_reduce_scatter"] = fused.phase_clocks(comm) if world > 1 else {}
        fused.set_phase_clocks(comm, False)
        gathered = [None] * world
        if world > 1:
            dist.all_gather_object(gathered, ph)
        else:
            gathered = [ph]
        if rank == 0:
            Path(a.phases).parent.mkdir(parents=True, exist_ok=True)
            Path(a.phases).write_text(json.dumps({"n_gpus": world, "per_rank": gathered}, indent=1))

    if world > 1 and not a.no_collectives:
        from hcomm_b200.utils.coll_bench import run_sweep
        sizes = [8, 4096, 262144, 4 << 20, 64 << 20, 256 << 20]
        rows_ar = run_sweep(comm, ["allreduce"], sizes, torch.bfloat16, iters=20, warmup=5, with_nccl=True)
        extra["allreduce_vs_nccl"] = [{"bytes": r["bytes"], "ours_busbw_gbs": round(r["ours_busbw_gbs"], 2), "nccl_busbw_gbs": round(r["nccl_busbw_gbs"], 2),
                                       "speedup": round(r["speedup_vs_nccl"], 3)} for r in rows_ar]

    if rank == 0:
        out = {
            "metric": "tp_mlp_fused_tokens_per_s", "value": TOKENS / (ms_per_step * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "tflops_per_gpu": flops / world / (ms_per_step * 1e-3) / 1e12, "config": config_block(world),
            "clocks": clocks.summary(), "prespin_s": round(spin_s, 2), "cpus_bound_near_gpu": a.cpus_bound, "max_err_vs_cublas_nccl": max_err, "mode": a.mode,
            "e2e": {"value": TOKENS / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": bi, "d2h_bytes_per_step": bo,
                    "note": "every step copies its input from pinned host memory and its whole result back to pinned host memory; the copies run on "
                            "copy streams beside the neighbouring steps' compute"},
            "gpu_launches": mlp.launches_per_step * a.steps,
        }
        out.update(extra)
        print(json.dumps(out))
    comm.destroy()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
