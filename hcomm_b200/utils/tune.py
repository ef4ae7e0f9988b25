"""Builds the selector's size-bucket table from measurements on the machine at hand.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m hcomm_b200.utils.tune --out tune_8.json
    HCCL_TUNE_FILE=tune_8.json python ...            # the selector then uses the measured buckets

For every collective and message size the candidates (mesh one-shot, mesh two-shot, in-switch reduction, each with
a few CTA counts) are timed with the same rules as the benchmarks (CUDA events, L2 flush, maximum over ranks); the
fastest candidate per size wins and neighbouring sizes with the same winner are merged into one bucket.
The file format is what ``HCCL_TUNE_FILE`` expects: {op: {ranks: [{"max_bytes", "algo", "engine", "ctas"}, ...]}};
``max_bytes`` counts what the selector sees: the whole vector for all-reduce and broadcast, one rank's block for
all-gather, reduce-scatter and all-to-all.

The same table can be built without a GPU from sweeps that ``coll_bench --out`` wrote earlier, one file per forced
algorithm (a file whose rows say ``auto`` stands for the family given with ``--auto-is``):

    python -m hcomm_b200.utils.tune --from-sweeps mesh.json nvls.json --auto-is mesh --ops allgather,reducescatter --out tune_8.json
"""
from __future__ import annotations

import argparse
import json
import os

CANDIDATES = {
    "allreduce": [("mesh_oneshot", "sm"), ("mesh", "sm"), ("nvls", "nvls")],
    "allgather": [("mesh", "sm"), ("nvls", "nvls")],
    "reducescatter": [("mesh", "sm"), ("nvls", "nvls")],
    "alltoall": [("mesh", "sm")],
    "broadcast": [("mesh_oneshot", "sm"), ("mesh", "sm"), ("nvls", "nvls")],
}
CTA_CHOICES = (0, 16, 32, 64, 128)        # 0 = the library's own heuristic


def merge_buckets(winners):
    """winners: [(bytes, algo, engine, ctas)] sorted by bytes -> bucket list with merged neighbours.

    A bucket ends halfway (geometrically: at the smaller size) between two sizes with different winners; the last one is
    open-ended (max_bytes = -1)."""
    buckets = []
    for i, (nbytes, algo, engine, ctas) in enumerate(winners):
        key = (algo, engine, ctas)
        if buckets and buckets[-1]["_key"] == key:
            buckets[-1]["max_bytes"] = nbytes
        else:
            buckets.append({"max_bytes": nbytes, "algo": algo, "engine": engine, "ctas": ctas, "_key": key})
    for b in buckets:
        del b["_key"]
    if buckets:
        buckets[-1]["max_bytes"] = -1
    return buckets


def pick_winners(measurements):
    """measurements: {bytes: {(algo, engine, ctas): microseconds}} -> [(bytes, algo, engine, ctas)] sorted by bytes.
    A candidate must beat the incumbent of the previous size by more than 3 % to replace it (keeps buckets stable)."""
    winners, prev = [], None
    for nbytes in sorted(measurements):
        cands = measurements[nbytes]
        best = min(cands, key=cands.get)
        if prev in cands and cands[prev] <= cands[best] * 1.03:
            best = prev
        winners.append((nbytes, *best))
        prev = best
    return winners


def selector_bytes(op, nbytes, world):
    """The size the selector compares with ``max_bytes`` for an operand of `nbytes` as the benchmarks count them."""
    return nbytes // world if op in ("allgather", "reducescatter", "alltoall") else nbytes


def family_of(label, op, auto_is):
    """(algo, engine) of a sweep row's ``algo`` label, e.g. ``allgather=level0:nvls/reducescatter=level0:nvls``."""
    name = auto_is
    if label and label != "auto":
        for part in label.split("/"):
            key, _, val = part.partition("=")
            if not val:                                   # "level0:ring" applies to every operator
                key, val = op, part
            if key.strip() == op:
                name = val.split(":")[-1].strip().lower()
    name = {"fullmesh": "mesh", "oneshot": "mesh_oneshot"}.get(name, name)
    return name, ("nvls" if name == "nvls" else "sm")


def table_from_sweeps(paths, ops, auto_is="mesh"):
    """Builds the bucket table from ``coll_bench --out`` files (lists of rows with op, bytes, n, algo, ours_us)."""
    meas = {}
    for path in paths:
        with open(path) as f:
            for row in json.load(f):
                if row["op"] not in ops or row.get("registered"):
                    continue
                algo, engine = family_of(row.get("algo", "auto"), row["op"], auto_is)
                key = (row["op"], str(row["n"]))
                meas.setdefault(key, {}).setdefault(selector_bytes(row["op"], row["bytes"], row["n"]), {})[(algo, engine, 0)] = row["ours_us"]
    table = {}
    for (op, ranks), by_size in sorted(meas.items()):
        table.setdefault(op, {})[ranks] = merge_buckets(pick_winners(by_size))
    return table


def algo_config(op, algo, engine):
    level0 = {"mesh": "fullmesh", "mesh_oneshot": "fullmesh", "nvls": "nvls"}[algo]
    return f"{op}=level0:{level0}"


def main():
    import torch
    import torch.distributed as dist
    from .coll_bench import parse_size
    from .launch import env_rank
    from .timing import time_cuda
    from ..comm import Communicator, get_root_info

    ap = argparse.ArgumentParser()
    ap.add_argument("--ops", default="allreduce,allgather,reducescatter,alltoall")
    ap.add_argument("--min-bytes", default="1K")
    ap.add_argument("--max-bytes", default="256M")
    ap.add_argument("--factor", type=int, default=4)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--out", default="hccl_tune.json")
    ap.add_argument("--from-sweeps", nargs="+", default=None, help="build the table from coll_bench --out files instead of measuring")
    ap.add_argument("--auto-is", default="mesh", help="family that rows labelled 'auto' stand for (with --from-sweeps)")
    a = ap.parse_args()
    if a.from_sweeps:
        table = table_from_sweeps(a.from_sweeps, a.ops.split(","), a.auto_is)
        with open(a.out, "w") as f:
            json.dump(table, f, indent=1)
        print(json.dumps(table))
        return
    rank, world, local = env_rank()
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    sizes, s = [], parse_size(a.min_bytes)
    while s <= parse_size(a.max_bytes):
        sizes.append(s)
        s *= a.factor
    table = {}
    for op in a.ops.split(","):
        meas = {}
        for algo, engine in CANDIDATES[op]:
            if algo == "mesh_oneshot":
                os.environ["HCCL_LL_MAX_BYTES"] = "0"
            for ctas in CTA_CHOICES:
                os.environ["HCCL_FORCE_CTAS"] = str(ctas)
                from .. import _lib
                _lib.load().HcommToolReloadEnv()
                box = [get_root_info() if rank == 0 else None]
                dist.broadcast_object_list(box, src=0)
                try:
                    comm = Communicator(world, box[0], rank, buffer_mb=512, algo=algo_config(op, algo, engine))
                except Exception:                                   # e.g. in-switch reduction not available
                    continue
                for nbytes in sizes:
                    if algo == "mesh_oneshot" and nbytes > (1 << 20):
                        continue
                    count = max(world, nbytes // 2) // world * world
                    x = torch.randn(count, device="cuda").to(torch.bfloat16)
                    y = torch.empty_like(x)
                    fn = {"allreduce": lambda: comm.all_reduce(x, y), "allgather": lambda: comm.all_gather(x[:count // world], y),
                          "reducescatter": lambda: comm.reduce_scatter(x, y[:count // world]), "alltoall": lambda: comm.all_to_all(x, y),
                          "broadcast": lambda: comm.broadcast(x, 0)}[op]
                    try:
                        med, _ = time_cuda(fn, a.iters, 3, nbytes < (160 << 20), dist.barrier)
                    except Exception:
                        continue
                    t = torch.tensor([med], device="cuda", dtype=torch.float64)
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                    meas.setdefault(selector_bytes(op, nbytes, world), {})[(algo, engine, ctas)] = t.item() * 1e3
                torch.cuda.synchronize()
                comm.destroy()
        table[op] = {str(world): merge_buckets(pick_winners(meas))}
    if rank == 0:
        with open(a.out, "w") as f:
            json.dump(table, f, indent=1)
        print(json.dumps(table))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
