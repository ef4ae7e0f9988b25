"""AllReduce inside a captured CUDA graph (reference sample: examples/02_aclgraphs/allreduce_aclgraph_demo.py).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/02_graphs/allreduce_cuda_graph_demo.py

Every rank captures one all-reduce of this library into a ``torch.cuda.CUDAGraph`` and replays it with new data in the
captured input buffer.  A captured launch replays correctly because what changes from call to call - the barrier
epoch, which half of the communication buffer the operator uses, the sequence numbers in its flags - lives in device
memory and is advanced by the kernels themselves; nothing the host counted is baked into the launch.
"""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent.parent))
import hcomm_b200 as hb  # noqa: E402


def main():
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("gloo")
        box = [hb.get_root_info() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        info = box[0]
    else:
        info = hb.get_root_info()
    comm = hb.Communicator(world, info, rank, buffer_mb=64)
    n = 1 << 20
    x = torch.zeros(n, device="cuda")
    y = torch.zeros(n, device="cuda")
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        x.fill_(float(rank + 1))
        comm.all_reduce(x, y)                 # warm-up outside the graph (first use of the kernels)
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        comm.all_reduce(x, y)
    for step in range(1, 6):
        x.fill_(float(rank + step))
        graph.replay()
        torch.cuda.synchronize()
        want = sum(float(r + step) for r in range(world))
        assert torch.all(y == want), (step, y[:4].tolist(), want)
    assert comm.async_error() == 0
    if rank == 0:
        print(f"allreduce_cuda_graph_demo: {world} ranks, 5 replays ok")
    comm.destroy()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
