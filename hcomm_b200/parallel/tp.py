"""Tensor-parallel building blocks on the fused GEMM + collective kernels.

Sequence-parallel convention: between layers the activations are sharded by rows (tokens); a
column-parallel linear gathers the rows while it multiplies (AllGather -> GEMM), a row-parallel linear
scatters the reduced rows while it multiplies (GEMM -> ReduceScatter).
"""
from __future__ import annotations

import torch

from ..comm import Communicator
from ..ops.fused import all_gather_gemm, gemm_reduce_scatter
from ..ops.gemm import gemm_bf16


class ColumnParallelLinear:
    """weight shard [out_features / tp, in_features]; input [tokens / tp, in_features] -> [tokens, out_features / tp]."""

    def __init__(self, comm: Communicator, weight_shard: torch.Tensor, mode: str = "auto"):
        self.comm, self.weight, self.mode = comm, weight_shard, mode

    def __call__(self, x_shard: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        if self.comm.size == 1:
            return gemm_bf16(x_shard, self.weight, out)
        return all_gather_gemm(self.comm, x_shard, self.weight, out, self.mode)


class RowParallelLinear:
    """weight shard [out_features, in_features / tp]; input [tokens, in_features / tp] -> [tokens / tp, out_features]."""

    def __init__(self, comm: Communicator, weight_shard: torch.Tensor, mode: str = "auto"):
        self.comm, self.weight, self.mode = comm, weight_shard, mode

    def __call__(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        if self.comm.size == 1:
            return gemm_bf16(x, self.weight, out)
        return gemm_reduce_scatter(self.comm, x, self.weight, out, self.mode)


class TensorParallelMlp:
    """Up projection (column-parallel) followed by down projection (row-parallel): the Llama-3-70B MLP shape
    of the tensor-parallel benchmark (hidden 8192, intermediate 28672).  Weights are random-initialised
    N(0, 0.02) shards unless given."""

    def __init__(self, comm: Communicator, hidden: int, intermediate: int, device=None, seed: int = 0, w_up=None, w_down=None, mode: str = "auto"):
        tp = comm.size
        assert intermediate % tp == 0
        dev = device or torch.device("cuda", torch.cuda.current_device())
        g = torch.Generator(device=dev).manual_seed(seed + 1000 * comm.rank)
        if w_up is None:
            w_up = (torch.randn(intermediate // tp, hidden, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        if w_down is None:
            w_down = (torch.randn(hidden, intermediate // tp, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        self.up, self.down = ColumnParallelLinear(comm, w_up, mode), RowParallelLinear(comm, w_down, mode)
        self.comm = comm
        self._h = None
        # kernels of this library per forward: one per projection; the split form adds the push / reduce-scatter kernel
        self.launches_per_step = 2 if (mode != "split" or comm.size == 1) else 4

    def forward(self, x_shard: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        tokens = x_shard.shape[0] * self.comm.size
        if self._h is None or self._h.shape[0] != tokens:
            self._h = torch.empty((tokens, self.up.weight.shape[0]), dtype=torch.bfloat16, device=x_shard.device)
        h = self.up(x_shard, self._h)
        return self.down(h, out)

    __call__ = forward
