"""Data parallelism over the ``hccl`` backend.

``fused_scale_hook`` is a DistributedDataParallel communication hook: every gradient bucket is reduced by ONE
kernel that sums the ranks' values in fp32, multiplies by 1/world_size and writes the bucket's dtype back
(HcclAllReduceScaled), instead of a division kernel followed by an all-reduce.  Buckets are reduced on the
backend's communication stream while autograd keeps producing the next bucket.
"""
import torch
import torch.distributed as dist
from torch.nn.parallel import DistributedDataParallel

from . import backend as _backend


class HookState:
    def __init__(self, group=None):
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self._native = None

    def native(self, device):
        if self._native is None:
            self._native = _backend.native_backend(self.group, device)
        return self._native


def fused_scale_hook(state: HookState, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    buf = bucket.buffer()
    work = state.native(buf.device).allreduce_scaled(buf, buf, 1.0 / state.world)
    return work.get_future().then(lambda f: f.value()[0])


def wrap(module: torch.nn.Module, *, group=None, bucket_cap_mb: int = 64, **ddp_kw) -> DistributedDataParallel:
    """DistributedDataParallel with the fused scale hook installed (gradients stay views of the buckets)."""
    dev = next(module.parameters()).device
    kw = dict(gradient_as_bucket_view=True, bucket_cap_mb=bucket_cap_mb, process_group=group)
    if dev.type == "cuda":
        kw["device_ids"] = [dev.index]
    kw.update(ddp_kw)
    ddp = DistributedDataParallel(module, **kw)
    ddp.register_comm_hook(HookState(group), fused_scale_hook)
    return ddp
