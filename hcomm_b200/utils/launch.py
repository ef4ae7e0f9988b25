"""Bringing a communicator up from the environment of a multi-process launcher.

``init_from_env()`` reads RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT (what
``torch.distributed.run`` exports), binds the process to its GPU, lets rank 0 create the rendezvous
ticket and distributes it through a ``torch.distributed.TCPStore`` on MASTER_PORT + ``port_offset``.
"""
from __future__ import annotations

import os
from datetime import timedelta

from ..comm import Communicator, get_root_info


def env_rank() -> tuple[int, int, int]:
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", os.environ.get("RANK", "0")))


def exchange_root_info(rank: int, world: int, key: str = "hccl_root_info", port_offset: int = 17, store=None) -> bytes:
    if world == 1:
        return get_root_info()
    import torch.distributed as dist
    if store is None:
        addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
        port = int(os.environ.get("MASTER_PORT", "29500")) + port_offset
        store = dist.TCPStore(addr, port, world, is_master=(rank == 0), timeout=timedelta(seconds=120), wait_for_workers=False)
    if rank == 0:
        store.set(key, get_root_info())
    return bytes(store.get(key))


def init_from_env(set_device: bool = True, **comm_kwargs) -> Communicator:
    rank, world, local = env_rank()
    if set_device:
        try:
            import torch
            if torch.cuda.is_available():
                torch.cuda.set_device(local % torch.cuda.device_count())
        except ImportError:
            pass
    info = exchange_root_info(rank, world)
    return Communicator(world, info, rank, **comm_kwargs)
