"""torch.distributed backend ``"hccl"``.

    import hcomm_b200.parallel.backend            # registers the backend
    torch.distributed.init_process_group("hccl", ...)

The backend object is the C++ class ``ProcessGroupHCCL`` (csrc/torch/process_group_hccl.cpp): one communicator per
process group, operators on a dedicated communication stream, ``Work.wait()`` stream-ordered.  CUDA tensors use the
GPU platform; CPU tensors are served when the library runs on its host simulator (``HCCL_SIM=1``), which is how the
backend is tested without a GPU.

The role is that of the reference's ``torch_npu`` process group over the same C API (reference: python/hccl/manage/api.py
exposes the communicator management that backend sits on).
"""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import torch
import torch.distributed as dist

from .. import _lib
from ..comm import Communicator

_EXT = None
BACKEND_NAME = "hccl"


def extension():
    """The compiled extension module; built on first use when the shared object is missing."""
    global _EXT
    if _EXT is not None:
        return _EXT
    _lib.load()                                   # libhcomm.so first: the extension links against it
    path = Path(__file__).resolve().parent.parent / "lib" / "_hcomm_torch.so"
    if not path.exists():
        from .. import build
        build.build_torch_extension()
    spec = importlib.util.spec_from_file_location("_hcomm_torch", str(path))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules["_hcomm_torch"] = mod
    _EXT = mod
    return mod


def _create(store, rank, size, timeout):
    return extension().create_backend(store, rank, size, timeout)


def register() -> None:
    """Registers the backend with torch.distributed (idempotent)."""
    if hasattr(dist.Backend, BACKEND_NAME.upper()):
        return
    dist.Backend.register_backend(BACKEND_NAME, _create, devices=["cuda", "cpu"])


def native_backend(group=None, device: torch.device | None = None):
    """The ``ProcessGroupHCCL`` object behind a torch process group (default group when None)."""
    group = group if group is not None else dist.group.WORLD
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    return group._get_backend(device)


def communicator_of(group=None, device: torch.device | None = None) -> Communicator:
    """The library communicator of a torch process group, for the C API and the fused operators."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    return Communicator.from_handle(native_backend(group, device).comm_handle(device))


register()
