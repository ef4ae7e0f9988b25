"""hcomm_b200 - a Blackwell-native collective communication library with the HCCL / HCOMM API.

Layout
    hcomm_b200.comm      Communicator (ctypes over libhcomm.so), group calls
    hcomm_b200.ops       fused compute + collective operators and their unfused baselines
    hcomm_b200.parallel  tensor / expert / data parallel building blocks, torch ProcessGroup backend
    hcomm_b200.models    reference model definitions used by the benchmarks
    hcomm_b200.utils     launch helpers, tuning, timing
The C ABI (headers under ``include/``) is served by ``hcomm_b200/lib/libhcomm.so``.
"""
from ._lib import HcclError, load as load_library  # noqa: F401
from .comm import Communicator, get_root_info, group_end, group_start  # noqa: F401

__version__ = "0.1.0"
