"""ctypes binding of ``libhcomm.so``: loads the library (building it on first use) and declares
the C structures of ``include/hccl``."""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

_LIB = None

HCCL_ROOT_INFO_BYTES = 4108

# HcclDataType
INT8, INT16, INT32, FP16, FP32, INT64, UINT64, UINT8, UINT16, UINT32, FP64, BF16 = range(12)
FP8E4M3, FP8E5M2 = 15, 16
# HcclReduceOp
SUM, PROD, MAX, MIN = range(4)

ERROR_NAMES = {
    0: "HCCL_SUCCESS", 1: "HCCL_E_PARA", 2: "HCCL_E_PTR", 3: "HCCL_E_MEMORY", 4: "HCCL_E_INTERNAL", 5: "HCCL_E_NOT_SUPPORT",
    6: "HCCL_E_NOT_FOUND", 7: "HCCL_E_UNAVAIL", 8: "HCCL_E_SYSCALL", 9: "HCCL_E_TIMEOUT", 10: "HCCL_E_OPEN_FILE_FAILURE",
    11: "HCCL_E_TCP_CONNECT", 13: "HCCL_E_TCP_TRANSFER", 15: "HCCL_E_RUNTIME", 16: "HCCL_E_DRV", 19: "HCCL_E_NETWORK",
    20: "HCCL_E_AGAIN", 21: "HCCL_E_REMOTE", 22: "HCCL_E_SUSPENDING", 23: "HCCL_E_OPRETRY_FAIL", 24: "HCCL_E_OOM",
}


class HcclError(RuntimeError):
    def __init__(self, code: int, what: str):
        self.code = code
        super().__init__(f"{what} failed: {ERROR_NAMES.get(code, code)} ({code})")


class HcclRootInfo(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_char * HCCL_ROOT_INFO_BYTES)]


class HcclCommConfig(ctypes.Structure):
    _fields_ = [
        ("reserved", ctypes.c_char * 24),
        ("hcclBufferSize", ctypes.c_uint32),
        ("hcclDeterministic", ctypes.c_uint32),
        ("hcclCommName", ctypes.c_char * 128),
        ("hcclUdi", ctypes.c_char * 128),
        ("hcclOpExpansionMode", ctypes.c_uint32),
        ("hcclRdmaTrafficClass", ctypes.c_uint32),
        ("hcclRdmaServiceLevel", ctypes.c_uint32),
        ("hcclWorldRankID", ctypes.c_uint32),
        ("hcclJobID", ctypes.c_uint64),
        ("aclGraphZeroCopyEnable", ctypes.c_uint8),
        ("hcclExecTimeOut", ctypes.c_int32),
        ("hcclAlgo", ctypes.c_char * 1600),
        ("hcclRetryEnable", ctypes.c_char * 50),
        ("hcclRetryParams", ctypes.c_char * 128),
        ("hcclBufferName", ctypes.c_char * 128),
        ("hcclQos", ctypes.c_uint32),
        ("hcclSymWinMaxMemSizePerRank", ctypes.c_uint64),
        ("hcclChannelSqDepth", ctypes.c_uint32),
    ]

    class _Header(ctypes.Structure):
        _fields_ = [("size", ctypes.c_size_t), ("magicWord", ctypes.c_uint32), ("version", ctypes.c_uint32), ("reserved", ctypes.c_uint64)]

    @classmethod
    def default(cls) -> "HcclCommConfig":
        """Python rendering of the inline C function HcclCommConfigInit."""
        cfg = cls()
        hdr = cls._Header.from_buffer(cfg)
        hdr.size = ctypes.sizeof(cls)
        hdr.magicWord = 0xF0F0F0F0
        hdr.version = 11
        cfg.hcclBufferSize = 0xFFFFFFFF
        cfg.hcclDeterministic = 0xFFFFFFFF
        cfg.hcclRdmaTrafficClass = 0xFFFFFFFF
        cfg.hcclRdmaServiceLevel = 0xFFFFFFFF
        cfg.hcclExecTimeOut = -1
        cfg.hcclQos = 0xFFFFFFFF
        cfg.hcclSymWinMaxMemSizePerRank = 16
        cfg.hcclChannelSqDepth = 0xFFFFFFFF
        return cfg


class HcclSendRecvItem(ctypes.Structure):
    _fields_ = [("sendRecvType", ctypes.c_int), ("buf", ctypes.c_void_p), ("count", ctypes.c_uint64), ("dataType", ctypes.c_int),
                ("remoteRank", ctypes.c_uint32)]


def lib_path() -> Path:
    # HCOMM_LIBRARY=bounds selects the bounds-checking build, HCOMM_LIBRARY=asan the AddressSanitizer build of the host runtime
    # (hcomm_b200.build.build_core(bounds=True) / (asan=True))
    name = {"bounds": "libhcomm_bounds.so", "asan": "libhcomm_asan.so", "tsan": "libhcomm_tsan.so", "ubsan": "libhcomm_ubsan.so", "cov": "libhcomm_cov.so"}.get(os.environ.get("HCOMM_LIBRARY", ""), "libhcomm.so")
    return Path(__file__).resolve().parent / "lib" / name


def load() -> ctypes.CDLL:
    """Returns the loaded library.  Builds it when the shared object is missing and the sources are present."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = lib_path()
    if not path.exists() or os.environ.get("HCOMM_REBUILD") == "1":
        from . import build
        build.build_core(bounds=os.environ.get("HCOMM_LIBRARY") == "bounds", asan=os.environ.get("HCOMM_LIBRARY") == "asan",
                         tsan=os.environ.get("HCOMM_LIBRARY") == "tsan", ubsan=os.environ.get("HCOMM_LIBRARY") == "ubsan",
                         cov=os.environ.get("HCOMM_LIBRARY") == "cov")
    _LIB = ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
    _LIB.HcclGetErrorString.restype = ctypes.c_char_p
    return _LIB


def check(code: int, what: str) -> None:
    if code != 0:
        raise HcclError(code, what)
