"""Python face of the communicator API.

``Communicator`` wraps an ``HcclComm`` handle and accepts NumPy arrays (simulator platform) or torch
tensors (CUDA platform, or CPU tensors on the simulator).  Every method maps one-to-one onto a C entry
point of ``include/hccl/hccl.h`` / ``hccl_comm.h``; errors raise :class:`HcclError` carrying the
``HcclResult`` code.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import numpy as np

from . import _lib
from ._lib import HcclError, check

_NP_DTYPES = {
    np.dtype(np.int8): _lib.INT8, np.dtype(np.int16): _lib.INT16, np.dtype(np.int32): _lib.INT32, np.dtype(np.float16): _lib.FP16,
    np.dtype(np.float32): _lib.FP32, np.dtype(np.int64): _lib.INT64, np.dtype(np.uint64): _lib.UINT64, np.dtype(np.uint8): _lib.UINT8,
    np.dtype(np.uint16): _lib.UINT16, np.dtype(np.uint32): _lib.UINT32, np.dtype(np.float64): _lib.FP64,
}
_OPS = {"sum": _lib.SUM, "prod": _lib.PROD, "max": _lib.MAX, "min": _lib.MIN}


def _torch_dtype_code(dt):
    import torch
    table = {torch.int8: _lib.INT8, torch.int16: _lib.INT16, torch.int32: _lib.INT32, torch.float16: _lib.FP16, torch.float32: _lib.FP32,
             torch.int64: _lib.INT64, torch.uint8: _lib.UINT8, torch.float64: _lib.FP64, torch.bfloat16: _lib.BF16}
    for name, code in (("float8_e4m3fn", _lib.FP8E4M3), ("float8_e5m2", _lib.FP8E5M2), ("uint16", _lib.UINT16), ("uint32", _lib.UINT32),
                       ("uint64", _lib.UINT64)):
        if hasattr(torch, name):
            table[getattr(torch, name)] = code
    return table[dt]


def describe(buf):
    """(address, element count, HcclDataType, cuda stream or None) of an array-like."""
    if isinstance(buf, np.ndarray):
        if not buf.flags["C_CONTIGUOUS"]:
            raise ValueError("buffers must be contiguous")
        return buf.ctypes.data, buf.size, _NP_DTYPES[buf.dtype], None
    import torch
    if isinstance(buf, torch.Tensor):
        if not buf.is_contiguous():
            raise ValueError("buffers must be contiguous")
        stream = torch.cuda.current_stream(buf.device).cuda_stream if buf.is_cuda else None
        return buf.data_ptr(), buf.numel(), _torch_dtype_code(buf.dtype), stream
    raise TypeError(f"unsupported buffer type {type(buf)}")


def get_root_info() -> bytes:
    """Starts the rendezvous server in this process and returns the ticket to hand to every rank."""
    info = _lib.HcclRootInfo()
    check(_lib.load().HcclGetRootInfo(ctypes.byref(info)), "HcclGetRootInfo")
    return ctypes.string_at(ctypes.addressof(info), _lib.HCCL_ROOT_INFO_BYTES)


def _u64_array(values: Sequence[int]):
    return (ctypes.c_uint64 * len(values))(*[int(v) for v in values])


class Communicator:
    def __init__(self, n_ranks: int, root_info: bytes, rank: int, *, buffer_mb: Optional[int] = None, name: Optional[str] = None,
                 deterministic: Optional[int] = None, algo: Optional[str] = None, op_expansion_mode: Optional[int] = None,
                 exec_timeout: Optional[int] = None):
        self._lib = _lib.load()
        info = _lib.HcclRootInfo()
        ctypes.memmove(ctypes.addressof(info), root_info, min(len(root_info), _lib.HCCL_ROOT_INFO_BYTES))
        cfg = _lib.HcclCommConfig.default()
        if buffer_mb is not None:
            cfg.hcclBufferSize = buffer_mb
        if name is not None:
            cfg.hcclCommName = name.encode()
        if deterministic is not None:
            cfg.hcclDeterministic = deterministic
        if algo is not None:
            cfg.hcclAlgo = algo.encode()
        if op_expansion_mode is not None:
            cfg.hcclOpExpansionMode = op_expansion_mode
        if exec_timeout is not None:
            cfg.hcclExecTimeOut = exec_timeout
        self._h = ctypes.c_void_p()
        check(self._lib.HcclCommInitRootInfoConfig(n_ranks, ctypes.byref(info), rank, ctypes.byref(cfg), ctypes.byref(self._h)),
              "HcclCommInitRootInfoConfig")
        self.rank, self.size = rank, n_ranks

    @classmethod
    def from_handle(cls, handle: int) -> "Communicator":
        self = cls.__new__(cls)
        self._lib = _lib.load()
        self._h = ctypes.c_void_p(handle)
        r, n = ctypes.c_uint32(), ctypes.c_uint32()
        check(self._lib.HcclGetRankId(self._h, ctypes.byref(r)), "HcclGetRankId")
        check(self._lib.HcclGetRankSize(self._h, ctypes.byref(n)), "HcclGetRankSize")
        self.rank, self.size = r.value, n.value
        return self

    @classmethod
    def from_rank_table(cls, path: str, rank: int) -> "Communicator":
        self = cls.__new__(cls)
        self._lib = _lib.load()
        self._h = ctypes.c_void_p()
        check(self._lib.HcclCommInitClusterInfo(path.encode(), rank, ctypes.byref(self._h)), "HcclCommInitClusterInfo")
        n = ctypes.c_uint32()
        check(self._lib.HcclGetRankSize(self._h, ctypes.byref(n)), "HcclGetRankSize")
        self.rank, self.size = rank, n.value
        return self

    # ------------------------------------------------------------------ properties
    @property
    def handle(self) -> int:
        return self._h.value

    @property
    def name(self) -> str:
        buf = ctypes.create_string_buffer(128)
        check(self._lib.HcclGetCommName(self._h, buf), "HcclGetCommName")
        return buf.value.decode()

    def async_error(self) -> int:
        e = ctypes.c_int()
        check(self._lib.HcclGetCommAsyncError(self._h, ctypes.byref(e)), "HcclGetCommAsyncError")
        return e.value

    def split(self, rank_ids: Sequence[int], sub_id: int = 0, **cfg_kw) -> Optional["Communicator"]:
        """Sub communicator over ``rank_ids`` (ranks of this communicator); collective over the members."""
        if self.rank not in rank_ids:
            return None
        cfg = _lib.HcclCommConfig.default()
        if "buffer_mb" in cfg_kw:
            cfg.hcclBufferSize = cfg_kw["buffer_mb"]
        if "name" in cfg_kw:
            cfg.hcclCommName = cfg_kw["name"].encode()
        if "algo" in cfg_kw:
            cfg.hcclAlgo = cfg_kw["algo"].encode()
        if "deterministic" in cfg_kw:
            cfg.hcclDeterministic = cfg_kw["deterministic"]
        if "op_expansion_mode" in cfg_kw:
            cfg.hcclOpExpansionMode = cfg_kw["op_expansion_mode"]
        ids = (ctypes.c_uint32 * len(rank_ids))(*rank_ids)
        sub = ctypes.c_void_p()
        check(self._lib.HcclCreateSubCommConfig(ctypes.byref(self._h), len(rank_ids), ids, ctypes.c_uint64(sub_id), list(rank_ids).index(self.rank),
                                                ctypes.byref(cfg), ctypes.byref(sub)), "HcclCreateSubCommConfig")
        return Communicator.from_handle(sub.value)

    # ------------------------------------------------------------------ operators
    def _stream(self, stream, inferred):
        if stream is not None:
            return ctypes.c_void_p(int(stream))
        return ctypes.c_void_p(inferred) if inferred else None

    def all_reduce(self, send, recv=None, op: str = "sum", stream=None):
        recv = send if recv is None else recv
        sp, n, dt, st = describe(send)
        rp, _, _, _ = describe(recv)
        check(self._lib.HcclAllReduce(ctypes.c_void_p(sp), ctypes.c_void_p(rp), ctypes.c_uint64(n), dt, _OPS[op], self._h, self._stream(stream, st)),
              "HcclAllReduce")
        return recv

    def all_reduce_scaled(self, send, recv=None, scale: float = 1.0, stream=None):
        recv = send if recv is None else recv
        sp, n, dt, st = describe(send)
        rp, _, rdt, _ = describe(recv)
        check(self._lib.HcclAllReduceScaled(ctypes.c_void_p(sp), ctypes.c_void_p(rp), ctypes.c_uint64(n), dt, rdt, ctypes.c_float(scale), self._h,
                                            self._stream(stream, st)), "HcclAllReduceScaled")
        return recv

    def broadcast(self, buf, root: int = 0, stream=None):
        p, n, dt, st = describe(buf)
        check(self._lib.HcclBroadcast(ctypes.c_void_p(p), ctypes.c_uint64(n), dt, root, self._h, self._stream(stream, st)), "HcclBroadcast")
        return buf

    def reduce_scatter(self, send, recv, op: str = "sum", stream=None):
        sp, _, dt, st = describe(send)
        rp, n, _, _ = describe(recv)
        check(self._lib.HcclReduceScatter(ctypes.c_void_p(sp), ctypes.c_void_p(rp), ctypes.c_uint64(n), dt, _OPS[op], self._h, self._stream(stream, st)),
              "HcclReduceScatter")
        return recv

    def reduce_scatter_v(self, send, counts, displs, recv, op: str = "sum", stream=None):
        sp, _, dt, st = describe(send)
        rp, n, _, _ = describe(recv)
        check(self._lib.HcclReduceScatterV(ctypes.c_void_p(sp), _u64_array(counts), _u64_array(displs), ctypes.c_void_p(rp),
                                           ctypes.c_uint64(counts[self.rank]), dt, _OPS[op], self._h, self._stream(stream, st)), "HcclReduceScatterV")
        return recv

    def all_gather(self, send, recv, stream=None):
        sp, n, dt, st = describe(send)
        rp, _, _, _ = describe(recv)
        check(self._lib.HcclAllGather(ctypes.c_void_p(sp), ctypes.c_void_p(rp), ctypes.c_uint64(n), dt, self._h, self._stream(stream, st)), "HcclAllGather")
        return recv

    def all_gather_v(self, send, recv, counts, displs, stream=None):
        sp, _, dt, st = describe(send)
        rp, _, _, _ = describe(recv)
        check(self._lib.HcclAllGatherV(ctypes.c_void_p(sp), ctypes.c_uint64(counts[self.rank]), ctypes.c_void_p(rp), _u64_array(counts),
                                       _u64_array(displs), dt, self._h, self._stream(stream, st)), "HcclAllGatherV")
        return recv

    def all_to_all(self, send, recv, stream=None):
        sp, n, dt, st = describe(send)
        rp, _, _, _ = describe(recv)
        per = n // self.size
        check(self._lib.HcclAlltoAll(ctypes.c_void_p(sp), ctypes.c_uint64(per), dt, ctypes.c_void_p(rp), ctypes.c_uint64(per), dt, self._h,
                                     self._stream(stream, st)), "HcclAlltoAll")
        return recv

    def all_to_all_v(self, send, send_counts, send_displs, recv, recv_counts, recv_displs, stream=None):
        sp, _, dt, st = describe(send)
        rp, _, _, _ = describe(recv)
        check(self._lib.HcclAlltoAllV(ctypes.c_void_p(sp), _u64_array(send_counts), _u64_array(send_displs), dt, ctypes.c_void_p(rp),
                                      _u64_array(recv_counts), _u64_array(recv_displs), dt, self._h, self._stream(stream, st)), "HcclAlltoAllV")
        return recv

    def all_to_all_vc(self, send, count_matrix, recv, stream=None):
        sp, _, dt, st = describe(send)
        rp, _, _, _ = describe(recv)
        flat = [int(v) for row in count_matrix for v in row]
        check(self._lib.HcclAlltoAllVC(ctypes.c_void_p(sp), _u64_array(flat), dt, ctypes.c_void_p(rp), dt, self._h, self._stream(stream, st)),
              "HcclAlltoAllVC")
        return recv

    def reduce(self, send, recv, root: int = 0, op: str = "sum", stream=None):
        sp, n, dt, st = describe(send)
        rp = describe(recv)[0] if recv is not None else 0
        check(self._lib.HcclReduce(ctypes.c_void_p(sp), ctypes.c_void_p(rp), ctypes.c_uint64(n), dt, _OPS[op], root, self._h, self._stream(stream, st)),
              "HcclReduce")
        return recv

    def scatter(self, send, recv, root: int = 0, stream=None):
        rp, n, dt, st = describe(recv)
        sp = describe(send)[0] if send is not None else 0
        check(self._lib.HcclScatter(ctypes.c_void_p(sp), ctypes.c_void_p(rp), ctypes.c_uint64(n), dt, root, self._h, self._stream(stream, st)), "HcclScatter")
        return recv

    def gather(self, send, recv, root: int = 0, stream=None):
        sp, n, dt, st = describe(send)
        rp = describe(recv)[0] if recv is not None else 0
        check(self._lib.HcclGather(ctypes.c_void_p(sp), ctypes.c_void_p(rp), ctypes.c_uint64(n), dt, root, self._h, self._stream(stream, st)), "HcclGather")
        return recv

    def send(self, buf, dst: int, stream=None):
        p, n, dt, st = describe(buf)
        check(self._lib.HcclSend(ctypes.c_void_p(p), ctypes.c_uint64(n), dt, dst, self._h, self._stream(stream, st)), "HcclSend")

    def recv(self, buf, src: int, stream=None):
        p, n, dt, st = describe(buf)
        check(self._lib.HcclRecv(ctypes.c_void_p(p), ctypes.c_uint64(n), dt, src, self._h, self._stream(stream, st)), "HcclRecv")
        return buf

    def batch_send_recv(self, items, stream=None):
        """items: iterable of ("send" | "recv", buffer, peer)."""
        arr = (_lib.HcclSendRecvItem * len(items))()
        st0 = None
        for i, (kind, buf, peer) in enumerate(items):
            p, n, dt, st = describe(buf)
            st0 = st0 or st
            arr[i].sendRecvType = 0 if kind == "send" else 1
            arr[i].buf, arr[i].count, arr[i].dataType, arr[i].remoteRank = p, n, dt, peer
        check(self._lib.HcclBatchSendRecv(arr, len(items), self._h, self._stream(stream, st0)), "HcclBatchSendRecv")

    def barrier(self, stream=None):
        check(self._lib.HcclBarrier(self._h, self._stream(stream, None)), "HcclBarrier")

    # ------------------------------------------------------------------ diagnostics
    def set_profiling(self, enable: bool = True):
        """Operator records, device timestamps of the kernels and one NVTX range per operator, from now on."""
        check(self._lib.HcclDiagSetProfiling(self._h, 1 if enable else 0), "HcclDiagSetProfiling")

    def kernel_times(self):
        """[(start_ns, end_ns)] of the most recent kernels on the GPU's global timer, oldest first (profiling must be on;
        at most 16 are kept; a kernel that still runs has end 0)."""
        cap = 16
        start, end = (ctypes.c_uint64 * cap)(), (ctypes.c_uint64 * cap)()
        n = ctypes.c_uint32()
        check(self._lib.HcclDiagGetKernelTimes(self._h, start, end, cap, ctypes.byref(n)), "HcclDiagGetKernelTimes")
        return [(int(start[i]), int(end[i])) for i in range(n.value)]

    def dump(self) -> str:
        """The newest operator records and the device wait status, as text."""
        buf = ctypes.create_string_buffer(16384)
        check(self._lib.HcclDiagDump(self._h, buf, len(buf)), "HcclDiagDump")
        return buf.value.decode(errors="replace")

    def suspend(self):
        check(self._lib.HcclCommSuspend(self._h), "HcclCommSuspend")

    def resume(self):
        check(self._lib.HcclCommResume(self._h), "HcclCommResume")

    def recover(self, timeout: int = 30):
        """Collective over the ranks that are left after others were lost (the rank that hosted the rendezvous among them
        or not): returns ``(communicator over the survivors, old rank of every new rank)``.  This communicator stays as it is."""
        h, size = ctypes.c_void_p(), ctypes.c_uint32()
        old = (ctypes.c_uint32 * self.size)()
        check(self._lib.HcclCommRecover(self._h, ctypes.c_uint32(timeout), ctypes.byref(h), ctypes.byref(size), old), "HcclCommRecover")
        return Communicator.from_handle(h.value), list(old[:size.value])

    # ---------------------------------------------------------------- registered (symmetric) memory
    def alloc_registered(self, shape, dtype):
        """Collective: allocates exportable device memory of the given torch shape / dtype on every rank, registers it as a
        symmetric window and returns it as a torch tensor.  Operators whose buffers lie inside such a window read and
        write the ranks' copies in place (zero-copy) instead of staging through the CCL buffer.  Every rank must pass the
        same size.  The memory lives until the communicator is destroyed (or :meth:`free_registered`)."""
        import torch
        n = 1
        for s_ in (shape if isinstance(shape, (tuple, list)) else (shape,)):
            n *= int(s_)
        nbytes = max(16, n * torch.tensor([], dtype=dtype).element_size())
        ptr = ctypes.c_void_p()
        check(self._lib.HcommMemAlloc(ctypes.byref(ptr), ctypes.c_size_t(nbytes)), "HcommMemAlloc")
        win = ctypes.c_void_p()
        rc = self._lib.HcclCommSymWinRegister(self._h, ptr, ctypes.c_uint64(nbytes), ctypes.byref(win), 0)
        if rc != 0:
            self._lib.HcommMemFree(ptr)
            check(rc, "HcclCommSymWinRegister")
        typestr = {1: "|u1", 2: "<u2", 4: "<u4", 8: "<u8"}[torch.tensor([], dtype=dtype).element_size()]

        class _View:
            pass
        v = _View()
        v.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr.value, False), "version": 3, "strides": None}
        t = torch.as_tensor(v, device=torch.device("cuda", torch.cuda.current_device())).view(dtype).view(shape)
        if not hasattr(self, "_registered"):
            self._registered = {}
        self._registered[t.data_ptr()] = (ptr, win)
        return t

    def free_registered(self, tensor):
        """Collective: deregisters and frees a tensor obtained from :meth:`alloc_registered`."""
        ptr, win = self._registered.pop(tensor.data_ptr())
        check(self._lib.HcclCommSymWinDeregister(win), "HcclCommSymWinDeregister")
        check(self._lib.HcommMemFree(ptr), "HcommMemFree")

    # ---------------------------------------------------------------- host messages over the control plane
    def send_bytes(self, data: bytes, dst: int, tag: int = 0):
        """Sends a small host message (control data, not tensors) to rank ``dst``; complete when the call returns."""
        buf = (ctypes.c_char * max(1, len(data))).from_buffer_copy(data if data else b"\0")
        req = ctypes.c_void_p()
        check(self._lib.HcclIsend(buf, len(data), _lib.INT8, dst, tag, self._h, ctypes.byref(req)), "HcclIsend")
        done = ctypes.c_int()
        check(self._lib.HcclTestSome(1, ctypes.byref(req), ctypes.byref(done), None, None), "HcclTestSome")

    def probe_bytes(self, src: Optional[int] = None, tag: Optional[int] = None):
        """Takes the oldest queued message from ``src`` with ``tag`` (``None``: any) without waiting.  Returns
        ``(source, tag, bytes)`` or ``None`` when nothing has arrived."""
        class _Status(ctypes.Structure):
            _fields_ = [("srcRank", ctypes.c_int), ("tag", ctypes.c_int), ("error", ctypes.c_int), ("cancelled", ctypes.c_int), ("count", ctypes.c_int)]
        flag, msg, st = ctypes.c_int(), ctypes.c_void_p(), _Status()
        check(self._lib.HcclImprobe(-1 if src is None else src, -1 if tag is None else tag, self._h, ctypes.byref(flag), ctypes.byref(msg), ctypes.byref(st)),
              "HcclImprobe")
        if not flag.value:
            return None
        buf = ctypes.create_string_buffer(max(1, st.count))
        req = ctypes.c_void_p()
        check(self._lib.HcclImrecv(buf, st.count, _lib.INT8, ctypes.byref(msg), ctypes.byref(req)), "HcclImrecv")
        done = ctypes.c_int()
        check(self._lib.HcclTestSome(1, ctypes.byref(req), ctypes.byref(done), None, None), "HcclTestSome")
        return st.srcRank, st.tag, buf.raw[:st.count]

    def recv_bytes(self, src: Optional[int] = None, tag: Optional[int] = None, timeout: float = 30.0):
        """Waits for a message as :meth:`probe_bytes` describes it; ``TimeoutError`` after ``timeout`` seconds."""
        import time
        deadline = time.time() + timeout
        while True:
            got = self.probe_bytes(src, tag)
            if got is not None:
                return got
            if time.time() > deadline:
                raise TimeoutError(f"no message from rank {src} with tag {tag} within {timeout} s")
            time.sleep(0.0005)

    def destroy(self):
        if self._h:
            regs = getattr(self, "_registered", {})
            check(self._lib.HcclCommDestroy(self._h), "HcclCommDestroy")
            for ptr, _ in regs.values():
                self._lib.HcommMemFree(ptr)
            regs.clear()
            self._h = ctypes.c_void_p()


def group_start():
    check(_lib.load().HcclGroupStart(), "HcclGroupStart")


def group_end():
    check(_lib.load().HcclGroupEnd(), "HcclGroupEnd")
