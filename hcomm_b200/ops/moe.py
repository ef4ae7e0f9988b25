"""Expert-parallel dispatch / combine for mixture-of-experts layers (``csrc/device/moe_kernels.cu``).

    moe = MoeExchange(comm, num_experts=256, topk=8, hidden=7168, max_tokens=4096)
    recv = moe.dispatch(x, topk_idx)          # x [T, H] bf16, topk_idx [T, k] int32 (global expert ids)
    ... run the local experts on recv.rows (fp8 e4m3) / recv.scales, grouped by recv.expert_offsets ...
    out = moe.combine(y, gates)               # y [recv.num_rows, H] bf16 in the received row order

``dispatch`` quantises every token once to fp8 e4m3 with one fp32 scale per 128 values and stores it directly
into the receive buffer of each rank that owns one of its experts; ``combine`` sends the expert outputs back
and applies the gate-weighted sum.  A combine must follow every dispatch before the next dispatch.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from .. import _lib
from ..comm import Communicator


class MoeLayout(ctypes.Structure):
    _fields_ = [("numExperts", ctypes.c_int32), ("topk", ctypes.c_int32), ("hidden", ctypes.c_int32), ("maxTokens", ctypes.c_int32),
                ("maxRecvRows", ctypes.c_int32), ("reserved", ctypes.c_int32), ("offCounts", ctypes.c_uint64), ("offExpertOffsets", ctypes.c_uint64),
                ("offOrigin", ctypes.c_uint64), ("offScales", ctypes.c_uint64), ("offRows", ctypes.c_uint64), ("offCombine", ctypes.c_uint64),
                ("totalBytes", ctypes.c_uint64), ("offValid", ctypes.c_uint64)]


class _DevView:
    """Exposes a raw device address to torch through the CUDA array interface."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 3, "strides": None}


def _view(ptr: int, shape, dtype: torch.dtype, device) -> torch.Tensor:
    typestr = {torch.uint8: "|u1", torch.float32: "<f4", torch.int32: "<i4", torch.int64: "<i8", torch.bfloat16: "<u2"}[dtype]
    t = torch.as_tensor(_DevView(ptr, shape, typestr), device=device)
    return t.view(torch.bfloat16) if dtype == torch.bfloat16 else t


@dataclass
class Received:
    rows: torch.Tensor            # [capacity, hidden] float8_e4m3fn (first num_rows valid), grouped by local expert
    scales: torch.Tensor          # [capacity, hidden // 128] float32
    origin: torch.Tensor          # [capacity] int64: (source rank << 32) | (token * topk + k)
    expert_offsets: torch.Tensor  # [experts_per_rank + 1] int32, on device

    @property
    def num_rows(self) -> int:
        return int(self.expert_offsets[-1].item())

    def dequantized(self, n: int | None = None) -> torch.Tensor:
        n = self.num_rows if n is None else n
        r = self.rows[:n].float().view(n, -1, 128) * self.scales[:n].unsqueeze(-1)
        return r.view(n, -1)


class MoeExchange:
    def __init__(self, comm: Communicator, num_experts: int, topk: int, hidden: int, max_tokens: int, capacity_factor: float = 2.0):
        self.comm, self.num_experts, self.topk, self.hidden, self.max_tokens = comm, num_experts, topk, hidden, max_tokens
        self._lib = _lib.load()
        self._h = ctypes.c_void_p()
        self.layout = MoeLayout()
        _lib.check(self._lib.HcommMoeCreate(ctypes.c_void_p(comm.handle), num_experts, topk, hidden, max_tokens, ctypes.c_float(capacity_factor),
                                            ctypes.byref(self._h), ctypes.byref(self.layout)), "HcommMoeCreate")
        ptrs = [ctypes.c_void_p() for _ in range(5)]
        _lib.check(self._lib.HcommMoeGetBuffers(self._h, *[ctypes.byref(p) for p in ptrs]), "HcommMoeGetBuffers")
        dev = torch.device("cuda", torch.cuda.current_device())
        cap, epr = self.layout.maxRecvRows, num_experts // comm.size
        self._rows = _view(ptrs[0].value, (cap, hidden), torch.uint8, dev).view(torch.float8_e4m3fn)
        self._scales = _view(ptrs[1].value, (cap, hidden // 128), torch.float32, dev)
        self._origin = _view(ptrs[2].value, (cap,), torch.int64, dev)
        self._offsets = _view(ptrs[3].value, (epr + 1,), torch.int32, dev)
        # one byte per (local token, k): 1 when the last dispatch sent that row, 0 when the index was masked or the row was dropped
        self.sent = _view(ptrs[0].value - self.layout.offRows + self.layout.offValid, (max_tokens, topk), torch.uint8, dev)

    def dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor) -> Received:
        assert x.dtype == torch.bfloat16 and x.is_contiguous() and x.shape[1] == self.hidden
        assert topk_idx.dtype == torch.int32 and topk_idx.is_contiguous() and topk_idx.shape == (x.shape[0], self.topk)
        stream = torch.cuda.current_stream(x.device).cuda_stream
        _lib.check(self._lib.HcommMoeDispatch(self._h, ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(topk_idx.data_ptr()), x.shape[0],
                                              ctypes.c_void_p(stream)), "HcommMoeDispatch")
        return Received(self._rows, self._scales, self._origin, self._offsets)

    def combine(self, y: torch.Tensor, gates: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        assert y.dtype == torch.bfloat16 and y.is_contiguous() and y.shape[1] == self.hidden
        assert gates.dtype == torch.float32 and gates.is_contiguous()
        t = gates.shape[0]
        if out is None:
            out = torch.empty((t, self.hidden), dtype=torch.bfloat16, device=y.device)
        stream = torch.cuda.current_stream(y.device).cuda_stream
        _lib.check(self._lib.HcommMoeCombine(self._h, ctypes.c_void_p(y.data_ptr()), ctypes.c_void_p(gates.data_ptr()), ctypes.c_void_p(out.data_ptr()), t,
                                             ctypes.c_void_p(stream)), "HcommMoeCombine")
        return out

    def overflow(self) -> int:
        return int(self._lib.HcommMoeTakeOverflow(self._h))

    def destroy(self):
        if self._h:
            _lib.check(self._lib.HcommMoeDestroy(self._h), "HcommMoeDestroy")
            self._h = ctypes.c_void_p()


def quantize_e4m3_1x128(x: torch.Tensor):
    """Reference quantiser with the kernel's rule: scale = max(|block|, 1e-4) / 448."""
    t, h = x.shape
    xb = x.float().view(t, h // 128, 128)
    amax = xb.abs().amax(dim=-1).clamp_min(1e-4)
    scale = amax / torch.full_like(amax, 448.0)     # tensor / tensor is a true division; tensor / python scalar multiplies by a rounded reciprocal
    q = (xb / scale.unsqueeze(-1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)   # saturate like the kernel does
    return q.view(t, h), scale
