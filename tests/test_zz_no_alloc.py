"""HcommMoeDispatchStaticScratch: the dispatch kernel with its counters in the library's built-in device array.

Called through the exported C symbol and compared with HcommMoeDispatch on the same inputs, twice in a row with
different inputs (the second call finds the first call's leftovers in the shared array).
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

HCCL_E_PARA = 1


def _snapshot(moe, rec):
    """Received rows in a canonical order: the position inside an expert's segment depends on atomics."""
    n = rec.num_rows
    origin = rec.origin[:n].clone()
    order = torch.argsort(origin)
    offs = rec.expert_offsets.clone()
    seg = torch.bucketize(torch.arange(n, device=origin.device), offs[1:].long(), right=True)   # expert of every row
    return offs, origin[order], rec.rows[:n].view(torch.uint8)[order].clone(), rec.scales[:n][order].clone(), seg[order]


def test_static_scratch_dispatch_matches_allocating_dispatch():
    import hcomm_b200 as hb
    from hcomm_b200 import _lib
    from hcomm_b200.ops.moe import MoeExchange, Received

    torch.cuda.set_device(0)
    lib = _lib.load()
    fn = lib.HcommMoeDispatchStaticScratch
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]

    comm = hb.Communicator(1, hb.get_root_info(), 0, buffer_mb=8)
    experts, topk, hidden, tokens = 16, 4, 1024, 96
    moe = MoeExchange(comm, experts, topk, hidden, tokens)
    big = MoeExchange(comm, 512, 2, 512, 8)
    try:
        g = torch.Generator(device="cuda").manual_seed(11)
        stream = torch.cuda.current_stream().cuda_stream
        cases = []
        for _ in range(2):
            x = torch.randn(tokens, hidden, device="cuda", generator=g).to(torch.bfloat16)
            idx = torch.stack([torch.randperm(experts, device="cuda", generator=g)[:topk] for _ in range(tokens)]).to(torch.int32).contiguous()
            rec = moe.dispatch(x, idx)
            torch.cuda.synchronize()
            cases.append((x, idx, _snapshot(moe, rec)))
        received = Received(moe._rows, moe._scales, moe._origin, moe._offsets)
        for x, idx, want in cases:          # two calls of the new entry point in a row
            torch.cuda.synchronize()
            free_before, allocated_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
            rc = fn(moe._h, ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(idx.data_ptr()), tokens, ctypes.c_void_p(stream))
            assert rc == 0
            torch.cuda.synchronize()
            # the call took no memory from the driver nor from torch's allocator
            assert torch.cuda.mem_get_info()[0] == free_before and torch.cuda.memory_allocated() == allocated_before
            got = _snapshot(moe, received)
            assert torch.equal(got[0], want[0]), "expert offsets"
            assert torch.equal(got[1], want[1]), "origins"
            assert torch.equal(got[2], want[2]), "fp8 rows"
            assert torch.allclose(got[3], want[3], rtol=1e-6, atol=0), "scales"
            assert torch.equal(got[4], want[4]), "rows sit in the same expert's segment"
        assert moe.overflow() == 0 and comm.async_error() == 0
        # more experts than the built-in array serves: refused, nothing launched
        x = torch.zeros(8, 512, device="cuda", dtype=torch.bfloat16)
        idx = torch.zeros(8, 2, device="cuda", dtype=torch.int32)
        assert fn(big._h, ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(idx.data_ptr()), 8, ctypes.c_void_p(stream)) == HCCL_E_PARA
        # called with another device current: the built-in table belongs to the exchange's GPU, the call is refused before anything is queued
        if torch.cuda.device_count() > 1:
            x2, idx2 = cases[0][0], cases[0][1]
            torch.cuda.set_device(1)
            try:
                assert fn(moe._h, ctypes.c_void_p(x2.data_ptr()), ctypes.c_void_p(idx2.data_ptr()), tokens, ctypes.c_void_p(stream)) == HCCL_E_PARA
            finally:
                torch.cuda.set_device(0)
    finally:
        big.destroy()
        moe.destroy()
        comm.destroy()
