"""Fused GEMM + collective kernels, ranks sharing one GPU in one cooperative launch, against plain
PyTorch fp32 references."""
import pytest
import torch

from helpers import run_ranks

pytestmark = pytest.mark.gpu


def _make(n, buffer_mb):
    import hcomm_b200 as hb
    info = hb.get_root_info()

    def init(r):
        torch.cuda.set_device(0)
        return hb.Communicator(n, info, r, buffer_mb=buffer_mb)
    return run_ranks(n, init)


@pytest.mark.parametrize("n,m,nn,k", [(2, 512, 512, 256), (4, 1024, 256, 192), (2, 256, 1024, 1024), (1, 256, 256, 128)])
def test_gemm_reduce_scatter(n, m, nn, k):
    from hcomm_b200.ops.fused import gemm_reduce_scatter
    from hcomm_b200.ops.gemm import take_kernel_error
    comms = _make(n, 16)
    try:
        torch.manual_seed(1)
        a = [torch.randn(m, k, device="cuda").to(torch.bfloat16) for _ in range(n)]
        b = [(torch.randn(nn, k, device="cuda") * 0.1).to(torch.bfloat16) for _ in range(n)]
        outs = [None] * n
        for rep in range(3):     # arrival counters must keep working across calls
            def op(r):
                torch.cuda.set_device(0)
                outs[r] = gemm_reduce_scatter(comms[r], a[r], b[r])
                torch.cuda.synchronize()
            run_ranks(n, op)
            assert take_kernel_error() == 0
            ref = sum(a[r].float() @ b[r].float().t() for r in range(n))
            rows = m // n
            for r in range(n):
                err = (outs[r].float() - ref[r * rows:(r + 1) * rows]).abs().max().item()
                assert err <= 2e-2 * max(1.0, ref.abs().max().item()), (rep, r, err)
            assert all(c.async_error() == 0 for c in comms)
    finally:
        run_ranks(n, lambda r: comms[r].destroy())


@pytest.mark.parametrize("n,ms,nn,k", [(2, 256, 256, 256), (4, 128, 512, 320), (2, 512, 128, 1024), (1, 256, 256, 64)])
def test_all_gather_gemm(n, ms, nn, k):
    from hcomm_b200.ops.fused import all_gather_gemm
    from hcomm_b200.ops.gemm import take_kernel_error
    comms = _make(n, 16)
    try:
        torch.manual_seed(2)
        x = [torch.randn(ms, k, device="cuda").to(torch.bfloat16) for _ in range(n)]
        w = [(torch.randn(nn, k, device="cuda") * 0.1).to(torch.bfloat16) for _ in range(n)]
        outs = [None] * n
        for rep in range(3):
            def op(r):
                torch.cuda.set_device(0)
                outs[r] = all_gather_gemm(comms[r], x[r], w[r])
                torch.cuda.synchronize()
            run_ranks(n, op)
            assert take_kernel_error() == 0
            full = torch.cat(x).float()
            for r in range(n):
                ref = full @ w[r].float().t()
                err = (outs[r].float() - ref).abs().max().item()
                assert err <= 2e-2 * max(1.0, ref.abs().max().item()), (rep, r, err)
    finally:
        run_ranks(n, lambda r: comms[r].destroy())


def test_fused_ops_interleave_with_collectives(n=2):
    from hcomm_b200.ops.fused import all_gather_gemm, gemm_reduce_scatter
    comms = _make(n, 16)
    try:
        a = [torch.randn(256, 128, device="cuda").to(torch.bfloat16) for _ in range(n)]
        b = [torch.randn(256, 128, device="cuda").to(torch.bfloat16) for _ in range(n)]
        w2 = [torch.randn(128, 256, device="cuda").to(torch.bfloat16) for _ in range(n)]
        v = [torch.full((1000,), float(r + 1), device="cuda") for r in range(n)]
        res = [None] * n

        def op(r):
            torch.cuda.set_device(0)
            c = comms[r]
            y1 = gemm_reduce_scatter(c, a[r], b[r])
            c.all_reduce(v[r])
            y2 = all_gather_gemm(c, y1, w2[r])
            c.all_reduce(v[r])
            torch.cuda.synchronize()
            res[r] = (y1, y2)
        run_ranks(n, op)
        s = sum(range(1, n + 1))
        assert (v[0] == s * n).all()
        ref1 = sum(a[r].float() @ b[r].float().t() for r in range(n))
        for r in range(n):
            assert torch.allclose(res[r][0].float(), ref1[r * 128:(r + 1) * 128], atol=0.6, rtol=3e-2)
    finally:
        run_ranks(n, lambda r: comms[r].destroy())


def test_fused_ops_with_changing_shapes():
    """Arrival counters are shared by all calls on a communicator: shapes that change from call to call (other
    numbers of tiles and row blocks) must not disturb each other."""
    from hcomm_b200.ops.fused import all_gather_gemm, gemm_reduce_scatter
    from hcomm_b200.ops.gemm import take_kernel_error
    n = 2
    comms = _make(n, 16)
    try:
        torch.manual_seed(5)
        shapes = [(512, 512, 256), (256, 256, 128), (1024, 256, 192), (512, 512, 256), (256, 768, 64)]
        for i, (m, nn, k) in enumerate(shapes):
            a = [torch.randn(m, k, device="cuda").to(torch.bfloat16) for _ in range(n)]
            b = [(torch.randn(nn, k, device="cuda") * 0.1).to(torch.bfloat16) for _ in range(n)]
            x = [torch.randn(m // n, k, device="cuda").to(torch.bfloat16) for _ in range(n)]
            outs, outs2 = [None] * n, [None] * n

            def op(r):
                torch.cuda.set_device(0)
                outs[r] = gemm_reduce_scatter(comms[r], a[r], b[r])
                outs2[r] = all_gather_gemm(comms[r], x[r], b[r])
                torch.cuda.synchronize()
            run_ranks(n, op)
            assert take_kernel_error() == 0, i
            ref = sum(a[r].float() @ b[r].float().t() for r in range(n))
            rows = m // n
            xa = torch.cat(x).float()
            for r in range(n):
                err = (outs[r].float() - ref[r * rows:(r + 1) * rows]).abs().max().item()
                assert err <= 2e-2 * max(1.0, ref.abs().max().item()), ("rs", i, r, err)
                ref2 = xa @ b[r].float().t()
                err2 = (outs2[r].float() - ref2).abs().max().item()
                assert err2 <= 2e-2 * max(1.0, ref2.abs().max().item()), ("ag", i, r, err2)
    finally:
        run_ranks(n, lambda r: comms[r].destroy())
