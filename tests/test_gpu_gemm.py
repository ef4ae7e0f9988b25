"""Numerics of the tcgen05 GEMM against a plain PyTorch fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 512), (256, 512, 256), (1024, 1024, 1024), (384, 128, 192), (200, 136, 72),
                                   (2048, 3584, 1024)])
def test_gemm_matches_fp32_reference(m, n, k):
    from hcomm_b200.ops.gemm import gemm_bf16, take_kernel_error
    torch.manual_seed(m * 7 + n * 3 + k)
    a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    b = (torch.randn(n, k, device="cuda", dtype=torch.float32) * 0.05).to(torch.bfloat16)
    c = gemm_bf16(a, b)
    torch.cuda.synchronize()
    assert take_kernel_error() == 0
    ref = a.float() @ b.float().t()
    err = (c.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * max(scale, 1.0), f"max abs err {err} vs scale {scale}"


def test_gemm_strided_operands():
    from hcomm_b200.ops.gemm import gemm_bf16
    a_full = torch.randn(256, 1024, device="cuda", dtype=torch.bfloat16)
    b_full = torch.randn(512, 1024, device="cuda", dtype=torch.bfloat16)
    a, b = a_full[:, 256:768], b_full[:, 256:768]   # K slice: pitch 1024, 512 columns used
    c = gemm_bf16(a, b)
    ref = a.float() @ b.float().t()
    assert torch.allclose(c.float(), ref, atol=0.5, rtol=2e-2)


@pytest.mark.parametrize("m,n,k,group", [(512, 1024, 256, 0), (2048, 4096, 1032, 0), (4096, 8192, 512, 12), (256, 512, 72, 1)])
def test_wide_tile_kernel_matches_fp32_reference(m, n, k, group):
    # 256 x 512 tiles (one accumulator, TMA-store epilogue) forced for shapes the selection rule would give narrower tiles,
    # including more tiles than CTA pairs, a K that is not a multiple of the 64-wide block, and a strided result
    from hcomm_b200 import _lib
    from hcomm_b200.ops.gemm import gemm_bf16, take_kernel_error
    lib = _lib.load()
    torch.manual_seed(m + n + k)
    a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    b = (torch.randn(n, k, device="cuda", dtype=torch.float32) * 0.05).to(torch.bfloat16)
    out_full = torch.zeros(m, n + 64, device="cuda", dtype=torch.bfloat16)
    out = out_full[:, :n]                       # pitch n + 64: the columns beyond n must stay untouched
    lib.HcommGemmSetTuning(group, 512)
    try:
        gemm_bf16(a, b, out)
        torch.cuda.synchronize()
    finally:
        lib.HcommGemmSetTuning(0, 0)
    assert take_kernel_error() == 0
    ref = a.float() @ b.float().t()
    err = (out.float() - ref).abs().max().item()
    assert err <= 1e-2 * max(ref.abs().max().item(), 1.0), f"max abs err {err}"
    assert out_full[:, n:].abs().max().item() == 0
