"""MoE dispatch / combine kernels, ranks sharing one GPU, against a PyTorch reference of the same routing."""
import pytest
import torch

from helpers import run_ranks

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,experts,topk,hidden,tokens", [(2, 8, 2, 512, 64), (4, 16, 4, 1024, 96), (2, 32, 8, 7168, 128)])
def test_dispatch_and_combine(n, experts, topk, hidden, tokens):
    import hcomm_b200 as hb
    from hcomm_b200.ops.moe import MoeExchange, quantize_e4m3_1x128
    info = hb.get_root_info()

    def init(r):
        torch.cuda.set_device(0)
        return hb.Communicator(n, info, r, buffer_mb=8)
    comms = run_ranks(n, init)
    moes = run_ranks(n, lambda r: (torch.cuda.set_device(0), MoeExchange(comms[r], experts, topk, hidden, tokens))[1])
    try:
        epr = experts // n
        g = torch.Generator(device="cuda").manual_seed(7)
        xs = [torch.randn(tokens, hidden, device="cuda", generator=g).to(torch.bfloat16) for _ in range(n)]
        idx = [torch.stack([torch.randperm(experts, device="cuda", generator=g)[:topk] for _ in range(tokens)]).to(torch.int32).contiguous() for _ in range(n)]
        gates = [torch.rand(tokens, topk, device="cuda", generator=g).float().contiguous() for _ in range(n)]
        outs = [None] * n
        recv_snap = [None] * n
        for rep in range(2):
            def op(r):
                torch.cuda.set_device(0)
                rec = moes[r].dispatch(xs[r], idx[r])
                torch.cuda.synchronize()
                nrows = rec.num_rows
                recv_snap[r] = (rec.rows[:nrows].clone(), rec.scales[:nrows].clone(), rec.origin[:nrows].clone(), rec.expert_offsets.clone())
                # "expert": y = 2 * dequantised row + local expert index
                deq = rec.dequantized(nrows)
                offs = rec.expert_offsets.tolist()
                y = torch.empty(nrows, hidden, device="cuda", dtype=torch.bfloat16)
                for el in range(epr):
                    y[offs[el]:offs[el + 1]] = (2 * deq[offs[el]:offs[el + 1]] + el).to(torch.bfloat16)
                outs[r] = moes[r].combine(y, gates[r])
                torch.cuda.synchronize()
            run_ranks(n, op)
            assert all(m.overflow() == 0 for m in moes)
            for r in range(n):
                rows, scales, origin, offs = recv_snap[r]
                offs = offs.tolist()
                expected_total = sum(int(((idx[s] // epr) == r).sum().item()) for s in range(n))
                assert offs[-1] == expected_total
                for el in range(epr):
                    e = r * epr + el
                    seg = slice(offs[el], offs[el + 1])
                    src_rank = (origin[seg] >> 32).tolist()
                    tk = (origin[seg] & 0xffffffff).tolist()
                    assert src_rank == sorted(src_rank), "rows of one expert are grouped by source rank"
                    want = sorted((s, int(t) * topk + int(k)) for s in range(n) for t, k in (idx[s] == e).nonzero().tolist())
                    assert sorted(zip(src_rank, tk)) == want
                    for i, (s, key) in enumerate(zip(src_rank, tk)):
                        if i % 7:      # spot-check rows
                            continue
                        q, sc = quantize_e4m3_1x128(xs[s][key // topk:key // topk + 1])
                        assert torch.equal(rows[offs[el] + i].view(torch.uint8), q[0].view(torch.uint8))
                        assert torch.allclose(scales[offs[el] + i], sc[0])
            for r in range(n):
                q, sc = quantize_e4m3_1x128(xs[r])
                deq = (q.float().view(tokens, -1, 128) * sc.unsqueeze(-1)).view(tokens, hidden)
                ref = torch.zeros(tokens, hidden, device="cuda")
                for k in range(topk):
                    el = (idx[r][:, k] % epr).float().unsqueeze(1)
                    ref += gates[r][:, k:k + 1] * (2 * deq + el).to(torch.bfloat16).float()
                err = (outs[r].float() - ref).abs().max().item()
                assert err <= 3e-2 * max(1.0, ref.abs().max().item()), (rep, r, err)
    finally:
        run_ranks(n, lambda r: moes[r].destroy())
        run_ranks(n, lambda r: comms[r].destroy())


@pytest.mark.parametrize("capacity_factor,masked", [(2.0, True), (0.3, False)])
def test_masked_experts_and_dropped_rows_stay_out_of_the_sum(capacity_factor, masked):
    """An expert index outside the range masks that choice, and rows beyond the receive capacity are dropped: combine must
    add neither - the landing slot of such a (token, k) holds whatever an earlier step left there."""
    import hcomm_b200 as hb
    from hcomm_b200.ops.moe import MoeExchange, quantize_e4m3_1x128
    n, experts, topk, hidden, tokens = 2, 8, 4, 512, 64
    info = hb.get_root_info()

    def init(r):
        torch.cuda.set_device(0)
        return hb.Communicator(n, info, r, buffer_mb=8)
    comms = run_ranks(n, init)
    moes = run_ranks(n, lambda r: (torch.cuda.set_device(0), MoeExchange(comms[r], experts, topk, hidden, tokens, capacity_factor=capacity_factor))[1])
    try:
        g = torch.Generator(device="cuda").manual_seed(3)
        xs = [torch.randn(tokens, hidden, device="cuda", generator=g).to(torch.bfloat16) for _ in range(n)]
        gates = [torch.rand(tokens, topk, device="cuda", generator=g).float().contiguous() for _ in range(n)]
        outs, sent = [None] * n, [None] * n
        for step in range(2):
            # step 0 fills every landing slot with large values (nothing masked), step 1 is the one that is checked
            idx = [torch.stack([torch.randperm(experts, device="cuda", generator=g)[:topk] for _ in range(tokens)]).to(torch.int32).contiguous() for _ in range(n)]
            if masked and step == 1:
                for r in range(n):
                    idx[r][::3, 1] = -1
                    idx[r][1::5, 3] = experts + 7
            scale = 1000.0 if step == 0 else 1.0

            def op(r):
                torch.cuda.set_device(0)
                rec = moes[r].dispatch(xs[r], idx[r])
                torch.cuda.synchronize()
                nrows = rec.num_rows
                offs = rec.expert_offsets.tolist()
                assert all(0 <= o <= moes[r].layout.maxRecvRows for o in offs) and offs == sorted(offs)
                y = (rec.dequantized(nrows) * scale).to(torch.bfloat16)
                outs[r] = moes[r].combine(y, gates[r])
                torch.cuda.synchronize()
                sent[r] = moes[r].sent[:tokens].clone()
            run_ranks(n, op)
            dropped = sum(m.overflow() for m in moes)
            if step == 0:
                continue
            if capacity_factor < 1:
                assert dropped > 0, "the capacity was meant to overflow"
            for r in range(n):
                in_range = (idx[r] >= 0) & (idx[r] < experts)
                assert torch.all(sent[r].bool() <= in_range), "a masked choice was marked as sent"
                if capacity_factor >= 1:
                    assert torch.equal(sent[r].bool(), in_range)
                q, sc = quantize_e4m3_1x128(xs[r])
                deq = (q.float().view(tokens, -1, 128) * sc.unsqueeze(-1)).view(tokens, hidden).to(torch.bfloat16).float()
                ref = deq * (gates[r] * sent[r].float()).sum(dim=1, keepdim=True)
                assert torch.isfinite(outs[r].float()).all()
                err = (outs[r].float() - ref).abs().max().item()
                assert err <= 3e-2 * max(1.0, ref.abs().max().item()), (r, err)
    finally:
        run_ranks(n, lambda r: moes[r].destroy())
        run_ranks(n, lambda r: comms[r].destroy())
