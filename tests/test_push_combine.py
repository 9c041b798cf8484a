"""GEMM fused with the combine all-to-all (push epilogue) on a single-GPU virtual group: each
virtual rank's down-projection GEMM stores its result rows straight into the home ranks' staging
slots; ``combine_pushed`` then sums K rows per token.  Checked against a PyTorch fp32 reference
and against the unfused path (GEMM into the shard, then the pull combine)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _cleanup():
    yield
    from moonep_b200.api import destroy_live_buffers
    destroy_live_buffers()
    torch.cuda.synchronize()


@pytest.mark.parametrize("R,maxvio", [(1, 0.0), (4, 3.0), (2, 0.0)])
def test_push_combine_matches_reference_and_unfused(R, maxvio):
    from moonep_b200 import Buffer
    from moonep_b200.ops import gemm
    from moonep_b200.utils.routing import routing_for_maxvio, tokens_per_expert
    S, K, E, H, Hp, tp = 128, 4, 4 * R, 256, 128, 64
    epn = E // R
    buf = Buffer(S, H, K, E, R, num_sms=2, token_padding=tp, virtual=True, timeout_s=3.0)
    topk, w, _, _ = routing_for_maxvio(S, K, E, R, maxvio, seed=21)
    tpe = torch.stack([tokens_per_expert(topk[r], E) for r in range(R)]).cuda()
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(R, S, H, device="cuda", generator=g).bfloat16()
    wd_all = (torch.randn(E, H, Hp, device="cuda", generator=g) * 0.08).bfloat16()
    proj = (torch.randn(H, Hp, device="cuda", generator=g) * 0.08).bfloat16()
    hidden, w_nvs, cu, plan = buf.dispatch(x, w.cuda(), topk.cuda(), tpe)
    buf.check()
    # source records: every real row names the entry that owns it
    N = S * K
    src = plan.src_info.cpu()
    dst = plan.dst.cpu()
    for r in range(R):
        raw = torch.where(dst[r] < 0, -dst[r] - 1, dst[r]).long()
        assert torch.equal(src[raw // buf.NvS, raw % buf.NvS], (r * N + torch.arange(N)).to(torch.int32))
    etc = plan.experts_to_copy[0].cpu()
    act = (hidden.float() @ proj.float()).bfloat16() * 1.0            # a stand-in activation
    act = (act.float() * w_nvs[:, :, None]).bfloat16()
    scal = torch.rand(R, buf.NvS, device="cuda", generator=g)
    push = buf.push_target(plan)
    y_unfused = torch.zeros(R, buf.NvS, H, device="cuda", dtype=torch.bfloat16)
    for r in range(R):
        slot_ids = etc[r].clamp(min=0).long()
        wd_slot = wd_all[slot_ids].contiguous()
        wd_loc = wd_all[r * epn:(r + 1) * epn].contiguous()
        p_r = dict(push, src_info=plan.src_info[r])
        gemm.down(act[r].contiguous(), wd_loc, plan.cu_seqlens[r], wd_slot=wd_slot, split=epn, push=p_r)
        gemm.down(act[r].contiguous(), wd_loc, plan.cu_seqlens[r], wd_slot=wd_slot, split=epn, out=y_unfused[r])
    out, sk = buf.combine_pushed(plan, scal)
    buf.check()
    gemm.check_status()
    # fp32 reference: token s of rank r sums, over its K entries, act_row @ Wd[expert]^T
    ref = torch.zeros(R, S, H, device="cuda")
    sk_ref = torch.zeros(R, S, K, device="cuda")
    for r in range(R):
        raw = torch.where(dst[r] < 0, -dst[r] - 1, dst[r]).long().cuda()
        dr, lo = raw // buf.NvS, raw % buf.NvS
        ex = topk[r].flatten().long().cuda()
        rows = act[dr, lo].float()                                           # [N, Hp]
        yk = torch.einsum("nh,nmh->nm", rows, wd_all[ex].float())            # [N, H]
        ref[r] = yk.view(S, K, H).sum(1)
        sk_ref[r] = scal[dr, lo].view(S, K)
    assert torch.equal(sk, sk_ref)
    scale = float(ref.abs().max())
    assert float((out.float() - ref).abs().max()) / scale < 2e-2
    out_u, _, _ = buf.combine(plan, y_unfused, None)
    assert float((out.float() - out_u.float()).abs().max()) / scale < 2e-2
