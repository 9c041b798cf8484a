"""MoE layer (EP=1) forward, backward and SGD step against a dense PyTorch fp32 reference of the
same math: softmax-over-top-k router, SwiGLU experts, weighted sum."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def reference_layer(x, wr, wg, wu, wd, K, bias=None):
    """fp32 autograd reference.  x [S,H]; wr [H,E]; wg/wu/wd [E,H,Hp]."""
    logits = x @ wr
    sel = logits + (bias if bias is not None else 0)
    idx = sel.topk(K, dim=1).indices
    w = torch.softmax(logits.gather(1, idx), dim=1)
    y = torch.zeros_like(x)
    for k in range(K):
        for e in idx[:, k].unique().tolist():
            m = idx[:, k] == e
            xe = x[m]
            act = torch.nn.functional.silu(xe @ wg[e]) * (xe @ wu[e]) * w[m, k:k + 1]
            y = y.index_add(0, m.nonzero().flatten(), act @ wd[e].t())
    return y, idx


def test_moe_layer_matches_reference():
    from moonep_b200 import Buffer
    from moonep_b200.models.moe_layer import MoELayer
    from moonep_b200.ops import gemm
    S, H, Hp, K, E = 256, 256, 128, 4, 8
    buf = Buffer(S, H, K, E, 1, num_sms=4, token_padding=64, timeout_s=5.0)
    layer = MoELayer(buf, Hp, None, seed=3, init_std=0.06)
    g = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn(S, H, device="cuda", generator=g).bfloat16()
    xr = x.float().requires_grad_(True)
    params = [layer.w_router, layer.w_gate, layer.w_up, layer.w_down]
    wr, wg, wu, wd = [p.float().clone().requires_grad_(True) for p in params]
    y_ref, idx = reference_layer(xr, wr, wg, wu, wd, K)
    dy = torch.randn(S, H, device="cuda", generator=g).bfloat16()
    y_ref.backward(dy.float())

    xo = x.clone().requires_grad_(True)
    y = layer(xo)
    y.backward(dy)
    buf.check()
    gemm.check_status()

    def close(a, b, tol):
        scale = float(b.abs().max()) + 1e-9
        err = float((a.float() - b).abs().max()) / scale
        assert err < tol, err

    close(y, y_ref.detach(), 3e-2)
    close(xo.grad, xr.grad, 5e-2)
    close(layer.g_gate, wg.grad, 5e-2)
    close(layer.g_up, wu.grad, 5e-2)
    close(layer.g_down, wd.grad, 5e-2)
    close(layer.g_router[0], wr.grad, 8e-2)
    before = layer.w_gate.float().clone()
    layer.sgd_step(0.5)
    close(layer.w_gate, before - 0.5 * layer.g_gate, 1e-2)
    sd = layer.state_dict()
    layer.w_gate.zero_()
    layer.load_state_dict(sd)
    assert torch.equal(layer.w_gate.cpu(), sd["gate"])
    buf.destroy()


def test_fused_sgd_step_is_bit_identical():
    """SGD fused into the weight-grad epilogues == weight grads stored, then the SGD kernel."""
    from moonep_b200 import Buffer
    from moonep_b200.models.moe_layer import MoELayer
    from moonep_b200.ops import gemm
    S, H, Hp, K, E = 512, 256, 384, 4, 8
    buf = Buffer(S, H, K, E, 1, num_sms=4, token_padding=64, timeout_s=5.0)
    g = torch.Generator(device="cuda").manual_seed(21)
    x = torch.randn(S, H, device="cuda", generator=g).bfloat16()
    dy = torch.randn(S, H, device="cuda", generator=g).bfloat16()
    bias = torch.zeros(E, device="cuda")
    bias[3] = -100.0                                   # one expert without tokens: weights untouched
    res = []
    for fused in (False, True):
        layer = MoELayer(buf, Hp, None, seed=3, init_std=0.06, router_bias=bias)
        if fused:
            layer.fuse_sgd(0.5)
        xo = x.clone().requires_grad_(True)
        y = layer(xo)
        y.backward(dy)
        layer.sgd_step(0.5)
        torch.cuda.synchronize()
        buf.check()
        gemm.check_status()
        res.append((y.detach().clone(), xo.grad.clone(), layer.w_gate.clone(), layer.w_up.clone(),
                    layer.w_down.clone(), layer.w_router.clone()))
    for a, b in zip(*res):
        assert torch.equal(a, b)
    init = MoELayer(buf, Hp, None, seed=3, init_std=0.06)
    assert torch.equal(res[1][2][3], init.w_gate[3]) and not torch.equal(res[1][2][0], init.w_gate[0])
    buf.destroy()


def test_forward_rows_kept_in_second_shard():
    """``hidden_in_place`` (forward dispatch lands in a second shard and is used in place) gives
    the same step as copying the rows out, and ``Buffer.dispatch(shard=1)`` returns the same rows."""
    from moonep_b200 import Buffer
    from moonep_b200.models.moe_layer import MoELayer
    from moonep_b200.ops import gemm
    S, H, Hp, K, E = 256, 256, 128, 4, 8
    buf = Buffer(S, H, K, E, 1, num_sms=4, token_padding=64, timeout_s=5.0)
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(S, H, device="cuda", generator=g).bfloat16()
    dy = torch.randn(S, H, device="cuda", generator=g).bfloat16()
    res = []
    for in_place in (False, True):
        layer = MoELayer(buf, Hp, None, seed=3, init_std=0.06, hidden_in_place=in_place)
        for _ in range(2):                       # twice: the shards are reused step after step
            xo = x.clone().requires_grad_(True)
            y = layer(xo)
            y.backward(dy)
            layer.sgd_step(0.1)
        torch.cuda.synchronize()
        buf.check()
        gemm.check_status()
        res.append((y.detach().clone(), xo.grad.clone(), layer.w_gate.clone(), layer.w_down.clone()))
    for a, b in zip(*res):
        assert torch.equal(a, b)
    topk = torch.randint(0, E, (S, K), device="cuda", dtype=torch.int32)
    tpe = torch.bincount(topk.flatten().long(), minlength=E).to(torch.int32)
    h0, _, _, plan = buf.dispatch(x, None, topk, tpe)
    h1, _, _, _ = buf.dispatch(x, None, plan=plan, zero_copy=True, shard=1)
    assert h1.data_ptr() == buf.hidden_view(1).data_ptr() != buf.hidden_view(0).data_ptr()
    rows = int(plan.cu_seqlens[-1])
    assert torch.equal(h0[:rows], h1[:rows])
    buf.destroy()


def test_router_topk_kernel():
    from moonep_b200.ops import elementwise as ew
    g = torch.Generator(device="cuda").manual_seed(1)
    logits = torch.randn(500, 96, device="cuda", generator=g)
    bias = torch.randn(96, device="cuda", generator=g)
    topk, w, tpe = ew.router_topk(logits, 6, bias)
    ref_idx = (logits + bias).topk(6, dim=1).indices
    assert torch.equal(topk.long().sort(1).values, ref_idx.sort(1).values)
    ref_w = torch.softmax(logits.gather(1, topk.long()), dim=1)
    torch.testing.assert_close(w, ref_w, rtol=1e-4, atol=1e-6)
    assert torch.equal(tpe.long(), torch.bincount(topk.flatten().long(), minlength=96))
    dw = torch.randn(500, 6, device="cuda", generator=g)
    dl = ew.router_topk_bwd(w, dw, topk, 96).float()
    lw = logits.clone().requires_grad_(True)
    torch.softmax(lw.gather(1, topk.long()), dim=1).backward(dw)
    torch.testing.assert_close(dl, lw.grad, rtol=2e-2, atol=2e-3)


def test_swiglu_bwd_kernel():
    from moonep_b200.ops import elementwise as ew
    g = torch.Generator(device="cuda").manual_seed(2)
    rows, Hp = 300, 192
    gate = torch.randn(rows, Hp, device="cuda", generator=g).bfloat16()
    up = torch.randn(rows, Hp, device="cuda", generator=g).bfloat16()
    dact = torch.randn(rows, Hp, device="cuda", generator=g).bfloat16()
    ws = torch.rand(rows, device="cuda", generator=g) + 0.5
    nrows = torch.tensor([260], dtype=torch.int32, device="cuda")
    dg, du, ds = ew.swiglu_bwd(dact, gate, up, ws, rows_ptr=nrows)
    gf, uf, wf = gate.float().requires_grad_(True), up.float().requires_grad_(True), ws.clone().requires_grad_(True)
    (torch.nn.functional.silu(gf) * uf * wf[:, None]).backward(dact.float())
    torch.testing.assert_close(dg[:260].float(), gf.grad[:260], rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(du[:260].float(), uf.grad[:260], rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(ds[:260], wf.grad[:260], rtol=1e-3, atol=1e-3)
    assert float(ds[260:].abs().max()) == 0


def test_tiny_decoder_trains_and_checkpoints():
    """Config-5-shaped stack at toy size on one GPU (EP=1): loss falls over a few steps and a
    state-dict round trip restores every parameter, expert weights in their home layout."""
    from moonep_b200 import Buffer
    from moonep_b200.models.decoder import MoEDecoder
    from moonep_b200.models.moe_layer import MoELayer
    S, Hd, E, K, Hp, V = 128, 128, 8, 2, 64, 97
    buf = Buffer(S, Hd, K, E, 1, num_sms=4, token_padding=64, timeout_s=5.0)
    torch.manual_seed(0)
    model = MoEDecoder(V, Hd, 2, 4, lambda i: MoELayer(buf, Hp, None, seed=i, init_std=0.05)).cuda()
    g = torch.Generator(device="cuda").manual_seed(1)
    tok = torch.randint(0, V, (S,), device="cuda", generator=g)
    tgt = torch.randint(0, V, (S,), device="cuda", generator=g)
    sd0 = model.state_dict_all()
    losses = [float(model.train_step(tok, tgt, 0.05)) for _ in range(8)]
    buf.check()
    assert losses[-1] < losses[0] - 0.05, losses
    changed = model.state_dict_all()
    assert not torch.equal(changed["moe.0.gate"], sd0["moe.0.gate"])
    model.load_state_dict_all(sd0)
    back = model.state_dict_all()
    assert all(torch.equal(back[k], sd0[k]) for k in sd0)
    buf.destroy()
