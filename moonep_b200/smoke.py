"""Tiny end-to-end run on one GPU: one MoE layer forward + backward + SGD step (EP=1), then a
4-rank virtual EP group round trip so that the multi-rank kernels run too."""
import torch


def run_smoke() -> None:
    from . import Buffer
    from .models.moe_layer import MoELayer
    from .ops import gemm
    from .utils.routing import routing_for_maxvio, tokens_per_expert

    dev = torch.device("cuda", torch.cuda.current_device())
    buf = Buffer(256, 512, 4, 16, 1, num_sms=8, token_padding=128, timeout_s=5.0)
    layer = MoELayer(buf, 256, None, seed=1, init_std=0.05)
    x = torch.randn(256, 512, device=dev).bfloat16().requires_grad_(True)
    y = layer(x)
    loss = y.float().pow(2).mean()
    loss.backward()
    layer.sgd_step(1e-3)
    buf.check()
    gemm.check_status(dev)
    assert torch.isfinite(y.float()).all() and torch.isfinite(x.grad.float()).all()
    assert float(layer.g_gate.abs().sum()) > 0
    buf.destroy()

    R, S, K, E, H = 4, 64, 4, 16, 256
    topk, w, _, _ = routing_for_maxvio(S, K, E, R, 2.0, seed=1)
    tpe = torch.stack([tokens_per_expert(topk[r], E) for r in range(R)])
    vb = Buffer(S, H, K, E, R, num_sms=4, token_padding=16, virtual=True, timeout_s=5.0)
    xv = torch.randn(R, S, H, device=dev).bfloat16()
    hidden, w_nvs, cu, plan = vb.dispatch(xv, w.to(dev), topk.to(dev), tpe.to(dev))
    out, _, _ = vb.combine(plan, (hidden.float() * w_nvs[:, :, None]).bfloat16())
    vb.check()
    ref = xv.float() * w.to(dev).sum(2, keepdim=True)
    err = float((out.float() - ref).abs().max())
    assert err < 0.1, err
    vb.destroy()
    print(f"smoke ok: loss {float(loss):.5f}, virtual round-trip max err {err:.4f}")
