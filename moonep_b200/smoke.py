"""Tiny end-to-end run on one GPU: a 4-rank virtual EP group dispatches, "computes" and combines."""
import torch


def run_smoke() -> None:
    from . import Buffer
    from .utils.routing import routing_for_maxvio, tokens_per_expert

    R, S, K, E, H = 4, 64, 4, 16, 256
    topk, w, _, _ = routing_for_maxvio(S, K, E, R, 2.0, seed=1)
    tpe = torch.stack([tokens_per_expert(topk[r], E) for r in range(R)])
    buf = Buffer(S, H, K, E, R, num_sms=4, token_padding=16, virtual=True, timeout_s=5.0)
    x = torch.randn(R, S, H, device="cuda").bfloat16()
    hidden, w_nvs, cu, plan = buf.dispatch(x, w.cuda(), topk.cuda(), tpe.cuda())
    y = (hidden.float() * w_nvs[:, :, None]).bfloat16()
    out, _, _ = buf.combine(plan, y)
    buf.check()
    ref = x.float() * w.cuda().sum(2, keepdim=True)
    err = float((out.float() - ref).abs().max())
    assert err < 0.1, err
    buf.destroy()
    print(f"smoke ok: max err {err:.4f}")
