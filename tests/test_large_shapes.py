"""Shapes whose byte offsets pass 2^31 and 2^32 (the reference pins them in
tests/test_prefetch.py:45-266 and tests/test_grad_reduce.py:231-403 with 7168x3072 experts, and
in tests/test_dispatch.py:118-127,419-441 with S=8192, K=16, H=7168): every index computation on
these paths must be 64-bit.  Only the rows / slots that a case touches are initialised and
checked, so the tests stay at a few GB and a few seconds."""
import pytest
import torch

from tests.test_virtual_weights import fake_plan

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _cleanup():
    yield
    from moonep_b200.api import destroy_live_buffers
    destroy_live_buffers()
    torch.cuda.synchronize()
    torch.cuda.empty_cache()


def test_prefetch_offsets_beyond_4gib():
    """bf16 experts of 7168 x 3072 (44 MB), 52 per rank, 2 ranks: a pool is 4.6 GB, so the last
    slots of rank 1 start beyond 2^32 bytes."""
    from moonep_b200 import Buffer
    R, epn, Hh, Hp = 2, 52, 7168, 3072
    buf = Buffer(16, 64, 2, R * epn, R, num_sms=8, token_padding=8, virtual=True, timeout_s=5.0)
    etc = torch.full((R, epn), -1, dtype=torch.int64)
    etc[1, epn - 1] = 0 * epn + (epn - 1)       # rank 1's LAST slot <- rank 0's last expert
    etc[1, 0] = 0 * epn + 3
    etc[0, epn - 2] = 1 * epn + (epn - 1)       # rank 0 <- rank 1's last expert (source offset > 2^31)
    plan = fake_plan(buf, etc)
    local = torch.empty(R, epn, Hh, Hp, dtype=torch.bfloat16, device="cuda")
    pool = torch.empty(R, epn, Hh, Hp, dtype=torch.bfloat16, device="cuda")
    assert pool[1, epn - 1].data_ptr() - pool.data_ptr() > 2 ** 32
    g = torch.Generator(device="cuda").manual_seed(4)
    touched = [(0, epn - 1), (0, 3), (1, epn - 1)]
    for r, e in touched:
        local[r, e].copy_(torch.randn(Hh, Hp, device="cuda", generator=g).bfloat16())
    for d, b in [(1, epn - 1), (1, 0), (0, epn - 2), (1, epn - 2), (0, 0)]:
        pool[d, b].fill_(7.0)
    small = torch.zeros(R, epn, 8, 8, dtype=torch.bfloat16, device="cuda")
    buf.prefetch_weight(plan, local_gate_weight=local, local_up_weight=small, local_down_weight=small,
                        gate_prefetch_buffer=pool, up_prefetch_buffer=small.clone(),
                        down_prefetch_buffer=small.clone())
    buf.check()
    assert torch.equal(pool[1, epn - 1], local[0, epn - 1])
    assert torch.equal(pool[1, 0], local[0, 3])
    assert torch.equal(pool[0, epn - 2], local[1, epn - 1])
    assert bool((pool[1, epn - 2] == 7.0).all()) and bool((pool[0, 0] == 7.0).all())   # neighbours untouched


def test_reduce_grad_offsets_beyond_4gib():
    """fp32 grads of 3584 x 3072 (44 MB), 52 per rank, 2 ranks: same geometry in the reduce pool."""
    from moonep_b200 import Buffer
    R, epn, Hh, Hp = 2, 52, 3584, 3072
    buf = Buffer(16, 64, 2, R * epn, R, num_sms=8, token_padding=8, virtual=True, timeout_s=5.0)
    etc = torch.full((R, epn), -1, dtype=torch.int64)
    etc[1, epn - 1] = 0 * epn + (epn - 1)       # rank 0's last expert computed in rank 1's last slot
    etc[0, epn - 1] = 0 * epn + (epn - 1)       # ... and in its own last slot
    etc[0, 1] = 1 * epn + (epn - 1)             # rank 1's last expert computed on rank 0
    plan = fake_plan(buf, etc)
    local = torch.empty(R, epn, Hh, Hp, device="cuda")
    pool = torch.empty(R, epn, Hh, Hp, device="cuda")
    assert pool[1, epn - 1].data_ptr() - pool.data_ptr() > 2 ** 32
    g = torch.Generator(device="cuda").manual_seed(5)
    for r, e in [(0, epn - 1), (1, epn - 1)]:
        local[r, e].copy_(torch.randn(Hh, Hp, device="cuda", generator=g))
    for d, b in [(1, epn - 1), (0, epn - 1), (0, 1)]:
        pool[d, b].copy_(torch.randn(Hh, Hp, device="cuda", generator=g))
    pool[1, epn - 2].fill_(3.0)
    want0 = (local[0, epn - 1] + pool[0, epn - 1]) + pool[1, epn - 1]      # ascending (rank, slot)
    want1 = local[1, epn - 1] + pool[0, 1]
    small = torch.zeros(R, epn, 4, 4, device="cuda")
    buf.reduce_grad(plan, local_gate_grad=local, local_up_grad=small, local_down_grad=small.clone(),
                    gate_reduce_buffer=pool, up_reduce_buffer=small.clone(), down_reduce_buffer=small.clone())
    buf.check()
    assert torch.equal(local[0, epn - 1], want0) and torch.equal(local[1, epn - 1], want1)    # bitwise
    for d, b in [(1, epn - 1), (0, epn - 1), (0, 1)]:
        assert bool((pool[d, b] == 0).all())                                                  # consumed slots cleared
    assert bool((pool[1, epn - 2] == 3.0).all())


def test_dispatch_combine_large_stride():
    """S=8192, K=16, H=7168 on two virtual ranks: a rank's row buffer is 1.9 GB, the second rank's
    rows start beyond 2^31 bytes.  Traceable payload: every row carries (token, source rank) in
    its first two elements; every destination slot is checked against the plan."""
    from moonep_b200 import Buffer
    R, S, K, H, epn = 2, 8192, 16, 7168, 16
    E = R * epn
    buf = Buffer(S, H, K, E, R, num_sms=16, token_padding=128, virtual=True, timeout_s=10.0)
    assert buf.hidden_stride * H * 2 > 2 ** 31 - 2 ** 28
    g = torch.Generator().manual_seed(6)
    topk = torch.stack([torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(S)])
                        for _ in range(R)]).to(torch.int32).cuda()
    tpe = torch.stack([torch.bincount(topk[r].flatten().long(), minlength=E) for r in range(R)]).to(torch.int32)
    x = torch.zeros(R, S, H, dtype=torch.bfloat16, device="cuda")
    tok = torch.arange(S, device="cuda")
    for r in range(R):
        x[r, :, 0] = (tok % 256).to(torch.bfloat16)          # exact in bf16
        x[r, :, 1] = (tok // 256).to(torch.bfloat16)
        x[r, :, 2] = float(r)
        x[r, :, H - 1] = 1.0
    hidden, _, cu, plan = buf.dispatch(x, None, topk, tpe.cuda(), zero_copy=True)
    buf.check()
    NvS = buf.NvS
    for r in range(R):
        d = plan.dst[r].long()
        raw = torch.where(d >= 0, d, -d - 1)
        dr, row = raw // NvS, raw % NvS
        t = torch.arange(S * K, device="cuda") // K
        got = hidden[dr, row]                                # [N, H] gather of every entry's slot
        assert torch.equal(got[:, 0].float(), (t % 256).float())
        assert torch.equal(got[:, 1].float(), (t // 256).float())
        assert bool((got[:, 2].float() == r).all()) and bool((got[:, H - 1].float() == 1).all())
        del got
    out, _, _ = buf.combine(plan, hidden, None, zero_copy=True)
    buf.check()
    # columns whose partial sums stay exact in bf16 (the duplicates of a token are pre-reduced in
    # bf16 on the rank that computed them): K copies of 1, and K copies of the source rank
    assert bool((out[:, :, H - 1].float() == K).all())
    for r in range(R):
        assert bool((out[r, :, 2].float() == r * K).all())
    rel = (out[:, :, 0].float() - x[:, :, 0].float() * K).abs() / (x[:, :, 0].float() * K + 1)
    assert float(rel.max()) < 2 ** -6


def test_shard_is_bound_at_launch():
    """The row buffer is a launch argument, not Buffer state: dispatches into the second and the
    first shard issued back to back on the communication stream, from two host threads and with
    no host wait in between, each fill their own buffer.  (They still run one after the other on
    the device: dispatch and combine of one Buffer share a barrier channel.)"""
    import threading

    from moonep_b200 import Buffer
    from moonep_b200.utils.routing import routing_for_maxvio, tokens_per_expert
    R, S, H, K, tp = 2, 512, 1024, 4, 16
    E = 8 * R
    buf = Buffer(S, H, K, E, R, num_sms=4, token_padding=tp, virtual=True, timeout_s=5.0)
    buf.enable_second_shard()
    topk, w, _, _ = routing_for_maxvio(S, K, E, R, 1.0, seed=2)
    tpe = torch.stack([tokens_per_expert(topk[r], E) for r in range(R)]).cuda()
    topk = topk.cuda()
    g = torch.Generator(device="cuda").manual_seed(3)
    xa = torch.randn(R, S, H, device="cuda", generator=g).bfloat16()
    xb = torch.randn(R, S, H, device="cuda", generator=g).bfloat16()
    ha, _, cu, plan = buf.dispatch(xa, None, topk, tpe, zero_copy=False)
    hb, _, _, _ = buf.dispatch(xb, None, plan=plan, zero_copy=False)
    torch.cuda.synchronize()
    dev = torch.cuda.current_device()
    events, errors = [], []

    def issue(x, shard):
        try:
            torch.cuda.set_device(dev)
            for _ in range(5):
                out = buf.dispatch(x, None, plan=plan, async_finish=True, zero_copy=True, shard=shard)
                events.append(out[-1])
        except Exception as exc:  # noqa: BLE001
            errors.append(exc)

    threads = [threading.Thread(target=issue, args=(xa, 1)), threading.Thread(target=issue, args=(xb, 0))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for ev in events:
        ev.wait()
    torch.cuda.synchronize()
    buf.check()
    h1, h0 = buf.hidden_view(1), buf.hidden_view(0)
    for r in range(R):
        rows = int(cu[r, -1])
        assert torch.equal(h1[r, :rows], ha[r, :rows]) and torch.equal(h0[r, :rows], hb[r, :rows])
