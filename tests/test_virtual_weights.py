"""prefetch_weight / reduce_grad on a single-GPU virtual group.  Case shapes follow the
reference's suites (tests/test_prefetch.py:45-266, tests/test_grad_reduce.py:231-403): empty
plans, holes, duplicates, self slots, several owners, fan-in larger than the ring, uint8
payloads with scale tensors, strided pools with padding sentinels, repeated launches."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _cleanup():
    yield
    from moonep_b200.api import destroy_live_buffers
    destroy_live_buffers()
    torch.cuda.synchronize()


def fake_plan(buf, etc):
    from moonep_b200 import CommPlan
    R, epn = buf.R, buf.epn
    etc_all = etc.to(torch.int32).cuda()[None].expand(R, R, epn).contiguous()
    z = lambda *s: torch.zeros(*s, dtype=torch.int32, device="cuda")
    return CommPlan(dst=z(R, buf.N), experts_to_copy=etc_all, zero_fill_ranges=z(R, 2 * epn, 2),
                    remote_stats=z(R, 2), cu_seqlens=z(R, 2 * epn), link=z(R, buf.NvS),
                    N=buf.N, R=R, E=buf.E, NvS=buf.NvS, K=buf.K)


def plans(R, epn, kind, seed=0):
    E = R * epn
    etc = torch.full((R, epn), -1, dtype=torch.int64)
    g = torch.Generator().manual_seed(seed)
    if kind == "empty":
        pass
    elif kind == "ring":            # every rank computes one expert of its right neighbour
        for d in range(R):
            etc[d, 0] = ((d + 1) % R) * epn
    elif kind == "fan_in":          # every slot of every other rank holds rank 0's expert 0..
        for d in range(1, R):
            for b in range(epn):
                etc[d, b] = b % epn
    elif kind == "holes_dups_self":
        for d in range(R):
            etc[d, epn - 1] = ((d + 1) % R) * epn + (epn - 1)      # hole before it
            if epn > 2:
                etc[d, 1] = ((d + 1) % R) * epn + (epn - 1)        # duplicate of the same expert
            etc[d, 0] = d * epn                                     # self slot
    elif kind == "random":
        mask = torch.rand(R, epn, generator=g) < 0.5
        vals = torch.randint(0, E, (R, epn), generator=g)
        etc = torch.where(mask, vals, etc)
    return etc


def expected_prefetch(local, pool0, etc, R, epn):
    """local [R, epn, ...]; returns the pool after the copy."""
    out = pool0.clone()
    for d in range(R):
        for b in range(epn):
            e = int(etc[d, b])
            if e >= 0:
                out[d, b] = local[e // epn, e % epn]
    return out


@pytest.mark.parametrize("kind", ["empty", "ring", "fan_in", "holes_dups_self", "random"])
@pytest.mark.parametrize("R,epn,Hh,Hp", [(4, 4, 128, 128), (8, 2, 256, 384), (2, 3, 64, 40)])
def test_prefetch_bf16(kind, R, epn, Hh, Hp):
    from moonep_b200 import Buffer
    buf = Buffer(16, 64, 2, R * epn, R, num_sms=3, token_padding=8, virtual=True, timeout_s=2.0)
    etc = plans(R, epn, kind, seed=R * 100 + epn)
    plan = fake_plan(buf, etc)
    g = torch.Generator(device="cuda").manual_seed(1)
    locs = [torch.randn(R, epn, Hh, Hp, device="cuda", generator=g).bfloat16() for _ in range(3)]
    # strided pools: room for one extra expert per rank acts as padding that must stay untouched
    raw = [torch.full((R, epn + 1, Hh, Hp), 7.0, device="cuda").bfloat16() for _ in range(3)]
    pools = [r[:, :epn] for r in raw]
    want = [expected_prefetch(l, p, etc, R, epn) for l, p in zip(locs, pools)]
    for rep in range(2):      # repeats on one Buffer
        buf.prefetch_weight(plan, local_gate_weight=locs[0], local_up_weight=locs[1],
                            local_down_weight=locs[2], gate_prefetch_buffer=pools[0],
                            up_prefetch_buffer=pools[1], down_prefetch_buffer=pools[2])
        buf.check()
        for p, w_, r in zip(pools, want, raw):
            assert torch.equal(p, w_)
            assert bool((r[:, epn] == 7.0).all())


def test_prefetch_uint8_with_scales_async():
    from moonep_b200 import Buffer
    R, epn = 4, 2
    buf = Buffer(16, 64, 2, R * epn, R, num_sms=2, token_padding=8, virtual=True, timeout_s=2.0)
    etc = plans(R, epn, "ring")
    plan = fake_plan(buf, etc)
    g = torch.Generator(device="cuda").manual_seed(2)
    rnd = lambda *s: torch.randint(0, 256, s, device="cuda", generator=g, dtype=torch.uint8)
    locs = [rnd(R, epn, 128, 64) for _ in range(3)]                  # packed 4-bit payload
    scs = [rnd(R, epn, 128, 4), rnd(R, epn, 128, 4), torch.randn(R, epn, 32, 12, device="cuda", generator=g)]
    pools = [torch.zeros(R, epn, 128, 64, device="cuda", dtype=torch.uint8) for _ in range(3)]
    spools = [torch.zeros_like(s) for s in scs]
    ev = buf.prefetch_weight(plan, async_finish=True, local_gate_weight=locs[0], local_up_weight=locs[1],
                             local_down_weight=locs[2], gate_prefetch_buffer=pools[0],
                             up_prefetch_buffer=pools[1], down_prefetch_buffer=pools[2],
                             local_gate_scale=scs[0], local_up_scale=scs[1], local_down_scale=scs[2],
                             gate_scale_prefetch_buffer=spools[0], up_scale_prefetch_buffer=spools[1],
                             down_scale_prefetch_buffer=spools[2])
    ev.wait()
    buf.check()
    for l, p in zip(locs + scs, pools + spools):
        assert torch.equal(p, expected_prefetch(l, torch.zeros_like(p), etc, R, epn))
    with pytest.raises(AssertionError):
        buf.prefetch_weight(plan, local_gate_weight=locs[0], local_up_weight=locs[1],
                            local_down_weight=locs[2], gate_prefetch_buffer=pools[0],
                            up_prefetch_buffer=pools[1], down_prefetch_buffer=pools[2],
                            local_gate_scale=scs[0])


@pytest.mark.parametrize("kind", ["empty", "ring", "fan_in", "holes_dups_self", "random"])
@pytest.mark.parametrize("R,epn,Hh,Hp", [(4, 4, 128, 128), (8, 1, 64, 72), (2, 3, 256, 132)])
def test_reduce_grad_bitwise(kind, R, epn, Hh, Hp):
    from moonep_b200 import Buffer
    buf = Buffer(16, 64, 2, R * epn, R, num_sms=3, token_padding=8, virtual=True, timeout_s=2.0)
    etc = plans(R, epn, kind, seed=R * 10 + epn)
    plan = fake_plan(buf, etc)
    g = torch.Generator(device="cuda").manual_seed(3)
    local = [torch.randn(R, epn, Hh, Hp, device="cuda", generator=g) for _ in range(3)]
    raw = [torch.randn(R, epn + 1, Hh, Hp, device="cuda", generator=g) for _ in range(3)]
    pools = [r[:, :epn] for r in raw]
    for rep in range(2):
        pool0 = [p.clone() for p in pools]
        pad0 = [r[:, epn].clone() for r in raw]
        want = [l.clone() for l in local]
        for t in range(3):
            for d in range(R):                       # ascending (rank, slot) order
                for b in range(epn):
                    e = int(etc[d, b])
                    if e >= 0:
                        want[t][e // epn, e % epn] += pool0[t][d, b]
        buf.reduce_grad(plan, local_gate_grad=local[0], local_up_grad=local[1], local_down_grad=local[2],
                        gate_reduce_buffer=pools[0], up_reduce_buffer=pools[1], down_reduce_buffer=pools[2])
        buf.check()
        for t in range(3):
            assert torch.equal(local[t], want[t])                      # bitwise
            for d in range(R):
                for b in range(epn):
                    if int(etc[d, b]) >= 0:
                        assert bool((pools[t][d, b] == 0).all())        # consumed slots cleared
                    else:
                        assert torch.equal(pools[t][d, b], pool0[t][d, b])
            assert torch.equal(raw[t][:, epn], pad0[t])                 # padding untouched
        for p in pools:                                                 # refill for the next round
            p.copy_(torch.randn(p.shape, device="cuda", generator=g))
