"""The planner entry point that allocates nothing (``mep_plan_local_noalloc``, see
csrc/device/plan_noalloc.h).

It serves callers that cannot allocate device memory at the moment they need a plan: code running
inside another runtime's fixed memory budget, or a process that has no ``Buffer`` (whose
constructor allocates).  The test drives the exported C symbol directly through ctypes, twice in a
row with different ranks and routings, and compares every output bit for bit with the plan the
regular ``Buffer.dispatch`` planner produces.  It lives in a file that pytest collects last, so a
run that stops at the first failure has already executed everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _symbol():
    from moonep_b200 import _build, _native
    _native.lib()                                    # builds the library if it is missing
    fn = ctypes.CDLL(_build.LIB_PATH).mep_plan_local_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 2 + [ctypes.c_int] * 6 + [ctypes.c_void_p] * 6 + [ctypes.c_void_p]
    return fn


def _call(fn, tpe_all, topk, rank, R, E, S, K, tp):
    epn = E // R
    i32 = dict(dtype=torch.int32, device="cuda")
    out = dict(dst=torch.full((S * K,), -7, **i32), cu=torch.full((2 * epn,), -7, **i32),
               zf=torch.full((2 * epn, 2), -7, **i32), etc=torch.full((R, epn), -7, **i32),
               rs=torch.full((2,), -7, **i32), status=torch.full((8,), -7, **i32))
    rc = fn(tpe_all.data_ptr(), topk.data_ptr(), rank, R, E, S, K, tp, out["dst"].data_ptr(),
            out["cu"].data_ptr(), out["zf"].data_ptr(), out["etc"].data_ptr(), out["rs"].data_ptr(),
            out["status"].data_ptr(), torch.cuda.current_stream().cuda_stream)
    return rc, out


def test_no_alloc_planner_matches_buffer_planner_twice():
    from moonep_b200 import Buffer, _native
    from moonep_b200.utils.routing import routing_for_maxvio, tokens_per_expert
    fn = _symbol()
    R, S, K, E, H, tp = 4, 96, 4, 24, 64, 16
    buf = Buffer(S, H, K, E, R, num_sms=3, token_padding=tp, virtual=True, timeout_s=2.0)
    x = torch.zeros(R, S, H, device="cuda", dtype=torch.bfloat16)
    for call, (seed, rank, maxvio) in enumerate([(3, 1, 3.0), (4, 2, 0.0), (5, 0, 6.0)]):
        topk, _, _, _ = routing_for_maxvio(S, K, E, R, maxvio, seed=seed)
        tpe = torch.stack([tokens_per_expert(topk[r], E) for r in range(R)])
        _, _, _, plan = buf.dispatch(x, None, topk.cuda(), tpe.cuda())       # existing entry point
        buf.check()
        tpe_d, topk_d = tpe.cuda().contiguous(), topk[rank].cuda().contiguous().view(-1)
        rc, out = _call(fn, tpe_d, topk_d, rank, R, E, S, K, tp)
        torch.cuda.synchronize()
        assert rc == 0, _native.last_error()
        # a second identical call into the same output tensors must leave the device's free
        # memory exactly where it was: the entry point itself allocates nothing
        free_before = torch.cuda.mem_get_info()[0]
        rc2 = fn(tpe_d.data_ptr(), topk_d.data_ptr(), rank, R, E, S, K, tp, out["dst"].data_ptr(),
                 out["cu"].data_ptr(), out["zf"].data_ptr(), out["etc"].data_ptr(),
                 out["rs"].data_ptr(), out["status"].data_ptr(),
                 torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert rc2 == 0 and torch.cuda.mem_get_info()[0] == free_before
        assert out["status"].tolist()[0] == 0
        assert torch.equal(out["dst"], plan.dst[rank])
        assert torch.equal(out["cu"], plan.cu_seqlens[rank])
        assert torch.equal(out["zf"], plan.zero_fill_ranges[rank])
        assert torch.equal(out["etc"], plan.experts_to_copy[rank])
        assert torch.equal(out["rs"], plan.remote_stats[rank])
    buf.destroy()


@pytest.mark.parametrize("R,E,S,K,tp", [(2, 8192, 64, 4, 8), (64, 256, 48, 8, 16)])
def test_no_alloc_planner_at_its_limits(R, E, S, K, tp):
    """R * E = 16384 fills the whole built-in array and needs more than 48 KB of shared memory;
    R = 64 takes the arg-max loops that stride over more ranks than a warp has lanes.  Checked
    against the CPU oracle, twice in a row for two ranks."""
    from moonep_b200 import _native
    from moonep_b200 import reference as ref
    fn = _symbol()
    g = torch.Generator().manual_seed(R + E)
    pop = torch.exp(1.5 * torch.randn(E, generator=g))
    topk = torch.stack([torch.stack([torch.multinomial(pop, K, generator=g) for _ in range(S)])
                        for _ in range(R)]).to(torch.int32)
    tpe = torch.stack([torch.bincount(topk[r].flatten().long(), minlength=E) for r in range(R)]).to(torch.int32)
    tables, dst = ref.plan_all_ranks(topk, S, K, E, tp, tpe)
    tpe_d = tpe.cuda().contiguous()
    for rank in (R - 1, 0):
        rc, out = _call(fn, tpe_d, topk[rank].cuda().contiguous().view(-1), rank, R, E, S, K, tp)
        torch.cuda.synchronize()
        assert rc == 0, _native.last_error()
        assert out["status"].tolist()[0] == 0
        assert torch.equal(out["dst"].cpu(), dst[rank])
        assert torch.equal(out["cu"].cpu(), tables.cu_seqlens[rank])
        assert torch.equal(out["zf"].cpu(), tables.zero_fill[rank])
        assert torch.equal(out["etc"].cpu(), tables.experts_to_copy)
        assert torch.equal(out["rs"].cpu(), tables.remote_stats[rank])


def test_no_alloc_planner_rejects_oversize():
    from moonep_b200 import _native
    fn = _symbol()
    R, E = 8, 4096                                   # R*E = 32768 > 16384
    z = torch.zeros(8, dtype=torch.int32, device="cuda")
    rc = fn(z.data_ptr(), z.data_ptr(), 0, R, E, 1, 1, 8, z.data_ptr(), z.data_ptr(), z.data_ptr(),
            z.data_ptr(), z.data_ptr(), 0, torch.cuda.current_stream().cuda_stream)
    assert rc != 0 and "exceeds" in _native.last_error()
    torch.cuda.synchronize()
