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


def test_no_alloc_planner_rejects_oversize():
    from moonep_b200 import _native
    fn = _symbol()
    R, E = 8, 4096                                   # R*E = 32768 > 16384
    z = torch.zeros(8, dtype=torch.int32, device="cuda")
    rc = fn(z.data_ptr(), z.data_ptr(), 0, R, E, 1, 1, 8, z.data_ptr(), z.data_ptr(), z.data_ptr(),
            z.data_ptr(), z.data_ptr(), 0, torch.cuda.current_stream().cuda_stream)
    assert rc != 0 and "exceeds" in _native.last_error()
    torch.cuda.synchronize()
