"""The public ``Buffer`` surface keeps the reference's call signatures (moonep/api.py:425-438,
698-836, 838-969, 971-1104, 1106-1193): same positional order, same keyword names and defaults.
Extra keyword-only parameters of this implementation must have defaults, so that a caller
written against the reference runs unchanged.  CPU only: nothing is constructed."""
import inspect

from moonep_b200 import Buffer, MoonEPCommPlan
from moonep_b200.plan import CommPlan

P = inspect.Parameter


def _params(fn):
    return list(inspect.signature(fn).parameters.values())[1:]          # drop self


def _check(fn, positional, keyword_only):
    ps = _params(fn)
    pos = [p for p in ps if p.kind == P.POSITIONAL_OR_KEYWORD]
    kwo = {p.name: p for p in ps if p.kind == P.KEYWORD_ONLY}
    assert [p.name for p in pos[: len(positional)]] == [n for n, _ in positional]
    for p, (name, default) in zip(pos, positional):
        if default is not P.empty:
            assert p.default == default, f"{fn.__name__}: default of {name}"
    for name, default in keyword_only:
        assert name in kwo, f"{fn.__name__}: missing keyword {name}"
        if default is not P.empty:
            assert kwo[name].default == default, f"{fn.__name__}: default of {name}"
    known = {n for n, _ in keyword_only}
    for name, p in kwo.items():          # extensions are optional
        if name not in known:
            assert p.default is not P.empty, f"{fn.__name__}: extra keyword {name} must have a default"
    for p in pos[len(positional):]:
        assert p.default is not P.empty


def test_constructor_signature():
    _check(Buffer.__init__,
           [("S", P.empty), ("H", P.empty), ("K", P.empty), ("E", P.empty), ("num_ep_ranks", P.empty),
            ("num_sms", None), ("token_padding", 128), ("group", None), ("comm_stream_priority", -1),
            ("enable_pdl", True), ("explicitly_destroy", False)], [])


def test_dispatch_and_combine_signatures():
    _check(Buffer.dispatch,
           [("hidden_sh", P.empty), ("route_weights_sk", None), ("topk_experts_sk", None),
            ("tokens_per_expert", None), ("plan", None), ("async_finish", False)],
           [("inter_rank_sync", True), ("zero_copy", False), ("router_weights_zero_copy", False)])
    _check(Buffer.combine,
           [("plan", None), ("hidden_nvsh", None), ("route_weights_nvs", None), ("async_finish", False),
            ("inter_rank_sync", True)],
           [("zero_copy", False), ("router_weights_zero_copy", False)])
    assert "hidden_sh" not in inspect.signature(Buffer.combine).parameters    # a TypeError in the reference too


def test_weight_op_signatures():
    w = ["local_gate_weight", "local_up_weight", "local_down_weight",
         "gate_prefetch_buffer", "up_prefetch_buffer", "down_prefetch_buffer"]
    s = ["local_gate_scale", "local_up_scale", "local_down_scale",
         "gate_scale_prefetch_buffer", "up_scale_prefetch_buffer", "down_scale_prefetch_buffer"]
    _check(Buffer.prefetch_weight, [("plan", P.empty), ("async_finish", False)],
           [(n, P.empty) for n in w] + [(n, None) for n in s])
    g = ["local_gate_grad", "local_up_grad", "local_down_grad",
         "gate_reduce_buffer", "up_reduce_buffer", "down_reduce_buffer"]
    _check(Buffer.reduce_grad, [("plan", P.empty), ("async_finish", False)], [(n, P.empty) for n in g])
    for n in w:
        assert inspect.signature(Buffer.prefetch_weight).parameters[n].default is P.empty
    for n in g:
        assert inspect.signature(Buffer.reduce_grad).parameters[n].default is P.empty


def test_plan_type_and_views():
    assert MoonEPCommPlan is CommPlan
    fields = set(CommPlan.__dataclass_fields__)
    assert {"dst", "experts_to_copy", "zero_fill_ranges", "remote_stats", "cu_seqlens"} <= fields
    for name in ("dup_groups", "dup_loffs", "dup_counts", "clone"):
        assert hasattr(CommPlan, name)
    for name in ("hidden_nvsh_buffer_view", "router_weight_buffer_view", "inter_rank_sync", "destroy"):
        assert hasattr(Buffer, name)
