"""Peer-loss detection on the host (gloo ranks on CPU, no GPU): a rank that leaves between steps
is reported to the others before they launch anything, as a PeerLostError naming the rank."""
import os

import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from moonep_b200.utils.health import Heartbeat, PeerLostError
    hb = Heartbeat.from_default_group()
    for step in range(3):
        hb.step(step, timeout_s=10.0)                 # everybody alive
    if rank == world - 1:
        os._exit(0)                                   # leaves between steps, nothing in flight
    try:
        hb.step(3, timeout_s=1.0)
        raise AssertionError("expected PeerLostError")
    except PeerLostError as exc:
        assert exc.missing == [world - 1] and exc.step == 3
    os._exit(0)                                       # no collective teardown with a dead peer


def test_heartbeat_detects_a_rank_that_left():
    mp.spawn(_worker, args=(3, 29741), nprocs=3, join=True)
