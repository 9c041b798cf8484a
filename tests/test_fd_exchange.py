"""Host-side handle exchange on CPU: gloo ranks pass file descriptors over AF_UNIX datagram
sockets (SCM_RIGHTS), the same path that carries the VMM memory handles between GPU ranks."""
import os
import tempfile

import pytest
import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from moonep_b200.buffer import exchange_fds
    path = os.path.join(tmp, f"payload{rank}")
    with open(path, "w") as fh:
        fh.write(f"rank-{rank}")
    fd = os.open(path, os.O_RDONLY)
    fds = exchange_fds(fd, dist.group.WORLD)
    assert len(fds) == world and fds[rank] == fd
    for r, f in enumerate(fds):
        os.lseek(f, 0, os.SEEK_SET)
        assert os.read(f, 64).decode() == f"rank-{r}"
        os.close(f)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_fd_exchange_gloo(world):
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_worker, args=(world, 29720 + world, tmp), nprocs=world, join=True)


def _short_timeout_worker(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import moonep_b200.buffer as B
    B._FD_TIMEOUT_S = 0.5
    fd = os.open(os.devnull, os.O_RDONLY)
    if rank == 1:
        # a peer that takes part in the rendezvous but never sends its handle
        import socket
        real = socket.socket.sendmsg
        socket.socket.sendmsg = lambda self, *a, **k: 0
        try:
            B.exchange_fds(fd, dist.group.WORLD)
        except RuntimeError:
            pass          # the waiting rank gave up and left; this rank's next collective fails
        finally:
            socket.socket.sendmsg = real
    else:
        try:
            B.exchange_fds(fd, dist.group.WORLD)
            raise AssertionError("expected a SymmetricMemoryError")
        except B.SymmetricMemoryError as exc:
            assert "timed out" in str(exc)


def test_fd_exchange_reports_a_silent_peer():
    """A dropped handle message surfaces as an exception on the waiting rank, not as a hang or
    an exit() (failure injected on the host; no GPU involved)."""
    mp.spawn(_short_timeout_worker, args=(2, 29731), nprocs=2, join=True)
