"""Symmetric (peer-mapped) tensors: Python side of the VMM allocator in ``csrc/host/symm_heap.cc``.

Public surface mirrors the reference's ``moonep/buffer.py``:

* ``create_nvl_dist_tensor(shape, dtype, group)``  (buffer.py:217)  -> ``[R * shape[0], ...]``
  tensor whose slice ``r`` lives on rank ``r`` and is readable / writable from every rank;
* ``create_nvl_dist_multicast_tensor``              (buffer.py:244)  -> the same plus an NVLS
  multicast alias (``None`` when the group has one rank or the device has no multicast);
* ``create_nvl_single_owner_tensor``                (buffer.py:338)  -> memory on one rank mapped
  by all;
* ``pad_to_granularity`` / ``pad_dim0_for_alignment`` (buffer.py:89-110);
* env ``MOONEP_MEM_HANDLE_TYPE=auto|fabric|fd``      (buffer.py:25-57).

Additions: ``create_local_group_tensor`` builds all R chunks on ONE device (single-GPU virtual
groups); handle exchange failures raise exceptions instead of exiting the process; tensors
are wrapped through a DLPack capsule (which names the device explicitly) and unmapped when the last view dies or on an
explicit ``release()``.
"""
from __future__ import annotations

import array
import ctypes
import os
import shutil
import socket
import tempfile
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from . import _native as nat
from ._native import I, L, P

U64P = ctypes.POINTER(ctypes.c_uint64)
IP = ctypes.POINTER(ctypes.c_int)

nat.declare("mep_driver_available", I, [])
nat.declare("mep_vmm_supported", I, [I])
nat.declare("mep_launch_multimem_bcast", I, [P, P, L, P])
nat.declare("mep_fabric_supported", I, [I])
nat.declare("mep_multicast_supported", I, [I])
nat.declare("mep_vmm_granularity", L, [I, I])
nat.declare("mep_multicast_granularity", L, [I, L])
nat.declare("mep_symm_alloc", I, [I, L, I, U64P])
nat.declare("mep_symm_export_fd", I, [ctypes.c_uint64, IP])
nat.declare("mep_symm_import_fd", I, [I, U64P])
nat.declare("mep_symm_export_fabric", I, [ctypes.c_uint64, P])
nat.declare("mep_symm_import_fabric", I, [P, U64P])
nat.declare("mep_symm_release", I, [ctypes.c_uint64])
nat.declare("mep_symm_map", I, [I, U64P, I, L, U64P])
nat.declare("mep_symm_unmap", I, [ctypes.c_uint64, I, L])
nat.declare("mep_mc_create", I, [I, L, U64P])
nat.declare("mep_mc_add_device", I, [ctypes.c_uint64, I])
nat.declare("mep_mc_bind", I, [ctypes.c_uint64, ctypes.c_uint64, L])
nat.declare("mep_mc_unbind", I, [ctypes.c_uint64, I, L])

FABRIC_HANDLE_BYTES = 64
_FD_TIMEOUT_S = 120.0


class SymmetricMemoryError(RuntimeError):
    pass


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise SymmetricMemoryError(f"{what}: {nat.last_error()} (code {rc})")


def nvl_fabric_supported(device: Optional[int] = None) -> bool:
    """Fabric (multi-node NVLink) memory handles are usable on this device."""
    device = torch.cuda.current_device() if device is None else device
    return bool(nat.call("mep_fabric_supported", device))


def nvl_multicast_supported(device: Optional[int] = None) -> bool:
    """The device and driver can create NVSwitch multicast objects."""
    device = torch.cuda.current_device() if device is None else device
    return bool(nat.call("mep_multicast_supported", device))


def get_multicast_granularity(num_devices: int, nbytes: int) -> int:
    g = nat.call("mep_multicast_granularity", num_devices, nbytes)
    if g <= 0:
        raise SymmetricMemoryError(f"multicast granularity query failed: {nat.last_error()}")
    return int(g)


def get_vmm_granularity(device: Optional[int] = None, fabric: bool = False) -> int:
    device = torch.cuda.current_device() if device is None else device
    g = nat.call("mep_vmm_granularity", device, int(fabric))
    if g <= 0:
        raise SymmetricMemoryError(f"granularity query failed: {nat.last_error()}")
    return int(g)


def pad_to_granularity(nbytes: int, granularity: Optional[int] = None) -> int:
    """Round ``nbytes`` up to the VMM granularity (moonep/buffer.py:89)."""
    granularity = get_vmm_granularity() if granularity is None else granularity
    return (nbytes + granularity - 1) // granularity * granularity


def pad_dim0_for_alignment(chunk_shape, dtype, granularity: Optional[int] = None) -> int:
    """Smallest ``d >= dim0`` such that a chunk of ``d`` rows is a whole number of VMM granules.

    Called like the reference, ``pad_dim0_for_alignment([epn, H, Hp], torch.bfloat16)``
    (moonep/buffer.py:95), or with plain numbers, ``pad_dim0_for_alignment(dim0, row_bytes, gran)``.
    """
    import math

    if isinstance(chunk_shape, (list, tuple, torch.Size)):
        dim0 = int(chunk_shape[0])
        row_bytes = torch.empty((), dtype=dtype).element_size()
        for d in chunk_shape[1:]:
            row_bytes *= int(d)
    else:
        dim0, row_bytes = int(chunk_shape), int(dtype)
    granularity = get_vmm_granularity() if granularity is None else granularity
    step = granularity // math.gcd(granularity, row_bytes)
    return (dim0 + step - 1) // step * step


def handle_type_for_group(group, device: int) -> str:
    """``fd`` or ``fabric`` per ``MOONEP_MEM_HANDLE_TYPE`` (auto = fabric iff every rank can)."""
    mode = os.environ.get("MOONEP_MEM_HANDLE_TYPE", "auto").lower()
    if mode not in ("auto", "fabric", "fd"):
        raise ValueError(f"MOONEP_MEM_HANDLE_TYPE must be auto|fabric|fd, got {mode!r}")
    if mode != "auto":
        return mode
    mine = torch.tensor([nat.call("mep_fabric_supported", device)], dtype=torch.int32,
                        device=f"cuda:{device}")
    if group is not None and dist.get_world_size(group) > 1:
        all_ = [torch.zeros_like(mine) for _ in range(dist.get_world_size(group))]
        dist.all_gather(all_, mine, group=group)
        ok = all(int(t.item()) for t in all_)
    else:
        ok = bool(int(mine.item()))
    # as in the reference (moonep/buffer.py:28-57): fabric handles iff every rank can really
    # create one (the probe allocates a granule), POSIX file descriptors otherwise
    return "fabric" if ok else "fd"


def exchange_fds(fd: int, group, tag: str = "h") -> list[int]:
    """All-gather one file descriptor per rank over AF_UNIX datagram sockets (SCM_RIGHTS).

    Works with any backend (the directory name travels through ``broadcast_object_list``).
    Returns the R descriptors in rank order; the caller owns (and must close) all of them
    except its own input.  Raises ``SymmetricMemoryError`` on timeout or a short message.
    """
    rank, R = dist.get_rank(group), dist.get_world_size(group)
    box = [tempfile.mkdtemp(prefix="moonep_b200_") if rank == 0 else None]
    dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group else 0, group=group)
    root = box[0]
    path = lambda r: os.path.join(root, f"{tag}{r}")
    sock = socket.socket(socket.AF_UNIX, socket.SOCK_DGRAM)
    out = [-1] * R
    try:
        sock.bind(path(rank))
        sock.settimeout(_FD_TIMEOUT_S)
        dist.barrier(group=group)           # every socket is bound
        for r in range(R):
            if r != rank:
                # sendmsg directly: socket.send_fds() drops its address argument on some
                # Python versions, which a datagram socket cannot live without
                sock.sendmsg([rank.to_bytes(4, "little")],
                             [(socket.SOL_SOCKET, socket.SCM_RIGHTS, array.array("i", [fd]))],
                             0, path(r))
        out[rank] = fd
        for _ in range(R - 1):
            try:
                msg, fds, _flags, _addr = socket.recv_fds(sock, 16, 4)
            except socket.timeout as exc:
                raise SymmetricMemoryError("timed out waiting for a peer's memory handle") from exc
            if len(msg) != 4 or len(fds) != 1:
                raise SymmetricMemoryError("malformed handle message from a peer")
            out[int.from_bytes(msg, "little")] = fds[0]
        dist.barrier(group=group)           # nobody unlinks before all have received
    finally:
        sock.close()
        try:
            os.unlink(path(rank))
        except OSError:
            pass
        if rank == 0:
            shutil.rmtree(root, ignore_errors=True)
    if any(f < 0 for f in out):
        raise SymmetricMemoryError("a peer's memory handle never arrived")
    return out


class _Mapping:
    """Owner of one virtual range (n chunks) and of the physical handles that must outlive it."""

    def __init__(self, device, va, n, chunk_bytes, handles, owned_local=None):
        self.device, self.va, self.n, self.chunk_bytes = device, va, n, chunk_bytes
        self.handles = list(handles)
        self.owned_local = owned_local
        self.alive = True

    def release(self):
        if not self.alive:
            return
        self.alive = False
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            nat.call("mep_symm_unmap", self.va, self.n, self.chunk_bytes)
            for h in self.handles:
                nat.call("mep_symm_release", h)

    def __del__(self):  # pragma: no cover - best effort
        try:
            self.release()
        except Exception:
            pass


# ---- raw device pointer -> torch tensor, through a hand-built DLPack capsule ----------------
# A peer-mapped range starts with rank 0's chunk, so inferring the tensor's device from the
# pointer would be wrong on every other rank; DLPack states the device explicitly.
class _DLDevice(ctypes.Structure):
    _fields_ = [("device_type", ctypes.c_int32), ("device_id", ctypes.c_int32)]


class _DLDataType(ctypes.Structure):
    _fields_ = [("code", ctypes.c_uint8), ("bits", ctypes.c_uint8), ("lanes", ctypes.c_uint16)]


class _DLTensor(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("device", _DLDevice), ("ndim", ctypes.c_int32),
                ("dtype", _DLDataType), ("shape", ctypes.POINTER(ctypes.c_int64)),
                ("strides", ctypes.POINTER(ctypes.c_int64)), ("byte_offset", ctypes.c_uint64)]


class _DLManagedTensor(ctypes.Structure):
    pass


_DELETER = ctypes.CFUNCTYPE(None, ctypes.POINTER(_DLManagedTensor))
_DLManagedTensor._fields_ = [("dl_tensor", _DLTensor), ("manager_ctx", ctypes.c_void_p),
                             ("deleter", _DELETER)]
_LIVE: dict[int, tuple] = {}


@_DELETER
def _dl_deleter(ptr):
    _LIVE.pop(ctypes.addressof(ptr.contents), None)


def _bytes_tensor(mapping: "_Mapping") -> torch.Tensor:
    """uint8 view of the whole mapped range, on ``mapping.device``; keeps ``mapping`` alive."""
    shape = (ctypes.c_int64 * 1)(mapping.n * mapping.chunk_bytes)
    mt = _DLManagedTensor()
    mt.dl_tensor.data = mapping.va
    mt.dl_tensor.device = _DLDevice(2, mapping.device)      # kDLCUDA
    mt.dl_tensor.ndim = 1
    mt.dl_tensor.dtype = _DLDataType(1, 8, 1)               # kDLUInt, 8 bits
    mt.dl_tensor.shape = shape
    mt.dl_tensor.strides = None
    mt.dl_tensor.byte_offset = 0
    mt.manager_ctx = None
    mt.deleter = _dl_deleter
    _LIVE[ctypes.addressof(mt)] = (mt, shape, mapping)
    new_capsule = ctypes.pythonapi.PyCapsule_New
    new_capsule.restype = ctypes.py_object
    new_capsule.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p]
    capsule = new_capsule(ctypes.addressof(mt), b"dltensor", None)
    return torch.from_dlpack(capsule)


def _wrap(mapping: _Mapping, shape: Sequence[int], dtype: torch.dtype, rows_per_chunk: int):
    raw = _bytes_tensor(mapping)
    t = raw.view(dtype).view(mapping.n * rows_per_chunk, *shape[1:])
    t._symm_mapping = mapping
    return t


def _alloc_chunk(device: int, chunk_bytes: int, fabric: bool) -> int:
    h = ctypes.c_uint64()
    _check(nat.call("mep_symm_alloc", device, chunk_bytes, int(fabric), ctypes.byref(h)),
           "allocating a symmetric chunk")
    return h.value


def _map(device: int, handles: list[int], chunk_bytes: int) -> int:
    arr = (ctypes.c_uint64 * len(handles))(*handles)
    va = ctypes.c_uint64()
    _check(nat.call("mep_symm_map", device, arr, len(handles), chunk_bytes, ctypes.byref(va)),
           "mapping symmetric chunks")
    return va.value


def _chunk_geometry(shape, dtype, device, fabric=False):
    esize = torch.empty((), dtype=dtype).element_size()
    row_bytes = esize
    for s in shape[1:]:
        row_bytes *= s
    gran = get_vmm_granularity(device, fabric)
    rows = pad_dim0_for_alignment(int(shape[0]), row_bytes, gran)
    return rows, rows * row_bytes


def create_local_group_tensor(shape, dtype, R: int, device: Optional[int] = None) -> torch.Tensor:
    """``[R * rows, ...]`` with all R chunks on ONE device (single-GPU virtual group).

    ``rows`` is ``shape[0]`` rounded up so that a chunk is a whole number of VMM granules; use
    ``t.shape[0] // R`` as the per-rank stride.
    """
    device = torch.cuda.current_device() if device is None else device
    if not nat.call("mep_vmm_supported", device):
        raise SymmetricMemoryError("device does not support CUDA virtual memory management")
    rows, chunk_bytes = _chunk_geometry(shape, dtype, device)
    handles = [_alloc_chunk(device, chunk_bytes, False) for _ in range(R)]
    va = _map(device, handles, chunk_bytes)
    m = _Mapping(device, va, R, chunk_bytes, handles)
    return _wrap(m, shape, dtype, rows)


def _exchange_and_map(local_handle: int, chunk_bytes: int, group, device: int, fabric: bool):
    rank, R = dist.get_rank(group), dist.get_world_size(group)
    handles = [0] * R
    if fabric:
        buf = (ctypes.c_uint8 * FABRIC_HANDLE_BYTES)()
        _check(nat.call("mep_symm_export_fabric", local_handle, buf), "exporting a fabric handle")
        mine = torch.tensor(list(buf), dtype=torch.uint8, device=f"cuda:{device}")
        allh = torch.empty(R * FABRIC_HANDLE_BYTES, dtype=torch.uint8, device=f"cuda:{device}")
        dist.all_gather_into_tensor(allh, mine, group=group)
        allh = allh.cpu().view(R, FABRIC_HANDLE_BYTES)
        for r in range(R):
            if r == rank:
                handles[r] = local_handle
                continue
            blob = (ctypes.c_uint8 * FABRIC_HANDLE_BYTES)(*allh[r].tolist())
            h = ctypes.c_uint64()
            _check(nat.call("mep_symm_import_fabric", blob, ctypes.byref(h)), "importing a fabric handle")
            handles[r] = h.value
    else:
        fd = ctypes.c_int(-1)
        _check(nat.call("mep_symm_export_fd", local_handle, ctypes.byref(fd)), "exporting a memory handle")
        fds = exchange_fds(fd.value, group)
        try:
            for r in range(R):
                if r == rank:
                    handles[r] = local_handle
                    continue
                h = ctypes.c_uint64()
                _check(nat.call("mep_symm_import_fd", fds[r], ctypes.byref(h)), "importing a memory handle")
                handles[r] = h.value
        finally:
            for f in fds:
                if f >= 0:
                    os.close(f)
    va = _map(device, handles, chunk_bytes)
    return handles, va


def create_nvl_dist_tensor(shape, dtype, local_rank=None, world_size=None, group=None,
                           device: Optional[int] = None) -> torch.Tensor:
    """Symmetric tensor ``[R * rows, *shape[1:]]``: slice ``r`` is rank ``r``'s memory.

    Accepts the reference's call ``create_nvl_dist_tensor(chunk_shape, dtype, rank, R, group)``
    (moonep/buffer.py:217); ``rank`` / ``R`` are then checked against the group.  Unlike the
    reference, a ``shape[0]`` that is not granule-aligned is padded (``rows >= shape[0]``).
    """
    if local_rank is not None and not isinstance(local_rank, int):
        group, local_rank = local_rank, None          # (shape, dtype, group) call style
    if not dist.is_initialized():
        assert world_size in (None, 1), "a process group is required for more than one rank"
        device = torch.cuda.current_device() if device is None else device
        return create_local_group_tensor(shape, dtype, 1, device)
    group = group if group is not None else dist.group.WORLD
    device = torch.cuda.current_device() if device is None else device
    R = dist.get_world_size(group)
    assert world_size in (None, R), f"world_size={world_size} but the group has {R} ranks"
    assert local_rank in (None, dist.get_rank(group)), "local_rank does not match the group"
    if R == 1:
        return create_local_group_tensor(shape, dtype, 1, device)
    if not nat.call("mep_vmm_supported", device):
        raise SymmetricMemoryError("device does not support CUDA virtual memory management")
    fabric = handle_type_for_group(group, device) == "fabric"
    rows, chunk_bytes = _chunk_geometry(shape, dtype, device, fabric)
    local = _alloc_chunk(device, chunk_bytes, fabric)
    handles, va = _exchange_and_map(local, chunk_bytes, group, device, fabric)
    m = _Mapping(device, va, R, chunk_bytes, handles, owned_local=local)
    t = _wrap(m, shape, dtype, rows)
    dist.barrier(group=group)
    return t


def create_nvl_dist_multicast_tensor(shape, dtype, local_rank=None, world_size=None, group=None,
                                     device: Optional[int] = None):
    """``(tensor, multicast_alias | None)``.

    The alias addresses the NVSwitch multicast object bound to every rank's chunk: a
    ``multimem.st`` through it lands in all R copies.  It is ``None`` for one-rank groups, on
    devices without multicast support, and unless ``MOONEP_B200_NVLS=1`` is set (a rank that
    dies while its memory is bound to a multicast object can fault its peers, so the overlay is
    opt-in).
    """
    if local_rank is not None and not isinstance(local_rank, int):
        group, local_rank = local_rank, None
    group = group if group is not None else dist.group.WORLD
    device = torch.cuda.current_device() if device is None else device
    t = create_nvl_dist_tensor(shape, dtype, local_rank, world_size, group, device)
    R = dist.get_world_size(group)
    want = os.environ.get("MOONEP_B200_NVLS") == "1"
    if R == 1 or not want or not nat.call("mep_multicast_supported", device):
        return t, None
    if handle_type_for_group(group, device) == "fabric":
        return t, None          # the overlay below shares its multicast object through file descriptors
    m: _Mapping = t._symm_mapping
    rank = dist.get_rank(group)
    gran = nat.call("mep_multicast_granularity", R, m.chunk_bytes)
    if gran <= 0 or m.chunk_bytes % gran != 0:
        return t, None
    mc = ctypes.c_uint64()
    if rank == 0:
        _check(nat.call("mep_mc_create", R, m.chunk_bytes, ctypes.byref(mc)), "creating the multicast object")
        fd = ctypes.c_int(-1)
        _check(nat.call("mep_symm_export_fd", mc.value, ctypes.byref(fd)), "exporting the multicast handle")
        my_fd = fd.value
    else:
        my_fd = os.open(os.devnull, os.O_RDONLY)   # placeholder so that everyone sends one fd
    fds = exchange_fds(my_fd, group, tag="m")
    try:
        if rank != 0:
            _check(nat.call("mep_symm_import_fd", fds[0], ctypes.byref(mc)), "importing the multicast handle")
    finally:
        for f in set(fds):
            if f >= 0:
                os.close(f)
    _check(nat.call("mep_mc_add_device", mc.value, device), "adding the device to the multicast object")
    dist.barrier(group=group)
    _check(nat.call("mep_mc_bind", mc.value, m.owned_local, m.chunk_bytes), "binding memory to the multicast object")
    va = _map(device, [mc.value], m.chunk_bytes)
    dist.barrier(group=group)
    mm = _Mapping(device, va, 1, m.chunk_bytes, [mc.value])
    rows = t.shape[0] // R
    alias = _wrap(mm, shape, dtype, rows)
    return t, alias


def create_nvl_single_owner_tensor(shape, dtype, owner: int, group=None, device: Optional[int] = None):
    """Memory that lives on rank ``owner`` only and is mapped read/write by every rank."""
    group = group if group is not None else dist.group.WORLD
    device = torch.cuda.current_device() if device is None else device
    rank, R = dist.get_rank(group), dist.get_world_size(group)
    rows, chunk_bytes = _chunk_geometry(shape, dtype, device)
    if R == 1:
        return create_local_group_tensor(shape, dtype, 1, device)[: shape[0]]
    local = _alloc_chunk(device, chunk_bytes, False) if rank == owner else None
    if rank == owner:
        fd = ctypes.c_int(-1)
        _check(nat.call("mep_symm_export_fd", local, ctypes.byref(fd)), "exporting a memory handle")
        my_fd = fd.value
    else:
        my_fd = os.open(os.devnull, os.O_RDONLY)
    fds = exchange_fds(my_fd, group, tag="s")
    try:
        if rank == owner:
            handle = local
        else:
            h = ctypes.c_uint64()
            _check(nat.call("mep_symm_import_fd", fds[owner], ctypes.byref(h)), "importing a memory handle")
            handle = h.value
    finally:
        for f in set(fds):
            if f >= 0:
                os.close(f)
    va = _map(device, [handle], chunk_bytes)
    m = _Mapping(device, va, 1, chunk_bytes, [handle], owned_local=local)
    t = _wrap(m, shape, dtype, rows)
    dist.barrier(group=group)
    return t[: shape[0]]


def multimem_broadcast(alias: torch.Tensor, src: torch.Tensor, offset: int = 0) -> None:
    """Store ``src`` (any 4-byte dtype, contiguous, local) through the multicast ``alias`` of a
    symmetric tensor at element ``offset``: the words land at the same place in EVERY rank's chunk
    (NVSwitch ``multimem.st``, the reference's plan broadcast, moonep/planning.py:147-156).  They
    are visible on the other ranks after the caller's next cross-rank synchronisation."""
    assert alias.element_size() == 4 and src.element_size() == 4 and src.is_contiguous() and src.is_cuda
    assert 0 <= offset and offset + src.numel() <= alias.numel()
    rc = nat.call("mep_launch_multimem_bcast", alias.data_ptr() + 4 * offset, src.data_ptr(), src.numel(),
                  torch.cuda.current_stream().cuda_stream)
    if rc != 0:
        raise SymmetricMemoryError(f"multimem broadcast: {nat.last_error()}")


def release(t: torch.Tensor) -> None:
    """Unmap a symmetric tensor now (all its views become dangling)."""
    m = getattr(t, "_symm_mapping", None)
    if m is not None:
        m.release()
