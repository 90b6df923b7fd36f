"""Peer-mapped buffers of the sequence-parallel group, for the exchange steps that the library's own kernels do
over NVLink (`schedule="p2p"`): one buffer per role on every rank, mapped into every other rank's address space
through torch's symmetric memory (CUDA VMM handles exchanged over the group's store), plus the flag array of the
signal/wait protocol (csrc/p2p.cu).

Nothing here has a counterpart in the reference, which sends every block through NCCL point-to-point calls
(send_recv_fwd_q, send_recv_fwd_Lo, send_recv_bwd_comp_reqs, send_recv_bwd_rescale_reqs,
lv_xattn/async_communication.py:210-289).

Every rank must create the same buffers in the same order (creation is a collective). Multicast (NVLS) binding of
the buffers is switched off: only plain peer loads and stores are used.
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from . import _lib
from .async_communication import get_sequence_parallel_group, get_sequence_parallel_rank, get_sequence_parallel_size

SLOT_FWD_Q, SLOT_FWD_PARTS, SLOT_BWD_IN, SLOT_BWD_DQ = 0, 1, 2, 3

_BUFFERS = {}
_FLAGS = None
_EPOCHS = [0] * _lib.P2P_SLOTS


class PeerBuffer:
    """`local`: this rank's buffer (uint8 tensor); `peers`: the LvxPeers table of every rank's copy."""

    def __init__(self, nbytes: int, device):
        import torch.distributed._symmetric_memory as symm_mem
        group = get_sequence_parallel_group()
        W = get_sequence_parallel_size()
        if W > _lib.MAX_PEERS:
            raise ValueError(f"at most {_lib.MAX_PEERS} ranks can share peer buffers")
        self.nbytes = nbytes
        self.local = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        handle = symm_mem.rendezvous(self.local, group)
        ptrs = [int(p) for p in handle.buffer_ptrs]
        if len(ptrs) != W or ptrs[get_sequence_parallel_rank()] != self.local.data_ptr():
            raise RuntimeError("symmetric-memory rendezvous returned an unexpected peer table")
        self._handle = handle          # keeps the mappings alive
        self.peers = _lib.LvxPeers()
        self.peers.world, self.peers.rank = W, get_sequence_parallel_rank()
        self.peers.nbytes = nbytes
        for i, a in enumerate(ptrs):
            self.peers.ptr[i] = a


def _ensure_env():
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")


_TIMEOUT_SET = False


def apply_wait_limit():
    """The in-kernel flag waits share the host waits' limit (LVX_P2P_TIMEOUT_S, 120 s unless set)."""
    global _TIMEOUT_SET
    if not _TIMEOUT_SET:
        from .async_communication import P2P_TIMEOUT_S
        _lib.check(_lib.load().lvx_p2p_set_timeout(float(P2P_TIMEOUT_S)), "lvx_p2p_set_timeout")
        _TIMEOUT_SET = True


def get_peer_buffer(name: str, nbytes: int, device) -> PeerBuffer:
    """Buffer for role `name`, at least nbytes long; re-created (collectively) when it has to grow."""
    _ensure_env()
    key = (name, str(device))
    buf = _BUFFERS.get(key)
    if buf is None or buf.nbytes < nbytes:
        n = (max(nbytes, 4096) + 4095) // 4096 * 4096
        buf = PeerBuffer(n, device)
        _BUFFERS[key] = buf
    return buf


def get_flags(device):
    """(peer table of the flag arrays, this rank's flag array as an int32 tensor)."""
    global _FLAGS
    _ensure_env()
    if _FLAGS is None:
        apply_wait_limit()
        buf = PeerBuffer(4096, device)
        buf.local.zero_()
        torch.cuda.current_stream(device).synchronize()
        dist.barrier(group=get_sequence_parallel_group())     # nobody signals before every array is zero
        _FLAGS = (buf, buf.local.view(torch.int32))
    return _FLAGS[0].peers, _FLAGS[1]


_AVAILABLE = None


def peer_memory_available(device) -> bool:
    """True when every rank of the group could map the flag arrays (decided once, collectively, so that all
    ranks pick the same schedule). A failure on any rank -- no peer access, symmetric memory not supported by
    the driver, more than MAX_PEERS ranks -- makes it False everywhere, with the reason in a warning."""
    global _AVAILABLE
    if _AVAILABLE is None:
        ok = 1
        try:
            if dist.get_backend(get_sequence_parallel_group()) != "nccl":
                raise RuntimeError("the process group is not NCCL")
            get_flags(device)
        except Exception as e:  # noqa: BLE001 - any failure means "use the NCCL schedule"
            import warnings
            warnings.warn(f"peer-mapped exchange unavailable, using NCCL collectives instead: {e}")
            ok = 0
        t = torch.tensor([ok], dtype=torch.int32, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=get_sequence_parallel_group())
        _AVAILABLE = bool(t.item())
    return _AVAILABLE


class StatusWatch:
    """Notices, without synchronising the host, that a bounded in-kernel wait ran out (a peer that never
    signalled). After the last kernel of a call `post()` enqueues a copy of the device status word into pinned
    host memory; `poll()` at the start of the next call (and `check()` on demand) reads what has arrived and raises
    P2PTimeoutError. While the word is set every kernel of the library returns at once, so the outputs of the
    failing call -- and of anything launched before the error is raised -- hold no result and must be dropped."""

    def __init__(self):
        self._slots = []          # [pinned int32 tensor, event or None]
        self._next = 0

    def _slot(self):
        if len(self._slots) < 4:
            self._slots.append([torch.zeros(1, dtype=torch.int32).pin_memory(), None])
            return self._slots[-1]
        s = self._slots[self._next % 4]
        self._next += 1
        if s[1] is not None:      # still unread from four calls ago: read it now
            self._read(s)
        return s

    def _read(self, s):
        ev = s[1]
        s[1] = None
        ev.synchronize()
        code = int(s[0].item())
        if code:
            _lib.device_status()                      # clears the word (and synchronises)
            from .async_communication import P2PTimeoutError
            what = f"rank {code & 0xFF} did not signal within the limit" if (code & 0xFF00) == 0x1300 else "a pipeline wait ran out"
            raise P2PTimeoutError(f"device status word {code:#x}: {what}; the results of the affected call are invalid")

    def post(self):
        s = self._slot()
        _lib.check(_lib.load().lvx_device_status_peek(_lib.stream_ptr(), ctypes.c_void_p(s[0].data_ptr())),
                   "lvx_device_status_peek")
        ev = torch.cuda.Event()
        ev.record()
        s[1] = ev

    def poll(self):
        """Reads every posted copy whose stream position has been reached; never blocks."""
        for s in self._slots:
            if s[1] is not None and s[1].query():
                self._read(s)

    def check(self):
        """Blocks until every posted copy has arrived and raises if any is non-zero."""
        for s in self._slots:
            if s[1] is not None:
                self._read(s)


status_watch = StatusWatch()


def check_device_status():
    """Blocking form of the check the step loop does one call late: raises P2PTimeoutError if any exchange since
    the last check gave up on a peer. Call it before trusting a step's results (before an optimizer step or a
    checkpoint), or set LVX_STATUS_CHECK=sync to have every backward end with it."""
    status_watch.check()


_SIDE = {}


def side_stream(device):
    """The stream the outgoing stores of the fused schedule run on, one per device."""
    key = str(device)
    if key not in _SIDE:
        _SIDE[key] = torch.cuda.Stream(device)
    return _SIDE[key]


def next_epoch(slot: int) -> int:
    _EPOCHS[slot] += 1
    return _EPOCHS[slot]


def reset_peer_memory():
    """Forgets every buffer (collective: all ranks must call it together, with no exchange in flight)."""
    global _FLAGS, _AVAILABLE, _TIMEOUT_SET
    _TIMEOUT_SET = False
    _BUFFERS.clear()
    _FLAGS = None
    _AVAILABLE = None
    for i in range(len(_EPOCHS)):
        _EPOCHS[i] = 0
