"""Sequence-parallel group, ring neighbours, double-buffered slabs and the P2P helpers of the step loop.

Mirrors the interface of the reference's lv_xattn/async_communication.py (same function names and env
contract) on a different transport plan:
  * one process per GPU, `torch.distributed` P2P (NCCL on GPUs; any initialised backend is accepted, which
    is what lets the step loop run on gloo CPU ranks in the tests)        -> reference :38-59, :292-299
  * every step moves ONE coalesced slab per direction instead of 2-5 tensors:
      forward   Q block (W-1 hops)              and  [O | lse] accumulator (W hops)
      backward  [Q | dO | lse | delta] (W-1 hops) and  fp32 dQ accumulator (W hops)
    (the reference sends q, L, o, dO separately and recomputes delta on every rank: :247-273)
  * waits carry a deadline and raise P2PTimeoutError instead of blocking forever (reference :301-305).
"""
from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as dist
from torch.distributed import P2POp, irecv, isend

_SEQUENCE_PARALLEL_GROUP = None
_SEQUENCE_PARALLEL_RANK = None
_SEQUENCE_PARALLEL_SIZE = None

# slab pools: {key: [buf0, buf1]}
_POOL: dict = {}

# seconds a wait may take before P2PTimeoutError is raised (host-visible backends only; NCCL waits are
# stream-ordered and bounded by the process group's own timeout)
P2P_TIMEOUT_S = float(os.environ.get("LVX_P2P_TIMEOUT_S", "120"))


class P2PTimeoutError(RuntimeError):
    """A peer did not deliver within the deadline (lost or stalled rank)."""


# --------------------------------------------------------------------------------------------------
# group management (reference :38-93, :183-208)
# --------------------------------------------------------------------------------------------------
def initialize_distributed(backend: str | None = None):
    """Creates the world process group from RANK / WORLD_SIZE / LOCAL_RANK if none exists, then (re)builds
    the sequence-parallel group over all ranks. An already initialised process group of any backend is
    reused as is (reference :39-45)."""
    if not dist.is_initialized():
        rank = int(os.environ["RANK"])
        world = int(os.environ["WORLD_SIZE"])
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        kwargs = {}
        if backend == "nccl":
            local = int(os.environ.get("LOCAL_RANK", rank))
            torch.cuda.set_device(local)
            kwargs["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend=backend, rank=rank, world_size=world, **kwargs)
    destroy_sequence_parallel()
    _initialize_sequence_parallel()


def _initialize_sequence_parallel(sequence_parallel_size=None):
    global _SEQUENCE_PARALLEL_GROUP, _SEQUENCE_PARALLEL_RANK, _SEQUENCE_PARALLEL_SIZE
    if sequence_parallel_size is not None:
        raise NotImplementedError("Multiple sequence parallel group not implemented.")
    if not dist.is_initialized():
        raise RuntimeError("torch.distributed is not initialised")
    if _SEQUENCE_PARALLEL_GROUP is not None:
        raise RuntimeError("sequence parallel group is already initialized")
    world = dist.get_world_size()
    _SEQUENCE_PARALLEL_GROUP = dist.new_group(list(range(world)))
    _SEQUENCE_PARALLEL_RANK = dist.get_rank()
    _SEQUENCE_PARALLEL_SIZE = world


def sequence_parallel_is_initialized() -> bool:
    return _SEQUENCE_PARALLEL_GROUP is not None


def get_sequence_parallel_group():
    if _SEQUENCE_PARALLEL_GROUP is None:
        raise RuntimeError("sequence parallel group is not initialized")
    return _SEQUENCE_PARALLEL_GROUP


def get_sequence_parallel_rank() -> int:
    """Rank inside the sequence-parallel group; 0 when no group exists (single-GPU use needs none)."""
    if _SEQUENCE_PARALLEL_GROUP is None:
        return 0
    return _SEQUENCE_PARALLEL_RANK


def get_sequence_parallel_size() -> int:
    if _SEQUENCE_PARALLEL_GROUP is None:
        return 1
    return _SEQUENCE_PARALLEL_SIZE


def destroy_sequence_parallel():
    global _SEQUENCE_PARALLEL_GROUP, _SEQUENCE_PARALLEL_RANK, _SEQUENCE_PARALLEL_SIZE
    _SEQUENCE_PARALLEL_GROUP = None
    _SEQUENCE_PARALLEL_RANK = None
    _SEQUENCE_PARALLEL_SIZE = None


def ring_neighbours():
    """(send_to, recv_from) = (rank+1, rank-1) mod W as global ranks (reference :217-218)."""
    r, w = get_sequence_parallel_rank(), get_sequence_parallel_size()
    return (r + 1) % w, (r - 1) % w


# --------------------------------------------------------------------------------------------------
# slab pools (reference :95-156)
# --------------------------------------------------------------------------------------------------
def get_slabs(kind: str, nbytes: int, device, count: int = 2):
    """`count` reusable byte buffers of at least `nbytes` for the role `kind` ("fwd_q", "fwd_acc", ...).
    Buffers are module-owned scratch, reused across calls of the same size and dropped by
    reset_global_memory_buffer()."""
    key = (kind, str(device))
    bufs = _POOL.get(key)
    if bufs is None or len(bufs) < count or bufs[0].numel() < nbytes:
        # 256-byte granularity keeps every carved view 16-byte aligned
        n = (max(nbytes, 256) + 255) // 256 * 256
        bufs = [torch.empty(n, dtype=torch.uint8, device=device) for _ in range(count)]
        _POOL[key] = bufs
    return bufs


def maybe_get_set_global_memory_buffer(q, acc_nbytes: int):
    """Forward ring pools: two Q slabs, two outgoing and two incoming [O | lse] accumulator slabs
    (the reference keeps 2x{Q, M, L, O}, lv_xattn/async_communication.py:95-108)."""
    n = q.numel() * q.element_size()
    return (get_slabs("fwd_q", n, q.device, 2), get_slabs("fwd_acc_send", acc_nbytes, q.device, 2),
            get_slabs("fwd_acc_recv", acc_nbytes, q.device, 2))


def maybe_get_set_global_memory_buffer_bwd(slab_nbytes: int, dq_nbytes: int, device):
    """Backward ring pools: three [Q | dO | lse | delta] slabs, two outgoing and two incoming fp32 dQ slabs
    (reference: lv_xattn/async_communication.py:110-133)."""
    return (get_slabs("bwd_in", slab_nbytes, device, 3), get_slabs("bwd_dq_send", dq_nbytes, device, 2),
            get_slabs("bwd_dq_recv", dq_nbytes, device, 2))


def reset_global_memory_buffer():
    """Drops every pooled slab and the kernels' scratch workspace (reference :135-156)."""
    _POOL.clear()
    from . import ops
    ops.release_workspaces()


# --------------------------------------------------------------------------------------------------
# P2P (reference :210-305)
# --------------------------------------------------------------------------------------------------
def _exchange(send_tensors, recv_tensors, comm_mode):
    group = get_sequence_parallel_group()
    send_rank, recv_rank = ring_neighbours()
    ops_ = []
    # receives first: a rank whose send blocks until matched still has its receive posted
    for t in recv_tensors:
        ops_.append(P2POp(op=irecv, tensor=t, peer=recv_rank, group=group))
    for t in send_tensors:
        ops_.append(P2POp(op=isend, tensor=t, peer=send_rank, group=group))
    return [launch_async_handles(ops_, comm_mode)]


def send_recv_fwd_q(q_send, q_recv, bias_args_send, bias_args_recv, comm_mode):
    """Q block to rank+1, next Q block from rank-1 (reference :210-227)."""
    return _exchange([q_send, *bias_args_send], [q_recv, *bias_args_recv], comm_mode)


def send_recv_fwd_Lo(acc_send, acc_recv, comm_mode):
    """Travelling [O | lse] accumulator slab to rank+1 / from rank-1 (reference :229-245, one slab here)."""
    return _exchange([acc_send], [acc_recv], comm_mode)


def send_recv_bwd_comp_reqs(slab_send, slab_recv, bias_args_send, bias_args_recv, comm_mode):
    """[Q | dO | lse | delta] slab to rank+1 / from rank-1 (reference :247-273, one slab here)."""
    return _exchange([slab_send, *bias_args_send], [slab_recv, *bias_args_recv], comm_mode)


def send_recv_bwd_rescale_reqs(dq_send, dq_recv, comm_mode):
    """Travelling dQ accumulator to rank+1 / from rank-1 (reference :275-289)."""
    return _exchange([dq_send], [dq_recv], comm_mode)


def all_gather_blocks(local_tensors, gathered, comm_mode):
    """gathered[i][s] <- rank s's local_tensors[i] for every rank s; gathered[i] is a contiguous [W, ...]
    tensor. One NCCL all-gather per tensor (every pair exchanges directly over NVSwitch; the bytes per GPU
    equal W-1 ring hops of the same block)."""
    if comm_mode == "nocomm":
        for t, g in zip(local_tensors, gathered):
            g[get_sequence_parallel_rank()].copy_(t)
        return []
    group = get_sequence_parallel_group()
    works = []
    for t, g in zip(local_tensors, gathered):
        works.append(dist.all_gather_into_tensor(g.view(-1), t.contiguous().view(-1), group=group, async_op=True))
    return [works]


def all_to_all_blocks(pairs, comm_mode):
    """For every (send, recv) pair of contiguous [W, ...] tensors: send[s] goes to rank s, recv[s] comes from
    rank s (one NCCL all-to-all per pair)."""
    if comm_mode == "nocomm":
        r = get_sequence_parallel_rank()
        for sd, rv in pairs:
            rv[r].copy_(sd[r])
        return []
    group = get_sequence_parallel_group()
    works = []
    for sd, rv in pairs:
        works.append(dist.all_to_all_single(rv.view(-1), sd.view(-1), group=group, async_op=True))
    return [works]


def launch_async_handles(handles, comm_mode):
    if comm_mode == "nocomm":
        return []
    if len(handles) > 0:
        return dist.batch_isend_irecv(handles)
    return []


def wait_async_handles(reqs, timeout_s: float | None = None):
    """Completes every request. On NCCL this only orders the current stream after the transfer (no host
    block, so compute keeps overlapping; a lost peer surfaces through the process group's own timeout).
    On host backends it blocks up to `timeout_s` (default P2P_TIMEOUT_S) and raises P2PTimeoutError."""
    if not reqs:
        return
    limit = P2P_TIMEOUT_S if timeout_s is None else timeout_s
    on_stream = dist.get_backend(get_sequence_parallel_group()) == "nccl"
    for group in reqs:
        for r in group:
            if on_stream:
                r.wait()
                continue
            try:
                ok = r.wait(datetime.timedelta(seconds=limit))
            except RuntimeError as e:
                if "timeout" in str(e).lower() or "timed out" in str(e).lower():
                    raise P2PTimeoutError(f"P2P wait exceeded {limit} s: {e}") from e
                raise
            if ok is False:
                raise P2PTimeoutError(f"P2P wait exceeded {limit} s")
