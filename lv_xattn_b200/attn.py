"""LV-XAttn step loop: sequence-parallel cross-attention forward and backward.

Same entry points, argument order and return conventions as the reference's lv_xattn/attn.py
(`_attn_forward` :297-435, `_attn_backward` :437-545), plus the two autograd wrappers the reference's
drivers build around them (test.py:38-77 "save q,k,v"; test_llama3.py:180-245 "recompute q,k,v").

Sharding (reference test.py:164-178): rank r holds rows [r*Sq/W, (r+1)*Sq/W) of Q/dO/O and rows
[r*Skv/W, (r+1)*Skv/W) of K/V. K/V never move. At step t a rank works on the Q block born on rank r-t:
  forward   partials = flash block(Q_blk, local K/V)            (tensor-core kernel, independent of the ring)
            acc_out  = merge(acc_in, partials)                  (one HBM-bound kernel; acc_in arrives from r-1)
            acc_out -> rank r+1; after W hops the finished (O, lse) is back home
  backward  dQ_delta, dK+=, dV+= = flash bwd block(Q_blk, dO_blk, lse_blk, delta_blk, local K/V)
            dQ_out = dQ_in + dQ_delta -> rank r+1; after W hops dQ is home
Differences from the reference that are deliberate: the travelling accumulators are fp32 (reference: fp16,
:448,:527), the empty accumulator is (0, -inf) instead of lse = 0 (:319), the result is taken from the slot
that actually holds it for every W (reference returns slot 0, wrong for odd W, :435), delta is computed once
at home and travels instead of O (:926-942 recomputes it on every rank), K/V are used at their own head
count (no expansion, :392-393), and key padding has a native form (a per-batch valid length, handled inside the
tensor-core kernels). The reference's general bias protocol -- bias_func(*local_bias_args, *remote_bias_args),
the remote arguments travelling with the query block (:359-360, :373-374, :386-389) -- is kept: with a bias_func
the step loop runs one block per step and the block kernels are the general FP32-FMA ones.
"""
from __future__ import annotations

import os

import torch

from . import ops
from .async_communication import (
    _exchange,
    get_sequence_parallel_rank,
    get_sequence_parallel_size,
    get_slabs,
    maybe_get_set_global_memory_buffer,
    maybe_get_set_global_memory_buffer_bwd,
    all_gather_blocks,
    all_to_all_blocks,
    reset_global_memory_buffer,
    send_recv_bwd_comp_reqs,
    send_recv_bwd_rescale_reqs,
    send_recv_fwd_Lo,
    send_recv_fwd_q,
    wait_async_handles,
)

_SUPPORTED = (torch.bfloat16, torch.float16, torch.float32)


_DEFAULT_SCHEDULE = "auto"
_PUSH_DMA = os.environ.get("LVX_PUSH", "dma") == "dma"   # outgoing blocks of the fused schedule: copy engines or a kernel
# The peer-memory form "auto" picks. Unset: the fused form ("p2p") up to four ranks, the pull form above that --
# the fused form issues one copy-engine transfer per peer and segment, and on eight B200s that host work outweighs
# the exchange it hides (measured 2.45 ms against 2.39 ms per pass; at two and four ranks the fused form is ahead).
_AUTO_PEER_SCHEDULE = os.environ.get("LVX_AUTO_PEER_SCHEDULE", "")
_FUSED_MAX_RANKS = 4


def _schedule(schedule, like=None):
    """"auto" (default): a peer-memory form ("p2p" up to four ranks, "p2p_pull" above) when every rank of the group
    can map its peers' memory, else "gather".
    "gather": every rank fetches all W query blocks, makes ONE pass over its K/V shard and the
    partial results are exchanged and reduced at home -- one kernel launch per pass, dK/dV written once.
    "ring": the reference's step loop, one query block per step with travelling accumulators
    (lv_xattn/attn.py:364-429). "p2p": the "gather" schedule with every exchange done by this library over
    peer-mapped memory instead of NCCL calls (peer_memory.py; CUDA devices of one NVLink domain only): each rank's
    copy engines store its query-side block into the consumers' buffers while the consumers' kernel already works
    on its own block and waits, per block, for the flag that follows each transfer. "p2p_pull": consumers load the
    blocks from the producers' buffers with one gather kernel before the compute kernel starts. All move the same
    bytes per GPU; LVX_SCHEDULE overrides the default."""
    s = schedule or os.environ.get("LVX_SCHEDULE", _DEFAULT_SCHEDULE)
    if s == "auto":
        # p2p where every rank can map its peers' memory (decided once, collectively), NCCL collectives otherwise
        s = "gather"
        if like is not None and like.is_cuda and get_sequence_parallel_size() > 1:
            from .peer_memory import peer_memory_available
            if peer_memory_available(like.device):
                s = _AUTO_PEER_SCHEDULE or ("p2p" if get_sequence_parallel_size() <= _FUSED_MAX_RANKS else "p2p_pull")
    if s not in ("gather", "ring", "p2p", "p2p_pull"):
        raise ValueError(f"unknown schedule {s!r}")
    return s


def _check_common(q, k, v, causal, bias_func, local_bias_args, remote_bias_args):
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("q, k, v must be [batch, heads, seq, head_dim]")
    Dq, Dk, Dv = q.shape[-1], k.shape[-1], v.shape[-1]
    if not (Dq == Dk == Dv):
        raise ValueError(f"head dimensions differ: {Dq}, {Dk}, {Dv}")
    if Dq != 128:
        raise ValueError(f"head dimension {Dq} unsupported (128 only)")
    if k.shape[-2] != v.shape[-2] or k.shape[1] != v.shape[1]:
        raise ValueError("k and v must agree on heads and sequence length")
    if q.shape[1] % k.shape[1]:
        raise ValueError(f"{q.shape[1]} query heads are not a multiple of {k.shape[1]} KV heads")
    if q.dtype not in _SUPPORTED or k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("q, k, v must share one dtype out of bfloat16, float16, float32")
    if bias_func is None:
        if len(local_bias_args) or len(remote_bias_args):
            raise ValueError("bias arguments given without a bias_func")
    elif not callable(bias_func):
        raise ValueError("bias_func must be callable: bias_func(*local_bias_args, *remote_bias_args) -> bias")
    if causal:
        raise NotImplementedError(
            "causal=True is not supported: cross-attention has no causal order, and the reference applies "
            "the mask with rank-local indices at every step (lv_xattn/attn.py:229,237)")


def _local_valid(kv_valid_len, skv_local: int, device):
    """Global key-padding lengths [B] -> this rank's clamp min(max(valid - rank*Skv_l, 0), Skv_l)."""
    if kv_valid_len is None:
        return None
    t = torch.as_tensor(kv_valid_len, device=device).to(torch.int64)
    t = (t - get_sequence_parallel_rank() * skv_local).clamp_(0, skv_local)
    return t.to(torch.int32).contiguous()


def _build_bias(bias_func, local_bias_args, peer_bias_args, q, k):
    """The reference's bias protocol (lv_xattn/attn.py:386-389): the additive bias of one step is
    bias_func(*local_bias_args, *peer_bias_args) -> [B, 1 or H, Sq_local, Skv_local], where the local arguments
    belong to this rank's K/V shard and the peer arguments arrived with the query block. It is added to the scaled
    scores (S = sm_scale*q.k + bias); steps with a bias run the general FP32-FMA kernels."""
    if bias_func is None:
        return None
    bias = bias_func(*(list(local_bias_args) + list(peer_bias_args)))
    if not torch.is_tensor(bias) or bias.dim() != 4:
        raise ValueError("bias_func must return a 4-D tensor broadcastable to [B, H, Sq, Skv]")
    return bias.to(device=q.device, dtype=torch.float32)


def _status_poll(t):
    """Start of a call: raise if a kernel of an earlier call gave up on a bounded wait (see peer_memory.StatusWatch)."""
    if t.is_cuda:
        from .peer_memory import status_watch
        status_watch.poll()


def _status_post(t):
    """End of a call: queue a look at the device status word behind the call's last kernel (no synchronisation)."""
    if t.is_cuda:
        from .peer_memory import status_watch
        status_watch.post()


def _carve(buf: torch.Tensor, offset: int, shape, dtype) -> torch.Tensor:
    n = 1
    for s in shape:
        n *= s
    nbytes = n * torch.empty((), dtype=dtype).element_size()
    return buf[offset:offset + nbytes].view(dtype).view(*shape)


def _attn_forward(q, k, v, causal, sm_scale, comm_mode, bias_func=None, local_bias_args=[], remote_bias_args=[],
                  no_overlap=False, kv_valid_len=None, schedule=None):
    """Returns (q, k, v, o, L): o like q, L fp32 [B*Hq, Sq_local] natural-log lse (reference :297-435).

    comm_mode == "nocomm" runs the W-step schedule without any transfer (timing ablation, as in the
    reference :294-296); the result is then the attention of the local Q block over the local K/V only.
    kv_valid_len: optional global number of valid K/V rows per batch entry (key padding)."""
    _check_common(q, k, v, causal, bias_func, local_bias_args, remote_bias_args)
    _status_poll(q)
    W = get_sequence_parallel_size()
    B, Hq, Sq, D = q.shape
    dev, dt = q.device, q.dtype
    es = q.element_size()
    qc, kc, vc = q.contiguous(), k.contiguous(), v.contiguous()
    kvl = _local_valid(kv_valid_len, k.shape[2], dev)
    o = torch.empty(B, Hq, Sq, D, dtype=dt, device=dev)
    L = torch.empty(B * Hq, Sq, dtype=torch.float32, device=dev)

    if W == 1 or comm_mode == "nocomm":
        bias = _build_bias(bias_func, local_bias_args, remote_bias_args, qc, kc)
        for _ in range(W):
            part = ops.fwd_partials(qc, kc, vc, sm_scale, kvl, bias=bias)
            ops.fwd_combine(part, None, None, o, L, True)
        _status_post(q)
        return q, k, v, o, L

    n_o, n_l = B * Hq * Sq * D, B * Hq * Sq
    # a bias is built per step from arguments that travel with the query block: the step loop is the only schedule
    sched = "ring" if bias_func is not None else _schedule(schedule, q)
    if sched in ("p2p", "p2p_pull") and (n_l * 4) % 16:
        if (schedule or os.environ.get("LVX_SCHEDULE", _DEFAULT_SCHEDULE)) != "auto":
            raise ValueError("the p2p schedules need B*Hq*Sq to be a multiple of 4")
        sched = "gather"          # picked by "auto": the exchange kernels copy 16 bytes at a time
    if sched == "p2p":
        from . import peer_memory as pm
        pm.status_watch.poll()
        rank = pm.get_sequence_parallel_rank()
        flag_peers, my_flags = pm.get_flags(dev)
        main, side = torch.cuda.current_stream(dev), pm.side_stream(dev)
        # Fused exchange + compute. The Q block goes into this rank's own slot of the gathered buffer with a local
        # copy and to the peers' slots from a side stream (posted NVLink stores + epoch); the multi-block kernel
        # starts at once with the local block and waits, inside the kernel and block by block, for the others.
        e = pm.next_epoch(pm.SLOT_FWD_Q)
        qbuf = pm.get_peer_buffer("p2p_q_all", 2 * W * n_o * es, dev)
        q_off = (e & 1) * W * n_o * es
        q_all = _carve(qbuf.local, q_off, (W, B, Hq, Sq, D), dt)
        q_all[rank].copy_(qc)
        ready = torch.cuda.Event()
        ready.record(main)
        with torch.cuda.stream(side):
            side.wait_event(ready)              # after everything the caller queued, and after the previous exchange
            # by the copy engines: they need no SM, so they make progress whatever kernel fills the GPU (a store
            # kernel queued behind a compute kernel that waits for the peer's stores would never start)
            ops.p2p_push(qbuf.peers, flag_peers, [(qc, False, q_off, n_o * es)], pm.SLOT_FWD_Q, e, skip_self=True,
                         dma=_PUSH_DMA)
            pushed = torch.cuda.Event()
            pushed.record(side)
        if not _PUSH_DMA:
            main.wait_event(pushed)             # a store kernel must have run before the kernel that waits for peers
        wait = (my_flags, pm.SLOT_FWD_Q, e, rank) if dt != torch.float32 else None
        if wait is None:
            ops.p2p_wait(my_flags, W, pm.SLOT_FWD_Q, e)
        part = ops.fwd_partials(q_all, kc, vc, sm_scale, kvl, block_wait=wait)
        sbuf = get_slabs("g_acc_send", W * (n_o + n_l) * 4, dev, 1)[0]
        o_parts = _carve(sbuf, 0, (W, B, Hq, Sq, D), torch.float32)
        l_parts = _carve(sbuf, W * n_o * 4, (W * B * Hq, Sq), torch.float32)
        ops.fwd_combine(part, None, None, o_parts, l_parts, False)
        # partial (O, lse) of block s goes to rank s; the owner merges what it received
        e = pm.next_epoch(pm.SLOT_FWD_PARTS)
        blk = W * (n_o + n_l) * 4
        pbuf = pm.get_peer_buffer("p2p_parts_recv", 2 * blk, dev)
        p_off = (e & 1) * blk
        ops.p2p_push(pbuf.peers, flag_peers, [(o_parts, True, p_off, n_o * 4), (l_parts, True, p_off + W * n_o * 4, n_l * 4)],
                     pm.SLOT_FWD_PARTS, e)
        ops.p2p_wait(my_flags, W, pm.SLOT_FWD_PARTS, e)
        o_recv = _carve(pbuf.local, p_off, (W, B, Hq, Sq, D), torch.float32)
        l_recv = _carve(pbuf.local, p_off + W * n_o * 4, (W, B * Hq, Sq), torch.float32)
        ops.fwd_merge_parts(o_recv, l_recv, dt, o_out=o, lse_out=L)
        main.wait_event(pushed)                 # the caller may reuse q once this call's work is done
        pm.status_watch.post()
        return q, k, v, o, L
    if sched == "p2p_pull":
        from . import peer_memory as pm
        pm.status_watch.poll()
        rank = pm.get_sequence_parallel_rank()
        flag_peers, my_flags = pm.get_flags(dev)
        # the Q block is published in a peer-mapped buffer and every rank pulls all W of them
        e = pm.next_epoch(pm.SLOT_FWD_Q)
        qbuf = pm.get_peer_buffer("p2p_q", 2 * n_o * es, dev)
        q_off = (e & 1) * n_o * es
        _carve(qbuf.local, q_off, (B, Hq, Sq, D), dt).copy_(qc)
        ops.p2p_signal(flag_peers, pm.SLOT_FWD_Q, e)
        q_all = _carve(get_slabs("g_q", W * n_o * es, dev, 1)[0], 0, (W, B, Hq, Sq, D), dt)
        ops.p2p_gather(qbuf.peers, q_off, n_o * es, q_all, my_flags, pm.SLOT_FWD_Q, e)
        part = ops.fwd_partials(q_all, kc, vc, sm_scale, kvl)
        # the W partial (O, lse) blocks stay here; each owner merges its block straight out of the peers' memory
        e = pm.next_epoch(pm.SLOT_FWD_PARTS)
        blk = W * (n_o + n_l) * 4
        pbuf = pm.get_peer_buffer("p2p_parts", 2 * blk, dev)
        p_off = (e & 1) * blk
        o_parts = _carve(pbuf.local, p_off, (W, B, Hq, Sq, D), torch.float32)
        l_parts = _carve(pbuf.local, p_off + W * n_o * 4, (W * B * Hq, Sq), torch.float32)
        ops.fwd_combine(part, None, None, o_parts, l_parts, False)
        ops.p2p_signal(flag_peers, pm.SLOT_FWD_PARTS, e)
        ops.p2p_fwd_merge(pbuf.peers, p_off + rank * n_o * 4, p_off + W * n_o * 4 + rank * n_l * 4, o, L, my_flags,
                          pm.SLOT_FWD_PARTS, e)
        pm.status_watch.post()
        return q, k, v, o, L
    if sched == "gather":
        q_all = _carve(get_slabs("g_q", W * n_o * es, dev, 1)[0], 0, (W, B, Hq, Sq, D), dt)
        wait_async_handles(all_gather_blocks([qc], [q_all], comm_mode))
        part = ops.fwd_partials(q_all, kc, vc, sm_scale, kvl)
        sbuf = get_slabs("g_acc_send", W * (n_o + n_l) * 4, dev, 1)[0]
        rbuf = get_slabs("g_acc_recv", W * (n_o + n_l) * 4, dev, 1)[0]
        o_parts = _carve(sbuf, 0, (W, B, Hq, Sq, D), torch.float32)
        l_parts = _carve(sbuf, W * n_o * 4, (W, B * Hq, Sq), torch.float32)
        o_recv = _carve(rbuf, 0, (W, B, Hq, Sq, D), torch.float32)
        l_recv = _carve(rbuf, W * n_o * 4, (W, B * Hq, Sq), torch.float32)
        ops.fwd_combine(part, None, None, o_parts, l_parts.view(W * B * Hq, Sq), False)
        wait_async_handles(all_to_all_blocks([(o_parts, o_recv), (l_parts, l_recv)], comm_mode))
        ops.fwd_merge_parts(o_recv, l_recv, dt, o_out=o, lse_out=L)
        _status_post(q)
        return q, k, v, o, L

    acc_bytes = n_o * 4 + n_l * 4
    q_bufs, send_bufs, recv_bufs = maybe_get_set_global_memory_buffer(qc, acc_bytes)

    def acc_views(buf, final):
        odt = dt if final else torch.float32
        o_v = _carve(buf, 0, (B, Hq, Sq, D), odt)
        l_v = _carve(buf, n_o * (es if final else 4), (B * Hq, Sq), torch.float32)
        return o_v, l_v

    q_cur = qc
    args_cur = [a.contiguous() for a in remote_bias_args] if bias_func is not None else []
    args_bufs = [[torch.empty_like(a) for a in args_cur] for _ in range(2)]
    q_reqs, acc_reqs = [], []
    for t in range(W):
        last = t == W - 1
        wait_async_handles(q_reqs)          # the block this step works on has arrived
        q_reqs = []
        if not last:
            q_next = _carve(q_bufs[t % 2], 0, (B, Hq, Sq, D), dt)
            args_next = args_bufs[t % 2]
            q_reqs = send_recv_fwd_q(q_cur, q_next, args_cur, args_next, comm_mode)
            if no_overlap:
                wait_async_handles(q_reqs)
                q_reqs = []
        bias = _build_bias(bias_func, local_bias_args, args_cur, q_cur, kc)
        part = ops.fwd_partials(q_cur, kc, vc, sm_scale, kvl, bias=bias)
        wait_async_handles(acc_reqs)        # travelling accumulator of this block (and last step's send)
        o_in = l_in = None
        if t > 0:
            o_in, l_in = acc_views(recv_bufs[(t - 1) % 2], False)
        o_out, l_out = acc_views(send_bufs[t % 2], last)
        ops.fwd_combine(part, o_in, l_in, o_out, l_out, last)
        if last:
            # the finished block goes home; this rank's own finished block arrives from rank-1
            acc_reqs = _exchange_final(o_out, l_out, o, L, comm_mode)
        else:
            sv = send_bufs[t % 2][:acc_bytes]
            rv = recv_bufs[t % 2][:acc_bytes]
            acc_reqs = send_recv_fwd_Lo(sv, rv, comm_mode)
        if no_overlap:
            wait_async_handles(acc_reqs)
            acc_reqs = []
        if not last:
            q_cur, args_cur = q_next, args_next
    wait_async_handles(acc_reqs)
    _status_post(q)
    return q, k, v, o, L


def _end_of_backward_status(pm):
    """Peer-memory schedules: a flag wait that ran out leaves the outputs unwritten. The status word is copied to
    the host after the last kernel and read at the start of the next call (no host synchronisation); with
    LVX_STATUS_CHECK=sync it is read here, at the price of one synchronisation per backward."""
    pm.status_watch.post()
    if os.environ.get("LVX_STATUS_CHECK", "") == "sync":
        pm.status_watch.check()


def _exchange_final(o_send, l_send, o_recv, l_recv, comm_mode):
    return _exchange([o_send, l_send], [o_recv, l_recv], comm_mode)


def _attn_backward(do, q, k, v, o, L, causal, sm_scale, comm_mode, backward_engine, bias_func=None,
                   local_bias_args=[], remote_bias_args=[], no_overlap=False, kv_valid_len=None, schedule=None):
    """Returns (dq, dk, dv): dq like q, dk/dv like k/v (summed over the query heads of each KV group)
    (reference :437-545). `backward_engine` is accepted and ignored, as in the reference."""
    _check_common(q, k, v, causal, bias_func, local_bias_args, remote_bias_args)
    _status_poll(q)
    W = get_sequence_parallel_size()
    B, Hq, Sq, D = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    dev, dt = q.device, q.dtype
    es = q.element_size()
    qc, kc, vc, oc, doc = (x.contiguous() for x in (q, k, v, o, do))
    if L.dtype != torch.float32 or L.numel() != B * Hq * Sq:
        raise ValueError("L must be the fp32 [B*Hq, Sq] log-sum-exp returned by _attn_forward")
    Lc = L.contiguous().view(B * Hq, Sq)
    kvl = _local_valid(kv_valid_len, Skv, dev)

    n_q, n_r, n_kv = B * Hq * Sq * D, B * Hq * Sq, B * Hkv * Skv * D
    delta = ops.bwd_prep(oc, doc)                       # once, at home; travels instead of O
    dq = torch.empty(B, Hq, Sq, D, dtype=dt, device=dev)

    sched = ("ring" if bias_func is not None else _schedule(schedule, q)) if W > 1 else "gather"
    if W == 1 or comm_mode == "nocomm":
        dq_acc = _carve(get_slabs("bwd_dq_delta", n_q * 4, dev, 1)[0], 0, (B, Hq, Sq, D), torch.float32)
        dk = torch.empty(B, Hkv, Skv, D, dtype=dt, device=dev)
        dv = torch.empty(B, Hkv, Skv, D, dtype=dt, device=dev)
        bias = _build_bias(bias_func, local_bias_args, remote_bias_args, qc, kc)
        for t in range(W):
            dq_acc.zero_()
            ops.bwd_block(qc, doc, Lc, delta, kc, vc, sm_scale, dq_acc, dk, dv, "final", kvl, bias=bias)
        ops.add_cast(dq_acc, None, dt, out=dq)
        _status_post(q)
        return dq, dk, dv
    if sched in ("p2p", "p2p_pull") and (n_r * 4) % 16:
        if (schedule or os.environ.get("LVX_SCHEDULE", _DEFAULT_SCHEDULE)) != "auto":
            raise ValueError("the p2p schedules need B*Hq*Sq to be a multiple of 4")
        sched = "gather"          # picked by "auto": the exchange kernels copy 16 bytes at a time
    if sched == "p2p":
        from . import peer_memory as pm
        pm.status_watch.poll()
        rank = pm.get_sequence_parallel_rank()
        flag_peers, my_flags = pm.get_flags(dev)
        main, side = torch.cuda.current_stream(dev), pm.side_stream(dev)
        e = pm.next_epoch(pm.SLOT_BWD_IN)
        blk = W * (2 * n_q * es + 2 * n_r * 4)
        ibuf = pm.get_peer_buffer("p2p_bwd_all", 2 * blk, dev)
        base = (e & 1) * blk
        offs = (base, base + W * n_q * es, base + 2 * W * n_q * es, base + 2 * W * n_q * es + W * n_r * 4)
        q_all = _carve(ibuf.local, offs[0], (W, B, Hq, Sq, D), dt)
        do_all = _carve(ibuf.local, offs[1], (W, B, Hq, Sq, D), dt)
        l_all = _carve(ibuf.local, offs[2], (W * B * Hq, Sq), torch.float32)
        d_all = _carve(ibuf.local, offs[3], (W * B * Hq, Sq), torch.float32)
        # own block with local copies; the peers' slots from the side stream while the kernel already works
        q_all[rank].copy_(qc)
        do_all[rank].copy_(doc)
        l_all.view(W, B * Hq, Sq)[rank].copy_(Lc)
        d_all.view(W, B * Hq, Sq)[rank].copy_(delta)
        ready = torch.cuda.Event()
        ready.record(main)
        with torch.cuda.stream(side):
            side.wait_event(ready)
            ops.p2p_push(ibuf.peers, flag_peers, [(qc, False, offs[0], n_q * es), (doc, False, offs[1], n_q * es),
                                                  (Lc, False, offs[2], n_r * 4), (delta, False, offs[3], n_r * 4)],
                         pm.SLOT_BWD_IN, e, skip_self=True, dma=_PUSH_DMA)
            pushed = torch.cuda.Event()
            pushed.record(side)
        dq_parts = _carve(get_slabs("g_dq_send", W * n_q * 4, dev, 1)[0], 0, (W, B, Hq, Sq, D), torch.float32)
        dq_parts.zero_()                        # overlaps the stores on the side stream
        dk = torch.empty(B, Hkv, Skv, D, dtype=dt, device=dev)
        dv = torch.empty(B, Hkv, Skv, D, dtype=dt, device=dev)
        if not _PUSH_DMA:
            main.wait_event(pushed)             # see _attn_forward
        wait = (my_flags, pm.SLOT_BWD_IN, e, rank) if dt != torch.float32 else None
        if wait is None:
            ops.p2p_wait(my_flags, W, pm.SLOT_BWD_IN, e)
        ops.bwd_block(q_all, do_all, l_all, d_all, kc, vc, sm_scale, dq_parts, dk, dv, "final", kvl, block_wait=wait)
        e = pm.next_epoch(pm.SLOT_BWD_DQ)
        dbuf = pm.get_peer_buffer("p2p_dq_recv", 2 * W * n_q * 4, dev)
        d_off = (e & 1) * W * n_q * 4
        ops.p2p_push(dbuf.peers, flag_peers, [(dq_parts, True, d_off, n_q * 4)], pm.SLOT_BWD_DQ, e)
        ops.p2p_wait(my_flags, W, pm.SLOT_BWD_DQ, e)
        ops.sum_cast(_carve(dbuf.local, d_off, (W, B, Hq, Sq, D), torch.float32), dt, out=dq)
        main.wait_event(pushed)
        _end_of_backward_status(pm)
        return dq, dk, dv
    elif sched == "p2p_pull":
        from . import peer_memory as pm
        pm.status_watch.poll()
        rank = pm.get_sequence_parallel_rank()
        flag_peers, my_flags = pm.get_flags(dev)
        e = pm.next_epoch(pm.SLOT_BWD_IN)
        blk = 2 * n_q * es + 2 * n_r * 4
        ibuf = pm.get_peer_buffer("p2p_bwd_in", 2 * blk, dev)
        base = (e & 1) * blk
        offs = (base, base + n_q * es, base + 2 * n_q * es, base + 2 * n_q * es + n_r * 4)
        _carve(ibuf.local, offs[0], (B, Hq, Sq, D), dt).copy_(qc)
        _carve(ibuf.local, offs[1], (B, Hq, Sq, D), dt).copy_(doc)
        _carve(ibuf.local, offs[2], (B * Hq, Sq), torch.float32).copy_(Lc)
        _carve(ibuf.local, offs[3], (B * Hq, Sq), torch.float32).copy_(delta)
        ops.p2p_signal(flag_peers, pm.SLOT_BWD_IN, e)
        gbuf = get_slabs("g_bwd_in", W * blk, dev, 1)[0]
        q_all = _carve(gbuf, 0, (W, B, Hq, Sq, D), dt)
        do_all = _carve(gbuf, W * n_q * es, (W, B, Hq, Sq, D), dt)
        l_all = _carve(gbuf, 2 * W * n_q * es, (W * B * Hq, Sq), torch.float32)
        d_all = _carve(gbuf, 2 * W * n_q * es + W * n_r * 4, (W * B * Hq, Sq), torch.float32)
        for dst, off, nb in ((q_all, offs[0], n_q * es), (do_all, offs[1], n_q * es), (l_all, offs[2], n_r * 4),
                             (d_all, offs[3], n_r * 4)):
            ops.p2p_gather(ibuf.peers, off, nb, dst, my_flags, pm.SLOT_BWD_IN, e)
        e = pm.next_epoch(pm.SLOT_BWD_DQ)
        dbuf = pm.get_peer_buffer("p2p_dq", 2 * W * n_q * 4, dev)
        d_off = (e & 1) * W * n_q * 4
        dq_parts = _carve(dbuf.local, d_off, (W, B, Hq, Sq, D), torch.float32)
        dq_parts.zero_()
        dk = torch.empty(B, Hkv, Skv, D, dtype=dt, device=dev)
        dv = torch.empty(B, Hkv, Skv, D, dtype=dt, device=dev)
        ops.bwd_block(q_all, do_all, l_all, d_all, kc, vc, sm_scale, dq_parts, dk, dv, "final", kvl)
        ops.p2p_signal(flag_peers, pm.SLOT_BWD_DQ, e)
        ops.p2p_sum_cast(dbuf.peers, d_off + rank * n_q * 4, dq, my_flags, pm.SLOT_BWD_DQ, e)   # each owner sums its block
        _end_of_backward_status(pm)
        return dq, dk, dv
    elif sched == "gather":
        gbuf = get_slabs("g_bwd_in", W * (2 * n_q * es + 2 * n_r * 4), dev, 1)[0]
        q_all = _carve(gbuf, 0, (W, B, Hq, Sq, D), dt)
        do_all = _carve(gbuf, W * n_q * es, (W, B, Hq, Sq, D), dt)
        l_all = _carve(gbuf, 2 * W * n_q * es, (W, B * Hq, Sq), torch.float32)
        d_all = _carve(gbuf, 2 * W * n_q * es + W * n_r * 4, (W, B * Hq, Sq), torch.float32)
        wait_async_handles(all_gather_blocks([qc, doc, Lc, delta], [q_all, do_all, l_all, d_all], comm_mode))
        dq_parts = _carve(get_slabs("g_dq_send", W * n_q * 4, dev, 1)[0], 0, (W, B, Hq, Sq, D), torch.float32)
        dq_recv = _carve(get_slabs("g_dq_recv", W * n_q * 4, dev, 1)[0], 0, (W, B, Hq, Sq, D), torch.float32)
        dq_parts.zero_()
        dk = torch.empty(B, Hkv, Skv, D, dtype=dt, device=dev)
        dv = torch.empty(B, Hkv, Skv, D, dtype=dt, device=dev)
        ops.bwd_block(q_all, do_all, l_all.view(W * B * Hq, Sq), d_all.view(W * B * Hq, Sq), kc, vc, sm_scale,
                      dq_parts, dk, dv, "final", kvl)       # one pass: dK/dV leave the kernel in their final dtype
        wait_async_handles(all_to_all_blocks([(dq_parts, dq_recv)], comm_mode))
        ops.sum_cast(dq_recv, dt, out=dq)
        _status_post(q)
        return dq, dk, dv
    else:
        slab_bytes = 2 * n_q * es + 2 * n_r * 4
        in_bufs, send_bufs, recv_bufs = maybe_get_set_global_memory_buffer_bwd(slab_bytes, n_q * 4, dev)
        # fp32 dK/dV accumulate across the W steps (only this schedule revisits the shard)
        acc = get_slabs("bwd_dkdv", 2 * n_kv * 4, dev, 1)[0]
        dk_acc = _carve(acc, 0, (B, Hkv, Skv, D), torch.float32)
        dv_acc = _carve(acc, n_kv * 4, (B, Hkv, Skv, D), torch.float32)
        dq_delta = _carve(get_slabs("bwd_dq_delta", n_q * 4, dev, 1)[0], 0, (B, Hq, Sq, D), torch.float32)

        def slab_views(buf):
            return (_carve(buf, 0, (B, Hq, Sq, D), dt), _carve(buf, n_q * es, (B, Hq, Sq, D), dt),
                    _carve(buf, 2 * n_q * es, (B * Hq, Sq), torch.float32),
                    _carve(buf, 2 * n_q * es + n_r * 4, (B * Hq, Sq), torch.float32))

        # home slab: [Q | dO | lse | delta]
        cur = in_bufs[2]
        cq, cdo, cl, cd = slab_views(cur)
        cq.copy_(qc)
        cdo.copy_(doc)
        cl.copy_(Lc)
        cd.copy_(delta)
        comp_reqs, dq_reqs = [], []
        args_cur = [a.contiguous() for a in remote_bias_args] if bias_func is not None else []
        args_bufs = [[torch.empty_like(a) for a in args_cur] for _ in range(2)]
        for t in range(W):
            last = t == W - 1
            wait_async_handles(comp_reqs)
            comp_reqs = []
            cq, cdo, cl, cd = slab_views(cur)
            if not last:
                nxt = in_bufs[t % 2]
                args_next = args_bufs[t % 2]
                comp_reqs = send_recv_bwd_comp_reqs(cur[:slab_bytes], nxt[:slab_bytes], args_cur, args_next, comm_mode)
                if no_overlap:
                    wait_async_handles(comp_reqs)
                    comp_reqs = []
            # step 0 accumulates straight into the buffer that is sent on; later steps into a scratch
            # delta that is added to the accumulator received from rank-1
            send_v = _carve(send_bufs[t % 2], 0, (B, Hq, Sq, D), torch.float32)
            target = send_v if t == 0 else dq_delta
            target.zero_()
            bias = _build_bias(bias_func, local_bias_args, args_cur, cq, kc)
            ops.bwd_block(cq, cdo, cl, cd, kc, vc, sm_scale, target, dk_acc, dv_acc, t > 0, kvl, bias=bias)
            wait_async_handles(dq_reqs)
            if t > 0:
                recv_v = _carve(recv_bufs[(t - 1) % 2], 0, (B, Hq, Sq, D), torch.float32)
                if last:
                    fin = _carve(send_bufs[t % 2], 0, (B, Hq, Sq, D), dt)
                    ops.add_cast(recv_v, dq_delta, dt, out=fin)
                else:
                    ops.add_cast(recv_v, dq_delta, torch.float32, out=send_v)
            if last:
                fin = _carve(send_bufs[t % 2], 0, (B, Hq, Sq, D), dt)
                dq_reqs = send_recv_bwd_rescale_reqs(fin, dq, comm_mode)
            else:
                dq_reqs = send_recv_bwd_rescale_reqs(send_bufs[t % 2][:n_q * 4], recv_bufs[t % 2][:n_q * 4],
                                                     comm_mode)
            if no_overlap:
                wait_async_handles(dq_reqs)
                dq_reqs = []
            if not last:
                cur, args_cur = nxt, args_next
        wait_async_handles(dq_reqs)

    dk = ops.add_cast(dk_acc, None, dt)
    dv = ops.add_cast(dv_acc, None, dt)
    _status_post(q)
    return dq, dk, dv


# --------------------------------------------------------------------------------------------------
# autograd wrappers
# --------------------------------------------------------------------------------------------------
class LVXAttnFunc(torch.autograd.Function):
    """attention(q, k, v, causal, sm_scale, bias_func=None, local_bias_args=[], remote_bias_args=[]) -> o.
    Saves q, k, v, o, L for backward; same call shape as the class built in reference test.py:38-77."""

    @staticmethod
    def forward(ctx, q, k, v, causal, sm_scale, bias_func=None, local_bias_args=[], remote_bias_args=[],
                kv_valid_len=None):
        q, k, v, o, L = _attn_forward(q, k, v, causal, sm_scale, None, bias_func=bias_func,
                                      local_bias_args=local_bias_args, remote_bias_args=remote_bias_args,
                                      kv_valid_len=kv_valid_len)
        ctx.save_for_backward(q, k, v, o, L)
        ctx.sm_scale = sm_scale
        ctx.causal = causal
        ctx.kv_valid_len = kv_valid_len
        ctx.bias = (bias_func, local_bias_args, remote_bias_args)      # as the reference keeps them, test.py:52-54
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, L = ctx.saved_tensors
        bias_func, local_bias_args, remote_bias_args = ctx.bias
        dq, dk, dv = _attn_backward(do, q, k, v, o, L, ctx.causal, ctx.sm_scale, None, "flash", bias_func=bias_func,
                                    local_bias_args=local_bias_args, remote_bias_args=remote_bias_args,
                                    kv_valid_len=ctx.kv_valid_len)
        return dq, dk, dv, None, None, None, None, None, None


def _make_recompute_class(name, fwd, bwd, doc):
    """The recompute-QKV wrapper over a given pair of step-loop functions (LV-XAttn or the ring baseline)."""

    class _Recompute(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x, run_function, is_causal, states_getter, kv_valid_len, *params):
            with torch.no_grad():
                q, k, v = run_function(x, states_getter())
            sm_scale = q.shape[-1] ** -0.5
            _, _, _, o, L = fwd()(q, k, v, is_causal, sm_scale, None, kv_valid_len=kv_valid_len)
            ctx.save_for_backward(x, o, L, *params)
            ctx.run_function = run_function
            ctx.states_getter = states_getter
            ctx.is_causal = is_causal
            ctx.sm_scale = sm_scale
            ctx.kv_valid_len = kv_valid_len
            del q, k, v
            return o

        @staticmethod
        def backward(ctx, do):
            x, o, L, *params = ctx.saved_tensors
            with torch.enable_grad():
                x_ = x.detach().requires_grad_(x.requires_grad)
                q, k, v = ctx.run_function(x_, ctx.states_getter())
            dq, dk, dv = bwd()(do, q.detach(), k.detach(), v.detach(), o, L, ctx.is_causal, ctx.sm_scale, None, "flash",
                               kv_valid_len=ctx.kv_valid_len)
            inputs = [t for t in ([x_] + list(params)) if t.requires_grad]
            grads = torch.autograd.grad((q, k, v), inputs, (dq, dk, dv), allow_unused=True) if inputs else ()
            it = iter(grads)
            gx = next(it) if x_.requires_grad else None
            gparams = [next(it) if p.requires_grad else None for p in params]
            return (gx, None, None, None, None, *gparams)

    _Recompute.__name__ = _Recompute.__qualname__ = name
    _Recompute.__doc__ = doc
    return _Recompute


LVXAttnRecomputeFunc = _make_recompute_class(
    "LVXAttnRecomputeFunc", lambda: _attn_forward, lambda: _attn_backward,
    """attention(x, run_function, is_causal, states_getter, kv_valid_len, *params) -> o, where
    run_function(x, states) -> (q, k, v) is the projection of the layer and `states` are the visual features held in a
    module global (see hf_patch.set_global_cross_attention_states). Only (x, o, L) are saved: K/V are recomputed in
    backward, which keeps the per-layer activation memory independent of the visual sequence length
    (reference test_llama3.py:180-245). Unlike the reference (:243 returns None for every input), backward
    re-runs the projection under autograd and propagates dq, dk, dv into x and into `params` (the tensors
    run_function closes over, passed so that autograd sees them).""")


def _ring():
    from . import ring
    return ring


RingAttnRecomputeFunc = _make_recompute_class(
    "RingAttnRecomputeFunc", lambda: _ring()._attn_forward, lambda: _ring()._attn_backward,
    """The same recompute-QKV wrapper over the ring (K/V-rotating) baseline, lv_xattn_b200.ring
    (reference test_llama3.py:180-245 with attention_mode="ring").""")


def create_attention_class(attention_mode="lv_xattn"):
    """Same factory as reference test.py:38: returns the autograd class for `attention_mode`
    ("lv_xattn", or "ring" for the K/V-rotating baseline on the same kernels)."""
    if attention_mode == "lv_xattn":
        return LVXAttnFunc
    if attention_mode in ("ring", "ring_self"):
        return _ring().RingAttnFunc
    raise NotImplementedError(f"attention_mode {attention_mode!r}: expected 'lv_xattn' or 'ring'")


attention = LVXAttnFunc.apply

__all__ = ["_attn_forward", "_attn_backward", "LVXAttnFunc", "LVXAttnRecomputeFunc", "RingAttnRecomputeFunc",
           "create_attention_class",
           "attention", "reset_global_memory_buffer"]
