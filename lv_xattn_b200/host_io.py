"""Forward + backward of the cross-attention layer when the tensors live in (pinned) host memory.

Long visual K/V can be too large, or too short-lived, to keep on the device between layers; then the cost of
a layer is dominated by the host link, not by the kernels. `HostStreamedAttention` hides the copies behind the
kernels in two ways.

Inside a step (one GPU), the K/V shard is cut into chunks along the key axis:

  forward   chunk c is copied host->device on a copy stream while chunk c-1 runs through the forward block;
            chunk results are merged with the same (O, lse) merge the sequence-parallel schedules use
  backward  the K/V-stationary backward block runs chunk by chunk (dQ accumulates across chunks in fp32) and
            each chunk's dK/dV goes device->host while the next chunk computes

Across steps (any number of GPUs), the device side holds two sets of input buffers: `prefetch` starts the copy of
the NEXT step's inputs while the current step computes, and `step(..., wait=False)` returns as soon as its work is
queued, so its results drain to the host while the next step runs. Every hazard between the three streams (an input
set still being read, an output buffer still draining) is ordered with events; nothing blocks the host until
`finish` (or a `step` with `wait=True`).

With a sequence-parallel group every rank's shard is already 1/W of the keys: the step is not chunked (the plain
entry points run once on the whole shard), the cross-step overlap is the same. Nothing here replaces a reference
function: the reference keeps everything on the device (test.py:103-107).
"""
from __future__ import annotations

import torch

from . import ops
from .async_communication import get_sequence_parallel_size
from .attn import _attn_backward, _attn_forward


class _InputSet:
    """One of the two device-side sets of input buffers."""
    __slots__ = ("index", "key", "filled", "free", "ready", "q", "do", "k", "v", "bounds")

    def __init__(self, index):
        self.index, self.key, self.filled = index, None, False
        self.free = None          # event: the kernels that read this set have finished
        self.ready = []           # events: chunk i has arrived
        self.q = self.do = None
        self.k, self.v, self.bounds = [], [], []


def _key(q, k, v, do):
    return tuple((t.data_ptr(), tuple(t.shape), t.dtype) for t in (q, k, v, do))


class HostStreamedAttention:
    def __init__(self, device=None, chunks: int = 4):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.chunks = max(1, int(chunks))
        self.copy_in = torch.cuda.Stream(self.device)
        self.copy_out = torch.cuda.Stream(self.device)
        self._bufs = {}
        self._sets = [_InputSet(0), _InputSet(1)]
        self._turn = 0
        self._fifo = []           # filled input sets, oldest first
        self._drained = {}        # output buffer name -> event: its device->host copy has finished
        self._last = None         # event: every copy queued so far on the output stream has finished
        self._kvl = {}            # (valid lengths, chunk bounds) -> per-chunk valid-length tensors
        self._steps = 0           # the dK/dV output buffers alternate between two sets by step parity, so that a
                                  # step's backward does not wait for the previous step's gradients to drain

    # ---- buffers and ordering -------------------------------------------------------------------------
    def _buf(self, name, shape, dtype):
        t = self._bufs.get(name)
        if t is None or t.shape != torch.Size(shape) or t.dtype != dtype:
            if t is not None:
                torch.cuda.synchronize(self.device)      # copies into the old buffer may still be in flight
            t = torch.empty(shape, dtype=dtype, device=self.device)
            self._bufs[name] = t
        return t

    def _before_write(self, name, stream):
        ev = self._drained.pop(name, None)
        if ev is not None:
            stream.wait_event(ev)

    def _drain(self, pairs, after, names):
        """Queues host_dst.copy_(dev_src) for every pair on the output stream once `after` has happened."""
        with torch.cuda.stream(self.copy_out):
            self.copy_out.wait_event(after)
            for dst, src in pairs:
                dst.copy_(src, non_blocking=True)
                src.record_stream(self.copy_out)
            ev = torch.cuda.Event()
            ev.record(self.copy_out)
        for n in names:
            self._drained[n] = ev
        self._last = ev

    def _bounds(self, Skv):
        if get_sequence_parallel_size() > 1 or self.chunks == 1:
            return [(0, Skv)]
        tiles = (Skv + 127) // 128                      # chunk boundaries on 128-row tiles
        per = (tiles + self.chunks - 1) // self.chunks * 128
        return [(c0, min(Skv, c0 + per)) for c0 in range(0, Skv, per)]

    # ---- host -> device -------------------------------------------------------------------------------
    def prefetch(self, q, k, v, do):
        """Starts the host->device copy of a coming step's inputs (pinned host tensors, shapes as in `step`) into
        the input set that is not in use. The host tensors must stay unchanged until that step has been queued.
        At most two sets can be filled at a time (the step being queued and the next)."""
        for t in (q, k, v, do):
            if t.is_cuda or not t.is_pinned():
                raise ValueError("HostStreamedAttention takes pinned host tensors")
        s = self._sets[self._turn]
        if s.filled:
            raise RuntimeError("both input sets are filled: call step() before the next prefetch()")
        self._turn ^= 1
        dt = q.dtype
        B, Hkv, Skv, D = k.shape
        s.bounds = self._bounds(Skv)
        s.q = self._buf(f"in{s.index}_q", q.shape, dt)
        s.do = self._buf(f"in{s.index}_do", do.shape, dt)
        s.k, s.v, s.ready = [], [], []
        if s.free is not None:
            self.copy_in.wait_event(s.free)
        with torch.cuda.stream(self.copy_in):
            s.q.copy_(q, non_blocking=True)
            for i, (c0, c1) in enumerate(s.bounds):
                kc = self._buf(f"in{s.index}_k{i}", (B, Hkv, c1 - c0, D), dt)
                vc = self._buf(f"in{s.index}_v{i}", (B, Hkv, c1 - c0, D), dt)
                if c0 == 0 and c1 == Skv:
                    kc.copy_(k, non_blocking=True)
                    vc.copy_(v, non_blocking=True)
                else:                                    # a strided source: one contiguous run per (batch, head)
                    for b in range(B):
                        for h in range(Hkv):
                            kc[b, h].copy_(k[b, h, c0:c1], non_blocking=True)
                            vc[b, h].copy_(v[b, h, c0:c1], non_blocking=True)
                if i == 0:
                    s.do.copy_(do, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.copy_in)
                s.ready.append(ev)
                s.k.append(kc)
                s.v.append(vc)
        s.key, s.filled = _key(q, k, v, do), True
        self._fifo.append(s)

    def _take(self, q, k, v, do):
        key = _key(q, k, v, do)
        for i, s in enumerate(self._fifo):
            if s.key == key:
                return self._fifo.pop(i)
        self.prefetch(q, k, v, do)
        return self._fifo.pop()

    # ---- one step -------------------------------------------------------------------------------------
    def step(self, q, k, v, do, sm_scale, out_o, out_dq, out_dk, out_dv, kv_valid_len=None, wait=True):
        """q, do: pinned host [B,Hq,Sq,D]; k, v: pinned host [B,Hkv,Skv,D]; outputs are pinned host tensors of
        the matching shapes. Uses the inputs a matching `prefetch` has already started, else copies them now.
        wait=True returns when every output has landed in host memory; wait=False returns once the step is queued
        (`finish` waits for everything queued)."""
        for t in (q, k, v, do, out_o, out_dq, out_dk, out_dv):
            if t.is_cuda or not t.is_pinned():
                raise ValueError("HostStreamedAttention takes pinned host tensors")
        dev = self.device
        main = torch.cuda.current_stream(dev)
        s = self._take(q, k, v, do)
        if get_sequence_parallel_size() > 1:
            self._step_group(s, main, sm_scale, out_o, out_dq, out_dk, out_dv, kv_valid_len)
        else:
            self._step_chunked(s, main, sm_scale, out_o, out_dq, out_dk, out_dv, kv_valid_len)
        s.free = torch.cuda.Event()
        s.free.record(main)
        s.filled = False
        if wait:
            self.finish()

    def finish(self):
        """Returns when every output of every queued step has landed in host memory; the compute stream is ordered
        after those copies too (so events recorded on it afterwards cover them)."""
        if self._last is not None:
            torch.cuda.current_stream(self.device).wait_event(self._last)
            self._last.synchronize()

    def _step_chunked(self, s, main, sm_scale, out_o, out_dq, out_dk, out_dv, kv_valid_len):
        dev, dt = self.device, s.q.dtype
        B, Hq, Sq, D = s.q.shape
        Hkv = s.k[0].shape[1]
        bounds = s.bounds
        valid = None if kv_valid_len is None else [int(x) for x in kv_valid_len]

        kvl = [None] * len(bounds)
        if valid is not None:
            kkey = (tuple(valid), tuple(bounds))
            if kkey not in self._kvl:                    # built once: creating them copies from pageable memory
                self._kvl[kkey] = [torch.tensor([min(max(n - c0, 0), c1 - c0) for n in valid], dtype=torch.int32,
                                                device=dev) for c0, c1 in bounds]
            kvl = self._kvl[kkey]

        # ---- forward: chunk by chunk, merged through the travelling accumulator ----
        acc = [(self._buf(f"acc_o{i}", (B, Hq, Sq, D), torch.float32),
                self._buf(f"acc_l{i}", (B * Hq, Sq), torch.float32)) for i in range(2)]
        o = self._buf("o", (B, Hq, Sq, D), dt)
        lse = self._buf("lse", (B * Hq, Sq), torch.float32)
        o_in = l_in = None
        for i in range(len(bounds)):
            main.wait_event(s.ready[i])
            part = ops.fwd_partials(s.q, s.k[i], s.v[i], sm_scale, kvl[i])
            last = i == len(bounds) - 1
            if last:
                self._before_write("o", main)
            o_out, l_out = (o, lse) if last else acc[i % 2]
            ops.fwd_combine(part, o_in, l_in, o_out, l_out, last)
            o_in, l_in = o_out, l_out
        fwd_done = torch.cuda.Event()
        fwd_done.record(main)
        self._drain([(out_o, o)], fwd_done, ["o"])

        # ---- backward: K/V-stationary, chunk by chunk; dK/dV leave as soon as a chunk is done ----
        delta = ops.bwd_prep(o, s.do)
        dq_acc = self._buf("dq_acc", (B, Hq, Sq, D), torch.float32)
        dq_acc.zero_()
        par = self._steps & 1
        self._steps += 1
        for i, (c0, c1) in enumerate(bounds):
            dkc = self._buf(f"dk{par}_{i}", (B, Hkv, c1 - c0, D), dt)
            dvc = self._buf(f"dv{par}_{i}", (B, Hkv, c1 - c0, D), dt)
            self._before_write(f"dkv{par}_{i}", main)
            ops.bwd_block(s.q, s.do, lse, delta, s.k[i], s.v[i], sm_scale, dq_acc, dkc, dvc, "final", kvl[i])
            ev = torch.cuda.Event()
            ev.record(main)
            if c0 == 0 and c1 == out_dk.shape[2]:
                pairs = [(out_dk, dkc), (out_dv, dvc)]
            else:
                pairs = [(out[b, h, c0:c1], src[b, h]) for b in range(B) for h in range(Hkv)
                         for out, src in ((out_dk, dkc), (out_dv, dvc))]
            self._drain(pairs, ev, [f"dkv{par}_{i}"])
        self._before_write("dq", main)
        dq = ops.add_cast(dq_acc, None, dt, out=self._buf("dq", (B, Hq, Sq, D), dt))
        ev = torch.cuda.Event()
        ev.record(main)
        self._drain([(out_dq, dq)], ev, ["dq"])

    def _step_group(self, s, main, sm_scale, out_o, out_dq, out_dk, out_dv, kv_valid_len):
        """Sequence-parallel group: the plain entry points on this rank's whole shard; the results are fresh
        tensors, handed to the output stream as they appear."""
        main.wait_event(s.ready[-1])
        qd, dod, kd, vd = s.q, s.do, s.k[0], s.v[0]
        _, _, _, o, L = _attn_forward(qd, kd, vd, False, sm_scale, None, kv_valid_len=kv_valid_len)
        ev = torch.cuda.Event()
        ev.record(main)
        self._drain([(out_o, o)], ev, [])
        dq, dk, dv = _attn_backward(dod, qd, kd, vd, o, L, False, sm_scale, None, "flash", kv_valid_len=kv_valid_len)
        ev = torch.cuda.Event()
        ev.record(main)
        self._drain([(out_dq, dq), (out_dk, dk), (out_dv, dv)], ev, [])
