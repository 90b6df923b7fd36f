"""Forward + backward of the cross-attention layer when the tensors live in (pinned) host memory.

Long visual K/V can be too large, or too short-lived, to keep on the device between layers; then the cost of
a layer is dominated by the host link, not by the kernels. `HostStreamedAttention.step` hides most of the
kernel time behind the copies by cutting the K/V shard into chunks along the key axis:

  forward   chunk c is copied host->device on a copy stream while chunk c-1 runs through the forward block;
            chunk results are merged with the same (O, lse) merge the sequence-parallel schedules use
  backward  the K/V-stationary backward block runs chunk by chunk (dQ accumulates across chunks in fp32) and
            each chunk's dK/dV goes device->host while the next chunk computes

Single-GPU (W = 1) only; with a sequence-parallel group every rank's shard is already 1/W of the keys and the
plain entry points are used after one copy. Nothing here replaces a reference function: the reference keeps
everything on the device (test.py:103-107).
"""
from __future__ import annotations

import torch

from . import ops
from .async_communication import get_sequence_parallel_size
from .attn import _attn_backward, _attn_forward


class HostStreamedAttention:
    def __init__(self, device=None, chunks: int = 4):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.chunks = max(1, int(chunks))
        self.copy_in = torch.cuda.Stream(self.device)
        self.copy_out = torch.cuda.Stream(self.device)
        self._bufs = {}

    def _buf(self, name, shape, dtype):
        t = self._bufs.get(name)
        if t is None or t.shape != torch.Size(shape) or t.dtype != dtype:
            t = torch.empty(shape, dtype=dtype, device=self.device)
            self._bufs[name] = t
        return t

    def step(self, q, k, v, do, sm_scale, out_o, out_dq, out_dk, out_dv, kv_valid_len=None):
        """q, do: pinned host [B,Hq,Sq,D]; k, v: pinned host [B,Hkv,Skv,D]; outputs are pinned host tensors of
        the matching shapes. Returns when every output has landed in host memory."""
        for t in (q, k, v, do, out_o, out_dq, out_dk, out_dv):
            if t.is_cuda or not t.is_pinned():
                raise ValueError("HostStreamedAttention takes pinned host tensors")
        dev, dt = self.device, q.dtype
        B, Hq, Sq, D = q.shape
        Hkv, Skv = k.shape[1], k.shape[2]
        main = torch.cuda.current_stream(dev)
        if get_sequence_parallel_size() > 1:
            return self._step_plain(q, k, v, do, sm_scale, out_o, out_dq, out_dk, out_dv, kv_valid_len)

        # chunk boundaries on 128-row tiles
        tiles = (Skv + 127) // 128
        per = (tiles + self.chunks - 1) // self.chunks * 128
        bounds = [(c0, min(Skv, c0 + per)) for c0 in range(0, Skv, per)]
        valid = None if kv_valid_len is None else [int(x) for x in kv_valid_len]

        qd, dod = self._buf("q", q.shape, dt), self._buf("do", do.shape, dt)
        start = torch.cuda.Event()
        start.record(main)
        self.copy_in.wait_event(start)                 # buffers of the previous step are no longer in use
        self.copy_out.wait_event(start)
        ready = []
        kd, vd = [], []
        with torch.cuda.stream(self.copy_in):
            qd.copy_(q, non_blocking=True)
            for i, (c0, c1) in enumerate(bounds):
                kc = self._buf(f"k{i}", (B, Hkv, c1 - c0, D), dt)
                vc = self._buf(f"v{i}", (B, Hkv, c1 - c0, D), dt)
                for b in range(B):
                    for h in range(Hkv):
                        kc[b, h].copy_(k[b, h, c0:c1], non_blocking=True)
                        vc[b, h].copy_(v[b, h, c0:c1], non_blocking=True)
                if i == 0:
                    dod.copy_(do, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.copy_in)
                ready.append(ev)
                kd.append(kc)
                vd.append(vc)

        def chunk_valid(i):
            if valid is None:
                return None
            c0, c1 = bounds[i]
            return torch.tensor([min(max(n - c0, 0), c1 - c0) for n in valid], dtype=torch.int32, device=dev)

        kvl = [chunk_valid(i) for i in range(len(bounds))]

        # ---- forward: chunk by chunk, merged through the travelling accumulator ----
        acc = [(self._buf(f"acc_o{i}", (B, Hq, Sq, D), torch.float32),
                self._buf(f"acc_l{i}", (B * Hq, Sq), torch.float32)) for i in range(2)]
        o = self._buf("o", (B, Hq, Sq, D), dt)
        lse = self._buf("lse", (B * Hq, Sq), torch.float32)
        o_in = l_in = None
        for i in range(len(bounds)):
            main.wait_event(ready[i])
            part = ops.fwd_partials(qd, kd[i], vd[i], sm_scale, kvl[i])
            last = i == len(bounds) - 1
            o_out, l_out = (o, lse) if last else acc[i % 2]
            ops.fwd_combine(part, o_in, l_in, o_out, l_out, last)
            o_in, l_in = o_out, l_out
        fwd_done = torch.cuda.Event()
        fwd_done.record(main)
        with torch.cuda.stream(self.copy_out):
            self.copy_out.wait_event(fwd_done)
            out_o.copy_(o, non_blocking=True)

        # ---- backward: K/V-stationary, chunk by chunk; dK/dV leave as soon as a chunk is done ----
        delta = ops.bwd_prep(o, dod)
        dq_acc = self._buf("dq_acc", (B, Hq, Sq, D), torch.float32)
        dq_acc.zero_()
        for i, (c0, c1) in enumerate(bounds):
            dkc = self._buf(f"dk{i}", (B, Hkv, c1 - c0, D), dt)
            dvc = self._buf(f"dv{i}", (B, Hkv, c1 - c0, D), dt)
            ops.bwd_block(qd, dod, lse, delta, kd[i], vd[i], sm_scale, dq_acc, dkc, dvc, "final", kvl[i])
            ev = torch.cuda.Event()
            ev.record(main)
            with torch.cuda.stream(self.copy_out):
                self.copy_out.wait_event(ev)
                for b in range(B):
                    for h in range(Hkv):
                        out_dk[b, h, c0:c1].copy_(dkc[b, h], non_blocking=True)
                        out_dv[b, h, c0:c1].copy_(dvc[b, h], non_blocking=True)
        dq = ops.add_cast(dq_acc, None, dt, out=self._buf("dq", (B, Hq, Sq, D), dt))
        ev = torch.cuda.Event()
        ev.record(main)
        with torch.cuda.stream(self.copy_out):
            self.copy_out.wait_event(ev)
            out_dq.copy_(dq, non_blocking=True)
        done = torch.cuda.Event()
        done.record(self.copy_out)
        main.wait_event(done)
        done.synchronize()

    def _step_plain(self, q, k, v, do, sm_scale, out_o, out_dq, out_dk, out_dv, kv_valid_len):
        dev = self.device
        qd, kd, vd, dod = (t.to(dev, non_blocking=True) for t in (q, k, v, do))
        _, _, _, o, L = _attn_forward(qd, kd, vd, False, sm_scale, None, kv_valid_len=kv_valid_len)
        out_o.copy_(o, non_blocking=True)
        dq, dk, dv = _attn_backward(dod, qd, kd, vd, o, L, False, sm_scale, None, "flash", kv_valid_len=kv_valid_len)
        out_dq.copy_(dq, non_blocking=True)
        out_dk.copy_(dk, non_blocking=True)
        out_dv.copy_(dv, non_blocking=True)
        torch.cuda.current_stream(dev).synchronize()
