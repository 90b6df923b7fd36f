"""Tensor-level wrappers over the C ABI (include/lvx.h). All compute happens in liblvx.so; torch only owns
the device memory and the stream. Inputs must be CUDA tensors; anything else raises."""
from __future__ import annotations

import ctypes

import torch

from . import _lib

_workspaces: dict = {}

# Launch accounting for benchmarks: number of kernels of this library launched since the last reset, and
# (when profiling is on) CUDA event pairs around the two tensor-core kernels, recorded on the launch stream.
launch_count = 0
_profile = None   # None, or {"fwd": [(start, end), ...], "bwd": [...], "proj": [...]}


def set_profiling(on: bool) -> None:
    global _profile
    _profile = {"fwd": [], "bwd": [], "proj": []} if on else None


def take_profile():
    """Returns {"fwd": [ms, ...], "bwd": [ms, ...]} for the launches since set_profiling(True); the caller
    must have synchronised the device."""
    global _profile
    out = {k: [a.elapsed_time(b) for a, b in v] for k, v in (_profile or {}).items()}
    if _profile is not None:
        _profile = {"fwd": [], "bwd": [], "proj": []}
    return out


class _Timed:
    def __init__(self, kind):
        self.kind = kind

    def __enter__(self):
        if _profile is not None:
            self.a = torch.cuda.Event(enable_timing=True)
            self.b = torch.cuda.Event(enable_timing=True)
            self.a.record()

    def __exit__(self, *exc):
        if _profile is not None:
            self.b.record()
            _profile[self.kind].append((self.a, self.b))
        return False


def _count(n=1):
    global launch_count
    launch_count += n


def _require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise _lib.LvxError("lv_xattn_b200 runs on CUDA tensors only; there is no CPU path")


def _contig(t):
    return t if t.is_contiguous() else t.contiguous()


def _workspace(device, nbytes: int) -> torch.Tensor:
    """One cached scratch buffer per device, grown on demand (module-owned; see release_workspaces)."""
    key = (device.type, device.index)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def release_workspaces() -> None:
    _workspaces.clear()


def shape_of(q, k) -> _lib.LvxShape:
    """q is [B, Hq, Sq, D], or [n, B, Hq, Sq, D] for n query blocks that all attend the same K/V batch."""
    nblk = 1
    if q.dim() == 5:
        nblk = q.shape[0]
    B, Hq, Sq, D = q.shape[-4:]
    Bk, Hkv, Skv, Dk = k.shape
    if Bk != B or Dk != D:
        raise ValueError(f"q {tuple(q.shape)} and k {tuple(k.shape)} disagree on batch or head dimension")
    if Hq % Hkv:
        raise ValueError(f"{Hq} query heads are not a multiple of {Hkv} KV heads")
    return _lib.make_shape(B, Hq, Hkv, Sq, Skv, D, q.dtype, nblk)


class FwdPartials:
    """Handle on the split-KV partials of one forward block (they live in the module's workspace until
    the next forward block on the same device overwrites them)."""
    __slots__ = ("shape", "ws", "dims", "dtype", "device")

    def __init__(self, shape, ws, dims, dtype, device):
        self.shape, self.ws, self.dims, self.dtype, self.device = shape, ws, dims, dtype, device


def _bias_view(bias, q, k):
    """lvx_bias for an fp32 tensor broadcastable to [B, Hq, Sq, Skv] (size-1 dims broadcast, as after the
    reference's `.expand(B, H, Lq, Lk)`, lv_xattn/attn.py:389). Returns (struct, tensor kept alive)."""
    _require_cuda(bias)
    if bias.dtype != torch.float32:
        bias = bias.float()
    if q.dim() != 4:
        raise ValueError("a dense bias is supported for a single query block only")
    B, Hq, Sq, _ = q.shape
    Skv = k.shape[2]
    if bias.dim() != 4:
        raise ValueError(f"bias must be 4-D, broadcastable to {(B, Hq, Sq, Skv)}; got {tuple(bias.shape)}")
    try:
        e = bias.expand(B, Hq, Sq, Skv)
    except RuntimeError as err:
        raise ValueError(f"bias {tuple(bias.shape)} does not broadcast to {(B, Hq, Sq, Skv)}") from err
    sb, sh, sq_, skv_ = e.stride()
    return _lib.LvxBias(e.data_ptr(), 0, sb, sh, sq_, skv_), e


def _block_wait(block_wait):
    """(my_flags tensor or None, slot, epoch, first_block) -> LvxBlockWait (see lvx_fwd_block_gathered)."""
    flags, slot, epoch, first = block_wait
    return _lib.LvxBlockWait(None if flags is None else flags.data_ptr(), slot, epoch & 0xFFFFFFFF, first)


def fwd_partials(q, k, v, sm_scale, kv_valid_len=None, bias=None, block_wait=None) -> FwdPartials:
    """Launches the forward block: Q block x local K/V shard -> split-KV partials in the workspace.
    bias: optional dense additive fp32 bias on the scores (S = sm_scale*q.k + bias); runs the general kernels."""
    _require_cuda(q, k, v, kv_valid_len)
    lib = _lib.load()
    q, k, v = _contig(q), _contig(k), _contig(v)
    if v.shape != k.shape or v.dtype != q.dtype or k.dtype != q.dtype:
        raise ValueError("k and v must have the same shape, and q/k/v the same dtype")
    shp = shape_of(q, k)
    fwd_bytes, _ = _lib.query_workspace(shp)
    ws = _workspace(q.device, fwd_bytes)
    B = k.shape[0]
    if kv_valid_len is not None:
        if kv_valid_len.dtype != torch.int32 or kv_valid_len.numel() != B:
            raise ValueError("kv_valid_len must be an int32 tensor with one entry per batch element")
        kv_valid_len = _contig(kv_valid_len)
    with _Timed("fwd"):
        if bias is not None:
            bv, keep = _bias_view(bias, q, k)
            _lib.check(lib.lvx_fwd_block_bias(ctypes.byref(shp), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v),
                                              _lib.ptr(kv_valid_len), ctypes.byref(bv), ctypes.c_float(sm_scale),
                                              _lib.ptr(ws), ws.numel(), _lib.stream_ptr()), "lvx_fwd_block_bias")
        elif block_wait is not None:
            bw = _block_wait(block_wait)
            _lib.check(lib.lvx_fwd_block_gathered(ctypes.byref(shp), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v),
                                                  _lib.ptr(kv_valid_len), ctypes.c_float(sm_scale), _lib.ptr(ws),
                                                  ws.numel(), ctypes.byref(bw), _lib.stream_ptr()),
                       "lvx_fwd_block_gathered")
        else:
            _lib.check(lib.lvx_fwd_block(ctypes.byref(shp), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v),
                                         _lib.ptr(kv_valid_len), ctypes.c_float(sm_scale), _lib.ptr(ws), ws.numel(),
                                         _lib.stream_ptr()), "lvx_fwd_block")
    _count()
    return FwdPartials(shp, ws, tuple(q.shape), q.dtype, q.device)


def fwd_combine(part: FwdPartials, o_in, lse_in, o_out, lse_out, final: bool) -> None:
    """partials (+) travelling (o_in, lse_in) -> (o_out, lse_out). o_in/lse_in None = empty accumulator.
    final=True writes O in the input dtype, otherwise fp32 (the travelling form)."""
    _require_cuda(o_in, lse_in, o_out, lse_out)
    lib = _lib.load()
    want = part.dtype if final else torch.float32
    if o_out.dtype != want or lse_out.dtype != torch.float32 or not o_out.is_contiguous() or not lse_out.is_contiguous():
        raise ValueError(f"o_out must be contiguous {want}, lse_out contiguous fp32")
    if (o_in is None) != (lse_in is None):
        raise ValueError("o_in and lse_in go together")
    if o_in is not None and (o_in.dtype != torch.float32 or lse_in.dtype != torch.float32
                             or not o_in.is_contiguous() or not lse_in.is_contiguous()):
        raise ValueError("the travelling accumulator (o_in, lse_in) must be contiguous fp32")
    _lib.check(lib.lvx_fwd_combine_merge(ctypes.byref(part.shape), _lib.ptr(part.ws), _lib.ptr(o_in),
                                         _lib.ptr(lse_in), _lib.ptr(o_out), _lib.ptr(lse_out), 1 if final else 0,
                                         _lib.stream_ptr()), "lvx_fwd_combine_merge")
    _count()


def fwd_block(q, k, v, sm_scale, kv_valid_len=None, o_in=None, lse_in=None, final=True, bias=None):
    """(O, lse) of the Q block against the local K/V shard, merged into the travelling (o_in, lse_in).

    final=True  -> O in q.dtype (the caller's result); final=False -> fp32 travelling form.
    lse is fp32 [B*Hq, Sq]."""
    part = fwd_partials(q, k, v, sm_scale, kv_valid_len, bias)
    Hq, Sq = q.shape[-3], q.shape[-2]
    o_out = torch.empty(q.shape, dtype=q.dtype if final else torch.float32, device=q.device)
    lse_out = torch.empty(q.numel() // (Hq * Sq * q.shape[-1]) * Hq, Sq, dtype=torch.float32, device=q.device)
    fwd_combine(part, o_in, lse_in, o_out, lse_out, final)
    return o_out, lse_out


def bwd_prep(o, do):
    """delta [B*Hq, Sq] fp32 = rowsum(O * dO)."""
    _require_cuda(o, do)
    lib = _lib.load()
    o, do = _contig(o), _contig(do)
    Hq, Sq, D = o.shape[-3:]
    B = o.numel() // (Hq * Sq * D)
    shp = _lib.make_shape(B, Hq, Hq, Sq, 0, D, o.dtype)
    delta = torch.empty(B * Hq, Sq, dtype=torch.float32, device=o.device)
    _lib.check(lib.lvx_bwd_prep(ctypes.byref(shp), _lib.ptr(o), _lib.ptr(do), _lib.ptr(delta), _lib.stream_ptr()),
               "lvx_bwd_prep")
    _count()
    return delta


def bwd_block(q, do, lse, delta, k, v, sm_scale, dq_acc, dk_acc, dv_acc, accumulate_dkdv, kv_valid_len=None,
              bias=None, block_wait=None):
    """dq_acc += dS K ; dk_acc, dv_acc (+)= dS^T Q, P^T dO.

    accumulate_dkdv: False -> overwrite the fp32 dk_acc/dv_acc; True -> add to them; "final" -> dk_acc/dv_acc
    are tensors of q.dtype and receive the finished gradients (single-pass use, no later accumulation)."""
    _require_cuda(q, do, lse, delta, k, v, dq_acc, dk_acc, dv_acc, kv_valid_len)
    lib = _lib.load()
    q, do, k, v = _contig(q), _contig(do), _contig(k), _contig(v)
    shp = shape_of(q, k)
    final = accumulate_dkdv == "final"
    for t, name in ((lse, "lse"), (delta, "delta"), (dq_acc, "dq_acc")):
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous fp32 tensor")
    for t, name in ((dk_acc, "dk_acc"), (dv_acc, "dv_acc")):
        if t.dtype != (q.dtype if final else torch.float32) or not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous {'in the input dtype' if final else 'fp32'}")
    if dq_acc.numel() != q.numel() or dk_acc.numel() != k.numel() or dv_acc.numel() != v.numel():
        raise ValueError("accumulator sizes do not match q / k / v")
    if kv_valid_len is not None:
        kv_valid_len = _contig(kv_valid_len)
    mode = 2 if final else (1 if accumulate_dkdv else 0)
    if bias is not None:
        bv, keep = _bias_view(bias, q, k)
        with _Timed("bwd"):
            _lib.check(lib.lvx_bwd_block_bias(ctypes.byref(shp), _lib.ptr(q), _lib.ptr(do), _lib.ptr(lse),
                                              _lib.ptr(delta), _lib.ptr(k), _lib.ptr(v), _lib.ptr(kv_valid_len),
                                              ctypes.byref(bv), ctypes.c_float(sm_scale), _lib.ptr(dq_acc),
                                              _lib.ptr(dk_acc), _lib.ptr(dv_acc), mode, _lib.stream_ptr()),
                       "lvx_bwd_block_bias")
        _count()
        return
    if block_wait is not None:
        bw = _block_wait(block_wait)
        with _Timed("bwd"):
            _lib.check(lib.lvx_bwd_block_gathered(ctypes.byref(shp), _lib.ptr(q), _lib.ptr(do), _lib.ptr(lse),
                                                  _lib.ptr(delta), _lib.ptr(k), _lib.ptr(v), _lib.ptr(kv_valid_len),
                                                  ctypes.c_float(sm_scale), _lib.ptr(dq_acc), _lib.ptr(dk_acc),
                                                  _lib.ptr(dv_acc), mode, ctypes.byref(bw), _lib.stream_ptr()),
                       "lvx_bwd_block_gathered")
        _count()
        return
    with _Timed("bwd"):
        _lib.check(lib.lvx_bwd_block(ctypes.byref(shp), _lib.ptr(q), _lib.ptr(do), _lib.ptr(lse), _lib.ptr(delta),
                                     _lib.ptr(k), _lib.ptr(v), _lib.ptr(kv_valid_len), ctypes.c_float(sm_scale),
                                     _lib.ptr(dq_acc), _lib.ptr(dk_acc), _lib.ptr(dv_acc),
                                     2 if final else (1 if accumulate_dkdv else 0), None, 0,
                                     _lib.stream_ptr()), "lvx_bwd_block")
    _count()


def kv_project_supported(states, wk, wv, n_kv_heads: int) -> bool:
    """True when lvx_kv_project can take these tensors (CUDA, bf16/fp16, head dim 128, Kd a multiple of 64, an even
    number of KV heads, plain [out, in] weights)."""
    return (states.is_cuda and states.dtype in (torch.bfloat16, torch.float16) and states.dim() == 3
            and wk.dtype == states.dtype and wv.dtype == states.dtype and wk.shape == wv.shape
            and wk.shape == (n_kv_heads * 128, states.shape[-1]) and states.shape[-1] % 64 == 0
            and n_kv_heads % 2 == 0)


def kv_project(states, wk, wv, norm_weight, eps: float, n_kv_heads: int):
    """K = rmsnorm_per_head(states @ wk^T) * norm_weight, V = states @ wv^T in one tensor-core GEMM, written as
    [B, Hkv, S, 128]; also rstd [B, Hkv, S] fp32. norm_weight None = no norm."""
    _require_cuda(states, wk, wv, norm_weight)
    lib = _lib.load()
    if not kv_project_supported(states, wk, wv, n_kv_heads):
        raise ValueError("kv_project: unsupported shapes or dtypes (see kv_project_supported)")
    states, wk, wv = _contig(states), _contig(wk), _contig(wv)
    B, S, Kd = states.shape
    if norm_weight is not None:
        if norm_weight.numel() != 128:
            raise ValueError("norm_weight must have 128 entries")
        norm_weight = _contig(norm_weight.to(states.dtype))
    k = torch.empty(B, n_kv_heads, S, 128, dtype=states.dtype, device=states.device)
    v = torch.empty_like(k)
    rstd = torch.empty(B, n_kv_heads, S, dtype=torch.float32, device=states.device)
    with _Timed("proj"):
        _lib.check(lib.lvx_kv_project(_lib.dtype_code(states.dtype), _lib.ptr(states), _lib.ptr(wk), _lib.ptr(wv),
                                      _lib.ptr(norm_weight), ctypes.c_float(eps), B, S, Kd, n_kv_heads, _lib.ptr(k),
                                      _lib.ptr(v), _lib.ptr(rstd), _lib.stream_ptr()), "lvx_kv_project")
    _count()
    return k, v, rstd


def knorm_bwd(k, dk, rstd, norm_weight):
    """Backward of the fused K norm: (dKpre like k, dw fp32 [128])."""
    _require_cuda(k, dk, rstd, norm_weight)
    lib = _lib.load()
    k, dk, rstd = _contig(k), _contig(dk), _contig(rstd)
    if dk.dtype != k.dtype or dk.shape != k.shape or rstd.dtype != torch.float32 or rstd.numel() * 128 != k.numel():
        raise ValueError("knorm_bwd: k, dk [.., 128] in one 16-bit dtype and fp32 rstd with one entry per row")
    w = _contig(norm_weight.to(k.dtype))
    dkpre = torch.empty_like(k)
    dw = torch.zeros(128, dtype=torch.float32, device=k.device)
    _lib.check(lib.lvx_knorm_bwd(_lib.dtype_code(k.dtype), _lib.ptr(k), _lib.ptr(dk), _lib.ptr(rstd), _lib.ptr(w),
                                 _lib.ptr(dkpre), _lib.ptr(dw), ctypes.c_size_t(rstd.numel()), _lib.stream_ptr()),
               "lvx_knorm_bwd")
    _count()
    return dkpre, dw


def fwd_merge_parts(o_parts, lse_parts, out_dtype, o_out=None, lse_out=None):
    """Merge of finished partials of the same query block: o_parts fp32 [n, B, Hq, Sq, D], lse_parts fp32
    [n, B*Hq, Sq] -> (o [B, Hq, Sq, D] in out_dtype, lse [B*Hq, Sq])."""
    _require_cuda(o_parts, lse_parts, o_out, lse_out)
    lib = _lib.load()
    if o_parts.dtype != torch.float32 or lse_parts.dtype != torch.float32:
        raise ValueError("partials must be fp32")
    o_parts, lse_parts = _contig(o_parts), _contig(lse_parts)
    n, B, Hq, Sq, D = o_parts.shape
    shp = _lib.make_shape(B, Hq, Hq, Sq, 0, D, out_dtype)
    if o_out is None:
        o_out = torch.empty(B, Hq, Sq, D, dtype=out_dtype, device=o_parts.device)
    if lse_out is None:
        lse_out = torch.empty(B * Hq, Sq, dtype=torch.float32, device=o_parts.device)
    _lib.check(lib.lvx_fwd_merge_parts(ctypes.byref(shp), _lib.ptr(o_parts), _lib.ptr(lse_parts), n, B * Hq * Sq * D,
                                       B * Hq * Sq, _lib.ptr(o_out), _lib.ptr(lse_out), _lib.stream_ptr()),
               "lvx_fwd_merge_parts")
    _count()
    return o_out, lse_out


def sum_cast(parts, out_dtype, out=None):
    """cast(sum over the leading axis) of an fp32 tensor [n, ...]."""
    _require_cuda(parts, out)
    lib = _lib.load()
    if parts.dtype != torch.float32:
        raise ValueError("sum_cast takes an fp32 tensor")
    parts = _contig(parts)
    n = parts.shape[0]
    inner = parts.numel() // n
    if out is None:
        out = torch.empty(parts.shape[1:], dtype=out_dtype, device=parts.device)
    _lib.check(lib.lvx_sum_cast(_lib.ptr(parts), n, inner, _lib.ptr(out), _lib.dtype_code(out_dtype), inner,
                                _lib.stream_ptr()), "lvx_sum_cast")
    _count()
    return out


# ---- exchange over peer-mapped memory (see peer_memory.py for the buffers) ---------------------------------
def p2p_signal(flags_peers, slot: int, epoch: int):
    """Publishes `epoch` for `slot` to every rank, ordered after the kernels already on the current stream."""
    lib = _lib.load()
    _lib.check(lib.lvx_p2p_signal(ctypes.byref(flags_peers), slot, ctypes.c_uint32(epoch & 0xFFFFFFFF), _lib.stream_ptr()),
               "lvx_p2p_signal")
    _count()


def p2p_gather(src_peers, src_offset: int, nbytes: int, dst, my_flags, slot: int, epoch: int):
    """dst[s] <- rank s's bytes [src_offset, src_offset + nbytes) for every rank s; dst is a contiguous
    [W, ...] tensor whose blocks are nbytes long."""
    _require_cuda(dst, my_flags)
    lib = _lib.load()
    W = src_peers.world
    if dst.numel() * dst.element_size() != W * nbytes or not dst.is_contiguous():
        raise ValueError("p2p_gather: dst must be a contiguous [W, ...] tensor of W blocks of nbytes")
    _lib.check(lib.lvx_p2p_gather(ctypes.byref(src_peers), ctypes.c_size_t(src_offset), ctypes.c_size_t(nbytes),
                                  _lib.ptr(dst), ctypes.c_size_t(nbytes), _lib.ptr(my_flags), slot,
                                  ctypes.c_uint32(epoch & 0xFFFFFFFF), _lib.stream_ptr()), "lvx_p2p_gather")
    _count()


def p2p_fwd_merge(parts_peers, o_offset: int, lse_offset: int, o_out, lse_out, my_flags, slot: int, epoch: int):
    """fwd_merge_parts with partial c read from rank c's buffer (O fp32 at byte o_offset, lse at lse_offset)."""
    _require_cuda(o_out, lse_out, my_flags)
    lib = _lib.load()
    B, Hq, Sq, D = o_out.shape
    shp = _lib.make_shape(B, Hq, Hq, Sq, 0, D, o_out.dtype)
    _lib.check(lib.lvx_p2p_fwd_merge(ctypes.byref(shp), ctypes.byref(parts_peers), ctypes.c_size_t(o_offset),
                                     ctypes.c_size_t(lse_offset), _lib.ptr(o_out), _lib.ptr(lse_out), _lib.ptr(my_flags),
                                     slot, ctypes.c_uint32(epoch & 0xFFFFFFFF), _lib.stream_ptr()), "lvx_p2p_fwd_merge")
    _count()


def p2p_sum_cast(parts_peers, offset: int, out, my_flags, slot: int, epoch: int):
    """out <- cast(sum over ranks c of the fp32 block at byte `offset` of rank c's buffer)."""
    _require_cuda(out, my_flags)
    lib = _lib.load()
    _lib.check(lib.lvx_p2p_sum_cast(ctypes.byref(parts_peers), ctypes.c_size_t(offset), _lib.ptr(out),
                                    _lib.dtype_code(out.dtype), ctypes.c_size_t(out.numel()), _lib.ptr(my_flags), slot,
                                    ctypes.c_uint32(epoch & 0xFFFFFFFF), _lib.stream_ptr()), "lvx_p2p_sum_cast")
    _count()


def p2p_push(dst_peers, flags_peers, segments, slot: int, epoch: int, skip_self: bool = False, dma: bool = False):
    """One launch: for every rank s and every segment (src tensor, all_to_all, dst_offset, dst_rank_stride),
    copies src (all_to_all False: the whole tensor to everyone; True: its block s, src being [W, ...]) into rank
    s's buffer at dst_offset + rank*dst_rank_stride, then publishes `epoch` for `slot` to every rank.
    skip_self: this rank's own buffer is not written (the caller fills it), the epoch still goes to everyone.
    dma: the copies are done by the copy engines (lvx_p2p_push_dma), which need no SM."""
    lib = _lib.load()
    W = dst_peers.world
    arr = (_lib.LvxPushSegment * len(segments))()
    keep = []
    for i, (src, a2a, dst_offset, dst_rank_stride) in enumerate(segments):
        _require_cuda(src)
        src = _contig(src)
        keep.append(src)
        total = src.numel() * src.element_size()
        nbytes = total // W if a2a else total
        arr[i].src = src.data_ptr()
        arr[i].src_stride = nbytes if a2a else 0
        arr[i].dst_offset = dst_offset
        arr[i].dst_rank_stride = dst_rank_stride
        arr[i].bytes = nbytes
        arr[i].src_bytes = total
    fn = lib.lvx_p2p_push_dma if dma else lib.lvx_p2p_push
    _lib.check(fn(ctypes.byref(dst_peers), ctypes.byref(flags_peers), arr, len(segments), slot,
                  ctypes.c_uint32(epoch & 0xFFFFFFFF), 1 if skip_self else 0, _lib.stream_ptr()),
               "lvx_p2p_push_dma" if dma else "lvx_p2p_push")
    if not dma:
        _count()


def p2p_wait(my_flags, world: int, slot: int, epoch: int):
    """Orders the current stream after every rank's push of `epoch` on `slot` (bounded wait on the device)."""
    _require_cuda(my_flags)
    lib = _lib.load()
    _lib.check(lib.lvx_p2p_wait(_lib.ptr(my_flags), world, slot, ctypes.c_uint32(epoch & 0xFFFFFFFF), _lib.stream_ptr()),
               "lvx_p2p_wait")
    _count()


def add_cast(a, b, out_dtype, out=None):
    """cast(a + b) for fp32 a (and optional fp32 b of the same shape); written into `out` when given."""
    _require_cuda(a, b)
    lib = _lib.load()
    a = _contig(a)
    if a.dtype != torch.float32 or (b is not None and (b.dtype != torch.float32 or b.shape != a.shape)):
        raise ValueError("add_cast takes fp32 tensors of equal shape")
    if b is not None:
        b = _contig(b)
    if out is None:
        out = torch.empty(a.shape, dtype=out_dtype, device=a.device)
    elif out.dtype != out_dtype or out.numel() != a.numel() or not out.is_contiguous() or not out.is_cuda:
        raise ValueError("out must be a contiguous CUDA tensor of the requested dtype and size")
    _lib.check(lib.lvx_add_cast(_lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.dtype_code(out_dtype), a.numel(),
                                _lib.stream_ptr()), "lvx_add_cast")
    _count()
    return out


def selftest_mma(mode: int, a, b, n_cols: int):
    _require_cuda(a, b)
    lib = _lib.load()
    d = torch.empty(128, n_cols, dtype=torch.float32, device=a.device)
    _lib.check(lib.lvx_selftest_mma(mode, _lib.ptr(a), _lib.ptr(b), _lib.ptr(d), _lib.stream_ptr()),
               "lvx_selftest_mma")
    return d
