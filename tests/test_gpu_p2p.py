"""The peer-memory exchange entry points (include/lvx.h, lvx_p2p_*) on ONE GPU: the "ranks" are separate buffers
of the same device, every signal is launched before the kernel that waits for it (same stream), so no kernel
ever waits for a later launch. Checks the gather, the partial-(O, lse) merge and the dQ sum against torch."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _peers(tensors, rank):
    from lv_xattn_b200 import _lib
    p = _lib.LvxPeers()
    p.world, p.rank = len(tensors), rank
    p.nbytes = min(t.numel() * t.element_size() for t in tensors)
    for i, t in enumerate(tensors):
        p.ptr[i] = t.data_ptr()
    return p


@pytest.fixture()
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda", 0)


@pytest.mark.parametrize("world", [1, 3, 8])
def test_gather_merge_sum(dev, world):
    from lv_xattn_b200 import _lib, ops
    torch.manual_seed(world)
    B, Hq, Sq, D = 1, 4, 96, 128
    n_o, n_l = B * Hq * Sq * D, B * Hq * Sq
    flags = [torch.zeros(_lib.P2P_SLOTS * _lib.MAX_PEERS, dtype=torch.int32, device=dev) for _ in range(world)]
    # ---- gather: rank s owns block s ----
    nbytes = n_o * 2
    bufs = [torch.randn(n_o, device=dev).bfloat16() for _ in range(world)]
    for epoch in (1, 2):
        for r in range(world):
            ops.p2p_signal(_peers(flags, r), 0, epoch)
        for r in range(world):
            dst = torch.zeros(world, n_o, dtype=torch.bfloat16, device=dev)
            ops.p2p_gather(_peers(bufs, r), 0, nbytes, dst, flags[r], 0, epoch)
            assert torch.equal(dst, torch.stack(bufs))
    # ---- merge: rank c holds partials for every block; block r is merged by rank r ----
    blk = world * (n_o + n_l) * 4
    parts = [torch.zeros(blk, dtype=torch.uint8, device=dev) for _ in range(world)]
    o_p = torch.randn(world, world, n_o, device=dev)                      # [holder c][block r]
    l_p = torch.randn(world, world, n_l, device=dev) * 3
    if world > 1:
        l_p[0, :, :5] = float("-inf")                                     # a holder with nothing valid for some rows
    for c in range(world):
        parts[c][: world * n_o * 4].view(torch.float32).view(world, n_o).copy_(o_p[c])
        parts[c][world * n_o * 4:].view(torch.float32).view(world, n_l).copy_(l_p[c])
    for r in range(world):
        ops.p2p_signal(_peers(flags, r), 1, 1)
    for r in range(world):
        o = torch.empty(B, Hq, Sq, D, dtype=torch.float32, device=dev)
        lse = torch.empty(B * Hq, Sq, dtype=torch.float32, device=dev)
        ops.p2p_fwd_merge(_peers(parts, r), r * n_o * 4, world * n_o * 4 + r * n_l * 4, o, lse, flags[r], 1, 1)
        lr = l_p[:, r]                                                    # [world, n_l]
        ref_l = torch.logsumexp(lr, dim=0)
        w = torch.exp(lr - ref_l).nan_to_num(0.0)
        ref_o = (o_p[:, r].view(world, n_l, D) * w[:, :, None]).sum(0)
        assert (lse.view(-1) - ref_l).abs().max().item() < 1e-5
        assert (o.view(n_l, D) - ref_o).abs().max().item() < 1e-5
    # ---- sum: dQ partials ----
    dq_parts = [torch.randn(world, n_o, device=dev) for _ in range(world)]
    for r in range(world):
        ops.p2p_signal(_peers(flags, r), 2, 1)
    for r in range(world):
        out = torch.empty(B, Hq, Sq, D, dtype=torch.bfloat16, device=dev)
        ops.p2p_sum_cast(_peers(dq_parts, r), r * n_o * 4, out, flags[r], 2, 1)
        ref = torch.stack([dq_parts[c][r] for c in range(world)]).sum(0)
        assert (out.view(-1).float() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())
    torch.cuda.synchronize()
    assert _lib.device_status() == 0


@pytest.mark.parametrize("world", [1, 3, 8])
def test_push_all_gather_and_all_to_all(dev, world):
    """lvx_p2p_push / lvx_p2p_wait with emulated ranks: an all-gather segment and an all-to-all segment in one
    launch per rank, two epochs (both halves of a double buffer)."""
    from lv_xattn_b200 import _lib, ops
    torch.manual_seed(10 + world)
    n = 4096                                      # floats per block
    flags = [torch.zeros(_lib.P2P_SLOTS * _lib.MAX_PEERS, dtype=torch.int32, device=dev) for _ in range(world)]
    recv = [torch.zeros(2, 2, world, n, device=dev) for _ in range(world)]          # [parity][segment][from][n]
    for epoch in (1, 2, 3):
        par = epoch & 1
        own = [torch.randn(n, device=dev) for _ in range(world)]                      # gathered by everyone
        parts = [torch.randn(world, n, device=dev) for _ in range(world)]             # block s goes to rank s
        for r in range(world):
            base = par * 2 * world * n * 4
            ops.p2p_push(_peers(recv, r), _peers(flags, r),
                         [(own[r], False, base, n * 4), (parts[r], True, base + world * n * 4, n * 4)], 5, epoch)
        for r in range(world):
            ops.p2p_wait(flags[r], world, 5, epoch)
        torch.cuda.synchronize()
        for r in range(world):
            assert torch.equal(recv[r][par, 0], torch.stack(own))
            assert torch.equal(recv[r][par, 1], torch.stack([parts[c][r] for c in range(world)]))
    # the same exchange by the copy engines (lvx_p2p_push_dma)
    recv3 = [torch.zeros(2, world, n, device=dev) for _ in range(world)]
    own = [torch.randn(n, device=dev) for _ in range(world)]
    parts = [torch.randn(world, n, device=dev) for _ in range(world)]
    for r in range(world):
        ops.p2p_push(_peers(recv3, r), _peers(flags, r), [(own[r], False, 0, n * 4), (parts[r], True, world * n * 4, n * 4)],
                     7, 1, dma=True)
    for r in range(world):
        ops.p2p_wait(flags[r], world, 7, 1)
    torch.cuda.synchronize()
    for r in range(world):
        assert torch.equal(recv3[r][0], torch.stack(own))
        assert torch.equal(recv3[r][1], torch.stack([parts[c][r] for c in range(world)]))
    # skip_self: the peers are written, this rank's own buffer is left to the caller, the epoch reaches everyone
    recv2 = [torch.zeros(world, n, device=dev) for _ in range(world)]
    own = [torch.randn(n, device=dev) for _ in range(world)]
    for r in range(world):
        ops.p2p_push(_peers(recv2, r), _peers(flags, r), [(own[r], False, 0, n * 4)], 6, 1, skip_self=True)
    for r in range(world):
        ops.p2p_wait(flags[r], world, 6, 1)
    torch.cuda.synchronize()
    for r in range(world):
        for c in range(world):
            assert torch.equal(recv2[r][c], own[c] if c != r else torch.zeros(n, device=dev))
    assert _lib.device_status() == 0


def test_argument_checks(dev):
    from lv_xattn_b200 import _lib, ops
    flags = torch.zeros(_lib.P2P_SLOTS * _lib.MAX_PEERS, dtype=torch.int32, device=dev)
    buf = torch.zeros(256, dtype=torch.uint8, device=dev)
    p = _peers([buf], 0)
    with pytest.raises(_lib.LvxError):
        ops.p2p_signal(p, _lib.P2P_SLOTS, 1)                 # slot out of range
    p.world = _lib.MAX_PEERS + 1
    with pytest.raises(_lib.LvxError):
        ops.p2p_signal(p, 0, 1)                              # too many peers
    p = _peers([buf], 0)
    dst = torch.zeros(1, 24, dtype=torch.uint8, device=dev)
    with pytest.raises(_lib.LvxError):
        ops.p2p_gather(p, 0, 24, dst, flags, 0, 1)           # not a multiple of 16 bytes


def test_bounds_checks_against_the_peer_buffer_size(dev):
    """Offsets and extents are checked on the host against lvx_peers.nbytes before anything is launched."""
    from lv_xattn_b200 import _lib, ops
    flags = torch.zeros(_lib.P2P_SLOTS * _lib.MAX_PEERS, dtype=torch.int32, device=dev)
    bufs = [torch.zeros(4096, dtype=torch.uint8, device=dev) for _ in range(2)]
    p = _peers(bufs, 0)
    dst = torch.zeros(2, 4096, dtype=torch.uint8, device=dev)
    with pytest.raises(_lib.LvxError, match="runs past"):
        ops.p2p_gather(p, 16, 4096, dst, flags, 0, 1)                        # source range ends 16 bytes too far
    out = torch.empty(1, 1, 8, 128, dtype=torch.float32, device=dev)
    with pytest.raises(_lib.LvxError, match="runs past"):
        ops.p2p_sum_cast(p, 2048, out, flags, 2, 1)                          # 4 KiB partial at offset 2 KiB
    src = torch.zeros(2, 4096, dtype=torch.uint8, device=dev)
    with pytest.raises(_lib.LvxError, match="runs past"):
        ops.p2p_push(p, _peers([flags, flags], 0), [(src, True, 0, 4096)], 5, 1)   # rank 1's block lands at 4096
    p.nbytes = 0
    with pytest.raises(_lib.LvxError, match="no buffer size"):
        ops.p2p_gather(p, 0, 16, torch.zeros(2, 16, dtype=torch.uint8, device=dev), flags, 0, 1)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0


def test_wait_for_a_peer_that_never_signals_gives_up_cleanly(dev):
    """A flag that nothing sets: with the limit lowered to a millisecond the wait kernel gives up, records
    0x1300 | peer in the status word and returns -- nothing faults or hangs. While the word is set the library's
    kernels return at once; reading the word clears it and the next call works again. The host-side watch turns
    the word into P2PTimeoutError."""
    import lv_xattn_b200 as lvx
    from lv_xattn_b200 import _lib, ops, peer_memory as pm
    lib = _lib.load()
    world = 4
    flags = torch.zeros(_lib.P2P_SLOTS * _lib.MAX_PEERS, dtype=torch.int32, device=dev)
    flags.view(_lib.P2P_SLOTS, _lib.MAX_PEERS)[6, :2] = 1                  # ranks 0 and 1 signalled epoch 1; 2 and 3 never do
    torch.cuda.synchronize()
    assert lib.lvx_p2p_set_timeout(ctypes.c_double(0.0)) != 0               # refused: must be positive
    try:
        _lib.check(lib.lvx_p2p_set_timeout(ctypes.c_double(1e-3)), "lvx_p2p_set_timeout")
        ops.p2p_wait(flags, world, 6, 1)
        # a kernel launched while the word is set returns without writing anything
        a = torch.ones(1024, device=dev)
        out = torch.full((1024,), 7.0, device=dev)
        ops.add_cast(a, None, torch.float32, out=out)
        torch.cuda.synchronize()
        assert torch.equal(out, torch.full((1024,), 7.0, device=dev))
        pm.status_watch.post()
        with pytest.raises(lvx.P2PTimeoutError, match="rank 2"):
            pm.status_watch.check()
        assert _lib.device_status() == 0                                    # the watch cleared the word
        ops.add_cast(a, None, torch.float32, out=out)                       # and the library works again
        torch.cuda.synchronize()
        assert torch.equal(out, a)
        # same through the raw status call
        ops.p2p_wait(flags, world, 6, 1)
        torch.cuda.synchronize()
        assert _lib.device_status() == (0x1300 | 2)
        assert _lib.device_status() == 0
    finally:
        _lib.check(lib.lvx_p2p_set_timeout(ctypes.c_double(120.0)), "lvx_p2p_set_timeout")
        _lib.device_status()
