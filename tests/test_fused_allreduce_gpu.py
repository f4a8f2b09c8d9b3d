"""The all-reduce fused into K2's epilogue (ob_chain_allreduce), on ONE GPU with the exchange done by hand: the test plays
the other rank.  It puts the peer's staged partial and its per-tile flags for the coming call into the buffers before
the launch -- nothing waits for another kernel -- and then checks that this rank's kernel (a) stored y = its own partial
+ the peer's in rank order, bitwise what the chain followed by the stand-alone all-reduce gives, (b) staged its own
partial and announced every tile in the peer's buffer, (c) advanced the call count; for the direct-store epilogue and
for the split-K one, both base formats, and twice in a row (the staged copies alternate)."""
from __future__ import annotations

import ctypes as C

import pytest
import torch

from helpers import build_fp8_op, build_nvfp4_op, device_meta, make_index
from oracle import configs
from onebase_b200 import _lib

pytestmark = pytest.mark.gpu

STATE_BYTES, TILE_FLAGS_OFF, MAX_TILES = 16384, 4096, 384      # layout of a communication buffer (ob_comm_bytes)


class HandComm:
    """Two ranks' communication buffers on one device; `comm` is rank `me`'s view."""

    def __init__(self, slot_bytes: int, me: int):
        size = C.c_size_t()
        _lib.call("ob_comm_bytes", slot_bytes, C.byref(size))
        self.bufs = [torch.zeros(size.value, dtype=torch.uint8, device="cuda") for _ in range(2)]
        self.slot_bytes, self.me = slot_bytes, me
        self.comm = _lib.ObComm()
        self.comm.world, self.comm.rank, self.comm.slot_bytes = 2, me, slot_bytes
        for r in range(2):
            self.comm.bufs[r] = self.bufs[r].data_ptr()

    def state(self, r):
        return self.bufs[r][:32].view(torch.int32)

    def tile_flags(self, r):
        return self.bufs[r][TILE_FLAGS_OFF:TILE_FLAGS_OFF + 2 * MAX_TILES * 4].view(torch.int32).view(2, MAX_TILES)

    def staged(self, r, parity, M, N):
        o = STATE_BYTES + parity * self.slot_bytes
        return self.bufs[r][o:o + M * N * 2].view(torch.bfloat16).view(M, N)


@pytest.mark.parametrize("base,split2,me", [("fp8", 1, 0), ("fp8", 3, 1), ("nvfp4", 1, 1), ("fp8", 0, 0)])
def test_fused_epilogue_allreduce_with_a_hand_played_peer(base, split2, me):
    K, widths, R, L, M = 1024, (384, 128), 32, 4, 19
    N = sum(widths)
    d = configs.draw(K, widths, R, L, M, seed=21, ids_low=-1, w_std=0.05, b_std=0.05)
    if base == "fp8":
        op = build_fp8_op(configs.with_fp8_base(d), max_m=32)
    else:
        op = build_nvfp4_op(configs.with_nvfp4_base(d), max_m=32, rcp_approx=True)
    idx = make_index(d["ids"], L, 32)
    meta = device_meta(idx, M)
    x = d["x"].cuda()
    cfg = {"split2": split2, "stream": 2} if split2 else {"stream": 2}
    y_part = op(x, meta, cfg=cfg).clone()                      # this rank's partial output (no exchange)
    torch.cuda.synchronize()
    n_tiles = sum((w + 127) // 128 for w in widths)
    peer = 1 - me
    hc = HandComm(slot_bytes=32 * N * 2, me=me)
    g = torch.Generator(device="cuda").manual_seed(7)
    for call in range(2):
        epoch = call + 1
        theirs = (torch.randn(M, N, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
        hc.staged(peer, epoch & 1, M, N).copy_(theirs)                     # the peer's partial for this call ...
        hc.tile_flags(me)[peer, :n_tiles] = epoch                          # ... and its announcements, in OUR buffer
        y = torch.full_like(y_part, float("nan"))

        class Peer:                                                        # what op() needs of a tp.PeerComm
            comm = hc.comm
        op(x, meta, out=y, cfg=cfg, allreduce=Peer)
        torch.cuda.synchronize()
        assert op.scratch.status()[0] == 0
        parts = [y_part, theirs] if me == 0 else [theirs, y_part]          # rank order, fp32 accumulation, one rounding
        want = (parts[0].float() + parts[1].float()).to(torch.bfloat16)
        assert torch.equal(y, want), f"call {call}"
        assert torch.equal(hc.staged(me, epoch & 1, M, N), y_part)         # our partial, staged for the peer
        assert bool((hc.tile_flags(peer)[me, :n_tiles] == epoch).all())   # announced in the peer's buffer, tile by tile
        assert int(hc.state(me)[0]) == epoch and int(hc.state(me)[7]) == 0


def test_fused_allreduce_peer_missing_runs_into_the_wait_limit():
    K, widths, R, L, M = 512, (256,), 16, 2, 8
    d = configs.with_fp8_base(configs.draw(K, widths, R, L, M, seed=2, ids_low=-1))
    op = build_fp8_op(d, max_m=32)
    idx = make_index(d["ids"], L, 32)
    meta = device_meta(idx, M)
    hc = HandComm(slot_bytes=32 * 256 * 2, me=0)               # the peer announces nothing
    y = torch.full((M, 256), 5.0, dtype=torch.bfloat16, device="cuda")

    class Peer:
        comm = hc.comm
    op(d["x"].cuda(), meta, out=y, cfg={"stream": 2, "wait_ms": 5}, allreduce=Peer)
    torch.cuda.synchronize()
    st = op.scratch.status()
    assert st[0] == 1 and st[1] == 21, st[:8]                   # a wait ran out: tile flag of rank 1
    assert bool((y == 5.0).all())
