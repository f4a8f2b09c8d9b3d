"""The peer-memory all-reduce kernel (ob_allreduce), on ONE GPU: several ranks emulated by one cooperative launch over
buffers that all live on the device (ranks on one GPU must not be separate launches that wait for one another), both
forms, both dtypes, several calls in a row (the staged copies alternate by call parity); and a wait that runs out -- a
rank whose peer never publishes anything -- which must leave the output untouched and report which rank was missing."""
from __future__ import annotations

import ctypes as C

import pytest
import torch

from onebase_b200 import _lib

pytestmark = pytest.mark.gpu


def _comms(n: int, slot_bytes: int):
    size = C.c_size_t()
    _lib.call("ob_comm_bytes", slot_bytes, C.byref(size))
    bufs = [torch.zeros(size.value, dtype=torch.uint8, device="cuda") for _ in range(n)]
    comms = (_lib.ObComm * n)()
    for q in range(n):
        comms[q].world, comms[q].rank, comms[q].slot_bytes = n, q, slot_bytes
        for r in range(n):
            comms[q].bufs[r] = bufs[r].data_ptr()
    return comms, bufs


def _rank_order_sum(xs):
    acc = torch.zeros_like(xs[0], dtype=torch.float32)
    for x in xs:                                              # rank 0 first, fp32 accumulation, one rounding at the end
        acc = acc + x.float()
    return acc.to(xs[0].dtype)


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("dtype,mode", [(torch.bfloat16, _lib.OB_AR_ONE_SHOT), (torch.bfloat16, _lib.OB_AR_TWO_SHOT),
                                        (torch.float32, _lib.OB_AR_ONE_SHOT), (torch.float32, _lib.OB_AR_TWO_SHOT)])
def test_emulated_ranks_sum_in_rank_order(n, dtype, mode):
    count = 32 * 4096 + 1016                                  # a decode batch's y of the o projection, plus a ragged tail
    esz = 2 if dtype == torch.bfloat16 else 4
    comms, bufs = _comms(n, slot_bytes=(count * esz + 15) // 16 * 16)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    g = torch.Generator(device="cuda").manual_seed(n)
    for call in range(3):
        xs = [torch.randn(count, device="cuda", generator=g).to(dtype) for _ in range(n)]
        outs = [torch.full_like(x, float("nan")) for x in xs]
        src = (C.c_void_p * n)(*[x.data_ptr() for x in xs])
        dst = (C.c_void_p * n)(*[o.data_ptr() for o in outs])
        _lib.call("ob_allreduce_emulated", comms, n, src, dst, count, 0 if dtype == torch.bfloat16 else 1, mode, 2000, stream)
        torch.cuda.synchronize()
        want = _rank_order_sum(xs)
        for q in range(n):
            st = (C.c_int32 * 8)()
            _lib.call("ob_comm_status", C.byref(comms[q]), st, stream)
            assert st[3] == 0 and st[0] == call + 1, list(st)
            assert torch.equal(outs[q], want), (call, q)


def test_in_place_and_inside_a_cuda_graph():
    n, count = 2, 8 * 4096
    comms, bufs = _comms(n, slot_bytes=count * 2)
    xs = [torch.zeros(count, dtype=torch.bfloat16, device="cuda") for _ in range(n)]
    src = (C.c_void_p * n)(*[x.data_ptr() for x in xs])

    def launch():
        _lib.call("ob_allreduce_emulated", comms, n, src, src, count, 0, _lib.OB_AR_AUTO, 2000,
                  C.c_void_p(torch.cuda.current_stream().cuda_stream))

    launch()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        launch()
    g = torch.Generator(device="cuda").manual_seed(1)
    for _ in range(4):                                        # the call count lives in the buffer: replays keep alternating
        vals = [torch.randn(count, device="cuda", generator=g).to(torch.bfloat16) for _ in range(n)]
        for x, v in zip(xs, vals):
            x.copy_(v)
        graph.replay()
        torch.cuda.synchronize()
        want = _rank_order_sum(vals)
        assert torch.equal(xs[0], want) and torch.equal(xs[1], want)


def test_missing_peer_runs_into_the_wait_limit():
    count = 4096
    comms, bufs = _comms(2, slot_bytes=count * 2)
    x = torch.ones(count, dtype=torch.bfloat16, device="cuda")
    out = torch.full_like(x, 7.0)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    # only rank 0 calls: rank 1's flag is never written
    _lib.call("ob_allreduce", C.byref(comms[0]), C.c_void_p(x.data_ptr()), C.c_void_p(out.data_ptr()), count, 0, 0, 5, stream)
    torch.cuda.synchronize()
    st = (C.c_int32 * 8)()
    _lib.call("ob_comm_status", C.byref(comms[0]), st, stream)
    assert st[3] == 1 and st[4] == 1 and st[5] == 1, list(st)  # a wait ran out: the partials' wait, rank 1 missing
    assert bool((out == 7.0).all())
    for b in bufs:                                            # the ranks start over from zeroed buffers
        b.zero_()
    xs = [x, x * 2]
    outs = [torch.empty_like(x), torch.empty_like(x)]
    _lib.call("ob_allreduce_emulated", comms, 2, (C.c_void_p * 2)(*[t.data_ptr() for t in xs]),
              (C.c_void_p * 2)(*[t.data_ptr() for t in outs]), count, 0, 0, 2000, stream)
    torch.cuda.synchronize()
    assert bool((outs[0] == 3.0).all()) and bool((outs[1] == 3.0).all())


def test_rejects_bad_arguments():
    comms, bufs = _comms(2, slot_bytes=1024)
    x = torch.zeros(4096, dtype=torch.bfloat16, device="cuda")
    st = _lib.lib().ob_allreduce(C.byref(comms[0]), C.c_void_p(x.data_ptr()), C.c_void_p(x.data_ptr()), 4096, 0, 0, 5,
                                 C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == -9                                           # larger than the buffer's slots
    st = _lib.lib().ob_allreduce(C.byref(comms[0]), C.c_void_p(x.data_ptr()), C.c_void_p(x.data_ptr()), 12, 0, 0, 5, None)
    assert st == -2                                           # not a multiple of 16 bytes
