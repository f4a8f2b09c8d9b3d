"""The persistent decode GEMM (one CTA per SM streaming a contiguous share of the weight k-blocks across output tiles)
against the oracle and against the tile-per-CTA GEMM, through the C ABI: shapes whose tiles are shared between CTAs in
every way (more tiles than CTAs, fewer, a CTA spanning three tiles), slices, K tails, partial output tiles, padded and
stale metadata, both base formats, serialized and chained launches, repeat launches bitwise equal, counters back to zero."""
from __future__ import annotations

import pytest
import torch

from helpers import (build_fp8_op, build_nvfp4_op, device_meta, make_index, max_err_ratio, oracle_y, oracle_y_nvfp4)
from oracle import configs, fp8 as ofp8, segments as oseg

pytestmark = pytest.mark.gpu
TOL = 2e-2
S1 = {"stream": 1}                                            # ask for the persistent GEMM (the tile GEMM is the default)


def _status_ok(op):
    st = op.scratch.status()
    assert st[0] == 0, f"device status {st[:8]}"


@pytest.mark.parametrize("K,widths,R,L,M,ids_low", [
    (4096, (4096,), 16, 4, 16, -1),            # configuration 0: 32 tiles x 32 k-blocks over 148 CTAs (about 7 per CTA)
    (128, (128,), 16, 2, 1, 0),                # one tile, one k-block: a single CTA owns everything
    (256, (128, 64, 64), 16, 4, 21, -1),       # three slices with partial tiles, two k-blocks each
    (384, (200,), 32, 3, 5, -1),               # K of three k-blocks, an output tile with a ragged edge
    (2048, (2560, 512), 64, 8, 32, 0),         # 24 tiles x 16 k-blocks: CTAs cross tile and slice boundaries
    (8192, (256,), 64, 32, 32, 0),             # two tiles of 64 k-blocks: every tile shared by dozens of CTAs
    (1024, (19200,), 64, 6, 24, -1),           # 150 tiles of 8 k-blocks: a CTA's share spans whole tiles and two shared ones
    (512, (256,), 256, 3, 9, -1),              # rank 256: four rank chunks per tenant
    (4096, (4096, 1024, 1024), 64, 32, 32, 0),  # the qkv projection of the benchmark layer
])
def test_stream_gemm_matches_oracle_and_tile_gemm(K, widths, R, L, M, ids_low):
    d = configs.with_fp8_base(configs.draw(K, widths, R, L, M, seed=K + M + len(widths), ids_low=ids_low, w_std=0.05, b_std=0.05))
    op = build_fp8_op(d, max_m=32)
    idx = make_index(d["ids"], L, 32)
    meta = device_meta(idx, M)
    x = d["x"].cuda()
    assert op.resolved_tile(M, S1)["stream"] == 1 and op.resolved_tile(M)["stream"] == 2
    y = op(x, meta, cfg=S1)                                   # the chain: K1 -> persistent GEMM
    y_again = op(x, meta, cfg=S1)
    y_serial = op(x, meta, cfg=S1, pdl=False)                 # the same two kernels without the programmatic edge
    y_tiles = op(x, meta)
    torch.cuda.synchronize()
    _status_ok(op)
    ref = oracle_y(d, d["x"], d["ids"])
    assert max_err_ratio(y, ref) <= TOL and max_err_ratio(y_tiles, ref) <= TOL
    assert float((y.float().cpu() - ref).norm() / ref.norm()) < 1e-2
    assert torch.equal(y, y_again) and torch.equal(y, y_serial)
    assert max_err_ratio(y, y_tiles.float().cpu()) <= 8e-3    # the two GEMMs add a shared tile's parts in different orders
    counters = op.scratch.region("counters", 4 * (4096 + 16)).view(torch.int32)
    assert int(counters.abs().sum()) == 0
    rows, _ = oseg.resolve_positions(M, *idx.args(M))
    q_ref, sx_ref = ofp8.quant_per_token(d["x"])
    assert torch.equal(op.scratch.xq(M, K).view(torch.uint8).cpu(), q_ref.view(torch.uint8)[rows])
    assert torch.equal(op.scratch.sx(M).cpu().view(torch.int32), sx_ref[rows].view(torch.int32))


@pytest.mark.parametrize("kind", ["none", "single", "padded"])
def test_stream_gemm_metadata_states(kind):
    """No adapter right after an adapter batch (stale index), a single tenant, CUDA-graph padding with poisoned entries."""
    K, widths, R, L, M = 512, (384, 128), 32, 5, 24
    d = configs.with_fp8_base(configs.draw(K, widths, R, L, M, seed=17, ids_low=-1, w_std=0.05, b_std=0.05))
    op = build_fp8_op(d, max_m=32)
    idx = oseg.SegmentIndex(L, 32)
    g = torch.Generator().manual_seed(3)
    idx.prepare(torch.randint(0, L, (32,), generator=g, dtype=torch.int32))          # a previous batch leaves its state
    if kind == "none":
        ids = torch.full((M,), -1, dtype=torch.int32)
        idx.prepare(ids)
    elif kind == "single":
        ids = torch.full((M,), L - 1, dtype=torch.int32)
        idx.prepare(ids)
    else:
        ids = torch.randint(-1, L, (M,), generator=g, dtype=torch.int32)
        ids[0] = 0
        idx.srt[M - 5:M] = 10 ** 6
        idx.tok[M - 5:M] = L - 1
        idx.prepare(ids[: M - 5])
        ids[M - 5:] = -1
    eff = oseg.effective_token_lora(M, *idx.args(M))
    assert torch.equal(eff, ids)
    y = op(d["x"].cuda(), device_meta(idx, M), cfg=S1)
    torch.cuda.synchronize()
    _status_ok(op)
    assert op.resolved_tile(M, S1)["stream"] == 1
    assert max_err_ratio(y, oracle_y(d, d["x"], eff)) <= TOL


@pytest.mark.parametrize("K,widths,R,L,M", [(512, (256, 128), 32, 4, 19), (4096, (1024, 512), 64, 16, 32), (256, (640,), 16, 3, 7)])
@pytest.mark.parametrize("approx", [False, True])
def test_stream_gemm_nvfp4_base(K, widths, R, L, M, approx):
    from oracle import nvfp4 as on4
    d = configs.with_nvfp4_base(configs.draw(K, widths, R, L, M, seed=K + M, ids_low=-1, w_std=0.05, b_std=0.05))
    op = build_nvfp4_op(d, max_m=32, rcp_approx=approx)
    idx = make_index(d["ids"], L, 32)
    meta = device_meta(idx, M)
    x = d["x"].cuda()
    y = op(x, meta, cfg=S1)
    y_again = op(x, meta, cfg=S1)
    y_tiles = op(x, meta)
    torch.cuda.synchronize()
    _status_ok(op)
    assert op.resolved_tile(M, S1)["stream"] == 1
    ref = oracle_y_nvfp4(d, d["x"], d["ids"])
    assert max_err_ratio(y, ref) <= TOL and max_err_ratio(y_tiles, ref) <= TOL
    assert torch.equal(y, y_again)
    if not approx:
        rows, _ = oseg.resolve_positions(M, *idx.args(M))
        q_ref, sf_ref = on4.quant(d["x"], d["x_global"])
        xq, xsf = op.codes(M)
        assert torch.equal(xq.cpu(), q_ref[rows]) and torch.equal(xsf.view(torch.uint8).cpu(), sf_ref.view(torch.uint8)[rows])


def test_stream_gemm_in_a_cuda_graph_with_changing_batches():
    """One captured chain replayed over batches of different tenants: the segment index and x change in place."""
    K, widths, R, L, M = 1024, (512, 256), 64, 8, 32
    d = configs.with_fp8_base(configs.draw(K, widths, R, L, M, seed=5, ids_low=-1, w_std=0.05, b_std=0.05))
    op = build_fp8_op(d, max_m=32)
    from onebase_b200.metadata import KernelMeta
    km = KernelMeta.make(L, 32, "cuda")
    x = torch.zeros(M, K, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(M, sum(widths), dtype=torch.bfloat16, device="cuda")
    km.prepare_tensors(d["ids"].cuda())
    op(x, km.meta_args(M), out=y, cfg=S1)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        op(x, km.meta_args(M), out=y, cfg=S1)
    gen = torch.Generator().manual_seed(9)
    for step in range(4):
        ids = torch.randint(-1, L, (M,), generator=gen, dtype=torch.int32) if step != 2 else torch.full((M,), -1, dtype=torch.int32)
        xs = torch.randn(M, K, generator=gen).to(torch.bfloat16)
        km.prepare_tensors(ids.cuda())
        x.copy_(xs)
        g.replay()
        torch.cuda.synchronize()
        _status_ok(op)
        assert max_err_ratio(y, oracle_y(d, xs, ids)) <= TOL, step
