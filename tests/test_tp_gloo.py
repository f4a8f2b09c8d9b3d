"""Tensor-parallel sharding on two CPU ranks (gloo): the shard functions the GPU path uses, with the CPU oracle standing
in for the kernels.  Column-parallel shards concatenate to the unsharded result exactly; row-parallel partials, summed by
the all-reduce, equal the hand-written sum of per-rank results (each rank quantizes its own K slice of x, as vLLM does)."""
from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import configs, fp8 as ofp8


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.set_num_threads(2)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from onebase_b200 import tp
    try:
        # column-parallel, 3 slices
        d = configs.with_fp8_base(configs.draw(256, (128, 64, 64), 16, 4, 12, seed=3, w_std=0.05, b_std=0.05))
        A, B = ofp8.stack_slices(d["a_stacked"], d["b_stacked"])
        full = ofp8.fused_projection(d["x"], d["ids"], d["w_q"], d["s_w"], A, B, d["widths"])
        w_r, a_r, b_r = tp.shard_column(d["w_q"].view(torch.uint8), d["a_stacked"], d["b_stacked"], world, rank)
        Ar, Br = ofp8.stack_slices(a_r, b_r)
        widths_r = [t.shape[2] for t in b_r]
        y_r = ofp8.fused_projection(d["x"], d["ids"], w_r.view(torch.float8_e4m3fn), d["s_w"], Ar, Br, widths_r)
        parts = [torch.empty_like(y_r) for _ in range(world)]
        dist.all_gather(parts, y_r)
        off, cols = 0, []
        for w in d["widths"]:                                    # rank r holds columns [r*w/tp, (r+1)*w/tp) of every slice
            ws = w // world
            cols.append(torch.cat([parts[r][:, off // world: off // world + ws] for r in range(world)], 1))
            off += w
        col_err = float((torch.cat(cols, 1) - full).abs().max())
        # row-parallel
        d2 = configs.with_fp8_base(configs.draw(512, (192,), 32, 3, 9, seed=5, w_std=0.05, b_std=0.05))
        A2, B2 = ofp8.stack_slices(d2["a_stacked"], d2["b_stacked"])
        full2 = ofp8.fused_projection(d2["x"], d2["ids"], d2["w_q"], d2["s_w"], A2, B2, d2["widths"])
        w2, a2, b2 = tp.shard_row(d2["w_q"].view(torch.uint8), d2["a_stacked"], d2["b_stacked"], world, rank)
        x2 = tp.shard_input_row(d2["x"], world, rank)
        A2r, B2r = ofp8.stack_slices(a2, b2)
        y2 = ofp8.fused_projection(x2, d2["ids"], w2.view(torch.float8_e4m3fn), d2["s_w"], A2r, B2r, d2["widths"])
        y2 = tp.all_reduce_output(y2)
        # expected: the same partial sums written out by hand (each rank quantizes its own K slice of x, as vLLM does)
        expect = torch.zeros_like(full2)
        ks = 512 // world
        for r in range(world):
            xs = d2["x"][:, r * ks:(r + 1) * ks]
            xq, sx = ofp8.quant_per_token(xs)
            expect += (xq.float() * sx[:, None]) @ (d2["w_q"].float()[:, r * ks:(r + 1) * ks] * d2["s_w"]).t()
            expect += ofp8.lora_term(xs, d2["ids"], A2[:, :, r * ks:(r + 1) * ks], B2, d2["widths"])
        row_err = float((y2 - expect).abs().max() / expect.abs().max())
        # and the sharded result stays close to the unsharded one (two different quantizations of x: twice the noise)
        assert float((y2 - full2).norm() / full2.norm()) < 6e-2
        # row-parallel with sharded adapters: all-reduce of the fp32 shrink partials, then each rank expands its own rows of B
        d3 = configs.with_fp8_base(configs.draw(256, (256, 256), 16, 3, 7, seed=8, w_std=0.05, b_std=0.05))
        A3, B3 = ofp8.stack_slices(d3["a_stacked"], d3["b_stacked"])
        w3, a3, b3, b_shard = tp.shard_row_sharded_lora(d3["w_q"].view(torch.uint8), d3["a_stacked"], d3["b_stacked"], world, rank)
        x3 = tp.shard_input_row(d3["x"], world, rank)
        A3r = torch.cat([t[:, 0] for t in a3], dim=1).float()                     # [L, S*R, K/tp]
        ids3 = d3["ids"].to(torch.int64)
        h = torch.zeros(x3.shape[0], A3r.shape[1])
        for m in range(x3.shape[0]):
            if ids3[m] >= 0:
                h[m] = x3[m].float() @ A3r[ids3[m]].t()                           # this rank's partial of the shrink
        dist.all_reduce(h)                                                        # exchange 1
        hb = h.to(torch.bfloat16).float()
        xq3, sx3 = ofp8.quant_per_token(x3)
        y3 = (xq3.float() * sx3[:, None]) @ (w3.view(torch.float8_e4m3fn).float() * d3["s_w"]).t()
        R3, off = 16, 0
        for s_i, (row0, rows, width) in enumerate(b_shard):
            for m in range(x3.shape[0]):
                if ids3[m] >= 0:
                    y3[m, off + row0: off + row0 + rows] += b3[s_i][ids3[m], 0].float() @ hb[m, s_i * R3:(s_i + 1) * R3]
            off += width
        dist.all_reduce(y3)                                                       # exchange 2
        expect3 = ofp8.lora_term(d3["x"], d3["ids"], A3, B3, d3["widths"])        # the LoRA term is now the unsharded one
        ks3 = 256 // world
        for r in range(world):
            xs = d3["x"][:, r * ks3:(r + 1) * ks3]
            xq, sx = ofp8.quant_per_token(xs)
            expect3 += (xq.float() * sx[:, None]) @ (d3["w_q"].float()[:, r * ks3:(r + 1) * ks3] * d3["s_w"]).t()
        sharded_err = float((y3 - expect3).abs().max() / expect3.abs().max())
        assert [tuple(t.shape) for t in b3] == [(3, 1, 256 // world, 16)] * 2 and b_shard[0] == (rank * 128, 128, 256)
        if rank == 0:
            out.put((col_err, row_err, tuple(w_r.shape), tuple(w2.shape), tuple(a2[0].shape), sharded_err))
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_shards_two_ranks():
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
        assert p.exitcode == 0
    col_err, row_err, w_shape, w2_shape, a2_shape, sharded_err = out.get()
    assert col_err == 0.0                                        # column shards are exact slices of the unsharded result
    assert row_err <= 1e-5
    assert sharded_err <= 2e-3                                   # h is summed over the ranks in another order than one long dot
    assert w_shape == (128, 256) and w2_shape == (192, 256) and a2_shape == (3, 1, 32, 256)


def test_qkv_kv_replication_when_fewer_kv_heads_than_ranks():
    from onebase_b200 import tp
    w = torch.arange(64 * 8, dtype=torch.uint8).reshape(64, 8)
    a = (torch.zeros(2, 1, 16, 8, dtype=torch.bfloat16),) * 3
    b = tuple(torch.zeros(2, 1, n, 16, dtype=torch.bfloat16) for n in (32, 16, 16))
    # 4 ranks, kv slices of 16 rows shared by 2 ranks each: q splits 4 ways (8 rows), k / v split 2 ways (8 rows)
    shapes = []
    for rank in range(4):
        w_r, _, b_r = tp.shard_column(w, a, b, 4, rank, replicate=(1, 2, 2))
        shapes.append([t.shape[2] for t in b_r])
        assert torch.equal(w_r[:8], w[rank * 8: rank * 8 + 8])
        assert torch.equal(w_r[8:16], w[32 + (rank // 2) * 8: 32 + (rank // 2) * 8 + 8])
    assert shapes == [[8, 8, 8]] * 4


def test_nvfp4_base_shards():
    """NVFP4 base under tensor parallelism (shard arithmetic only, the oracle standing in for the kernels): column shards
    concatenate to the unsharded result exactly; row shards, whose activation codes equal the unsharded ones block for
    block, sum to it up to the fp32 summation order and one bf16 rounding of each rank's partial h."""
    from onebase_b200 import tp
    from oracle import nvfp4 as on4
    world = 2
    d = configs.with_nvfp4_base(configs.draw(256, (128, 64), 16, 4, 11, seed=13, w_std=0.05, b_std=0.05))
    A, B = ofp8.stack_slices(d["a_stacked"], d["b_stacked"])
    full = on4.fused_projection(d["x"], d["ids"], d["w_q4"], d["w_sf"], d["w_global"], d["x_global"], A, B, d["widths"])
    parts = []
    for rank in range(world):
        q_r, sf_r, a_r, b_r = tp.shard_column_nvfp4(d["w_q4"], d["w_sf"], d["a_stacked"], d["b_stacked"], world, rank)
        assert q_r.shape == (96, 128) and sf_r.shape == (96, 16) and sf_r.dtype == d["w_sf"].dtype
        Ar, Br = ofp8.stack_slices(a_r, b_r)
        parts.append(on4.fused_projection(d["x"], d["ids"], q_r, sf_r, d["w_global"], d["x_global"], Ar, Br, [t.shape[2] for t in b_r]))
    cols, off = [], 0
    for w in d["widths"]:
        ws = w // world
        cols.append(torch.cat([parts[r][:, off // world: off // world + ws] for r in range(world)], 1))
        off += w
    assert torch.equal(torch.cat(cols, 1), full)
    total = torch.zeros_like(full)
    for rank in range(world):
        q_r, sf_r, a_r, b_r = tp.shard_row_nvfp4(d["w_q4"], d["w_sf"], d["a_stacked"], d["b_stacked"], world, rank)
        assert q_r.shape == (192, 64) and sf_r.shape == (192, 8) and a_r[0].shape[-1] == 128
        x_r = tp.shard_input_row(d["x"], world, rank)
        xq_full, xsf_full = on4.quant(d["x"], d["x_global"])
        xq_r, xsf_r = on4.quant(x_r, d["x_global"])
        assert torch.equal(xq_r, xq_full[:, rank * 64:(rank + 1) * 64]) and torch.equal(xsf_r.view(torch.uint8), xsf_full.view(torch.uint8)[:, rank * 8:(rank + 1) * 8])
        Ar, Br = ofp8.stack_slices(a_r, b_r)
        total += on4.fused_projection(x_r, d["ids"], q_r, sf_r, d["w_global"], d["x_global"], Ar, Br, d["widths"])
    assert float((total - full).abs().max() / full.abs().max()) <= 2e-3
    with pytest.raises(AssertionError):
        tp.shard_row_nvfp4(d["w_q4"][:, :24], d["w_sf"][:, :3], d["a_stacked"], d["b_stacked"], world, 0)   # K = 48: 24 per rank
