"""Parity on the per-GPU shapes of the 72B-class configuration under tensor parallelism 2 / 4 / 8 (hidden 8192, 64 query /
8 kv heads of 128, intermediate 29568; the reference lists the same per-GPU shapes for its sweeps,
bench/pdl_k2_bench.py:63-68, but refuses slices that are not multiples of 64, lowbit_lora/plugin.py:253).  The shards are
the awkward ones: gate_up slices of 14784 / 7392 / 3696 rows (a partial last output tile per slice), down's K of
14784 / 7392 / 3696 (a K tail that is not a whole 128-byte block: TMA fills it with zeros), qkv with 128-row kv slices.
Each shard runs at full size on the device and is checked against the CPU oracle on a sample of output features (the
first and last rows of every slice plus random ones), as tests/test_fullsize_gpu.py does; codes and scales in full."""
from __future__ import annotations

import pytest
import torch

from helpers import device_meta, max_err_ratio
from oracle import configs, fp8 as ofp8, segments as oseg

pytestmark = pytest.mark.gpu
L, R = 32, 64
TOL = 2e-2


def shard_shape(name: str, tp: int):
    """(K, widths) of one rank's shard: column-parallel layers split every slice's rows, row-parallel layers split K."""
    K, widths = configs.L72B[name]
    if name in ("qkv", "gate_up"):
        return K, tuple(w // tp for w in widths)
    return K // tp, widths


CASES = [(name, tp, M) for tp in (2, 4, 8) for name in ("qkv", "o", "gate_up", "down") for M in (32,)]
CASES += [("gate_up", 4, 8), ("down", 4, 8), ("gate_up", 8, 128), ("down", 8, 128), ("gate_up", 2, 128), ("down", 2, 8)]


@pytest.mark.parametrize("name,tp,M", CASES)
def test_tp_shard_shapes_of_the_72b_layer(name, tp, M):
    from onebase_b200.kernels.fp8_lora_vllm import VllmFusedFP8LoRA
    K, widths = shard_shape(name, tp)
    N = sum(widths)
    g = torch.Generator(device="cuda").manual_seed(1000 * tp + 10 * len(name) + M)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.02
    s_w = (w.abs().max() / 448.0).reshape(1).float()
    w_q = (w / s_w).to(torch.float8_e4m3fn)
    del w
    a_st = tuple(((torch.rand(L, 1, R, K, device="cuda", generator=g) * 2 - 1) / K ** 0.5).to(torch.bfloat16) for _ in widths)
    b_st = tuple((torch.randn(L, 1, n, R, device="cuda", generator=g) * 0.01).to(torch.bfloat16) for n in widths)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    op = VllmFusedFP8LoRA(w_q, s_w, a_st, b_st, max_m=M)
    g_cpu = torch.Generator().manual_seed(M + tp)
    ids = torch.randint(-1, L, (M,), generator=g_cpu, dtype=torch.int32)
    idx = oseg.SegmentIndex(L, M)
    idx.prepare(ids)
    meta = device_meta(idx, M)
    y = op(x, meta)
    y2 = op(x, meta)
    torch.cuda.synchronize()
    assert op.scratch.status()[0] == 0, op.scratch.status()[:8]
    assert torch.equal(y, y2)
    x_cpu = x.cpu()
    rows, _ = oseg.resolve_positions(M, *idx.args(M))
    q_ref, sx_ref = ofp8.quant_per_token(x_cpu)
    assert torch.equal(op.scratch.xq(M, K).view(torch.uint8).cpu(), q_ref.view(torch.uint8)[rows])
    assert torch.equal(op.scratch.sx(M).cpu().view(torch.int32), sx_ref[rows].view(torch.int32))
    # sampled output features per slice: the first and last 8 (the ragged last tile) and random ones
    glob, local, off = [], [], 0
    for n in widths:
        pick = torch.unique(torch.cat([torch.arange(8), torch.arange(n - 8, n), torch.randint(0, n, (24,), generator=g_cpu)]))
        local.append(pick)
        glob.append(pick + off)
        off += n
    sel = torch.cat(glob)
    a_red = tuple(t.cpu() for t in a_st)
    b_red = tuple(t[:, :, loc.to(t.device)].cpu() for t, loc in zip(b_st, local))
    A, B = ofp8.stack_slices(a_red, b_red)
    ref = ofp8.fused_projection(x_cpu, ids, w_q.view(torch.uint8)[sel.cuda()].cpu().view(torch.float8_e4m3fn), s_w.cpu(), A, B,
                                [len(loc) for loc in local])
    got = y[:, sel.cuda()]
    err = max_err_ratio(got, ref)
    assert err <= TOL, f"{name} TP{tp} shard K={K} widths={widths} M={M}: max-abs-err / ||y||inf = {err:.3e}"
    assert float((got.float().cpu() - ref).norm() / ref.norm()) < 1e-2
    if M <= 32:                                               # the persistent GEMM on the same shard
        y3 = op(x, meta, cfg={"stream": 1})
        torch.cuda.synchronize()
        assert op.scratch.status()[0] == 0
        assert max_err_ratio(y3[:, sel.cuda()], ref) <= TOL
