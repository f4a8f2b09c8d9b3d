"""The ops either side of the projection, fused: silu(gate) * up formed inside K1 (down_proj's input, read once instead of
written and re-read by a kernel of its own) and the residual add inside K2's stores (after o_proj / down_proj), against
the oracle's restatement of vLLM's SiluAndMul and of the residual half of its fused add + RMSNorm.

The activation goes through expf: the device's and the host's may differ in the last fp32 bit, which flips a bf16
rounding of silu(g) on a few elements in a million.  So: the activation scales and codes are compared with the oracle
quantizer applied to the ORACLE's activation and must agree on all but a few per million codes (and every scale but
such rows'), and the outputs hold the usual 2e-2 * ||y||inf bound against the oracle chain."""
from __future__ import annotations

import pytest
import torch

from helpers import build_fp8_op, build_nvfp4_op, device_meta, make_index, max_err_ratio
from oracle import configs, fp8 as ofp8, neighbours as onb, segments as oseg

pytestmark = pytest.mark.gpu
TOL = 2e-2


def _gate_up(M, K, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(M, 2 * K, generator=g) * 1.5).to(torch.bfloat16)


@pytest.mark.parametrize("K,widths,R,L,M,cfg", [
    (12288, (4096,), 64, 32, 32, None),                        # down_proj of the benchmark layer, decode
    (1024, (256, 128), 16, 4, 7, {"stream": 1}),               # the looped K1 beside the persistent GEMM
    (2048, (512,), 32, 6, 200, {"prefill": 2}),                # a prefill batch, warp-level shrink
    (1024, (256,), 64, 4, 300, {"prefill": 1}),                # ... tensor-core shrink (the sorted copy of x is the activation)
])
def test_silu_mul_inside_k1_fp8(K, widths, R, L, M, cfg):
    d = configs.with_fp8_base(configs.draw(K, widths, R, L, M, seed=K + M, ids_low=-1, w_std=0.05, b_std=0.05))
    gu = _gate_up(M, K, seed=M)
    act = onb.silu_mul(gu)                                      # what vLLM would hand the projection
    op = build_fp8_op(d, max_m=max(32, M))
    idx = make_index(d["ids"], L, max(32, M))
    meta = device_meta(idx, M)
    y = op(gu.cuda(), meta, cfg=cfg, silu_mul=True)
    y_plain = op(act.cuda(), meta, cfg=cfg)                     # the unfused route: the same projection on the oracle's activation
    torch.cuda.synchronize()
    assert op.scratch.status()[0] == 0
    A, B = ofp8.stack_slices(d["a_stacked"], d["b_stacked"])
    ref = ofp8.fused_projection(act, d["ids"], d["w_q"], d["s_w"], A, B, d["widths"])
    assert max_err_ratio(y, ref) <= TOL and max_err_ratio(y_plain, ref) <= TOL
    assert max_err_ratio(y, y_plain.float().cpu()) <= 4e-3    # the two routes differ only where an expf bit flipped a rounding
    op(gu.cuda(), meta, cfg=cfg, silu_mul=True, gemm=False)
    torch.cuda.synchronize()
    rows, _ = oseg.resolve_positions(M, *idx.args(M))
    q_ref, sx_ref = ofp8.quant_per_token(act)
    codes = op.scratch.xq(M, K).view(torch.uint8).cpu()
    differing = int((codes != q_ref.view(torch.uint8)[rows]).sum())
    assert differing <= max(4, M * K // 100000), f"{differing} of {M * K} codes differ from the oracle's"
    assert int((op.scratch.sx(M).cpu().view(torch.int32) != sx_ref[rows].view(torch.int32)).sum()) <= 1


def test_silu_mul_inside_k1_nvfp4():
    from oracle import nvfp4 as on4
    K, widths, R, L, M = 2048, (512, 256), 32, 4, 21
    d = configs.with_nvfp4_base(configs.draw(K, widths, R, L, M, seed=5, ids_low=-1, w_std=0.05, b_std=0.05))
    gu = _gate_up(M, K, seed=9)
    act = onb.silu_mul(gu)
    d["x_global"] = on4.global_scale_for(act.float())
    op = build_nvfp4_op(d, max_m=32)
    idx = make_index(d["ids"], L, 32)
    y = op(gu.cuda(), device_meta(idx, M), silu_mul=True)
    torch.cuda.synchronize()
    assert op.scratch.status()[0] == 0
    A, B = ofp8.stack_slices(d["a_stacked"], d["b_stacked"])
    ref = on4.fused_projection(act, d["ids"], d["w_q4"], d["w_sf"], d["w_global"], d["x_global"], A, B, d["widths"])
    assert max_err_ratio(y, ref) <= TOL


@pytest.mark.parametrize("cfg", [None, {"split2": 1}, {"split2": 3}, {"stream": 1}])
@pytest.mark.parametrize("in_place", [False, True])
def test_residual_add_inside_k2_store(cfg, in_place):
    K, widths, R, L, M = 2048, (512, 200), 32, 4, 23          # a ragged last output tile too
    N = sum(widths)
    d = configs.with_fp8_base(configs.draw(K, widths, R, L, M, seed=12, ids_low=-1, w_std=0.05, b_std=0.05))
    op = build_fp8_op(d, max_m=32)
    idx = make_index(d["ids"], L, 32)
    meta = device_meta(idx, M)
    x = d["x"].cuda()
    g = torch.Generator().manual_seed(3)
    res = torch.randn(M, N, generator=g).to(torch.bfloat16)
    y_plain = op(x, meta, cfg=cfg).clone()
    want = onb.add_residual(y_plain.cpu(), res)               # bf16(y) + residual in fp32, one rounding: exact, no tolerance
    r_dev = res.cuda()
    out = r_dev if in_place else torch.empty_like(y_plain)
    y = op(x, meta, cfg=cfg, out=out, residual=r_dev)
    torch.cuda.synchronize()
    assert op.scratch.status()[0] == 0
    assert torch.equal(y.cpu(), want)
