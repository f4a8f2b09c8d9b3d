"""GPU parity of the NVFP4 path through the C ABI: activation codes and ue4m3 block scales bit-exact against the oracle
(the torch recipe with IEEE reciprocals) and against the fixture the reference itself produced; with rcp.approx.ftz
reciprocals (vLLM's CUDA quantizer) at most 0.1 % of codes / scales may differ (the reference's own bound,
tests/test_nvfp4_lora_vllm_interp.py:98); bf16 outputs within max-abs-error <= 2e-2 * ||y||_inf of the fp32 oracle."""
from __future__ import annotations

import pytest
import torch

from conftest import bf16, e4m3, t
from helpers import build_nvfp4_op, device_meta, make_index, max_err_ratio, oracle_y_nvfp4
from oracle import configs, nvfp4 as on4, segments as oseg

pytestmark = pytest.mark.gpu
TOL = 2e-2


def u8(x):
    return x.contiguous().view(torch.uint8)


def _case(K, widths, R, L, M, seed=0):
    d = configs.draw(K, widths, R, L, M, seed=seed, ids_low=-1, w_std=0.05, b_std=0.05)
    d["x"][:, :3] *= 8                                        # outlier channels, as the reference's test
    return configs.with_nvfp4_base(d)


def _status_ok(op):
    st = op.scratch.status()
    assert st[0] == 0, f"device status {st[:8]}"


@pytest.mark.parametrize("ci", [0, 1, 2])
def test_quant_codes_and_scales_bit_exact_golden(golden, ci):
    g = golden("nvfp4")
    p = f"c{ci}_"
    x = bf16(g[p + "x"])
    M, K = x.shape
    widths = tuple(int(v) for v in g[p + "widths"])
    S, L, R = len(widths), int(g[p + "L"]), int(g[p + "R"])
    d = {"w_q4": t(g[p + "w_q"]), "w_sf": e4m3(g[p + "w_sf"]), "w_global": float(g[p + "w_global"]),
         "x_global": float(g[p + "x_global"]), "widths": widths,
         "a_stacked": tuple(bf16(g[p + f"a{s}"]) for s in range(S)), "b_stacked": tuple(bf16(g[p + f"b{s}"]) for s in range(S))}
    op = build_nvfp4_op(d, max_m=64)
    tok = t(g[p + "tok"])
    idx = make_index(tok, L, 64)
    y = op(x.cuda(), device_meta(idx, M))
    torch.cuda.synchronize()
    _status_ok(op)
    rows, _ = oseg.resolve_positions(M, *idx.args(M))
    xq, xsf = op.codes(M)
    assert torch.equal(xq.cpu(), t(g[p + "xq"])[rows])
    assert torch.equal(u8(xsf).cpu(), t(g[p + "xsf"])[rows])
    assert max_err_ratio(y, t(g[p + "y"])) <= TOL


def test_e2m1_ties_fixture(golden):
    g = golden("nvfp4")
    x16 = t(g["ties_x"]).to(torch.bfloat16)                   # every tie point is exactly representable in bf16 ...
    keep = (x16.float() == t(g["ties_x"]))                    # ... except the "just above" probes, which are masked out
    x = torch.cat([x16, torch.zeros_like(x16)], dim=1)        # K must be a multiple of 32: one more (all-zero) block per row
    M, K = x.shape
    d = _case(K, (128,), 16, 2, M)
    d["x_global"] = 1.0
    op = build_nvfp4_op(d, max_m=16)
    idx = make_index(torch.full((M,), -1, dtype=torch.int32), 2, 16)
    op(x.cuda(), device_meta(idx, M), gemm=False)
    torch.cuda.synchronize()
    xq, xsf = op.codes(M)
    q_ref, sf_ref = on4.quant(x, 1.0)
    assert torch.equal(xq.cpu(), q_ref) and torch.equal(u8(xsf).cpu(), u8(sf_ref))
    assert int(u8(xsf).cpu()[:, 1].sum()) == 0                # the zero-scale guard: an all-zero block has scale 0, codes 0
    want = t(g["ties_q"])
    both = keep.reshape(M, 8, 2).all(-1)
    assert torch.equal(xq.cpu()[:, :8][both], want[both])


@pytest.mark.parametrize("K,widths,R,L,M,kind", [
    (256, (128, 128), 16, 4, 16, "mixed"),
    (64, (32, 16, 16), 16, 4, 21, "mixed"),
    (96, (64,), 32, 3, 5, "mixed"),
    (512, (256,), 64, 8, 13, "none"),
    (1024, (384, 128), 64, 6, 40, "single"),
    (128, (64,), 128, 2, 24, "padded"),
    (2048, (256, 128, 128), 32, 32, 32, "all32"),
    (4096, (512,), 64, 6, 100, "mixed"),                       # 128-token tile, two 32-row scale groups and more
])
def test_fused_projection_matches_oracle(K, widths, R, L, M, kind):
    d = _case(K, widths, R, L, M, seed=K + M)
    max_m = 128
    op = build_nvfp4_op(d, max_m=max_m)
    idx = oseg.SegmentIndex(L, max_m)
    g = torch.Generator().manual_seed(7)
    idx.prepare(torch.randint(0, L, (max_m,), generator=g, dtype=torch.int32))
    if kind == "mixed":
        ids = torch.randint(-1, L, (M,), generator=g, dtype=torch.int32)
        idx.prepare(ids)
    elif kind == "all32":
        ids = torch.arange(M, dtype=torch.int32) % L
        idx.prepare(ids)
    elif kind == "single":
        ids = torch.full((M,), L - 1, dtype=torch.int32)
        idx.prepare(ids)
    elif kind == "none":
        ids = torch.full((M,), -1, dtype=torch.int32)
        idx.prepare(ids)
    else:
        ids = torch.randint(-1, L, (M,), generator=g, dtype=torch.int32)
        ids[0] = 0
        idx.srt[M - 5:M] = 10 ** 6
        idx.tok[M - 5:M] = L - 1
        idx.prepare(ids[: M - 5])
        ids[M - 5:] = -1
    meta_cpu = idx.args(M)
    x = d["x"]
    meta = device_meta(idx, M)
    y = op(x.cuda(), meta)
    torch.cuda.synchronize()
    _status_ok(op)
    rows, _ = oseg.resolve_positions(M, *meta_cpu)
    q_ref, sf_ref = on4.quant(x, d["x_global"])
    xq, xsf = op.codes(M)
    assert torch.equal(xq.cpu(), q_ref[rows])
    assert torch.equal(u8(xsf).cpu(), u8(sf_ref)[rows])
    ref = oracle_y_nvfp4(d, x, ids)
    err = max_err_ratio(y, ref)
    assert err <= TOL, f"max-abs-err / ||y||inf = {err:.3e}"
    assert float((y.float().cpu() - ref).norm() / ref.norm()) < 1e-2
    y2 = op(x.cuda(), meta, pdl=False)
    torch.cuda.synchronize()
    assert torch.equal(y, y2)
    if M <= 32:                                                # the one-kernel form of the chain, twice in a row
        y4 = op(x.cuda(), meta, cfg={"fused": 1})
        y5 = op(x.cuda(), meta, cfg={"fused": 1})
        torch.cuda.synchronize()
        assert torch.equal(y, y4) and torch.equal(y, y5)
        xq2, xsf2 = op.codes(M)
        assert torch.equal(xq2.cpu(), q_ref[rows]) and torch.equal(u8(xsf2).cpu(), u8(sf_ref)[rows])
    _status_ok(op)


def test_rcp_approx_mode_stays_within_reference_bound():
    d = _case(2048, (256,), 16, 2, 64, seed=5)
    op = build_nvfp4_op(d, max_m=64, rcp_approx=True)
    idx = make_index(torch.full((64,), -1, dtype=torch.int32), 2, 64)
    op(d["x"].cuda(), device_meta(idx, 64), gemm=False)
    torch.cuda.synchronize()
    xq, xsf = op.codes(64)
    q_ref, sf_ref = on4.quant(d["x"], d["x_global"])
    assert float((xq.cpu() != q_ref).float().mean()) < 1e-3
    assert float((u8(xsf).cpu() != u8(sf_ref)).float().mean()) < 1e-3


def test_weight_scale_packing_round_trip():
    from onebase_b200.kernels.nvfp4_lora_vllm import pack_weight_scales
    K, widths = 1280, (200, 72)                                # partial tiles in both slices, 5 K slots
    N = sum(widths)
    sf = torch.randint(1, 120, (N, K // 16), dtype=torch.uint8)
    packed = pack_weight_scales(sf.cuda(), K, widths).cpu()
    kslots = (K + 255) // 256
    tiles = sum((w + 127) // 128 for w in widths)
    v = packed.view(tiles, kslots, 4, 32, 4, 4)                # [tile, K slot, mma, r32, r4, j]
    row0, tile0 = 0, 0
    for w in widths:
        for tl in range((w + 127) // 128):
            blk = v[tile0 + tl].permute(3, 2, 0, 1, 4).reshape(128, kslots * 16)   # [r4, r32, kb, mma, j] -> rows x cols
            n = min(128, w - tl * 128)
            assert torch.equal(blk[:n, : K // 16], sf[row0 + tl * 128: row0 + tl * 128 + n])
            assert int(blk[n:].sum()) == 0
        row0 += w
        tile0 += (w + 127) // 128


@pytest.mark.parametrize("fmt", ["fp8", "nvfp4"])
def test_nvfp4_base_with_stored_adapters(fmt):
    """NVFP4 base with FP8- or NVFP4-stored adapters (the benchmark's third configuration): outputs against the oracle run
    on the dequantized adapters."""
    from oracle import fp8 as ofp8
    d = _case(1024, (256, 128), 64, 6, 29, seed=13)
    op = build_nvfp4_op(d, max_m=64, lora_fmt=fmt)
    As, Bs = [], []
    for s in range(2):
        for src, acc in ((d["a_stacked"][s], As), (d["b_stacked"][s], Bs)):
            if fmt == "fp8":
                codes, scale = ofp8.store_rows_fp8(src[:, 0])
                acc.append(codes.float() * scale[..., None])
            else:
                acc.append(on4.dequant_stack(*on4.quant_stack(src[:, 0])))
    idx = make_index(d["ids"], 6, 64)
    y = op(d["x"].cuda(), device_meta(idx, 29))
    torch.cuda.synchronize()
    _status_ok(op)
    ref = on4.fused_projection(d["x"], d["ids"], d["w_q4"], d["w_sf"], d["w_global"], d["x_global"], torch.cat(As, 1),
                               torch.cat(Bs, 1), d["widths"])
    assert max_err_ratio(y, ref) <= TOL
