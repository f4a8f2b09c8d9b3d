"""The CPU oracle against the golden files that the reference itself produced (tests/golden/make_golden.py)."""
from __future__ import annotations

import numpy as np
import torch

from conftest import bf16, e4m3, t
from oracle import fp8, nvfp4, segments


def u8(x: torch.Tensor) -> torch.Tensor:
    return x.contiguous().view(torch.uint8)


def test_fp8_per_token_quant_bit_exact(golden):
    g = golden("fp8_quant")
    codes, sx = fp8.quant_per_token(bf16(g["x"]))
    assert torch.equal(u8(codes), t(g["codes"]))
    assert torch.equal(sx.view(torch.int32), t(g["sx"]).view(torch.int32))
    # known answers: the floor on an all-zero row, and a row whose scale is exactly 1
    assert sx[1].item() == np.float32(1.0 / (448.0 * 512.0))
    assert sx[4].item() == 1.0


def test_segment_index_matches_vllm_sequence(golden):
    g = golden("segment_index")
    idx = segments.SegmentIndex(int(g["L"]), int(g["max_m"]))
    for i in range(len(g["kinds"])):
        m = int(g[f"s{i}_m"])
        idx.prepare(t(g[f"s{i}_given"]))
        got = idx.args(m)
        for name, have in zip(("tok", "srt", "seg_n", "seg_start", "seg_ids"), got):
            want = t(g[f"s{i}_{name}"])
            kind = str(g["kinds"][i])
            if kind == "padded" and name in ("tok", "srt"):
                n = int(g[f"s{i}_given"].shape[0])          # beyond the real tokens the fixture holds poisoned entries
                assert torch.equal(have[:n], want[:n]), (i, name)
            else:
                assert torch.equal(have, want), (i, kind, name)


def _stacks(g, p, S):
    return tuple(bf16(g[p + f"a{s}"]) for s in range(S)), tuple(bf16(g[p + f"b{s}"]) for s in range(S))


def test_fp8_projection_matches_reference(golden):
    g = golden("fp8_projection")
    for ci in range(int(g["n_cases"])):
        p = f"c{ci}_"
        widths = tuple(int(v) for v in g[p + "widths"])
        a_st, b_st = _stacks(g, p, len(widths))
        A, B = fp8.stack_slices(a_st, b_st)
        x, tok = bf16(g[p + "x"]), t(g[p + "tok"])
        y = fp8.fused_projection(x, tok, e4m3(g[p + "w_q"]), t(g[p + "s_w"]), A, B, widths)
        want = t(g[p + "y"])
        assert float((y - want).abs().max()) <= 2e-5 * float(want.abs().max())


def test_fp8_stored_adapters_bit_exact(golden):
    g = golden("fp8_projection")
    for ci in range(int(g["n_cases"])):
        p = f"c{ci}_"
        widths = tuple(int(v) for v in g[p + "widths"])
        a_st, b_st = _stacks(g, p, len(widths))
        As, Bs = [], []
        for s in range(len(widths)):
            for src, qn, sn, acc in ((a_st[s], "aq", "as", As), (b_st[s], "bq", "bs", Bs)):
                codes, scale = fp8.store_rows_fp8(src[:, 0])
                assert torch.equal(u8(codes), t(g[p + f"fp8_{qn}{s}"])[:, 0])
                assert torch.equal(scale.view(torch.int32), t(g[p + f"fp8_{sn}{s}"]).view(torch.int32))
                acc.append(codes.float() * scale[..., None])
        y = fp8.fused_projection(bf16(g[p + "x"]), t(g[p + "tok"]), e4m3(g[p + "w_q"]), t(g[p + "s_w"]),
                                 torch.cat(As, 1), torch.cat(Bs, 1), widths)
        want = t(g[p + "fp8_y"])
        assert float((y - want).abs().max()) <= 2e-5 * float(want.abs().max())


def test_nvfp4_stored_adapters_bit_exact(golden):
    g = golden("fp8_projection")
    for ci in range(int(g["n_cases"])):
        p = f"c{ci}_"
        widths = tuple(int(v) for v in g[p + "widths"])
        a_st, b_st = _stacks(g, p, len(widths))
        As, Bs = [], []
        for s in range(len(widths)):
            for src, qn, sn, gn, acc in ((a_st[s], "aq", "as", "ag", As), (b_st[s], "bq", "bs", "bg", Bs)):
                packed, sf, inv_g = nvfp4.quant_stack(src[:, 0])
                assert torch.equal(packed, t(g[p + f"nvfp4_{qn}{s}"])[:, 0])
                assert torch.equal(u8(sf), t(g[p + f"nvfp4_{sn}{s}"])[:, 0])
                assert torch.equal(inv_g.view(torch.int32), t(g[p + f"nvfp4_{gn}"])[s].view(torch.int32))
                acc.append(nvfp4.dequant_stack(packed, sf, inv_g))
        y = fp8.fused_projection(bf16(g[p + "x"]), t(g[p + "tok"]), e4m3(g[p + "w_q"]), t(g[p + "s_w"]),
                                 torch.cat(As, 1), torch.cat(Bs, 1), widths)
        want = t(g[p + "nvfp4_y"])
        assert float((y - want).abs().max()) <= 2e-5 * float(want.abs().max())


def test_nvfp4_quant_dequant_projection(golden):
    g = golden("nvfp4")
    for ci in range(int(g["n_cases"])):
        p = f"c{ci}_"
        widths = tuple(int(v) for v in g[p + "widths"])
        w = t(g[p + "w"])
        w_global = nvfp4.global_scale_for(w)
        assert w_global == float(g[p + "w_global"])
        w_q, w_sf = nvfp4.quant(w, w_global)
        assert torch.equal(w_q, t(g[p + "w_q"])) and torch.equal(u8(w_sf), t(g[p + "w_sf"]))
        x = bf16(g[p + "x"])
        x_global = nvfp4.global_scale_for(x)
        assert x_global == float(g[p + "x_global"])
        xq, xsf = nvfp4.quant(x, x_global)
        assert torch.equal(xq, t(g[p + "xq"])) and torch.equal(u8(xsf), t(g[p + "xsf"]))
        assert torch.equal(nvfp4.dequant(w_q, w_sf, w_global), t(g[p + "w_deq"]))
        a_st, b_st = _stacks(g, p, len(widths))
        A, B = fp8.stack_slices(a_st, b_st)
        y = nvfp4.fused_projection(x, t(g[p + "tok"]), w_q, w_sf, w_global, x_global, A, B, widths)
        want = t(g[p + "y"])
        assert float((y - want).abs().max()) <= 2e-5 * float(want.abs().max())


def test_e2m1_ties_and_saturation(golden):
    g = golden("nvfp4")
    q, sf = nvfp4.quant(t(g["ties_x"]), 1.0)
    assert torch.equal(q, t(g["ties_q"])) and torch.equal(u8(sf), t(g["ties_sf"]))
    # known answers, independent of the fixture: ties go to the even code, the grid saturates at 6
    v = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 7.0, -0.75, -100.0])
    assert nvfp4.e2m1_codes(v).tolist() == [0, 2, 2, 4, 4, 6, 6, 7, 7, 10, 15]
    assert nvfp4.E2M1_VALUES == (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
    packed = torch.tensor([[0x21]], dtype=torch.uint8)                   # element 0 in the low nibble
    assert nvfp4.unpack_values(packed).tolist() == [[0.5, 1.0]]


def test_resolve_positions_padding_and_stale():
    idx = segments.SegmentIndex(4, 32)
    tok = torch.tensor([1, -1, 0, 1, 3, 0], dtype=torch.int32)
    idx.prepare(tok)
    rows, ads = segments.resolve_positions(8, *idx.args(8))              # two padding rows beyond the six tokens
    assert rows.tolist() == [1, 2, 5, 0, 3, 4, 6, 7]
    assert ads.tolist() == [-1, 0, 0, 1, 1, 3, -1, -1]
    idx.prepare(torch.full((6,), -1, dtype=torch.int32))                 # no adapter: stale sort must be ignored
    rows, ads = segments.resolve_positions(6, *idx.args(6))
    assert rows.tolist() == list(range(6)) and ads.tolist() == [-1] * 6


def test_port_equals_the_references_own_modules_when_built():
    """`python -m oracle.build_ref` puts the reference's three source files under oracle/_ref (git-ignored).  Where that
    copy exists -- the build machine, and any box the snapshot travels to -- the restatement must agree with the
    reference's own functions on freshly drawn inputs, not only with the committed fixtures."""
    from oracle import build_ref, configs
    ref = build_ref.load()
    if ref is None:
        pytest.skip("oracle/_ref has not been built on this machine")
    ref8, ref4 = ref
    d = configs.with_fp8_base(configs.draw(512, (256, 128), 16, 4, 24, seed=11, ids_low=-1))
    A, B = fp8.stack_slices(d["a_stacked"], d["b_stacked"])
    want = ref8.reference_multi(d["x"], d["ids"], d["w_q"], d["s_w"], A, B, list(d["widths"]), 1.0)
    got = fp8.fused_projection(d["x"], d["ids"], d["w_q"], d["s_w"], A, B, d["widths"])
    assert float((got - want.float()).abs().max()) <= 2e-5 * float(want.float().abs().max())
    x = torch.randn(8, 256, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    gs = ref4.global_scale_for(x.float())
    assert gs == nvfp4.global_scale_for(x.float())
    q_ref, sf_ref = ref4.nvfp4_quant_torch(x, gs)
    q, sf = nvfp4.quant(x, gs)
    assert torch.equal(q, q_ref) and torch.equal(u8(sf), u8(sf_ref))
    assert torch.equal(nvfp4.dequant(q, sf, gs), ref4.nvfp4_dequant_torch(q_ref, sf_ref, gs))
