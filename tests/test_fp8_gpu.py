"""GPU parity of the FP8 path through the C ABI: quantization codes / scales and the token sort bit-exact against the
oracle, bf16 outputs within max-abs-error <= 2e-2 * ||y||_inf of the oracle's fp32 result (the acceptance bound);
edge cases as the reference's CPU tests (tests/test_fp8_lora_vllm_interp.py): mixed adapters with tokens without one,
a single adapter, none right after an adapter batch (stale metadata), CUDA-graph padding with poisoned stale entries,
one to four slices, ranks 16..128, K tails, split-K variants, repeat-launch determinism, counters back to zero."""
from __future__ import annotations

import ctypes as C

import numpy as np
import pytest
import torch

from conftest import bf16, e4m3, t
from helpers import build_fp8_op, device_meta, make_index, max_err_ratio, oracle_y
from oracle import configs, fp8 as ofp8, segments as oseg

pytestmark = pytest.mark.gpu
TOL = 2e-2


def u8(x):
    return x.contiguous().view(torch.uint8)


def _case(K, widths, R, L, M, seed=0, ids_low=-1):
    return configs.with_fp8_base(configs.draw(K, widths, R, L, M, seed=seed, ids_low=ids_low, w_std=0.05, b_std=0.05))


def _check_status(op):
    st = op.scratch.status()
    assert st[0] == 0, f"device status {st[:8]}"


def test_segment_index_bit_exact_sequence(golden):
    from onebase_b200 import _lib
    g = golden("segment_index")
    L, max_m = int(g["L"]), int(g["max_m"])
    dev = "cuda"
    tok = torch.zeros(max_m, dtype=torch.int32, device=dev)
    srt = torch.zeros(max_m, dtype=torch.int32, device=dev)
    seg_n = torch.zeros(L + 1, dtype=torch.int32, device=dev)
    seg_start = torch.zeros(L + 2, dtype=torch.int32, device=dev)
    seg_ids = torch.zeros(L + 1, dtype=torch.int32, device=dev)
    ref = oseg.SegmentIndex(L, max_m)
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for i in range(len(g["kinds"])):
        given = t(g[f"s{i}_given"])
        m = int(g[f"s{i}_m"])
        ref.prepare(given)
        gd = given.to(dev)
        _lib.call("ob_segment_index", C.c_void_p(gd.data_ptr()), given.numel(), L, C.c_void_p(tok.data_ptr()),
                  C.c_void_p(srt.data_ptr()), C.c_void_p(seg_n.data_ptr()), C.c_void_p(seg_start.data_ptr()),
                  C.c_void_p(seg_ids.data_ptr()), st)
        torch.cuda.synchronize()
        n = given.numel()
        for name, have, want in (("tok", tok[:n], ref.tok[:n]), ("srt", srt[:n], ref.srt[:n]), ("seg_n", seg_n, ref.seg_n),
                                 ("seg_start", seg_start, ref.seg_start), ("seg_ids", seg_ids, ref.seg_ids)):
            assert torch.equal(have.cpu(), want), (i, str(g["kinds"][i]), name)
        # and against the file vLLM itself produced
        assert torch.equal(seg_n.cpu(), t(g[f"s{i}_seg_n"])) and torch.equal(seg_start.cpu(), t(g[f"s{i}_seg_start"]))
        assert torch.equal(seg_ids.cpu(), t(g[f"s{i}_seg_ids"]))


def test_segment_index_large_batch():
    from onebase_b200 import _lib
    L, M = 32, 4099
    ids = configs.zipf_request_ids(M, L, seed=3)
    ids[::7] = -1
    ref = make_index(ids, L, M)
    dev = "cuda"
    out = [torch.zeros(n, dtype=torch.int32, device=dev) for n in (M, M, L + 1, L + 2, L + 1)]
    gd = ids.to(dev)
    _lib.call("ob_segment_index", C.c_void_p(gd.data_ptr()), M, L, *[C.c_void_p(o.data_ptr()) for o in out],
              C.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    for have, want in zip(out, (ref.tok[:M], ref.srt[:M], ref.seg_n, ref.seg_start, ref.seg_ids)):
        assert torch.equal(have.cpu(), want)


def test_segment_index_hook_device_path():
    """The replacement for vLLM's LoRAKernelMeta.prepare_tensors (LOWBIT_SEGMENT_INDEX=1) on device tensors: the five
    tensors bit-equal to the oracle over a sequence of batches on the same object, and vLLM's host-side flags."""
    from onebase_b200.plugin import segment_index_prepare
    L, max_m = 6, 48

    class Meta:   # the attributes of vllm/lora/ops/triton_ops/lora_kernel_metadata.py:14-60 the replacement touches
        def __init__(self):
            z = lambda n: torch.zeros(n, dtype=torch.int32, device="cuda")   # noqa: E731
            self.token_lora_mapping, self.token_indices_sorted_by_lora_ids = z(max_m), z(max_m)
            self.active_lora_ids = torch.full((L + 1,), -1, dtype=torch.int32, device="cuda")
            self.num_tokens_per_lora, self.lora_token_start_loc = z(L + 1), z(L + 2)
            self.no_lora_flag_cpu = torch.tensor([False])
            self.num_active_loras_cpu = torch.tensor([0], dtype=torch.int32)
            self.captured_lora_counts = [1, 2, 4, 7]

    def never(self, t):
        raise AssertionError("fell back to vLLM's own code")

    hook = segment_index_prepare(never)
    m, ref = Meta(), oseg.SegmentIndex(L, max_m)
    g = torch.Generator().manual_seed(5)
    batches = [torch.randint(-1, L, (40,), generator=g, dtype=torch.int32), torch.full((17,), -1, dtype=torch.int32),
               torch.full((9,), 3, dtype=torch.int32), torch.arange(48, dtype=torch.int32) % L]
    want_active = [7, 0, 1, 7]                                  # unique ids ("-1" included), rounded up to a captured count
    for t, active in zip(batches, want_active):
        hook(m, t.cuda())
        ref.prepare(t)
        n = t.numel()
        for have, want in ((m.token_lora_mapping[:n], ref.tok[:n]), (m.token_indices_sorted_by_lora_ids[:n], ref.srt[:n]),
                           (m.num_tokens_per_lora, ref.seg_n), (m.lora_token_start_loc, ref.seg_start),
                           (m.active_lora_ids, ref.seg_ids)):
            assert torch.equal(have.cpu(), want)
        assert bool(m.no_lora_flag_cpu[0]) == bool((t == -1).all()) and int(m.num_active_loras_cpu[0]) == active


def test_quant_codes_and_scales_bit_exact_golden(golden):
    """K1's codes and scales on the fixture the reference's own rule produced (edge rows: zeros, floor, ties, large)."""
    g = golden("fp8_quant")
    x = bf16(g["x"])
    M, K = x.shape
    d = _case(K, (128,), 16, 2, M)
    op = build_fp8_op(d, max_m=M)
    ids = torch.full((M,), -1, dtype=torch.int32)
    idx = make_index(ids, 2, M)
    op(x.cuda(), device_meta(idx, M), gemm=False)
    torch.cuda.synchronize()
    assert torch.equal(u8(op.scratch.xq(M, K)).cpu(), t(g["codes"]))
    assert torch.equal(op.scratch.sx(M).cpu().view(torch.int32), t(g["sx"]).view(torch.int32))


@pytest.mark.parametrize("K,widths,R,L,M,kind", [
    (4096, (4096,), 16, 4, 16, "mixed"),                       # configuration 0
    (64, (32, 16, 16), 16, 4, 21, "mixed"),
    (96, (64,), 32, 3, 5, "mixed"),
    (64, (32, 32), 16, 5, 13, "none"),
    (256, (128, 64), 64, 8, 40, "single"),
    (64, (32,), 128, 2, 24, "padded"),
    (128, (32, 16, 16, 32), 16, 3, 24, "padded"),              # four slices
    (512, (256, 128), 64, 32, 32, "all32"),
    (1024, (384,), 64, 6, 77, "mixed"),                        # M > 64: 128-token tile, partial N tile
    (256, (128,), 256, 3, 9, "mixed"),                         # rank 256: four rank chunks
    (512, (256, 512), 64, 8, 300, "mixed"),                    # > 128 tokens, widths in 256s: the 256 x 256 prefill GEMM
    (1024, (768,), 128, 3, 200, "padded"),                     # ... with two rank chunks and padded metadata
    (384, (512, 256, 256), 64, 40, 517, "all32"),              # ... three token tiles, more tenants than a block's width
    (4096, (4096,), 64, 32, 160, "mixed"),                     # a shape with swept decode rows in the tile table, at a prefill size
])
def test_fused_projection_matches_oracle(K, widths, R, L, M, kind):
    torch.manual_seed(1)
    d = _case(K, widths, R, L, M, seed=K + M)
    max_m = max(96, M + 3)
    op = build_fp8_op(d, max_m=max_m)
    idx = oseg.SegmentIndex(L, max_m)
    g = torch.Generator().manual_seed(7)
    # a previous, larger adapter batch leaves its state behind (stale entries)
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
    else:   # padded: metadata for the first M-5 tokens, poisoned stale entries beyond
        ids = torch.randint(-1, L, (M,), generator=g, dtype=torch.int32)
        ids[0] = 0
        idx.srt[M - 5:M] = 10 ** 6
        idx.tok[M - 5:M] = L - 1
        idx.prepare(ids[: M - 5])
        ids[M - 5:] = -1
    meta_cpu = idx.args(M)
    eff = oseg.effective_token_lora(M, *meta_cpu)
    assert torch.equal(eff, ids)
    x = d["x"]
    meta = device_meta(idx, M)
    y = op(x.cuda(), meta)
    torch.cuda.synchronize()
    _check_status(op)
    if M > 128:   # also through the tensor-core shrink and the 256 x 256 GEMM tiles, whatever the library's size rule says
        y_big = op(x.cuda(), meta, cfg={"prefill": 1})
        y_small = op(x.cuda(), meta, cfg={"prefill": 2})
        torch.cuda.synchronize()
        _check_status(op)
        for other in (y_big, y_small):
            assert max_err_ratio(other, oracle_y(d, x, eff)) <= TOL
        y = op(x.cuda(), meta)
        torch.cuda.synchronize()
    # codes / scales bit-exact (kernel rows are sorted positions)
    rows, _ = oseg.resolve_positions(M, *meta_cpu)
    q_ref, sx_ref = ofp8.quant_per_token(x)
    assert torch.equal(u8(op.scratch.xq(M, K)).cpu(), u8(q_ref)[rows])
    assert torch.equal(op.scratch.sx(M).cpu().view(torch.int32), sx_ref[rows].view(torch.int32))
    ref = oracle_y(d, x, eff)
    err = max_err_ratio(y, ref)
    assert err <= TOL, f"max-abs-err / ||y||inf = {err:.3e}"
    # relative L2 as the reference's own tests measure it (< 1e-2)
    rel = float((y.float().cpu() - ref).norm() / ref.norm())
    assert rel < 1e-2, rel
    # serialized launch (no PDL attribute) and a repeat launch are bitwise identical
    y2 = op(x.cuda(), meta, pdl=False)
    y3 = op(x.cuda(), meta)
    torch.cuda.synchronize()
    assert torch.equal(y, y2) and torch.equal(y, y3)
    if M <= 32:
        # the one-kernel form of the chain: same codes, same output bits, twice in a row (its work counters clear themselves)
        op.scratch.xq(M, K).zero_()
        y4 = op(x.cuda(), meta, cfg={"fused": 1})
        y5 = op(x.cuda(), meta, cfg={"fused": 1})
        torch.cuda.synchronize()
        assert torch.equal(y, y4) and torch.equal(y, y5)
        assert torch.equal(u8(op.scratch.xq(M, K)).cpu(), u8(q_ref)[rows])
    counters = op.scratch.region("counters", 4 * (4096 + 16)).view(torch.int32)
    assert int(counters.abs().sum()) == 0
    _check_status(op)


@pytest.mark.parametrize("split1,split2,tn,stages", [(1, 1, 0, 2), (3, 2, 32, 3), (8, 4, 0, 0), (2, 8, 64, 5)])
def test_tile_variants_agree(split1, split2, tn, stages):
    d = _case(2048, (256, 128, 128), 32, 6, 19, seed=3)
    op = build_fp8_op(d, max_m=64)
    idx = make_index(d["ids"], 6, 64)
    meta = device_meta(idx, 19)
    x = d["x"].cuda()
    y = op(x, meta, cfg={"split1": split1, "split2": split2, "tn": tn, "stages": stages})
    torch.cuda.synchronize()
    _check_status(op)
    ref = oracle_y(d, d["x"], d["ids"])
    assert max_err_ratio(y, ref) <= TOL


def test_golden_projection_cases(golden):
    """The CUDA path on the inputs the reference itself was run on (tests/golden/fp8_projection.npz)."""
    g = golden("fp8_projection")
    for ci in range(int(g["n_cases"])):
        p = f"c{ci}_"
        widths = tuple(int(v) for v in g[p + "widths"])
        S = len(widths)
        L, R, K = int(g[p + "L"]), int(g[p + "R"]), int(g[p + "K"])
        d = {"w_q": e4m3(g[p + "w_q"]), "s_w": t(g[p + "s_w"]), "widths": widths,
             "a_stacked": tuple(bf16(g[p + f"a{s}"]) for s in range(S)),
             "b_stacked": tuple(bf16(g[p + f"b{s}"]) for s in range(S))}
        x, tok = bf16(g[p + "x"]), t(g[p + "tok"])
        M = x.shape[0]
        op = build_fp8_op(d, max_m=64)
        idx = make_index(tok, L, 64)
        y = op(x.cuda(), device_meta(idx, M))
        torch.cuda.synchronize()
        _check_status(op)
        assert max_err_ratio(y, t(g[p + "y"])) <= TOL


def test_rejects_bad_arguments_before_launch():
    from onebase_b200 import _lib
    d = _case(128, (128,), 16, 2, 4)
    op = build_fp8_op(d, max_m=8)
    idx = make_index(d["ids"], 2, 8)
    meta = device_meta(idx, 4)
    with pytest.raises(_lib.ObError) as e:
        op(d["x"].cuda(), meta, cfg={"tn": 24})
    assert e.value.status == -5
    with pytest.raises(_lib.ObError) as e:
        op(torch.zeros(9, 128, dtype=torch.bfloat16, device="cuda"), device_meta(make_index(torch.zeros(9, dtype=torch.int32), 2, 16), 9))
    assert e.value.status == -7
    torch.cuda.synchronize()
    _check_status(op)


@pytest.mark.parametrize("fmt", ["fp8", "nvfp4"])
def test_stored_adapter_formats_golden(golden, fmt):
    """FP8- / NVFP4-stored adapters: the device copies are bit-identical to the ones the reference's AdapterStore made, and
    the outputs match the reference run on the dequantized adapters (tests/golden/fp8_projection.npz)."""
    g = golden("fp8_projection")
    for ci in range(int(g["n_cases"])):
        p = f"c{ci}_"
        widths = tuple(int(v) for v in g[p + "widths"])
        S = len(widths)
        L = int(g[p + "L"])
        d = {"w_q": e4m3(g[p + "w_q"]), "s_w": t(g[p + "s_w"]), "widths": widths,
             "a_stacked": tuple(bf16(g[p + f"a{s}"]) for s in range(S)),
             "b_stacked": tuple(bf16(g[p + f"b{s}"]) for s in range(S))}
        x, tok = bf16(g[p + "x"]), t(g[p + "tok"])
        M = x.shape[0]
        op = build_fp8_op(d, max_m=64, lora_fp8=fmt == "fp8", lora_fp4=fmt == "nvfp4")
        for s in range(S):
            for have, name in ((op.store.a_q[s], "aq"), (op.store.a_s[s], "as"), (op.store.b_q[s], "bq"), (op.store.b_s[s], "bs")):
                want = t(g[p + f"{fmt}_{name}{s}"])
                assert torch.equal(have.cpu().view(want.dtype) if have.element_size() == want.element_size() else have.cpu(), want), (ci, fmt, name, s)
        if fmt == "nvfp4":
            assert torch.equal(op.store.ag.cpu(), t(g[p + "nvfp4_ag"])) and torch.equal(op.store.bg.cpu(), t(g[p + "nvfp4_bg"]))
        idx = make_index(tok, L, 64)
        y = op(x.cuda(), device_meta(idx, M))
        torch.cuda.synchronize()
        _check_status(op)
        want_y = t(g[p + f"{fmt}_y"])
        assert max_err_ratio(y, want_y) <= TOL, (ci, fmt, max_err_ratio(y, want_y))
        assert float((y.float().cpu() - want_y).norm() / want_y.norm()) < 1e-2


@pytest.mark.parametrize("fmt", ["fp8", "nvfp4"])
@pytest.mark.parametrize("M", [1, 24])
def test_stored_adapters_any_ring_depth_long_k(fmt, M):
    """Stored adapters with a long K and few expand steps: the weight ring runs many slots ahead of the warps that
    dequantize the B tiles, whatever the ring depth (3 and 5 slots included) and the K split."""
    d = _case(4096, (256, 128), 32, 4, M, seed=31, ids_low=0)
    op = build_fp8_op(d, max_m=32, lora_fp8=fmt == "fp8", lora_fp4=fmt == "nvfp4")
    op.wait_ms = 200
    idx = make_index(d["ids"], 4, 32)
    meta = device_meta(idx, M)
    x = d["x"].cuda()
    ref = op(x, meta, cfg={"split2": 1, "stages": 4}).clone()
    torch.cuda.synchronize()
    _check_status(op)
    for split2 in (1, 2, 4):
        for stages in (2, 3, 5, 6):
            y = op(x, meta, cfg={"split2": split2, "stages": stages})
            torch.cuda.synchronize()
            _check_status(op)
            assert max_err_ratio(y, ref.float().cpu()) <= 8e-3, (fmt, M, split2, stages)   # one bf16 ulp: the K split moves the fp32 sum


def test_released_slots_serve_from_the_copies_alone():
    """After release(), vLLM writes every adapter through one staging slot and requantize(index) files it under its slot
    (reference: tests/test_release_slots.py): the outputs equal those of the fully populated bf16 slots' copies."""
    d = _case(512, (256, 128), 32, 4, 24, seed=9)
    full = build_fp8_op(d, max_m=32, lora_fp8=True)
    a_stage = tuple(torch.zeros_like(t_[:1]).cuda() for t_ in d["a_stacked"])
    b_stage = tuple(torch.zeros_like(t_[:1]).cuda() for t_ in d["b_stacked"])
    rel = build_fp8_op(d, max_m=32, lora_fp8=True)
    rel.release(a_stage, b_stage)
    for slot in (2, 0, 3, 1):                                   # slots written in any order through the staging slot
        for s in range(2):
            a_stage[s][0].copy_(d["a_stacked"][s][slot])
            b_stage[s][0].copy_(d["b_stacked"][s][slot])
        rel.requantize(slot)
    for s in range(2):
        assert torch.equal(rel.store.a_q[s].view(torch.uint8), full.store.a_q[s].view(torch.uint8))
        assert torch.equal(rel.store.b_s[s], full.store.b_s[s])
    idx = make_index(d["ids"], 4, 32)
    meta = device_meta(idx, 24)
    x = d["x"].cuda()
    assert torch.equal(rel(x, meta), full(x, meta))


def test_large_batch_three_token_tiles():
    """M = 600: 256-token tiles (three of them), Zipf-distributed contiguous requests, the shrink's 4-position passes."""
    d = _case(1024, (256, 128), 32, 8, 600, seed=21)
    ids = configs.zipf_request_ids(600, 8, seed=4, mean_len=40)
    ids[100:130] = -1
    op = build_fp8_op(d, max_m=600)
    idx = make_index(ids, 8, 600)
    y = op(d["x"].cuda(), device_meta(idx, 600))
    torch.cuda.synchronize()
    _check_status(op)
    rows, _ = oseg.resolve_positions(600, *idx.args(600))
    q_ref, sx_ref = ofp8.quant_per_token(d["x"])
    assert torch.equal(u8(op.scratch.xq(600, 1024)).cpu(), u8(q_ref)[rows])
    A, B = ofp8.stack_slices(d["a_stacked"], d["b_stacked"])
    ref = ofp8.fused_projection(d["x"], ids, d["w_q"], d["s_w"], A, B, d["widths"])
    assert max_err_ratio(y, ref) <= TOL
