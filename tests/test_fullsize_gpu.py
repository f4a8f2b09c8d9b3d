"""Parity at the benchmark's full sizes: the four Qwen3-8B projections (FP8 base, 32 tenants of rank 64) at a decode and
a prefill batch, checked against the CPU oracle on a SAMPLE of output features.

Output feature n of the fused projection depends only on row n of W and row n of every tenant's B, so the oracle runs
the same batch on a reduced layer that keeps just the sampled rows (a few dozen per slice, spread over the first, the
last and random tiles); the kernels run the full layer.  The quantization codes and scales are compared in full.
Inputs are drawn on the device from a seeded generator and copied to the host for the oracle.
"""
import pytest
import torch

from oracle import fp8 as ofp8
from oracle import segments as oseg
from helpers import device_meta, max_err_ratio

pytestmark = pytest.mark.gpu

PROJECTIONS = {"qkv": (4096, (4096, 1024, 1024)), "o": (4096, (4096,)), "gate_up": (4096, (12288, 12288)),
               "down": (12288, (4096,))}
L, R = 32, 64
TOL = 2e-2   # max-abs-err / ||y||inf, the bound the reference's own tests hold the fused path to


def _layer(name, seed):
    from onebase_b200.kernels.fp8_lora_vllm import VllmFusedFP8LoRA
    K, widths = PROJECTIONS[name]
    N = sum(widths)
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.02
    s_w = (w.abs().max() / 448.0).reshape(1).float()
    w_q = (w / s_w).to(torch.float8_e4m3fn)
    del w
    a_st = tuple(((torch.rand(L, 1, R, K, device="cuda", generator=g) * 2 - 1) / K ** 0.5).to(torch.bfloat16) for _ in widths)
    b_st = tuple((torch.randn(L, 1, n, R, device="cuda", generator=g) * 0.01).to(torch.bfloat16) for n in widths)
    return K, widths, N, w_q, s_w, a_st, b_st, g, VllmFusedFP8LoRA


def _sample_rows(widths, g_cpu, per_slice=48):
    """Per slice: the first and last 8 rows plus random ones -> (global row indices, per-slice local indices)."""
    glob, local, off = [], [], 0
    for n in widths:
        pick = torch.cat([torch.arange(8), torch.arange(n - 8, n), torch.randint(0, n, (per_slice - 16,), generator=g_cpu)])
        pick = torch.unique(pick)
        local.append(pick)
        glob.append(pick + off)
        off += n
    return torch.cat(glob), local


# M = 1000 on gate_up gives every CTA pair of the prefill GEMM several tiles; M = 2500 on down does the same for the
# single-CTA form (the long-K projection keeps it): the persistent loops' hand-overs between tiles are exercised.
@pytest.mark.parametrize("name,M", [(n, m) for m in (32, 300) for n in PROJECTIONS] + [("gate_up", 1000), ("down", 2500)])
def test_full_size_projection_sampled_features(name, M):
    K, widths, N, w_q, s_w, a_st, b_st, g, Op = _layer(name, seed=len(name) * 100 + M)
    op = Op(w_q, s_w, a_st, b_st, max_m=M)
    g_cpu = torch.Generator().manual_seed(M)
    if M <= 32:
        ids = torch.randint(-1, L, (M,), generator=g_cpu, dtype=torch.int32)          # mixed decode batch, some tokens bare
    else:   # prefill: contiguous requests of random length, each with its own tenant (or none)
        ids = torch.empty(M, dtype=torch.int32)
        p = 0
        while p < M:
            n = int(torch.randint(5, 90, (1,), generator=g_cpu))
            ids[p:p + n] = int(torch.randint(-1, L, (1,), generator=g_cpu))
            p += n
    idx = oseg.SegmentIndex(L, M)
    idx.prepare(ids)
    meta = device_meta(idx, M)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    cfg = {"prefill": 1} if M > 32 else None               # prefill: the tensor-core shrink and the 256 x 256 GEMM tiles
    y = op(x, meta, cfg=cfg)
    y2 = op(x, meta, cfg=cfg)
    torch.cuda.synchronize()
    assert op.scratch.status()[0] == 0, op.scratch.status()[:8]
    assert torch.equal(y, y2)
    # quantization: every code and scale, against the oracle, at the kernel's adapter-sorted positions
    x_cpu = x.cpu()
    rows, _ = oseg.resolve_positions(M, *idx.args(M))
    q_ref, sx_ref = ofp8.quant_per_token(x_cpu)
    assert torch.equal(op.scratch.xq(M, K).view(torch.uint8).cpu(), q_ref.view(torch.uint8)[rows])
    assert torch.equal(op.scratch.sx(M).cpu().view(torch.int32), sx_ref[rows].view(torch.int32))
    # outputs: the sampled features through the oracle on the reduced layer
    sel, local = _sample_rows(widths, g_cpu)
    a_red = tuple(t.cpu() for t in a_st)
    b_red = tuple(t[:, :, loc.to(t.device)].cpu() for t, loc in zip(b_st, local))
    A, B = ofp8.stack_slices(a_red, b_red)
    ref = ofp8.fused_projection(x_cpu, ids, w_q.view(torch.uint8)[sel.cuda()].cpu().view(torch.float8_e4m3fn), s_w.cpu(), A, B, [len(loc) for loc in local])
    got = y[:, sel.cuda()]
    err = max_err_ratio(got, ref)
    assert err <= TOL, f"{name} M={M}: max-abs-err / ||y||inf = {err:.3e}"
    rel = float((got.float().cpu() - ref).norm() / ref.norm())
    assert rel < 1e-2, rel


@pytest.mark.parametrize("name", ["qkv", "down"])
@pytest.mark.parametrize("M,cfg", [(32, None), (300, None), (300, {"prefill": 1}), (1000, None)])
def test_full_size_nvfp4_projection_sampled_features(name, M, cfg):
    """The same check with an NVFP4 base.  The weight codes and block scales are random (every nibble and every scale byte
    of 0.5..1.9 is a valid weight); both sides consume the same bytes, so parity does not depend on how they were made.
    M = 300 runs the 64-token tiles by default and the large-tile prefill GEMM (128 features x 256 tokens) when asked;
    M = 1000 takes the large tiles by the library's own rule."""
    from onebase_b200.kernels.nvfp4_lora_vllm import VllmFusedNVFP4LoRA
    from oracle import nvfp4 as on4
    K, widths = PROJECTIONS[name]
    N = sum(widths)
    g = torch.Generator(device="cuda").manual_seed(7 * len(name) + M)
    w_q4 = torch.randint(0, 256, (N, K // 2), device="cuda", generator=g, dtype=torch.uint8)
    w_sf = torch.randint(0x30, 0x40, (N, K // 16), device="cuda", generator=g, dtype=torch.uint8).view(torch.float8_e4m3fn)
    a_st = tuple(((torch.rand(L, 1, R, K, device="cuda", generator=g) * 2 - 1) / K ** 0.5).to(torch.bfloat16) for _ in widths)
    b_st = tuple((torch.randn(L, 1, n, R, device="cuda", generator=g) * 0.01).to(torch.bfloat16) for n in widths)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    x_cpu = x.cpu()
    w_global, x_global = 2688.0 / 0.1, on4.global_scale_for(x_cpu.float())
    op = VllmFusedNVFP4LoRA(w_q4, w_sf, w_global, x_global, a_st, b_st, max_m=M)
    g_cpu = torch.Generator().manual_seed(M + 1)
    ids = torch.randint(-1, L, (M,), generator=g_cpu, dtype=torch.int32)
    if M > 32:
        ids = torch.sort(ids).values[torch.randperm(M, generator=g_cpu)]              # any order: the kernels sort by tenant
    idx = oseg.SegmentIndex(L, M)
    idx.prepare(ids)
    meta = device_meta(idx, M)
    y = op(x, meta, cfg=cfg)
    y2 = op(x, meta, cfg=cfg)
    torch.cuda.synchronize()
    assert op.scratch.status()[0] == 0, op.scratch.status()[:8]
    assert torch.equal(y, y2)
    big = op.resolved_tile(M, cfg)["prefill"] == 1
    assert big == (cfg is not None or M >= 1000)
    rows, _ = oseg.resolve_positions(M, *idx.args(M))
    q_ref, sf_ref = on4.quant(x_cpu, x_global)
    xq, xsf = op.codes(M, tn=256 if big else None)
    assert torch.equal(xq.cpu(), q_ref[rows])
    assert torch.equal(xsf.view(torch.uint8).cpu(), sf_ref.view(torch.uint8)[rows])
    sel, local = _sample_rows(widths, g_cpu)
    a_red = tuple(t.cpu() for t in a_st)
    b_red = tuple(t[:, :, loc.to(t.device)].cpu() for t, loc in zip(b_st, local))
    A, B = ofp8.stack_slices(a_red, b_red)
    ref = on4.fused_projection(x_cpu, ids, w_q4[sel.cuda()].cpu(), w_sf.view(torch.uint8)[sel.cuda()].cpu().view(torch.float8_e4m3fn),
                               w_global, x_global, A, B, [len(loc) for loc in local])
    got = y[:, sel.cuda()]
    err = max_err_ratio(got, ref)
    assert err <= TOL, f"{name} M={M}: max-abs-err / ||y||inf = {err:.3e}"


def _zipf_ids(M, seed=0, exponent=1.1):
    """Contiguous requests whose sizes follow Zipf(1.1) over the L tenants, in a seeded tenant order (the prefill batches
    of the NVFP4 configuration)."""
    g = torch.Generator().manual_seed(seed)
    share = 1.0 / torch.arange(1, L + 1, dtype=torch.float64) ** exponent
    exact = share / share.sum() * M
    counts = exact.floor().long()
    order = torch.argsort(exact - counts, descending=True)
    counts[order[: M - int(counts.sum())]] += 1
    return torch.repeat_interleave(torch.randperm(L, generator=g).to(torch.int32), counts)


def _dequantized_like_the_store(stacked, fmt):
    """What the kernels see of adapters stored as `fmt` (the reference's AdapterStore.dequantized,
    lowbit_lora/kernels/adapter_store.py:82-94), per slice as fp32 [L, rows, cols]."""
    from oracle import nvfp4 as on4
    out = []
    for t in stacked:
        m = t[:, 0].cpu()
        if fmt == "bf16":
            out.append(m.float())
        elif fmt == "fp8":
            codes, scale = ofp8.store_rows_fp8(m)
            out.append(codes.float() * scale[..., None])
        else:
            out.append(on4.dequant_stack(*on4.quant_stack(m)))
    return out


@pytest.mark.parametrize("adapters", ["bf16", "fp8", "nvfp4"])
@pytest.mark.parametrize("M", [512, 2048])
def test_config2_nvfp4_base_stored_adapters_zipf_prefill(adapters, M):
    """Configuration 2 at full size: NVFP4 base, adapters stored as bf16 / FP8 / NVFP4, a prefill batch split across the
    32 tenants by Zipf(1.1), under the library's own tile rule; the o projection (4096 -> 4096) on sampled features."""
    from onebase_b200.kernels.nvfp4_lora_vllm import VllmFusedNVFP4LoRA
    from oracle import nvfp4 as on4
    K, widths = PROJECTIONS["o"]
    N = sum(widths)
    g = torch.Generator(device="cuda").manual_seed(1000 + M)
    w_q4 = torch.randint(0, 256, (N, K // 2), device="cuda", generator=g, dtype=torch.uint8)
    w_sf = torch.randint(0x30, 0x40, (N, K // 16), device="cuda", generator=g, dtype=torch.uint8).view(torch.float8_e4m3fn)
    a_st = tuple(((torch.rand(L, 1, R, K, device="cuda", generator=g) * 2 - 1) / K ** 0.5).to(torch.bfloat16) for _ in widths)
    b_st = tuple((torch.randn(L, 1, n, R, device="cuda", generator=g) * 0.01).to(torch.bfloat16) for n in widths)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    x_cpu = x.cpu()
    w_global, x_global = 2688.0 / 0.1, on4.global_scale_for(x_cpu.float())
    op = VllmFusedNVFP4LoRA(w_q4, w_sf, w_global, x_global, a_st, b_st, max_m=M, lora_fmt=adapters)
    ids = _zipf_ids(M, seed=M)
    idx = oseg.SegmentIndex(L, M)
    idx.prepare(ids)
    meta = device_meta(idx, M)
    y = op(x, meta)
    y2 = op(x, meta)
    torch.cuda.synchronize()
    assert op.scratch.status()[0] == 0, op.scratch.status()[:8]
    assert torch.equal(y, y2)
    g_cpu = torch.Generator().manual_seed(M)
    sel, local = _sample_rows(widths, g_cpu)
    a_deq = _dequantized_like_the_store(a_st, adapters)
    b_deq = [t[:, loc] for t, loc in zip(_dequantized_like_the_store(b_st, adapters), local)]
    A, B = torch.cat(a_deq, 1), torch.cat(b_deq, 1)
    ref = on4.fused_projection(x_cpu, ids, w_q4[sel.cuda()].cpu(), w_sf.view(torch.uint8)[sel.cuda()].cpu().view(torch.float8_e4m3fn),
                               w_global, x_global, A, B, [len(loc) for loc in local])
    err = max_err_ratio(y[:, sel.cuda()], ref)
    assert err <= TOL, f"adapters {adapters} M={M}: max-abs-err / ||y||inf = {err:.3e}"


@pytest.mark.parametrize("name,M", [("o", 512), ("gate_up", 2048)])
def test_fp8_base_zipf_prefill_default_rule(name, M):
    """FP8 base, bf16 adapters, Zipf(1.1) prefill batches under the library's OWN rule (no tile override): from 512 tokens
    on both take the tensor-core shrink and the large-tile kernels (o at M = 512: 16 pair tiles, most pairs idle)."""
    K, widths, N, w_q, s_w, a_st, b_st, g, Op = _layer(name, seed=31 + M)
    op = Op(w_q, s_w, a_st, b_st, max_m=M)
    ids = _zipf_ids(M, seed=M + 1)
    idx = oseg.SegmentIndex(L, M)
    idx.prepare(ids)
    meta = device_meta(idx, M)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    y = op(x, meta)
    y2 = op(x, meta)
    torch.cuda.synchronize()
    assert op.scratch.status()[0] == 0, op.scratch.status()[:8]
    assert torch.equal(y, y2)
    assert op.resolved_tile(M)["prefill"] == 1
    x_cpu = x.cpu()
    rows, _ = oseg.resolve_positions(M, *idx.args(M))
    q_ref, sx_ref = ofp8.quant_per_token(x_cpu)
    assert torch.equal(op.scratch.xq(M, K).view(torch.uint8).cpu(), q_ref.view(torch.uint8)[rows])
    assert torch.equal(op.scratch.sx(M).cpu().view(torch.int32), sx_ref[rows].view(torch.int32))
    g_cpu = torch.Generator().manual_seed(M)
    sel, local = _sample_rows(widths, g_cpu)
    a_red = tuple(t.cpu() for t in a_st)
    b_red = tuple(t[:, :, loc.to(t.device)].cpu() for t, loc in zip(b_st, local))
    A, B = ofp8.stack_slices(a_red, b_red)
    ref = ofp8.fused_projection(x_cpu, ids, w_q.view(torch.uint8)[sel.cuda()].cpu().view(torch.float8_e4m3fn), s_w.cpu(), A, B, [len(loc) for loc in local])
    err = max_err_ratio(y[:, sel.cuda()], ref)
    assert err <= TOL, f"{name} M={M}: max-abs-err / ||y||inf = {err:.3e}"
