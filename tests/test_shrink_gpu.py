"""The shrink's own output against the oracle's h = x A_l^T, not just through y: K1's fp32 split-K partials `hp`
(decode, warp-level shrink) and the tensor-core shrink's finished bf16 `hb` (prefill), read back from the workspace at
their adapter-sorted positions.  The reference computes h per token in fp32 and rounds it to bf16 once
(lowbit_lora/kernels/fp8_lora_multi.py:303-309)."""
from __future__ import annotations

import pytest
import torch

from helpers import build_fp8_op, device_meta, make_index
from oracle import configs, fp8 as ofp8, segments as oseg

pytestmark = pytest.mark.gpu


def _oracle_h(d, ids):
    """fp32 h [M, S, R] of every token with an adapter (zeros for tokens without)."""
    A, _ = ofp8.stack_slices(d["a_stacked"], d["b_stacked"])
    S, R = len(d["widths"]), d["R"]
    M = d["x"].shape[0]
    h = torch.zeros(M, S, R)
    xf = d["x"].float()
    for m in range(M):
        l = int(ids[m])
        if l >= 0:
            h[m] = (xf[m] @ A[l].float().t()).view(S, R)
    return h


@pytest.mark.parametrize("K,widths,R,L,M,cfg", [
    (4096, (4096, 1024, 1024), 64, 32, 32, None),              # decode, the benchmark's qkv shape
    (4096, (4096, 1024, 1024), 64, 32, 32, {"stream": 1}),     # ... and the looped one-CTA-per-SM grid beside the persistent GEMM
    (1024, (512,), 16, 3, 7, {"split1": 3}),
    (12288, (256,), 64, 8, 1, None),
])
def test_decode_shrink_partials_sum_to_oracle_h(K, widths, R, L, M, cfg):
    d = configs.with_fp8_base(configs.draw(K, widths, R, L, M, seed=K + M, ids_low=-1))
    op = build_fp8_op(d, max_m=32)
    idx = make_index(d["ids"], L, 32)
    op.scratch.region("hp", op.scratch.sizes["hp"]).zero_()
    op(d["x"].cuda(), device_meta(idx, M), cfg=cfg, gemm=False)
    torch.cuda.synchronize()
    assert op.scratch.status()[0] == 0
    hp = op.shrink_partials(M, cfg).double().sum(0).float().cpu()        # [S, max_m, R] at sorted positions
    rows, eff = oseg.resolve_positions(M, *idx.args(M))
    want = _oracle_h(d, d["ids"])[rows]                                   # position p holds token rows[p]
    got = hp[:, :M].permute(1, 0, 2)
    has = (d["ids"][rows] >= 0)
    assert has.any() or M == 1
    err = float((got[has] - want[has]).abs().max()) if has.any() else 0.0
    scale = float(want.abs().max().clamp_min(1e-30))
    assert err <= 2e-5 * scale + 1e-7, f"max |hp sum - h| = {err:.3e} against ||h||inf = {scale:.3e}"


@pytest.mark.parametrize("K,split1,L", [(1024, 0, 8), (1024, 1, 8), (1024, 2, 8), (4096, 8, 8),
                                         (1024, 0, 32), (1024, 1, 32), (1024, 2, 32), (4096, 8, 32)])
def test_prefill_tensor_core_shrink_h_equals_oracle_h(K, split1, L):
    """split1 = 0: the library's rule (four K splits here: one thread-block cluster that sums over distributed shared
    memory); 1: no split (the accumulator row is the finished h); 2: a cluster of two; 8 (on a longer K): partials through
    the workspace and the arrival counter, the last arriver adds them.  L = 8: one CTA per 128-position tile; L = 32: the
    host expects six or more tenants per tile and deals each tile's tenants out four at a time to CTAs of their own
    (a grid sized by the host's bound, some CTAs without a work item)."""
    widths, R, M = (256, 512), 64, 300
    d = configs.with_fp8_base(configs.draw(K, widths, R, L, M, seed=4, ids_low=-1))
    ids = configs.zipf_request_ids(M, L, seed=6, mean_len=25 if L == 8 else 9)
    ids[40:70] = -1
    op = build_fp8_op(d, max_m=M)
    idx = make_index(ids, L, M)
    cfg = {"prefill": 1, "tn": 128, **({"split1": split1} if split1 else {})}
    op(d["x"].cuda(), device_meta(idx, M), cfg=cfg, gemm=False)   # tensor-core shrink -> finished h
    torch.cuda.synchronize()
    assert op.scratch.status()[0] == 0
    hb = op.scratch.hb(len(widths), R).float().cpu()[:, :M].permute(1, 0, 2)
    rows, _ = oseg.resolve_positions(M, *idx.args(M))
    want = _oracle_h(d, ids)[rows]
    has = ids[rows] >= 0
    got, ref = hb[has], want[has]
    # bf16 of an fp32 sum taken in another order: equal to the oracle's rounding or its neighbour.  `ref` is the unrounded
    # fp32 value, so a neighbour of its rounding lies up to 1.5 bf16 spacings away, and a spacing is at most 2^-7 |ref|.
    # (Elements that are small against their own terms also carry the fp32 sums' reordering error: 2e-5 of |h|inf.)
    ulp = ref.abs().clamp_min(1e-30) * 2.0 ** -7
    slack = 2e-5 * float(ref.abs().max())
    assert bool(((got - ref).abs() <= 1.5 * ulp + slack).all()), float(((got - ref).abs() / (1.5 * ulp + slack)).max())
    assert float((got != ref.to(torch.bfloat16).float()).float().mean()) < 0.02
