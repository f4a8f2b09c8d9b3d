"""Row-parallel projection with sharded adapters (vLLM's RowParallelLinearWithShardedLoRA) on ONE GPU: the ranks of a
tensor-parallel group are run one after the other, and the two exchange steps -- the all-reduce of the fp32 shrink
partials between K1 and K2, and the all-reduce of y -- are done by hand.  Checks the kernels' side of the form: K1 on a K
slice, K2 adding the expand only to the output features whose B rows the rank holds.
"""
import pytest
import torch

from helpers import device_meta, max_err_ratio
from oracle import fp8 as ofp8
from oracle import segments as oseg

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tp,M,K,widths,R,L", [(2, 24, 1024, (512,), 64, 6), (4, 9, 2048, (1024, 512), 32, 4),
                                                (2, 150, 512, (256, 256), 64, 5)])
def test_sharded_adapters_row_parallel_one_gpu(tp, M, K, widths, R, L):
    from onebase_b200 import tp as obtp
    from onebase_b200.kernels.fp8_lora_vllm import VllmFusedFP8LoRA
    g = torch.Generator().manual_seed(tp * 1000 + M)
    N = sum(widths)
    w = torch.randn(N, K, generator=g) * 0.02
    s_w = (w.abs().max() / 448.0).reshape(1).float()
    w_q = (w / s_w).to(torch.float8_e4m3fn)
    a_st = tuple(((torch.rand(L, 1, R, K, generator=g) * 2 - 1) / K ** 0.5).to(torch.bfloat16) for _ in widths)
    b_st = tuple((torch.randn(L, 1, n, R, generator=g) * 0.01).to(torch.bfloat16) for n in widths)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    ids = torch.randint(-1, L, (M,), generator=g, dtype=torch.int32)
    idx = oseg.SegmentIndex(L, M)
    idx.prepare(ids)
    meta = device_meta(idx, M)
    ops, xs = [], []
    for rank in range(tp):
        w_r, a_r, b_r, b_shard = obtp.shard_row_sharded_lora(w_q.view(torch.uint8), a_st, b_st, tp, rank)
        ops.append(VllmFusedFP8LoRA(w_r.view(torch.float8_e4m3fn).cuda(), s_w.cuda(), tuple(t.cuda() for t in a_r),
                                    tuple(t.cuda() for t in b_r), max_m=M, b_shard=b_shard))
        xs.append(obtp.shard_input_row(x, tp, rank).cuda())
    split1 = ops[0].resolved_tile(M)["split1"]
    assert all(op.resolved_tile(M)["split1"] == split1 for op in ops)
    # exchange 1: every rank's shrink partials, summed (what the all-reduce leaves in every rank's workspace)
    total = None
    for op, x_r in zip(ops, xs):
        op(x_r, meta, gemm=False)
        part = op.shrink_partials(M).clone()
        total = part if total is None else total + part
    # exchange 2: the ranks' outputs, summed.  The ranks share one workspace here, so K1 runs again before each K2 and the
    # summed partials are put in its place.
    y = torch.zeros(M, N, dtype=torch.float32, device="cuda")
    for op, x_r in zip(ops, xs):
        op(x_r, meta, gemm=False)
        op.shrink_partials(M).copy_(total)
        y += op(x_r, meta, shrink=False).float()
        assert op.scratch.status()[0] == 0, op.scratch.status()[:8]
    # the oracle of the same form: per-rank quantized base partials, h summed over the ranks' K slices before its bf16 rounding
    ks = K // tp
    ref = torch.zeros(M, N)
    for rank in range(tp):
        xr = x[:, rank * ks:(rank + 1) * ks]
        xq, sx = ofp8.quant_per_token(xr)
        ref += (xq.float() * sx.unsqueeze(1)) @ (w_q[:, rank * ks:(rank + 1) * ks].float() * s_w).t()
    A, B = ofp8.stack_slices(a_st, b_st)
    ref += ofp8.lora_term(x, ids, A, B, list(widths), 1.0)
    err = max_err_ratio(y, ref)
    assert err <= 2e-2, f"max-abs-err / ||y||inf = {err:.3e}"
    assert float((y.cpu() - ref).norm() / ref.norm()) < 1e-2
