"""K1's activation codes and scales byte for byte against vLLM's own CUDA quantizers on the same device tensors:
`ops.scaled_fp8_quant(x, use_per_token_if_dynamic=True)` for the FP8 base and
`ops.scaled_fp4_quant(x, x_global, is_sf_swizzled_layout=False)` for the NVFP4 base in its rcp.approx mode -- the checks
the reference records for every configuration it ships (bench/pdl_k2_bench.py:627-639, bench/nvfp4_check.py:119-125).
Skipped when vLLM's compiled ops cannot be imported."""
from __future__ import annotations

import pytest
import torch

from helpers import build_fp8_op, build_nvfp4_op, device_meta, make_index
from oracle import configs

pytestmark = pytest.mark.gpu


def _vllm_ops():
    try:
        import vllm._custom_ops as ops
        torch.ops._C.dynamic_per_token_scaled_fp8_quant   # noqa: B018 - the compiled extension must be there
        return ops
    except Exception as e:   # noqa: BLE001
        pytest.skip(f"vLLM's compiled quantizers are not importable here: {type(e).__name__}: {e}")


def _activations(M: int, K: int, seed: int) -> torch.Tensor:
    """Rows of the configurations' distribution plus the hard ones: an outlier row, a tiny row, a zero row, exact ties."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    if M >= 4:
        x[1, 7] = 300.0                                        # an outlier sets the row's scale
        x[2] *= 1e-4                                           # scale at the floor
        x[3] = 0.0
    if M >= 6:
        x[4] = torch.randint(-8, 9, (K,), generator=g).float() * 0.25   # values on code boundaries
        x[5, ::2] = 448.0
    return x.to(torch.bfloat16)


@pytest.mark.parametrize("M,K", [(1, 4096), (32, 4096), (32, 12288), (300, 4096)])
def test_fp8_codes_and_scales_equal_vllm(M, K):
    ops = _vllm_ops()
    d = configs.with_fp8_base(configs.draw(K, (128,), 16, 2, M, seed=1))
    x = _activations(M, K, seed=M + K).cuda()
    op = build_fp8_op(d, max_m=M)
    ids = torch.full((M,), -1, dtype=torch.int32)              # no adapter: positions are the token rows themselves
    op(x, device_meta(make_index(ids, 2, M), M), gemm=False)
    q_v, s_v = ops.scaled_fp8_quant(x, use_per_token_if_dynamic=True)
    torch.cuda.synchronize()
    codes = op.scratch.xq(M, K).view(torch.uint8)
    n_codes = int((codes != q_v.view(torch.uint8)).sum())
    n_scales = int((op.scratch.sx(M).view(torch.int32) != s_v.reshape(-1).view(torch.int32)).sum())
    assert n_codes == 0 and n_scales == 0, f"differing from vLLM: {n_codes} of {M * K} codes, {n_scales} of {M} scales"


@pytest.mark.parametrize("M,K", [(1, 4096), (32, 4096), (32, 12288), (300, 4096)])
def test_nvfp4_codes_and_scales_equal_vllm_in_approx_mode(M, K):
    ops = _vllm_ops()
    from oracle import nvfp4 as on4
    d = configs.with_nvfp4_base(configs.draw(K, (128,), 16, 2, M, seed=2))
    xc = _activations(M, K, seed=M + K + 1)
    xc[xc.abs() > 64] = 64.0                                   # keep the static global scale meaningful
    x = xc.cuda()
    d["x_global"] = on4.global_scale_for(xc.float())
    op = build_nvfp4_op(d, max_m=M, rcp_approx=True)
    ids = torch.full((M,), -1, dtype=torch.int32)
    op(x, device_meta(make_index(ids, 2, M), M), gemm=False)
    xg = torch.tensor([d["x_global"]], dtype=torch.float32, device="cuda")
    q_v, sf_v = ops.scaled_fp4_quant(x, xg, is_sf_swizzled_layout=False)
    torch.cuda.synchronize()
    xq, xsf = op.codes(M)
    n_codes = int((xq != q_v.view(torch.uint8)[:, : K // 2]).sum())
    n_scales = int((xsf.view(torch.uint8) != sf_v.view(torch.uint8).reshape(M, -1)[:, : K // 16]).sum())
    assert n_codes == 0 and n_scales == 0, \
        f"differing from vLLM: {n_codes} of {M * K // 2} code bytes, {n_scales} of {M * K // 16} block scales"
