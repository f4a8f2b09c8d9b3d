"""The device-side adapter (re)quantization kernels against the oracle's recipes, bit for bit: FP8 rows (one scale per
row) and NVFP4 matrices (one global per matrix, ue4m3 scale per 16 elements, packed e2m1 codes)."""
import pytest
import torch

from oracle import fp8 as ofp8
from oracle import nvfp4 as on4

pytestmark = pytest.mark.gpu


def _inputs(shape, seed):
    g = torch.Generator().manual_seed(seed)
    t = torch.randn(shape, generator=g) * torch.rand(shape[:-1] + (1,), generator=g) * 3.0
    t[..., 0, :] = 0.0                                          # an all-zero row: floor of the scale, zero codes
    flat = t.reshape(-1, shape[-1])
    flat[1, 3] = 1e4                                            # an outlier that sets its row's (and matrix's) scale
    flat[2, :8] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -2.5])   # e2m1 tie points (before scaling)
    return t.to(torch.bfloat16)


@pytest.mark.parametrize("shape", [(3, 16, 64), (2, 64, 4096), (5, 384, 16), (1, 8, 12288)])
def test_fp8_rows_bit_exact(shape):
    from onebase_b200.kernels.adapter_store import store_rows_fp8
    t = _inputs(shape, seed=sum(shape))
    codes, scale = store_rows_fp8(t.cuda())
    ref_codes, ref_scale = ofp8.store_rows_fp8(t)
    assert torch.equal(scale.cpu().view(torch.int32), ref_scale.view(torch.int32))
    assert torch.equal(codes.cpu().view(torch.uint8), ref_codes.view(torch.uint8))


@pytest.mark.parametrize("shape", [(3, 16, 64), (2, 64, 4096), (5, 384, 16), (32, 64, 1024)])
def test_nvfp4_matrices_bit_exact(shape):
    from onebase_b200.kernels.adapter_store import quant_stack_nvfp4
    t = _inputs(shape, seed=7 + sum(shape))
    packed, sf, inv_g = quant_stack_nvfp4(t.cuda())
    ref_packed, ref_sf, ref_inv = on4.quant_stack(t)
    assert torch.equal(inv_g.cpu().view(torch.int32), ref_inv.view(torch.int32))
    assert torch.equal(sf.cpu().view(torch.uint8), ref_sf.view(torch.uint8))
    assert torch.equal(packed.cpu(), ref_packed)
