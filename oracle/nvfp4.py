"""Oracle (test infrastructure, CPU torch): the NVFP4 side of the path (e2m1 codes, one ue4m3 scale per 16 elements,
one fp32 global scale per tensor).

Follows the reference's torch recipe, which is vLLM's `scaled_fp4_quant` recipe with exact reciprocals:
  * quantizer ...................... lowbit_lora/kernels/nvfp4_lora_vllm.py:361-376 (`nvfp4_quant_torch`)
  * stacked adapters ............... lowbit_lora/kernels/nvfp4_lora_vllm.py:379-397 (`nvfp4_quant_batched`)
  * dequantizer .................... lowbit_lora/kernels/nvfp4_lora_vllm.py:400-407 (`nvfp4_dequant_torch`)
  * global scale ................... lowbit_lora/kernels/nvfp4_lora_vllm.py:410-412 (`global_scale_for`)
  * e2m1 rounding thresholds / ties  lowbit_lora/kernels/nvfp4_lora_vllm.py:70-76; value table :56,79-85
  * fused projection, fp32 ......... lowbit_lora/kernels/nvfp4_lora_vllm.py:633-649 (`reference`)
Packing: two codes per byte along the quantized axis, element 2i in the low nibble (:113-115, :374-375).
"""
from __future__ import annotations

import torch

from oracle.fp8 import lora_term

E2M1_MAX = 6.0
E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
BLOCK = 16


def global_scale_for(t: torch.Tensor) -> float:
    """The multiplier that maps the tensor's amax to 448 * 6 (ModelOpt's per-tensor global scale)."""
    return float(448.0 * E2M1_MAX / t.abs().amax().clamp_min(1e-12))


def e2m1_codes(v: torch.Tensor) -> torch.Tensor:
    """fp32 -> 4-bit code (bit 3 = sign), round-to-nearest-even on the grid {0,.5,1,1.5,2,3,4,6}, saturating at 6.
    The midpoints .25, 1.25, 2.5, 5 round down on a tie (strict >) and .75, 1.75, 3.5 round up (>=): ties to even."""
    a = v.abs()
    mag = ((a > 0.25).to(torch.int32) + (a >= 0.75).to(torch.int32) + (a > 1.25).to(torch.int32)
           + (a >= 1.75).to(torch.int32) + (a > 2.5).to(torch.int32) + (a >= 3.5).to(torch.int32)
           + (a > 5.0).to(torch.int32))
    return mag + 8 * (v < 0).to(torch.int32)


def _quant_blocks(xb: torch.Tensor, gs: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """xb [..., nblk, 16] fp32, gs broadcastable fp32 -> (codes int32 [..., nblk, 16], block scales e4m3 [..., nblk, 1]).
    sf = e4m3_rn(min(gs * (blockmax * (1/6)), 448)); out_scale = sf != 0 ? 1 / (sf * (1 / gs)) : 0; code = e2m1(x * out_scale).
    All in fp32 with IEEE reciprocals."""
    vmax = xb.abs().amax(dim=-1, keepdim=True)
    sf = (gs * (vmax * (1.0 / E2M1_MAX))).clamp(max=448.0).to(torch.float8_e4m3fn)
    sff = sf.to(torch.float32)
    out_scale = torch.where(sff != 0, 1.0 / (sff * (1.0 / gs)), torch.zeros_like(sff))
    return e2m1_codes(xb * out_scale), sf


def _pack(codes: torch.Tensor) -> torch.Tensor:
    pair = codes.reshape(*codes.shape[:-1], codes.shape[-1] // 2, 2)
    return (pair[..., 0] | (pair[..., 1] << 4)).to(torch.uint8)


def quant(x: torch.Tensor, global_scale: float) -> tuple[torch.Tensor, torch.Tensor]:
    """x [m, k] -> (packed codes [m, k/2] uint8, block scales [m, k/16] float8_e4m3fn)."""
    m, k = x.shape
    gs = torch.tensor(global_scale, dtype=torch.float32)
    codes, sf = _quant_blocks(x.to(torch.float32).reshape(m, k // BLOCK, BLOCK), gs)
    return _pack(codes.reshape(m, k)), sf.reshape(m, k // BLOCK)


def quant_stack(t: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """t [l, rows, cols] -> (packed [l, rows, cols/2], block scales [l, rows, cols/16], inverse global scales [l]);
    one global scale 448*6/amax per matrix; value = code * block_scale * inv_global."""
    l, rows, cols = t.shape
    tf = t.to(torch.float32)
    gs = (448.0 * E2M1_MAX / tf.abs().amax(dim=(1, 2)).clamp_min(1e-12)).to(torch.float32)
    codes, sf = _quant_blocks(tf.reshape(l, rows, cols // BLOCK, BLOCK), gs.view(l, 1, 1, 1))
    return _pack(codes.reshape(l, rows, cols)), sf.reshape(l, rows, cols // BLOCK), (1.0 / gs).to(torch.float32)


def unpack_values(packed: torch.Tensor) -> torch.Tensor:
    """packed [..., k/2] uint8 -> e2m1 values fp32 [..., k]."""
    p = packed.to(torch.int64)
    codes = torch.stack([p & 15, (p >> 4) & 15], dim=-1).reshape(*p.shape[:-1], 2 * p.shape[-1])
    lut = torch.tensor(E2M1_VALUES, dtype=torch.float32)
    return lut[codes & 7] * torch.where((codes & 8) != 0, -1.0, 1.0)


def dequant(packed: torch.Tensor, sf: torch.Tensor, global_scale: float) -> torch.Tensor:
    """(packed [m, k/2], scales [m, k/16]) -> fp32 [m, k] = value * block_scale / global_scale."""
    v = unpack_values(packed)
    m, k = v.shape
    return (v.reshape(m, k // BLOCK, BLOCK) * sf.to(torch.float32).reshape(m, k // BLOCK, 1)).reshape(m, k) / global_scale


def dequant_stack(packed, sf, inv_global) -> torch.Tensor:
    """Stored adapter stack (quant_stack's outputs) -> fp32 [l, rows, cols], as the reference's
    `AdapterStore.dequantized` (lowbit_lora/kernels/adapter_store.py:82-94)."""
    return torch.stack([dequant(packed[i], sf[i], 1.0) * inv_global[i] for i in range(packed.shape[0])])


def fused_projection(x, token_lora, w_q, w_sf, w_global, x_global, a, b, widths, xq=None, xsf=None) -> torch.Tensor:
    """fp32 reference of y = dequant(x_q) @ dequant(W)^T + LoRA on the bf16 x (nvfp4_lora_vllm.py:633-649)."""
    if xq is None:
        xq, xsf = quant(x, x_global)
    base = dequant(xq, xsf, x_global) @ dequant(w_q, w_sf, w_global).t()
    return base + lora_term(x, token_lora, a, b, widths, 1.0)
