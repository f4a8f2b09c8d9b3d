"""Oracle (test infrastructure, CPU torch): the two elementwise ops that sit either side of the fused projection in a
decoder layer and that the kernels can take in -- restated from vLLM's own pure-torch forms (vLLM 0.22; the reference
leaves both to vLLM).

  * `silu_mul`      SiluAndMul.forward_native, vllm/model_executor/layers/activation.py:
                        d = x.shape[-1] // 2;  return F.silu(x[..., :d]) * x[..., d:]
                    on bf16 tensors: silu is evaluated in fp32 and rounded to bf16, the product is one more bf16 rounding.
  * `add_residual`  the first half of RMSNorm.forward_native with a residual, vllm/model_executor/layers/layernorm.py:
                        x = x.to(float32) + residual.to(float32);  residual = x.to(orig_dtype)
                    i.e. the new residual stream is the fp32 sum of the two bf16 tensors, rounded once.
"""
from __future__ import annotations

import torch


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """gate_up [M, 2K] bf16 (gate | up) -> [M, K] bf16."""
    d = gate_up.shape[-1] // 2
    return torch.nn.functional.silu(gate_up[..., :d]) * gate_up[..., d:]


def add_residual(y: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
    """y, residual [M, N] bf16 -> the new residual stream [M, N] bf16."""
    return (y.to(torch.float32) + residual.to(torch.float32)).to(y.dtype)
