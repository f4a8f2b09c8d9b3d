"""Oracle (test infrastructure, CPU torch): the FP8 e4m3 side of the path.

Follows the reference's torch restatement of vLLM's dynamic per-token FP8 quantization and its fp32 reference of the
fused projection:
  * per-token activation quantization ......... lowbit_lora/kernels/fp8_lora_multi.py:298-300 and the stand-alone rule
                                                `tq()` in tests/pdl_k2_interp_check.py:56-59
  * per-tensor weight quantization ............ tests/test_fp8_lora_vllm_interp.py:33-35, bench/pdl_k2_bench.py:195-197
  * FP8-stored adapters (per-row fp32 scale) .. lowbit_lora/kernels/fp8_lora_vllm.py:517-524,
                                                lowbit_lora/kernels/adapter_store.py:72-76
  * fused projection, fp32 .................... lowbit_lora/kernels/fp8_lora_multi.py:295-314 (`reference_multi`)
"""
from __future__ import annotations

import torch

FP8_MAX = 448.0
MIN_TOKEN_SCALE = 1.0 / (FP8_MAX * 512.0)   # vLLM's floor on a dynamic per-token scale (fp8_lora_vllm.py:27)
ADAPTER_SCALE_FLOOR = 1e-12                 # floor of a stored adapter row's scale (fp8_lora_vllm.py:522)


def quant_per_token(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """x [M, K] (bf16 or fp32) -> (codes [M, K] float8_e4m3fn, s_x [M] fp32).

    amax over the row in fp32; s_x = max(amax / 448, 1/(448*512)) (IEEE division); code = e4m3 round-to-nearest-even
    of clamp(x / s_x, +-448) (IEEE division, one rounding step)."""
    xf = x.to(torch.float32)
    s_x = torch.clamp_min(xf.abs().amax(dim=1) / FP8_MAX, MIN_TOKEN_SCALE)
    codes = torch.clamp(xf / s_x.unsqueeze(1), -FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return codes, s_x


def quant_weight_per_tensor(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """w [N, K] fp32 -> (codes float8_e4m3fn, s_w [1] fp32) with s_w = amax / 448, as the reference's tests and
    benches build their FP8 base weights."""
    s_w = (w.abs().max() / FP8_MAX).reshape(1).to(torch.float32)
    return (w / s_w).to(torch.float8_e4m3fn), s_w


def store_rows_fp8(t: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """FP8 storage of adapter matrices t [..., rows, cols]: one fp32 scale per row, amax / 448 floored at 1e-12."""
    tf = t.to(torch.float32)
    scale = torch.clamp_min(tf.abs().amax(dim=-1) / FP8_MAX, ADAPTER_SCALE_FLOOR)
    codes = torch.clamp(tf / scale.unsqueeze(-1), -FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return codes, scale


def lora_term(x: torch.Tensor, token_lora: torch.Tensor, a: torch.Tensor, b: torch.Tensor, widths,
              scale: float = 1.0, grouped: bool = False) -> torch.Tensor:
    """The adapters' contribution [M, N] in fp32: for token m with adapter l >= 0,
    h = bf16(scale * x[m] @ A_l^T) (one rounding of the whole shrink, fp32 accumulate) and, per slice s,
    out[m, slice s] = B_l[slice s] @ h[s*R:(s+1)*R].  a [L, S*R, K], b [L, N, R] (already dequantized to fp32 if the
    adapters are stored in a low-precision format).  Token by token, as fp8_lora_multi.py:303-313; grouped=True batches
    the tokens of each adapter into one matmul (same dot products in another summation order: a bf16 rounding of h may
    flip, so results agree to ~1e-4 relative, not to fp32 round-off)."""
    M = x.shape[0]
    N = b.shape[1]
    R = b.shape[2]
    out = torch.zeros(M, N, dtype=torch.float32)
    xf = x.to(torch.float32)
    ids = token_lora.to(torch.int64)
    groups = ([torch.nonzero(ids == l).flatten() for l in torch.unique(ids).tolist() if l >= 0] if grouped
              else [torch.tensor([m]) for m in range(M) if int(ids[m]) >= 0])
    for rows in groups:
        l = int(ids[rows[0]])
        h = (xf[rows] @ a[l].to(torch.float32).t() * scale).to(torch.bfloat16).to(torch.float32)   # [n, S*R]
        bl = b[l].to(torch.float32)
        off = 0
        for s, n_s in enumerate(widths):
            out[rows, off:off + n_s] = h[:, s * R:(s + 1) * R] @ bl[off:off + n_s].t()
            off += n_s
    return out


def fused_projection(x, token_lora, w_q, s_w, a, b, widths, scale: float = 1.0, xq=None, sx=None) -> torch.Tensor:
    """fp32 reference of y = s_x * s_w * (x_q @ W_q^T) + LoRA (fp8_lora_multi.py:295-314).  x_q / s_x are computed here
    unless given (the tests pass the kernel's own codes once those were checked bit-exact)."""
    if xq is None:
        xq, sx = quant_per_token(x)
    base = (xq.to(torch.float32) * sx.unsqueeze(1)) @ (w_q.to(torch.float32) * s_w.to(torch.float32)).t()
    return base + lora_term(x, token_lora, a, b, widths, scale)


def stack_slices(a_stacked, b_stacked) -> tuple[torch.Tensor, torch.Tensor]:
    """vLLM's per-slice buffers (a_stacked[s] [L,1,R,K], b_stacked[s] [L,1,N_s,R]) -> (A [L,S*R,K], B [L,N,R]),
    the layout the reference functions take (tests/test_fp8_lora_vllm_interp.py:38-39)."""
    return torch.cat([t[:, 0] for t in a_stacked], dim=1), torch.cat([t[:, 0] for t in b_stacked], dim=1)
