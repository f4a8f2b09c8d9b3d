"""Oracle (test infrastructure): seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations, drawn on the CPU in one fixed order (x, W, A per slice, B per slice, ids) so that the CPU oracle and
the CUDA kernels see identical bits.

Distributions follow the reference's tests and benches: x ~ N(0,1) bf16; W ~ N(0,1)*0.02 quantized per tensor
(bench/pdl_k2_bench.py:193-197); A ~ U(+-1/sqrt(K)) and B ~ N(0,1)*0.01 bf16 in vLLM's stacked per-slice layout
[L,1,R,K] / [L,1,N_s,R] (lowbit_lora/kernels/fp8_lora_vllm.py:4-8); slot ids uniform.
Projection shapes are Qwen3-8B's (bench/kernel_bench.py:29-31).
"""
from __future__ import annotations

import torch

from oracle import fp8, nvfp4

QWEN3_8B = {          # projection -> (K, slice widths)
    "qkv": (4096, (4096, 1024, 1024)),
    "o": (4096, (4096,)),
    "gate_up": (4096, (12288, 12288)),
    "down": (12288, (4096,)),
}
L72B = {              # 72B-class architecture (hidden 8192, 64 q / 8 kv heads of 128, intermediate 29568)
    "qkv": (8192, (8192, 1024, 1024)),
    "o": (8192, (8192,)),
    "gate_up": (8192, (29568, 29568)),
    "down": (29568, (8192,)),
}


def draw(K: int, widths, R: int, L: int, M: int, seed: int = 0, ids_low: int = -1, w_std: float = 0.02,
         b_std: float = 0.01) -> dict:
    """One projection's inputs.  ids uniform over {ids_low, ..., L-1} (ids_low = -1 includes "no adapter")."""
    g = torch.Generator().manual_seed(seed)
    N = sum(widths)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, generator=g) * w_std
    a_st = tuple(((torch.rand(L, 1, R, K, generator=g) * 2 - 1) / K ** 0.5).to(torch.bfloat16) for _ in widths)
    b_st = tuple((torch.randn(L, 1, n, R, generator=g) * b_std).to(torch.bfloat16) for n in widths)
    ids = torch.randint(ids_low, L, (M,), generator=g, dtype=torch.int32)
    return {"x": x, "w": w, "a_stacked": a_st, "b_stacked": b_st, "ids": ids, "K": K, "N": N, "widths": tuple(widths),
            "R": R, "L": L, "M": M}


def with_fp8_base(d: dict) -> dict:
    d["w_q"], d["s_w"] = fp8.quant_weight_per_tensor(d["w"])
    return d


def with_nvfp4_base(d: dict) -> dict:
    d["w_global"] = nvfp4.global_scale_for(d["w"])
    d["w_q4"], d["w_sf"] = nvfp4.quant(d["w"], d["w_global"])
    d["x_global"] = nvfp4.global_scale_for(d["x"].float())
    return d


def config0(seed: int = 0) -> dict:
    """Single FP8 projection: M 16, K = N = 4096, 4 bf16 adapters of rank 16, ids uniform over {-1, 0..3}."""
    return with_fp8_base(draw(4096, (4096,), 16, 4, 16, seed=seed, ids_low=-1))


def zipf_request_ids(M: int, L: int, seed: int, alpha: float = 1.1, mean_len: int = 64) -> torch.Tensor:
    """Prefill batches: requests of contiguous tokens, each request's slot drawn Zipf(alpha) over the L slots."""
    g = torch.Generator().manual_seed(seed)
    p = 1.0 / torch.arange(1, L + 1, dtype=torch.float64) ** alpha
    p = p / p.sum()
    ids = torch.empty(M, dtype=torch.int32)
    pos = 0
    while pos < M:
        n = int(torch.randint(max(1, mean_len // 2), 2 * mean_len, (1,), generator=g))
        slot = int(torch.multinomial(p, 1, generator=g))
        ids[pos:pos + n] = slot
        pos += n
    return ids
