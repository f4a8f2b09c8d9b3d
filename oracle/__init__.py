"""CPU oracle for the fused low-precision base GEMM + multi-tenant LoRA projection.

TEST INFRASTRUCTURE ONLY.  This package restates, in plain torch on the CPU, the arithmetic of the reference's own
"torch dequantize-and-matmul" path (every function cites the reference file:line it follows).  It exists so that the
CUDA kernels can be checked against it; the product (`onebase_b200`) never imports it and has no CPU fallback.  Only
the tests, `__graft_entry__.smoke()` and the CPU-baseline legs of `bench.py` may import it.

Parity is PINNED: `tests/golden/make_golden.py` imported the reference (`lowbit_lora.kernels.fp8_lora_multi`,
`lowbit_lora.kernels.nvfp4_lora_vllm`, `lowbit_lora.kernels.adapter_store`) and vLLM's `LoRAKernelMeta` on the CPU,
ran them on seeded inputs and stored their outputs under `tests/golden/`; `tests/test_oracle_golden.py` checks this
restatement against those files bit for bit (codes, scales, indices) or to fp32 round-off (matmul outputs).
"""
from oracle import fp8, nvfp4, segments  # noqa: F401
