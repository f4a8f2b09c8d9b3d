"""Oracle (test infrastructure): put the reference's OWN torch path for the fused projection next to the oracle, so that
benchmarks on a machine without the reference checkout can time the reference itself and not only its restatement.

    python -m oracle.build_ref [<reference checkout>]        (default: $ONEBASE_REFERENCE_DIR, else the build container's mount)

The reference is pure Python: "building" it means copying the modules that hold its CPU path
(lowbit_lora/kernels/{fp8_lora_multi, nvfp4_lora_vllm, common}.py: `reference_multi`, `reference`, the NVFP4 torch
recipes and the e4m3 helper they import) with their empty package markers into oracle/_ref/, which is git-ignored like
any other built artefact: the sources never enter this repository's history.  `load()` imports them from there; it
returns None when the directory has not been built.  The modules import triton at module level (their kernels live in
the same files); only their torch functions are called.
"""
from __future__ import annotations

import importlib
import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_DIR = HERE / "_ref"
MODULES = ("fp8_lora_multi", "nvfp4_lora_vllm", "common")
# ... and, for the opt-in GPU timing of the reference's own kernels (bench.py --reference-gpu), its Triton op for vLLM
GPU_MODULES = ("fp8_lora_vllm", "adapter_store")


DEFAULT_REFERENCE = os.environ.get("ONEBASE_REFERENCE_DIR", "/root/reference")


def build(reference: str | Path = DEFAULT_REFERENCE) -> Path | None:
    src = Path(reference) / "lowbit_lora" / "kernels"
    if not all((src / f"{m}.py").exists() for m in MODULES):
        return None
    dst = REF_DIR / "lowbit_lora" / "kernels"
    dst.mkdir(parents=True, exist_ok=True)
    (REF_DIR / "lowbit_lora" / "__init__.py").write_text("")
    (dst / "__init__.py").write_text("")
    for m in MODULES + tuple(m for m in GPU_MODULES if (src / f"{m}.py").exists()):
        shutil.copyfile(src / f"{m}.py", dst / f"{m}.py")
    return REF_DIR


def load():
    """(fp8_lora_multi module, nvfp4_lora_vllm module) of the built copy, or None if it is absent or does not import."""
    if not (REF_DIR / "lowbit_lora" / "kernels" / "fp8_lora_multi.py").exists():
        return None
    if str(REF_DIR) not in sys.path:
        sys.path.insert(0, str(REF_DIR))
    try:
        return (importlib.import_module("lowbit_lora.kernels.fp8_lora_multi"),
                importlib.import_module("lowbit_lora.kernels.nvfp4_lora_vllm"))
    except Exception:   # noqa: BLE001 - e.g. no triton on this machine: the caller falls back to the restatement
        return None


def load_gpu_op():
    """The reference's `VllmFusedFP8LoRA` class (its serialized Triton launches `_shrink_vllm` + `_gemm_vllm`,
    lowbit_lora/kernels/fp8_lora_vllm.py:416-765) out of the built copy, or None."""
    if load() is None or not (REF_DIR / "lowbit_lora" / "kernels" / "fp8_lora_vllm.py").exists():
        return None
    try:
        return importlib.import_module("lowbit_lora.kernels.fp8_lora_vllm").VllmFusedFP8LoRA
    except Exception:   # noqa: BLE001
        return None


if __name__ == "__main__":
    out = build(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_REFERENCE)
    print(out if out else "reference checkout not found: nothing built")
