"""vLLM plugin: serve LoRA layers whose base is per-tensor FP8 or ModelOpt NVFP4 through the fused B200 kernels.

Same contract as the reference's `lowbit_lora.plugin` (lowbit_lora/plugin.py:1-355): vLLM loads `install` through the
`vllm.general_plugins` entry-point group in every process; it is no-arg, idempotent and does nothing unless
LOWBIT_FUSED=1.  It registers the opaque custom op `torch.ops.vllm.lowbit_fused_fp8_lora(x, layer_id, tok, srt, seg_n,
seg_start, seg_ids)` (CUDA-graph capturable: it only reads vLLM's static LoRA buffers and Punica metadata) and patches
`BaseLinearLayerWithLoRA.{set_mapping, _apply_sync, apply}`.  Beyond the reference it also wraps every class-level
`apply` override of the LoRA linear classes: in newer vLLM the merged column-parallel / replicated / sharded classes
define their own `apply` that never reaches the base class.

Switches (environment, read at install / layer build; same names and meaning as the reference where they still apply):
  LOWBIT_FUSED=1          enable the plugin
  LOWBIT_PDL=0            launch K1 and K2 serialized instead of chained by programmatic dependent launch (default: chained)
  LOWBIT_PDL_MAX_M=<n>    chain only batches of at most n tokens (default: all)
  LOWBIT_PDL_CFG=<file>   extra tile-table rows (onebase_b200.tile_table)
  LOWBIT_TP=1             also serve tensor-parallel shards and layers with a bias (bias added after the fused call)
  LOWBIT_NVFP4_RCP=exact  NVFP4 activation quantizer with IEEE reciprocals (default: rcp.approx.ftz, vLLM's kernel)
  LOWBIT_REPORT=<file>    one pid-tagged line per layer decision, and an `op-called` line
  LOWBIT_VERBOSE=1        print what was installed
  LOWBIT_WARMUP=0         skip the load-time scratch growth
  LOWBIT_COMPILE_CACHE=0  disable vLLM's compile cache instead of keying it
  LOWBIT_LORA_FP8=1 / LOWBIT_LORA_FP4=1   serve the adapters FP8-stored (e4m3, per-row scales) / NVFP4-stored from low-precision
                          copies refreshed on every slot write; LOWBIT_RELEASE_SLOTS=0 keeps vLLM's bf16 slots as well
  LOWBIT_SEGMENT_INDEX=1  (not in the reference) build vLLM's per-step token sort / segment index with the ob_segment_index
                          kernel instead of torch sort / unique / cumsum (LoRAKernelMeta.prepare_tensors): one launch and
                          one small copy to the host per step
  LOWBIT_DISPATCH*, LOWBIT_HYBRIDQ, LOWBIT_LEAN_BASE, LOWBIT_TUNE_MAX_M   accepted and ignored: there is no timed
                          dispatch; tiles come from the table.
"""
from __future__ import annotations

import os

import torch

_REGISTRY: list = []          # layer id -> op object
_INSTALLED = False
_CALLED = [False]
_STATS = {"fused_layers": 0, "fallback_layers": 0}


def _on(name: str, default: str = "0") -> bool:
    return os.environ.get(name, default) not in ("0", "", "false", "False")


def _report(line: str) -> None:
    rep = os.environ.get("LOWBIT_REPORT")
    if rep:
        with open(rep, "a") as fh:
            fh.write(f"{os.getpid()} {line}\n")


def _device_segment_index(meta, token_lora_mapping: torch.Tensor, max_loras: int) -> None:
    """Fill the five metadata tensors of a vLLM LoRAKernelMeta with one launch of the segment index kernel."""
    import ctypes as C

    from onebase_b200 import _lib
    t = token_lora_mapping
    p = lambda x: C.c_void_p(x.data_ptr())   # noqa: E731
    _lib.call("ob_segment_index", p(t), t.numel(), max_loras, p(meta.token_lora_mapping),
              p(meta.token_indices_sorted_by_lora_ids), p(meta.num_tokens_per_lora), p(meta.lora_token_start_loc),
              p(meta.active_lora_ids), C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream))


def segment_index_prepare(orig, index_fn=None):
    """A replacement for vLLM's `LoRAKernelMeta.prepare_tensors` (vllm/lora/ops/triton_ops/lora_kernel_metadata.py:110-168)
    that leaves the same five tensors, bit for bit and with the same statefulness (an all -1 batch resets the segment arrays
    and keeps the token map and sorted indices), through `index_fn(meta, mapping, max_loras)` -- the ob_segment_index kernel
    unless a test passes its own -- and then sets the host-side flags vLLM's own LoRA ops and its CUDA-graph dispatch read
    (`no_lora_flag_cpu`, `num_active_loras_cpu` rounded up to a captured count) from ONE copy of the per-segment token
    counts.  Inputs the kernel does not take (not int32 / not contiguous / not on a GPU / more than 256 slots) go to `orig`."""
    import bisect

    def prepare_tensors(self, token_lora_mapping: torch.Tensor) -> None:
        t = token_lora_mapping
        max_loras = self.active_lora_ids.numel() - 1
        fits = (t.dtype == torch.int32 and t.is_contiguous() and t.ndim == 1 and 0 < max_loras <= 256 and
                t.numel() <= self.token_lora_mapping.numel())
        if not fits or (index_fn is None and not t.is_cuda):
            return orig(self, t)
        (index_fn or _device_segment_index)(self, t, max_loras)
        counts = self.num_tokens_per_lora.cpu()                 # the step's only device -> host copy (it synchronizes)
        groups = int((counts > 0).sum())                        # unique ids of the batch, the "-1" group included
        if hasattr(self, "no_lora_flag_cpu"):
            self.no_lora_flag_cpu[0] = groups == 0              # the kernel leaves every count 0 for an all -1 batch
        if hasattr(self, "num_active_loras_cpu"):
            captured = getattr(self, "captured_lora_counts", None)
            if captured and groups > 0:
                i = bisect.bisect_left(captured, groups)
                if i < len(captured):
                    groups = captured[i]
            self.num_active_loras_cpu[0] = groups

    return prepare_tensors


def _cache_root() -> str:
    """vLLM's compile-cache root keyed on this package's source and every LOWBIT_* setting (as the reference's
    `_cache_root`, plugin.py:31-51): a graph compiled without the plugin would silently bypass it."""
    import hashlib
    from pathlib import Path

    import vllm.envs as envs
    h = hashlib.sha256()
    pkg = Path(__file__).resolve().parent
    for f in sorted(list(pkg.rglob("*.py")) + list(pkg.rglob("*.cu")) + list(pkg.rglob("*.cuh")) + list(pkg.rglob("*.jsonl"))):
        h.update(str(f.relative_to(pkg)).encode())
        h.update(f.read_bytes())
    for k in sorted(os.environ):
        if k.startswith("LOWBIT_") and k not in ("LOWBIT_REPORT", "LOWBIT_VERBOSE"):
            h.update(f"{k}={os.environ[k]}\n".encode())
    base = envs.VLLM_CACHE_ROOT
    key = f"lowbit-{h.hexdigest()[:12]}"
    return base if os.path.basename(base) == key else os.path.join(base, key)


def _fused(x: torch.Tensor, layer_id: int, tok: torch.Tensor, srt: torch.Tensor, seg_n: torch.Tensor,
           seg_start: torch.Tensor, seg_ids: torch.Tensor) -> torch.Tensor:
    if not _CALLED[0]:          # once per process: proof that the compiled graph calls this op
        _CALLED[0] = True
        _report("op-called")
    op = _REGISTRY[layer_id]
    pdl = _on("LOWBIT_PDL", "1")
    max_m = int(os.environ.get("LOWBIT_PDL_MAX_M", "0") or 0)
    if max_m and x.shape[0] > max_m:
        pdl = False
    return op(x, (tok, srt, seg_n, seg_start, seg_ids), pdl=pdl)


def _fused_fake(x: torch.Tensor, layer_id: int, tok: torch.Tensor, srt: torch.Tensor, seg_n: torch.Tensor,
                seg_start: torch.Tensor, seg_ids: torch.Tensor) -> torch.Tensor:
    return torch.empty(x.shape[0], _REGISTRY[layer_id].N, dtype=torch.bfloat16, device=x.device)


def _op_classes():
    from onebase_b200.kernels.fp8_lora_vllm import VllmFusedFP8LoRA
    from onebase_b200.kernels.nvfp4_lora_vllm import VllmFusedNVFP4LoRA
    return VllmFusedFP8LoRA, VllmFusedNVFP4LoRA


def _adapters_ok(layer) -> bool:
    a, b = getattr(layer, "lora_a_stacked", None), getattr(layer, "lora_b_stacked", None)
    if a is None or b is None or not (1 <= len(a) <= 4) or len(a) != len(b):
        return False
    if not all(t.dtype == torch.bfloat16 for t in (*a, *b)):
        return False
    return a[0].shape[2] in (16, 32, 64, 128, 256)


def _is_fp8_per_tensor(base, qm) -> bool:
    """A linear layer whose weight vLLM holds as per-tensor e4m3 codes with one fp32 scale and whose activations are
    quantized dynamically (reference: isinstance checks on vLLM's classes, plugin.py:243-248).  Recognised by the
    quantized tensors plus the method's class NAME -- vLLM has moved and renamed these classes between releases
    (`Fp8PerTensorOnlineLinearMethod` under quantization/online, `Fp8OnlineLinearMethod` / `Fp8LinearMethod` in
    quantization/fp8.py) -- and never for block-quantized weights or a static activation scale."""
    w, ws = getattr(base, "weight", None), getattr(base, "weight_scale", None)
    if w is None or ws is None or w.dtype != torch.float8_e4m3fn or ws.numel() != 1:
        return False
    if qm is None or getattr(qm, "block_quant", False) or getattr(base, "input_scale", None) is not None:
        return False
    return type(qm).__name__ in ("Fp8PerTensorOnlineLinearMethod", "Fp8OnlineLinearMethod", "Fp8LinearMethod")


def _hook_slot_writes(layer, op) -> None:
    """Per instance: requantize a slot's low-precision copy after vLLM writes or clears it (reference: plugin.py:89-130).
    By default (LOWBIT_RELEASE_SLOTS=0 keeps vLLM's buffers) the copies become the only per-slot storage: vLLM's bf16 slots
    shrink to one staging slot that every write goes through."""
    set_lora, reset_lora = layer.set_lora, layer.reset_lora
    if _on("LOWBIT_RELEASE_SLOTS", "1"):
        layer.lora_a_stacked = tuple(t[:1].clone() for t in layer.lora_a_stacked)
        layer.lora_b_stacked = tuple(t[:1].clone() for t in layer.lora_b_stacked)
        op.release(layer.lora_a_stacked, layer.lora_b_stacked)
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
        writing = [False]

        def set_lora_s(index, *args, **kw):
            writing[0] = True
            try:
                set_lora(0, *args, **kw)          # its reset_lora(0) lands in reset_lora_s
            finally:
                writing[0] = False
            op.requantize(index)

        def reset_lora_s(index):
            reset_lora(0)
            if not writing[0]:
                op.requantize(index)              # a cleared slot: the copy of the zeroed staging slot

        layer.set_lora, layer.reset_lora = set_lora_s, reset_lora_s
        layer._lowbit_released = True
        return

    def set_lora_q(index, *args, **kw):
        set_lora(index, *args, **kw)
        op.requantize(index)

    def reset_lora_q(index):
        reset_lora(index)
        op.requantize(index)

    layer.set_lora, layer.reset_lora = set_lora_q, reset_lora_q


def _build(layer) -> int:
    """Decide and construct once per layer (vLLM calls set_mapping right after wrapping a layer, after the base weights
    were quantized, before CUDA graphs are captured).  Returns the layer id or -1 (fallback to vLLM's own path)."""
    base = layer.base_layer
    qm = getattr(base, "quant_method", None)
    tp_ok = _on("LOWBIT_TP")
    why = ""
    lid = -1
    kind = "fused"
    fp8_cls, nvfp4_cls = _op_classes()
    st4 = getattr(base, "_lowbit_nvfp4", None)
    max_m = layer.punica_wrapper._token_lora_indices.numel()
    fmt = "nvfp4" if _on("LOWBIT_LORA_FP4") else "fp8" if _on("LOWBIT_LORA_FP8") else "bf16"
    if not _adapters_ok(layer):
        why = "adapter buffers (dtype / slices / rank)"
    elif (getattr(layer, "tp_size", 1) != 1 or getattr(base, "bias", None) is not None) and not tp_ok:
        why = "tensor-parallel shard or bias without LOWBIT_TP=1"
    elif st4 is not None:
        w_q, w_sf = st4["w_q"], st4["w_sf"]
        widths = [t.shape[2] for t in layer.lora_b_stacked]
        if w_q.shape[0] == sum(widths) and 2 * w_q.shape[1] == layer.lora_a_stacked[0].shape[3] and w_q.shape[1] % 16 == 0:
            op = nvfp4_cls(w_q, w_sf, 1.0 / st4["weight_scale_2"], 1.0 / st4["input_scale"], layer.lora_a_stacked,
                           layer.lora_b_stacked, max_m, lora_fmt=fmt,
                           rcp_approx=os.environ.get("LOWBIT_NVFP4_RCP", "approx") != "exact")
            kind = "fused-nvfp4"
            _REGISTRY.append(op)
            lid = len(_REGISTRY) - 1
        else:
            why = "NVFP4 weight shape"
    elif _is_fp8_per_tensor(base, qm):
        w_q = base.weight.t()                                   # [N, K], the storage vLLM quantized into
        widths = [t.shape[2] for t in layer.lora_b_stacked]
        if w_q.is_contiguous() and w_q.shape[0] == sum(widths) and w_q.shape[1] == layer.lora_a_stacked[0].shape[3] \
                and w_q.shape[1] % 16 == 0:
            op = fp8_cls(w_q, base.weight_scale.reshape(1).float(), layer.lora_a_stacked, layer.lora_b_stacked, max_m,
                         lora_fp8=fmt == "fp8", lora_fp4=fmt == "nvfp4")
            _REGISTRY.append(op)
            lid = len(_REGISTRY) - 1
        else:
            why = "FP8 weight layout"
    else:
        why = "base is neither per-tensor FP8 nor ModelOpt NVFP4"
    if lid >= 0 and fmt != "bf16":
        _hook_slot_writes(layer, _REGISTRY[lid])
    if lid >= 0:
        if _on("LOWBIT_WARMUP", "1"):
            _REGISTRY[lid].warmup()
        _STATS["fused_layers"] += 1
    else:
        _STATS["fallback_layers"] += 1
    _report(f"{type(layer).__name__} {kind if lid >= 0 else 'fallback'} {getattr(base, 'prefix', '')} "
            f"dispatch=table{(' reason=' + why.replace(' ', '_')) if lid < 0 else ''}")
    return lid


def install() -> None:
    global _INSTALLED
    if _INSTALLED or not _on("LOWBIT_FUSED"):
        return
    if _on("LOWBIT_COMPILE_CACHE", "1"):
        try:
            os.environ["VLLM_CACHE_ROOT"] = _cache_root()
        except Exception:   # noqa: BLE001 - an unkeyable cache is disabled rather than shared with stock graphs
            os.environ["VLLM_DISABLE_COMPILE_CACHE"] = "1"
    else:
        os.environ["VLLM_DISABLE_COMPILE_CACHE"] = "1"
    import inspect

    import vllm.lora.layers as lora_layers
    from vllm.lora.layers.base_linear import BaseLinearLayerWithLoRA
    from vllm.utils.torch_utils import direct_register_custom_op

    try:   # keep the NVFP4 checkpoint layout (codes, linear block scales) before the backend re-layouts it
        from vllm.model_executor.layers.quantization.modelopt import ModelOptNvFp4LinearMethod
        orig_process = ModelOptNvFp4LinearMethod.process_weights_after_loading

        def nvfp4_process(self, layer):
            layer._lowbit_nvfp4 = st = {"w_q": layer.weight.data.clone(),
                                        "w_sf": layer.weight_scale.data.view(torch.float8_e4m3fn).clone(),
                                        "input_scale": float(layer.input_scale.max()),
                                        "weight_scale_2": float(layer.weight_scale_2.max())}
            out = orig_process(self, layer)
            w = layer.weight.data
            if w.dtype == st["w_q"].dtype and w.shape == st["w_q"].shape and w.is_contiguous() and torch.equal(w, st["w_q"]):
                st["w_q"] = w                                   # the backend kept the codes in place: share them
            return out

        ModelOptNvFp4LinearMethod.process_weights_after_loading = nvfp4_process
    except Exception:   # noqa: BLE001
        pass

    if _on("LOWBIT_SEGMENT_INDEX"):
        try:
            from vllm.lora.ops.triton_ops.lora_kernel_metadata import LoRAKernelMeta
            LoRAKernelMeta.prepare_tensors = segment_index_prepare(LoRAKernelMeta.prepare_tensors)
            _report("segment-index kernel installed in LoRAKernelMeta.prepare_tensors")
        except Exception as e:   # noqa: BLE001 - vLLM keeps its own metadata code
            _report(f"segment-index kernel not installed: {type(e).__name__}")

    direct_register_custom_op(op_name="lowbit_fused_fp8_lora", op_func=_fused, mutates_args=[], fake_impl=_fused_fake)
    fused_op = torch.ops.vllm.lowbit_fused_fp8_lora
    orig_sync = BaseLinearLayerWithLoRA._apply_sync
    orig_apply = BaseLinearLayerWithLoRA.apply
    orig_set_mapping = BaseLinearLayerWithLoRA.set_mapping
    tp_bias = _on("LOWBIT_TP")

    def set_mapping(self, punica_wrapper):
        orig_set_mapping(self, punica_wrapper)
        if "_lowbit_id" not in self.__dict__:
            self._lowbit_id = _build(self)

    def _note_fallback(layer, why: str) -> None:
        if not layer.__dict__.get("_lowbit_fb"):
            layer.__dict__["_lowbit_fb"] = True
            _report(f"{type(layer).__name__} runtime-fallback {why}")

    def fused_or_none(self, x, bias):
        """The fused call if this layer and this input can be served, else None."""
        lid = getattr(self, "_lowbit_id", -1)
        if lid < 0:
            return None
        if bias is not None and not tp_bias:
            return None
        if x.dtype != torch.bfloat16:
            if not torch.compiler.is_compiling():
                _note_fallback(self, f"dtype={x.dtype}")
            return None
        shape = x.shape
        x2 = x if x.ndim == 2 and x.is_contiguous() else x.reshape(-1, shape[-1]).contiguous()
        tok, srt, seg_n, seg_start, seg_ids = self.punica_wrapper.token_mapping_meta.meta_args(
            x2.size(0), self.lora_config.specialize_active_lora)[:5]
        y = fused_op(x2, lid, tok, srt, seg_n, seg_start, seg_ids)
        if bias is not None:
            y = y + bias
        return y if x.ndim == 2 else y.reshape(*shape[:-1], -1)

    def _stock_allowed(layer) -> None:
        """vLLM's own path indexes the per-slot bf16 buffers; once a layer serves from the low-precision copies alone those
        buffers are a single staging slot, and a call the fused path cannot take must fail loudly instead of reading past it."""
        if layer.__dict__.get("_lowbit_released"):
            raise RuntimeError("onebase_b200: this layer's bf16 adapter slots were released (LOWBIT_RELEASE_SLOTS) and the call "
                               "cannot be served by the fused path (input dtype or bias); set LOWBIT_RELEASE_SLOTS=0")

    def _apply_sync(self, x, bias=None):
        y = fused_or_none(self, x, bias)
        if y is None:
            _stock_allowed(self)
        return y if y is not None else orig_sync(self, x, bias)

    def apply(self, x, bias=None):
        y = fused_or_none(self, x, bias)
        if y is None:
            _stock_allowed(self)
        return y if y is not None else orig_apply(self, x, bias)

    BaseLinearLayerWithLoRA.set_mapping = set_mapping
    BaseLinearLayerWithLoRA._apply_sync = _apply_sync
    BaseLinearLayerWithLoRA.apply = apply
    wrapped = []
    for name, cls in inspect.getmembers(lora_layers, inspect.isclass):
        if cls is BaseLinearLayerWithLoRA or not issubclass(cls, BaseLinearLayerWithLoRA) or "apply" not in cls.__dict__:
            continue

        def make(orig):
            def apply_override(self, x, bias=None):
                y = fused_or_none(self, x, bias)
                if y is None:
                    _stock_allowed(self)
                return y if y is not None else orig(self, x, bias)
            return apply_override

        cls.apply = make(cls.__dict__["apply"])
        wrapped.append(name)
    _INSTALLED = True
    _report(f"installed wrapped-apply={','.join(wrapped) or '-'}")
    if os.environ.get("LOWBIT_VERBOSE"):
        print(f"[lowbit] onebase_b200 fused FP8/NVFP4 + LoRA plugin installed (class-level apply wrapped: {wrapped})", flush=True)
