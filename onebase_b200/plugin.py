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
_STATS = {"fused_layers": 0, "fallback_layers": 0, "segment_index_kernel": 0, "segment_index_stock": 0}
_LAUNCH = {"pdl": True, "pdl_max_m": 0}   # how the op launches its two kernels; filled from the environment by install()


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
    counts.  int64 mappings (what vLLM's Punica wrapper passes) are cast to int32 on the device first.  Inputs the kernel
    does not take (another dtype, empty, not on a GPU, more than 256 slots) go to `orig`."""
    import bisect

    def prepare_tensors(self, token_lora_mapping: torch.Tensor) -> None:
        t = token_lora_mapping
        max_loras = self.active_lora_ids.numel() - 1
        fits = (t.dtype in (torch.int32, torch.int64) and t.ndim == 1 and 0 < max_loras <= 256 and
                0 < t.numel() <= self.token_lora_mapping.numel())
        if not fits or (index_fn is None and not t.is_cuda):
            _STATS["segment_index_stock"] += 1
            return orig(self, t)               # (an empty mapping too: vLLM treats it as a batch without adapters)
        if t.dtype != torch.int32 or not t.is_contiguous():
            # vLLM's PunicaWrapperGPU hands over a slice of its int64 `_token_lora_indices` (punica_base.py): slot ids
            # fit 32 bits, and the cast is one small device-side copy in the same stream
            t = t.to(torch.int32).contiguous()
        (index_fn or _device_segment_index)(self, t, max_loras)
        _STATS["segment_index_kernel"] += 1
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


def _settings_digest() -> str:
    """Twelve hex digits that change with anything that changes what a compiled graph would call: the built library, the
    tile rows, this package's Python, and every LOWBIT_* switch except the two that only steer reporting."""
    import hashlib
    from pathlib import Path
    pkg = Path(__file__).resolve().parent
    digest = hashlib.blake2b(digest_size=6)
    tracked = [q for pat in ("*.py", "kernels/*.py", "tiles/*.jsonl", "csrc/*.cu", "csrc/*.cuh") for q in pkg.glob(pat)]
    for q in sorted(tracked, key=lambda q: q.as_posix()):
        digest.update(q.relative_to(pkg).as_posix().encode() + b"\0" + q.read_bytes() + b"\0")
    switches = {k: v for k, v in os.environ.items() if k.startswith("LOWBIT_") and k not in ("LOWBIT_REPORT", "LOWBIT_VERBOSE")}
    digest.update(repr(sorted(switches.items())).encode())
    return digest.hexdigest()


def _cache_root() -> str:
    """Where vLLM should keep graphs compiled with this plugin active: a sub-directory of its cache root named after
    `_settings_digest()`, so that a graph compiled without the plugin (or with other switches) is never reused -- it
    would bypass the fused op without any error (the reference keys its cache the same way, lowbit_lora/plugin.py:31-51).
    A child process that inherits an already keyed root keeps it."""
    import vllm.envs as envs
    root = envs.VLLM_CACHE_ROOT
    leaf = "lowbit-" + _settings_digest()
    return root if os.path.basename(os.path.normpath(root)) == leaf else os.path.join(root, leaf)


def _fused(x: torch.Tensor, layer_id: int, tok: torch.Tensor, srt: torch.Tensor, seg_n: torch.Tensor,
           seg_start: torch.Tensor, seg_ids: torch.Tensor) -> torch.Tensor:
    if not _CALLED[0]:          # once per process: proof that the compiled graph calls this op
        _CALLED[0] = True
        _report("op-called")
    op = _REGISTRY[layer_id]
    limit = _LAUNCH["pdl_max_m"]
    chained = _LAUNCH["pdl"] and not (limit and x.shape[0] > limit)
    return op(x, (tok, srt, seg_n, seg_start, seg_ids), pdl=chained)


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
    if not all(t.dtype == torch.bfloat16 and t.ndim == 4 for t in (*a, *b)):
        return False
    rank = a[0].shape[2]
    # every slice: A [L,1,R,K] and B [L,1,N_s,R] with the SAME R -- vLLM's fully sharded classes keep A as [L,1,R/tp,K] and
    # all-gather the shrink, which this op does not do
    if any(ta.shape[2] != rank or tb.shape[3] != rank for ta, tb in zip(a, b)):
        return False
    return rank in (16, 32, 64, 128, 256)


def _fully_sharded(layer) -> bool:
    """vLLM's `fully_sharded_loras` classes (…WithShardedLoRA): their shrink output is all-gathered / their expand input
    all-reduced between the two LoRA kernels, a collective the fused call does not contain."""
    return any("ShardedLoRA" in c.__name__ for c in type(layer).__mro__)


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


def _fp8_backend(qm) -> str:
    """Name of the scaled-mm kernel object vLLM chose for this layer (the reference insists on the CUTLASS one, which
    quantizes activations per token: lowbit_lora/plugin.py:244).  Reported per layer; LOWBIT_FP8_BACKEND_STRICT=1 makes any
    other backend a fallback."""
    for attr in ("fp8_linear", "kernel", "fp8_linear_op"):
        k = getattr(qm, attr, None)
        if k is not None:
            return type(getattr(k, "kernel", k)).__name__
    return "unknown"


class _SlotWrites:
    """Keeps an op's low-precision adapter copies in step with vLLM's slot writes on ONE layer instance, by standing in
    for the instance's `set_lora` / `reset_lora` (what the reference does per instance too, lowbit_lora/plugin.py:89-130;
    subclasses of the LoRA layers override these methods, hence the instance and not the class).

    keep_bf16 = True   vLLM's L bf16 slots stay; after each write or reset of slot i the copy of slot i is refreshed.
    keep_bf16 = False  (default, LOWBIT_RELEASE_SLOTS=1) vLLM's buffers are cut down to ONE staging slot: every write goes
                       into staging slot 0 and is then filed under its real index in the copies, which become the only
                       per-slot storage (32 rank-64 slots of an 8B model are about 10 GB of bf16 otherwise).
    vLLM's own `set_lora(i, ...)` begins with `reset_lora(i)`; while a write is under way that inner reset must not refresh
    the copy (it would file a zeroed slot under i and the write would then quantize twice)."""

    def __init__(self, layer, op, keep_bf16: bool):
        self.op, self.keep = op, keep_bf16
        self.vllm_set, self.vllm_reset = layer.set_lora, layer.reset_lora
        self.mid_write = False
        if not keep_bf16:
            layer.lora_a_stacked = tuple(buf.narrow(0, 0, 1).clone() for buf in layer.lora_a_stacked)
            layer.lora_b_stacked = tuple(buf.narrow(0, 0, 1).clone() for buf in layer.lora_b_stacked)
            op.release(layer.lora_a_stacked, layer.lora_b_stacked)
            layer._lowbit_released = True
            if torch.cuda.is_available():
                torch.cuda.empty_cache()
        layer.set_lora, layer.reset_lora = self.write, self.clear

    def _vllm_index(self, index: int) -> int:
        return index if self.keep else 0

    def write(self, index, *args, **kwargs):
        self.mid_write = True
        try:
            self.vllm_set(self._vllm_index(index), *args, **kwargs)
        finally:
            self.mid_write = False
        self.op.requantize(index)

    def clear(self, index):
        self.vllm_reset(self._vllm_index(index))
        if not self.mid_write:
            self.op.requantize(index)


def _hook_slot_writes(layer, op) -> None:
    _SlotWrites(layer, op, keep_bf16=not _on("LOWBIT_RELEASE_SLOTS", "1"))


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
    if _fully_sharded(layer):
        why = "fully sharded adapters"
    elif not _adapters_ok(layer):
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
    elif _is_fp8_per_tensor(base, qm) and _on("LOWBIT_FP8_BACKEND_STRICT") and "Cutlass" not in _fp8_backend(qm):
        why = f"FP8 backend {_fp8_backend(qm)} (LOWBIT_FP8_BACKEND_STRICT=1 wants vLLM's CUTLASS per-token kernel)"
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
            f"dispatch=table{(' fp8_backend=' + _fp8_backend(qm)) if lid >= 0 and kind == 'fused' else ''}"
            f"{(' reason=' + why.replace(' ', '_')) if lid < 0 else ''}")
    return lid


def _keep_nvfp4_checkpoint_layout() -> None:
    """vLLM's NVFP4 backends re-layout a ModelOpt checkpoint's tensors when the weights have been loaded (swizzled block
    scales, possibly shuffled codes).  K2 wants the checkpoint's own layout -- codes [N, K/2], linear ue4m3 block scales
    [N, K/16] -- so a snapshot is taken just before (`layer._lowbit_nvfp4`), with the two per-tensor scales as vLLM itself
    reduces them (the maximum over fused shards).  When the backend turns out to have left the codes untouched the snapshot
    of the codes is dropped in favour of vLLM's tensor, so only the scales are held twice.  (The reference does the same
    around the same method, lowbit_lora/plugin.py:155-174.)  No-op when this vLLM has no ModelOpt NVFP4 method."""
    try:
        from vllm.model_executor.layers.quantization.modelopt import ModelOptNvFp4LinearMethod as Method
    except Exception:   # noqa: BLE001
        return
    if getattr(Method.process_weights_after_loading, "_lowbit_wrapped", False):
        return
    backend_relayout = Method.process_weights_after_loading

    def process_weights_after_loading(self, layer):
        codes = layer.weight.data.clone()
        snap = {"w_q": codes, "w_sf": layer.weight_scale.data.view(torch.float8_e4m3fn).clone(),
                "input_scale": float(layer.input_scale.max()), "weight_scale_2": float(layer.weight_scale_2.max())}
        layer._lowbit_nvfp4 = snap
        result = backend_relayout(self, layer)
        after = layer.weight.data
        same_storage_layout = after.dtype == codes.dtype and after.shape == codes.shape and after.is_contiguous()
        if same_storage_layout and torch.equal(after, codes):
            snap["w_q"] = after
        return result

    process_weights_after_loading._lowbit_wrapped = True
    Method.process_weights_after_loading = process_weights_after_loading


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
    _LAUNCH["pdl"] = _on("LOWBIT_PDL", "1")
    _LAUNCH["pdl_max_m"] = int(os.environ.get("LOWBIT_PDL_MAX_M", "0") or 0)
    import inspect

    import vllm.lora.layers as lora_layers
    from vllm.lora.layers.base_linear import BaseLinearLayerWithLoRA
    from vllm.utils.torch_utils import direct_register_custom_op

    _keep_nvfp4_checkpoint_layout()

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
        # vLLM calls this once per wrapped layer, after the base weights are final and before any graph capture: the one
        # point where the layer can be inspected and its op built.  The decision is kept on the instance.
        orig_set_mapping(self, punica_wrapper)
        if vars(self).get("_lowbit_id") is None:
            vars(self)["_lowbit_id"] = _build(self)

    reported_fallbacks: set = set()

    def _note_fallback(layer, why: str) -> None:
        if id(layer) not in reported_fallbacks:                # one line per layer, however often it falls back
            reported_fallbacks.add(id(layer))
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


def install_pdl() -> None:
    """Entry point `lowbit_pdl`: in the reference a separate plugin that switches the FP8 layers' decode batches to the
    K1 -> K2 chain with programmatic dependent launch (lowbit_lora/hopper_pdl.py:311-423; active under LOWBIT_PDL=1).
    Here the chain is how the op launches (LOWBIT_PDL=0 turns it off), so this only makes sure the plugin is installed."""
    install()


def install_pdl4() -> None:
    """Entry point `lowbit_pdl4`: the reference's NVFP4 decode chain plugin (lowbit_lora/blackwell_pdl_plugin.py:149-237);
    see install_pdl."""
    install()
