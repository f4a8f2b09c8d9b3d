"""Low-precision copies of vLLM's stacked LoRA buffers, for serving adapters FP8- or NVFP4-stored.

vLLM keeps each slice's adapters as lora_a_stacked[s] [L,1,R,K] and lora_b_stacked[s] [L,1,N_s,R] (bf16).  The fused
kernels can read, instead, one low-precision copy per buffer and dequantize it in registers (K1: A, K2: B):
  fp8    e4m3 codes of the same shape + one fp32 scale per matrix row (A: [L,R], B: [L,N_s]): amax / 448, floor 1e-12
  nvfp4  e2m1 codes packed two per byte along the last axis (A: [L,1,R,K/2], B: [L,1,N_s,R/2]), one ue4m3 scale per 16
         elements ([.., last/16]) and one inverse global scale per (slice, slot) ([S,L]): global = 448 * 6 / amax
The storage formats, the attribute names (`a_q`, `b_q`, `a_s`, `b_s`, `ag`, `bg`) and the calls (`requantize`, `release`)
are those of the reference's `AdapterStore` (lowbit_lora/kernels/adapter_store.py:21-94) and of
`VllmFusedFP8LoRA.requantize` (lowbit_lora/kernels/fp8_lora_vllm.py:504-524), because the op objects and the plugin are
written against them.  The copies themselves are made by the library's requantization kernels -- one launch per buffer,
bit-identical to the reference's torch recipes (tests/test_requant_gpu.py) -- and only on CUDA tensors: like the rest of
the package there is no host path.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from onebase_b200 import _lib


def _ptr(t: torch.Tensor) -> C.c_void_p:
    return C.c_void_p(t.data_ptr())


def _stream(t: torch.Tensor) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _device_only(t: torch.Tensor, multiple: int) -> torch.Tensor:
    if not t.is_cuda or t.dtype != torch.bfloat16 or t.shape[-1] % multiple != 0:
        raise RuntimeError(f"onebase_b200 requantizes bf16 CUDA tensors whose last dimension is a multiple of {multiple} "
                           f"(got {t.dtype} {tuple(t.shape)} on {t.device}); there is no host path")
    return t.contiguous()


def store_rows_fp8(t: torch.Tensor):
    """t [..., cols] bf16 on the device -> (e4m3 codes of the same shape, fp32 scale per row), one kernel launch."""
    src = _device_only(t, 8)
    codes = torch.empty(src.shape, dtype=torch.float8_e4m3fn, device=src.device)
    scale = torch.empty(src.shape[:-1], dtype=torch.float32, device=src.device)
    with torch.cuda.device(src.device):
        _lib.call("ob_requant_fp8_rows", _ptr(src), src.numel() // src.shape[-1], src.shape[-1], _ptr(codes), _ptr(scale),
                  _stream(src))
    return codes, scale


def quant_stack_nvfp4(t: torch.Tensor):
    """t [l, rows, cols] bf16 on the device -> (packed [l, rows, cols/2] uint8, block scales [l, rows, cols/16] e4m3,
    inverse global scales [l] fp32): one amax pass and one quantizing pass."""
    src = _device_only(t, 16)
    l, rows, cols = src.shape
    packed = torch.empty(l, rows, cols // 2, dtype=torch.uint8, device=src.device)
    sf = torch.empty(l, rows, cols // 16, dtype=torch.float8_e4m3fn, device=src.device)
    inv_g = torch.empty(l, dtype=torch.float32, device=src.device)
    amax = torch.empty(l, dtype=torch.int32, device=src.device)
    with torch.cuda.device(src.device):
        _lib.call("ob_requant_nvfp4", _ptr(src), l, rows, cols, _ptr(packed), _ptr(sf), _ptr(inv_g), _ptr(amax), _stream(src))
    return packed, sf, inv_g


@dataclass
class _Copy:
    """The low-precision copy of ONE stacked buffer (matrix A or B of one slice)."""
    codes: torch.Tensor                # fp8: [L,1,rows,cols] e4m3; nvfp4: [L,1,rows,cols/2] uint8
    scales: torch.Tensor               # fp8: [L,rows] fp32;        nvfp4: [L,1,rows,cols/16] e4m3
    inv_global: torch.Tensor | None    # nvfp4: this slice's row of the [S,L] table (a view); fp8: None

    def refresh(self, fmt: str, src: torch.Tensor, slots: slice) -> None:
        """Requantize `src` [n,1,rows,cols] (n slots of vLLM's buffer, or the one staging slot) into slots `slots`."""
        mats = src[:, 0]
        if fmt == "fp8":
            codes, scale = store_rows_fp8(mats)
            self.codes[slots, 0] = codes
            self.scales[slots] = scale
        else:
            packed, sf, inv_g = quant_stack_nvfp4(mats)
            self.codes[slots, 0] = packed
            self.scales[slots, 0] = sf
            self.inv_global[slots] = inv_g


def _blank_copy(fmt: str, like: torch.Tensor, inv_global: torch.Tensor | None) -> _Copy:
    L, _, rows, cols = like.shape
    dev = like.device
    if fmt == "fp8":
        return _Copy(torch.zeros(L, 1, rows, cols, dtype=torch.float8_e4m3fn, device=dev),
                     torch.zeros(L, rows, dtype=torch.float32, device=dev), None)
    if cols % 16 != 0:
        raise RuntimeError(f"NVFP4-stored adapters need a last dimension that is a multiple of 16, got {cols}")
    return _Copy(torch.zeros(L, 1, rows, cols // 2, dtype=torch.uint8, device=dev),
                 torch.zeros(L, 1, rows, cols // 16, dtype=torch.float8_e4m3fn, device=dev), inv_global)


class AdapterStore:
    """fmt "bf16": nothing is copied, the kernels read vLLM's buffers in place.  "fp8" / "nvfp4": one `_Copy` per buffer,
    filled at construction and refreshed per slot by `requantize`."""

    def __init__(self, a_stacked, b_stacked, fmt: str):
        if fmt not in ("bf16", "fp8", "nvfp4"):
            raise ValueError(f"unknown adapter storage format {fmt!r}")
        self.fmt = fmt
        self.a_stacked, self.b_stacked = a_stacked, b_stacked
        self.staged = False               # after release(): a_stacked / b_stacked are ONE staging slot each, not L slots
        self.S = len(a_stacked)
        self.L, _, self.R, self.K = a_stacked[0].shape
        self.ag = self.bg = None
        self._a: list[_Copy] = []
        self._b: list[_Copy] = []
        if fmt == "bf16":
            return
        dev = a_stacked[0].device
        if fmt == "nvfp4":
            self.ag = torch.zeros(self.S, self.L, dtype=torch.float32, device=dev)
            self.bg = torch.zeros(self.S, self.L, dtype=torch.float32, device=dev)
        for s in range(self.S):
            self._a.append(_blank_copy(fmt, a_stacked[s], None if self.ag is None else self.ag[s]))
            self._b.append(_blank_copy(fmt, b_stacked[s], None if self.bg is None else self.bg[s]))
        self.requantize()

    # what the kernels' pointer tables and the tests read: per-slice tuples of codes and scales
    @property
    def a_q(self):
        return tuple(self.a_stacked) if self.fmt == "bf16" else tuple(c.codes for c in self._a)

    @property
    def b_q(self):
        return tuple(self.b_stacked) if self.fmt == "bf16" else tuple(c.codes for c in self._b)

    @property
    def a_s(self):
        return None if self.fmt == "bf16" else tuple(c.scales for c in self._a)

    @property
    def b_s(self):
        return None if self.fmt == "bf16" else tuple(c.scales for c in self._b)

    def release(self, a_stage, b_stage) -> None:
        """From now on the copies are the only per-slot storage: vLLM's L bf16 slots are replaced by one staging slot per
        buffer (a_stage[s] [1,1,R,K], b_stage[s] [1,1,N_s,R]) that it writes every adapter through; `requantize(i)`
        then files the staging slot's content under slot i."""
        if self.fmt == "bf16":
            raise RuntimeError("bf16 adapters are served from vLLM's own slots: there is nothing to release them to")
        self.a_stacked, self.b_stacked, self.staged = a_stage, b_stage, True

    @torch.no_grad()
    def requantize(self, index: int | None = None) -> None:
        """Refresh slot `index` (all slots if None) of every copy from vLLM's buffers, after vLLM wrote or cleared it."""
        if self.fmt == "bf16":
            return
        if self.staged and index is None:
            raise RuntimeError("with released slots only one slot at a time can be refreshed (from the staging slot)")
        dst = slice(None) if index is None else slice(index, index + 1)
        src = slice(0, 1) if self.staged else dst
        for s in range(self.S):
            self._a[s].refresh(self.fmt, self.a_stacked[s][src], dst)
            self._b[s].refresh(self.fmt, self.b_stacked[s][src], dst)
