"""Shared helpers of the GPU parity tests: move oracle-side inputs to the device, build ops, compare."""
from __future__ import annotations

import torch

from oracle import fp8 as ofp8
from oracle import segments as oseg


def device_meta(idx: oseg.SegmentIndex, m: int, device="cuda"):
    """The five metadata tensors of `idx` for an m-token call, on the device (full-capacity buffers, sliced like vLLM)."""
    tok, srt = idx.tok.to(device), idx.srt.to(device)
    return tok[:m], srt[:m], idx.seg_n.to(device), idx.seg_start.to(device), idx.seg_ids.to(device)


def make_index(ids: torch.Tensor, L: int, max_m: int) -> oseg.SegmentIndex:
    idx = oseg.SegmentIndex(L, max_m)
    idx.prepare(ids)
    return idx


def build_fp8_op(d: dict, max_m: int, device="cuda", **kw):
    from onebase_b200.kernels.fp8_lora_vllm import VllmFusedFP8LoRA
    a_st = tuple(t.to(device) for t in d["a_stacked"])
    b_st = tuple(t.to(device) for t in d["b_stacked"])
    return VllmFusedFP8LoRA(d["w_q"].to(device), d["s_w"].to(device), a_st, b_st, max_m, **kw)


def oracle_y(d: dict, x: torch.Tensor, eff_ids: torch.Tensor) -> torch.Tensor:
    A, B = ofp8.stack_slices(d["a_stacked"], d["b_stacked"])
    return ofp8.fused_projection(x, eff_ids, d["w_q"], d["s_w"], A, B, d["widths"])


def max_err_ratio(y: torch.Tensor, ref: torch.Tensor) -> float:
    """max-abs-error / ||ref||_inf (the acceptance bound is 2e-2)."""
    return float((y.float().cpu() - ref).abs().max() / ref.abs().max().clamp_min(1e-30))


def build_nvfp4_op(d: dict, max_m: int, device="cuda", **kw):
    from onebase_b200.kernels.nvfp4_lora_vllm import VllmFusedNVFP4LoRA
    a_st = tuple(t.to(device) for t in d["a_stacked"])
    b_st = tuple(t.to(device) for t in d["b_stacked"])
    return VllmFusedNVFP4LoRA(d["w_q4"].to(device), d["w_sf"].to(device), d["w_global"], d["x_global"], a_st, b_st, max_m, **kw)


def oracle_y_nvfp4(d: dict, x: torch.Tensor, eff_ids: torch.Tensor) -> torch.Tensor:
    from oracle import nvfp4 as on4
    A, B = ofp8.stack_slices(d["a_stacked"], d["b_stacked"])
    return on4.fused_projection(x, eff_ids, d["w_q4"], d["w_sf"], d["w_global"], d["x_global"], A, B, d["widths"])
