"""Fused NVFP4 (W4A4) base + multi-tenant LoRA for one vLLM LoRA layer, on B200 through libonebase_b200.so.

Host-side mirror of the reference's `VllmFusedNVFP4LoRA` (lowbit_lora/kernels/nvfp4_lora_vllm.py:437-630) and of its
decode-chain launcher `run_pdl4` (lowbit_lora/blackwell_pdl.py:59-133), in vLLM's ModelOpt NVFP4 linear format:
W as e2m1 codes packed two per byte along K ([N, K/2] uint8, element 2i in the low nibble), one ue4m3 scale per 16
elements ([N, K/16], the checkpoint's linear layout) and a per-tensor global scale w_global; x quantized per 16-element
block on the fly against a static global scale x_global; y = alpha * sum(v(x) s_x v(w) s_w) + LoRA with
alpha = 1 / (x_global * w_global).  x_global and alpha live on the device ([1] fp32) and may be refilled between calls,
as the reference's tests do.
"""
from __future__ import annotations

import ctypes as C

import torch

from onebase_b200 import _lib
from onebase_b200.kernels.adapter_store import AdapterStore
from onebase_b200.kernels.fp8_lora_vllm import Scratch, VllmFusedFP8LoRA, fill_adapter_pointers, shared_scratch

E2M1_MAX = 6.0


def pack_weight_scales(w_sf: torch.Tensor, K: int, widths) -> torch.Tensor:
    """Linear [N, K/16] ue4m3 block scales -> the per-(tile, K slot) atom order K2 copies to TMEM (one kernel launch)."""
    assert w_sf.is_cuda and w_sf.is_contiguous() and w_sf.element_size() == 1
    wa = (C.c_int32 * len(widths))(*widths)
    n = C.c_size_t()
    _lib.call("ob_nvfp4_packed_scale_bytes", K, len(widths), wa, C.byref(n))
    out = torch.empty(n.value, dtype=torch.uint8, device=w_sf.device)
    _lib.call("ob_nvfp4_pack_scales", C.c_void_p(w_sf.data_ptr()), K, len(widths), wa, C.c_void_p(out.data_ptr()), n.value,
              C.c_void_p(torch.cuda.current_stream(w_sf.device).cuda_stream))
    return out


class VllmFusedNVFP4LoRA(VllmFusedFP8LoRA):
    """w_q [N, K/2] uint8 (packed e2m1), w_sf [N, K/16] float8_e4m3fn (linear layout), w_global and x_global the global
    scales (multipliers: amax -> 448 * 6), a_stacked / b_stacked vLLM's per-slice bf16 adapter buffers.
    rcp_approx=True computes the quantizer's reciprocals with rcp.approx.ftz as vLLM's CUDA kernel does; False uses IEEE
    reciprocals as the torch recipe does (bit-identical to it)."""

    _K1, _K2, _CHAIN, _FMT = "ob_k1_nvfp4", "ob_k2_nvfp4", "ob_chain_nvfp4", "nvfp4"

    def __init__(self, w_q, w_sf, w_global, x_global, a_stacked, b_stacked, max_m, *, split_k=None, lora_fmt="bf16",
                 rcp_approx=False):
        if w_q.device.type != "cuda":
            raise RuntimeError("onebase_b200 runs on CUDA devices only (there is no CPU path)")
        self.w_q, self.w_sf = w_q, w_sf
        self.N = w_q.shape[0]
        self.K = 2 * w_q.shape[1]
        self.S = len(a_stacked)
        self.L, _, self.R, k_a = a_stacked[0].shape
        assert w_q.dtype == torch.uint8 and w_q.is_contiguous() and tuple(w_sf.shape) == (self.N, self.K // 16)
        assert k_a == self.K and all(t.dtype == torch.bfloat16 and t.is_contiguous() for t in (*a_stacked, *b_stacked))
        widths = [t.shape[2] for t in b_stacked]
        assert sum(widths) == self.N and self.S <= 4
        ends = [sum(widths[:i + 1]) for i in range(self.S)]
        self.end0 = ends[0] if self.S >= 2 else self.N
        self.end1 = ends[1] if self.S >= 3 else self.N
        self.end2 = ends[2] if self.S >= 4 else self.N
        self.widths = widths
        self.a_stacked, self.b_stacked = a_stacked, b_stacked
        self.max_m = int(max_m)
        self.split_k = split_k
        self.lora_fmt = lora_fmt
        self.lora_fp8, self.lora_fp4 = lora_fmt == "fp8", lora_fmt == "nvfp4"
        self.device = w_q.device
        self.store = AdapterStore(a_stacked, b_stacked, lora_fmt)
        self.w_global = float(w_global)
        self.x_global = torch.tensor([float(x_global)], dtype=torch.float32, device=self.device)
        self.alpha = torch.tensor([1.0 / (float(x_global) * float(w_global))], dtype=torch.float32, device=self.device)
        self.w_sf_packed = pack_weight_scales(w_sf.contiguous().view(torch.uint8), self.K, widths)
        self.scratch = shared_scratch(self.device)
        self.scratch.ensure(self.max_m, self.K, self.N, self.S * self.R, Scratch.MAX_SPLIT2, self.L)
        self.dispatch = {}
        self.wait_ms = 2000
        d = _lib.ObLayerDesc()
        d.base_fmt = _lib.OB_BASE_NVFP4
        d.N, d.K, d.S, d.L, d.R, d.max_m = self.N, self.K, self.S, self.L, self.R, self.max_m
        for s in range(self.S):
            d.widths[s] = widths[s]
        fill_adapter_pointers(d, self.store)
        d.w_q, d.w_sf = w_q.data_ptr(), self.w_sf_packed.data_ptr()
        d.x_global, d.alpha = self.x_global.data_ptr(), self.alpha.data_ptr()
        d.quant_rcp_approx = 1 if rcp_approx else 0
        self._desc = d
        h = C.c_void_p()
        with torch.cuda.device(self.device):
            _lib.call("ob_layer_create", C.byref(d), C.byref(h))
        self._h = h

    def set_x_global(self, x_global: float) -> None:
        """Refill the static activation scale and alpha on the device (reference: op.x_global.fill_ / op.alpha.fill_)."""
        self.x_global.fill_(float(x_global))
        self.alpha.fill_(1.0 / (float(x_global) * self.w_global))

    def codes(self, M: int, tn: int | None = None):
        """The last call's activation codes and block scales in POSITION order: (packed [M, K/2] uint8, scales [M, K/16]
        float8_e4m3fn, read back out of the scale-factor atoms)."""
        K = self.K
        xq = self.scratch.region("xq", M * (K // 2)).view(M, K // 2)
        if tn is None:   # the token tile the library's own rule gave the last call; 256 under the large-tile prefill GEMM
            rt = self.resolved_tile(M)
            tn = 256 if rt["prefill"] == 1 else rt["tn"]
        nblk = 2 if tn > 128 else 1
        kslots = (K + 255) // 256
        m_tiles = (M + tn - 1) // tn
        raw = self.scratch.region("xsf", m_tiles * kslots * nblk * 2048).view(m_tiles, kslots, nblk, 4, 32, 4, 4)
        # [mt, kb, blk, mma, r32, r4, j] -> [mt, blk, r4, r32, kb, mma, j] = [positions, scale columns]
        lin = raw.permute(0, 2, 5, 4, 1, 3, 6).reshape(m_tiles, nblk * 128, kslots * 16)[:, :tn].reshape(m_tiles * tn, kslots * 16)
        return xq, lin[:M, : K // 16].contiguous().view(torch.float8_e4m3fn)
