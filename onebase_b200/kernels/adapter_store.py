"""Low-precision copies of vLLM's stacked LoRA buffers (FP8- and NVFP4-stored adapter modes).

Mirror of the reference's `AdapterStore` (lowbit_lora/kernels/adapter_store.py:21-94) and of
`VllmFusedFP8LoRA.requantize` (lowbit_lora/kernels/fp8_lora_vllm.py:504-524).  vLLM keeps each slice's adapters as
lora_a_stacked[s] [L,1,R,K] and lora_b_stacked[s] [L,1,N_s,R] (bf16); the store holds, per slice,
  fp8:   e4m3 copies with one fp32 scale per row of A ([L,R]) and of B ([L,N_s]): amax / 448 floored at 1e-12;
  nvfp4: e2m1 codes packed along K (A: [L,1,R,K/2]) and along R (B: [L,1,N_s,R/2]), ue4m3 scales per 16 elements and
         one inverse global scale per adapter and slice ([S,L]): global = 448 * 6 / amax (the reference's batched recipe,
         lowbit_lora/kernels/nvfp4_lora_vllm.py:379-397, exact reciprocals).
The kernels dequantize these in registers (K1: A; K2: B).  `requantize(index)` refreshes one slot (or all) after vLLM
writes or clears it; after `release()`, vLLM writes every slot through one staging slot and the copies are the only
per-slot storage.  On the device the copies are made by the library's requantization kernels (one launch per buffer;
the reference does it with torch ops: slot writes happen outside CUDA graphs); host tensors take the torch recipe.
"""
from __future__ import annotations

import torch

FP8_MAX = 448.0
E2M1_MAX = 6.0


def _c(value: float, like: torch.Tensor) -> torch.Tensor:
    """A 0-dim fp32 tensor on `like`'s device.  Divisions are written tensor / tensor on purpose: on CUDA torch turns
    `tensor / python_scalar` into a multiplication by the scalar's reciprocal, which is not the IEEE quotient and would
    move a scale by one ulp (and with it some codes) against the CPU recipe."""
    return torch.tensor(value, dtype=torch.float32, device=like.device)


def _stream(t: torch.Tensor):
    import ctypes as C
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def store_rows_fp8(t: torch.Tensor):
    """t [..., cols] bf16 -> (e4m3 codes of the same shape, fp32 scale per row).  On a CUDA tensor this is one launch of
    the library's requantization kernel (ob_requant_fp8_rows); the torch lines below are the same arithmetic for host
    tensors (the CPU tests compare the two through the golden fixtures)."""
    if t.is_cuda and t.dtype == torch.bfloat16 and t.shape[-1] % 8 == 0:
        import ctypes as C
        from onebase_b200 import _lib
        src = t.contiguous()
        rows = src.numel() // src.shape[-1]
        codes = torch.empty(src.shape, dtype=torch.float8_e4m3fn, device=t.device)
        scale = torch.empty(src.shape[:-1], dtype=torch.float32, device=t.device)
        with torch.cuda.device(t.device):
            _lib.call("ob_requant_fp8_rows", C.c_void_p(src.data_ptr()), rows, src.shape[-1], C.c_void_p(codes.data_ptr()),
                      C.c_void_p(scale.data_ptr()), _stream(t))
        return codes, scale
    tf = t.float()
    scale = torch.div(tf.abs().amax(-1), _c(FP8_MAX, tf)).clamp_min(1e-12)
    return torch.div(tf, scale[..., None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn), scale


def quant_stack_nvfp4(t: torch.Tensor):
    """t [l, rows, cols] -> (packed [l, rows, cols/2] uint8, block scales [l, rows, cols/16] e4m3, inverse globals [l])."""
    l, rows, cols = t.shape
    if t.is_cuda and t.dtype == torch.bfloat16 and cols % 16 == 0:   # one amax pass + one quantizing pass on the device
        import ctypes as C
        from onebase_b200 import _lib
        src = t.contiguous()
        packed = torch.empty(l, rows, cols // 2, dtype=torch.uint8, device=t.device)
        sf = torch.empty(l, rows, cols // 16, dtype=torch.float8_e4m3fn, device=t.device)
        inv_g = torch.empty(l, dtype=torch.float32, device=t.device)
        amax = torch.empty(l, dtype=torch.int32, device=t.device)
        with torch.cuda.device(t.device):
            _lib.call("ob_requant_nvfp4", C.c_void_p(src.data_ptr()), l, rows, cols, C.c_void_p(packed.data_ptr()),
                      C.c_void_p(sf.data_ptr()), C.c_void_p(inv_g.data_ptr()), C.c_void_p(amax.data_ptr()), _stream(t))
        return packed, sf, inv_g
    tf = t.float()
    one = _c(1.0, tf)
    # `scalar / tensor` in torch is reciprocal(tensor) * scalar (two roundings): the reference's global scale is that value
    gs = (torch.reciprocal(tf.abs().amax(dim=(1, 2)).clamp_min(1e-12)) * (448.0 * E2M1_MAX)).float()
    xb = tf.reshape(l, rows, cols // 16, 16)
    g = gs.view(l, 1, 1, 1)
    vmax = xb.abs().amax(-1, keepdim=True)
    sf = (g * (vmax * (1.0 / E2M1_MAX))).clamp(max=448.0).to(torch.float8_e4m3fn)
    sff = sf.float()
    osc = torch.where(sff != 0, torch.div(one, sff * torch.div(one, g)), torch.zeros_like(sff))
    v = xb * osc
    a = v.abs()
    code = ((a > 0.25).int() + (a >= 0.75).int() + (a > 1.25).int() + (a >= 1.75).int() + (a > 2.5).int()
            + (a >= 3.5).int() + (a > 5.0).int() + 8 * (v < 0).int()).reshape(l, rows, cols // 2, 2)
    packed = (code[..., 0] | (code[..., 1] << 4)).to(torch.uint8)
    return packed, sf.reshape(l, rows, cols // 16), torch.div(one, gs).float()


class AdapterStore:
    def __init__(self, a_stacked, b_stacked, fmt: str):
        assert fmt in ("bf16", "fp8", "nvfp4")
        self.fmt, self.a_stacked, self.b_stacked = fmt, a_stacked, b_stacked
        self.staged = False
        dev = a_stacked[0].device
        self.S = len(a_stacked)
        self.L, _, self.R, self.K = a_stacked[0].shape
        widths = [t.shape[2] for t in b_stacked]
        self.ag = self.bg = None
        if fmt == "bf16":
            self.a_q, self.b_q, self.a_s, self.b_s = a_stacked, b_stacked, None, None
            return
        if fmt == "fp8":
            self.a_q = tuple(torch.zeros(t.shape, dtype=torch.float8_e4m3fn, device=dev) for t in a_stacked)
            self.b_q = tuple(torch.zeros(t.shape, dtype=torch.float8_e4m3fn, device=dev) for t in b_stacked)
            self.a_s = tuple(torch.zeros(self.L, self.R, dtype=torch.float32, device=dev) for _ in a_stacked)
            self.b_s = tuple(torch.zeros(self.L, w, dtype=torch.float32, device=dev) for w in widths)
        else:
            assert self.R % 16 == 0 and self.K % 16 == 0
            self.a_q = tuple(torch.zeros(self.L, 1, self.R, self.K // 2, dtype=torch.uint8, device=dev) for _ in a_stacked)
            self.a_s = tuple(torch.zeros(self.L, 1, self.R, self.K // 16, dtype=torch.float8_e4m3fn, device=dev)
                             for _ in a_stacked)
            self.b_q = tuple(torch.zeros(self.L, 1, w, self.R // 2, dtype=torch.uint8, device=dev) for w in widths)
            self.b_s = tuple(torch.zeros(self.L, 1, w, self.R // 16, dtype=torch.float8_e4m3fn, device=dev) for w in widths)
            self.ag = torch.zeros(self.S, self.L, dtype=torch.float32, device=dev)
            self.bg = torch.zeros(self.S, self.L, dtype=torch.float32, device=dev)
        self.requantize()

    def release(self, a_stage, b_stage) -> None:
        """Serve from the low-precision copies alone: vLLM's per-slot bf16 buffers give way to one staging slot
        (a_stage[s] [1,1,R,K], b_stage[s] [1,1,N_s,R]); requantize(index) then reads slot 0 of the staging buffers."""
        assert self.fmt != "bf16"
        self.a_stacked, self.b_stacked, self.staged = a_stage, b_stage, True

    @torch.no_grad()
    def requantize(self, index: int | None = None) -> None:
        if self.fmt == "bf16":
            return
        assert not (self.staged and index is None)
        idx = slice(None) if index is None else slice(index, index + 1)
        sidx = slice(0, 1) if self.staged else idx
        for src, q, sc, g in ((self.a_stacked, self.a_q, self.a_s, self.ag), (self.b_stacked, self.b_q, self.b_s, self.bg)):
            for s in range(self.S):
                t = src[s][sidx, 0]
                if self.fmt == "fp8":
                    codes, scale = store_rows_fp8(t)
                    q[s][idx, 0] = codes
                    sc[s][idx] = scale
                else:
                    packed, sf, inv_g = quant_stack_nvfp4(t)
                    q[s][idx, 0], sc[s][idx, 0], g[s, idx] = packed, sf, inv_g
