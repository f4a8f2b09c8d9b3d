"""Fused FP8 base + multi-tenant LoRA for one vLLM LoRA layer, on B200 through libonebase_b200.so.

Host-side mirror of the reference's op object `VllmFusedFP8LoRA` (lowbit_lora/kernels/fp8_lora_vllm.py:416-765) and of
its decode-chain launcher `run_pdl` (lowbit_lora/hopper_pdl.py:104-175): same constructor arguments, same call
signature `op(x, meta_args, out=None)`, same attributes (N, K, S, L, R, widths, end0..2, scratch, max_m), same slot
maintenance calls (`requantize`, `release`), same shared per-device scratch grown before any CUDA graph is captured.
What differs is below the call: two hand-written sm_100a kernels (K1 quantize+shrink, K2 tcgen05 GEMM+expand) linked by
programmatic dependent launch, chosen by a per-shape tile table instead of a timed dispatch.
"""
from __future__ import annotations

import ctypes as C

import torch

from onebase_b200 import _lib
from onebase_b200.kernels.adapter_store import AdapterStore
from onebase_b200.tile_table import tile_for

FP8_MAX = 448.0
_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192, 1 << 30)   # fp8_lora_vllm.py:349


def _bucket(M: int) -> int:
    return next(b for b in _BUCKETS if M <= b)


def fill_adapter_pointers(d: "_lib.ObLayerDesc", store: AdapterStore) -> None:
    """The adapter pointer tables of a layer descriptor (reference: a_ptrs / b_ptrs / sa_ptrs / sb_ptrs, fp8_lora_vllm.py:
    440-441,477-493)."""
    d.lora_fmt = {"bf16": _lib.OB_LORA_BF16, "fp8": _lib.OB_LORA_FP8, "nvfp4": _lib.OB_LORA_NVFP4}[store.fmt]
    for s in range(store.S):
        d.a[s] = store.a_q[s].data_ptr()
        d.b[s] = store.b_q[s].data_ptr()
        if store.fmt != "bf16":
            d.sa[s] = store.a_s[s].data_ptr()
            d.sb[s] = store.b_s[s].data_ptr()
    if store.fmt == "nvfp4":
        d.ag, d.bg = store.ag.data_ptr(), store.bg.data_ptr()


class Scratch:
    """The workspace shared by every fused layer on one device (reference: `Scratch`, fp8_lora_vllm.py:315-346): status
    words, split-K counters, per-position scales `sx`, activation codes `xq`, shrink partials `hp`, GEMM split-K partials.
    `ensure` grows it to the largest request; it must reach its final size before a CUDA graph is captured."""

    MAX_SPLIT1 = 32
    MAX_SPLIT2 = 8

    def __init__(self, device):
        self.device = torch.device(device)
        self.shape = _lib.ObWorkspaceShape(0, 0, 0, 0, self.MAX_SPLIT1, 1)
        self.buf = None
        self.offsets = None

    def ensure(self, max_m: int, K: int, N: int, SR: int, split2: int = 1, L: int = 0) -> None:
        s = self.shape
        want = (max(s.max_m, max_m), max(s.max_k, K), max(s.max_n, N), max(s.max_sr, SR), max(s.max_split2, split2),
                max(s.max_l, L))
        if self.buf is not None and want == (s.max_m, s.max_k, s.max_n, s.max_sr, s.max_split2, s.max_l):
            return
        s.max_m, s.max_k, s.max_n, s.max_sr, s.max_split2, s.max_l = want
        nbytes = C.c_size_t()
        _lib.call("ob_workspace_bytes", C.byref(s), C.byref(nbytes))
        self.offsets, self.sizes = {}, {}
        for name, rid in _lib.OB_WS.items():
            off, size = C.c_size_t(), C.c_size_t()
            _lib.call("ob_workspace_region", C.byref(s), rid, C.byref(off), C.byref(size))
            self.offsets[name], self.sizes[name] = int(off.value), int(size.value)
        # over-allocate so that the base can be rounded up to the 1024-byte alignment the TMA descriptors need
        raw = torch.zeros(nbytes.value + 1024, dtype=torch.uint8, device=self.device)
        skew = (-raw.data_ptr()) % 1024
        self._raw = raw
        self.buf = raw[skew: skew + nbytes.value]

    @property
    def ptr(self) -> int:
        return self.buf.data_ptr()

    def region(self, name: str, nbytes: int) -> torch.Tensor:
        o = self.offsets[name]
        return self.buf[o: o + nbytes]

    def sx(self, M: int) -> torch.Tensor:
        """Per-POSITION activation scales of the last call, fp32 [M]."""
        return self.region("sx", 4 * M).view(torch.float32)

    def xq(self, M: int, K: int) -> torch.Tensor:
        """Per-POSITION e4m3 codes of the last call, [M, K] (position p holds the token row the sort put there)."""
        return self.region("xq", M * K).view(torch.float8_e4m3fn).view(M, K)

    def hb(self, S: int, R: int) -> torch.Tensor:
        """The tensor-core shrink's finished h of the last prefill call, bf16 [S, max_m, R] at adapter-sorted positions."""
        max_m = self.shape.max_m
        return self.region("hb", 2 * S * max_m * R).view(torch.bfloat16).view(S, max_m, R)

    def status(self, stream=None) -> list[int]:
        out = (C.c_int32 * _lib.OB_STATUS_WORDS)()
        st = stream if stream is not None else torch.cuda.current_stream(self.device).cuda_stream
        _lib.call("ob_read_status", C.c_void_p(self.ptr), out, C.c_void_p(st))
        return list(out)


_SCRATCH: dict = {}


def shared_scratch(device) -> Scratch:
    key = str(torch.device(device))
    if key not in _SCRATCH:
        _SCRATCH[key] = Scratch(device)
    return _SCRATCH[key]


class VllmFusedFP8LoRA:
    """Fused base + LoRA for one vLLM LoRA layer whose base is per-tensor FP8 (e4m3).

    w_q [N, K] float8_e4m3fn (= base_layer.weight.t(), contiguous), s_w [1] fp32; a_stacked / b_stacked: vLLM's tuples of
    per-slice buffers [L, 1, R, K] / [L, 1, N_s, R] (bf16, alpha/r folded into B); max_m = the engine's max tokens per
    forward.  Tokens are described by vLLM's LoRAKernelMeta tensors (tok, srt, seg_n, seg_start, seg_ids)."""

    _K1, _K2, _CHAIN, _FMT = "ob_k1_fp8", "ob_k2_fp8", "ob_chain_fp8", "fp8"   # entry points and tile-table format key

    def __init__(self, w_q, s_w, a_stacked, b_stacked, max_m, *, split_k=None, lora_fp8=False, lora_fp4=False,
                 b_shard=None):
        if w_q.device.type != "cuda":
            raise RuntimeError("onebase_b200 runs on CUDA devices only (there is no CPU path)")
        self.w_q, self.s_w = w_q, s_w.reshape(1).to(torch.float32)
        self.N, self.K = w_q.shape
        self.S = len(a_stacked)
        self.L, _, self.R, k_a = a_stacked[0].shape
        assert w_q.dtype == torch.float8_e4m3fn and w_q.is_contiguous()
        assert k_a == self.K and all(t.dtype == torch.bfloat16 and t.is_contiguous() for t in (*a_stacked, *b_stacked))
        # b_shard = [(first row, rows, slice width), ...] per slice: this rank holds only those rows of each slice's B
        # (vLLM's row-parallel layers with sharded adapters); the expand then covers those output features only
        self.b_shard = b_shard
        widths = [t.shape[2] for t in b_stacked] if b_shard is None else [int(w) for _, _, w in b_shard]
        assert sum(widths) == self.N and self.S <= 4
        assert b_shard is None or (not lora_fp8 and not lora_fp4 and
                                   all(t.shape[2] == rows for t, (_, rows, _) in zip(b_stacked, b_shard)))
        ends = [sum(widths[:i + 1]) for i in range(self.S)]
        self.end0 = ends[0] if self.S >= 2 else self.N
        self.end1 = ends[1] if self.S >= 3 else self.N
        self.end2 = ends[2] if self.S >= 4 else self.N
        self.widths = widths
        self.a_stacked, self.b_stacked = a_stacked, b_stacked            # keep the buffers alive
        self.max_m = int(max_m)
        self.split_k = split_k                                           # shrink split-K override (None: tile table)
        self.lora_fp8, self.lora_fp4 = lora_fp8, lora_fp4
        assert not (lora_fp8 and lora_fp4)
        self.device = w_q.device
        self.store = AdapterStore(a_stacked, b_stacked, "nvfp4" if lora_fp4 else "fp8" if lora_fp8 else "bf16")
        self.scratch = shared_scratch(self.device)
        self.scratch.ensure(self.max_m, self.K, self.N, self.S * self.R, Scratch.MAX_SPLIT2, self.L)
        self.dispatch = {}                                               # kept for report compatibility: always fused
        self.wait_ms = 2000
        d = _lib.ObLayerDesc()
        d.base_fmt = _lib.OB_BASE_FP8
        d.N, d.K, d.S, d.L, d.R, d.max_m = self.N, self.K, self.S, self.L, self.R, self.max_m
        for s in range(self.S):
            d.widths[s] = widths[s]
        fill_adapter_pointers(d, self.store)
        if b_shard is not None:
            for s, (row0, rows, _) in enumerate(b_shard):
                d.b_row0[s], d.b_rows[s] = int(row0), int(rows)
        d.w_q, d.s_w = w_q.data_ptr(), self.s_w.data_ptr()
        self._desc = d
        h = C.c_void_p()
        with torch.cuda.device(self.device):
            _lib.call("ob_layer_create", C.byref(d), C.byref(h))
        self._h = h

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            try:
                _lib.lib().ob_layer_destroy(h)
            except Exception:   # noqa: BLE001 - interpreter shutdown: the library may already be gone
                pass
            self._h = None

    # ------------------------------------------------------------------------------------------------- tile choice
    def tile(self, M: int, cfg: dict | None = None) -> _lib.ObTileCfg:
        # rows are keyed by the adapters' storage too: one swept with bf16 adapters is not applied to stored ones
        adapters = "nvfp4" if self.lora_fp4 else "fp8" if self.lora_fp8 else "bf16"
        c = dict(tile_for(_bucket(M), self.N, self.K, self.S, self.R, self._FMT, adapters))
        if self.split_k:
            c["split1"] = self.split_k
        if cfg:
            c.update(cfg)
        return _lib.ObTileCfg(c.get("tn", 0), c.get("split2", 0), c.get("split1", 0), c.get("stages", 0),
                              c.get("wait_ms", self.wait_ms), c.get("fused", 0), c.get("prefill", 0), c.get("stream", 0))

    def resolved_tile(self, M: int, cfg: dict | None = None) -> dict:
        """The tile choice a call of M tokens runs with, the library's own rule filled in (ob_resolve_tile)."""
        out = _lib.ObTileCfg()
        _lib.call("ob_resolve_tile", self._h, int(M), C.byref(self.tile(M, cfg)), C.byref(out))
        return {k: getattr(out, k) for k in ("tn", "split2", "split1", "stages", "fused", "stream", "prefill")}

    def shrink_partials(self, M: int, cfg: dict | None = None) -> torch.Tensor:
        """The fp32 shrink partials the last K1 call of M tokens wrote, [split1, S, max_m, R], as a view of the workspace:
        what a row-parallel layer with sharded adapters all-reduces between K1 and K2."""
        split1 = self.resolved_tile(M, cfg)["split1"]
        max_m = self.scratch.shape.max_m
        n = split1 * self.S * max_m * self.R
        return self.scratch.region("hp", 4 * n).view(torch.float32).view(split1, self.S, max_m, self.R)

    # ------------------------------------------------------------------------------------------------- the call
    def _batch(self, x, meta_args, out, silu_mul: bool = False, residual=None):
        tok, srt, seg_n, seg_start, seg_ids = meta_args[:5]
        M = x.shape[0]
        assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
        assert x.shape[1] == (2 * self.K if silu_mul else self.K)
        y = out if out is not None else torch.empty(M, self.N, dtype=torch.bfloat16, device=x.device)
        assert y.dtype == torch.bfloat16 and y.stride(1) == 1
        for t in (tok, srt, seg_n, seg_start, seg_ids):
            assert t.dtype == torch.int32 and t.is_cuda
        b = _lib.ObBatch(M, x.data_ptr(), x.stride(0), y.data_ptr(), y.stride(0), tok.data_ptr(), srt.data_ptr(),
                         seg_n.data_ptr(), seg_start.data_ptr(), seg_ids.data_ptr())
        b.x_op = _lib.OB_X_SILU_MUL if silu_mul else _lib.OB_X_PLAIN
        if residual is not None:
            assert residual.dtype == torch.bfloat16 and residual.shape == (M, self.N) and residual.stride(1) == 1
            b.residual, b.ldr = residual.data_ptr(), residual.stride(0)
        return b, y

    def __call__(self, x, meta_args, out=None, cfg: dict | None = None, pdl: bool = True, shrink: bool = True,
                 gemm: bool = True, allreduce=None, silu_mul: bool = False, residual=None):
        """y = x W^T (FP8, x quantized per token as vLLM does) + every tenant's expansion.  pdl=False runs the same two
        kernels serialized; shrink=False / gemm=False run one kernel alone (breakdowns and tests).  allreduce = a
        tp.PeerComm: this is a row-parallel shard and y is summed over the ranks inside K2's epilogue (ob_chain_allreduce).
        silu_mul=True: x is the merged gate | up output [M, 2K] and the projection's input is silu(gate) * up, formed inside
        K1 (down_proj).  residual = [M, N] bf16: K2 stores y + residual, the new residual stream (o_proj, down_proj)."""
        b, y = self._batch(x, meta_args, out, silu_mul, residual)
        t = self.tile(b.M, cfg)
        ws, sh = C.c_void_p(self.scratch.ptr), C.byref(self.scratch.shape)
        st = C.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)
        if allreduce is not None:
            assert shrink and gemm and y.is_contiguous()
            _lib.call("ob_chain_allreduce", self._h, C.byref(b), ws, sh, C.byref(t), C.byref(allreduce.comm), st)
        elif shrink and gemm and pdl:
            _lib.call(self._CHAIN, self._h, C.byref(b), ws, sh, C.byref(t), st)
        else:
            if shrink:
                _lib.call(self._K1, self._h, C.byref(b), ws, sh, C.byref(t), st)
            if gemm:
                _lib.call(self._K2, self._h, C.byref(b), ws, sh, C.byref(t), 0, st)
        return y

    def warmup(self) -> None:
        """Nothing to compile or time at load: kernels are prebuilt and tiles come from the table.  Grows the scratch to
        its final size (before CUDA-graph capture), as the reference's warm-up does (fp8_lora_vllm.py:598-617)."""
        self.scratch.ensure(self.max_m, self.K, self.N, self.S * self.R, Scratch.MAX_SPLIT2, self.L)

    def requantize(self, index: int | None = None) -> None:
        """Refresh the low-precision copy of one slot (or all) from vLLM's bf16 slots after vLLM wrote or cleared it
        (reference: fp8_lora_vllm.py:504-524).  bf16 adapters are read in place: nothing to do."""
        self.store.requantize(index)

    def release(self, a_stage, b_stage) -> None:
        """Serve from the low-precision copies alone; vLLM then writes every adapter through one staging slot
        (reference: fp8_lora_vllm.py:498-502)."""
        assert self.lora_fp8 or self.lora_fp4
        self.store.release(a_stage, b_stage)
        self.a_stacked, self.b_stacked = a_stage, b_stage

    # the reference exposes the copies under these names (tests read them)
    a8 = property(lambda self: self.store.a_q)
    b8 = property(lambda self: self.store.b_q)
    sa = property(lambda self: self.store.a_s)
    sb = property(lambda self: self.store.b_s)
    a4 = property(lambda self: self.store.a_q)
    b4 = property(lambda self: self.store.b_q)
    a4s = property(lambda self: self.store.a_s)
    b4s = property(lambda self: self.store.b_s)
    ag = property(lambda self: self.store.ag)
    bg = property(lambda self: self.store.bg)


def run_pdl(op: VllmFusedFP8LoRA, x, meta_args, cfg: dict | None = None, out=None, pdl: bool = True, shrink: bool = True,
            gemm: bool = True):
    """The decode chain K1 -> K2 with programmatic dependent launch (reference: lowbit_lora/hopper_pdl.py:104-175)."""
    return op(x, meta_args, out=out, cfg=cfg, pdl=pdl, shrink=shrink, gemm=gemm)
