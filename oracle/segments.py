"""Oracle (test infrastructure, CPU torch): the token sort / segment index the kernels consume.

Producer side: vLLM's `LoRAKernelMeta.prepare_tensors` (vllm/lora/ops/triton_ops/lora_kernel_metadata.py:110-168), the
third-party step that builds the five int32 tensors (token map, token indices sorted by slot id, tokens per segment,
segment start offsets, segment slot ids).  Restated here with its statefulness: the buffers persist across steps, a
batch without any adapter only resets the three segment arrays and leaves the token map and the sorted indices stale.
Consumer side: how the reference's GEMM turns those tensors into the row and adapter of every tile position
(lowbit_lora/kernels/fp8_lora_vllm.py:147-163), including CUDA-graph padding rows and stale entries.
"""
from __future__ import annotations

import torch


class SegmentIndex:
    """Persistent metadata buffers for up to `max_loras` slots and `max_tokens` tokens."""

    def __init__(self, max_loras: int, max_tokens: int):
        self.L = max_loras
        self.tok = torch.zeros(max_tokens, dtype=torch.int32)            # token -> slot id (-1: none)
        self.srt = torch.zeros(max_tokens, dtype=torch.int32)            # token indices sorted by slot id (stable)
        self.seg_n = torch.zeros(max_loras + 1, dtype=torch.int32)       # tokens per segment
        self.seg_start = torch.zeros(max_loras + 2, dtype=torch.int32)   # exclusive prefix sum, first entry 0
        self.seg_ids = torch.full((max_loras + 1,), -1, dtype=torch.int32)   # slot id of each segment, -1 padded

    def prepare(self, token_lora: torch.Tensor) -> None:
        self.seg_ids.fill_(-1)
        self.seg_n.fill_(0)
        self.seg_start.fill_(0)
        ids = token_lora.to(torch.int32)
        if bool((ids == -1).all()):
            return                                                       # token map and sorted indices stay stale
        n = ids.numel()
        self.tok[:n] = ids
        # stable sort by slot id: counting sort keeps the arrival order inside a segment
        order = sorted(range(n), key=lambda i: int(ids[i]))
        self.srt[:n] = torch.tensor(order, dtype=torch.int32)
        uniq = sorted(set(int(v) for v in ids))
        counts = [int((ids == u).sum()) for u in uniq]
        self.seg_ids[: len(uniq)] = torch.tensor(uniq, dtype=torch.int32)
        self.seg_n[: len(uniq)] = torch.tensor(counts, dtype=torch.int32)
        self.seg_start[1: 1 + len(uniq)] = torch.cumsum(torch.tensor(counts, dtype=torch.int32), 0).to(torch.int32)

    def args(self, m: int):
        """The five tensors in the order the fused op takes them: tok[:m], srt[:m], seg_n, seg_start, seg_ids."""
        return self.tok[:m], self.srt[:m], self.seg_n, self.seg_start, self.seg_ids


def resolve_positions(m: int, tok, srt, seg_n, seg_start, seg_ids) -> tuple[torch.Tensor, torch.Tensor]:
    """Row and adapter of each of the m tile positions, as the reference's GEMM derives them:
    n_all = sum(seg_n), n_ad = sum of seg_n over segments with a slot id >= 0.  If n_ad > 0, positions p < n_all run the
    adapter-sorted order (row = clamp(srt[p], 0, m-1), adapter = tok[row]); every other position is its own row without
    an adapter (natural order; CUDA-graph padding).  Returns (rows int64 [m], adapters int64 [m])."""
    n_all = int(seg_n.sum())
    n_ad = int(seg_n[seg_ids >= 0].sum())
    rows = torch.arange(m, dtype=torch.int64)
    ads = torch.full((m,), -1, dtype=torch.int64)
    if n_ad > 0:
        k = min(n_all, m)
        r = srt[:k].to(torch.int64).clamp(0, m - 1)
        rows[:k] = r
        ads[:k] = tok.to(torch.int64)[r]
    return rows, ads


def effective_token_lora(m: int, tok, srt, seg_n, seg_start, seg_ids) -> torch.Tensor:
    """The adapter each TOKEN ROW ends up with (what a reference call with these tensors computes): -1 for padding rows
    and for every row of a batch whose metadata names no adapter."""
    rows, ads = resolve_positions(m, tok, srt, seg_n, seg_start, seg_ids)
    out = torch.full((m,), -1, dtype=torch.int32)
    out[rows] = ads.to(torch.int32)
    return out
