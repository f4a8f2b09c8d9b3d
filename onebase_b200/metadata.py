"""Token sort / segment index on the device.

`KernelMeta` has the interface of vLLM's `LoRAKernelMeta` (vllm/lora/ops/triton_ops/lora_kernel_metadata.py:14-200:
`make`, `prepare_tensors`, `meta_args`) and produces the same five tensors bit for bit, but with ONE kernel launch
(`ob_segment_index`) instead of torch sort / unique / cumsum and their small copies.  The stand-alone benches and
tests use it where the plugin receives vLLM's own tensors.
"""
from __future__ import annotations

import ctypes as C

import torch

from onebase_b200 import _lib


class KernelMeta:
    def __init__(self, max_loras: int, max_num_tokens: int, device):
        dev = torch.device(device)
        self.max_loras = max_loras
        self.token_lora_mapping = torch.zeros(max_num_tokens, dtype=torch.int32, device=dev)
        self.token_indices_sorted_by_lora_ids = torch.zeros(max_num_tokens, dtype=torch.int32, device=dev)
        self.num_tokens_per_lora = torch.zeros(max_loras + 1, dtype=torch.int32, device=dev)
        self.lora_token_start_loc = torch.zeros(max_loras + 2, dtype=torch.int32, device=dev)
        self.active_lora_ids = torch.full((max_loras + 1,), -1, dtype=torch.int32, device=dev)

    @staticmethod
    def make(max_loras: int, max_num_tokens: int, device) -> "KernelMeta":
        return KernelMeta(max_loras, max_num_tokens, device)

    def prepare_tensors(self, token_lora_mapping: torch.Tensor) -> None:
        """token_lora_mapping [M] int32 on the device (-1 = no adapter)."""
        t = token_lora_mapping
        assert t.dtype == torch.int32 and t.is_cuda and t.is_contiguous()
        assert t.numel() <= self.token_lora_mapping.numel()
        p = lambda x: C.c_void_p(x.data_ptr())   # noqa: E731
        _lib.call("ob_segment_index", p(t), t.numel(), self.max_loras, p(self.token_lora_mapping),
                  p(self.token_indices_sorted_by_lora_ids), p(self.num_tokens_per_lora), p(self.lora_token_start_loc),
                  p(self.active_lora_ids), C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream))

    def meta_args(self, token_nums: int, specialize_active_lora: bool = False):
        """(tok[:m], srt[:m], seg_n, seg_start, seg_ids): the first five of vLLM's meta_args, in its order."""
        return (self.token_lora_mapping[:token_nums], self.token_indices_sorted_by_lora_ids[:token_nums],
                self.num_tokens_per_lora, self.lora_token_start_loc, self.active_lora_ids)
