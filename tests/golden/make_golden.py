"""Generate the golden fixtures in this directory by RUNNING THE REFERENCE on the CPU.

Run once, in a container that has the reference checkout and vLLM importable:

    REFERENCE_ROOT=<path to the fatebreaker/onebase checkout> python tests/golden/make_golden.py

It imports the reference's own torch path (lowbit_lora.kernels.fp8_lora_multi.reference_multi,
lowbit_lora.kernels.nvfp4_lora_vllm.{nvfp4_quant_torch,nvfp4_quant_batched,nvfp4_dequant_torch,reference,
global_scale_for}, lowbit_lora.kernels.adapter_store.AdapterStore) and vLLM's LoRAKernelMeta, feeds them seeded inputs
and stores inputs + outputs as .npz files (bf16 as raw uint16, e4m3 as raw uint8).  The tests never import the
reference; they read these files.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, os.environ.get("REFERENCE_ROOT", "/root/reference"))

from lowbit_lora.kernels import fp8_lora_multi as FM                      # noqa: E402
from lowbit_lora.kernels import nvfp4_lora_vllm as N4                     # noqa: E402
from lowbit_lora.kernels.adapter_store import AdapterStore               # noqa: E402
from vllm.lora.ops.triton_ops.lora_kernel_metadata import LoRAKernelMeta  # noqa: E402


def raw(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float8_e4m3fn:
        return t.contiguous().view(torch.uint8).numpy()
    return t.contiguous().numpy()


def tq(x):
    """The reference's stand-alone per-token rule (tests/pdl_k2_interp_check.py:56-59), run through reference_multi's own
    lines by calling it with an empty adapter set would not expose the codes, so the same two torch lines are used."""
    xf = x.float()
    sx = (xf.abs().amax(dim=1) / 448.0).clamp_min(1.0 / (448.0 * 512.0))
    return (xf / sx[:, None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn), sx


def fp8_quant_case() -> None:
    g = torch.Generator().manual_seed(11)
    x = torch.randn(24, 256, generator=g)
    x[1] = 0.0                                   # all-zero row: the scale floor
    x[2] *= 1e-6                                 # below the floor
    x[3] *= 300.0                                # large
    x[4, :16] = torch.tensor([448.0, -448.0, 0.0625, 17.0, 18.0, 19.0, 20.0, 22.0, 26.0, 30.0, 1.0, -1.0,
                              3.5, 4.5, 5.5, 6.5])  # scale 1: ties between e4m3 codes
    x[4, 16:] = 0.0
    x[5] = x[5].abs() * 0 + 7.0                  # constant row
    x = x.to(torch.bfloat16)
    q, sx = tq(x)
    np.savez_compressed(HERE / "fp8_quant.npz", x=raw(x), codes=raw(q), sx=raw(sx))


def meta_sequence_case() -> None:
    """A sequence of steps through ONE LoRAKernelMeta (state carries over): mixed, smaller mixed, none (stale), single,
    padded (poisoned stale entries beyond the real tokens)."""
    L, max_m = 6, 48
    meta = LoRAKernelMeta.make(L, max_m, device="cpu")
    meta.token_lora_mapping.zero_()
    meta.token_indices_sorted_by_lora_ids.zero_()
    g = torch.Generator().manual_seed(5)
    out = {"L": np.int32(L), "max_m": np.int32(max_m)}
    steps = []
    for i, (m, kind) in enumerate([(21, "mixed"), (5, "mixed"), (13, "none"), (40, "single"), (24, "padded"),
                                   (1, "one"), (33, "nolast"), (7, "none")]):
        if kind == "mixed":
            tok = torch.randint(-1, L - 1, (m,), generator=g, dtype=torch.int32)
        elif kind == "single":
            tok = torch.full((m,), L - 1, dtype=torch.int32)
        elif kind == "one":
            tok = torch.tensor([2], dtype=torch.int32)
        elif kind == "nolast":
            tok = torch.randint(0, L, (m,), generator=g, dtype=torch.int32)
        else:
            tok = torch.full((m,), -1, dtype=torch.int32)
        given = tok
        if kind == "padded":
            tok = torch.randint(-1, L - 1, (m,), generator=g, dtype=torch.int32)
            tok[0] = 0
            meta.token_indices_sorted_by_lora_ids[m - 5:m] = 10 ** 6
            meta.token_lora_mapping[m - 5:m] = L - 1
            given = tok[: m - 5]
        meta.prepare_tensors(given)
        a = meta.meta_args(m, False)
        out[f"s{i}_given"] = raw(given)
        out[f"s{i}_m"] = np.int32(m)
        for name, t in zip(("tok", "srt", "seg_n", "seg_start", "seg_ids"), a[:5]):
            out[f"s{i}_{name}"] = raw(t.clone())
        steps.append(kind)
    out["kinds"] = np.array(steps)
    np.savez_compressed(HERE / "segment_index.npz", **out)


def fp8_projection_cases() -> None:
    torch.manual_seed(0)
    out = {}
    cases = [(64, (32, 16, 16), 16, 4, 21), (96, (64,), 32, 3, 40), (128, (32, 16, 16, 32), 16, 3, 13),
             (256, (128, 128), 64, 8, 32)]
    for ci, (K, widths, R, L, M) in enumerate(cases):
        N, S = sum(widths), len(widths)
        w = torch.randn(N, K) * 0.05
        s_w = (w.abs().max() / 448.0).reshape(1).float()
        w_q = (w / s_w).to(torch.float8_e4m3fn)
        a_st = tuple((torch.randn(L, 1, R, K) / K ** 0.5).to(torch.bfloat16) for _ in range(S))
        b_st = tuple((torch.randn(L, 1, n, R) * 0.05).to(torch.bfloat16) for n in widths)
        A = torch.cat([t[:, 0] for t in a_st], dim=1)
        B = torch.cat([t[:, 0] for t in b_st], dim=1)
        x = torch.randn(M, K).to(torch.bfloat16)
        tok = torch.randint(-1, L, (M,), dtype=torch.int32)
        y = FM.reference_multi(x, tok, w_q, s_w, A, B, widths, 1.0)
        p = f"c{ci}_"
        out.update({p + "K": np.int32(K), p + "widths": np.array(widths, dtype=np.int32), p + "R": np.int32(R),
                    p + "L": np.int32(L), p + "x": raw(x), p + "w_q": raw(w_q), p + "s_w": raw(s_w), p + "tok": raw(tok),
                    p + "y": raw(y)})
        for s in range(S):
            out[p + f"a{s}"] = raw(a_st[s])
            out[p + f"b{s}"] = raw(b_st[s])
        for fmt in ("fp8", "nvfp4"):
            st = AdapterStore(a_st, b_st, fmt)
            Ad, Bd = st.dequantized()
            out[p + f"{fmt}_y"] = raw(FM.reference_multi(x, tok, w_q, s_w, Ad, Bd, widths, 1.0))
            for s in range(S):
                out[p + f"{fmt}_aq{s}"] = raw(st.a_q[s])
                out[p + f"{fmt}_as{s}"] = raw(st.a_s[s])
                out[p + f"{fmt}_bq{s}"] = raw(st.b_q[s])
                out[p + f"{fmt}_bs{s}"] = raw(st.b_s[s])
            if fmt == "nvfp4":
                out[p + "nvfp4_ag"] = raw(st.ag)
                out[p + "nvfp4_bg"] = raw(st.bg)
    out["n_cases"] = np.int32(len(cases))
    np.savez_compressed(HERE / "fp8_projection.npz", **out)


def nvfp4_cases() -> None:
    torch.manual_seed(0)
    out = {}
    cases = [(64, (32, 16, 16), 16, 4, 21), (128, (64,), 32, 3, 24), (256, (128, 64), 64, 5, 32)]
    for ci, (K, widths, R, L, M) in enumerate(cases):
        N, S = sum(widths), len(widths)
        w = torch.randn(N, K) * 0.05
        w_global = N4.global_scale_for(w)
        w_q, w_sf = N4.nvfp4_quant_torch(w, w_global)
        a_st = tuple((torch.randn(L, 1, R, K) / K ** 0.5).to(torch.bfloat16) for _ in range(S))
        b_st = tuple((torch.randn(L, 1, n, R) * 0.05).to(torch.bfloat16) for n in widths)
        A = torch.cat([t[:, 0] for t in a_st], dim=1)
        B = torch.cat([t[:, 0] for t in b_st], dim=1)
        x = torch.randn(M, K).to(torch.bfloat16)
        x[:, :3] *= 8
        if ci == 0:
            x[2] = 0.0                                                   # zero blocks: the zero-scale guard
        x_global = N4.global_scale_for(x)
        xq, xsf = N4.nvfp4_quant_torch(x, x_global)
        tok = torch.randint(-1, L, (M,), dtype=torch.int32)
        y = N4.reference(x, tok, w_q, w_sf, w_global, x_global, A, B, widths)
        p = f"c{ci}_"
        out.update({p + "K": np.int32(K), p + "widths": np.array(widths, dtype=np.int32), p + "R": np.int32(R),
                    p + "L": np.int32(L), p + "x": raw(x), p + "w": raw(w), p + "w_q": raw(w_q), p + "w_sf": raw(w_sf),
                    p + "w_global": np.float64(w_global), p + "x_global": np.float64(x_global), p + "xq": raw(xq),
                    p + "xsf": raw(xsf), p + "tok": raw(tok), p + "y": raw(y),
                    p + "w_deq": raw(N4.nvfp4_dequant_torch(w_q, w_sf, w_global))})
        for s in range(S):
            out[p + f"a{s}"] = raw(a_st[s])
            out[p + f"b{s}"] = raw(b_st[s])
    # e2m1 rounding: every threshold, its neighbours, and saturation, at out_scale 1 (block scale 1 with global 1)
    pts = [0.0, 0.2, 0.25, 0.2500001, 0.3, 0.7, 0.75, 0.8, 1.2, 1.25, 1.2500001, 1.3, 1.7, 1.75, 1.8, 2.4, 2.5, 2.5000002,
           2.6, 3.4, 3.5, 3.6, 4.9, 5.0, 5.0000005, 5.1, 6.0, 7.0, 100.0, 6.0, 6.0, 6.0]
    v = torch.tensor(pts + [-p_ for p_ in pts], dtype=torch.float32).reshape(4, 16)
    v[:, 15] = 6.0                                                       # each block's max is 6: block scale exactly 1
    q, sf = N4.nvfp4_quant_torch(v, 1.0)
    out.update({"ties_x": raw(v), "ties_q": raw(q), "ties_sf": raw(sf)})
    out["n_cases"] = np.int32(len(cases))
    np.savez_compressed(HERE / "nvfp4.npz", **out)


if __name__ == "__main__":
    fp8_quant_case()
    meta_sequence_case()
    fp8_projection_cases()
    nvfp4_cases()
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size, "bytes")
