"""Sweep the tile choices of the FP8 decode chain on this GPU and write the rows of a tile table.

    python -m onebase_b200.tiles.sweep [--out onebase_b200/tiles/qwen3_8b_fp8.jsonl] [--ms 1,2,4,8,16,32]

For every Qwen3-8B projection shape and decode batch size it times the K1 -> K2 chain (one CUDA-graph replay, L2
flushed before each, median of the replays) over GEMM split-K x ring depth, then over the shrink's split-K at the best
pair, and keeps the fastest.  This replaces the reference's load-time timed dispatch by a table measured once per GPU
model (the reference ships such sweeps as results/pdl_k2*.jsonl).
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

PROJECTIONS = {"qkv": (4096, (4096, 1024, 1024)), "o": (4096, (4096,)), "gate_up": (4096, (12288, 12288)),
               "down": (12288, (4096,))}
L_SLOTS, RANK = 32, 64


def time_chain(op, x, meta, y, cfg, flush, reps=15):
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        op(x, meta, out=y, cfg=cfg)
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        op(x, meta, out=y, cfg=cfg)
    ts = []
    for i in range(reps + 3):
        flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        e1.synchronize()
        if i >= 3:
            ts.append(e0.elapsed_time(e1) * 1e3)
    return statistics.median(ts)


def main() -> None:
    from onebase_b200 import _lib
    from onebase_b200.kernels.fp8_lora_vllm import VllmFusedFP8LoRA
    from onebase_b200.metadata import KernelMeta
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=str(Path(__file__).resolve().parent / "qwen3_8b_fp8.jsonl"))
    ap.add_argument("--ms", default="1,2,4,8,16,32")
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    g = torch.Generator(device=dev).manual_seed(0)
    rows = []
    for name, (K, widths) in PROJECTIONS.items():
        N = sum(widths)
        w_q = (torch.randn(N, K, device=dev, generator=g) * 0.5).to(torch.float8_e4m3fn)
        s_w = torch.full((1,), 0.01, device=dev)
        a_st = tuple((torch.randn(L_SLOTS, 1, RANK, K, device=dev, generator=g) / K ** 0.5).to(torch.bfloat16) for _ in widths)
        b_st = tuple((torch.randn(L_SLOTS, 1, n, RANK, device=dev, generator=g) * 0.01).to(torch.bfloat16) for n in widths)
        op = VllmFusedFP8LoRA(w_q, s_w, a_st, b_st, max_m=32)
        for M in (int(v) for v in args.ms.split(",")):
            ids = torch.randint(0, L_SLOTS, (M,), generator=torch.Generator().manual_seed(M), dtype=torch.int32).to(dev)
            km = KernelMeta.make(L_SLOTS, M, dev)
            km.prepare_tensors(ids)
            meta = km.meta_args(M)
            x = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
            y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
            default_us = time_chain(op, x, meta, y, {}, flush, reps=25)
            best = (default_us, {})
            tried = 1
            for split2 in (1, 2, 3, 4, 6, 8):
                for stages in (0, 3, 4):
                    cfg = {"split2": split2, **({"stages": stages} if stages else {})}
                    try:
                        us = time_chain(op, x, meta, y, cfg, flush)
                    except _lib.ObError:
                        continue
                    tried += 1
                    if us < best[0]:
                        best = (us, dict(cfg))
            for split1 in (1, 2, 4, 8, 16):
                cfg = dict(best[1], split1=split1)
                try:
                    us = time_chain(op, x, meta, y, cfg, flush)
                except _lib.ObError:
                    continue
                tried += 1
                if us < best[0]:
                    best = (us, cfg)
            if best[1]:   # confirm with more replays; a choice must beat the library's own rule by 3 % to enter the table
                again = time_chain(op, x, meta, y, best[1], flush, reps=25)
                best = (again, best[1]) if again < 0.97 * default_us else (default_us, {})
            status = op.scratch.status()
            assert status[0] == 0, status[:8]
            row = {"M": M, "N": N, "K": K, "S": len(widths), "R": RANK, "fmt": "fp8", **best[1], "us": round(best[0], 2),
                   "default_us": round(default_us, 2), "proj": name, "tried": tried, "gpu": torch.cuda.get_device_name(0)}
            rows.append(row)
            print(json.dumps(row), flush=True)
        del op
    Path(args.out).write_text("".join(json.dumps(r) + "\n" for r in rows))


if __name__ == "__main__":
    main()
