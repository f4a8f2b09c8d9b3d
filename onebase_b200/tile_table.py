"""Per-shape tile table: which token tile, GEMM split-K, shrink split-K and ring depth a call uses.

Replaces the reference's load-time timed dispatch (`tune_dispatch`, lowbit_lora/kernels/fp8_lora_vllm.py:554-596) with a
lookup, keyed like the reference's swept tables (lowbit_lora/hopper_pdl.py:268-298): (M bucket, N, K, S, R, base format)
plus the adapters' storage format ("adapters": "bf16" when a row does not say; a row swept with bf16 adapters says
nothing about a layer whose B tiles are dequantized inside the kernel).
Rows live in `tiles/*.jsonl` next to this file (one JSON object per line: the key fields plus tn / split2 / split1 /
stages).  A shape without a row falls back to the M bucket next to it of the same (N, K, S, R, formats), then to the
library's own rule (an empty dict: every field 0 = default).  LOWBIT_PDL_CFG=<file> adds rows from another file, which
win over the shipped ones.
"""
from __future__ import annotations

import json
import os
from pathlib import Path

_TABLE: dict | None = None


def _load() -> dict:
    table: dict = {}
    files = sorted((Path(__file__).resolve().parent / "tiles").glob("*.jsonl"))
    extra = os.environ.get("LOWBIT_PDL_CFG")
    if extra:
        files.append(Path(extra))
    for f in files:
        if not f.exists():
            continue
        for line in f.read_text().splitlines():
            line = line.strip()
            if not line or line.startswith("#"):
                continue
            row = json.loads(line)
            key = (int(row["M"]), int(row["N"]), int(row["K"]), int(row["S"]), int(row["R"]), str(row.get("fmt", "fp8")),
                   str(row.get("adapters", "bf16")))
            table[key] = {k: int(row[k]) for k in ("tn", "split2", "split1", "stages", "fused", "prefill", "stream") if k in row}
    return table


def tile_for(m_bucket: int, N: int, K: int, S: int, R: int, fmt: str, adapters: str = "bf16") -> dict:
    global _TABLE
    if _TABLE is None:
        _TABLE = _load()
    hit = _TABLE.get((m_bucket, N, K, S, R, fmt, adapters))
    if hit is not None:
        return hit
    # A neighbouring bucket's choice carries over only within one doubling: the swept rows are decode sizes, and their
    # split-K choices are not even valid for a prefill batch (several token tiles cannot be split along K).
    near = [(abs(k[0].bit_length() - m_bucket.bit_length()), k) for k in _TABLE if k[1:] == (N, K, S, R, fmt, adapters)]
    near = [n for n in near if n[0] <= 1]
    if near:
        cfg = dict(_TABLE[min(near)[1]])
        cfg.pop("tn", None)                      # the token tile follows the batch, not the neighbouring bucket
        return cfg
    return {}


def reload() -> None:
    global _TABLE
    _TABLE = None
