"""A bounded device-side wait that runs out: the kernel records it in the workspace's status words, stores nothing, leaves
the context usable, and the next ordinary call is correct.

The wait is made to expire on the host's side only -- nothing faults or spins without a limit: the one-kernel form of the
decode chain (ObTileCfg.fused) hands out the quantization of the batch's positions from a work counter in the workspace;
the test presets that counter past the batch, so no CTA quantizes anything, the count of quantized positions every CTA's
weight producer waits for is never reached, and each wait gives up after `wait_ms` (5 ms here).  The reference bounds
its device-side spins the same way (lowbit_lora/kernels/fp8_lora_pdl.py:302-311)."""
from __future__ import annotations

import pytest
import torch

from helpers import build_fp8_op, device_meta, make_index, max_err_ratio, oracle_y
from oracle import configs

pytestmark = pytest.mark.gpu

ARRIVAL_COUNTERS = 4096          # the split-K arrival counters; the chain's work counters follow them in the same region
WORK_QUANT = ARRIVAL_COUNTERS + 2


def test_expired_wait_sets_status_stores_nothing_and_next_call_is_correct():
    d = configs.with_fp8_base(configs.draw(1024, (256, 128), 32, 4, 12, seed=3, ids_low=-1, w_std=0.05, b_std=0.05))
    op = build_fp8_op(d, max_m=32)
    idx = make_index(d["ids"], 4, 32)
    meta = device_meta(idx, 12)
    x = d["x"].cuda()
    y_ok = op(x, meta).clone()
    torch.cuda.synchronize()
    assert op.scratch.status()[0] == 0

    counters = op.scratch.region("counters", 4 * (ARRIVAL_COUNTERS + 16)).view(torch.int32)
    counters[WORK_QUANT] = 1 << 20                              # "every position is already taken": nobody quantizes
    sentinel = 123.0
    y = torch.full_like(y_ok, sentinel)
    op(x, meta, out=y, cfg={"fused": 1, "wait_ms": 5})
    torch.cuda.synchronize()                                    # the launch ends by itself, a few wait limits later
    status = op.scratch.status()                                # reads and clears the status words
    assert status[0] == 1, status[:8]                           # OB_DEV_WAIT_TIMEOUT
    assert status[1] != 0                                       # ... and where
    assert bool((y == sentinel).all()), "a launch whose wait ran out must not store"

    counters.zero_()                                            # the workspace is the caller's: back to its initial state
    y_after = op(x, meta)
    torch.cuda.synchronize()
    assert op.scratch.status()[0] == 0
    assert torch.equal(y_after, y_ok)
    assert max_err_ratio(y_after, oracle_y(d, d["x"], d["ids"])) <= 2e-2
