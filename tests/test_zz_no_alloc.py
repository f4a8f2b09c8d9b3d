"""ob_k2_fp8_static: the K2 entry point that keeps its split-K scratch in a fixed device array inside the library.

Some hosts of this library may not allocate device memory at the point where the projection runs: a serving thread
whose memory pool was frozen after warm-up, code running under a stream capture, or a runtime that passes the
library nothing but its tensors.  They cannot grow a workspace when a tile choice needs split-K room, so this variant
takes the room from the library's own static array.  The test runs K1 once, then the GEMM through the ordinary entry
point and through the static one -- twice in a row, since all calls share the one array and each must leave its
arrival counters at zero -- and expects bitwise identical outputs.  (This file sorts last on purpose: if it fails under
`pytest -x`, every other test has already run.)
"""
from __future__ import annotations

import ctypes as C

import pytest
import torch

from helpers import build_fp8_op, device_meta, make_index, max_err_ratio, oracle_y
from oracle import configs

pytestmark = pytest.mark.gpu


def test_static_scratch_gemm_matches_workspace_gemm_twice():
    from onebase_b200 import _lib
    d = configs.with_fp8_base(configs.draw(2048, (384, 128), 32, 6, 19, seed=11, ids_low=-1, w_std=0.05, b_std=0.05))
    op = build_fp8_op(d, max_m=32)
    idx = make_index(d["ids"], 6, 32)
    meta = device_meta(idx, 19)
    x = d["x"].cuda()
    cfg = {"split2": 4, "split1": 2}                       # split-K of the GEMM: the scratch is really used
    y_ref = op(x, meta, pdl=False, cfg=cfg)                # K1 + K2 through the existing entry points
    torch.cuda.synchronize()
    assert op.scratch.status()[0] == 0
    assert max_err_ratio(y_ref, oracle_y(d, d["x"], d["ids"])) <= 2e-2

    tile = op.tile(19, cfg)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    ws, shape = C.c_void_p(op.scratch.ptr), C.byref(op.scratch.shape)
    for call in range(2):
        y = torch.full_like(y_ref, float("nan"))
        batch, _ = op._batch(x, meta, y)
        _lib.call("ob_k2_fp8_static", op._h, C.byref(batch), ws, shape, C.byref(tile), 0, stream)
        torch.cuda.synchronize()
        assert op.scratch.status()[0] == 0
        assert torch.equal(y, y_ref), f"call {call}: static-scratch GEMM differs from the workspace GEMM"


def test_static_scratch_gemm_as_programmatic_dependent_of_k1():
    """K1 through its own entry point, then the static-scratch GEMM launched with the programmatic-launch attribute
    (pdl = 1), twice in a row: bitwise what the workspace GEMM of the same tile choice gives."""
    from onebase_b200 import _lib
    d = configs.with_fp8_base(configs.draw(1024, (256, 256), 64, 8, 27, seed=5, ids_low=-1, w_std=0.05, b_std=0.05))
    op = build_fp8_op(d, max_m=32)
    idx = make_index(d["ids"], 8, 32)
    meta = device_meta(idx, 27)
    x = d["x"].cuda()
    cfg = {"split2": 2, "split1": 4}
    y_ref = op(x, meta, cfg=cfg)
    torch.cuda.synchronize()
    tile = op.tile(27, cfg)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    ws, shape = C.c_void_p(op.scratch.ptr), C.byref(op.scratch.shape)
    for call in range(2):
        y = torch.full_like(y_ref, float("nan"))
        batch, _ = op._batch(x, meta, y)
        _lib.call("ob_k1_fp8", op._h, C.byref(batch), ws, shape, C.byref(tile), stream)
        _lib.call("ob_k2_fp8_static", op._h, C.byref(batch), ws, shape, C.byref(tile), 1, stream)
        torch.cuda.synchronize()
        assert op.scratch.status()[0] == 0
        assert torch.equal(y, y_ref), f"call {call}"


def test_static_scratch_gemm_several_token_tiles_and_large_tiles():
    """Batches of more than one token tile take the same grid order as the workspace GEMM (no split-K there), and a prefill
    batch that the 256 x 256 GEMM serves needs no scratch at all: both bitwise equal to ob_k2_fp8."""
    from onebase_b200 import _lib
    d = configs.with_fp8_base(configs.draw(512, (256, 512), 64, 8, 300, seed=8, ids_low=-1, w_std=0.05, b_std=0.05))
    op = build_fp8_op(d, max_m=300)
    ids = configs.zipf_request_ids(300, 8, seed=2, mean_len=30)
    idx = make_index(ids, 8, 300)
    meta = device_meta(idx, 300)
    x = d["x"].cuda()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    ws, shape = C.c_void_p(op.scratch.ptr), C.byref(op.scratch.shape)
    for cfg in ({"prefill": 2, "tn": 64}, {"prefill": 1}):
        y_ref = op(x, meta, pdl=False, cfg=cfg)
        torch.cuda.synchronize()
        assert max_err_ratio(y_ref, oracle_y(d, d["x"], ids)) <= 2e-2
        tile = op.tile(300, cfg)
        y = torch.full_like(y_ref, float("nan"))
        batch, _ = op._batch(x, meta, y)
        _lib.call("ob_k2_fp8_static", op._h, C.byref(batch), ws, shape, C.byref(tile), 0, stream)
        torch.cuda.synchronize()
        assert op.scratch.status()[0] == 0
        assert torch.equal(y, y_ref), cfg


def test_static_scratch_rejects_oversized_requests():
    from onebase_b200 import _lib
    # 192 output tiles x split 8 x 256 tokens x 128 x 4 B = 201 MB of partials: far beyond the 8 MiB array
    d = configs.with_fp8_base(configs.draw(1024, (24576,), 16, 2, 8, seed=2))
    op = build_fp8_op(d, max_m=256)
    idx = make_index(torch.zeros(200, dtype=torch.int32), 2, 256)
    x = torch.zeros(200, 1024, dtype=torch.bfloat16, device="cuda")
    y = torch.empty(200, 24576, dtype=torch.bfloat16, device="cuda")
    batch, _ = op._batch(x, device_meta(idx, 200), y)
    tile = op.tile(200, {"split2": 8, "tn": 256})
    st = _lib.lib().ob_k2_fp8_static(op._h, C.byref(batch), C.c_void_p(op.scratch.ptr), C.byref(op.scratch.shape),
                                     C.byref(tile), 0, C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == -9
