"""ctypes binding of libonebase_b200.so (the C ABI declared in include/onebase_b200.h).

The library is the only compute path: there is no CPU or eager-torch fallback.  If the shared object is missing the
import of this module raises with the build command; every entry point's status is checked and a non-zero status raises.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "lib" / "libonebase_b200.so"

OB_MAX_SLICES = 4
OB_STATUS_WORDS = 16
OB_BASE_FP8, OB_BASE_NVFP4 = 0, 1
OB_LORA_BF16, OB_LORA_FP8, OB_LORA_NVFP4 = 0, 1, 2
OB_X_PLAIN, OB_X_SILU_MUL = 0, 1
OB_WS = {name: i for i, name in enumerate(("status", "counters", "sx", "xq", "xsf", "hp", "part", "xs", "hb", "hcat"))}


class ObError(RuntimeError):
    def __init__(self, fn: str, status: int, text: str):
        super().__init__(f"{fn} failed with status {status}: {text}")
        self.status = status


class ObLayerDesc(C.Structure):
    _fields_ = [
        ("base_fmt", C.c_int32), ("lora_fmt", C.c_int32), ("N", C.c_int32), ("K", C.c_int32), ("S", C.c_int32),
        ("L", C.c_int32), ("R", C.c_int32), ("widths", C.c_int32 * OB_MAX_SLICES), ("max_m", C.c_int32),
        ("w_q", C.c_void_p), ("w_sf", C.c_void_p), ("s_w", C.c_void_p), ("x_global", C.c_void_p), ("alpha", C.c_void_p),
        ("a", C.c_void_p * OB_MAX_SLICES), ("b", C.c_void_p * OB_MAX_SLICES), ("sa", C.c_void_p * OB_MAX_SLICES),
        ("sb", C.c_void_p * OB_MAX_SLICES), ("ag", C.c_void_p), ("bg", C.c_void_p), ("quant_rcp_approx", C.c_int32),
        ("b_row0", C.c_int32 * OB_MAX_SLICES), ("b_rows", C.c_int32 * OB_MAX_SLICES),
    ]


class ObBatch(C.Structure):
    _fields_ = [
        ("M", C.c_int32), ("x", C.c_void_p), ("ldx", C.c_int64), ("y", C.c_void_p), ("ldy", C.c_int64),
        ("tok", C.c_void_p), ("srt", C.c_void_p), ("seg_n", C.c_void_p), ("seg_start", C.c_void_p), ("seg_ids", C.c_void_p),
        ("x_op", C.c_int32), ("residual", C.c_void_p), ("ldr", C.c_int64),
    ]


class ObWorkspaceShape(C.Structure):
    _fields_ = [("max_m", C.c_int32), ("max_k", C.c_int32), ("max_n", C.c_int32), ("max_sr", C.c_int32),
                ("max_split1", C.c_int32), ("max_split2", C.c_int32), ("max_l", C.c_int32)]


OB_MAX_RANKS = 8
OB_DTYPE_BF16, OB_DTYPE_F32 = 0, 1
OB_AR_AUTO, OB_AR_ONE_SHOT, OB_AR_TWO_SHOT = 0, 1, 2


class ObComm(C.Structure):
    _fields_ = [("world", C.c_int32), ("rank", C.c_int32), ("bufs", C.c_void_p * OB_MAX_RANKS), ("slot_bytes", C.c_size_t)]


class ObTileCfg(C.Structure):
    _fields_ = [("tn", C.c_int32), ("split2", C.c_int32), ("split1", C.c_int32), ("stages", C.c_int32),
                ("wait_ms", C.c_int32), ("fused", C.c_int32), ("prefill", C.c_int32), ("stream", C.c_int32)]


# every symbol include/onebase_b200.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "ob_version": (C.c_int, []),
    "ob_status_string": (C.c_char_p, [C.c_int]),
    "ob_workspace_bytes": (C.c_int, [C.POINTER(ObWorkspaceShape), C.POINTER(C.c_size_t)]),
    "ob_workspace_offsets": (C.c_int, [C.POINTER(ObWorkspaceShape), C.POINTER(C.c_size_t)]),
    "ob_workspace_region": (C.c_int, [C.POINTER(ObWorkspaceShape), C.c_int, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "ob_layer_create": (C.c_int, [C.POINTER(ObLayerDesc), C.POINTER(C.c_void_p)]),
    "ob_layer_destroy": (C.c_int, [C.c_void_p]),
    "ob_requant_fp8_rows": (C.c_int, [C.c_void_p, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]),
    "ob_requant_nvfp4": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                   C.c_void_p]),
    "ob_resolve_tile": (C.c_int, [C.c_void_p, C.c_int32, C.POINTER(ObTileCfg), C.POINTER(ObTileCfg)]),
    "ob_k1_fp8": (C.c_int, [C.c_void_p, C.POINTER(ObBatch), C.c_void_p, C.POINTER(ObWorkspaceShape), C.POINTER(ObTileCfg),
                            C.c_void_p]),
    "ob_k2_fp8": (C.c_int, [C.c_void_p, C.POINTER(ObBatch), C.c_void_p, C.POINTER(ObWorkspaceShape), C.POINTER(ObTileCfg),
                            C.c_int, C.c_void_p]),
    "ob_k2_fp8_static": (C.c_int, [C.c_void_p, C.POINTER(ObBatch), C.c_void_p, C.POINTER(ObWorkspaceShape),
                                   C.POINTER(ObTileCfg), C.c_int, C.c_void_p]),
    "ob_chain_fp8": (C.c_int, [C.c_void_p, C.POINTER(ObBatch), C.c_void_p, C.POINTER(ObWorkspaceShape),
                               C.POINTER(ObTileCfg), C.c_void_p]),
    "ob_k1_nvfp4": (C.c_int, [C.c_void_p, C.POINTER(ObBatch), C.c_void_p, C.POINTER(ObWorkspaceShape), C.POINTER(ObTileCfg),
                              C.c_void_p]),
    "ob_k2_nvfp4": (C.c_int, [C.c_void_p, C.POINTER(ObBatch), C.c_void_p, C.POINTER(ObWorkspaceShape), C.POINTER(ObTileCfg),
                              C.c_int, C.c_void_p]),
    "ob_chain_nvfp4": (C.c_int, [C.c_void_p, C.POINTER(ObBatch), C.c_void_p, C.POINTER(ObWorkspaceShape),
                                 C.POINTER(ObTileCfg), C.c_void_p]),
    "ob_nvfp4_packed_scale_bytes": (C.c_int, [C.c_int32, C.c_int32, C.POINTER(C.c_int32), C.POINTER(C.c_size_t)]),
    "ob_nvfp4_pack_scales": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.POINTER(C.c_int32), C.c_void_p, C.c_size_t,
                                       C.c_void_p]),
    "ob_segment_index": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                   C.c_void_p, C.c_void_p]),
    "ob_comm_bytes": (C.c_int, [C.c_size_t, C.POINTER(C.c_size_t)]),
    "ob_ipc_export": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_size_t)]),
    "ob_ipc_open": (C.c_int, [C.c_char_p, C.c_size_t, C.POINTER(C.c_void_p)]),
    "ob_ipc_close": (C.c_int, [C.c_void_p, C.c_size_t]),
    "ob_allreduce": (C.c_int, [C.POINTER(ObComm), C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "ob_allreduce_emulated": (C.c_int, [C.POINTER(ObComm), C.c_int32, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_int64,
                                        C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "ob_chain_allreduce": (C.c_int, [C.c_void_p, C.POINTER(ObBatch), C.c_void_p, C.POINTER(ObWorkspaceShape), C.POINTER(ObTileCfg),
                                     C.POINTER(ObComm), C.c_void_p]),
    "ob_comm_status": (C.c_int, [C.POINTER(ObComm), C.POINTER(C.c_int32), C.c_void_p]),
    "ob_trace_buffer": (C.c_int, [C.c_void_p, C.c_int64]),
    "ob_read_status": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32), C.c_void_p]),
}

_lib = None


def lib() -> C.CDLL:
    """The loaded library (loaded once).  Raises if it has not been built."""
    global _lib
    if _lib is None:
        path = Path(os.environ.get("ONEBASE_B200_LIB", LIB_PATH))
        if not path.exists():
            raise ImportError(f"{path} not found: build it with `python -m onebase_b200.build` "
                              "(onebase_b200 has no fallback path without its CUDA library)")
        handle = C.CDLL(str(path))
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(fn: str, status: int) -> None:
    if status != 0:
        raise ObError(fn, status, lib().ob_status_string(status).decode())


def call(fn: str, *args) -> None:
    check(fn, getattr(lib(), fn)(*args))
