"""CPU-side checks of the C-ABI boundary: the library loads, exports every symbol the header declares, sizes the
workspace, and rejects bad arguments with a negative status before any launch.  No compute call is made."""
from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

import pytest
import torch

from onebase_b200 import _lib

HEADER = Path(__file__).resolve().parent.parent / "include" / "onebase_b200.h"


def declared_symbols() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(ob_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.lib()
    names = declared_symbols()
    assert len(names) >= 11
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
        assert n in _lib.SYMBOLS, f"{n} has no ctypes signature"
    assert set(_lib.SYMBOLS) == set(names)
    assert lib.ob_version() == 1
    assert b"tile" in lib.ob_status_string(-5)


def test_struct_sizes_match_header_layout(tmp_path):
    """Compile the header as plain C and compare sizeof / offsetof with the ctypes mirrors."""
    import shutil
    import subprocess
    if not shutil.which("gcc"):
        pytest.skip("no gcc")
    src = tmp_path / "sizes.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "onebase_b200.h"\nint main(void) {\n'
                   'printf("%zu %zu %zu %zu %zu %zu %zu\\n", sizeof(ObLayerDesc), sizeof(ObBatch), sizeof(ObWorkspaceShape),'
                   ' sizeof(ObTileCfg), offsetof(ObLayerDesc, w_q), offsetof(ObLayerDesc, bg), offsetof(ObBatch, seg_ids));\n'
                   'return 0; }\n')
    exe = tmp_path / "sizes"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", str(HEADER.parent), str(src), "-o", str(exe)], check=True)
    got = [int(v) for v in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    want = [C.sizeof(_lib.ObLayerDesc), C.sizeof(_lib.ObBatch), C.sizeof(_lib.ObWorkspaceShape), C.sizeof(_lib.ObTileCfg),
            _lib.ObLayerDesc.w_q.offset, _lib.ObLayerDesc.bg.offset, _lib.ObBatch.seg_ids.offset]
    assert got == want


def test_workspace_sizing():
    n1, n2 = C.c_size_t(), C.c_size_t()
    s = _lib.ObWorkspaceShape(32, 12288, 24576, 192, 32, 8)
    _lib.call("ob_workspace_bytes", C.byref(s), C.byref(n1))
    offs = (C.c_size_t * 7)()
    _lib.call("ob_workspace_offsets", C.byref(s), offs)
    o = [int(v) for v in offs]
    assert o == sorted(o) and all(v % 1024 == 0 for v in o) and o[-1] < n1.value
    s2 = _lib.ObWorkspaceShape(64, 12288, 24576, 192, 32, 8)
    _lib.call("ob_workspace_bytes", C.byref(s2), C.byref(n2))
    assert n2.value > n1.value
    bad = _lib.ObWorkspaceShape(0, 12288, 24576, 192, 32, 8)
    assert _lib.lib().ob_workspace_bytes(C.byref(bad), C.byref(n1)) == -2
    assert _lib.lib().ob_workspace_bytes(None, C.byref(n1)) == -1


def _desc(**over):
    d = _lib.ObLayerDesc()
    d.base_fmt, d.lora_fmt = 0, 0
    d.N, d.K, d.S, d.L, d.R, d.max_m = 256, 256, 2, 4, 16, 8
    d.widths[0], d.widths[1] = 128, 128
    fake = 0x10000                                        # never dereferenced on the host
    d.w_q, d.s_w = fake, fake
    for s in range(2):
        d.a[s], d.b[s] = fake, fake
    for k, v in over.items():
        setattr(d, k, v)
    return d


@pytest.mark.parametrize("over,status", [
    ({"R": 24}, -2), ({"K": 100}, -2), ({"S": 5}, -2), ({"N": 300}, -2), ({"base_fmt": 7}, -6), ({"lora_fmt": 9}, -6),
    ({"w_q": None}, -1), ({"s_w": None}, -1), ({"w_q": 0x10004}, -3), ({"max_m": 0}, -2), ({"L": 0}, -2),
])
def test_layer_create_rejects_before_touching_the_device(over, status):
    h = C.c_void_p()
    assert _lib.lib().ob_layer_create(C.byref(_desc(**over)), C.byref(h)) == status
    assert not h.value


def test_layer_create_without_a_driver_reports_it():
    if torch.cuda.is_available():
        pytest.skip("a CUDA driver is present")
    h = C.c_void_p()
    assert _lib.lib().ob_layer_create(C.byref(_desc()), C.byref(h)) == -8
    assert _lib.lib().ob_layer_create(C.byref(_desc()), None) == -1


def test_compute_entry_points_reject_null_arguments():
    lib = _lib.lib()
    assert lib.ob_k1_fp8(None, None, None, None, None, None) == -1
    assert lib.ob_k2_fp8(None, None, None, None, None, 0, None) == -1
    assert lib.ob_chain_fp8(None, None, None, None, None, None) == -1
    assert lib.ob_segment_index(None, 4, 4, None, None, None, None, None, None) == -1
    assert lib.ob_read_status(None, None, None) == -1


def test_product_has_no_cpu_path():
    from onebase_b200.kernels.fp8_lora_vllm import VllmFusedFP8LoRA
    w = torch.zeros(128, 128).to(torch.float8_e4m3fn)
    a = (torch.zeros(2, 1, 16, 128, dtype=torch.bfloat16),)
    b = (torch.zeros(2, 1, 128, 16, dtype=torch.bfloat16),)
    with pytest.raises(RuntimeError, match="CUDA devices only"):
        VllmFusedFP8LoRA(w, torch.ones(1), a, b, 8)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setenv("ONEBASE_B200_LIB", str(tmp_path / "nope.so"))
    monkeypatch.setattr(_lib, "_lib", None)
    with pytest.raises(ImportError, match="no fallback"):
        _lib.lib()
    monkeypatch.undo()
    _lib.lib()


def test_tile_table_lookup_and_fallback(tmp_path, monkeypatch):
    from onebase_b200 import tile_table
    f = tmp_path / "extra.jsonl"
    f.write_text('{"M": 32, "N": 1000, "K": 512, "S": 1, "R": 16, "fmt": "fp8", "tn": 32, "split2": 3, "split1": 2, "stages": 4}\n'
                 '{"M": 32, "N": 1000, "K": 512, "S": 1, "R": 16, "fmt": "fp8", "adapters": "nvfp4", "split2": 2}\n')
    monkeypatch.setenv("LOWBIT_PDL_CFG", str(f))
    tile_table.reload()
    assert tile_table.tile_for(32, 1000, 512, 1, 16, "fp8") == {"tn": 32, "split2": 3, "split1": 2, "stages": 4}
    near = tile_table.tile_for(16, 1000, 512, 1, 16, "fp8")     # the bucket next to it of the same shape, token tile not inherited
    assert near == {"split2": 3, "split1": 2, "stages": 4}
    assert tile_table.tile_for(2048, 1000, 512, 1, 16, "fp8") == {}   # a decode row says nothing about a prefill batch
    assert tile_table.tile_for(32, 999, 512, 1, 16, "fp8") == {}
    # rows are per adapter storage: a bf16-adapter row is not applied to stored adapters, nor the other way round
    assert tile_table.tile_for(32, 1000, 512, 1, 16, "fp8", "fp8") == {}
    assert tile_table.tile_for(32, 1000, 512, 1, 16, "fp8", "nvfp4") == {"split2": 2}
    assert tile_table.tile_for(16, 1000, 512, 1, 16, "fp8", "nvfp4") == {"split2": 2}
    monkeypatch.delenv("LOWBIT_PDL_CFG")
    tile_table.reload()


def test_bench_workload_helpers():
    """The bench's host-side arithmetic: the Zipf(1.1) prefill split covers every token and every tenant in contiguous
    runs, and the per-format algorithmic bytes agree with the per-projection table the main line reports."""
    import bench
    for M in (512, 2048, 8192):
        ids = bench.zipf_ids(M, seed=1)
        assert ids.numel() == M and ids.dtype == torch.int32
        counts = torch.bincount(ids.long(), minlength=bench.L_SLOTS)
        assert int(counts.min()) >= 1 and int(counts.sum()) == M
        top = counts.sort(descending=True).values.double()
        assert abs(float(top[0] / top[1]) - 2 ** 1.1) < 0.15            # sizes follow 1 / rank^1.1
        assert int((ids[1:] != ids[:-1]).sum()) == bench.L_SLOTS - 1    # one contiguous run per tenant
    fp8_bf16 = bench.format_bytes(32, 23, "fp8", "bf16")
    assert fp8_bf16 == sum(v["total"] for v in bench.layer_bytes(32, 23).values())
    w_fp8 = sum(sum(w) * K for K, w in bench.PROJECTIONS.values())
    assert fp8_bf16 - bench.format_bytes(32, 23, "nvfp4", "bf16") == int(w_fp8 * (1 - 0.5625))
    assert bench.format_bytes(32, 23, "fp8", "nvfp4") < bench.format_bytes(32, 23, "fp8", "fp8") < fp8_bf16
