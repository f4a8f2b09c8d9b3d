"""Plugin wiring on the CPU with fakes (as the reference's tests/pdl_plugin_check.py and test_release_slots.py do):
install() is inert without LOWBIT_FUSED, idempotent, registers the op with the reference's name and schema, patches
the base class and every class-level `apply` override, builds an op only for eligible layers and reports each decision."""
from __future__ import annotations

import types

import pytest
import torch

vllm = pytest.importorskip("vllm")


class FakeOp:
    made = []

    def __init__(self, *args, **kw):
        self.args, self.kw = args, kw
        self.N = args[0].shape[0]
        self.calls = []
        FakeOp.made.append(self)

    def warmup(self):
        self.warm = True

    def __call__(self, x, meta, pdl=True):
        self.calls.append((tuple(x.shape), pdl))
        return torch.zeros(x.shape[0], self.N, dtype=torch.bfloat16)


def fake_layer(K=64, widths=(32, 32), R=16, L=3, fp8=True, tp=1, bias=None, a_dtype=torch.bfloat16):
    from vllm.model_executor.layers.quantization.online.fp8 import Fp8PerTensorOnlineLinearMethod
    N = sum(widths)
    qm = object.__new__(Fp8PerTensorOnlineLinearMethod) if fp8 else object()
    base = types.SimpleNamespace(weight=torch.zeros(N, K).to(torch.float8_e4m3fn).t() if fp8 else torch.zeros(N, K).t(),   # vLLM stores W^T views
                                 weight_scale=torch.ones(1), quant_method=qm, bias=bias, prefix="model.layers.0.x")
    meta = types.SimpleNamespace(meta_args=lambda m, spec: tuple(torch.zeros(4, dtype=torch.int32) for _ in range(7)))
    return types.SimpleNamespace(
        base_layer=base, tp_size=tp,
        lora_a_stacked=tuple(torch.zeros(L, 1, R, K, dtype=a_dtype) for _ in widths),
        lora_b_stacked=tuple(torch.zeros(L, 1, w, R, dtype=torch.bfloat16) for w in widths),
        punica_wrapper=types.SimpleNamespace(_token_lora_indices=torch.zeros(48), token_mapping_meta=meta),
        lora_config=types.SimpleNamespace(specialize_active_lora=False))


@pytest.fixture()
def plugin(monkeypatch, tmp_path):
    from onebase_b200 import plugin as P
    monkeypatch.setattr(P, "_op_classes", lambda: (FakeOp, FakeOp))
    monkeypatch.setattr(P, "_REGISTRY", [])
    monkeypatch.setenv("LOWBIT_REPORT", str(tmp_path / "report.txt"))
    FakeOp.made.clear()
    P._report_path = tmp_path / "report.txt"
    return P


def test_build_decisions_and_report(plugin, monkeypatch):
    P = plugin
    assert P._build(fake_layer()) == 0                                   # eligible FP8 layer
    assert FakeOp.made[0].args[0].shape == (64, 64) and FakeOp.made[0].args[4] == 48 and FakeOp.made[0].warm
    assert P._build(fake_layer(fp8=False)) == -1                         # unquantized base
    assert P._build(fake_layer(tp=2)) == -1                              # TP shard without LOWBIT_TP
    assert P._build(fake_layer(bias=torch.zeros(64))) == -1
    assert P._build(fake_layer(a_dtype=torch.float16)) == -1             # adapters must be bf16
    assert P._build(fake_layer(R=24)) == -1                              # unsupported rank
    monkeypatch.setenv("LOWBIT_TP", "1")
    assert P._build(fake_layer(tp=2)) == 1
    monkeypatch.setenv("LOWBIT_LORA_FP8", "1")                           # FP8-stored adapters: slots released to one staging slot
    lay = fake_layer()
    writes = []
    lay.set_lora = lambda index, *a, **k: (lay.reset_lora(index), writes.append(("set", index)))
    lay.reset_lora = lambda index: writes.append(("reset", index))
    FakeOp.requantize = lambda self, index=None: writes.append(("requant", index))
    FakeOp.release = lambda self, a, b: writes.append(("release", a[0].shape[0]))
    assert P._build(lay) == 2 and FakeOp.made[-1].kw["lora_fp8"] is True and lay._lowbit_released
    assert lay.lora_a_stacked[0].shape[0] == 1                           # vLLM's L slots shrank to the staging slot
    lay.set_lora(2, "A", "B")
    lay.reset_lora(1)
    assert writes == [("release", 1), ("reset", 0), ("set", 0), ("requant", 2), ("reset", 0), ("requant", 1)]
    lines = P._report_path.read_text().splitlines()
    assert sum(" fused " in ln for ln in lines) == 3 and sum(" fallback " in ln for ln in lines) == 5
    assert all(ln.split()[0].isdigit() for ln in lines)                  # pid-tagged


def test_nvfp4_layer_uses_checkpoint_layout(plugin):
    P = plugin
    lay = fake_layer(fp8=False)
    lay.base_layer._lowbit_nvfp4 = {"w_q": torch.zeros(64, 32, dtype=torch.uint8),
                                    "w_sf": torch.zeros(64, 4).to(torch.float8_e4m3fn), "input_scale": 0.5,
                                    "weight_scale_2": 0.25}
    assert P._build(lay) == 0
    op = FakeOp.made[0]
    assert op.args[2] == 4.0 and op.args[3] == 2.0 and op.kw["rcp_approx"] is True      # 1 / weight_scale_2, 1 / input_scale


def test_install_is_inert_without_the_switch(monkeypatch):
    from onebase_b200 import plugin as P
    from vllm.lora.layers.base_linear import BaseLinearLayerWithLoRA
    monkeypatch.delenv("LOWBIT_FUSED", raising=False)
    before = BaseLinearLayerWithLoRA.apply
    P.install()
    assert BaseLinearLayerWithLoRA.apply is before and not P._INSTALLED


def test_install_patches_and_routes_calls(plugin, monkeypatch, tmp_path):
    P = plugin
    import vllm.lora.layers as LL
    from vllm.lora.layers.base_linear import BaseLinearLayerWithLoRA
    monkeypatch.setenv("LOWBIT_FUSED", "1")
    monkeypatch.setenv("LOWBIT_COMPILE_CACHE", "0")
    monkeypatch.setenv("LOWBIT_PDL_MAX_M", "8")
    saved = {c: dict(c.__dict__) for c in [BaseLinearLayerWithLoRA] + [getattr(LL, n) for n in dir(LL) if isinstance(getattr(LL, n), type)]}
    try:
        monkeypatch.setattr(P, "_INSTALLED", False)
        BaseLinearLayerWithLoRA.set_mapping = lambda self, pw: setattr(self, "punica_wrapper", pw)   # stands in for vLLM's
        P.install()
        P.install()                                                       # idempotent
        assert P._INSTALLED and hasattr(torch.ops.vllm, "lowbit_fused_fp8_lora")
        assert "wrapped-apply=" in P._report_path.read_text()
        lay = fake_layer()
        pw = lay.punica_wrapper
        BaseLinearLayerWithLoRA.set_mapping(lay, pw)                      # builds the op once
        assert lay._lowbit_id == 0
        BaseLinearLayerWithLoRA.set_mapping(lay, pw)
        assert len(FakeOp.made) == 1
        y = BaseLinearLayerWithLoRA.apply(lay, torch.zeros(5, 64, dtype=torch.bfloat16))
        assert y.shape == (5, 64) and FakeOp.made[0].calls[-1] == ((5, 64), True)
        y = LL.MergedColumnParallelLinearWithLoRA.apply(lay, torch.zeros(2, 6, 64, dtype=torch.bfloat16))   # class-level override, 3-D x
        assert y.shape == (2, 6, 64) and FakeOp.made[0].calls[-1] == ((12, 64), False)   # above LOWBIT_PDL_MAX_M: serialized
        assert "op-called" in P._report_path.read_text()
    finally:
        for c, d in saved.items():
            for k in ("apply", "_apply_sync", "set_mapping"):
                if k in d:
                    setattr(c, k, d[k])
                elif k in c.__dict__:
                    delattr(c, k)
        monkeypatch.setattr(P, "_INSTALLED", False)


def test_segment_index_hook_matches_vllm_metadata():
    """LOWBIT_SEGMENT_INDEX: the replacement for LoRAKernelMeta.prepare_tensors leaves vLLM's own tensors and host flags,
    over a sequence of batches on the SAME object (stale state included).  The kernel is stood in for by the CPU oracle
    of the segment index (the GPU tests hold the kernel to that oracle bit for bit)."""
    meta_mod = pytest.importorskip("vllm.lora.ops.triton_ops.lora_kernel_metadata")
    from onebase_b200.plugin import segment_index_prepare
    from oracle import segments as oseg
    L, max_m = 6, 48
    captured = [1, 2, 4, 7]

    def index_fn(meta, t, max_loras):
        assert max_loras == L
        idx = oseg.SegmentIndex(L, max_m)
        idx.tok.copy_(meta.token_lora_mapping)
        idx.srt.copy_(meta.token_indices_sorted_by_lora_ids)
        idx.prepare(t)
        meta.token_lora_mapping.copy_(idx.tok)
        meta.token_indices_sorted_by_lora_ids.copy_(idx.srt)
        meta.num_tokens_per_lora.copy_(idx.seg_n)
        meta.lora_token_start_loc.copy_(idx.seg_start)
        meta.active_lora_ids.copy_(idx.seg_ids)

    stock = meta_mod.LoRAKernelMeta.make(L, max_m, "cpu", captured_lora_counts=captured)
    ours = meta_mod.LoRAKernelMeta.make(L, max_m, "cpu", captured_lora_counts=captured)
    for m in (stock, ours):                                    # vLLM allocates these with torch.empty
        m.token_lora_mapping.zero_()
        m.token_indices_sorted_by_lora_ids.zero_()
    hooked = segment_index_prepare(meta_mod.LoRAKernelMeta.prepare_tensors, index_fn=index_fn)
    g = torch.Generator().manual_seed(5)
    batches = [torch.randint(-1, L, (40,), generator=g, dtype=torch.int32), torch.full((17,), -1, dtype=torch.int32),
               torch.full((9,), 3, dtype=torch.int32), torch.randint(0, 2, (48,), generator=g, dtype=torch.int32),
               torch.tensor([5, -1, 5, 0], dtype=torch.int32), torch.full((3,), -1, dtype=torch.int32),
               torch.arange(48, dtype=torch.int32) % L]
    for t in batches:
        stock.prepare_tensors(t)
        hooked(ours, t)
        n = t.numel()
        for spec in (False, True):
            a, b = stock.meta_args(n, spec), ours.meta_args(n, spec)
            for x, y in zip(a, b):
                assert torch.equal(x, y), (t.tolist(), spec)
    # vLLM's Punica wrapper hands over a slice of its int64 index buffer: the hook serves it too (cast to int32 first)
    calls = []
    counting = segment_index_prepare(meta_mod.LoRAKernelMeta.prepare_tensors,
                                     index_fn=lambda m, t, n: (calls.append(t.dtype), index_fn(m, t, n)))
    wide = torch.zeros(64, dtype=torch.int64)
    wide[:40] = batches[0]
    counting(ours, wide[:40])                                  # a slice of a longer int64 buffer, as punica_base.py passes it
    stock.prepare_tensors(wide[:40])
    assert calls == [torch.int32]
    assert all(torch.equal(x, y) for x, y in zip(stock.meta_args(40, True), ours.meta_args(40, True)))
    # inputs the kernel does not take go to vLLM's own code: another dtype, an empty mapping
    def never(m, t, n):
        raise AssertionError("the kernel path was taken")
    refusing = segment_index_prepare(meta_mod.LoRAKernelMeta.prepare_tensors, index_fn=never)
    refusing(ours, batches[0].to(torch.int16))
    stock.prepare_tensors(batches[0].to(torch.int16))
    assert all(torch.equal(x, y) for x, y in zip(stock.meta_args(40, True), ours.meta_args(40, True)))
    refusing(ours, torch.zeros(0, dtype=torch.int32))
    stock.prepare_tensors(torch.zeros(0, dtype=torch.int32))
    assert all(torch.equal(x, y) for x, y in zip(stock.meta_args(4, True), ours.meta_args(4, True)))


def test_fully_sharded_adapters_fall_back(plugin):
    """vLLM's fully sharded LoRA classes hold A as [L,1,R/tp,K] and gather the shrink between their two LoRA kernels: a
    rank mismatch between A and B, or such a class anywhere in the layer's type, must not build a fused op."""
    P = plugin
    layer = fake_layer(R=16)
    layer.lora_a_stacked = tuple(t[:, :, :8].contiguous() for t in layer.lora_a_stacked)      # R/tp rows of A, B keeps R
    assert P._build(layer) == -1

    class ColumnParallelLinearWithShardedLoRA(types.SimpleNamespace):
        pass

    ok = fake_layer()
    sharded = ColumnParallelLinearWithShardedLoRA(**vars(ok))
    assert P._build(sharded) == -1
    assert P._build(ok) >= 0
    text = P._report_path.read_text()
    assert "fully_sharded_adapters" in text and "adapter_buffers" in text
