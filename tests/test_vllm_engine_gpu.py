"""The plugin inside a real vLLM engine (runs whenever vLLM imports; ONEBASE_VLLM_ENGINE_TEST=0 skips it; ~2 minutes a case).

A child process builds a small random-init Qwen3-architecture checkpoint (2 layers, hidden 1024, GQA 8/2) and three
random rank-16 LoRA adapters under a temporary directory -- bf16 weights that vLLM quantizes online to per-tensor FP8, or
a ModelOpt NVFP4 checkpoint (packed e2m1 codes, linear ue4m3 block scales, weight_scale_2, input_scale) quantized with
the oracle's recipe --, starts `vllm.LLM(..., enable_lora=True)` in eager mode with the plugin installed, and wraps every LoRA linear class that overrides `apply` so that each call runs BOTH
the fused path and vLLM's own path on the same input.  Checked: every LoRA linear layer was taken over (no fallback), the
opaque op was called, and the two paths agree within the output bound on every call of a mixed batch (prefill and decode,
one request without an adapter).  A third case runs the FP8 engine with LOWBIT_SEGMENT_INDEX=1, i.e. with vLLM's per-step
token sort / segment index built by the ob_segment_index kernel, and checks that the kernel path was really taken on the
mappings vLLM's Punica wrapper passes.  The engine runs in a child process so that its memory pool and process groups do not
outlive the test.
"""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu

CHILD = textwrap.dedent('''
    import collections, inspect, json, os, sys, tempfile
    BASE = sys.argv[1]                                   # "fp8": online per-tensor FP8; "nvfp4": a ModelOpt NVFP4 checkpoint
    if BASE.endswith("+segidx"):                         # ... "+segidx": the segment index kernel behind vLLM's metadata
        BASE = BASE[:-7]
        os.environ["LOWBIT_SEGMENT_INDEX"] = "1"
    os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")
    os.environ["LOWBIT_FUSED"] = "1"
    work = tempfile.mkdtemp(prefix="ob_vllm_")
    os.environ["LOWBIT_REPORT"] = f"{work}/report.txt"
    import torch
    from safetensors.torch import save_file
    H, LAYERS, HEADS, KV, HD, INTER, VOCAB, R, NL = 1024, 2, 8, 2, 128, 3072, 2048, 16, 3
    model_dir = f"{work}/model"
    os.makedirs(model_dir)
    cfg = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": H, "num_hidden_layers": LAYERS,
           "num_attention_heads": HEADS, "num_key_value_heads": KV, "head_dim": HD, "intermediate_size": INTER,
           "vocab_size": VOCAB, "max_position_embeddings": 2048, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
           "hidden_act": "silu", "tie_word_embeddings": False, "torch_dtype": "bfloat16", "attention_bias": False,
           "bos_token_id": 1, "eos_token_id": 2}
    if BASE == "nvfp4":
        q = {"quant_algo": "NVFP4", "kv_cache_quant_algo": None, "group_size": 16, "exclude_modules": ["lm_head"]}
        cfg["quantization_config"] = dict(q, quant_method="modelopt")
        json.dump({"producer": {"name": "modelopt", "version": "0.0"}, "quantization": q}, open(f"{model_dir}/hf_quant_config.json", "w"))
    json.dump(cfg, open(f"{model_dir}/config.json", "w"))
    g = torch.Generator().manual_seed(123)
    rn = lambda *s, std=0.04: (torch.randn(*s, generator=g) * std).to(torch.bfloat16)
    one = lambda n: torch.ones(n, dtype=torch.bfloat16)
    w = {"model.embed_tokens.weight": rn(VOCAB, H, std=1.0), "model.norm.weight": one(H), "lm_head.weight": rn(VOCAB, H, std=0.05)}
    proj = {"self_attn.q_proj": (HEADS * HD, H), "self_attn.k_proj": (KV * HD, H), "self_attn.v_proj": (KV * HD, H),
            "self_attn.o_proj": (H, HEADS * HD), "mlp.gate_proj": (INTER, H), "mlp.up_proj": (INTER, H), "mlp.down_proj": (H, INTER)}
    merged = [["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"], ["self_attn.o_proj"],
              ["mlp.gate_proj", "mlp.up_proj"], ["mlp.down_proj"]]
    for l in range(LAYERS):
        pre = f"model.layers.{l}"
        w[f"{pre}.input_layernorm.weight"], w[f"{pre}.post_attention_layernorm.weight"] = one(H), one(H)
        w[f"{pre}.self_attn.q_norm.weight"], w[f"{pre}.self_attn.k_norm.weight"] = one(HD), one(HD)
        for names in merged:
            mats = {n: rn(*proj[n]) for n in names}
            if BASE != "nvfp4":
                for n, m in mats.items():
                    w[f"{pre}.{n}.weight"] = m
                continue
            # ModelOpt layout, quantized with the oracle's recipe; one global scale per merged module, as vLLM requires
            from oracle import nvfp4 as on4
            w_global = 448.0 * 6.0 / max(float(m.float().abs().max()) for m in mats.values())
            for n, m in mats.items():
                w[f"{pre}.{n}.weight"], w[f"{pre}.{n}.weight_scale"] = on4.quant(m.float(), w_global)
                w[f"{pre}.{n}.weight_scale_2"] = torch.tensor(1.0 / w_global, dtype=torch.float32)
                w[f"{pre}.{n}.input_scale"] = torch.tensor(8.0 / (448.0 * 6.0), dtype=torch.float32)
    save_file(w, f"{model_dir}/model.safetensors")
    loras = []
    for li in range(NL):
        d = f"{work}/lora{li}"
        os.makedirs(d)
        t = {}
        for l in range(LAYERS):
            for name, (n_out, k_in) in proj.items():
                base = f"base_model.model.model.layers.{l}.{name}"
                t[f"{base}.lora_A.weight"] = rn(R, k_in, std=k_in ** -0.5)
                t[f"{base}.lora_B.weight"] = rn(n_out, R, std=0.2)
        save_file(t, f"{d}/adapter_model.safetensors")
        json.dump({"peft_type": "LORA", "r": R, "lora_alpha": R, "target_modules": [n.split(".")[1] for n in proj], "bias": "none",
                   "base_model_name_or_path": model_dir, "task_type": "CAUSAL_LM"}, open(f"{d}/adapter_config.json", "w"))
        loras.append(d)
    import vllm.lora.layers as lora_layers
    from vllm.lora.layers.base_linear import BaseLinearLayerWithLoRA
    stock = {cls: cls.__dict__["apply"] for _, cls in inspect.getmembers(lora_layers, inspect.isclass)
             if issubclass(cls, BaseLinearLayerWithLoRA) and "apply" in cls.__dict__}
    from onebase_b200 import plugin
    plugin.install()
    errs = collections.defaultdict(list)
    def wrap(cls, fused_apply, stock_apply):
        def both(self, x, bias=None):
            y = fused_apply(self, x, bias)
            if getattr(self, "_lowbit_id", -1) >= 0 and x.shape[0] > 0:
                ys = stock_apply(self, x, bias)
                errs[self.base_layer.prefix].append(float((y.float() - ys.float()).abs().max()) / (float(ys.float().abs().max()) + 1e-30))
            return y
        cls.apply = both
    for cls, st in stock.items():
        wrap(cls, cls.__dict__["apply"], st)
    from vllm import LLM, SamplingParams
    from vllm.lora.request import LoRARequest
    llm = LLM(model=model_dir, quantization="fp8" if BASE == "fp8" else None, dtype="bfloat16", enable_lora=True, max_loras=NL, max_lora_rank=R,
              skip_tokenizer_init=True, enforce_eager=True, gpu_memory_utilization=0.2, max_model_len=1024, max_num_seqs=16, seed=0)
    gp = torch.Generator().manual_seed(1)
    prompts = [{"prompt_token_ids": torch.randint(3, VOCAB, (int(n),), generator=gp).tolist()} for n in (17, 40, 9, 64, 33, 5)]
    reqs = [LoRARequest(f"a{i % NL}", i % NL + 1, loras[i % NL]) if i != 2 else None for i in range(len(prompts))]
    errs.clear()
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, detokenize=False), lora_request=reqs)
    rep = open(os.environ["LOWBIT_REPORT"]).read().splitlines()
    print("RESULT " + json.dumps({"fused": sum(" fused" in l for l in rep), "fallback": sum("fallback" in l for l in rep),
                                  "op_called": any("op-called" in l for l in rep), "generated": [len(o.outputs[0].token_ids) for o in outs],
                                  "max_err": {k: max(v) for k, v in errs.items()}, "calls": {k: len(v) for k, v in errs.items()},
                                  "segment_index": {"installed": any("segment-index kernel installed" in l for l in rep),
                                                    "kernel": plugin._STATS["segment_index_kernel"], "stock": plugin._STATS["segment_index_stock"]}}))
''')


@pytest.mark.skipif(os.environ.get("ONEBASE_VLLM_ENGINE_TEST") == "0", reason="ONEBASE_VLLM_ENGINE_TEST=0 (starts a vLLM engine)")
@pytest.mark.parametrize("base", ["fp8", "nvfp4", "fp8+segidx"])
def test_plugin_inside_vllm_engine(base):
    import json
    pytest.importorskip("vllm")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
    p = subprocess.run([sys.executable, "-c", CHILD, base], capture_output=True, text=True, timeout=900, env=env)
    lines = [l for l in p.stdout.splitlines() if l.startswith("RESULT ")]
    assert p.returncode == 0 and lines, (p.stdout[-2000:], p.stderr[-4000:])
    r = json.loads(lines[-1][7:])
    assert r["fused"] == 8 and r["fallback"] == 0 and r["op_called"], r          # 2 layers x (qkv, o, gate_up, down)
    assert r["generated"] == [8] * 6, r
    assert r["max_err"] and all(c > 0 for c in r["calls"].values()), r
    assert max(r["max_err"].values()) <= 2e-2, r                                 # fused vs vLLM's own path, same inputs
    if base.endswith("+segidx"):
        assert r["segment_index"]["installed"] and r["segment_index"]["kernel"] > 0, r
