"""End-to-end decode throughput through a vLLM engine, with and without the plugin (the reference's protocol for its
serving numbers, bench/overhead.py:126-138: random token ids, fixed output length, every request on its own adapter).

    python -m onebase_b200.bench_vllm --mode fused|stock [--layers 36] [--requests 32] [--prompt 512] [--out-tokens 128]

Builds, under a temporary directory, the config of a Qwen3-8B-shaped model (hidden 4096, GQA 32/8, head_dim 128,
intermediate 12288, vocab 151936; `--layers` of its 36 layers) and ONE random rank-64 adapter file that is registered under
`--tenants` different adapter ids (default: one per request; vLLM gives each id its own slot, so the kernels see that
many tenants).  The base
weights are vLLM's dummy initialisation quantized online to per-tensor FP8 -- throughput does not depend on the values,
and no checkpoint exists offline.  Prints one JSON line: tokens/s over a timed `generate` (prefill + decode) after a
warm-up call, and the per-output-token time of the decode phase estimated from two output lengths.
"""
from __future__ import annotations

import argparse
import json
import os
import tempfile
import time


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", choices=["fused", "stock"], required=True)
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--requests", type=int, default=32)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--out-tokens", type=int, default=128)
    ap.add_argument("--rank", type=int, default=64)
    ap.add_argument("--tenants", type=int, default=0, help="adapter ids the requests cycle over (default: one per request)")
    ap.add_argument("--eager", action="store_true")
    args = ap.parse_args()
    os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")
    os.environ["LOWBIT_FUSED"] = "1" if args.mode == "fused" else "0"
    work = tempfile.mkdtemp(prefix="ob_vllm_bench_")
    os.environ["LOWBIT_REPORT"] = f"{work}/report.txt"
    import torch
    from safetensors.torch import save_file
    H, HEADS, KV, HD, INTER, VOCAB = 4096, 32, 8, 128, 12288, 151936
    model_dir = f"{work}/model"
    os.makedirs(model_dir)
    json.dump({"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": H, "num_hidden_layers": args.layers,
               "num_attention_heads": HEADS, "num_key_value_heads": KV, "head_dim": HD, "intermediate_size": INTER,
               "vocab_size": VOCAB, "max_position_embeddings": 4096, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
               "hidden_act": "silu", "tie_word_embeddings": False, "torch_dtype": "bfloat16", "attention_bias": False,
               "bos_token_id": 1, "eos_token_id": 2}, open(f"{model_dir}/config.json", "w"))
    proj = {"self_attn.q_proj": (HEADS * HD, H), "self_attn.k_proj": (KV * HD, H), "self_attn.v_proj": (KV * HD, H),
            "self_attn.o_proj": (H, HEADS * HD), "mlp.gate_proj": (INTER, H), "mlp.up_proj": (INTER, H), "mlp.down_proj": (H, INTER)}
    g = torch.Generator().manual_seed(0)
    t = {}
    for l in range(args.layers):
        for name, (n_out, k_in) in proj.items():
            base = f"base_model.model.model.layers.{l}.{name}"
            t[f"{base}.lora_A.weight"] = (torch.randn(args.rank, k_in, generator=g) * k_in ** -0.5).to(torch.bfloat16)
            t[f"{base}.lora_B.weight"] = (torch.randn(n_out, args.rank, generator=g) * 1e-3).to(torch.bfloat16)
    lora_dir = f"{work}/lora"
    os.makedirs(lora_dir)
    save_file(t, f"{lora_dir}/adapter_model.safetensors")
    json.dump({"peft_type": "LORA", "r": args.rank, "lora_alpha": args.rank, "target_modules": [n.split(".")[1] for n in proj],
               "bias": "none", "base_model_name_or_path": model_dir, "task_type": "CAUSAL_LM"},
              open(f"{lora_dir}/adapter_config.json", "w"))
    if args.mode == "fused":
        from onebase_b200 import plugin
        plugin.install()
    from vllm import LLM, SamplingParams
    from vllm.lora.request import LoRARequest
    t0 = time.time()
    tenants = args.tenants or args.requests
    llm = LLM(model=model_dir, load_format="dummy", quantization="fp8", dtype="bfloat16", enable_lora=True,
              max_loras=tenants, max_lora_rank=args.rank, skip_tokenizer_init=True, enforce_eager=args.eager,
              gpu_memory_utilization=0.6, max_model_len=args.prompt + args.out_tokens + 16, max_num_seqs=max(args.requests, 8),
              max_num_batched_tokens=8192, seed=0)
    up = time.time() - t0
    gp = torch.Generator().manual_seed(1)
    prompts = [{"prompt_token_ids": torch.randint(3, VOCAB, (args.prompt,), generator=gp).tolist()} for _ in range(args.requests)]
    reqs = [LoRARequest(f"a{i % tenants}", i % tenants + 1, lora_dir) for i in range(args.requests)]

    def run(n_out: int) -> float:
        sp = SamplingParams(temperature=0.0, max_tokens=n_out, min_tokens=n_out, ignore_eos=True, detokenize=False)
        torch.cuda.synchronize()
        t1 = time.time()
        outs = llm.generate(prompts, sp, lora_request=reqs, use_tqdm=False)
        torch.cuda.synchronize()
        assert all(len(o.outputs[0].token_ids) == n_out for o in outs)
        return time.time() - t1

    run(8)                                                     # warm-up: adapter loads, lazy compilation
    short, full = run(args.out_tokens // 4), run(args.out_tokens)
    decode_s = (full - short) / (args.out_tokens - args.out_tokens // 4)     # seconds per decode step of the whole batch
    rep = open(os.environ["LOWBIT_REPORT"]).read().splitlines() if os.path.exists(os.environ["LOWBIT_REPORT"]) else []
    print(json.dumps({"mode": args.mode, "layers": args.layers, "requests": args.requests, "tenants": tenants, "prompt": args.prompt,
                      "out_tokens": args.out_tokens, "engine_up_s": round(up, 1), "generate_s": round(full, 3),
                      "tokens_per_s": round(args.requests * args.out_tokens / full, 1),
                      "decode_step_ms": round(decode_s * 1e3, 3), "decode_tokens_per_s": round(args.requests / decode_s, 1),
                      "fused_layers": sum(" fused " in l for l in rep), "fallback_layers": sum("fallback" in l for l in rep),
                      "cuda_graphs": not args.eager}))


if __name__ == "__main__":
    main()
