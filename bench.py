"""Benchmark of the fused FP8 + multi-tenant LoRA decoder layer (the decode chain K1 -> K2 per projection).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--m M] [--impl reference]

Workload (N = 1): one Qwen3-8B-shaped decoder layer, FP8 per-tensor base (qkv 4096->6144, o 4096->4096, gate_up
4096->2x12288, down 12288->4096), decode batch M = 32 tokens, 32 bf16 tenants of rank 64 with slot ids uniform random
per token, the four projections' K1 -> K2 chains captured in ONE CUDA graph; a "step" is one replay of that graph.
Synthetic data with the shapes and distributions of that configuration (random-init weights; no dataset).
Timing: CUDA events around each replay on the replay's stream, a 256 MB write flushes L2 before every replay (outside
the timed events), W >= 3 warm-up replays, max over ranks.  Prints ONE JSON line (rank 0).

`value`   tokens/s through the layer with inputs resident in HBM (M / mean replay time).
`e2e`     the same through the public op call with HOST buffers: every step copies the four projections' activations from
          pinned host memory, runs the layer, and copies the four outputs back (copies inside the timed region).
          Headline: steady state with two steps in flight (step i+1 uploads and step i-1 downloads while step i computes;
          all steps timed as one region).  `single_step`: one step alone as one CUDA graph over three streams (a
          projection waits only for its own input, its output goes down while the next projection runs); `serial`:
          uploads, layer, downloads one after the other.
`roofline` for the dominant kernel (K2 of gate_up): algorithmic bytes (W + x + the distinct tenants' B + y) / its
          CUDA-event time when launched alone, against the measured HBM copy bandwidth.
`cpu_baseline` the CPU oracle (a torch port of the reference's dequantize-and-matmul path) on this host's cores.
`--impl reference` times only that CPU path and prints the same line shape with "impl": "reference".
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

PROJECTIONS = {"qkv": (4096, (4096, 1024, 1024)), "o": (4096, (4096,)), "gate_up": (4096, (12288, 12288)),
               "down": (12288, (4096,))}
L_SLOTS, RANK = 32, 64
METRIC = "decode tok/s at 32 tenants through one fused FP8+LoRA decoder layer (layer us and HBM roofline % alongside)"


def workload_name(M: int) -> str:
    """The same string in both arms' lines (the batch is seeded: both draw the same tenants)."""
    ids = torch.randint(0, L_SLOTS, (M,), generator=torch.Generator().manual_seed(0), dtype=torch.int32)
    return (f"Qwen3-8B decoder layer (qkv, o, gate_up, down), FP8 per-tensor base, decode M={M}, 32 bf16 tenants rank 64 "
            f"({int(torch.unique(ids).numel())} distinct in the batch)")


def measured_peaks() -> tuple[float, str]:
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.stop_flag, self.max_mhz = index, [], set(), False, None

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            names = {nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap", nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
                     nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
                     nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown"}
            while not self.stop_flag:
                self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
                time.sleep(0.002)
        except Exception as e:   # noqa: BLE001 - clocks are reported as unavailable, the measurement itself stands
            self.reasons.add(f"nvml-unavailable:{type(e).__name__}")

    def result(self) -> dict:
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def physical_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except (ValueError, IndexError):
            return local
    return local


def zipf_ids(M: int, seed: int = 0, exponent: float = 1.1) -> torch.Tensor:
    """Prefill batch of the NVFP4 configuration: the M tokens are split across the 32 tenants in contiguous runs whose
    sizes follow Zipf(1.1) (tenant of rank i gets a share proportional to 1 / i^1.1), tenants in a seeded random order."""
    g = torch.Generator().manual_seed(seed)
    share = 1.0 / torch.arange(1, L_SLOTS + 1, dtype=torch.float64) ** exponent
    exact = share / share.sum() * M
    counts = exact.floor().long()
    order = torch.argsort(exact - counts, descending=True)
    counts[order[: M - int(counts.sum())]] += 1              # largest remainders take the tokens the floors left over
    tenants = torch.randperm(L_SLOTS, generator=g)
    return torch.repeat_interleave(tenants.to(torch.int32), counts)


def make_layer(M: int, device, seed: int = 0, base: str = "fp8", lora_fmt: str = "bf16", ids=None):
    """Random-init layer with the configuration's distributions, generated on the device (values do not matter for
    timing; the parity tests use CPU-drawn inputs).  Returns {proj: (op, x, meta)} plus the ids."""
    from onebase_b200.kernels.fp8_lora_vllm import VllmFusedFP8LoRA
    g = torch.Generator(device=device).manual_seed(seed)
    if ids is None:
        ids = torch.randint(0, L_SLOTS, (M,), generator=torch.Generator().manual_seed(seed), dtype=torch.int32)
    from onebase_b200.metadata import KernelMeta
    km = KernelMeta.make(L_SLOTS, M, device)
    km.prepare_tensors(ids.to(device))
    meta = km.meta_args(M)
    layer = {}
    for name, (K, widths) in PROJECTIONS.items():
        N = sum(widths)
        w = torch.randn(N, K, device=device, generator=g) * 0.02
        if base == "fp8":
            s_w = (w.abs().max() / 448.0).reshape(1).float()
            w_q = (w / s_w).to(torch.float8_e4m3fn)
        else:   # NVFP4: timing does not depend on the code values: random nibbles, block scales near 1
            w_q = torch.randint(0, 256, (N, K // 2), device=device, generator=g, dtype=torch.uint8)
            w_sf = torch.randint(0x30, 0x40, (N, K // 16), device=device, generator=g, dtype=torch.uint8).view(torch.float8_e4m3fn)
        del w
        a_st = tuple(((torch.rand(L_SLOTS, 1, RANK, K, device=device, generator=g) * 2 - 1) / K ** 0.5).to(torch.bfloat16)
                     for _ in widths)
        b_st = tuple((torch.randn(L_SLOTS, 1, n, RANK, device=device, generator=g) * 0.01).to(torch.bfloat16) for n in widths)
        x = torch.randn(M, K, device=device, generator=g).to(torch.bfloat16)
        if base == "fp8":
            op = VllmFusedFP8LoRA(w_q, s_w, a_st, b_st, max_m=M, lora_fp8=lora_fmt == "fp8", lora_fp4=lora_fmt == "nvfp4")
        else:
            from onebase_b200.kernels.nvfp4_lora_vllm import VllmFusedNVFP4LoRA
            op = VllmFusedNVFP4LoRA(w_q, w_sf, 2688.0 / 0.1, 2688.0 / 4.0, a_st, b_st, max_m=M, lora_fmt=lora_fmt, rcp_approx=True)
        layer[name] = (op, x, torch.empty(M, N, dtype=torch.bfloat16, device=device))
    return layer, meta, ids


def layer_bytes(M: int, distinct: int) -> dict:
    """Algorithmic bytes per projection: W + x + the distinct tenants' A and B + y (bf16 adapters)."""
    out = {}
    for name, (K, widths) in PROJECTIONS.items():
        N, S = sum(widths), len(widths)
        out[name] = {"w": N * K, "x": M * K * 2, "y": M * N * 2, "a": distinct * S * RANK * K * 2, "b": distinct * N * RANK * 2}
        out[name]["total"] = sum(out[name].values())
    return out


def run_layer(layer, meta):
    for name in ("qkv", "o", "gate_up", "down"):
        op, x, y = layer[name]
        op(x, meta, out=y)


def time_events(fn, steps: int, warmup: int, flush) -> list[float]:
    for _ in range(warmup):
        flush.fill_(1)
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(steps):
        flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1))
    return ts   # milliseconds


def profile_case(args, dev) -> None:
    """One projection, K1 and K2 launched separately (no graph, no PDL) so that a profiler can pick either kernel."""
    global PROJECTIONS
    keep = {args.profile: PROJECTIONS[args.profile]}
    saved, PROJECTIONS = PROJECTIONS, keep
    try:
        layer, meta, ids = make_layer(args.m, dev, base=args.base, lora_fmt=args.lora_fmt)
    finally:
        PROJECTIONS = saved
    op, x, y = layer[args.profile]
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    op(x, meta, out=y)
    torch.cuda.synchronize()
    k1 = time_events(lambda: op(x, meta, out=y, gemm=False), args.steps, 2, flush)
    k2 = time_events(lambda: op(x, meta, out=y, shrink=False, pdl=False), args.steps, 2, flush)
    chain = time_events(graph_of(lambda: op(x, meta, out=y)).replay, args.steps, 2, flush)
    by = layer_bytes(args.m, int(torch.unique(ids).numel()))[args.profile]
    print(json.dumps({"profile": args.profile, "M": args.m, "base": args.base, "lora_fmt": args.lora_fmt,
                      "distinct": int(torch.unique(ids).numel()),
                      "k1_us": statistics.fmean(k1) * 1e3, "k2_us": statistics.fmean(k2) * 1e3,
                      "chain_us": statistics.fmean(chain) * 1e3, "bytes": by}))


def format_bytes(M: int, distinct: int, base: str, lora_fmt: str) -> int:
    """Algorithmic bytes of one layer pass for a base / adapter storage format: W (+ its block scales), x, y and the distinct
    tenants' A and B with their scales; intermediates excluded."""
    w_b = 1.0 if base == "fp8" else 0.5625                  # NVFP4: half a byte per code + one scale byte per 16
    total = 0.0
    for K, widths in PROJECTIONS.values():
        N, S = sum(widths), len(widths)
        n_ab = S * RANK * K + N * RANK                      # adapter elements per tenant
        if lora_fmt == "bf16":
            ad = 2.0 * n_ab
        elif lora_fmt == "fp8":
            ad = 1.0 * n_ab + 4.0 * (S * RANK + N)          # codes + one fp32 scale per row of A and of B
        else:
            ad = 0.5625 * n_ab + 8.0 * S                    # codes + block scales + the two matrices' global scales
        total += N * K * w_b + M * K * 2 + M * N * 2 + distinct * ad
    return int(total)


def measure_cell(base: str, lora_fmt: str, M: int, dev, flush, peak: float, kind: str) -> dict:
    """One cell of the configurations' grid: the four-projection layer for a base format, adapter storage and batch size as
    one CUDA graph, L2 flushed before every replay, CUDA events.  Decode batches (at most 64 tokens) draw a tenant per token
    and report algorithmic bytes against the HBM peak; prefill batches split the tokens across the tenants by Zipf(1.1) and
    report the base GEMM's flops against the nominal dense peak of the base format and against 2x / 4x the measured bf16
    GEMM throughput (an FP8 / FP4 ceiling of the same silicon)."""
    ids = zipf_ids(M) if M > 64 else None
    layer, meta, ids = make_layer(M, dev, base=base, lora_fmt=lora_fmt, ids=ids)
    run_layer(layer, meta)
    torch.cuda.synchronize()
    status = [int(layer[n][0].scratch.status()[0]) for n in PROJECTIONS]
    g = graph_of(lambda: run_layer(layer, meta))
    steps = 30 if M <= 64 else 10
    us = statistics.fmean(time_events(g.replay, steps, 3, flush)) * 1e3
    distinct = int(torch.unique(ids).numel())
    nbytes = format_bytes(M, distinct, base, lora_fmt)
    flops = sum(2.0 * M * sum(w) * K for K, w in PROJECTIONS.values())
    line = {"base": base, "adapters": lora_fmt, "M": M, "distinct": distinct, "layer_us": round(us, 1),
            "tokens_per_s": round(M / us * 1e6), "device_status": status}
    if M <= 64:
        line.update({"bytes": nbytes, "gbs": round(nbytes / us / 1e3, 1), "hbm_frac": round(nbytes / us / 1e3 / peak, 3),
                     "hbm_frac_of_nominal_8tbs": round(nbytes / us / 1e3 / 8000.0, 3), "peak_gbs": peak, "peak_kind": kind})
    else:
        bf16 = measured_bf16_tflops()
        mult = 2.0 if base == "fp8" else 4.0
        line.update({"base_gemm_gflop": round(flops / 1e9, 1), "pflops": round(flops / us / 1e9, 3),
                     "frac_of_nominal": round(flops / us / 1e9 / (4.5 if base == "fp8" else 9.0), 3),
                     "frac_of_measured_bf16_x%d" % int(mult): (round(flops / us / 1e6 / (bf16 * mult), 3) if bf16 else None)})
    del layer, g
    torch.cuda.empty_cache()
    return line


def measured_bf16_tflops() -> float | None:
    f = ROOT / "MEASURED_PEAKS.json"
    return float(json.loads(f.read_text())["bf16_tflops"]) if f.exists() else None


def matrix_case(args, dev) -> None:
    """The configurations' grid, one JSON line per cell: base format x adapter storage x batch size."""
    peak, kind = measured_peaks()
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    cells = [("fp8", "bf16"), ("nvfp4", "bf16"), ("fp8", "fp8"), ("nvfp4", "fp8"), ("nvfp4", "nvfp4")]
    sizes = [int(v) for v in args.matrix.split(",")] if args.matrix != "all" else [1, 2, 4, 8, 16, 32, 512, 2048, 8192]
    for base, lora_fmt in cells:
        for M in sizes:
            print(json.dumps(dict(measure_cell(base, lora_fmt, M, dev, flush, peak, kind), matrix=True)), flush=True)


def e2e_object(M, h2d, d2h, stream_ms, step_ms, step_kind, serial_ms) -> dict:
    """The end-to-end entry of the line: the steady-state form (two steps in flight) where it ran, else the single step;
    the other forms beside it."""
    single = {"value": M / (step_ms * 1e-3), "ms_per_step": step_ms,
              "how": step_kind + "; every step timed alone, L2 flushed before it"}
    serial = {"value": M / (serial_ms * 1e-3), "ms_per_step": serial_ms,
              "how": "uploads, one graph replay, downloads, one after the other on one stream; every step timed alone, L2 flushed"}
    head = {"unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
    if stream_ms is not None:
        head.update(value=M / (stream_ms * 1e-3), ms_per_step=stream_ms,
                    how="steady state, two steps in flight: step i+1 uploads and step i-1 downloads while step i computes "
                        "(three streams, two buffer sets, upload / layer / download graphs ordered by events); all steps "
                        "timed as one region; no L2 flush inside it (a step streams 193 MB of weights and the tenants' adapters "
                        "through a 126 MB L2; what survives from the step before can put this below `value`'s flushed step)",
                    single_step=single, serial=serial)
    else:
        head.update(value=single["value"], ms_per_step=step_ms, how=single["how"], serial=serial)
    return head


def graph_of(fn) -> "torch.cuda.CUDAGraph":
    """Capture fn's launches in a CUDA graph (replays carry no host launch latency)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    return g


def cpu_layer_seconds(M: int, reps: int, threads: int) -> tuple[float, str, str]:
    """The reference's CPU torch path on one layer (all four projections), same shapes and distributions; median seconds
    per pass.  Runs the reference's own `reference_multi` (its per-token Python loop timed as written) when its modules
    were put under oracle/_ref by `python -m oracle.build_ref`, else the oracle's restatement of it.  Returns
    (seconds, sample description, "reference" | "port")."""
    from oracle import build_ref, configs, fp8 as ofp8
    torch.set_num_threads(threads)
    ref = build_ref.load()
    ds = {}
    for i, (name, (K, widths)) in enumerate(PROJECTIONS.items()):
        d = configs.with_fp8_base(configs.draw(K, widths, RANK, L_SLOTS, M, seed=i, ids_low=0))
        d["A"], d["B"] = ofp8.stack_slices(d["a_stacked"], d["b_stacked"])
        ds[name] = d
    ts = []
    for r in range(reps + 1):
        t0 = time.perf_counter()
        for name, d in ds.items():
            if ref is not None:
                ref[0].reference_multi(d["x"], d["ids"], d["w_q"], d["s_w"], d["A"], d["B"], list(d["widths"]), 1.0)
            else:
                ofp8.fused_projection(d["x"], d["ids"], d["w_q"], d["s_w"], d["A"], d["B"], d["widths"])
        if r:
            ts.append(time.perf_counter() - t0)
    kind = "reference" if ref is not None else "port"
    what = ("the reference's own reference_multi (lowbit_lora/kernels/fp8_lora_multi.py:295-314), per-token loop as written"
            if ref is not None else "the oracle's restatement of reference_multi")
    return (statistics.median(ts),
            f"one Qwen3-8B layer (4 projections), M={M}, 32 slots rank 64, {reps} timed passes after 1 warm-up; {what}", kind)


def reference_gpu_layer(layer, meta, M: int, flush, steps: int) -> dict:
    """The reference's own GPU path for the same layer on this GPU: its `VllmFusedFP8LoRA` (serialized Triton launches,
    the form its plugin runs wherever its PDL chain is not available) built over the SAME tensors, the four projections
    captured in one CUDA graph, L2 flushed before every replay, CUDA events.  Its outputs are checked against this
    repository's on the way.  Part of the reference leg: nothing of the product path runs through it."""
    from oracle import build_ref
    RefOp = build_ref.load_gpu_op()
    if RefOp is None:
        return {"unavailable": "the reference's modules are not under oracle/_ref (python -m oracle.build_ref) or do not import"}
    try:
        ref, outs, errs = {}, {}, {}
        for name, (op, x, y) in layer.items():
            ref[name] = RefOp(op.w_q, op.s_w, op.a_stacked, op.b_stacked, max_m=M)
            outs[name] = torch.empty_like(y)

        def run_ref():
            for name in ("qkv", "o", "gate_up", "down"):
                ref[name](layer[name][1], meta, out=outs[name])

        for _ in range(3):                                    # Triton compiles here
            run_ref()
        torch.cuda.synchronize()
        for name, (op, x, y) in layer.items():
            ours = op(x, meta).float()
            errs[name] = float((outs[name].float() - ours).abs().max() / ours.abs().max())
        g = graph_of(run_ref)
        ts = time_events(g.replay, steps, 5, flush)
        per = {}
        for name in layer:
            g1 = graph_of(lambda n=name: ref[n](layer[n][1], meta, out=outs[n]))
            per[name] = statistics.fmean(time_events(g1.replay, 20, 3, flush)) * 1e3
        return {"layer_us": statistics.fmean(ts) * 1e3, "projection_us": per, "max_abs_err_over_ymax_vs_this_repo": errs,
                "how": "lowbit_lora.kernels.fp8_lora_vllm.VllmFusedFP8LoRA (Triton _shrink_vllm + _gemm_vllm, its own tile "
                       "tables) from oracle/_ref, same tensors, one CUDA graph, L2 flushed, CUDA events",
                "triton": __import__("triton").__version__}
    except Exception as exc:   # noqa: BLE001 - the reference's kernels may not compile for this GPU
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}


def reference_gpu_in_child(M: int, steps: int) -> dict:
    """`reference_gpu_layer` in a process of its own: a compile error, a time-out or a fault in the reference's kernels
    then costs this one object, not the run's line."""
    import subprocess
    cmd = [sys.executable, os.path.abspath(__file__), "--reference-gpu-child", "--m", str(M), "--steps", str(steps)]
    try:
        out = subprocess.run(cmd, capture_output=True, text=True, timeout=420)
        rows = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
        if out.returncode != 0 or not rows:
            return {"unavailable": f"child exited {out.returncode}: {out.stderr.strip()[-200:]}"}
        return json.loads(rows[-1])
    except subprocess.TimeoutExpired:
        return {"unavailable": "the reference's kernels did not finish within 420 s"}


def reference_gpu_child(args) -> None:
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    layer, meta, _ = make_layer(args.m, dev)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    print(json.dumps(reference_gpu_layer(layer, meta, args.m, flush, args.steps)))


def reference_arm(args, rank: int) -> None:
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    M = args.m
    steps = max(1, min(args.steps, 3))
    sec, sample, kind = cpu_layer_seconds(M, steps, threads)
    value = M / sec
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": steps,
            "warmup": 1, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "fp32 (CPU dequantize-and-matmul)", "data": "synthetic",
            "config": {"workload": workload_name(M), "how": "the reference's CPU torch path on this host's cores"},
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--m", type=int, default=32, help="decode batch (tokens per step)")
    ap.add_argument("--impl", default="onebase_b200")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-tables", action="store_true", help="skip the decode / prefill tables beside the headline cell")
    ap.add_argument("--no-reference-gpu", action="store_true",
                    help="skip the `reference_gpu` object: the reference's own Triton kernels (out of oracle/_ref) timed on "
                         "the same layer and GPU in a child process, beside the CPU baseline")
    ap.add_argument("--reference-gpu-child", action="store_true", help=argparse.SUPPRESS)
    ap.add_argument("--base", default="fp8", choices=["fp8", "nvfp4"], help="base format of the --profile case")
    ap.add_argument("--lora-fmt", default="bf16", choices=["bf16", "fp8", "nvfp4"], help="adapter storage of the --profile case")
    ap.add_argument("--tp-form", default="partial", choices=["partial", "sharded"],
                    help="N > 1: row-parallel layers add partial LoRA terms (vLLM's default) or shard the adapters too and "
                         "all-reduce the shrink partials first")
    ap.add_argument("--tp-comm", default="peer", choices=["peer", "fused", "nccl"],
                    help="N > 1: the row-parallel layers' all-reduce -- the peer-memory kernel inside the layer's CUDA graph "
                         "(default; measured fastest), the same exchange fused into K2's epilogue, or NCCL between graph replays")
    ap.add_argument("--no-config4", action="store_true", help="N > 1: skip the 72B-class layer's timings")
    ap.add_argument("--matrix", default=None, metavar="SIZES",
                    help="measure the grid of base formats x adapter storage formats at these batch sizes (comma-separated, "
                         "or 'all' for 1,2,4,8,16,32,512,2048,8192); one JSON line per cell")
    ap.add_argument("--profile", default=None, metavar="PROJ",
                    help="small profiling case: build only this projection (qkv|o|gate_up|down) and launch K1 and K2 "
                         "separately --steps times each (for ncu captures); prints their mean times")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.reference_gpu_child:
        reference_gpu_child(args)
        return
    if args.impl == "reference":
        reference_arm(args, rank)
        return
    if world > 1:
        from onebase_b200.tp import bench_tp
        bench_tp(args, rank, world, local, METRIC)
        return

    warmup = max(3, args.warmup)
    M = args.m
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    if args.profile:
        profile_case(args, dev)
        return
    if args.matrix:
        matrix_case(args, dev)
        return
    layer, meta, ids = make_layer(M, dev)
    distinct = int(torch.unique(ids).numel())
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    run_layer(layer, meta)                                   # scratch reaches its final size before capture
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        run_layer(layer, meta)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run_layer(layer, meta)
    torch.cuda.synchronize()

    sampler = ClockSampler(physical_index(local))
    sampler.start()
    ts = time_events(graph.replay, args.steps, warmup, flush)
    ms = statistics.fmean(ts)

    # per-projection chain time and the dominant kernel (K2 of gate_up) alone
    per_proj = {}
    for name in PROJECTIONS:
        op, x, y = layer[name]
        g1 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g1):
            op(x, meta, out=y)
        per_proj[name] = statistics.fmean(time_events(g1.replay, 30, 5, flush)) * 1e3
    op, x, y = layer["gate_up"]
    op(x, meta, out=y)
    k2_ms = statistics.fmean(time_events(graph_of(lambda: op(x, meta, out=y, shrink=False, pdl=False)).replay, 50, 5, flush))
    k1_ms = statistics.fmean(time_events(graph_of(lambda: op(x, meta, out=y, gemm=False)).replay, 50, 5, flush))

    # end to end: host buffers in, host buffers out, copies inside the timed region
    host_x = {n: layer[n][1].cpu().pin_memory() for n in PROJECTIONS}
    host_y = {n: torch.empty(layer[n][2].shape, dtype=torch.bfloat16).pin_memory() for n in PROJECTIONS}
    h2d = sum(t.numel() * 2 for t in host_x.values())
    d2h = sum(t.numel() * 2 for t in host_y.values())

    def e2e_serial():
        for n in PROJECTIONS:
            layer[n][1].copy_(host_x[n], non_blocking=True)
        graph.replay()
        for n in PROJECTIONS:
            host_y[n].copy_(layer[n][2], non_blocking=True)

    def e2e_pipelined_graph():
        """The same step as one CUDA graph over three streams: the inputs go up on a copy stream, each projection's chain
        waits only for its own input, and each output goes down on another copy stream while the next chain runs."""
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        g2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g2):
            cap = torch.cuda.current_stream()
            s_in.wait_stream(cap)
            s_out.wait_stream(cap)
            arrived = {}
            with torch.cuda.stream(s_in):
                for n in PROJECTIONS:
                    layer[n][1].copy_(host_x[n], non_blocking=True)
                    arrived[n] = torch.cuda.Event()
                    arrived[n].record(s_in)
            for n in PROJECTIONS:
                op_n, x_n, y_n = layer[n]
                cap.wait_event(arrived[n])
                op_n(x_n, meta, out=y_n)
                done = torch.cuda.Event()
                done.record(cap)
                s_out.wait_event(done)
                with torch.cuda.stream(s_out):
                    host_y[n].copy_(y_n, non_blocking=True)
            cap.wait_stream(s_in)
            cap.wait_stream(s_out)
        return g2

    def e2e_streamed(steps: int, warm: int) -> float:
        """Steady-state serving, two steps in flight: step i + 1's inputs go up and step i - 1's outputs come down while
        step i computes.  Two sets of device and pinned host buffers; uploads, the layer and downloads are three CUDA
        graphs per set on three streams, ordered by events (a set's upload waits for the compute that last read it, its
        compute for the download that last emptied its outputs; the computes themselves run one after the other: they
        share one workspace).  Returns milliseconds per step over `steps` steps timed as ONE region (CUDA events on the
        first upload's and the last download's streams).  No L2 flush inside the region: a step streams 193 MB of
        weights plus the tenants' adapters through a 126 MB L2."""
        names = list(PROJECTIONS)
        xs = [{n: layer[n][1] for n in names}, {n: torch.empty_like(layer[n][1]) for n in names}]
        ys = [{n: layer[n][2] for n in names}, {n: torch.empty_like(layer[n][2]) for n in names}]
        hx = [host_x, {n: host_x[n].clone().pin_memory() for n in names}]
        hy = [host_y, {n: torch.empty_like(host_y[n]).pin_memory() for n in names}]
        s_in, s_run, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()

        def captured(stream, fn):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                fn()
            return g

        def upload(b):
            for n in names:
                xs[b][n].copy_(hx[b][n], non_blocking=True)

        def compute(b):
            for n in names:
                layer[n][0](xs[b][n], meta, out=ys[b][n])

        def download(b):
            for n in names:
                hy[b][n].copy_(ys[b][n], non_blocking=True)

        torch.cuda.synchronize()
        up = [captured(s_in, lambda b=b: upload(b)) for b in (0, 1)]
        run = [captured(s_run, lambda b=b: compute(b)) for b in (0, 1)]
        down = [captured(s_out, lambda b=b: download(b)) for b in (0, 1)]
        in_done = [torch.cuda.Event(), torch.cuda.Event()]
        run_done = [torch.cuda.Event(), torch.cuda.Event()]
        out_done = [torch.cuda.Event(), torch.cuda.Event()]

        def steps_in_flight(k: int) -> float:
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(s_in)
            for i in range(k):
                b = i & 1
                with torch.cuda.stream(s_in):
                    if i >= 2:
                        s_in.wait_event(run_done[b])
                    up[b].replay()
                    in_done[b].record(s_in)
                with torch.cuda.stream(s_run):
                    s_run.wait_event(in_done[b])
                    if i >= 2:
                        s_run.wait_event(out_done[b])
                    run[b].replay()
                    run_done[b].record(s_run)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(run_done[b])
                    down[b].replay()
                    out_done[b].record(s_out)
            s_out.wait_stream(s_run)
            s_out.wait_stream(s_in)
            e1.record(s_out)
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / k

        steps_in_flight(max(2, warm))
        ms_step = steps_in_flight(steps)
        for n in names:                                        # both sets carried the same inputs: the same bytes come back
            assert torch.equal(hy[0][n], hy[1][n]) and torch.equal(hy[0][n], ys[0][n].cpu())
        return ms_step

    e2e_kind = "one CUDA graph over three streams: uploads, the four chains and downloads overlap"
    try:
        e2e_step = e2e_pipelined_graph().replay
        e2e_step()
        torch.cuda.synchronize()
        for n in PROJECTIONS:                                  # the pipelined step must deliver the same bytes
            assert torch.equal(host_y[n], layer[n][2].cpu())
    except Exception as exc:   # noqa: BLE001 - a driver that cannot capture the multi-stream step: run it serially
        print(f"[bench] pipelined end-to-end step unavailable ({type(exc).__name__}: {exc}); timing the serial form", file=sys.stderr)
        e2e_step, e2e_kind = e2e_serial, "serial: uploads, one graph replay, downloads"
    e2e_ms = statistics.fmean(time_events(e2e_step, args.steps, warmup, flush))
    e2e_serial_ms = statistics.fmean(time_events(e2e_serial, args.steps, warmup, flush))
    e2e_stream_ms = None
    try:
        e2e_stream_ms = e2e_streamed(args.steps, warmup)
    except Exception as exc:   # noqa: BLE001 - report the single-step forms alone
        print(f"[bench] two-steps-in-flight end-to-end run unavailable ({type(exc).__name__}: {exc})", file=sys.stderr)
    sampler.stop_flag = True
    sampler.join(timeout=2)
    status = layer["qkv"][0].scratch.status()
    assert status[0] == 0, f"device status {status[:8]}"

    by = layer_bytes(M, distinct)
    total_bytes = sum(v["total"] for v in by.values())
    peak, peak_kind = measured_peaks()
    gu = by["gate_up"]
    k2_bytes = gu["w"] + gu["x"] + gu["b"] + gu["y"]
    k2_gbs = k2_bytes / (k2_ms * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": M / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3",
        "data": "synthetic",
        "config": {"workload": workload_name(M), "how": "K1->K2 PDL chains of the four projections in one CUDA graph",
                   "l2": "flushed by a 256 MB write before every timed replay"},
        "layer_us": ms * 1e3, "layer_us_median": statistics.median(ts) * 1e3, "projection_us": per_proj,
        "layer_bytes": total_bytes, "layer_gbs": total_bytes / (ms * 1e-3) / 1e9,
        "layer_frac_of_peak": total_bytes / (ms * 1e-3) / 1e9 / peak,
        "roofline": {"kernel": "k2_kernel<FP8 base, bf16 adapters> (gate_up, launched alone)", "bound": "hbm", "achieved": k2_gbs, "peak": peak,
                     "peak_kind": peak_kind, "unit": "GB/s", "frac": k2_gbs / peak, "traffic": None,
                     "traffic_note": "DRAM bytes are not readable from inside the run; one ncu capture of this launch "
                                     "(k2_kernel, gate_up, M = 32) read 178.5 MB against 174.85 MB algorithmic",
                     "bytes": k2_bytes,
                     "us": k2_ms * 1e3, "k1_us_alone": k1_ms * 1e3},
        "e2e": e2e_object(M, h2d, d2h, e2e_stream_ms, e2e_ms, e2e_kind, e2e_serial_ms),
        "gpu_launches": 8 * args.steps,
        "clocks": sampler.result(),
    }
    if not args.no_reference_gpu:
        line["reference_gpu"] = reference_gpu_in_child(M, min(args.steps, 50))
        if "layer_us" in line["reference_gpu"]:
            line["reference_gpu"]["reference_over_this_repo"] = line["reference_gpu"]["layer_us"] / line["layer_us"]
    if not args.no_tables:
        # the rest of the metric beside the headline cell: decode at M = 1 / 8 / 32 and one prefill batch, both base formats
        del layer, graph
        torch.cuda.empty_cache()
        line["decode_table"] = [measure_cell(b, "bf16", m, dev, flush, peak, peak_kind) for b in ("fp8", "nvfp4") for m in (1, 8, 32)]
        line["prefill_table"] = [measure_cell(b, "bf16", 2048, dev, flush, peak, peak_kind) for b in ("fp8", "nvfp4")]
    if not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        sec, sample, kind = cpu_layer_seconds(M, 2, threads)
        line["cpu_baseline"] = {"value": M / sec, "unit": "tokens/s", "cores": threads, "kind": kind, "sample": sample}
    print(json.dumps(line))


if __name__ == "__main__":
    main()
