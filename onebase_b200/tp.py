"""Tensor-parallel sharding of the fused projection, as vLLM shards LoRA linear layers.

Column-parallel (qkv, gate_up): every slice's output rows are split across ranks -- W rows and B rows
`[rank * w_s, (rank + 1) * w_s)` of each slice with `w_s = width_s / tp` (vllm/lora/layers/column_parallel_linear.py:
251-262; for qkv the kv slices are replicated when there are fewer kv heads than ranks, :442-463); A is not sliced, so
the whole shrink runs on every rank and there is NO collective.
Row-parallel (o, down): K is split -- W columns and A columns `[rank * K/tp, (rank + 1) * K/tp)`, all of B
(vllm/lora/layers/row_parallel_linear.py:32-40); each rank computes a partial base GEMM plus a partial LoRA term and the
layer all-reduces `y [M, N]` (bf16, NCCL over NVLink) (:73-76).  This is the form the reference's plugin serves under
LOWBIT_TP=1 (lowbit_lora/plugin.py:239-245).  With sharded adapters (:118-160) B is split by output rows as well: the
ranks first all-reduce the fp32 shrink partials, then each adds the expand to its own output features before the
all-reduce of y.  The shard functions are plain tensor slicing and work on any device.
"""
from __future__ import annotations

import json
import os
import statistics

import torch


def shard_column(w_q, a_stacked, b_stacked, tp: int, rank: int, replicate=()):
    """Per-rank (w_q, a_stacked, b_stacked) of a column-parallel projection.  `replicate[s]` > 1 means slice s is
    replicated over that many consecutive ranks (kv heads fewer than ranks)."""
    widths = [t.shape[2] for t in b_stacked]
    rows, b_out, off = [], [], 0
    for s, w in enumerate(widths):
        rep = replicate[s] if s < len(replicate) else 1
        parts = max(1, tp // rep)
        assert w % parts == 0, f"slice {s} of width {w} does not split into {parts} shards"
        ws = w // parts
        sid = rank // rep if rep > 1 else rank
        lo = (sid % parts) * ws
        rows.append(w_q[off + lo: off + lo + ws])
        b_out.append(b_stacked[s][:, :, lo:lo + ws].contiguous())
        off += w
    return torch.cat(rows, 0).contiguous(), tuple(a_stacked), tuple(b_out)


def shard_row(w_q, a_stacked, b_stacked, tp: int, rank: int):
    """Per-rank (w_q, a_stacked, b_stacked) of a row-parallel projection (K split; B whole)."""
    K = w_q.shape[1]
    assert K % tp == 0
    ks = K // tp
    lo = rank * ks
    return (w_q[:, lo:lo + ks].contiguous(), tuple(a[..., lo:lo + ks].contiguous() for a in a_stacked), tuple(b_stacked))


def shard_row_sharded_lora(w_q, a_stacked, b_stacked, tp: int, rank: int):
    """Per-rank (w_q, a_stacked, b_stacked, b_shard) of a row-parallel projection whose adapters are sharded too (vLLM's
    RowParallelLinearWithShardedLoRA, vllm/lora/layers/row_parallel_linear.py:118-160): W and A by K as in shard_row, and
    of each slice's B only rows [rank * N_s / tp, (rank + 1) * N_s / tp).  `b_shard` = [(first row, rows, slice width)]
    is what the op's constructor takes.  The shard boundaries must fall on 128-row tiles."""
    w_r, a_r, _ = shard_row(w_q, a_stacked, b_stacked, tp, rank)
    b_r, b_shard = [], []
    for b in b_stacked:
        n_s = b.shape[2]
        assert n_s % tp == 0 and (n_s // tp) % 128 == 0, f"slice of width {n_s} does not split into {tp} shards of whole tiles"
        rows = n_s // tp
        b_r.append(b[:, :, rank * rows:(rank + 1) * rows].contiguous())
        b_shard.append((rank * rows, rows, n_s))
    return w_r, a_r, tuple(b_r), b_shard


def shard_column_nvfp4(w_q4, w_sf, a_stacked, b_stacked, tp: int, rank: int, replicate=()):
    """Column-parallel shard of an NVFP4 base (the reference's plugin refuses NVFP4 under tensor parallelism,
    lowbit_lora/plugin.py:199): the rank's rows of the packed codes [N, K/2] and of the linear block scales [N, K/16]; the
    two global scales are per tensor and stay.  Returns (w_q4, w_sf, a_stacked, b_stacked)."""
    q_r, a_r, b_r = shard_column(w_q4, a_stacked, b_stacked, tp, rank, replicate)
    sf_r, _, _ = shard_column(w_sf.view(torch.uint8), a_stacked, b_stacked, tp, rank, replicate)
    return q_r, sf_r.view(w_sf.dtype), a_r, b_r


def shard_row_nvfp4(w_q4, w_sf, a_stacked, b_stacked, tp: int, rank: int):
    """Row-parallel shard of an NVFP4 base: K elements [rank * K/tp, (rank + 1) * K/tp) are columns [lo/2, hi/2) of the
    packed codes and [lo/16, hi/16) of the block scales (K/tp must be a multiple of 32: whole scale blocks, and code rows
    that keep the 16-byte stride TMA needs).  The activation quantization is block-local against a static global scale, so
    a rank's codes of its K slice equal the unsharded ones.  Returns (w_q4, w_sf, a_stacked, b_stacked)."""
    K = w_q4.shape[1] * 2
    assert K % tp == 0 and (K // tp) % 32 == 0, f"K = {K} does not split into {tp} shards of whole 32-element groups"
    ks = K // tp
    lo = rank * ks
    return (w_q4[:, lo // 2:(lo + ks) // 2].contiguous(), w_sf[:, lo // 16:(lo + ks) // 16].contiguous(),
            tuple(a[..., lo:lo + ks].contiguous() for a in a_stacked), tuple(b_stacked))


def run_row_parallel_sharded(op, x_r, meta_args, out=None, cfg=None, group=None):
    """One row-parallel projection with sharded adapters on this rank: K1 on the rank's K slice, all-reduce of the fp32
    shrink partials (a few hundred KB at most), K2 with the expand on the rank's output features only, all-reduce of y.
    The two collectives are the exchange steps of this form (row_parallel_linear.py:135-160 and :73-76)."""
    import torch.distributed as dist
    M = x_r.shape[0]
    y = op(x_r, meta_args, out=out, cfg=cfg, gemm=False)
    multi = dist.is_initialized() and dist.get_world_size(group) > 1
    if multi:
        dist.all_reduce(op.shrink_partials(M, cfg), op=dist.ReduceOp.SUM, group=group)
    y = op(x_r, meta_args, out=y, cfg=cfg, shrink=False)
    if multi:
        dist.all_reduce(y, op=dist.ReduceOp.SUM, group=group)
    return y


def shard_input_row(x, tp: int, rank: int):
    """A row-parallel layer's input is already split along K (the previous column-parallel layer's output shard)."""
    ks = x.shape[1] // tp
    return x[:, rank * ks:(rank + 1) * ks].contiguous()


def all_reduce_output(y: torch.Tensor, group=None) -> torch.Tensor:
    """The row-parallel layer's exchange step: sum of the ranks' partial outputs (vLLM's tensor_model_parallel_all_reduce)."""
    import torch.distributed as dist
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(y, op=dist.ReduceOp.SUM, group=group)
    return y


# ------------------------------------------------------------------------------------------------------ benchmark
QWEN3_8B = {"qkv": (4096, (4096, 1024, 1024), "col"), "o": (4096, (4096,), "row"),
            "gate_up": (4096, (12288, 12288), "col"), "down": (12288, (4096,), "row")}
L_SLOTS, RANK = 32, 64


def bench_tp(args, rank: int, world: int, local: int, metric: str) -> None:
    """One Qwen3-8B decoder layer at tensor-parallel size `world` (one process per GPU, NCCL): column-parallel qkv /
    gate_up, row-parallel o / down each followed by an all-reduce of y.  Strong scaling: the same M tokens on every N.
    Device time per step with CUDA events (max over ranks), L2 flushed before every step."""
    import torch.distributed as dist
    from onebase_b200.kernels.fp8_lora_vllm import VllmFusedFP8LoRA
    from onebase_b200.metadata import KernelMeta
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    import datetime
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
    M = args.m
    sharded = getattr(args, "tp_form", "partial") == "sharded"   # row-parallel layers with sharded adapters
    warmup = max(3, args.warmup)
    g = torch.Generator(device=dev).manual_seed(0)            # same seed on every rank: identical full tensors, then sharded
    ids = torch.randint(0, L_SLOTS, (M,), generator=torch.Generator().manual_seed(0), dtype=torch.int32).to(dev)
    km = KernelMeta.make(L_SLOTS, M, dev)
    km.prepare_tensors(ids)
    meta = km.meta_args(M)
    layer = {}
    for name, (K, widths, kind) in QWEN3_8B.items():
        N = sum(widths)
        w = torch.randn(N, K, device=dev, generator=g) * 0.02
        s_w = (w.abs().max() / 448.0).reshape(1).float()
        w_q = (w / s_w).to(torch.float8_e4m3fn)
        del w
        a_st = tuple(((torch.rand(L_SLOTS, 1, RANK, K, device=dev, generator=g) * 2 - 1) / K ** 0.5).to(torch.bfloat16)
                     for _ in widths)
        b_st = tuple((torch.randn(L_SLOTS, 1, n, RANK, device=dev, generator=g) * 0.01).to(torch.bfloat16) for n in widths)
        x = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
        b_shard = None
        if kind == "col":
            rep = (1, max(1, world // 8), max(1, world // 8)) if name == "qkv" else ()
            w_r, a_r, b_r = shard_column(w_q.view(torch.uint8), a_st, b_st, world, rank, rep)
            x_r = x
        elif sharded:
            w_r, a_r, b_r, b_shard = shard_row_sharded_lora(w_q.view(torch.uint8), a_st, b_st, world, rank)
            x_r = shard_input_row(x, world, rank)
        else:
            w_r, a_r, b_r = shard_row(w_q.view(torch.uint8), a_st, b_st, world, rank)
            x_r = shard_input_row(x, world, rank)
        del w_q, a_st, b_st
        op = VllmFusedFP8LoRA(w_r.view(torch.float8_e4m3fn), s_w, a_r, b_r, max_m=M, b_shard=b_shard)
        layer[name] = (op, x_r, torch.empty(M, op.N, dtype=torch.bfloat16, device=dev), kind)
    torch.cuda.empty_cache()

    def half(names):
        for name in names:
            op, x, y, _ = layer[name]
            op(x, meta, out=y)

    def col_then_k1(col, row):       # sharded adapters: the column-parallel chain, then the row-parallel layer's K1
        op, x, y, _ = layer[col]
        op(x, meta, out=y)
        op, x, y, _ = layer[row]
        op(x, meta, out=y, gemm=False)

    def k2_only(row):
        op, x, y, _ = layer[row]
        op(x, meta, out=y, shrink=False)

    hp_o = layer["o"][0].shrink_partials(M) if sharded else None
    hp_down = layer["down"][0].shrink_partials(M) if sharded else None

    def log(msg):
        if os.environ.get("LOWBIT_VERBOSE"):
            print(f"[tp rank {rank}] {msg}", flush=True)

    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    y_o, y_down = layer["o"][2], layer["down"][2]
    def eager_step():
        if sharded:
            col_then_k1("qkv", "o")
            dist.all_reduce(hp_o)
            k2_only("o")
            dist.all_reduce(y_o)
            col_then_k1("gate_up", "down")
            dist.all_reduce(hp_down)
            k2_only("down")
            dist.all_reduce(y_down)
        else:
            half(("qkv", "o"))
            dist.all_reduce(y_o)
            half(("gate_up", "down"))
            dist.all_reduce(y_down)

    for _ in range(2):                                        # eager warm-up: kernels, scratch, NCCL communicator
        eager_step()
    torch.cuda.synchronize()
    log("eager warm-up done")
    # The kernels of each half are captured in a CUDA graph; the two all-reduces are issued between the replays (NCCL is
    # not captured: the collective stays an ordinary stream-ordered launch).
    graphs = []
    pieces = ([lambda: col_then_k1("qkv", "o"), lambda: k2_only("o"), lambda: col_then_k1("gate_up", "down"),
               lambda: k2_only("down")] if sharded else [lambda: half(("qkv", "o")), lambda: half(("gate_up", "down"))])
    for piece in pieces:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            piece()
        torch.cuda.current_stream().wait_stream(side)
        gph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gph):
            piece()
        graphs.append(gph)
    torch.cuda.synchronize()
    log("graphs captured")
    graphed = True

    def run():
        if sharded:
            graphs[0].replay()
            dist.all_reduce(hp_o)
            graphs[1].replay()
            dist.all_reduce(y_o)
            graphs[2].replay()
            dist.all_reduce(hp_down)
            graphs[3].replay()
            dist.all_reduce(y_down)
        else:
            graphs[0].replay()
            dist.all_reduce(y_o)
            graphs[1].replay()
            dist.all_reduce(y_down)

    for _ in range(warmup):
        flush.fill_(1)
        run()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    ts = []
    for _ in range(args.steps):
        flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1))
    torch.cuda.synchronize()
    dist.barrier()
    ms = torch.tensor([statistics.fmean(ts)], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    status = layer["qkv"][0].scratch.status()
    ok = torch.tensor([1 if status[0] == 0 else 0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        ms_v = float(ms.item())
        print(json.dumps({
            "metric": metric, "value": M / (ms_v * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_v, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "fp8_e4m3", "data": "synthetic",
            "config": {"workload": f"Qwen3-8B decoder layer at tensor-parallel {world}: column-parallel qkv / gate_up, row-parallel "
                                   f"o / down + NCCL all-reduce of y"
                                   f"{' (adapters sharded too: all-reduce of the shrink partials before the expand)' if sharded else ''}"
                                   f"; FP8 base, decode M={M}, 32 bf16 tenants rank 64",
                       "l2": "flushed by a 256 MB write before every timed step",
                       "cuda_graph": f"{len(graphs)} graphs; the NCCL all-reduces are launched between them" if graphed else "no"},
            "layer_us": ms_v * 1e3, "gpu_launches": 8 * args.steps,   # our kernels: four K1 + four K2 per step
            "device_status_ok": bool(ok.item()),
            "e2e": None, "roofline": None, "cpu_baseline": None}))
    dist.destroy_process_group()
