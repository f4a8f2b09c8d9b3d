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


class PeerComm:
    """This rank's end of the peer-memory all-reduce (ob_allreduce): a zeroed communication buffer on the current device,
    exported by CUDA IPC and mapped into every other rank of `group`; handles travel through torch.distributed (host
    side, once).  `all_reduce(t)` is then ONE stream-ordered kernel launch, capturable in a CUDA graph, in place of the
    NCCL call vLLM makes after a row-parallel layer (tensor_model_parallel_all_reduce, row_parallel_linear.py:73-76).
    Every rank of the group must make the same calls in the same order."""

    def __init__(self, max_bytes: int, device, group=None, wait_ms: int = 2000):
        import ctypes as C

        import torch.distributed as dist

        from onebase_b200 import _lib
        self._lib, self._C = _lib, C
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert 2 <= self.world <= _lib.OB_MAX_RANKS
        self.wait_ms = wait_ms
        self.slot_bytes = (int(max_bytes) + 15) // 16 * 16
        size = C.c_size_t()
        _lib.call("ob_comm_bytes", self.slot_bytes, C.byref(size))
        with torch.cuda.device(device):
            self.buf = torch.zeros(size.value, dtype=torch.uint8, device=device)
            handle = C.create_string_buffer(64)
            offset = C.c_size_t()
            _lib.call("ob_ipc_export", C.c_void_p(self.buf.data_ptr()), handle, C.byref(offset))
            torch.cuda.synchronize(device)                     # the zeros are in memory before any peer may write a flag
            mine = (bytes(handle.raw), int(offset.value))
            everyone = [None] * self.world
            dist.all_gather_object(everyone, mine, group=group)
            self.comm = _lib.ObComm()
            self.comm.world, self.comm.rank, self.comm.slot_bytes = self.world, self.rank, self.slot_bytes
            self._mapped = []
            for r, (h, off) in enumerate(everyone):
                if r == self.rank:
                    self.comm.bufs[r] = self.buf.data_ptr()
                    continue
                ptr = C.c_void_p()
                _lib.call("ob_ipc_open", h, off, C.byref(ptr))
                self.comm.bufs[r] = ptr.value
                self._mapped.append((ptr.value, off))
        dist.barrier(group=group)                               # every rank has mapped every buffer

    def all_reduce(self, t: torch.Tensor, out: torch.Tensor | None = None, mode: int = 0) -> torch.Tensor:
        C, _lib = self._C, self._lib
        assert t.is_cuda and t.is_contiguous() and t.dtype in (torch.bfloat16, torch.float32)
        out = t if out is None else out
        _lib.call("ob_allreduce", C.byref(self.comm), C.c_void_p(t.data_ptr()), C.c_void_p(out.data_ptr()), t.numel(),
                  _lib.OB_DTYPE_BF16 if t.dtype == torch.bfloat16 else _lib.OB_DTYPE_F32, mode, self.wait_ms,
                  C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream))
        return out

    def status(self) -> list[int]:
        C = self._C
        st = (C.c_int32 * 8)()
        self._lib.call("ob_comm_status", C.byref(self.comm), st, C.c_void_p(torch.cuda.current_stream(self.buf.device).cuda_stream))
        return list(st)

    def close(self) -> None:
        for ptr, off in self._mapped:
            self._lib.lib().ob_ipc_close(self._C.c_void_p(ptr), off)
        self._mapped = []


# ------------------------------------------------------------------------------------------------------ benchmark
QWEN3_8B = {"qkv": (4096, (4096, 1024, 1024), "col"), "o": (4096, (4096,), "row"),
            "gate_up": (4096, (12288, 12288), "col"), "down": (12288, (4096,), "row")}
# the 72B-class layer of the tensor-parallel configuration: hidden 8192, 64 query / 8 kv heads of 128, intermediate 29568
L72B = {"qkv": (8192, (8192, 1024, 1024), "col"), "o": (8192, (8192,), "row"),
        "gate_up": (8192, (29568, 29568), "col"), "down": (29568, (8192,), "row")}


def time_sharded_layer(spec: dict, world: int, rank: int, dev, batch_sizes, comm, steps: int, flush) -> dict:
    """Layer time (us, mean over `steps` graph replays, L2 flushed, max over ranks) of `spec`'s decoder layer at tensor-
    parallel `world` for each batch size: this rank's shards are drawn directly at their shard shapes (timing only), the
    layer -- eight fused kernels and the two peer-memory all-reduces -- is one CUDA graph per batch size."""
    import torch.distributed as dist

    from onebase_b200.kernels.fp8_lora_vllm import VllmFusedFP8LoRA
    from onebase_b200.metadata import KernelMeta
    max_m = max(batch_sizes)
    g = torch.Generator(device=dev).manual_seed(1 + rank)
    ops = {}
    for name, (K, widths, kind) in spec.items():
        if kind == "col":
            kv_rep = max(1, world // 8) if name == "qkv" else 1        # kv slices are replicated when ranks outnumber kv heads
            widths_r = tuple(w // (world if s == 0 or name != "qkv" else max(1, world // kv_rep)) for s, w in enumerate(widths))
            K_r = K
        else:
            widths_r, K_r = widths, K // world
        N_r = sum(widths_r)
        w_q = torch.randint(0, 120, (N_r, K_r), device=dev, generator=g, dtype=torch.uint8).view(torch.float8_e4m3fn)
        s_w = torch.full((1,), 1e-3, device=dev)
        a_r = tuple(((torch.rand(L_SLOTS, 1, RANK, K_r, device=dev, generator=g) * 2 - 1) / K ** 0.5).to(torch.bfloat16) for _ in widths_r)
        b_r = tuple((torch.randn(L_SLOTS, 1, n, RANK, device=dev, generator=g) * 0.01).to(torch.bfloat16) for n in widths_r)
        ops[name] = (VllmFusedFP8LoRA(w_q, s_w, a_r, b_r, max_m=max_m), K_r, N_r, kind)
    out = {}
    for M in batch_sizes:
        ids = torch.randint(0, L_SLOTS, (M,), generator=torch.Generator().manual_seed(M), dtype=torch.int32).to(dev)
        km = KernelMeta.make(L_SLOTS, M, dev)
        km.prepare_tensors(ids)
        meta = km.meta_args(M)
        xs = {n: torch.randn(M, k, device=dev, generator=g).to(torch.bfloat16) for n, (_, k, _, _) in ops.items()}
        ys = {n: torch.empty(M, nn, dtype=torch.bfloat16, device=dev) for n, (_, _, nn, _) in ops.items()}

        def step():
            for n in ("qkv", "o", "gate_up", "down"):
                ops[n][0](xs[n], meta, out=ys[n])
                if ops[n][3] == "row":
                    comm.all_reduce(ys[n])

        for _ in range(2):
            step()
        torch.cuda.synchronize()
        dist.barrier()
        gph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gph):
            step()
        ts = []
        for i in range(steps + 3):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            gph.replay()
            e1.record()
            e1.synchronize()
            if i >= 3:
                ts.append(e0.elapsed_time(e1))
        ms = torch.tensor([statistics.fmean(ts)], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        out[str(M)] = round(float(ms.item()) * 1e3, 1)
        del gph
    st = ops["qkv"][0].scratch.status()
    out["device_status_ok"] = st[0] == 0
    return out
L_SLOTS, RANK = 32, 64


def nvfp4_layer_check(world: int, rank: int, dev, comm, M: int, steps: int, flush) -> dict:
    """The Qwen3-8B layer with an NVFP4 base at tensor-parallel `world`: every rank draws the same full tensors (random
    codes and block scales: both sides consume the same bytes), keeps its column / row shard (`shard_column_nvfp4`,
    `shard_row_nvfp4`), runs the layer -- eight fused kernels and the two peer-memory all-reduces -- as one CUDA graph, and
    checks (a) its all-reduced o / down outputs against the rank-ordered sum of every rank's partial output, gathered by
    NCCL (exact), (b) them against the unsharded NVFP4 op on the same tensors: the activation quantization is block-local
    against a static global scale, so sharding K changes only the summation order.  Returns errors and the layer time."""
    import torch.distributed as dist

    from onebase_b200.kernels.nvfp4_lora_vllm import VllmFusedNVFP4LoRA
    from onebase_b200.metadata import KernelMeta
    g = torch.Generator(device=dev).manual_seed(5)
    ids = torch.randint(0, L_SLOTS, (M,), generator=torch.Generator().manual_seed(0), dtype=torch.int32).to(dev)
    km = KernelMeta.make(L_SLOTS, M, dev)
    km.prepare_tensors(ids)
    meta = km.meta_args(M)
    w_global = 2688.0 / 0.1
    layer, y_full = {}, {}
    for name, (K, widths, kind) in QWEN3_8B.items():
        N = sum(widths)
        w_q4 = torch.randint(0, 256, (N, K // 2), device=dev, generator=g, dtype=torch.uint8)
        w_sf = torch.randint(0x30, 0x40, (N, K // 16), device=dev, generator=g, dtype=torch.uint8).view(torch.float8_e4m3fn)
        a_st = tuple(((torch.rand(L_SLOTS, 1, RANK, K, device=dev, generator=g) * 2 - 1) / K ** 0.5).to(torch.bfloat16) for _ in widths)
        b_st = tuple((torch.randn(L_SLOTS, 1, n, RANK, device=dev, generator=g) * 0.01).to(torch.bfloat16) for n in widths)
        x = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
        x_global = float(448.0 * 6.0 / x.float().abs().amax().clamp_min(1e-12))
        if kind == "row":
            full = VllmFusedNVFP4LoRA(w_q4, w_sf, w_global, x_global, a_st, b_st, max_m=M)
            y_full[name] = full(x, meta).clone()
            torch.cuda.synchronize()
            del full
            q_r, sf_r, a_r, b_r = shard_row_nvfp4(w_q4, w_sf, a_st, b_st, world, rank)
            x_r = shard_input_row(x, world, rank)
        else:
            rep = (1, max(1, world // 8), max(1, world // 8)) if name == "qkv" else ()
            q_r, sf_r, a_r, b_r = shard_column_nvfp4(w_q4, w_sf, a_st, b_st, world, rank, rep)
            x_r = x
        del w_q4, w_sf, a_st, b_st
        op = VllmFusedNVFP4LoRA(q_r, sf_r, w_global, x_global, a_r, b_r, max_m=M)
        layer[name] = (op, x_r, torch.empty(M, op.N, dtype=torch.bfloat16, device=dev), kind)
    torch.cuda.empty_cache()

    def step():
        for n in ("qkv", "o", "gate_up", "down"):
            op, x_n, y_n, kind = layer[n]
            op(x_n, meta, out=y_n)
            if kind == "row":
                comm.all_reduce(y_n)

    for _ in range(2):
        step()
    torch.cuda.synchronize()
    exact, check = {}, {}
    for n in ("o", "down"):
        op, x_n, y_n, _ = layer[n]
        part = torch.empty_like(y_n)
        op(x_n, meta, out=part)
        parts = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(parts, part)
        acc = torch.zeros_like(part, dtype=torch.float32)
        for t in parts:
            acc += t.float()
        exact[n] = float((y_n.float() - acc.to(torch.bfloat16).float()).abs().max() / acc.abs().max())
        ref = y_full[n].float()
        check[n] = float((y_n.float() - ref).abs().max() / ref.abs().max())
    dist.barrier()
    gph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gph):
        step()
    ts = []
    for i in range(steps + 3):
        flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        gph.replay()
        e1.record()
        e1.synchronize()
        if i >= 3:
            ts.append(e0.elapsed_time(e1))
    ms = torch.tensor([statistics.fmean(ts), max(exact.values()), max(check.values())], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    st = layer["qkv"][0].scratch.status()
    return {"layer_us": round(float(ms[0].item()) * 1e3, 1), "max_abs_err_over_ymax_vs_sum_of_rank_partials": float(ms[1].item()),
            "max_abs_err_over_ymax_vs_unsharded_op": float(ms[2].item()), "unsharded_bound": 2e-2,
            "ok": float(ms[1].item()) == 0.0 and float(ms[2].item()) <= 2e-2 and st[0] == 0,
            "workload": f"Qwen3-8B decoder layer, NVFP4 base, tensor-parallel {world}, decode M={M}, 32 bf16 tenants rank 64"}


def bench_tp(args, rank: int, world: int, local: int, metric: str) -> None:
    """One Qwen3-8B decoder layer at tensor-parallel size `world` (one process per GPU): column-parallel qkv / gate_up,
    row-parallel o / down each followed by an all-reduce of y -- by default the peer-memory kernel (ob_allreduce), so the
    whole layer (eight fused kernels + two all-reduces) is ONE CUDA graph; `--tp-comm nccl` issues NCCL all-reduces
    between two graphs instead.  Strong scaling: the same M tokens on every N.  Before timing, rank 0's all-reduced o /
    down outputs are checked against the unsharded op on the same seeded tensors.  Device time per step with CUDA events
    (max over ranks), L2 flushed before every step."""
    import datetime

    import torch.distributed as dist

    from onebase_b200.kernels.fp8_lora_vllm import VllmFusedFP8LoRA
    from onebase_b200.metadata import KernelMeta
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
    M = args.m
    sharded = getattr(args, "tp_form", "partial") == "sharded"   # row-parallel layers with sharded adapters
    use_nccl = getattr(args, "tp_comm", "peer") == "nccl"
    fuse_ar = getattr(args, "tp_comm", "peer") == "fused" and not sharded   # the all-reduce inside K2's epilogue
    warmup = max(3, args.warmup)
    g = torch.Generator(device=dev).manual_seed(0)            # same seed on every rank: identical full tensors, then sharded
    ids = torch.randint(0, L_SLOTS, (M,), generator=torch.Generator().manual_seed(0), dtype=torch.int32).to(dev)
    distinct = int(torch.unique(ids).numel())
    km = KernelMeta.make(L_SLOTS, M, dev)
    km.prepare_tensors(ids)
    meta = km.meta_args(M)
    layer, y_full = {}, {}
    rank_bytes = {}
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
        if kind == "row":                                        # the unsharded projection on the same tensors: the check's reference
            full = VllmFusedFP8LoRA(w_q, s_w, a_st, b_st, max_m=M)
            y_full[name] = full(x, meta).clone()
            torch.cuda.synchronize()
            del full
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
        # algorithmic bytes this rank moves for the projection: its W shard, its x, the distinct tenants' A and B shards, y
        rank_bytes[name] = (w_r.numel() + x_r.numel() * 2 + M * op.N * 2 +
                            distinct * (sum(t.shape[2] * t.shape[3] for t in a_r) + sum(t.shape[2] * t.shape[3] for t in b_r)) * 2)
    torch.cuda.empty_cache()

    y_o, y_down = layer["o"][2], layer["down"][2]
    hp_o = layer["o"][0].shrink_partials(M) if sharded else None
    hp_down = layer["down"][0].shrink_partials(M) if sharded else None
    comm = None
    if not use_nccl:
        largest = max(y_o.numel() * 2, y_down.numel() * 2, (hp_o.numel() * 4 if sharded else 0), (hp_down.numel() * 4 if sharded else 0))
        comm = PeerComm(largest, dev)

    def reduce(t):
        if use_nccl:
            dist.all_reduce(t)
        else:
            comm.all_reduce(t)

    def chain(name, **kw):
        op, x, y, _ = layer[name]
        op(x, meta, out=y, **kw)

    def step():
        """The whole layer in stream order."""
        chain("qkv")
        if sharded:
            chain("o", gemm=False)
            reduce(hp_o)
            chain("o", shrink=False)
            reduce(y_o)
        elif fuse_ar:
            chain("o", allreduce=comm)
        else:
            chain("o")
            reduce(y_o)
        chain("gate_up")
        if sharded:
            chain("down", gemm=False)
            reduce(hp_down)
            chain("down", shrink=False)
            reduce(y_down)
        elif fuse_ar:
            chain("down", allreduce=comm)
        else:
            chain("down")
            reduce(y_down)

    def log(msg):
        if os.environ.get("LOWBIT_VERBOSE"):
            print(f"[tp rank {rank}] {msg}", flush=True)

    for _ in range(2):                                        # eager warm-up: kernels, scratch, communicator
        step()
    torch.cuda.synchronize()
    log("eager warm-up done")
    # ---- correctness of the exchange before timing.  (a) The all-reduced o / down outputs against the sum of every rank's
    # partial output, gathered by NCCL and added in rank order in fp32: exact for the peer-memory kernel, one bf16 rounding
    # per hop off for NCCL's ring.  (b) Against the unsharded projection on the same seeded tensors: equal up to the two
    # activation quantizations (a rank scales its K slice of a token by the slice's own amax).
    check, exact = {}, {}
    for name, y in (("o", y_o), ("down", y_down)):
        op_n, x_n, _, _ = layer[name]
        part = torch.empty_like(y)
        if sharded:
            op_n(x_n, meta, out=part, gemm=False)
            reduce(op_n.shrink_partials(M))
            op_n(x_n, meta, out=part, shrink=False)
        else:
            op_n(x_n, meta, out=part)
        parts = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(parts, part)
        acc = torch.zeros_like(part, dtype=torch.float32)
        for t in parts:
            acc += t.float()
        exact[name] = float((y.float() - acc.to(torch.bfloat16).float()).abs().max() / acc.abs().max())
        ref = y_full[name].float()
        check[name] = float((y.float() - ref).abs().max() / ref.abs().max())
    worst = torch.tensor([max(check.values()), max(exact.values())], device=dev)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    same = torch.stack([y_o.float().sum(), y_down.float().sum()])
    lo, hi = same.clone(), same.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    ranks_agree = bool(torch.equal(lo, hi))                   # every rank holds the same reduced outputs
    exact_bound = 0.0 if not use_nccl else 1e-2
    tp_ok = float(worst[1].item()) <= exact_bound and float(worst[0].item()) <= 6e-2 and ranks_agree
    log(f"exchange check: vs sum of partials {exact}, vs the unsharded op {check}, ranks agree = {ranks_agree}")

    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    graphs = []
    if use_nccl:
        # NCCL stays outside the graphs: the kernels of each half are captured, the collectives are issued between replays
        pieces = ([lambda: (chain("qkv"), chain("o", gemm=False)), lambda: chain("o", shrink=False),
                   lambda: (chain("gate_up"), chain("down", gemm=False)), lambda: chain("down", shrink=False)] if sharded
                  else [lambda: (chain("qkv"), chain("o")), lambda: (chain("gate_up"), chain("down"))])
    else:
        pieces = [step]
    for piece in pieces:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            piece()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        dist.barrier()
        gph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gph):
            piece()
        graphs.append(gph)
    torch.cuda.synchronize()
    dist.barrier()
    log("graphs captured")

    def run():
        if not use_nccl:
            graphs[0].replay()
        elif sharded:
            graphs[0].replay(); dist.all_reduce(hp_o); graphs[1].replay(); dist.all_reduce(y_o)
            graphs[2].replay(); dist.all_reduce(hp_down); graphs[3].replay(); dist.all_reduce(y_down)
        else:
            graphs[0].replay(); dist.all_reduce(y_o); graphs[1].replay(); dist.all_reduce(y_down)

    def timed(fn, steps):
        ts = []
        for _ in range(steps):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            ts.append(e0.elapsed_time(e1))
        return ts

    for _ in range(warmup):
        flush.fill_(1)
        run()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    ts = timed(run, args.steps)
    torch.cuda.synchronize()
    dist.barrier()
    ms = torch.tensor([statistics.fmean(ts)], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)

    # ---- end to end: this rank's activations from pinned host memory, the layer, rank outputs back to the host
    host_x = {n: layer[n][1].cpu().pin_memory() for n in layer}
    host_y = {n: torch.empty(layer[n][2].shape, dtype=torch.bfloat16).pin_memory() for n in layer}

    def e2e_step():
        for n in layer:
            layer[n][1].copy_(host_x[n], non_blocking=True)
        run()
        for n in layer:
            host_y[n].copy_(layer[n][2], non_blocking=True)

    for _ in range(3):
        flush.fill_(1)
        e2e_step()
    torch.cuda.synchronize()
    dist.barrier()
    e2e_ts = timed(e2e_step, args.steps)
    e2e_ms = torch.tensor([statistics.fmean(e2e_ts)], device=dev)
    dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    h2d = sum(t.numel() * 2 for t in host_x.values())
    d2h = sum(t.numel() * 2 for t in host_y.values())

    # ---- the dominant kernel on this rank: K2 of the gate_up shard, launched alone
    op_g, x_g, y_g, _ = layer["gate_up"]
    op_g(x_g, meta, out=y_g)
    gk2 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gk2):
        op_g(x_g, meta, out=y_g, shrink=False, pdl=False)
    k2_ms = statistics.fmean(timed(gk2.replay, 30))
    k2_bytes = (op_g.w_q.numel() + M * op_g.K + M * op_g.N * 2 + distinct * op_g.N * RANK * 2)

    # ---- the exchange alone (one all-reduce of y_o in a graph of its own), and the 72B-class layer of the tensor-parallel
    # configuration at this N (decode M = 8, 32, 128); both with the peer-memory kernel only
    ar_us, config4, nvfp4_tp = None, None, None
    status = layer["qkv"][0].scratch.status()
    if comm is not None:
        g_ar = torch.cuda.CUDAGraph()                          # eight in a row: the ranks' start skew is paid once, not per call
        with torch.cuda.graph(g_ar):
            for _ in range(8):
                comm.all_reduce(y_o)
        dist.barrier()
        ar_ms = torch.tensor([statistics.fmean(timed(g_ar.replay, 30)) / 8], device=dev)
        dist.all_reduce(ar_ms, op=dist.ReduceOp.MAX)
        ar_us = float(ar_ms.item()) * 1e3
        if not getattr(args, "no_config4", False):
            del layer, op_g, x_g, y_g, gk2, graphs
            torch.cuda.empty_cache()
            big = PeerComm(128 * 8192 * 2, dev)
            config4 = time_sharded_layer(L72B, world, rank, dev, (8, 32, 128), big, 20, flush)
            config4["workload"] = (f"72B-class decoder layer (hidden 8192, intermediate 29568) at tensor-parallel {world}, FP8 base, "
                                   "32 bf16 tenants rank 64, one CUDA graph per batch size; layer us by decode batch size")
            big.close()
            nvfp4_tp = nvfp4_layer_check(world, rank, dev, comm, M, 20, flush)
    ok = torch.tensor([1 if status[0] == 0 and (comm is None or comm.status()[3] == 0) and
                       (config4 is None or config4["device_status_ok"]) else 0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        import json as _json
        from pathlib import Path
        ms_v = float(ms.item())
        peaks = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
        peak, peak_kind = (float(_json.loads(peaks.read_text())["hbm_gbs"]), "measured") if peaks.exists() else (6650.0, "fallback")
        k2_gbs = k2_bytes / (k2_ms * 1e-3) / 1e9
        total_rank_bytes = sum(rank_bytes.values())
        print(json.dumps({
            "metric": metric, "value": M / (ms_v * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_v, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "fp8_e4m3", "data": "synthetic",
            "config": {"workload": f"Qwen3-8B decoder layer at tensor-parallel {world}: column-parallel qkv / gate_up, row-parallel "
                                   f"o / down + all-reduce of y ({'NCCL' if use_nccl else 'over peer memory inside K2 epilogues' if fuse_ar else 'peer-memory kernel, in the graph'})"
                                   f"{' (adapters sharded too: all-reduce of the shrink partials before the expand)' if sharded else ''}"
                                   f"; FP8 base, decode M={M}, 32 bf16 tenants rank 64 ({distinct} distinct)",
                       "l2": "flushed by a 256 MB write before every timed step",
                       "cuda_graph": (f"{len(graphs)} graphs; the NCCL all-reduces are launched between them" if use_nccl
                                      else "one graph: 8 fused kernels per rank, the two all-reduces inside K2's epilogues" if fuse_ar
                                      else "one graph: 8 fused kernels + 2 all-reduce kernels per rank")},
            "layer_us": ms_v * 1e3, "allreduce_us_alone": ar_us, "config4": config4, "nvfp4_tp": nvfp4_tp,
            "gpu_launches": (8 if use_nccl or fuse_ar else 10) * args.steps,   # our kernels per step: four K1, four K2 (+ two all-reduces)
            "device_status_ok": bool(ok.item()),
            "tp_check": {"max_abs_err_over_ymax_vs_sum_of_rank_partials": exact, "exchange_bound": exact_bound,
                         "max_abs_err_over_ymax_vs_unsharded_op": check, "unsharded_bound": 6e-2,
                         "note": "the unsharded op quantizes a token's activations once, a rank its K slice with the slice's own "
                                 "scale: two FP8 roundings of the same activations, not an exchange error",
                         "ranks_bitwise_equal": ranks_agree, "ok": tp_ok},
            "rank_bytes_per_step": total_rank_bytes, "rank_gbs": total_rank_bytes / (ms_v * 1e-3) / 1e9,
            "remaining_per_rank": "every rank still runs the whole shrink of the column-parallel layers (A is not sharded) "
                                  "and K1's latency does not shrink with N",
            "e2e": {"value": M / (float(e2e_ms.item()) * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": float(e2e_ms.item()),
                    "how": "per rank: uploads, the layer, downloads, serial on one stream; max over ranks"},
            "roofline": {"kernel": "k2_kernel<FP8 base, bf16 adapters> (this rank's gate_up shard, launched alone)", "bound": "hbm",
                         "achieved": k2_gbs, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": k2_gbs / peak,
                         "traffic": None, "bytes": k2_bytes, "us": k2_ms * 1e3},
            "cpu_baseline": None}))
    if comm is not None:
        comm.close()
    dist.destroy_process_group()
