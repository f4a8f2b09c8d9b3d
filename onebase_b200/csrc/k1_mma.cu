// K1b: the LoRA shrink h = x A^T of a prefill batch on the tensor cores (bf16 adapters, more than 32 tokens).
//
// The CUDA-core shrink of k1_fp8.cu re-reads an adapter's A once per four tokens; with hundreds of tokens per tenant that
// is hundreds of megabytes of L2 traffic.  Here a CTA owns (128 adapter-sorted positions, slice, K split) and multiplies
// its 128 x K tile of x with the A of EVERY tenant that has a position in the tile, one fp32 accumulator of R columns in
// tensor memory per tenant (tcgen05.mma kind::f16, M = 128 positions, N = R).  Rows of a tenant's accumulator that belong
// to other tenants' positions are computed and thrown away -- a tile of a sorted batch holds two or three tenants, and the
// shrink is a small share of the layer's flops.  Operands arrive by TMA through a shared-memory ring: the x tile comes
// from the adapter-sorted bf16 copy of x that K1's quantizing CTAs leave in the workspace, the A tiles straight from the
// stacked adapters.  Output: the split-K partials hp[split][slice][position][rank] (fp32) that K2 adds in split order,
// the same array the CUDA-core shrink writes.  Computes what lowbit_lora/kernels/fp8_lora_vllm.py:72-120 computes.
//
// K splits: the splits of a (tile, slice) are ONE thread-block cluster where the launch allows (2 or 4 splits, the
// rank divisible among them, one accumulator pass): each CTA leaves its positions' own-tenant rows (fp32) in its idle
// ring, the cluster meets at a barrier, and split j adds rows j * 128 / splits ... of all the splits in split order over
// distributed shared memory and writes the finished h -- no partials in the workspace, no arrival counter, no last
// arriver that reduces alone (that tail took 7 of the kernel's 25 us).  Otherwise the partials go through the
// workspace: the splits count their arrivals and the last one adds them, in the same order.
//
// Warp roles: 0 = TMA producer, 1 = MMA issuer (and the owner of the tensor-memory allocation), 2..5 = epilogue (warp w
// reads the 32 accumulator lanes w % 4 may touch).  Every wait is bounded; a wait that runs out records where in the
// workspace's status words and the CTA leaves without storing.
#include "ob_common.cuh"
#include "ob_ptx.cuh"

namespace ob {

constexpr int kMmaThreads = 192;
constexpr int kMmaTile = 128;          // positions per CTA (the MMA's M)
constexpr int kMmaKStep = 64;          // bf16 elements per ring slot: one 128-byte swizzle atom
constexpr int kMmaXBytes = kMmaTile * kMmaKStep * 2;       // 16 KB
constexpr int kMmaMaxCols = 512;       // tensor-memory columns: R per tenant in flight
constexpr int kMmaMaxStages = 8;
constexpr int kMmaMaxList = 128;       // tenants with a position in one tile
constexpr int kMmaMaxSeg = 257;        // segments of a batch: at most 256 tenants and the positions without one

struct K1mCtrl {
    uint64_t full[kMmaMaxStages];
    uint64_t empty[kMmaMaxStages];
    uint64_t acc_full;
    uint64_t acc_empty;
    uint32_t tmem_base;
    volatile int abort_flag;
    int n_list;
    int wi_tile;                       // this CTA's work item: position tile and first list entry of its tenant group
    int wi_g0;
    int wait_before_exit;
    int last_flag;
    int lora[kMmaMaxList];             // the tile's tenants in segment order
    short gidx[kMmaTile];              // list entry of each position (-1: no adapter)
};

__device__ __forceinline__ void k1m_timeout(const K1mParams& p, K1mCtrl* c, int where, int it) {
    c->abort_flag = 1;
    if (atomicCAS(p.status, OB_DEV_OK, OB_DEV_WAIT_TIMEOUT) == OB_DEV_OK) {
        p.status[1] = 100 + where;
        p.status[2] = blockIdx.x;
        p.status[3] = blockIdx.y;
        p.status[4] = blockIdx.z;
        p.status[5] = it;
    }
}

// GROUPS: a tile's tenants are dealt out to several CTAs (p.tg_cap of them each); false: one CTA per tile, the grid's x is
// the tile (two instantiations: the one-CTA-per-tile form compiled with the group logic beside it measured slower).
template <bool GROUPS>
__global__ void __launch_bounds__(kMmaThreads, 1)
k1_mma_kernel(const K1mParams p, const __grid_constant__ CUtensorMap tm_xs, const __grid_constant__ CUtensorMap tm_a0,
              const __grid_constant__ CUtensorMap tm_a1, const __grid_constant__ CUtensorMap tm_a2,
              const __grid_constant__ CUtensorMap tm_a3) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* ring = smem;
    K1mCtrl* ctrl = reinterpret_cast<K1mCtrl*>(smem + p.ring_bytes);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    griddep_launch_dependents();
    const uint64_t limit_ns = (uint64_t)p.wait_ms * 1000000ull;
    // Work item, slice and K split of this CTA, numbered so that CTAs are dispatched in work-item order (the grid's x runs
    // fastest): the CTAs beyond the launch's last item -- the grid is the host's upper bound -- then come last instead of
    // taking SMs ahead of working ones.  A cluster is the grid's z extent (rank = split), so only x and y are folded there.
    int wi, s, j;
    if (!GROUPS) {                                            // one CTA per tile: every CTA has a work item
        wi = (int)blockIdx.x; s = (int)blockIdx.y; j = (int)blockIdx.z;
    } else if (p.cluster) {
        const int lin = (int)(blockIdx.x + gridDim.x * blockIdx.y);
        j = (int)blockIdx.z; s = lin % p.S; wi = lin / p.S;
    } else {
        int lin = (int)(blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z));
        j = lin % p.split1; lin /= p.split1; s = lin % p.S; wi = lin / p.S;
    }
    const int k0 = j * p.k_per_split, k1 = min(p.K, k0 + p.k_per_split);
    const int n_ksteps = k1 > k0 ? (k1 - k0 + kMmaKStep - 1) / kMmaKStep : 0;
    const int a_bytes = p.R * kMmaKStep * 2;                  // one tenant's A tile of a ring slot
    const int group = kMmaMaxCols / p.R;                      // tenants whose accumulators fit tensor memory at once

    if (tid == 0) {
        for (int i = 0; i < kMmaMaxStages; ++i) {
            mbar_init(&ctrl->full[i], 1);
            mbar_init(&ctrl->empty[i], 1);
        }
        mbar_init(&ctrl->acc_full, 1);
        mbar_init(&ctrl->acc_empty, 4);
        ctrl->abort_flag = 0;
        ctrl->n_list = 0;
        fence_mbar_init();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tm_xs);
        tma_prefetch_desc(s == 0 ? &tm_a0 : s == 1 ? &tm_a1 : s == 2 ? &tm_a2 : &tm_a3);
    }
    for (int c = tid; c < kMmaTile; c += kMmaThreads) ctrl->gidx[c] = -1;
    __syncthreads();
    // ---- this CTA's work item and the tile's tenants, from the segment index (static during the preceding kernels)
    if (warp == 2) {
        int n_all, n_ad;
        segment_totals(p.meta, p.L, lane, n_all, n_ad);
        n_all = min(n_all, p.M);
        // (tile, tenant group) number wi in tile order.  First and last tile of every segment go to shared memory;
        // then a lane is one tile of a batch of 32 and counts the segments that cover it.
        const int n_tiles = (p.M + kMmaTile - 1) / kMmaTile, w = wi;
        // (the two arrays lie in the still idle operand ring, not in the control block: a launch whose shared memory crosses
        // 196 KB measured 10-16 us slower -- the SM then has no first-level cache left.  The fence below orders this warp's
        // accesses before the TMA writes that follow the block's barrier.)
        const int n_seg = GROUPS ? min(p.L + 1, kMmaMaxSeg) : 0;
        int* seg_first = reinterpret_cast<int*>(ring);
        int* seg_last = seg_first + kMmaMaxSeg;
        for (int i = lane; i < n_seg; i += 32) {
            const int lora = __ldg(p.meta.seg_ids + i), n = __ldg(p.meta.seg_n + i), sst = __ldg(p.meta.seg_start + i);
            const int end = min(sst + n, n_all);
            const bool ok = lora >= 0 && lora < p.L && n > 0 && sst >= 0 && sst < end;
            seg_first[i] = ok ? sst / kMmaTile : 0x7fffffff;
            seg_last[i] = ok ? (end - 1) / kMmaTile : -1;
        }
        __syncwarp();
        int acc = 0, tile = -1, first = 0;
        if (!GROUPS) {                                        // one CTA per tile: the work item is the tile
            tile = (w < n_tiles && n_ad > 0) ? w : -1;
            acc = 0;
        }
        // (the CTA of the grid's last work item counts on to the end: more items than the host's bound allowed for means the
        // index is not made of disjoint contiguous segments, and the status words say so instead of a silently short h)
        const bool count_all = GROUPS && w == (int)gridDim.x - 1 && s == 0 && j == 0;
        for (int tb = 0; GROUPS && tb < n_tiles && (tile < 0 || count_all) && n_ad > 0; tb += 32) {
            const int t = tb + lane;
            int cnt = 0;
            for (int i = 0; i < n_seg; ++i) cnt += (seg_first[i] <= t && t <= seg_last[i]) ? 1 : 0;
            const int items = t < n_tiles ? (min(cnt, kMmaMaxList) + p.tg_cap - 1) / p.tg_cap : 0;
            int pre = items;                                  // inclusive prefix over the batch's tiles
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, pre, o);
                if (lane >= o) pre += v;
            }
            const uint32_t hit = tile < 0 ? __ballot_sync(0xffffffffu, w >= acc + pre - items && w < acc + pre) : 0u;
            if (hit) {
                const int src = __ffs(hit) - 1;
                tile = tb + src;
                first = (w - acc - __shfl_sync(0xffffffffu, pre - items, src)) * p.tg_cap;
            }
            acc += __shfl_sync(0xffffffffu, pre, 31);
        }
        // a CTA beyond the launch's last work item leaves at once -- unless the launch has none at all: then nobody else
        // would keep this grid from completing before the grid it depends on
        if (count_all && acc > (int)gridDim.x && lane == 0 && atomicCAS(p.status, OB_DEV_OK, OB_DEV_BAD_INDEX) == OB_DEV_OK) {
            p.status[1] = 150;
            p.status[2] = acc;
            p.status[3] = (int)gridDim.x;
        }
        if (GROUPS) fence_proxy_async_smem();
        if (lane == 0) ctrl->wait_before_exit = (tile < 0 && acc == 0) ? 1 : 0;
        int total = 0;
        if (tile >= 0) {
            const int t0w = tile * kMmaTile;
            for (int base = 0; base <= p.L; base += 32) {
                const int i = base + lane;
                int lora = -1, lo = 0, hi = 0;
                if (i <= p.L) {
                    lora = p.meta.seg_ids[i];
                    const int cnt = p.meta.seg_n[i], sst = p.meta.seg_start[i];
                    lo = max(sst, t0w);
                    hi = min(min(sst + cnt, t0w + kMmaTile), n_all);
                    if (cnt <= 0 || sst < 0) lora = -1;
                }
                const bool ok = lora >= 0 && lora < p.L && lo < hi;
                const uint32_t mask = __ballot_sync(0xffffffffu, ok);
                if (ok) {
                    const int idx = total + __popc(mask & ((1u << lane) - 1u));
                    if (idx < kMmaMaxList) {
                        ctrl->lora[idx] = lora;
                        for (int pos = lo; pos < hi; ++pos) ctrl->gidx[pos - t0w] = (short)idx;
                    }
                }
                total += __popc(mask);
            }
        }
        if (lane == 0) {
            ctrl->n_list = min(total, kMmaMaxList);
            ctrl->wi_tile = tile;
            ctrl->wi_g0 = first;
        }
    }
    __syncthreads();
    const int t0 = ctrl->wi_tile * kMmaTile;
    const int g_lo = GROUPS ? ctrl->wi_g0 : 0;                // list entries [g_lo, g_lo + n_list) are this CTA's tenants
    const int n_list = ctrl->wi_tile < 0 ? 0 : GROUPS ? min(p.tg_cap, ctrl->n_list - g_lo) : ctrl->n_list;
    if (n_list <= 0 || n_ksteps == 0) {                       // the launch has fewer work items than CTAs (or no tenant at all)
        // this grid must not be complete before the grid it depends on is: the CTAs with a work item see to that
        if (!GROUPS || n_ksteps == 0 || ctrl->wait_before_exit) griddep_wait();
        return;
    }
    const int n_pass = (n_list + group - 1) / group;
    const bool csum = p.cluster != 0 && n_pass == 1 && p.split1 > 1;      // the same in every CTA of the cluster (same tile)
    const int first_group = min(n_list, group);
    uint32_t tmem_cols = 32;
    while (tmem_cols < (uint32_t)(first_group * p.R)) tmem_cols *= 2;
    const int stage_bytes = kMmaXBytes + first_group * a_bytes;           // slot size of the widest pass
    int stages = p.ring_bytes / stage_bytes;
    stages = stages > kMmaMaxStages ? kMmaMaxStages : stages;
    if (warp == 1) {
        tmem_alloc(&ctrl->tmem_base, tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctrl->tmem_base;

    if (warp == 0) {
        // =========================================================== TMA producer
        if (lane == 0) {
            const CUtensorMap* tma = s == 0 ? &tm_a0 : s == 1 ? &tm_a1 : s == 2 ? &tm_a2 : &tm_a3;
            griddep_wait();                                   // the sorted copy of x comes from the preceding kernel
            int it = 0;
            for (int pass = 0; pass < n_pass && !ctrl->abort_flag; ++pass) {
                const int g0 = pass * group, ng = min(group, n_list - g0);
                for (int ks = 0; ks < n_ksteps; ++ks, ++it) {
                    const int st = it % stages;
                    if (it >= stages && !mbar_wait(&ctrl->empty[st], (uint32_t)((it / stages - 1) & 1), limit_ns)) {
                        k1m_timeout(p, ctrl, 1, it);
                        break;
                    }
                    uint8_t* slot = ring + (size_t)st * stage_bytes;
                    mbar_arrive_expect_tx(&ctrl->full[st], (uint32_t)(kMmaXBytes + ng * a_bytes));
                    tma_load_2d(slot, &tm_xs, &ctrl->full[st], k0 + ks * kMmaKStep, t0);
                    for (int g = 0; g < ng; ++g)
                        tma_load_2d(slot + kMmaXBytes + (size_t)g * a_bytes, tma, &ctrl->full[st], k0 + ks * kMmaKStep,
                                    ctrl->lora[g_lo + g0 + g] * p.R);
                }
            }
        }
    } else if (warp == 1) {
        // =========================================================== MMA issuer
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(1, 1, kMmaTile, (uint32_t)p.R);
            int it = 0;
            bool ok = true;
            for (int pass = 0; pass < n_pass && ok; ++pass) {
                const int g0 = pass * group, ng = min(group, n_list - g0);
                if (pass > 0) {                               // the epilogue has read the previous pass's accumulators
                    if (!mbar_wait(&ctrl->acc_empty, (uint32_t)((pass - 1) & 1), limit_ns)) { k1m_timeout(p, ctrl, 2, pass); break; }
                    tc_fence_after();
                }
                for (int ks = 0; ks < n_ksteps; ++ks, ++it) {
                    const int st = it % stages;
                    if (ctrl->abort_flag || !mbar_wait(&ctrl->full[st], (uint32_t)((it / stages) & 1), limit_ns)) {
                        if (!ctrl->abort_flag) k1m_timeout(p, ctrl, 3, it);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t xa = smem_u32(ring + (size_t)st * stage_bytes);
                    const uint64_t dx = umma_smem_desc(xa, 1024, 2);
                    // The tenants' A tiles lie one after the other in the slot and their accumulators side by side in tensor
                    // memory, so up to 256 / R of them are ONE B operand: an MMA of N = (tenants in the batch) x R columns
                    // instead of one MMA per tenant (every tcgen05.mma costs its issuer some 60 cycles).
                    const int batch = 256 / p.R > 0 ? 256 / p.R : 1;
                    for (int g = 0; g < ng; g += batch) {
                        const int nb = min(batch, ng - g);
                        const uint32_t idesc_b = nb == 1 ? idesc : umma_idesc(1, 1, kMmaTile, (uint32_t)(nb * p.R));
                        const uint64_t da = umma_smem_desc(xa + kMmaXBytes + (uint32_t)(g * a_bytes), 1024, 2);
#pragma unroll
                        for (int kk = 0; kk < kMmaKStep / 16; ++kk)
                            umma_f16(tmem_base + (uint32_t)(g * p.R), dx + (uint64_t)(kk * 2), da + (uint64_t)(kk * 2), idesc_b,
                                     (ks > 0 || kk > 0) ? 1u : 0u);
                    }
                    umma_commit(&ctrl->empty[st]);
                }
                if (ok) umma_commit(&ctrl->acc_full);
            }
        }
    } else {
        // =========================================================== epilogue: accumulator rows -> hp partials
        const int q = warp & 3;                               // the 32 tensor-memory lanes this warp may read
        const int row = q * 32 + lane, pos = t0 + row;
        const int mine = ctrl->gidx[row];
        float* dst = p.hp + (((size_t)j * p.S + s) * p.max_m + (size_t)pos) * p.R;
        __nv_bfloat16* hdst = p.hb + ((size_t)s * p.max_m + (size_t)pos) * p.R;
        const bool direct = p.split1 == 1;                     // no partials: the accumulator row is the finished h
        const bool cat = p.hcat != nullptr;                    // per-tenant blocks, pre-divided by the output scale
        __nv_bfloat16* cdst = cat ? p.hcat + ((size_t)s * p.max_m + (size_t)pos) * ((size_t)p.lc * p.R) : nullptr;
        // (the per-token scales come from the quantizing kernel this launch is a programmatic dependent of: they may be read
        // only after griddepcontrol.wait, which every thread that reads them executes itself)
        griddep_wait();
        const float inv = (cat && pos < p.M) ? 1.0f / ((p.sx ? __ldcg(p.sx + pos) : 1.0f) * __ldg(p.s_w)) : 0.0f;   // NVFP4 base: one scale for every token
        for (int pass = 0; pass < n_pass; ++pass) {
            const int g0 = pass * group, ng = min(group, n_list - g0);
            int go = 1;
            if (lane == 0) {
                go = ctrl->abort_flag ? 0 : 1;
                if (go && !mbar_wait(&ctrl->acc_full, (uint32_t)(pass & 1), limit_ns)) {
                    k1m_timeout(p, ctrl, 4, pass);
                    go = 0;
                }
            }
            go = __shfl_sync(0xffffffffu, go, 0);
            if (!go) break;
            tc_fence_after();
            for (int g = 0; g < ng; ++g) {
                const bool own = mine == g_lo + g0 + g && pos < p.M;
                if (cat && direct) {                          // every row of the block: the tenant's rows scaled, zeros elsewhere
                    for (int c0 = 0; c0 < p.R; c0 += 16) {
                        uint32_t r[16];
                        tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(g * p.R + c0), r);
                        tmem_ld_wait();
                        uint32_t o[8];
#pragma unroll
                        for (int v = 0; v < 8; ++v) {
                            __nv_bfloat162 b = __floats2bfloat162_rn(own ? __uint_as_float(r[2 * v]) * inv : 0.0f,
                                                                     own ? __uint_as_float(r[2 * v + 1]) * inv : 0.0f);
                            o[v] = *reinterpret_cast<uint32_t*>(&b);
                        }
                        if (pos < p.max_m) {
                            uint4* d4 = reinterpret_cast<uint4*>(cdst + (size_t)(g_lo + g0 + g) * p.R + c0);
                            d4[0] = make_uint4(o[0], o[1], o[2], o[3]);
                            d4[1] = make_uint4(o[4], o[5], o[6], o[7]);
                        }
                    }
                    continue;
                }
                if (!__any_sync(0xffffffffu, own)) continue;  // none of this warp's positions belongs to the tenant
                for (int c0 = 0; c0 < p.R; c0 += 16) {
                    uint32_t r[16];
                    tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(g * p.R + c0), r);
                    tmem_ld_wait();
                    if (own && direct) {                  // (not cat)
                        uint32_t o[8];
#pragma unroll
                        for (int v = 0; v < 8; ++v) {
                            __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(r[2 * v]), __uint_as_float(r[2 * v + 1]));
                            o[v] = *reinterpret_cast<uint32_t*>(&b);
                        }
                        reinterpret_cast<uint4*>(hdst + c0)[0] = make_uint4(o[0], o[1], o[2], o[3]);
                        reinterpret_cast<uint4*>(hdst + c0)[1] = make_uint4(o[4], o[5], o[6], o[7]);
                    } else if (own && csum) {             // the row stays in this CTA's (idle) ring for the cluster's sum
                        float4* sr = reinterpret_cast<float4*>(ring) + ((size_t)row * p.R + c0) / 4;
#pragma unroll
                        for (int v = 0; v < 4; ++v)
                            sr[v] = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                                __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
                    } else if (own) {
#pragma unroll
                        for (int v = 0; v < 4; ++v)
                            reinterpret_cast<float4*>(dst + c0)[v] =
                                make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                            __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctrl->acc_empty);
        }
        if (!direct && !csum) {
            // The K splits of a (tile, slice) count their arrivals; the last one adds the partials in split order and writes
            // the finished h once, so that K2's CTAs -- one per output tile -- need not each add them again.
            const int te = tid - 64;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (te == 0) {
                int old;
                asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(old) : "l"(p.counters + wi * p.S + s) : "memory");
                ctrl->last_flag = (old == p.split1 - 1) ? 1 : 0;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (ctrl->last_flag && !ctrl->abort_flag && cat && pos < p.max_m) {
                // zeros for the group's other entries first; the position's own entry is written below
                for (int li = g_lo; li < g_lo + n_list; ++li) {
                    if (li == mine && pos < p.M) continue;
                    uint4* d4 = reinterpret_cast<uint4*>(cdst + (size_t)li * p.R);
                    for (int c = 0; c < p.R / 8; ++c) d4[c] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            if (ctrl->last_flag && !ctrl->abort_flag) {
                if (mine >= g_lo && mine < g_lo + n_list && pos < p.M) {
                    __nv_bfloat16* odst = cat ? cdst + (size_t)mine * p.R : hdst;
                    const float osc = cat ? inv : 1.0f;
                    const size_t jstride = (size_t)p.S * p.max_m * p.R;
                    const float* src = p.hp + ((size_t)s * p.max_m + (size_t)pos) * p.R;
                    // 32 columns at a time, four splits' loads of all of them in flight together: a plain loop would pay
                    // one L2 round trip per 8 columns and split
                    for (int cb = 0; cb < p.R; cb += 32) {
                        float4 acc[8];
#pragma unroll
                        for (int q4 = 0; q4 < 8; ++q4) acc[q4] = make_float4(0.f, 0.f, 0.f, 0.f);
                        for (int j1 = 0; j1 < p.split1; j1 += 4) {
                            float4 v[4][8];
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
#pragma unroll
                                for (int q4 = 0; q4 < 8; ++q4) {
                                    v[u][q4] = (j1 + u < p.split1 && cb + q4 * 4 < p.R)
                                                   ? __ldcg(reinterpret_cast<const float4*>(src + (size_t)(j1 + u) * jstride + cb) + q4)
                                                   : make_float4(0.f, 0.f, 0.f, 0.f);
                                }
                            }
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
#pragma unroll
                                for (int q4 = 0; q4 < 8; ++q4) {
                                    acc[q4].x += v[u][q4].x; acc[q4].y += v[u][q4].y; acc[q4].z += v[u][q4].z; acc[q4].w += v[u][q4].w;
                                }
                            }
                        }
#pragma unroll
                        for (int q8 = 0; q8 < 4; ++q8) {
                            if (cb + q8 * 8 < p.R) {
                                const float4 a0 = acc[2 * q8], a1 = acc[2 * q8 + 1];
                                __nv_bfloat162 b0 = __floats2bfloat162_rn(a0.x * osc, a0.y * osc), b1 = __floats2bfloat162_rn(a0.z * osc, a0.w * osc);
                                __nv_bfloat162 b2 = __floats2bfloat162_rn(a1.x * osc, a1.y * osc), b3 = __floats2bfloat162_rn(a1.z * osc, a1.w * osc);
                                *reinterpret_cast<uint4*>(odst + cb + q8 * 8) =
                                    make_uint4(*reinterpret_cast<uint32_t*>(&b0), *reinterpret_cast<uint32_t*>(&b1),
                                               *reinterpret_cast<uint32_t*>(&b2), *reinterpret_cast<uint32_t*>(&b3));
                            }
                        }
                    }
                }
                if (te == 0) p.counters[wi * p.S + s] = 0;
            }
        }
    }
    // ---- teardown: nobody leaves while tensor memory is in use or copies may still land in this CTA's shared memory
    if (ctrl->abort_flag) __nanosleep(200000);
    tc_fence_before();
    __syncthreads();
    if (p.cluster != 0) {
        // ---- the cluster's sum (see the header).  Both barriers are unconditional: a CTA whose wait ran out still joins
        // them (its rows are then garbage, but the status words say so), and no CTA leaves while a partner reads its ring.
        __syncwarp();
        cluster_sync_all();
        if (csum && warp >= 2 && !ctrl->abort_flag) {
            const int te = tid - 64;
            const int rank = (int)blockIdx.z;                 // cluster = the grid's z extent: rank = split index
            const int rows_per = kMmaTile / p.split1, tpr = p.split1;          // rows this CTA finishes; threads per row
            const int row = rank * rows_per + te / tpr, sub = te % tpr;
            const int cols = p.R / tpr, c_lo = sub * cols;                     // a multiple of 4 columns per thread
            const int pos = t0 + row, mine = ctrl->gidx[row];
            const bool cat = p.hcat != nullptr;
            const bool valid = mine >= g_lo && mine < g_lo + n_list && pos < p.M;
            if (cat && pos < p.max_m) {                       // zeros for the group's other entries, shared among the row's threads
                __nv_bfloat16* cdst = p.hcat + ((size_t)s * p.max_m + (size_t)pos) * ((size_t)p.lc * p.R);
                for (int li = g_lo + sub; li < g_lo + n_list; li += tpr) {
                    if (valid && li == mine) continue;
                    uint4* d4 = reinterpret_cast<uint4*>(cdst + (size_t)li * p.R);
                    for (int c = 0; c < p.R / 8; ++c) d4[c] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            if (valid) {
                const float osc = cat ? 1.0f / ((p.sx ? __ldcg(p.sx + pos) : 1.0f) * __ldg(p.s_w)) : 1.0f;
                __nv_bfloat16* odst = cat ? p.hcat + ((size_t)s * p.max_m + (size_t)pos) * ((size_t)p.lc * p.R) + (size_t)mine * p.R
                                          : p.hb + ((size_t)s * p.max_m + (size_t)pos) * p.R;
                const uint32_t own_addr = smem_u32(ring) + (uint32_t)(((size_t)row * p.R + c_lo) * 4);
                for (int c = 0; c < cols; c += 4) {
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int q = 0; q < p.split1; ++q) {      // split order: the same sum as the workspace path
                        const float4 v = ld_cluster_f4(cluster_peer_addr(own_addr + (uint32_t)(c * 4), (uint32_t)q));
                        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                    }
                    __nv_bfloat162 b0 = __floats2bfloat162_rn(acc.x * osc, acc.y * osc), b1 = __floats2bfloat162_rn(acc.z * osc, acc.w * osc);
                    *reinterpret_cast<uint2*>(odst + c_lo + c) = make_uint2(*reinterpret_cast<uint32_t*>(&b0), *reinterpret_cast<uint32_t*>(&b1));
                }
            }
        }
        __syncwarp();
        cluster_sync_all();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, tmem_cols);
    }
}

size_t k1_mma_smem_bytes(int ring_bytes) { return 1024 + (size_t)ring_bytes + sizeof(K1mCtrl) + 64; }

cudaError_t launch_k1_mma(const K1mParams& p, const CUtensorMap& tm_xs, const CUtensorMap* tm_a, dim3 grid, cudaStream_t stream) {
    static int configured_for[64] = {0};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const size_t smem = k1_mma_smem_bytes(p.ring_bytes);
    if (dev >= 0 && dev < 64 && !configured_for[dev]) {
        e = cudaFuncSetAttribute(k1_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
        if (e != cudaSuccess) return e;
        e = cudaFuncSetAttribute(k1_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
        if (e != cudaSuccess) return e;
        configured_for[dev] = 1;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kMmaThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // always a programmatic dependent of K1
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;                  // the K splits of a (tile, slice) as one cluster
    attr[1].val.clusterDim.x = 1;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = grid.z;
    cfg.attrs = attr;
    cfg.numAttrs = p.cluster ? 2 : 1;
    if (p.tg_cap < kMmaMaxList) return cudaLaunchKernelEx(&cfg, k1_mma_kernel<true>, p, tm_xs, tm_a[0], tm_a[1], tm_a[2], tm_a[3]);
    return cudaLaunchKernelEx(&cfg, k1_mma_kernel<false>, p, tm_xs, tm_a[0], tm_a[1], tm_a[2], tm_a[3]);
}

}  // namespace ob
