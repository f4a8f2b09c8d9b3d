// K2 for prefill batches (more than 128 tokens), bf16 adapters: one CTA per 256 output features x 256 tokens (FP8 base) or
// per 128 output features x 256 tokens (NVFP4 base).
//
// Why another GEMM kernel: with 128 x 128 tiles a CTA moves 32 KB of operands into shared memory per 4.2 MFLOP
// (131 FLOP per byte), and at prefill sizes the L2-to-SM traffic, not the tensor pipe, is what saturates (measured
// ~7.8 TB/s, i.e. ~1.0 PFLOP/s).  A 256 x 256 tile moves 64 KB per 16.8 MFLOP -- twice the flops per byte.
// Its two 128-row halves are two tcgen05.mma accumulators of 256 columns each: all 512 columns of tensor memory.  That
// leaves no room for the separate LoRA accumulator of k2_gemm.cu, so the expand is folded into the base accumulator:
//     y[t, n] = s_x[t] s_w * ( sum_k Wq[n,k] xq[t,k]  +  sum_r B_l[n,r] * h[t,r] / (s_x[t] s_w) )
// The tensor-core shrink (k1_mma.cu) leaves h already divided by the token's output scale, as one block per (position,
// tenant of the position's 128-block) with zeros in the blocks of the other tenants, so an expand step is a plain pair of
// TMA tiles -- B_l [256 x 64] and the tenant's h block [128 tokens x 64] -- and four more MMAs per half, like one more K
// block of the GEMM.  (The division moves one bf16 rounding of h: the result differs from k2_gemm.cu's by about 2^-9 of
// the LoRA term, far inside the 2e-2 * |y|inf bound the outputs are held to.)
// Computes what lowbit_lora/kernels/fp8_lora_vllm.py:123-284 (`_gemm_vllm`) computes for a prefill batch.
//
// The kernel is persistent: one CTA per SM walks the launch's tiles (token tiles fastest, so a wave shares a few W tiles
// in L2).  Warps: 0 = TMA producer (one thread), 1 = MMA issuer (one thread; owns the tensor-memory allocation), 2 = tile
// scout (row map, output scales and the tile's expand steps from the segment index, double-buffered, one tile ahead),
// 3..6 = epilogue (tcgen05.ld, scale, 32 tokens at a time staged in shared memory, whole token rows scattered back
// through the sort).  The accumulators fill tensor memory, so a tile's MMAs wait until the previous tile has been read
// out; but the producer does not: while the epilogue drains, it fills the ring with the next tile's first k-blocks, and
// the MMAs catch up at tensor-core speed (the main loop is bound by the L2-to-SM stream, not by the tensor pipe).
// Ring slots of 64 KB: a W k-block [256 x 128 B] with its x_q tile [256 tokens x 128 B], or an expand step's B and h
// tiles.  A tile's W k-blocks come first, its expand steps last.  Every wait is bounded.
//
// NVFP4 base (template FP4): a 128-byte k-block holds 256 e2m1 codes, so the same slot carries twice the K and the flops
// per byte double; but the block scales of kind::mxf4nvf4 live in tensor memory beside the accumulator, so the tile is one
// 128-row half (256 accumulator columns) and each ring slot owns 48 more columns: 16 for the W scales of its four K = 64
// MMAs, 32 for the two 128-token blocks of activation scales (tcgen05.cp from the slot, as in k2_gemm.cu).  Slot: W
// [128 x 128 B], x_q [256 x 128 B], W scales 2 KB, activation scales 4 KB = 54 KB.  Computes what
// lowbit_lora/kernels/nvfp4_lora_vllm.py:219-357 computes for a prefill batch.
#include "ob_common.cuh"
#include "ob_ptx.cuh"

namespace ob {

constexpr int kPfThreads = 224;              // warps: 0 TMA producer, 1 MMA issuer, 2 tile scout, 3..6 epilogue
constexpr int kPfTokens = 256;               // tokens per tile (the MMAs' N)
constexpr int kPfHalfBytes = 128 * 128;      // one 128-row half of a W or B tile
constexpr int kPfSfCols = 48;                // NVFP4: tensor-memory columns of one slot's scale factors (16 W + 32 activation)
constexpr int kPfChunk = 32;                 // tokens of the output tile staged in shared memory at a time
constexpr int kPfMaxStages = 3;
constexpr int kPfMaxSteps = 512;             // expand steps of one tile (two 128-token blocks x tenants x rank chunks)
// output features per tile (FP8: two MMA halves of 128; NVFP4: one) and the ring slot that feeds them
__host__ __device__ constexpr int pf_halves(bool fp4) { return fp4 ? 1 : 2; }
__host__ __device__ constexpr int pf_rows(bool fp4) { return 128 * pf_halves(fp4); }
__host__ __device__ constexpr int pf_slot_bytes(bool fp4) {
    return pf_halves(fp4) * kPfHalfBytes + kPfTokens * 128 + (fp4 ? 3 * kSfSlotBytes : 0);
}
__host__ __device__ constexpr int pf_stage_bytes(bool fp4) { return kPfChunk * pf_rows(fp4) * 2; }

struct PfStep {
    uint16_t lora, entry, block, chunk;      // tenant, its entry in the 128-block's list, 128-block of the tile, rank chunk
};

// What the scout prepares per tile, double-buffered so that it runs one tile ahead of the other roles.
struct PfMeta {
    int n_steps;
    int rowmap[kPfTokens];
    float scale[kPfTokens];
    PfStep steps[kPfMaxSteps];
};

struct PfCtrl {
    uint64_t full[kPfMaxStages];
    uint64_t empty[kPfMaxStages];
    uint64_t meta_full[2];
    uint64_t meta_empty[2];
    uint64_t acc_full;
    uint64_t acc_empty;
    uint32_t tmem_base;
    volatile int abort_flag;
    int go_flag;
    PfMeta meta[2];
};

__device__ __forceinline__ void pf_timeout(const K2pParams& p, PfCtrl* c, int where, int it) {
    c->abort_flag = 1;
    if (atomicCAS(p.status, OB_DEV_OK, OB_DEV_WAIT_TIMEOUT) == OB_DEV_OK) {
        p.status[1] = 200 + where;
        p.status[2] = blockIdx.x;
        p.status[3] = blockIdx.y;
        p.status[4] = blockIdx.z;
        p.status[5] = it;
    }
}

// Tile t of the launch: token tiles vary fastest, so the CTAs of one wave share a few W tiles (HBM once, L2 after).
struct PfTile {
    int t0, s, n_s, slice_off, n0_local, n_idx, m_idx;
};
template <bool FP4>
__device__ __forceinline__ PfTile pf_tile(const K2pParams& p, int t, int m_tiles) {
    PfTile r;
    r.m_idx = t % m_tiles;
    r.n_idx = t / m_tiles;
    r.t0 = r.m_idx * kPfTokens;
    int s = 0, n_tile = r.n_idx, off = 0;
    while (s < p.S - 1 && n_tile >= p.widths[s] / pf_rows(FP4)) {
        n_tile -= p.widths[s] / pf_rows(FP4);
        off += p.widths[s];
        ++s;
    }
    r.s = s;
    r.n_s = p.widths[s];
    r.slice_off = off;
    r.n0_local = n_tile * pf_rows(FP4);
    return r;
}

template <bool FP4>
__global__ void __launch_bounds__(kPfThreads, 1)
k2_prefill_kernel(const K2pParams p, const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                  const __grid_constant__ CUtensorMap tm_h, const __grid_constant__ CUtensorMap tm_b0,
                  const __grid_constant__ CUtensorMap tm_b1, const __grid_constant__ CUtensorMap tm_b2,
                  const __grid_constant__ CUtensorMap tm_b3) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int kPfRows = pf_rows(FP4), kHalves = pf_halves(FP4), kPfSlotBytes = pf_slot_bytes(FP4);
    constexpr int kXOff = kHalves * kPfHalfBytes;             // the x_q (or h) tile follows the W (or B) tile in a slot
    uint8_t* ring = smem;
    uint8_t* stage = smem + (size_t)p.stages * kPfSlotBytes;  // [kPfChunk tokens][kPfRows] bf16 of the output tile
    PfCtrl* ctrl = reinterpret_cast<PfCtrl*>(stage + pf_stage_bytes(FP4));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    griddep_launch_dependents();
    const uint64_t limit_ns = (uint64_t)p.wait_ms * 1000000ull;
    const int m_tiles = (p.M + kPfTokens - 1) / kPfTokens;
    const int n_tiles = m_tiles * (p.N / kPfRows);
    const int n_chunks = p.R / 64;

    if (tid == 0) {
        for (int i = 0; i < kPfMaxStages; ++i) {
            mbar_init(&ctrl->full[i], 1);
            mbar_init(&ctrl->empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&ctrl->meta_full[i], 1);
            mbar_init(&ctrl->meta_empty[i], 4);
        }
        mbar_init(&ctrl->acc_full, 1);
        mbar_init(&ctrl->acc_empty, 4);
        ctrl->abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(&ctrl->tmem_base, 512);
        tmem_relinquish();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tm_w);
        tma_prefetch_desc(&tm_x);
        tma_prefetch_desc(&tm_h);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctrl->tmem_base;

    if (warp == 0) {
        // =========================================================== TMA producer: runs ahead through the tiles, ring-deep
        if (lane == 0) {
            griddep_wait();                                   // x_q and the h blocks come from the preceding kernels
            int it = 0;
            bool ok = true;
            for (int t = blockIdx.x, i = 0; t < n_tiles && ok; t += gridDim.x, ++i) {
                const PfTile tl = pf_tile<FP4>(p, t, m_tiles);
                const CUtensorMap* tmb = (tl.s == 0) ? &tm_b0 : (tl.s == 1) ? &tm_b1 : (tl.s == 2) ? &tm_b2 : &tm_b3;
                for (int kb = 0; kb < p.kblocks && ok; ++kb, ++it) {
                    const int st = it % p.stages;
                    if (ctrl->abort_flag ||
                        (it >= p.stages && !mbar_wait(&ctrl->empty[st], (uint32_t)((it / p.stages - 1) & 1), limit_ns))) {
                        if (!ctrl->abort_flag) pf_timeout(p, ctrl, 1, it);
                        ok = false;
                        break;
                    }
                    uint8_t* slot = ring + (size_t)st * kPfSlotBytes;
                    mbar_arrive_expect_tx(&ctrl->full[st], (uint32_t)(kXOff + kPfTokens * 128 + (FP4 ? 3 * kSfSlotBytes : 0)));
                    tma_load_2d(slot, &tm_w, &ctrl->full[st], kb * 128, tl.slice_off + tl.n0_local);
                    tma_load_2d(slot + kXOff, &tm_x, &ctrl->full[st], kb * 128, tl.t0);
                    if (FP4) {
                        uint8_t* sf = slot + kXOff + kPfTokens * 128;
                        bulk_load(sf, p.wsf + ((size_t)tl.n_idx * p.kblocks + kb) * kSfSlotBytes, kSfSlotBytes, &ctrl->full[st]);
                        bulk_load(sf + kSfSlotBytes, p.xsf + ((size_t)tl.m_idx * p.kblocks + kb) * 2 * kSfSlotBytes,
                                  2 * kSfSlotBytes, &ctrl->full[st]);
                    }
                }
                if (!ok) break;
                const PfMeta& mt = ctrl->meta[i & 1];
                if (!mbar_wait(&ctrl->meta_full[i & 1], (uint32_t)((i >> 1) & 1), limit_ns)) {
                    pf_timeout(p, ctrl, 2, it);
                    break;
                }
                const int n_steps = mt.n_steps;
                for (int li = 0; li < n_steps && ok; ++li, ++it) {
                    const int st = it % p.stages;
                    if (ctrl->abort_flag ||
                        (it >= p.stages && !mbar_wait(&ctrl->empty[st], (uint32_t)((it / p.stages - 1) & 1), limit_ns))) {
                        if (!ctrl->abort_flag) pf_timeout(p, ctrl, 3, it);
                        ok = false;
                        break;
                    }
                    const PfStep e = mt.steps[li];
                    uint8_t* slot = ring + (size_t)st * kPfSlotBytes;
                    mbar_arrive_expect_tx(&ctrl->full[st], (uint32_t)(kXOff + 128 * 128));
                    tma_load_2d(slot, tmb, &ctrl->full[st], (int)e.chunk * 64, (int)e.lora * tl.n_s + tl.n0_local);
                    tma_load_2d(slot + kXOff, &tm_h, &ctrl->full[st], (int)e.entry * p.R + (int)e.chunk * 64,
                                tl.s * p.max_m + tl.t0 + (int)e.block * 128);
                }
            }
        }
    } else if (warp == 1) {
        // =========================================================== MMA issuer
        if (lane == 0) {
            const uint32_t idesc8 = umma_idesc(0, 0, 128, kPfTokens);
            const uint32_t idesc4 = umma_idesc_nvfp4(128, kPfTokens);
            const uint32_t idesc16 = umma_idesc(1, 1, 128, 128);
            int it = 0;
            bool ok = true;
            for (int t = blockIdx.x, i = 0; t < n_tiles && ok; t += gridDim.x, ++i) {
                if (i > 0) {                                  // the epilogue has read the previous tile out of tensor memory
                    if (ctrl->abort_flag || !mbar_wait(&ctrl->acc_empty, (uint32_t)((i - 1) & 1), limit_ns)) {
                        if (!ctrl->abort_flag) pf_timeout(p, ctrl, 8, i);
                        break;
                    }
                    tc_fence_after();
                }
                for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
                    const int st = it % p.stages;
                    if (ctrl->abort_flag || !mbar_wait(&ctrl->full[st], (uint32_t)((it / p.stages) & 1), limit_ns)) {
                        if (!ctrl->abort_flag) pf_timeout(p, ctrl, 4, it);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t wa = smem_u32(ring + (size_t)st * kPfSlotBytes);
                    const uint64_t dx = umma_smem_desc(wa + kXOff, 1024, 2);
                    if (FP4) {
                        // the slot's scale factors: shared memory -> the slot's own tensor-memory columns, then the four K = 64 MMAs
                        const uint64_t dw = umma_smem_desc(wa, 1024, 2);
                        const uint32_t sfs = wa + (uint32_t)(kXOff + kPfTokens * 128);
                        const uint32_t sft = tmem_base + (uint32_t)kPfTokens + (uint32_t)(st * kPfSfCols);
                        // (all twelve copies first: a copy issued between two MMAs would hold the second one back)
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint32_t ta = sft + (uint32_t)k * 4u, tb = sft + 16u + (uint32_t)k * 8u;
                            tmem_cp_sf(ta, sf_smem_desc(sfs + (uint32_t)k * 512u));
                            tmem_cp_sf(tb, sf_smem_desc(sfs + kSfSlotBytes + (uint32_t)k * 512u));
                            tmem_cp_sf(tb + 4u, sf_smem_desc(sfs + 2 * kSfSlotBytes + (uint32_t)k * 512u));
                        }
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint32_t ta = sft + (uint32_t)k * 4u, tb = sft + 16u + (uint32_t)k * 8u;
                            umma_nvfp4(tmem_base, dw + (uint64_t)(k * 2), dx + (uint64_t)(k * 2), idesc4, ta, tb, (kb > 0 || k > 0) ? 1u : 0u);
                        }
                    } else {
#pragma unroll
                        for (int half = 0; half < kHalves; ++half) {
                            const uint64_t dw = umma_smem_desc(wa + (uint32_t)(half * kPfHalfBytes), 1024, 2);
#pragma unroll
                            for (int k = 0; k < 4; ++k)
                                umma_f8f6f4(tmem_base + (uint32_t)(half * kPfTokens), dw + (uint64_t)(k * 2), dx + (uint64_t)(k * 2), idesc8,
                                            (kb > 0 || k > 0) ? 1u : 0u);
                        }
                    }
                    umma_commit(&ctrl->empty[st]);
                }
                if (!ok) break;
                const PfMeta& mt = ctrl->meta[i & 1];
                if (!mbar_wait(&ctrl->meta_full[i & 1], (uint32_t)((i >> 1) & 1), limit_ns)) {
                    pf_timeout(p, ctrl, 5, it);
                    break;
                }
                const int n_steps = mt.n_steps;
                for (int li = 0; li < n_steps; ++li, ++it) {
                    const int st = it % p.stages;
                    if (ctrl->abort_flag || !mbar_wait(&ctrl->full[st], (uint32_t)((it / p.stages) & 1), limit_ns)) {
                        if (!ctrl->abort_flag) pf_timeout(p, ctrl, 6, it);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const PfStep e = mt.steps[li];
                    const uint32_t ba = smem_u32(ring + (size_t)st * kPfSlotBytes);
                    const uint64_t dh = umma_smem_desc(ba + kXOff, 1024, 2);
#pragma unroll
                    for (int half = 0; half < kHalves; ++half) {
                        const uint64_t db = umma_smem_desc(ba + (uint32_t)(half * kPfHalfBytes), 1024, 2);
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            umma_f16(tmem_base + (uint32_t)(half * kPfTokens + (int)e.block * 128), db + (uint64_t)(k * 2),
                                     dh + (uint64_t)(k * 2), idesc16, 1u);
                    }
                    umma_commit(&ctrl->empty[st]);
                }
                if (ok) umma_commit(&ctrl->acc_full);
            }
        }
    } else if (warp == 2) {
        // =========================================================== tile scout: row map, output scales and expand steps,
        // one tile ahead of the roles that consume them
        int n_all, n_ad;
        segment_totals(p.meta, p.L, lane, n_all, n_ad);
        n_all = min(n_all, p.M);
        griddep_wait();                                       // K1's s_x from here on
        const float s_w = __ldg(p.s_w);
        for (int t = blockIdx.x, i = 0; t < n_tiles; t += gridDim.x, ++i) {
            PfMeta& mt = ctrl->meta[i & 1];
            int go = 1;
            if (lane == 0 && i >= 2) {                        // the epilogue of the tile before last has let go of this buffer
                go = ctrl->abort_flag ? 0 : 1;
                if (go && !mbar_wait(&ctrl->meta_empty[i & 1], (uint32_t)(((i >> 1) - 1) & 1), limit_ns)) {
                    pf_timeout(p, ctrl, 9, i);
                    go = 0;
                }
            }
            go = __shfl_sync(0xffffffffu, go, 0);
            if (!go) break;
            const PfTile tl = pf_tile<FP4>(p, t, m_tiles);
            for (int c = lane; c < kPfTokens; c += 32) {
                const int pos = tl.t0 + c;
                mt.rowmap[c] = pos < p.M ? position_row(p.meta, pos, p.M, n_all, n_ad) : -1;
                mt.scale[c] = pos < p.M ? (p.sx ? __ldcg(p.sx + pos) : 1.0f) * s_w : 0.0f;   // NVFP4: one scale for every token
            }
            // per 128-position block, the segments that reach into it, in segment order: the order in which the shrink
            // numbered the block's h entries
            int total = 0;
            if (n_ad > 0) {
                for (int blk = 0; blk < 2; ++blk) {
                    const int b0 = tl.t0 + blk * 128;
                    int entries = 0;
                    for (int base = 0; base <= p.L; base += 32) {
                        const int j = base + lane;
                        int lora = -1, lo = 0, hi = 0;
                        if (j <= p.L) {
                            lora = p.meta.seg_ids[j];
                            const int cnt = p.meta.seg_n[j], sst = p.meta.seg_start[j];
                            lo = max(sst, b0);
                            hi = min(min(sst + cnt, b0 + 128), n_all);
                            if (cnt <= 0 || sst < 0) lora = -1;
                        }
                        const bool hit = lora >= 0 && lora < p.L && lo < hi;
                        const uint32_t mask = __ballot_sync(0xffffffffu, hit);
                        if (hit) {
                            const int rank = __popc(mask & ((1u << lane) - 1u));   // hits of lower lanes in this ballot
                            const int entry = entries + rank;
                            if (entry < kMaxTileTenants)
                                for (int c = 0; c < n_chunks; ++c) {
                                    const int li = total + rank * n_chunks + c;
                                    if (li < kPfMaxSteps)
                                        mt.steps[li] = PfStep{(uint16_t)lora, (uint16_t)entry, (uint16_t)blk, (uint16_t)c};
                                }
                        }
                        entries += __popc(mask);
                        total += __popc(mask) * n_chunks;
                    }
                }
            }
            if (lane == 0) mt.n_steps = min(total, kPfMaxSteps);
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctrl->meta_full[i & 1]);
        }
    } else {
        // =========================================================== epilogue (warps 3..6): tensor memory -> y
        const int te = tid - 96;
        const int q = warp & 3;                               // the 32 tensor-memory lanes this warp may read
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        constexpr int kLanesPerTok = kPfRows / 8, kTokPerWarp = 32 / kLanesPerTok;   // copy-out: 16 bytes per lane
        for (int t = blockIdx.x, i = 0; t < n_tiles; t += gridDim.x, ++i) {
            const PfMeta& mt = ctrl->meta[i & 1];
            if (te == 0) {
                int go = ctrl->abort_flag ? 0 : 1;
                if (go && !mbar_wait(&ctrl->meta_full[i & 1], (uint32_t)((i >> 1) & 1), limit_ns)) {
                    pf_timeout(p, ctrl, 10, i);
                    go = 0;
                }
                if (go && !mbar_wait(&ctrl->acc_full, (uint32_t)(i & 1), limit_ns)) {
                    pf_timeout(p, ctrl, 7, i);
                    go = 0;
                }
                ctrl->go_flag = go;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const int go = ctrl->go_flag;
            asm volatile("bar.sync 1, 128;" ::: "memory");    // everyone has read the flag before its next writer runs
            if (!go) break;
            tc_fence_after();
            const PfTile tl = pf_tile<FP4>(p, t, m_tiles);
            const int n_tok = min(kPfTokens, p.M - tl.t0);
            __nv_bfloat16* ybase = p.y + tl.slice_off + tl.n0_local + (lane % kLanesPerTok) * 8;
            // kPfChunk tokens at a time through shared memory as [token][features] bf16, so that each token's 512 (256)
            // bytes leave in one coalesced store instead of 2-byte stores per feature
#pragma unroll 1
            for (int c0 = 0; c0 < n_tok; c0 += kPfChunk) {
#pragma unroll
                for (int half = 0; half < kHalves; ++half) {
                    uint32_t r[32];
                    tmem_ld32(tmem_base + lane_addr + (uint32_t)(half * kPfTokens + c0), r);
                    tmem_ld_wait();
                    uint8_t* col = stage + (size_t)(half * 128 + q * 32 + lane) * 2;
#pragma unroll
                    for (int c = 0; c < 32; ++c)
                        *reinterpret_cast<__nv_bfloat16*>(col + (size_t)c * (kPfRows * 2)) =
                            __float2bfloat16_rn(__uint_as_float(r[c]) * mt.scale[c0 + c]);
                }
                if (c0 + kPfChunk >= n_tok) {                 // the accumulators are in registers or beyond: the next tile's MMAs may start
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&ctrl->acc_empty);
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                for (int c = q * kTokPerWarp + lane / kLanesPerTok; c < kPfChunk && c0 + c < n_tok; c += 4 * kTokPerWarp) {
                    const int row = mt.rowmap[c0 + c];
                    if (row >= 0)
                        *reinterpret_cast<uint4*>(ybase + (int64_t)row * p.ldy) =
                            *reinterpret_cast<const uint4*>(stage + (size_t)c * (kPfRows * 2) + (lane % kLanesPerTok) * 16);
                }
                asm volatile("bar.sync 1, 128;" ::: "memory"); // the chunk has left before the next one is staged
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctrl->meta_empty[i & 1]);
        }
    }
    // ---- teardown: nobody leaves while tensor memory is in use or copies may still land in this CTA's shared memory
    if (ctrl->abort_flag) __nanosleep(200000);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

size_t k2_prefill_smem_bytes(int stages, int fp4) {
    return 1024 + (size_t)stages * (size_t)pf_slot_bytes(fp4 != 0) + (size_t)pf_stage_bytes(fp4 != 0) + sizeof(PfCtrl) + 64;
}
int k2_prefill_max_steps() { return kPfMaxSteps; }

template <bool FP4>
static cudaError_t launch_k2_prefill_impl(const K2pParams& p, const CUtensorMap& tm_w, const CUtensorMap& tm_x, const CUtensorMap& tm_h,
                                          const CUtensorMap* tm_b, dim3 grid, int pdl, cudaStream_t stream) {
    static int configured_for[64] = {0};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64 && !configured_for[dev]) {
        e = cudaFuncSetAttribute(k2_prefill_kernel<FP4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
        if (e != cudaSuccess) return e;
        configured_for[dev] = 1;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kPfThreads);
    cfg.dynamicSmemBytes = k2_prefill_smem_bytes(p.stages, FP4 ? 1 : 0);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, k2_prefill_kernel<FP4>, p, tm_w, tm_x, tm_h, tm_b[0], tm_b[1], tm_b[2], tm_b[3]);
}

cudaError_t launch_k2_prefill(const K2pParams& p, const CUtensorMap& tm_w, const CUtensorMap& tm_x, const CUtensorMap& tm_h,
                              const CUtensorMap* tm_b, dim3 grid, int fp4, int pdl, cudaStream_t stream) {
    return fp4 ? launch_k2_prefill_impl<true>(p, tm_w, tm_x, tm_h, tm_b, grid, pdl, stream)
               : launch_k2_prefill_impl<false>(p, tm_w, tm_x, tm_h, tm_b, grid, pdl, stream);
}

}  // namespace ob
