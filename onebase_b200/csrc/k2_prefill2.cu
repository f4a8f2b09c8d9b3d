// K2 for prefill batches, bf16 adapters, on CTA PAIRS: two CTAs of a cluster compute one tile of 256 tokens x 256 (NVFP4
// base) or 512 (FP8 base) output features with tcgen05.mma.cta_group::2 (kind::mxf4nvf4.block_scale or kind::f8f6f4, M =
// 256 tokens, N = 256 features, the FP8 tile as two such MMAs filling all 512 accumulator columns: unlike
// the decode kernels the tokens are the MMA's rows here, so an accumulator lane is a token and its columns are
// consecutive features -- a thread of the epilogue stores 64 contiguous bytes of a row of y per tensor-memory load).
//
// Why pairs: the single-CTA kernel of k2_prefill.cu takes 54 KB (NVFP4; FP8 64 KB) of operands into shared memory per
// 16.8 MFLOP and its tensor pipe idles most of the time -- a ring slot costs its single-thread roles a fixed ~0.8 us
// (every wait, copy issue, tcgen05.cp / mma / commit costs its issuing thread 50-250 cycles), whatever the slot holds,
// and only three such slots fit.  In a pair each CTA supplies its own 128 rows of W and only HALF of the token tile (the
// MMA reads the other half out of the partner's shared memory), so a CTA takes in 38 KB for the same 16.8 MFLOP -- five
// slots fit, and with the tokens on the accumulator's lanes the epilogue needs no staging: W [128 x
// 128 B], x_q [128 tokens x 128 B], its tokens' block scales (2 KB) and the W block scales of all 256 features (4 KB;
// every CTA needs the scales of all of B's rows in its own tensor memory).  No load is multicast.
//
// Per CTA (448 threads): warp 0 = TMA producer of the CTA's own operands -- every load a tensor load of the
// cta_group::2 form, whose bytes are counted on the slot barrier of the pair's rank-0 CTA, so one wait there covers
// both CTAs' operands (the block scales are fetched as 8 x 256-byte boxes of a [rows, 256] byte tensor for that
// reason); warp 1 = in the pair's rank-0 CTA the MMA issuer for both; warp 2 = tile
// scout (row map, output scale, expand steps; both CTAs compute the same list); warps 3..6 and 8..11 = epilogue of the CTA's own
// 128 tokens (straight from tensor memory to y; two warps per lane quarter, half of the features each);
// warps 7, 12, 13 = in rank 0 the scale copiers (tcgen05.cp of a slot's scale factors into both CTAs' tensor memory).  The issuer's commits arrive on the slot-free and accumulator-full barriers of BOTH CTAs
// (tcgen05.commit ... multicast::cluster, an arrival, not a load).  The kernel is persistent: a pair walks the launch's
// tiles; accumulators are single-buffered (256 columns + 5 x 48 scale columns), the five-slot ring runs ahead into the
// next tile while the epilogue drains.  The LoRA expand is folded into the accumulator as in k2_prefill.cu: per
// (128-token block, tenant, rank chunk) one M = 256, N = 256 MMA of kind::f16 of the tenant's h block with B_l's 256 rows;
// the block is one CTA's tokens, the other CTA's A rows are a zero tile (a TMA box outside the tensor).  Every wait is bounded; a CTA whose wait runs out records where,
// stops, and still joins the cluster barrier of the teardown, so its partner's own waits run out and both leave.
// Computes what lowbit_lora/kernels/nvfp4_lora_vllm.py:219-357 computes for a prefill batch.
#include <atomic>

#include "ob_common.cuh"
#include "ob_ptx.cuh"

namespace ob {

constexpr int kP2Threads = 448;
constexpr int kP2Tokens = 256;               // tokens per tile: 128 per CTA (the MMA's M)
constexpr int kP2WBytes = 128 * 128;         // 128 rows of W (or B_l) of a slot
constexpr int kP2XBytes = 128 * 128;         // this CTA's half of the token tile
constexpr int kP2SfCols = 48;                // NVFP4: tensor-memory columns of one slot's scale factors (16 tokens' + 32 W)
constexpr int kP2MaxSteps = 512;
// features per tile (NVFP4: one N = 256 MMA; FP8: two, all 512 accumulator columns), ring depth and slot size
__host__ __device__ constexpr int p2_halves(bool fp4) { return fp4 ? 1 : 2; }
__host__ __device__ constexpr int p2_rows(bool fp4) { return 256 * p2_halves(fp4); }
__host__ __device__ constexpr int p2_stages(bool fp4) { return fp4 ? 5 : 4; }
__host__ __device__ constexpr int p2_slot_bytes(bool fp4) {
    return p2_halves(fp4) * kP2WBytes + kP2XBytes + (fp4 ? 3 * kSfSlotBytes : 0);   // 38 KB / 48 KB
}

struct P2Step {
    uint16_t lora, entry, block, chunk;      // tenant, its entry in the 128-block's list, 128-block of the tile, rank chunk
};

struct P2Meta {
    int n_steps;
    int rowmap[kP2Tokens];
    float scale[kP2Tokens];
    P2Step steps[kP2MaxSteps];
};

struct P2Ctrl {
    uint64_t full[5];                // rank 0's: both CTAs' operands of the slot have landed (rank 1's is unused)
    uint64_t sf_ready[5];            // rank 0 only (NVFP4): the slot's scale factors are in both CTAs' tensor memory
    uint64_t empty[5];               // the pair's MMAs on the slot are done (arrives in both CTAs)
    uint64_t meta_full[2];
    uint64_t meta_empty[2];
    uint64_t acc_full;               // arrives in both CTAs
    uint64_t acc_empty;              // rank 0 only: both CTAs' epilogue warps (16 arrivals)
    uint32_t tmem_base;
    volatile int abort_flag;
    int go_flag;
    P2Meta meta[2];
};

__device__ __forceinline__ void p2_timeout(const K2pParams& p, P2Ctrl* c, int where, int it) {
    c->abort_flag = 1;
    if (atomicCAS(p.status, OB_DEV_OK, OB_DEV_WAIT_TIMEOUT) == OB_DEV_OK) {
        p.status[1] = 300 + where;
        p.status[2] = blockIdx.x;
        p.status[3] = 0;
        p.status[4] = 0;
        p.status[5] = it;
    }
}

struct P2Tile {
    int t0, s, n_s, slice_off, n0_local, n_idx, m_idx;
};
template <bool FP4>
__device__ __forceinline__ P2Tile p2_tile(const K2pParams& p, int t, int m_tiles) {
    P2Tile r;
    r.m_idx = t % m_tiles;
    r.n_idx = t / m_tiles;
    r.t0 = r.m_idx * kP2Tokens;
    int s = 0, n_tile = r.n_idx, off = 0;
    while (s < p.S - 1 && n_tile >= p.widths[s] / p2_rows(FP4)) {
        n_tile -= p.widths[s] / p2_rows(FP4);
        off += p.widths[s];
        ++s;
    }
    r.s = s;
    r.n_s = p.widths[s];
    r.slice_off = off;
    r.n0_local = n_tile * p2_rows(FP4);
    return r;
}

template <bool FP4>
__global__ void __launch_bounds__(kP2Threads, 1)
k2_prefill_pair_kernel(const K2pParams p, const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                       const __grid_constant__ CUtensorMap tm_h, const __grid_constant__ CUtensorMap tm_b0,
                       const __grid_constant__ CUtensorMap tm_b1, const __grid_constant__ CUtensorMap tm_b2,
                       const __grid_constant__ CUtensorMap tm_b3, const __grid_constant__ CUtensorMap tm_wsf,
                       const __grid_constant__ CUtensorMap tm_xsf) {
    extern __shared__ uint8_t smem_raw[];
    // (the dynamic shared memory starts at the same offset in both CTAs of a pair: the MMA applies one descriptor to both)
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int kHalves = p2_halves(FP4), kRows = p2_rows(FP4), kStages = p2_stages(FP4), kSlot = p2_slot_bytes(FP4);
    constexpr int kXOff = kHalves * kP2WBytes;                // the token tile (or h block) follows the W (or B_l) rows in a slot
    uint8_t* ring = smem;
    P2Ctrl* ctrl = reinterpret_cast<P2Ctrl*>(smem + (size_t)kStages * kSlot);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_cta_rank();                 // 0: issues the pair's MMAs
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    griddep_launch_dependents();
    const uint64_t limit_ns = (uint64_t)p.wait_ms * 1000000ull;
    const int m_tiles = (p.M + kP2Tokens - 1) / kP2Tokens;
    const int n_tiles = m_tiles * (p.N / kRows);
    const int n_chunks = p.R / 64;

    if (tid == 0) {
        for (int i = 0; i < kStages; ++i) {
            // rank 0's: one arrival whose transaction count covers both CTAs' bytes (every load is a tensor load, and the
            // partner's complete on this barrier directly); rank 1's is never used
            mbar_init(&ctrl->full[i], 1);
            mbar_init(&ctrl->sf_ready[i], 3);   // one commit per copier thread
            mbar_init(&ctrl->empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&ctrl->meta_full[i], 1);
            mbar_init(&ctrl->meta_empty[i], 8);
        }
        mbar_init(&ctrl->acc_full, 1);
        mbar_init(&ctrl->acc_empty, 16);
        ctrl->abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(&ctrl->tmem_base, 512);
        tmem_relinquish_pair();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tm_w);
        tma_prefetch_desc(&tm_x);
        tma_prefetch_desc(&tm_h);
    }
    tc_fence_before();
    __syncthreads();
    cluster_arrive();                                         // both CTAs' barriers exist before either is signalled from outside
    cluster_wait();
    tc_fence_after();
    const uint32_t tmem_base = ctrl->tmem_base;

    if (warp == 0) {
        // =========================================================== TMA producer of this CTA's operands
        if (lane == 0) {
            griddep_wait();                                   // x_q and the h blocks come from the preceding kernels
            int it = 0;
            bool ok = true;
            for (int t = pair, i = 0; t < n_tiles && ok; t += n_pairs, ++i) {
                const P2Tile tl = p2_tile<FP4>(p, t, m_tiles);
                const CUtensorMap* tmb = (tl.s == 0) ? &tm_b0 : (tl.s == 1) ? &tm_b1 : (tl.s == 2) ? &tm_b2 : &tm_b3;
                const int row0 = tl.n0_local + (int)rank * 128;           // this CTA's rows of each 256-feature half
                for (int kb = 0; kb < p.kblocks && ok; ++kb, ++it) {
                    const int st = it % kStages;
                    if (ctrl->abort_flag ||
                        (it >= kStages && !mbar_wait_cluster(&ctrl->empty[st], (uint32_t)((it / kStages - 1) & 1), limit_ns))) {
                        if (!ctrl->abort_flag) p2_timeout(p, ctrl, 1, it);
                        ok = false;
                        break;
                    }
                    uint8_t* slot = ring + (size_t)st * kSlot;
                    // every load is a tensor load, so both CTAs' bytes are counted on rank 0's barrier and no relay stands
                    // between the partner's data and the MMAs
                    const uint32_t bar0 = cluster_peer_addr(smem_u32(&ctrl->full[st]), 0);
                    if (rank == 0) mbar_arrive_expect_tx(&ctrl->full[st], (uint32_t)(2 * kSlot));
#pragma unroll
                    for (int h = 0; h < kHalves; ++h)
                        tma_load_2d_pair(slot + h * kP2WBytes, &tm_w, bar0, kb * 128, tl.slice_off + row0 + h * 256);
                    tma_load_2d_pair(slot + kXOff, &tm_x, bar0, kb * 128, tl.t0 + (int)rank * 128);
                    if (FP4) {
                        // scales, as 8 x 256-byte rows of a [rows, 256] byte tensor per 2 KB atom: this CTA's 128 tokens (the
                        // MMA's A rows), then both 128-feature tiles of W (every CTA needs the scales of all of B's 256 rows in
                        // its own tensor memory)
                        uint8_t* sf = slot + kXOff + kP2XBytes;
                        tma_load_2d_pair(sf, &tm_xsf, bar0, 0, ((tl.m_idx * p.kblocks + kb) * 2 + (int)rank) * 8);
                        tma_load_2d_pair(sf + kSfSlotBytes, &tm_wsf, bar0, 0, ((tl.n_idx * 2) * p.kblocks + kb) * 8);
                        tma_load_2d_pair(sf + 2 * kSfSlotBytes, &tm_wsf, bar0, 0, ((tl.n_idx * 2 + 1) * p.kblocks + kb) * 8);
                    }
                }
                if (!ok) break;
                const P2Meta& mt = ctrl->meta[i & 1];
                if (!mbar_wait(&ctrl->meta_full[i & 1], (uint32_t)((i >> 1) & 1), limit_ns)) {
                    p2_timeout(p, ctrl, 2, it);
                    break;
                }
                const int n_steps = mt.n_steps;
                for (int li = 0; li < n_steps && ok; ++li, ++it) {
                    const int st = it % kStages;
                    if (ctrl->abort_flag ||
                        (it >= kStages && !mbar_wait_cluster(&ctrl->empty[st], (uint32_t)((it / kStages - 1) & 1), limit_ns))) {
                        if (!ctrl->abort_flag) p2_timeout(p, ctrl, 3, it);
                        ok = false;
                        break;
                    }
                    const P2Step e = mt.steps[li];
                    uint8_t* slot = ring + (size_t)st * kSlot;
                    // B_l: this CTA's 128 features of each half.  h: the step's 128-token block belongs to ONE CTA of the pair
                    // (block b = rank b's tokens); the other CTA's rows of the M = 256 MMA must add nothing, so it fetches a
                    // box that lies wholly outside the tensor, which TMA fills with zeros.
                    const int h_row = (int)e.block == (int)rank ? tl.s * p.max_m + tl.t0 + (int)e.block * 128 : p.S * p.max_m + 128;
                    const uint32_t bar0 = cluster_peer_addr(smem_u32(&ctrl->full[st]), 0);
                    if (rank == 0) mbar_arrive_expect_tx(&ctrl->full[st], (uint32_t)(2 * (kXOff + kP2XBytes)));
#pragma unroll
                    for (int h = 0; h < kHalves; ++h)
                        tma_load_2d_pair(slot + h * kP2WBytes, tmb, bar0, (int)e.chunk * 64, (int)e.lora * tl.n_s + row0 + h * 256);
                    tma_load_2d_pair(slot + kXOff, &tm_h, bar0, (int)e.entry * p.R + (int)e.chunk * 64, h_row);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // =========================================================== MMA issuer of the pair
            // A = tokens (each CTA's 128 are its accumulator's lanes), B = features (128 from each CTA per 256-wide half)
            const uint32_t idesc4 = umma_idesc_nvfp4(256, 256);
            const uint32_t idesc8 = umma_idesc(0, 0, 256, 256);
            const uint32_t idesc16 = umma_idesc(1, 1, 256, 256);
            int it = 0;
            bool ok = true;
            uint32_t sf_par = 0;                              // per slot: phase of its scale barrier
            for (int t = pair, i = 0; t < n_tiles && ok; t += n_pairs, ++i) {
                if (i > 0) {                                  // both epilogues have read the previous tile out of tensor memory
                    if (ctrl->abort_flag || !mbar_wait_cluster(&ctrl->acc_empty, (uint32_t)((i - 1) & 1), limit_ns)) {
                        if (!ctrl->abort_flag) p2_timeout(p, ctrl, 8, i);
                        break;
                    }
                    tc_fence_after();
                }
                for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
                    const int st = it % kStages;
                    const uint32_t par = (uint32_t)((it / kStages) & 1);
                    bool landed;
                    if (FP4) {
                        // the scale copier saw both CTAs' operands land before it copied: one wait covers data and scales; the
                        // barrier completes once per K-BLOCK use of the slot -- expand steps pass it by -- so it has its own parity
                        landed = !ctrl->abort_flag && mbar_wait(&ctrl->sf_ready[st], (sf_par >> st) & 1u, limit_ns);
                        sf_par ^= 1u << st;
                    } else {
                        landed = !ctrl->abort_flag && mbar_wait_cluster(&ctrl->full[st], par, limit_ns);
                    }
                    if (!landed) {
                        if (!ctrl->abort_flag) p2_timeout(p, ctrl, 4, it);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t wa = smem_u32(ring + (size_t)st * kSlot);
                    const uint64_t dx = umma_smem_desc(wa + kXOff, 1024, 2);
                    if (FP4) {
                        const uint64_t dw = umma_smem_desc(wa, 1024, 2);
                        const uint32_t sft = tmem_base + 256u + (uint32_t)(st * kP2SfCols);
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint32_t ta = sft + (uint32_t)k * 4u, tb = sft + 16u + (uint32_t)k * 8u;
                            umma_nvfp4_pair(tmem_base, dx + (uint64_t)(k * 2), dw + (uint64_t)(k * 2), idesc4, ta, tb, (kb > 0 || k > 0) ? 1u : 0u);
                        }
                    } else {
#pragma unroll
                        for (int h = 0; h < kHalves; ++h) {
                            const uint64_t dw = umma_smem_desc(wa + (uint32_t)(h * kP2WBytes), 1024, 2);
#pragma unroll
                            for (int k = 0; k < 4; ++k)
                                umma_f8f6f4_pair(tmem_base + (uint32_t)(h * 256), dx + (uint64_t)(k * 2), dw + (uint64_t)(k * 2), idesc8,
                                                 (kb > 0 || k > 0) ? 1u : 0u);
                        }
                    }
                    umma_commit_pair(&ctrl->empty[st], 3);
                }
                if (!ok) break;
                if (!mbar_wait(&ctrl->meta_full[i & 1], (uint32_t)((i >> 1) & 1), limit_ns)) {
                    p2_timeout(p, ctrl, 5, it);
                    break;
                }
                const int n_steps = ctrl->meta[i & 1].n_steps;
                for (int li = 0; li < n_steps; ++li, ++it) {
                    const int st = it % kStages;
                    const uint32_t par = (uint32_t)((it / kStages) & 1);
                    if (ctrl->abort_flag || !mbar_wait_cluster(&ctrl->full[st], par, limit_ns)) {
                        if (!ctrl->abort_flag) p2_timeout(p, ctrl, 6, it);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t ba = smem_u32(ring + (size_t)st * kSlot);
                    const uint64_t dh = umma_smem_desc(ba + kXOff, 1024, 2);
#pragma unroll
                    for (int h = 0; h < kHalves; ++h) {
                        const uint64_t db = umma_smem_desc(ba + (uint32_t)(h * kP2WBytes), 1024, 2);
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            umma_f16_pair(tmem_base + (uint32_t)(h * 256), dh + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc16, 1u);
                    }
                    umma_commit_pair(&ctrl->empty[st], 3);
                }
                if (ok) umma_commit_pair(&ctrl->acc_full, 3);
            }
        }
    } else if (warp == 7 || warp >= 12) {
        // =========================================================== scale copiers (NVFP4, rank 0; warps 7, 12, 13): a k-block
        // slot's scale factors -> both CTAs' tensor memory, ahead of the MMAs.  Threads of their own because every tcgen05
        // instruction costs its issuer some 50 cycles: twelve copies per slot from one thread (with its wait and commit, 920
        // cycles) bounded the main loop, whose four MMAs take the tensor pipe some 540.  Copier 0 moves the tokens' scales,
        // copiers 1 and 2 those of the two 128-feature halves of W: four copies each per slot.
        const int cpi = warp == 7 ? 0 : warp - 11;
        if (FP4 && lane == 0 && rank == 0) {
            int it = 0;
            bool ok = true;
            for (int t = pair, i = 0; t < n_tiles && ok; t += n_pairs, ++i) {
                // the tile's expand steps use ring slots too: read their number now (the scout is a tile ahead), while this
                // thread's own copies still stand between the read and the buffer's next writer
                if (!mbar_wait(&ctrl->meta_full[i & 1], (uint32_t)((i >> 1) & 1), limit_ns)) {
                    p2_timeout(p, ctrl, 14, it);
                    break;
                }
                const int n_steps = ctrl->meta[i & 1].n_steps;
                for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
                    const int st = it % kStages;
                    const uint32_t par = (uint32_t)((it / kStages) & 1);
                    if (ctrl->abort_flag || !mbar_wait_cluster(&ctrl->full[st], par, limit_ns)) {
                        if (!ctrl->abort_flag) p2_timeout(p, ctrl, 13, it);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sfs = smem_u32(ring + (size_t)st * kSlot) + (uint32_t)(kXOff + kP2XBytes);
                    const uint32_t sft = tmem_base + 256u + (uint32_t)(st * kP2SfCols);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint32_t dst = cpi == 0 ? sft + (uint32_t)k * 4u : sft + 16u + (uint32_t)k * 8u + (uint32_t)(cpi - 1) * 4u;
                        tmem_cp_sf_pair(dst, sf_smem_desc(sfs + (uint32_t)cpi * kSfSlotBytes + (uint32_t)k * 512u));
                    }
                    umma_commit_pair(&ctrl->sf_ready[st], 1);      // (arrives in rank 0 only)
                }
                // The expand steps' slots carry no scales, but this thread still follows their barriers phase by phase: a
                // parity wait entered a whole phase early would pass at once.
                for (int li = 0; li < n_steps && ok; ++li, ++it) {
                    const int st = it % kStages;
                    const uint32_t par = (uint32_t)((it / kStages) & 1);
                    if (ctrl->abort_flag || !mbar_wait_cluster(&ctrl->full[st], par, limit_ns)) {
                        if (!ctrl->abort_flag) p2_timeout(p, ctrl, 15, it);
                        ok = false;
                    }
                }
            }
        }
    } else if (warp == 2) {
        // =========================================================== tile scout (the same list in both CTAs)
        int n_all, n_ad;
        segment_totals(p.meta, p.L, lane, n_all, n_ad);
        n_all = min(n_all, p.M);
        griddep_wait();                                       // K1's s_x from here on
        const float s_w = __ldg(p.s_w);
        for (int t = pair, i = 0; t < n_tiles; t += n_pairs, ++i) {
            P2Meta& mt = ctrl->meta[i & 1];
            int go = 1;
            if (lane == 0 && i >= 2) {
                go = ctrl->abort_flag ? 0 : 1;
                if (go && !mbar_wait(&ctrl->meta_empty[i & 1], (uint32_t)(((i >> 1) - 1) & 1), limit_ns)) {
                    p2_timeout(p, ctrl, 9, i);
                    go = 0;
                }
            }
            go = __shfl_sync(0xffffffffu, go, 0);
            if (!go) break;
            const P2Tile tl = p2_tile<FP4>(p, t, m_tiles);
            for (int c = lane; c < kP2Tokens; c += 32) {
                const int pos = tl.t0 + c;
                mt.rowmap[c] = pos < p.M ? position_row(p.meta, pos, p.M, n_all, n_ad) : -1;
                // FP8: the token's activation scale times the weight scale; NVFP4: alpha = 1 / (x_global * w_global) for all
                mt.scale[c] = pos < p.M ? (p.sx ? __ldcg(p.sx + pos) : 1.0f) * s_w : 0.0f;
            }
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
                            const int rk = __popc(mask & ((1u << lane) - 1u));
                            const int entry = entries + rk;
                            if (entry < kMaxTileTenants)
                                for (int c = 0; c < n_chunks; ++c) {
                                    const int li = total + rk * n_chunks + c;
                                    if (li < kP2MaxSteps)
                                        mt.steps[li] = P2Step{(uint16_t)lora, (uint16_t)entry, (uint16_t)blk, (uint16_t)c};
                                }
                        }
                        entries += __popc(mask);
                        total += __popc(mask) * n_chunks;
                    }
                }
            }
            if (lane == 0) mt.n_steps = min(total, kP2MaxSteps);
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctrl->meta_full[i & 1]);
        }
    } else {
        // =========================================================== epilogue (warps 3..6 and 8..11): this CTA's 128 tokens -> y
        // Two warps per 32-lane quarter of tensor memory, one per half of the tile's features.
        const int te = tid - 96;
        const int q = warp & 3;                               // the 32 tensor-memory lanes this warp may read
        const int c_beg = warp >= 8 ? kRows / 2 : 0, c_end = c_beg + kRows / 2;
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        const uint32_t acc_empty_addr = cluster_peer_addr(smem_u32(&ctrl->acc_empty), 0);
        for (int t = pair, i = 0; t < n_tiles; t += n_pairs, ++i) {
            const P2Meta& mt = ctrl->meta[i & 1];
            if (te == 0) {
                int go = ctrl->abort_flag ? 0 : 1;
                if (go && !mbar_wait(&ctrl->meta_full[i & 1], (uint32_t)((i >> 1) & 1), limit_ns)) {
                    p2_timeout(p, ctrl, 10, i);
                    go = 0;
                }
                if (go && !mbar_wait_cluster(&ctrl->acc_full, (uint32_t)(i & 1), limit_ns)) {
                    p2_timeout(p, ctrl, 7, i);
                    go = 0;
                }
                ctrl->go_flag = go;
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
            const int go = ctrl->go_flag;
            asm volatile("bar.sync 1, 256;" ::: "memory");    // everyone has read the flag before its next writer runs
            if (!go) break;
            tc_fence_after();
            const P2Tile tl = p2_tile<FP4>(p, t, m_tiles);
            // Thread = one token (tensor-memory lane); a load brings 32 consecutive features of it, 64 contiguous bytes of
            // the token's row in y.  Stored as they come, a warp's store instruction would touch 32 rows with 16 bytes each and
            // the tile's read-out is bound by the store unit (measured: 18 k cycles per 512-feature tile, a third of the
            // kernel, spent with the tensor pipe idle).  So every four lanes transpose their 4 x 4 sixteen-byte pieces first
            // (two shuffle stages): lane j of a group then holds piece j of each of the group's four tokens, and a store
            // instruction writes 64 contiguous bytes of 8 rows.  No staging in shared memory, no barrier between the warps.
            // Two register buffers: the next load is in flight while this one is converted and stored.
            const int c_tok = (int)rank * 128 + q * 32 + lane;
            const int row = mt.rowmap[c_tok];
            const float sc = mt.scale[c_tok];
            const int lj = lane & 3;
            __nv_bfloat16* yr4[4];
            bool live4[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int rr = __shfl_sync(0xffffffffu, row, (lane & ~3) + r);
                live4[r] = rr >= 0;
                yr4[r] = p.y + (int64_t)(rr < 0 ? 0 : rr) * p.ldy + tl.slice_off + tl.n0_local + lj * 8;
            }
            auto store32 = [&](const uint32_t (&r)[32], int c0) {
                uint32_t o[16];                               // o[4 v + u]: piece v (8 features), register u
#pragma unroll
                for (int u = 0; u < 16; ++u) {
                    const __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(r[2 * u]) * sc, __uint_as_float(r[2 * u + 1]) * sc);
                    o[u] = *reinterpret_cast<const uint32_t*>(&b2);
                }
#pragma unroll
                for (int v = 0; v < 2; ++v)                   // 2 x 2 blocks of pieces change places between lanes j and j ^ 2
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const uint32_t send = (lj & 2) ? o[v * 4 + u] : o[(v + 2) * 4 + u];
                        const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, 2);
                        if (lj & 2) o[v * 4 + u] = recv; else o[(v + 2) * 4 + u] = recv;
                    }
#pragma unroll
                for (int v = 0; v < 4; v += 2)                // then the pieces inside each block between lanes j and j ^ 1
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const uint32_t send = (lj & 1) ? o[v * 4 + u] : o[(v + 1) * 4 + u];
                        const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, 1);
                        if (lj & 1) o[v * 4 + u] = recv; else o[(v + 1) * 4 + u] = recv;
                    }
#pragma unroll
                for (int r4 = 0; r4 < 4; ++r4)                // o[4 r4 ..]: piece lj of the group's token r4
                    if (live4[r4])
                        *reinterpret_cast<uint4*>(yr4[r4] + c0) = make_uint4(o[r4 * 4], o[r4 * 4 + 1], o[r4 * 4 + 2], o[r4 * 4 + 3]);
            };
            uint32_t ra[32], rb[32];
            tmem_ld32(tmem_base + lane_addr + (uint32_t)c_beg, ra);
#pragma unroll 1
            for (int c0 = c_beg; c0 < c_end; c0 += 64) {
                tmem_ld_wait();
                tmem_ld32(tmem_base + lane_addr + (uint32_t)(c0 + 32), rb);
                store32(ra, c0);
                tmem_ld_wait();
                if (c0 + 64 < c_end) {
                    tmem_ld32(tmem_base + lane_addr + (uint32_t)(c0 + 64), ra);
                } else {                                      // tensor memory has been read: the next tile's MMAs may start
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_remote(acc_empty_addr);
                }
                store32(rb, c0 + 32);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctrl->meta_empty[i & 1]);
        }
    }
    // ---- teardown: neither CTA leaves (or frees tensor memory) while its partner may still read its shared memory, write
    // its tensor memory or arrive on its barriers
    if (ctrl->abort_flag) __nanosleep(200000);
    tc_fence_before();
    __syncthreads();
    __syncwarp();
    cluster_arrive();
    cluster_wait();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

size_t k2_prefill_pair_smem_bytes(int fp4) {
    return 1024 + (size_t)p2_stages(fp4 != 0) * (size_t)p2_slot_bytes(fp4 != 0) + sizeof(P2Ctrl) + 64;
}
int k2_prefill_pair_max_steps() { return kP2MaxSteps; }
int k2_prefill_pair_rows(int fp4) { return p2_rows(fp4 != 0); }

template <bool FP4>
static void pair_launch_config(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* attr, int pairs, int pdl, cudaStream_t stream) {
    *cfg = cudaLaunchConfig_t{};
    cfg->gridDim = dim3((unsigned)(2 * pairs));
    cfg->blockDim = dim3(kP2Threads);
    cfg->dynamicSmemBytes = k2_prefill_pair_smem_bytes(FP4 ? 1 : 0);
    cfg->stream = stream;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg->attrs = attr;
    cfg->numAttrs = pdl ? 2 : 1;
}

// Resident pairs of the kernel on the current device (a pair sits inside one GPC, so fewer may fit than SMs / 2); also
// raises the kernel's dynamic shared-memory limit, so it is called before the first launch.
template <bool FP4>
static int pair_capacity() {
    static std::atomic<int> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { (void)cudaGetLastError(); return 0; }
    int n = cached[dev].load();
    if (n > 0) return n;
    cudaError_t e = cudaFuncSetAttribute(k2_prefill_pair_kernel<FP4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
    if (e != cudaSuccess) { (void)cudaGetLastError(); return 0; }
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[2];
    pair_launch_config<FP4>(&cfg, attr, 148, 0, nullptr);
    n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, k2_prefill_pair_kernel<FP4>, &cfg);
    if (e != cudaSuccess) { (void)cudaGetLastError(); return 0; }
    cached[dev].store(n);
    return n;
}
int k2_prefill_pair_capacity(int fp4) { return fp4 ? pair_capacity<true>() : pair_capacity<false>(); }

cudaError_t launch_k2_prefill_pair(const K2pParams& p, const CUtensorMap& tm_w, const CUtensorMap& tm_x, const CUtensorMap& tm_h,
                                   const CUtensorMap* tm_b, const CUtensorMap* tm_sf, int pairs, int fp4, int pdl,
                                   cudaStream_t stream) {
    // tm_sf: NVFP4 base only, the packed W block scales and the workspace's token block scales as [rows, 256] byte tensors
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[2];
    if (fp4) {
        pair_launch_config<true>(&cfg, attr, pairs, pdl, stream);
        return cudaLaunchKernelEx(&cfg, k2_prefill_pair_kernel<true>, p, tm_w, tm_x, tm_h, tm_b[0], tm_b[1], tm_b[2], tm_b[3], tm_sf[0],
                                  tm_sf[1]);
    }
    pair_launch_config<false>(&cfg, attr, pairs, pdl, stream);
    return cudaLaunchKernelEx(&cfg, k2_prefill_pair_kernel<false>, p, tm_w, tm_x, tm_h, tm_b[0], tm_b[1], tm_b[2], tm_b[3], tm_w, tm_w);
}

}  // namespace ob
