// K2 for prefill batches (more than 128 tokens), FP8 base, bf16 adapters: one CTA per 256 output features x 256 tokens.
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
// Warps: 0 = TMA producer (one thread), 1 = MMA issuer (one thread; owns the tensor-memory allocation), 2..5 = the tile's
// expand steps from the segment index, then the epilogue (tcgen05.ld, scale, the bf16 tile staged in shared memory, whole
// token rows scattered back through the sort).
// Ring slots of 64 KB: a W k-block [256 x 128 B] with its x_q tile [256 tokens x 128 B], or an expand step's B and h
// tiles.  All W k-blocks come first, the expand steps last.  Every wait is bounded.
#include "ob_common.cuh"
#include "ob_ptx.cuh"

namespace ob {

constexpr int kPfThreads = 192;
constexpr int kPfRows = 256;                 // output features per CTA (two MMA halves of 128)
constexpr int kPfTokens = 256;               // tokens per CTA (the MMAs' N)
constexpr int kPfSlotBytes = 64 * 1024;
constexpr int kPfHalfBytes = 128 * 128;      // one 128-row half of a W or B tile
constexpr int kPfMaxStages = 3;
constexpr int kPfMaxSteps = 1024;

struct PfStep {
    uint16_t lora, entry, block, chunk;      // tenant, its entry in the 128-block's list, 128-block of the tile, rank chunk
};

struct PfCtrl {
    uint64_t full[kPfMaxStages];
    uint64_t empty[kPfMaxStages];
    uint64_t list_ready;
    uint64_t acc_full;
    uint32_t tmem_base;
    volatile int abort_flag;
    int n_steps;
    int go_flag;
    int rowmap[kPfTokens];
    float scale[kPfTokens];
    PfStep steps[kPfMaxSteps];
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

__global__ void __launch_bounds__(kPfThreads, 1)
k2_prefill_kernel(const K2pParams p, const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                  const __grid_constant__ CUtensorMap tm_h, const __grid_constant__ CUtensorMap tm_b0,
                  const __grid_constant__ CUtensorMap tm_b1, const __grid_constant__ CUtensorMap tm_b2,
                  const __grid_constant__ CUtensorMap tm_b3) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* ring = smem;
    PfCtrl* ctrl = reinterpret_cast<PfCtrl*>(smem + (size_t)p.stages * kPfSlotBytes);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    griddep_launch_dependents();
    const uint64_t limit_ns = (uint64_t)p.wait_ms * 1000000ull;

    // grid x walks the token tiles (consecutive CTAs share a W tile: HBM once, L2 after), z the 256-row output tiles
    const int t0 = blockIdx.x * kPfTokens;
    int s = 0, n_tile = blockIdx.z, slice_off = 0;
    while (s < p.S - 1 && n_tile >= p.widths[s] / kPfRows) {
        n_tile -= p.widths[s] / kPfRows;
        slice_off += p.widths[s];
        ++s;
    }
    const int n_s = p.widths[s];
    const int n0_local = n_tile * kPfRows;
    const int n_chunks = p.R / 64;

    if (tid == 0) {
        for (int i = 0; i < kPfMaxStages; ++i) {
            mbar_init(&ctrl->full[i], 1);
            mbar_init(&ctrl->empty[i], 1);
        }
        mbar_init(&ctrl->list_ready, 1);
        mbar_init(&ctrl->acc_full, 1);
        ctrl->abort_flag = 0;
        ctrl->n_steps = 0;
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
        // =========================================================== TMA producer
        if (lane == 0) {
            const CUtensorMap* tmb = (s == 0) ? &tm_b0 : (s == 1) ? &tm_b1 : (s == 2) ? &tm_b2 : &tm_b3;
            griddep_wait();                                   // x_q, s_x and the h blocks come from the preceding kernels
            int it = 0;
            bool ok = true;
            for (int kb = 0; kb < p.kblocks && ok; ++kb, ++it) {
                const int st = it % p.stages;
                if (ctrl->abort_flag ||
                    (it >= p.stages && !mbar_wait(&ctrl->empty[st], (uint32_t)((it / p.stages - 1) & 1), limit_ns))) {
                    if (!ctrl->abort_flag) pf_timeout(p, ctrl, 1, it);
                    ok = false;
                    break;
                }
                uint8_t* slot = ring + (size_t)st * kPfSlotBytes;
                mbar_arrive_expect_tx(&ctrl->full[st], (uint32_t)(2 * kPfHalfBytes + kPfTokens * 128));
                tma_load_2d(slot, &tm_w, &ctrl->full[st], kb * 128, slice_off + n0_local);
                tma_load_2d(slot + 2 * kPfHalfBytes, &tm_x, &ctrl->full[st], kb * 128, t0);
            }
            if (ok && !mbar_wait(&ctrl->list_ready, 0, limit_ns)) {
                pf_timeout(p, ctrl, 2, it);
                ok = false;
            }
            const int n_steps = ok ? ctrl->n_steps : 0;
            for (int li = 0; li < n_steps && ok; ++li, ++it) {
                const int st = it % p.stages;
                if (ctrl->abort_flag ||
                    (it >= p.stages && !mbar_wait(&ctrl->empty[st], (uint32_t)((it / p.stages - 1) & 1), limit_ns))) {
                    if (!ctrl->abort_flag) pf_timeout(p, ctrl, 3, it);
                    break;
                }
                const PfStep e = ctrl->steps[li];
                uint8_t* slot = ring + (size_t)st * kPfSlotBytes;
                mbar_arrive_expect_tx(&ctrl->full[st], (uint32_t)(2 * kPfHalfBytes + 128 * 128));
                tma_load_2d(slot, tmb, &ctrl->full[st], (int)e.chunk * 64, (int)e.lora * n_s + n0_local);
                tma_load_2d(slot + 2 * kPfHalfBytes, &tm_h, &ctrl->full[st], (int)e.entry * p.R + (int)e.chunk * 64,
                            s * p.max_m + t0 + (int)e.block * 128);
            }
        }
    } else if (warp == 1) {
        // =========================================================== MMA issuer
        if (lane == 0) {
            const uint32_t idesc8 = umma_idesc(0, 0, 128, kPfTokens);
            const uint32_t idesc16 = umma_idesc(1, 1, 128, 128);
            int it = 0;
            bool ok = true;
            for (int kb = 0; kb < p.kblocks; ++kb, ++it) {
                const int st = it % p.stages;
                if (ctrl->abort_flag || !mbar_wait(&ctrl->full[st], (uint32_t)((it / p.stages) & 1), limit_ns)) {
                    if (!ctrl->abort_flag) pf_timeout(p, ctrl, 4, it);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t wa = smem_u32(ring + (size_t)st * kPfSlotBytes);
                const uint64_t dx = umma_smem_desc(wa + 2 * kPfHalfBytes, 1024, 2);
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const uint64_t dw = umma_smem_desc(wa + (uint32_t)(half * kPfHalfBytes), 1024, 2);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_f8f6f4(tmem_base + (uint32_t)(half * kPfTokens), dw + (uint64_t)(k * 2), dx + (uint64_t)(k * 2), idesc8,
                                    (kb > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(&ctrl->empty[st]);
            }
            if (ok && !mbar_wait(&ctrl->list_ready, 0, limit_ns)) {
                pf_timeout(p, ctrl, 5, it);
                ok = false;
            }
            const int n_steps = ok ? ctrl->n_steps : 0;
            for (int li = 0; li < n_steps; ++li, ++it) {
                const int st = it % p.stages;
                if (ctrl->abort_flag || !mbar_wait(&ctrl->full[st], (uint32_t)((it / p.stages) & 1), limit_ns)) {
                    if (!ctrl->abort_flag) pf_timeout(p, ctrl, 6, it);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const PfStep e = ctrl->steps[li];
                const uint32_t ba = smem_u32(ring + (size_t)st * kPfSlotBytes);
                const uint64_t dh = umma_smem_desc(ba + 2 * kPfHalfBytes, 1024, 2);
#pragma unroll
                for (int half = 0; half < 2; ++half) {
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
    } else {
        // =========================================================== expand steps, then the epilogue
        const int te = tid - 64;
        int n_all, n_ad;
        segment_totals(p.meta, p.L, lane, n_all, n_ad);
        n_all = min(n_all, p.M);
        for (int c = te; c < kPfTokens; c += 128) {
            const int pos = t0 + c;
            ctrl->rowmap[c] = pos < p.M ? position_row(p.meta, pos, p.M, n_all, n_ad) : -1;
        }
        if (warp == 2) {
            // per 128-position block, the segments that reach into it, in segment order: the order in which the shrink
            // numbered the block's h entries
            int total = 0;
            if (n_ad > 0) {
                for (int blk = 0; blk < 2; ++blk) {
                    const int b0 = t0 + blk * 128;
                    int entries = 0;
                    for (int base = 0; base <= p.L; base += 32) {
                        const int i = base + lane;
                        int lora = -1, lo = 0, hi = 0;
                        if (i <= p.L) {
                            lora = p.meta.seg_ids[i];
                            const int cnt = p.meta.seg_n[i], sst = p.meta.seg_start[i];
                            lo = max(sst, b0);
                            hi = min(min(sst + cnt, b0 + 128), n_all);
                            if (cnt <= 0 || sst < 0) lora = -1;
                        }
                        const bool ok = lora >= 0 && lora < p.L && lo < hi;
                        const uint32_t mask = __ballot_sync(0xffffffffu, ok);
                        if (ok) {
                            const int rank = __popc(mask & ((1u << lane) - 1u));   // hits of lower lanes in this ballot
                            const int entry = entries + rank;
                            if (entry < kMaxTileTenants)
                                for (int c = 0; c < n_chunks; ++c) {
                                    const int li = total + rank * n_chunks + c;
                                    if (li < kPfMaxSteps)
                                        ctrl->steps[li] = PfStep{(uint16_t)lora, (uint16_t)entry, (uint16_t)blk, (uint16_t)c};
                                }
                        }
                        entries += __popc(mask);
                        total += __popc(mask) * n_chunks;
                    }
                }
            }
            if (lane == 0) ctrl->n_steps = min(total, kPfMaxSteps);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (te == 0) mbar_arrive(&ctrl->list_ready);

        griddep_wait();                                       // K1's s_x from here on
        const float s_w = __ldg(p.s_w);
        for (int c = te; c < kPfTokens; c += 128) ctrl->scale[c] = (t0 + c < p.M) ? __ldcg(p.sx + t0 + c) * s_w : 0.0f;
        asm volatile("bar.sync 1, 128;" ::: "memory");

        if (te == 0) {
            int go = ctrl->abort_flag ? 0 : 1;
            if (go && !mbar_wait(&ctrl->acc_full, 0u, limit_ns)) {
                pf_timeout(p, ctrl, 7, 0);
                go = 0;
            }
            ctrl->go_flag = go;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        tc_fence_after();
        if (ctrl->go_flag) {
            // The ring is idle now (every tile was consumed): it stages the output tile as [token][256 features] bf16, so
            // that each token's 512 bytes leave in one coalesced store instead of 2-byte stores per feature.
            const int q = warp & 3;
            const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
            const int n_tok = min(kPfTokens, p.M - t0);
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {
                uint8_t* col = ring + (size_t)(half * 128 + q * 32 + lane) * 2;
#pragma unroll 1
                for (int c0 = 0; c0 < n_tok; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld32(tmem_base + lane_addr + (uint32_t)(half * kPfTokens + c0), r);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; ++c)
                        *reinterpret_cast<__nv_bfloat16*>(col + (size_t)(c0 + c) * (kPfRows * 2)) =
                            __float2bfloat16_rn(__uint_as_float(r[c]) * ctrl->scale[c0 + c]);
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            __nv_bfloat16* ybase = p.y + slice_off + n0_local + lane * 8;
            for (int c = warp - 2; c < n_tok; c += 4) {
                const int row = ctrl->rowmap[c];
                if (row >= 0)
                    *reinterpret_cast<uint4*>(ybase + (int64_t)row * p.ldy) =
                        *reinterpret_cast<const uint4*>(ring + (size_t)c * (kPfRows * 2) + lane * 16);
            }
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

size_t k2_prefill_smem_bytes(int stages) { return 1024 + (size_t)stages * kPfSlotBytes + sizeof(PfCtrl) + 64; }

cudaError_t launch_k2_prefill(const K2pParams& p, const CUtensorMap& tm_w, const CUtensorMap& tm_x, const CUtensorMap& tm_h,
                              const CUtensorMap* tm_b, dim3 grid, int pdl, cudaStream_t stream) {
    static int configured_for[64] = {0};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64 && !configured_for[dev]) {
        e = cudaFuncSetAttribute(k2_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
        if (e != cudaSuccess) return e;
        configured_for[dev] = 1;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kPfThreads);
    cfg.dynamicSmemBytes = k2_prefill_smem_bytes(p.stages);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, k2_prefill_kernel, p, tm_w, tm_x, tm_h, tm_b[0], tm_b[1], tm_b[2], tm_b[3]);
}

}  // namespace ob
