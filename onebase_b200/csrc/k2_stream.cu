// K2 for decode batches (one token tile of at most 32 adapter-sorted positions, bf16 adapters), as ONE persistent CTA per
// SM that streams a contiguous share of the launch's weight bytes, whatever the number of output tiles:
//
//   The launch's work is the sequence of W k-blocks (128 output features x 128 bytes of K) of all output tiles, tile
//   after tile.  CTA c of G owns k-blocks [c*U/G, (c+1)*U/G) of that sequence (U = tiles x k-blocks per tile), so its
//   share crosses tile boundaries: it is cut into per-tile SEGMENTS.  For a segment that covers k-blocks [ka, ke) of a
//   tile the CTA also takes the same fraction of the tile's expand steps, [ka*ns/kb, ke*ns/kb) of the batch's ns
//   (segment, rank chunk) steps, so the tenants' B tiles are spread over the CTAs like the weights.
//
//   Two rings of shared-memory slots, each with its own producer thread and its own consumer, so that neither stream
//   holds up the other:
//     W ring   W tile [128 x 128 B] + its x_q tile (+ NVFP4 scale blocks); consumed by the tcgen05.mma issuer into one of
//              four accumulator buffers in tensor memory (segment i uses buffer i % 4).  Needs only K1's codes.
//     B ring   the expand steps' B tiles [128 features x rank chunk] bf16; consumed by the four epilogue warps, which add
//              each tenant's expansion on the CUDA cores: thread n owns output feature n and accumulates
//              sum_r B[n][r] * h[token][r] (fp32 FMAs on bf16 inputs, as the reference's bf16 dot with fp32 accumulate)
//              for the step's one or two tokens into its column of a [tokens x 128] fp32 tile in shared memory.
//              Needs K1's h, i.e. K1's end.  (On the tensor cores a step's four 128 x 32 x 16 MMAs cost more than its
//              16 KB of B take to arrive, and consumed ring slots in order with the weights.)
//   In a K1 -> K2 chain the weight stream therefore runs WHILE K1's shrink warps are still streaming A: K1 counts the
//   positions whose codes and scales are in memory, the W producer starts on that count, and only the expand waits for
//   K1's end.
//
//   A segment that covers its whole tile stores bf16 rows directly.  Otherwise the CTA leaves an fp32 partial tile
//   (scaled base + expand) in the workspace and counts its arrival on the tile's counter; the LAST CTA to arrive adds the
//   tile's partials in CTA order -- the same order on every launch, so results repeat bit for bit -- stores the rows
//   and returns the counter to zero.  No CTA ever waits for another CTA.
//
//   warp 0   W producer (TMA, evict-first on W)          warp 1   MMA issuer: kind::f8f6f4, or kind::mxf4nvf4.block_scale
//   warp 2   B producer (TMA)                                     with the scales copied slot -> TMEM by tcgen05.cp
//   warps 4-7 segment index -> expand step list; after K1: h tables (K1's split-K partials added in split order, one
//            bf16 rounding); per segment the expand steps, the epilogue and, for shared tiles, the fix-up
//
// Every wait is bounded (wait_ms) and a wait that runs out records where and makes the CTA leave without storing.
//
// Computes what lowbit_lora/kernels/fp8_lora_pdl.py:324-495 (`_k2_body`) and lowbit_lora/kernels/nvfp4_lora_pdl.py:
// 192-257 compute; positions, padding and stale metadata follow lowbit_lora/kernels/fp8_lora_vllm.py:147-163.
#include <atomic>

#include "k1_device.cuh"

namespace ob {

constexpr int kKsThreads = 256;
constexpr int kKsWTileBytes = kTileN * kBlockK;   // 16 KB
constexpr int kKsCtrlBytes = 4096;
constexpr int kKsMaxSteps = 256;                  // (segment, rank chunk) steps of a batch: min(L, 32) x R / 64 at most 128
constexpr int kKsMaxStages = 16;

struct KsStep {
    uint16_t lora;    // adapter slot
    uint16_t chunk;   // rank chunk index
    uint16_t lo, hi;  // token positions [lo, hi) of the segment
};

constexpr int kKsAccBufs = 4;                     // accumulator buffers in tensor memory (segment i uses i % 4)
constexpr int kKsBStages = 6;                     // slots of the B ring
constexpr int kKsHTiles = 6;                      // masked H tiles in flight

struct KsCtrl {
    uint64_t full[kKsMaxStages];      // W ring
    uint64_t empty[kKsMaxStages];
    uint64_t full_b[kKsBStages];      // B ring
    uint64_t empty_b[kKsBStages];
    uint64_t acc_full[kKsAccBufs];    // two arrivals: the base GEMM's issuer and the expand's
    uint64_t acc_empty[kKsAccBufs];
    uint64_t h_full[kKsHTiles];       // a masked H tile is built
    uint64_t h_empty[kKsHTiles];      // ... and may be rebuilt: the MMAs that read it are complete
    uint64_t htab_ready;
    uint64_t list_ready;
    uint32_t tmem_base;
    volatile int abort_flag;
    int n_steps;
    int last_flag;
    int go_flag;
    int h_prev[kKsHTiles];   // the step whose rows each masked H tile holds (expand warp only)
    float sx[32];
    int rowmap[32];
    KsStep steps[kKsMaxSteps];
};
static_assert(sizeof(KsCtrl) <= kKsCtrlBytes, "control block too large");

// The share of CTA c.  With n_tiles = Q * G + Rm, every CTA owns Q WHOLE tiles (tiles c*Q .. c*Q+Q-1: stored directly, no
// fix-up) and an even share of the k-blocks of the Rm remainder tiles (tiles Q*G ..): k-blocks [w0, w1) of the remainder's
// sequence, cut into per-tile segments -- only these tiles are shared between CTAs.  The remainder segments come FIRST,
// so that their fix-ups run under the weight stream of the whole tiles and a CTA's last epilogue is a plain store.
struct KsSpan {
    long long w0, w1;     // this CTA's k-blocks of the remainder sequence
    int kb;               // k-blocks per tile
    int q_whole;          // whole tiles per CTA
    int rem0;             // first remainder tile
    int r_first, r_nseg;  // remainder segments: tiles rem0 + r_first ..
    int c;
    int nseg;
    __device__ static long long start_of(long long units, int G, int c) { return units * c / G; }
    __device__ KsSpan(int n_tiles, int kblocks, int G, int cta) : kb(kblocks), c(cta) {
        q_whole = n_tiles / G;
        rem0 = q_whole * G;
        const long long units = (long long)(n_tiles - rem0) * kblocks;
        w0 = start_of(units, G, cta);
        w1 = start_of(units, G, cta + 1);
        r_first = (int)(w0 / kb);
        r_nseg = w1 > w0 ? (int)((w1 - 1) / kb) - r_first + 1 : 0;
        nseg = r_nseg + q_whole;
    }
    __device__ void segment(int i, int& tile, int& ka, int& ke) const {
        if (i >= r_nseg) {                                   // a whole tile
            tile = c * q_whole + (i - r_nseg);
            ka = 0;
            ke = kb;
            return;
        }
        tile = rem0 + r_first + i;
        const long long base = (long long)(r_first + i) * kb;
        ka = (int)(w0 > base ? w0 - base : 0);
        ke = (int)(w1 < base + kb ? w1 - base : kb);
    }
};

// The CTA whose share holds unit u of the remainder sequence.
__device__ __forceinline__ int ks_owner(long long units, int G, long long u) {
    int c = (int)((u + 1) * G / units);
    if (c > G - 1) c = G - 1;
    while (c > 0 && KsSpan::start_of(units, G, c) > u) --c;
    while (c < G - 1 && KsSpan::start_of(units, G, c + 1) <= u) ++c;
    return c;
}

struct KsTile {
    int s, n0_local, slice_off, n_s;
    bool has_b;           // sharded B: only the tiles whose rows this rank holds carry an expand
};

__device__ __forceinline__ KsTile ks_tile(const K2Params& p, int tile) {
    KsTile g;
    g.s = 0;
    g.slice_off = 0;
    int n_tile = tile;
    while (g.s < p.S - 1 && n_tile >= (p.widths[g.s] + kTileN - 1) / kTileN) {
        n_tile -= (p.widths[g.s] + kTileN - 1) / kTileN;
        g.slice_off += p.widths[g.s];
        ++g.s;
    }
    g.n_s = p.widths[g.s];
    g.n0_local = n_tile * kTileN;
    g.has_b = g.n0_local >= p.b_row0[g.s] && g.n0_local < p.b_row0[g.s] + p.b_rows[g.s];
    return g;
}

__device__ __forceinline__ void ks_timeout(const K2Params& p, KsCtrl* c, int where, int it) {
    c->abort_flag = 1;
    if (atomicCAS(p.status, OB_DEV_OK, OB_DEV_WAIT_TIMEOUT) == OB_DEV_OK) {
        p.status[1] = 100 + where;      // 100+: the persistent decode kernel
        p.status[2] = blockIdx.x;
        p.status[3] = 0;
        p.status[4] = 0;
        p.status[5] = it;
    }
}

#define KS_TRACE(ev) \
    if (p.trace != nullptr && (long long)blockIdx.x < p.trace_ctas) p.trace[(long long)blockIdx.x * OB_TRACE_EVENTS + (ev)] = global_timer_ns();

template <bool FP4>
__global__ void __launch_bounds__(kKsThreads, 2)
k2_stream_kernel(const K2Params p, const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                 const __grid_constant__ CUtensorMap tm_b0, const __grid_constant__ CUtensorMap tm_b1,
                 const __grid_constant__ CUtensorMap tm_b2, const __grid_constant__ CUtensorMap tm_b3) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tn = p.tn;                                         // 16 or 32
    const int stages = p.stages;
    const int sf_bytes = FP4 ? 2 * kSfSlotBytes : 0;             // W scales + activation scales of one K slot
    const int stage_bytes = kKsWTileBytes + tn * kBlockK + sf_bytes;
    const int b_bytes = kTileN * p.rc * 2;                       // one B tile: 128 features x rank chunk, bf16
    const int b_stage_bytes = (int)align_up((size_t)b_bytes, 1024);
    const int htab_bytes = (int)align_up((size_t)tn * p.R * 2, 1024);
    uint8_t* ring = smem;
    uint8_t* bring = ring + (size_t)stages * stage_bytes;
    const int h_bytes = (int)align_up((size_t)tn * p.rc * 2, 1024);
    uint8_t* hbuf = bring + (size_t)kKsBStages * b_stage_bytes;     // masked H tiles (UMMA layout)
    uint8_t* htab = hbuf + (size_t)kKsHTiles * h_bytes;             // bf16 h tables [S][tn][R]
    KsCtrl* ctrl = reinterpret_cast<KsCtrl*>(htab + (size_t)p.S * htab_bytes);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    griddep_launch_dependents();
    const uint64_t limit_ns = (uint64_t)p.wait_ms * 1000000ull;
    const int G = (int)gridDim.x, cta = (int)blockIdx.x;
    const KsSpan span(p.n_tiles, p.kblocks, G, cta);
    const int nseg = span.nseg;
    const int kb = p.kblocks;
    const int n_chunks = p.R / p.rc;
    if (tid == 0) { KS_TRACE(0) }

    if (tid == 0) {
        for (int i = 0; i < stages; ++i) {
            mbar_init(&ctrl->full[i], 1);
            mbar_init(&ctrl->empty[i], 1);
        }
        for (int i = 0; i < kKsBStages; ++i) {
            mbar_init(&ctrl->full_b[i], 1);
            mbar_init(&ctrl->empty_b[i], 1);
        }
        for (int i = 0; i < kKsAccBufs; ++i) {
            mbar_init(&ctrl->acc_full[i], 2);
            mbar_init(&ctrl->acc_empty[i], 1);
        }
        for (int i = 0; i < kKsHTiles; ++i) {
            mbar_init(&ctrl->h_full[i], 1);
            mbar_init(&ctrl->h_empty[i], 1);
        }
        mbar_init(&ctrl->htab_ready, 1);
        mbar_init(&ctrl->list_ready, 1);
        ctrl->abort_flag = 0;
        ctrl->n_steps = 0;
        ctrl->last_flag = 0;
        ctrl->go_flag = 0;
        fence_mbar_init();
    }
    // TMEM: four buffers of two fp32 accumulators (base, expand) of tn columns; NVFP4 adds 32 scale-factor columns per W slot
    const uint32_t sf_cols_per_slot = FP4 ? 32u : 0u;
    uint32_t tmem_cols = 32;
    while (tmem_cols < (uint32_t)(2 * kKsAccBufs * tn) + sf_cols_per_slot * (uint32_t)stages) tmem_cols *= 2;
    if (warp == 1) {
        tmem_alloc(&ctrl->tmem_base, tmem_cols);
        tmem_relinquish();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tm_w);
        tma_prefetch_desc(&tm_x);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctrl->tmem_base;
    if (tid == 0) { KS_TRACE(1) }

    if (warp == 0) {
        // =========================================================== W producer
        if (lane == 0) {
            const uint64_t pol = l2_policy_evict_first();          // W streams through once: it should not displace the adapters
            const uint32_t wx_bytes = (uint32_t)kKsWTileBytes + (uint32_t)tn * kBlockK + (uint32_t)sf_bytes;
            int git = 0;                                           // slots handed out so far (ring position git % stages)
            bool k1_done = false, ok = true;
            auto load_xq = [&](int st, int k) {
                uint8_t* slot = ring + (size_t)st * stage_bytes;
                tma_load_2d(slot + kKsWTileBytes, &tm_x, &ctrl->full[st], k * kBlockK, 0);
                if (FP4)
                    bulk_load(slot + kKsWTileBytes + tn * kBlockK + kSfSlotBytes, p.xsf + (size_t)k * kSfSlotBytes,
                              (uint32_t)kSfSlotBytes, &ctrl->full[st]);
            };
            // K1's codes: in a chain, the count of quantized positions (the shrink may still be running); else the end of
            // the preceding kernel.  Then the x_q tile of every slot handed out so far.
            auto wait_k1 = [&]() -> bool {
                KS_TRACE(15)
                if (p.xq_ready != nullptr) {
                    const uint64_t t_start = global_timer_ns();
                    bool ready = false;
                    for (uint32_t spin = 0;; ++spin) {
                        if (ld_acquire(p.xq_ready) >= p.M) { ready = true; break; }
                        if ((spin & 31u) == 31u && global_timer_ns() - t_start > limit_ns) break;
                    }
                    if (!ready) { ks_timeout(p, ctrl, 15, git); return false; }
                    fence_proxy_async_all();
                } else {
                    griddep_wait();
                }
                KS_TRACE(4)
                k1_done = true;
                int g = 0;
                for (int i = 0; i < nseg && g < git; ++i) {
                    int tile, ka, ke;
                    span.segment(i, tile, ka, ke);
                    for (int k = ka; k < ke && g < git; ++k, ++g) load_xq(g % stages, k);
                }
                return true;
            };
            for (int i = 0; i < nseg && ok; ++i) {
                int tile, ka, ke;
                span.segment(i, tile, ka, ke);
                const KsTile g = ks_tile(p, tile);
                for (int k = ka; k < ke; ++k) {
                    if (ctrl->abort_flag) { ok = false; break; }
                    if (!k1_done && git >= stages && !wait_k1()) { ok = false; break; }
                    const int st = git % stages;
                    if (git >= stages && !mbar_wait(&ctrl->empty[st], (uint32_t)((git / stages - 1) & 1), limit_ns)) {
                        ks_timeout(p, ctrl, 1, git);
                        ok = false;
                        break;
                    }
                    uint8_t* slot = ring + (size_t)st * stage_bytes;
                    mbar_arrive_expect_tx(&ctrl->full[st], wx_bytes);
                    tma_load_2d_hint(slot, &tm_w, &ctrl->full[st], k * kBlockK, g.slice_off + g.n0_local, pol);
                    if (git == 0) { KS_TRACE(2) }
                    if (FP4)
                        bulk_load(slot + kKsWTileBytes + tn * kBlockK, p.wsf + ((size_t)tile * kb + k) * kSfSlotBytes,
                                  kSfSlotBytes, &ctrl->full[st]);
                    if (k1_done) load_xq(st, k);
                    ++git;
                }
            }
            if (ok && !k1_done) wait_k1();
            KS_TRACE(3)
        }
    } else if (warp == 1) {
        // =========================================================== MMA issuer: base GEMM and expand, two cursors
        // One thread serves both rings, taking whichever has a slot ready: W slots (kind::f8f6f4 / mxf4nvf4 into the base
        // accumulator of the segment's buffer) in k-block order, B slots (kind::f16 into the expand accumulator, against the
        // step's masked H tile) in step order.  Neither cursor waits for the other, so the base GEMM of later segments runs
        // while the expand still waits for K1.  A segment's accumulators are final when both cursors have passed it: each
        // commits its arrival on acc_full.
        if (lane == 0) {
            const uint32_t idesc8 = umma_idesc(0, 0, kTileN, (uint32_t)tn);
            const uint32_t idesc4 = umma_idesc_nvfp4(kTileN, (uint32_t)tn);
            const uint32_t idesc16 = umma_idesc(1, 1, kTileN, (uint32_t)tn);
            const uint32_t row_bytes = (uint32_t)p.rc * 2;                 // 32, 64 or 128
            const uint32_t lt = row_bytes == 128 ? 2u : row_bytes == 64 ? 4u : 6u;
            const uint32_t sbo = row_bytes * 8;
            // base cursor
            int wi = 0, wk = 0, wke = 0, wka = 0, git = 0;
            bool w_open = false, w_fin = nseg == 0;
            // expand cursor
            int bi = 0, bl = 0, bsb = 0, bsa = 0, gb = 0, n_steps = -1;
            bool b_open = false, b_fin = nseg == 0;
            uint64_t t_idle = 0;
            bool ok = true;
            while (ok && !(w_fin && b_fin)) {
                bool progress = false;
                if (ctrl->abort_flag) { ok = false; break; }
                if (!w_fin) {
                    const int buf = wi % kKsAccBufs;
                    if (!w_open) {                                  // enter segment wi: its buffer must have been drained
                        if (wi < kKsAccBufs || mbar_try_wait(&ctrl->acc_empty[buf], (uint32_t)((wi / kKsAccBufs - 1) & 1))) {
                            int tile;
                            span.segment(wi, tile, wka, wke);
                            wk = wka;
                            w_open = true;
                            tc_fence_after();
                            progress = true;
                        }
                    }
                    if (w_open) {
                        const int st = git % stages;
                        if (mbar_try_wait(&ctrl->full[st], (uint32_t)((git / stages) & 1))) {
                            if (git == 0) { KS_TRACE(5) }
                            tc_fence_after();
                            const uint32_t acc0 = tmem_base + (uint32_t)(buf * 2 * tn);
                            const uint32_t wa = smem_u32(ring + (size_t)st * stage_bytes);
                            const uint64_t dw = umma_smem_desc(wa, 1024, 2);
                            const uint64_t dx = umma_smem_desc(wa + kKsWTileBytes, 1024, 2);
                            if (FP4) {
                                const uint32_t sfs = wa + kKsWTileBytes + (uint32_t)tn * kBlockK;
                                const uint32_t sft = tmem_base + (uint32_t)(2 * kKsAccBufs * tn) + (uint32_t)st * sf_cols_per_slot;
#pragma unroll
                                for (int q = 0; q < kBlockK / 32; ++q) {
                                    const uint32_t ta = sft + (uint32_t)q * 4u;
                                    const uint32_t tb = sft + 16u + (uint32_t)q * 4u;
                                    tmem_cp_sf(ta, sf_smem_desc(sfs + (uint32_t)q * 512u));
                                    tmem_cp_sf(tb, sf_smem_desc(sfs + kSfSlotBytes + (uint32_t)q * 512u));
                                    umma_nvfp4(acc0, dw + (uint64_t)(q * 2), dx + (uint64_t)(q * 2), idesc4, ta, tb, (wk > wka || q > 0) ? 1u : 0u);
                                }
                            } else {
#pragma unroll
                                for (int q = 0; q < kBlockK / 32; ++q)
                                    umma_f8f6f4(acc0, dw + (uint64_t)(q * 2), dx + (uint64_t)(q * 2), idesc8, (wk > wka || q > 0) ? 1u : 0u);
                            }
                            umma_commit(&ctrl->empty[st]);
                            ++git;
                            ++wk;
                            progress = true;
                            if (wk == wke) {                        // the base half of segment wi is issued
                                umma_commit(&ctrl->acc_full[buf]);
                                if (wi == nseg - 1) { KS_TRACE(6) }
                                w_open = false;
                                if (++wi == nseg) w_fin = true;
                            }
                        }
                    }
                }
                if (!b_fin) {
                    if (n_steps < 0 && mbar_try_wait(&ctrl->list_ready, 0)) n_steps = ctrl->n_steps;
                    if (n_steps >= 0) {
                        const int buf = bi % kKsAccBufs;
                        if (!b_open) {
                            int tile, ka, ke;
                            span.segment(bi, tile, ka, ke);
                            const int ns = ks_tile(p, tile).has_b ? n_steps : 0;
                            bsa = (int)((long long)ka * ns / kb);
                            bsb = (int)((long long)ke * ns / kb);
                            if (bsb == bsa) {                       // no expand step here: this half is final at once
                                umma_commit(&ctrl->acc_full[buf]);
                                if (++bi == nseg) b_fin = true;
                                progress = true;
                            } else if (bi < kKsAccBufs || mbar_try_wait(&ctrl->acc_empty[buf], (uint32_t)((bi / kKsAccBufs - 1) & 1))) {
                                bl = bsa;
                                b_open = true;
                                tc_fence_after();
                                progress = true;
                            }
                        }
                        if (b_open) {
                            const int st = gb % kKsBStages, hb = gb % kKsHTiles;
                            if (mbar_try_wait(&ctrl->full_b[st], (uint32_t)((gb / kKsBStages) & 1)) &&
                                mbar_try_wait(&ctrl->h_full[hb], (uint32_t)((gb / kKsHTiles) & 1))) {
                                tc_fence_after();
                                const uint32_t acc1 = tmem_base + (uint32_t)(buf * 2 * tn + tn);
                                const uint64_t db = umma_smem_desc(smem_u32(bring + (size_t)st * b_stage_bytes), sbo, lt);
                                const uint64_t dh = umma_smem_desc(smem_u32(hbuf + (size_t)hb * h_bytes), sbo, lt);
                                for (int q = 0; q < p.rc / 16; ++q)
                                    umma_f16(acc1, db + (uint64_t)(q * 2), dh + (uint64_t)(q * 2), idesc16, (bl > bsa || q > 0) ? 1u : 0u);
                                umma_commit(&ctrl->empty_b[st]);
                                umma_commit(&ctrl->h_empty[hb]);
                                ++gb;
                                ++bl;
                                progress = true;
                                if (bl == bsb) {
                                    umma_commit(&ctrl->acc_full[buf]);
                                    b_open = false;
                                    if (++bi == nseg) b_fin = true;
                                }
                            }
                        }
                    }
                }
                if (progress) {
                    t_idle = 0;
                } else {                                            // bounded: no slot of either ring became ready for wait_ms
                    const uint64_t now = global_timer_ns();
                    if (t_idle == 0) t_idle = now;
                    else if (now - t_idle > limit_ns) { ks_timeout(p, ctrl, 5, git * 1000 + gb); ok = false; }
                }
            }
        }
    } else if (warp == 2) {
        // =========================================================== B producer: the expand steps' tiles, in step order
        if (lane == 0) {
            bool ok = mbar_wait(&ctrl->list_ready, 0, limit_ns);
            if (!ok) ks_timeout(p, ctrl, 2, 0);
            const int n_steps = ok ? ctrl->n_steps : 0;
            int gb = 0;
            for (int i = 0; i < nseg && ok; ++i) {
                int tile, ka, ke;
                span.segment(i, tile, ka, ke);
                const KsTile g = ks_tile(p, tile);
                const int ns = g.has_b ? n_steps : 0;
                const int sa = (int)((long long)ka * ns / kb), sb = (int)((long long)ke * ns / kb);
                const CUtensorMap* tmb = (g.s == 0) ? &tm_b0 : (g.s == 1) ? &tm_b1 : (g.s == 2) ? &tm_b2 : &tm_b3;
                for (int li = sa; li < sb; ++li, ++gb) {
                    if (ctrl->abort_flag) { ok = false; break; }
                    const int st = gb % kKsBStages;
                    if (gb >= kKsBStages && !mbar_wait(&ctrl->empty_b[st], (uint32_t)((gb / kKsBStages - 1) & 1), limit_ns)) {
                        ks_timeout(p, ctrl, 3, gb);
                        ok = false;
                        break;
                    }
                    const KsStep e = ctrl->steps[li];
                    if (gb == 0) { KS_TRACE(9) }
                    mbar_arrive_expect_tx(&ctrl->full_b[st], (uint32_t)b_bytes);
                    tma_load_2d(bring + (size_t)st * b_stage_bytes, tmb, &ctrl->full_b[st], e.chunk * p.rc,
                                e.lora * p.b_rows[g.s] + (g.n0_local - p.b_row0[g.s]));
                }
            }
        }
    } else if (warp == 3) {
        // =========================================================== masked H tiles of the expand steps, in step order
        // Step li multiplies B_l's tile with H = the h rows of tenant l's tokens, zero elsewhere.  The H tiles start as
        // zeros; per step the warp clears the rows the tile's previous step filled and copies this step's rows out of the
        // slice's h table.
        for (int i = lane; i < kKsHTiles * h_bytes / 16; i += 32) reinterpret_cast<uint4*>(hbuf)[i] = make_uint4(0u, 0u, 0u, 0u);
        bool ok = mbar_wait(&ctrl->list_ready, 0, limit_ns);
        const int n_steps = ok ? ctrl->n_steps : 0;
        if (ok && n_steps > 0) ok = mbar_wait(&ctrl->htab_ready, 0, limit_ns);
        if (!ok && lane == 0) ks_timeout(p, ctrl, 13, 0);
        const int row_bytes = p.rc * 2, cpr = row_bytes / 16;
        const uint32_t swz = (uint32_t)cpr - 1u;
        int gb = 0;
        for (int i = 0; i < nseg && ok; ++i) {
            int tile, ka, ke;
            span.segment(i, tile, ka, ke);
            const KsTile g = ks_tile(p, tile);
            const int ns = g.has_b ? n_steps : 0;
            const int sa = (int)((long long)ka * ns / kb), sb = (int)((long long)ke * ns / kb);
            const uint8_t* tab = htab + (size_t)g.s * htab_bytes;
            for (int li = sa; li < sb; ++li, ++gb) {
                const int hb = gb % kKsHTiles, hu = gb / kKsHTiles;
                if (ctrl->abort_flag) { ok = false; break; }
                uint8_t* tile_h = hbuf + (size_t)hb * h_bytes;
                if (hu > 0) {
                    if (!mbar_wait(&ctrl->h_empty[hb], (uint32_t)((hu - 1) & 1), limit_ns)) {
                        if (lane == 0) ks_timeout(p, ctrl, 10, li);
                        ok = false;
                        break;
                    }
                    const KsStep o = ctrl->steps[ctrl->h_prev[hb]];
                    for (int c = lane; c < ((int)o.hi - (int)o.lo) * cpr; c += 32) {
                        uint32_t off = (uint32_t)((int)o.lo + c / cpr) * (uint32_t)row_bytes + (uint32_t)(c % cpr) * 16u;
                        off ^= ((off >> 7) & swz) << 4;
                        *reinterpret_cast<uint4*>(tile_h + off) = make_uint4(0u, 0u, 0u, 0u);
                    }
                    __syncwarp();
                }
                const KsStep e = ctrl->steps[li];
                for (int c = lane; c < ((int)e.hi - (int)e.lo) * cpr; c += 32) {
                    const int row = (int)e.lo + c / cpr, c16 = c % cpr;
                    const uint4 v = *reinterpret_cast<const uint4*>(tab + ((size_t)row * p.R + (size_t)e.chunk * p.rc) * 2 + (size_t)c16 * 16);
                    uint32_t off = (uint32_t)row * (uint32_t)row_bytes + (uint32_t)c16 * 16u;
                    off ^= ((off >> 7) & swz) << 4;
                    *reinterpret_cast<uint4*>(tile_h + off) = v;
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    ctrl->h_prev[hb] = li;
                    mbar_arrive(&ctrl->h_full[hb]);
                }
                __syncwarp();
            }
        }
    } else if (warp >= 4) {
        // =========================================================== segment index, h tables, expand, epilogues
        const int te = tid - 128;
        for (int i = lane; i <= p.L; i += 32) prefetch_l1(p.meta.seg_start + i);
        int srt_v = 0;
        if (te < tn && te < p.M) srt_v = p.meta.srt[te];
        int n_all, n_ad;
        segment_totals(p.meta, p.L, lane, n_all, n_ad);
        n_all = min(n_all, p.M);
        if (te < tn) {
            int row = te < p.M ? te : -1;
            if (n_ad > 0 && te < n_all) row = srt_v < 0 ? 0 : (srt_v > p.M - 1 ? p.M - 1 : srt_v);
            ctrl->rowmap[te] = row;
        }
        if (warp == 4) {
            int total = 0;
            if (n_ad > 0) {
                for (int base = 0; base <= p.L; base += 32) {
                    const int i = base + lane;
                    int lora = -1, lo = 0, hi = 0;
                    if (i <= p.L) {
                        lora = p.meta.seg_ids[i];
                        const int cnt = p.meta.seg_n[i], sst = p.meta.seg_start[i];
                        lo = max(sst, 0);
                        hi = min(min(sst + cnt, tn), n_all);
                        if (cnt <= 0 || sst < 0) lora = -1;
                    }
                    const bool okseg = lora >= 0 && lora < p.L && lo < hi;
                    const uint32_t mask = __ballot_sync(0xffffffffu, okseg);
                    if (okseg) {
                        const int idx = total / n_chunks + __popc(mask & ((1u << lane) - 1u));
                        for (int c = 0; c < n_chunks; ++c) {
                            const int e = idx * n_chunks + c;
                            if (e < kKsMaxSteps) ctrl->steps[e] = KsStep{(uint16_t)lora, (uint16_t)c, (uint16_t)lo, (uint16_t)hi};
                        }
                    }
                    total += __popc(mask) * n_chunks;
                }
            }
            if (lane == 0) ctrl->n_steps = min(total, kKsMaxSteps);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (te == 0) { mbar_arrive(&ctrl->list_ready); KS_TRACE(7) }
        const int n_steps = ctrl->n_steps;

        griddep_wait();                                       // K1's s_x and shrink partials from here on
        if (te == 0) { KS_TRACE(8) }
        if (te < tn) ctrl->sx[te] = FP4 ? 1.0f : (te < p.M ? __ldcg(p.sx + te) : 0.0f);

        // ---- h tables of the slices this CTA's segments touch: bf16( sum over K1's splits, in split order ), once
        if (n_steps > 0 && nseg > 0) {
            int s_lo = p.S, s_hi = -1;                        // slices of this CTA's tiles
            for (int i = 0; i < nseg; ++i) {
                int tile, ka, ke;
                span.segment(i, tile, ka, ke);
                const int sl = ks_tile(p, tile).s;
                s_lo = min(s_lo, sl);
                s_hi = max(s_hi, sl);
            }
            const int groups = p.R / 8;
            const size_t jstride = (size_t)p.S * p.max_m * p.R;
            for (int s = s_lo; s <= s_hi; ++s) {
                uint8_t* tab = htab + (size_t)s * htab_bytes;
                for (int idx = te; idx < tn * groups; idx += 128) {
                    const int row = idx / groups, g8 = idx % groups;
                    float acc[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) acc[u] = 0.0f;
                    if (row < n_all) {
                        const float* src0 = p.hp + ((size_t)s * p.max_m + (size_t)row) * p.R + (size_t)g8 * 8;
                        for (int j1 = 0; j1 < p.split1; j1 += 4) {
                            float4 v[4][2];
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                if (j1 + q < p.split1) {
                                    const float4* src = reinterpret_cast<const float4*>(src0 + (size_t)(j1 + q) * jstride);
                                    v[q][0] = __ldcg(src);
                                    v[q][1] = __ldcg(src + 1);
                                } else {
                                    v[q][0] = v[q][1] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                                }
                            }
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                acc[0] += v[q][0].x; acc[1] += v[q][0].y; acc[2] += v[q][0].z; acc[3] += v[q][0].w;
                                acc[4] += v[q][1].x; acc[5] += v[q][1].y; acc[6] += v[q][1].z; acc[7] += v[q][1].w;
                            }
                        }
                    }
                    __nv_bfloat162 b0 = __floats2bfloat162_rn(acc[0], acc[1]);
                    __nv_bfloat162 b1 = __floats2bfloat162_rn(acc[2], acc[3]);
                    __nv_bfloat162 b2 = __floats2bfloat162_rn(acc[4], acc[5]);
                    __nv_bfloat162 b3 = __floats2bfloat162_rn(acc[6], acc[7]);
                    uint4 out;
                    out.x = *reinterpret_cast<uint32_t*>(&b0);
                    out.y = *reinterpret_cast<uint32_t*>(&b1);
                    out.z = *reinterpret_cast<uint32_t*>(&b2);
                    out.w = *reinterpret_cast<uint32_t*>(&b3);
                    *reinterpret_cast<uint4*>(tab + ((size_t)row * p.R + (size_t)g8 * 8) * 2) = out;
                }
            }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");         // h tables, sx and rowmap visible to warps 4-7

        if (te == 0) mbar_arrive(&ctrl->htab_ready);

        // ---- per segment: epilogue (+ fix-up of a tile shared with other CTAs)
        const int q4 = warp & 3;
        const int n_local = q4 * 32 + lane;                    // the output feature (TMEM lane) this thread owns
        const uint32_t lane_addr = (uint32_t)(q4 * 32) << 16;
        const float s_w = FP4 ? __ldg(p.alpha) : __ldg(p.s_w);
        const long long units = (long long)(p.n_tiles - span.rem0) * kb;      // the remainder tiles' k-blocks
        for (int i = 0; i < nseg; ++i) {
            int tile, ka, ke;
            span.segment(i, tile, ka, ke);
            const KsTile g = ks_tile(p, tile);
            const int buf = i % kKsAccBufs;
            const int ns = g.has_b ? n_steps : 0;
            const bool has_lora = (int)((long long)ke * ns / kb) > (int)((long long)ka * ns / kb);
            if (te == 0) {
                int go = ctrl->abort_flag ? 0 : 1;
                if (go && !mbar_wait(&ctrl->acc_full[buf], (uint32_t)((i / kKsAccBufs) & 1), limit_ns)) {
                    ks_timeout(p, ctrl, 11, i);
                    go = 0;
                }
                ctrl->go_flag = go;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (!ctrl->go_flag) break;
            tc_fence_after();
            if (te == 0 && i == 0) { KS_TRACE(11) }
            const bool whole = ka == 0 && ke == kb;
            const bool n_ok = g.n0_local + n_local < g.n_s;
            const int n_glob = g.slice_off + g.n0_local + n_local;
            const uint32_t acc0 = tmem_base + (uint32_t)(buf * 2 * tn) + lane_addr, acc1 = acc0 + (uint32_t)tn;
            float* part = p.part + (size_t)(2 * cta + (i > 0 ? 1 : 0)) * (size_t)tn * kTileN;
            for (int c0 = 0; c0 < tn; c0 += 16) {
                uint32_t r0[16], r1[16];
                tmem_ld16(acc0 + (uint32_t)c0, r0);
                if (has_lora) tmem_ld16(acc1 + (uint32_t)c0, r1);
                tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    float v = __uint_as_float(r0[c]) * (ctrl->sx[c0 + c] * s_w);
                    if (has_lora) v += __uint_as_float(r1[c]);
                    if (whole) {
                        const int row = ctrl->rowmap[c0 + c];
                        if (row >= 0 && n_ok) p.y[(int64_t)row * p.ldy + n_glob] = __float2bfloat16_rn(v);
                    } else {
                        part[(size_t)(c0 + c) * kTileN + n_local] = v;
                    }
                }
            }
            tc_fence_before();
            asm volatile("bar.sync 1, 128;" ::: "memory");    // all 128 threads have drained the buffer / written their partials
            if (te == 0) mbar_arrive(&ctrl->acc_empty[buf]);
            if (whole) continue;
            // the tile is shared: CTAs c_lo .. c_hi hold parts of it
            const int rt = tile - span.rem0;                  // (a shared tile is a remainder tile)
            const int c_lo = ks_owner(units, G, (long long)rt * kb), c_hi = ks_owner(units, G, (long long)rt * kb + kb - 1);
            if (te == 0) {
                int holders = 0;                              // (with fewer remainder k-blocks than CTAs some shares are empty)
                for (int cc = c_lo; cc <= c_hi; ++cc)
                    holders += KsSpan::start_of(units, G, cc + 1) > KsSpan::start_of(units, G, cc) ? 1 : 0;
                int old;                                      // release our partial, acquire the others'
                asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(old) : "l"(p.counters + tile) : "memory");
                ctrl->last_flag = (old == holders - 1) ? 1 : 0;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (ctrl->last_flag) {
                // Thread = 4 output features x every 4th token; 8 tokens' loads in flight per contributor.
                const int tg = te >> 5, n4 = (te & 31) * 4;
                for (int cb = 0; cb < tn; cb += 32) {
                    float4 acc[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) acc[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    for (int cc = c_lo; cc <= c_hi; ++cc) {
                        if (KsSpan::start_of(units, G, cc + 1) <= KsSpan::start_of(units, G, cc)) continue;   // an empty share
                        const int first_tile = (int)(KsSpan::start_of(units, G, cc) / kb);
                        const float* pb = p.part + (size_t)(2 * cc + (first_tile == rt ? 0 : 1)) * (size_t)tn * kTileN;
#pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            const int c = cb + u * 4 + tg;
                            if (c < tn) {
                                const float4 v = __ldcg(reinterpret_cast<const float4*>(pb + (size_t)c * kTileN + n4));
                                acc[u].x += v.x; acc[u].y += v.y; acc[u].z += v.z; acc[u].w += v.w;
                            }
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int c = cb + u * 4 + tg;
                        const int row = c < tn ? ctrl->rowmap[c] : -1;
                        if (row >= 0) {
                            __nv_bfloat16* yr = p.y + (int64_t)row * p.ldy + g.slice_off + g.n0_local + n4;
                            const int left = g.n_s - (g.n0_local + n4);
                            if (left >= 4 && (((uintptr_t)yr) & 7) == 0) {
                                __nv_bfloat162 lo2 = __floats2bfloat162_rn(acc[u].x, acc[u].y), hi2 = __floats2bfloat162_rn(acc[u].z, acc[u].w);
                                *reinterpret_cast<uint2*>(yr) = make_uint2(*reinterpret_cast<uint32_t*>(&lo2), *reinterpret_cast<uint32_t*>(&hi2));
                            } else {
                                if (left > 0) yr[0] = __float2bfloat16_rn(acc[u].x);
                                if (left > 1) yr[1] = __float2bfloat16_rn(acc[u].y);
                                if (left > 2) yr[2] = __float2bfloat16_rn(acc[u].z);
                                if (left > 3) yr[3] = __float2bfloat16_rn(acc[u].w);
                            }
                        }
                    }
                }
                if (te == 0) p.counters[tile] = 0;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");    // last_flag is rewritten by the next shared segment
        }
    }

    // ---- teardown: nobody leaves while TMEM is in use or copies may still land in this CTA's shared memory
    if (ctrl->abort_flag) __nanosleep(200000);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, tmem_cols);
    }
    if (p.chain_done != nullptr && tid == 0) {       // the last CTA of a chained launch clears K1's count for the next call
        if (atomicAdd(p.chain_done, 1) == G - 1) {
            *const_cast<volatile int32_t*>(p.xq_ready) = 0;
            *const_cast<volatile int32_t*>(p.chain_done) = 0;
        }
    }
    if (tid == 0) { KS_TRACE(14) }
}

int k2_stream_h_tiles(int tn) { (void)tn; return kKsHTiles; }

size_t k2_stream_smem_bytes(int tn, int stages, int rc, int R, int S, int fp4) {
    const size_t sf = fp4 ? 2 * (size_t)kSfSlotBytes : 0;
    const size_t aux = (size_t)kKsBStages * align_up((size_t)kTileN * rc * 2, 1024) + (size_t)S * align_up((size_t)tn * R * 2, 1024) +
                       (size_t)kKsHTiles * align_up((size_t)tn * rc * 2, 1024);
    return 1024 + (size_t)stages * (kKsWTileBytes + (size_t)tn * kBlockK + sf) + aux + kKsCtrlBytes;
}

template <bool FP4>
static cudaError_t launch_k2_stream_impl(const K2Params& p, const CUtensorMap& tm_w, const CUtensorMap& tm_x, const CUtensorMap* tm_b,
                                         int grid, size_t smem, int pdl, cudaStream_t stream) {
    static std::atomic<unsigned long long> configured{0};     // bit per device: the shared-memory opt-in was made
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || !(configured.load() & (1ull << dev))) {
        cudaFuncAttributes fa;
        e = cudaFuncGetAttributes(&fa, k2_stream_kernel<FP4>);
        if (e != cudaSuccess) return e;
        e = cudaFuncSetAttribute(k2_stream_kernel<FP4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - (int)fa.sharedSizeBytes);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured.fetch_or(1ull << dev);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kKsThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, k2_stream_kernel<FP4>, p, tm_w, tm_x, tm_b[0], tm_b[1], tm_b[2], tm_b[3]);
}

cudaError_t launch_k2_stream(const K2Params& p, const CUtensorMap& tm_w, const CUtensorMap& tm_x, const CUtensorMap* tm_b,
                             int grid, size_t smem, int fp4, int pdl, cudaStream_t stream) {
    return fp4 ? launch_k2_stream_impl<true>(p, tm_w, tm_x, tm_b, grid, smem, pdl, stream)
               : launch_k2_stream_impl<false>(p, tm_w, tm_x, tm_b, grid, smem, pdl, stream);
}

}  // namespace ob
