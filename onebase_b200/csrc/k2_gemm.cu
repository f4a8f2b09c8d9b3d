// K2: y = bf16( scale * (x_q W_q^T) + sum over tenants of h B^T ) for an FP8 (e4m3, scale = s_x * s_w) or NVFP4 (e2m1 with
// ue4m3 block scales, scale = alpha) base, one CTA per (128 output features,
// token tile, K split), two CTAs per SM, hand-written for sm_100a:
//
//   swap-AB orientation -- the 128 rows of the W tile sit on the MMA's M side, the tokens (16..256 per tile, adapter-
//   sorted positions written by K1) on its N side, so a decode batch of 1..32 tokens wastes no tensor-core rows and the
//   kernel is a pure stream of W (and the tenants' B) from HBM.
//
//   warp 0   the TMA producer.  One ring of shared-memory slots carries W tiles [128 x 128 B] (128-byte swizzle, L2
//            evict-first) each with its x_q tile [tokens x 128 B], and the expand steps' B tiles [128 x rank chunk]
//            (bf16), interleaved (SlotWalk) so that the tenants' B streams in between the W tiles instead of after them.
//            W and B do not depend on K1: under programmatic dependent launch the ring fills while K1 still runs; the
//            x_q tiles are requested after griddepcontrol.wait.
//   warp 1   allocates TMEM and issues tcgen05.mma: kind::f8f6f4 (e4m3 x e4m3, fp32) into accumulator 0 for the base
//            GEMM -- or, for an NVFP4 base, kind::mxf4nvf4.block_scale.scale_vec::4X with both operands' ue4m3 block
//            scales copied from the slot into TMEM by tcgen05.cp -- and kind::f16 (bf16) into accumulator 1 for each
//            expand step; tcgen05.commit releases ring slots.
//   warp 2   (decode tiles, <= 32 tokens) keeps masked H tiles ready: H of a step = the h rows of that tenant's tokens,
//            zero elsewhere, in the UMMA layout; it only rewrites the one or two rows that change between steps.
//   warps 4-7  read vLLM's segment index, list the (segment, rank chunk) expand steps of this tile; after K1 they sum
//            its split-K partials once into a bf16 h table in shared memory (decode tiles) or build the masked H tiles
//            themselves (larger tiles); finally the epilogue: tcgen05.ld both accumulators, s_x*s_w*acc0 + acc1, bf16
//            rows scattered back through the sort.  With split-K > 1 they write fp32 partials instead and the last CTA
//            to arrive adds them in split order (deterministic) and resets the arrival counter.
//
// What it computes is lowbit_lora/kernels/fp8_lora_vllm.py:123-284 (`_gemm_vllm`, BASE=True) and the decode-chain GEMM
// lowbit_lora/kernels/fp8_lora_pdl.py:324-495; positions, padding and stale metadata follow fp8_lora_vllm.py:147-163.
// Every wait is bounded (wait_ms); a wait that runs out records where in the workspace status words and the CTA leaves
// without storing.
#include "k1_device.cuh"

namespace ob {

constexpr int kK2Threads = 256;
constexpr int kWTileBytes = kTileN * kBlockK;   // 16 KB
constexpr int kCtrlBytes = 8192;

struct LoraStep {
    uint16_t lora;    // adapter slot
    uint16_t chunk;   // rank chunk index
    uint16_t lo, hi;  // tile-local token rows [lo, hi) of the segment
};

struct K2Ctrl {
    uint64_t full_w[12];
    uint64_t full_b[12];   // B tiles of the expand steps: own barriers, so their consumers need not follow the base phases
    uint64_t empty[12];
    uint64_t empty_b[12];  // release of a slot that held a B tile (4 arrivals: one per expanding warp; 1 from the MMA warp)
    uint64_t h_full[8];
    uint64_t h_empty[8];
    uint64_t htab_ready;
    uint64_t list_ready;
    uint64_t acc_full;
    uint32_t tmem_base;
    volatile int abort_flag;
    volatile int b_grant; // stored adapters: expand steps whose ring slot the producer has acquired for warps 4-7 to fill
    int n_steps;          // expand steps of this CTA
    int last_flag;
    int go_flag;          // the epilogue warps' shared continue / stop decision
    int claim;            // fused: the position the four epilogue warps claimed together
    int lora_pos[32];     // fused: adapter slot of each of the tile's positions (-1: none)
    float sx[256];
    int rowmap[256];
    LoraStep steps[kMaxLoraIters];
    uint64_t code_full[12];   // stored adapters: the step's codes and scales have landed in the slot
};
static_assert(sizeof(K2Ctrl) <= kCtrlBytes, "control block too large");

// The ring's slot sequence, identical in every role.  Slot `it` (ring position it % stages) holds either the next W
// k-block together with its x_q tile, or the next expand step's B tile.  The first `lead` slots (one ring fill) are W
// tiles whatever the batch, so the stream starts without waiting for the segment index; after them the n_steps B tiles
// are spread evenly among the remaining W tiles (an error-accumulating line walk), so that the tenants' B streams in
// between the W tiles and both kinds run out together.  The number of expand steps is needed from slot `lead` on.
struct SlotWalk {
    int it = 0, k = 0, li = 0;
    int lead;   // slots at the start that are W tiles regardless
    int acc = 0;
    __device__ explicit SlotWalk(int lead_slots) : lead(lead_slots) {}
    __device__ bool needs_list(int n_base) const { return it >= lead || k >= n_base; }
    __device__ bool is_b(int n_base, int n_steps) const {
        if (li >= n_steps) return false;
        if (k >= n_base) return true;
        if (it < lead) return false;
        const int total = (n_base > lead ? n_base - lead : 0) + n_steps;
        return acc + n_steps >= total;
    }
    __device__ bool done(int n_base, int n_steps) const { return k >= n_base && li >= n_steps; }
    __device__ void advance(bool was_b, int n_base, int n_steps) {
        if (it >= lead && k < n_base && li < n_steps) {      // the line walk only runs while both kinds remain
            acc += n_steps;
            if (was_b) acc -= (n_base > lead ? n_base - lead : 0) + n_steps;
        }
        ++it;
        if (was_b) ++li; else ++k;
    }
};

// Per-slot bookkeeping of the ring, identical in every role that hands slots out: which barrier frees slot `st` for reuse
// (the one of its previous tenant: `empty` after a W tile, `empty_b` after a B tile) and with which phase parity.  Every
// role that calls acquire() for EVERY slot, in order, stays in step whether or not it actually waits.
struct RingBook {
    uint32_t par_w = 0, par_b = 0, last_b = 0;
    // returns 0: slot never used; 1: wait `empty[st]`; 2: wait `empty_b[st]`; the parity to wait for goes to `parity`
    __device__ int acquire(int it, int st, int stages, bool is_b, uint32_t& parity) {
        const uint32_t bit = 1u << st;
        int kind = 0;
        if (it >= stages) {
            if (last_b & bit) {
                kind = 2;
                parity = (par_b >> st) & 1u;
                par_b ^= bit;
            } else {
                kind = 1;
                parity = (par_w >> st) & 1u;
                par_w ^= bit;
            }
        }
        if (is_b) last_b |= bit; else last_b &= ~bit;
        return kind;
    }
};

__device__ __forceinline__ void record_timeout(const K2Params& p, K2Ctrl* c, int where, int it) {
    c->abort_flag = 1;
    if (atomicCAS(p.status, OB_DEV_OK, OB_DEV_WAIT_TIMEOUT) == OB_DEV_OK) {
        p.status[1] = where;
        p.status[2] = blockIdx.x;
        p.status[3] = blockIdx.y;
        p.status[4] = blockIdx.z;
        p.status[5] = it;
    }
}

// Timeline stamp `ev` of this CTA (profiling only; off unless a trace buffer is set).
#define OB_TRACE(ev)                                                                                      \
    if (p.trace != nullptr && trace_cta < p.trace_ctas) p.trace[trace_cta * OB_TRACE_EVENTS + (ev)] = global_timer_ns();

#define OB_WAIT(bar, parity, where, it)                   \
    if (!mbar_wait((bar), (parity), limit_ns)) {          \
        record_timeout(p, ctrl, (where), (it));           \
        break;                                            \
    }

__device__ __forceinline__ float k2_e2m1_value(uint32_t code) {
    const uint32_t mag = code & 7u;
    float v = __uint_as_float(0x3F000000u + (mag << 22));
    v = mag == 0 ? 0.0f : (mag == 1 ? 0.5f : v);
    return (code & 8u) ? -v : v;
}

__device__ __forceinline__ float k2_e4m3_value(uint32_t code) {
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((uint16_t)code));
    return __half2float(__ushort_as_half((unsigned short)(h2 & 0xFFFFu)));
}

// The value K2 stores for an accumulated fp32 result: bf16(acc), or with a residual stream bf16(bf16(acc) + residual): the
// "x + residual" of vLLM's fused add + RMSNorm (layernorm.py, forward_native: fp32 sum of the two bf16 tensors).
template <bool EXTRA>
__device__ __forceinline__ __nv_bfloat16 k2_out(const K2Params& p, float v, int64_t row, int64_t col) {
    const __nv_bfloat16 y = __float2bfloat16_rn(v);
    if (!EXTRA || p.residual == nullptr) return y;
    return __float2bfloat16_rn(__bfloat162float(y) + __bfloat162float(p.residual[row * p.ldr + col]));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&b);
}

// Expand step e's B tile [128 rows x rank chunk] from a stored-format adapter, in two halves so that a step's codes can
// be requested one step ahead: load_b_codes() fetches thread `te`'s row of codes and scales (output row n0_local + te) into
// registers, store_b_tile() dequantizes them to bf16 with the scales folded in (one rounding) into the ring slot in the
// UMMA layout.  FP8-stored: bf16(code * sb[l, n]); NVFP4-stored: bf16(e2m1 * block scale * bg[s, l])
// (lowbit_lora/kernels/fp8_lora_vllm.py:249-278).  Rows past the slice's width are zero.  The rank chunk is at most 64:
// four groups of 16 codes.
struct BCodes {
    uint4 c[4];     // FP8: 16 codes each; NVFP4: .x/.y = 16 codes, .z = the block's scale byte
    float sc;       // FP8: the row's scale; NVFP4: the matrix's global scale
};

__device__ __forceinline__ void load_b_codes(const K2Params& p, const LoraStep& e, int s, int n_s, int n0_local, int te, BCodes& r) {
    const int n = n0_local + te;
    const bool ok = n < n_s;
    const size_t row = (size_t)e.lora * n_s + (size_t)(ok ? n : 0);
    const int groups = p.rc / 16;
    if (p.lora_fmt == kLoraFp8) {
        const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(p.b[s]) + row * p.R + (size_t)e.chunk * p.rc);
        r.sc = ok ? __ldg(static_cast<const float*>(p.sb[s]) + row) : 0.0f;
#pragma unroll
        for (int g = 0; g < 4; ++g) r.c[g] = (ok && g < groups) ? __ldg(src + g) : make_uint4(0u, 0u, 0u, 0u);
    } else {
        const uint2* src = reinterpret_cast<const uint2*>(static_cast<const uint8_t*>(p.b[s]) + (row * p.R + (size_t)e.chunk * p.rc) / 2);
        const uint8_t* sfp = static_cast<const uint8_t*>(p.sb[s]) + row * (p.R / 16) + (size_t)e.chunk * p.rc / 16;
        r.sc = __ldg(p.bg + (size_t)s * p.L + e.lora);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const bool in = ok && g < groups;
            const uint2 c = in ? __ldg(src + g) : make_uint2(0u, 0u);
            r.c[g] = make_uint4(c.x, c.y, in ? (uint32_t)__ldg(sfp + g) : 0u, 0u);
        }
    }
}

// The same row of codes and scales out of the ring slot, where the producer's bulk copies put them: codes of row r at
// slot + 8192 + r * (R or R/2) bytes, scales (fp32 per row, or one ue4m3 byte per 16 elements) at slot + 16384.  (The rank
// chunk is the whole rank in this form.)
__device__ __forceinline__ void load_b_codes_smem(const K2Params& p, const LoraStep& e, int s, int n_s, int n0_local, int te,
                                                  const uint8_t* slot, BCodes& r) {
    const bool ok = n0_local + te < n_s;
    const int groups = p.rc / 16;
    if (p.lora_fmt == kLoraFp8) {
        const uint4* src = reinterpret_cast<const uint4*>(slot + 8192 + (size_t)te * p.R);
        r.sc = ok ? *reinterpret_cast<const float*>(slot + 16384 + (size_t)te * 4) : 0.0f;
#pragma unroll
        for (int g = 0; g < 4; ++g) r.c[g] = (ok && g < groups) ? src[g] : make_uint4(0u, 0u, 0u, 0u);
    } else {
        const uint2* src = reinterpret_cast<const uint2*>(slot + 8192 + (size_t)te * (p.R / 2));
        const uint8_t* sfp = slot + 16384 + (size_t)te * (p.R / 16);
        r.sc = __ldg(p.bg + (size_t)s * p.L + e.lora);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const bool in = ok && g < groups;
            const uint2 c = in ? src[g] : make_uint2(0u, 0u);
            r.c[g] = make_uint4(c.x, c.y, in ? (uint32_t)sfp[g] : 0u, 0u);
        }
    }
}

// Four e2m1 codes (the nibbles of the low 16 bits of w4) -> four bf16 values of bf16(value * block scale * global), through
// byte tables of the block's eight magnitudes: two byte permutes pick the low and the high bytes of the four results,
// two more interleave them, the codes' sign bits are ORed in.
__device__ __forceinline__ void e2m1x4_lookup(uint32_t w4, const uint32_t (&lo)[2], const uint32_t (&hi)[2], uint32_t& out01, uint32_t& out23) {
    const uint32_t sel = w4 & 0x7777u;
    const uint32_t L = __byte_perm(lo[0], lo[1], sel), H = __byte_perm(hi[0], hi[1], sel);
    out01 = __byte_perm(L, H, 0x5140u) | ((w4 & 0x8u) << 12) | ((w4 & 0x80u) << 24);
    out23 = __byte_perm(L, H, 0x7362u) | ((w4 & 0x800u) << 4) | ((w4 & 0x8000u) << 16);
}

__device__ __forceinline__ void store_b_tile(const K2Params& p, const BCodes& r, uint8_t* tile, int te, int row_bytes, uint32_t swz) {
    const uint32_t row_off = (uint32_t)te * (uint32_t)row_bytes;
    const int groups = p.rc / 16;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        if (g < groups) {
            uint32_t o[8];
            if (p.lora_fmt == kLoraFp8) {                      // 16 codes -> two 16-byte chunks of bf16
                const uint32_t w[4] = {r.c[g].x, r.c[g].y, r.c[g].z, r.c[g].w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    o[2 * q] = pack_bf16x2(k2_e4m3_value(w[q] & 0xFFu) * r.sc, k2_e4m3_value((w[q] >> 8) & 0xFFu) * r.sc);
                    o[2 * q + 1] = pack_bf16x2(k2_e4m3_value((w[q] >> 16) & 0xFFu) * r.sc, k2_e4m3_value(w[q] >> 24) * r.sc);
                }
            } else {                                           // one block of 16 codes (8 bytes) + its scale
                const float sf = k2_e4m3_value(r.c[g].z);      // (0 for rows past the slice's width: their codes are 0 too)
                // the block's eight magnitudes bf16((value * block scale) * global) -- the reference's order of the two
                // products, one fp32 rounding -- as byte tables
                const uint32_t m01 = pack_bf16x2(0.0f, (0.5f * sf) * r.sc), m23 = pack_bf16x2((1.0f * sf) * r.sc, (1.5f * sf) * r.sc);
                const uint32_t m45 = pack_bf16x2((2.0f * sf) * r.sc, (3.0f * sf) * r.sc), m67 = pack_bf16x2((4.0f * sf) * r.sc, (6.0f * sf) * r.sc);
                const uint32_t lo[2] = {__byte_perm(m01, m23, 0x6420u), __byte_perm(m45, m67, 0x6420u)};
                const uint32_t hi[2] = {__byte_perm(m01, m23, 0x7531u), __byte_perm(m45, m67, 0x7531u)};
                e2m1x4_lookup(r.c[g].x, lo, hi, o[0], o[1]);   // element 2q in the low nibble of byte q: nibble order = element order
                e2m1x4_lookup(r.c[g].x >> 16, lo, hi, o[2], o[3]);
                e2m1x4_lookup(r.c[g].y, lo, hi, o[4], o[5]);
                e2m1x4_lookup(r.c[g].y >> 16, lo, hi, o[6], o[7]);
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t off = row_off + (uint32_t)(2 * g + h) * 16u;
                off ^= ((off >> 7) & swz) << 4;
                *reinterpret_cast<uint4*>(tile + off) = make_uint4(o[4 * h], o[4 * h + 1], o[4 * h + 2], o[4 * h + 3]);
            }
        }
    }
}

// ---- all-reduce fused into the epilogue (see K2Params.ar_*).  System-scope flag and data accesses as in allreduce.cu.
__device__ __forceinline__ void ar_st_release_sys(int32_t* p, int32_t v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ar_ld_acquire_sys(const int32_t* p) {
    int32_t v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ar_ld_peer16(const void* p) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// Called by the 128 epilogue threads of the CTA that holds the FINISHED values of output tile `tile` once they are staged
// (bf16, [token row][N]) in this rank's communication buffer: announce the tile to every rank, wait (bounded) for every
// rank's copy of it, add the copies in rank order with fp32 accumulation, store y.  Same arithmetic as the stand-alone
// all-reduce kernel, so the results are bitwise equal to "K2, then ob_allreduce".
__device__ void ar_finish_tile(const K2Params& p, K2Ctrl* ctrl, int te, int tile, int32_t epoch, int tn, int slice_off, int n0_local,
                               int n_s, uint64_t limit_ns) {
    uint8_t* own = p.ar_bufs[p.ar_rank];
    const size_t data_off = (size_t)kArStateBytes + (size_t)(epoch & 1) * (size_t)p.ar_slot_bytes;
    asm volatile("bar.sync 1, 128;" ::: "memory");            // every thread's staged values precede the announcement
    if (te < p.ar_world) {
        __threadfence();
        ar_st_release_sys(reinterpret_cast<int32_t*>(p.ar_bufs[te] + kArTileFlagsOff) + p.ar_rank * kArMaxTiles + tile, epoch);
        const int32_t* flag = reinterpret_cast<const int32_t*>(own + kArTileFlagsOff) + te * kArMaxTiles + tile;
        const uint64_t t0 = global_timer_ns();
        bool ok = false;
        for (uint32_t spin = 0;; ++spin) {
            if (ar_ld_acquire_sys(flag) - epoch >= 0) { ok = true; break; }
            if ((spin & 63u) == 63u && global_timer_ns() - t0 > limit_ns) break;
        }
        if (!ok) record_timeout(p, ctrl, 20 + te, tile);     // 20 + the rank whose tile did not arrive
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (ctrl->abort_flag) return;
    for (int idx = te; idx < tn * (kTileN / 8); idx += 128) {
        const int c = idx / (kTileN / 8), n8 = (idx % (kTileN / 8)) * 8;
        const int row = ctrl->rowmap[c];
        const int left = n_s - (n0_local + n8);
        if (row < 0 || left <= 0) continue;
        const size_t off = data_off + ((size_t)row * p.N + (size_t)(slice_off + n0_local + n8)) * 2;
        uint4 v[OB_MAX_RANKS];
#pragma unroll
        for (int r = 0; r < OB_MAX_RANKS; ++r)
            if (r < p.ar_world) v[r] = ar_ld_peer16(p.ar_bufs[r] + off);
        float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int r = 0; r < OB_MAX_RANKS; ++r)
            if (r < p.ar_world) {
                acc[0] += bf16_lo(v[r].x); acc[1] += bf16_hi(v[r].x); acc[2] += bf16_lo(v[r].y); acc[3] += bf16_hi(v[r].y);
                acc[4] += bf16_lo(v[r].z); acc[5] += bf16_hi(v[r].z); acc[6] += bf16_lo(v[r].w); acc[7] += bf16_hi(v[r].w);
            }
        __nv_bfloat16* yr = p.y + (int64_t)row * p.ldy + slice_off + n0_local + n8;
        if (p.residual != nullptr) {
            for (int u = 0; u < 8 && u < left; ++u) yr[u] = k2_out<true>(p, acc[u], row, slice_off + n0_local + n8 + u);
        } else if (left >= 8 && (((uintptr_t)yr) & 15) == 0) {
            *reinterpret_cast<uint4*>(yr) = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                                      pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
        } else {
            for (int u = 0; u < 8 && u < left; ++u) yr[u] = __float2bfloat16_rn(acc[u]);
        }
    }
}

// Fused decode form: the warps of every CTA except the producer and the MMA issuer claim the shrink kernel's work
// (positions to quantize, then shrink units) from two counters before they take up their GEMM roles.  A claimed piece of
// work never waits for another CTA, so the launch cannot deadlock however its CTAs are scheduled.
template <int FMT>
__device__ __forceinline__ void fused_shrink_units(const K2Params& p, const K1Params& k1, const K2Ctrl* ctrl, int lane) {
    const int groups = k1.R >> 3;
    for (;;) {
        int u = 0;
        if (lane == 0) u = atomicAdd(p.work_shrink, 1);
        u = __shfl_sync(0xffffffffu, u, 0);
        if (u >= p.shrink_units) break;
        // unit -> (position, slice, group of 8 rank rows, K split); the position's row and adapter were worked out once
        // per CTA together with the expand steps
        const int pos = u / k1.units_per_block, uu = u % k1.units_per_block;
        const int lora = ctrl->lora_pos[pos], row = ctrl->rowmap[pos];
        if (lora >= 0 && row >= 0) {
            const int j = uu % k1.split1, rg = (uu / k1.split1) % groups, sl = uu / (k1.split1 * groups);
            const int k0 = j * k1.k_per_split;
            shrink_pass1<FMT>(k1, lora, sl, rg, j, k0, min(k1.K, k0 + k1.k_per_split), pos, row, lane);
        }
        __syncwarp();
        if (lane == 0) red_release_add(p.hp_ready, 1);      // the unit's partial sums are in memory
    }
}

// EXTRA: the launch adds a residual stream in its stores; every other launch runs an instantiation without that code (a
// launch's instruction lines are cold fetches after an L2 flush, and the per-element branches lengthen the epilogue).
template <bool FP4, bool STORED, bool FUSED, bool EXTRA>
__global__ void __launch_bounds__(kK2Threads, 2)
k2_kernel(const K2Params p, const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
              const __grid_constant__ CUtensorMap tm_b0, const __grid_constant__ CUtensorMap tm_b1,
              const __grid_constant__ CUtensorMap tm_b2, const __grid_constant__ CUtensorMap tm_b3, const K1Params k1) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tn = p.tn;
    const int sf_bytes = FP4 ? kSfSlotBytes * (1 + p.nblk) : 0;   // W scales + activation scales of one K slot
    const int stage_bytes = kWTileBytes + tn * kBlockK + sf_bytes;
    const bool small = tn <= 32;                               // decode tiles: h table in shared memory + a builder warp
    const int nh = p.nh;                                       // masked H tiles in flight
    const int h_bytes = (int)align_up((size_t)tn * p.rc * 2, 1024);
    uint8_t* ring = smem;
    uint8_t* hbuf = ring + (size_t)p.stages * stage_bytes;    // nh masked H tiles (UMMA layout)
    uint8_t* htab = hbuf + (size_t)nh * h_bytes;              // small: bf16 h table [tn][R]
    K2Ctrl* ctrl = reinterpret_cast<K2Ctrl*>(htab + (small ? align_up((size_t)tn * p.R * 2, 1024) : 0));

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    griddep_launch_dependents();                               // the next kernel in the stream may start its own prologue
    const uint64_t limit_ns = (uint64_t)p.wait_ms * 1000000ull;

    // ---- tile coordinates: blockIdx.x walks the slices' 128-wide tiles, .y the K splits, .z the token tiles.  With more
    // than one token tile the two swap: consecutive CTAs then share a W tile, which comes from HBM once and from L2 after.
    const int n_idx = p.m_fast ? (int)blockIdx.z : (int)blockIdx.x;
    const int m_idx = p.m_fast ? (int)blockIdx.x : (int)blockIdx.z;
    const int n_count = p.m_fast ? (int)gridDim.z : (int)gridDim.x;
    int s = 0, n_tile = n_idx, slice_off = 0;
    while (s < p.S - 1 && n_tile >= (p.widths[s] + kTileN - 1) / kTileN) {
        n_tile -= (p.widths[s] + kTileN - 1) / kTileN;
        slice_off += p.widths[s];
        ++s;
    }
    const int n_s = p.widths[s];
    const int n0_local = n_tile * kTileN;
    const int j = blockIdx.y;
    const int t0 = m_idx * tn;
    const int kb0 = (int)(((int64_t)p.kblocks * j) / p.split2);
    const int kb1 = (int)(((int64_t)p.kblocks * (j + 1)) / p.split2);
    const int n_base = kb1 - kb0;
    const int n_chunks = p.R / p.rc;
    const int tile_lin = m_idx * n_count + n_idx;
    const int lead = FUSED ? max(p.stages, n_base) : p.stages;   // fused: every W tile first -- the shrink runs beside them
    const long long trace_cta = blockIdx.x + (long long)gridDim.x * (blockIdx.y + (long long)gridDim.y * blockIdx.z);
    if (tid == 0) { OB_TRACE(0) }

    // ---- one-time setup
    if (tid == 0) {
        for (int i = 0; i < p.stages; ++i) {
            mbar_init(&ctrl->full_w[i], 1);
            mbar_init(&ctrl->full_b[i], 1);
            mbar_init(&ctrl->empty[i], 1);
            mbar_init(&ctrl->empty_b[i], 1);
            if (STORED) mbar_init(&ctrl->code_full[i], 1);
        }
        for (int i = 0; i < 8; ++i) {
            mbar_init(&ctrl->h_full[i], 1);
            mbar_init(&ctrl->h_empty[i], 1);
        }
        mbar_init(&ctrl->htab_ready, 1);
        mbar_init(&ctrl->list_ready, 1);
        mbar_init(&ctrl->acc_full, 1);
        ctrl->abort_flag = 0;
        ctrl->b_grant = 0;
        ctrl->n_steps = 0;
        ctrl->last_flag = 0;
        fence_mbar_init();
    }
    // TMEM: two fp32 accumulators of tn columns; NVFP4 adds, per ring slot, 4 MMAs x (4 columns of W scales + 4 per
    // 128-token block of activation scales)
    const uint32_t sf_cols_per_slot = FP4 ? 16u * (1u + (uint32_t)p.nblk) : 0u;
    uint32_t tmem_cols = 32;
    while (tmem_cols < 2u * (uint32_t)tn + sf_cols_per_slot * (uint32_t)p.stages) tmem_cols *= 2;
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
    if (tid == 0) { OB_TRACE(1) }
    const uint32_t acc0 = tmem_base, acc1 = tmem_base + (uint32_t)tn;

    if (warp == 0) {
        // =========================================================== TMA producer: W tiles + their x_q tiles, B tiles
        if (lane == 0) {
            // one token tile: W streams through once, so it should not displace the adapters; several token tiles re-read it
            const uint64_t pol = p.m_fast ? l2_policy_evict_last() : l2_policy_evict_first();
            const CUtensorMap* tmb = (s == 0) ? &tm_b0 : (s == 1) ? &tm_b1 : (s == 2) ? &tm_b2 : &tm_b3;
            const uint32_t b_bytes = (uint32_t)kTileN * p.rc * 2;
            const uint32_t wx_bytes = (uint32_t)kWTileBytes + (uint32_t)tn * kBlockK + (uint32_t)sf_bytes;
            SlotWalk w(lead);
            RingBook book;
            const bool b_by_tma = !STORED;
            int n_steps = 0;
            bool have_list = false, k1_done = false;
            // Progress beyond the slots issued so far needs K1's x_q: wait for K1, then request the x_q tile of every W slot
            // issued so far.  (All of those slots are W tiles: the walk hands out no B tile before the list is known.)
            auto wait_k1 = [&]() -> bool {
                OB_TRACE(15)
                griddep_wait();     // the preceding kernel is complete: K1's outputs, or (fused) x and the cleared counters
                if constexpr (FUSED) {
                    // The CTAs' epilogue warps count the positions they quantized; those codes are enough to start the
                    // base GEMM while the shrink units keep running beside it.
                    const uint64_t t_start = global_timer_ns();
                    bool ready = false;
                    for (uint32_t spin = 0;; ++spin) {
                        if (ld_acquire(p.xq_ready) >= p.M) { ready = true; break; }
                        if ((spin & 31u) == 31u && global_timer_ns() - t_start > limit_ns) break;
                    }
                    if (!ready) { record_timeout(p, ctrl, 15, w.it); return false; }
                    fence_proxy_async_all();
                }
                OB_TRACE(4)
                k1_done = true;
                SlotWalk r(lead);
                while (r.it < w.it) {
                    const bool rb = r.is_b(n_base, n_steps);
                    if (!rb) {
                        const int st = r.it % p.stages;
                        uint8_t* slot = ring + (size_t)st * stage_bytes;
                        tma_load_2d(slot + kWTileBytes, &tm_x, &ctrl->full_w[st], (kb0 + r.k) * kBlockK, t0);
                        if (FP4)
                            bulk_load(slot + kWTileBytes + tn * kBlockK + kSfSlotBytes,
                                      p.xsf + ((size_t)m_idx * p.kblocks + (kb0 + r.k)) * p.nblk * kSfSlotBytes,
                                      (uint32_t)(kSfSlotBytes * p.nblk), &ctrl->full_w[st]);
                    }
                    r.advance(rb, n_base, n_steps);
                }
                return true;
            };
            for (;;) {
                if (ctrl->abort_flag) break;
                // A full ring of W tiles needs no list: K1's codes first, so that the MMAs start while warps 4-7 still list
                // the tile's expand steps.
                if (!k1_done && w.it >= p.stages && w.it <= lead && w.k < n_base && !wait_k1()) break;
                if (!have_list && w.needs_list(n_base)) {
                    if (!mbar_wait(&ctrl->list_ready, 0, limit_ns)) { record_timeout(p, ctrl, 2, w.it); break; }
                    n_steps = ctrl->n_steps;
                    have_list = true;
                }
                const bool finished = w.done(n_base, n_steps);
                if (!k1_done && (finished || w.it >= p.stages) && !wait_k1()) break;
                if (finished) break;
                const int st = w.it % p.stages;
                const bool isb = w.is_b(n_base, n_steps);
                uint32_t parity = 0;
                const int kind = book.acquire(w.it, st, p.stages, isb, parity);   // wait until the slot's previous tenant was consumed
                if (kind == 2) {
                    OB_WAIT(&ctrl->empty_b[st], parity, 3, w.it)
                } else if (kind == 1) {
                    OB_WAIT(&ctrl->empty[st], parity, 1, w.it)
                }
                if (isb) {
                    if (b_by_tma) {       // bf16 adapters: the B tile comes by TMA; stored formats are dequantized by warps 4-7
                        const LoraStep e = ctrl->steps[w.li];
                        mbar_arrive_expect_tx(&ctrl->full_b[st], b_bytes);
                        tma_load_2d(ring + (size_t)st * stage_bytes, tmb, &ctrl->full_b[st], e.chunk * p.rc,
                                    e.lora * p.b_rows[s] + (n0_local - p.b_row0[s]));
                    } else {
                        // The slot is free (this thread saw its release, in order, like every slot's): hand it to warps
                        // 4-7 through a count, which -- unlike a barrier phase awaited late -- cannot be mistaken.
                        if (p.b_staged) {
                            // ... with the step's codes and scales already on their way into the slot's upper half (the
                            // dequantized tile will overwrite them only after every thread has taken its row into
                            // registers): the ring's depth, not one step, is how far the adapter bytes run ahead.
                            const LoraStep e = ctrl->steps[w.li];
                            const uint32_t rows = (uint32_t)min(kTileN, n_s - n0_local);
                            const size_t row0 = (size_t)e.lora * n_s + (size_t)n0_local;
                            uint8_t* slot = ring + (size_t)st * stage_bytes;
                            const uint32_t code_bytes = p.lora_fmt == kLoraFp8 ? rows * (uint32_t)p.R : rows * (uint32_t)p.R / 2;
                            const uint32_t scale_bytes = p.lora_fmt == kLoraFp8 ? rows * 4u : rows * (uint32_t)p.R / 16;
                            const size_t code_off = p.lora_fmt == kLoraFp8 ? row0 * p.R : row0 * p.R / 2;
                            const size_t scale_off = p.lora_fmt == kLoraFp8 ? row0 * 4 : row0 * p.R / 16;
                            mbar_arrive_expect_tx(&ctrl->code_full[st], code_bytes + scale_bytes);
                            bulk_load(slot + 8192, static_cast<const uint8_t*>(p.b[s]) + code_off, code_bytes, &ctrl->code_full[st]);
                            bulk_load(slot + 16384, static_cast<const uint8_t*>(p.sb[s]) + scale_off, scale_bytes, &ctrl->code_full[st]);
                        }
                        __threadfence_block();
                        ctrl->b_grant = w.li + 1;
                    }
                } else {
                    mbar_arrive_expect_tx(&ctrl->full_w[st], wx_bytes);
                    tma_load_2d_hint(ring + (size_t)st * stage_bytes, &tm_w, &ctrl->full_w[st], (kb0 + w.k) * kBlockK,
                                     slice_off + n0_local, pol);
                    if (w.it == 0) { OB_TRACE(2) }
                    uint8_t* slot = ring + (size_t)st * stage_bytes;
                    if (FP4)
                        bulk_load(slot + kWTileBytes + tn * kBlockK, p.wsf + ((size_t)n_idx * p.kblocks + (kb0 + w.k)) * kSfSlotBytes,
                                  kSfSlotBytes, &ctrl->full_w[st]);
                    if (k1_done) {
                        tma_load_2d(slot + kWTileBytes, &tm_x, &ctrl->full_w[st], (kb0 + w.k) * kBlockK, t0);
                        if (FP4)
                            bulk_load(slot + kWTileBytes + tn * kBlockK + kSfSlotBytes,
                                      p.xsf + ((size_t)m_idx * p.kblocks + (kb0 + w.k)) * p.nblk * kSfSlotBytes,
                                      (uint32_t)(kSfSlotBytes * p.nblk), &ctrl->full_w[st]);
                    }
                }
                w.advance(isb, n_base, n_steps);
            }
            OB_TRACE(3)
        }
    } else if (warp == 1) {
        // =========================================================== MMA issuer
        if (lane == 0) {
            const uint32_t idesc8 = umma_idesc(0, 0, kTileN, (uint32_t)tn);
            const uint32_t idesc16 = umma_idesc(1, 1, kTileN, (uint32_t)tn);
            const uint32_t idesc4 = umma_idesc_nvfp4(kTileN, (uint32_t)tn);
            const uint32_t row_bytes = (uint32_t)p.rc * 2;                 // 32, 64 or 128
            const uint32_t lt = row_bytes == 128 ? 2u : row_bytes == 64 ? 4u : 6u;
            const uint32_t sbo = row_bytes * 8;
            SlotWalk w(lead);
            uint32_t par_w = 0, par_b = 0;
            int n_steps = 0;
            bool have_list = false, ok = true;
            for (;;) {
                if (ctrl->abort_flag) { ok = false; break; }
                if (!have_list && w.needs_list(n_base)) {
                    if (!mbar_wait(&ctrl->list_ready, 0, limit_ns)) { record_timeout(p, ctrl, 7, w.it); ok = false; break; }
                    n_steps = ctrl->n_steps;
                    have_list = true;
                }
                if (w.done(n_base, n_steps)) break;
                const int st = w.it % p.stages;
                const uint32_t bit = 1u << st;
                const bool isb = w.is_b(n_base, n_steps);
                if (!isb) {
                    if (!mbar_wait(&ctrl->full_w[st], (par_w >> st) & 1u, limit_ns)) { record_timeout(p, ctrl, 5, w.it); ok = false; break; }
                    par_w ^= bit;
                    if (w.k == 0) { OB_TRACE(5) }
                    tc_fence_after();
                    const uint32_t wa = smem_u32(ring + (size_t)st * stage_bytes);
                    const uint64_t dw = umma_smem_desc(wa, 1024, 2);
                    const uint64_t dx = umma_smem_desc(wa + kWTileBytes, 1024, 2);
                    if (FP4) {
                        // scale factors of this slot: shared memory -> this slot's TMEM columns, then the block-scaled MMAs
                        const uint32_t sfs = wa + kWTileBytes + (uint32_t)tn * kBlockK;
                        const uint32_t sft = tmem_base + 2u * (uint32_t)tn + (uint32_t)st * sf_cols_per_slot;
#pragma unroll
                        for (int k = 0; k < kBlockK / 32; ++k) {
                            const uint32_t ta = sft + (uint32_t)k * 4u;
                            const uint32_t tb = sft + 16u + (uint32_t)k * 4u * (uint32_t)p.nblk;
                            tmem_cp_sf(ta, sf_smem_desc(sfs + (uint32_t)k * 512u));
                            for (int b = 0; b < p.nblk; ++b)
                                tmem_cp_sf(tb + 4u * (uint32_t)b, sf_smem_desc(sfs + kSfSlotBytes + ((uint32_t)b * 4u + (uint32_t)k) * 512u));
                            umma_nvfp4(acc0, dw + (uint64_t)(k * 2), dx + (uint64_t)(k * 2), idesc4, ta, tb, (w.k > 0 || k > 0) ? 1u : 0u);
                        }
                    } else {
#pragma unroll
                        for (int k = 0; k < kBlockK / 32; ++k)
                            umma_f8f6f4(acc0, dw + (uint64_t)(k * 2), dx + (uint64_t)(k * 2), idesc8, (w.k > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(&ctrl->empty[st]);
                    if (w.k == n_base - 1) { OB_TRACE(6) }
                } else {
                    const int hb = w.li % nh, hu = w.li / nh;
                    if (!mbar_wait(&ctrl->full_b[st], (par_b >> st) & 1u, limit_ns)) { record_timeout(p, ctrl, 8, w.it); ok = false; break; }
                    par_b ^= bit;
                    if (!mbar_wait(&ctrl->h_full[hb], (uint32_t)(hu & 1), limit_ns)) { record_timeout(p, ctrl, 9, w.it); ok = false; break; }
                    tc_fence_after();
                    const uint64_t db = umma_smem_desc(smem_u32(ring + (size_t)st * stage_bytes), sbo, lt);
                    const uint64_t dh = umma_smem_desc(smem_u32(hbuf + (size_t)hb * h_bytes), sbo, lt);
                    for (int k = 0; k < p.rc / 16; ++k)
                        umma_f16(acc1, db + (uint64_t)(k * 2), dh + (uint64_t)(k * 2), idesc16, (w.li > 0 || k > 0) ? 1u : 0u);
                    umma_commit(&ctrl->empty_b[st]);
                    umma_commit(&ctrl->h_empty[hb]);
                }
                w.advance(isb, n_base, n_steps);
            }
            if (ok) umma_commit(&ctrl->acc_full);
        }
    } else if (warp == 2) {
        // =========================================================== masked-H builder (decode tiles)
        // Step li multiplies B_l's tile with H = the h rows of tenant l's tokens, zero elsewhere.  The nh tiles start as
        // zeros; per step the warp clears the rows the tile's previous step filled and copies this step's rows out of the h
        // table -- one or two 128-byte rows in a mixed decode batch -- so it runs far ahead of the B tiles' arrival.
        if (small) {
            for (int i = lane; i < nh * h_bytes / 16; i += 32) reinterpret_cast<uint4*>(hbuf)[i] = make_uint4(0u, 0u, 0u, 0u);
            bool ok = mbar_wait(&ctrl->list_ready, 0, limit_ns);
            if constexpr (FUSED) {
                griddep_wait();
                if (ok) fused_shrink_units<kLoraBf16>(p, k1, ctrl, lane);
            }
            const int n_steps = ok ? ctrl->n_steps : 0;
            if (ok && n_steps > 0) ok = mbar_wait(&ctrl->htab_ready, 0, limit_ns);
            if (!ok && lane == 0) record_timeout(p, ctrl, 13, 0);
            const int row_bytes = p.rc * 2, cpr = row_bytes / 16;
            const uint32_t swz = (uint32_t)cpr - 1u;
            for (int li = 0; ok && li < n_steps; ++li) {
                const int hb = li % nh, hu = li / nh;
                if (ctrl->abort_flag) break;
                uint8_t* tile = hbuf + (size_t)hb * h_bytes;
                if (hu > 0) {
                    if (!mbar_wait(&ctrl->h_empty[hb], (uint32_t)((hu - 1) & 1), limit_ns)) {
                        if (lane == 0) record_timeout(p, ctrl, 10, li);
                        break;
                    }
                    const LoraStep o = ctrl->steps[li - nh];
                    for (int c = lane; c < ((int)o.hi - (int)o.lo) * cpr; c += 32) {
                        uint32_t off = (uint32_t)((int)o.lo + c / cpr) * (uint32_t)row_bytes + (uint32_t)(c % cpr) * 16u;
                        off ^= ((off >> 7) & swz) << 4;
                        *reinterpret_cast<uint4*>(tile + off) = make_uint4(0u, 0u, 0u, 0u);
                    }
                    __syncwarp();
                }
                const LoraStep e = ctrl->steps[li];
                for (int c = lane; c < ((int)e.hi - (int)e.lo) * cpr; c += 32) {
                    const int row = (int)e.lo + c / cpr, c16 = c % cpr;
                    const uint4 v = *reinterpret_cast<const uint4*>(htab + ((size_t)row * p.R + (size_t)e.chunk * p.rc) * 2 + (size_t)c16 * 16);
                    uint32_t off = (uint32_t)row * (uint32_t)row_bytes + (uint32_t)c16 * 16u;
                    off ^= ((off >> 7) & swz) << 4;
                    *reinterpret_cast<uint4*>(tile + off) = v;
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&ctrl->h_full[hb]);
            }
        }
    } else if (warp == 3) {
        if constexpr (FUSED) {
            const bool ok = mbar_wait(&ctrl->list_ready, 0, limit_ns);
            griddep_wait();
            if (ok) fused_shrink_units<kLoraBf16>(p, k1, ctrl, lane);
        }
    } else if (warp >= 4) {
        // =========================================================== segment index, H tiles, epilogue
        const int te = tid - 128;
        // The index's loads do not depend on one another: request the sorted rows and the segment starts before the
        // totals are summed, so that the list costs one memory round trip and not three.
        for (int i = lane; i <= p.L; i += 32) prefetch_l1(p.meta.seg_start + i);
        int srt_v[2] = {0, 0};                                // tn <= 256: at most two positions per thread
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int c = te + u * 128;
            if (c < tn && t0 + c < p.M) srt_v[u] = p.meta.srt[t0 + c];
        }
        int n_all, n_ad;
        segment_totals(p.meta, p.L, lane, n_all, n_ad);
        n_all = min(n_all, p.M);
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int c = te + u * 128, pos = t0 + c;
            if (c < tn) {
                int row = pos < p.M ? pos : -1;
                if (n_ad > 0 && pos < n_all) row = srt_v[u] < 0 ? 0 : (srt_v[u] > p.M - 1 ? p.M - 1 : srt_v[u]);
                ctrl->rowmap[c] = row;
            }
        }
        if (FUSED) {
            for (int c = te; c < 32; c += 128) ctrl->lora_pos[c] = -1;
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        if (warp == 4) {
            int total = 0;                                   // (segment, chunk) steps of this tile so far, all splits
            // sharded B: only the tiles whose rows this rank holds carry an expand
            const bool has_b = n0_local >= p.b_row0[s] && n0_local < p.b_row0[s] + p.b_rows[s];
            if (n_ad > 0) {
                for (int base = 0; base <= p.L; base += 32) {
                    const int i = base + lane;
                    int lora = -1, lo = 0, hi = 0;
                    if (i <= p.L) {
                        lora = p.meta.seg_ids[i];
                        const int cnt = p.meta.seg_n[i], sst = p.meta.seg_start[i];
                        lo = max(sst, t0);
                        hi = min(min(sst + cnt, t0 + tn), n_all);
                        if (cnt <= 0 || sst < 0) lora = -1;
                    }
                    const bool seg = lora >= 0 && lora < p.L && lo < hi;
                    if (FUSED && seg)                        // (the shrink covers every position, with or without an expand here)
                        for (int pos = lo; pos < hi; ++pos) ctrl->lora_pos[pos - t0] = lora;
                    const bool ok = seg && has_b;
                    const uint32_t mask = __ballot_sync(0xffffffffu, ok);
                    if (ok) {
                        const int idx = total / n_chunks + __popc(mask & ((1u << lane) - 1u));
                        for (int c = 0; c < n_chunks; ++c) {
                            const int e = idx * n_chunks + c;
                            if (e % p.split2 == j) {
                                const int li = e / p.split2;
                                if (li < kMaxLoraIters)
                                    ctrl->steps[li] = LoraStep{(uint16_t)lora, (uint16_t)c, (uint16_t)(lo - t0), (uint16_t)(hi - t0)};
                            }
                        }
                    }
                    total += __popc(mask) * n_chunks;
                }
            }
            if (lane == 0) {
                int mine = total > j ? (total - j + p.split2 - 1) / p.split2 : 0;
                ctrl->n_steps = min(mine, kMaxLoraIters);
            }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (te == 0) { mbar_arrive(&ctrl->list_ready); OB_TRACE(7) }
        const int n_steps = ctrl->n_steps;

        griddep_wait();                                       // K1's s_x and shrink partials from here on
        if constexpr (FUSED) {
            // x is final now.  Quantize positions, one per claim of the four warps together; then shrink units, one per
            // claim of a warp; then wait until every position and every unit of the launch is done.
            for (;;) {
                if (te == 0) ctrl->claim = atomicAdd(p.work_quant, 1);
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const int qpos = ctrl->claim;
                if (qpos >= p.M) break;
                const int qrow = ctrl->rowmap[qpos];          // t0 = 0: the fused form serves one token tile
                if (FP4) quantize_row_nvfp4<128>(k1, qpos, qrow, te);
                else quantize_row<128, 1>(k1, qpos, qrow, te);
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (te == 0) red_release_add(p.xq_ready, 1);
            }
            fused_shrink_units<kLoraBf16>(p, k1, ctrl, lane);
            if (te == 0) {
                const uint64_t t_start = global_timer_ns();
                bool ready = false;
                for (uint32_t spin = 0;; ++spin) {
                    if (ld_acquire(p.xq_ready) >= p.M && ld_acquire(p.hp_ready) >= p.shrink_units) { ready = true; break; }
                    if ((spin & 31u) == 31u && global_timer_ns() - t_start > limit_ns) break;
                }
                if (!ready) record_timeout(p, ctrl, 16, 0);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        if (te == 0) { OB_TRACE(8) }
        for (int c = te; c < tn; c += 128) ctrl->sx[c] = FP4 ? 1.0f : ((t0 + c < p.M) ? __ldcg(p.sx + t0 + c) : 0.0f);

        const int row_bytes = p.rc * 2;
        const int cpr = row_bytes / 16;                       // 16-byte chunks per tile row
        const uint32_t swz = (uint32_t)cpr - 1u;
        const int q = warp & 3;
        const int n_local = q * 32 + lane;
        if (small) {
            // ---- h table: bf16( sum over K1's splits, in split order ) for every token of the tile, once
            if (n_steps > 0) {
                const int groups = p.R / 8;
                for (int idx = te; idx < tn * groups; idx += 128) {
                    const int row = idx / groups, g8 = idx % groups;
                    float acc[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) acc[u] = 0.0f;
                    if (t0 + row < n_all) {
                        // four splits' loads in flight at a time (a plain loop would pay one L2 round trip per split),
                        // added in split order
                        const size_t jstride = (size_t)p.S * p.max_m * p.R;
                        const float* src0 = p.hp + ((size_t)s * p.max_m + (size_t)(t0 + row)) * p.R + (size_t)g8 * 8;
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
                    *reinterpret_cast<uint4*>(htab + ((size_t)row * p.R + (size_t)g8 * 8) * 2) = out;
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (te == 0) { mbar_arrive(&ctrl->htab_ready); }
        }
        constexpr bool stored = STORED;                       // FP8- / NVFP4-stored adapters: these warps produce the B tiles
        if (stored || !small) {
            SlotWalk w(lead);
            BCodes cur;                                       // stored adapters: this step's codes, requested a step ahead
            const bool staged = STORED && p.b_staged != 0;    // ... or brought into the slot by the producer's bulk copies
            uint32_t par_c = 0;                               // per slot: phase of its code barrier
            if (STORED && !staged && n_steps > 0) load_b_codes(p, ctrl->steps[0], s, n_s, n0_local, te, cur);
            for (int li = 0; li < n_steps; ++li) {
                while (!w.is_b(n_base, n_steps)) w.advance(false, n_base, n_steps);   // the W slots in between
                const int st = w.it % p.stages;
                const int hb = li % nh, hu = li / nh;
                if (te == 0) {                                    // one thread decides, so that all 128 leave together
                    int go = ctrl->abort_flag ? 0 : 1;
                    if (go && stored) {
                        // Wait until the producer has acquired this step's slot.  (These warps start late -- after K1's
                        // partials -- while the ring runs ahead; a wait of their own on the slot's release barrier could
                        // meet a phase two ahead of the awaited one and never return.)
                        const uint64_t t_start = global_timer_ns();
                        for (uint32_t spin = 0; ctrl->b_grant <= li; ++spin) {
                            if (ctrl->abort_flag) { go = 0; break; }
                            if ((spin & 63u) == 63u && global_timer_ns() - t_start > limit_ns) {
                                record_timeout(p, ctrl, 14, w.it);
                                go = 0;
                                break;
                            }
                        }
                        __threadfence_block();
                        if (go && staged && !mbar_wait(&ctrl->code_full[st], (par_c >> st) & 1u, limit_ns)) {
                            record_timeout(p, ctrl, 17, w.it);
                            go = 0;
                        }
                    }
                    if (go && !small && hu > 0 && !mbar_wait(&ctrl->h_empty[hb], (uint32_t)((hu - 1) & 1), limit_ns)) {
                        record_timeout(p, ctrl, 10, li);
                        go = 0;
                    }
                    ctrl->go_flag = go;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (!ctrl->go_flag) break;
                const LoraStep e = ctrl->steps[li];
                if constexpr (STORED) {
                    if (staged) {
                        par_c ^= 1u << st;
                        load_b_codes_smem(p, e, s, n_s, n0_local, te, ring + (size_t)st * stage_bytes, cur);
                        asm volatile("bar.sync 1, 128;" ::: "memory");    // every row is in registers before the tile overwrites the codes
                        store_b_tile(p, cur, ring + (size_t)st * stage_bytes, te, row_bytes, swz);
                    } else {
                        BCodes nxt = cur;
                        if (li + 1 < n_steps) load_b_codes(p, ctrl->steps[li + 1], s, n_s, n0_local, te, nxt);   // in flight during the stores
                        store_b_tile(p, cur, ring + (size_t)st * stage_bytes, te, row_bytes, swz);
                        cur = nxt;
                    }
                }
                if (!small) {
                uint8_t* hdst = hbuf + (size_t)hb * h_bytes;
                for (int ch = te; ch < tn * cpr; ch += 128) {
                    const int row = ch / cpr, c16 = ch % cpr;
                    uint4 out = make_uint4(0u, 0u, 0u, 0u);
                    if (p.hb != nullptr) {                 // the tensor-core shrink left the finished h
                        if (row >= (int)e.lo && row < (int)e.hi)
                            out = __ldcg(reinterpret_cast<const uint4*>(
                                p.hb + ((size_t)s * p.max_m + (size_t)(t0 + row)) * p.R + (size_t)e.chunk * p.rc + (size_t)c16 * 8));
                    } else if (row >= (int)e.lo && row < (int)e.hi) {
                        float acc[8];
#pragma unroll
                        for (int u = 0; u < 8; ++u) acc[u] = 0.0f;
                        const size_t col = (size_t)e.chunk * p.rc + (size_t)c16 * 8;
                        for (int j1 = 0; j1 < p.split1; ++j1) {
                            const float4* src = reinterpret_cast<const float4*>(
                                p.hp + (((size_t)j1 * p.S + s) * p.max_m + (size_t)(t0 + row)) * p.R + col);
                            const float4 u0 = __ldcg(src), u1 = __ldcg(src + 1);
                            acc[0] += u0.x; acc[1] += u0.y; acc[2] += u0.z; acc[3] += u0.w;
                            acc[4] += u1.x; acc[5] += u1.y; acc[6] += u1.z; acc[7] += u1.w;
                        }
                        __nv_bfloat162 b0 = __floats2bfloat162_rn(acc[0], acc[1]);
                        __nv_bfloat162 b1 = __floats2bfloat162_rn(acc[2], acc[3]);
                        __nv_bfloat162 b2 = __floats2bfloat162_rn(acc[4], acc[5]);
                        __nv_bfloat162 b3 = __floats2bfloat162_rn(acc[6], acc[7]);
                        out.x = *reinterpret_cast<uint32_t*>(&b0);
                        out.y = *reinterpret_cast<uint32_t*>(&b1);
                        out.z = *reinterpret_cast<uint32_t*>(&b2);
                        out.w = *reinterpret_cast<uint32_t*>(&b3);
                    }
                    uint32_t off = (uint32_t)row * (uint32_t)row_bytes + (uint32_t)c16 * 16u;
                    off ^= ((off >> 7) & swz) << 4;
                    *reinterpret_cast<uint4*>(hdst + off) = out;
                }
                }
                fence_proxy_async_smem();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (te == 0) {
                    if (stored) mbar_arrive(&ctrl->full_b[st]);
                    if (!small) mbar_arrive(&ctrl->h_full[hb]);
                }
                w.advance(true, n_base, n_steps);
            }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");            // sx / rowmap visible to all epilogue threads

        // ---- epilogue
        if (te == 0) {
            int go = ctrl->abort_flag ? 0 : 1;
            if (go && !mbar_wait(&ctrl->acc_full, 0u, limit_ns)) {
                record_timeout(p, ctrl, 11, 0);
                go = 0;
            }
            ctrl->go_flag = go;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const bool done = ctrl->go_flag != 0;
        tc_fence_after();
        if (te == 0) { OB_TRACE(11) }
        if (done) {
            const bool n_ok = n0_local + n_local < n_s;
            const int n_glob = slice_off + n0_local + n_local;
            const float s_w = FP4 ? __ldg(p.alpha) : __ldg(p.s_w);   // NVFP4: one scale 1 / (x_global * w_global)
            const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
            const bool has_lora = n_steps > 0;
            float* part = p.part + ((size_t)tile_lin * p.split2 + j) * (size_t)tn * kTileN;
            // fused all-reduce: finished values go to this rank's staged copy ([token row][N] bf16) instead of y
            const bool ar = p.ar_world > 0;   // a run-time flag in every instantiation: measured faster than compiling it out
            const int32_t ar_epoch = ar ? *reinterpret_cast<const volatile int32_t*>(p.ar_bufs[p.ar_rank]) + 1 : 0;
            __nv_bfloat16* ydst = ar ? reinterpret_cast<__nv_bfloat16*>(p.ar_bufs[p.ar_rank] + kArStateBytes +
                                                                      (size_t)(ar_epoch & 1) * (size_t)p.ar_slot_bytes)
                                     : p.y;
            const int64_t yld = ar ? (int64_t)p.N : p.ldy;
            {
                for (int c0 = 0; c0 < tn; c0 += 16) {
                    uint32_t r0[16], r1[16];
                    tmem_ld16(acc0 + lane_addr + (uint32_t)c0, r0);
                    if (has_lora) tmem_ld16(acc1 + lane_addr + (uint32_t)c0, r1);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 16; ++c) {
                        const int row = ctrl->rowmap[c0 + c];
                        float v = __uint_as_float(r0[c]) * (ctrl->sx[c0 + c] * s_w);
                        if (has_lora) v += __uint_as_float(r1[c]);
                        if (p.split2 == 1) {
                            if (row >= 0 && n_ok) ydst[(int64_t)row * yld + n_glob] = ar ? __float2bfloat16_rn(v) : k2_out<EXTRA>(p, v, row, n_glob);
                        } else if (p.cluster_reduce) {
                            reinterpret_cast<float*>(ring)[(c0 + c) * kTileN + n_local] = v;   // the ring is idle by now
                        } else {
                            part[(size_t)(c0 + c) * kTileN + n_local] = v;
                        }
                    }
                }
            }
            if (ar && p.split2 == 1) ar_finish_tile(p, ctrl, te, tile_lin, ar_epoch, tn, slice_off, n0_local, n_s, limit_ns);
            if (p.split2 > 1 && !p.cluster_reduce) {
                asm volatile("bar.sync 1, 128;" ::: "memory");    // all 128 threads' partials precede the arrival below
                if (te == 0) {
                    int old;                                      // release our partials, acquire the other splits'
                    asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(old) : "l"(p.counters + tile_lin) : "memory");
                    ctrl->last_flag = (old == p.split2 - 1) ? 1 : 0;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (ctrl->last_flag) {
                    // The last CTA of the tile adds the partials in split order.  Thread = 4 output features x every 4th
                    // token; 8 tokens' loads are in flight per split so the sum is not a chain of dependent L2 round trips.
                    const float* pbase = p.part + (size_t)tile_lin * p.split2 * (size_t)tn * kTileN;
                    const int tg = te >> 5, n4 = (te & 31) * 4;
                    for (int cb = 0; cb < tn; cb += 32) {
                        float4 acc[8];
#pragma unroll
                        for (int u = 0; u < 8; ++u) acc[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                        for (int jj = 0; jj < p.split2; ++jj) {
#pragma unroll
                            for (int u = 0; u < 8; ++u) {
                                const int c = cb + u * 4 + tg;
                                if (c < tn) {
                                    const float4 v = __ldcg(reinterpret_cast<const float4*>(pbase + ((size_t)jj * tn + c) * kTileN + n4));
                                    acc[u].x += v.x; acc[u].y += v.y; acc[u].z += v.z; acc[u].w += v.w;
                                }
                            }
                        }
#pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            const int c = cb + u * 4 + tg;
                            const int row = c < tn ? ctrl->rowmap[c] : -1;
                            if (row >= 0) {
                                const int64_t col = slice_off + n0_local + n4;
                                __nv_bfloat16* yr = ydst + (int64_t)row * yld + col;
                                const int left = n_s - (n0_local + n4);
                                const float vv[4] = {acc[u].x, acc[u].y, acc[u].z, acc[u].w};
#pragma unroll
                                for (int e = 0; e < 4; ++e)
                                    if (left > e) yr[e] = ar ? __float2bfloat16_rn(vv[e]) : k2_out<EXTRA>(p, vv[e], row, col + e);
                            }
                        }
                    }
                    if (te == 0) p.counters[tile_lin] = 0;
                    if (ar) ar_finish_tile(p, ctrl, te, tile_lin, ar_epoch, tn, slice_off, n0_local, n_s, limit_ns);
                }
            }
        }
    }

    if (p.cluster_reduce) {
        // The K splits of a tile are the CTAs of one cluster.  Each has left its fp32 partial tile at the start of its own
        // shared memory; split j now sums tokens j, j + split2, ... over the cluster in split order and writes those rows.
        // Every thread of every CTA takes part in both barriers, whatever happened to it before.
        __syncthreads();
        cluster_sync_all();
        if (warp >= 4 && ctrl->go_flag) {
            const int te = tid - 128, tg = te >> 5, n4 = (te & 31) * 4;
            const uint32_t own = smem_u32(ring);
            for (int c = j + p.split2 * tg; c < tn; c += p.split2 * 4) {
                float4 v[8];
#pragma unroll
                for (int jj = 0; jj < 8; ++jj)
                    if (jj < p.split2) v[jj] = ld_cluster_f4(cluster_peer_addr(own + (uint32_t)(c * kTileN + n4) * 4u, (uint32_t)jj));
                float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                for (int jj = 0; jj < 8; ++jj)
                    if (jj < p.split2) { acc.x += v[jj].x; acc.y += v[jj].y; acc.z += v[jj].z; acc.w += v[jj].w; }
                const int row = ctrl->rowmap[c];
                if (row >= 0) {
                    __nv_bfloat16* yr = p.y + (int64_t)row * p.ldy + slice_off + n0_local + n4;
                    const int left = n_s - (n0_local + n4);
                    if (EXTRA && p.residual != nullptr) {
                        const float vv[4] = {acc.x, acc.y, acc.z, acc.w};
                        for (int e = 0; e < 4 && e < left; ++e) yr[e] = k2_out<true>(p, vv[e], row, slice_off + n0_local + n4 + e);
                    } else if (left >= 4 && (((uintptr_t)yr) & 7) == 0) {
                        __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
                        *reinterpret_cast<uint2*>(yr) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
                    } else {
                        if (left > 0) yr[0] = __float2bfloat16_rn(acc.x);
                        if (left > 1) yr[1] = __float2bfloat16_rn(acc.y);
                        if (left > 2) yr[2] = __float2bfloat16_rn(acc.z);
                        if (left > 3) yr[3] = __float2bfloat16_rn(acc.w);
                    }
                }
            }
        }
        cluster_sync_all();
    }
    // ---- teardown: nobody leaves while TMEM is in use or copies may still land in this CTA's shared memory
    if (ctrl->abort_flag) __nanosleep(200000);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, tmem_cols);
    }
    if (p.ar_world > 0 && tid == 0) {      // fused all-reduce: the last CTA of the launch advances the call count
        int32_t* state = reinterpret_cast<int32_t*>(p.ar_bufs[p.ar_rank]);
        const int32_t epoch = *reinterpret_cast<volatile int32_t*>(state) + 1;
        __threadfence();
        if (atomicAdd(state + 7, 1) == (int)(gridDim.x * gridDim.y * gridDim.z) - 1) {
            state[7] = 0;
            __threadfence();
            *reinterpret_cast<volatile int32_t*>(state) = epoch;
        }
    }
    if (FUSED && tid == 0) {                        // the last CTA of the launch clears the work counters for the next call
        const int total = (int)(gridDim.x * gridDim.y * gridDim.z);
        if (atomicAdd(p.chain_done, 1) == total - 1) {
            *const_cast<volatile int32_t*>(p.xq_ready) = 0;
            if constexpr (FUSED) {
                *const_cast<volatile int32_t*>(p.work_quant) = 0;
                *const_cast<volatile int32_t*>(p.work_shrink) = 0;
                *const_cast<volatile int32_t*>(p.hp_ready) = 0;
            }
            *const_cast<volatile int32_t*>(p.chain_done) = 0;
        }
    }
    if (tid == 0) { OB_TRACE(14) }
}

int k2_fp8_h_tiles(int tn) { return tn <= 16 ? 8 : tn <= 32 ? 4 : 2; }

size_t k2_fp8_smem_bytes(int tn, int stages, int rc, int R, int fp4) {
    const size_t sf = fp4 ? (size_t)kSfSlotBytes * (1 + (tn > 128 ? 2 : 1)) : 0;
    const size_t aux = (size_t)k2_fp8_h_tiles(tn) * align_up((size_t)tn * rc * 2, 1024) +
                       (tn <= 32 ? align_up((size_t)tn * R * 2, 1024) : 0);
    return 1024 + (size_t)stages * (kWTileBytes + (size_t)tn * kBlockK + sf) + aux + kCtrlBytes;
}

template <bool FP4, bool STORED, bool FUSED, bool EXTRA = false>
static cudaError_t launch_k2_impl(const K2Params& p, const CUtensorMap& tm_w, const CUtensorMap& tm_x, const CUtensorMap* tm_b,
                                  dim3 grid, size_t smem, int pdl, cudaStream_t stream, const K1Params& k1) {
    static int configured_for[64] = {0};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64 && !configured_for[dev]) {
        cudaFuncAttributes fa;                    // the opt-in limit covers static + dynamic shared memory
        e = cudaFuncGetAttributes(&fa, k2_kernel<FP4, STORED, FUSED, EXTRA>);
        if (e != cudaSuccess) return e;
        e = cudaFuncSetAttribute(k2_kernel<FP4, STORED, FUSED, EXTRA>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 227 * 1024 - (int)fa.sharedSizeBytes);
        if (e != cudaSuccess) return e;
        configured_for[dev] = 1;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kK2Threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (pdl) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    if (p.cluster_reduce) {                      // the K splits of one tile (grid y) are one cluster
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = 1;
        attr[n_attr].val.clusterDim.y = (unsigned)p.split2;
        attr[n_attr].val.clusterDim.z = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    return cudaLaunchKernelEx(&cfg, k2_kernel<FP4, STORED, FUSED, EXTRA>, p, tm_w, tm_x, tm_b[0], tm_b[1], tm_b[2], tm_b[3], k1);
}

// How many clusters of `split2` CTAs (grid y) of this kernel the current device keeps resident at once; 0 on error.
template <bool FP4, bool STORED>
static int max_clusters_impl(int split2, size_t smem) {
    cudaError_t e = cudaFuncSetAttribute(k2_kernel<FP4, STORED, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(64, (unsigned)split2, 1);
    cfg.blockDim = dim3(kK2Threads);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = (unsigned)split2;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, k2_kernel<FP4, STORED, false, false>, &cfg);
    if (e != cudaSuccess) { (void)cudaGetLastError(); return 0; }
    return n;
}

int k2_max_active_clusters(int fp4, int stored, int split2, size_t smem) {
    return fp4 ? (stored ? max_clusters_impl<true, true>(split2, smem) : max_clusters_impl<true, false>(split2, smem))
               : (stored ? max_clusters_impl<false, true>(split2, smem) : max_clusters_impl<false, false>(split2, smem));
}

cudaError_t launch_k2_fp8(const K2Params& p, const CUtensorMap& tm_w, const CUtensorMap& tm_x, const CUtensorMap* tm_b,
                          dim3 grid, size_t smem, int pdl, cudaStream_t stream) {
    const K1Params none = {};
    if (p.residual != nullptr)
        return p.lora_fmt == kLoraBf16 ? launch_k2_impl<false, false, false, true>(p, tm_w, tm_x, tm_b, grid, smem, pdl, stream, none)
                                       : launch_k2_impl<false, true, false, true>(p, tm_w, tm_x, tm_b, grid, smem, pdl, stream, none);
    return p.lora_fmt == kLoraBf16 ? launch_k2_impl<false, false, false>(p, tm_w, tm_x, tm_b, grid, smem, pdl, stream, none)
                                   : launch_k2_impl<false, true, false>(p, tm_w, tm_x, tm_b, grid, smem, pdl, stream, none);
}

cudaError_t launch_k2_nvfp4(const K2Params& p, const CUtensorMap& tm_w, const CUtensorMap& tm_x, const CUtensorMap* tm_b,
                            dim3 grid, size_t smem, int pdl, cudaStream_t stream) {
    const K1Params none = {};
    if (p.residual != nullptr)
        return p.lora_fmt == kLoraBf16 ? launch_k2_impl<true, false, false, true>(p, tm_w, tm_x, tm_b, grid, smem, pdl, stream, none)
                                       : launch_k2_impl<true, true, false, true>(p, tm_w, tm_x, tm_b, grid, smem, pdl, stream, none);
    return p.lora_fmt == kLoraBf16 ? launch_k2_impl<true, false, false>(p, tm_w, tm_x, tm_b, grid, smem, pdl, stream, none)
                                   : launch_k2_impl<true, true, false>(p, tm_w, tm_x, tm_b, grid, smem, pdl, stream, none);
}

// The fused decode kernel (bf16 adapters, one token tile of at most 32 tokens): quantization, shrink and GEMM in one launch.
cudaError_t launch_fused(const K2Params& p, const K1Params& k1, const CUtensorMap& tm_w, const CUtensorMap& tm_x,
                         const CUtensorMap* tm_b, dim3 grid, size_t smem, cudaStream_t stream) {
    return k1.base_fmt == OB_BASE_NVFP4 ? launch_k2_impl<true, false, true>(p, tm_w, tm_x, tm_b, grid, smem, 1, stream, k1)
                                        : launch_k2_impl<false, false, true>(p, tm_w, tm_x, tm_b, grid, smem, 1, stream, k1);
}

}  // namespace ob
