// Device code of K1 -- activation quantization of one tile position and the LoRA shrink of one warp's unit -- shared by
// the stand-alone K1 kernel and by the fused decode kernel, whose warps run the same units before their GEMM roles.
#pragma once
#include "ob_common.cuh"
#include "ob_ptx.cuh"

namespace ob {

template <int BAR, int NT>
__device__ __forceinline__ void named_bar_sync() {
    asm volatile("bar.sync %0, %1;" ::"n"(BAR), "n"(NT) : "memory");
}

#define OB_TRACE1(ev) \
    if (p.trace != nullptr && (long long)blockIdx.x < p.trace_ctas && threadIdx.x == 0) \
        p.trace[(long long)blockIdx.x * OB_TRACE_EVENTS + (ev)] = global_timer_ns();

constexpr float kFp8Max = 448.0f;
constexpr float kMinTokenScale = 1.0f / (448.0f * 512.0f);

__device__ __forceinline__ float amax8(const uint4& v) {
    float m = fmaxf(fabsf(bf16_lo(v.x)), fabsf(bf16_hi(v.x)));
    m = fmaxf(m, fmaxf(fabsf(bf16_lo(v.y)), fabsf(bf16_hi(v.y))));
    m = fmaxf(m, fmaxf(fabsf(bf16_lo(v.z)), fabsf(bf16_hi(v.z))));
    return fmaxf(m, fmaxf(fabsf(bf16_lo(v.w)), fabsf(bf16_hi(v.w))));
}

__device__ __forceinline__ float q1(float v, float sx) {
    return fminf(fmaxf(__fdiv_rn(v, sx), -kFp8Max), kFp8Max);
}

__device__ __forceinline__ uint2 quant8(const uint4& v, float sx) {
    uint2 o;
    o.x = (uint32_t)cvt_e4m3x2(q1(bf16_lo(v.x), sx), q1(bf16_hi(v.x), sx)) |
          ((uint32_t)cvt_e4m3x2(q1(bf16_lo(v.y), sx), q1(bf16_hi(v.y), sx)) << 16);
    o.y = (uint32_t)cvt_e4m3x2(q1(bf16_lo(v.z), sx), q1(bf16_hi(v.z), sx)) |
          ((uint32_t)cvt_e4m3x2(q1(bf16_lo(v.w), sx), q1(bf16_hi(v.w), sx)) << 16);
    return o;
}

// Eight consecutive elements k .. k+7 of the projection's INPUT row as bf16 pairs.  Plain: the row of x itself.  SiLU * mul
// (down_proj): x holds the merged gate | up output [2K]; the input is silu(gate) * up, formed as vLLM's SiluAndMul forms
// it: silu in fp32, rounded to bf16, times up, rounded to bf16 (activation.py, forward_native).
// XOP is a template parameter: the plain kernels must not carry the activation's code (after an L2 flush every
// instruction line of a launch is a cold fetch, and K1 sits on the chain's critical path).
template <bool XOP>
__device__ __forceinline__ uint4 x_load8(const K1Params& p, const __nv_bfloat16* xrow, int k) {
    const uint4 g = __ldg(reinterpret_cast<const uint4*>(xrow + k));
    if (!XOP) return g;
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(xrow + p.K + k));
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float g0 = bf16_lo(gw[i]), g1 = bf16_hi(gw[i]);
        const __nv_bfloat162 s2 = __floats2bfloat162_rn(__fdiv_rn(g0, 1.0f + expf(-g0)), __fdiv_rn(g1, 1.0f + expf(-g1)));
        const uint32_t sb = *reinterpret_cast<const uint32_t*>(&s2);
        const __nv_bfloat162 r2 = __floats2bfloat162_rn(bf16_lo(sb) * bf16_lo(uw[i]), bf16_hi(sb) * bf16_hi(uw[i]));
        o[i] = *reinterpret_cast<const uint32_t*>(&r2);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

// The row of x that tile position `pos` stands for (warp-wide call).
__device__ __forceinline__ int row_of_position(const K1Params& p, int pos, int lane) {
    const int sorted_row = p.meta.srt[pos];            // requested together with the segment index (one latency, not two)
    int n_all, n_ad;
    segment_totals(p.meta, p.L, lane, n_all, n_ad);
    n_all = min(n_all, p.M);
    return (n_ad > 0 && pos < n_all) ? min(max(sorted_row, 0), p.M - 1) : pos;
}

// NT threads (tid in [0, NT)) that meet at named barrier BAR quantize row `row` of x into position `pos`.
template <int NT, int BAR, bool XOP = false>
__device__ void quantize_row(const K1Params& p, int pos, int row, int tid) {
    __shared__ float s_part[NT / 32];
    __shared__ float s_scale;
    const int lane = tid & 31, warp = tid >> 5;
    const __nv_bfloat16* xr = p.x + (int64_t)row * p.ldx;
    const int nvec = p.K >> 3;
    // Pass 1: every load of the row in flight at once (the loop is short code: a row has at most a few vectors per thread).
    float amax = 0.0f;
#pragma unroll 4
    for (int i = tid; i < nvec; i += NT) amax = fmaxf(amax, amax8(x_load8<XOP>(p, xr, i * 8)));
#pragma unroll
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0) s_part[warp] = amax;
    named_bar_sync<BAR, NT>();
    if (tid == 0) {
        float m = s_part[0];
        for (int w = 1; w < NT / 32; ++w) m = fmaxf(m, s_part[w]);
        const float sx = fmaxf(__fdiv_rn(m, kFp8Max), kMinTokenScale);
        s_scale = sx;
        p.sx[pos] = sx;
    }
    named_bar_sync<BAR, NT>();
    const float sx = s_scale;
    uint2* out = reinterpret_cast<uint2*>(p.xq + (size_t)pos * (size_t)p.K);
    // Pass 2 re-reads the row (it is in L1 now) in a rolled loop: the eight IEEE divisions per vector are long code, and a
    // batch runs this code on few SMs, so every instruction line of an unrolled copy would be fetched cold.
#pragma unroll 1
    for (int i = tid; i < nvec; i += NT) out[i] = quant8(x_load8<XOP>(p, xr, i * 8), sx);
    named_bar_sync<BAR, NT>();                        // s_part / s_scale may be reused by the group's next position
}

// The same quantization for the prefill launches' one-row CTAs, with the row held in registers between the two passes
// (NV vectors of 8 elements per thread: K <= 8 * NV * NT) and the adapter-sorted bf16 copy written from the same
// registers: thousands of such CTAs keep the code warm, so the unrolled second pass costs no cold fetches, and a row
// of up to 4096 elements needs so few registers that eight CTAs share an SM.
template <int NT, int BAR, int NV>
__device__ void quantize_row_regs(const K1Params& p, int pos, int row, int tid) {
    __shared__ float s_part[NT / 32];
    __shared__ float s_scale;
    const int lane = tid & 31, warp = tid >> 5;
    const __nv_bfloat16* xr = p.x + (int64_t)row * p.ldx;
    const int nvec = p.K >> 3;
    uint4 v[NV];
    float amax = 0.0f;
#pragma unroll
    for (int q = 0; q < NV; ++q) {
        const int i = tid + q * NT;
        v[q] = i < nvec ? __ldg(reinterpret_cast<const uint4*>(xr + i * 8)) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int q = 0; q < NV; ++q) amax = fmaxf(amax, amax8(v[q]));
#pragma unroll
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0) s_part[warp] = amax;
    if (p.xs != nullptr) {                            // the tensor-core shrink reads x in position order by TMA
        uint4* xo = reinterpret_cast<uint4*>(p.xs + (size_t)pos * (size_t)p.K);
#pragma unroll
        for (int q = 0; q < NV; ++q) {
            const int i = tid + q * NT;
            if (i < nvec) xo[i] = v[q];
        }
    }
    named_bar_sync<BAR, NT>();
    if (tid == 0) {
        float m = s_part[0];
        for (int w = 1; w < NT / 32; ++w) m = fmaxf(m, s_part[w]);
        const float sx = fmaxf(__fdiv_rn(m, kFp8Max), kMinTokenScale);
        s_scale = sx;
        p.sx[pos] = sx;
    }
    named_bar_sync<BAR, NT>();
    const float sx = s_scale;
    uint2* out = reinterpret_cast<uint2*>(p.xq + (size_t)pos * (size_t)p.K);
#pragma unroll
    for (int q = 0; q < NV; ++q) {
        const int i = tid + q * NT;
        if (i < nvec) out[i] = quant8(v[q], sx);
    }
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x); f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
    f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z); f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}

// e2m1 code of v (bit 3 = sign): round to nearest even on {0,.5,1,1.5,2,3,4,6}, saturating -- the threshold chain of
// lowbit_lora/kernels/nvfp4_lora_vllm.py:70-76 (ties .25/1.25/2.5/5 go down, .75/1.75/3.5 go up).
__device__ __forceinline__ uint32_t e2m1_code(float v) {
    const float a = fabsf(v);
    const uint32_t mag = (uint32_t)(a > 0.25f) + (uint32_t)(a >= 0.75f) + (uint32_t)(a > 1.25f) + (uint32_t)(a >= 1.75f) +
                         (uint32_t)(a > 2.5f) + (uint32_t)(a >= 3.5f) + (uint32_t)(a > 5.0f);
    return mag | (v < 0.0f ? 8u : 0u);
}

__device__ __forceinline__ float e4m3_to_float(uint32_t code) {
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((uint16_t)code));
    return __half2float(__ushort_as_half((unsigned short)(h2 & 0xFFFFu)));
}

// NVFP4 activation quantization of one position (vLLM's scaled_fp4_quant recipe, lowbit_lora/kernels/nvfp4_lora_vllm.py:
// 102-115 / 361-376): per 16-element block sf = e4m3_rn(min(gs * (blockmax * rcp(6)), 448)), out_scale = sf != 0 ?
// rcp(sf * rcp(gs)) : 0, code = e2m1_rn(x * out_scale); codes packed two per byte (element 2i in the low nibble).  One
// thread per block.  The scales go straight into K2's scale-factor atoms: [token tile][K slot][128-token block][MMA][r%32]
// [r/32][4], r = position within the token tile.
// COPY: also write the row's bf16 values to the adapter-sorted copy p.xs (prefill: the tensor-core shrink's input) from
// the vectors just loaded, instead of a second pass over the row.
template <int NT, bool XOP = false, bool COPY = false>
__device__ void quantize_row_nvfp4(const K1Params& p, int pos, int row, int tid) {
    const float gs = __ldg(p.x_global);
    const __nv_bfloat16* xr = p.x + (int64_t)row * p.ldx;
    const float rcp6 = p.rcp_approx ? rcp_approx_ftz(6.0f) : __frcp_rn(6.0f);
    const float rgs = p.rcp_approx ? rcp_approx_ftz(gs) : __frcp_rn(gs);
    const int nblocks = p.K >> 4;
    const int mt = pos / p.tn, r = pos % p.tn;
    uint8_t* sf_tile = p.xsf + (size_t)mt * p.kslots * p.nblk * kSfSlotBytes;
    const int sf_row = (r >> 7) * kSfSlotBytes + (r & 31) * 16 + ((r & 127) >> 5) * 4;
    for (int b = tid; b < p.kslots * 16; b += NT) {
        uint32_t sf_code = 0;
        if (b < nblocks) {
            float v[16];
            const uint4 u0 = x_load8<XOP>(p, xr, 16 * b), u1 = x_load8<XOP>(p, xr, 16 * b + 8);
            if (COPY && p.xs != nullptr) {
                uint4* xo = reinterpret_cast<uint4*>(p.xs + (size_t)pos * (size_t)p.K) + 2 * b;
                xo[0] = u0;
                xo[1] = u1;
            }
            unpack8(u0, *reinterpret_cast<float(*)[8]>(&v[0]));
            unpack8(u1, *reinterpret_cast<float(*)[8]>(&v[8]));
            float vmax = 0.0f;
#pragma unroll
            for (int e = 0; e < 16; ++e) vmax = fmaxf(vmax, fabsf(v[e]));
            const float sfv = fminf(__fmul_rn(gs, __fmul_rn(vmax, rcp6)), 448.0f);
            sf_code = (uint32_t)cvt_e4m3x2(sfv, 0.0f) & 0xFFu;
            const float sff = e4m3_to_float(sf_code);
            float osc = 0.0f;
            if (sff != 0.0f) {
                const float den = __fmul_rn(sff, rgs);
                osc = p.rcp_approx ? rcp_approx_ftz(den) : __frcp_rn(den);
            }
            uint32_t lo = 0, hi = 0;
            // The sign bit of a code: the torch recipe sets it for values below zero (so -0.0 and negative values under a
            // zero block scale encode as +0), vLLM's CUDA kernel converts with cvt.rn.satfinite.e2m1x2.f32, which keeps the
            // product's own sign bit (they encode as -0: code 8).  Each mode follows its model, bit for bit.
            const uint32_t approx = p.rcp_approx ? 1u : 0u;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float a = __fmul_rn(v[e], osc), b = __fmul_rn(v[8 + e], osc);
                uint32_t ca = e2m1_code(a), cb = e2m1_code(b);
                if (approx) {
                    ca = (ca & 7u) | ((__float_as_uint(a) >> 31) << 3);
                    cb = (cb & 7u) | ((__float_as_uint(b) >> 31) << 3);
                }
                lo |= ca << (4 * e);
                hi |= cb << (4 * e);
            }
            *reinterpret_cast<uint2*>(p.xq + (size_t)pos * (size_t)(p.K >> 1) + (size_t)b * 8) = make_uint2(lo, hi);
        }
        // K slot b / 16, MMA (b % 16) / 4, scale b % 4; blocks past K are zero scales
        sf_tile[(size_t)(b >> 4) * p.nblk * kSfSlotBytes + sf_row + ((b & 15) >> 2) * 512 + (b & 3)] = (uint8_t)sf_code;
    }
}

// 32 lane-partial values per lane -> lane i holds the warp-wide sum of value i (31 shuffles).
__device__ __forceinline__ float transpose_reduce32(float (&v)[32], int lane) {
#pragma unroll
    for (int off = 16, n = 32; off >= 1; off >>= 1, n >>= 1) {
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < n / 2; ++i) {
            const float send = upper ? v[i] : v[i + n / 2];
            const float keep = upper ? v[i + n / 2] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
    }
    return v[0];
}

// The 8 rank rows a warp owns, in the adapter's storage format: bf16, e4m3 codes (fp32 scale per row, applied after the
// dot) or packed e2m1 codes with one ue4m3 scale per 16 elements (and one fp32 global per adapter and slice, applied
// after the dot) -- lowbit_lora/kernels/fp8_lora_vllm.py:85-118.  A lane always covers 8 consecutive K elements of each
// row: 16, 8 or 4 bytes of codes (+ 1 scale byte).
template <int FMT>
struct ARows {
    const uint8_t* base;      // row 0 of the 8 rows, element 0
    const uint8_t* sbase;     // NVFP4: block scales of row 0
    size_t row_bytes, srow_bytes;
    __device__ __forceinline__ ARows(const K1Params& p, int lora, int s, int rg) {
        const size_t row = (size_t)lora * p.R + (size_t)rg * 8;
        row_bytes = FMT == kLoraBf16 ? (size_t)p.K * 2 : FMT == kLoraFp8 ? (size_t)p.K : (size_t)p.K / 2;
        srow_bytes = (size_t)p.K / 16;
        base = static_cast<const uint8_t*>(p.a[s]) + row * row_bytes;
        sbase = FMT == kLoraNvfp4 ? static_cast<const uint8_t*>(p.sa[s]) + row * srow_bytes : nullptr;
    }
    // raw codes of the lane's 8 elements at column k of each row (x: codes; y: the block's scale byte for NVFP4)
    __device__ __forceinline__ void load(uint4 (&av)[8], int k, bool act) const {
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (act) {
                if (FMT == kLoraBf16) {
                    v = __ldg(reinterpret_cast<const uint4*>(base + r * row_bytes + (size_t)k * 2));
                } else if (FMT == kLoraFp8) {
                    const uint2 c = __ldg(reinterpret_cast<const uint2*>(base + r * row_bytes + (size_t)k));
                    v.x = c.x; v.y = c.y;
                } else {
                    v.x = __ldg(reinterpret_cast<const uint32_t*>(base + r * row_bytes + (size_t)k / 2));
                    v.y = __ldg(sbase + r * srow_bytes + (size_t)k / 16);
                }
            }
            av[r] = v;
        }
    }
};

__device__ __forceinline__ float2 e4m3x2_to_float2(uint32_t two_codes) {
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((uint16_t)two_codes));
    return __half22float2(*reinterpret_cast<__half2*>(&h2));
}

__device__ __forceinline__ float e2m1_value(uint32_t code) {
    const uint32_t mag = code & 7u;
    float v = __uint_as_float(0x3F000000u + (mag << 22));          // magnitudes 2..7: 1, 1.5, 2, 3, 4, 6
    v = mag == 0 ? 0.0f : (mag == 1 ? 0.5f : v);
    return (code & 8u) ? -v : v;
}

template <int FMT>
__device__ __forceinline__ void unpack_a(const uint4& v, float (&f)[8]) {
    if (FMT == kLoraBf16) {
        unpack8(v, f);
    } else if (FMT == kLoraFp8) {
        const float2 a = e4m3x2_to_float2(v.x & 0xFFFFu), b = e4m3x2_to_float2(v.x >> 16);
        const float2 c = e4m3x2_to_float2(v.y & 0xFFFFu), d = e4m3x2_to_float2(v.y >> 16);
        f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
    } else {
        const float sf = e4m3_to_float(v.y & 0xFFu);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = e2m1_value((v.x >> (4 * e)) & 15u) * sf;    // exact in bf16, as the reference notes
    }
}

// Scale applied to a finished dot product: the row's fp32 scale (FP8-stored) or the adapter's inverse global (NVFP4-stored).
template <int FMT>
__device__ __forceinline__ float post_scale(const K1Params& p, int lora, int s, int row_in_slice) {
    if (FMT == kLoraFp8) return __ldg(static_cast<const float*>(p.sa[s]) + (size_t)lora * p.R + row_in_slice);
    if (FMT == kLoraNvfp4) return __ldg(p.ag + (size_t)s * p.L + lora);
    return 1.0f;
}

// One pass of a warp: 8 rank rows [k0, k1) of adapter `lora`, slice s, times the `nt` (<= 4) tokens whose x rows are
// rows[0..nt); writes the split-K partial hp[j][s][pos0 + t][rg*8 .. +8].  bf16 adapters.  The first block of A is
// requested before the wait on the preceding kernel (A is static); x is read and hp written only after it.
template <int FMT, bool XOP = false>
__device__ __forceinline__ void shrink_pass(const K1Params& p, int lora, int s, int rg, int j, int k0, int k1, int pos0,
                                                 const int* rows, int nt, int lane) {
    const ARows<FMT> a(p, lora, s, rg);
    uint4 av[8];
    a.load(av, k0 + lane * 8, k0 + lane * 8 < k1);
    OB_TRACE1(1)
    griddep_wait();
    OB_TRACE1(2)
    const __nv_bfloat16* xrow[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) xrow[t] = p.x + (int64_t)rows[t < nt ? t : 0] * p.ldx;
    float acc[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) acc[i] = 0.0f;
    for (int kk = k0; kk < k1; kk += 256) {
        const int k = kk + lane * 8;
        const bool act = k < k1;
        float xf[4][8];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            if (t < nt && act) {
                unpack8(x_load8<XOP>(p, xrow[t], k), xf[t]);
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) xf[t][e] = 0.0f;
            }
        }
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            float af[8];
            unpack_a<FMT>(av[r], af);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                float sacc = acc[r * 4 + t];
#pragma unroll
                for (int e = 0; e < 8; ++e) sacc = fmaf(af[e], xf[t][e], sacc);
                acc[r * 4 + t] = sacc;
            }
        }
        if (kk + 256 < k1) a.load(av, k + 256, k + 256 < k1);
    }
    const float total = transpose_reduce32(acc, lane);
    const int r = lane >> 2, t = lane & 3;
    if (t < nt) p.hp[(((size_t)j * p.S + s) * p.max_m + (pos0 + t)) * p.R + rg * 8 + r] = total * post_scale<FMT>(p, lora, s, rg * 8 + r);
}

template <int FMT>
__device__ __forceinline__ void fma8(float (&acc)[8], const uint4 (&av)[8], const float (&xf)[8]) {
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        float af[8];
        unpack_a<FMT>(av[r], af);
        float sacc = acc[r];
#pragma unroll
        for (int e = 0; e < 8; ++e) sacc = fmaf(af[e], xf[e], sacc);
        acc[r] = sacc;
    }
}

// Decode form of the pass (one token): two K steps of A in flight per lane (8 KB per warp), both requested before the wait
// on the preceding kernel.  8 lane-partials -> lanes 0..7 hold the 8 rank rows' sums (2 butterfly + 3 transposing steps).
template <int FMT, bool XOP = false>
__device__ __forceinline__ void shrink_pass1(const K1Params& p, int lora, int s, int rg, int j, int k0, int k1, int pos,
                                                  int row, int lane) {
    const ARows<FMT> a(p, lora, s, rg);
    const int kl = k0 + lane * 8;
    uint4 a0[8], a1[8];
    a.load(a0, kl, kl < k1);
    a.load(a1, kl + 256, kl + 256 < k1);
    OB_TRACE1(1)
    griddep_wait();
    OB_TRACE1(2)
    const __nv_bfloat16* xrow = p.x + (int64_t)row * p.ldx;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
    for (int k = kl; k < k1; k += 512) {
        float x0[8], x1[8];
        unpack8(x_load8<XOP>(p, xrow, k), x0);
        if (k + 256 < k1) {
            unpack8(x_load8<XOP>(p, xrow, k + 256), x1);
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) x1[e] = 0.0f;
        }
        fma8<FMT>(acc, a0, x0);
        a.load(a0, k + 512, k + 512 < k1);
        fma8<FMT>(acc, a1, x1);
        a.load(a1, k + 768, k + 768 < k1);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], 16);
        acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], 8);
    }
#pragma unroll
    for (int off = 4, n = 8; off >= 1; off >>= 1, n >>= 1) {
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < n / 2; ++i) {
            const float send = upper ? acc[i] : acc[i + n / 2];
            const float keep = upper ? acc[i + n / 2] : acc[i];
            acc[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
    }
    if (lane < 8) p.hp[(((size_t)j * p.S + s) * p.max_m + pos) * p.R + rg * 8 + lane] = acc[0] * post_scale<FMT>(p, lora, s, rg * 8 + lane);
}

// One warp: block `pb` of p.pb consecutive sorted positions, unit `u` -> (slice, group of 8 rank rows, K split).
// One warp-wide read of the segment index gives the batch totals and the segment (adapter) of each of the warp's
// positions; the positions' token rows are requested at the same time.  Then one pass per run of positions that share
// an adapter.
template <int FMT, bool XOP = false>
__device__ void shrink_unit(const K1Params& p, int pb, int u, int lane) {
    const int p0 = pb * p.pb;
    int rows[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        int r = (q < p.pb && p0 + q < p.M) ? p.meta.srt[p0 + q] : 0;
        rows[q] = r < 0 ? 0 : (r > p.M - 1 ? p.M - 1 : r);
    }
    int lora_of[4] = {-1, -1, -1, -1};
    int n_all = 0, n_ad = 0;
    for (int base = 0; base <= p.L; base += 32) {
        const int i = base + lane;
        int id = -1, st = 0, cnt = 0;
        if (i <= p.L) {
            id = p.meta.seg_ids[i];
            st = p.meta.seg_start[i];
            cnt = p.meta.seg_n[i];
        }
        n_all += cnt;
        n_ad += id >= 0 ? cnt : 0;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const bool hit = q < p.pb && id >= 0 && id < p.L && st <= p0 + q && p0 + q < st + cnt;
            const uint32_t m = __ballot_sync(0xffffffffu, hit);
            if (m) lora_of[q] = __shfl_sync(0xffffffffu, id, __ffs(m) - 1);
        }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        n_all += __shfl_xor_sync(0xffffffffu, n_all, o);
        n_ad += __shfl_xor_sync(0xffffffffu, n_ad, o);
    }
    n_all = min(n_all, p.M);
    if (n_ad <= 0) return;
    const int np = min(p.pb, n_all - p0);
    if (np <= 0) return;
    const int groups = p.R >> 3;
    const int j = u % p.split1;
    const int rg = (u / p.split1) % groups;
    const int s = u / (p.split1 * groups);
    const int k0 = j * p.k_per_split;
    const int k1 = min(p.K, k0 + p.k_per_split);
    if (p.pb == 1) {
        if (lora_of[0] >= 0) shrink_pass1<FMT, XOP>(p, lora_of[0], s, rg, j, k0, k1, p0, rows[0], lane);
        return;
    }
    int q = 0;
    while (q < np) {
        const int lora = lora_of[q];
        int nt = 1;
        while (q + nt < np && lora_of[q + nt] == lora) ++nt;
        if (lora >= 0) shrink_pass<FMT, XOP>(p, lora, s, rg, j, k0, k1, p0 + q, rows + q, nt, lane);
        q += nt;
    }
}

}  // namespace ob
