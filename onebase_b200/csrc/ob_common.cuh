// Shared between the kernels and the C-ABI: the workspace layout, kernel parameter blocks and the position rule.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/onebase_b200.h"

namespace ob {

constexpr int kTileN = 128;          // output features per GEMM tile (rows of W; the MMA's M)
constexpr int kBlockK = 128;         // bytes of K per ring stage row (one 128-byte swizzle row)
constexpr int kMaxLoraIters = 512;   // capacity of a CTA's list of (segment, rank chunk) expand steps
constexpr int kMaxTileTenants = 128;  // tenants with a position in one 128-position block
constexpr int kBigTileMinTokens = 128; // larger batches of bf16 adapters take the large-tile prefill GEMM (k2_prefill.cu)
constexpr int kMmaShrinkGroup = 4;      // tenants of a 128-position tile per CTA of the tensor-core shrink
constexpr int kMmaShrinkTokens = 512;   // batches from this size on shrink on the tensor cores (bf16 adapters)
constexpr int kDecodeTokens = 32;     // batches up to this size take the decode forms (one position per shrink warp)
constexpr int kCounterSlots = 4096;  // split-K arrival counters in the workspace
constexpr int kStreamMaxCtas = 256;  // most CTAs of the persistent decode GEMM (one per SM)
constexpr int kSfSlotBytes = 2048;
// Peer-memory all-reduce: layout of a rank's communication buffer (see allreduce.cu)
constexpr int kArStateBytes = 16384;  // state words, rank flags, per-tile flags; the staged copies follow
constexpr int kArFlagsOff = 1024, kArFlags2Off = 2048, kArTileFlagsOff = 4096;
constexpr int kArMaxTiles = 384;      // per-tile flags [world][kArMaxTiles] of the all-reduce fused into K2's epilogue   // NVFP4: scale factors of 128 rows x one 256-element K slot (4 atoms of 512 bytes)

__host__ __device__ inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Offsets of the regions inside the shared workspace (bytes).  All regions are 1024-byte aligned.
struct WorkspaceLayout {
    size_t status;     // int32 [OB_STATUS_WORDS]
    size_t counters;   // int32 [kCounterSlots]   zero between launches
    size_t sx;         // fp32  [max_m]           per-position activation scale
    size_t xq;         // bytes [max_m * max_k]   quantized activations, row pitch = the calling layer's K (FP8) or K/2
    size_t xsf;        // bytes NVFP4 activation block scales: [token tile][256-element K slot][128-token block][2048]
    size_t hp;         // fp32  [max_split1 * max_sr * max_m]  shrink partials [split][slice][position][rank]
    size_t part;       // fp32  [max_split2 * token tile * (max_n rounded to tiles)]  GEMM split-K partials
    size_t xs;         // bf16  [max_m * max_k]   adapter-sorted copy of x for the tensor-core shrink (max_m > 32 only)
    size_t hb;         // bf16  [max_sr * max_m]  the tensor-core shrink's finished h [slice][position][rank] (max_m > 32 only)
    size_t hcat;       // bf16  [max_sr * max_m * min(max_l, 128)]  per-tenant h blocks of the large-tile prefill GEMM
    size_t total;
};

__host__ __device__ inline WorkspaceLayout workspace_layout(const ObWorkspaceShape& s) {
    WorkspaceLayout l;
    size_t off = 0;
    l.status = off;   off = align_up(off + sizeof(int32_t) * OB_STATUS_WORDS, 1024);
    l.counters = off; off = align_up(off + sizeof(int32_t) * (kCounterSlots + 16), 1024);   // + chain flags (x_q ready, CTAs done)
    l.sx = off;       off = align_up(off + sizeof(float) * (size_t)s.max_m, 1024);
    l.xq = off;       off = align_up(off + (size_t)s.max_m * (size_t)s.max_k, 1024);
    l.xsf = off;      off = align_up(off + ((size_t)s.max_m + 15) / 16 * (((size_t)s.max_k + 255) / 256) * kSfSlotBytes, 1024);
    l.hp = off;       off = align_up(off + sizeof(float) * (size_t)s.max_split1 * (size_t)s.max_sr * (size_t)s.max_m, 1024);
    const size_t n_pad = align_up((size_t)s.max_n, kTileN) + (size_t)OB_MAX_SLICES * kTileN;
    size_t m_pad = 16;                                        // split-K serves one token tile: min(max_m, 256) tokens
    while (m_pad < (size_t)s.max_m && m_pad < 256) m_pad *= 2;
    // ... or the persistent decode GEMM's partial tiles: two of 32 tokens x 128 features per CTA
    const size_t units_cap = (n_pad / kTileN) * (((size_t)s.max_k + kBlockK - 1) / kBlockK);
    const size_t stream_part = (size_t)2 * (units_cap < (size_t)kStreamMaxCtas ? units_cap : (size_t)kStreamMaxCtas) * kDecodeTokens * kTileN;
    const size_t split_part = s.max_split2 > 1 ? (size_t)s.max_split2 * m_pad * n_pad : 0;
    l.part = off;     off = align_up(off + sizeof(float) * (split_part > stream_part ? split_part : stream_part), 1024);
    l.xs = off;       off = align_up(off + (s.max_m > kDecodeTokens ? (size_t)s.max_m * (size_t)s.max_k * 2 : 0), 1024);
    l.hb = off;       off = align_up(off + (s.max_m > kDecodeTokens ? (size_t)s.max_sr * (size_t)s.max_m * 2 : 0), 1024);
    const size_t lc = s.max_l < kMaxTileTenants ? (s.max_l > 0 ? s.max_l : 0) : kMaxTileTenants;
    l.hcat = off;     off = align_up(off + (s.max_m > kBigTileMinTokens ? (size_t)s.max_sr * (size_t)s.max_m * lc * 2 : 0), 1024);
    l.total = off;
    return l;
}

// vLLM's five metadata tensors.
struct Meta {
    const int32_t* tok;
    const int32_t* srt;
    const int32_t* seg_n;
    const int32_t* seg_start;
    const int32_t* seg_ids;
};

enum : int { kLoraBf16 = OB_LORA_BF16, kLoraFp8 = OB_LORA_FP8, kLoraNvfp4 = OB_LORA_NVFP4 };

struct K1Params {
    int M, K, S, R, L;
    int lora_fmt;
    int split1;            // K splits of the shrink
    int k_per_split;       // elements of K per split (multiple of the warp's K step)
    int n_quant_ctas;      // leading CTAs that quantize (one position each)
    int looped;            // 1: the grid is capped at one CTA per SM; every warp walks the shrink units with the grid's stride
    int pb;                // sorted positions per shrink warp: 1 (decode) or 4
    int n_pblocks;         // ceil(M / pb)
    int units_per_block;   // shrink warps per position block: S * (R / 8) * split1
    const __nv_bfloat16* x;
    int64_t ldx;
    int x_op;              // OB_X_SILU_MUL: x is [M, 2K] (gate | up) and the projection's input is bf16(bf16(silu(g)) * u)
    Meta meta;
    const void* a[OB_MAX_SLICES];
    const void* sa[OB_MAX_SLICES];
    const float* ag;
    uint8_t* xq;           // [M, K] codes at sorted positions
    float* sx;             // [M]
    float* hp;             // [split1][S][max_m][R]
    int max_m;
    int base_fmt;          // OB_BASE_FP8: per-token e4m3 quantization; OB_BASE_NVFP4: e2m1 codes + ue4m3 scale per 16
    int tn, nblk, kslots;  // NVFP4: K2's token tile, its 128-token scale blocks, 256-element K slots (scale layout)
    int rcp_approx;        // NVFP4: 1 = rcp.approx.ftz reciprocals (vLLM's CUDA quantizer), 0 = IEEE (the torch recipe)
    const float* x_global; // NVFP4: [1] static activation global scale
    uint8_t* xsf;          // NVFP4: activation block scales, packed per (token tile, K slot) in scale-factor atoms
    __nv_bfloat16* xs;     // prefill with a tensor-core shrink: the quantizing CTAs also copy their row here (null: no copy)
    int32_t* xq_ready;     // chain: counts the positions whose codes and scale are written (null: no signal)
    unsigned long long* trace;   // optional timeline buffer (null: off); K1 stamps go after K2's region
    long long trace_ctas;
};

// The tensor-core shrink of a prefill batch (k1_mma.cu).
struct K1mParams {
    int M, K, S, R, L, max_m;
    int split1;            // K splits (grid z); K2 adds the partials in split order
    int k_per_split;       // elements of K per split, a multiple of 64
    int ring_bytes;        // shared memory of the operand ring
    uint32_t wait_ms;
    Meta meta;
    float* hp;             // [split1][S][max_m][R] partials (split1 > 1)
    __nv_bfloat16* hb;     // [S][max_m][R] the finished h: bf16 of the partials' sum in split order
    // Large-tile prefill GEMM: instead of hb, block (position, list entry) of hcat [S][max_m][lc * R] receives
    // h / (s_x[position] * s_w) for the entry that is the position's tenant and zeros for the block's other entries, so
    // that the GEMM can add the expand into the base accumulator with plain TMA tiles (no masking, one final scale).
    __nv_bfloat16* hcat;   // null: write hb
    int lc;                // list entries per position in hcat: min(L, 128)
    const float* sx;       // [max_m] per-position activation scales (K1's)
    const float* s_w;      // [1]
    int32_t* counters;     // one arrival counter per (position tile, slice); zero between launches
    int32_t* status;
    int tg_cap;            // tenants of a tile per CTA (work item = tile x tenant group; grid x = the host's bound on their number)
    int cluster;           // the K splits of a (tile, slice) were launched as one thread-block cluster (grid z): their partial
                           // rows are added over distributed shared memory instead of the workspace and the counters
};

// The large-tile prefill GEMM (k2_prefill.cu): FP8 base 256 x 256, NVFP4 base 128 x 256; bf16 adapters.
struct K2pParams {
    int M, N, K, S, R, L;
    int widths[OB_MAX_SLICES];
    int kblocks;           // 128-byte k-blocks of a W row: ceil(K / 128), NVFP4 ceil(K / 256)
    int stages;
    const uint8_t* wsf;    // NVFP4: packed W block scales [128-row tile][k-block][2 KB]
    const uint8_t* xsf;    // NVFP4: K1's activation block scales [256-token tile][k-block][2][2 KB]
    int lc;                // list entries per position in hcat
    int max_m;
    uint32_t wait_ms;
    const float* s_w;
    const float* sx;
    Meta meta;
    __nv_bfloat16* y;
    int64_t ldy;
    int32_t* status;
};

struct K2Params {
    int M, N, K, S, R, L;
    int widths[OB_MAX_SLICES];
    int lora_fmt;
    int tn;                // tokens per tile (MMA N)
    int split2;            // GEMM split-K
    int m_fast;            // several token tiles: grid x walks the token tiles and grid z the output tiles
    int cluster_reduce;    // split2 > 1: the splits of a tile form one thread-block cluster and add their partials through shared memory
    int split1;            // shrink partials to sum
    int kblocks;           // ceil(K / 128)
    int n_tiles;           // persistent decode kernel: 128-wide output tiles over all slices
    int stages;
    int rc;                // rank chunk per expand step: min(R, 64)
    int nh;                // masked H tiles in flight (expand steps the builder may run ahead of the B tiles)
    int max_m;
    uint32_t wait_ms;
    const float* s_w;
    const float* sx;
    const float* hp;
    const __nv_bfloat16* hb;   // prefill after the tensor-core shrink: finished h [S][max_m][R] (null: sum hp's partials)
    Meta meta;
    __nv_bfloat16* y;
    int64_t ldy;
    const __nv_bfloat16* residual;   // y = bf16(bf16(acc) + residual) (null: plain store)
    int64_t ldr;
    float* part;
    int32_t* counters;
    int32_t* status;
    const void* b[OB_MAX_SLICES];
    const void* sb[OB_MAX_SLICES];
    int b_staged;          // stored adapters: a step's codes and scales come by bulk copy into its ring slot (see k2_gemm.cu)
    int b_row0[OB_MAX_SLICES];   // first output feature of each slice whose B rows this rank holds (0 unless B is sharded)
    int b_rows[OB_MAX_SLICES];   // number of those rows (the slice's width unless B is sharded)
    const float* bg;
    const uint8_t* wsf;    // NVFP4 base: W block scales, packed per (128-row tile, 256-element K slot) in scale-factor atoms
    const uint8_t* xsf;    // NVFP4 base: K1's activation block scales, packed per (token tile, K slot)
    const float* alpha;    // NVFP4 base: [1] 1 / (x_global * w_global)
    int nblk;              // NVFP4 base: 128-token scale-factor blocks per token tile (1, or 2 for 256-token tiles)
    int32_t* xq_ready;     // chain: K1's count of quantized positions; the producer polls it instead of waiting for all of K1
    int32_t* chain_done;   // chain: CTAs of this launch that finished; the last one clears the chain's words
    int32_t* work_quant;   // fused: next position to quantize (claimed by a CTA's four epilogue warps together)
    int32_t* work_shrink;  // fused: next shrink unit (claimed by one warp)
    int32_t* hp_ready;     // fused: shrink units finished
    int shrink_units;      // fused: position blocks x units per block
    unsigned long long* trace;   // optional timeline buffer (null: off)
    long long trace_ctas;
    // All-reduce fused into the epilogue (row-parallel layers under tensor parallelism; ar_world = 0: off): a finished tile is
    // staged in this rank's communication buffer, announced to every peer by a per-tile flag, and the CTA then adds the
    // ranks' copies of ITS tile in rank order and stores y -- no separate all-reduce launch, no second pass over y.
    int ar_world, ar_rank;
    long long ar_slot_bytes;
    uint8_t* ar_bufs[OB_MAX_RANKS];
};

// Warp-wide: n_all = sum of seg_n, n_ad = sum of seg_n over segments whose slot id >= 0 (L+1 segments).
__device__ __forceinline__ void segment_totals(const Meta& m, int L, int lane, int& n_all, int& n_ad) {
    int a = 0, d = 0;
    for (int i = lane; i <= L; i += 32) {
        const int c = m.seg_n[i];
        a += c;
        d += (m.seg_ids[i] >= 0) ? c : 0;
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, o);
        d += __shfl_xor_sync(0xffffffffu, d, o);
    }
    n_all = a;
    n_ad = d;
}

// Row of x / y that tile position p stands for: the adapter-sorted order when the batch has an adapter and p is a real
// token, else the position itself (no-adapter batches, CUDA-graph padding).  Indices are clamped as a last guard.
__device__ __forceinline__ int position_row(const Meta& m, int p, int M, int n_all, int n_ad) {
    if (n_ad > 0 && p < n_all) {
        int r = m.srt[p];
        return r < 0 ? 0 : (r > M - 1 ? M - 1 : r);
    }
    return p;
}

}  // namespace ob
