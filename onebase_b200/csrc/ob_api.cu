// The C ABI (include/onebase_b200.h): argument validation, launch geometry, TMA descriptor construction, launches.
// Host code only allocates host memory; device memory always belongs to the caller.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "ob_common.cuh"

namespace ob {
size_t k2_fp8_smem_bytes(int tn, int stages, int rc, int R, int fp4);
cudaError_t launch_k2_nvfp4(const K2Params& p, const CUtensorMap& tm_w, const CUtensorMap& tm_x, const CUtensorMap* tm_b,
                            dim3 grid, size_t smem, int pdl, cudaStream_t stream);
int k2_fp8_h_tiles(int tn);
int k2_max_active_clusters(int fp4, int stored, int split2, size_t smem);
cudaError_t launch_k1_mma(const K1mParams& p, const CUtensorMap& tm_xs, const CUtensorMap* tm_a, dim3 grid, cudaStream_t stream);
cudaError_t launch_k2_prefill(const K2pParams& p, const CUtensorMap& tm_w, const CUtensorMap& tm_x, const CUtensorMap& tm_h,
                              const CUtensorMap* tm_b, dim3 grid, int fp4, int pdl, cudaStream_t stream);
int k2_prefill_max_steps();
cudaError_t launch_k2_prefill_pair(const K2pParams& p, const CUtensorMap& tm_w, const CUtensorMap& tm_x, const CUtensorMap& tm_h,
                                   const CUtensorMap* tm_b, const CUtensorMap* tm_sf, int pairs, int fp4, int pdl,
                                   cudaStream_t stream);
int k2_prefill_pair_capacity(int fp4);
int k2_prefill_pair_max_steps();
int k2_prefill_pair_rows(int fp4);
cudaError_t launch_requant_fp8(const void* src, long long rows, int cols, void* codes, float* scales, cudaStream_t stream);
cudaError_t launch_requant_nvfp4(const void* src, int l, int rows, int cols, void* packed, void* sf, float* inv_global,
                                 unsigned int* amax_bits, cudaStream_t stream);
cudaError_t launch_fused(const K2Params& p, const K1Params& k1, const CUtensorMap& tm_w, const CUtensorMap& tm_x,
                         const CUtensorMap* tm_b, dim3 grid, size_t smem, cudaStream_t stream);
cudaError_t launch_k1_fp8(const K1Params& p, int grid, int pdl, cudaStream_t stream);
cudaError_t launch_k2_fp8(const K2Params& p, const CUtensorMap& tm_w, const CUtensorMap& tm_x, const CUtensorMap* tm_b,
                          dim3 grid, size_t smem, int pdl, cudaStream_t stream);
size_t k2_stream_smem_bytes(int tn, int stages, int rc, int R, int S, int fp4);
int k2_stream_h_tiles(int tn);
cudaError_t launch_k2_stream(const K2Params& p, const CUtensorMap& tm_w, const CUtensorMap& tm_x, const CUtensorMap* tm_b,
                             int grid, size_t smem, int fp4, int pdl, cudaStream_t stream);
cudaError_t launch_pack_scales(const uint8_t* linear, int K, int S, const int32_t* widths, uint8_t* packed, size_t bytes,
                               cudaStream_t stream);
cudaError_t launch_segment_index(const int32_t* token_lora, int M, int L, int32_t* tok, int32_t* srt, int32_t* seg_n,
                                 int32_t* seg_start, int32_t* seg_ids, cudaStream_t stream);
struct ArParams {
    int world, rank;
    int dtype;
    int two_shot;
    long long count;
    long long slot_bytes;
    uint32_t wait_ms;
    const void* src;
    void* dst;
    uint8_t* bufs[OB_MAX_RANKS];
};
struct ArBatch {
    ArParams r[OB_MAX_RANKS];
};
cudaError_t launch_allreduce(const ArBatch& b, int n_emulated, int grid_x, cudaStream_t stream);
}  // namespace ob

using namespace ob;

namespace {

constexpr size_t kSmemLimit = 226 * 1024;    // dynamic part; the kernels keep a few static words besides
constexpr size_t kSmemStream = 216 * 1024;   // the persistent decode GEMM: leaves 10 KB of the SM for co-resident K1 CTAs
constexpr size_t kSmemTwoPerSm = 112 * 1024;   // two CTAs of this size (+1 KB reserved each) fit one SM's 228 KB

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
        else
            (void)cudaGetLastError();
    });
    return fn;
}

// 2-D row-major tensor [rows, inner] of `elem_bytes` elements -> tiled map with box [box_rows, box_inner], swizzle by the
// box's inner bytes (32 / 64 / 128); `linear` asks for an unswizzled box (rows of up to 256 elements, back to back).
int encode_2d(CUtensorMap* tm, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t inner, uint64_t rows,
              uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_rows, bool linear = false) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return OB_ERR_DRIVER;
    const uint32_t inner_bytes = box_inner * (uint32_t)elem_bytes;
    CUtensorMapSwizzle sw = inner_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                            : inner_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                            : inner_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                                : CU_TENSOR_MAP_SWIZZLE_NONE;
    if (linear) sw = CU_TENSOR_MAP_SWIZZLE_NONE;
    if ((sw == CU_TENSOR_MAP_SWIZZLE_NONE && !linear) || box_inner > 256 || box_rows > 256) return OB_ERR_SHAPE;
    cuuint64_t gdim[2] = {inner, rows};
    cuuint64_t gstride[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_inner, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(tm, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? OB_OK : 1000 + (int)r;
}

unsigned long long* g_trace = nullptr;
long long g_trace_ctas = 0;

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

struct XMap {
    const void* base;
    int rows, tn;
    CUtensorMap tm;
};

}  // namespace

struct ObLayer {
    ObLayerDesc d;
    int rc;                       // rank chunk of an expand step
    int n_tiles;                  // 128-wide output tiles over all slices
    CUtensorMap tm_w;
    CUtensorMap tm_b[OB_MAX_SLICES];
    CUtensorMap tm_a[OB_MAX_SLICES];   // bf16 adapters: A of each slice as [L * R, K], for the tensor-core shrink
    bool big_ok;                       // bf16 adapters of rank >= 64, slice widths in multiples of 256 (NVFP4 base: 128):
    CUtensorMap tm_w2;                 //   the large-tile prefill GEMM applies; FP8 base: W and B in 256-row boxes
    CUtensorMap tm_b2[OB_MAX_SLICES];
    CUtensorMap tm_wsf;                //   NVFP4 base: the packed W block scales as a [rows, 256] byte tensor (8 rows per atom)
    std::mutex mu;
    std::vector<XMap> xmaps;      // x_q maps by (workspace region, rows, token tile)
};

namespace {

int validate_desc(const ObLayerDesc* d) {
    if (!d) return OB_ERR_NULL;
    if (d->base_fmt != OB_BASE_FP8 && d->base_fmt != OB_BASE_NVFP4) return OB_ERR_FORMAT;
    if (d->lora_fmt != OB_LORA_BF16 && d->lora_fmt != OB_LORA_FP8 && d->lora_fmt != OB_LORA_NVFP4) return OB_ERR_FORMAT;
    if (d->N <= 0 || d->K <= 0 || d->K % 16 != 0 || d->S < 1 || d->S > OB_MAX_SLICES || d->L < 1 || d->L > 256 ||
        d->max_m < 1)
        return OB_ERR_SHAPE;
    if (!(d->R == 16 || d->R == 32 || d->R == 64 || d->R == 128 || d->R == 256)) return OB_ERR_SHAPE;
    int sum = 0;
    for (int s = 0; s < d->S; ++s) {
        if (d->widths[s] <= 0) return OB_ERR_SHAPE;
        sum += d->widths[s];
    }
    if (sum != d->N) return OB_ERR_SHAPE;
    if (!d->w_q) return OB_ERR_NULL;
    if (d->base_fmt == OB_BASE_FP8 && !d->s_w) return OB_ERR_NULL;
    if (d->base_fmt == OB_BASE_NVFP4 && (!d->w_sf || !d->x_global || !d->alpha)) return OB_ERR_NULL;
    if (d->base_fmt == OB_BASE_NVFP4 && d->K % 32 != 0) return OB_ERR_SHAPE;
    if (!aligned16(d->w_q) || (d->w_sf && !aligned16(d->w_sf))) return OB_ERR_ALIGN;
    for (int s = 0; s < d->S; ++s) {
        if (!d->a[s] || !d->b[s]) return OB_ERR_NULL;
        if (!aligned16(d->a[s]) || !aligned16(d->b[s])) return OB_ERR_ALIGN;
        if (d->lora_fmt != OB_LORA_BF16 && (!d->sa[s] || !d->sb[s])) return OB_ERR_NULL;
    }
    if (d->lora_fmt == OB_LORA_NVFP4 && (!d->ag || !d->bg)) return OB_ERR_NULL;
    for (int s = 0; s < d->S; ++s) {   // sharded B rows: whole 128-row tiles of the slice, bf16 adapters
        if (d->b_rows[s] == 0 && d->b_row0[s] == 0) continue;
        if (d->lora_fmt != OB_LORA_BF16) return OB_ERR_FORMAT;
        if (d->b_row0[s] < 0 || d->b_rows[s] <= 0 || d->b_row0[s] % kTileN != 0 || d->b_row0[s] + d->b_rows[s] > d->widths[s] ||
            (d->b_rows[s] % kTileN != 0 && d->b_row0[s] + d->b_rows[s] != d->widths[s]))
            return OB_ERR_SHAPE;
    }
    return OB_OK;
}

bool b_sharded(const ObLayerDesc& d) {
    for (int s = 0; s < d.S; ++s)
        if (d.b_rows[s] != 0) return true;
    return false;
}

int validate_batch(const ObLayer* l, const ObBatch* b) {
    if (!l || !b) return OB_ERR_NULL;
    if (b->M < 1 || b->M > l->d.max_m) return OB_ERR_BATCH;
    if (!b->x || !b->y || !b->tok || !b->srt || !b->seg_n || !b->seg_start || !b->seg_ids) return OB_ERR_NULL;
    if (b->x_op != OB_X_PLAIN && b->x_op != OB_X_SILU_MUL) return OB_ERR_FORMAT;
    if (!aligned16(b->x) || b->ldx < (b->x_op == OB_X_SILU_MUL ? 2 : 1) * (int64_t)l->d.K || b->ldx % 8 != 0) return OB_ERR_ALIGN;
    if (b->residual && ((reinterpret_cast<uintptr_t>(b->residual) & 1u) || b->ldr < l->d.N)) return OB_ERR_ALIGN;
    if ((reinterpret_cast<uintptr_t>(b->y) & 1u) || b->ldy < l->d.N) return OB_ERR_ALIGN;
    return OB_OK;
}

int validate_workspace(const ObLayer* l, const void* ws, const ObWorkspaceShape* sh, int split1, int split2) {
    if (!ws || !sh) return OB_ERR_NULL;
    if ((reinterpret_cast<uintptr_t>(ws) & 1023u) != 0) return OB_ERR_ALIGN;
    if (sh->max_m < l->d.max_m || sh->max_k < l->d.K || sh->max_n < l->d.N || sh->max_sr < l->d.S * l->d.R ||
        sh->max_split1 < split1 || sh->max_split2 < split2)
        return OB_ERR_WORKSPACE;
    return OB_OK;
}

int k_bytes(const ObLayerDesc& d) { return d.base_fmt == OB_BASE_NVFP4 ? d.K / 2 : d.K; }

struct Resolved {
    int tn, split1, split2, stages, m_tiles, k_per_split, pb, fused, mma_shrink, big;
    int stream;        // the persistent decode GEMM (k2_stream.cu) serves this call; `grid_s` CTAs, `stages` ring slots
    int grid_s;
    uint32_t wait_ms;
};

// Streaming multiprocessors of the current device (148 on a B200); 0 if it cannot be read.
int sm_count() {
    static std::mutex mu;
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { (void)cudaGetLastError(); return 0; }
    std::lock_guard<std::mutex> g(mu);
    if (dev >= 0 && dev < 64 && cached[dev] > 0) return cached[dev];
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) { (void)cudaGetLastError(); return 0; }
    if (dev >= 0 && dev < 64) cached[dev] = n;
    return n;
}

// Token tile by default: the smallest of 16..128 that covers the batch.  Prefill batches stay at 128-token tiles: two
// such CTAs share an SM (256 TMEM columns and a two-slot ring each), so one's epilogue runs under the other's main loop,
// which measured faster than one 256-token CTA per SM.
int default_tn(int M) {
    int tn = 16;
    while (tn < M && tn < 128) tn *= 2;
    return tn;
}

// Tenants with a position in one 128-position tile of an adapter-sorted batch, estimated for L tenants of equal size:
// 128 L / M of them and one more that straddles the tile's edge.
int shrink_tenants_per_tile(int L, int M) { return (int)std::min<long long>(L, (128LL * L + M - 1) / M + 1); }
// Tenants per CTA of the tensor-core shrink.  Tiles of six or more tenants are dealt out in groups of kMmaShrinkGroup
// to CTAs of their own (measured at 512 tokens over 32 tenants: K1 55-75 -> 32-52 us per projection); with fewer
// tenants per tile one CTA per tile measured better (no CTAs without a work item, one pass over the segment index).
int shrink_group_cap(int L, int M) { return shrink_tenants_per_tile(L, M) >= 6 ? kMmaShrinkGroup : kMaxTileTenants; }

int resolve_cfg(const ObLayer* l, int M, const ObTileCfg* cfg, Resolved* r) {
    const ObLayerDesc& d = l->d;
    const bool fp4 = d.base_fmt == OB_BASE_NVFP4;
    const int kblocks = (k_bytes(d) + kBlockK - 1) / kBlockK;
    r->tn = (cfg && cfg->tn) ? cfg->tn : default_tn(M);
    // NVFP4: the scale factors share tensor memory with the accumulators; 64-token tiles leave room for two CTAs per SM
    if (fp4 && r->tn > 64 && !(cfg && cfg->tn)) r->tn = 64;
    if (fp4 && r->tn > 128) return OB_ERR_TILE;   // (the large-tile prefill GEMM has its own 256-token tile: `big` below)
    if (!(r->tn == 16 || r->tn == 32 || r->tn == 64 || r->tn == 128 || r->tn == 256)) return OB_ERR_TILE;
    r->m_tiles = (M + r->tn - 1) / r->tn;
    // Decode batches of bf16 adapters may take the persistent GEMM (k2_stream.cu): one CTA per SM streams a contiguous share
    // of the launch's weight bytes.  ObTileCfg.stream = 1 (or LOWBIT_K2_STREAM=1 for every call) asks for it; 0 and 2 keep
    // the tile-per-CTA kernel, which measured as fast or faster on a B200 at every shape of the benchmark layer (the
    // persistent form's start-up, expand pipeline and shared-tile fix-ups cost what its weight stream gains).
    static const bool env_stream = [] { const char* v = std::getenv("LOWBIT_K2_STREAM"); return v && v[0] == '1'; }();
    r->stream = 0;
    r->grid_s = 0;
    {
        const int want = cfg ? cfg->stream : 0;
        const int sms = sm_count();
        const long long units = (long long)l->n_tiles * kblocks;
        if ((want == 1 || (env_stream && want != 2)) && !(cfg && cfg->fused) && sms > 0 &&
            M <= kDecodeTokens && r->tn <= 32 && r->m_tiles == 1 && d.lora_fmt == kLoraBf16 && l->n_tiles <= kCounterSlots &&
            (long long)(d.L < r->tn ? d.L : r->tn) * (d.R / l->rc) <= 256) {
            // Ring depth: measured on a B200, the stream rate does not grow beyond 4-6 slots (HBM, not latency, bounds it), and
            // the footprint must leave room for K1's CTAs (a few static bytes + 1 KB reserved each) on the same SM, or the
            // two kernels of a chain cannot overlap.
            int stages = (cfg && cfg->stages) ? cfg->stages : 4;
            if (stages > 16) stages = 16;
            while (stages > 3 && k2_stream_smem_bytes(r->tn, stages, l->rc, d.R, d.S, fp4 ? 1 : 0) > kSmemStream) --stages;
            if (fp4) while (stages > 3 && 4 * r->tn + 32 * stages > 512) --stages;   // tensor memory: four accumulators + scale columns
            if (stages >= 3 && k2_stream_smem_bytes(r->tn, stages, l->rc, d.R, d.S, fp4 ? 1 : 0) <= kSmemStream) {
                r->stream = 1;
                r->stages = stages;
                r->grid_s = (int)(units < sms ? units : sms);
                if (r->grid_s > kStreamMaxCtas) r->grid_s = kStreamMaxCtas;
            }
        }
    }
    int split2 = (cfg && cfg->split2) ? cfg->split2 : 0;
    if (r->stream) split2 = 1;
    if (split2 == 0) {   // one co-resident wave: as many CTAs as fit the GPU's 2 x 148 slots, at least 4 K blocks each
        split2 = 1;
        if (r->m_tiles == 1)
            while (split2 < 8 && l->n_tiles * (split2 + 1) <= 296 && kblocks / (split2 + 1) >= 4) ++split2;
    }
    if (split2 < 1 || split2 > 16 || split2 > kblocks || (split2 > 1 && r->m_tiles > 1)) return OB_ERR_TILE;
    if (split2 > 1 && (long long)l->n_tiles * r->m_tiles > kCounterSlots) return OB_ERR_TOO_LARGE;   // one arrival counter per split tile
    r->split2 = split2;
    int split1 = (cfg && cfg->split1) ? cfg->split1 : 0;
    const int pb = M <= kDecodeTokens ? 1 : 4;
    // Prefill batches of bf16 adapters shrink on the tensor cores (LOWBIT_SHRINK_CUDA_CORES=1 keeps the warp-level form).
    static const bool no_mma = [] { const char* v = std::getenv("LOWBIT_SHRINK_CUDA_CORES"); return v && v[0] == '1'; }();
    // (not for sharded adapters: their shrink partials are all-reduced between K1 and K2, so they must stay partials).
    // From kMmaShrinkTokens on: below it a 128-position tile of a many-tenant batch holds too many tenants for one
    // accumulator pass (measured at 32 tenants: 60-120 us for the tensor-core form at 64-256 tokens, 35-50 us warp-level).
    const int pf = cfg ? cfg->prefill : 0;             // 1 / 2 force the tensor-core / warp-level forms
    r->mma_shrink = (!no_mma && pf != 2 && M > kDecodeTokens && (pf == 1 || M >= kMmaShrinkTokens) &&
                     d.lora_fmt == kLoraBf16 && !b_sharded(d)) ? 1 : 0;
    // Larger batches go to the 256 x 256 prefill GEMM unless the caller names a token tile (LOWBIT_PREFILL_SMALL_TILES=1
    // keeps k2_gemm.cu's tiles); prepare_call() drops the choice again when the workspace has no room for its h blocks.
    static const bool no_big = [] { const char* v = std::getenv("LOWBIT_PREFILL_SMALL_TILES"); return v && v[0] == '1'; }();
    // (LOWBIT_PREFILL_MIN_TILES=n sends launches of fewer than n 256-token tiles back to k2_gemm.cu's 128 x 128 tiles; with
    // the CTA-pair kernel the large tiles measured equal or faster from 512 tokens on for every projection, so n = 1)
    static const int min_big_tiles = [] { const char* v = std::getenv("LOWBIT_PREFILL_MIN_TILES"); return v ? std::atoi(v) : 1; }();
    const long long big_tiles = (long long)((M + 255) / 256) * (d.N / (fp4 ? 128 : 256));
    const long long big_steps = 2LL * (d.L < kMaxTileTenants ? d.L : kMaxTileTenants) * (d.R / 64);   // a tile's expand steps at most
    r->big = (!no_big && r->mma_shrink && l->big_ok && M > kBigTileMinTokens && !(cfg && cfg->tn) &&
              big_steps <= k2_prefill_max_steps() && (pf == 1 || big_tiles >= min_big_tiles)) ? 1 : 0;
    if (split1 == 0 && r->mma_shrink) {   // one wave of (128-position tile, tenant group, slice, K split) CTAs, at least 256 elements each
        // (tenant groups per tile, where the shrink deals a tile's tenants out to several CTAs: see shrink_group_cap)
        const int cap = shrink_group_cap(d.L, M);
        const int groups = (shrink_tenants_per_tile(d.L, M) + cap - 1) / cap;
        const int tiles = ((M + 127) / 128) * groups * d.S;
        split1 = 1;
        while (split1 < 16 && tiles * (split1 * 2) <= 148 && d.K / (split1 * 2) >= 256) split1 *= 2;
        // four splits are one cluster that sums over shared memory; eight go through the workspace and their last arriver:
        // unless that halves a long K (1024 elements or more per split), four measured faster
        if (split1 == 8 && d.K / 8 < 1024 && d.R % 16 == 0) split1 = 4;
    }
    if (split1 == 0) {
        const long long units = (long long)((M + pb - 1) / pb) * d.S * (d.R / 8);
        split1 = 1;
        if (pb == 1 && r->stream)   // beside the persistent GEMM the shrink runs as one CTA per SM: one unit per warp of that grid
            while (split1 < 16 && d.K / (split1 * 2) >= 512 && units * split1 * 2 <= (long long)r->grid_s * 8) split1 *= 2;
        else if (pb == 1)   // decode: as many K splits as keep the whole shrink in one wave of the GPU's 2 x 148 CTA slots (8 warps each)
            while (split1 < 16 && d.K / (split1 * 2) >= 512 && (units * split1 * 2 + 7) / 8 + M <= 296) split1 *= 2;
        else {         // four positions per warp: two to three waves of warps measured best (each re-reads A through L2);
                       // every CTA of K2 adds the partials again, so a projection with many output tiles wants fewer of them
            const int cap = l->n_tiles > 100 ? 4 : 16;
            while (split1 < cap && d.K / (split1 * 2) >= 512 && units * split1 * 2 <= 6144) split1 *= 2;
        }
    }
    if (split1 < 1 || split1 > 32) return OB_ERR_TILE;
    r->split1 = split1;
    r->k_per_split = (int)align_up((size_t)(d.K + split1 - 1) / split1, 256);
    if (r->mma_shrink)   // every split must hold part of K: the splits of a tile count their arrivals
        while (r->split1 > 1 && (long long)(r->split1 - 1) * r->k_per_split >= d.K) --r->split1;
    r->pb = pb;
    const int rc = l->rc;
    int stages = r->stream ? r->stages : (cfg && cfg->stages) ? cfg->stages : 0;
    if (r->stream) {
        r->wait_ms = (cfg && cfg->wait_ms > 0) ? (uint32_t)cfg->wait_ms : 2000u;
        r->fused = 0;
        return OB_OK;
    }
    if (stages == 0) {   // prefer a footprint that lets two CTAs share an SM (3+ stages; 2+ for 128-token tiles), else the deepest ring that fits
        stages = 12;
        const int floor_stages = r->tn >= 128 ? 2 : 3;
        while (stages > floor_stages && k2_fp8_smem_bytes(r->tn, stages, rc, d.R, d.base_fmt == OB_BASE_NVFP4) > kSmemTwoPerSm) --stages;
        if (k2_fp8_smem_bytes(r->tn, stages, rc, d.R, d.base_fmt == OB_BASE_NVFP4) > kSmemTwoPerSm) stages = 12;
    }
    if (stages < 2 || stages > 12) return OB_ERR_TILE;
    while (stages > 2 && k2_fp8_smem_bytes(r->tn, stages, rc, d.R, d.base_fmt == OB_BASE_NVFP4) > kSmemLimit) --stages;
    if (k2_fp8_smem_bytes(r->tn, stages, rc, d.R, d.base_fmt == OB_BASE_NVFP4) > kSmemLimit) return OB_ERR_TILE;
    if (fp4)   // TMEM: 2 tn accumulator columns + 32 scale-factor columns per ring slot, 512 in all
        while (stages > 2 && 2 * r->tn + 32 * stages > 512) --stages;
    r->stages = stages;
    if ((long long)(d.L < r->tn ? d.L : r->tn) * (d.R / rc) > kMaxLoraIters) return OB_ERR_TOO_LARGE;
    r->wait_ms = (cfg && cfg->wait_ms > 0) ? (uint32_t)cfg->wait_ms : 2000u;
    r->fused = (cfg && cfg->fused) ? 1 : 0;
    return OB_OK;
}

Meta meta_of(const ObBatch* b) { return Meta{b->tok, b->srt, b->seg_n, b->seg_start, b->seg_ids}; }

int get_xmap(ObLayer* l, const void* xq, int rows, int tn, CUtensorMap* out) {
    std::lock_guard<std::mutex> g(l->mu);
    for (const XMap& m : l->xmaps)
        if (m.base == xq && m.rows == rows && m.tn == tn) {
            *out = m.tm;
            return OB_OK;
        }
    XMap m;
    m.base = xq;
    m.rows = rows;
    m.tn = tn;
    const uint64_t lc = (uint64_t)(l->d.L < kMaxTileTenants ? l->d.L : kMaxTileTenants);
    int st = tn == -4   // NVFP4 activation block scales as a [rows, 256] byte tensor: one 2 KB atom = an unswizzled 8-row box
                 ? encode_2d(&m.tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, 256, (uint64_t)rows, 256, 256, 8, true)
             : tn == -2   // the shrink's per-tenant h blocks [S * rows, lc * R] bf16: 64-element x 128-row boxes
                 ? encode_2d(&m.tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, xq, lc * (uint64_t)l->d.R, (uint64_t)l->d.S * (uint64_t)rows,
                             lc * (uint64_t)l->d.R * 2, 64, 128)
             : tn < 0   // the adapter-sorted bf16 copy of x: 64-element x 128-row boxes for the tensor-core shrink
                 ? encode_2d(&m.tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, xq, (uint64_t)l->d.K, (uint64_t)rows, (uint64_t)l->d.K * 2, 64, 128)
                 : encode_2d(&m.tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, (uint64_t)k_bytes(l->d), (uint64_t)rows,
                             (uint64_t)k_bytes(l->d), kBlockK, (uint32_t)tn);
    if (st != OB_OK) return st;
    l->xmaps.push_back(m);
    *out = m.tm;
    return OB_OK;
}

K1Params k1_params(ObLayer* l, const ObBatch* b, void* ws, const ObWorkspaceShape* sh, const Resolved& r, bool chain) {
    const ObLayerDesc& d = l->d;
    const WorkspaceLayout lay = workspace_layout(*sh);
    uint8_t* base = static_cast<uint8_t*>(ws);
    K1Params p = {};
    p.M = b->M; p.K = d.K; p.S = d.S; p.R = d.R; p.L = d.L;
    p.lora_fmt = d.lora_fmt;
    p.split1 = r.split1;
    p.k_per_split = r.k_per_split;
    p.n_quant_ctas = b->M;
    p.looped = r.stream;
    p.pb = r.pb;
    p.n_pblocks = (b->M + r.pb - 1) / r.pb;
    p.units_per_block = d.S * (d.R / 8) * r.split1;
    p.x = static_cast<const __nv_bfloat16*>(b->x);
    p.ldx = b->ldx;
    p.x_op = b->x_op;
    p.meta = meta_of(b);
    for (int s = 0; s < d.S; ++s) { p.a[s] = d.a[s]; p.sa[s] = d.sa[s]; }
    p.ag = d.ag;
    p.xq = base + lay.xq;
    p.sx = reinterpret_cast<float*>(base + lay.sx);
    p.hp = reinterpret_cast<float*>(base + lay.hp);
    p.max_m = sh->max_m;
    p.base_fmt = d.base_fmt;
    p.tn = (r.big && d.base_fmt == OB_BASE_NVFP4) ? 256 : r.tn;   // the activation scales are laid out per token tile of K2
    p.nblk = p.tn > 128 ? 2 : 1;
    p.kslots = (d.K + 255) / 256;
    p.rcp_approx = d.quant_rcp_approx;
    p.x_global = d.x_global;
    p.xsf = base + lay.xsf;
    p.xq_ready = chain ? reinterpret_cast<int32_t*>(base + lay.counters) + kCounterSlots : nullptr;
    p.xs = r.mma_shrink ? reinterpret_cast<__nv_bfloat16*>(base + lay.xs) : nullptr;
    p.trace = g_trace ? g_trace + g_trace_ctas * OB_TRACE_EVENTS : nullptr;   // K1's stamps follow K2's
    p.trace_ctas = g_trace_ctas;
    return p;
}

int k1_fp8_impl(ObLayer* l, const ObBatch* b, void* ws, const ObWorkspaceShape* sh, const Resolved& r, int pdl,
                cudaStream_t stream, bool chain = false) {
    const K1Params p = k1_params(l, b, ws, sh, r, chain);
    const long long warps = r.mma_shrink ? 0 : (long long)p.n_pblocks * p.units_per_block;
    long long grid = p.n_quant_ctas + (warps + 7) / 8;
    if (p.looped) {   // at most one CTA per SM (never fewer than the quantizing CTAs): the warps walk the units with the grid's stride
        const long long cap = r.grid_s > p.n_quant_ctas ? r.grid_s : p.n_quant_ctas;
        const long long need = (warps + 7) / 8 > p.n_quant_ctas ? (warps + 7) / 8 : p.n_quant_ctas;
        grid = need < cap ? need : cap;
    }
    if (grid > 0x7fffffffLL) return OB_ERR_TOO_LARGE;
    cudaError_t e = launch_k1_fp8(p, (int)grid, pdl, stream);
    if (e != cudaSuccess) return (int)e;
    if (!r.mma_shrink) return OB_OK;
    // the shrink itself: one CTA per (128 positions, slice, K split), a programmatic dependent of the launch above
    const ObLayerDesc& d = l->d;
    const WorkspaceLayout lay = workspace_layout(*sh);
    uint8_t* base = static_cast<uint8_t*>(ws);
    CUtensorMap tm_xs;
    int st = get_xmap(l, base + lay.xs, sh->max_m, -1, &tm_xs);
    if (st != OB_OK) return st;
    K1mParams m = {};
    m.M = b->M; m.K = d.K; m.S = d.S; m.R = d.R; m.L = d.L; m.max_m = sh->max_m;
    m.split1 = r.split1;
    m.k_per_split = r.k_per_split;
    m.ring_bytes = 192 * 1024;
    m.tg_cap = shrink_group_cap(d.L, b->M);
    m.wait_ms = r.wait_ms;
    m.meta = meta_of(b);
    m.hp = reinterpret_cast<float*>(base + lay.hp);
    m.hb = reinterpret_cast<__nv_bfloat16*>(base + lay.hb);
    m.counters = reinterpret_cast<int32_t*>(base + lay.counters);
    m.status = reinterpret_cast<int32_t*>(base + lay.status);
    if (r.big) {
        m.hcat = reinterpret_cast<__nv_bfloat16*>(base + lay.hcat);
        m.lc = d.L < kMaxTileTenants ? d.L : kMaxTileTenants;
        const bool fp4 = d.base_fmt == OB_BASE_NVFP4;     // NVFP4: the output scale is alpha = 1 / (x_global * w_global) alone
        m.sx = fp4 ? nullptr : reinterpret_cast<const float*>(base + lay.sx);
        m.s_w = fp4 ? d.alpha : d.s_w;
    }
    // 2 or 4 splits whose share of the rank is whole float4s: one thread-block cluster per (tile, slice), sums over
    // distributed shared memory (LOWBIT_SHRINK_GLOBAL_SUM=1 keeps the workspace partials and the arrival counters).
    // Clusters of 8 measured slower than the workspace path: a cluster sits inside one GPC with one such CTA per SM, so
    // few of them are resident at once.
    static const bool global_sum = [] { const char* v = std::getenv("LOWBIT_SHRINK_GLOBAL_SUM"); return v && v[0] == '1'; }();
    m.cluster = (!global_sum && (r.split1 == 2 || r.split1 == 4) && d.R % (4 * r.split1) == 0 &&
                 (size_t)128 * d.R * 4 <= (size_t)m.ring_bytes) ? 1 : 0;
    // work items (tile, tenant group): sum over tiles of ceil(tenants / cap) <= (pairs + tiles (cap - 1)) / cap with
    // pairs = (tile, tenant) incidences <= segments + tiles - 1 (a tile boundary is crossed by one segment at most), and
    // never more than ceil(min(L, 128) / cap) per tile
    const long long mtiles = (b->M + 127) / 128;
    const long long per_tile_max = ((d.L < kMaxTileTenants ? d.L : kMaxTileTenants) + m.tg_cap - 1) / m.tg_cap;
    const long long pairs = std::min<long long>(d.L + 1, b->M) + mtiles - 1;   // (L + 1: every entry of the index)
    const long long items = std::min(mtiles * per_tile_max, (pairs + mtiles * (m.tg_cap - 1)) / m.tg_cap);
    if (items * d.S > kCounterSlots || items > 0x7fffffffLL) return OB_ERR_TOO_LARGE;
    dim3 mgrid((unsigned)items, (unsigned)d.S, (unsigned)r.split1);
    e = launch_k1_mma(m, tm_xs, l->tm_a, mgrid, stream);
    return e == cudaSuccess ? OB_OK : (int)e;
}

// Split-K through a cluster: up to 8 splits, a partial tile that fits the operand ring, and all of the launch's clusters
// resident at once (a cluster is placed whole inside one GPC, so fewer fit than single CTAs would).  Otherwise, and under
// LOWBIT_SPLITK_GLOBAL=1, the partials go through the workspace and the arrival counters.
bool cluster_reduce_fits(const ObLayer* l, const Resolved& r, size_t smem) {
    static const bool force_global = [] { const char* v = std::getenv("LOWBIT_SPLITK_GLOBAL"); return v && v[0] == '1'; }();
    if (force_global || r.split2 < 2 || r.split2 > 8) return false;
    const size_t ring_bytes = (size_t)r.stages * ((size_t)kTileN * kBlockK + (size_t)r.tn * kBlockK);
    if ((size_t)r.tn * kTileN * sizeof(float) > ring_bytes) return false;
    static std::mutex mu;
    static std::vector<std::pair<unsigned long long, int>> cache;   // (device, formats, split2, smem) -> resident clusters
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return false;
    const int fp4 = l->d.base_fmt == OB_BASE_NVFP4 ? 1 : 0, stored = l->d.lora_fmt == kLoraBf16 ? 0 : 1;
    const unsigned long long key = ((unsigned long long)dev << 48) | ((unsigned long long)(fp4 * 2 + stored) << 44) |
                                   ((unsigned long long)r.split2 << 40) | (unsigned long long)smem;
    std::lock_guard<std::mutex> g(mu);
    int n = -1;
    for (const auto& kv : cache) if (kv.first == key) n = kv.second;
    if (n < 0) {
        n = k2_max_active_clusters(fp4, stored, r.split2, smem);
        cache.emplace_back(key, n);
        if (std::getenv("LOWBIT_VERBOSE"))
            std::fprintf(stderr, "[onebase_b200] split-K clusters of %d CTAs, %zu B shared memory: %d resident at once\n", r.split2, smem, n);
    }
    return l->n_tiles <= n;
}

// K2's launch: parameters, tensor map of the quantized activations, grid and shared memory.
struct K2Launch {
    K2Params p;
    CUtensorMap tm_x;
    dim3 grid;
    size_t smem;
    bool fp4;
};

// `scratch` (optional): split-K partial tiles and arrival counters somewhere else than in the workspace's own split-K
// region -- the partials then go through global memory (no cluster form) and the workspace need not have room for them.
struct SplitScratch {
    float* part;
    int32_t* counters;
};

int k2_prepare(ObLayer* l, const ObBatch* b, void* ws, const ObWorkspaceShape* sh, const Resolved& r, bool chain, K2Launch* out,
               const SplitScratch* scratch = nullptr, const ObComm* fused_ar = nullptr) {
    const ObLayerDesc& d = l->d;
    const WorkspaceLayout lay = workspace_layout(*sh);
    uint8_t* base = static_cast<uint8_t*>(ws);
    int st = get_xmap(l, base + lay.xq, sh->max_m, r.tn, &out->tm_x);
    if (st != OB_OK) return st;
    out->p = K2Params{};
    K2Params& p = out->p;
    p.M = b->M; p.N = d.N; p.K = d.K; p.S = d.S; p.R = d.R; p.L = d.L;
    for (int s = 0; s < OB_MAX_SLICES; ++s) p.widths[s] = s < d.S ? d.widths[s] : 0;
    p.lora_fmt = d.lora_fmt;
    p.tn = r.tn;
    p.split2 = r.split2;
    p.split1 = r.split1;
    p.kblocks = (k_bytes(d) + kBlockK - 1) / kBlockK;
    p.stages = r.stages;
    p.rc = l->rc;
    p.nh = k2_fp8_h_tiles(r.tn);
    p.wsf = static_cast<const uint8_t*>(d.w_sf);
    p.xsf = base + lay.xsf;
    p.alpha = d.alpha;
    p.nblk = r.tn > 128 ? 2 : 1;
    p.max_m = sh->max_m;
    p.wait_ms = r.wait_ms;
    p.s_w = d.s_w;
    p.sx = reinterpret_cast<const float*>(base + lay.sx);
    p.hp = reinterpret_cast<const float*>(base + lay.hp);
    p.hb = r.mma_shrink ? reinterpret_cast<const __nv_bfloat16*>(base + lay.hb) : nullptr;
    p.meta = meta_of(b);
    p.y = static_cast<__nv_bfloat16*>(b->y);
    p.ldy = b->ldy;
    p.residual = static_cast<const __nv_bfloat16*>(b->residual);
    p.ldr = b->ldr;
    p.part = reinterpret_cast<float*>(base + lay.part);
    p.counters = reinterpret_cast<int32_t*>(base + lay.counters);
    p.status = reinterpret_cast<int32_t*>(base + lay.status);
    int32_t* chain_words = reinterpret_cast<int32_t*>(base + lay.counters) + kCounterSlots;
    p.xq_ready = chain ? chain_words : nullptr;
    p.chain_done = chain ? chain_words + 1 : nullptr;
    for (int s = 0; s < d.S; ++s) { p.b[s] = d.b[s]; p.sb[s] = d.sb[s]; }
    for (int s = 0; s < OB_MAX_SLICES; ++s) {
        p.b_row0[s] = s < d.S ? d.b_row0[s] : 0;
        p.b_rows[s] = s < d.S ? (d.b_rows[s] ? d.b_rows[s] : d.widths[s]) : 0;
    }
    p.bg = d.bg;
    {   // stored adapters: bulk copies of a step's codes need whole-rank chunks and 16-byte granular rows
        static const bool unstaged = [] { const char* v = std::getenv("LOWBIT_B_UNSTAGED"); return v && v[0] == '1'; }();
        bool ok = d.lora_fmt != kLoraBf16 && d.R == l->rc && !unstaged;
        for (int s = 0; s < d.S; ++s) ok = ok && d.widths[s] % 16 == 0;
        p.b_staged = ok ? 1 : 0;
    }
    p.trace = g_trace;
    p.trace_ctas = g_trace_ctas;
    if (scratch != nullptr) {
        p.part = scratch->part;
        p.counters = scratch->counters;
    } else if (r.split2 > 1) {   // the partials of this call must fit the workspace's split-K region
        const size_t need = (size_t)r.split2 * (size_t)l->n_tiles * (size_t)r.tn * kTileN * sizeof(float);
        if (lay.part + need > lay.total) return OB_ERR_WORKSPACE;
    }
    p.m_fast = r.m_tiles > 1 ? 1 : 0;
    if (p.m_fast && l->n_tiles > 65535) return OB_ERR_TOO_LARGE;
    out->grid = p.m_fast ? dim3((unsigned)r.m_tiles, 1u, (unsigned)l->n_tiles)
                         : dim3((unsigned)l->n_tiles, (unsigned)r.split2, (unsigned)r.m_tiles);
    out->fp4 = d.base_fmt == OB_BASE_NVFP4;
    out->smem = k2_fp8_smem_bytes(r.tn, r.stages, l->rc, d.R, out->fp4 ? 1 : 0);
    p.cluster_reduce = (scratch == nullptr && fused_ar == nullptr && cluster_reduce_fits(l, r, out->smem)) ? 1 : 0;
    if (fused_ar != nullptr) {      // the all-reduce of a row-parallel layer's output, inside the epilogue
        p.ar_world = fused_ar->world;
        p.ar_rank = fused_ar->rank;
        p.ar_slot_bytes = (long long)fused_ar->slot_bytes;
        for (int q = 0; q < fused_ar->world; ++q) p.ar_bufs[q] = static_cast<uint8_t*>(fused_ar->bufs[q]);
    }
    return OB_OK;
}

int k2_prefill_impl(ObLayer* l, const ObBatch* b, void* ws, const ObWorkspaceShape* sh, const Resolved& r, int pdl,
                    cudaStream_t stream) {
    const ObLayerDesc& d = l->d;
    const WorkspaceLayout lay = workspace_layout(*sh);
    uint8_t* base = static_cast<uint8_t*>(ws);
    // Slices in whole tiles of the pair kernel (256 features with an NVFP4 base, 512 with FP8): CTA pairs (k2_prefill2.cu)
    // unless LOWBIT_PREFILL_PAIRS=0
    static const bool no_pairs = [] { const char* v = std::getenv("LOWBIT_PREFILL_PAIRS"); return v && v[0] == '0'; }();
    const int is_fp4 = d.base_fmt == OB_BASE_NVFP4 ? 1 : 0;
    const int pair_rows = k2_prefill_pair_rows(is_fp4);
    bool pairs = !no_pairs;
    for (int s = 0; s < d.S; ++s) pairs = pairs && d.widths[s] % pair_rows == 0;
    const int pair_cap = pairs ? k2_prefill_pair_capacity(is_fp4) : 0;
    pairs = pairs && pair_cap > 0;
    if (std::getenv("LOWBIT_VERBOSE")) std::fprintf(stderr, "[onebase_b200] prefill GEMM: pairs=%d (resident pairs %d)\n", (int)pairs, pair_cap);
    CUtensorMap tm_x, tm_h;
    int st = get_xmap(l, base + lay.xq, sh->max_m, pairs ? 128 : 256, &tm_x);
    if (st == OB_OK) st = get_xmap(l, base + lay.hcat, sh->max_m, -2, &tm_h);
    if (st != OB_OK) return st;
    K2pParams p = {};
    p.M = b->M; p.N = d.N; p.K = d.K; p.S = d.S; p.R = d.R; p.L = d.L;
    for (int s = 0; s < OB_MAX_SLICES; ++s) p.widths[s] = s < d.S ? d.widths[s] : 0;
    const bool fp4 = d.base_fmt == OB_BASE_NVFP4;
    p.kblocks = (k_bytes(d) + kBlockK - 1) / kBlockK;
    p.stages = 3;
    p.wsf = static_cast<const uint8_t*>(d.w_sf);
    p.xsf = base + lay.xsf;
    p.lc = d.L < kMaxTileTenants ? d.L : kMaxTileTenants;
    p.max_m = sh->max_m;
    p.wait_ms = r.wait_ms;
    p.s_w = fp4 ? d.alpha : d.s_w;               // NVFP4: one output scale, no per-token factor
    p.sx = fp4 ? nullptr : reinterpret_cast<const float*>(base + lay.sx);
    p.meta = meta_of(b);
    p.y = static_cast<__nv_bfloat16*>(b->y);
    p.ldy = b->ldy;
    p.status = reinterpret_cast<int32_t*>(base + lay.status);
    if (pairs) {
        CUtensorMap tm_sf[2] = {l->tm_wsf, l->tm_w};
        if (is_fp4) {
            st = get_xmap(l, base + lay.xsf, (int)((lay.hp - lay.xsf) / 256), -4, &tm_sf[1]);
            if (st != OB_OK) return st;
        }
        const long long ptiles = (long long)((b->M + 255) / 256) * (d.N / pair_rows);
        const int n = (int)(ptiles < pair_cap ? ptiles : pair_cap);
        cudaError_t e = launch_k2_prefill_pair(p, l->tm_w, tm_x, tm_h, l->tm_b, tm_sf, n, is_fp4, pdl, stream);
        return e == cudaSuccess ? OB_OK : (int)e;
    }
    const int rows = fp4 ? 128 : 256;            // output features per CTA
    const long long tiles = (long long)((b->M + 255) / 256) * (d.N / rows);
    const int sms = sm_count();
    if (tiles > 0x7fffffffLL || sms <= 0) return OB_ERR_TOO_LARGE;
    dim3 grid((unsigned)(tiles < sms ? tiles : sms), 1u, 1u);   // persistent: one CTA per SM walks the tiles
    cudaError_t e = fp4 ? launch_k2_prefill(p, l->tm_w, tm_x, tm_h, l->tm_b, grid, 1, pdl, stream)
                        : launch_k2_prefill(p, l->tm_w2, tm_x, tm_h, l->tm_b2, grid, 0, pdl, stream);
    return e == cudaSuccess ? OB_OK : (int)e;
}

// The persistent decode GEMM: same parameters as the tile kernel's launch; its fp32 partial tiles (two per CTA at most: the
// first and the last tile of a CTA's share may be shared with its neighbours) live in the workspace's split-K region.
int k2_stream_impl(ObLayer* l, const ObBatch* b, void* ws, const ObWorkspaceShape* sh, const Resolved& r, int pdl,
                   cudaStream_t stream, bool chain) {
    K2Launch k;
    const int st = k2_prepare(l, b, ws, sh, r, chain, &k);
    if (st != OB_OK) return st;
    const WorkspaceLayout lay = workspace_layout(*sh);
    const size_t need = (size_t)2 * (size_t)r.grid_s * (size_t)r.tn * kTileN * sizeof(float);
    if (lay.part + need > lay.total) return OB_ERR_WORKSPACE;
    k.p.n_tiles = l->n_tiles;
    k.p.nh = k2_stream_h_tiles(r.tn);
    k.p.cluster_reduce = 0;
    k.p.m_fast = 0;
    const size_t smem = k2_stream_smem_bytes(r.tn, r.stages, l->rc, l->d.R, l->d.S, k.fp4 ? 1 : 0);
    cudaError_t e = launch_k2_stream(k.p, l->tm_w, k.tm_x, l->tm_b, r.grid_s, smem, k.fp4 ? 1 : 0, pdl, stream);
    return e == cudaSuccess ? OB_OK : (int)e;
}

int k2_fp8_impl(ObLayer* l, const ObBatch* b, void* ws, const ObWorkspaceShape* sh, const Resolved& r, int pdl,
                cudaStream_t stream, bool chain = false) {
    if (r.big) return k2_prefill_impl(l, b, ws, sh, r, pdl, stream);
    if (r.stream) return k2_stream_impl(l, b, ws, sh, r, pdl, stream, chain);
    K2Launch k;
    const int st = k2_prepare(l, b, ws, sh, r, chain, &k);
    if (st != OB_OK) return st;
    cudaError_t e = k.fp4 ? launch_k2_nvfp4(k.p, l->tm_w, k.tm_x, l->tm_b, k.grid, k.smem, pdl, stream)
                          : launch_k2_fp8(k.p, l->tm_w, k.tm_x, l->tm_b, k.grid, k.smem, pdl, stream);
    return e == cudaSuccess ? OB_OK : (int)e;
}

// ObTileCfg.fused: a decode chain of bf16 adapters as ONE kernel.  Every CTA of the GEMM first takes a share of the
// quantization and of the shrink from two work counters, so the weight stream starts with the launch and no second launch
// sits in between; in exchange the shrink's dependent loads queue behind the CTA's own weight stream.  Which form wins
// depends on the shape, so the tile table decides.
bool fused_applies(const ObLayer* l, const Resolved& r) {
    return r.fused && l->d.lora_fmt == kLoraBf16 && r.pb == 1 && r.m_tiles == 1 && r.tn <= 32;
}

int fused_impl(ObLayer* l, const ObBatch* b, void* ws, const ObWorkspaceShape* sh, const Resolved& r, cudaStream_t stream) {
    K2Launch k;
    const int st = k2_prepare(l, b, ws, sh, r, true, &k);
    if (st != OB_OK) return st;
    K1Params k1 = k1_params(l, b, ws, sh, r, true);
    k1.trace = g_trace ? g_trace + g_trace_ctas * OB_TRACE_EVENTS : nullptr;
    k.p.work_quant = k.p.counters + kCounterSlots + 2;
    k.p.work_shrink = k.p.counters + kCounterSlots + 3;
    k.p.hp_ready = k.p.counters + kCounterSlots + 4;
    const long long units = (long long)k1.n_pblocks * k1.units_per_block;
    if (units > 0x3fffffffLL) return OB_ERR_TOO_LARGE;
    k.p.shrink_units = (int)units;
    cudaError_t e = launch_fused(k.p, k1, l->tm_w, k.tm_x, l->tm_b, k.grid, k.smem, stream);
    return e == cudaSuccess ? OB_OK : (int)e;
}

int prepare_call(ObLayer* l, const ObBatch* b, void* ws, const ObWorkspaceShape* sh, const ObTileCfg* cfg, Resolved* r,
                 int base_fmt = OB_BASE_FP8) {
    int st = validate_batch(l, b);
    if (st != OB_OK) return st;
    if (l->d.base_fmt != base_fmt) return OB_ERR_FORMAT;
    st = resolve_cfg(l, b->M, cfg, r);
    if (st != OB_OK) return st;
    if (b->residual != nullptr) {                // the residual add lives in the tile kernel's stores
        r->big = 0;
        r->stream = 0;
        r->fused = 0;
    }
    if (b->x_op != OB_X_PLAIN) {                 // the input transform lives in the two-CTAs-per-SM K1 only
        r->fused = 0;
        r->stream = 0;
    }
    if (r->big && (!sh || sh->max_l < l->d.L)) r->big = 0;
    if (r->big && (b->ldy % 8 != 0 || !aligned16(b->y))) r->big = 0;   // its epilogue stores 16 bytes at a time
    return validate_workspace(l, ws, sh, r->split1, r->split2);
}

// ---------------------------------------------------------------------------------------------------------------
// ob_k2_fp8_static: K2 for callers that cannot allocate device memory.  Its split-K scratch (fp32 partial tiles and
// the per-tile arrival counters) lives in the file-scope device array below instead of the caller's workspace.  Every
// GPU that loads this library holds the array until the process exits.
constexpr size_t kStaticCounterBytes = sizeof(int32_t) * kCounterSlots;                      // 16 KiB of arrival counters
constexpr size_t kStaticPartBytes = (size_t)OB_STATIC_SCRATCH_BYTES - kStaticCounterBytes;   // the rest: partial tiles
static __device__ __align__(256) unsigned char g_k2_static_scratch[OB_STATIC_SCRATCH_BYTES];

// Device address of the array on the current device, resolved once per device.  In host code the array's name is only a
// stand-in symbol, not a device address, so the kernel must be given what cudaGetSymbolAddress returns.  The first call
// on a device also zeroes the counters (a memset on the caller's stream; later launches return them to zero themselves).
constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
unsigned char* g_static_addr[kMaxDevices] = {nullptr};

int static_scratch_for_current_device(cudaStream_t stream, unsigned char** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return OB_ERR_TOO_LARGE;
    std::lock_guard<std::mutex> g(g_static_mu);
    if (g_static_addr[dev] == nullptr) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_k2_static_scratch);
        if (e != cudaSuccess) return (int)e;
        e = cudaMemsetAsync(ptr, 0, kStaticCounterBytes, stream);
        if (e != cudaSuccess) return (int)e;
        g_static_addr[dev] = static_cast<unsigned char*>(ptr);
    }
    *out = g_static_addr[dev];
    return OB_OK;
}

// A launch that recorded a wait time-out may have left arrival counters of the static array above zero (a CTA that gave
// up never arrived), and no caller can reach the array.  ob_read_status -- the call by which a host learns of the
// time-out -- therefore clears them whenever it reads a non-zero status word on a device whose array is in use.
cudaError_t rezero_static_counters(cudaStream_t stream) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaSuccess;
    std::lock_guard<std::mutex> g(g_static_mu);
    if (g_static_addr[dev] == nullptr) return cudaSuccess;
    return cudaMemsetAsync(g_static_addr[dev], 0, kStaticCounterBytes, stream);
}

}  // namespace

extern "C" {

int ob_k2_fp8_static(ObLayer* layer, const ObBatch* batch, void* workspace, const ObWorkspaceShape* shape,
                     const ObTileCfg* cfg, int pdl, void* cuda_stream) {
    Resolved r;
    int st = validate_batch(layer, batch);
    if (st != OB_OK) return st;
    if (layer->d.base_fmt != OB_BASE_FP8 || layer->d.lora_fmt != OB_LORA_BF16) return OB_ERR_FORMAT;
    st = resolve_cfg(layer, batch->M, cfg, &r);
    if (st != OB_OK) return st;
    r.stream = 0;   // this entry point runs the tile-per-CTA kernel: its split-K partials are what lives in the array
    // the workspace only has to hold what K1 wrote (and the status words): its own split-K region is not used
    st = validate_workspace(layer, workspace, shape, r.split1, 1);
    if (st != OB_OK) return st;
    if (r.big && (shape->max_l < layer->d.L || batch->ldy % 8 != 0 || !aligned16(batch->y))) r.big = 0;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    // a prefill batch on the 256 x 256 GEMM needs no split-K scratch at all: the same launch as ob_k2_fp8
    if (r.big) return k2_prefill_impl(layer, batch, workspace, shape, r, pdl, stream);
    const size_t need = r.split2 > 1 ? (size_t)r.split2 * (size_t)layer->n_tiles * (size_t)r.tn * kTileN * sizeof(float) : 0;
    if (need > kStaticPartBytes) return OB_ERR_TOO_LARGE;   // beyond the static scratch: use ob_k2_fp8 with a workspace
    unsigned char* scratch = nullptr;
    st = static_scratch_for_current_device(stream, &scratch);
    if (st != OB_OK) return st;
    // the same launch as ob_k2_fp8 builds, with the split-K partial tiles and arrival counters taken from the array
    const SplitScratch ss = {reinterpret_cast<float*>(scratch + kStaticCounterBytes), reinterpret_cast<int32_t*>(scratch)};
    K2Launch k;
    st = k2_prepare(layer, batch, workspace, shape, r, false, &k, &ss);
    if (st != OB_OK) return st;
    k.p.trace = nullptr;
    k.p.trace_ctas = 0;
    cudaError_t e = launch_k2_fp8(k.p, layer->tm_w, k.tm_x, layer->tm_b, k.grid, k.smem, pdl, stream);
    return e == cudaSuccess ? OB_OK : (int)e;
}

int ob_version(void) { return OB_ABI_VERSION; }

const char* ob_status_string(int status) {
    switch (status) {
        case OB_OK: return "ok";
        case OB_ERR_NULL: return "a required pointer is null";
        case OB_ERR_SHAPE: return "unsupported layer shape";
        case OB_ERR_ALIGN: return "pointer or pitch not aligned";
        case OB_ERR_WORKSPACE: return "workspace too small";
        case OB_ERR_TILE: return "invalid tile configuration";
        case OB_ERR_FORMAT: return "format not served by this entry point";
        case OB_ERR_BATCH: return "token count out of range";
        case OB_ERR_DRIVER: return "CUDA driver entry points unavailable";
        case OB_ERR_TOO_LARGE: return "request exceeds a fixed capacity";
        default: break;
    }
    if (status >= 1000) return "CUDA driver error (status - 1000 is the CUresult)";
    if (status > 0) return cudaGetErrorString((cudaError_t)status);
    return "unknown status";
}

int ob_workspace_bytes(const ObWorkspaceShape* shape, size_t* bytes) {
    if (!shape || !bytes) return OB_ERR_NULL;
    if (shape->max_m < 1 || shape->max_k < 16 || shape->max_k % 16 != 0 || shape->max_n < 1 || shape->max_sr < 16 ||
        shape->max_split1 < 1 || shape->max_split1 > 32 || shape->max_split2 < 1 || shape->max_split2 > 16)
        return OB_ERR_SHAPE;
    *bytes = workspace_layout(*shape).total;
    return OB_OK;
}

int ob_workspace_offsets(const ObWorkspaceShape* shape, size_t out[7]) {
    size_t total;
    int st = ob_workspace_bytes(shape, &total);
    if (st != OB_OK) return st;
    if (!out) return OB_ERR_NULL;
    const WorkspaceLayout l = workspace_layout(*shape);
    out[0] = l.status; out[1] = l.counters; out[2] = l.sx; out[3] = l.xq; out[4] = l.xsf; out[5] = l.hp; out[6] = l.part;
    return OB_OK;
}

int ob_workspace_region(const ObWorkspaceShape* shape, int region, size_t* offset, size_t* bytes) {
    size_t total;
    int st = ob_workspace_bytes(shape, &total);
    if (st != OB_OK) return st;
    if (!offset || !bytes) return OB_ERR_NULL;
    if (region < 0 || region >= OB_WS_REGIONS) return OB_ERR_SHAPE;
    const WorkspaceLayout l = workspace_layout(*shape);
    const size_t start[OB_WS_REGIONS + 1] = {l.status, l.counters, l.sx, l.xq, l.xsf, l.hp, l.part, l.xs, l.hb, l.hcat, l.total};
    *offset = start[region];
    *bytes = start[region + 1] - start[region];
    return OB_OK;
}

int ob_layer_create(const ObLayerDesc* desc, ObLayer** out) {
    if (!out) return OB_ERR_NULL;
    *out = nullptr;
    int st = validate_desc(desc);
    if (st != OB_OK) return st;
    ObLayer* l = new (std::nothrow) ObLayer();
    if (!l) return (int)cudaErrorMemoryAllocation;
    l->d = *desc;
    l->rc = desc->R < 64 ? desc->R : 64;
    l->n_tiles = 0;
    for (int s = 0; s < desc->S; ++s) l->n_tiles += (desc->widths[s] + kTileN - 1) / kTileN;
    {
        const uint64_t kb = (uint64_t)k_bytes(*desc);   // bytes of one W row: K e4m3 codes or K/2 packed e2m1 pairs
        st = encode_2d(&l->tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, desc->w_q, kb, (uint64_t)desc->N, kb, kBlockK, kTileN);
        if (st == OB_OK && desc->lora_fmt == OB_LORA_BF16) {
            for (int s = 0; s < OB_MAX_SLICES && st == OB_OK; ++s) {
                const int ss = s < desc->S ? s : 0;   // unused slots repeat slice 0 so every kernel argument is a valid map
                const int b_rows = desc->b_rows[ss] ? desc->b_rows[ss] : desc->widths[ss];   // rows of B this rank holds
                st = encode_2d(&l->tm_b[s], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, desc->b[ss], (uint64_t)desc->R,
                               (uint64_t)desc->L * (uint64_t)b_rows, (uint64_t)desc->R * 2, (uint32_t)l->rc, kTileN);
                if (st == OB_OK)
                    st = encode_2d(&l->tm_a[s], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, desc->a[ss], (uint64_t)desc->K,
                                   (uint64_t)desc->L * (uint64_t)desc->R, (uint64_t)desc->K * 2, 64, (uint32_t)desc->R);
            }
        }
    }
    l->big_ok = desc->lora_fmt == OB_LORA_BF16 && desc->R >= 64 && !b_sharded(*desc);
    for (int s = 0; s < desc->S; ++s) l->big_ok = l->big_ok && desc->widths[s] % (desc->base_fmt == OB_BASE_NVFP4 ? 128 : 256) == 0;
    if (desc->base_fmt == OB_BASE_NVFP4 && desc->K % 256 != 0) l->big_ok = false;   // whole 256-element k-blocks
    if (st == OB_OK && l->big_ok && desc->base_fmt == OB_BASE_FP8) {
        st = encode_2d(&l->tm_w2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, desc->w_q, (uint64_t)desc->K, (uint64_t)desc->N, (uint64_t)desc->K,
                       kBlockK, 256);
        for (int s = 0; s < OB_MAX_SLICES && st == OB_OK; ++s) {
            const int ss = s < desc->S ? s : 0;
            st = encode_2d(&l->tm_b2[s], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, desc->b[ss], (uint64_t)desc->R,
                           (uint64_t)desc->L * (uint64_t)desc->widths[ss], (uint64_t)desc->R * 2, 64, 256);
        }
    }
    if (st == OB_OK && l->big_ok && desc->base_fmt == OB_BASE_NVFP4)
        st = encode_2d(&l->tm_wsf, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, desc->w_sf, 256,
                       (uint64_t)l->n_tiles * (uint64_t)((desc->K + 255) / 256) * (kSfSlotBytes / 256), 256, 256, 8, true);
    if (st != OB_OK) {
        delete l;
        return st;
    }
    *out = l;
    return OB_OK;
}

int ob_layer_destroy(ObLayer* layer) {
    delete layer;
    return OB_OK;
}

int ob_resolve_tile(ObLayer* layer, int32_t M, const ObTileCfg* cfg, ObTileCfg* out) {
    if (!layer || !out) return OB_ERR_NULL;
    if (M < 1 || M > layer->d.max_m) return OB_ERR_BATCH;
    Resolved r;
    const int st = resolve_cfg(layer, M, cfg, &r);
    if (st != OB_OK) return st;
    out->tn = r.tn;
    out->split2 = r.split2;
    out->split1 = r.split1;
    out->stages = r.stages;
    out->wait_ms = (int32_t)r.wait_ms;
    out->fused = r.fused;
    out->stream = r.stream ? 1 : 2;                          // which GEMM kernel serves the call
    out->prefill = r.big ? 1 : r.mma_shrink ? 0 : 2;       // what will run (the workspace may still veto the large tiles)
    return OB_OK;
}

int ob_k1_fp8(ObLayer* layer, const ObBatch* batch, void* workspace, const ObWorkspaceShape* shape, const ObTileCfg* cfg,
              void* cuda_stream) {
    Resolved r;
    int st = prepare_call(layer, batch, workspace, shape, cfg, &r);
    if (st != OB_OK) return st;
    return k1_fp8_impl(layer, batch, workspace, shape, r, 0, static_cast<cudaStream_t>(cuda_stream));
}

int ob_k2_fp8(ObLayer* layer, const ObBatch* batch, void* workspace, const ObWorkspaceShape* shape, const ObTileCfg* cfg,
              int pdl, void* cuda_stream) {
    Resolved r;
    int st = prepare_call(layer, batch, workspace, shape, cfg, &r);
    if (st != OB_OK) return st;
    return k2_fp8_impl(layer, batch, workspace, shape, r, pdl, static_cast<cudaStream_t>(cuda_stream));
}

int ob_chain_fp8(ObLayer* layer, const ObBatch* batch, void* workspace, const ObWorkspaceShape* shape, const ObTileCfg* cfg,
                 void* cuda_stream) {
    Resolved r;
    int st = prepare_call(layer, batch, workspace, shape, cfg, &r);
    if (st != OB_OK) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    if (fused_applies(layer, r)) return fused_impl(layer, batch, workspace, shape, r, stream);
    // (persistent decode GEMM: K1 counts the positions it has quantized and K2 starts its base GEMM on that count)
    st = k1_fp8_impl(layer, batch, workspace, shape, r, 1, stream, r.stream != 0);
    if (st != OB_OK) return st;
    return k2_fp8_impl(layer, batch, workspace, shape, r, 1, stream, r.stream != 0);
}

int ob_k1_nvfp4(ObLayer* layer, const ObBatch* batch, void* workspace, const ObWorkspaceShape* shape, const ObTileCfg* cfg,
                void* cuda_stream) {
    Resolved r;
    int st = prepare_call(layer, batch, workspace, shape, cfg, &r, OB_BASE_NVFP4);
    if (st != OB_OK) return st;
    return k1_fp8_impl(layer, batch, workspace, shape, r, 0, static_cast<cudaStream_t>(cuda_stream));
}

int ob_k2_nvfp4(ObLayer* layer, const ObBatch* batch, void* workspace, const ObWorkspaceShape* shape, const ObTileCfg* cfg,
                int pdl, void* cuda_stream) {
    Resolved r;
    int st = prepare_call(layer, batch, workspace, shape, cfg, &r, OB_BASE_NVFP4);
    if (st != OB_OK) return st;
    return k2_fp8_impl(layer, batch, workspace, shape, r, pdl, static_cast<cudaStream_t>(cuda_stream));
}

int ob_chain_nvfp4(ObLayer* layer, const ObBatch* batch, void* workspace, const ObWorkspaceShape* shape, const ObTileCfg* cfg,
                   void* cuda_stream) {
    Resolved r;
    int st = prepare_call(layer, batch, workspace, shape, cfg, &r, OB_BASE_NVFP4);
    if (st != OB_OK) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    if (fused_applies(layer, r)) return fused_impl(layer, batch, workspace, shape, r, stream);
    // (persistent decode GEMM: K1 counts the positions it has quantized and K2 starts its base GEMM on that count)
    st = k1_fp8_impl(layer, batch, workspace, shape, r, 1, stream, r.stream != 0);
    if (st != OB_OK) return st;
    return k2_fp8_impl(layer, batch, workspace, shape, r, 1, stream, r.stream != 0);
}

int ob_nvfp4_packed_scale_bytes(int32_t K, int32_t S, const int32_t* widths, size_t* bytes) {
    if (!widths || !bytes) return OB_ERR_NULL;
    if (K < 32 || K % 32 != 0 || S < 1 || S > OB_MAX_SLICES) return OB_ERR_SHAPE;
    size_t tiles = 0;
    for (int s = 0; s < S; ++s) {
        if (widths[s] <= 0) return OB_ERR_SHAPE;
        tiles += (size_t)(widths[s] + kTileN - 1) / kTileN;
    }
    *bytes = tiles * (size_t)((K + 255) / 256) * kSfSlotBytes;
    return OB_OK;
}

int ob_nvfp4_pack_scales(const void* w_sf_linear, int32_t K, int32_t S, const int32_t* widths, void* packed,
                         size_t packed_bytes, void* cuda_stream) {
    size_t need = 0;
    int st = ob_nvfp4_packed_scale_bytes(K, S, widths, &need);
    if (st != OB_OK) return st;
    if (!w_sf_linear || !packed) return OB_ERR_NULL;
    if (packed_bytes < need) return OB_ERR_WORKSPACE;
    cudaError_t e = launch_pack_scales(static_cast<const uint8_t*>(w_sf_linear), K, S, widths, static_cast<uint8_t*>(packed),
                                       need, static_cast<cudaStream_t>(cuda_stream));
    return e == cudaSuccess ? OB_OK : (int)e;
}

int ob_requant_fp8_rows(const void* src, int64_t rows, int32_t cols, void* codes, float* scales, void* cuda_stream) {
    if (!src || !codes || !scales) return OB_ERR_NULL;
    if (rows < 1 || rows > 0x7fffffffLL || cols < 8 || cols % 8 != 0) return OB_ERR_SHAPE;
    if (!aligned16(src) || (reinterpret_cast<uintptr_t>(codes) & 7u)) return OB_ERR_ALIGN;
    cudaError_t e = launch_requant_fp8(src, rows, cols, codes, scales, static_cast<cudaStream_t>(cuda_stream));
    return e == cudaSuccess ? OB_OK : (int)e;
}

int ob_requant_nvfp4(const void* src, int32_t l, int32_t rows, int32_t cols, void* packed, void* sf, float* inv_global,
                     void* amax_scratch, void* cuda_stream) {
    if (!src || !packed || !sf || !inv_global || !amax_scratch) return OB_ERR_NULL;
    if (l < 1 || l > 65535 || rows < 1 || cols < 16 || cols % 16 != 0) return OB_ERR_SHAPE;
    if (!aligned16(src) || (reinterpret_cast<uintptr_t>(packed) & 7u) || (reinterpret_cast<uintptr_t>(amax_scratch) & 3u))
        return OB_ERR_ALIGN;
    cudaError_t e = launch_requant_nvfp4(src, l, rows, cols, packed, sf, inv_global, static_cast<unsigned int*>(amax_scratch),
                                         static_cast<cudaStream_t>(cuda_stream));
    return e == cudaSuccess ? OB_OK : (int)e;
}

int ob_segment_index(const int32_t* token_lora, int32_t M, int32_t L, int32_t* tok, int32_t* srt, int32_t* seg_n,
                     int32_t* seg_start, int32_t* seg_ids, void* cuda_stream) {
    if (!token_lora || !tok || !srt || !seg_n || !seg_start || !seg_ids) return OB_ERR_NULL;
    if (M < 1 || L < 1 || L > 1023) return OB_ERR_SHAPE;
    cudaError_t e = launch_segment_index(token_lora, M, L, tok, srt, seg_n, seg_start, seg_ids,
                                         static_cast<cudaStream_t>(cuda_stream));
    return e == cudaSuccess ? OB_OK : (int)e;
}

// ---------------------------------------------------------------------------------------------------------------
// all-reduce over peer-mapped memory
namespace {
int ar_fill(const ObComm* c, const void* src, void* dst, int64_t count, int32_t dtype, int32_t mode, int32_t wait_ms, ArParams* p) {
    if (!c || !src || !dst) return OB_ERR_NULL;
    if (c->world < 2 || c->world > OB_MAX_RANKS || c->rank < 0 || c->rank >= c->world) return OB_ERR_SHAPE;
    if (dtype != OB_DTYPE_BF16 && dtype != OB_DTYPE_F32) return OB_ERR_FORMAT;
    const size_t esz = dtype == OB_DTYPE_BF16 ? 2 : 4;
    if (count < 1 || ((size_t)count * esz) % 16 != 0) return OB_ERR_SHAPE;
    if ((size_t)count * esz > c->slot_bytes || c->slot_bytes % 16 != 0) return OB_ERR_TOO_LARGE;
    if (!aligned16(src) || !aligned16(dst)) return OB_ERR_ALIGN;
    for (int r = 0; r < c->world; ++r)
        if (!c->bufs[r] || !aligned16(c->bufs[r])) return OB_ERR_NULL;
    if (mode != OB_AR_AUTO && mode != OB_AR_ONE_SHOT && mode != OB_AR_TWO_SHOT) return OB_ERR_TILE;
    *p = ArParams{};
    p->world = c->world;
    p->rank = c->rank;
    p->dtype = dtype;
    p->two_shot = mode == OB_AR_TWO_SHOT || (mode == OB_AR_AUTO && c->world > 2 && (size_t)count * esz > 512 * 1024) ? 1 : 0;
    p->count = count;
    p->slot_bytes = (long long)c->slot_bytes;
    p->wait_ms = wait_ms > 0 ? (uint32_t)wait_ms : 2000u;
    p->src = src;
    p->dst = dst;
    for (int r = 0; r < c->world; ++r) p->bufs[r] = static_cast<uint8_t*>(c->bufs[r]);
    return OB_OK;
}

int ar_grid(int64_t count, int32_t dtype) {
    const long long nvec = (count * (dtype == OB_DTYPE_BF16 ? 2 : 4) + 15) / 16;
    long long g = (nvec + 255) / 256;
    const long long cap = nvec > 32768 ? 128 : 64;        // payloads above 512 KB: more CTAs, two vectors per thread and pass
    return (int)(g < 1 ? 1 : g > cap ? cap : g);
}
}  // namespace

// Can K2's epilogue carry the all-reduce of this call?  Decode batches on the tile-per-CTA kernel, features in whole 16-byte
// groups, one flag per output tile, and the [M, N] bf16 partial must fit a slot of the communication buffer.
static bool fused_allreduce_applies(const ObLayer* l, const ObBatch* b, const Resolved& r, const ObComm* c) {
    if (r.big || r.stream || r.m_tiles != 1 || r.tn > kDecodeTokens) return false;
    if (l->n_tiles > kArMaxTiles || l->d.N % 8 != 0) return false;
    for (int s = 0; s < l->d.S; ++s)
        if (l->d.widths[s] % 8 != 0) return false;
    return (size_t)b->M * (size_t)l->d.N * 2 <= c->slot_bytes;
}

int ob_chain_allreduce(ObLayer* layer, const ObBatch* batch, void* workspace, const ObWorkspaceShape* shape, const ObTileCfg* cfg,
                       const ObComm* comm, void* cuda_stream) {
    if (!comm) return OB_ERR_NULL;
    if (comm->world < 2 || comm->world > OB_MAX_RANKS || comm->rank < 0 || comm->rank >= comm->world || comm->slot_bytes % 16 != 0)
        return OB_ERR_SHAPE;
    for (int q = 0; q < comm->world; ++q)
        if (!comm->bufs[q] || !aligned16(comm->bufs[q])) return OB_ERR_NULL;
    if (!layer) return OB_ERR_NULL;
    Resolved r;
    int st = prepare_call(layer, batch, workspace, shape, cfg, &r, layer->d.base_fmt);
    if (st != OB_OK) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    const int wait_ms = (cfg && cfg->wait_ms > 0) ? cfg->wait_ms : 2000;
    if (!fused_allreduce_applies(layer, batch, r, comm)) {
        // the chain as usual, then the stand-alone all-reduce kernel over y (which must then be a dense [M, N] matrix)
        if (batch->ldy != layer->d.N || !aligned16(batch->y)) return OB_ERR_ALIGN;
        if (fused_applies(layer, r)) st = fused_impl(layer, batch, workspace, shape, r, stream);
        else {
            st = k1_fp8_impl(layer, batch, workspace, shape, r, 1, stream, r.stream != 0);
            if (st == OB_OK) st = k2_fp8_impl(layer, batch, workspace, shape, r, 1, stream, r.stream != 0);
        }
        if (st != OB_OK) return st;
        return ob_allreduce(comm, batch->y, batch->y, (int64_t)batch->M * layer->d.N, OB_DTYPE_BF16, OB_AR_AUTO, wait_ms, cuda_stream);
    }
    st = k1_fp8_impl(layer, batch, workspace, shape, r, 1, stream);
    if (st != OB_OK) return st;
    K2Launch k;
    st = k2_prepare(layer, batch, workspace, shape, r, false, &k, nullptr, comm);
    if (st != OB_OK) return st;
    cudaError_t e = k.fp4 ? launch_k2_nvfp4(k.p, layer->tm_w, k.tm_x, layer->tm_b, k.grid, k.smem, 1, stream)
                          : launch_k2_fp8(k.p, layer->tm_w, k.tm_x, layer->tm_b, k.grid, k.smem, 1, stream);
    return e == cudaSuccess ? OB_OK : (int)e;
}

int ob_comm_bytes(size_t slot_bytes, size_t* bytes) {
    if (!bytes) return OB_ERR_NULL;
    if (slot_bytes < 16 || slot_bytes % 16 != 0) return OB_ERR_SHAPE;
    *bytes = kArStateBytes + 4 * slot_bytes;     // state and flags; two staged copies; two reduced copies
    return OB_OK;
}

int ob_ipc_export(const void* dev_ptr, unsigned char handle[OB_IPC_HANDLE_BYTES], size_t* offset) {
    if (!dev_ptr || !handle || !offset) return OB_ERR_NULL;
    static_assert(sizeof(cudaIpcMemHandle_t) == OB_IPC_HANDLE_BYTES, "handle size");
    // the handle names the whole allocation the pointer lies in: report where in it the pointer is
    typedef CUresult (*RangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
    void* fp = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fp, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) {
        (void)cudaGetLastError();
        return OB_ERR_DRIVER;
    }
    CUdeviceptr base = 0;
    size_t size = 0;
    const CUresult r = reinterpret_cast<RangeFn>(fp)(&base, &size, reinterpret_cast<CUdeviceptr>(dev_ptr));
    if (r != CUDA_SUCCESS) return 1000 + (int)r;
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base));
    if (e != cudaSuccess) return (int)e;
    std::memcpy(handle, &h, sizeof(h));
    *offset = reinterpret_cast<CUdeviceptr>(dev_ptr) - base;
    return OB_OK;
}

int ob_ipc_open(const unsigned char handle[OB_IPC_HANDLE_BYTES], size_t offset, void** mapped) {
    if (!handle || !mapped) return OB_ERR_NULL;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    void* base = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return (int)e;
    *mapped = static_cast<unsigned char*>(base) + offset;
    return OB_OK;
}

int ob_ipc_close(void* mapped, size_t offset) {
    if (!mapped) return OB_ERR_NULL;
    const cudaError_t e = cudaIpcCloseMemHandle(static_cast<unsigned char*>(mapped) - offset);
    return e == cudaSuccess ? OB_OK : (int)e;
}

int ob_allreduce(const ObComm* comm, const void* src, void* dst, int64_t count, int32_t dtype, int32_t mode, int32_t wait_ms,
                 void* cuda_stream) {
    ArBatch b = {};
    const int st = ar_fill(comm, src, dst, count, dtype, mode, wait_ms, &b.r[0]);
    if (st != OB_OK) return st;
    const cudaError_t e = launch_allreduce(b, 1, ar_grid(count, dtype), static_cast<cudaStream_t>(cuda_stream));
    return e == cudaSuccess ? OB_OK : (int)e;
}

int ob_allreduce_emulated(const ObComm* comms, int32_t n, const void* const* src, void* const* dst, int64_t count,
                          int32_t dtype, int32_t mode, int32_t wait_ms, void* cuda_stream) {
    if (!comms || !src || !dst) return OB_ERR_NULL;
    if (n < 1 || n > OB_MAX_RANKS) return OB_ERR_SHAPE;
    ArBatch b = {};
    for (int q = 0; q < n; ++q) {
        const int st = ar_fill(&comms[q], src[q], dst[q], count, dtype, mode, wait_ms, &b.r[q]);
        if (st != OB_OK) return st;
    }
    int grid = ar_grid(count, dtype);
    const int sms = sm_count();
    if (sms > 0 && grid * n > sms) grid = sms / n > 0 ? sms / n : 1;      // a cooperative launch must fit the GPU at once
    const cudaError_t e = launch_allreduce(b, n, grid, static_cast<cudaStream_t>(cuda_stream));
    return e == cudaSuccess ? OB_OK : (int)e;
}

int ob_comm_status(const ObComm* comm, int32_t host_out[8], void* cuda_stream) {
    if (!comm || !host_out || !comm->bufs[comm->rank]) return OB_ERR_NULL;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    int32_t* state = static_cast<int32_t*>(comm->bufs[comm->rank]);
    cudaError_t e = cudaMemcpyAsync(host_out, state, sizeof(int32_t) * 8, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(state + 3, 0, sizeof(int32_t) * 4, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    return e == cudaSuccess ? OB_OK : (int)e;
}

int ob_trace_buffer(void* device_u64_buffer, int64_t max_ctas) {
    g_trace = static_cast<unsigned long long*>(device_u64_buffer);
    g_trace_ctas = device_u64_buffer ? max_ctas : 0;
    return OB_OK;
}

int ob_read_status(void* workspace, int32_t* host_out, void* cuda_stream) {
    if (!workspace || !host_out) return OB_ERR_NULL;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    cudaError_t e = cudaMemcpyAsync(host_out, workspace, sizeof(int32_t) * OB_STATUS_WORDS, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(workspace, 0, sizeof(int32_t) * OB_STATUS_WORDS, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e == cudaSuccess && host_out[0] != OB_DEV_OK) {
        e = rezero_static_counters(stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    }
    return e == cudaSuccess ? OB_OK : (int)e;
}

}  // extern "C"
