/*
 * onebase_b200 -- C ABI of the B200 (sm_100a) implementation of OneBase's fused multi-tenant LoRA + low-precision
 * base GEMM projection.
 *
 * The reference (fatebreaker/onebase) has no native layer: its host code launches Triton kernels directly from
 * Python.  Every entry point below therefore replaces a Python->Triton launch site of the reference; each comment
 * names that site as `file:line` inside the reference checkout.
 *
 * Conventions
 *   - every function returns an int status: 0 = OB_OK, < 0 = argument / geometry rejected BEFORE any launch,
 *     > 0 = a cudaError_t (or 1000 + CUresult for driver calls) from the launch path.  Nothing throws.
 *   - every pointer inside the structs is a borrowed DEVICE pointer that the caller keeps alive; the library never
 *     allocates or frees device memory and never synchronizes (except ob_read_status, which copies 64 bytes back).
 *   - scratch ("workspace") is one caller-allocated, zero-initialized device buffer per device, sized by
 *     ob_workspace_bytes() for the largest layer that will use it; layers share it and run one after another on one
 *     stream (as the reference's shared `Scratch`, lowbit_lora/kernels/fp8_lora_vllm.py:315-346).  Kernels return its
 *     counters to zero, so a captured CUDA graph can be replayed.
 *   - device-side waits are bounded: a wait that runs out sets status word 0 of the workspace (see ob_read_status)
 *     and the kernel returns without writing out of bounds.
 *   - reentrant per (device, stream); two calls that share a workspace must not overlap on the GPU.
 */
#ifndef ONEBASE_B200_H
#define ONEBASE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OB_ABI_VERSION 1

/* status codes (< 0: rejected before any launch) */
#define OB_OK 0
#define OB_ERR_NULL (-1)         /* a required pointer is null */
#define OB_ERR_SHAPE (-2)        /* unsupported N / K / R / S / L / widths */
#define OB_ERR_ALIGN (-3)        /* a pointer or pitch is not 16-byte aligned */
#define OB_ERR_WORKSPACE (-4)    /* the workspace is too small for this call */
#define OB_ERR_TILE (-5)         /* the tile configuration is not valid for this shape */
#define OB_ERR_FORMAT (-6)       /* unknown base / adapter format, or a format this entry point does not serve */
#define OB_ERR_BATCH (-7)        /* M out of range (0 < M <= max_m) */
#define OB_ERR_DRIVER (-8)       /* the CUDA driver entry points could not be resolved (no GPU / no driver) */
#define OB_ERR_TOO_LARGE (-9)    /* the request exceeds a fixed capacity of the entry point */

/* device-side status word 0 (ob_read_status) */
#define OB_DEV_OK 0
#define OB_DEV_WAIT_TIMEOUT 1    /* a bounded wait ran out; words 1..7 say where */
#define OB_DEV_BAD_INDEX 2       /* the segment index holds more (tile, tenant) incidences than disjoint contiguous segments
                                    can: the tensor-core shrink's launch did not cover them; word 2 = work items found,
                                    word 3 = work items launched */

enum { OB_BASE_FP8 = 0, OB_BASE_NVFP4 = 1 };
enum { OB_X_PLAIN = 0, OB_X_SILU_MUL = 1 };
enum { OB_LORA_BF16 = 0, OB_LORA_FP8 = 1, OB_LORA_NVFP4 = 2 };

#define OB_MAX_SLICES 4
#define OB_STATUS_WORDS 16

/* One LoRA linear layer: the constructor arguments of the reference's op objects
 *   VllmFusedFP8LoRA(w_q, s_w, a_stacked, b_stacked, max_m, lora_fp8=, lora_fp4=)
 *       lowbit_lora/kernels/fp8_lora_vllm.py:416-496
 *   VllmFusedNVFP4LoRA(w_q, w_sf, w_global, x_global, a_stacked, b_stacked, max_m, lora_fmt=)
 *       lowbit_lora/kernels/nvfp4_lora_vllm.py:437-502
 * with vLLM's per-slice stacked adapter buffers a[s] = [L,1,R,K], b[s] = [L,1,N_s,R]. */
typedef struct ObLayerDesc {
    int32_t base_fmt;                /* OB_BASE_* */
    int32_t lora_fmt;                /* OB_LORA_* */
    int32_t N, K;                    /* output / input features of this (shard of the) projection */
    int32_t S;                       /* slices (1..4): q/k/v, gate/up */
    int32_t L;                       /* adapter slots */
    int32_t R;                       /* LoRA rank: 16, 32, 64, 128 or 256 */
    int32_t widths[OB_MAX_SLICES];   /* N_s, sum = N */
    int32_t max_m;                   /* largest token count of a call */
    const void* w_q;                 /* FP8: [N,K] e4m3.  NVFP4: [N,K/2] packed e2m1, element 2i in the low nibble */
    const void* w_sf;                /* NVFP4: ue4m3 block scales PACKED by ob_nvfp4_pack_scales from the checkpoint's linear
                                        [N,K/16] layout (ob_nvfp4_packed_scale_bytes bytes).  FP8: null */
    const float* s_w;                /* FP8: [1] per-tensor weight scale */
    const float* x_global;           /* NVFP4: [1] static activation global scale (1 / input_scale) */
    const float* alpha;              /* NVFP4: [1] 1 / (x_global * w_global) */
    const void* a[OB_MAX_SLICES];    /* adapter A per slice: bf16 [L,1,R,K] | e4m3 [L,1,R,K] | packed [L,1,R,K/2] */
    const void* b[OB_MAX_SLICES];    /* adapter B per slice: bf16 [L,1,N_s,R] | e4m3 | packed [L,1,N_s,R/2] */
    const void* sa[OB_MAX_SLICES];   /* FP8: fp32 [L,R] row scales.  NVFP4: ue4m3 [L,1,R,K/16] block scales */
    const void* sb[OB_MAX_SLICES];   /* FP8: fp32 [L,N_s].           NVFP4: ue4m3 [L,1,N_s,R/16] */
    const float* ag;                 /* NVFP4 adapters: fp32 [S,L] inverse global scales of A */
    const float* bg;                 /* NVFP4 adapters: fp32 [S,L] inverse global scales of B */
    int32_t quant_rcp_approx;        /* NVFP4 base: 1 = reciprocals by rcp.approx.ftz (bit-identical to vLLM's CUDA quantizer,
                                        nvfp4_lora_vllm.py:61-67), 0 = IEEE reciprocals (the torch recipe, :361-376) */
    /* Row-parallel layers with sharded adapters (vLLM's RowParallelLinearWithShardedLoRA,
     * vllm/lora/layers/row_parallel_linear.py:118-160): this rank holds W and A for its K slice but only rows
     * [b_row0[s], b_row0[s] + b_rows[s]) of each slice's B (`b[s]` is then [L,1,b_rows[s],R]); the expand is added to those
     * output features only, after the caller has all-reduced the shrink partials in the workspace.  Both zero: the whole
     * slice.  bf16 adapters only; b_row0 must be a multiple of 128, b_rows too unless the range ends with the slice. */
    int32_t b_row0[OB_MAX_SLICES];
    int32_t b_rows[OB_MAX_SLICES];
} ObLayerDesc;

/* One call's inputs and output: the arguments of `op(x, meta_args, out=...)`
 * (lowbit_lora/kernels/fp8_lora_vllm.py:619-629) with vLLM's LoRAKernelMeta tensors
 * (vllm/lora/ops/triton_ops/lora_kernel_metadata.py:170-200), all int32 on the device. */
typedef struct ObBatch {
    int32_t M;                       /* tokens in this call (rows of x and y), 0 < M <= max_m */
    const void* x;                   /* [M,K] bf16, row pitch ldx elements */
    int64_t ldx;
    void* y;                         /* [M,N] bf16, row pitch ldy elements */
    int64_t ldy;
    const int32_t* tok;              /* [M]   token -> slot id (-1: none)            token_lora_mapping */
    const int32_t* srt;              /* [M]   token indices sorted by slot id        token_indices_sorted_by_lora_ids */
    const int32_t* seg_n;            /* [L+1] tokens per segment                     num_tokens_per_lora */
    const int32_t* seg_start;        /* [L+2] segment start offsets                  lora_token_start_loc */
    const int32_t* seg_ids;          /* [L+1] slot id per segment, -1 padded         active_lora_ids */
    /* The ops either side of the projection, fused (all optional; zero / null = off):
     *   x_op = OB_X_SILU_MUL   the projection's input is silu(gate) * up of the preceding merged projection: x is its
     *        output [M, 2K] (gate | up, row pitch ldx >= 2K) and K1 forms bf16(bf16(silu(g)) * u) on the fly -- vLLM's
     *        SiluAndMul (vllm/model_executor/layers/activation.py, forward_native) without its pass over memory -- before
     *        quantizing and shrinking it.  For down_proj.
     *   residual   [M, N] bf16, row pitch ldr: K2 stores y = bf16(bf16(acc) + residual) -- the "x + residual" of vLLM's
     *        fused add + RMSNorm that follows o_proj and down_proj (vllm/model_executor/layers/layernorm.py,
     *        forward_native: the sum in fp32, rounded to the residual's dtype).  May be the same memory as y. */
    int32_t x_op;
    const void* residual;
    int64_t ldr;
} ObBatch;

/* Capacity of a shared workspace (what the reference's Scratch.ensure / _Work.ensure grow,
 * lowbit_lora/kernels/fp8_lora_vllm.py:329-346, lowbit_lora/kernels/fp8_lora_pdl.py:620-643). */
typedef struct ObWorkspaceShape {
    int32_t max_m;                   /* tokens */
    int32_t max_k;                   /* largest K */
    int32_t max_n;                   /* largest N */
    int32_t max_sr;                  /* largest S*R */
    int32_t max_split1;              /* largest split-K of the shrink */
    int32_t max_split2;              /* largest split-K of the GEMM */
    int32_t max_l;                   /* most adapter slots L of any layer sharing the workspace; 0 = no room for the
                                      * per-tenant h blocks of the large-tile prefill GEMM, which is then not used */
} ObWorkspaceShape;

/* Per-call tile choice (what the reference's pick_cfg / plugin_cfg return,
 * lowbit_lora/kernels/fp8_lora_vllm.py:287-312, lowbit_lora/hopper_pdl.py:268-298).  0 = library default. */
typedef struct ObTileCfg {
    int32_t tn;                      /* tokens per GEMM tile (the MMA's N): 16, 32, 64, 128 or 256 */
    int32_t split2;                  /* GEMM split-K (1..16) */
    int32_t split1;                  /* shrink split-K (1..32) */
    int32_t stages;                  /* shared-memory ring depth of the GEMM (2..12) */
    int32_t wait_ms;                 /* bound of every device-side wait in milliseconds (default 2000) */
    int32_t fused;                   /* ob_chain_*: 1 = one kernel for the whole chain where that form applies (bf16
                                      * adapters, at most 32 tokens): every GEMM CTA first takes a share of the
                                      * quantization and of the shrink from work counters in the workspace */
    int32_t prefill;                 /* batches of more than 32 tokens, bf16 adapters: 0 = library rule (tensor-core shrink
                                      * from 512 tokens; 256 x 256 GEMM tiles when they fill the GPU), 1 = tensor-core
                                      * shrink and, where the layer allows, 256 x 256 tiles whatever the size, 2 = the
                                      * warp-level shrink and 64..128-token tiles */
    int32_t stream;                  /* decode batches (at most 32 tokens) of bf16 adapters: 1 = the persistent GEMM, one CTA per
                                      * SM streaming a contiguous share of the launch's weight k-blocks across output tiles, the
                                      * expand steps' B tiles in a ring of their own (tiles shared between CTAs are finished by
                                      * the last CTA to arrive; tn and stages apply, split2 does not); 0 or 2 = one CTA per
                                      * (output tile, K split), the default.  ob_resolve_tile reports which one a call takes
                                      * (1 or 2) */
} ObTileCfg;

typedef struct ObLayer ObLayer;      /* opaque: validated descriptor + TMA tensor maps (host memory only) */

int ob_version(void);
const char* ob_status_string(int status);

/* Bytes of the shared workspace for `shape`.  Replaces Scratch.ensure (fp8_lora_vllm.py:329-346). */
int ob_workspace_bytes(const ObWorkspaceShape* shape, size_t* bytes);

/* Byte offsets of the workspace regions, for inspection (the reference exposes them as Scratch.xq / .sx / .hp,
 * fp8_lora_vllm.py:321-327): out[0..6] = status words, split-K counters, s_x [max_m] fp32, x_q codes (row pitch = the
 * calling layer's K; rows are adapter-sorted POSITIONS), NVFP4 activation block scales, shrink partials
 * [split1][S][max_m][R] fp32, GEMM split-K partials.  Behind them the workspace holds regions only the kernels use (for
 * max_m > 32: an adapter-sorted bf16 copy of x and the tensor-core shrink's finished h; for max_m > 128 and max_l > 0: the
 * per-tenant h blocks of the large-tile prefill GEMM); ob_workspace_bytes counts them. */
int ob_workspace_offsets(const ObWorkspaceShape* shape, size_t out[7]);

/* Offset and size of ONE workspace region, the kernel-only ones included (same purpose as above: the reference's
 * tests read its scratch tensors, e.g. `op.scratch.hp`, lowbit_lora/kernels/fp8_lora_vllm.py:321-327).
 * OB_WS_XS: adapter-sorted bf16 copy of x [max_m, K]; OB_WS_HB: the tensor-core shrink's finished h [S][max_m][R] bf16;
 * OB_WS_HCAT: per-tenant h blocks of the large-tile prefill GEMM.  A region the shape has no room for has 0 bytes. */
enum { OB_WS_STATUS = 0, OB_WS_COUNTERS, OB_WS_SX, OB_WS_XQ, OB_WS_XSF, OB_WS_HP, OB_WS_PART, OB_WS_XS, OB_WS_HB, OB_WS_HCAT,
       OB_WS_REGIONS };
int ob_workspace_region(const ObWorkspaceShape* shape, int region, size_t* offset, size_t* bytes);

/* Validate a layer and build its TMA descriptors.  Replaces VllmFusedFP8LoRA.__init__ / VllmFusedNVFP4LoRA.__init__
 * (fp8_lora_vllm.py:425-496, nvfp4_lora_vllm.py:446-502): pointer tables, slice ends, format flags. */
int ob_layer_create(const ObLayerDesc* desc, ObLayer** out);
int ob_layer_destroy(ObLayer* layer);

/* The tile choice a call of M tokens would run with: `cfg`'s non-zero fields, the rest filled in by the library's rule
 * (tn, split2, split1, stages, wait_ms; fused as given).  For callers that need the shrink's split count -- e.g. to
 * all-reduce exactly the partials [split1][S][max_m][R] that were written.  No counterpart in the reference, whose
 * Python host code holds these numbers itself (`pick_cfg`, lowbit_lora/kernels/fp8_lora_vllm.py:287-312). */
int ob_resolve_tile(ObLayer* layer, int32_t M, const ObTileCfg* cfg, ObTileCfg* out);

/* K1, FP8 base: per-token dynamic e4m3 quantization of x (codes + scales into the workspace, at each token's
 * adapter-sorted position) fused with every tenant's shrink h = x A^T (split-K partials into the workspace).
 * Replaces the launch `_shrink_vllm[grid]` (fp8_lora_vllm.py:732-745) / `_shrink_pdl` (lowbit_lora/hopper_pdl.py:153-165). */
int ob_k1_fp8(ObLayer* layer, const ObBatch* batch, void* workspace, const ObWorkspaceShape* shape,
              const ObTileCfg* cfg, void* cuda_stream);

/* K2, FP8 base: TMA-fed tcgen05 e4m3 GEMM over the adapter-sorted tokens K1 wrote, scaled by s_x*s_w, plus each
 * tenant's expand h B^T, bf16 out.  Replaces `_gemm_vllm[grid]` (fp8_lora_vllm.py:747-765) / `_gemm_pdl`
 * (lowbit_lora/hopper_pdl.py:167-174).  `pdl` != 0 launches it with programmatic stream serialization. */
int ob_k2_fp8(ObLayer* layer, const ObBatch* batch, void* workspace, const ObWorkspaceShape* shape,
              const ObTileCfg* cfg, int pdl, void* cuda_stream);

/* K2 for callers that cannot allocate device memory for scratch: the same tile-per-CTA kernel, launch geometry and
 * result as ob_k2_fp8 with ObTileCfg.stream = 2, but its split-K scratch (fp32 partial tiles, per-tile arrival counters)
 * lives in a fixed device array inside the library instead of the workspace's split-K region.  Meant for hosts that
 * must not call cudaMalloc where this runs -- inside a stream capture, on a serving thread whose memory pool is frozen
 * after warm-up, or from a runtime that hands the library nothing but its tensors -- and so cannot grow a workspace
 * when a tile choice needs more split-K room.
 * This entry point has no counterpart in the reference (its Triton host code allocates torch tensors freely).
 *   - `workspace` must still hold what ob_k1_fp8 wrote for this batch (x_q, s_x, shrink partials) and receives the
 *     status words; its own split-K region is neither needed nor touched (a shape with max_split2 = 1 is enough).
 *   - limit: split2 * n_tiles * tn * 128 * 4 bytes of partials must fit OB_STATIC_SCRATCH_BYTES minus 16 KiB of
 *     counters; larger requests return OB_ERR_TOO_LARGE before any launch.  Every GPU that loads the library holds
 *     the array (OB_STATIC_SCRATCH_BYTES) until the process exits.
 *   - the first call on each device resolves the array's device address and zeroes its counters on `cuda_stream`;
 *     make that first call before any stream capture.  It calls no cudaMalloc / cudaFree or other allocating routine.
 *   - all calls on a device share the one array: two calls that overlap on the GPU (different streams) race.  A call
 *     that completes leaves the counters at zero; the partial tiles keep the last call's contents and are overwritten
 *     before use.  A call whose device-side wait ran out (status word 0 = OB_DEV_WAIT_TIMEOUT) may leave counters
 *     above zero: ob_read_status, by which the host learns of it, clears the array's counters on the current device
 *     whenever it reads a non-zero status, so call it (with that device current) before the next static call. */
#define OB_STATIC_SCRATCH_BYTES (8u << 20)
int ob_k2_fp8_static(ObLayer* layer, const ObBatch* batch, void* workspace, const ObWorkspaceShape* shape,
                     const ObTileCfg* cfg, int pdl, void* cuda_stream);

/* K1 then K2 linked by programmatic dependent launch: the decode chain `run_pdl` (lowbit_lora/hopper_pdl.py:104-175). */
int ob_chain_fp8(ObLayer* layer, const ObBatch* batch, void* workspace, const ObWorkspaceShape* shape,
                 const ObTileCfg* cfg, void* cuda_stream);

/* The NVFP4-base counterparts of ob_k1_fp8 / ob_k2_fp8 / ob_chain_fp8.  K1 quantizes x to e2m1 codes with one ue4m3
 * scale per 16 elements against the static global scale (vLLM's scaled_fp4_quant recipe) and shrinks; K2 is the
 * block-scaled tcgen05 GEMM (kind::mxf4nvf4, scale factors in TMEM) with the same expand.  Replace the launches of
 * `_shrink_nvfp4` / `_gemm_nvfp4` (lowbit_lora/kernels/nvfp4_lora_vllm.py:591-630) and `run_pdl4`
 * (lowbit_lora/blackwell_pdl.py:59-133). */
int ob_k1_nvfp4(ObLayer* layer, const ObBatch* batch, void* workspace, const ObWorkspaceShape* shape,
                const ObTileCfg* cfg, void* cuda_stream);
int ob_k2_nvfp4(ObLayer* layer, const ObBatch* batch, void* workspace, const ObWorkspaceShape* shape,
                const ObTileCfg* cfg, int pdl, void* cuda_stream);
int ob_chain_nvfp4(ObLayer* layer, const ObBatch* batch, void* workspace, const ObWorkspaceShape* shape,
                   const ObTileCfg* cfg, void* cuda_stream);

/* One-time re-layout of an NVFP4 weight's block scales from the checkpoint's linear [N, K/16] ue4m3 matrix (what the
 * reference keeps before vLLM swizzles it, lowbit_lora/plugin.py:155-174) into the order K2 copies to TMEM: per
 * (128-row output tile of a slice, 256-element K slot) four 512-byte atoms [row % 32][row / 32][4 scales], zero padded.
 * `widths` are host integers.  The caller allocates `packed` (ob_nvfp4_packed_scale_bytes). */
int ob_nvfp4_packed_scale_bytes(int32_t K, int32_t S, const int32_t* widths, size_t* bytes);
int ob_nvfp4_pack_scales(const void* w_sf_linear, int32_t K, int32_t S, const int32_t* widths, void* packed,
                         size_t packed_bytes, void* cuda_stream);

/* Adapter slot (re)quantization on the device, bit-identical to the reference's torch recipes; used when vLLM writes or
 * clears an adapter slot (lowbit_lora/kernels/adapter_store.py:63-80, VllmFusedFP8LoRA.requantize
 * lowbit_lora/kernels/fp8_lora_vllm.py:504-524).  `src` is bf16, rows contiguous, cols a multiple of 8 (16 for NVFP4).
 *   FP8:   per row scale = max(amax / 448, 1e-12), codes = e4m3(x / scale)            -> codes [rows, cols], scales [rows]
 *   NVFP4: per matrix m of `l` matrices [rows, cols]: global = 2688 / amax (the reference's two roundings), ue4m3 scale per
 *          16 elements, packed e2m1 codes  -> packed [l, rows, cols/2], sf [l, rows, cols/16], inv_global [l] = 1 / global
 *          (lowbit_lora/kernels/nvfp4_lora_vllm.py:379-397).  `amax_scratch` = l * 4 bytes of device memory. */
int ob_requant_fp8_rows(const void* src, int64_t rows, int32_t cols, void* codes, float* scales, void* cuda_stream);
int ob_requant_nvfp4(const void* src, int32_t l, int32_t rows, int32_t cols, void* packed, void* sf, float* inv_global,
                     void* amax_scratch, void* cuda_stream);

/* Token sort + segment index on the device: vLLM's LoRAKernelMeta.prepare_tensors
 * (vllm/lora/ops/triton_ops/lora_kernel_metadata.py:110-168) incl. its stale-on-no-adapter behaviour.
 * token_lora [M] int32 in; the five metadata tensors out (tok/srt of capacity >= M, seg_* of L+1 / L+2 / L+1). */
int ob_segment_index(const int32_t* token_lora, int32_t M, int32_t L, int32_t* tok, int32_t* srt, int32_t* seg_n,
                     int32_t* seg_start, int32_t* seg_ids, void* cuda_stream);

/* ---- All-reduce of a row-parallel layer's partial outputs over peer-mapped memory (one NVSwitch box, one process per
 * GPU).  Replaces the NCCL all-reduce vLLM issues after a row-parallel LoRA layer (tensor_model_parallel_all_reduce,
 * vllm/lora/layers/row_parallel_linear.py:73-76; served by the reference's plugin under LOWBIT_TP=1,
 * lowbit_lora/plugin.py:239-245) with one stream-ordered kernel per rank that can sit inside a CUDA graph.
 *
 * Every rank allocates one communication buffer (device memory, zero-initialized, ob_comm_bytes(slot_bytes) bytes, where
 * slot_bytes >= the largest payload), exports it (ob_ipc_export), hands handle + offset to the other ranks by any host
 * channel, and maps theirs (ob_ipc_open).  ObComm.bufs[r] is rank r's buffer as mapped in THIS process (bufs[rank] = the
 * own buffer's ordinary pointer).  All ranks must call ob_allreduce the same number of times with the same count / dtype /
 * mode; the result is bitwise identical on all ranks (partials added in rank order, fp32 accumulation).  Waits on peers are
 * bounded by wait_ms: when one runs out the call's output is left unwritten and ob_comm_status reports it; the ranks must
 * then zero their buffers together before the next call.  Plain peer loads and stores only (no multicast, no TMA). */
#define OB_MAX_RANKS 8
#define OB_IPC_HANDLE_BYTES 64
enum { OB_DTYPE_BF16 = 0, OB_DTYPE_F32 = 1 };
enum { OB_AR_AUTO = 0, OB_AR_ONE_SHOT = 1, OB_AR_TWO_SHOT = 2 };   /* auto: two shots above 512 KB on more than 2 ranks */
typedef struct ObComm {
    int32_t world, rank;             /* 2..OB_MAX_RANKS ranks */
    void* bufs[OB_MAX_RANKS];
    size_t slot_bytes;               /* as given to ob_comm_bytes (a multiple of 16) */
} ObComm;
int ob_comm_bytes(size_t slot_bytes, size_t* bytes);
int ob_ipc_export(const void* dev_ptr, unsigned char handle[OB_IPC_HANDLE_BYTES], size_t* offset);
int ob_ipc_open(const unsigned char handle[OB_IPC_HANDLE_BYTES], size_t offset, void** mapped);
int ob_ipc_close(void* mapped, size_t offset);
/* dst[i] = sum over ranks of src[i], i < count; count * element size a multiple of 16 and <= slot_bytes; src and dst 16-byte
 * aligned device pointers of this rank (they may be the same). */
int ob_allreduce(const ObComm* comm, const void* src, void* dst, int64_t count, int32_t dtype, int32_t mode, int32_t wait_ms,
                 void* cuda_stream);
/* The same exchange for `n` ranks that all live on the CURRENT device, as ONE cooperative launch (ranks on one GPU must not
 * be separate launches that wait for one another): for tests without a second GPU.  comms[q].bufs are ordinary pointers. */
int ob_allreduce_emulated(const ObComm* comms, int32_t n, const void* const* src, void* const* dst, int64_t count,
                          int32_t dtype, int32_t mode, int32_t wait_ms, void* cuda_stream);
/* A row-parallel projection with its all-reduce: K1, then K2 whose epilogue stages each finished output tile in this rank's
 * communication buffer, announces it to the peers with a per-tile flag, waits (bounded) for every rank's copy of that tile
 * and stores the sum -- the exchange of vLLM's row-parallel LoRA layers (row_parallel_linear.py:73-76) without a launch of
 * its own and without a second pass over y.  Bitwise the same result as the chain followed by ob_allreduce (same rank
 * order, fp32 accumulation).  Serves decode batches (at most 32 tokens) on the tile-per-CTA kernel for either base
 * format; any other call runs the chain and then the stand-alone kernel (y must then be dense: ldy = N).  Counts as one
 * call of the communication buffer on every rank, like ob_allreduce. */
int ob_chain_allreduce(ObLayer* layer, const ObBatch* batch, void* workspace, const ObWorkspaceShape* shape, const ObTileCfg* cfg,
                       const ObComm* comm, void* cuda_stream);

/* Copy the buffer's 8 state words to the host (synchronizes the stream): [0] calls completed, [3] 0 = ok / 1 = a wait ran out,
 * [4] which wait (1 = partials, 2 = reduced slices), [5] the rank that was missing, [6] the call.  Clears [3..6]. */
int ob_comm_status(const ObComm* comm, int32_t host_out[8], void* cuda_stream);

/* In-kernel timeline for profiling (the reference has no counterpart: it profiles with torch.profiler only,
 * bench/overhead.py:111-113).  While a buffer is set, every K2 CTA stores OB_TRACE_EVENTS global-timer stamps (ns) at
 * buffer[cta * OB_TRACE_EVENTS + event], cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z); CTAs beyond
 * `max_ctas` store nothing.  K1 CTAs store 4 stamps each (start, segment index read, dependency wait passed, end of
 * warp 0) in a second region of the same size that follows the first: the buffer holds 2 * max_ctas * OB_TRACE_EVENTS
 * 64-bit words.  Pass a null pointer to switch it off (the default).  Process-wide, not thread-safe. */
#define OB_TRACE_EVENTS 16
int ob_trace_buffer(void* device_u64_buffer, int64_t max_ctas);

/* Copy the workspace's OB_STATUS_WORDS status words to host memory (synchronizes the stream) and clear them.  If word 0
 * is not OB_DEV_OK it also zeroes the arrival counters of ob_k2_fp8_static's array on the current device. */
int ob_read_status(void* workspace, int32_t* host_out, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* ONEBASE_B200_H */
