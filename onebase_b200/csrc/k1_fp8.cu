// K1: activation quantization -- per-token dynamic e4m3 for an FP8 base, or e2m1 codes with one ue4m3 scale per 16
// elements against a static global scale for an NVFP4 base -- fused in one launch with every tenant's LoRA shrink
// h = x A^T.
//
// One launch, two kinds of CTA (256 threads each):
//   * CTAs [0, M): quantize one tile POSITION each.  Position p stands for row `position_row(p)` of x: the adapter-sorted
//     order whenever the batch has an adapter, so that K2 can fetch contiguous rows by TMA.  amax over the row in fp32,
//     s_x = max(amax / 448, 1/(448*512)) and code = e4m3_rn(clamp(x / s_x)) with IEEE divisions and ONE rounding step:
//     the rule of lowbit_lora/kernels/fp8_lora_vllm.py:47-71 (vLLM's dynamic per-token quantization), bit for bit.
//   * the remaining CTAs: 8 independent warps each; a warp owns (block of 1 or 4 sorted positions, slice, 8 rank rows,
//     K split) and streams that [8, K/split] block of the positions' adapter A from HBM with 16-byte loads, multiplying it
//     into up to 4 tokens at a time (their x rows come from L2; tokens of one tenant handled by different warps re-read
//     A through L2, not HBM).  The 32 lane-partial sums per warp (8 rank rows x 4 tokens) are
//     reduced with a transposing butterfly -- 31 shuffles for 32 sums, lane i ends up with sum i -- and written as
//     split-K partials hp[split][slice][position][rank] (fp32), which K2 adds in split order (deterministic).
//     Computes what lowbit_lora/kernels/fp8_lora_vllm.py:72-120 computes per adapter segment.
// The kernel starts with griddepcontrol.launch_dependents so that a dependent K2 may begin streaming W at once, and it
// may itself be launched as a programmatic dependent of the preceding kernel: it reads the segment index and requests
// its first block of A before griddepcontrol.wait, and touches x and the scratch only after it.
#include <atomic>

#include "k1_device.cuh"

namespace ob {

constexpr int kK1Threads = 256;

// One instantiation per (adapter storage, base format): each launch carries only the code of its own case.
// LOOPED: the one-CTA-per-SM form that runs beside the persistent GEMM; a function of its own, because the shared-memory
// carve-out it needs (see launch_k1_impl) is a per-function attribute and costs the other form its L1 cache.
// XOP: the projection's input is formed from x on the fly (OB_X_SILU_MUL); plain launches run an instantiation without it.
template <int LORA_FMT, bool FP4_BASE, bool LOOPED, bool XOP>
__global__ void __launch_bounds__(kK1Threads, XOP ? 2 : 0) k1_kernel(const K1Params p) {
    griddep_launch_dependents();
    OB_TRACE1(0)
    if ((int)blockIdx.x < p.n_quant_ctas) {
        const int row = row_of_position(p, blockIdx.x, threadIdx.x & 31);
        griddep_wait();                               // x comes from the preceding kernel; the scratch may still be read by it
        if (FP4_BASE) quantize_row_nvfp4<kK1Threads, XOP>(p, blockIdx.x, row, threadIdx.x);
        else quantize_row<kK1Threads, 0, XOP>(p, blockIdx.x, row, threadIdx.x);
        if (p.xs != nullptr) {                        // the tensor-core shrink reads x in position order by TMA
            const __nv_bfloat16* xr = p.x + (int64_t)row * p.ldx;
            uint4* xo = reinterpret_cast<uint4*>(p.xs + (size_t)blockIdx.x * (size_t)p.K);
            for (int i = threadIdx.x; i < (p.K >> 3); i += kK1Threads) xo[i] = x_load8<XOP>(p, xr, i * 8);
        }
        if (p.xq_ready != nullptr) {          // chain: tell K2 that this position's codes and scale are in memory
            __syncthreads();
            if (threadIdx.x == 0) red_release_add(p.xq_ready, 1);
        }
        OB_TRACE1(3)
        if (!LOOPED) return;
    }
    const int lane = threadIdx.x & 31;
    if (LOOPED) {
        // One CTA per SM at most (so that a dependent GEMM's CTAs fit beside this kernel's and stream weights while it
        // runs): every warp of the grid walks the shrink units with the grid's stride; the quantizing CTAs join after
        // their position.
        const long long total = (long long)p.n_pblocks * p.units_per_block;
        const long long stride = (long long)gridDim.x * (kK1Threads / 32);
        for (long long w = (long long)blockIdx.x * (kK1Threads / 32) + (threadIdx.x >> 5); w < total; w += stride)
            shrink_unit<LORA_FMT, XOP>(p, (int)(w / p.units_per_block), (int)(w % p.units_per_block), lane);
        OB_TRACE1(3)
        return;
    }
    const int w = ((int)blockIdx.x - p.n_quant_ctas) * (kK1Threads / 32) + (threadIdx.x >> 5);
    const int pb = w / p.units_per_block;
    if (pb >= p.n_pblocks) return;
    shrink_unit<LORA_FMT, XOP>(p, pb, w % p.units_per_block, lane);
    OB_TRACE1(3)
}

// Quantization alone, for batches whose shrink runs on the tensor cores: without the shrink's registers four of these
// CTAs share an SM instead of two, which is what a launch of thousands of one-row CTAs needs.
template <bool FP4_BASE>
__global__ void __launch_bounds__(kK1Threads, 4) k1_quant_kernel(const K1Params p) {
    griddep_launch_dependents();
    const int row = row_of_position(p, blockIdx.x, threadIdx.x & 31);
    griddep_wait();
    if (FP4_BASE) quantize_row_nvfp4<kK1Threads, false, true>(p, blockIdx.x, row, threadIdx.x);
    else quantize_row<kK1Threads, 0>(p, blockIdx.x, row, threadIdx.x);
    if (!FP4_BASE && p.xs != nullptr) {
        const __nv_bfloat16* xr = p.x + (int64_t)row * p.ldx;
        uint4* xo = reinterpret_cast<uint4*>(p.xs + (size_t)blockIdx.x * (size_t)p.K);
        for (int i = threadIdx.x; i < (p.K >> 3); i += kK1Threads) xo[i] = x_load8<false>(p, xr, i * 8);
    }
}

// The FP8 base's form of it with the row in registers (NV vectors per thread): one read of x serves the amax, the codes
// and the sorted copy; rows of up to 4096 elements run eight CTAs per SM (the launch is bound by how many rows an SM has
// in flight, not by bytes).
template <int NV>
__global__ void __launch_bounds__(kK1Threads, NV <= 2 ? 8 : 4) k1_quant_regs_kernel(const K1Params p) {
    griddep_launch_dependents();
    const int row = row_of_position(p, blockIdx.x, threadIdx.x & 31);
    griddep_wait();
    quantize_row_regs<kK1Threads, 0, NV>(p, blockIdx.x, row, threadIdx.x);
}

template <int LORA_FMT, bool FP4_BASE>
static cudaError_t launch_k1_impl(const K1Params& p, int grid, int pdl, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kK1Threads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    if (p.looped) {
        // Beside the persistent GEMM, K1 needs next to no shared memory but must leave the SMs it runs on configured for the
        // LARGEST shared-memory carve-out: the split between L1 and shared memory only changes on an idle SM, so with the
        // default (small) carve-out the dependent GEMM's CTAs (150-200 KB each) could not become resident beside K1's and
        // the two kernels of the chain would run one after the other.  (It costs this form most of its L1 cache.)
        static std::atomic<unsigned long long> carved{0};
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64 && !(carved.load() & (1ull << dev))) {
            cudaError_t e = cudaFuncSetAttribute(k1_kernel<LORA_FMT, FP4_BASE, true, false>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                                 (int)cudaSharedmemCarveoutMaxShared);
            if (e != cudaSuccess) return e;
            carved.fetch_or(1ull << dev);
        }
        return cudaLaunchKernelEx(&cfg, k1_kernel<LORA_FMT, FP4_BASE, true, false>, p);
    }
    if (p.x_op != OB_X_PLAIN) return cudaLaunchKernelEx(&cfg, k1_kernel<LORA_FMT, FP4_BASE, false, true>, p);
    if (grid == p.n_quant_ctas && p.xq_ready == nullptr && p.trace == nullptr) {   // no shrink warps in this launch
        if (!FP4_BASE && p.K <= 16 * kK1Threads) return cudaLaunchKernelEx(&cfg, k1_quant_regs_kernel<2>, p);
        if (!FP4_BASE && p.K <= 48 * kK1Threads) return cudaLaunchKernelEx(&cfg, k1_quant_regs_kernel<6>, p);
        return cudaLaunchKernelEx(&cfg, k1_quant_kernel<FP4_BASE>, p);
    }
    return cudaLaunchKernelEx(&cfg, k1_kernel<LORA_FMT, FP4_BASE, false, false>, p);
}

cudaError_t launch_k1_fp8(const K1Params& p, int grid, int pdl, cudaStream_t stream) {
    const bool fp4 = p.base_fmt == OB_BASE_NVFP4;
    switch (p.lora_fmt) {
        case kLoraFp8:
            return fp4 ? launch_k1_impl<kLoraFp8, true>(p, grid, pdl, stream) : launch_k1_impl<kLoraFp8, false>(p, grid, pdl, stream);
        case kLoraNvfp4:
            return fp4 ? launch_k1_impl<kLoraNvfp4, true>(p, grid, pdl, stream) : launch_k1_impl<kLoraNvfp4, false>(p, grid, pdl, stream);
        default:
            return fp4 ? launch_k1_impl<kLoraBf16, true>(p, grid, pdl, stream) : launch_k1_impl<kLoraBf16, false>(p, grid, pdl, stream);
    }
}

}  // namespace ob
