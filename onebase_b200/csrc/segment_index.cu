// Token sort + segment index on the device: the five tensors vLLM's LoRAKernelMeta.prepare_tensors builds with torch
// sort / unique / cumsum (vllm/lora/ops/triton_ops/lora_kernel_metadata.py:110-168), bit for bit, including its
// statefulness: the three segment arrays are always reset; a batch whose every token is -1 stops there and leaves the
// token map and the sorted indices as they were.
//
// One CTA.  Histogram of slot ids in shared memory (bin 0 = "-1"), compaction of the non-empty bins to the front
// (sorted unique ids), exclusive scan for the start offsets, then a stable counting sort: one warp per bin walks the
// tokens in order, 32 at a time, and ranks the matching lanes with ballot + popc.
#include "ob_common.cuh"

namespace ob {

constexpr int kSegThreads = 1024;

__global__ void __launch_bounds__(kSegThreads) segment_index_kernel(const int32_t* __restrict__ token_lora, int M, int L,
                                                                    int32_t* tok, int32_t* srt, int32_t* seg_n,
                                                                    int32_t* seg_start, int32_t* seg_ids) {
    extern __shared__ int32_t sm[];
    int32_t* count = sm;                  // [L+1] tokens per bin
    int32_t* start = sm + (L + 1);        // [L+1] first sorted position of each bin
    __shared__ int any_adapter;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int bins = L + 1;
    for (int i = tid; i < bins; i += kSegThreads) {
        count[i] = 0;
        seg_n[i] = 0;
        seg_ids[i] = -1;
    }
    for (int i = tid; i < L + 2; i += kSegThreads) seg_start[i] = 0;
    if (tid == 0) any_adapter = 0;
    __syncthreads();
    int mine = 0;
    for (int i = tid; i < M; i += kSegThreads) {
        const int id = token_lora[i];
        if (id >= 0 && id < L) {
            mine = 1;
            atomicAdd(&count[id + 1], 1);
        } else {
            atomicAdd(&count[0], 1);
        }
    }
    if (mine) any_adapter = 1;
    __syncthreads();
    if (!any_adapter) return;             // the reset is all that happens; tok / srt stay stale
    for (int i = tid; i < M; i += kSegThreads) tok[i] = token_lora[i];
    if (warp == 0) {                      // compaction + scan over the bins, 32 at a time, in order
        int n_seg = 0, run = 0;
        for (int base = 0; base < bins; base += 32) {
            const int b = base + lane;
            const int c = b < bins ? count[b] : 0;
            const uint32_t m = __ballot_sync(0xffffffffu, c > 0);
            int incl = c;                 // inclusive scan of the counts within the warp
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            if (b < bins) start[b] = run + incl - c;
            if (c > 0) {
                const int slot = n_seg + __popc(m & ((1u << lane) - 1u));
                seg_ids[slot] = b - 1;
                seg_n[slot] = c;
                seg_start[slot + 1] = run + incl;
            }
            n_seg += __popc(m);
            run += __shfl_sync(0xffffffffu, incl, 31);
        }
    }
    __syncthreads();
    for (int b = warp; b < bins; b += kSegThreads / 32) {
        if (count[b] == 0) continue;
        const int want = b - 1;
        int rank = start[b];
        for (int base = 0; base < M; base += 32) {
            const int i = base + lane;
            int id = -2;
            if (i < M) {
                id = token_lora[i];
                if (id < 0 || id >= L) id = -1;
            }
            const uint32_t m = __ballot_sync(0xffffffffu, id == want);
            if (id == want) srt[rank + __popc(m & ((1u << lane) - 1u))] = i;
            rank += __popc(m);
        }
    }
}

cudaError_t launch_segment_index(const int32_t* token_lora, int M, int L, int32_t* tok, int32_t* srt, int32_t* seg_n,
                                 int32_t* seg_start, int32_t* seg_ids, cudaStream_t stream) {
    segment_index_kernel<<<1, kSegThreads, sizeof(int32_t) * 2 * (L + 1), stream>>>(token_lora, M, L, tok, srt, seg_n,
                                                                                   seg_start, seg_ids);
    return cudaGetLastError();
}

}  // namespace ob
