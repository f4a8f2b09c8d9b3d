// All-reduce (sum) of a row-parallel layer's partial outputs over the GPUs of one NVSwitch box, as ONE kernel per rank
// that reads its peers' buffers directly (peer-mapped memory, plain loads over NVLink): the exchange step vLLM performs
// with tensor_model_parallel_all_reduce after a row-parallel LoRA layer (vllm/lora/layers/row_parallel_linear.py:73-76),
// which the reference serves under LOWBIT_TP=1 (lowbit_lora/plugin.py:239-245) through NCCL.
//
// Why not NCCL: the payload is 64 KB - 2 MB per layer call and the call sits between two kernels of a CUDA graph; a
// library collective costs its launch and protocol latency twice per decoder layer.  This kernel is stream-ordered like
// any other launch (so a whole layer is one graph), takes one flag round per call, and every rank adds the partials in
// rank order with fp32 accumulation, so all ranks hold bitwise the same result.
//
// Each rank owns a communication buffer (caller-allocated, zero-initialized, mapped into every peer by CUDA IPC):
//     [0, 1 KB)      state   int32: [0] calls completed (the epoch), [1] CTAs that staged, [2] CTAs that reduced their slice,
//                            [3] status (0 ok, 1 = a wait ran out), [4..6] which wait / rank / call, [7] CTAs finished
//     [1 KB, 2 KB)   flags   int32[world]: flags[r] = last epoch for which rank r's data is ready (written BY rank r)
//     [2 KB, 3 KB)   flags2  int32[world]: two-shot form: rank r's reduced slice is ready
//     [4 KB, 16 KB)  per-tile flags int32[world][384] of the all-reduce fused into K2's epilogue (k2_gemm.cu)
//     [16 KB, ...)   data[2][slot] then red[2][slot]: the staged partials (by epoch parity) and the reduced slices
// One call on rank q:  (1) every CTA copies its share of `src` into data[epoch & 1] of its OWN buffer; the last CTA to
// finish that (an arrival counter -- no CTA waits for another CTA of its grid) publishes flags[q] = epoch in every
// peer's buffer with a system-scope release.  (2) every CTA waits, bounded, until its own buffer's flags[r] >= epoch for
// all r (system-scope acquire).  (3a) one-shot form (small payloads): each thread adds element i of every rank's staged
// copy, r = 0 .. world-1, and writes dst[i].  (3b) two-shot form: rank q reduces only slice q that way into red[epoch & 1]
// of its own buffer, publishes flags2[q], then gathers every slice from the rank that reduced it.
// The staged copies are double-buffered by epoch parity: a rank can only overwrite data[p] two calls later, and it cannot
// get there before every peer has published the epoch in between, i.e. finished reading.  The epoch lives in the buffer
// and is advanced by the last CTA to finish, so a captured graph can be replayed.
// Every wait is bounded (wait_ms); a wait that runs out sets the status word and the CTA goes on WITHOUT reading peers.
// No multicast / multimem and no TMA: plain ld.global / st.global on peer pointers.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ob_common.cuh"

namespace ob {

constexpr int kArThreads = 256;

struct ArParams {
    int world, rank;
    int dtype;                 // 0 = bf16, 1 = fp32
    int two_shot;
    long long count;           // elements
    long long slot_bytes;      // bytes of one staged copy
    uint32_t wait_ms;
    const void* src;
    void* dst;
    uint8_t* bufs[OB_MAX_RANKS];   // every rank's communication buffer as mapped into THIS process (bufs[rank] = own)
};

// Several ranks emulated by one launch on one GPU (tests): blockIdx.y picks the rank's parameter block.
struct ArBatch {
    ArParams r[OB_MAX_RANKS];
};

__device__ __forceinline__ uint64_t ar_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
    int32_t v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_peer16(const void* p) {     // data another GPU wrote: never from a stale local cache line
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// Bounded wait until flags[r] >= epoch for every rank r (thread r of the CTA polls rank r's flag).  Returns false if the
// limit ran out; the status words then say which rank was missing.
__device__ bool ar_wait_flags(const ArParams& p, int32_t* state, const int32_t* flags, int32_t epoch, int where) {
    __shared__ int s_ok;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if ((int)threadIdx.x < p.world) {
        const uint64_t limit = (uint64_t)p.wait_ms * 1000000ull, t0 = ar_timer_ns();
        bool ok = false;
        for (uint32_t spin = 0;; ++spin) {
            if (ld_acquire_sys(flags + threadIdx.x) - epoch >= 0) { ok = true; break; }
            if ((spin & 63u) == 63u && ar_timer_ns() - t0 > limit) break;
        }
        if (!ok) {
            s_ok = 0;
            if (atomicCAS(state + 3, 0, 1) == 0) {
                state[4] = where;
                state[5] = (int32_t)threadIdx.x;      // the rank whose flag did not arrive
                state[6] = epoch;
            }
        }
    }
    __syncthreads();
    return s_ok != 0;
}

template <typename T> struct ArVec;
template <> struct ArVec<__nv_bfloat16> {
    static __device__ __forceinline__ void add(float (&acc)[8], const uint4& v) {
        acc[0] += __uint_as_float(v.x << 16); acc[1] += __uint_as_float(v.x & 0xFFFF0000u);
        acc[2] += __uint_as_float(v.y << 16); acc[3] += __uint_as_float(v.y & 0xFFFF0000u);
        acc[4] += __uint_as_float(v.z << 16); acc[5] += __uint_as_float(v.z & 0xFFFF0000u);
        acc[6] += __uint_as_float(v.w << 16); acc[7] += __uint_as_float(v.w & 0xFFFF0000u);
    }
    static __device__ __forceinline__ uint4 pack(const float (&acc)[8]) {
        __nv_bfloat162 a = __floats2bfloat162_rn(acc[0], acc[1]), b = __floats2bfloat162_rn(acc[2], acc[3]);
        __nv_bfloat162 c = __floats2bfloat162_rn(acc[4], acc[5]), d = __floats2bfloat162_rn(acc[6], acc[7]);
        return make_uint4(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b), *reinterpret_cast<uint32_t*>(&c),
                          *reinterpret_cast<uint32_t*>(&d));
    }
    static constexpr int kPerVec = 8;
};
template <> struct ArVec<float> {
    static __device__ __forceinline__ void add(float (&acc)[8], const uint4& v) {
        acc[0] += __uint_as_float(v.x); acc[1] += __uint_as_float(v.y); acc[2] += __uint_as_float(v.z); acc[3] += __uint_as_float(v.w);
    }
    static __device__ __forceinline__ uint4 pack(const float (&acc)[8]) {
        return make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]), __float_as_uint(acc[3]));
    }
    static constexpr int kPerVec = 4;
};

template <typename T>
__global__ void __launch_bounds__(kArThreads) allreduce_kernel(const ArBatch batch) {
    const ArParams& p = batch.r[blockIdx.y];
    uint8_t* own = p.bufs[p.rank];
    int32_t* state = reinterpret_cast<int32_t*>(own);
    const int32_t epoch = state[0] + 1;                       // this call's epoch (the previous call on this rank has finished)
    const int par = epoch & 1;
    const long long nvec = (p.count + ArVec<T>::kPerVec - 1) / ArVec<T>::kPerVec;   // 16-byte vectors (count is a multiple)
    const long long gsize = (long long)gridDim.x * kArThreads, gid = (long long)blockIdx.x * kArThreads + threadIdx.x;
    __shared__ int s_last;

    // (1) stage this rank's partial in its own buffer; the last CTA publishes "ready" to every rank
    uint4* stage = reinterpret_cast<uint4*>(own + kArStateBytes + (size_t)par * p.slot_bytes);
    const uint4* src = reinterpret_cast<const uint4*>(p.src);
    for (long long i = gid; i < nvec; i += gsize) stage[i] = src[i];
    // The staged copy is in this GPU's own memory, where peers read it through this GPU's L2: a device-scope fence orders it
    // before the arrival; the last CTA has then observed every CTA's arrival, and its system-scope release (cumulative)
    // publishes the whole copy.  (A system-scope fence in every thread cost several microseconds per call.)
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(state + 1, 1) == (int)gridDim.x - 1 ? 1 : 0;
    __syncthreads();
    if (s_last) {
        __threadfence();
        if ((int)threadIdx.x < p.world)
            st_release_sys(reinterpret_cast<int32_t*>(p.bufs[threadIdx.x] + kArFlagsOff) + p.rank, epoch);
    }

    // (2) wait for every rank's partial
    const bool ok = ar_wait_flags(p, state, reinterpret_cast<const int32_t*>(own + kArFlagsOff), epoch, 1);

    uint4* dst = reinterpret_cast<uint4*>(p.dst);
    if (ok && !p.two_shot) {
        // (3a) one shot: every rank adds all partials, in rank order; two vectors per thread in flight per pass, so that a
        // large payload is not one NVLink round trip per 16 bytes and thread
        for (long long i0 = gid; i0 < nvec; i0 += 2 * gsize) {
            const long long i1 = i0 + gsize;
            const bool two = i1 < nvec;
            uint4 v0[OB_MAX_RANKS], v1[OB_MAX_RANKS];
#pragma unroll
            for (int r = 0; r < OB_MAX_RANKS; ++r)
                if (r < p.world) {
                    const uint8_t* base = p.bufs[r] + kArStateBytes + (size_t)par * p.slot_bytes;
                    v0[r] = ld_peer16(base + (size_t)i0 * 16);
                    if (two) v1[r] = ld_peer16(base + (size_t)i1 * 16);
                }
            float a0[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f}, a1[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int r = 0; r < OB_MAX_RANKS; ++r)
                if (r < p.world) {
                    ArVec<T>::add(a0, v0[r]);
                    if (two) ArVec<T>::add(a1, v1[r]);
                }
            dst[i0] = ArVec<T>::pack(a0);
            if (two) dst[i1] = ArVec<T>::pack(a1);
        }
    } else if (ok) {
        // (3b) two shots: this rank reduces slice `rank` (vectors [lo, hi)), publishes it, then gathers every slice
        const long long per = (nvec + p.world - 1) / p.world;
        const long long lo = per * p.rank, hi = (lo + per < nvec) ? lo + per : nvec;
        const size_t red_off = kArStateBytes + 2 * (size_t)p.slot_bytes + (size_t)par * p.slot_bytes;
        uint4* red = reinterpret_cast<uint4*>(own + red_off);
        for (long long i = lo + gid; i < hi; i += gsize) {
            uint4 v[OB_MAX_RANKS];
#pragma unroll
            for (int r = 0; r < OB_MAX_RANKS; ++r)
                if (r < p.world) v[r] = ld_peer16(p.bufs[r] + kArStateBytes + (size_t)par * p.slot_bytes + (size_t)i * 16);
            float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int r = 0; r < OB_MAX_RANKS; ++r)
                if (r < p.world) ArVec<T>::add(acc, v[r]);
            red[i] = ArVec<T>::pack(acc);
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) s_last = atomicAdd(state + 2, 1) == (int)gridDim.x - 1 ? 1 : 0;
        __syncthreads();
        if (s_last) {
            __threadfence();
            if ((int)threadIdx.x < p.world)
                st_release_sys(reinterpret_cast<int32_t*>(p.bufs[threadIdx.x] + kArFlags2Off) + p.rank, epoch);
        }
        if (ar_wait_flags(p, state, reinterpret_cast<const int32_t*>(own + kArFlags2Off), epoch, 2)) {
            for (long long i = gid; i < nvec; i += gsize) {
                const int r = (int)(i / per);
                dst[i] = ld_peer16(p.bufs[r] + red_off + (size_t)i * 16);
            }
        }
    }

    // the last CTA to finish advances the epoch and returns the arrival counters to zero (for the next call / replay)
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(state + 7, 1) == (int)gridDim.x - 1) {
            state[1] = 0;
            state[2] = 0;
            state[7] = 0;
            __threadfence();
            state[0] = epoch;
        }
    }
}

cudaError_t launch_allreduce(const ArBatch& b, int n_emulated, int grid_x, cudaStream_t stream) {
    const dim3 grid((unsigned)grid_x, (unsigned)n_emulated);
    if (n_emulated > 1) {
        // Ranks emulated on ONE GPU wait for one another inside one launch: every CTA must be resident at once.
        void* args[] = {const_cast<ArBatch*>(&b)};
        return b.r[0].dtype == 0
                   ? cudaLaunchCooperativeKernel(reinterpret_cast<void*>(allreduce_kernel<__nv_bfloat16>), grid, dim3(kArThreads), args, 0, stream)
                   : cudaLaunchCooperativeKernel(reinterpret_cast<void*>(allreduce_kernel<float>), grid, dim3(kArThreads), args, 0, stream);
    }
    if (b.r[0].dtype == 0) allreduce_kernel<__nv_bfloat16><<<grid, kArThreads, 0, stream>>>(b);
    else allreduce_kernel<float><<<grid, kArThreads, 0, stream>>>(b);
    return cudaGetLastError();
}

}  // namespace ob
