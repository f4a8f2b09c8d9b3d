// Adapter slot (re)quantization: the low-precision copies of vLLM's bf16 LoRA buffers, made on the device when a slot is
// written.  Bit-identical to the reference's torch recipes:
//   * FP8 (lowbit_lora/kernels/adapter_store.py:63-80, `_store`): per row, scale = max(amax / 448, 1e-12) (IEEE division),
//     code = e4m3_rn(clamp(x / scale, -448, 448)) (IEEE division, one rounding).
//   * NVFP4 (lowbit_lora/kernels/nvfp4_lora_vllm.py:379-397, `nvfp4_quant_batched`): per matrix, global = rcp(max(amax,
//     1e-12)) * 2688 (reciprocal, then the product: the two roundings torch's `scalar / tensor` makes); per 16-element
//     block sf = e4m3_rn(min(global * (blockmax * (1/6)), 448)), out = sf != 0 ? 1 / (sf * (1 / global)) : 0,
//     code = e2m1_rn(x * out) with the reference's threshold chain; codes packed two per byte (element 2i in the low
//     nibble); the matrix's inverse global 1 / global is stored beside them.
// One CTA per row; the NVFP4 form needs the matrix's amax first (a kernel of its own, atomicMax on the float's bits).
#include "k1_device.cuh"

namespace ob {

constexpr int kRqThreads = 128;

__global__ void __launch_bounds__(kRqThreads)
requant_fp8_rows_kernel(const __nv_bfloat16* __restrict__ src, int cols, uint8_t* __restrict__ codes, float* __restrict__ scales) {
    __shared__ float s_part[kRqThreads / 32];
    __shared__ float s_scale;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t row = blockIdx.x;
    const uint4* xr = reinterpret_cast<const uint4*>(src + row * (size_t)cols);
    const int nvec = cols >> 3;                       // 8 bf16 per 16-byte vector; a tail of < 8 elements follows
    float amax = 0.0f;
    for (int i = tid; i < nvec; i += kRqThreads) amax = fmaxf(amax, amax8(__ldg(xr + i)));
    for (int c = nvec * 8 + tid; c < cols; c += kRqThreads) amax = fmaxf(amax, fabsf(__bfloat162float(src[row * (size_t)cols + c])));
#pragma unroll
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0) s_part[warp] = amax;
    __syncthreads();
    if (tid == 0) {
        float m = s_part[0];
        for (int w = 1; w < kRqThreads / 32; ++w) m = fmaxf(m, s_part[w]);
        const float sc = fmaxf(__fdiv_rn(m, kFp8Max), 1e-12f);
        s_scale = sc;
        scales[row] = sc;
    }
    __syncthreads();
    const float sc = s_scale;
    uint2* out = reinterpret_cast<uint2*>(codes + row * (size_t)cols);
#pragma unroll 1
    for (int i = tid; i < nvec; i += kRqThreads) out[i] = quant8(__ldg(xr + i), sc);
    for (int c = nvec * 8 + tid; c < cols; c += kRqThreads) {
        const float v = q1(__bfloat162float(src[row * (size_t)cols + c]), sc);
        codes[row * (size_t)cols + c] = (uint8_t)(cvt_e4m3x2(v, 0.0f) & 0xFFu);
    }
}

// amax of each of the `l` matrices of `per` elements (grid: x = chunks of a matrix, y = matrix).  amax_bits[] starts at 0.
__global__ void __launch_bounds__(256)
requant_amax_kernel(const __nv_bfloat16* __restrict__ src, size_t per, unsigned int* __restrict__ amax_bits) {
    const __nv_bfloat16* m = src + (size_t)blockIdx.y * per;
    float amax = 0.0f;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < per; i += (size_t)gridDim.x * blockDim.x)
        amax = fmaxf(amax, fabsf(__bfloat162float(m[i])));
#pragma unroll
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) atomicMax(amax_bits + blockIdx.y, __float_as_uint(amax));   // non-negative floats order as integers
}

// One CTA per row of one matrix (grid: x = row, y = matrix); one thread per 16-element block.
__global__ void __launch_bounds__(kRqThreads)
requant_nvfp4_kernel(const __nv_bfloat16* __restrict__ src, int rows, int cols, const unsigned int* __restrict__ amax_bits,
                     uint8_t* __restrict__ packed, uint8_t* __restrict__ sf, float* __restrict__ inv_global) {
    const int l = blockIdx.y;
    const size_t row = (size_t)l * rows + blockIdx.x;
    const float amax = fmaxf(__uint_as_float(amax_bits[l]), 1e-12f);
    const float gs = __fmul_rn(__frcp_rn(amax), 448.0f * 6.0f);
    if (blockIdx.x == 0 && threadIdx.x == 0) inv_global[l] = __frcp_rn(gs);
    const float rgs = __frcp_rn(gs);
    const float rcp6 = 1.0f / 6.0f;                   // the fp32 constant torch multiplies by
    const __nv_bfloat16* xr = src + row * (size_t)cols;
    for (int b = threadIdx.x; b < cols / 16; b += kRqThreads) {
        float v[16];
        unpack8(__ldg(reinterpret_cast<const uint4*>(xr) + 2 * b), *reinterpret_cast<float(*)[8]>(&v[0]));
        unpack8(__ldg(reinterpret_cast<const uint4*>(xr) + 2 * b + 1), *reinterpret_cast<float(*)[8]>(&v[8]));
        float vmax = 0.0f;
#pragma unroll
        for (int e = 0; e < 16; ++e) vmax = fmaxf(vmax, fabsf(v[e]));
        const float sfv = fminf(__fmul_rn(gs, __fmul_rn(vmax, rcp6)), 448.0f);
        const uint32_t sf_code = (uint32_t)cvt_e4m3x2(sfv, 0.0f) & 0xFFu;
        const float sff = e4m3_to_float(sf_code);
        const float osc = sff != 0.0f ? __frcp_rn(__fmul_rn(sff, rgs)) : 0.0f;
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            lo |= e2m1_code(__fmul_rn(v[e], osc)) << (4 * e);
            hi |= e2m1_code(__fmul_rn(v[8 + e], osc)) << (4 * e);
        }
        *reinterpret_cast<uint2*>(packed + row * (size_t)(cols / 2) + (size_t)b * 8) = make_uint2(lo, hi);
        sf[row * (size_t)(cols / 16) + b] = (uint8_t)sf_code;
    }
}

cudaError_t launch_requant_fp8(const void* src, long long rows, int cols, void* codes, float* scales, cudaStream_t stream) {
    requant_fp8_rows_kernel<<<(unsigned)rows, kRqThreads, 0, stream>>>(static_cast<const __nv_bfloat16*>(src), cols,
                                                                      static_cast<uint8_t*>(codes), scales);
    return cudaGetLastError();
}

cudaError_t launch_requant_nvfp4(const void* src, int l, int rows, int cols, void* packed, void* sf, float* inv_global,
                                 unsigned int* amax_bits, cudaStream_t stream) {
    cudaError_t e = cudaMemsetAsync(amax_bits, 0, sizeof(unsigned int) * (size_t)l, stream);
    if (e != cudaSuccess) return e;
    const size_t per = (size_t)rows * cols;
    unsigned chunks = (unsigned)((per + 256 * 16 - 1) / (256 * 16));
    if (chunks > 512) chunks = 512;
    if (chunks < 1) chunks = 1;
    requant_amax_kernel<<<dim3(chunks, (unsigned)l), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(src), per, amax_bits);
    requant_nvfp4_kernel<<<dim3((unsigned)rows, (unsigned)l), kRqThreads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(src), rows, cols, amax_bits, static_cast<uint8_t*>(packed), static_cast<uint8_t*>(sf),
        inv_global);
    return cudaGetLastError();
}

}  // namespace ob
