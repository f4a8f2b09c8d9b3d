// One-time re-layout of an NVFP4 weight's ue4m3 block scales: linear [N, K/16] (the checkpoint's layout) -> the order in
// which K2 moves them to TMEM.  Per (128-row output tile of a slice, 256-element K slot) 2048 bytes = 4 atoms (one per
// 64-element MMA) of 512 bytes [row % 32][row / 32][4 scales]: the scale-factor atom of the block-scaled tcgen05 MMA.
// Rows past a slice's width and scale columns past K/16 are zero.
#include "ob_common.cuh"

namespace ob {

struct PackArgs {
    int K16, kslots, S;
    int widths[OB_MAX_SLICES];
};

__global__ void pack_scales_kernel(const uint8_t* __restrict__ linear, uint8_t* __restrict__ packed, size_t bytes, PackArgs a) {
    for (size_t o = blockIdx.x * (size_t)blockDim.x + threadIdx.x; o < bytes; o += (size_t)gridDim.x * blockDim.x) {
        const int j = (int)(o & 3), r4 = (int)((o >> 2) & 3), r32 = (int)((o >> 4) & 31), m = (int)((o >> 9) & 3);
        const size_t slot = o >> 11;
        const int kb = (int)(slot % a.kslots);
        int tile = (int)(slot / a.kslots), s = 0, row0 = 0;
        while (s < a.S - 1 && tile >= (a.widths[s] + kTileN - 1) / kTileN) {
            tile -= (a.widths[s] + kTileN - 1) / kTileN;
            row0 += a.widths[s];
            ++s;
        }
        const int r = tile * kTileN + r4 * 32 + r32, col = kb * 16 + m * 4 + j;
        packed[o] = (r < a.widths[s] && col < a.K16) ? linear[(size_t)(row0 + r) * a.K16 + col] : (uint8_t)0;
    }
}

cudaError_t launch_pack_scales(const uint8_t* linear, int K, int S, const int32_t* widths, uint8_t* packed, size_t bytes,
                               cudaStream_t stream) {
    PackArgs a = {};
    a.K16 = K / 16;
    a.kslots = (K + 255) / 256;
    a.S = S;
    for (int s = 0; s < S; ++s) a.widths[s] = widths[s];
    const int threads = 256;
    size_t blocks = (bytes + threads - 1) / threads;
    if (blocks > 148 * 32) blocks = 148 * 32;
    pack_scales_kernel<<<(unsigned)blocks, threads, 0, stream>>>(linear, packed, bytes, a);
    return cudaGetLastError();
}

}  // namespace ob
