// Trellis decoders: packed codes -> dense fp16 (m, n).
//
// decode_hyb_kernel   HYB (L=16, V=2, Q=9) kernel layout; one warp per 2x2 block of 16x16 tiles,
//                     a lane reads its 4K contiguous bytes, gets the wrap-around bits from lane+1,
//                     and looks its 16 states up in a 512-entry LUT held in shared memory.
//                     Same mapping as decode_compressed upstream (lib/utils/kernel_decompress.py:4-55).
// decode_plain_kernel any code, plain layout (lib/codebook/bitshift.py:329-353, 378-381): one warp
//                     per tile, each lane decodes 8 consecutive sequence elements of one tile row half.
#include "common.cuh"

namespace qtip {
namespace {

constexpr int kDecodeThreads = 256;

// Row stride of a warp's staging tile in 32-bit words: 16 data words + 4 of padding, so that the scattered 4-byte
// stores of the eight fragment rows fall into distinct banks while rows stay 16-byte aligned for the read-back.
constexpr int kStageStride = 20;

template <int K>
__global__ void __launch_bounds__(kDecodeThreads) decode_hyb_kernel(__half *__restrict__ W,
                                                                   const uint8_t *__restrict__ codes,
                                                                   const uint32_t *__restrict__ tlut, int m, int n) {
    __shared__ uint32_t lut[512];
    __shared__ __align__(16) uint32_t stage_all[kDecodeThreads / 32][32 * kStageStride];
    for (int i = threadIdx.x; i < 512; i += blockDim.x) lut[i] = tlut[i];
    __syncthreads();

    const int lane = threadIdx.x & 31;
    uint32_t *stage = stage_all[threadIdx.x >> 5];
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int nb = n >> 5;
    const long blocks = (long)(m >> 5) * nb;
    const int a = lane >> 2, b = lane & 3;
    for (long blk = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; blk < blocks; blk += warps) {
        const int M = (int)(blk / nb), N = (int)(blk % nb);
        LaneCodes<K> own = load_lane_codes<K>(codes + blk * (128 * K) + lane * (4 * K));
        LaneCodes<K> nxt = shfl_next_lane<K>(own, lane);
        // decode into the warp's 32 x 32 staging tile (fragment order -> row-major) ...
#pragma unroll
        for (int t = 0; t < 4; t++) {
            const int ks = t >> 1, ms = t & 1;
            uint32_t st[4];
            lane_states<K>(lane_slice<K>(own, t), lane_slice<K>(nxt, t), st);
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const int c = q >> 1, d = q & 1;
                uint32_t h = hyb_hash(st[q]);
                uint32_t w = lut[(h >> 6) & 511u] ^ (h & 0x8000u);
                stage[(16 * ms + 8 * d + a) * kStageStride + 8 * ks + 4 * c + b] = w;     // cols 16ks + 8c + 2b, +1
            }
        }
        __syncwarp();
        // ... and write it out as 64-byte row segments: one 16-byte store per lane covers 8 rows x 64 bytes
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int r = 8 * i + a;
            const uint4 v = *reinterpret_cast<const uint4 *>(stage + r * kStageStride + 4 * b);
            *reinterpret_cast<uint4 *>(W + ((size_t)32 * M + r) * n + (size_t)32 * N + 8 * b) = v;
        }
        __syncwarp();
    }
}

// 48 stream bits of a tile starting at bit `pos` (circular over nbits = 256*K), first bit at bit 47.
__device__ __forceinline__ uint64_t tile_bits48(const uint16_t *__restrict__ words, int nwords, int pos) {
    int w = pos >> 4;
    uint64_t v = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int wi = w + i;
        if (wi >= nwords) wi -= nwords;
        v = (v << 16) | words[wi];
    }
    return (v << (pos & 15)) >> 16;  // drop the bits before pos, keep 48
}

template <int CODE>
__global__ void __launch_bounds__(kDecodeThreads) decode_plain_kernel(__half *__restrict__ W,
                                                                     const uint16_t *__restrict__ codes,
                                                                     const uint32_t *__restrict__ tlut, int K, int m,
                                                                     int n) {
    __shared__ uint32_t lut[CODE == QTIP_CODE_HYB ? 512 : 1];
    if constexpr (CODE == QTIP_CODE_HYB) {
        for (int i = threadIdx.x; i < 512; i += blockDim.x) lut[i] = tlut[i];
        __syncthreads();
    }
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int tn = n >> 4;
    const long tiles = (long)(m >> 4) * tn;
    const int nwords = 16 * K;
    const int r = lane >> 1, hf = lane & 1;  // tile row, half of the row (8 elements)
    for (long tile = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; tile < tiles; tile += warps) {
        const uint16_t *words = codes + tile * nwords;
        const int e0 = r * 16 + hf * 8;  // first sequence element of this lane
        __half out[8];
        if constexpr (CODE == QTIP_CODE_HYB) {
            // V = 2: state i covers elements 2i, 2i+1; window starts at bit i*2K
#pragma unroll
            for (int j = 0; j < 4; j++) {
                int i = (e0 >> 1) + j;
                uint32_t s = (uint32_t)(tile_bits48(words, nwords, i * 2 * K) >> 32) & 0xFFFFu;
                uint32_t h = hyb_hash(s);
                uint32_t w = lut[(h >> 6) & 511u] ^ (h & 0x8000u);
                *reinterpret_cast<uint32_t *>(&out[2 * j]) = w;
            }
        } else {
            // V = 1: 8 states from 7K+16 <= 44 consecutive bits
            uint64_t bits = tile_bits48(words, nwords, e0 * K);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                uint32_t s = (uint32_t)(bits >> (32 - j * K)) & 0xFFFFu;
                out[j] = (CODE == QTIP_CODE_3INST) ? decode_3inst(s) : decode_1mad(s);
            }
        }
        size_t row = (size_t)(tile / tn) * 16 + r, col = (size_t)(tile % tn) * 16 + hf * 8;
        *reinterpret_cast<uint4 *>(W + row * n + col) = *reinterpret_cast<uint4 *>(out);
    }
}

int decode_grid(long warps_needed) {
    long ctas = (warps_needed + (kDecodeThreads / 32) - 1) / (kDecodeThreads / 32);
    long cap = (long)sm_count() * 8;
    return (int)(ctas < cap ? (ctas < 1 ? 1 : ctas) : cap);
}

}  // namespace
}  // namespace qtip

using namespace qtip;

extern "C" int qtip_decode_hyb(void *W, const void *codes, const void *tlut, int K, int m, int n, void *stream) {
    if (!W || !codes || !tlut || K < 2 || K > 4) return QTIP_ERR_BAD_ARG;
    if (m <= 0 || n <= 0 || (m & 31) || (n & 31)) return QTIP_ERR_BAD_SHAPE;
    if (!aligned(codes, 16) || !aligned(W, 16) || !aligned(tlut, 4)) return QTIP_ERR_ALIGNMENT;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int grid = decode_grid((long)(m >> 5) * (n >> 5));
    auto *Wh = static_cast<__half *>(W);
    auto *c = static_cast<const uint8_t *>(codes);
    auto *t = static_cast<const uint32_t *>(tlut);
    if (K == 2) decode_hyb_kernel<2><<<grid, kDecodeThreads, 0, s>>>(Wh, c, t, m, n);
    else if (K == 3) decode_hyb_kernel<3><<<grid, kDecodeThreads, 0, s>>>(Wh, c, t, m, n);
    else decode_hyb_kernel<4><<<grid, kDecodeThreads, 0, s>>>(Wh, c, t, m, n);
    return check_launch();
}

extern "C" int qtip_decode_plain(void *W, const void *codes, int code, const void *tlut, int K, int m, int n,
                                 void *stream) {
    if (!W || !codes || K < 2 || K > 4) return QTIP_ERR_BAD_ARG;
    if (code == QTIP_CODE_HYB && !tlut) return QTIP_ERR_BAD_ARG;
    if (m <= 0 || n <= 0 || (m & 15) || (n & 15)) return QTIP_ERR_BAD_SHAPE;
    if (!aligned(codes, 2) || !aligned(W, 16)) return QTIP_ERR_ALIGNMENT;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int grid = decode_grid((long)(m >> 4) * (n >> 4));
    auto *Wh = static_cast<__half *>(W);
    auto *c = static_cast<const uint16_t *>(codes);
    auto *t = static_cast<const uint32_t *>(tlut);
    switch (code) {
        case QTIP_CODE_HYB: decode_plain_kernel<QTIP_CODE_HYB><<<grid, kDecodeThreads, 0, s>>>(Wh, c, t, K, m, n); break;
        case QTIP_CODE_3INST: decode_plain_kernel<QTIP_CODE_3INST><<<grid, kDecodeThreads, 0, s>>>(Wh, c, t, K, m, n); break;
        case QTIP_CODE_1MAD: decode_plain_kernel<QTIP_CODE_1MAD><<<grid, kDecodeThreads, 0, s>>>(Wh, c, t, K, m, n); break;
        default: return QTIP_ERR_BAD_ARG;
    }
    return check_launch();
}
