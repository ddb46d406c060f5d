// Producers of the packed formats the decode path consumes (the quantizer side of the format):
//   * pack_trellis: trellis states -> tail-biting bitstream words, plain layout
//     (bitshift_codebook.pack_trellis upstream, lib/codebook/bitshift.py:294-327, including its overlap check);
//   * the byte shuffle between the plain layout and the kernel layout
//     (lib/algo/finetune.py:196-201 upstream, inverse at lib/utils/kernel_decompress.py:19-24).
// All three are pure bit / byte movement: results are bit-exact by construction, the kernels are bound by HBM
// (one read and one write of the packed bytes; pack_trellis reads 4 bytes per state and writes K*V/8).
#include "common.cuh"

namespace qtip {
namespace {

// One thread per output word.  Stream bit p of a tile (p < 256*K) is bit 15 - (p - i*KV) of state i, for the state
// whose window covers p; upstream takes state 0 for the first 16 bits and afterwards the state that ENDS last at or
// after p, i = (p - 16) / KV + 1 (the states agree on their overlap, which `violations` counts when it is not so).
__global__ void pack_trellis_kernel(uint16_t *__restrict__ words, const int *__restrict__ states, long tiles, int T, int KV,
                                    int words_per_tile, unsigned *__restrict__ violations) {
    const long total = tiles * words_per_tile;
    for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
        const long tile = idx / words_per_tile;
        const int w = (int)(idx - tile * words_per_tile);
        const int *st = states + tile * T;
        uint32_t out = 0;
#pragma unroll
        for (int b = 0; b < 16; b++) {
            const int p = 16 * w + b;
            int i, bit;
            if (p < 16) { i = 0; bit = 15 - p; }
            else { i = (p - 16) / KV + 1; bit = KV - 1 - (p - 16) % KV; }
            out = (out << 1) | ((uint32_t)(st[i] >> bit) & 1u);
        }
        words[idx] = (uint16_t)out;
    }
    if (violations) {
        // the overlap check of pack_trellis upstream: low L-KV bits of state i-1 == state i >> KV
        const long pairs = tiles * (T - 1);
        const int mask = (1 << (16 - KV)) - 1;
        for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < pairs; idx += (long)gridDim.x * blockDim.x) {
            const long tile = idx / (T - 1);
            const int i = (int)(idx - tile * (T - 1)) + 1;
            const int *st = states + tile * T;
            if ((st[i - 1] & mask) != ((st[i] & 0xFFFF) >> KV)) atomicAdd(violations, 1u);
        }
    }
}

// Kernel layout bytes  [M][N][lane 32][ks 2][ms 2][K]  <->  plain layout words [tile row 2M+ms][tile col 2N+ks][16K],
// where lane l's K bytes are bytes l*K .. l*K+K-1 of the tile's big-endian byte stream, stored reversed.
// One thread per byte of the kernel layout.
template <bool TO_KERNEL>
__global__ void layout_kernel(uint8_t *__restrict__ dst, const uint8_t *__restrict__ src, int K, int mb, int nb) {
    const long total = (long)mb * nb * 128 * K;
    for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
        long r = idx;
        const int kb = (int)(r % K); r /= K;
        const int ms = (int)(r & 1); r >>= 1;
        const int ks = (int)(r & 1); r >>= 1;
        const int lane = (int)(r & 31); r >>= 5;
        const int N = (int)(r % nb);
        const int M = (int)(r / nb);
        // byte position in the tile's big-endian stream, then in the little-endian uint16 words of the plain layout
        const int sb = lane * K + (K - 1 - kb);
        const long tile = (long)(2 * M + ms) * (2 * nb) + (2 * N + ks);
        const long plain = tile * (32 * K) + (sb ^ 1);      // big-endian byte sb of word sb/2 is byte (sb ^ 1) in memory
        if (TO_KERNEL) dst[idx] = src[plain];
        else dst[plain] = src[idx];
    }
}

int grid_for(long items, int threads) {
    long g = (items + threads - 1) / threads;
    const long cap = (long)sm_count() * 16;
    return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace
}  // namespace qtip

using namespace qtip;

extern "C" int qtip_pack_trellis(void *words, const int *states, long tiles, int K, int V, unsigned *violations, void *stream) {
    if (!words || !states || tiles <= 0 || K < 1 || K > 8 || (V != 1 && V != 2) || K * V > 16 || (256 * K) % 16) return QTIP_ERR_BAD_ARG;
    if (!aligned(words, 2) || !aligned(states, 4) || (violations && !aligned(violations, 4))) return QTIP_ERR_ALIGNMENT;
    const int T = 256 / V, wpt = 16 * K;
    const long items = tiles * (long)(wpt > T ? wpt : T);
    pack_trellis_kernel<<<grid_for(items, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint16_t *>(words), states, tiles, T, K * V, wpt, violations);
    return check_launch();
}

extern "C" int qtip_plain_to_kernel_layout(void *kernel_codes, const void *plain_words, int K, int m, int n, void *stream) {
    if (!kernel_codes || !plain_words || kernel_codes == plain_words || K < 2 || K > 4) return QTIP_ERR_BAD_ARG;
    if (m <= 0 || n <= 0 || (m & 31) || (n & 31)) return QTIP_ERR_BAD_SHAPE;
    const long items = (long)(m >> 5) * (n >> 5) * 128 * K;
    layout_kernel<true><<<grid_for(items, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint8_t *>(kernel_codes), static_cast<const uint8_t *>(plain_words), K, m >> 5, n >> 5);
    return check_launch();
}

extern "C" int qtip_kernel_to_plain_layout(void *plain_words, const void *kernel_codes, int K, int m, int n, void *stream) {
    if (!kernel_codes || !plain_words || kernel_codes == plain_words || K < 2 || K > 4) return QTIP_ERR_BAD_ARG;
    if (m <= 0 || n <= 0 || (m & 31) || (n & 31)) return QTIP_ERR_BAD_SHAPE;
    const long items = (long)(m >> 5) * (n >> 5) * 128 * K;
    layout_kernel<false><<<grid_for(items, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint8_t *>(plain_words), static_cast<const uint8_t *>(kernel_codes), K, m >> 5, n >> 5);
    return check_launch();
}
