// Fused trellis-decode + matvec (batch 1..8) for B200.
//
// Work decomposition.  The packed matrix is cut into "units": a unit is one 32-row block of the
// output (a row of 2x2 blocks of 16x16 tiles, contiguous in memory) restricted to one contiguous
// range of columns.  A persistent grid (a multiple of the SM count) walks the units; inside a unit
// the warps of a CTA take 2x2 blocks round-robin, each lane pulls its 4K contiguous bytes with one
// streaming load, borrows the wrap-around bits from lane+1, decodes 16 states into four
// mma.m16n8k16 A fragments held in registers, and multiplies them with x placed in the B fragment
// (column j of B = batch row j, so up to 8 batch rows cost nothing extra).  Warps of a CTA are
// summed through shared memory; column ranges of one row block are summed, in a fixed order, by
// whichever CTA finishes that row block last (a ticket counter in the workspace), so the result is
// deterministic and `out` is overwritten, never accumulated into.
//
// Upstream counterpart: kernel_decompress_matvec, qtip-kernels/src/inference.cu:168-425.
#include "common.cuh"

namespace qtip {
namespace {

constexpr int kThreads = 512;             // 16 warps per CTA
constexpr int kWarps = kThreads / 32;
constexpr int kLutBytes = 512 * 32 * 4;   // 512 entries x 32 lane-private copies x half2
constexpr int kMaxBatch = 8;

struct MatvecPlan {
    int split;        // column ranges per row block
    int chunk;        // 2x2 blocks per column range (last range may be shorter)
    int units;
    int grid;
};

// Workspace: [row blocks] uint32 ticket counters (padded to 256 B), then partial sums
// [row block][split][8 batch][32 rows] fp32.
constexpr int kMaxSplit = 64;

inline size_t counters_bytes(int m) { return (((size_t)(m >> 5) * 4) + 255) & ~(size_t)255; }

MatvecPlan make_plan(int m, int n) {
    MatvecPlan p;
    const int mb = m >> 5, nb = n >> 5;
    const int ctas = sm_count();
    // aim for >= 4 units per CTA, at least one block per warp-iteration pair in a unit
    int split = 1;
    while (split < kMaxSplit && (long)mb * split < 4L * ctas && nb / (split * 2) >= kWarps) split *= 2;
    p.chunk = (nb + split - 1) / split;
    p.split = (nb + p.chunk - 1) / p.chunk;
    p.units = mb * p.split;
    p.grid = p.units < ctas ? p.units : ctas;
    return p;
}

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Cross-warp sum of the per-warp 32x8 accumulators, then either the final store or the
// partial-sum / ticket protocol.  red: [kWarps][256] floats in shared memory.
__device__ __forceinline__ void finish_unit(float (&acc)[2][4], float *red, float *__restrict__ out,
                                            float *__restrict__ partial, unsigned *__restrict__ counters, int M,
                                            int cidx, int split, int m, int bs) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    // accumulator element (ms, i): row = 16*ms + g + 8*(i>>1), batch = 2*t + (i&1); slot = batch*32 + row
#pragma unroll
    for (int ms = 0; ms < 2; ms++)
#pragma unroll
        for (int i = 0; i < 4; i++)
            red[warp * 256 + (2 * t + (i & 1)) * 32 + 16 * ms + g + 8 * (i >> 1)] = acc[ms][i];
    __syncthreads();
    __shared__ int s_last;
    float v = 0.f;
    if (threadIdx.x < 256) {
#pragma unroll
        for (int w = 0; w < kWarps; w++) v += red[w * 256 + threadIdx.x];
    }
    const int b = threadIdx.x >> 5, r = threadIdx.x & 31;
    if (split == 1) {
        if (threadIdx.x < 256 && b < bs) out[(size_t)b * m + 32 * M + r] = v;
        __syncthreads();
        return;
    }
    if (threadIdx.x < 256) partial[((size_t)M * split + cidx) * 256 + threadIdx.x] = v;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned prev = atomicAdd(&counters[M], 1u);
        s_last = (prev == (unsigned)(split - 1));
    }
    __syncthreads();
    if (s_last) {
        __threadfence();
        if (threadIdx.x < 256 && b < bs) {
            float s = 0.f;
            const float *p = partial + (size_t)M * split * 256 + threadIdx.x;
            for (int c = 0; c < split; c++) s += __ldcg(p + (size_t)c * 256);
            out[(size_t)b * m + 32 * M + r] = s;
        }
        if (threadIdx.x == 0) counters[M] = 0;  // leave the workspace ready for the next call
    }
    __syncthreads();
}

template <int K>
__global__ void __launch_bounds__(kThreads, 1)
    matvec_hyb_kernel(float *__restrict__ out, const uint8_t *__restrict__ codes, const __half *__restrict__ x,
                      const uint32_t *__restrict__ tlut, int m, int n, int bs, int split, int chunk, int units,
                      unsigned *__restrict__ counters, float *__restrict__ partial) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint32_t *lut = reinterpret_cast<uint32_t *>(smem);                 // [512][32]
    float *red = reinterpret_cast<float *>(smem + kLutBytes);           // [kWarps][256]

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // lane-private LUT copies: entry e of copy l at word e*32 + l  -> conflict-free gathers
    for (int i = threadIdx.x; i < 512 * 32; i += kThreads) lut[i] = tlut[i >> 5];
    __syncthreads();

    const int nb = n >> 5;
    const int g = lane >> 2, t = lane & 3;
    const __half *xrow = x + (size_t)(g < bs ? g : 0) * n + 2 * t;
    const bool xvalid = g < bs;
    const uint32_t *lut_lane = lut + lane;

    for (int u = blockIdx.x; u < units; u += gridDim.x) {
        const int M = u / split, cidx = u % split;
        const int n0 = cidx * chunk;
        const int n1 = min(nb, n0 + chunk);
        float acc[2][4] = {};
        const uint8_t *base = codes + ((size_t)M * nb) * (128 * K) + lane * (4 * K);

        for (int N = n0 + warp; N < n1; N += kWarps) {
            LaneCodes<K> own = load_lane_codes<K>(base + (size_t)N * (128 * K));
            uint32_t xb[4] = {0u, 0u, 0u, 0u};  // [ks][0: cols 2t,2t+1 | 1: cols 2t+8,2t+9]
            if (xvalid) {
                const uint32_t *xp = reinterpret_cast<const uint32_t *>(xrow + 32 * N);
                xb[0] = __ldg(xp); xb[1] = __ldg(xp + 4); xb[2] = __ldg(xp + 8); xb[3] = __ldg(xp + 12);
            }
            LaneCodes<K> nxt = shfl_next_lane<K>(own, lane);
#pragma unroll
            for (int tt = 0; tt < 4; tt++) {
                const int ks = tt >> 1, ms = tt & 1;
                uint32_t st[4], a[4];
                lane_states<K>(lane_slice<K>(own, tt), lane_slice<K>(nxt, tt), st);
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    uint32_t h = hyb_hash(st[q]);
                    a[q] = lut_lane[(h >> 1) & (511u << 5)] ^ (h & 0x8000u);
                }
                mma_16816(acc[ms], a, xb[2 * ks], xb[2 * ks + 1]);
            }
        }
        finish_unit(acc, red, out, partial, counters, M, cidx, split, m, bs);
    }
}

// ---- 3INST / 1MAD, plain layout, V = 1 ---------------------------------------------------------
// One warp per 16x16 tile pair stacked along m (32 rows x 16 cols).  Within a tile lane (g, t)
// decodes elements (row g, cols 4t..4t+3) and (row g+8, cols 4t..4t+3): two runs of four
// consecutive states, each cut from <= 28+... consecutive stream bits.  The A fragment wants
// columns {2t, 2t+1, 2t+8, 2t+9}; instead of moving weights between lanes the k index of the MMA is
// permuted: fragment column j of this lane pair is matrix column perm(j), and x is loaded with the
// same permutation, which leaves every dot product unchanged.
template <int CODE>
__device__ __forceinline__ uint32_t decode_pair(uint32_t s0, uint32_t s1) {
    __half lo, hi;
    if constexpr (CODE == QTIP_CODE_3INST) { lo = decode_3inst(s0 & 0xFFFFu); hi = decode_3inst(s1 & 0xFFFFu); }
    else { lo = decode_1mad(s0 & 0xFFFFu); hi = decode_1mad(s1 & 0xFFFFu); }
    __half2 p = __halves2half2(lo, hi);
    return *reinterpret_cast<uint32_t *>(&p);
}

// 32 + 16 stream bits of a tile starting at bit pos (circular), first bit at bit 47
__device__ __forceinline__ uint64_t tile_bits48(const uint16_t *__restrict__ words, int nwords, int pos) {
    int w = pos >> 4;
    uint64_t v = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int wi = w + i;
        if (wi >= nwords) wi -= nwords;
        v = (v << 16) | __ldg(words + wi);
    }
    return (v << (pos & 15)) >> 16;
}

template <int CODE>
__global__ void __launch_bounds__(kThreads, 1)
    matvec_plain_kernel(float *__restrict__ out, const uint16_t *__restrict__ codes, const __half *__restrict__ x, int K,
                        int m, int n, int bs, int split, int chunk, int units, unsigned *__restrict__ counters,
                        float *__restrict__ partial) {
    extern __shared__ __align__(128) uint8_t smem[];
    float *red = reinterpret_cast<float *>(smem);  // [kWarps][256]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tn = n >> 4;       // tiles per tile row
    const int nwords = 16 * K;
    const int g = lane >> 2, t = lane & 3;
    const bool xvalid = g < bs;
    const __half *xrow = x + (size_t)(xvalid ? g : 0) * n;

    // chunk / split are expressed in 32-column blocks like the HYB kernel; here a block is two k-tiles
    const int nb = n >> 5;
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
        const int M = u / split, cidx = u % split;
        const int n0 = cidx * chunk, n1 = min(nb, n0 + chunk);
        float acc[2][4] = {};
        for (int kt = 2 * n0 + warp; kt < 2 * n1; kt += kWarps) {
            // B fragment with the permuted k order: fragment k = 2t+{0,1} -> matrix cols 4t+{0,1};
            // fragment k = 2t+8+{0,1} -> matrix cols 4t+{2,3}
            uint32_t b0 = 0u, b1 = 0u;
            if (xvalid) {
                const uint32_t *xp = reinterpret_cast<const uint32_t *>(xrow + 16 * kt + 4 * t);
                b0 = __ldg(xp); b1 = __ldg(xp + 1);
            }
#pragma unroll
            for (int ms = 0; ms < 2; ms++) {
                const uint16_t *words = codes + ((size_t)(2 * M + ms) * tn + kt) * nwords;
                uint32_t a[4];
#pragma unroll
                for (int hr = 0; hr < 2; hr++) {  // rows g, g+8
                    const int e0 = (g + 8 * hr) * 16 + 4 * t;
                    uint64_t bits = tile_bits48(words, nwords, e0 * K);
                    uint32_t s0 = (uint32_t)(bits >> 32), s1 = (uint32_t)(bits >> (32 - K));
                    uint32_t s2 = (uint32_t)(bits >> (32 - 2 * K)), s3 = (uint32_t)(bits >> (32 - 3 * K));
                    a[hr] = decode_pair<CODE>(s0, s1);       // a0 / a1: fragment cols 2t, 2t+1
                    a[2 + hr] = decode_pair<CODE>(s2, s3);   // a2 / a3: fragment cols 2t+8, 2t+9
                }
                mma_16816(acc[ms], a, b0, b1);
            }
        }
        finish_unit(acc, red, out, partial, counters, M, cidx, split, m, bs);
    }
}

int check_common(const void *out, const void *codes, const void *x, int K, int m, int n, int bs, void *workspace,
                 size_t workspace_bytes) {
    if (!out || !codes || !x || K < 2 || K > 4 || bs < 1 || bs > kMaxBatch) return QTIP_ERR_BAD_ARG;
    if (m <= 0 || n <= 0 || (m & 31) || (n & 31)) return QTIP_ERR_BAD_SHAPE;
    if (!workspace || workspace_bytes < qtip_matvec_workspace_bytes(m, n, bs)) return QTIP_ERR_WORKSPACE;
    if (!aligned(workspace, 256) || !aligned(codes, 16) || !aligned(x, 4) || !aligned(out, 4)) return QTIP_ERR_ALIGNMENT;
    return QTIP_OK;
}

}  // namespace
}  // namespace qtip

using namespace qtip;

extern "C" size_t qtip_matvec_workspace_bytes(int m, int n, int bs) {
    (void)n; (void)bs;
    if (m <= 0) return 256;
    return counters_bytes(m) + (size_t)(m >> 5) * kMaxSplit * 256 * sizeof(float);
}

template <int K>
static int launch_hyb(float *out, const uint8_t *codes, const __half *x, const uint32_t *tlut, int m, int n, int bs,
                      const MatvecPlan &p, unsigned *counters, float *partial, cudaStream_t s) {
    static bool attr_set[64] = {};
    int dev = 0;
    QTIP_CUDA_TRY(cudaGetDevice(&dev));
    constexpr int smem = kLutBytes + kWarps * 256 * (int)sizeof(float);
    if (dev < 64 && !attr_set[dev]) {
        QTIP_CUDA_TRY(cudaFuncSetAttribute(matvec_hyb_kernel<K>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        attr_set[dev] = true;
    }
    matvec_hyb_kernel<K><<<p.grid, kThreads, smem, s>>>(out, codes, x, tlut, m, n, bs, p.split, p.chunk, p.units,
                                                        counters, partial);
    return check_launch();
}

extern "C" int qtip_decompress_matvec(float *out, const void *codes, const void *x, const void *tlut, int K, int m,
                                      int n, int bs, void *workspace, size_t workspace_bytes, void *stream) {
    if (!tlut) return QTIP_ERR_BAD_ARG;
    int st = check_common(out, codes, x, K, m, n, bs, workspace, workspace_bytes);
    if (st != QTIP_OK) return st;
    if (!aligned(tlut, 4)) return QTIP_ERR_ALIGNMENT;
    MatvecPlan p = make_plan(m, n);
    auto *counters = static_cast<unsigned *>(workspace);
    auto *partial = reinterpret_cast<float *>(static_cast<uint8_t *>(workspace) + counters_bytes(m));
    auto *c = static_cast<const uint8_t *>(codes);
    auto *xh = static_cast<const __half *>(x);
    auto *t = static_cast<const uint32_t *>(tlut);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (K == 2) return launch_hyb<2>(out, c, xh, t, m, n, bs, p, counters, partial, s);
    if (K == 3) return launch_hyb<3>(out, c, xh, t, m, n, bs, p, counters, partial, s);
    return launch_hyb<4>(out, c, xh, t, m, n, bs, p, counters, partial, s);
}

extern "C" int qtip_decompress_matvec_plain(float *out, const void *codes, const void *x, int code, int K, int m, int n,
                                            int bs, void *workspace, size_t workspace_bytes, void *stream) {
    if (code != QTIP_CODE_3INST && code != QTIP_CODE_1MAD) return QTIP_ERR_BAD_ARG;
    int st = check_common(out, codes, x, K, m, n, bs, workspace, workspace_bytes);
    if (st != QTIP_OK) return st;
    MatvecPlan p = make_plan(m, n);
    auto *counters = static_cast<unsigned *>(workspace);
    auto *partial = reinterpret_cast<float *>(static_cast<uint8_t *>(workspace) + counters_bytes(m));
    auto *c = static_cast<const uint16_t *>(codes);
    auto *xh = static_cast<const __half *>(x);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    constexpr int smem = kWarps * 256 * (int)sizeof(float);
    if (code == QTIP_CODE_3INST)
        matvec_plain_kernel<QTIP_CODE_3INST><<<p.grid, kThreads, smem, s>>>(out, c, xh, K, m, n, bs, p.split, p.chunk,
                                                                           p.units, counters, partial);
    else
        matvec_plain_kernel<QTIP_CODE_1MAD><<<p.grid, kThreads, smem, s>>>(out, c, xh, K, m, n, bs, p.split, p.chunk,
                                                                          p.units, counters, partial);
    return check_launch();
}
