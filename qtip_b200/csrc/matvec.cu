// Fused trellis-decode + matvec (batch 1..8) for B200.
//
// Partition ("stream-K").  The packed matrix is a sequence of B = (m/32)*(n/32) blocks (a block is
// a 2x2 group of 16x16 tiles, 128*K contiguous bytes; blocks of one 32-row block are contiguous).
// The grid has one CTA per SM and CTA c owns the contiguous block range [c*B/G, (c+1)*B/G), so
// every SM streams the same number of bytes (+-1 block) from one contiguous address range.  A
// range is cut into "segments" at 32-row-block boundaries.
//
// Data path.  A producer warp streams the CTA's byte range through a ring of shared-memory
// stages with cp.async.bulk (TMA, completion on an mbarrier per stage), running ahead of the
// consumers across segment boundaries.  Sixteen consumer warps take the blocks of a stage
// round-robin: a lane reads its 4K contiguous bytes and those of lane+1 (wrap-around bits) from
// the stage, decodes 16 trellis states into four mma.m16n8k16 A fragments in registers - HYB:
// h = s*(s+1), entry (h>>6)&511 of a LUT kept as 32 lane-private copies in shared memory, sign
// flip from bit 15 - and multiplies them with x held in the B fragment (column j of B = batch row
// j, so up to 8 batch rows ride along for free).  fp32 accumulation in the MMA.
//
// Reduction.  Warps of a CTA are summed through shared memory at the end of a segment.  When a
// row block is shared by several CTAs each stores its partial sums to the workspace and takes a
// ticket; the CTA that draws the last ticket adds the partials in CTA order and writes the result,
// so the output is deterministic and is overwritten, never accumulated into.
//
// Every wait on an mbarrier is bounded: after kSpinLimit polls the thread records an error code in
// the workspace status word, raises a CTA-wide abort flag that makes all later waits fall through,
// and the kernel runs to its end (with meaningless results) instead of hanging.
//
// Upstream counterpart: kernel_decompress_matvec, qtip-kernels/src/inference.cu:168-425.
#include "common.cuh"

namespace qtip {
namespace {

constexpr int kConsumerWarps = 16;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;  // + producer warp
constexpr int kStageBlocks = 32;                 // blocks per ring stage (two per consumer warp)
constexpr int kLutBytes = 512 * 32 * 4;          // 512 entries x 32 lane-private copies x half2 = 64 KiB
constexpr int kRedBytes = kConsumerWarps * 256 * 4;
constexpr int kMaxStages = 8;
constexpr int kMaxBatch = 8;
constexpr unsigned kSpinLimit = 1u << 22;        // polls of ~20-40 ns each: gives up after ~0.1 s

// ---- workspace layout (all offsets fixed, independent of the problem) -----------------------------
// [0, 64 KiB)   ticket counters, one uint32 per 32-row block (m <= 524288); zero between calls
// [64 KiB, +256) status word (0 = ok) and padding
// [.., end)     partial sums: [row block][contributor][8 batch x 32 rows] fp32
constexpr size_t kCounterBytes = 64 * 1024;
constexpr size_t kStatusOffset = kCounterBytes;
constexpr size_t kPartialOffset = kCounterBytes + 256;
constexpr int kMaxGrid = 256;  // sizing bound for the number of CTAs

// A row block (nb consecutive blocks) meets at most floor(nb / minlen) CTAs that lie entirely inside
// it plus two partial ones, where minlen = floor(B / G) is the shortest CTA range.
inline int max_contributors(long nb, long B, long G) {
    const long minlen = B / G > 0 ? B / G : 1;
    return (int)(nb / minlen) + 2;
}

struct Partition {
    int grid;       // CTAs
    int kmax;       // contributor slots per row block
    long blocks;    // B
};

Partition make_partition(int m, int n) {
    Partition p;
    p.blocks = (long)(m >> 5) * (n >> 5);
    const long sms = sm_count();
    p.grid = (int)(p.blocks < sms ? p.blocks : sms);
    p.kmax = max_contributors(n >> 5, p.blocks, p.grid);
    return p;
}

// ---- PTX wrappers -----------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  `abort_flag` lives in shared memory; once set every wait returns immediately.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                          unsigned *status, int code) {
    if (mbar_try_wait(bar, parity)) return;
    for (unsigned spin = 0; spin < kSpinLimit; spin++) {
        if (mbar_try_wait(bar, parity)) return;
        if (*abort_flag) return;
    }
    *abort_flag = 1;
    atomicCAS(status, 0u, (unsigned)code);
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory"); }

__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// ---- partition arithmetic (identical on host and device) ------------------------------------------------
__host__ __device__ __forceinline__ long range_start(long c, long B, long G) { return c * B / G; }
__host__ __device__ __forceinline__ long cta_of_block(long b, long B, long G) { return ((b + 1) * G - 1) / B; }

struct Shared {            // small control block at the start of dynamic shared memory
    unsigned long long full[kMaxStages];
    unsigned long long empty[kMaxStages];
    uint32_t stage_addr[kMaxStages];
    int abort_flag;
    int is_last;
};

// Cross-warp sum of the per-warp 32x8 accumulators of one segment, then the final store or the
// partial-sum / ticket protocol.  Consumer threads only.
__device__ __forceinline__ void finish_segment(float (&acc)[2][4], float *red, Shared *sh, float *__restrict__ out,
                                               float *__restrict__ partial, unsigned *__restrict__ counters, long M,
                                               long nb, long B, long G, int kmax, int m, int bs) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    // accumulator (ms, i): row = 16*ms + g + 8*(i>>1), batch = 2*t + (i&1); slot = batch*32 + row
#pragma unroll
    for (int ms = 0; ms < 2; ms++)
#pragma unroll
        for (int i = 0; i < 4; i++)
            red[warp * 256 + (2 * t + (i & 1)) * 32 + 16 * ms + g + 8 * (i >> 1)] = acc[ms][i];
    consumer_sync();
    float v = 0.f;
    if (tid < 256) {
#pragma unroll
        for (int w = 0; w < kConsumerWarps; w++) v += red[w * 256 + tid];
    }
    const int b = tid >> 5, r = tid & 31;
    const long c_first = cta_of_block(M * nb, B, G), c_last = cta_of_block((M + 1) * nb - 1, B, G);
    const int contributors = (int)(c_last - c_first) + 1;
    if (contributors == 1) {
        if (tid < 256 && b < bs) out[(size_t)b * m + 32 * M + r] = v;
        consumer_sync();
        return;
    }
    const int k = (int)(blockIdx.x - c_first);
    float *slot = partial + ((size_t)M * kmax) * 256;
    if (tid < 256) __stcg(slot + (size_t)k * 256 + tid, v);
    __threadfence();
    consumer_sync();
    if (tid == 0) {
        unsigned prev = atomicAdd(&counters[M], 1u);
        sh->is_last = (prev == (unsigned)(contributors - 1));
    }
    consumer_sync();
    if (sh->is_last) {
        __threadfence();
        if (tid < 256 && b < bs) {
            float s = 0.f;
            for (int c = 0; c < contributors; c++) s += __ldcg(slot + (size_t)c * 256 + tid);
            out[(size_t)b * m + 32 * M + r] = s;
        }
        if (tid == 0) counters[M] = 0;  // leave the workspace ready for the next call
    }
    consumer_sync();
}

template <int K>
__global__ void __launch_bounds__(kThreads, 1)
    matvec_hyb_kernel(float *__restrict__ out, const uint8_t *__restrict__ codes, const __half *__restrict__ x,
                      const uint32_t *__restrict__ tlut, int m, int n, int bs, int kmax, int nstages,
                      uint8_t *__restrict__ workspace, uint32_t smem_total) {
    constexpr int kBlockBytes = 128 * K;
    constexpr int kStageBytes = kStageBlocks * kBlockBytes;
    extern __shared__ __align__(128) uint8_t smem[];

    unsigned *counters = reinterpret_cast<unsigned *>(workspace);
    unsigned *status = reinterpret_cast<unsigned *>(workspace + kStatusOffset);
    float *partial = reinterpret_cast<float *>(workspace + kPartialOffset);

    // ---- carve shared memory.  The LUT must sit on a 64 KiB boundary of the shared window so that a
    // gather address is (hash bits) | (lane*4): one logic op, no add.  Whatever lies below and above
    // it holds the control block, the cross-warp reduction buffer and the ring stages.
    const uint32_t base = smem_u32(smem);
    const uint32_t lut_addr = (base + 0xFFFFu) & ~0xFFFFu;
    Shared *sh = reinterpret_cast<Shared *>(smem);  // control block first if it fits below the LUT, else above
    uint32_t lo = base, lo_end = lut_addr, hi = lut_addr + kLutBytes, hi_end = base + smem_total;
    auto carve = [&](uint32_t bytes) -> uint32_t {
        bytes = (bytes + 127u) & ~127u;
        if (lo + bytes <= lo_end) { uint32_t a = lo; lo += bytes; return a; }
        uint32_t a = hi; hi += bytes; return a;  // host sized smem_total so that this fits
    };
    const uint32_t sh_addr = carve(sizeof(Shared));
    const uint32_t red_addr = carve(kRedBytes);
    sh = reinterpret_cast<Shared *>(smem + (sh_addr - base));
    float *red = reinterpret_cast<float *>(smem + (red_addr - base));
    if (threadIdx.x == 0) {
        for (int s = 0; s < nstages; s++) {
            sh->stage_addr[s] = carve(kStageBytes);
            mbar_init(smem_u32(&sh->full[s]), 1);
            mbar_init(smem_u32(&sh->empty[s]), kConsumerWarps);
        }
        sh->abort_flag = 0;
        sh->is_last = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (hi > hi_end) atomicCAS(status, 0u, 3u);  // cannot happen when the host sizes smem_total
    }
    __syncthreads();

    const long nb = n >> 5;
    const long B = (long)(m >> 5) * nb, G = gridDim.x;
    const long r0 = range_start(blockIdx.x, B, G), r1 = range_start(blockIdx.x + 1, B, G);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int *abort_flag = &sh->abort_flag;

    if (warp == kConsumerWarps) {
        // ------------------------------- producer warp ---------------------------------------------
        if (lane == 0) {
            uint32_t it = 0;
            for (long seg0 = r0; seg0 < r1;) {
                const long seg1 = min(r1, (seg0 / nb + 1) * nb);
                for (long b = seg0; b < seg1 && !*abort_flag; b += kStageBlocks, it++) {
                    const uint32_t cnt = (uint32_t)min((long)kStageBlocks, seg1 - b);
                    const uint32_t s = it % nstages, round = it / nstages;
                    if (round > 0) mbar_wait(smem_u32(&sh->empty[s]), (round - 1) & 1, abort_flag, status, 1);
                    const uint32_t bar = smem_u32(&sh->full[s]);
                    mbar_expect_tx(bar, cnt * kBlockBytes);
                    bulk_g2s(sh->stage_addr[s], codes + (size_t)b * kBlockBytes, cnt * kBlockBytes, bar);
                }
                seg0 = seg1;
            }
        }
        return;  // every copy issued above is consumed (waited for) by the consumer warps below
    }

    // ------------------------------------ consumer warps ------------------------------------------------
    // lane-private LUT copies: entry e, copy l at byte e*128 + l*4 -> conflict-free gathers
    {
        uint32_t *lut = reinterpret_cast<uint32_t *>(smem + (lut_addr - base));
        for (int i = threadIdx.x; i < 512 * 8; i += kConsumerThreads) {
            const uint32_t e = tlut[i >> 3];
            reinterpret_cast<uint4 *>(lut)[i] = make_uint4(e, e, e, e);
        }
    }
    consumer_sync();

    const int g = lane >> 2, t = lane & 3;
    const bool xvalid = g < bs;
    const __half *xrow = x + (size_t)(xvalid ? g : 0) * n + 2 * t;
    const uint32_t lut_lane = lut_addr + lane * 4;
    const uint32_t own_off = lane * (4 * K), nxt_off = ((lane + 1) & 31) * (4 * K);

    uint32_t it = 0;
    for (long seg0 = r0; seg0 < r1;) {
        const long M = seg0 / nb;
        const long seg1 = min(r1, (M + 1) * nb);
        float acc[2][4] = {};
        for (long b = seg0; b < seg1; b += kStageBlocks, it++) {
            const int cnt = (int)min((long)kStageBlocks, seg1 - b);
            const uint32_t s = it % nstages, round = it / nstages;
            mbar_wait(smem_u32(&sh->full[s]), round & 1, abort_flag, status, 2);
            const uint32_t stage = sh->stage_addr[s];
#pragma unroll 2
            for (int j = warp; j < cnt; j += kConsumerWarps) {
                const int N = (int)(b + j - M * nb);
                uint32_t xb[4] = {0u, 0u, 0u, 0u};  // [ks][cols 2t,2t+1 | cols 2t+8,2t+9]
                if (xvalid) {
                    const uint32_t *xp = reinterpret_cast<const uint32_t *>(xrow + 32 * N);
                    xb[0] = __ldg(xp); xb[1] = __ldg(xp + 4); xb[2] = __ldg(xp + 8); xb[3] = __ldg(xp + 12);
                }
                LaneCodes<K> own, nxt;
                const uint32_t blk = stage + j * kBlockBytes;
#pragma unroll
                for (int i = 0; i < K; i++) {
                    own.w[i] = lds_u32(blk + own_off + 4 * i);
                    nxt.w[i] = lds_u32(blk + nxt_off + 4 * i);
                }
#pragma unroll
                for (int tt = 0; tt < 4; tt++) {
                    const int ks = tt >> 1, ms = tt & 1;
                    uint32_t st[4], a[4];
                    lane_states<K>(lane_slice<K>(own, tt), lane_slice<K>(nxt, tt), st);
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const uint32_t h = hyb_hash(st[q]);
                        a[q] = lds_u32(((h << 1) & 0xFF80u) | lut_lane) ^ (h & 0x8000u);
                    }
                    mma_16816(acc[ms], a, xb[2 * ks], xb[2 * ks + 1]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sh->empty[s]));
        }
        finish_segment(acc, red, sh, out, partial, counters, M, nb, B, G, kmax, m, bs);
        seg0 = seg1;
    }
    if (*abort_flag) {
        // a wait gave up: give copies that may still be in flight time to land before the CTA retires
        for (int i = 0; i < 1000; i++) __nanosleep(1000);
    }
}

// ---- 3INST / 1MAD, plain layout, V = 1 ---------------------------------------------------------------------
// Same partition and reduction; the codes are read straight from global memory (the tile words a
// lane needs are 2-3 consecutive 16-bit words, shared with its neighbours through L1).  Within a
// tile lane (g, t) decodes elements (row g, cols 4t..4t+3) and (row g+8, cols 4t..4t+3): two runs
// of four consecutive states.  The A fragment wants columns {2t, 2t+1, 2t+8, 2t+9}; instead of
// moving weights between lanes the k index of the MMA is permuted (fragment column 2t+e is matrix
// column 4t+e, fragment column 2t+8+e is matrix column 4t+2+e) and x is loaded with the same
// permutation, which leaves every dot product unchanged.
template <int CODE>
__device__ __forceinline__ uint32_t decode_pair(uint32_t s0, uint32_t s1) {
    __half lo, hi;
    if constexpr (CODE == QTIP_CODE_3INST) { lo = decode_3inst(s0 & 0xFFFFu); hi = decode_3inst(s1 & 0xFFFFu); }
    else { lo = decode_1mad(s0 & 0xFFFFu); hi = decode_1mad(s1 & 0xFFFFu); }
    __half2 p = __halves2half2(lo, hi);
    return *reinterpret_cast<uint32_t *>(&p);
}

// 48 stream bits of a tile starting at bit pos (circular over the tile's words), first bit at bit 47
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
__global__ void __launch_bounds__(kConsumerThreads, 1)
    matvec_plain_kernel(float *__restrict__ out, const uint16_t *__restrict__ codes, const __half *__restrict__ x, int K,
                        int m, int n, int bs, int kmax, uint8_t *__restrict__ workspace) {
    extern __shared__ __align__(128) uint8_t smem[];
    Shared *sh = reinterpret_cast<Shared *>(smem);
    float *red = reinterpret_cast<float *>(smem + 256);
    unsigned *counters = reinterpret_cast<unsigned *>(workspace);
    float *partial = reinterpret_cast<float *>(workspace + kPartialOffset);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tn = n >> 4, nwords = 16 * K;
    const int g = lane >> 2, t = lane & 3;
    const bool xvalid = g < bs;
    const __half *xrow = x + (size_t)(xvalid ? g : 0) * n;
    const long nb = n >> 5;
    const long B = (long)(m >> 5) * nb, G = gridDim.x;
    const long r0 = range_start(blockIdx.x, B, G), r1 = range_start(blockIdx.x + 1, B, G);

    for (long seg0 = r0; seg0 < r1;) {
        const long M = seg0 / nb;
        const long seg1 = min(r1, (M + 1) * nb);
        float acc[2][4] = {};
        const int kt0 = 2 * (int)(seg0 - M * nb), kt1 = 2 * (int)(seg1 - M * nb);
        for (int kt = kt0 + warp; kt < kt1; kt += kConsumerWarps) {
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
                    const uint64_t bits = tile_bits48(words, nwords, e0 * K);
                    const uint32_t s0 = (uint32_t)(bits >> 32), s1 = (uint32_t)(bits >> (32 - K));
                    const uint32_t s2 = (uint32_t)(bits >> (32 - 2 * K)), s3 = (uint32_t)(bits >> (32 - 3 * K));
                    a[hr] = decode_pair<CODE>(s0, s1);       // a0 / a1: fragment cols 2t, 2t+1
                    a[2 + hr] = decode_pair<CODE>(s2, s3);   // a2 / a3: fragment cols 2t+8, 2t+9
                }
                mma_16816(acc[ms], a, b0, b1);
            }
        }
        finish_segment(acc, red, sh, out, partial, counters, M, nb, B, G, kmax, m, bs);
        seg0 = seg1;
    }
}

int check_common(const void *out, const void *codes, const void *x, int K, int m, int n, int bs, void *workspace,
                 size_t workspace_bytes) {
    if (!out || !codes || !x || K < 2 || K > 4 || bs < 1 || bs > kMaxBatch) return QTIP_ERR_BAD_ARG;
    if (m <= 0 || n <= 0 || (m & 31) || (n & 31) || (size_t)(m >> 5) * 4 > kCounterBytes) return QTIP_ERR_BAD_SHAPE;
    if (!workspace || workspace_bytes < qtip_matvec_workspace_bytes(m, n, bs)) return QTIP_ERR_WORKSPACE;
    if (!aligned(workspace, 256) || !aligned(codes, 16) || !aligned(x, 4) || !aligned(out, 4)) return QTIP_ERR_ALIGNMENT;
    return QTIP_OK;
}

template <int K>
int launch_hyb(float *out, const uint8_t *codes, const __half *x, const uint32_t *tlut, int m, int n, int bs,
               uint8_t *workspace, cudaStream_t s) {
    constexpr int kStageBytes = kStageBlocks * 128 * K;
    // ring depth: about 64 KiB in flight per SM
    constexpr int nstages = (64 * 1024 / kStageBytes) < kMaxStages ? (64 * 1024 / kStageBytes) : kMaxStages;
    // worst case the LUT alignment wastes just under 64 KiB below it only if nothing fits there; the
    // carve order (control, reduction buffer, stages) fills the low part first, so size for: slack to
    // the boundary + LUT + everything else
    constexpr uint32_t payload = 256 + kRedBytes + nstages * kStageBytes;  // control block, reduction buffer, ring
    constexpr uint32_t smem_total = 64 * 1024 + kLutBytes + payload > 227 * 1024 ? 227 * 1024
                                                                                   : 64 * 1024 + kLutBytes + payload;
    static_assert(kLutBytes + payload + 1024 + kStageBytes <= 227 * 1024, "ring does not fit");
    static bool attr_set[64] = {};
    int dev = 0;
    QTIP_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 64 && !attr_set[dev]) {
        QTIP_CUDA_TRY(cudaFuncSetAttribute(matvec_hyb_kernel<K>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)smem_total));
        attr_set[dev] = true;
    }
    const Partition p = make_partition(m, n);
    matvec_hyb_kernel<K><<<p.grid, kThreads, smem_total, s>>>(out, codes, x, tlut, m, n, bs, p.kmax, nstages, workspace,
                                                             smem_total);
    return check_launch();
}

}  // namespace
}  // namespace qtip

using namespace qtip;

extern "C" size_t qtip_matvec_workspace_bytes(int m, int n, int bs) {
    (void)bs;
    if (m < 32 || n < 32) return kPartialOffset;
    const long nb = n >> 5, B = (long)(m >> 5) * nb;
    const long G = B < kMaxGrid ? B : kMaxGrid;
    return kPartialOffset + (size_t)(m >> 5) * max_contributors(nb, B, G) * 256 * sizeof(float);
}

extern "C" int qtip_decompress_matvec(float *out, const void *codes, const void *x, const void *tlut, int K, int m,
                                      int n, int bs, void *workspace, size_t workspace_bytes, void *stream) {
    if (!tlut) return QTIP_ERR_BAD_ARG;
    int st = check_common(out, codes, x, K, m, n, bs, workspace, workspace_bytes);
    if (st != QTIP_OK) return st;
    if (!aligned(tlut, 4)) return QTIP_ERR_ALIGNMENT;
    auto *c = static_cast<const uint8_t *>(codes);
    auto *xh = static_cast<const __half *>(x);
    auto *t = static_cast<const uint32_t *>(tlut);
    auto *ws = static_cast<uint8_t *>(workspace);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (K == 2) return launch_hyb<2>(out, c, xh, t, m, n, bs, ws, s);
    if (K == 3) return launch_hyb<3>(out, c, xh, t, m, n, bs, ws, s);
    return launch_hyb<4>(out, c, xh, t, m, n, bs, ws, s);
}

extern "C" int qtip_decompress_matvec_plain(float *out, const void *codes, const void *x, int code, int K, int m, int n,
                                            int bs, void *workspace, size_t workspace_bytes, void *stream) {
    if (code != QTIP_CODE_3INST && code != QTIP_CODE_1MAD) return QTIP_ERR_BAD_ARG;
    int st = check_common(out, codes, x, K, m, n, bs, workspace, workspace_bytes);
    if (st != QTIP_OK) return st;
    const Partition p = make_partition(m, n);
    auto *c = static_cast<const uint16_t *>(codes);
    auto *xh = static_cast<const __half *>(x);
    auto *ws = static_cast<uint8_t *>(workspace);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    constexpr int smem = 256 + kRedBytes;
    if (code == QTIP_CODE_3INST)
        matvec_plain_kernel<QTIP_CODE_3INST><<<p.grid, kConsumerThreads, smem, s>>>(out, c, xh, K, m, n, bs, p.kmax, ws);
    else
        matvec_plain_kernel<QTIP_CODE_1MAD><<<p.grid, kConsumerThreads, smem, s>>>(out, c, xh, K, m, n, bs, p.kmax, ws);
    return check_launch();
}
