// Fused trellis-decode + matvec (batch 1..8) for B200.
//
// Partition.  The packed matrix is a sequence of B = (m/32)*(n/32) blocks (a block is a 2x2 group of
// 16x16 tiles, 128*K contiguous bytes; the blocks of one 32-row block are contiguous).  The grid
// has at most one CTA per SM.  Two schedules exist and the host picks the cheaper one per shape:
//   rows     CTA c owns whole 32-row blocks c, c+G, ...: no cross-CTA reduction at all;
//   stream-K CTA c owns the contiguous block range [c*B/G, (c+1)*B/G), cut into segments at
//            row-block boundaries: perfectly balanced bytes, but row blocks shared by several
//            CTAs need the ticket reduction below.
//
// Data path.  A producer warp streams the CTA's segments through a ring of shared-memory stages
// with cp.async.bulk (TMA, completion on an mbarrier per stage), running ahead of the consumers
// across segment boundaries.  31 consumer warps take the blocks of a stage two at a time: a lane
// reads its 4K contiguous bytes and those of lane+1 (wrap-around bits) from the stage, decodes 16
// trellis states into four mma.m16n8k16 A fragments in registers - HYB: h = s*(s+1), entry
// (h>>6)&1023 of a 1024-entry table (the 512-entry LUT and its sign-flipped twin) kept as 32
// lane-private copies in shared memory, so gathers never conflict - and multiplies them with x held in the B fragment (column j of B = batch row
// j, so up to 8 batch rows ride along for free).  fp32 accumulation in the MMA.
//
// Reduction.  Warps of a CTA are summed through shared memory at the end of a segment.  When a
// row block is shared by several CTAs each stores its partial sums to the workspace and takes a
// ticket; the CTA that draws the last ticket adds the partials in CTA order and writes the result,
// so the output is deterministic and is overwritten, never accumulated into.
//
// Launch overlap.  The kernel is launched with programmatic stream serialization: everything that
// touches only weights (barrier setup, LUT replication, the first ring fills) runs before
// griddepcontrol.wait, i.e. while the previous kernel of the stream drains; x, out and the
// workspace are touched only after it.
//
// Every wait on an mbarrier is bounded: after kSpinLimit polls the thread records an error code in
// the workspace status word, raises a CTA-wide abort flag that makes all later waits fall through,
// and the kernel runs to its end (with meaningless results) instead of hanging.
//
// Upstream counterpart: kernel_decompress_matvec, qtip-kernels/src/inference.cu:168-425.
#include <cstdlib>

#include "common.cuh"

namespace qtip {
namespace {

constexpr int kConsumerWarps = 32;               // all 32 warps decode; lane 0 of warp 0 also feeds the ring
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = 1024;
constexpr int kStageBlocks = 2 * kConsumerWarps; // blocks per ring stage: two per warp
// Gather table: 1024 entries (sign bit of the hash folded in as the top index bit, so no separate
// sign flip is needed) x 32 lane-private copies x half2 = 128 KiB.  Entry e, copy l at byte e*128 + l*4:
// every lane reads its own bank, so a warp's 32 random lookups never conflict.
constexpr int kLutBytes = 1024 * 32 * 4;
constexpr int kCtrlBytes = 256;
constexpr int kSmemLimit = 227 * 1024;
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
constexpr int kMaxGrid = 1024;  // sizing bound for the number of CTAs

// A row block (nb consecutive blocks) meets at most floor(nb / minlen) CTAs that lie entirely inside
// it plus two partial ones, where minlen = floor(B / G) is the shortest CTA range.
inline int max_contributors(long nb, long B, long G) {
    const long minlen = B / G > 0 ? B / G : 1;
    return (int)(nb / minlen) + 2;
}

enum { kModeStreamK = 1, kModeRows = 2 };

struct Partition {
    int grid;       // CTAs
    int kmax;       // contributor slots per row block
    int mode;
};

// Cost model in bytes streamed by the busiest SM; the ticket reduction of a shared row block costs
// about as much time as streaming kTailBytes.
constexpr long kTailBytes = 40 * 1024;

Partition make_partition(int m, int n, int K) {
    static const int forced = [] { const char *e = getenv("QTIP_MATVEC_MODE"); return e ? atoi(e) : 0; }();
    Partition p;
    const long mb = m >> 5, nb = n >> 5, B = mb * nb, sms = sm_count(), bb = 128 * K;
    const long g_stream = B < sms ? B : sms, g_rows = mb < sms ? mb : sms;
    const long cost_rows = ((mb + g_rows - 1) / g_rows) * nb * bb;
    const bool shared_rows = (B % g_stream) != 0 || ((B / g_stream) % nb) != 0;
    const long cost_stream = ((B + g_stream - 1) / g_stream) * bb + (shared_rows ? kTailBytes : 0);
    p.mode = forced ? forced : (cost_rows <= cost_stream ? kModeRows : kModeStreamK);
    p.grid = (int)(p.mode == kModeRows ? g_rows : g_stream);
    p.kmax = max_contributors(nb, B, g_stream);
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
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// A lane's 4K bytes of a block staged in shared memory.
template <int K>
__device__ __forceinline__ LaneCodes<K> lds_lane_codes(uint32_t addr) {
    LaneCodes<K> c;
    if constexpr (K == 2) {
        asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(c.w[0]), "=r"(c.w[1]) : "r"(addr) : "memory");
    } else if constexpr (K == 3) {
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(c.w[0]) : "r"(addr) : "memory");
        asm volatile("ld.shared.u32 %0, [%1+4];" : "=r"(c.w[1]) : "r"(addr) : "memory");
        asm volatile("ld.shared.u32 %0, [%1+8];" : "=r"(c.w[2]) : "r"(addr) : "memory");
    } else {
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(c.w[0]), "=r"(c.w[1]), "=r"(c.w[2]), "=r"(c.w[3])
                     : "r"(addr)
                     : "memory");
    }
    return c;
}

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// ---- partition arithmetic -------------------------------------------------------------------------------
__host__ __device__ __forceinline__ long range_start(long c, long B, long G) { return c * B / G; }
__host__ __device__ __forceinline__ long cta_of_block(long b, long B, long G) { return ((b + 1) * G - 1) / B; }

// The segments (row block M, blocks [s0, s1) in the global block numbering) of one CTA, in order.
struct SegmentIter {
    long nb, end, pos, step;  // rows mode: pos = M*nb, step = G*nb;  stream-K: pos walks [r0, r1)
    int mode;
    __device__ __forceinline__ SegmentIter(int mode_, long mb, long nb_, long G, long c) : nb(nb_), mode(mode_) {
        if (mode == kModeRows) { pos = c * nb; end = mb * nb; step = G * nb; }
        else { const long B = mb * nb; pos = range_start(c, B, G); end = range_start(c + 1, B, G); step = 0; }
    }
    __device__ __forceinline__ bool next(long &s0, long &s1) {
        if (pos >= end) return false;
        s0 = pos;
        if (mode == kModeRows) { s1 = pos + nb; pos += step; }
        else { s1 = min(end, (pos / nb + 1) * nb); pos = s1; }
        return true;
    }
};

struct Shared {            // control block at the start of dynamic shared memory
    unsigned long long full[kMaxStages];
    unsigned long long empty[kMaxStages];
    int abort_flag;
    int is_last;
    // cursor of the ring producer (touched by thread 0 only)
    long p_pos, p_end, p_step, p_seg_end;   // next block to fetch; end of the CTA's work; rows-mode stride; end of the current segment
    unsigned p_slot, p_round;
};
static_assert(sizeof(Shared) <= kCtrlBytes, "control block too large");

// Cross-warp sum of the per-warp 32 x 8 accumulators of one segment, then the final store or the
// partial-sum / ticket protocol.  Consumer threads only (NW warps).  Only the first `bs` batch
// columns are kept: red holds [NW][bs][32] floats.
// trailing_sync = false is allowed only when the caller alternates between two `red` buffers, so
// that the next segment's stores cannot overtake this segment's readers.
template <int NW>
__device__ __forceinline__ void finish_segment(float (&acc)[2][4], float *red, Shared *sh, float *__restrict__ out,
                                               float *__restrict__ partial, unsigned *__restrict__ counters, long M,
                                               long nb, long B, long G, int kmax, int m, int bs, bool whole_row,
                                               bool trailing_sync = true) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int stride = 32 * bs;
    // accumulator (ms, i): row = 16*ms + g + 8*(i>>1), batch = 2*t + (i&1); slot = batch*32 + row
#pragma unroll
    for (int ms = 0; ms < 2; ms++)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int batch = 2 * t + (i & 1);
            if (batch < bs) red[warp * stride + batch * 32 + 16 * ms + g + 8 * (i >> 1)] = acc[ms][i];
        }
    asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");
    float v = 0.f;
    if (tid < stride) {
#pragma unroll 4
        for (int w = 0; w < NW; w++) v += red[w * stride + tid];
    }
    const int b = tid >> 5, r = tid & 31;
    int contributors = 1;
    long c_first = 0;
    if (!whole_row) {
        c_first = cta_of_block(M * nb, B, G);
        contributors = (int)(cta_of_block((M + 1) * nb - 1, B, G) - c_first) + 1;
    }
    if (contributors == 1) {
        if (tid < stride) out[(size_t)b * m + 32 * M + r] = v;
        if (trailing_sync) asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");
        return;
    }
    const int k = (int)(blockIdx.x - c_first);
    float *slot = partial + ((size_t)M * kmax) * 256;
    if (tid < stride) __stcg(slot + (size_t)k * 256 + tid, v);
    __threadfence();
    asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");
    if (tid == 0) {
        unsigned prev = atomicAdd(&counters[M], 1u);
        sh->is_last = (prev == (unsigned)(contributors - 1));
    }
    asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");
    if (sh->is_last) {
        __threadfence();
        if (tid < stride) {
            float s = 0.f;
            for (int c = 0; c < contributors; c++) s += __ldcg(slot + (size_t)c * 256 + tid);
            out[(size_t)b * m + 32 * M + r] = s;
        }
        if (tid == 0) counters[M] = 0;  // leave the workspace ready for the next call
    }
    asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");
}

// The four states of tile tt (= ks*2 + ms) of a lane, from the lane's own words and those of lane+1.
// Only the low 16 bits of each st[q] are meaningful (the hash ignores the rest), which saves the
// masks and, for the state that already sits in the low half of a word, the shift.  Shifts are
// funnel shifts of (own : next) so no 64-bit value is ever formed.
template <int K>
__device__ __forceinline__ void tile_states(const LaneCodes<K> &own, const LaneCodes<K> &nxt, int tt, uint32_t (&st)[4]) {
    if constexpr (K == 2) {
        // word ks holds slice(ms=1) << 16 | slice(ms=0); state q = low 16 bits of (own slice << 4q | next slice >> (16-4q))
        const uint32_t w = own.w[tt >> 1], nw = nxt.w[tt >> 1];
        if ((tt & 1) == 0) {
            const uint32_t lo = nw << 16;  // next slice in the top half
            st[0] = w; st[1] = __funnelshift_l(lo, w, 4); st[2] = __funnelshift_l(lo, w, 8); st[3] = __funnelshift_l(lo, w, 12);
        } else {
            const uint32_t hi = w >> 16;   // nw already has the next slice in its top half
            st[0] = hi; st[1] = __funnelshift_l(nw, hi, 4); st[2] = __funnelshift_l(nw, hi, 8); st[3] = __funnelshift_l(nw, hi, 12);
        }
    } else if constexpr (K == 3) {
        // 24-bit slices at byte offset 3*tt.  S: own slice in the low 24 bits (junk above is shifted
        // out); N: next slice with its top 16 bits in the top half of the register.
        uint32_t S, N;
        if (tt == 0) { S = own.w[0]; N = nxt.w[0] << 8; }
        else if (tt == 1) { S = __funnelshift_r(own.w[0], own.w[1], 24); N = __funnelshift_r(nxt.w[0], nxt.w[1], 16); }
        else if (tt == 2) { S = __funnelshift_r(own.w[1], own.w[2], 16); N = __funnelshift_r(nxt.w[1], nxt.w[2], 8); }
        else { S = own.w[2] >> 8; N = nxt.w[2]; }
        // window bit 47 = first bit of S; state q = window bits [47-6q .. 32-6q]
        st[0] = S >> 8; st[1] = S >> 2; st[2] = __funnelshift_l(N, S, 4); st[3] = __funnelshift_l(N, S, 10);
    } else {
        const uint32_t S = own.w[tt], N = nxt.w[tt];
        st[0] = S >> 16; st[1] = S >> 8; st[2] = S; st[3] = __funnelshift_l(N, S, 8);
    }
}

// One HYB lookup: h = t*t + t; entry = h bits 15..6 (bit 15 = sign flip of the first weight, folded
// into the table); 128 bytes per entry, the lane's copy selected by lut_lane.  Two of the four
// instructions are integer multiply-adds, which issue at full rate; logic ops are half rate.
__device__ __forceinline__ uint32_t hyb_lookup(uint32_t t, uint32_t lut_lane) {
    uint32_t w;
    asm("{\n\t.reg .b32 h, a;\n\t"
        "mad.lo.u32 h, %1, %1, %1;\n\t"
        "and.b32 h, h, 0xFFC0;\n\t"
        "mad.lo.u32 a, h, 2, %2;\n\t"
        "ld.shared.u32 %0, [a];\n\t}"
        : "=r"(w)
        : "r"(t), "r"(lut_lane));
    return w;
}

// 16 states of one lane -> four A fragments -> four MMAs (2 k-subtiles x 2 m-subtiles).
template <int K>
__device__ __forceinline__ void decode_block(const LaneCodes<K> &own, const LaneCodes<K> &nxt, const uint32_t (&xb)[4],
                                             float (&acc)[2][4], uint32_t lut_lane) {
#pragma unroll
    for (int tt = 0; tt < 4; tt++) {
        const int ks = tt >> 1, ms = tt & 1;
        uint32_t st[4], a[4];
        tile_states<K>(own, nxt, tt, st);
#pragma unroll
        for (int q = 0; q < 4; q++) a[q] = hyb_lookup(st[q], lut_lane);
        mma_16816(acc[ms], a, xb[2 * ks], xb[2 * ks + 1]);
    }
}

// Ring producer step (thread 0 only): fetch the next stage of this CTA's work, if any, into ring slot
// p_slot.  A slot may be refilled once all 32 warps have pulled their bytes of its previous use.
template <int K>
__device__ __forceinline__ void produce_stage(Shared *sh, const uint8_t *__restrict__ codes, uint32_t ring, int nstages,
                                              int mode, long nb, unsigned *status) {
    constexpr int kBlockBytes = 128 * K;
    constexpr int kStageBytes = kStageBlocks * kBlockBytes;
    long pos = sh->p_pos;
    if (pos >= sh->p_end) return;
    volatile int *abort_flag = &sh->abort_flag;
    if (*abort_flag) return;
    long seg_end = sh->p_seg_end;
    if (pos >= seg_end) {  // open the next segment
        if (mode == kModeRows) { pos += sh->p_step - nb; seg_end = pos + nb; if (pos >= sh->p_end) { sh->p_pos = pos; return; } }
        else seg_end = min(sh->p_end, (pos / nb + 1) * nb);
        sh->p_seg_end = seg_end;
    }
    const unsigned slot = sh->p_slot, round = sh->p_round;
    if (round > 0) mbar_wait(smem_u32(&sh->empty[slot]), (round - 1) & 1, abort_flag, status, 1);
    const uint32_t bytes = (uint32_t)min((long)kStageBlocks, seg_end - pos) * kBlockBytes;
    const uint32_t bar = smem_u32(&sh->full[slot]);
    mbar_expect_tx(bar, bytes);
    bulk_g2s(ring + slot * kStageBytes, codes + (size_t)pos * kBlockBytes, bytes, bar);
    sh->p_pos = pos + min((long)kStageBlocks, seg_end - pos);
    if (slot + 1 == (unsigned)nstages) { sh->p_slot = 0; sh->p_round = round + 1; }
    else sh->p_slot = slot + 1;
}

// XS: x is staged once per CTA in shared memory, permuted so that a lane's four B-fragment words of
// a block are one 16-byte load; otherwise they are read from global memory (L1-resident) per block.
// DB: the cross-warp reduction buffer is double-buffered, which drops one CTA barrier per segment.
template <int K, bool XS, bool DB>
__global__ void __launch_bounds__(kThreads, 1)
    matvec_hyb_kernel(float *__restrict__ out, const uint8_t *__restrict__ codes, const __half *__restrict__ x,
                      const uint32_t *__restrict__ tlut, int m, int n, int bs, int kmax, int mode, int nstages,
                      uint8_t *__restrict__ workspace) {
    constexpr int kBlockBytes = 128 * K;
    constexpr int kStageBytes = kStageBlocks * kBlockBytes;
    extern __shared__ __align__(128) uint8_t smem[];
    // layout: control block | LUT | ring stages | reduction buffer(s) [32][bs][32] fp32 | x (bs, n) fp16 permuted
    Shared *sh = reinterpret_cast<Shared *>(smem);
    uint32_t *lut = reinterpret_cast<uint32_t *>(smem + kCtrlBytes);
    const uint32_t ring = smem_u32(smem + kCtrlBytes + kLutBytes);
    const int red_floats = kConsumerWarps * 32 * bs;
    float *red = reinterpret_cast<float *>(smem + kCtrlBytes + kLutBytes + nstages * kStageBytes);
    uint4 *xs = reinterpret_cast<uint4 *>(red + (DB ? 2 : 1) * red_floats);

    unsigned *counters = reinterpret_cast<unsigned *>(workspace);
    unsigned *status = reinterpret_cast<unsigned *>(workspace + kStatusOffset);
    float *partial = reinterpret_cast<float *>(workspace + kPartialOffset);

    const int nb = n >> 5, mb = m >> 5;
    const int G = gridDim.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < nstages; s++) {
            mbar_init(smem_u32(&sh->full[s]), 1);
            mbar_init(smem_u32(&sh->empty[s]), kConsumerWarps);
        }
        sh->abort_flag = 0;
        sh->is_last = 0;
        SegmentIter it(mode, mb, nb, G, blockIdx.x);
        sh->p_pos = it.pos; sh->p_end = it.end; sh->p_step = it.step;
        sh->p_seg_end = mode == kModeRows ? it.pos + nb : min(it.end, (it.pos / nb + 1) * nb);
        sh->p_slot = 0; sh->p_round = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // fill the ring: packed codes are weights, no need to wait for the previous kernel
        for (int s = 0; s < nstages; s++) produce_stage<K>(sh, codes, ring, nstages, mode, nb, status);
    }
    // lane-private LUT copies: entry e = sign << 9 | index, copy l at byte e*128 + l*4; the sign bit
    // flips the sign of the first (low) half of the pair
    for (int i = threadIdx.x; i < 1024 * 8; i += kThreads) {
        const uint32_t e = __ldg(tlut + ((i >> 3) & 511)) ^ ((uint32_t)(i >> 12) << 15);
        reinterpret_cast<uint4 *>(lut)[i] = make_uint4(e, e, e, e);
    }
    grid_launch_dependents();  // the next kernel of the stream may start its own weight-only prologue
    grid_dependency_wait();    // x, out and the workspace belong to the stream's data flow
    if constexpr (XS) {
        // xs[(b*nb + N)*4 + t] = { x[b][32N+2t..+1], x[..+8..], x[..+16..], x[..+24..] }
        const uint32_t *xw = reinterpret_cast<const uint32_t *>(x);
        const int words = bs * (n >> 1);
        for (int i = threadIdx.x; i < words; i += kThreads) {
            const int blk = i >> 4, w = i & 15;          // 16 words per 32-column block
            reinterpret_cast<uint32_t *>(xs)[blk * 16 + (w & 3) * 4 + (w >> 2)] = __ldg(xw + i);
        }
    }
    __syncthreads();

    volatile int *abort_flag = &sh->abort_flag;
    const int g = lane >> 2, t = lane & 3;
    const int xg = g < bs ? g : 0;  // lanes of unused batch columns alias row 0; their results are never stored
    const uint32_t *xrow = reinterpret_cast<const uint32_t *>(x + (size_t)xg * n + 2 * t);
    const uint4 *xsrow = xs + (size_t)xg * nb * 4 + t;
    const uint32_t lut_lane = smem_u32(lut) + lane * 4;
    const uint32_t own_off = lane * (4 * K), nxt_off = ((lane + 1) & 31) * (4 * K);
    const uint32_t off0 = warp * kBlockBytes, off1 = (warp + kConsumerWarps) * kBlockBytes;

    uint32_t s = 0, phase = 0, segno = 0;  // ring slot, parity its "full" barrier completes next
    SegmentIter segs(mode, mb, nb, G, blockIdx.x);
    long seg0, seg1;
    while (segs.next(seg0, seg1)) {
        const int M = (int)(seg0 / nb);
        float acc[2][4] = {};
        int N0 = (int)(seg0 - (long)M * nb) + warp;  // this warp's first block of the stage inside the row block
        for (int left = (int)(seg1 - seg0); left > 0; left -= kStageBlocks, N0 += kStageBlocks) {
            const bool v0 = warp < left, v1 = warp + kConsumerWarps < left;
            LaneCodes<K> own0, nxt0, own1, nxt1;
            uint32_t xb0[4], xb1[4];  // [ks][cols 2t,2t+1 | cols 2t+8,2t+9]
            if (v0) {
                if constexpr (XS) {
                    const uint4 a = xsrow[N0 * 4];
                    xb0[0] = a.x; xb0[1] = a.y; xb0[2] = a.z; xb0[3] = a.w;
                    if (v1) { const uint4 b = xsrow[(N0 + kConsumerWarps) * 4]; xb1[0] = b.x; xb1[1] = b.y; xb1[2] = b.z; xb1[3] = b.w; }
                } else {
                    const uint32_t *xp = xrow + 16 * N0;
                    xb0[0] = __ldg(xp); xb0[1] = __ldg(xp + 4); xb0[2] = __ldg(xp + 8); xb0[3] = __ldg(xp + 12);
                    if (v1) {
                        xp += 16 * kConsumerWarps;
                        xb1[0] = __ldg(xp); xb1[1] = __ldg(xp + 4); xb1[2] = __ldg(xp + 8); xb1[3] = __ldg(xp + 12);
                    }
                }
                mbar_wait(smem_u32(&sh->full[s]), phase, abort_flag, status, 2);
                const uint32_t stage = ring + s * kStageBytes;
                own0 = lds_lane_codes<K>(stage + off0 + own_off);
                nxt0 = lds_lane_codes<K>(stage + off0 + nxt_off);
                if (v1) {
                    own1 = lds_lane_codes<K>(stage + off1 + own_off);
                    nxt1 = lds_lane_codes<K>(stage + off1 + nxt_off);
                }
            }
            // the warp's bytes of this stage are in registers: release the slot before decoding
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sh->empty[s]));
            if (++s == (uint32_t)nstages) { s = 0; phase ^= 1; }
            if (v0) {
                decode_block<K>(own0, nxt0, xb0, acc, lut_lane);
                if (v1) decode_block<K>(own1, nxt1, xb1, acc, lut_lane);
            }
            if (threadIdx.x == 0) produce_stage<K>(sh, codes, ring, nstages, mode, nb, status);
        }
        finish_segment<kConsumerWarps>(acc, DB ? red + (segno & 1) * red_floats : red, sh, out, partial, counters, M, nb,
                                       (long)mb * nb, G, kmax, m, bs, mode == kModeRows, !DB);
        segno++;
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

constexpr int kPlainWarps = 16;

template <int CODE>
__global__ void __launch_bounds__(kPlainWarps * 32, 2)
    matvec_plain_kernel(float *__restrict__ out, const uint16_t *__restrict__ codes, const __half *__restrict__ x, int K,
                        int m, int n, int bs, int kmax, int mode, uint8_t *__restrict__ workspace) {
    extern __shared__ __align__(128) uint8_t smem[];
    Shared *sh = reinterpret_cast<Shared *>(smem);
    float *red = reinterpret_cast<float *>(smem + kCtrlBytes);
    unsigned *counters = reinterpret_cast<unsigned *>(workspace);
    float *partial = reinterpret_cast<float *>(workspace + kPartialOffset);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tn = n >> 4, nwords = 16 * K;
    const int g = lane >> 2, t = lane & 3;
    const bool xvalid = g < bs;
    const __half *xrow = x + (size_t)(xvalid ? g : 0) * n;
    const long nb = n >> 5, mb = m >> 5;
    const long B = mb * nb, G = gridDim.x;

    SegmentIter segs(mode, mb, nb, G, blockIdx.x);
    long seg0, seg1;
    while (segs.next(seg0, seg1)) {
        const long M = seg0 / nb;
        float acc[2][4] = {};
        const int kt0 = 2 * (int)(seg0 - M * nb), kt1 = 2 * (int)(seg1 - M * nb);
        for (int kt = kt0 + warp; kt < kt1; kt += kPlainWarps) {
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
        finish_segment<kPlainWarps>(acc, red, sh, out, partial, counters, M, nb, B, G, kmax, m, bs, mode == kModeRows);
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

template <int K, bool XS, bool DB>
int launch_hyb_variant(float *out, const uint8_t *codes, const __half *x, const uint32_t *tlut, int m, int n, int bs,
                       uint8_t *workspace, int nstages, int smem_total, cudaStream_t s) {
    static bool attr_set[64] = {};
    int dev = 0;
    QTIP_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 64 && !attr_set[dev]) {
        QTIP_CUDA_TRY(cudaFuncSetAttribute(matvec_hyb_kernel<K, XS, DB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           kSmemLimit));
        attr_set[dev] = true;
    }
    const Partition p = make_partition(m, n, K);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_total;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    QTIP_CUDA_TRY(cudaLaunchKernelEx(&cfg, matvec_hyb_kernel<K, XS, DB>, out, codes, x, tlut, m, n, bs, p.kmax, p.mode,
                                     nstages, workspace));
    return check_launch();
}

template <int K>
int launch_hyb(float *out, const uint8_t *codes, const __half *x, const uint32_t *tlut, int m, int n, int bs,
               uint8_t *workspace, cudaStream_t s) {
    constexpr int kStageBytes = kStageBlocks * 128 * K;
    // shared memory: control + table are fixed; the ring gets what the reduction buffer(s) and the
    // staged x leave.  Prefer (double-buffered reduction, x in shared memory) while >= 3 stages remain.
    const int red_bytes = kConsumerWarps * 32 * bs * (int)sizeof(float);
    const int x_bytes = bs * n * 2;
    const int avail = kSmemLimit - kCtrlBytes - kLutBytes;
    const bool db = bs <= 2;
    const int fixed = (db ? 2 : 1) * red_bytes;
    const bool xs = (avail - fixed - x_bytes) / kStageBytes >= 3;
    int nstages = (avail - fixed - (xs ? x_bytes : 0)) / kStageBytes;
    if (nstages > kMaxStages) nstages = kMaxStages;
    if (nstages < 2) return QTIP_ERR_BAD_ARG;
    const int smem_total = kCtrlBytes + kLutBytes + nstages * kStageBytes + fixed + (xs ? x_bytes : 0);
    if (xs && db) return launch_hyb_variant<K, true, true>(out, codes, x, tlut, m, n, bs, workspace, nstages, smem_total, s);
    if (xs) return launch_hyb_variant<K, true, false>(out, codes, x, tlut, m, n, bs, workspace, nstages, smem_total, s);
    if (db) return launch_hyb_variant<K, false, true>(out, codes, x, tlut, m, n, bs, workspace, nstages, smem_total, s);
    return launch_hyb_variant<K, false, false>(out, codes, x, tlut, m, n, bs, workspace, nstages, smem_total, s);
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
    Partition p = make_partition(m, n, K);
    // two CTAs of 16 warps per SM
    if (p.mode == kModeStreamK) {
        const long B = (long)(m >> 5) * (n >> 5);
        p.grid = (int)(B < 2L * p.grid ? B : 2L * p.grid);
        p.kmax = max_contributors(n >> 5, B, p.grid);
    }
    auto *c = static_cast<const uint16_t *>(codes);
    auto *xh = static_cast<const __half *>(x);
    auto *ws = static_cast<uint8_t *>(workspace);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int smem = kCtrlBytes + kPlainWarps * 32 * bs * 4;
    if (code == QTIP_CODE_3INST)
        matvec_plain_kernel<QTIP_CODE_3INST><<<p.grid, kPlainWarps * 32, smem, s>>>(out, c, xh, K, m, n, bs, p.kmax,
                                                                                  p.mode, ws);
    else
        matvec_plain_kernel<QTIP_CODE_1MAD><<<p.grid, kPlainWarps * 32, smem, s>>>(out, c, xh, K, m, n, bs, p.kmax,
                                                                                 p.mode, ws);
    return check_launch();
}
