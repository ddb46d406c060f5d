// Fused trellis-decode + matvec (batch 1..8) for B200.
//
// Partition.  The packed matrix is a sequence of B = (m/32)*(n/32) blocks (a block is a 2x2 group of
// 16x16 tiles, 128*K contiguous bytes; the blocks of one 32-row block are contiguous).  The grid
// has at most one CTA (32 warps) per SM.  Two schedules exist and the host picks the cheaper one:
//   rows     CTA c owns whole 32-row blocks c, c+G, ...: no cross-CTA reduction at all;
//   stream-K CTA c owns the contiguous block range [c*B/G, (c+1)*B/G), cut into segments at
//            row-block boundaries: perfectly balanced bytes, but row blocks shared by several
//            CTAs need the ticket reduction below.
//
// Data path.  Inside a segment warp w owns a CONTIGUOUS run of blocks (1/32 of the segment).  It pulls the
// run in chunks of up to 1 KiB with one bulk copy (cp.async.bulk, the 1-D form of TMA) per chunk into a
// two-slot ring of its own in shared memory, completion on an mbarrier of its own; the next chunk -
// of this or of the following segment - is always in flight while one is decoded (up to 64 KiB in
// flight per SM, no registers held, no load-latency stalls in the loop).  A lane reads its 4K bytes of a
// block and those of lane+1 (the wrap-around bits of the tail-biting stream) from the ring, so the loop
// has no shuffles.  A lane decodes its 16 trellis states into four mma.m16n8k16 A
// fragments in registers - HYB: h = s*(s+1), entry (h>>6)&1023 of a 1024-entry table (the 512-entry
// LUT and its sign-flipped twin) kept as 32 lane-private copies in shared memory, so gathers never
// conflict - and multiplies them with x held in the B fragment (column j of B = batch row j, so up
// to 8 batch rows share one decode).  fp32 accumulation in the MMA.  x is staged once per CTA
// in shared memory in fragment order (one 16-byte load per block and lane) when it fits beside the
// table; 8 rows of a wide layer do not, and are then read from L1/L2 per block (about 1.5x the time
// of a single row).
//
// The kernel is instruction-issue bound, not HBM bound (about 5 instructions per state are
// irreducible: shift, multiply-add hash, mask, multiply-add address, shared load; multiply-add, logic
// and shift instructions each issue once per two cycles per sub-partition on this part).  The ring costs about one instruction per block because it is
// private to a warp: no producer warp, no CTA barrier, one bounded mbarrier wait per chunk.
//
// Reduction.  Warps of a CTA are summed through shared memory at the end of a segment.  When a
// row block is shared by several CTAs each stores its partial sums to the workspace and takes a
// ticket; the CTA that draws the last ticket adds the partials in CTA order and writes the result,
// so the output is deterministic and is overwritten, never accumulated into.
//
// Launch overlap.  The kernel is launched with programmatic stream serialization: everything that
// touches only weights (the first code loads, the table build) runs before griddepcontrol.wait,
// i.e. while the previous kernel of the stream drains; x, out and the workspace are touched only
// after it.  Waits: the per-chunk mbarrier wait (bounded; a time-out sets word 1 of the workspace's control
// area and the kernel runs to its end with meaningless results) and, in the tensor-parallel instantiation
// (TP), one bounded wait for the other GPUs' result values (see PeerIn below).
//
// Upstream counterpart: kernel_decompress_matvec, qtip-kernels/src/inference.cu:168-425.
#include <mutex>

#include <cstddef>

#include "fwht.cuh"

namespace qtip {
namespace {

constexpr int kConsumerWarps = 32;
// Gather table: 1024 entries (sign bit of the hash folded in as the top index bit, so no separate
// sign flip is needed) x 32 lane-private copies x half2 = 128 KiB.  Entry e, copy l at byte e*128 + l*4:
// every lane reads its own bank, so a warp's 32 random lookups never conflict.
constexpr int kLutBytes = 1024 * 32 * 4;
constexpr int kCtrlBytes = 1024;      // Shared (256 bytes) + two mbarriers per warp
constexpr int kBarOffset = 256;
constexpr int kMaxChunkBytes = 1024;  // bytes of packed codes per bulk copy
constexpr unsigned kRingSpinLimit = 1u << 22;
constexpr int kSmemLimit = 227 * 1024;
constexpr int kMaxBatch = 8;

// ---- workspace layout (all offsets fixed, independent of the problem) -----------------------------
// [0, 64 KiB)   ticket counters, one uint32 per 32-row block (m <= 524288); zero between calls
// [64 KiB, +256) word 0: counter of finished CTAs (fused output transform); zero between calls
//               word 1: sticky flag, set if a wait for a bulk copy ever ran out (never cleared by the kernels)
// [.., end)     partial sums: [row block][contributor][8 batch x 32 rows] fp32
constexpr size_t kCounterBytes = 64 * 1024;
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

// nprob problems of the same shape share one launch: each gets sm_count / nprob CTAs.
Partition make_partition(int m, int n, int K, int nprob = 1) {
    Partition p;
    const long mb = m >> 5, nb = n >> 5, B = mb * nb, bb = 128 * K;
    const long sms = sm_count() / nprob > 0 ? sm_count() / nprob : 1;
    const long g_stream = B < sms ? B : sms, g_rows = mb < sms ? mb : sms;
    const long cost_rows = ((mb + g_rows - 1) / g_rows) * nb * bb;
    const bool shared_rows = (B % g_stream) != 0 || ((B / g_stream) % nb) != 0;
    const long cost_stream = ((B + g_stream - 1) / g_stream) * bb + (shared_rows ? kTailBytes : 0);
    p.mode = cost_rows <= cost_stream ? kModeRows : kModeStreamK;
    p.grid = (int)(p.mode == kModeRows ? g_rows : g_stream);
    p.kmax = max_contributors(nb, B, g_stream);
    return p;
}

// ---- PTX wrappers -----------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

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

// Extra destinations of a result row block (tensor parallelism): this rank's slot in every GPU's peer-mapped
// buffer.  Each value travels as ONE 64-bit scalar store {value in the low word, stamp in the high word}; the reader
// knows a value has arrived when its stamp is the expected sequence number, so no fence, flag or atomic sits between
// producer and consumers.  A 64-bit scalar access is single-copy atomic in the PTX memory model (a vector access of
// two 32-bit elements would not be), so value and stamp can never be observed apart.
struct OutCopies {
    uint2 *dst[8];
    int n;
};
__device__ __forceinline__ void store_stamped(uint2 *p, float v, unsigned stamp) {
    const unsigned long long q = ((unsigned long long)stamp << 32) | (unsigned long long)__float_as_uint(v);
    asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(q) : "memory");
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Upper bound on the time one launch spends waiting for the other GPUs' values, whatever the poll limit says.
constexpr unsigned long long kPeerWaitNs = 200ull * 1000ull * 1000ull;

struct Shared {            // control block at the start of dynamic shared memory
    int is_last;
    int pad_[7];
    float warp_sums[32];   // scratch of block_sum
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
                                               bool trailing_sync, const OutCopies &copies, unsigned stamp) {
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
        if (tid < stride) {
            out[(size_t)b * m + 32 * M + r] = v;
            for (int q = 0; q < copies.n; q++) store_stamped(copies.dst[q] + (size_t)b * m + 32 * M + r, v, stamp);
        }
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
            for (int q = 0; q < copies.n; q++) store_stamped(copies.dst[q] + (size_t)b * m + 32 * M + r, s, stamp);
        }
        if (tid == 0) counters[M] = 0;  // leave the workspace ready for the next call
    }
    asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");
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

// One linear of a launch.  `in` / `ep` describe the optional transforms fused around the matvec.
struct FusedIn {    // x_raw != nullptr: x = fp16( H^T( sign_in * [silu(gate) *] [RMSNorm](x_raw [+ residual]) ) * scale )
    const __half *x_raw, *residual, *norm_weight, *gate, *sign_in;
    __half *residual_out;
    float scale, eps;
    // y_prev != nullptr: x_raw is not read; it is fp16(prev_sign * H(y_prev) * prev_scale), the deferred
    // output side of the linear that produced y_prev
    const float *y_prev, *prev_sign;
    float prev_scale;
};
struct FusedOut {   // final != nullptr: final = sign_out * H(out) * scale, computed by the last CTA to finish
    void *final;
    const float *sign_out;
    float scale;
    int dtype;
};
// Tensor parallelism without a separate all-reduce launch.  A row-parallel linear leaves a PARTIAL y on every
// GPU; the consumer's deferred output side (FusedIn::y_prev) then has to start from the sum over GPUs.
// Signal (producer): every result value is also stored, stamped with the sequence number *seq + 1, into this
// rank's vector on every GPU (copies); the CTA that finishes last then advances *seq.
// PeerIn (consumer): y[p] is GPU p's stamped vector in THIS GPU's memory; a thread re-reads its elements until
// they carry the stamp *seq (its own GPU's producer launch has already advanced it), at most max_polls times -
// then it sets *status and goes on (wrong numbers, but the kernel terminates).
constexpr int kMaxPeers = 8;
struct PeerIn {
    const uint2 *y[kMaxPeers];
    const unsigned *seq;
    unsigned *status;
    unsigned max_polls;
    int n;
};
struct Signal {
    unsigned *seq;
    OutCopies copies;
};
struct MatvecProblem {
    float *out;
    const uint8_t *codes;
    const __half *x;
    const uint32_t *tlut;
    uint8_t *workspace;
    FusedIn in;
    FusedOut ep;
    PeerIn peer;
    Signal sig;
};
constexpr int kMaxProblems = 4;
struct MatvecBatch {
    MatvecProblem p[kMaxProblems];
};

// ---- per-warp staging ring ----------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
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
// One bulk copy global -> shared (addresses and size multiples of 16 bytes), completion counted on `bar`.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// A lane's 4K bytes of a block in the ring (address = block start + lane * 4K); every access pattern below is
// conflict-free (8 / 16 bytes per lane contiguous, or words at stride 3).
template <int K>
__device__ __forceinline__ LaneCodes<K> lds_lane_codes(uint32_t addr) {
    LaneCodes<K> c;
    if constexpr (K == 2) {
        asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(c.w[0]), "=r"(c.w[1]) : "r"(addr));
    } else if constexpr (K == 3) {
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(c.w[0]) : "r"(addr));
        asm volatile("ld.shared.u32 %0, [%1+4];" : "=r"(c.w[1]) : "r"(addr));
        asm volatile("ld.shared.u32 %0, [%1+8];" : "=r"(c.w[2]) : "r"(addr));
    } else {
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(c.w[0]), "=r"(c.w[1]), "=r"(c.w[2]), "=r"(c.w[3]) : "r"(addr));
    }
    return c;
}

// E consecutive stamped values of one GPU's partial vector, read once; false if a stamp is not `want`
template <int E>
__device__ __forceinline__ bool loadE_stamped(const uint2 *p, size_t i, unsigned want, float (&o)[E]) {
    bool ok = true;
#pragma unroll
    for (int k = 0; k < E; k += 2) {
        unsigned long long a, b;   // two 64-bit elements, each {value, stamp} read atomically
        asm volatile("ld.relaxed.sys.global.v2.b64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(p + i + k) : "memory");
        o[k] = __uint_as_float((unsigned)a); o[k + 1] = __uint_as_float((unsigned)b);
        ok = ok && (unsigned)(a >> 32) == want && (unsigned)(b >> 32) == want;
    }
    return ok;
}

// Before the whole CTA reads the vectors, one warp watches 32 sample elements of each until they are current:
// the other 31 warps stay off the memory system while the data is still on its way (150 000 threads re-reading
// with system scope slow the arriving stores down by orders of magnitude).  Bounded like the reads themselves.
__device__ __forceinline__ void await_samples(const PeerIn &peer, int n, unsigned want, unsigned long long t_start,
                                              bool dead) {
    // `dead` may differ between threads (another CTA can set the status word at any time): the warp agrees on it,
    // and the CTA barrier below is reached by every thread whatever it saw
    if (threadIdx.x < 32 && !__any_sync(kFullMask, dead)) {
        const size_t idx = (size_t)threadIdx.x * (n >> 5);
        for (int p = 0; p < peer.n; p++) {
            for (unsigned polls = 0; polls < peer.max_polls; polls++) {
                unsigned long long q;
                asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(q) : "l"(peer.y[p] + idx) : "memory");
                if (__all_sync(kFullMask, (unsigned)(q >> 32) == want)) break;
                if (globaltimer_ns() - t_start > kPeerWaitNs) break;
                __nanosleep(200);
            }
        }
    }
    __syncthreads();
}

// Fused input side for n = 1024*E (E = 4, 8, 16): a thread owns E consecutive values, everything up to the
// Walsh-Hadamard transform stays in registers (see fwht_regs), the result goes to xs in fragment order.
template <int E, bool TP>
__device__ __forceinline__ void fused_input_regs(const FusedIn &I, const PeerIn &peer, int n, uint4 *xs, float *buf, float *warp_sums) {
    // ownership of the E consecutive values a thread works on: tid*E ("A"), or, after one fwht_regs,
    // (lane*32 + warp)*E ("B").  The transform maps A to B and B to A, every other step is element-wise or
    // a sum over everything, so the deferred-producer path simply does its element-wise work in B.
    const bool use_peers = TP && peer.n > 0;
    const bool deferred = I.y_prev != nullptr || use_peers;
    const size_t jA = (size_t)threadIdx.x * E;
    const size_t jB = (size_t)((threadIdx.x & 31) * 32 + (threadIdx.x >> 5)) * E;
    const size_t j = deferred ? jB : jA;
    float v[E], rs[E], wn[E], gt[E], sg[E];
    // all operand vectors are requested before any is used
    if (use_peers) {
        const unsigned want = *reinterpret_cast<const volatile unsigned *>(peer.seq);
        // A wait that ran out in an EARLIER launch (a lost or desynchronised GPU) leaves *status set: every later
        // launch then reads once and goes on instead of spinning again, so a dead peer costs one bounded wait in
        // total, not one per launch.  The host reads the word and stops or falls back.
        const bool dead = *reinterpret_cast<const volatile unsigned *>(peer.status) != 0u;
        const unsigned long long t_start = globaltimer_ns();
        await_samples(peer, n, want, t_start, dead);
        // A warp reads, checks and - for stragglers - retries as a unit: the loop is uniform over the warp (vote), so
        // no lane ever spins on its own while its warp waits for it, and it ends after max_polls rounds or
        // kPeerWaitNs at the latest.
        bool ok;
        for (unsigned round = 0;; round++) {
            ok = loadE_stamped<E>(peer.y[0], jA, want, v);
            for (int p = 1; p < peer.n; p++) {      // same order on every GPU: the sums are bit-identical
                float t[E];
                ok = loadE_stamped<E>(peer.y[p], jA, want, t) && ok;
#pragma unroll
                for (int k = 0; k < E; k++) v[k] += t[k];
            }
            if (__all_sync(kFullMask, ok || dead) || round >= peer.max_polls) break;
            if (__any_sync(kFullMask, globaltimer_ns() - t_start > kPeerWaitNs)) break;
            __nanosleep(200);
        }
        if (!ok) atomicOr(peer.status, 1u);
    } else if (deferred) loadE_f32<E>(I.y_prev, jA, v, true);
    else loadE_f16<E>(I.x_raw, j, v);
    if (I.residual) loadE_f16<E>(I.residual, j, rs);
    if (I.norm_weight) loadE_f16<E>(I.norm_weight, j, wn);
    if (I.gate) loadE_f16<E>(I.gate, j, gt);
    if (I.sign_in) loadE_f16<E>(I.sign_in, j, sg);
    if (deferred) {
        float ps[E];
        if (I.prev_sign) loadE_f32<E>(I.prev_sign, jB, ps, false);
        fwht_regs<E>(v, buf);
#pragma unroll
        for (int k = 0; k < E; k++) {
            v[k] *= I.prev_scale;
            if (I.prev_sign) v[k] *= ps[k];
            v[k] = __half2float(__float2half_rn(v[k]));      // the producer's output is an fp16 tensor
        }
        __syncthreads();                                       // buf is used again below
    }
    if (I.residual) {
#pragma unroll
        for (int k = 0; k < E; k++) v[k] = __half2float(__float2half_rn(v[k] + rs[k]));   // fp16 residual stream
        if (I.residual_out && blockIdx.x == 0) storeE_f16<E>(I.residual_out, j, v);
    }
    if (I.norm_weight) {
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < E; k++) ss += v[k] * v[k];
        const float r = rsqrtf(block_sum(ss, warp_sums) / (float)n + I.eps);
#pragma unroll
        for (int k = 0; k < E; k++) v[k] = __half2float(__hmul(__float2half_rn(wn[k]), __float2half_rn(v[k] * r)));  // LlamaRMSNorm
    }
#pragma unroll
    for (int k = 0; k < E; k++) {
        if (I.gate) v[k] = swiglu_fp16(gt[k], v[k]);
        if (I.sign_in) v[k] *= sg[k];
    }
    fwht_regs<E>(v, buf);
    const int i0 = (int)(deferred ? jA : jB);                  // ownership after the transform
#pragma unroll
    for (int k = 0; k < E; k += 2) {
        const int wi = (i0 + k) >> 1, blk = wi >> 4, w = wi & 15;   // 16 words per 32-column block
        reinterpret_cast<__half2 *>(xs)[blk * 16 + (w & 3) * 4 + (w >> 2)] = __floats2half2_rn(v[k] * I.scale, v[k + 1] * I.scale);
    }
}

// Fused output side for m = 1024*E, run by the CTA that finished last.
template <int E>
__device__ __forceinline__ void fused_output_regs(const FusedOut &O, const float *out, int m, int bs, float *buf) {
    const size_t j = (size_t)threadIdx.x * E;
    const size_t i0 = (size_t)((threadIdx.x & 31) * 32 + (threadIdx.x >> 5)) * E;   // ownership after the transform
    float sg[E];
    if (O.sign_out) loadE_f32<E>(O.sign_out, i0, sg, false);
    for (int b = 0; b < bs; b++) {
        float v[E];
        loadE_f32<E>(out + (size_t)b * m, j, v, true);
        fwht_regs<E>(v, buf);
#pragma unroll
        for (int k = 0; k < E; k++) {
            v[k] *= O.scale;
            if (O.sign_out) v[k] *= sg[k];
        }
        if (O.dtype == QTIP_F16) storeE_f16<E>(static_cast<__half *>(O.final), (size_t)b * m + i0, v);
        else storeE_f32<E>(static_cast<float *>(O.final), (size_t)b * m + i0, v);
        __syncthreads();
    }
}

// XS: x is staged once per CTA in shared memory, permuted so that a lane's four B-fragment words of
// a block are one 16-byte load; otherwise they are read from global memory (L1-resident) per block.
// db: the cross-warp reduction buffer is double-buffered, which drops one CTA barrier per segment.
// blockIdx.y selects the problem of the batch (all problems have the same m, n, K, bs).
// TP: the tensor-parallel fields (PeerIn / Signal) are live; the single-GPU instantiation carries none of that code.
// NW: warps per CTA (32: the register transforms of the fused sides are written for 1024 threads).
// C:  blocks per bulk copy; xs_offset: byte offset of the staged x in shared memory (the host fits the ring, the
// reduction buffers, x and the scratch of the fused input side into 227 KiB and picks C accordingly).
template <int K, bool XS, bool TP, int NW, int C>
__global__ void __launch_bounds__(NW * 32, 1)
    matvec_hyb_kernel(const __grid_constant__ MatvecBatch batch, int m, int n, int bs, int kmax, int mode, int db,
                      int xs_offset, int scratch_offset) {
    constexpr int kBlockBytes = 128 * K;
    constexpr int chunk_blocks = C;
    const bool DB = db != 0;
    constexpr int kConsumerWarps = NW, kThreads = NW * 32;     // shadow the file-scope defaults
    constexpr int kWarpShift = NW == 32 ? 5 : 4;
    static_assert(NW == 32 || NW == 16, "a segment is split over 16 or 32 warps");
    extern __shared__ __align__(128) uint8_t smem[];
    // layout: control block (incl. two mbarriers per warp) | LUT | ring slot 0 [NW][chunk] | ring slot 1 [NW][chunk] |
    //         reduction buffer(s) [NW][bs][32] fp32 | (padding) | x (bs, n) fp16 permuted
    // The fp32 scratch of the fused input transform lies behind x when everything fits (scratch_offset > 0); otherwise
    // it overlays ring slot 1 and what follows it up to x, and slot 1 is first filled after the transform is done.
    const MatvecProblem &P = batch.p[blockIdx.y];
    float *__restrict__ out = P.out;
    const uint8_t *__restrict__ codes = P.codes;
    const __half *__restrict__ x = P.x;
    const uint32_t *__restrict__ tlut = P.tlut;
    Shared *sh = reinterpret_cast<Shared *>(smem);
    uint32_t *lut = reinterpret_cast<uint32_t *>(smem + kCtrlBytes);
    const int slot_bytes = chunk_blocks * kBlockBytes;             // per warp
    uint8_t *ring = smem + kCtrlBytes + kLutBytes;
    const int red_floats = kConsumerWarps * 32 * bs;
    float *red = reinterpret_cast<float *>(ring + 2 * NW * slot_bytes);
    (void)chunk_blocks;
    uint4 *xs = reinterpret_cast<uint4 *>(smem + xs_offset);
    float *fscratch = reinterpret_cast<float *>(scratch_offset > 0 ? smem + scratch_offset : ring + NW * slot_bytes);

    unsigned *counters = reinterpret_cast<unsigned *>(P.workspace);
    unsigned *done_counter = reinterpret_cast<unsigned *>(P.workspace + kCounterBytes);
    float *partial = reinterpret_cast<float *>(P.workspace + kPartialOffset);

    const int nb = n >> 5, mb = m >> 5;
    const int G = gridDim.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // Segment bookkeeping in 32-bit block indices (B = mb*nb < 2^30 is checked by the host).
    // rows mode: segments are whole row blocks c, c+G, ...; stream-K: [r0, r1) cut at row boundaries.  Both are
    // "the part of row block M from pos up to min(end, (M+1)*nb), then on to row block M + mstep at seg_end + gap",
    // so the loops below carry no mode branches and no divisions.
    const int B = mb * nb;
    int pos, end, M, mstep, gap;
    if (mode == kModeRows) { pos = blockIdx.x * nb; end = B; M = blockIdx.x; mstep = G; gap = (G - 1) * nb; }
    else {
        pos = (int)range_start(blockIdx.x, B, G); end = (int)range_start(blockIdx.x + 1, B, G);
        M = pos / nb; mstep = 1; gap = 0;
    }
    // warp w's run of a segment [p, e): an even split of its blocks, contiguous in memory
    auto run_of = [&](int p, int e, int &r0, int &r1) {
        const int cnt = e - p;
        r0 = p + ((warp * cnt) >> kWarpShift);
        r1 = p + (((warp + 1) * cnt) >> kWarpShift);
    };
    int seg_end = min(end, (M + 1) * nb);

    // The ring of this warp: slot s at ring + (s*NW + warp)*slot_bytes, its barrier at bar_w + 8s.
    const uint32_t ring_w = smem_u32(ring) + warp * slot_bytes;
    const uint32_t slot_stride = NW * slot_bytes;
    const uint32_t bar_w = smem_u32(smem + kBarOffset) + warp * 16;
    if (lane == 0) { mbar_init(bar_w, 1); mbar_init(bar_w + 8, 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncwarp();
    // Issue cursor: walks this warp's chunks (over all segments of the CTA, in order) one or two chunks ahead of
    // the decoding; uniform over the warp, lane 0 issues the copy.
    int i_M = M, i_seg_end = seg_end, i_blk = 0, i_run_end = 0;
    bool i_valid = pos < end;
    unsigned ichunk = 0;
    if (i_valid) run_of(pos, i_seg_end, i_blk, i_run_end);
    auto issue = [&]() {
        while (i_valid && i_blk >= i_run_end) {
            const int i_pos = i_seg_end + gap;
            i_M += mstep;
            if (i_pos >= end) { i_valid = false; break; }
            i_seg_end = min(end, (i_M + 1) * nb);
            run_of(i_pos, i_seg_end, i_blk, i_run_end);
        }
        if (!i_valid) return;
        const int nblk = min(chunk_blocks, i_run_end - i_blk);
        if (lane == 0)
            bulk_load(ring_w + (ichunk & 1u) * slot_stride, codes + (size_t)i_blk * kBlockBytes, (uint32_t)(nblk * kBlockBytes),
                      bar_w + (ichunk & 1u) * 8);
        i_blk += nblk;
        ichunk++;
    };
    // First chunk of this warp: packed codes are weights, so the copy starts before the table build and before
    // waiting for the previous kernel of the stream.
    issue();
    if (scratch_offset > 0) issue();      // ring slot 1 is free from the start: second chunk in flight as well
    if (threadIdx.x == 0) sh->is_last = 0;
    // lane-private LUT copies: entry e = sign << 9 | index, copy l at byte e*128 + l*4; the sign bit
    // flips the sign of the first (low) half of the pair.  Thread t writes the 16-byte groups t, t + kThreads, ...:
    // the LUT words it needs are requested first, then stored.
    {
        constexpr int kGroupsPerThread = 1024 * 8 / kThreads;     // 8 (or 16)
        uint32_t tl[kGroupsPerThread / 2];
#pragma unroll
        for (int j = 0; j < kGroupsPerThread / 2; j++) tl[j] = __ldg(tlut + (((threadIdx.x + kThreads * j) >> 3) & 511));
#pragma unroll
        for (int j = 0; j < kGroupsPerThread; j++) {
            // group i = t + kThreads*j: entry (i >> 3) & 511, sign bit i >> 12 (= j / (kGroupsPerThread/2))
            const uint32_t e = tl[j % (kGroupsPerThread / 2)] ^ ((uint32_t)(j / (kGroupsPerThread / 2)) << 15);
            reinterpret_cast<uint4 *>(lut)[threadIdx.x + kThreads * j] = make_uint4(e, e, e, e);
        }
    }
    grid_launch_dependents();  // the next kernel of the stream may start its own weight-only prologue
    grid_dependency_wait();    // x, out and the workspace belong to the stream's data flow
    // tensor parallelism: the stamp of this launch's result values (every CTA reads the counter before any CTA can
    // have taken its exit ticket, and only the last ticket holder advances it)
    unsigned stamp = 0u;
    if constexpr (TP) stamp = P.sig.seq ? *reinterpret_cast<const volatile unsigned *>(P.sig.seq) + 1u : 0u;
    if constexpr (XS) {
        // xs[(b*nb + N)*4 + t] = { x[b][32N+2t..+1], x[..+8..], x[..+16..], x[..+24..] }
        if (NW == 32 && (P.in.x_raw || P.in.y_prev || (TP && P.peer.n > 0))) {
            // fused input side (bs == 1, n a power of two): every CTA transforms the activation itself.
            // A thread owns 8 consecutive values; the loads of all operand vectors are issued together so
            // the whole prologue costs one L2 round trip, not one per array.
            const FusedIn &I = P.in;
#ifndef QTIP_PROLOGUE_SMEM
            if (NW == 32 && n == 4096) fused_input_regs<4, TP>(I, P.peer, n, xs, fscratch, sh->warp_sums);
            else if (NW == 32 && n == 8192) fused_input_regs<8, TP>(I, P.peer, n, xs, fscratch, sh->warp_sums);
            else
#endif
            {
            const int nvec = n >> 3;
            int p = 0;
            while ((1 << p) < n) p++;
            const bool use_peers = TP && P.peer.n > 0;
            const bool deferred = I.y_prev != nullptr || use_peers;
            if (deferred) {
                // the producer's raw result (or the sum of the GPUs' partial results) -> scratch -> transform; its
                // sign, scale and fp16 rounding are applied when the values are picked up below
                if (use_peers) {
                    const unsigned want = *reinterpret_cast<const volatile unsigned *>(P.peer.seq);
                    const bool dead = *reinterpret_cast<const volatile unsigned *>(P.peer.status) != 0u;
                    const unsigned long long t_start = globaltimer_ns();
                    await_samples(P.peer, n, want, t_start, dead);
                    for (int vi = threadIdx.x; vi < nvec; vi += kThreads) {      // trip counts are uniform per warp
                        const size_t j = (size_t)vi * 8;
                        float v[8];
                        bool ok;
                        for (unsigned round = 0;; round++) {
                            ok = loadE_stamped<8>(P.peer.y[0], j, want, v);
                            for (int q = 1; q < P.peer.n; q++) {
                                float t8[8];
                                ok = loadE_stamped<8>(P.peer.y[q], j, want, t8) && ok;
#pragma unroll
                                for (int k = 0; k < 8; k++) v[k] += t8[k];
                            }
                            if (__all_sync(kFullMask, ok || dead) || round >= P.peer.max_polls) break;
                            if (__any_sync(kFullMask, globaltimer_ns() - t_start > kPeerWaitNs)) break;
                            __nanosleep(200);
                        }
                        if (!ok) atomicOr(P.peer.status, 1u);
#pragma unroll
                        for (int k = 0; k < 8; k++) fscratch[pad((int)j + k)] = v[k];
                    }
                } else {
                    for (int vi = threadIdx.x; vi < nvec; vi += kThreads) {
                        const size_t j = (size_t)vi * 8;
                        float v[8];
                        loadE_f32<8>(I.y_prev, j, v, true);
#pragma unroll
                        for (int k = 0; k < 8; k++) fscratch[pad((int)j + k)] = v[k];
                    }
                }
                __syncthreads();
                fwht_shared(fscratch, n, p);
            }
            float ss = 0.f;
            for (int vi = threadIdx.x; vi < nvec; vi += kThreads) {
                const size_t j = (size_t)vi * 8;
                float v[8], rs[8], gt[8], sg[8];
                if (deferred) {
                    float ps[8];
                    if (I.prev_sign) load8_f32(I.prev_sign, j, ps);
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        float y = fscratch[pad((int)j + k)] * I.prev_scale;
                        if (I.prev_sign) y *= ps[k];
                        v[k] = __half2float(__float2half_rn(y));      // the producer's output is an fp16 tensor
                    }
                } else load8_f16(I.x_raw, j, v);
                if (I.residual) load8_f16(I.residual, j, rs);
                if (I.gate && !I.norm_weight) load8_f16(I.gate, j, gt);
                if (I.sign_in && !I.norm_weight) load8_f16(I.sign_in, j, sg);
                if (I.residual) {
#pragma unroll
                    for (int k = 0; k < 8; k++) v[k] = __half2float(__float2half_rn(v[k] + rs[k]));   // fp16 residual stream
                    if (I.residual_out && blockIdx.x == 0) store8_f16(I.residual_out, j, v);
                }
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    ss += v[k] * v[k];
                    // without a norm everything can be applied right away; with one the weight is folded in now
                    // and the common factor r after the reduction: w * fp16(v * r) needs r first, so stash v
                    if (!I.norm_weight) {
                        if (I.gate) v[k] = swiglu_fp16(gt[k], v[k]);
                        if (I.sign_in) v[k] *= sg[k];
                    }
                    fscratch[pad((int)j + k)] = v[k];
                }
            }
            if (I.norm_weight) {
                const float r = rsqrtf(block_sum(ss, sh->warp_sums) / (float)n + I.eps);
                for (int vi = threadIdx.x; vi < nvec; vi += kThreads) {   // each thread revisits its own values
                    const size_t j = (size_t)vi * 8;
                    float w[8], gt[8], sg[8];
                    load8_f16(I.norm_weight, j, w);
                    if (I.gate) load8_f16(I.gate, j, gt);
                    if (I.sign_in) load8_f16(I.sign_in, j, sg);
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        float v = fscratch[pad((int)j + k)];
                        v = __half2float(__hmul(__float2half_rn(w[k]), __float2half_rn(v * r)));   // LlamaRMSNorm
                        if (I.gate) v = swiglu_fp16(gt[k], v);
                        if (I.sign_in) v *= sg[k];
                        fscratch[pad((int)j + k)] = v;
                    }
                }
            }
            __syncthreads();
            fwht_shared(fscratch, n, p);
            for (int i = threadIdx.x; i < (n >> 1); i += kThreads) {
                const int blk = i >> 4, w = i & 15;
                const __half2 h = __floats2half2_rn(fscratch[pad(2 * i)] * I.scale, fscratch[pad(2 * i + 1)] * I.scale);
                reinterpret_cast<__half2 *>(xs)[blk * 16 + (w & 3) * 4 + (w >> 2)] = h;
            }
            }
        } else {
            // 4 words (8 values) per thread and trip
            const uint4 *xw = reinterpret_cast<const uint4 *>(x);
            const int quads = bs * (n >> 3);
            for (int i = threadIdx.x; i < quads; i += kThreads) {
                const uint4 q = __ldg(xw + i);
                const uint32_t wv[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const int wi = i * 4 + k, blk = wi >> 4, w = wi & 15;   // 16 words per 32-column block
                    reinterpret_cast<uint32_t *>(xs)[blk * 16 + (w & 3) * 4 + (w >> 2)] = wv[k];
                }
            }
        }
    }
    __syncthreads();
    if (scratch_offset <= 0) issue();   // second chunk: ring slot 1 (the scratch of the fused input side lay over it until now)

    const int g = lane >> 2, t = lane & 3;
    const int xg = g < bs ? g : 0;  // lanes of unused batch columns alias row 0; their results are never stored
    const uint32_t *xrow = reinterpret_cast<const uint32_t *>(x + (size_t)xg * n + 2 * t);
    const uint32_t xsrow = smem_u32(xs) + (uint32_t)(xg * nb * 4 + t) * 16u;   // shared-memory address of this lane's fragments
    const uint32_t lut_lane = smem_u32(lut) + lane * 4;
    const uint32_t own_off = lane * (4 * K), nxt_off = ((lane + 1) & 31) * (4 * K);   // lane 31 wraps to lane 0: tail-biting

    uint32_t segno = 0;
    unsigned cchunk = 0;       // chunks consumed so far: slot cchunk & 1, barrier phase (cchunk >> 1) & 1
    bool ring_dead = false;    // a wait ran out: stop waiting (the results are meaningless, the kernel terminates)
    while (pos < end) {
        int r0, r1;
        run_of(pos, seg_end, r0, r1);
        const int row0 = M * nb;
        float acc[2][4] = {};
        uint32_t xsp = xsrow + (uint32_t)(r0 - row0) * 64u;    // x fragments of the block being decoded (64 bytes per block)
        const uint32_t *xgp = xrow + 16 * (r0 - row0);
        for (int blk = r0; blk < r1; blk += C) {
            const int nblk = min(C, r1 - blk);
            const uint32_t slot = ring_w + (cchunk & 1u) * slot_stride;
            if (!ring_dead) {
                const uint32_t bar = bar_w + (cchunk & 1u) * 8, parity = (cchunk >> 1) & 1u;
                unsigned spins = 0;
                while (!mbar_try_wait(bar, parity)) {
                    if (++spins > kRingSpinLimit) {
                        ring_dead = true;
                        if (lane == 0) atomicOr(done_counter + 1, 1u);
                        break;
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < C; i++) {
                if (i < nblk) {
                    const LaneCodes<K> own = lds_lane_codes<K>(slot + i * kBlockBytes + own_off);
                    const LaneCodes<K> nxt = lds_lane_codes<K>(slot + i * kBlockBytes + nxt_off);
                    uint32_t xb[4];
                    if constexpr (XS) {
                        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(xb[0]), "=r"(xb[1]), "=r"(xb[2]), "=r"(xb[3]) : "r"(xsp + i * 64));
                    }
                    else { const uint32_t *xp = xgp + 16 * i; xb[0] = __ldg(xp); xb[1] = __ldg(xp + 4); xb[2] = __ldg(xp + 8); xb[3] = __ldg(xp + 12); }
                    decode_block<K>(own, nxt, xb, acc, lut_lane);
                }
            }
            if constexpr (XS) xsp += C * 64;
            else xgp += C * 16;
            __syncwarp();      // every lane has read the slot before it is filled again
            issue();
            cchunk++;
        }
        // a segment that covers its whole row block has no other contributor (true for every segment in rows mode)
        const bool whole = pos == row0 && seg_end - pos == nb;
        finish_segment<kConsumerWarps>(acc, DB ? red + (segno & 1) * red_floats : red, sh, out, partial, counters, M, nb,
                                       (long)B, G, kmax, m, bs, whole, !DB, TP ? P.sig.copies : OutCopies{}, stamp);
        segno++;
        pos = seg_end + gap;
        M += mstep;
        seg_end = min(end, (M + 1) * nb);
    }

    if (TP && P.sig.seq) {
        // row-parallel partial result: the values are already on their way to every GPU (stamped); the CTA that
        // finishes last advances the sequence counter that the stamps of the next launch are derived from
        __syncthreads();
        if (threadIdx.x == 0) {
            if (atomicAdd(done_counter, 1u) == gridDim.x - 1) {
                *P.sig.seq = stamp;
                *done_counter = 0;
            }
        }
    } else if (NW == 32 && P.ep.final) {
        // fused output side (m a power of two): the CTA that finishes last transforms the whole result
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) sh->is_last = (atomicAdd(done_counter, 1u) == gridDim.x - 1);
        __syncthreads();
        if (sh->is_last) {
            __threadfence();
            float *f = reinterpret_cast<float *>(lut);   // the table is no longer needed
            if (m == 4096) fused_output_regs<4>(P.ep, out, m, bs, f);
            else if (m == 8192) fused_output_regs<8>(P.ep, out, m, bs, f);
            else if (m == 16384) fused_output_regs<16>(P.ep, out, m, bs, f);
            else {
            int p = 0;
            while ((1 << p) < m) p++;
            const int mvec = m >> 3;
            // sign_out of this thread's first vector, requested together with the first y loads
            float sg0[8];
            if (P.ep.sign_out && threadIdx.x < mvec) load8_f32(P.ep.sign_out, (size_t)threadIdx.x * 8, sg0);
            for (int b = 0; b < bs; b++) {
                for (int vi = threadIdx.x; vi < mvec; vi += kThreads) {
                    const float4 *src = reinterpret_cast<const float4 *>(out + (size_t)b * m + (size_t)vi * 8);
                    const float4 a = __ldcg(src), c = __ldcg(src + 1);
                    const int j = vi * 8;
                    f[pad(j)] = a.x; f[pad(j + 1)] = a.y; f[pad(j + 2)] = a.z; f[pad(j + 3)] = a.w;
                    f[pad(j + 4)] = c.x; f[pad(j + 5)] = c.y; f[pad(j + 6)] = c.z; f[pad(j + 7)] = c.w;
                }
                __syncthreads();
                fwht_shared(f, m, p);
                for (int vi = threadIdx.x; vi < mvec; vi += kThreads) {
                    const size_t j = (size_t)vi * 8;
                    float y[8], sg[8];
                    if (P.ep.sign_out && vi != (int)threadIdx.x) load8_f32(P.ep.sign_out, j, sg);
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        y[k] = f[pad((int)j + k)] * P.ep.scale;
                        if (P.ep.sign_out) y[k] *= (vi == (int)threadIdx.x) ? sg0[k] : sg[k];
                    }
                    if (P.ep.dtype == QTIP_F16) store8_f16(static_cast<__half *>(P.ep.final), (size_t)b * m + j, y);
                    else store8_f32(static_cast<float *>(P.ep.final), (size_t)b * m + j, y);
                }
                __syncthreads();
            }
            }
            if (threadIdx.x == 0) *done_counter = 0;  // leave the workspace ready for the next call
        }
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
__device__ __forceinline__ uint32_t decode_pair(uint32_t s0, uint32_t s1, const __half *mad_tab) {
    __half lo, hi;
    if constexpr (CODE == QTIP_CODE_3INST) { lo = decode_3inst(s0 & 0xFFFFu); hi = decode_3inst(s1 & 0xFFFFu); }
    else { lo = decode_1mad_tab(s0 & 0xFFFFu, mad_tab); hi = decode_1mad_tab(s1 & 0xFFFFu, mad_tab); }
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
    __shared__ __half mad_tab[CODE == QTIP_CODE_1MAD ? kMadTableEntries : 1];
    if constexpr (CODE == QTIP_CODE_1MAD) {
        build_1mad_table(mad_tab);
        __syncthreads();
    }
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
                    a[hr] = decode_pair<CODE>(s0, s1, mad_tab);       // a0 / a1: fragment cols 2t, 2t+1
                    a[2 + hr] = decode_pair<CODE>(s2, s3, mad_tab);   // a2 / a3: fragment cols 2t+8, 2t+9
                }
                mma_16816(acc[ms], a, b0, b1);
            }
        }
        finish_segment<kPlainWarps>(acc, red, sh, out, partial, counters, M, nb, B, G, kmax, m, bs, mode == kModeRows, true,
                                    OutCopies{}, 0u);
    }
}

int check_common(const void *out, const void *codes, const void *x, int K, int m, int n, int bs, void *workspace,
                 size_t workspace_bytes) {
    if (!out || !codes || !x || K < 2 || K > 4 || bs < 1 || bs > kMaxBatch) return QTIP_ERR_BAD_ARG;
    if (m <= 0 || n <= 0 || (m & 31) || (n & 31) || (size_t)(m >> 5) * 4 > kCounterBytes) return QTIP_ERR_BAD_SHAPE;
    if ((long)(m >> 5) * (n >> 5) >= (1L << 30)) return QTIP_ERR_BAD_SHAPE;  // block indices are 32-bit
    if (!workspace || workspace_bytes < qtip_matvec_workspace_bytes(m, n, bs)) return QTIP_ERR_WORKSPACE;
    if (!aligned(workspace, 256) || !aligned(codes, 16) || !aligned(x, 16) || !aligned(out, 4)) return QTIP_ERR_ALIGNMENT;
    return QTIP_OK;
}

struct SmemPlan {
    int chunk_blocks, xs_offset, total, db, scratch_offset;
};

template <int K, bool XS, bool TP, int NW, int C>
int launch_hyb_variant_tp(const MatvecBatch &batch, int nprob, int m, int n, int bs, const SmemPlan &plan, cudaStream_t s) {
    static bool attr_set[64] = {};
    static std::mutex attr_mutex;
    int dev = 0;
    QTIP_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return QTIP_ERR_BAD_ARG;
    {
        std::lock_guard<std::mutex> lock(attr_mutex);
        if (!attr_set[dev]) {
            QTIP_CUDA_TRY(cudaFuncSetAttribute(matvec_hyb_kernel<K, XS, TP, NW, C>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               kSmemLimit));
            attr_set[dev] = true;
        }
    }
    const Partition p = make_partition(m, n, K, nprob);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.grid, nprob);
    cfg.blockDim = dim3(NW * 32);
    cfg.dynamicSmemBytes = plan.total;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    QTIP_CUDA_TRY(cudaLaunchKernelEx(&cfg, matvec_hyb_kernel<K, XS, TP, NW, C>, batch, m, n, bs, p.kmax, p.mode, plan.db,
                                     plan.xs_offset, plan.scratch_offset));
    return check_launch();
}

template <int K, bool XS, int C>
int launch_hyb_variant_c(const MatvecBatch &batch, int nprob, int m, int n, int bs, const SmemPlan &plan, cudaStream_t s) {
    bool tp = false;
    for (int i = 0; i < nprob; i++) {
        const MatvecProblem &q = batch.p[i];
        tp = tp || q.peer.n > 0 || q.sig.seq != nullptr;
    }
    if (tp) return launch_hyb_variant_tp<K, XS, true, 32, C>(batch, nprob, m, n, bs, plan, s);
    return launch_hyb_variant_tp<K, XS, false, 32, C>(batch, nprob, m, n, bs, plan, s);
}

template <int K, bool XS>
int launch_hyb_variant(const MatvecBatch &batch, int nprob, int m, int n, int bs, const SmemPlan &plan, cudaStream_t s) {
    constexpr int kMaxC = kMaxChunkBytes / (128 * K);      // 4 for K = 2, 2 for K = 3 and 4
    if constexpr (kMaxC >= 4) {
        if (plan.chunk_blocks >= 4) return launch_hyb_variant_c<K, XS, 4>(batch, nprob, m, n, bs, plan, s);
    }
    if (plan.chunk_blocks >= 2) return launch_hyb_variant_c<K, XS, 2>(batch, nprob, m, n, bs, plan, s);
    return launch_hyb_variant_c<K, XS, 1>(batch, nprob, m, n, bs, plan, s);
}

// Fit ring, reduction buffer(s), x and the scratch of the fused input side into the shared memory left beside
// the table.  Returns false if not even a one-block ring fits.
template <int K>
bool plan_smem(int n, int bs, bool xs, bool db, bool fused_in, SmemPlan &plan) {
    constexpr int NW = kConsumerWarps, BB = 128 * K;
    const int red_bytes = (db ? 2 : 1) * NW * 32 * bs * (int)sizeof(float);
    const int x_bytes = xs ? bs * n * 2 : 0;
    // fwht_shared wants n + n/32 + 8 floats, fwht_regs 32 rows of n/32 + 4
    const int scratch_bytes = fused_in ? (n + (n >> 5) + 136) * (int)sizeof(float) : 0;
    const int avail = kSmemLimit - kCtrlBytes - kLutBytes;
    plan.db = db ? 1 : 0;
    plan.scratch_offset = 0;
    for (int c = kMaxChunkBytes / BB; c >= 1; c >>= 1) {          // 4, 2, 1: the instantiated chunk sizes
        const int slot = NW * c * BB;                                   // one ring slot, all warps
        if (2 * slot + red_bytes + x_bytes + scratch_bytes <= avail) {  // room for a scratch area of its own
            plan.chunk_blocks = c;
            plan.xs_offset = kCtrlBytes + kLutBytes + 2 * slot + red_bytes;
            plan.scratch_offset = scratch_bytes > 0 ? plan.xs_offset + x_bytes : 1;   // > 0: both ring slots usable at once
            plan.total = kCtrlBytes + kLutBytes + 2 * slot + red_bytes + x_bytes + scratch_bytes;
            if (plan.scratch_offset == 1) plan.scratch_offset = plan.xs_offset;       // no scratch needed: any offset > 0
            return true;
        }
        const int after_slot1 = slot + red_bytes;                       // bytes from slot 1 up to x
        const int pad = scratch_bytes > after_slot1 ? scratch_bytes - after_slot1 : 0;
        const int total = 2 * slot + red_bytes + pad + x_bytes;
        if (total <= avail) {
            plan.chunk_blocks = c;
            plan.xs_offset = kCtrlBytes + kLutBytes + 2 * slot + red_bytes + pad;
            plan.total = kCtrlBytes + kLutBytes + total;
            return true;
        }
    }
    return false;
}

// fused_in: the batch uses the fused input transform (needs x staged in shared memory plus fp32 scratch)
template <int K>
int launch_hyb_batch(const MatvecBatch &batch, int nprob, int m, int n, int bs, bool fused_in, cudaStream_t s) {
    // shared memory: control + table are fixed; then the ring, the reduction buffer(s) and, when it fits, x.
    // Preference: x staged and double-buffered reduction; then give up the second reduction buffer; then x.
    SmemPlan plan;
    if (plan_smem<K>(n, bs, true, true, fused_in, plan)) return launch_hyb_variant<K, true>(batch, nprob, m, n, bs, plan, s);
    if (plan_smem<K>(n, bs, true, false, fused_in, plan)) return launch_hyb_variant<K, true>(batch, nprob, m, n, bs, plan, s);
    if (fused_in) return QTIP_ERR_BAD_SHAPE;      // the fused input side leaves x in shared memory
    if (plan_smem<K>(n, bs, false, true, false, plan)) return launch_hyb_variant<K, false>(batch, nprob, m, n, bs, plan, s);
    if (plan_smem<K>(n, bs, false, false, false, plan)) return launch_hyb_variant<K, false>(batch, nprob, m, n, bs, plan, s);
    return QTIP_ERR_BAD_SHAPE;
}

template <int K>
int launch_hyb(float *out, const uint8_t *codes, const __half *x, const uint32_t *tlut, int m, int n, int bs,
               uint8_t *workspace, cudaStream_t s) {
    MatvecBatch batch = {};
    batch.p[0].out = out; batch.p[0].codes = codes; batch.p[0].x = x; batch.p[0].tlut = tlut;
    batch.p[0].workspace = workspace;
    return launch_hyb_batch<K>(batch, 1, m, n, bs, false, s);
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

// sizeof(qtip_linear_desc) followed by the byte offset of every field in declaration order: lets a foreign-language
// mirror of the struct (ctypes, cgo, JNA ...) prove at start-up that it agrees with the compiled library.  A mirror
// that is one field out of step turns a pointer's low bits into peer_max_polls or a count.
extern "C" int qtip_linear_desc_layout(size_t *out, int capacity) {
#define QTIP_F(f) offsetof(qtip_linear_desc, f)
    const size_t v[] = {sizeof(qtip_linear_desc), QTIP_F(y), QTIP_F(codes), QTIP_F(tlut), QTIP_F(x), QTIP_F(workspace),
                        QTIP_F(workspace_bytes), QTIP_F(in_raw), QTIP_F(residual), QTIP_F(residual_out), QTIP_F(norm_weight),
                        QTIP_F(gate), QTIP_F(sign_in), QTIP_F(in_scale), QTIP_F(eps), QTIP_F(out), QTIP_F(out_dtype),
                        QTIP_F(sign_out), QTIP_F(out_scale), QTIP_F(in_y), QTIP_F(in_y_sign), QTIP_F(in_y_scale),
                        QTIP_F(peer_count), QTIP_F(peer_y), QTIP_F(peer_seq), QTIP_F(peer_status), QTIP_F(peer_max_polls),
                        QTIP_F(signal_count), QTIP_F(signal_y), QTIP_F(signal_seq)};
#undef QTIP_F
    const int count = (int)(sizeof(v) / sizeof(v[0]));
    if (out)
        for (int i = 0; i < count && i < capacity; i++) out[i] = v[i];
    return count;
}

extern "C" int qtip_linear_fused(const qtip_linear_desc *descs, int count, int K, int m, int n, int bs, void *stream) {
    if (!descs || count < 1 || count > kMaxProblems) return QTIP_ERR_BAD_ARG;
    MatvecBatch batch = {};
    bool fused_in = false;
    for (int i = 0; i < count; i++) {
        const qtip_linear_desc &d = descs[i];
        if (!d.tlut) return QTIP_ERR_BAD_ARG;
        const bool fin = d.in_raw != nullptr || d.in_y != nullptr || d.peer_count > 0, fout = d.out != nullptr;
        if (i > 0 && fin != fused_in) return QTIP_ERR_BAD_ARG;   // all or none: the shared-memory layout is per launch
        fused_in = fin;
        const void *x = d.peer_count > 0 ? d.peer_y[0] : d.in_y ? (const void *)d.in_y : fin ? d.in_raw : d.x;
        int st = check_common(d.y, d.codes, x, K, m, n, bs, d.workspace, d.workspace_bytes);
        if (st != QTIP_OK) return st;
        if (!aligned(d.tlut, 4)) return QTIP_ERR_ALIGNMENT;
        if (fin && (bs != 1 || (n & (n - 1)) || n > 16384)) return QTIP_ERR_BAD_SHAPE;
        if (d.in_y && n != 4096 && n != 8192) return QTIP_ERR_BAD_SHAPE;
        if (fout && ((m & (m - 1)) || m > 16384)) return QTIP_ERR_BAD_SHAPE;
        if (fout && d.out_dtype != QTIP_F16 && d.out_dtype != QTIP_F32) return QTIP_ERR_BAD_ARG;
        {
            const void *vecs[] = {d.in_raw, d.residual, d.residual_out, d.norm_weight, d.gate, d.sign_in, d.out, d.sign_out,
                                  d.in_y, d.in_y_sign,
                                  (fin || fout) ? (const void *)d.y : nullptr};
            for (const void *q : vecs)
                if (q && !aligned(q, 16)) return QTIP_ERR_ALIGNMENT;
        }
        if (d.residual_out && (d.residual_out == d.in_raw || d.residual_out == d.residual)) return QTIP_ERR_BAD_ARG;
        for (int j = 0; j < i; j++)
            if (descs[j].workspace == d.workspace || descs[j].y == d.y) return QTIP_ERR_BAD_ARG;
        MatvecProblem &P = batch.p[i];
        P.out = d.y; P.codes = static_cast<const uint8_t *>(d.codes); P.x = static_cast<const __half *>(d.x);
        P.tlut = static_cast<const uint32_t *>(d.tlut); P.workspace = static_cast<uint8_t *>(d.workspace);
        if (fin) {
            P.in.x_raw = static_cast<const __half *>(d.in_raw); P.in.residual = static_cast<const __half *>(d.residual);
            P.in.residual_out = static_cast<__half *>(d.residual_out);
            P.in.norm_weight = static_cast<const __half *>(d.norm_weight); P.in.gate = static_cast<const __half *>(d.gate);
            P.in.sign_in = static_cast<const __half *>(d.sign_in); P.in.scale = d.in_scale; P.in.eps = d.eps;
            P.in.y_prev = d.in_y; P.in.prev_sign = d.in_y_sign; P.in.prev_scale = d.in_y_scale;
        }
        if (fout) { P.ep.final = d.out; P.ep.sign_out = d.sign_out; P.ep.scale = d.out_scale; P.ep.dtype = d.out_dtype; }
        if (d.peer_count > 0) {
            if (d.peer_count > kMaxPeers || !d.peer_seq || !d.peer_status || !fin) return QTIP_ERR_BAD_ARG;
            if (n != 4096 && n != 8192) return QTIP_ERR_BAD_SHAPE;
            for (int q = 0; q < d.peer_count; q++) {
                if (!d.peer_y[q] || !aligned(d.peer_y[q], 16)) return QTIP_ERR_BAD_ARG;
                P.peer.y[q] = static_cast<const uint2 *>(d.peer_y[q]);
            }
            P.peer.n = d.peer_count; P.peer.seq = d.peer_seq; P.peer.status = d.peer_status;
            P.peer.max_polls = d.peer_max_polls ? d.peer_max_polls : (1u << 20);
            P.in.prev_sign = d.in_y_sign; P.in.prev_scale = d.in_y_scale;
        }
        if (d.signal_count > 0) {
            if (d.signal_count > kMaxPeers || !d.signal_seq || fout) return QTIP_ERR_BAD_ARG;
            for (int q = 0; q < d.signal_count; q++) {
                if (!d.signal_y[q] || !aligned(d.signal_y[q], 16)) return QTIP_ERR_BAD_ARG;
                P.sig.copies.dst[q] = static_cast<uint2 *>(d.signal_y[q]);
            }
            P.sig.copies.n = d.signal_count; P.sig.seq = d.signal_seq;
        }
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (K == 2) return launch_hyb_batch<2>(batch, count, m, n, bs, fused_in, s);
    if (K == 3) return launch_hyb_batch<3>(batch, count, m, n, bs, fused_in, s);
    return launch_hyb_batch<4>(batch, count, m, n, bs, fused_in, s);
}

// ---- allocation-free variant ------------------------------------------------------------------------------
// Scratch (ticket counters + partial sums) of qtip_decompress_matvec_static: a fixed array in the
// library's device image.  Every GPU that loads the library carries these 4 MiB + 64.25 KiB until the
// process exits.  In host code the name below is only a stand-in for the symbol; the address a kernel
// can use comes from cudaGetSymbolAddress, looked up once per device.
namespace qtip {
namespace {
constexpr size_t kStaticScratchBytes = kPartialOffset + 4u * 1024u * 1024u;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
std::mutex g_static_scratch_mutex;
void *g_static_scratch_ptr[64] = {};
}  // namespace
}  // namespace qtip

extern "C" int qtip_decompress_matvec_static(float *out, const void *codes, const void *x, const void *tlut, int K,
                                             int m, int n, int bs, void *stream) {
    if (!tlut) return QTIP_ERR_BAD_ARG;
    if (m > 0 && n > 0 && !(m & 31) && !(n & 31) && qtip_matvec_workspace_bytes(m, n, bs) > kStaticScratchBytes)
        return QTIP_ERR_TOO_LARGE;
    int dev = 0;
    QTIP_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return QTIP_ERR_BAD_ARG;
    void *scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
        if (!g_static_scratch_ptr[dev]) {
            // first call on this device (it is the current one): resolve the device address of the array
            void *p = nullptr;
            QTIP_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
            g_static_scratch_ptr[dev] = p;
        }
        scratch = g_static_scratch_ptr[dev];
    }
    int st = check_common(out, codes, x, K, m, n, bs, scratch, kStaticScratchBytes);
    if (st != QTIP_OK) return st;
    if (!aligned(tlut, 4)) return QTIP_ERR_ALIGNMENT;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // the array keeps whatever the previous call (or an interrupted one) left: the ticket counters of the
    // row blocks this call uses must start at zero
    QTIP_CUDA_TRY(cudaMemsetAsync(scratch, 0, (size_t)(m >> 5) * sizeof(unsigned), s));
    auto *c = static_cast<const uint8_t *>(codes);
    auto *xh = static_cast<const __half *>(x);
    auto *t = static_cast<const uint32_t *>(tlut);
    auto *ws = static_cast<uint8_t *>(scratch);
    if (K == 2) return launch_hyb<2>(out, c, xh, t, m, n, bs, ws, s);
    if (K == 3) return launch_hyb<3>(out, c, xh, t, m, n, bs, ws, s);
    return launch_hyb<4>(out, c, xh, t, m, n, bs, ws, s);
}
