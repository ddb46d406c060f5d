// Decompress-GEMM for batches 9..128 on the 5th-generation tensor cores (tcgen05 + TMEM).
//
//   out (bs, m) fp32 = X (bs, n) fp16 @ decode(codes)^T        HYB code, kernel layout
//
// One CTA owns 128 output rows (four 32-row blocks) and a contiguous range of input columns.  The
// weights are the A operand: D[128 x N] += A[128 x 16] * B[16 x N] with D in tensor memory, A and B
// in shared memory, K-major, 128-byte swizzle; N = batch rounded up to 16.
//   * 24 decode warps turn packed codes into fp16 and store them straight into the swizzled A tile
//     of a ring stage (128 rows x 64 columns = 8 tile blocks, one per warp; three stages are
//     filled concurrently).  The stores of a warp hit 32 distinct banks.  The same warps copy the 64-column
//     slice of X into the B tile of the stage.
//   * one thread issues four tcgen05.mma (K = 16 each) per stage and commits them to the stage's
//     "empty" barrier; a last commit signals the epilogue.
//   * warps 0-3 read the accumulator with tcgen05.ld (warp w owns TMEM lanes 32w..32w+31 = rows) and
//     write out (coalesced along rows); with a 2-way column split the two CTAs of a row range add
//     into a zeroed output (two addends: order-independent, so still deterministic).
// The compute codes (3INST / 1MAD, V = 1, plain layout) use the same kernel with another producer: a lane decodes
// eight consecutive states of a tile row (44 stream bits) and stores the eight weights as ONE 16-byte chunk of the
// swizzled A tile; no table is built.  That path is bound by the per-weight arithmetic, not by the tensor pipe.
// This replaces decode-to-HBM + dense GEMM of BitshiftLinearKernelAG upstream
// (lib/codebook/bitshift.py:476-489), which writes and re-reads 16x the packed bytes at 2 bits.
//
// Only the decode is expensive (one table lookup + one shared-memory store per state); the MMA work
// is negligible below batch 256, so the kernel runs at roughly the speed of the batch-1 matvec.
//
// Every mbarrier wait is bounded: after kSpinLimit polls the waiter records an error code in
// `status`, raises a CTA-wide abort flag that makes every later wait fall through, and the kernel
// still runs to its end, frees its tensor memory and returns (with meaningless results).
#include <mutex>

#include "common.cuh"

namespace qtip {
namespace {

constexpr int kGroups = 3;                               // groups of 8 decode warps; a group fills one stage
constexpr int kDecodeWarps = 8 * kGroups;
constexpr int kGemmThreads = (kDecodeWarps + 1) * 32;   // + one control warp (TMEM allocation, MMA issue)
constexpr int kStages = 4;                              // ring stages for batches up to 64; 3 for 65..128 (shared memory)
constexpr int kRows = 128;                               // output rows per CTA
constexpr int kStageCols = 64;                           // input columns per stage (128 bytes of fp16 per row)
constexpr int kAStageBytes = kRows * kStageCols * 2;     // 16 KiB
constexpr int kLut512Bytes = 1024 * 32 * 4;              // (512 entries + sign-flipped twins) x 32 lane-private copies
constexpr int kMaxN = 128;
constexpr unsigned kSpinLimit = 1u << 22;

struct GemmCtrl {
    unsigned long long full[kStages];
    unsigned long long empty[kStages];
    unsigned long long done;
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
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
// false: the wait gave up (its own limit, or another waiter raised the abort flag)
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, unsigned *status,
                                          unsigned code) {
    if (mbar_try_wait(bar, parity)) return true;
    for (unsigned spin = 0; spin < kSpinLimit; spin++) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    atomicCAS(status, 0u, code);
    return false;
}
// bounded wait that does not look at the abort flag (used before tensor memory is released)
__device__ __forceinline__ void mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    for (unsigned spin = 0; spin < kSpinLimit; spin++)
        if (mbar_try_wait(bar, parity)) return;
}

// Shared-memory matrix descriptor: K-major, 128-byte swizzle, rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);          // start address
    d |= (uint64_t)1 << 16;                            // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                  // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                            // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                            // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 48 stream bits of a plain-layout tile starting at bit pos (circular over the tile's 16K words), first bit at bit 47
__device__ __forceinline__ uint64_t plain_bits48(const uint16_t *__restrict__ words, int nwords, int pos) {
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

// STAGES: ring depth, 4 for batches up to 64 (B tile <= 8 KiB), 3 above (16 KiB B tiles); a compile-time value so that
// the ring arithmetic of the common case stays free of run-time divisions
template <int K, int CODE, int STAGES>
__global__ void __launch_bounds__(kGemmThreads, 1)
    decompress_gemm_kernel(float *__restrict__ out, const uint8_t *__restrict__ codes, const __half *__restrict__ x,
                           const uint32_t *__restrict__ tlut, int m, int n, int bs, int npad, int splitk,
                           unsigned *__restrict__ status) {
    constexpr int stages = STAGES;
    constexpr int kBlockBytes = 128 * K;
    constexpr bool kHyb = CODE == QTIP_CODE_HYB;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_addr(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                 // swizzled tiles need 1024-byte alignment
    uint8_t *smem = smem_raw + (base - raw);
    const int b_stage_bytes = npad * 128;
    // layout: A stages | B stages | LUT | control
    const uint32_t a_base = base, b_base = base + stages * kAStageBytes;
    uint32_t *lut = reinterpret_cast<uint32_t *>(smem + stages * (kAStageBytes + b_stage_bytes));
    GemmCtrl *ctl = reinterpret_cast<GemmCtrl *>(smem + stages * (kAStageBytes + b_stage_bytes) + kLut512Bytes);
    volatile int *abort_flag = &ctl->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tmem_cols = npad <= 32 ? 32 : (npad <= 64 ? 64 : 128);

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) {
            mbar_init(smem_addr(&ctl->full[s]), 8);     // eight decode warps fill a stage
            mbar_init(smem_addr(&ctl->empty[s]), 1);    // one tcgen05.commit frees it
        }
        mbar_init(smem_addr(&ctl->done), 1);
        ctl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kDecodeWarps) {
        // tensor memory for the accumulator: 128 lanes x tmem_cols 32-bit columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&ctl->tmem_base)),
                     "r"(tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // lane-private copies of the table: entry e = sign << 9 | index, copy l at byte e*128 + l*4; the sign bit of
    // the hash flips the first weight of the pair, so it is folded into the table (no per-state sign op)
    __half *mad_tab = reinterpret_cast<__half *>(lut);     // 1MAD: byte sum -> weight (the table area is otherwise unused)
    if constexpr (CODE == QTIP_CODE_1MAD) build_1mad_table(mad_tab);
    if constexpr (kHyb) {
        for (int i = threadIdx.x; i < 1024 * 8; i += kGemmThreads) {
            const uint32_t e = __ldg(tlut + ((i >> 3) & 511)) ^ ((uint32_t)(i >> 12) << 15);
            reinterpret_cast<uint4 *>(lut)[i] = make_uint4(e, e, e, e);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = ctl->tmem_base;

    const int nb = n >> 5;                                  // 32-column blocks per row block
    const int r0 = blockIdx.x * kRows;                      // first output row of this CTA
    const int cols_per_split = n / splitk;
    const int c0 = blockIdx.y * cols_per_split;             // first input column
    const int nsteps = cols_per_split / kStageCols;

    if (warp < kDecodeWarps) {
        // ---------------------------------- decode warps ------------------------------------------------
        const int group = warp >> 3;                        // this group fills steps group, group + kGroups, ...
        const int w8 = warp & 7, rb = w8 & 3, cb = w8 >> 2; // row block (of 4) and column block (of 2) of the stage
        const int a = lane >> 2, b = lane & 3;
        const uint32_t lut_lane = smem_addr(lut) + lane * 4;
        const uint8_t *src = codes + ((size_t)(r0 / 32 + rb) * nb + (c0 / 32 + cb)) * kBlockBytes + lane * (4 * K);
        // byte offset inside an A stage of this lane's element (ms, d, ks, c): row 32rb+16ms+8d+a, column 32cb+16ks+8c+2b
        const uint32_t row_off = (uint32_t)(4 * rb) * 1024u + (uint32_t)a * 128u + (uint32_t)b * 4u;
        const int tid8 = w8 * 32 + lane;                    // 0..255 within the stage's eight warps
        // The 64-column slice of x goes into the B tile of the stage: chunk ch of the tile = batch row ch >> 3, columns
        // 8*(ch & 7) .. +7, rows beyond bs zero.  Batches up to 64 (at most two 16-byte chunks per thread): the chunks of
        // the warp's NEXT step are requested into registers before the current step is decoded, so their latency hides
        // behind a step of work.  Larger batches: asynchronous copies straight into the tile (no registers), awaited
        // before the stage is handed over.
        const int chunks = npad * 8;
        constexpr bool small = STAGES == kStages;
        const bool has0 = small && tid8 < chunks, has1 = small && tid8 + 256 < chunks;
        auto load_x = [&](int step, int ch) -> uint4 {
            const int brow = ch >> 3, c = ch & 7;
            if (brow >= bs) return make_uint4(0u, 0u, 0u, 0u);
            return *reinterpret_cast<const uint4 *>(x + (size_t)brow * n + c0 + step * kStageCols + c * 8);
        };
        uint4 xv0_next = make_uint4(0u, 0u, 0u, 0u), xv1_next = xv0_next;
        // codes: two steps of this warp ahead (the warp's steps are kGroups apart)
        LaneCodes<K> own_next = {}, own_next2 = {};
        // plain layout (V = 1 codes): tile (tile row, tile column) = 16K words at ((row/16)*(n/16) + col/16)*16K; this
        // lane decodes row pr of each of the warp's four tiles, columns 8*ph .. 8*ph+7
        const uint16_t *pcodes = reinterpret_cast<const uint16_t *>(codes);
        const int tn = n >> 4, pr = lane >> 1, ph = lane & 1;
        if (group < nsteps) {
            if constexpr (kHyb) own_next = load_lane_codes<K>(src + (size_t)group * 2 * kBlockBytes);
            if (has0) xv0_next = load_x(group, tid8);
            if (has1) xv1_next = load_x(group, tid8 + 256);
        }
        if constexpr (kHyb)
            if (group + kGroups < nsteps) own_next2 = load_lane_codes<K>(src + (size_t)(group + kGroups) * 2 * kBlockBytes);
        // HYB: byte offsets of this lane's four 16-byte chunks (ks, c) inside a 128-byte row of the A tile, swizzled by
        // the row (row % 8 == a for every row this lane writes); rows (ms, d) are 1024-byte groups apart
        uint32_t chunk_off[4];
#pragma unroll
        for (int j = 0; j < 4; j++) chunk_off[j] = (((uint32_t)(4 * cb + j)) ^ (uint32_t)a) << 4;
        // ring position of this warp's step, kept incrementally (stages is a run-time value: no division in the loop)
        int s = group % stages, round = group / stages;
        for (int step = group; step < nsteps; step += kGroups) {
            const LaneCodes<K> own = own_next;
            const uint4 xv0 = xv0_next, xv1 = xv1_next;
            own_next = own_next2;
            if (step + kGroups < nsteps) {
                if (has0) xv0_next = load_x(step + kGroups, tid8);
                if (has1) xv1_next = load_x(step + kGroups, tid8 + 256);
            }
            if constexpr (kHyb)
                if (step + 2 * kGroups < nsteps) own_next2 = load_lane_codes<K>(src + (size_t)(step + 2 * kGroups) * 2 * kBlockBytes);
            // V = 1: the 44 bits this lane needs of each of its four tiles are requested before the wait for the stage
            uint64_t pbits[4];
            if constexpr (!kHyb) {
#pragma unroll
                for (int tt = 0; tt < 4; tt++) {
                    const int ks = tt >> 1, ms = tt & 1;
                    const size_t tile = (size_t)(r0 / 16 + 2 * rb + ms) * tn + (size_t)((c0 + step * kStageCols) / 16 + 2 * cb + ks);
                    pbits[tt] = plain_bits48(pcodes + tile * (16 * K), 16 * K, (pr * 16 + ph * 8) * K);
                }
            }
            if (round > 0) mbar_wait(smem_addr(&ctl->empty[s]), (round - 1) & 1, abort_flag, status, 1u);
            LaneCodes<K> nxt = {};
            if constexpr (kHyb) {
#pragma unroll
                for (int i = 0; i < K; i++) nxt.w[i] = __shfl_sync(kFullMask, own.w[i], lane + 1);
            }
            // B tile: rows = batch (zero beyond bs), 64 columns of x, 16-byte chunks swizzled by row % 8; the copies run
            // while this warp decodes and are awaited before the stage is handed to the MMA
            const uint32_t bst = b_base + s * b_stage_bytes;
            if (has0) {
                const int brow = tid8 >> 3, c = tid8 & 7;
                const uint32_t dst = bst + brow * 128 + ((c ^ (brow & 7)) << 4);
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(xv0.x), "r"(xv0.y), "r"(xv0.z), "r"(xv0.w) : "memory");
            }
            if (has1) {
                const int brow = (tid8 + 256) >> 3, c = tid8 & 7;
                const uint32_t dst = bst + brow * 128 + ((c ^ (brow & 7)) << 4);
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(xv1.x), "r"(xv1.y), "r"(xv1.z), "r"(xv1.w) : "memory");
            }
            if constexpr (!small) {
                for (int ch = tid8; ch < chunks; ch += 256) {
                    const int brow = ch >> 3, c = ch & 7;
                    const uint32_t dst = bst + brow * 128 + ((c ^ (brow & 7)) << 4);
                    const bool live = brow < bs;
                    const __half *srcx = live ? x + (size_t)brow * n + c0 + step * kStageCols + c * 8 : x;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(srcx), "r"(live ? 16 : 0) : "memory");
                }
            }
            if constexpr (kHyb) {
                const uint32_t ast = a_base + s * kAStageBytes + row_off;
                uint32_t dst4[4];                       // chunk (ks, c) of this lane's row with ms = 0, d = 0
#pragma unroll
                for (int j = 0; j < 4; j++) dst4[j] = ast + chunk_off[j];
#pragma unroll
                for (int tt = 0; tt < 4; tt++) {
                    const int ks = tt >> 1, ms = tt & 1;
                    uint32_t st[4];
                    tile_states<K>(own, nxt, tt, st);
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const int c = q >> 1, d = q & 1;
                        const uint32_t w = hyb_lookup(st[q], lut_lane);
                        // the row offset is a compile-time constant after unrolling: register + immediate addressing
                        asm volatile("st.shared.u32 [%0], %1;" ::"r"(dst4[2 * ks + c] + (uint32_t)(2 * ms + d) * 1024u), "r"(w) : "memory");
                    }
                }
            } else {
#pragma unroll
                for (int tt = 0; tt < 4; tt++) {
                    const int ks = tt >> 1, ms = tt & 1;
                    uint32_t wv[4];
#pragma unroll
                    for (int j = 0; j < 4; j++) {          // eight states, K bits apart, two weights per word
                        const uint32_t s0 = (uint32_t)(pbits[tt] >> (32 - 2 * j * K)) & 0xFFFFu;
                        const uint32_t s1 = (uint32_t)(pbits[tt] >> (32 - (2 * j + 1) * K)) & 0xFFFFu;
                        const __half lo = CODE == QTIP_CODE_3INST ? decode_3inst(s0) : decode_1mad_tab(s0, mad_tab);
                        const __half hi = CODE == QTIP_CODE_3INST ? decode_3inst(s1) : decode_1mad_tab(s1, mad_tab);
                        const __half2 p2 = __halves2half2(lo, hi);
                        wv[j] = *reinterpret_cast<const uint32_t *>(&p2);
                    }
                    // row 32rb + 16ms + pr of the stage, 16-byte chunk 4cb + 2ks + ph of its 128-byte row
                    const uint32_t row = (uint32_t)(32 * rb + 16 * ms + pr), chunk = (uint32_t)(4 * cb + 2 * ks + ph);
                    const uint32_t dst = a_base + s * kAStageBytes + (row >> 3) * 1024u + (row & 7u) * 128u + ((chunk ^ (row & 7u)) << 4);
                    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(wv[0]), "r"(wv[1]), "r"(wv[2]), "r"(wv[3]) : "memory");
                }
            }
            if constexpr (!small) asm volatile("cp.async.wait_all;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> visible to the MMA
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_addr(&ctl->full[s]));
            s += kGroups;
            if (s >= stages) { s -= stages; round++; }      // kGroups <= stages: at most one wrap
        }
    } else if (lane == 0) {
        // ------------------------------------ MMA issue ---------------------------------------------------
        // instruction descriptor: D fp32, A/B fp16, both K-major, N = npad, M = 128
        const uint32_t idesc = (1u << 4) | ((uint32_t)(npad >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
        int s = 0, round = 0;
        for (int step = 0; step < nsteps; step++) {
            // a wait that gave up ends the issue loop: no further MMA is started, and the commit below still
            // covers everything issued so far
            if (!mbar_wait(smem_addr(&ctl->full[s]), round & 1, abort_flag, status, 2u)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t adesc = umma_desc(a_base + s * kAStageBytes);
            const uint64_t bdesc = umma_desc(b_base + s * b_stage_bytes);
#pragma unroll
            for (int kk = 0; kk < 4; kk++)   // 16 columns = 32 bytes further inside the 128-byte swizzled row
                umma_f16(tmem_d, adesc + (uint64_t)(kk * 2), bdesc + (uint64_t)(kk * 2), idesc, (step | kk) != 0);
            umma_commit(smem_addr(&ctl->empty[s]));
            if (++s == stages) { s = 0; round++; }
        }
        umma_commit(smem_addr(&ctl->done));
    }

    if (warp < 4) {
        // ------------------------------------- epilogue ----------------------------------------------------
        mbar_wait(smem_addr(&ctl->done), 0u, abort_flag, status, 3u);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int row = r0 + warp * 32 + lane;
        for (int col = 0; col < npad; col += 8) {
            uint32_t r[8];
            const uint32_t taddr = tmem_d + ((uint32_t)(warp * 32) << 16) + (uint32_t)col;
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                         : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                         : "r"(taddr)
                         : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int bcol = col + j;
                if (bcol < bs) {
                    const float v = __uint_as_float(r[j]);
                    if (splitk == 1) out[(size_t)bcol * m + row] = v;
                    else atomicAdd(out + (size_t)bcol * m + row, v);
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == kDecodeWarps) {
        // tensor memory is released only after the last commit has arrived, i.e. after every MMA that was issued has
        // completed - also on the abort path, where the epilogue warps did not wait for it
        if (lane == 0) mbar_wait_bounded(smem_addr(&ctl->done), 0u);
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(tmem_cols) : "memory");
    }
}

template <int K, int CODE, int STAGES>
int launch_gemm_stages(float *out, const uint8_t *codes, const __half *x, const uint32_t *tlut, int m, int n, int bs, int npad,
                       int splitk, unsigned *status, cudaStream_t s) {
    const int smem = 1024 + STAGES * (kAStageBytes + npad * 128) + kLut512Bytes + 256;
    static bool attr_set[64] = {};
    static std::mutex attr_mutex;
    int dev = 0;
    QTIP_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return QTIP_ERR_BAD_ARG;
    {
        std::lock_guard<std::mutex> lock(attr_mutex);
        if (!attr_set[dev]) {
            QTIP_CUDA_TRY(cudaFuncSetAttribute(decompress_gemm_kernel<K, CODE, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               227 * 1024));
            attr_set[dev] = true;
        }
    }
    if (splitk > 1) QTIP_CUDA_TRY(cudaMemsetAsync(out, 0, (size_t)bs * m * sizeof(float), s));
    decompress_gemm_kernel<K, CODE, STAGES><<<dim3(m / kRows, splitk), kGemmThreads, smem, s>>>(out, codes, x, tlut, m, n, bs,
                                                                                                npad, splitk, status);
    return check_launch();
}

// four ring stages while the B tiles are small; batches above 64 (16 KiB per B tile) leave room for three
template <int K, int CODE>
int launch_gemm(float *out, const uint8_t *codes, const __half *x, const uint32_t *tlut, int m, int n, int bs, int npad,
                int splitk, unsigned *status, cudaStream_t s) {
    if (npad > 64) return launch_gemm_stages<K, CODE, 3>(out, codes, x, tlut, m, n, bs, npad, splitk, status, s);
    return launch_gemm_stages<K, CODE, kStages>(out, codes, x, tlut, m, n, bs, npad, splitk, status, s);
}

template <int CODE>
int launch_gemm_k(float *out, const uint8_t *c, const __half *xh, const uint32_t *t, int K, int m, int n, int bs, int npad,
                  int splitk, unsigned *status, cudaStream_t s) {
    if (K == 2) return launch_gemm<2, CODE>(out, c, xh, t, m, n, bs, npad, splitk, status, s);
    if (K == 3) return launch_gemm<3, CODE>(out, c, xh, t, m, n, bs, npad, splitk, status, s);
    return launch_gemm<4, CODE>(out, c, xh, t, m, n, bs, npad, splitk, status, s);
}

}  // namespace
}  // namespace qtip

using namespace qtip;

extern "C" int qtip_decompress_gemm(float *out, const void *codes, const void *x, const void *tlut, int K, int m, int n,
                                    int bs, unsigned *status, void *stream) {
    if (!out || !codes || !x || !tlut || !status || K < 2 || K > 4 || bs < 1 || bs > kMaxN) return QTIP_ERR_BAD_ARG;
    if (m <= 0 || n <= 0 || (m % kRows) || (n % kStageCols)) return QTIP_ERR_BAD_SHAPE;
    if ((long)(m >> 5) * (n >> 5) >= (1L << 30)) return QTIP_ERR_BAD_SHAPE;
    if (!aligned(codes, 16) || !aligned(x, 16) || !aligned(out, 4) || !aligned(tlut, 4) || !aligned(status, 4))
        return QTIP_ERR_ALIGNMENT;
    const int npad = (bs + 15) & ~15;
    // two CTAs per row range while that still leaves SMs idle and the column range divides
    const int splitk = ((m / kRows) * 2 <= sm_count() && (n % (2 * kStageCols)) == 0) ? 2 : 1;
    auto *c = static_cast<const uint8_t *>(codes);
    auto *xh = static_cast<const __half *>(x);
    auto *t = static_cast<const uint32_t *>(tlut);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return launch_gemm_k<QTIP_CODE_HYB>(out, c, xh, t, K, m, n, bs, npad, splitk, status, s);
}

extern "C" int qtip_decompress_gemm_plain(float *out, const void *codes, const void *x, int code, int K, int m, int n, int bs,
                                          unsigned *status, void *stream) {
    if (!out || !codes || !x || !status || K < 2 || K > 4 || bs < 1 || bs > kMaxN) return QTIP_ERR_BAD_ARG;
    if (code != QTIP_CODE_3INST && code != QTIP_CODE_1MAD) return QTIP_ERR_BAD_ARG;
    if (m <= 0 || n <= 0 || (m % kRows) || (n % kStageCols)) return QTIP_ERR_BAD_SHAPE;
    if ((long)(m >> 5) * (n >> 5) >= (1L << 30)) return QTIP_ERR_BAD_SHAPE;
    if (!aligned(codes, 16) || !aligned(x, 16) || !aligned(out, 4) || !aligned(status, 4)) return QTIP_ERR_ALIGNMENT;
    const int npad = (bs + 15) & ~15;
    const int splitk = ((m / kRows) * 2 <= sm_count() && (n % (2 * kStageCols)) == 0) ? 2 : 1;
    auto *c = static_cast<const uint8_t *>(codes);
    auto *xh = static_cast<const __half *>(x);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (code == QTIP_CODE_3INST) return launch_gemm_k<QTIP_CODE_3INST>(out, c, xh, nullptr, K, m, n, bs, npad, splitk, status, s);
    return launch_gemm_k<QTIP_CODE_1MAD>(out, c, xh, nullptr, K, m, n, bs, npad, splitk, status, s);
}
