// Viterbi quantizer over the bitshift trellis with tail-biting: the encoder that produces the trellis states the
// decoders of this library consume (bitshift_codebook.quantize upstream, lib/codebook/bitshift.py:203-292).
//
// A sequence of T values is quantized to S = T/V states of L = 16 bits, consecutive states overlapping by 16 - KV bits
// (KV = K*V).  Upstream keeps one cost per state (2^16 floats per sequence and step) and, per step, gathers the
// 2^KV predecessors of every group of states that share them.  Here the cost vector is never materialised:
//     cost_i[p] = err_i(p) + best_i[p >> KV],      best_{i+1}[g] = min over d of cost_i[g + d * G],   G = 2^(16-KV)
// so the dynamic-programming state of a sequence is the G values best_i (16 KiB at 2 bits with V = 2) and lives in
// shared memory; err_i(p) = sum over v of (recons_v(p) - x_{iV+v})^2 is recomputed from the code function, which is a
// handful of integer instructions and one small table lookup.  The arithmetic is upstream's, operation for operation in
// fp32 with round-to-nearest and no contraction (subtract, square, add over v, add best; strict "<" in ascending
// predecessor order = torch.min's first minimal index), so the chosen states are identical to upstream's, not merely
// equally good.  Tail-biting as upstream: a first pass over the sequence rolled by half its length with free ends
// yields the 16 - KV bits where the original sequence starts; the second pass forces its first state to begin and its
// last state to end with them.
//
// One CTA of 1024 threads per sequence (grid-stride over sequences).  Back-pointers (one byte per group and step) go to
// a per-CTA slab of the caller's workspace and are read back by one thread for the back-trace.  The kernel is bound by
// instruction issue: 65536 candidate evaluations of ~16 instructions per step and sequence.  No waits except CTA barriers.
#include "common.cuh"

namespace qtip {
namespace {

constexpr int kVitThreads = 1024;
constexpr int kMaxT = 1024;

// reconstruction of state p: r0 (and r1 for V = 2), upstream's recons_state[:, p].  `tl` is the code's table in shared
// memory: HYB the 512 x 2 fp32 LUT; 1MAD the 1021 possible values (byte sum - 510) / 147.800537109375 (the IEEE quotient
// upstream computes, tabulated once per CTA instead of divided per evaluation); 3INST needs none.
// (tl: 32-bit shared-memory address of the table - the loops are bound by instruction issue, and 64-bit generic
// address arithmetic would cost two more instructions per evaluation)
template <int CODE>
__device__ __forceinline__ void recons_of(uint32_t p, uint32_t tl, float &r0, float &r1) {
    if constexpr (CODE == QTIP_CODE_HYB) {
        const uint32_t h = hyb_hash(p);
        float vx, vy;
        asm("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(vx), "=f"(vy) : "r"(tl + ((h >> 3) & 0xFF8u)));    // entry (h >> 6) & 511
        // quantlut_sym multiplies the first value by -1 when bit 15 of the hash is set: flip the sign bit
        r0 = __uint_as_float(__float_as_uint(vx) ^ ((h << 16) & 0x80000000u));
        r1 = vy;
    } else if constexpr (CODE == QTIP_CODE_3INST) {
        r0 = __half2float(decode_3inst(p));
        r1 = 0.f;
    } else {
        const uint32_t x = p * 34038481u + 76625530u;
        asm("ld.shared.f32 %0, [%1];" : "=f"(r0) : "r"(tl + __vsadu4(x, 0u) * 4u));
        r1 = 0.f;
    }
}

template <int CODE>
__device__ __forceinline__ float err_of(uint32_t p, uint32_t tl, float x0, float x1) {
    float r0, r1;
    recons_of<CODE>(p, tl, r0, r1);
    const float d0 = __fsub_rn(r0, x0);
    float e = __fmul_rn(d0, d0);
    if constexpr (CODE == QTIP_CODE_HYB) {
        const float d1 = __fsub_rn(r1, x1);
        e = __fadd_rn(e, __fmul_rn(d1, d1));
    }
    return e;
}

struct __align__(16) Smem {    // sizeof is a multiple of 16: the table (8-byte loads) and the cost arrays follow it
    float x[kMaxT];            // the sequence as fp32 (second pass order)
    float red_v[32];
    uint32_t red_i[32];
    uint32_t arg;
};

// One pass of upstream's viterbi().  xoff: the pass reads x[(t + xoff) % T] (the rolled sequence of the first pass).
// Leaves the first minimal final state in sh->arg; back-pointers in bp[i*G + g], i = 1..S-1.
template <int CODE>
__device__ __forceinline__ void viterbi_pass(Smem *sh, float *best0, float *best1, uint32_t tl, uint8_t *__restrict__ bp, int T, int KV,
                             int xoff, bool has_overlap, uint32_t overlap, float *final_cost) {
    constexpr int V = CODE == QTIP_CODE_HYB ? 2 : 1;
    const int S = T / V;
    const uint32_t G = 65536u >> KV, D = 1u << KV, Gs = G >> KV;     // (g + d*G) >> KV = (g >> KV) + d * Gs
    const int tid = threadIdx.x;
    // best_0: adding 0 leaves the first step's error as it is; with an overlap only the states whose top bits equal it
    // may start the walk (upstream: min(cost + mask, inf))
    for (uint32_t q = tid; q < G; q += kVitThreads) best0[q] = (!has_overlap || q == overlap) ? 0.f : INFINITY;
    __syncthreads();
    // threads per group: 1 while there are at least as many groups as threads, else the predecessor range is split
    const uint32_t tpg = G >= (uint32_t)kVitThreads ? 1u : (uint32_t)kVitThreads / G;
    const uint32_t dchunk = D / tpg;
    float *cur = best0, *nxt = best1;
    for (int i = 0; i + 1 < S; i++) {
        int t0 = i * V + xoff;
        if (t0 >= T) t0 -= T;
        const float x0 = sh->x[t0], x1 = V == 2 ? sh->x[t0 + 1] : 0.f;      // T and xoff are multiples of V
        uint8_t *bpi = bp + (size_t)(i + 1) * G;
        for (uint32_t w = tid; w < G * tpg; w += kVitThreads) {
            const uint32_t g = w / tpg, sub = w - g * tpg;
            const uint32_t d0 = sub * dchunk;
            float bv = 0.f;
            uint32_t bd = d0;
            // ascending d with a strict "<": the first minimal predecessor wins, as torch.min does
            uint32_t pcur = g + d0 * G;
            uint32_t bcur = (uint32_t)__cvta_generic_to_shared(cur) + ((g >> KV) + d0 * Gs) * 4u;
            float bprev;
            asm volatile("ld.shared.f32 %0, [%1];" : "=f"(bprev) : "r"(bcur) : "memory");
            bv = __fadd_rn(err_of<CODE>(pcur, tl, x0, x1), bprev);
#pragma unroll 4
            for (uint32_t d = d0 + 1; d < d0 + dchunk; d++) {
                pcur += G;
                bcur += Gs * 4u;
                asm volatile("ld.shared.f32 %0, [%1];" : "=f"(bprev) : "r"(bcur) : "memory");
                const float c = __fadd_rn(err_of<CODE>(pcur, tl, x0, x1), bprev);
                if (c < bv) { bv = c; bd = d; }
            }
            // combine the sub-ranges of a group (adjacent lanes, ascending d): the lower range wins ties
            for (uint32_t o = 1; o < tpg; o <<= 1) {
                const float ov = __shfl_xor_sync(kFullMask, bv, o);
                const uint32_t od = __shfl_xor_sync(kFullMask, bd, o);
                const bool take = (sub & o) ? (ov <= bv) : (ov < bv);      // partner holds the lower range iff our bit is set
                if (take) { bv = ov; bd = od; }
            }
            if (sub == 0) { nxt[g] = bv; bpi[g] = (uint8_t)bd; }
        }
        __syncthreads();
        float *t = cur; cur = nxt; nxt = t;
    }
    // final costs: err_{S-1}(s) + best_{S-1}[s >> KV], masked to the states that end with the overlap bits; first minimum
    {
        int t0 = (S - 1) * V + xoff;
        if (t0 >= T) t0 -= T;
        const float x0 = sh->x[t0], x1 = V == 2 ? sh->x[t0 + 1] : 0.f;
        constexpr uint32_t kPer = 65536u / kVitThreads;
        float bv = INFINITY;
        uint32_t bi = 0xFFFFFFFFu;
        for (uint32_t s = tid * kPer; s < (tid + 1) * kPer; s++) {
            float c = __fadd_rn(err_of<CODE>(s, tl, x0, x1), cur[s >> KV]);
            if (has_overlap && (s & (G - 1)) != overlap) c = INFINITY;
            if (bi == 0xFFFFFFFFu || c < bv) { bv = c; bi = s; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(kFullMask, bv, o);
            const uint32_t oi = __shfl_xor_sync(kFullMask, bi, o);
            if (ov < bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if ((tid & 31) == 0) { sh->red_v[tid >> 5] = bv; sh->red_i[tid >> 5] = bi; }
        __syncthreads();
        if (tid < 32) {
            bv = sh->red_v[tid]; bi = sh->red_i[tid];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(kFullMask, bv, o);
                const uint32_t oi = __shfl_xor_sync(kFullMask, bi, o);
                if (ov < bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            if (tid == 0) {
                sh->arg = bi;
                if (final_cost) *final_cost = bv;
            }
        }
        __syncthreads();
    }
}

template <int CODE>
__global__ void __launch_bounds__(kVitThreads, 1)
    viterbi_kernel(int *__restrict__ states, float *__restrict__ final_cost, const __half *__restrict__ X, long N, int T, int KV,
                   const float2 *__restrict__ tlut, uint8_t *__restrict__ workspace) {
    constexpr int V = CODE == QTIP_CODE_HYB ? 2 : 1;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    Smem *sh = reinterpret_cast<Smem *>(smem_raw);
    static_assert(sizeof(Smem) % 16 == 0, "what follows the control block needs 8- and 16-byte alignment");
    float2 *tl = reinterpret_cast<float2 *>(smem_raw + sizeof(Smem));                 // 4 KiB: the code's table (HYB, 1MAD)
    const uint32_t G = 65536u >> KV;
    float *best0 = reinterpret_cast<float *>(smem_raw + sizeof(Smem) + 512 * sizeof(float2));
    float *best1 = best0 + G;
    const int S = T / V;
    uint8_t *bp = workspace + (size_t)blockIdx.x * S * G;
    if constexpr (CODE == QTIP_CODE_HYB)
        for (int i = threadIdx.x; i < 512; i += kVitThreads) tl[i] = tlut[i];
    if constexpr (CODE == QTIP_CODE_1MAD)
        for (int i = threadIdx.x; i < 1024; i += kVitThreads)
            reinterpret_cast<float *>(tl)[i] = __fdiv_rn((float)(i - 510), 147.800537109375f);
    const uint32_t tl_addr = (uint32_t)__cvta_generic_to_shared(tl);
    for (long b = blockIdx.x; b < N; b += gridDim.x) {
        __syncthreads();
        for (int t = threadIdx.x; t < T; t += kVitThreads) sh->x[t] = __half2float(X[b * T + t]);
        __syncthreads();
        // first pass: the sequence rolled by T/(2V)*V (rolled[t] = x[t - roll]), free ends
        const int roll = T / (2 * V) * V;
        viterbi_pass<CODE>(sh, best0, best1, tl_addr, bp, T, KV, T - roll, false, 0u, nullptr);
        // the state at step T/(2V) of the rolled walk is where the original sequence starts
        if (threadIdx.x == 0) {
            uint32_t st = sh->arg;
            for (int i = S - 1; i > T / (2 * V); i--) {
                const uint32_t g = st >> KV;
                st = g + (uint32_t)bp[(size_t)i * G + g] * G;
            }
            sh->arg = st >> KV;
        }
        __syncthreads();
        const uint32_t overlap = sh->arg;
        __syncthreads();
        viterbi_pass<CODE>(sh, best0, best1, tl_addr, bp, T, KV, 0, true, overlap, final_cost ? final_cost + b : nullptr);
        if (threadIdx.x == 0) {
            uint32_t st = sh->arg;
            int *out = states + b * S;
            out[S - 1] = (int)st;
            for (int i = S - 1; i > 0; i--) {
                const uint32_t g = st >> KV;
                st = g + (uint32_t)bp[(size_t)i * G + g] * G;
                out[i - 1] = (int)st;
            }
        }
    }
}

int viterbi_grid(long N) {
    const long cap = sm_count();
    return (int)(N < cap ? N : cap);
}

int kv_of(int code, int K) { return code == QTIP_CODE_HYB ? 2 * K : K; }

template <int CODE>
int launch_viterbi(int *states, float *final_cost, const __half *X, long N, int T, int KV, const float2 *tlut, uint8_t *ws,
                   cudaStream_t s) {
    const uint32_t G = 65536u >> KV;
    const int smem = (int)(sizeof(Smem) + 512 * sizeof(float2) + 2 * G * sizeof(float));
    QTIP_CUDA_TRY(cudaFuncSetAttribute(viterbi_kernel<CODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    viterbi_kernel<CODE><<<viterbi_grid(N), kVitThreads, smem, s>>>(states, final_cost, X, N, T, KV, tlut, ws);
    return check_launch();
}

}  // namespace
}  // namespace qtip

using namespace qtip;

extern "C" size_t qtip_viterbi_workspace_bytes(int code, int K, int T, long N) {
    if (K < 1 || K > 4 || T <= 0 || N <= 0 || code < QTIP_CODE_HYB || code > QTIP_CODE_1MAD) return 0;
    const int V = code == QTIP_CODE_HYB ? 2 : 1;
    return (size_t)viterbi_grid(N) * (size_t)(T / V) * (65536u >> kv_of(code, K));
}

extern "C" int qtip_viterbi_quantize(int *states, float *final_cost, const void *X, long N, int T, int code, int K,
                                     const float *tlut, void *workspace, size_t workspace_bytes, void *stream) {
    if (!states || !X || N <= 0 || K < 2 || K > 4) return QTIP_ERR_BAD_ARG;
    if (code != QTIP_CODE_HYB && code != QTIP_CODE_3INST && code != QTIP_CODE_1MAD) return QTIP_ERR_BAD_ARG;
    if (code == QTIP_CODE_HYB && !tlut) return QTIP_ERR_BAD_ARG;
    const int V = code == QTIP_CODE_HYB ? 2 : 1;
    // a tail-biting walk needs at least L = 16 stream bits (T*K): shorter sequences have no walk whose ends overlap
    if (T < 4 * V || T * K < 16 || T > kMaxT || (T % (2 * V))) return QTIP_ERR_BAD_SHAPE;
    if (!aligned(states, 4) || !aligned(X, 2) || (tlut && !aligned(tlut, 8)) || (final_cost && !aligned(final_cost, 4)))
        return QTIP_ERR_ALIGNMENT;
    if (!workspace || workspace_bytes < qtip_viterbi_workspace_bytes(code, K, T, N)) return QTIP_ERR_WORKSPACE;
    auto *xh = static_cast<const __half *>(X);
    auto *tl = reinterpret_cast<const float2 *>(tlut);
    auto *ws = static_cast<uint8_t *>(workspace);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int KV = kv_of(code, K);
    if (code == QTIP_CODE_HYB) return launch_viterbi<QTIP_CODE_HYB>(states, final_cost, xh, N, T, KV, tl, ws, s);
    if (code == QTIP_CODE_3INST) return launch_viterbi<QTIP_CODE_3INST>(states, final_cost, xh, N, T, KV, tl, ws, s);
    return launch_viterbi<QTIP_CODE_1MAD>(states, final_cost, xh, N, T, KV, tl, ws, s);
}
