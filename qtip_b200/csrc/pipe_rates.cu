// Measurement support: issue rates of the instructions the trellis decoders are made of, on the GPU at hand.
//
// The decode kernels are bound by instruction issue, not by HBM (two to four half-rate integer instructions and one
// shared-memory gather per state), so the ceiling their roofline is quoted against is a property of the SM's pipes.
// qtip_measure_pipe_rates runs, for each instruction class, one CTA per SM whose warps each execute a long stream of
// 8 independent dependency chains of that instruction and reports cycles per warp-instruction per SM sub-partition
// (clock64 around the loop, averaged over the CTAs).  `decode sequence` is the per-state sequence of the HYB decoders
// (funnel shift, multiply-add hash, mask, multiply-add address, lane-private shared load) counted per STATE.
// No waits, no peers; every loop has a fixed trip count.  Used by `python -m qtip_b200.microbench --pipes`.
#include "common.cuh"

namespace qtip {
namespace {

enum { OP_IMAD = 0, OP_LOP3, OP_SHF, OP_PRMT, OP_IADD, OP_IMADHI, OP_LDS, OP_HMMA, OP_DECODE, OP_DECODE_NOLDS, OP_COUNT };
const char *const kOpNames[OP_COUNT] = {"IMAD (mad.lo.u32)", "LOP3", "SHF (funnel shift)", "PRMT", "IADD", "IMAD.HI (mul.hi.u32)",
                                        "LDS (lane-private gather)", "HMMA (mma.sync.m16n8k16, fp32 accumulate)",
                                        "decode sequence per state (shf, imad, and, imad, lds)",
                                        "decode sequence per state without the lds"};

template <int OP>
__global__ void __launch_bounds__(1024, 1) pipe_rate_kernel(uint32_t *out, long long *cycles, int iters, uint32_t seed) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint32_t *lut = reinterpret_cast<uint32_t *>(smem);
    if (OP == OP_LDS || OP == OP_DECODE)
        for (int i = threadIdx.x; i < 1024 * 32; i += blockDim.x) lut[i] = i * 2654435761u;
    __syncthreads();
    const uint32_t lut_lane = (uint32_t)__cvta_generic_to_shared(lut) + (threadIdx.x & 31) * 4;
    uint32_t r[8];
#pragma unroll
    for (int j = 0; j < 8; j++) r[j] = (threadIdx.x * 2654435761u + j * 40503u + seed) | 1u;
    const uint32_t k1 = seed | 0x10001u, k2 = seed * 3 + 7;
    float acc[8][4] = {};
    const long long t0 = clock64();
    for (int it = 0; it < iters; it++) {
#pragma unroll
        for (int j = 0; j < 8; j++) {
            if (OP == OP_IMAD) asm volatile("mad.lo.u32 %0, %0, %0, %1;" : "+r"(r[j]) : "r"(k1));
            else if (OP == OP_LOP3) asm volatile("lop3.b32 %0, %0, %1, %2, 0x96;" : "+r"(r[j]) : "r"(k1), "r"(k2));
            else if (OP == OP_SHF) asm volatile("shf.l.wrap.b32 %0, %0, %1, %2;" : "+r"(r[j]) : "r"(k1), "r"(k2));
            else if (OP == OP_PRMT) asm volatile("prmt.b32 %0, %0, %1, %2;" : "+r"(r[j]) : "r"(k1), "r"(k2));
            else if (OP == OP_IADD) asm volatile("add.u32 %0, %0, %1;" : "+r"(r[j]) : "r"(k1));
            else if (OP == OP_IMADHI) asm volatile("mul.hi.u32 %0, %0, %1;" : "+r"(r[j]) : "r"(k1));
            else if (OP == OP_LDS) {
                const uint32_t a = lut_lane + ((r[j] & 0x3FFu) << 7);
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(r[j]) : "r"(a));
            } else if (OP == OP_HMMA) {
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                             : "+f"(acc[j][0]), "+f"(acc[j][1]), "+f"(acc[j][2]), "+f"(acc[j][3])
                             : "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(k1), "r"(k2));
            } else {
                // r[j] plays a code word: four states per word, as at 2 bits per weight
                const uint32_t w = r[j];
                uint32_t x = 0;
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    uint32_t t, h, a, v;
                    asm volatile("shf.l.wrap.b32 %0, %1, %2, %3;" : "=r"(t) : "r"(k1), "r"(w), "r"(4 * q + 1));
                    asm volatile("mad.lo.u32 %0, %1, %1, %1;" : "=r"(h) : "r"(t));
                    asm volatile("and.b32 %0, %1, 0xFFC0;" : "=r"(h) : "r"(h));
                    asm volatile("mad.lo.u32 %0, %1, 2, %2;" : "=r"(a) : "r"(h), "r"(lut_lane));
                    if (OP == OP_DECODE) asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
                    else v = a;
                    x ^= v;
                }
                r[j] = x + w;
            }
        }
    }
    const long long t1 = clock64();
    uint32_t s = 0;
#pragma unroll
    for (int j = 0; j < 8; j++) s ^= r[j] ^ __float_as_uint(acc[j][0] + acc[j][1] + acc[j][2] + acc[j][3]);
    out[blockIdx.x * blockDim.x + threadIdx.x] = s;       // keeps the chains alive
    if (threadIdx.x == 0) cycles[blockIdx.x] = t1 - t0;
}

template <int OP>
int run_op(int threads, int iters, uint32_t *out, long long *cyc, int ctas, double *result) {
    constexpr int kSmem = 128 * 1024;
    QTIP_CUDA_TRY(cudaFuncSetAttribute(pipe_rate_kernel<OP>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
    pipe_rate_kernel<OP><<<ctas, threads, kSmem>>>(out, cyc, 16, 1u);          // warm-up
    pipe_rate_kernel<OP><<<ctas, threads, kSmem>>>(out, cyc, iters, 1u);
    QTIP_CUDA_TRY(cudaDeviceSynchronize());
    long long h[512];
    QTIP_CUDA_TRY(cudaMemcpy(h, cyc, sizeof(long long) * ctas, cudaMemcpyDeviceToHost));
    double avg = 0;
    for (int i = 0; i < ctas; i++) avg += (double)h[i];
    avg /= ctas;
    const int per = (OP == OP_DECODE || OP == OP_DECODE_NOLDS) ? 4 : 1;        // states per inner step of the decode sequence
    const double warp_ops = (double)iters * 8 * per * (threads / 32);
    *result = avg / (warp_ops / 4);                                             // cycles per warp-op per sub-partition
    return QTIP_OK;
}

}  // namespace
}  // namespace qtip

using namespace qtip;

extern "C" int qtip_pipe_rate_count(void) { return OP_COUNT; }

extern "C" const char *qtip_pipe_rate_name(int i) { return (i >= 0 && i < OP_COUNT) ? kOpNames[i] : ""; }

extern "C" int qtip_measure_pipe_rates(double *cycles, int count, int threads_per_cta) {
    if (!cycles || count < OP_COUNT || threads_per_cta < 32 || threads_per_cta > 1024 || (threads_per_cta & 31)) return QTIP_ERR_BAD_ARG;
    const int ctas = sm_count() < 512 ? sm_count() : 512;
    uint32_t *out = nullptr;
    long long *cyc = nullptr;
    QTIP_CUDA_TRY(cudaMalloc(&out, (size_t)ctas * 1024 * sizeof(uint32_t)));
    if (cudaMalloc(&cyc, (size_t)ctas * sizeof(long long)) != cudaSuccess) { cudaFree(out); return QTIP_ERR_CUDA; }
    int st = QTIP_OK;
    const int t = threads_per_cta;
    auto go = [&](int rc) { if (st == QTIP_OK) st = rc; };
    go(run_op<OP_IMAD>(t, 4000, out, cyc, ctas, cycles + OP_IMAD));
    go(run_op<OP_LOP3>(t, 4000, out, cyc, ctas, cycles + OP_LOP3));
    go(run_op<OP_SHF>(t, 4000, out, cyc, ctas, cycles + OP_SHF));
    go(run_op<OP_PRMT>(t, 4000, out, cyc, ctas, cycles + OP_PRMT));
    go(run_op<OP_IADD>(t, 4000, out, cyc, ctas, cycles + OP_IADD));
    go(run_op<OP_IMADHI>(t, 4000, out, cyc, ctas, cycles + OP_IMADHI));
    go(run_op<OP_LDS>(t, 4000, out, cyc, ctas, cycles + OP_LDS));
    go(run_op<OP_HMMA>(t, 2000, out, cyc, ctas, cycles + OP_HMMA));
    go(run_op<OP_DECODE>(t, 2000, out, cyc, ctas, cycles + OP_DECODE));
    go(run_op<OP_DECODE_NOLDS>(t, 2000, out, cyc, ctas, cycles + OP_DECODE_NOLDS));
    cudaFree(out);
    cudaFree(cyc);
    return st;
}
