// The unquantized ends of a decode step at batch 1, as three small launches instead of about twenty
// framework kernels, so that the whole step is one chain of this library's launches in a CUDA graph:
//   embedding lookup                                (embed_tokens, model/llama.py LlamaModel.forward upstream)
//   final RMSNorm + fp16 lm_head matrix-vector      (LlamaForCausalLM.forward upstream; the head is not quantized)
//   temperature / top-k sampling without host sync  (eval/interactive_gen.py:15-40 upstream)
// The lm_head product is a plain HBM-bound GEMV: vocab x hidden fp16 read once.
#include "fwht.cuh"

namespace qtip {
namespace {

// res = embed[token]; delta = 0 (the residual update pending for the first layer)
__global__ void embed_kernel(__half *__restrict__ res, __half *__restrict__ delta, const __half *__restrict__ embed,
                             const long long *__restrict__ token, int hidden, int vocab, unsigned *status) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const long long tok = *token;
    if (tok < 0 || tok >= vocab) {            // not a row of the table: leave res / delta alone and report
        if (status && threadIdx.x == 0) atomicOr(status, 2u);
        return;
    }
    const uint4 *src = reinterpret_cast<const uint4 *>(embed + (size_t)tok * hidden);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < hidden / 8; i += gridDim.x * blockDim.x) {
        reinterpret_cast<uint4 *>(res)[i] = __ldg(src + i);
        reinterpret_cast<uint4 *>(delta)[i] = make_uint4(0u, 0u, 0u, 0u);
    }
}

constexpr int kHeadThreads = 256, kHeadWarps = kHeadThreads / 32, kHeadUnroll = 4;

__device__ __forceinline__ float dot8(const uint4 &w, const float4 &x0, const float4 &x1, float acc) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&w);
    const float2 a = __half22float2(h[0]), b = __half22float2(h[1]), c = __half22float2(h[2]), d = __half22float2(h[3]);
    acc = fmaf(a.x, x0.x, acc); acc = fmaf(a.y, x0.y, acc); acc = fmaf(b.x, x0.z, acc); acc = fmaf(b.y, x0.w, acc);
    acc = fmaf(c.x, x1.x, acc); acc = fmaf(c.y, x1.y, acc); acc = fmaf(d.x, x1.z, acc); acc = fmaf(d.y, x1.w, acc);
    return acc;
}

// logits[v] = sum_j W[v][j] * h[j],  h = fp16( fp16(RMSNorm(res + delta)) * norm_weight )  (LlamaRMSNorm).
// Every CTA normalises the hidden vector itself (fp32 copy in shared memory); a warp then takes two rows
// of W at a time, kHeadUnroll 16-byte loads per row and lane in flight.  The first loads of W are weights
// and are requested before the grid dependency wait.
__global__ void __launch_bounds__(kHeadThreads)
    lm_head_kernel(float *__restrict__ logits, const __half *__restrict__ res, const __half *__restrict__ delta,
                   const __half *__restrict__ norm_weight, const __half *__restrict__ W, int hidden, int vocab, float eps) {
    extern __shared__ __align__(16) float xs[];       // hidden floats, then block_sum scratch
    float *scratch = xs + hidden;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int chunks = hidden >> 3;                    // 16-byte chunks per row
    const int pair_stride = gridDim.x * kHeadWarps;
    int pair = blockIdx.x * kHeadWarps + warp;         // rows 2*pair, 2*pair + 1
    const int pairs = (vocab + 1) >> 1;

    uint4 w0[kHeadUnroll], w1[kHeadUnroll];
    auto request = [&](int p, int c0) {
        const size_t r0 = (size_t)2 * p, r1 = min((size_t)2 * p + 1, (size_t)vocab - 1);
#pragma unroll
        for (int u = 0; u < kHeadUnroll; u++) {
            const int c = c0 + u * 32 + lane;
            if (c < chunks) {
                w0[u] = ld_stream_u32x4(reinterpret_cast<const uint4 *>(W + r0 * hidden) + c);
                w1[u] = ld_stream_u32x4(reinterpret_cast<const uint4 *>(W + r1 * hidden) + c);
            }
        }
    };
    if (pair < pairs) request(pair, 0);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    float ss = 0.f;
    for (int j = threadIdx.x * 8; j < hidden; j += kHeadThreads * 8) {
        float a[8], b[8];
        load8_f16(res, j, a);
        load8_f16(delta, j, b);
#pragma unroll
        for (int k = 0; k < 8; k++) {
            a[k] = __half2float(__float2half_rn(a[k] + b[k]));     // fp16 residual stream
            ss += a[k] * a[k];
            xs[j + k] = a[k];
        }
    }
    const float r = rsqrtf(block_sum(ss, scratch) / (float)hidden + eps);
    for (int j = threadIdx.x * 8; j < hidden; j += kHeadThreads * 8) {
        float wn[8];
        load8_f16(norm_weight, j, wn);
#pragma unroll
        for (int k = 0; k < 8; k++) xs[j + k] = __half2float(__hmul(__float2half_rn(wn[k]), __float2half_rn(xs[j + k] * r)));
    }
    __syncthreads();

    for (; pair < pairs; pair += pair_stride) {
        float acc0 = 0.f, acc1 = 0.f;
        for (int c0 = 0; c0 < chunks; c0 += kHeadUnroll * 32) {
            uint4 a0[kHeadUnroll], a1[kHeadUnroll];
#pragma unroll
            for (int u = 0; u < kHeadUnroll; u++) { a0[u] = w0[u]; a1[u] = w1[u]; }
            // next batch: the rest of this pair of rows, or the start of the warp's next pair
            const int nc0 = c0 + kHeadUnroll * 32;
            if (nc0 < chunks) request(pair, nc0);
            else if (pair + pair_stride < pairs) request(pair + pair_stride, 0);
#pragma unroll
            for (int u = 0; u < kHeadUnroll; u++) {
                const int c = c0 + u * 32 + lane;
                if (c < chunks) {
                    const float4 x0 = *reinterpret_cast<const float4 *>(xs + c * 8), x1 = *reinterpret_cast<const float4 *>(xs + c * 8 + 4);
                    acc0 = dot8(a0[u], x0, x1, acc0);
                    acc1 = dot8(a1[u], x0, x1, acc1);
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            acc0 += __shfl_xor_sync(kFullMask, acc0, o);
            acc1 += __shfl_xor_sync(kFullMask, acc1, o);
        }
        if (lane == 0) {
            logits[2 * pair] = acc0;
            if (2 * pair + 1 < vocab) logits[2 * pair + 1] = acc1;
        }
    }
}

// ---- sampler ---------------------------------------------------------------------------------------------
constexpr int kSampleThreads = 1024, kMaxTopK = 16;

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// One CTA.  top_k rounds of a block-wide arg-max over the logits not yet taken (ties: lower index), then
// softmax(top / temperature) and one draw by inverse CDF from a counter-based generator keyed by (seed, *pos).
// Writes the token to `token` and to out_tokens[*pos + 1], then advances *pos.
__global__ void __launch_bounds__(kSampleThreads)
    sample_kernel(long long *__restrict__ token, long long *__restrict__ out_tokens, int *__restrict__ pos,
                  const float *__restrict__ logits, int vocab, float inv_temperature, int top_k, unsigned long long seed,
                  int max_tokens, unsigned *status) {
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    __shared__ float top_val[kMaxTopK];
    __shared__ int top_idx[kMaxTopK];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // up to 32 logits per thread stay in registers for all rounds (vocabularies up to 32768); larger ones are re-read
    constexpr int kHeld = 32;
    const bool held = vocab <= kHeld * kSampleThreads;
    float mine[kHeld];
    if (held) {
#pragma unroll
        for (int j = 0; j < kHeld; j++) {
            const int i = threadIdx.x + j * kSampleThreads;
            mine[j] = i < vocab ? __ldcg(logits + i) : -INFINITY;
        }
    }
    for (int round = 0; round < top_k; round++) {
        float best = -INFINITY;
        int bi = 0x7FFFFFFF;
        if (held) {
#pragma unroll
            for (int j = 0; j < kHeld; j++) {
                const float v = mine[j];
                if (v > best) { best = v; bi = threadIdx.x + j * kSampleThreads; }    // ascending index: ties keep the lower
            }
        } else {
            for (int i = threadIdx.x; i < vocab; i += kSampleThreads) {
                const float v = __ldcg(logits + i);
                bool taken = false;
                for (int q = 0; q < round; q++) taken |= (top_idx[q] == i);
                if (!taken && (v > best || (v == best && i < bi))) { best = v; bi = i; }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(kFullMask, best, o);
            const int oi = __shfl_xor_sync(kFullMask, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) { s_val[warp] = best; s_idx[warp] = bi; }
        __syncthreads();
        if (warp == 0) {
            best = s_val[lane]; bi = s_idx[lane];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(kFullMask, best, o);
                const int oi = __shfl_xor_sync(kFullMask, bi, o);
                if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
            }
            if (lane == 0) { top_val[round] = best; top_idx[round] = bi; }
        }
        __syncthreads();
        if (held) {
            const int win = top_idx[round];
#pragma unroll
            for (int j = 0; j < kHeld; j++)
                if (win == threadIdx.x + j * kSampleThreads) mine[j] = -INFINITY;     // (a -inf logit can be drawn twice)
        }
    }
    if (threadIdx.x == 0) {
        const int p = *pos;
        float prob[kMaxTopK], sum = 0.f;
        for (int q = 0; q < top_k; q++) { prob[q] = __expf((top_val[q] - top_val[0]) * inv_temperature); sum += prob[q]; }
        const unsigned long long bits = splitmix64(seed ^ splitmix64((unsigned long long)p));
        const float u = (float)(bits >> 40) * (1.0f / 16777216.0f) * sum;      // uniform in [0, sum)
        int pick = top_k - 1;
        float cum = 0.f;
        for (int q = 0; q < top_k; q++) {
            cum += prob[q];
            if (u < cum) { pick = q; break; }
        }
        const long long t = top_idx[pick];
        *token = t;
        if (p >= 0 && p + 1 < max_tokens) out_tokens[p + 1] = t;      // the token log is full: keep sampling, report
        else if (status) atomicOr(status, 4u);
        *pos = p + 1;
    }
}

template <typename... Args>
int launch_pdl(void (*kernel)(Args...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    QTIP_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, args...));
    return check_launch();
}

}  // namespace
}  // namespace qtip

using namespace qtip;

extern "C" int qtip_embed_token(void *res, void *delta, const void *embed, const long long *token, int hidden, int vocab,
                                unsigned *status, void *stream) {
    if (!res || !delta || !embed || !token || vocab <= 0) return QTIP_ERR_BAD_ARG;
    if (hidden <= 0 || (hidden & 7)) return QTIP_ERR_BAD_SHAPE;
    if (!aligned(res, 16) || !aligned(delta, 16) || !aligned(embed, 16) || !aligned(token, 8)) return QTIP_ERR_ALIGNMENT;
    return launch_pdl(embed_kernel, dim3(2), dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<__half *>(res),
                      static_cast<__half *>(delta), static_cast<const __half *>(embed), token, hidden, vocab, status);
}

extern "C" int qtip_lm_head(float *logits, const void *res, const void *delta, const void *norm_weight, const void *weight,
                            int hidden, int vocab, float eps, void *stream) {
    if (!logits || !res || !delta || !norm_weight || !weight) return QTIP_ERR_BAD_ARG;
    if (hidden <= 0 || (hidden & 7) || hidden > 32768 || vocab <= 0) return QTIP_ERR_BAD_SHAPE;
    const void *ptrs[] = {res, delta, norm_weight, weight};
    for (const void *p : ptrs)
        if (!aligned(p, 16)) return QTIP_ERR_ALIGNMENT;
    if (!aligned(logits, 4)) return QTIP_ERR_ALIGNMENT;
    const size_t smem = (size_t)(hidden + 32) * sizeof(float);
    static bool attr_set[64] = {};
    int dev = 0;
    QTIP_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 64 && !attr_set[dev]) {
        QTIP_CUDA_TRY(cudaFuncSetAttribute(lm_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (32768 + 32) * 4));
        attr_set[dev] = true;
    }
    const int pairs = (vocab + 1) / 2;
    int grid = sm_count() * 4;                              // 4 CTAs of 8 warps per SM
    if (grid * kHeadWarps > pairs) grid = (pairs + kHeadWarps - 1) / kHeadWarps;
    return launch_pdl(lm_head_kernel, dim3(grid), dim3(kHeadThreads), smem, static_cast<cudaStream_t>(stream), logits,
                      static_cast<const __half *>(res), static_cast<const __half *>(delta),
                      static_cast<const __half *>(norm_weight), static_cast<const __half *>(weight), hidden, vocab, eps);
}

extern "C" int qtip_sample_top_k(long long *token, long long *out_tokens, int *pos, const float *logits, int vocab,
                                 float temperature, int top_k, unsigned long long seed, int max_tokens, unsigned *status,
                                 void *stream) {
    if (!token || !out_tokens || !pos || !logits || max_tokens <= 0) return QTIP_ERR_BAD_ARG;
    if (vocab <= 0 || top_k < 1 || top_k > kMaxTopK || top_k > vocab) return QTIP_ERR_BAD_SHAPE;
    const float inv_t = 1.0f / fmaxf(temperature, 1e-5f);
    return launch_pdl(sample_kernel, dim3(1), dim3(kSampleThreads), 0, static_cast<cudaStream_t>(stream), token, out_tokens, pos,
                      logits, vocab, inv_t, top_k, seed, max_tokens, status);
}
