// Small per-token kernels of a Llama decoder layer at batch 1, so that a decode step is a short
// chain of our own launches inside one CUDA graph: rotary embedding + KV-cache append, and
// single-query attention over the cache.  They replace, for the decode loop only,
// apply_rotary_pos_emb / StaticCache.update / scaled_dot_product_attention as used by
// LlamaSdpaAttention.forward upstream (model/llama.py:797-898, model/cache_utils.py:1147-1193).
// The position is read from device memory so a captured graph can be replayed for every token.
#include "common.cuh"

namespace qtip {
namespace {

// q: (n_heads, hd) fp16 rotated in place.  k: (n_kv, hd) rotated and appended to cache_k[pos];
// v: (n_kv, hd) appended to cache_v[pos].  Caches are (max_pos, n_kv*hd) fp16.
// HF convention: out[i] = x[i]*cos - x[i+hd/2]*sin ; out[i+hd/2] = x[i+hd/2]*cos + x[i]*sin,
// angle = pos * theta^(-2i/hd).
__global__ void rope_kv_kernel(__half *__restrict__ q, const __half *__restrict__ k, const __half *__restrict__ v,
                               __half *__restrict__ cache_k, __half *__restrict__ cache_v,
                               const int *__restrict__ pos_ptr, int n_heads, int n_kv, int hd, float log2_theta) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int pos = *pos_ptr;
    const int half = hd >> 1;
    const int total = (n_heads + n_kv) * half;
    const size_t crow = (size_t)pos * n_kv * hd;
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        const int head = idx / half, i = idx % half;
        const float inv_freq = exp2f(-log2_theta * (float)(2 * i) / (float)hd);
        float sn, cs;
        sincosf((float)pos * inv_freq, &sn, &cs);
        if (head < n_heads) {
            __half *p = q + (size_t)head * hd;
            const float a = __half2float(p[i]), b = __half2float(p[i + half]);
            p[i] = __float2half_rn(a * cs - b * sn);
            p[i + half] = __float2half_rn(b * cs + a * sn);
        } else {
            const int kh = head - n_heads;
            const __half *p = k + (size_t)kh * hd;
            const float a = __half2float(p[i]), b = __half2float(p[i + half]);
            cache_k[crow + (size_t)kh * hd + i] = __float2half_rn(a * cs - b * sn);
            cache_k[crow + (size_t)kh * hd + i + half] = __float2half_rn(b * cs + a * sn);
            cache_v[crow + (size_t)kh * hd + i] = v[(size_t)kh * hd + i];
            cache_v[crow + (size_t)kh * hd + i + half] = v[(size_t)kh * hd + i + half];
        }
    }
}

// One CTA per query head, 8 warps; warp w scans cache positions w, w+8, ... <= pos with an online
// softmax, lanes split the head dimension (hd = 128: 4 values per lane); partial results of the
// warps are merged through shared memory.  out: (n_heads, hd) fp16.
constexpr int kAttnWarps = 8;

__global__ void __launch_bounds__(kAttnWarps * 32)
    attn_decode_kernel(__half *__restrict__ out, const __half *__restrict__ q, const __half *__restrict__ cache_k,
                       const __half *__restrict__ cache_v, const int *__restrict__ pos_ptr, int n_heads, int n_kv,
                       float scale) {
    constexpr int hd = 128;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int head = blockIdx.x, kvh = head / (n_heads / n_kv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ctx = *pos_ptr + 1;
    const size_t row = (size_t)n_kv * hd;
    float qv[4];
    {
        const uint2 raw = *reinterpret_cast<const uint2 *>(q + (size_t)head * hd + lane * 4);
        const __half2 a = *reinterpret_cast<const __half2 *>(&raw.x), b = *reinterpret_cast<const __half2 *>(&raw.y);
        qv[0] = __low2float(a) * scale; qv[1] = __high2float(a) * scale;
        qv[2] = __low2float(b) * scale; qv[3] = __high2float(b) * scale;
    }
    float mx = -INFINITY, den = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int t = warp; t < ctx; t += kAttnWarps) {
        const size_t off = (size_t)t * row + (size_t)kvh * hd + lane * 4;
        const uint2 kr = *reinterpret_cast<const uint2 *>(cache_k + off);
        const uint2 vr = *reinterpret_cast<const uint2 *>(cache_v + off);
        const __half2 k0 = *reinterpret_cast<const __half2 *>(&kr.x), k1 = *reinterpret_cast<const __half2 *>(&kr.y);
        float s = qv[0] * __low2float(k0) + qv[1] * __high2float(k0) + qv[2] * __low2float(k1) + qv[3] * __high2float(k1);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(kFullMask, s, o);
        const float nm = fmaxf(mx, s);
        const float corr = __expf(mx - nm), pr = __expf(s - nm);
        const __half2 v0 = *reinterpret_cast<const __half2 *>(&vr.x), v1 = *reinterpret_cast<const __half2 *>(&vr.y);
        acc[0] = acc[0] * corr + pr * __low2float(v0); acc[1] = acc[1] * corr + pr * __high2float(v0);
        acc[2] = acc[2] * corr + pr * __low2float(v1); acc[3] = acc[3] * corr + pr * __high2float(v1);
        den = den * corr + pr;
        mx = nm;
    }
    __shared__ float s_mx[kAttnWarps], s_den[kAttnWarps], s_acc[kAttnWarps][hd];
    if (lane == 0) { s_mx[warp] = mx; s_den[warp] = den; }
#pragma unroll
    for (int i = 0; i < 4; i++) s_acc[warp][lane * 4 + i] = acc[i];
    __syncthreads();
    if (threadIdx.x < hd) {
        float gm = -INFINITY;
        for (int w = 0; w < kAttnWarps; w++) gm = fmaxf(gm, s_mx[w]);
        float d = 0.f, a = 0.f;
        for (int w = 0; w < kAttnWarps; w++) {
            const float c = (s_mx[w] == -INFINITY) ? 0.f : __expf(s_mx[w] - gm);
            d += s_den[w] * c;
            a += s_acc[w][threadIdx.x] * c;
        }
        out[(size_t)head * hd + threadIdx.x] = __float2half_rn(a / d);
    }
}

template <typename... Args>
int launch_pdl(void (*kernel)(Args...), dim3 grid, dim3 block, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
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

extern "C" int qtip_rope_kv_append(void *q, const void *k, const void *v, void *cache_k, void *cache_v, const int *pos,
                                   int n_heads, int n_kv_heads, int head_dim, float theta, void *stream) {
    if (!q || !k || !v || !cache_k || !cache_v || !pos) return QTIP_ERR_BAD_ARG;
    if (n_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || (head_dim & 1) || n_heads % n_kv_heads) return QTIP_ERR_BAD_SHAPE;
    const int total = (n_heads + n_kv_heads) * (head_dim / 2);
    return launch_pdl(rope_kv_kernel, dim3((total + 255) / 256), dim3(256), static_cast<cudaStream_t>(stream),
                      static_cast<__half *>(q), static_cast<const __half *>(k), static_cast<const __half *>(v),
                      static_cast<__half *>(cache_k), static_cast<__half *>(cache_v), pos, n_heads, n_kv_heads, head_dim,
                      log2f(theta));
}

extern "C" int qtip_attn_decode(void *out, const void *q, const void *cache_k, const void *cache_v, const int *pos,
                                int n_heads, int n_kv_heads, int head_dim, void *stream) {
    if (!out || !q || !cache_k || !cache_v || !pos) return QTIP_ERR_BAD_ARG;
    if (head_dim != 128 || n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads) return QTIP_ERR_BAD_SHAPE;
    if (!aligned(q, 8) || !aligned(cache_k, 8) || !aligned(cache_v, 8)) return QTIP_ERR_ALIGNMENT;
    return launch_pdl(attn_decode_kernel, dim3(n_heads), dim3(kAttnWarps * 32), static_cast<cudaStream_t>(stream),
                      static_cast<__half *>(out), static_cast<const __half *>(q), static_cast<const __half *>(cache_k),
                      static_cast<const __half *>(cache_v), pos, n_heads, n_kv_heads, 1.0f / sqrtf((float)head_dim));
}
