// Small per-token kernels of a Llama decoder layer at batch 1, so that a decode step is a short
// chain of our own launches inside one CUDA graph: rotary embedding + KV-cache append, and
// single-query attention over the cache.  They replace, for the decode loop only,
// apply_rotary_pos_emb / StaticCache.update / scaled_dot_product_attention as used by
// LlamaSdpaAttention.forward upstream (model/llama.py:797-898, model/cache_utils.py:1147-1193).
// The position is read from device memory so a captured graph can be replayed for every token.
#include "common.cuh"
#include "fwht.cuh"

namespace qtip {
namespace {

// Cache capacity guard: a position outside [0, max_pos) must not be used as a cache row.  The whole grid sees the
// same position, so every CTA leaves together (before any barrier that later code relies on); the caller learns
// of it through the status word.
__device__ __forceinline__ bool position_ok(int pos, int max_pos, unsigned *status) {
    if ((unsigned)pos < (unsigned)max_pos) return true;
    if (status && threadIdx.x == 0) atomicOr(status, 1u);
    return false;
}

// q: (n_heads, hd) fp16 rotated in place.  k: (n_kv, hd) rotated and appended to cache_k[pos];
// v: (n_kv, hd) appended to cache_v[pos].  Caches are (max_pos, n_kv*hd) fp16.
// HF convention: out[i] = x[i]*cos - x[i+hd/2]*sin ; out[i+hd/2] = x[i+hd/2]*cos + x[i]*sin,
// angle = pos * theta^(-2i/hd).
__global__ void rope_kv_kernel(__half *__restrict__ q, const __half *__restrict__ k, const __half *__restrict__ v,
                               __half *__restrict__ cache_k, __half *__restrict__ cache_v,
                               const int *__restrict__ pos_ptr, int n_heads, int n_kv, int hd, float log2_theta,
                               int max_pos, unsigned *status) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int pos = *pos_ptr;
    if (!position_ok(pos, max_pos, status)) return;
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

// rope_kv_kernel with the output side of the q/k/v linears in front of it: CTA 0 / 1 / 2 takes the raw
// matvec result y_q / y_k / y_v (fp32), applies sign * H(y) * scale in registers (fwht_regs), rounds to
// fp16 as the linear's output tensor would be, and then rotates / appends as above.  The matvec launch
// then needs no last-CTA epilogue.  Widths are 1024*E, E in {1, 2, 4, 8, 16}.
struct QkvPostArgs {
    const float *y[3];
    const float *sv[3];
    float scale[3];
    int width[3];
    __half *q_out, *cache_k, *cache_v;
    const int *pos;
    int n_heads, n_kv, hd;
    float log2_theta;
    int max_pos;
    unsigned *status;
};

template <int E>
__device__ __forceinline__ void qkv_transform(const QkvPostArgs &a, int which, float *buf, float *vals) {
    const size_t jA = (size_t)threadIdx.x * E;
    const size_t jB = (size_t)((threadIdx.x & 31) * 32 + (threadIdx.x >> 5)) * E;
    float v[E], sg[E];
    if (a.sv[which]) loadE_f32<E>(a.sv[which], jB, sg, false);     // a weight: requested before the wait
    asm volatile("griddepcontrol.wait;" ::: "memory");
    loadE_f32<E>(a.y[which], jA, v, true);
    fwht_regs<E>(v, buf);
#pragma unroll
    for (int k = 0; k < E; k++) {
        v[k] *= a.scale[which];
        if (a.sv[which]) v[k] *= sg[k];
        vals[jB + k] = __half2float(__float2half_rn(v[k]));
    }
    __syncthreads();
}

__global__ void __launch_bounds__(1024) qkv_post_kernel(const QkvPostArgs a) {
    extern __shared__ __align__(16) float sm_post[];
    const int which = blockIdx.x, width = a.width[which];
    float *buf = sm_post, *vals = sm_post + width + 128;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    switch (width >> 10) {
        case 1: qkv_transform<1>(a, which, buf, vals); break;
        case 2: qkv_transform<2>(a, which, buf, vals); break;
        case 4: qkv_transform<4>(a, which, buf, vals); break;
        case 8: qkv_transform<8>(a, which, buf, vals); break;
        default: qkv_transform<16>(a, which, buf, vals); break;
    }
    const int pos = *a.pos, hd = a.hd, half = hd >> 1;
    if (!position_ok(pos, a.max_pos, a.status)) return;
    const size_t crow = (size_t)pos * a.n_kv * hd;
    if (which == 2) {
        for (int e = threadIdx.x * 2; e < width; e += blockDim.x * 2)
            *reinterpret_cast<__half2 *>(a.cache_v + crow + e) = __floats2half2_rn(vals[e], vals[e + 1]);
        return;
    }
    __half *dst = which == 0 ? a.q_out : a.cache_k + crow;
    for (int idx = threadIdx.x; idx < (width >> 1); idx += blockDim.x) {
        const int head = idx / half, i = idx - head * half;
        const float inv_freq = exp2f(-a.log2_theta * (float)(2 * i) / (float)hd);
        float sn, cs;
        sincosf((float)pos * inv_freq, &sn, &cs);
        const float x0 = vals[head * hd + i], x1 = vals[head * hd + i + half];
        dst[(size_t)head * hd + i] = __float2half_rn(x0 * cs - x1 * sn);
        dst[(size_t)head * hd + i + half] = __float2half_rn(x1 * cs + x0 * sn);
    }
}

// One CTA per query head, 512 threads = 32 groups of 16 lanes; a lane owns 8 of the 128 head dimensions
// (one 16-byte load per cache row), a group owns cache positions g, g+32, ...  The cache is read in
// batches of 8 rows per group with all loads of a batch in flight at once: at decode lengths the kernel
// is a handful of L2 round trips, not one per position.  Per chunk of kAttnChunk positions:
//   scores -> shared memory, chunk maximum, p = exp(s - max) and its sum, then the weighted sum of V
// (whose first batch is requested before the two block-wide reductions).  Chunks are merged with the
// usual running maximum / denominator.  out: (n_heads, hd) fp16.
constexpr int kAttnThreads = 512, kAttnGroups = kAttnThreads / 16, kAttnChunk = 2048, kAttnBatch = 8;

__device__ __forceinline__ void unpack8(const uint4 &r, float (&f)[8]) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&r);
#pragma unroll
    for (int i = 0; i < 4; i++) { f[2 * i] = __low2float(h[i]); f[2 * i + 1] = __high2float(h[i]); }
}

__global__ void __launch_bounds__(kAttnThreads)
    attn_decode_kernel(__half *__restrict__ out, const __half *__restrict__ q, const __half *__restrict__ cache_k,
                       const __half *__restrict__ cache_v, const int *__restrict__ pos_ptr, int n_heads, int n_kv,
                       float scale, int max_pos, unsigned *status) {
    constexpr int hd = 128, G = kAttnGroups, U = kAttnBatch;
    __shared__ float sc[kAttnChunk];
    __shared__ float red_max[kAttnThreads / 32], red_sum[kAttnThreads / 32];
    __shared__ float accs[G][hd + 4];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int head = blockIdx.x, kvh = head / (n_heads / n_kv);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, grp = tid >> 4, sub = tid & 15;
    if (!position_ok(*pos_ptr, max_pos, status)) return;
    const int ctx = *pos_ptr + 1;
    const size_t row = (size_t)n_kv * hd;
    float qv[8];
    unpack8(__ldg(reinterpret_cast<const uint4 *>(q + (size_t)head * hd + sub * 8)), qv);
#pragma unroll
    for (int i = 0; i < 8; i++) qv[i] *= scale;
    const __half *kb = cache_k + (size_t)kvh * hd + sub * 8, *vb = cache_v + (size_t)kvh * hd + sub * 8;

    float m_run = -INFINITY, d_run = 0.f, acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int c0 = 0; c0 < ctx; c0 += kAttnChunk) {
        const int cn = min(kAttnChunk, ctx - c0);
        // ---- scores of the chunk
        float lmax = -INFINITY;
        // the trip count and every shuffle are uniform over the CTA: a warp holds two groups whose
        // positions may fall on different sides of cn, so validity is a predicate, never a branch
        // around a warp-wide shuffle
        for (int tb = 0; tb < cn; tb += U * G) {
            uint4 kr[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int t = tb + grp + u * G;
                kr[u] = make_uint4(0u, 0u, 0u, 0u);
                if (t < cn) kr[u] = __ldg(reinterpret_cast<const uint4 *>(kb + (size_t)(c0 + t) * row));
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int t = tb + grp + u * G;
                float kf[8], s = 0.f;
                unpack8(kr[u], kf);
#pragma unroll
                for (int i = 0; i < 8; i++) s = fmaf(qv[i], kf[i], s);
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(kFullMask, s, o);
                if (t < cn) {
                    if (sub == 0) sc[t] = s;
                    lmax = fmaxf(lmax, s);
                }
            }
        }
        // first batch of V rows: in flight during the reductions below
        uint4 vr[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int t = grp + u * G;
            if (t < cn) vr[u] = __ldg(reinterpret_cast<const uint4 *>(vb + (size_t)(c0 + t) * row));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) lmax = fmaxf(lmax, __shfl_xor_sync(kFullMask, lmax, o));
        if (lane == 0) red_max[warp] = lmax;
        __syncthreads();
        float cmax = red_max[0];
#pragma unroll
        for (int w = 1; w < kAttnThreads / 32; w++) cmax = fmaxf(cmax, red_max[w]);
        const float m_new = fmaxf(m_run, cmax);
        const float corr = __expf(m_run - m_new);      // 0 for the first chunk
        float lsum = 0.f;
        for (int t = tid; t < cn; t += kAttnThreads) {
            const float pr = __expf(sc[t] - m_new);
            sc[t] = pr;
            lsum += pr;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) lsum += __shfl_xor_sync(kFullMask, lsum, o);
        if (lane == 0) red_sum[warp] = lsum;
        __syncthreads();
        float csum = 0.f;
#pragma unroll
        for (int w = 0; w < kAttnThreads / 32; w++) csum += red_sum[w];
        d_run = d_run * corr + csum;
        m_run = m_new;
#pragma unroll
        for (int i = 0; i < 8; i++) acc[i] *= corr;
        // ---- weighted sum of V
        for (int tb = 0; tb < cn; tb += U * G) {
            uint4 cur[U];
#pragma unroll
            for (int u = 0; u < U; u++) cur[u] = vr[u];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int t = tb + U * G + grp + u * G;
                if (t < cn) vr[u] = __ldg(reinterpret_cast<const uint4 *>(vb + (size_t)(c0 + t) * row));
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int t = tb + grp + u * G;
                if (t < cn) {
                    float vf[8];
                    unpack8(cur[u], vf);
                    const float pr = sc[t];
#pragma unroll
                    for (int i = 0; i < 8; i++) acc[i] = fmaf(pr, vf[i], acc[i]);
                }
            }
        }
        __syncthreads();    // sc and the reduction slots are reused by the next chunk
    }
#pragma unroll
    for (int i = 0; i < 8; i++) accs[grp][sub * 8 + i] = acc[i];
    __syncthreads();
    if (tid < hd) {
        float a = 0.f;
#pragma unroll
        for (int g = 0; g < G; g++) a += accs[g][tid];
        out[(size_t)head * hd + tid] = __float2half_rn(a / d_run);
    }
}

// attn_decode_kernel with everything between the q/k/v matvecs and the attention in front of it, so that a
// decoder layer needs no separate rotary / cache launch.  The Walsh-Hadamard transform over a width
// n_heads * 128 factors into one over the head index and one over the 128 values of a head, so the CTA of head h
// only needs  z[d] = sum_h2 (-1)^popc(h & h2) * y[h2*128 + d]  (a signed sum over heads, every CTA reads all of y)
// followed by a 128-point transform in one warp.  It does this for its q head and for its k / v head, applies
// sign * scale, rounds to fp16 like the linear's output tensor, rotates q and k, and the first q head of each
// k/v group appends k and v to the cache.  Attention then runs over cache rows 0..pos-1 plus the new row, which
// is taken from shared memory (the cache write of another CTA may not have landed).
struct AttnFusedArgs {
    const float *y_q, *y_k, *y_v, *sv_q, *sv_k, *sv_v;
    float scale_q, scale_kv;
    __half *out, *cache_k, *cache_v;
    const int *pos;
    int n_heads, n_kv;
    float log2_theta, softmax_scale;
    int max_pos;
    unsigned *status;
};

__global__ void __launch_bounds__(kAttnThreads) attn_decode_fused_kernel(const AttnFusedArgs a) {
    constexpr int hd = 128, G = kAttnGroups, U = kAttnBatch;
    __shared__ float sc[kAttnChunk + 1];
    __shared__ float red_max[kAttnThreads / 32], red_sum[kAttnThreads / 32];
    __shared__ float accs[G][hd + 4];
    __shared__ float part[3][4][hd];          // signed head sums of q, k, v: four partial sums each
    __shared__ __align__(16) float cur[3][hd];   // this position's q (rotated, pre-scaled), k (rotated), v
    const int head = blockIdx.x, rep = a.n_heads / a.n_kv, kvh = head / rep;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, grp = tid >> 4, sub = tid & 15;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int pos = *a.pos;
    if (!position_ok(pos, a.max_pos, a.status)) return;

    // ---- signed sums over heads: thread (quarter, d) adds a quarter of the heads (all three loads batches in flight)
    {
        const int d = tid & (hd - 1), quarter = tid >> 7;
        float s3[3];
#pragma unroll
        for (int w = 0; w < 3; w++) {
            const float *y = w == 0 ? a.y_q : w == 1 ? a.y_k : a.y_v;
            const int nh = w == 0 ? a.n_heads : a.n_kv, h = w == 0 ? head : kvh;
            const int per = (nh + 3) >> 2, h0 = quarter * per, h1 = min(nh, h0 + per);
            float s = 0.f;
#pragma unroll 8
            for (int h2 = h0; h2 < h1; h2++) {
                const float v = __ldcg(y + (size_t)h2 * hd + d);
                s += (__popc(h & h2) & 1) ? -v : v;
            }
            s3[w] = s;
        }
#pragma unroll
        for (int w = 0; w < 3; w++) part[w][quarter][d] = s3[w];
    }
    __syncthreads();
    if (warp < 3) {
        // warp 0: q, warp 1: k, warp 2: v.  Lane l holds d = l + 32*e, so the rotary partner d + 64 is e + 2.
        const int w = warp;
        const float *sv = w == 0 ? a.sv_q : w == 1 ? a.sv_k : a.sv_v;
        const int h = w == 0 ? head : kvh;
        const float scale = w == 0 ? a.scale_q : a.scale_kv;
        float v[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int d = lane + 32 * e;
            v[e] = part[w][0][d] + part[w][1][d] + part[w][2][d] + part[w][3][d];
        }
        fwht_warp<4>(v, lane);
#pragma unroll
        for (int e = 0; e < 4; e++) {
            v[e] *= scale;
            if (sv) v[e] *= sv[(size_t)h * hd + lane + 32 * e];
            v[e] = __half2float(__float2half_rn(v[e]));           // the linear's output is an fp16 tensor
        }
        if (w < 2) {
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int i = lane + 32 * e;
                const float inv_freq = exp2f(-a.log2_theta * (float)(2 * i) / (float)hd);
                float sn, cs;
                sincosf((float)pos * inv_freq, &sn, &cs);
                const float x0 = v[e], x1 = v[e + 2];
                v[e] = __half2float(__float2half_rn(x0 * cs - x1 * sn));
                v[e + 2] = __half2float(__float2half_rn(x1 * cs + x0 * sn));
            }
        }
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int d = lane + 32 * e;
            cur[w][d] = w == 0 ? v[e] * a.softmax_scale : v[e];
            if (w > 0 && head == kvh * rep) {
                __half *cache = w == 1 ? a.cache_k : a.cache_v;
                cache[(size_t)pos * a.n_kv * hd + (size_t)kvh * hd + d] = __float2half_rn(v[e]);
            }
        }
    }
    __syncthreads();

    // ---- attention over rows 0..pos (row pos from shared memory)
    const int ctx = pos + 1;
    const size_t row = (size_t)a.n_kv * hd;
    float qv[8];
#pragma unroll
    for (int i = 0; i < 8; i++) qv[i] = cur[0][sub * 8 + i];
    const __half *kb = a.cache_k + (size_t)kvh * hd + sub * 8, *vb = a.cache_v + (size_t)kvh * hd + sub * 8;
    auto load_row = [&](const __half *base, const float *fresh, int t_global, float (&f)[8], const uint4 &raw) {
        if (t_global == pos) {
#pragma unroll
            for (int i = 0; i < 8; i++) f[i] = fresh[sub * 8 + i];
        } else {
            unpack8(raw, f);
        }
    };
    float m_run = -INFINITY, d_run = 0.f, acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int c0 = 0; c0 < ctx; c0 += kAttnChunk) {
        const int cn = min(kAttnChunk, ctx - c0);
        float lmax = -INFINITY;
        for (int tb = 0; tb < cn; tb += U * G) {
            uint4 kr[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int t = tb + grp + u * G;
                kr[u] = make_uint4(0u, 0u, 0u, 0u);
                if (t < cn && c0 + t < pos) kr[u] = __ldg(reinterpret_cast<const uint4 *>(kb + (size_t)(c0 + t) * row));
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int t = tb + grp + u * G;
                float kf[8], s = 0.f;
                load_row(kb, cur[1], c0 + t, kf, kr[u]);
#pragma unroll
                for (int i = 0; i < 8; i++) s = fmaf(qv[i], kf[i], s);
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(kFullMask, s, o);
                if (t < cn) {
                    if (sub == 0) sc[t] = s;
                    lmax = fmaxf(lmax, s);
                }
            }
        }
        uint4 vr[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int t = grp + u * G;
            vr[u] = make_uint4(0u, 0u, 0u, 0u);
            if (t < cn && c0 + t < pos) vr[u] = __ldg(reinterpret_cast<const uint4 *>(vb + (size_t)(c0 + t) * row));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) lmax = fmaxf(lmax, __shfl_xor_sync(kFullMask, lmax, o));
        if (lane == 0) red_max[warp] = lmax;
        __syncthreads();
        float cmax = red_max[0];
#pragma unroll
        for (int w = 1; w < kAttnThreads / 32; w++) cmax = fmaxf(cmax, red_max[w]);
        const float m_new = fmaxf(m_run, cmax);
        const float corr = __expf(m_run - m_new);
        float lsum = 0.f;
        for (int t = tid; t < cn; t += kAttnThreads) {
            const float pr = __expf(sc[t] - m_new);
            sc[t] = pr;
            lsum += pr;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) lsum += __shfl_xor_sync(kFullMask, lsum, o);
        if (lane == 0) red_sum[warp] = lsum;
        __syncthreads();
        float csum = 0.f;
#pragma unroll
        for (int w = 0; w < kAttnThreads / 32; w++) csum += red_sum[w];
        d_run = d_run * corr + csum;
        m_run = m_new;
#pragma unroll
        for (int i = 0; i < 8; i++) acc[i] *= corr;
        for (int tb = 0; tb < cn; tb += U * G) {
            uint4 curv[U];
#pragma unroll
            for (int u = 0; u < U; u++) curv[u] = vr[u];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int t = tb + U * G + grp + u * G;
                if (t < cn && c0 + t < pos) vr[u] = __ldg(reinterpret_cast<const uint4 *>(vb + (size_t)(c0 + t) * row));
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int t = tb + grp + u * G;
                if (t < cn) {
                    float vf[8];
                    load_row(vb, cur[2], c0 + t, vf, curv[u]);
                    const float pr = sc[t];
#pragma unroll
                    for (int i = 0; i < 8; i++) acc[i] = fmaf(pr, vf[i], acc[i]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 8; i++) accs[grp][sub * 8 + i] = acc[i];
    __syncthreads();
    if (tid < hd) {
        float s = 0.f;
#pragma unroll
        for (int g = 0; g < G; g++) s += accs[g][tid];
        a.out[(size_t)head * hd + tid] = __float2half_rn(s / d_run);
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
                                   int n_heads, int n_kv_heads, int head_dim, float theta, int max_positions,
                                   unsigned *status, void *stream) {
    if (!q || !k || !v || !cache_k || !cache_v || !pos || max_positions <= 0) return QTIP_ERR_BAD_ARG;
    if (n_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || (head_dim & 1) || n_heads % n_kv_heads) return QTIP_ERR_BAD_SHAPE;
    const int total = (n_heads + n_kv_heads) * (head_dim / 2);
    return launch_pdl(rope_kv_kernel, dim3((total + 255) / 256), dim3(256), static_cast<cudaStream_t>(stream),
                      static_cast<__half *>(q), static_cast<const __half *>(k), static_cast<const __half *>(v),
                      static_cast<__half *>(cache_k), static_cast<__half *>(cache_v), pos, n_heads, n_kv_heads, head_dim,
                      log2f(theta), max_positions, status);
}

extern "C" int qtip_rope_kv_append_fused(void *q_out, const float *y_q, const float *y_k, const float *y_v,
                                         const float *sign_q, const float *sign_k, const float *sign_v, float scale_q,
                                         float scale_kv, void *cache_k, void *cache_v, const int *pos, int n_heads,
                                         int n_kv_heads, int head_dim, float theta, int max_positions,
                                         unsigned *status, void *stream) {
    if (!q_out || !y_q || !y_k || !y_v || !cache_k || !cache_v || !pos || max_positions <= 0) return QTIP_ERR_BAD_ARG;
    if (n_heads <= 0 || n_kv_heads <= 0 || head_dim <= 0 || (head_dim & 1) || n_heads % n_kv_heads) return QTIP_ERR_BAD_SHAPE;
    const int wq = n_heads * head_dim, wkv = n_kv_heads * head_dim;
    auto ok_width = [](int w) { return w == 1024 || w == 2048 || w == 4096 || w == 8192 || w == 16384; };
    if (!ok_width(wq) || !ok_width(wkv)) return QTIP_ERR_BAD_SHAPE;
    const void *ptrs[] = {q_out, y_q, y_k, y_v, sign_q, sign_k, sign_v, cache_k, cache_v};
    for (const void *p : ptrs)
        if (p && !aligned(p, 16)) return QTIP_ERR_ALIGNMENT;
    QkvPostArgs a = {};
    a.y[0] = y_q; a.y[1] = y_k; a.y[2] = y_v;
    a.sv[0] = sign_q; a.sv[1] = sign_k; a.sv[2] = sign_v;
    a.scale[0] = scale_q; a.scale[1] = scale_kv; a.scale[2] = scale_kv;
    a.width[0] = wq; a.width[1] = wkv; a.width[2] = wkv;
    a.q_out = static_cast<__half *>(q_out); a.cache_k = static_cast<__half *>(cache_k); a.cache_v = static_cast<__half *>(cache_v);
    a.pos = pos; a.n_heads = n_heads; a.n_kv = n_kv_heads; a.hd = head_dim; a.log2_theta = log2f(theta);
    a.max_pos = max_positions; a.status = status;
    const size_t smem = (size_t)(2 * wq + 128) * sizeof(float);
    static bool attr_set[64] = {};
    int dev = 0;
    QTIP_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 64 && !attr_set[dev]) {
        QTIP_CUDA_TRY(cudaFuncSetAttribute(qkv_post_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (2 * 16384 + 128) * 4));
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(3);
    cfg.blockDim = dim3(1024);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    QTIP_CUDA_TRY(cudaLaunchKernelEx(&cfg, qkv_post_kernel, a));
    return check_launch();
}

extern "C" int qtip_attn_decode(void *out, const void *q, const void *cache_k, const void *cache_v, const int *pos,
                                int n_heads, int n_kv_heads, int head_dim, int max_positions, unsigned *status,
                                void *stream) {
    if (!out || !q || !cache_k || !cache_v || !pos || max_positions <= 0) return QTIP_ERR_BAD_ARG;
    if (head_dim != 128 || n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads) return QTIP_ERR_BAD_SHAPE;
    if (!aligned(q, 16) || !aligned(cache_k, 16) || !aligned(cache_v, 16)) return QTIP_ERR_ALIGNMENT;
    return launch_pdl(attn_decode_kernel, dim3(n_heads), dim3(kAttnThreads), static_cast<cudaStream_t>(stream),
                      static_cast<__half *>(out), static_cast<const __half *>(q), static_cast<const __half *>(cache_k),
                      static_cast<const __half *>(cache_v), pos, n_heads, n_kv_heads, 1.0f / sqrtf((float)head_dim),
                      max_positions, status);
}

extern "C" int qtip_attn_decode_fused(void *out, const float *y_q, const float *y_k, const float *y_v, const float *sign_q,
                                      const float *sign_k, const float *sign_v, float scale_q, float scale_kv,
                                      void *cache_k, void *cache_v, const int *pos, int n_heads, int n_kv_heads,
                                      int head_dim, float theta, int max_positions, unsigned *status, void *stream) {
    if (!out || !y_q || !y_k || !y_v || !cache_k || !cache_v || !pos || max_positions <= 0) return QTIP_ERR_BAD_ARG;
    if (head_dim != 128 || n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads) return QTIP_ERR_BAD_SHAPE;
    if ((n_heads & (n_heads - 1)) || (n_kv_heads & (n_kv_heads - 1))) return QTIP_ERR_BAD_SHAPE;   // Hadamard over heads
    if (!aligned(cache_k, 16) || !aligned(cache_v, 16) || !aligned(y_q, 4)) return QTIP_ERR_ALIGNMENT;
    AttnFusedArgs a = {};
    a.y_q = y_q; a.y_k = y_k; a.y_v = y_v; a.sv_q = sign_q; a.sv_k = sign_k; a.sv_v = sign_v;
    a.scale_q = scale_q; a.scale_kv = scale_kv;
    a.out = static_cast<__half *>(out); a.cache_k = static_cast<__half *>(cache_k); a.cache_v = static_cast<__half *>(cache_v);
    a.pos = pos; a.n_heads = n_heads; a.n_kv = n_kv_heads; a.log2_theta = log2f(theta);
    a.softmax_scale = 1.0f / sqrtf((float)head_dim);
    a.max_pos = max_positions; a.status = status;
    return launch_pdl(attn_decode_fused_kernel, dim3(n_heads), dim3(kAttnThreads), static_cast<cudaStream_t>(stream), a);
}
