// Walsh-Hadamard transform of a vector held in (padded) shared memory, shared by the RHT kernel and the
// fused prologue / epilogue of the matvec kernel.
#pragma once

#include "common.cuh"

namespace qtip {

// Shared-memory index with one pad word per 32: a thread that walks 16 consecutive values (first
// butterfly pass) then hits 32 different banks across a warp instead of 2.
__device__ __forceinline__ int pad(int i) { return i + (i >> 5); }

template <int R>
__device__ __forceinline__ void butterfly_pass(float *v, int n, int b) {
    constexpr int E = 1 << R;
    const int groups = n >> R;
    for (int gidx = threadIdx.x; gidx < groups; gidx += blockDim.x) {
        const int lo = gidx & ((1 << b) - 1), hi = gidx >> b;
        const int base = (hi << (b + R)) | lo;
        float e[E];
#pragma unroll
        for (int k = 0; k < E; k++) e[k] = v[pad(base + (k << b))];
#pragma unroll
        for (int s = 0; s < R; s++) {
#pragma unroll
            for (int k = 0; k < E; k++) {
                if (!(k & (1 << s))) {
                    float a0 = e[k], a1 = e[k | (1 << s)];
                    e[k] = a0 + a1;
                    e[k | (1 << s)] = a0 - a1;
                }
            }
        }
#pragma unroll
        for (int k = 0; k < E; k++) v[pad(base + (k << b))] = e[k];
    }
}

// Unnormalised transform over the 2^p-long segments of v[0, n) (all threads of the CTA; starts and ends
// with the data visible to every thread, i.e. contains the barriers it needs after the first pass).
__device__ __forceinline__ void fwht_shared(float *v, int n, int p) {
    for (int b = 0; b < p;) {
        const int r = (p - b) >= 4 ? 4 : (p - b);
        switch (r) {
            case 4: butterfly_pass<4>(v, n, b); break;
            case 3: butterfly_pass<3>(v, n, b); break;
            case 2: butterfly_pass<2>(v, n, b); break;
            default: butterfly_pass<1>(v, n, b); break;
        }
        b += r;
        __syncthreads();
    }
}

// 8 consecutive values starting at element i (i % 8 == 0, pointer 16-byte aligned)
__device__ __forceinline__ void load8_f16(const __half *p, size_t i, float (&o)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4 *>(p + i);
    const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
    for (int k = 0; k < 4; k++) { o[2 * k] = __low2float(h[k]); o[2 * k + 1] = __high2float(h[k]); }
}
__device__ __forceinline__ void load8_f32(const float *p, size_t i, float (&o)[8]) {
    const float4 a = *reinterpret_cast<const float4 *>(p + i), b = *reinterpret_cast<const float4 *>(p + i + 4);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
__device__ __forceinline__ void store8_f16(__half *p, size_t i, const float (&o)[8]) {
    uint4 raw;
    __half2 *h = reinterpret_cast<__half2 *>(&raw);
#pragma unroll
    for (int k = 0; k < 4; k++) h[k] = __floats2half2_rn(o[2 * k], o[2 * k + 1]);
    *reinterpret_cast<uint4 *>(p + i) = raw;
}
__device__ __forceinline__ void store8_f32(float *p, size_t i, const float (&o)[8]) {
    *reinterpret_cast<float4 *>(p + i) = make_float4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<float4 *>(p + i + 4) = make_float4(o[4], o[5], o[6], o[7]);
}

// Walsh-Hadamard transform of n = 1024*E values held in the registers of a 1024-thread CTA.
// In : thread (warp w, lane l) holds elements (w*32 + l)*E + r, r < E   (E consecutive values).
// Out: thread (w, l) holds elements (l*32 + w)*E + r                      (warp and lane swapped).
// Butterflies over the low log2(E) index bits run in registers, over the 5 lane bits with shuffles; one
// pass through shared memory (buf: 32*(32E+4) floats; rows padded by 4 words so that 16-byte accesses of
// 8 lanes cover all banks) swaps the warp and lane bits, then the shuffles run again.  Contains one barrier.
template <int E>
__device__ __forceinline__ void fwht_regs(float (&v)[E], float *buf) {
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
#pragma unroll
    for (int s = 1; s < E; s <<= 1)
#pragma unroll
        for (int k = 0; k < E; k++)
            if (!(k & s)) { const float a = v[k], b = v[k | s]; v[k] = a + b; v[k | s] = a - b; }
#pragma unroll
    for (int bit = 1; bit < 32; bit <<= 1)
#pragma unroll
        for (int k = 0; k < E; k++) {
            const float o = __shfl_xor_sync(kFullMask, v[k], bit);
            v[k] = (l & bit) ? o - v[k] : v[k] + o;
        }
    constexpr int kRow = 32 * E + 4;
    float *dst = buf + w * kRow + l * E;
    if constexpr (E >= 4) {
#pragma unroll
        for (int k = 0; k < E; k += 4) *reinterpret_cast<float4 *>(dst + k) = make_float4(v[k], v[k + 1], v[k + 2], v[k + 3]);
    } else {
#pragma unroll
        for (int k = 0; k < E; k++) dst[k] = v[k];
    }
    __syncthreads();
    const float *src = buf + l * kRow + w * E;
    if constexpr (E >= 4) {
#pragma unroll
        for (int k = 0; k < E; k += 4) {
            const float4 q = *reinterpret_cast<const float4 *>(src + k);
            v[k] = q.x; v[k + 1] = q.y; v[k + 2] = q.z; v[k + 3] = q.w;
        }
    } else {
#pragma unroll
        for (int k = 0; k < E; k++) v[k] = src[k];
    }
#pragma unroll
    for (int bit = 1; bit < 32; bit <<= 1)
#pragma unroll
        for (int k = 0; k < E; k++) {
            const float o = __shfl_xor_sync(kFullMask, v[k], bit);
            v[k] = (l & bit) ? o - v[k] : v[k] + o;
        }
}

// E consecutive values starting at element i (i % E == 0, pointers aligned to E elements).
// The fp32 load takes E = 1, 2 or a multiple of 4; the fp16 forms and the stores E = 4 or a multiple of 8.
template <int E>
__device__ __forceinline__ void loadE_f16(const __half *p, size_t i, float (&o)[E]) {
    if constexpr (E == 4) {
        const uint2 raw = *reinterpret_cast<const uint2 *>(p + i);
        const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
        o[0] = __low2float(h[0]); o[1] = __high2float(h[0]); o[2] = __low2float(h[1]); o[3] = __high2float(h[1]);
    } else {
#pragma unroll
        for (int k = 0; k < E; k += 8) {
            float t[8];
            load8_f16(p, i + k, t);
#pragma unroll
            for (int q = 0; q < 8; q++) o[k + q] = t[q];
        }
    }
}
template <int E>
__device__ __forceinline__ void loadE_f32(const float *p, size_t i, float (&o)[E], bool bypass_l1) {
    if constexpr (E == 1) {
        o[0] = bypass_l1 ? __ldcg(p + i) : p[i];
    } else if constexpr (E == 2) {
        const float2 *q = reinterpret_cast<const float2 *>(p + i);
        const float2 a = bypass_l1 ? __ldcg(q) : *q;
        o[0] = a.x; o[1] = a.y;
    } else {
#pragma unroll
        for (int k = 0; k < E; k += 4) {
            const float4 *q = reinterpret_cast<const float4 *>(p + i + k);
            const float4 a = bypass_l1 ? __ldcg(q) : *q;
            o[k] = a.x; o[k + 1] = a.y; o[k + 2] = a.z; o[k + 3] = a.w;
        }
    }
}
template <int E>
__device__ __forceinline__ void storeE_f16(__half *p, size_t i, const float (&o)[E]) {
    if constexpr (E == 4) {
        uint2 raw;
        __half2 *h = reinterpret_cast<__half2 *>(&raw);
        h[0] = __floats2half2_rn(o[0], o[1]); h[1] = __floats2half2_rn(o[2], o[3]);
        *reinterpret_cast<uint2 *>(p + i) = raw;
    } else {
#pragma unroll
        for (int k = 0; k < E; k += 8) {
            float t[8];
#pragma unroll
            for (int q = 0; q < 8; q++) t[q] = o[k + q];
            store8_f16(p, i + k, t);
        }
    }
}
template <int E>
__device__ __forceinline__ void storeE_f32(float *p, size_t i, const float (&o)[E]) {
#pragma unroll
    for (int k = 0; k < E; k += 4) *reinterpret_cast<float4 *>(p + i + k) = make_float4(o[k], o[k + 1], o[k + 2], o[k + 3]);
}

// Walsh-Hadamard transform over the 32*E values of a warp; lane l holds j = l + 32*e
template <int E>
__device__ __forceinline__ void fwht_warp(float (&v)[E], int lane) {
#pragma unroll
    for (int s = 1; s < E; s <<= 1)
#pragma unroll
        for (int k = 0; k < E; k++)
            if (!(k & s)) { const float a = v[k], b = v[k | s]; v[k] = a + b; v[k | s] = a - b; }
#pragma unroll
    for (int bit = 1; bit < 32; bit <<= 1)
#pragma unroll
        for (int k = 0; k < E; k++) {
            const float o = __shfl_xor_sync(kFullMask, v[k], bit);
            v[k] = (lane & bit) ? o - v[k] : v[k] + o;
        }
}

// Sum over the CTA (scratch: one float per warp).  Contains two barriers.
__device__ __forceinline__ float block_sum(float x, float *scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(kFullMask, x, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) scratch[warp] = x;
    __syncthreads();
    float t = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); w++) t += scratch[w];
    return t;
}

// SwiGLU product as fp16 tensors would compute it: silu(gate) rounded to fp16, product rounded to fp16.
__device__ __forceinline__ float swiglu_fp16(float gate, float up) {
    const __half sg = __float2half_rn(__fdividef(gate, 1.0f + __expf(-gate)));
    return __half2float(__hmul(sg, __float2half_rn(up)));
}

}  // namespace qtip
