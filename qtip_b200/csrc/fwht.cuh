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

// SwiGLU product as fp16 tensors would compute it: silu(gate) rounded to fp16, product rounded to fp16.
__device__ __forceinline__ float swiglu_fp16(float gate, float up) {
    const __half sg = __float2half_rn(__fdividef(gate, 1.0f + __expf(-gate)));
    return __half2float(__hmul(sg, __float2half_rn(up)));
}

}  // namespace qtip
