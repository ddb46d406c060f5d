// Shared device/host helpers for the qtip_b200 kernels (sm_100a).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/qtip_b200.h"

namespace qtip {

// ---- host-side status plumbing -------------------------------------------------------------
void set_last_cuda_error(cudaError_t e);

inline int check_launch() {
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
        set_last_cuda_error(e);
        (void)cudaGetLastError();
        return QTIP_ERR_CUDA;
    }
    return QTIP_OK;
}

#define QTIP_CUDA_TRY(expr)                         \
    do {                                            \
        cudaError_t _e = (expr);                    \
        if (_e != cudaSuccess) {                    \
            ::qtip::set_last_cuda_error(_e);        \
            return QTIP_ERR_CUDA;                   \
        }                                           \
    } while (0)

inline bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// Number of SMs of the current device (cached per device; a property query on every launch is
// host overhead the upstream launcher pays, qtip-kernels/src/inference.cu:451-452).
int sm_count();

// ---- device helpers ------------------------------------------------------------------------
constexpr unsigned kFullMask = 0xFFFFFFFFu;

// HYB state function (lib/codebook/bitshift.py:72-80 upstream): h = s*(s+1) mod 2^16 where only
// the low 16 bits of `t` need to hold the state; LUT entry (h >> 6) & 511, sign of the first
// weight flipped when bit 15 of h is set.
__device__ __forceinline__ uint32_t hyb_hash(uint32_t t) { return t * t + t; }

// 3INST (lib/codebook/bitshift.py:43-60): two fp16 bit patterns masked out of an LCG, summed in fp16.
__device__ __forceinline__ __half decode_3inst(uint32_t s16) {
    uint32_t x = s16 * 89226354u + 64248484u;
    uint32_t r = (x & 0x8FFF8FFFu) ^ 0x3B603B60u;
    __half2 h = *reinterpret_cast<__half2 *>(&r);
    return __hadd(__low2half(h), __high2half(h));
}

// 1MAD (lib/codebook/bitshift.py:17-26): (byte sum of an LCG - 510) / 147.800537109375 in fp32
// (IEEE divide), rounded once to fp16.
__device__ __forceinline__ __half decode_1mad(uint32_t s16) {
    uint32_t x = s16 * 34038481u + 76625530u;
    int y = (int)__vsadu4(x, 0u) - 510;
    return __float2half_rn(__fdiv_rn((float)y, 147.800537109375f));
}

// The same value from a table over the 1021 possible byte sums (built with decode_1mad's own arithmetic, so it is
// bit-identical): one shared-memory load instead of a convert, an IEEE divide and a second convert.
constexpr int kMadTableEntries = 1024;
__device__ __forceinline__ void build_1mad_table(__half *tab) {
    for (int i = threadIdx.x; i < kMadTableEntries; i += blockDim.x)
        tab[i] = __float2half_rn(__fdiv_rn((float)(i - 510), 147.800537109375f));
}
__device__ __forceinline__ __half decode_1mad_tab(uint32_t s16, const __half *tab) {
    const uint32_t x = s16 * 34038481u + 76625530u;
    return tab[__vsadu4(x, 0u)];
}

// Streaming (read-once) global loads of packed codes: keep them out of L1.
__device__ __forceinline__ uint32_t ld_stream_u32(const void *p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ld_stream_u32x2(const void *p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ld_stream_u32x4(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// A lane's 4*K bytes of one 2x2 tile block in the kernel layout: [k-subtile 2][m-subtile 2][K bytes].
template <int K>
struct LaneCodes {
    uint32_t w[K];
};

template <int K>
__device__ __forceinline__ LaneCodes<K> load_lane_codes(const uint8_t *p) {
    LaneCodes<K> c;
    if constexpr (K == 2) {
        uint2 v = ld_stream_u32x2(p);
        c.w[0] = v.x; c.w[1] = v.y;
    } else if constexpr (K == 3) {
        c.w[0] = ld_stream_u32(p); c.w[1] = ld_stream_u32(p + 4); c.w[2] = ld_stream_u32(p + 8);
    } else {
        uint4 v = ld_stream_u32x4(p);
        c.w[0] = v.x; c.w[1] = v.y; c.w[2] = v.z; c.w[3] = v.w;
    }
    return c;
}

template <int K>
__device__ __forceinline__ LaneCodes<K> shfl_next_lane(const LaneCodes<K> &c, int lane) {
    LaneCodes<K> o;
#pragma unroll
    for (int i = 0; i < K; i++) o.w[i] = __shfl_sync(kFullMask, c.w[i], (lane + 1) & 31);
    return o;
}

// Slice t (= ks*2 + ms) of a lane: K bytes read as a little-endian integer, i.e. 8K stream bits
// with the first bit as MSB.
template <int K>
__device__ __forceinline__ uint32_t lane_slice(const LaneCodes<K> &c, int t) {
    if constexpr (K == 2) {
        return (t & 1) ? (c.w[t >> 1] >> 16) : (c.w[t >> 1] & 0xFFFFu);
    } else if constexpr (K == 3) {
        switch (t) {
            case 0: return c.w[0] & 0xFFFFFFu;
            case 1: return __funnelshift_r(c.w[0], c.w[1], 24) & 0xFFFFFFu;
            case 2: return __funnelshift_r(c.w[1], c.w[2], 16) & 0xFFFFFFu;
            default: return c.w[2] >> 8;
        }
    } else {
        return c.w[t];
    }
}

// The four 16-bit states of (lane, tile t): windows at bit offsets 0, 2K, 4K, 6K of own-slice || next-slice.
// Only the low 16 bits of each returned value are meaningful.
template <int K>
__device__ __forceinline__ void lane_states(uint32_t own, uint32_t next, uint32_t (&st)[4]) {
    uint64_t win = ((uint64_t)own << (8 * K)) | next;
#pragma unroll
    for (int q = 0; q < 4; q++) st[q] = (uint32_t)(win >> (16 * K - 16 - 2 * K * q));
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
// instructions are integer multiply-adds: one instruction each where shift + add or shift + or would take two
// (multiply-add, logic and shift instructions all issue at one warp-instruction per two cycles per sub-partition).
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


}  // namespace qtip
