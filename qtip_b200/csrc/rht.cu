// Randomized Hadamard transform with the sign flips and scales fused on both sides.
//
// One row of n = kfac * 2^p values is transformed entirely in shared memory:
//   1. load, multiply by sign_in;
//   2. Walsh-Hadamard over the 2^p-long segments: radix-16 passes over shared memory
//      (4 butterfly stages per pass in registers);
//   3. kfac > 1: multiply the (kfac, 2^p) view from the left by the +-1 matrix hadK.  This is the
//      only super-linear part (kfac^2 * 2^p adds), so it is spread over several CTAs: CTA (i, r) of
//      the grid repeats steps 1-2 for row r (cheap, data comes from L2) and produces kRowsPerCta
//      output rows of the (kfac, 2^p) view;
//   4. scale, multiply by sign_out, store as fp16 or fp32.
// Replaces hadamard::hadamard + the hadK matmul + the element-wise kernels of
// lib/utils/matmul_had.py:105-119 and lib/codebook/bitshift.py:428-441, 465-471 upstream.
#include "common.cuh"

namespace qtip {
namespace {

constexpr int kRhtThreads = 512;
constexpr int kRowsPerCta = 16;  // hadK output rows per CTA

template <int R>
__device__ __forceinline__ void butterfly_pass(float *v, int n, int b) {
    constexpr int E = 1 << R;
    const int groups = n >> R;
    for (int gidx = threadIdx.x; gidx < groups; gidx += blockDim.x) {
        const int lo = gidx & ((1 << b) - 1), hi = gidx >> b;
        const int base = (hi << (b + R)) | lo;
        float e[E];
#pragma unroll
        for (int k = 0; k < E; k++) e[k] = v[base + (k << b)];
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
        for (int k = 0; k < E; k++) v[base + (k << b)] = e[k];
    }
}

__device__ __forceinline__ float load_elem(const void *p, int dtype, size_t i) {
    return dtype == QTIP_F16 ? __half2float(static_cast<const __half *>(p)[i]) : static_cast<const float *>(p)[i];
}

__global__ void __launch_bounds__(kRhtThreads)
    rht_kernel(void *__restrict__ out, int out_dtype, const void *__restrict__ in, int in_dtype, int n, int p,
               const void *__restrict__ sign_in, int sign_in_dtype, const float *__restrict__ sign_out, int sign_rep,
               const uint32_t *__restrict__ hadk_bits, int kfac, int transpose, float scale) {
    extern __shared__ __align__(16) float sm[];
    float *v = sm;            // n values
    float *hs = sm + n;       // kRowsPerCta x kfac signs (+-1.0f), only when kfac > 1
    const long row = blockIdx.y;
    const size_t sign_off = (size_t)(row % sign_rep) * n;
    const size_t roff = (size_t)row * n;

    for (int j = threadIdx.x; j < n; j += blockDim.x) {
        float x = load_elem(in, in_dtype, roff + j);
        if (sign_in) x *= load_elem(sign_in, sign_in_dtype, sign_off + j);
        v[j] = x;
    }
    const int i0 = blockIdx.x * kRowsPerCta;
    const int rows_here = min(kRowsPerCta, kfac - i0);
    if (kfac > 1) {
        const int wpr = (kfac + 31) >> 5;
        for (int idx = threadIdx.x; idx < rows_here * kfac; idx += blockDim.x) {
            int il = idx / kfac, k = idx % kfac;
            // hadK[i][k], or hadK[k][i] for the transposed (input-side) transform
            int rr = transpose ? k : (i0 + il), cc = transpose ? (i0 + il) : k;
            uint32_t bit = (hadk_bits[rr * wpr + (cc >> 5)] >> (cc & 31)) & 1u;
            hs[il * kfac + k] = bit ? 1.0f : -1.0f;
        }
    }
    __syncthreads();

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

    const int len = 1 << p;
    if (kfac == 1) {
        for (int j = threadIdx.x; j < n; j += blockDim.x) {
            float y = v[j] * scale;
            if (sign_out) y *= sign_out[sign_off + j];
            if (out_dtype == QTIP_F16) static_cast<__half *>(out)[roff + j] = __float2half_rn(y);
            else static_cast<float *>(out)[roff + j] = y;
        }
        return;
    }
    // hadK multiply: output (i0 + il, j) = sum_k hs[il][k] * v[k*len + j]
    const int items = rows_here * len;
    for (int idx = threadIdx.x; idx < items; idx += blockDim.x) {
        const int il = idx / len, j = idx % len;
        const float *hrow = hs + il * kfac;
        float acc0 = 0.f, acc1 = 0.f;
        int k = 0;
        for (; k + 1 < kfac; k += 2) {
            acc0 = fmaf(hrow[k], v[k * len + j], acc0);
            acc1 = fmaf(hrow[k + 1], v[(k + 1) * len + j], acc1);
        }
        if (k < kfac) acc0 = fmaf(hrow[k], v[k * len + j], acc0);
        const size_t o = (size_t)(i0 + il) * len + j;
        float y = (acc0 + acc1) * scale;
        if (sign_out) y *= sign_out[sign_off + o];
        if (out_dtype == QTIP_F16) static_cast<__half *>(out)[roff + o] = __float2half_rn(y);
        else static_cast<float *>(out)[roff + o] = y;
    }
}

bool valid_kfac(int k) {
    static const int ks[] = {1, 12, 20, 28, 36, 52, 60, 108, 116, 124, 140, 156, 172};
    for (int v : ks)
        if (v == k) return true;
    return false;
}

}  // namespace
}  // namespace qtip

using namespace qtip;

extern "C" int qtip_rht(void *out, int out_dtype, const void *in, int in_dtype, long rows, int n, const void *sign_in,
                        int sign_in_dtype, const float *sign_out, long n_signs, const uint32_t *hadk_bits, int kfac,
                        int transpose, float scale, void *stream) {
    if (!out || !in || rows < 0) return QTIP_ERR_BAD_ARG;
    if ((out_dtype != QTIP_F16 && out_dtype != QTIP_F32) || (in_dtype != QTIP_F16 && in_dtype != QTIP_F32))
        return QTIP_ERR_BAD_ARG;
    if (sign_in && sign_in_dtype != QTIP_F16 && sign_in_dtype != QTIP_F32) return QTIP_ERR_BAD_ARG;
    if (!valid_kfac(kfac) || (kfac > 1 && !hadk_bits)) return QTIP_ERR_BAD_ARG;
    if (n <= 0 || n > 65536 || n % kfac) return QTIP_ERR_BAD_SHAPE;
    const int len = n / kfac;
    if (len < 2 || (len & (len - 1))) return QTIP_ERR_BAD_SHAPE;
    if ((sign_in || sign_out) && (n_signs < n || n_signs % n)) return QTIP_ERR_BAD_ARG;
    if (out == in && out_dtype != in_dtype) return QTIP_ERR_BAD_ARG;
    if (out == in && kfac > 1) return QTIP_ERR_BAD_ARG;  // several CTAs read the whole row
    if (rows == 0) return QTIP_OK;
    if (rows > 65535) return QTIP_ERR_BAD_SHAPE;
    int p = 0;
    while ((1 << p) < len) p++;
    const size_t smem = (size_t)n * sizeof(float) + (kfac > 1 ? (size_t)kRowsPerCta * kfac * sizeof(float) : 0);
    if (smem > 227 * 1024) return QTIP_ERR_BAD_SHAPE;
    static bool attr_set[64] = {};
    int dev = 0;
    QTIP_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 64 && !attr_set[dev]) {
        QTIP_CUDA_TRY(cudaFuncSetAttribute(rht_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        attr_set[dev] = true;
    }
    const int sign_rep = (sign_in || sign_out) ? (int)(n_signs / n) : 1;
    dim3 grid(kfac > 1 ? (kfac + kRowsPerCta - 1) / kRowsPerCta : 1, (unsigned)rows);
    rht_kernel<<<grid, kRhtThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        out, out_dtype, in, in_dtype, n, p, sign_in, sign_in_dtype, sign_out, sign_rep, hadk_bits, kfac, transpose,
        scale);
    return check_launch();
}
