// Randomized Hadamard transform with the sign flips and scales fused on both sides, plus the
// element-wise work that surrounds a QTIP linear inside a decoder layer.
//
// One row of n = kfac * 2^p values is transformed entirely in shared memory:
//   0. optional prologue, all fused into the load:  v = in (+ residual) ; residual_out = v ;
//      v = RMSNorm(v) * norm_weight ; v = silu(gate) * v
//   1. multiply by sign_in;
//   2. Walsh-Hadamard over the 2^p-long segments: radix-16 passes over shared memory
//      (4 butterfly stages per pass in registers);
//   3. kfac > 1: multiply the (kfac, 2^p) view from the left by the +-1 matrix hadK.  This is the
//      only super-linear part (kfac^2 * 2^p adds), so it is spread over several CTAs: CTA (i, r) of
//      the grid repeats steps 0-2 for row r (cheap, data comes from L2) and produces kRowsPerCta
//      output rows of the (kfac, 2^p) view;
//   4. scale, multiply by sign_out, store as fp16 or fp32.
// Replaces hadamard::hadamard + the hadK matmul + the element-wise kernels of
// lib/utils/matmul_had.py:105-119 and lib/codebook/bitshift.py:428-441, 465-471 upstream; the
// prologue options replace the residual add, LlamaRMSNorm (model/llama.py:129-136) and the
// SwiGLU product (model/llama.py:399-400) kernels that would otherwise run in between.
//
// Launched with programmatic stream serialization: the hadK sign table (weights) is expanded
// before griddepcontrol.wait, activations are touched after it.
#include "common.cuh"

namespace qtip {
namespace {

constexpr int kRhtThreads = 512;
constexpr int kRowsPerCta = 16;  // hadK output rows per CTA

struct RhtArgs {
    void *out; const void *in; const void *sign_in; const float *sign_out; const uint32_t *hadk_bits;
    const __half *residual; __half *residual_out; const __half *norm_weight; const __half *gate;
    long in_row_stride;  // elements between input rows (0 = every row reads the same input)
    int out_dtype, in_dtype, sign_in_dtype;
    int n, p, sign_rep, kfac, transpose;
    int vec_ok;          // every buffer is 16-byte aligned and n, strides are multiples of 8: 8-wide loads / stores
    float scale, eps;
};

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

__device__ __forceinline__ float load_elem(const void *p, int dtype, size_t i) {
    return dtype == QTIP_F16 ? __half2float(static_cast<const __half *>(p)[i]) : static_cast<const float *>(p)[i];
}

// 8 consecutive elements starting at element i (i % 8 == 0, base pointers 16-byte aligned)
__device__ __forceinline__ void load8(const void *p, int dtype, size_t i, float (&o)[8]) {
    if (dtype == QTIP_F16) {
        const uint4 raw = *reinterpret_cast<const uint4 *>(static_cast<const __half *>(p) + i);
        const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
        for (int k = 0; k < 4; k++) { o[2 * k] = __low2float(h[k]); o[2 * k + 1] = __high2float(h[k]); }
    } else {
        const float4 a = *reinterpret_cast<const float4 *>(static_cast<const float *>(p) + i);
        const float4 b = *reinterpret_cast<const float4 *>(static_cast<const float *>(p) + i + 4);
        o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
    }
}

__device__ __forceinline__ void store8(void *p, int dtype, size_t i, const float (&o)[8]) {
    if (dtype == QTIP_F16) {
        uint4 raw;
        __half2 *h = reinterpret_cast<__half2 *>(&raw);
#pragma unroll
        for (int k = 0; k < 4; k++) h[k] = __floats2half2_rn(o[2 * k], o[2 * k + 1]);
        *reinterpret_cast<uint4 *>(static_cast<__half *>(p) + i) = raw;
    } else {
        *reinterpret_cast<float4 *>(static_cast<float *>(p) + i) = make_float4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<float4 *>(static_cast<float *>(p) + i + 4) = make_float4(o[4], o[5], o[6], o[7]);
    }
}

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

// The fused prologue applied to one value (everything except the RMS statistic).
__device__ __forceinline__ float gate_and_sign(const RhtArgs &a, float x, size_t in_idx, size_t sign_idx) {
    if (a.gate) {
        // SwiGLU: silu(gate) in fp16 precision, product rounded to fp16 (the activations are fp16 tensors)
        const float gt = __half2float(a.gate[in_idx]);
        const __half sg = __float2half_rn(gt / (1.0f + __expf(-gt)));
        x = __half2float(__hmul(sg, __float2half_rn(x)));
    }
    if (a.sign_in) x *= load_elem(a.sign_in, a.sign_in_dtype, sign_idx);
    return x;
}

__global__ void __launch_bounds__(kRhtThreads) rht_kernel(const RhtArgs a) {
    extern __shared__ __align__(16) float sm[];
    const int n = a.n, kfac = a.kfac;
    float *v = sm;                            // n values, padded (see pad())
    float *hs = sm + pad(n) + 1;              // kfac x kRowsPerCta signs (+-1.0f), [k][row], only when kfac > 1
    hs = reinterpret_cast<float *>((reinterpret_cast<uintptr_t>(hs) + 15) & ~(uintptr_t)15);
    float *scratch = hs + (kfac > 1 ? kRowsPerCta * kfac : 0);  // 32 floats
    const long row = blockIdx.y;
    const size_t sign_off = (size_t)(row % a.sign_rep) * n;
    const size_t in_off = (size_t)row * a.in_row_stride, out_off = (size_t)row * n;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;

    const int i0 = blockIdx.x * kRowsPerCta;
    const int rows_here = min(kRowsPerCta, kfac - i0);
    if (kfac > 1) {
        // hs[k][il] = hadK[i0+il][k], or hadK[k][i0+il] for the transposed (input-side) transform
        const int wpr = (kfac + 31) >> 5;
        for (int il = warp; il < kRowsPerCta; il += nwarps)
            for (int k = lane; k < kfac; k += 32) {
                float sgn = 0.f;
                if (il < rows_here) {
                    const int rr = a.transpose ? k : (i0 + il), cc = a.transpose ? (i0 + il) : k;
                    sgn = ((a.hadk_bits[rr * wpr + (cc >> 5)] >> (cc & 31)) & 1u) ? 1.0f : -1.0f;
                }
                hs[k * kRowsPerCta + il] = sgn;
            }
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const bool vec = a.vec_ok;
    float ss = 0.f;
    if (vec) {
        for (int j = threadIdx.x * 8; j < n; j += blockDim.x * 8) {
            float x[8];
            load8(a.in, a.in_dtype, in_off + j, x);
            if (a.residual) {
                float r[8];
                load8(a.residual, QTIP_F16, in_off + j, r);
                // the residual stream is fp16: the sum is rounded to fp16 as an fp16 add would
#pragma unroll
                for (int k = 0; k < 8; k++) x[k] = __half2float(__float2half_rn(x[k] + r[k]));
                if (a.residual_out && blockIdx.x == 0 && (a.in_row_stride != 0 || row == 0))
                    store8(a.residual_out, QTIP_F16, in_off + j, x);
            }
#pragma unroll
            for (int k = 0; k < 8; k++) {
                ss += x[k] * x[k];
                if (!a.norm_weight) x[k] = gate_and_sign(a, x[k], in_off + j + k, sign_off + j + k);
                v[pad(j + k)] = x[k];
            }
        }
    } else {
        for (int j = threadIdx.x; j < n; j += blockDim.x) {
            float x = load_elem(a.in, a.in_dtype, in_off + j);
            if (a.residual) {
                x = __half2float(__float2half_rn(x + __half2float(a.residual[in_off + j])));
                if (a.residual_out && blockIdx.x == 0 && (a.in_row_stride != 0 || row == 0))
                    a.residual_out[in_off + j] = __float2half_rn(x);
            }
            ss += x * x;
            if (!a.norm_weight) x = gate_and_sign(a, x, in_off + j, sign_off + j);
            v[pad(j)] = x;
        }
    }
    if (a.norm_weight) {
        // LlamaRMSNorm: fp32 statistics, normalised value rounded to fp16, then times the fp16 weight
        const float r = rsqrtf(block_sum(ss, scratch) / (float)n + a.eps);
        for (int j = threadIdx.x; j < n; j += blockDim.x) {
            const __half hn = __float2half_rn(v[pad(j)] * r);
            v[pad(j)] = gate_and_sign(a, __half2float(__hmul(a.norm_weight[j], hn)), in_off + j, sign_off + j);
        }
    }
    __syncthreads();

    const int p = a.p;
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
    const float scale = a.scale;
    if (kfac == 1) {
        if (vec) {
            for (int j = threadIdx.x * 8; j < n; j += blockDim.x * 8) {
                float y[8];
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    y[k] = v[pad(j + k)] * scale;
                    if (a.sign_out) y[k] *= a.sign_out[sign_off + j + k];
                }
                store8(a.out, a.out_dtype, out_off + j, y);
            }
        } else {
            for (int j = threadIdx.x; j < n; j += blockDim.x) {
                float y = v[pad(j)] * scale;
                if (a.sign_out) y *= a.sign_out[sign_off + j];
                if (a.out_dtype == QTIP_F16) static_cast<__half *>(a.out)[out_off + j] = __float2half_rn(y);
                else static_cast<float *>(a.out)[out_off + j] = y;
            }
        }
        return;
    }
    // hadK multiply: output (i0 + il, j) = sum_k hs[k][il] * v[k*len + j].  A thread owns 4 rows of one
    // column: per k one value and one 16-byte broadcast load of 4 signs feed 4 multiply-adds.
    const int items = (kRowsPerCta / 4) * len;
    for (int idx = threadIdx.x; idx < items; idx += blockDim.x) {
        const int j = idx & (len - 1), il = (idx >> p) * 4;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
        for (int k = 0; k < kfac; k++) {
            const float x = v[pad(k * len + j)];
            const float4 h = *reinterpret_cast<const float4 *>(hs + k * kRowsPerCta + il);
            acc[0] = fmaf(h.x, x, acc[0]); acc[1] = fmaf(h.y, x, acc[1]);
            acc[2] = fmaf(h.z, x, acc[2]); acc[3] = fmaf(h.w, x, acc[3]);
        }
#pragma unroll
        for (int r = 0; r < 4; r++) {
            if (il + r < rows_here) {
                const size_t o = (size_t)(i0 + il + r) * len + j;
                float y = acc[r] * scale;
                if (a.sign_out) y *= a.sign_out[sign_off + o];
                if (a.out_dtype == QTIP_F16) static_cast<__half *>(a.out)[out_off + o] = __float2half_rn(y);
                else static_cast<float *>(a.out)[out_off + o] = y;
            }
        }
    }
}

bool valid_kfac(int k) {
    static const int ks[] = {1, 12, 20, 28, 36, 52, 60, 108, 116, 124, 140, 156, 172};
    for (int v : ks)
        if (v == k) return true;
    return false;
}

int launch_rht(RhtArgs a, long rows, void *stream) {
    const int len = a.n / a.kfac;
    int p = 0;
    while ((1 << p) < len) p++;
    a.p = p;
    const size_t smem = ((size_t)a.n + (a.n >> 5) + 8 + (a.kfac > 1 ? (size_t)kRowsPerCta * a.kfac : 0) + 32) * sizeof(float);
    {
        const void *ptrs[] = {a.out, a.in, a.residual, a.residual_out, a.gate};
        bool ok = (a.n % 8 == 0) && (a.in_row_stride % 8 == 0);
        for (const void *q : ptrs) ok = ok && aligned(q, 16);
        a.vec_ok = ok ? 1 : 0;
    }
    if (smem > 227 * 1024) return QTIP_ERR_BAD_SHAPE;
    static bool attr_set[64] = {};
    int dev = 0;
    QTIP_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 64 && !attr_set[dev]) {
        QTIP_CUDA_TRY(cudaFuncSetAttribute(rht_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.kfac > 1 ? (a.kfac + kRowsPerCta - 1) / kRowsPerCta : 1, (unsigned)rows);
    cfg.blockDim = dim3(kRhtThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    QTIP_CUDA_TRY(cudaLaunchKernelEx(&cfg, rht_kernel, a));
    return check_launch();
}

int check_rht(const void *out, int out_dtype, const void *in, int in_dtype, long rows, int n, const void *sign_in,
              int sign_in_dtype, const float *sign_out, long n_signs, const uint32_t *hadk_bits, int kfac) {
    if (!out || !in || rows < 0) return QTIP_ERR_BAD_ARG;
    if ((out_dtype != QTIP_F16 && out_dtype != QTIP_F32) || (in_dtype != QTIP_F16 && in_dtype != QTIP_F32))
        return QTIP_ERR_BAD_ARG;
    if (sign_in && sign_in_dtype != QTIP_F16 && sign_in_dtype != QTIP_F32) return QTIP_ERR_BAD_ARG;
    if (!valid_kfac(kfac) || (kfac > 1 && !hadk_bits)) return QTIP_ERR_BAD_ARG;
    if (n <= 0 || n > 65536 || n % kfac) return QTIP_ERR_BAD_SHAPE;
    const int len = n / kfac;
    if (len < 2 || (len & (len - 1))) return QTIP_ERR_BAD_SHAPE;
    if ((sign_in || sign_out) && (n_signs < n || n_signs % n)) return QTIP_ERR_BAD_ARG;
    if (rows > 65535) return QTIP_ERR_BAD_SHAPE;
    return QTIP_OK;
}

}  // namespace
}  // namespace qtip

using namespace qtip;

extern "C" int qtip_rht(void *out, int out_dtype, const void *in, int in_dtype, long rows, int n, const void *sign_in,
                        int sign_in_dtype, const float *sign_out, long n_signs, const uint32_t *hadk_bits, int kfac,
                        int transpose, float scale, void *stream) {
    int st = check_rht(out, out_dtype, in, in_dtype, rows, n, sign_in, sign_in_dtype, sign_out, n_signs, hadk_bits, kfac);
    if (st != QTIP_OK) return st;
    if (out == in && out_dtype != in_dtype) return QTIP_ERR_BAD_ARG;
    if (out == in && kfac > 1) return QTIP_ERR_BAD_ARG;  // several CTAs read the whole row
    if (rows == 0) return QTIP_OK;
    RhtArgs a = {};
    a.out = out; a.in = in; a.sign_in = sign_in; a.sign_out = sign_out; a.hadk_bits = hadk_bits;
    a.in_row_stride = n; a.out_dtype = out_dtype; a.in_dtype = in_dtype; a.sign_in_dtype = sign_in_dtype;
    a.n = n; a.sign_rep = (sign_in || sign_out) ? (int)(n_signs / n) : 1; a.kfac = kfac; a.transpose = transpose;
    a.scale = scale;
    return launch_rht(a, rows, stream);
}

extern "C" int qtip_rht_fused(void *out, int out_dtype, const void *in, int in_dtype, long rows, long in_row_stride,
                              int n, const void *residual, void *residual_out, const void *norm_weight, float eps,
                              const void *gate, const void *sign_in, int sign_in_dtype, const float *sign_out,
                              long n_signs, const uint32_t *hadk_bits, int kfac, int transpose, float scale,
                              void *stream) {
    int st = check_rht(out, out_dtype, in, in_dtype, rows, n, sign_in, sign_in_dtype, sign_out, n_signs, hadk_bits, kfac);
    if (st != QTIP_OK) return st;
    if (in_row_stride != 0 && in_row_stride < n) return QTIP_ERR_BAD_ARG;
    if (residual_out && !residual) return QTIP_ERR_BAD_ARG;
    // several CTAs (rows with stride 0, or kfac > 1) read the inputs while one writes residual_out / out
    if (out == in || out == residual || out == gate) return QTIP_ERR_BAD_ARG;
    if (residual_out && (residual_out == in || residual_out == residual || residual_out == out || residual_out == gate))
        return QTIP_ERR_BAD_ARG;
    if (rows == 0) return QTIP_OK;
    RhtArgs a = {};
    a.out = out; a.in = in; a.sign_in = sign_in; a.sign_out = sign_out; a.hadk_bits = hadk_bits;
    a.residual = static_cast<const __half *>(residual); a.residual_out = static_cast<__half *>(residual_out);
    a.norm_weight = static_cast<const __half *>(norm_weight); a.gate = static_cast<const __half *>(gate);
    a.in_row_stride = in_row_stride; a.out_dtype = out_dtype; a.in_dtype = in_dtype; a.sign_in_dtype = sign_in_dtype;
    a.n = n; a.sign_rep = (sign_in || sign_out) ? (int)(n_signs / n) : 1; a.kfac = kfac; a.transpose = transpose;
    a.scale = scale; a.eps = eps;
    return launch_rht(a, rows, stream);
}
