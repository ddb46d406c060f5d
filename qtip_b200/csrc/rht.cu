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
#include "fwht.cuh"

namespace qtip {
namespace {

constexpr int kRhtThreads = 1024;

struct RhtArgs {
    void *out; const void *in; const void *sign_in; const float *sign_out; const uint32_t *hadk_bits;
    const __half *residual; __half *residual_out; const __half *norm_weight; const __half *gate;
    long in_row_stride;  // elements between input rows (0 = every row reads the same input)
    int out_dtype, in_dtype, sign_in_dtype;
    int n, p, sign_rep, kfac, transpose;
    int rpc;             // hadK output rows per CTA (4, 8 or 16)
    int part_offset;     // float offset in shared memory of the partial-product buffer (short rows only)
    int sgn_offset;      // float offset of the staged sign_out slice (short rows only, else 0)
    int vec_ok;          // every buffer is 16-byte aligned and n, strides are multiples of 8: 8-wide loads / stores
    float scale, eps;
};

__device__ __forceinline__ float load_elem(const void *p, int dtype, size_t i) {
    return dtype == QTIP_F16 ? __half2float(static_cast<const __half *>(p)[i]) : static_cast<const float *>(p)[i];
}

// 8 consecutive elements starting at element i (i % 8 == 0, base pointers 16-byte aligned)
__device__ __forceinline__ void load8(const void *p, int dtype, size_t i, float (&o)[8]) {
    if (dtype == QTIP_F16) load8_f16(static_cast<const __half *>(p), i, o);
    else load8_f32(static_cast<const float *>(p), i, o);
}
__device__ __forceinline__ void store8(void *p, int dtype, size_t i, const float (&o)[8]) {
    if (dtype == QTIP_F16) store8_f16(static_cast<__half *>(p), i, o);
    else store8_f32(static_cast<float *>(p), i, o);
}

// 8 values from one (fp16) or two (fp32) raw 16-byte registers
__device__ __forceinline__ void unpack_raw(const uint4 *r, int dtype, float (&o)[8]) {
    if (dtype == QTIP_F16) {
        const __half2 *h = reinterpret_cast<const __half2 *>(r);
#pragma unroll
        for (int k = 0; k < 4; k++) { o[2 * k] = __low2float(h[k]); o[2 * k + 1] = __high2float(h[k]); }
    } else {
        const float *f = reinterpret_cast<const float *>(r);
#pragma unroll
        for (int k = 0; k < 8; k++) o[k] = f[k];
    }
}

// Power-of-two n = 1024*E with vector-aligned buffers: a thread owns E consecutive values and the whole
// row stays in registers (fwht_regs); shared memory is used for one transpose only.
template <int E>
__device__ __forceinline__ void rht_regs(const RhtArgs &a, float *buf, float *scratch) {
    const int n = a.n;
    const long row = blockIdx.y;
    const size_t sign_off = (size_t)(row % a.sign_rep) * n;
    const size_t in_off = (size_t)row * a.in_row_stride, out_off = (size_t)row * n;
    const size_t j = (size_t)threadIdx.x * E;
    const size_t jo = (size_t)((threadIdx.x & 31) * 32 + (threadIdx.x >> 5)) * E;   // ownership after the transform
    float v[E], rs[E], wn[E], gt[E], sg[E], so[E];
    if (a.in_dtype == QTIP_F16) loadE_f16<E>(static_cast<const __half *>(a.in), in_off + j, v);
    else loadE_f32<E>(static_cast<const float *>(a.in), in_off + j, v, false);
    if (a.residual) loadE_f16<E>(a.residual, in_off + j, rs);
    if (a.norm_weight) loadE_f16<E>(a.norm_weight, j, wn);
    if (a.gate) loadE_f16<E>(a.gate, in_off + j, gt);
    if (a.sign_in) {
        if (a.sign_in_dtype == QTIP_F16) loadE_f16<E>(static_cast<const __half *>(a.sign_in), sign_off + j, sg);
        else loadE_f32<E>(static_cast<const float *>(a.sign_in), sign_off + j, sg, false);
    }
    if (a.sign_out) loadE_f32<E>(a.sign_out, sign_off + jo, so, false);
    if (a.residual) {
#pragma unroll
        for (int k = 0; k < E; k++) v[k] = __half2float(__float2half_rn(v[k] + rs[k]));
        if (a.residual_out && (a.in_row_stride != 0 || row == 0)) storeE_f16<E>(a.residual_out, in_off + j, v);
    }
    if (a.norm_weight) {
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < E; k++) ss += v[k] * v[k];
        const float r = rsqrtf(block_sum(ss, scratch) / (float)n + a.eps);
#pragma unroll
        for (int k = 0; k < E; k++) v[k] = __half2float(__hmul(__float2half_rn(wn[k]), __float2half_rn(v[k] * r)));
    }
#pragma unroll
    for (int k = 0; k < E; k++) {
        if (a.gate) v[k] = swiglu_fp16(gt[k], v[k]);
        if (a.sign_in) v[k] *= sg[k];
    }
    fwht_regs<E>(v, buf);
#pragma unroll
    for (int k = 0; k < E; k++) {
        v[k] *= a.scale;
        if (a.sign_out) v[k] *= so[k];
    }
    if (a.out_dtype == QTIP_F16) storeE_f16<E>(static_cast<__half *>(a.out), out_off + jo, v);
    else storeE_f32<E>(static_cast<float *>(a.out), out_off + jo, v);
}

__global__ void __launch_bounds__(kRhtThreads) rht_kernel(const RhtArgs a) {
    extern __shared__ __align__(16) float sm[];
    const int n = a.n, kfac = a.kfac;
    float *v = sm;                            // n values, padded (see pad())
    const int rpc = a.rpc;
    float *hs = sm + pad(n) + 1;              // kfac x rpc signs (+-1.0f), [k][row], only when kfac > 1
    hs = reinterpret_cast<float *>((reinterpret_cast<uintptr_t>(hs) + 15) & ~(uintptr_t)15);
    float *scratch = hs + (kfac > 1 ? rpc * kfac : 0);            // 32 floats (block_sum)
    uint32_t *bits = reinterpret_cast<uint32_t *>(scratch + 32);  // the packed hadK matrix, kfac * ceil(kfac/32) words
    const long row = blockIdx.y;
    const size_t sign_off = (size_t)(row % a.sign_rep) * n;
    const size_t in_off = (size_t)row * a.in_row_stride, out_off = (size_t)row * n;

    const int i0 = blockIdx.x * rpc;
    const int rows_here = min(rpc, kfac - i0);
    if (kfac > 1) {
        // one coalesced read of the bit matrix, then hs[k][il] = hadK[i0+il][k]
        // (hadK[k][i0+il] for the transposed, input-side transform)
        const int wpr = (kfac + 31) >> 5;
        for (int i = threadIdx.x; i < kfac * wpr; i += blockDim.x) bits[i] = a.hadk_bits[i];
        __syncthreads();
        for (int idx = threadIdx.x; idx < rpc * kfac; idx += blockDim.x) {
            const int k = idx / rpc, il = idx - k * rpc;
            float sgn = 0.f;
            if (il < rows_here) {
                const int rr = a.transpose ? k : (i0 + il), cc = a.transpose ? (i0 + il) : k;
                sgn = ((bits[rr * wpr + (cc >> 5)] >> (cc & 31)) & 1u) ? 1.0f : -1.0f;
            }
            hs[idx] = sgn;
        }
    }
    // short rows: this CTA's slice of sign_out (a weight) is copied to shared memory asynchronously now,
    // so the final store does not wait for it
    const bool vec = a.vec_ok;
    const bool sign_staged = kfac > 1 && vec && a.sign_out && a.sgn_offset > 0 && ((n / kfac) & 7) == 0;
    if (sign_staged) {
        const int len_ = n / kfac;
        const float *src = a.sign_out + sign_off + (size_t)i0 * len_;
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(sm + a.sgn_offset);
        for (int c = threadIdx.x; c < (rows_here * len_) >> 2; c += blockDim.x)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + c * 16), "l"(src + c * 4) : "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    if (kfac == 1 && vec && (n == 4096 || n == 8192)) {
        if (n == 4096) rht_regs<4>(a, v, scratch);
        else rht_regs<8>(a, v, scratch);
        return;
    }
    const bool write_res = a.residual_out && blockIdx.x == 0 && (a.in_row_stride != 0 || row == 0);
    float ss = 0.f;
    if (vec && !a.residual && !a.norm_weight) {
        // two 8-value vectors per thread and trip, every load of both requested before the first use
        const int nvec = n >> 3;
        for (int j0 = threadIdx.x; j0 < nvec; j0 += 2 * blockDim.x) {
            const int jv[2] = {j0, j0 + (int)blockDim.x};
            uint4 xr[2][2], gr[2], sr[2][2];
#pragma unroll
            for (int u = 0; u < 2; u++) {
                if (jv[u] >= nvec) continue;
                const size_t j = (size_t)jv[u] * 8;
                if (a.in_dtype == QTIP_F16) xr[u][0] = *reinterpret_cast<const uint4 *>(static_cast<const __half *>(a.in) + in_off + j);
                else {
                    const uint4 *q = reinterpret_cast<const uint4 *>(static_cast<const float *>(a.in) + in_off + j);
                    xr[u][0] = q[0]; xr[u][1] = q[1];
                }
                if (a.gate) gr[u] = *reinterpret_cast<const uint4 *>(a.gate + in_off + j);
                if (a.sign_in) {
                    if (a.sign_in_dtype == QTIP_F16) sr[u][0] = *reinterpret_cast<const uint4 *>(static_cast<const __half *>(a.sign_in) + sign_off + j);
                    else {
                        const uint4 *q = reinterpret_cast<const uint4 *>(static_cast<const float *>(a.sign_in) + sign_off + j);
                        sr[u][0] = q[0]; sr[u][1] = q[1];
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < 2; u++) {
                if (jv[u] >= nvec) continue;
                const int j = jv[u] * 8;
                float x[8], gt[8], sg[8];
                unpack_raw(xr[u], a.in_dtype, x);
                if (a.gate) unpack_raw(&gr[u], QTIP_F16, gt);
                if (a.sign_in) unpack_raw(sr[u], a.sign_in_dtype, sg);
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    if (a.gate) x[k] = swiglu_fp16(gt[k], x[k]);
                    if (a.sign_in) x[k] *= sg[k];
                    v[pad(j + k)] = x[k];
                }
            }
        }
    } else if (vec) {
        // a thread owns 8 consecutive values; all operand vectors are requested before any is used
        for (int j = threadIdx.x * 8; j < n; j += blockDim.x * 8) {
            float x[8], rs[8], gt[8], sg[8];
            load8(a.in, a.in_dtype, in_off + j, x);
            if (a.residual) load8_f16(a.residual, in_off + j, rs);
            if (a.gate && !a.norm_weight) load8_f16(a.gate, in_off + j, gt);
            if (a.sign_in && !a.norm_weight) load8(a.sign_in, a.sign_in_dtype, sign_off + j, sg);
            if (a.residual) {
                // the residual stream is fp16: the sum is rounded to fp16 as an fp16 add would
#pragma unroll
                for (int k = 0; k < 8; k++) x[k] = __half2float(__float2half_rn(x[k] + rs[k]));
                if (write_res) store8_f16(a.residual_out, in_off + j, x);
            }
#pragma unroll
            for (int k = 0; k < 8; k++) {
                ss += x[k] * x[k];
                if (!a.norm_weight) {
                    if (a.gate) x[k] = swiglu_fp16(gt[k], x[k]);
                    if (a.sign_in) x[k] *= sg[k];
                }
                v[pad(j + k)] = x[k];
            }
        }
        if (a.norm_weight) {
            // LlamaRMSNorm: fp32 statistics, normalised value rounded to fp16, then times the fp16 weight
            const float r = rsqrtf(block_sum(ss, scratch) / (float)n + a.eps);
            for (int j = threadIdx.x * 8; j < n; j += blockDim.x * 8) {
                float w[8], gt[8], sg[8];
                load8_f16(a.norm_weight, j, w);
                if (a.gate) load8_f16(a.gate, in_off + j, gt);
                if (a.sign_in) load8(a.sign_in, a.sign_in_dtype, sign_off + j, sg);
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    float x = __half2float(__hmul(__float2half_rn(w[k]), __float2half_rn(v[pad(j + k)] * r)));
                    if (a.gate) x = swiglu_fp16(gt[k], x);
                    if (a.sign_in) x *= sg[k];
                    v[pad(j + k)] = x;
                }
            }
        }
    } else {
        for (int j = threadIdx.x; j < n; j += blockDim.x) {
            float x = load_elem(a.in, a.in_dtype, in_off + j);
            if (a.residual) {
                x = __half2float(__float2half_rn(x + __half2float(a.residual[in_off + j])));
                if (write_res) a.residual_out[in_off + j] = __float2half_rn(x);
            }
            ss += x * x;
            v[pad(j)] = x;
        }
        float r = 1.f;
        if (a.norm_weight) r = rsqrtf(block_sum(ss, scratch) / (float)n + a.eps);
        for (int j = threadIdx.x; j < n; j += blockDim.x) {
            float x = v[pad(j)];
            if (a.norm_weight) x = __half2float(__hmul(a.norm_weight[j], __float2half_rn(x * r)));
            if (a.gate) x = swiglu_fp16(__half2float(a.gate[in_off + j]), x);
            if (a.sign_in) x *= load_elem(a.sign_in, a.sign_in_dtype, sign_off + j);
            v[pad(j)] = x;
        }
    }
    __syncthreads();

    const int p = a.p;
    const int len = 1 << p;
    const float scale = a.scale;
    if (kfac == 1) {
        fwht_shared(v, n, p);
        if (vec) {
            for (int j = threadIdx.x * 8; j < n; j += blockDim.x * 8) {
                float y[8], sg[8];
                if (a.sign_out) load8_f32(a.sign_out, sign_off + j, sg);
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    y[k] = v[pad(j + k)] * scale;
                    if (a.sign_out) y[k] *= sg[k];
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
    // n = kfac * 2^p.  The two factors of the transform commute, so the +-1 multiply runs FIRST, on the
    // untransformed values, and only this CTA's rpc output rows go through the Walsh-Hadamard passes:
    //   w[il][j] = sum_k hs[k][il] * v[k*len + j]   then   FWHT over j of each row.
    // A thread owns 4 rows of one column: per k one value and one 16-byte broadcast load of 4 signs.
    // The products stay in registers until every thread has finished reading v; the rows are then written over
    // the start of v (the host guarantees at most 4 items per thread).
    const int items = (rpc >> 2) * len;
    float *wbuf = v;
    if (items * 2 <= (int)blockDim.x) {
        // short rows: the k range is cut into blockDim.x / items slices so that every thread takes part;
        // the slices' partial products meet in `part` ([slice][row][column]) and are summed below
        const int slices = blockDim.x / items, kper = (kfac + slices - 1) / slices;
        const int sl = threadIdx.x / items, item = threadIdx.x - sl * items;
        const int j = item & (len - 1), il = (item >> p) * 4;
        const int k0 = sl * kper, k1 = min(kfac, k0 + kper);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
        for (int k = k0; k < k1; k++) {
            const float x = v[pad(k * len + j)];
            const float4 h = *reinterpret_cast<const float4 *>(hs + k * rpc + il);
            acc[0] = fmaf(h.x, x, acc[0]); acc[1] = fmaf(h.y, x, acc[1]);
            acc[2] = fmaf(h.z, x, acc[2]); acc[3] = fmaf(h.w, x, acc[3]);
        }
        float *part = a.part_offset + sm;
#pragma unroll
        for (int r = 0; r < 4; r++) part[(sl * rpc + il + r) * len + j] = acc[r];
        __syncthreads();
        for (int e = threadIdx.x; e < rpc * len; e += blockDim.x) {
            float t = 0.f;
            for (int q = 0; q < slices; q++) t += part[q * rpc * len + e];
            wbuf[pad(e)] = t;
        }
        __syncthreads();
    } else {
        float acc[4][4];
#pragma unroll
        for (int t = 0; t < 4; t++) {
            const int idx = threadIdx.x + t * blockDim.x;
#pragma unroll
            for (int r = 0; r < 4; r++) acc[t][r] = 0.f;
            if (idx < items) {
                const int j = idx & (len - 1), il = (idx >> p) * 4;
#pragma unroll 4
                for (int k = 0; k < kfac; k++) {
                    const float x = v[pad(k * len + j)];
                    const float4 h = *reinterpret_cast<const float4 *>(hs + k * rpc + il);
                    acc[t][0] = fmaf(h.x, x, acc[t][0]); acc[t][1] = fmaf(h.y, x, acc[t][1]);
                    acc[t][2] = fmaf(h.z, x, acc[t][2]); acc[t][3] = fmaf(h.w, x, acc[t][3]);
                }
            }
        }
        __syncthreads();
#pragma unroll
        for (int t = 0; t < 4; t++) {
            const int idx = threadIdx.x + t * blockDim.x;
            if (idx < items) {
                const int j = idx & (len - 1), il = (idx >> p) * 4;
#pragma unroll
                for (int r = 0; r < 4; r++) wbuf[pad((il + r) * len + j)] = acc[t][r];
            }
        }
        __syncthreads();
    }
    if (sign_staged) asm volatile("cp.async.wait_all;" ::: "memory");   // made visible by the barriers below
    fwht_shared(wbuf, rpc * len, p);
    const int total = rows_here * len;
    if (vec && (len & 7) == 0) {
        for (int e = threadIdx.x * 8; e < total; e += blockDim.x * 8) {
            const size_t o = (size_t)i0 * len + e;      // rows of this CTA are contiguous in the output
            float y[8], sg[8];
            if (sign_staged) load8_f32(sm + a.sgn_offset, e, sg);
            else if (a.sign_out) load8_f32(a.sign_out, sign_off + o, sg);
#pragma unroll
            for (int k = 0; k < 8; k++) {
                y[k] = wbuf[pad(e + k)] * scale;
                if (a.sign_out) y[k] *= sg[k];
            }
            store8(a.out, a.out_dtype, out_off + o, y);
        }
    } else {
        for (int e = threadIdx.x; e < total; e += blockDim.x) {
            const size_t o = (size_t)i0 * len + e;
            float y = wbuf[pad(e)] * scale;
            if (a.sign_out) y *= a.sign_out[sign_off + o];
            if (a.out_dtype == QTIP_F16) static_cast<__half *>(a.out)[out_off + o] = __float2half_rn(y);
            else static_cast<float *>(a.out)[out_off + o] = y;
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
    // rows of the factor matrix per CTA: 8, or 4 when a row is long - a thread keeps at most 4 x 4 products
    // in registers, so (rpc / 4) * len <= 4 * kRhtThreads
    a.rpc = len >= 1024 ? 4 : 8;
    if (a.kfac > 1 && (a.rpc / 4) * len > 4 * kRhtThreads) return QTIP_ERR_BAD_SHAPE;
    // floats: values (padded) + alignment slack, signs of this CTA's rows, block_sum scratch, the bit matrix,
    // and for short rows the partial products of the k slices (4 per thread)
    size_t words = (size_t)a.n + (a.n >> 5) + 8 + (a.kfac > 1 ? (size_t)a.rpc * a.kfac : 0) + 32 +
                   (a.kfac > 1 ? (size_t)a.kfac * ((a.kfac + 31) / 32) : 0);
    words = (words + 3) & ~(size_t)3;
    a.part_offset = (int)words;
    if (a.kfac > 1 && (a.rpc / 4) * len * 2 <= kRhtThreads) {
        words += 4 * kRhtThreads;
        a.sgn_offset = (int)words;
        words += (size_t)a.rpc * len;
    }
    const size_t smem = words * sizeof(float);
    {
        const void *ptrs[] = {a.out, a.in, a.residual, a.residual_out, a.gate, a.sign_in, a.sign_out, a.norm_weight};
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
    cfg.gridDim = dim3(a.kfac > 1 ? (a.kfac + a.rpc - 1) / a.rpc : 1, (unsigned)rows);
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
