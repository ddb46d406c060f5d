// Everything between the gate/up matvecs and the down matvec of a Llama MLP at batch 1, in ONE launch of
// one 8-CTA cluster, for widths n = kfac * len whose Hadamard transform has a non-trivial +-1 factor
// (Llama-2-7B: 11008 = 172 * 64):
//     g = sv_gate * H(y_gate) * scale_out          output side of gate_proj   (bitshift.py:465-471 upstream)
//     u = sv_up   * H(y_up)   * scale_out          output side of up_proj
//     a = silu(g) * u                              model/llama.py:399-400 upstream, fp16 tensors
//     x = fp16( H^T( su_down * a ) * scale_in )    input side of down_proj    (bitshift.py:428-441 upstream)
// with H = hadK (x) Walsh-Hadamard(len).  The +-1 factor is a GEMM-shaped product (kfac x kfac by kfac x len)
// and runs on the tensor cores: the +-1 matrix is exact in fp16 and the data is split into an fp16 head and
// an fp16 remainder (two MMAs, fp32 accumulation), which keeps about 22 bits of the fp32 input.
//
// CTA c of the cluster owns rows [c*R, c*R + R) of the kfac x len matrix view.  Phases:
//   0  (weights only, before the grid dependency wait) bit matrix -> shared memory, the bit rows this
//      CTA needs for both products, its slices of the three sign vectors (cp.async)
//   1  y_gate, y_up -> shared memory as fp16 head / remainder planes, pairs of consecutive k packed in one
//      word ([k/2][j]): exactly the B-fragment layout of mma.m16n8k16
//   2  T = S[own rows, :] * Y for gate and up: one 16x8 output tile per warp, 11 k steps
//   3  one warp per pair of own rows: Walsh-Hadamard over j (registers + shuffles), signs, SwiGLU, signs,
//      Walsh-Hadamard again; the result is pushed, already split into head / remainder, into the planes of
//      ALL CTAs of the cluster (distributed shared memory), then one cluster barrier
//   4  X = S^T[own rows, :] * B on the tensor cores, scaled, rounded to fp16, stored
#include "fwht.cuh"

namespace qtip {
namespace {

constexpr int kMidThreads = 1024, kMidWarps = 32, kMidCluster = 8;
constexpr int kMaxFactor = 176;   // kfac padded to a multiple of 16
constexpr int kRowWords = 8;      // words per bit row (kfac <= 256 would fit; 6 used for 172)

struct MlpMidArgs {
    const float *y_gate, *y_up, *sv_gate, *sv_up;
    const __half *su_down;
    __half *out;
    const uint32_t *hadk_bits;
    int n, kfac, len, rows_per_cta;
    float scale_out, scale_in;
};

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// two matrix bits -> half2 of +-1.0 (bit set = +1): 0xBC00 is -1.0, flipping bit 15 gives +1.0
__device__ __forceinline__ uint32_t pm1_pair(uint32_t x) { return 0xBC00BC00u ^ ((x & 1u) << 15) ^ ((x & 2u) << 30); }

// A fragment (16 rows x 16 k) of a +-1 matrix whose rows are bit rows in shared memory
__device__ __forceinline__ void sign_fragment(const uint32_t *rowbits, int mt, int kt, int g, int t, uint32_t (&a)[4]) {
    const uint32_t w0 = rowbits[(mt * 16 + g) * kRowWords + (kt >> 1)], w1 = rowbits[(mt * 16 + g + 8) * kRowWords + (kt >> 1)];
    const int s = (kt & 1) * 16 + 2 * t;
    a[0] = pm1_pair(w0 >> s); a[1] = pm1_pair(w1 >> s); a[2] = pm1_pair(w0 >> (s + 8)); a[3] = pm1_pair(w1 >> (s + 8));
}

// fp32 -> fp16 head and fp16 remainder
__device__ __forceinline__ void split_f32(float x, __half &hi, __half &lo) {
    hi = __float2half_rn(x);
    lo = __float2half_rn(x - __half2float(hi));
}
__device__ __forceinline__ uint32_t pack_h2(__half a, __half b) {
    return (uint32_t)__half_as_ushort(a) | ((uint32_t)__half_as_ushort(b) << 16);
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

__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void store_remote(uint32_t local_addr, uint32_t cta, uint32_t v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(cta));
    asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(remote), "r"(v) : "memory");
}

struct MidLayout {     // offsets in 32-bit words from the start of dynamic shared memory
    int bits, rb_out, rb_in, sv_g, sv_u, su, planes1, tbuf, planes2, total;
    int ld;            // words per plane row: len + 8 (bank-conflict-free B fragments)
    int kp;            // plane rows: padded kfac / 2
};
__host__ __device__ inline MidLayout mid_layout(int kfac, int len, int R) {
    MidLayout L;
    const int wpr = (kfac + 31) >> 5, kpad = (kfac + 15) & ~15;
    L.ld = len + 8;
    L.kp = kpad >> 1;
    int o = 0;
    L.bits = o;    o += (kfac * wpr + 3) & ~3;
    L.rb_out = o;  o += 32 * kRowWords;
    L.rb_in = o;   o += 32 * kRowWords;
    L.sv_g = o;    o += R * len;
    L.sv_u = o;    o += R * len;
    L.su = o;      o += R * len / 2;
    L.planes1 = o; o += 4 * L.kp * L.ld;      // [gate, up][head, remainder][kp][ld]
    L.tbuf = o;    o += 2 * 32 * (len + 4);   // [gate, up][32 rows][len + 4] fp32
    L.planes2 = o; o += 2 * L.kp * L.ld;      // [head, remainder][kp][ld]
    L.total = o;
    return L;
}

template <int E>   // len = 32 * E
__global__ void __launch_bounds__(kMidThreads, 1) mlp_mid_kernel(const MlpMidArgs a) {
    extern __shared__ __align__(16) uint32_t smw[];
    constexpr int len = 32 * E;
    const int kfac = a.kfac, R = a.rows_per_cta, wpr = (kfac + 31) >> 5;
    const MidLayout L = mid_layout(kfac, len, R);
    const int KT = (kfac + 15) >> 4;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int rank = (int)cluster_rank();
    const int i0 = rank * R, rows_here = max(0, min(R, kfac - i0));
    uint32_t *bits = smw + L.bits, *rb_out = smw + L.rb_out, *rb_in = smw + L.rb_in;
    float *svg = reinterpret_cast<float *>(smw + L.sv_g), *svu = reinterpret_cast<float *>(smw + L.sv_u);
    __half *su = reinterpret_cast<__half *>(smw + L.su);
    uint32_t *planes1 = smw + L.planes1, *planes2 = smw + L.planes2;
    float *tbuf = reinterpret_cast<float *>(smw + L.tbuf);
    constexpr int ldt = len + 4;

    // ---- phase 0: weights only
    for (int i = tid; i < kfac * wpr; i += kMidThreads) bits[i] = __ldg(a.hadk_bits + i);
    if (rows_here > 0) {
        const int chunks32 = rows_here * len / 4, chunks16 = rows_here * len / 8;   // 16-byte chunks
        const size_t off = (size_t)i0 * len;
        for (int c = tid; c < chunks32; c += kMidThreads) {
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(svg + c * 4)),
                         "l"(a.sv_gate + off + c * 4) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(svu + c * 4)),
                         "l"(a.sv_up + off + c * 4) : "memory");
        }
        for (int c = tid; c < chunks16; c += kMidThreads)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(su + c * 8)),
                         "l"(a.su_down + off + c * 8) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    // zero rows of the second product's planes that no CTA writes (k >= kfac), and the whole first planes' tail
    for (int i = tid; i < 2 * (L.kp - kfac / 2) * L.ld; i += kMidThreads) {
        const int per = (L.kp - kfac / 2) * L.ld;
        planes2[(i / per) * L.kp * L.ld + (kfac / 2) * L.ld + (i % per)] = 0u;
    }
    __syncthreads();
    // bit rows of this CTA: rb_out[il] = row i0+il of S (first product), rb_in[il] = column i0+il of S (second)
    for (int i = tid; i < 32 * kRowWords; i += kMidThreads) {
        const int il = i / kRowWords, w = i % kRowWords;
        rb_out[i] = (il < rows_here && w < wpr) ? bits[(i0 + il) * wpr + w] : 0u;
    }
    for (int u = warp; u < 32 * kRowWords; u += kMidWarps) {
        const int il = u / kRowWords, w = u % kRowWords, k = 32 * w + lane, col = i0 + il;
        const bool bit = il < rows_here && k < kfac && ((bits[k * wpr + (col >> 5)] >> (col & 31)) & 1u);
        const uint32_t word = __ballot_sync(kFullMask, bit);
        if (lane == 0) rb_in[u] = word;
    }
    cluster_arrive();     // every CTA of the cluster is running; matched by the wait before the remote stores
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- phase 1: y_gate, y_up -> head / remainder planes, [k/2][j] words
    {
        constexpr int jq = len / 4;                      // float4 groups per row
        const int items = 2 * L.kp * jq;                 // (which, k pair, j group)
        for (int it0 = tid; it0 < items; it0 += 2 * kMidThreads) {
            float4 r0[2], r1[2];
            int which[2], kpi[2], jg[2];
            bool ok[2];
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const int it = it0 + u * kMidThreads;
                ok[u] = it < items;
                which[u] = it / (L.kp * jq);
                const int rem = it - which[u] * (L.kp * jq);
                kpi[u] = rem / jq; jg[u] = rem - kpi[u] * jq;
                r0[u] = r1[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (ok[u]) {
                    const float *src = (which[u] ? a.y_up : a.y_gate) + (size_t)(2 * kpi[u]) * len + 4 * jg[u];
                    if (2 * kpi[u] < kfac) r0[u] = __ldcg(reinterpret_cast<const float4 *>(src));
                    if (2 * kpi[u] + 1 < kfac) r1[u] = __ldcg(reinterpret_cast<const float4 *>(src + len));
                }
            }
#pragma unroll
            for (int u = 0; u < 2; u++) {
                if (!ok[u]) continue;
                const float e0[4] = {r0[u].x, r0[u].y, r0[u].z, r0[u].w}, e1[4] = {r1[u].x, r1[u].y, r1[u].z, r1[u].w};
                uint32_t hi[4], lo[4];
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    __half h0, l0, h1, l1;
                    split_f32(e0[q], h0, l0); split_f32(e1[q], h1, l1);
                    hi[q] = pack_h2(h0, h1); lo[q] = pack_h2(l0, l1);
                }
                uint32_t *dst = planes1 + (size_t)(which[u] * 2) * L.kp * L.ld + kpi[u] * L.ld + 4 * jg[u];
                *reinterpret_cast<uint4 *>(dst) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<uint4 *>(dst + L.kp * L.ld) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
            }
        }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();

    // ---- phase 2: T[which][il][j] = sum_k S[i0+il][k] * y_which[k][j]
    {
        constexpr int NT = len / 8;
        const int MT = (rows_here + 15) >> 4;
        for (int unit = warp; unit < 2 * MT * NT; unit += kMidWarps) {
            const int which = unit / (MT * NT), rem = unit - which * (MT * NT), mt = rem / NT, nt = rem - mt * NT;
            const uint32_t *ph = planes1 + (size_t)(which * 2) * L.kp * L.ld, *pl = ph + L.kp * L.ld;
            float c[4] = {0.f, 0.f, 0.f, 0.f};
            for (int kt = 0; kt < KT; kt++) {
                uint32_t af[4];
                sign_fragment(rb_out, mt, kt, g, t, af);
                const int o = (kt * 8 + t) * L.ld + nt * 8 + g;
                mma_16816(c, af, ph[o], ph[o + 4 * L.ld]);
                mma_16816(c, af, pl[o], pl[o + 4 * L.ld]);
            }
            float *dst = tbuf + (size_t)which * 32 * ldt + (mt * 16 + g) * ldt + nt * 8 + 2 * t;
            dst[0] = c[0]; dst[1] = c[1];
            dst[8 * ldt] = c[2]; dst[8 * ldt + 1] = c[3];
        }
    }
    __syncthreads();
    cluster_wait();       // (arrive above) every CTA runs, so its shared memory may be written

    // ---- phase 3: per pair of own rows: transform over j, signs, SwiGLU, signs, transform; push to all CTAs
    for (int rp = warp; 2 * rp < rows_here; rp += kMidWarps) {
        float b[2][E];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int il = 2 * rp + h;
            if (il < rows_here) {                      // uniform over the warp
                float gv[E], uv[E];
#pragma unroll
                for (int e = 0; e < E; e++) { gv[e] = tbuf[il * ldt + lane + 32 * e]; uv[e] = tbuf[32 * ldt + il * ldt + lane + 32 * e]; }
                fwht_warp<E>(gv, lane);
                fwht_warp<E>(uv, lane);
#pragma unroll
                for (int e = 0; e < E; e++) {
                    const int j = il * len + lane + 32 * e;
                    const float gg = __half2float(__float2half_rn(gv[e] * a.scale_out * svg[j]));   // fp16 output tensors
                    const float uu = __half2float(__float2half_rn(uv[e] * a.scale_out * svu[j]));
                    b[h][e] = swiglu_fp16(gg, uu) * __half2float(su[j]);
                }
                fwht_warp<E>(b[h], lane);
            } else {
#pragma unroll
                for (int e = 0; e < E; e++) b[h][e] = 0.f;
            }
        }
#pragma unroll
        for (int e = 0; e < E; e++) {
            __half h0, l0, h1, l1;
            split_f32(b[0][e], h0, l0); split_f32(b[1][e], h1, l1);
            const uint32_t hi = pack_h2(h0, h1), lo = pack_h2(l0, l1);
            uint32_t *dst = planes2 + (i0 / 2 + rp) * L.ld + lane + 32 * e;
            const uint32_t a_hi = (uint32_t)__cvta_generic_to_shared(dst), a_lo = (uint32_t)__cvta_generic_to_shared(dst + L.kp * L.ld);
#pragma unroll
            for (int q = 0; q < kMidCluster; q++) { store_remote(a_hi, q, hi); store_remote(a_lo, q, lo); }
        }
    }
    cluster_arrive();
    cluster_wait();       // all rows of B have landed in this CTA's planes; nobody touches remote memory afterwards

    // ---- phase 4: X[i0+il][j] = sum_i S[i][i0+il] * B[i][j]
    {
        constexpr int NT = len / 8;
        const int MT = (rows_here + 15) >> 4;
        const uint32_t *ph = planes2, *pl = planes2 + L.kp * L.ld;
        for (int unit = warp; unit < MT * NT; unit += kMidWarps) {
            const int mt = unit / NT, nt = unit - mt * NT;
            float c[4] = {0.f, 0.f, 0.f, 0.f};
            for (int kt = 0; kt < KT; kt++) {
                uint32_t af[4];
                sign_fragment(rb_in, mt, kt, g, t, af);
                const int o = (kt * 8 + t) * L.ld + nt * 8 + g;
                mma_16816(c, af, ph[o], ph[o + 4 * L.ld]);
                mma_16816(c, af, pl[o], pl[o + 4 * L.ld]);
            }
            const int il0 = mt * 16 + g, il1 = il0 + 8, j = nt * 8 + 2 * t;
            if (il0 < rows_here)
                *reinterpret_cast<__half2 *>(a.out + (size_t)(i0 + il0) * len + j) = __floats2half2_rn(c[0] * a.scale_in, c[1] * a.scale_in);
            if (il1 < rows_here)
                *reinterpret_cast<__half2 *>(a.out + (size_t)(i0 + il1) * len + j) = __floats2half2_rn(c[2] * a.scale_in, c[3] * a.scale_in);
        }
    }
}

int mid_rows_per_cta(int kfac) {
    int r = (kfac + kMidCluster - 1) / kMidCluster;
    return (r + 1) & ~1;    // even: two rows share a word of the planes
}

}  // namespace
}  // namespace qtip

using namespace qtip;

extern "C" int qtip_mlp_mid_supported(int n, int kfac) {
    if (kfac <= 1 || kfac > kMaxFactor || (kfac & 3) || n <= 0 || n % kfac) return 0;
    const int len = n / kfac;
    if (len != 32 && len != 64 && len != 128) return 0;
    const int R = mid_rows_per_cta(kfac);
    if (R > 32) return 0;
    return (size_t)mid_layout(kfac, len, R).total * 4 <= 227u * 1024u ? 1 : 0;
}

extern "C" int qtip_mlp_mid(void *out, const float *y_gate, const float *y_up, const float *sign_gate, const float *sign_up,
                            const void *sign_down, const uint32_t *hadk_bits, int n, int kfac, float scale_out,
                            float scale_in, void *stream) {
    if (!out || !y_gate || !y_up || !sign_gate || !sign_up || !sign_down || !hadk_bits) return QTIP_ERR_BAD_ARG;
    if (!qtip_mlp_mid_supported(n, kfac)) return QTIP_ERR_BAD_SHAPE;
    const void *ptrs[] = {out, y_gate, y_up, sign_gate, sign_up, sign_down};
    for (const void *p : ptrs)
        if (!aligned(p, 16)) return QTIP_ERR_ALIGNMENT;
    if (!aligned(hadk_bits, 4)) return QTIP_ERR_ALIGNMENT;
    MlpMidArgs a = {};
    a.y_gate = y_gate; a.y_up = y_up; a.sv_gate = sign_gate; a.sv_up = sign_up;
    a.su_down = static_cast<const __half *>(sign_down); a.out = static_cast<__half *>(out); a.hadk_bits = hadk_bits;
    a.n = n; a.kfac = kfac; a.len = n / kfac; a.rows_per_cta = mid_rows_per_cta(kfac);
    a.scale_out = scale_out; a.scale_in = scale_in;
    const size_t smem = (size_t)mid_layout(kfac, a.len, a.rows_per_cta).total * 4;
    void (*kernel)(const MlpMidArgs) = a.len == 32 ? mlp_mid_kernel<1> : a.len == 64 ? mlp_mid_kernel<2> : mlp_mid_kernel<4>;
    static bool attr_set[64][3] = {};
    int dev = 0;
    QTIP_CUDA_TRY(cudaGetDevice(&dev));
    const int which = a.len == 32 ? 0 : a.len == 64 ? 1 : 2;
    if (dev < 64 && !attr_set[dev][which]) {
        QTIP_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        attr_set[dev][which] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kMidCluster);
    cfg.blockDim = dim3(kMidThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kMidCluster; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    QTIP_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, a));
    return check_launch();
}
