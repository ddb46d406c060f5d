// Everything between the gate/up matvecs and the down matvec of a Llama MLP at batch 1, in ONE launch of
// one thread-block cluster (16 CTAs, or 8 where 16 cannot be co-scheduled), for widths n = kfac * len whose Hadamard transform has a non-trivial +-1 factor
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
//   0  (weights only, before the grid dependency wait) cp.async of the bit rows this CTA needs for both
//      products (a table derived once from the packed factor matrix) and of its slices of the sign vectors
//   1  y_gate, y_up -> shared memory as fp16 head / remainder planes, pairs of consecutive k packed in one
//      word ([k/2][j]): exactly the B-fragment layout of mma.m16n8k16
//   2  T = S[own rows, :] * Y for gate and up: one 16x8 output tile per warp, 11 k steps
//   3  one warp per own row: Walsh-Hadamard over j (registers + shuffles), signs, SwiGLU, sign; the result is
//      an fp16 number and is pushed as such into the planes of ALL CTAs of the cluster (distributed shared
//      memory), then one cluster barrier
//   4  X' = S^T[own rows, :] * A on the tensor cores - exact, so one MMA per step - and
//   5  Walsh-Hadamard over j of the own rows (it commutes with the factor), scale, round to fp16, store
#include <mutex>

#include "fwht.cuh"

namespace qtip {
namespace {

constexpr int kMidThreads = 1024, kMidWarps = 32;
constexpr int kMidClusterMax = 16;   // 16 (non-portable size) when the device can co-schedule it, else 8
constexpr int kMaxFactor = 176;   // kfac padded to a multiple of 16
constexpr int kRowWords = 8;      // words per bit row (kfac <= 256 would fit; 6 used for 172)

struct MlpMidArgs {
    const float *y_gate, *y_up, *sv_gate, *sv_up;
    const __half *su_down;
    __half *out;
    const uint32_t *table;      // mid_prepare_kernel's output
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

__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
constexpr int kTableWords = kMidClusterMax * 2 * 32 * kRowWords;   // [rank][first, second product][32 rows][kRowWords]

struct MidLayout {     // offsets in 32-bit words from the start of dynamic shared memory
    int rb, sv_g, sv_u, su, planes1, tbuf, planes2, total;
    int ld;            // words per plane row: len + 8 (bank-conflict-free B fragments)
    int kp;            // plane rows: padded kfac / 2
};
__host__ __device__ inline MidLayout mid_layout(int kfac, int len, int R) {
    MidLayout L;
    const int kpad = (kfac + 15) & ~15;
    L.ld = len + 8;
    L.kp = kpad >> 1;
    int o = 0;
    L.rb = o;      o += 2 * 32 * kRowWords;    // bit rows of the first product, then of the second
    L.sv_g = o;    o += R * len;
    L.sv_u = o;    o += R * len;
    L.su = o;      o += R * len / 2;
    L.planes1 = o; o += 4 * L.kp * L.ld;      // [gate, up][head, remainder][kp][ld]
    L.tbuf = o;    o += 2 * 32 * (len + 4);   // [gate, up][32 rows][len + 4] fp32
    L.planes2 = o; o += L.kp * L.ld;          // [kp][ld]: the SwiGLU result of all rows, fp16
    L.total = o;
    return L;
}


// The bit rows every CTA of the cluster needs, derived once per factor matrix:
// table[rank][0][il] = row (rank*R + il) of S, table[rank][1][il] = column (rank*R + il) of S, zero beyond kfac.
__global__ void mid_prepare_kernel(uint32_t *__restrict__ table, const uint32_t *__restrict__ bits, int kfac, int R) {
    const int rank = blockIdx.x, wpr = (kfac + 31) >> 5, i0 = rank * R;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t *out = table + rank * 2 * 32 * kRowWords;
    for (int i = threadIdx.x; i < 32 * kRowWords; i += blockDim.x) {
        const int il = i / kRowWords, w = i % kRowWords, row = i0 + il;
        out[i] = (il < R && row < kfac && w < wpr) ? bits[row * wpr + w] : 0u;
    }
    for (int u = warp; u < 32 * kRowWords; u += (int)(blockDim.x >> 5)) {
        const int il = u / kRowWords, w = u % kRowWords, k = 32 * w + lane, col = i0 + il;
        const bool bit = il < R && col < kfac && k < kfac && ((bits[k * wpr + (col >> 5)] >> (col & 31)) & 1u);
        const uint32_t word = __ballot_sync(kFullMask, bit);
        if (lane == 0) out[32 * kRowWords + u] = word;
    }
}

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src) : "memory");
}
template <int E>   // len = 32 * E
__global__ void __launch_bounds__(kMidThreads, 1) mlp_mid_kernel(const MlpMidArgs a) {
    extern __shared__ __align__(16) uint32_t smw[];
    constexpr int len = 32 * E;
    const int kfac = a.kfac, R = a.rows_per_cta;
    const MidLayout L = mid_layout(kfac, len, R);
    const int KT = (kfac + 15) >> 4;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int rank = (int)cluster_rank();
    const int i0 = rank * R, rows_here = max(0, min(R, kfac - i0));
    uint32_t *rb_out = smw + L.rb, *rb_in = rb_out + 32 * kRowWords;
    float *svg = reinterpret_cast<float *>(smw + L.sv_g), *svu = reinterpret_cast<float *>(smw + L.sv_u);
    __half *su = reinterpret_cast<__half *>(smw + L.su);
    uint32_t *planes1 = smw + L.planes1, *planes2 = smw + L.planes2;
    float *tbuf = reinterpret_cast<float *>(smw + L.tbuf);
    constexpr int ldt = len + 4;
    // ---- phase 0: weights only, all asynchronous (waited for before phase 2)
    for (int c = tid; c < 2 * 32 * kRowWords / 4; c += kMidThreads) cp_async16(rb_out + c * 4, a.table + rank * 2 * 32 * kRowWords + c * 4);
    if (rows_here > 0) {
        const size_t off = (size_t)i0 * len;
        for (int c = tid; c < rows_here * len / 4; c += kMidThreads) {
            cp_async16(svg + c * 4, a.sv_gate + off + c * 4);
            cp_async16(svu + c * 4, a.sv_up + off + c * 4);
        }
        for (int c = tid; c < rows_here * len / 8; c += kMidThreads) cp_async16(su + c * 8, a.su_down + off + c * 8);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    // rows of planes2 that no CTA writes (k >= kfac)
    for (int i = tid; i < (L.kp - kfac / 2) * L.ld; i += kMidThreads) planes2[(kfac / 2) * L.ld + i] = 0u;
    cluster_arrive();     // every CTA of the cluster is running; matched by the wait before the remote stores
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- phase 1: y_gate, y_up -> head / remainder planes, [k/2][j] words.  One item = (which, k pair, 4 columns);
    // a thread's items are all requested before the first is converted.
    {
        constexpr int jq = len / 4, U = 3;
        const int per = L.kp * jq, items = 2 * per;
        for (int it0 = tid; it0 < items; it0 += U * kMidThreads) {
            float4 r0[U], r1[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int it = it0 + u * kMidThreads;
                r0[u] = r1[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (it < items) {
                    const int which = it >= per, rem = it - which * per, kpi = rem / jq, jg = rem % jq;
                    const float *src = (which ? a.y_up : a.y_gate) + (size_t)(2 * kpi) * len + 4 * jg;
                    if (2 * kpi < kfac) r0[u] = __ldcg(reinterpret_cast<const float4 *>(src));
                    if (2 * kpi + 1 < kfac) r1[u] = __ldcg(reinterpret_cast<const float4 *>(src + len));
                }
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int it = it0 + u * kMidThreads;
                if (it >= items) continue;
                const int which = it >= per, rem = it - which * per, kpi = rem / jq, jg = rem % jq;
                const float e0[4] = {r0[u].x, r0[u].y, r0[u].z, r0[u].w}, e1[4] = {r1[u].x, r1[u].y, r1[u].z, r1[u].w};
                uint32_t hi[4], lo[4];
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    // rows k (low half) and k+1 (high half) of one column: one packed conversion each for head and remainder
                    const __half2 h2 = __floats2half2_rn(e0[q], e1[q]);
                    const float2 back = __half22float2(h2);
                    const __half2 l2 = __floats2half2_rn(e0[q] - back.x, e1[q] - back.y);
                    hi[q] = *reinterpret_cast<const uint32_t *>(&h2);
                    lo[q] = *reinterpret_cast<const uint32_t *>(&l2);
                }
                uint32_t *dst = planes1 + (size_t)(which * 2) * L.kp * L.ld + kpi * L.ld + 4 * jg;
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

    // ---- phase 3: one warp per own row: transform over j, signs, SwiGLU, sign; the fp16 result goes to the planes
    // of ALL CTAs of the cluster.  It is exactly representable in fp16 (sign_down is +-1), so the second product
    // needs no head / remainder split when it runs BEFORE the second transform over j (the two commute).
    if (warp < rows_here) {
        const int il = warp;
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
            const __half av = __float2half_rn(swiglu_fp16(gg, uu) * __half2float(su[j]));
            const int row = i0 + il;
            reinterpret_cast<__half *>(planes2 + (row >> 1) * L.ld + lane + 32 * e)[row & 1] = av;
        }
    }
    cluster_arrive();
    cluster_wait();       // every CTA has written its own rows into its own planes
    // pull the other CTAs' rows (16-byte distributed-shared-memory loads; same offsets in every CTA)
    {
        const int chunks = (kfac / 2) * L.ld / 4, rows2 = R / 2;
        const uint32_t base = (uint32_t)__cvta_generic_to_shared(planes2);
        for (int c0 = tid; c0 < chunks; c0 += 2 * kMidThreads) {
            uint4 v[2];
            bool take[2];
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const int c = c0 + u * kMidThreads;
                const int owner = c < chunks ? (c * 4 / L.ld) / rows2 : rank;
                take[u] = owner != rank;
                if (take[u]) {
                    uint32_t remote;
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(base + c * 16), "r"(owner));
                    asm volatile("ld.shared::cluster.v4.u32 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w) : "r"(remote) : "memory");
                }
            }
#pragma unroll
            for (int u = 0; u < 2; u++)
                if (take[u]) reinterpret_cast<uint4 *>(planes2)[c0 + u * kMidThreads] = v[u];
        }
    }
    cluster_arrive();     // this CTA no longer reads remote memory; matched by the wait at the end of the kernel
    __syncthreads();

    // ---- phase 4: X'[il][j] = sum_i S[i][i0+il] * a[i][j]  (exact: +-1 times fp16, fp32 accumulation)
    {
        constexpr int NT = len / 8;
        const int MT = (rows_here + 15) >> 4;
        for (int unit = warp; unit < MT * NT; unit += kMidWarps) {
            const int mt = unit / NT, nt = unit - mt * NT;
            float c[4] = {0.f, 0.f, 0.f, 0.f};
            for (int kt = 0; kt < KT; kt++) {
                uint32_t af[4];
                sign_fragment(rb_in, mt, kt, g, t, af);
                const int o = (kt * 8 + t) * L.ld + nt * 8 + g;
                mma_16816(c, af, planes2[o], planes2[o + 4 * L.ld]);
            }
            float *dst = tbuf + (mt * 16 + g) * ldt + nt * 8 + 2 * t;
            dst[0] = c[0]; dst[1] = c[1];
            dst[8 * ldt] = c[2]; dst[8 * ldt + 1] = c[3];
        }
    }
    __syncthreads();
    // ---- phase 5: transform over j of the own rows, scale, round, store
    if (warp < rows_here) {
        float v[E];
#pragma unroll
        for (int e = 0; e < E; e++) v[e] = tbuf[warp * ldt + lane + 32 * e];
        fwht_warp<E>(v, lane);
#pragma unroll
        for (int e = 0; e < E; e++) a.out[(size_t)(i0 + warp) * len + lane + 32 * e] = __float2half_rn(v[e] * a.scale_in);
    }
    cluster_wait();       // nobody is still reading this CTA's shared memory
}

int mid_rows_per_cta(int kfac, int cluster) {
    int r = (kfac + cluster - 1) / cluster;
    return (r + 1) & ~1;    // even: two rows share a word of the planes
}

template <int E>
int mid_max_clusters(int cluster, size_t smem) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cluster);
    cfg.blockDim = dim3(kMidThreads);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, mlp_mid_kernel<E>, &cfg) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}

// Cluster size for this device: 16 CTAs when the hardware can co-schedule them, else 8 (decided once per device).
template <int E>
int mid_cluster_size_for(int dev) {
    static int cached[64] = {};
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 0 || dev >= 64) return 8;
    if (!cached[dev]) {
        cudaFuncSetAttribute(mlp_mid_kernel<E>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        const bool np = cudaFuncSetAttribute(mlp_mid_kernel<E>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
        cudaGetLastError();
        cached[dev] = (np && mid_max_clusters<E>(16, 200 * 1024) >= 1) ? 16 : 8;
    }
    return cached[dev];
}

int mid_cluster_size(int len) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 8;
    return len == 32 ? mid_cluster_size_for<1>(dev) : len == 64 ? mid_cluster_size_for<2>(dev) : mid_cluster_size_for<4>(dev);
}

}  // namespace
}  // namespace qtip

using namespace qtip;


extern "C" int qtip_mlp_mid_supported(int n, int kfac) {
    if (kfac <= 1 || kfac > kMaxFactor || (kfac & 3) || n <= 0 || n % kfac) return 0;
    const int len = n / kfac;
    if (len != 32 && len != 64 && len != 128) return 0;
    const int R = mid_rows_per_cta(kfac, 8);     // the smaller cluster needs the most shared memory per CTA
    if (R > 32) return 0;
    return (size_t)mid_layout(kfac, len, R).total * 4 <= 227u * 1024u ? 1 : 0;
}

extern "C" size_t qtip_mlp_mid_table_bytes(void) { return (size_t)kTableWords * 4; }

extern "C" int qtip_mlp_mid_prepare(void *table, const uint32_t *hadk_bits, int n, int kfac, void *stream) {
    if (!table || !hadk_bits) return QTIP_ERR_BAD_ARG;
    if (!qtip_mlp_mid_supported(n, kfac)) return QTIP_ERR_BAD_SHAPE;
    if (!aligned(table, 16) || !aligned(hadk_bits, 4)) return QTIP_ERR_ALIGNMENT;
    const int cluster = mid_cluster_size(n / kfac);
    mid_prepare_kernel<<<cluster, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint32_t *>(table), hadk_bits, kfac,
                                                                                mid_rows_per_cta(kfac, cluster));
    return check_launch();
}

extern "C" int qtip_mlp_mid(void *out, const float *y_gate, const float *y_up, const float *sign_gate, const float *sign_up,
                            const void *sign_down, const void *table, int n, int kfac, float scale_out, float scale_in,
                            void *stream) {
    if (!out || !y_gate || !y_up || !sign_gate || !sign_up || !sign_down || !table) return QTIP_ERR_BAD_ARG;
    if (!qtip_mlp_mid_supported(n, kfac)) return QTIP_ERR_BAD_SHAPE;
    const void *ptrs[] = {out, y_gate, y_up, sign_gate, sign_up, sign_down, table};
    for (const void *p : ptrs)
        if (!aligned(p, 16)) return QTIP_ERR_ALIGNMENT;
    MlpMidArgs a = {};
    a.y_gate = y_gate; a.y_up = y_up; a.sv_gate = sign_gate; a.sv_up = sign_up;
    a.su_down = static_cast<const __half *>(sign_down); a.out = static_cast<__half *>(out);
    a.table = static_cast<const uint32_t *>(table);
    a.n = n; a.kfac = kfac; a.len = n / kfac;
    const int cluster = mid_cluster_size(a.len);   // also sets the kernel's shared-memory and cluster attributes
    a.rows_per_cta = mid_rows_per_cta(kfac, cluster);
    a.scale_out = scale_out; a.scale_in = scale_in;
    const size_t smem = (size_t)mid_layout(kfac, a.len, a.rows_per_cta).total * 4;
    void (*kernel)(const MlpMidArgs) = a.len == 32 ? mlp_mid_kernel<1> : a.len == 64 ? mlp_mid_kernel<2> : mlp_mid_kernel<4>;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cluster);
    cfg.blockDim = dim3(kMidThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    QTIP_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, a));
    return check_launch();
}
