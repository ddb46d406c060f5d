/*
 * CPU restatement (plain C + OpenMP) of the QTIP quantized-linear path.  TEST INFRASTRUCTURE ONLY.
 *
 * It is the checker the CUDA library is compared with at sizes the numpy restatement
 * (qtip_oracle.py) is too slow for, and the timed CPU baseline of the benchmark.  The product
 * library never links or calls it.  It is itself pinned against qtip_oracle.py and the golden
 * fixtures (tests/test_oracle.py), which in turn are pinned against the upstream torch code.
 *
 * Upstream lines each function follows (paths inside the QTIP project):
 *   qo_hyb_expand_lut      lib/codebook/bitshift.py:72-80          quantlut_sym
 *   qo_code_table          lib/codebook/bitshift.py:17-26, 43-60   decode_1mad, decode_3inst
 *   qo_decode_kernel       lib/utils/kernel_decompress.py:4-55     decode_compressed
 *   qo_decode_plain        lib/codebook/bitshift.py:329-353, 378-381  unpack_trellis + get_hatW
 *   qo_matvec_kernel       qtip-kernels/src/inference.cu:168-425   fused decode + matvec, fp32 accumulate
 *   qo_hadamard            lib/utils/matmul_had.py:105-119         matmul_hadU_cuda
 *   qo_layer_forward       lib/codebook/bitshift.py:415-472        BitshiftLinear.forward
 *
 * fp16 values are uint16_t bit patterns.  K = bits per weight, m = out, n = in.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static float g_h2f[65536];
static int g_h2f_ready = 0;

static float half_bits_to_float(uint16_t h) {
    uint32_t s = (uint32_t)(h >> 15) << 31, e = (h >> 10) & 31, f = h & 1023, u;
    if (e == 0) {
        if (f == 0) u = s;
        else {
            int sh = 0;
            while (!(f & 1024)) { f <<= 1; sh++; }
            u = s | ((uint32_t)(113 - sh) << 23) | ((f & 1023) << 13);
        }
    } else if (e == 31) u = s | 0x7F800000u | (f << 13);
    else u = s | ((e + 112) << 23) | (f << 13);
    float r; memcpy(&r, &u, 4); return r;
}

/* round-to-nearest-even fp32 -> fp16 */
static uint16_t float_to_half_bits(float x) {
    uint32_t u; memcpy(&u, &x, 4);
    uint32_t s = (u >> 16) & 0x8000u, a = u & 0x7FFFFFFFu;
    if (a >= 0x7F800000u) return (uint16_t)(s | 0x7C00u | ((a > 0x7F800000u) ? 0x200u : 0));
    if (a >= 0x477FF000u) return (uint16_t)(s | 0x7C00u);               /* rounds to inf */
    if (a < 0x33000001u) return (uint16_t)s;                             /* rounds to zero */
    int e = (int)(a >> 23) - 127;
    uint32_t mant = (a & 0x7FFFFFu) | 0x800000u;
    int shift = (e < -14) ? (13 + (-14 - e)) : 13;
    uint32_t half_mant = mant >> shift, rem = mant & ((1u << shift) - 1), halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (half_mant & 1))) half_mant++;
    uint32_t r = (e < -14) ? half_mant : (((uint32_t)(e + 15) << 10) + (half_mant - 1024u));
    return (uint16_t)(s | r);
}

void qo_init(void) {
    if (g_h2f_ready) return;
    for (int i = 0; i < 65536; i++) g_h2f[i] = half_bits_to_float((uint16_t)i);
    g_h2f_ready = 1;
}

/* launchers such as torchrun export OMP_NUM_THREADS=1; the CPU baseline wants every host core */
void qo_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int qo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void qo_float_to_half(const float *x, uint16_t *y, long cnt) {
    for (long i = 0; i < cnt; i++) y[i] = float_to_half_bits(x[i]);
}

static inline uint32_t hyb_hash(uint32_t s) { return (s * (s + 1u)) & 0xFFFFu; }

/* tlut: 512 x 2 fp16; lut16: 65536 x 2 fp16 */
void qo_hyb_expand_lut(const uint16_t *tlut, uint16_t *lut16) {
    for (uint32_t s = 0; s < 65536; s++) {
        uint32_t h = hyb_hash(s), idx = (h >> 6) & 511u;
        lut16[2 * s] = tlut[2 * idx] ^ (uint16_t)((h >> 15) << 15);
        lut16[2 * s + 1] = tlut[2 * idx + 1];
    }
}

/* code 1 = 3INST (exact fp16), code 2 = 1MAD (fp32 value rounded once to fp16); table: 65536 fp16 */
void qo_code_table(int code, uint16_t *table) {
    qo_init();
    for (uint32_t s = 0; s < 65536; s++) {
        if (code == 1) {
            uint32_t x = s * 89226354u + 64248484u;
            uint32_t r = (x & 0x8FFF8FFFu) ^ 0x3B603B60u;
            float sum = g_h2f[r >> 16] + g_h2f[r & 0xFFFF];  /* exact in fp32, one rounding = fp16 add */
            table[s] = float_to_half_bits(sum);
        } else {
            uint32_t x = s * 34038481u + 76625530u;
            int y = (int)((x & 255) + ((x >> 8) & 255) + ((x >> 16) & 255) + (x >> 24)) - 510;
            float v = (float)y / 147.800537109375f;
            table[s] = float_to_half_bits(v);
        }
    }
}

/* states of one lane of a 2x2 tile block in the kernel layout.
 * blk points at [lane 32][ks 2][ms 2][K bytes]; returns the 4 states of (lane, ks, ms). */
static inline void kernel_lane_states(const uint8_t *blk, int K, int lane, int ks, int ms, uint32_t st[4]) {
    const uint8_t *p = blk + ((lane * 2 + ks) * 2 + ms) * K;
    const uint8_t *q = blk + ((((lane + 1) & 31) * 2 + ks) * 2 + ms) * K;
    uint64_t a = 0, b = 0;
    for (int i = 0; i < K; i++) { a |= (uint64_t)p[i] << (8 * i); b |= (uint64_t)q[i] << (8 * i); }
    uint64_t win = (a << (8 * K)) | b;
    for (int s = 0; s < 4; s++) st[s] = (uint32_t)(win >> (16 * K - 16 - 2 * K * s)) & 0xFFFFu;
}

/* HYB kernel-layout decode: W (m x n fp16) */
void qo_decode_kernel(const uint8_t *codes, int m, int n, int K, const uint16_t *tlut, uint16_t *W) {
    uint16_t *lut16 = (uint16_t *)malloc(65536 * 2 * sizeof(uint16_t));
    qo_hyb_expand_lut(tlut, lut16);
    int MB = m / 32, NB = n / 32;
#pragma omp parallel for schedule(static)
    for (int M = 0; M < MB; M++)
        for (int N = 0; N < NB; N++) {
            const uint8_t *blk = codes + ((size_t)M * NB + N) * 128 * K;
            for (int lane = 0; lane < 32; lane++) {
                int a = lane >> 2, b = lane & 3;
                for (int ks = 0; ks < 2; ks++)
                    for (int ms = 0; ms < 2; ms++) {
                        uint32_t st[4];
                        kernel_lane_states(blk, K, lane, ks, ms, st);
                        for (int q = 0; q < 4; q++) {
                            int c = q >> 1, d = q & 1;
                            size_t row = 32 * M + 16 * ms + 8 * d + a, col = 32 * N + 16 * ks + 8 * c + 2 * b;
                            W[row * n + col] = lut16[2 * st[q]];
                            W[row * n + col + 1] = lut16[2 * st[q] + 1];
                        }
                    }
            }
        }
    free(lut16);
}

/* plain-layout decode, V weights per state; table is 65536 x V fp16 */
void qo_decode_plain(const uint16_t *codes, int m, int n, int K, int V, const uint16_t *table, uint16_t *W) {
    int TN = n / 16, tiles = (m / 16) * TN, T = 256 / V, nbits = 256 * K;
#pragma omp parallel for schedule(static)
    for (int t = 0; t < tiles; t++) {
        const uint16_t *w = codes + (size_t)t * 16 * K;
        int tr = t / TN, tc = t % TN;
        for (int i = 0; i < T; i++) {
            int pos = i * K * V;
            uint32_t s = 0;
            for (int j = 0; j < 16; j++) {
                int bit = (pos + j) % nbits;
                s = (s << 1) | ((w[bit >> 4] >> (15 - (bit & 15))) & 1u);
            }
            for (int v = 0; v < V; v++) {
                int e = i * V + v;
                W[(size_t)(tr * 16 + e / 16) * n + tc * 16 + (e % 16)] = table[s * V + v];
            }
        }
    }
}

/* dense fp16 matvec with wide accumulation: y[b][r] = sum_c W[r][c] * x[b][c] */
void qo_matvec_dense(const uint16_t *W, const uint16_t *x, int m, int n, int bs, float *y) {
    qo_init();
#pragma omp parallel for schedule(static)
    for (int r = 0; r < m; r++)
        for (int b = 0; b < bs; b++) {
            double acc = 0;
            for (int c = 0; c < n; c++) acc += (double)g_h2f[W[(size_t)r * n + c]] * (double)g_h2f[x[(size_t)b * n + c]];
            y[(size_t)b * m + r] = (float)acc;
        }
}

/* fused HYB kernel-layout decode + matvec, fp32 accumulation per output row (the upstream CUDA op) */
void qo_matvec_kernel(const uint8_t *codes, int m, int n, int K, const uint16_t *tlut, const uint16_t *x,
                      int bs, float *y) {
    qo_init();
    uint16_t *lut16 = (uint16_t *)malloc(65536 * 2 * sizeof(uint16_t));
    qo_hyb_expand_lut(tlut, lut16);
    int MB = m / 32, NB = n / 32;
#pragma omp parallel
    {
        float *xf = (float *)malloc(sizeof(float) * (size_t)n * bs);
        for (long i = 0; i < (long)n * bs; i++) xf[i] = g_h2f[x[i]];
        float *acc = (float *)malloc(sizeof(float) * 32 * bs);
#pragma omp for schedule(static)
        for (int M = 0; M < MB; M++) {
            memset(acc, 0, sizeof(float) * 32 * bs);
            for (int N = 0; N < NB; N++) {
                const uint8_t *blk = codes + ((size_t)M * NB + N) * 128 * K;
                for (int lane = 0; lane < 32; lane++) {
                    int a = lane >> 2, b = lane & 3;
                    for (int ks = 0; ks < 2; ks++)
                        for (int ms = 0; ms < 2; ms++) {
                            uint32_t st[4];
                            kernel_lane_states(blk, K, lane, ks, ms, st);
                            for (int q = 0; q < 4; q++) {
                                int c = q >> 1, d = q & 1;
                                int row = 16 * ms + 8 * d + a, col = 32 * N + 16 * ks + 8 * c + 2 * b;
                                float w0 = g_h2f[lut16[2 * st[q]]], w1 = g_h2f[lut16[2 * st[q] + 1]];
                                for (int bb = 0; bb < bs; bb++)
                                    acc[bb * 32 + row] += w0 * xf[(size_t)bb * n + col] + w1 * xf[(size_t)bb * n + col + 1];
                            }
                        }
                }
            }
            for (int bb = 0; bb < bs; bb++)
                for (int r = 0; r < 32; r++) y[(size_t)bb * m + 32 * M + r] = acc[bb * 32 + r];
        }
        free(acc);
        free(xf);
    }
    free(lut16);
}

/* in-place unnormalised Walsh-Hadamard transform (Sylvester order) of length len (power of two) */
static void fwht(float *v, int len) {
    for (int h = 1; h < len; h <<= 1)
        for (int i = 0; i < len; i += 2 * h)
            for (int j = i; j < i + h; j++) {
                float a = v[j], b = v[j + h];
                v[j] = a + b; v[j + h] = a - b;
            }
}

/* x: (rows, n) in place.  n = kfac * 2^p; hadK (kfac x kfac, +-1 floats, row-major) or NULL when kfac == 1.
 * transpose != 0 uses hadK^T (the input-side transform). */
void qo_hadamard(float *x, long rows, int n, const float *hadK, int kfac, int transpose) {
    float scale = (float)(1.0 / sqrt((double)n));
    int len = n / kfac;
#pragma omp parallel for schedule(static) if (rows > 1)
    for (long r = 0; r < rows; r++) {
        float *v = x + r * n;
        for (int k = 0; k < kfac; k++) fwht(v + (size_t)k * len, len);
        if (kfac > 1) {
            double *col = (double *)malloc(sizeof(double) * kfac);
            for (int j = 0; j < len; j++) {
                for (int i = 0; i < kfac; i++) {
                    double acc = 0;
                    for (int k = 0; k < kfac; k++)
                        acc += (double)(transpose ? hadK[k * kfac + i] : hadK[i * kfac + k]) * v[(size_t)k * len + j];
                    col[i] = acc;
                }
                for (int i = 0; i < kfac; i++) v[(size_t)i * len + j] = (float)col[i];
            }
            free(col);
        }
        for (int i = 0; i < n; i++) v[i] *= scale;
    }
}

/* BitshiftLinear.forward for HYB kernel-layout codes.  x (bs, n) fp32 -> y (bs, m) fp32.
 * rcp 0: plain; 1: input-side transform per chunk of n/tp; 2: output-side transform per chunk of m/tp.
 * had_left / had_right are the factor matrices for the (chunk) sizes, kl / kr their orders (1 = none). */
void qo_layer_forward(const float *x, int bs, const uint8_t *codes, int m, int n, int K, const uint16_t *tlut,
                      const float *SU, const float *SV, const float *had_left, int kl, const float *had_right, int kr,
                      int rcp, int tp, float *y) {
    float *xs = (float *)malloc(sizeof(float) * (size_t)bs * n);
    uint16_t *xh = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)bs * n);
    for (int b = 0; b < bs; b++)
        for (int i = 0; i < n; i++) xs[(size_t)b * n + i] = x[(size_t)b * n + i] * SU[i];
    if (rcp == 1) qo_hadamard(xs, (long)bs * tp, n / tp, had_left, kl, 1);
    else qo_hadamard(xs, bs, n, had_left, kl, 1);
    for (long i = 0; i < (long)bs * n; i++) xh[i] = float_to_half_bits(xs[i] / 32.0f);
    qo_matvec_kernel(codes, m, n, K, tlut, xh, bs, y);
    if (rcp == 2) qo_hadamard(y, (long)bs * tp, m / tp, had_right, kr, 0);
    else qo_hadamard(y, bs, m, had_right, kr, 0);
    for (int b = 0; b < bs; b++)
        for (int i = 0; i < m; i++) y[(size_t)b * m + i] *= SV[i] * 32.0f;
    free(xs);
    free(xh);
}

/* ------------------------------------------------------------------------------------------------------------------
 * Viterbi quantizer over the bitshift trellis with tail-biting: bitshift_codebook.quantize
 * (lib/codebook/bitshift.py:283-292) = quantize_seq / viterbi / update (:203-281), in upstream's own formulation:
 * a cost per state (2^16 floats), per step the minimum over the 2^(KV) predecessors of each group of 2^(KV) states
 * that share them (first minimal index wins, as torch.min), the squared error of the state's reconstruction added,
 * back-pointers per group, back-trace from the first minimal final state.
 * recons: [V][65536] fp32 (upstream's recons_state); X: N sequences of T fp16 values; states: N x T/V.
 * Arithmetic follows the eager torch ops in fp32: (r - x), square, sum over V, + best.  Built with -ffp-contract=off.
 * ------------------------------------------------------------------------------------------------------------------ */
static inline float seq_err(const float *recons, int V, uint32_t s, const float *x) {
    const float d0 = recons[s] - x[0];
    float e = d0 * d0;
    if (V == 2) {
        const float d1 = recons[65536 + s] - x[1];
        e = e + d1 * d1;
    }
    return e;
}

static void viterbi_pass(const float *x, int S, int KV, int V, const float *recons, int has_overlap, uint32_t overlap,
                         int32_t *out, float *cost, float *cost2, uint16_t *from, float *final_cost) {
    const uint32_t D = 1u << KV, G = 65536u >> KV;
    for (uint32_t s = 0; s < 65536; s++) cost[s] = seq_err(recons, V, s, x);
    if (has_overlap)   /* viterbi :225-231: only states whose top 16-KV bits equal `overlap` may start the walk */
        for (uint32_t s = 0; s < 65536; s++)
            if ((s >> KV) != overlap) cost[s] = INFINITY;
    for (int i = 1; i < S; i++) {
        uint16_t *fr = from + (size_t)i * G;
        for (uint32_t g = 0; g < G; g++) {
            float best = cost[g];
            uint32_t bd = 0;
            for (uint32_t d = 1; d < D; d++) {
                const float c = cost[g + d * G];
                if (c < best) { best = c; bd = d; }
            }
            fr[g] = (uint16_t)(g + bd * G);
            for (uint32_t j = 0; j < D; j++) {
                const uint32_t s = g * D + j;
                cost2[s] = seq_err(recons, V, s, x + (size_t)i * V) + best;
            }
        }
        float *t = cost; cost = cost2; cost2 = t;
    }
    if (has_overlap)   /* :244-249: the last state's low 16-KV bits must equal `overlap` */
        for (uint32_t s = 0; s < 65536; s++)
            if ((s & (G - 1)) != overlap) cost[s] = INFINITY;
    uint32_t arg = 0;
    for (uint32_t s = 1; s < 65536; s++)
        if (cost[s] < cost[arg]) arg = s;
    if (final_cost) *final_cost = cost[arg];
    out[S - 1] = (int32_t)arg;
    for (int i = S - 1; i > 0; i--) out[i - 1] = from[(size_t)i * G + ((uint32_t)out[i] >> KV)];
}

void qo_viterbi_quantize(const uint16_t *X, long N, int T, int K, int V, const float *recons, int32_t *states,
                         float *final_cost) {
    qo_init();
    const int KV = K * V, S = T / V;
    const uint32_t G = 65536u >> KV;
#pragma omp parallel
    {
        float *cost = (float *)malloc(65536 * sizeof(float)), *cost2 = (float *)malloc(65536 * sizeof(float));
        uint16_t *from = (uint16_t *)malloc((size_t)S * G * sizeof(uint16_t));
        float *x = (float *)malloc((size_t)T * sizeof(float)), *xr = (float *)malloc((size_t)T * sizeof(float));
        int32_t *tmp = (int32_t *)malloc((size_t)S * sizeof(int32_t));
#pragma omp for schedule(dynamic, 1)
        for (long b = 0; b < N; b++) {
            for (int t = 0; t < T; t++) x[t] = g_h2f[X[b * T + t]];
            /* quantize :286-289: first pass on the sequence rolled by T/(2V)*V, free ends; the state it finds where the
             * original sequence starts gives the overlap bits both ends of the second pass must agree on */
            const int roll = T / (2 * V) * V;
            for (int t = 0; t < T; t++) xr[(t + roll) % T] = x[t];
            viterbi_pass(xr, S, KV, V, recons, 0, 0u, tmp, cost, cost2, from, NULL);
            const uint32_t overlap = (uint32_t)tmp[T / (2 * V)] >> KV;
            viterbi_pass(x, S, KV, V, recons, 1, overlap, states + b * S, cost, cost2, from, final_cost ? final_cost + b : NULL);
        }
        free(cost); free(cost2); free(from); free(x); free(xr); free(tmp);
    }
}
