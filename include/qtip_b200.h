/*
 * qtip_b200 - C ABI of the B200 (sm_100a) kernels for the QTIP quantized-linear path.
 *
 * Every entry point takes plain device pointers and sizes, launches on the stream it is given
 * (a cudaStream_t passed as void*; NULL = the legacy default stream) on the CURRENT device, does
 * not synchronise, and returns a status code instead of terminating the process (the upstream
 * launcher exits on a launch error: qtip-kernels/src/inference.h:10-18).  Unless a comment says
 * otherwise an entry point allocates nothing, so it may be called while a stream is captured
 * into a CUDA graph.
 *
 * Naming: K = bits per weight (the upstream CUDA template parameter R), m = out_features
 * (upstream M), n = in_features (upstream template K), bs = batch rows.  fp16 buffers are IEEE
 * binary16 (uint16_t storage).  "kernel layout" is the packed trellis format written by
 * lib/algo/finetune.py:196-201 upstream for L=16, V=2, Q=9, 16x16 tiles; "plain layout" is the
 * output of bitshift_codebook.pack_trellis (lib/codebook/bitshift.py:294-327).
 */
#ifndef QTIP_B200_H
#define QTIP_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    QTIP_OK = 0,
    QTIP_ERR_BAD_ARG = 1,      /* NULL pointer, unsupported K / code / dtype, bs out of range */
    QTIP_ERR_BAD_SHAPE = 2,    /* m or n not a multiple of the tile block, size has no Hadamard factorisation */
    QTIP_ERR_WORKSPACE = 3,    /* workspace missing or too small */
    QTIP_ERR_CUDA = 4,         /* a CUDA runtime call or the launch failed; see qtip_last_cuda_error() */
    QTIP_ERR_ALIGNMENT = 5,    /* a pointer is not aligned as documented */
    QTIP_ERR_TOO_LARGE = 6     /* the problem needs more scratch than the built-in array of qtip_decompress_matvec_static */
};

enum { QTIP_CODE_HYB = 0, QTIP_CODE_3INST = 1, QTIP_CODE_1MAD = 2 };
enum { QTIP_F16 = 0, QTIP_F32 = 1 };

/* Human-readable text for a status code; never NULL. */
const char *qtip_status_string(int status);
/* cudaError_t (as int) recorded by the last failing call on this host thread, 0 if none. */
int qtip_last_cuda_error(void);
/* Library version, major*100 + minor. */
int qtip_version(void);

/* --------------------------------------------------------------------------------------------
 * Decoders (trellis codes -> dense fp16 matrix W, row-major (m, n), y = x @ W^T).
 * ------------------------------------------------------------------------------------------ */

/* HYB code, kernel layout.  Replaces decode_compressed (lib/utils/kernel_decompress.py:4-55) and
 * BitshiftLinear.get_hatW_kernel (lib/codebook/bitshift.py:383-387); bit-exact with them.
 * codes: K*m*n/8 bytes, 16-byte aligned; W 16-byte aligned; tlut: 512x2 fp16; m, n multiples of 32; K in {2,3,4}. */
int qtip_decode_hyb(void *W, const void *codes, const void *tlut, int K, int m, int n, void *stream);

/* Plain layout, any of the three codes.  Replaces unpack_trellis + recons + get_hatW
 * (lib/codebook/bitshift.py:329-353, 199-201, 378-381).  HYB uses V=2 and needs tlut; 3INST and
 * 1MAD use V=1, ignore tlut, and are the state functions decode_3inst / decode_1mad (:43-60,
 * :17-26); 1MAD's fp32 value is rounded once (nearest-even) to fp16.  m, n multiples of 16. */
int qtip_decode_plain(void *W, const void *codes, int code, const void *tlut, int K, int m, int n, void *stream);

/* --------------------------------------------------------------------------------------------
 * Measurement support (no counterpart in the reference): issue rates of the instruction classes the decoders are
 * made of, measured on the current device.  The decode kernels are bound by instruction issue rather than by HBM,
 * so these rates, not the memory bandwidth, set their ceiling.
 * qtip_measure_pipe_rates fills cycles[i], i < qtip_pipe_rate_count(), with the cycles one warp-instruction of class i
 * (qtip_pipe_rate_name(i)) costs per SM sub-partition when every sub-partition runs threads_per_cta/128 warps of
 * independent chains; the two "decode sequence" classes are counted per trellis state.  Host pointer; the call
 * allocates and frees its own device scratch and synchronises the device (not for use inside a serving loop).
 * ------------------------------------------------------------------------------------------ */
int qtip_pipe_rate_count(void);
const char *qtip_pipe_rate_name(int i);
int qtip_measure_pipe_rates(double *cycles, int count, int threads_per_cta);

/* --------------------------------------------------------------------------------------------
 * Producers of the packed formats (the quantizer side of the format; pure bit / byte movement, bit-exact).
 * ------------------------------------------------------------------------------------------ */

/* bitshift_codebook.pack_trellis (lib/codebook/bitshift.py:294-327): trellis states -> packed words, plain layout.
 * states: (tiles, 256/V) int32, each a 16-bit state (L = 16); words: (tiles, 16*K) uint16 - the tile's tail-biting
 * bitstream, MSB first: state 0's 16 bits, then the low K*V bits of each later state, the last 16 - K*V bits dropped.
 * violations (optional, one zero-initialised uint32): receives the number of consecutive state pairs that do not
 * overlap by 16 - K*V bits (upstream asserts this, :306-309); the words are written either way. */
int qtip_pack_trellis(void *words, const int *states, long tiles, int K, int V, unsigned *violations, void *stream);

/* bitshift_codebook.quantize (lib/codebook/bitshift.py:283-292; viterbi / update / quantize_seq :203-281): the Viterbi
 * quantizer over the L = 16 bitshift trellis with tail-biting.  X: N sequences of T fp16 values (upstream: the rows of
 * the (N, td_x*td_y) matrix handed to quantize(); T = 256 for 16x16 tiles).  states: (N, T/V) int32, the states of the
 * minimum-squared-error walk whose last state ends with the bits its first state begins with - identical to the states
 * upstream's implementation returns (same fp32 arithmetic, same tie-breaking), ready for qtip_pack_trellis.
 * final_cost (optional): the walk's total squared error per sequence.  code: QTIP_CODE_HYB (V = 2; tlut = 512 x 2 FP32,
 * the table the quantizer holds in fp32) or QTIP_CODE_3INST / QTIP_CODE_1MAD (V = 1, tlut ignored).  K in {2,3,4};
 * T a multiple of 2V, 4V <= T <= 1024 and T*K >= 16 (a tail-biting walk needs at least 16 stream bits).  workspace: qtip_viterbi_workspace_bytes() bytes of device memory
 * (back-pointers; no initialisation needed). */
size_t qtip_viterbi_workspace_bytes(int code, int K, int T, long N);
int qtip_viterbi_quantize(int *states, float *final_cost, const void *X, long N, int T, int code, int K, const float *tlut,
                          void *workspace, size_t workspace_bytes, void *stream);

/* The byte shuffle from the plain layout to the kernel layout for L = 16, V = 2, 16x16 tiles
 * (lib/algo/finetune.py:196-201) and its inverse (lib/utils/kernel_decompress.py:19-24).  Both buffers hold
 * K*m*n/8 bytes and must not alias; m, n multiples of 32. */
int qtip_plain_to_kernel_layout(void *kernel_codes, const void *plain_words, int K, int m, int n, void *stream);
int qtip_kernel_to_plain_layout(void *plain_words, const void *kernel_codes, int K, int m, int n, void *stream);

/* --------------------------------------------------------------------------------------------
 * Fused decode + matvec:  out[b][r] = sum_c W[r][c] * x[b][c],  fp16 operands, fp32 accumulate.
 * ------------------------------------------------------------------------------------------ */

/* Bytes of workspace qtip_decompress_matvec / _plain need for this problem (never 0). */
size_t qtip_matvec_workspace_bytes(int m, int n, int bs);

/* HYB code, kernel layout.  Replaces the 64 fixed-shape functions
 * decompress_matvec_16_9_{K}_1_{m}_1_{n}(out, compressed, x, codebook)
 * (qtip-kernels/src/qtip_torch.cu:14-57 and :60-671, kernel qtip-kernels/src/inference.cu:168-425)
 * with one shape-generic call, and extends them to bs <= 8 rows of x.
 * out: (bs, m) fp32, OVERWRITTEN (need not be zeroed); x: (bs, n) fp16, 16-byte aligned;
 * codes 16-byte aligned; tlut 512x2 fp16.  m, n multiples of 32.
 * workspace: qtip_matvec_workspace_bytes() bytes, 256-byte aligned, ZEROED ONCE by the caller
 * before its first use (the kernel leaves it zeroed again); calls that may overlap on the device
 * need separate workspaces. */
int qtip_decompress_matvec(float *out, const void *codes, const void *x, const void *tlut, int K, int m, int n,
                           int bs, void *workspace, size_t workspace_bytes, void *stream);

/* Decompress-GEMM for batches up to 128 on the tcgen05 tensor cores (accumulator in tensor memory):
 * out (bs, m) fp32 = x (bs, n) fp16 @ decode(codes)^T, HYB code, kernel layout.  Replaces
 * BitshiftLinearKernelAG.forward (lib/codebook/bitshift.py:476-489: decode_compressed to a dense fp16
 * matrix in HBM, then a dense GEMM) without ever materialising the matrix.
 * m a multiple of 128, n a multiple of 64; x and codes 16-byte aligned.  status: one zero-initialised
 * uint32 in device memory; the kernel leaves it 0, or a non-zero code if one of its (bounded) waits on
 * a shared-memory barrier gave up - the results are then meaningless, but the kernel still terminates
 * and frees its tensor memory.  When the row ranges leave SMs idle the input columns are split over
 * two CTAs and `out` is zeroed on the stream first (allocation-free, capturable). */
int qtip_decompress_gemm(float *out, const void *codes, const void *x, const void *tlut, int K, int m, int n, int bs,
                         unsigned *status, void *stream);

/* qtip_decompress_gemm for the compute codes: 3INST / 1MAD, V = 1, plain layout (no LUT).  The batched form of
 * BitshiftLinear.forward's dense branch for codes without a matvec kernel upstream (lib/codebook/bitshift.py:454-463:
 * unpack_trellis + get_hatW + matmul), again without materialising the matrix; the decoded weights are the ones
 * qtip_decode_plain produces (1MAD: the fp32 value rounded once to fp16).  Same shape and status rules. */
int qtip_decompress_gemm_plain(float *out, const void *codes, const void *x, int code, int K, int m, int n, int bs,
                               unsigned *status, void *stream);

/* One to four QTIP linears of the same shape in ONE launch (e.g. q/k/v, or gate/up), each optionally with
 * its input-side and output-side transforms fused into the matvec kernel, i.e. the whole of
 * BitshiftLinear.forward (lib/codebook/bitshift.py:428-472) for a decode step in one kernel:
 *   input side  (in_raw != NULL; needs bs == 1 and n a power of two <= 16384): every CTA computes
 *       x = fp16( H_n^T( sign_in * [silu(gate) *] [RMSNorm]( in_raw [+ residual] ) ) * in_scale )
 *       itself; residual_out (if given) receives in_raw + residual; norm_weight / gate / residual optional.
 *       With in_y != NULL (n = 4096 or 8192) in_raw is not read: the value it stands for is computed on the
 *       fly as fp16( in_y_sign * H_n(in_y) * in_y_scale ), i.e. the output side of the PRODUCER linear
 *       (whose raw y is in_y) is deferred into this launch instead of running in the producer's last CTA.
 *   matvec      y (bs, m) fp32 = x @ decode(codes)^T, always written.
 *   output side (out != NULL; needs m a power of two <= 16384): the CTA that finishes last computes
 *       out = sign_out * H_m(y) * out_scale  (fp16 or fp32).
 * H is the unnormalised Walsh-Hadamard transform; fold n^-1/2, /32 and x32 into the scales as for qtip_rht.
 *   tensor parallelism: a row-parallel linear leaves a partial y on every GPU.  Instead of an all-reduce launch
 *       between it and its consumer, the producer launch (signal_count > 0) also stores every value of y, stamped
 *       with a sequence number in the same 8-byte store, into a vector on every GPU (peer-mapped memory), and the
 *       consumer launch (peer_count > 0, n = 4096 or 8192) re-reads those vectors in its own memory until each
 *       value carries the expected stamp, adds the vectors in rank order and continues as for in_y.  No fence,
 *       flag or atomic lies between the GPUs.  Vectors may be reused every second producer/consumer pair (the
 *       protocol of qtip_b200/tp.py alternates two).  The wait is bounded; peer_status reports a time-out.
 * Either all descriptors of a call use the fused input side or none does.  Every descriptor needs its
 * own zero-initialised workspace (qtip_matvec_workspace_bytes) and its own y. */
typedef struct qtip_linear_desc {
    float *y;
    const void *codes;            /* kernel layout, K*m*n/8 bytes */
    const void *tlut;             /* 512 x 2 fp16 */
    const void *x;                /* (bs, n) fp16, used when in_raw == NULL */
    void *workspace;
    size_t workspace_bytes;
    const void *in_raw;           /* (n) fp16 */
    const void *residual;         /* (n) fp16 or NULL */
    void *residual_out;           /* (n) fp16 or NULL; must not alias in_raw / residual */
    const void *norm_weight;      /* (n) fp16 or NULL */
    const void *gate;             /* (n) fp16 or NULL */
    const void *sign_in;          /* (n) fp16 or NULL */
    float in_scale;
    float eps;
    void *out;                    /* (bs, m) of out_dtype or NULL */
    int out_dtype;
    const float *sign_out;        /* (m) fp32 or NULL */
    float out_scale;
    const float *in_y;            /* (n) fp32 raw output of the producer linear, or NULL */
    const float *in_y_sign;       /* (n) fp32, the producer's sign_out; or NULL */
    float in_y_scale;             /* the producer's out_scale */
    /* tensor parallelism without an all-reduce launch (see above); all zero / NULL when unused */
    int peer_count;               /* consumer: number of GPUs whose partial vectors are summed instead of in_y */
    const void *peer_y[8];        /* GPU p's stamped vector ((n) pairs {fp32 value, uint32 stamp}) in THIS GPU's memory */
    const unsigned *peer_seq;     /* this GPU's sequence counter (the one its own producer launch advances) */
    unsigned *peer_status;        /* set to non-zero if a wait ran out */
    unsigned peer_max_polls;      /* bound on the re-reads of one element group (0: 1 Mi) */
    int signal_count;             /* producer: number of GPUs that receive the result */
    void *signal_y[8];            /* GPU p's stamped vector for THIS rank (peer-mapped; this GPU's own included) */
    unsigned *signal_seq;         /* this GPU's sequence counter, advanced by one per launch */
} qtip_linear_desc;
int qtip_linear_fused(const qtip_linear_desc *descs, int count, int K, int m, int n, int bs, void *stream);

/* Writes sizeof(qtip_linear_desc) and then the byte offset of every field, in declaration order, into out (up to
 * `capacity` entries; out may be NULL) and returns the number of entries (1 + number of fields).  For bindings that
 * mirror the struct by hand: compare at start-up, refuse to run on a mismatch.  No device is touched. */
int qtip_linear_desc_layout(size_t *out, int capacity);

/* qtip_decompress_matvec for callers that must not allocate device memory and have none to spare for a
 * workspace - a serving loop that froze its memory pool at start-up, a plug-in whose host owns every
 * allocation, code running where a cudaMalloc would synchronise the device.  (No counterpart in the
 * reference, whose kernel needs no scratch.)  Same arguments and result as qtip_decompress_matvec minus
 * the workspace: the ticket counters and partial sums live in a 4 MiB + 64.25 KiB array built into the
 * library's device image (each GPU that loads the library holds it until the process exits).  Problems
 * whose qtip_matvec_workspace_bytes(m, n, bs) exceeds that size return QTIP_ERR_TOO_LARGE; every
 * Llama-2/3 layer shape up to 53248 x 16384 fits.  The call itself performs no cudaMalloc / cudaFree
 * and calls no allocating library routine.  The FIRST call on each device looks the array's device
 * address up (cudaGetSymbolAddress, with that device current) - make that call outside any stream
 * capture.  All calls on a device share the one array: its ticket counters are cleared on `stream`
 * before each launch, and two calls that can overlap on the GPU (different streams, or graph branches)
 * race - serialise them or use qtip_decompress_matvec with separate workspaces. */
int qtip_decompress_matvec_static(float *out, const void *codes, const void *x, const void *tlut, int K, int m, int n,
                                  int bs, void *stream);

/* 3INST / 1MAD, plain layout, V=1; same contract as qtip_decompress_matvec (no LUT).  The decoded weights are the
 * ones qtip_decode_plain produces.  m, n multiples of 32. */
int qtip_decompress_matvec_plain(float *out, const void *codes, const void *x, int code, int K, int m, int n,
                                 int bs, void *workspace, size_t workspace_bytes, void *stream);

/* --------------------------------------------------------------------------------------------
 * Randomized Hadamard transform.
 * ------------------------------------------------------------------------------------------ */

/* out[r][:] = sign_out ⊙ ( H_n ( sign_in ⊙ in[r][:] ) ) * scale      for each of `rows` rows.
 * H_n is the UNNORMALISED transform of matmul_hadU_cuda (lib/utils/matmul_had.py:105-119):
 * n = kfac * 2^p viewed (kfac, n/kfac), Walsh-Hadamard over the last dim, then hadK (kfac x kfac)
 * from the left - hadK^T when `transpose` is non-zero (matmul_hadUt_cuda, :118-119).  The caller
 * folds n^-1/2 and the /32, x32 factors of BitshiftLinear.forward (lib/codebook/bitshift.py:428-441,
 * 465-471) into `scale` and sign_out.  Replaces the hadamard::hadamard op (third-party
 * fast_hadamard_transform) plus the element-wise kernels around it.
 *   in / out      : (rows, n), dtype QTIP_F16 or QTIP_F32 each; may alias only if identical.
 *   sign_in       : NULL or n_signs values of dtype sign_in_dtype; sign_out: NULL or n_signs fp32.
 *   n_signs       : n, or a multiple t*n - then row r uses signs [(r % t)*n, (r % t + 1)*n)
 *                   (the per-chunk transforms of the tensor-parallel layouts, :437-441, :465-469).
 *   hadk_bits     : NULL when kfac == 1, else kfac rows of ceil(kfac/32) uint32 words, bit j of
 *                   word w of row i set when hadK[i][32w+j] == +1.
 *   kfac in {1,12,20,28,36,52,60,108,116,124,140,156,172}; n/kfac a power of two, 2 <= n/kfac,
 *   n <= 65536. */
int qtip_rht(void *out, int out_dtype, const void *in, int in_dtype, long rows, int n, const void *sign_in,
             int sign_in_dtype, const float *sign_out, long n_signs, const uint32_t *hadk_bits, int kfac,
             int transpose, float scale, void *stream);

/* qtip_rht with the element-wise neighbours of a QTIP linear in a decoder layer fused into the load:
 *   v = in (+ residual)            the sum rounded to fp16, written to residual_out when given
 *   v = RMSNorm(v) * norm_weight   LlamaRMSNorm, model/llama.py:129-136 (fp32 statistics, fp16 product)
 *   v = silu(gate) * v             the SwiGLU product of LlamaMLP.forward, model/llama.py:399-400
 * then sign_in, Hadamard, scale, sign_out as qtip_rht.  residual, residual_out, norm_weight and gate
 * are fp16 and optional (NULL); residual and gate use the row layout of `in`.
 * in_row_stride: elements between consecutive input rows, 0 = all rows read the same input row
 * (one launch transforms one activation with several sign vectors - q/k/v or gate/up - with
 * n_signs = rows*n).  out and residual_out must not alias any input. */
int qtip_rht_fused(void *out, int out_dtype, const void *in, int in_dtype, long rows, long in_row_stride, int n,
                   const void *residual, void *residual_out, const void *norm_weight, float eps, const void *gate,
                   const void *sign_in, int sign_in_dtype, const float *sign_out, long n_signs,
                   const uint32_t *hadk_bits, int kfac, int transpose, float scale, void *stream);

/* Everything between the gate/up matvecs and the down matvec of a Llama MLP for one token, in one launch
 * (one cluster of 16 CTAs, or 8 where 16 cannot be co-scheduled; the +-1 Hadamard factor runs on the tensor cores):
 *   out (n) fp16 = fp16( H^T( sign_down * silu(g) * u ) * scale_in ),
 *   g = fp16( sign_gate * H(y_gate) * scale_out ),  u = fp16( sign_up * H(y_up) * scale_out ),
 * i.e. the output side of gate_proj and up_proj (lib/codebook/bitshift.py:465-471), the SwiGLU product
 * (model/llama.py:399-400) and the input side of down_proj (bitshift.py:428-441).  y_* are the raw fp32 matvec
 * results, sign_gate / sign_up fp32, sign_down fp16 with entries +-1, all (n) and 16-byte aligned;
 * n = kfac * len with kfac > 1 from the table of qtip_rht and len in {32, 64, 128}
 * (qtip_mlp_mid_supported tells, 1 = yes).  `table` (qtip_mlp_mid_table_bytes() bytes of device memory,
 * 16-byte aligned) is derived from the packed factor matrix once, by qtip_mlp_mid_prepare on the same device,
 * and can be kept for the life of the model.  The first call on a device queries the cluster occupancy and
 * must happen outside stream capture. */
int qtip_mlp_mid_supported(int n, int kfac);
size_t qtip_mlp_mid_table_bytes(void);
int qtip_mlp_mid_prepare(void *table, const uint32_t *hadk_bits, int n, int kfac, void *stream);
int qtip_mlp_mid(void *out, const float *y_gate, const float *y_up, const float *sign_gate, const float *sign_up,
                 const void *sign_down, const void *table, int n, int kfac, float scale_out, float scale_in,
                 void *stream);

/* --------------------------------------------------------------------------------------------
 * Decode-loop support (batch 1): the per-token attention pieces between the QTIP linears, so that a
 * decode step is one CUDA graph of this library's launches.  fp16 tensors; `pos` points to the
 * token position in device memory (read at run time, so a captured graph can be replayed).
 * ------------------------------------------------------------------------------------------ */

/* Capacity guards of the decode-loop entry points below.  The token index and the position live in device memory
 * (so that one captured graph serves every step) and the host cannot check them per launch; every entry point
 * that uses one as an address therefore takes the capacity of the buffer it indexes (vocab, max_positions,
 * max_tokens) and an optional `status` word (one zero-initialised uint32 in device memory, may be NULL).  A kernel
 * that finds the index outside its buffer touches nothing, ORs a bit into *status (1: position outside the KV
 * cache, 2: token outside the embedding table, 4: token log full) and returns; the context stays usable. */

/* Embedding lookup for one token: res (hidden) fp16 = embed[*token] (embed is (vocab, hidden) fp16, token a
 * 64-bit index in device memory); delta (hidden) fp16 = 0.  Replaces embed_tokens of LlamaModel.forward
 * (model/llama.py) for the decode loop.  hidden a multiple of 8, pointers 16-byte aligned. */
int qtip_embed_token(void *res, void *delta, const void *embed, const long long *token, int hidden, int vocab,
                     unsigned *status, void *stream);

/* Final RMSNorm and the (unquantized, fp16) lm_head for one token:
 * logits (vocab) fp32 = weight (vocab, hidden) @ fp16( norm_weight * fp16( RMSNorm(res + delta) ) ), the tail of
 * LlamaForCausalLM.forward (model/llama.py).  An HBM-bound matrix-vector product; pointers 16-byte aligned. */
int qtip_lm_head(float *logits, const void *res, const void *delta, const void *norm_weight, const void *weight,
                 int hidden, int vocab, float eps, void *stream);

/* Temperature / top-k sampling without a host synchronisation (eval/interactive_gen.py:15-40: logits_to_probs +
 * multinomial_sample_one_no_sync): the top_k (<= 16) largest logits, softmax(top / temperature), one draw from a
 * counter-based generator keyed by (seed, *pos).  Writes the token to *token and out_tokens[*pos + 1] (out_tokens
 * holds max_tokens entries) and advances *pos (32-bit, device memory).  The draw is reproducible for a given seed
 * but is not torch's stream. */
int qtip_sample_top_k(long long *token, long long *out_tokens, int *pos, const float *logits, int vocab,
                      float temperature, int top_k, unsigned long long seed, int max_tokens, unsigned *status,
                      void *stream);

/* Rotary embedding of q (n_heads, head_dim; in place) and k (n_kv_heads, head_dim), and append of the
 * rotated k and of v to the caches at row *pos (caches are (max_positions, n_kv_heads*head_dim)).
 * Replaces apply_rotary_pos_emb + StaticCache.update (model/llama.py:797-898,
 * model/cache_utils.py:1147-1193) for a single new token. */
int qtip_rope_kv_append(void *q, const void *k, const void *v, void *cache_k, void *cache_v, const int *pos,
                        int n_heads, int n_kv_heads, int head_dim, float theta, int max_positions, unsigned *status,
                        void *stream);

/* qtip_rope_kv_append with the output side of the q / k / v linears in front of it: y_q / y_k / y_v are the raw
 * fp32 results of the three matvecs (e.g. the y of a qtip_linear_fused launch without fused output side); the
 * kernel computes fp16( sign * H(y) * scale ) - the tail of BitshiftLinear.forward, lib/codebook/bitshift.py:465-471
 * - then rotates q (written to q_out) and k and appends k, v to the caches (model/llama.py:797-898,
 * model/cache_utils.py:1147-1193).  n_heads*head_dim and n_kv_heads*head_dim in {1024, 2048, 4096, 8192, 16384};
 * all pointers 16-byte aligned; sign_* (fp32) may be NULL. */
int qtip_rope_kv_append_fused(void *q_out, const float *y_q, const float *y_k, const float *y_v, const float *sign_q,
                              const float *sign_k, const float *sign_v, float scale_q, float scale_kv, void *cache_k,
                              void *cache_v, const int *pos, int n_heads, int n_kv_heads, int head_dim, float theta,
                              int max_positions, unsigned *status, void *stream);

/* qtip_rope_kv_append_fused and qtip_attn_decode in one launch: from the raw fp32 results of the q / k / v matvecs
 * to the attention output (n_heads, head_dim) fp16 for one new token at row *pos, appending the rotated k and v
 * to the caches on the way.  head_dim 128; n_heads and n_kv_heads powers of two (the Walsh-Hadamard transform
 * over the width factors into one over heads and one inside a head).  Caches 16-byte aligned. */
int qtip_attn_decode_fused(void *out, const float *y_q, const float *y_k, const float *y_v, const float *sign_q,
                           const float *sign_k, const float *sign_v, float scale_q, float scale_kv, void *cache_k,
                           void *cache_v, const int *pos, int n_heads, int n_kv_heads, int head_dim, float theta,
                           int max_positions, unsigned *status, void *stream);

/* Single-query attention over cache rows 0..*pos: out (n_heads, head_dim).  head_dim must be 128;
 * q and the caches 16-byte aligned.
 * Replaces the scaled_dot_product_attention call of LlamaSdpaAttention.forward (model/llama.py:884-891)
 * for a single new token. */
int qtip_attn_decode(void *out, const void *q, const void *cache_k, const void *cache_v, const int *pos, int n_heads,
                     int n_kv_heads, int head_dim, int max_positions, unsigned *status, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* QTIP_B200_H */
