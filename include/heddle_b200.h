/*
 * heddle_b200 — C ABI of the B200-native attention / fused-GEMM hot path.
 *
 * The reference (DragonOV12341/Heddle) has no C boundary of its own: its device
 * kernels are generated at run time by TileLang and reached through Python
 * callables.  Each entry point below names the reference callable it replaces
 * (path inside the reference project : line).
 *
 * Conventions
 *   - every pointer named q/k/v/o/lse/a/w/out/... is a DEVICE pointer owned by the
 *     caller; the library never allocates or frees caller memory;
 *   - all calls are stream-ordered and asynchronous: they enqueue work on `stream`
 *     (a cudaStream_t passed as void*, NULL = legacy default stream) and return;
 *   - the return value is an hb_status; on failure hb_last_error() returns a
 *     thread-local, human readable message.  No exception, abort() or device trap
 *     ever crosses this boundary;
 *   - strides are in ELEMENTS of the tensor's dtype, the innermost (head_dim /
 *     K / N) dimension is contiguous.
 */
#ifndef HEDDLE_B200_H_
#define HEDDLE_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HB_VERSION 100

typedef enum hb_status {
  HB_OK = 0,
  HB_ERR_BAD_ARG = 1,     /* null pointer, negative size, inconsistent shape      */
  HB_ERR_UNSUPPORTED = 2, /* dtype / head_dim / epilogue not built for sm_100a     */
  HB_ERR_ALIGN = 3,       /* pointer or stride violates the 16-byte TMA rule       */
  HB_ERR_CUDA = 4,        /* a CUDA runtime / driver call failed                   */
  HB_ERR_TIMEOUT = 5      /* a device-side bounded wait gave up (see hb_status_word) */
} hb_status;

typedef enum hb_dtype {
  HB_BF16 = 0,
  HB_FP16 = 1,
  HB_FP8_E4M3 = 2
} hb_dtype;

/* hb_query() selectors */
enum {
  HB_QUERY_SM_COUNT = 0,
  HB_QUERY_SMEM_OPTIN = 1,
  HB_QUERY_CC = 2, /* major*10+minor of the current device */
  HB_QUERY_FA_SMEM = 3,
  HB_QUERY_GEMM_SMEM = 4
};

/*
 * FlashAttention forward:  O = softmax(Q K^T * softmax_scale + mask) V,
 * optionally LSE = log(sum(exp(scaled masked scores))) per query row (natural log).
 *
 * Replaces the kernels produced by
 *   Heddle/heddle/tileop/flash_attention.py:20-143   (flashattn)
 *   Heddle/heddle/tileop/flash_attention.py:158-300  (flashattn_lse)
 *   Heddle/heddle/frontend/backend.py:28-85, 92-156  (_build_fa_kernel[_with_lse])
 * and is what _tilelang_sdpa_direct (backend.py:205-224) and
 * TileLangFlashAttnFunc.forward (patterns.py:146-187) launch.
 *
 * Layout: q is [B, Hq, Sq, D], k/v are [B, Hkv, Skv, D], o is [B, Hq, Sq, D], each
 * addressed through explicit batch/head/seq strides so that both BHSD and BSHD
 * storage work without a transposed copy.  Query head h reads KV head
 * h / (Hq / Hkv).  Causal masking follows the reference's past_len rule
 * (flash_attention.py:27,44): query i may see key j iff j <= i + (Skv - Sq).
 *
 * FP8: q/k/v are e4m3 with per-tensor dequantisation scales q_scale/k_scale/v_scale;
 * P is requantised to e4m3 (scale p_scale, 0 = library default) before the PV MMA;
 * o is bf16.
 */
typedef struct hb_fa_args {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  float* lse; /* optional [B, Hq, Sq] fp32 contiguous; NULL = not written */
  int32_t B, Hq, Hkv, Sq, Skv, D;
  int64_t q_stride_b, q_stride_h, q_stride_s;
  int64_t k_stride_b, k_stride_h, k_stride_s;
  int64_t v_stride_b, v_stride_h, v_stride_s;
  int64_t o_stride_b, o_stride_h, o_stride_s;
  int32_t causal;
  float softmax_scale; /* <= 0 selects D^-1/2 */
  int32_t dtype;       /* hb_dtype of q/k/v (o: same dtype; bf16 for FP8) */
  float q_scale, k_scale, v_scale, p_scale, o_scale; /* FP8 only; 0 = 1.0 */
  void* stream;
} hb_fa_args;

int hb_fa_fwd(const hb_fa_args* args);

/*
 * hb_fa_fwd for callers that cannot allocate device memory.  No counterpart in the
 * reference (its kernels and their buffers are created by TileLang's JIT at run time).
 *
 * Who needs it: hb_fa_fwd obtains the device-side status word its kernel reports into
 * with cudaMalloc on the first call per device.  A host process that runs under a fixed
 * memory budget, forbids allocation once it has started serving, or calls from inside a
 * region where cudaMalloc is not permitted cannot make that first call.  This entry
 * point computes exactly the same result with the same kernel, but keeps that scratch
 * in a static device array compiled into the library (256 bytes; every GPU that loads
 * the library holds it until the process exits) and calls no cudaMalloc, cudaFree or
 * other allocating routine.  The caller still passes q, k, v, o and lse.
 *
 * Set-up: the first call on each device resolves the array's device address
 * (cudaGetSymbolAddress, with that device current).  Make that first call outside any
 * stream capture.  Limits: bf16 / fp16 only; at most 2^31-1 query blocks of 256 rows
 * (B * Hq * ceil(ceil(Sq/256)/2)) per call, larger problems are rejected with
 * HB_ERR_UNSUPPORTED.  All calls on a device share the one array, which keeps its contents
 * from call to call: the status word in it starts at zero when the library is loaded, a
 * kernel only moves it from zero to a failure code (the first failure wins) and only
 * hb_status_word_noalloc clears it.  Calls whose kernels overlap on the GPU (different
 * streams) therefore race on that word: a failure cannot be attributed to one of them —
 * issue them on one stream or order them with events if that matters.
 */
int hb_fa_fwd_noalloc(const hb_fa_args* args);

/*
 * Status word of the hb_fa_fwd_noalloc path on the current device (hb_status_word reads a
 * different, allocated word and allocates on first use, so a host that may not allocate
 * cannot call it).  Copies the word out of the static array on `stream`, waits for that
 * stream, and if it is non-zero clears it and returns HB_ERR_TIMEOUT with hb_last_error()
 * naming the kernel role whose wait gave up.  Allocates nothing.  No counterpart in the
 * reference.
 */
int hb_status_word_noalloc(uint32_t* out, void* stream);

/*
 * H2O score:  score[b,h,k] = sum_q exp(scaled masked score[q,k] - LSE[q])
 * Replaces Heddle/heddle/tileop/h2o_attention.py:27-136 (h2o_score), called from
 * backend.py:162-202 (_tilelang_h2o_attention).  lse is the natural-log LSE that
 * hb_fa_fwd writes; score is [B, Hq, Skv] fp32 and is overwritten.
 */
typedef struct hb_h2o_args {
  const void* q;
  const void* k;
  const float* lse;
  float* score;
  int32_t B, Hq, Hkv, Sq, Skv, D;
  int64_t q_stride_b, q_stride_h, q_stride_s;
  int64_t k_stride_b, k_stride_h, k_stride_s;
  int32_t causal;
  float softmax_scale;
  int32_t dtype;
  void* stream;
} hb_h2o_args;

int hb_h2o_score(const hb_h2o_args* args);

/*
 * GEMM + fused epilogue:  out[M, N_out] = epilogue(a[M, K] . w[N, K]^T)
 *
 * Replaces the kernels emitted by
 *   Heddle/heddle/frontend/codegen.py:980-1244 (auto_gemm_* : GEMM + unary epilogue,
 *     dual-GEMM / SwiGLU with the activation left in PyTorch at :1155-1160)
 *   Heddle/heddle/frontend/backend.py:227-252  (_build_gemm_kernel)
 * `w` is in nn.Linear layout [N, K] (K contiguous) — no transposed weight copy is
 * needed (the reference caches one, codegen.py:1124-1131).
 *
 * Epilogues (fp32 on the accumulator, then cast; formulas codegen.py:1232-1244):
 *   NONE, SILU, RELU, GELU_TANH, SIGMOID, TANH           out is [M, N]
 *   SWIGLU      w = [Wg ; Wu] stacked as [2*N_out, K];    out[M, N_out] = silu(g) * u
 *   ROWSCALE    out = row_scale[m] * acc   (RMSNorm with gamma folded into w)
 *   ROPE        rotate-half RoPE on head_dim-wide column groups,
 *               cos/sin tables [rope_seq, head_dim/2] fp32, position = m % rope_seq
 * Optional operands, any epilogue: row_scale (fp32 [M]) multiplies the accumulator
 * first; bias ([N], dtype) is added next, before the activation / gate / rotation;
 * residual ([M, N_out], dtype) is added last.
 * Constraints: K, N_out, lda, ldw, ldo, ldr multiples of 8 elements; 16-byte aligned
 * pointers; ROPE needs head_dim in {64, 128, 256} dividing N and rope_cols.
 */
typedef enum hb_epilogue {
  HB_EPI_NONE = 0,
  HB_EPI_SILU = 1,
  HB_EPI_RELU = 2,
  HB_EPI_GELU_TANH = 3,
  HB_EPI_SIGMOID = 4,
  HB_EPI_TANH = 5,
  HB_EPI_SWIGLU = 6,
  HB_EPI_ROPE = 7
} hb_epilogue;

typedef enum hb_w_layout { HB_W_NK = 0, HB_W_KN = 1 } hb_w_layout;
/* Which kernel runs the product.  AUTO: CTA pairs (two CTAs share a 256 x 256 tile through
 * tcgen05.mma.cta_group::2) when M > 128, else the single-CTA kernel (128 x 256 tiles).  SINGLE and
 * PAIR force one of them; the results are identical (same accumulation order per element). */
typedef enum hb_gemm_schedule { HB_GEMM_AUTO = 0, HB_GEMM_SINGLE = 1, HB_GEMM_PAIR = 2 } hb_gemm_schedule;

typedef struct hb_gemm_args {
  const void* a; /* [M, K], row stride lda */
  const void* w; /* [N, K], row stride ldw */
  void* out;     /* [M, N_out], row stride ldo */
  int32_t M, N, K;
  int64_t lda, ldw, ldo;
  int32_t dtype; /* HB_BF16 or HB_FP16 */
  int32_t epilogue;
  const float* row_scale;  /* optional fp32 [M] */
  const void* bias;        /* optional [N] */
  const void* residual;    /* optional [M, N_out], row stride ldr */
  int64_t ldr;
  const float* rope_cos;   /* ROPE: [rope_seq, head_dim/2] */
  const float* rope_sin;
  int32_t rope_seq, head_dim;
  int32_t rope_cols;       /* ROPE: columns [0, rope_cols) are rotated, the rest copied */
  void* stream;
  /* Batched products and the [K, N] operand layout (zero-initialised fields = one product, w [N, K]).
   * batch > 1: out[b] = epilogue(a[b] . w[b]) for b < batch, replacing the reference's batched kernel
   * (Heddle/heddle/frontend/backend.py:491-536, _build_bmm_kernel / _tilelang_bmm_wrapper); the batch
   * strides are in elements, 0 = densely packed; row_scale is [batch * M], bias [N] is shared.
   * w_layout HB_W_KN: w is [K, N] row-major with row stride ldw, as torch.mm / torch.bmm and the
   * reference's plain GEMM take it (backend.py:227-272, _build_gemm_kernel / _tilelang_gemm_wrapper);
   * plain epilogues only. */
  int32_t batch;
  int32_t w_layout;
  int64_t a_batch_stride, w_batch_stride, o_batch_stride, r_batch_stride;
  int32_t schedule; /* hb_gemm_schedule */
} hb_gemm_args;

int hb_gemm_epilogue(const hb_gemm_args* args);

/*
 * Row statistic for RMSNorm fused with the residual add:
 *   y = x (+ residual);  if y_out: y_out = y;  rstd[m] = rsqrt(mean(y^2) + eps)
 * The reference only analyses this fusion (Heddle/heddle/frontend/elementwise_fusion.py:73-80)
 * and runs RMSNorm in eager PyTorch; here it feeds the ROWSCALE GEMM epilogue.
 */
int hb_rms_rowstat(const void* x, const void* residual, void* y_out, float* rstd,
                   int32_t M, int32_t N, int64_t ldx, float eps, int32_t dtype, void* stream);

/*
 * One-off weight preparation for hb_gemm_epilogue: stacks up to four nn.Linear weights [rows_i, K]
 * along the row axis (Q|K|V for one projection GEMM, gate|up for SWIGLU) and, optionally, scales
 * column k by gamma[k] (the RMSNorm weight folded into the GEMM):
 *   out[off_i + r, k] = round(float(src_i[r, k]) * float(gamma[k]))
 * Replaces the host-side weight handling of the reference's GEMM wrapper, which transposes the
 * weight to [K, N] and caches it by data_ptr (Heddle/heddle/frontend/codegen.py:1106-1131) and
 * concatenates gate and up weights for the dual GEMM (:1146-1152); here weights keep the [N, K]
 * layout, so preparation is a single streaming pass.
 */
typedef struct hb_prepare_args {
  const void* src[4];   /* [rows[i], K] each, row stride ld_src[i] elements */
  int32_t rows[4];
  int64_t ld_src[4];
  int32_t n_src;        /* 1..4 */
  int32_t K;            /* multiple of 8 */
  const void* gamma;    /* [K] in the weights' dtype, or NULL */
  void* out;            /* [sum rows, K], row stride ld_out elements */
  int64_t ld_out;
  int32_t dtype;        /* HB_BF16 or HB_FP16 */
  void* stream;
} hb_prepare_args;

int hb_prepare_weight(const hb_prepare_args* args);

/*
 * Attention backward, split into three kernels with exclusive outputs (no atomic adds).  The
 * reference sketches this interface and leaves the kernels unwritten:
 *   Heddle/heddle/frontend/bwd_separator.py:366-455 (create_separated_bwd_function:
 *     delta = preprocess(O, dO);  dK, dV = dkdv(Q, K, V, O, dO, LSE, delta);  dQ = dq(...))
 *   delta[b,h,q] = sum_d O * dO
 *   P = exp(scale * Q K^T + mask - LSE),  dP = dO V^T,  dS = P o (dP - delta)
 *   dV = P^T dO,  dK = scale * dS^T Q,  dQ = scale * dS K
 * q, d_o, o are [B, Hq, Sq, D] and k, v [B, Hkv, Skv, D] by element strides (head_dim contiguous,
 * 16-byte aligned rows), lse is the natural-log LSE that hb_fa_fwd writes, lse and delta are
 * [B, Hq, Sq] fp32 contiguous.  Outputs are contiguous: dq [B, Hq, Sq, D], dk and dv
 * [B, Hkv, Skv, D] (with grouped queries a kv head's gradient is the sum over its query heads,
 * formed inside the one CTA that owns the key tile).  bf16 / fp16, D in {64, 128}, causal mask aligned
 * to the end of the keys (key <= query + Skv - Sq) as in hb_fa_fwd.
 *   hb_fa_bwd_preprocess reads o, d_o            and writes delta
 *   hb_fa_bwd_dkdv       reads q, k, v, d_o, lse, delta and writes dk, dv
 *   hb_fa_bwd_dq         reads q, k, v, d_o, lse, delta and writes dq
 */
typedef struct hb_fa_bwd_args {
  const void* q;
  const void* k;
  const void* v;
  const void* o;
  const void* d_o;
  const float* lse;
  float* delta;
  void* dq;
  void* dk;
  void* dv;
  int32_t B, Hq, Hkv, Sq, Skv, D;
  int64_t q_stride_b, q_stride_h, q_stride_s;
  int64_t k_stride_b, k_stride_h, k_stride_s;
  int64_t v_stride_b, v_stride_h, v_stride_s;
  int64_t o_stride_b, o_stride_h, o_stride_s;
  int64_t do_stride_b, do_stride_h, do_stride_s;
  int32_t causal;
  float softmax_scale; /* <= 0 selects D^-1/2 */
  int32_t dtype;       /* HB_BF16 or HB_FP16 */
  void* stream;
} hb_fa_bwd_args;

int hb_fa_bwd_preprocess(const hb_fa_bwd_args* args);
int hb_fa_bwd_dkdv(const hb_fa_bwd_args* args);
int hb_fa_bwd_dq(const hb_fa_bwd_args* args);

/*
 * y = softmax(scale * x) over the last axis of a [rows, cols] matrix (bf16 / fp16, fp32 math,
 * cols a multiple of 8 and at most 16384).  The native counterpart of the reference's generated
 * softmax-like reduction kernel (Heddle/heddle/frontend/codegen.py:1246-1400: one 32-thread CTA
 * per row, exp2 with log2(e), block-wise online merge); here a row is read and written once.
 */
int hb_row_softmax(const void* x, void* y, int64_t rows, int32_t cols, int64_t ld_x, int64_t ld_y,
                   float scale, int32_t dtype, void* stream);

/*
 * Pointwise chains and row reductions over a [rows, cols] matrix (bf16 / fp16 tensors, fp32 math),
 * driven by an op-code program.  The native counterpart of the kernels the reference generates as
 * source text and compiles at run time for its elementwise partitions
 * (Heddle/heddle/frontend/codegen.py:1457-1498, op table _map_op :1577-1609) and for its
 * softmax-like / sum / mean / max row reductions (:1246-1455: one pass per reduction that recomputes
 * the expression up to it, reduction results kept in fp32, then an output pass).
 *
 * The program runs once per group of 8 consecutive columns of a row on an accumulator machine:
 * `acc = op(acc, operand)`.  Operands: a full input tensor [rows, cols] (HB_SRC_INPUT), a [cols]
 * vector of the same dtype broadcast over rows (HB_SRC_ROWVEC), an fp32 [rows] vector broadcast
 * over columns (HB_SRC_ROWSCALAR), an immediate (HB_SRC_IMM), a saved value (HB_SRC_TMP, written
 * by HB_EW_STORE_TMP) or the result of an earlier row reduction (HB_SRC_REDUCED).  Unary ops use
 * no operand.  HB_EW_REDUCE_{SUM,MAX,MEAN} reduce acc over the whole row into slot `index` and leave
 * acc unchanged; a program with R of them is run R + 1 times (prefix passes, then the whole
 * program), so instructions in front of a reduction must not depend on that reduction.
 * HB_EW_STORE_OUT writes acc, rounded to the dtype, to output `index`; HB_EW_ROUND rounds acc to
 * the dtype and back (an intermediate 16-bit tensor of the eager graph).
 * Constraints: cols a multiple of 8; pointers 16-byte aligned; row strides multiples of 8.
 */
typedef enum hb_ew_op {
  HB_EW_LOAD = 0, /* acc = operand */
  HB_EW_ADD = 1,
  HB_EW_SUB = 2,  /* acc - operand */
  HB_EW_RSUB = 3, /* operand - acc */
  HB_EW_MUL = 4,
  HB_EW_DIV = 5,  /* acc / operand */
  HB_EW_RDIV = 6, /* operand / acc */
  HB_EW_MAX = 7,
  HB_EW_MIN = 8,
  HB_EW_POW = 9,  /* acc ** operand */
  HB_EW_NEG = 16,
  HB_EW_ABS = 17,
  HB_EW_EXP = 18,
  HB_EW_LOG = 19,
  HB_EW_LOG2 = 20,
  HB_EW_SQRT = 21,
  HB_EW_RSQRT = 22,
  HB_EW_RECIP = 23,
  HB_EW_SIGMOID = 24,   /* 1 / (1 + exp(-x)) */
  HB_EW_SILU = 25,      /* x * sigmoid(x) */
  HB_EW_RELU = 26,
  HB_EW_GELU_TANH = 27, /* 0.5 x (1 + tanh(0.7978845608 (x + 0.044715 x^3))) */
  HB_EW_GELU_ERF = 28,
  HB_EW_TANH = 29,
  HB_EW_ROUND = 30,
  HB_EW_STORE_TMP = 40,
  HB_EW_REDUCE_SUM = 48,
  HB_EW_REDUCE_MAX = 49,
  HB_EW_REDUCE_MEAN = 50,
  HB_EW_STORE_OUT = 56
} hb_ew_op;

typedef enum hb_ew_src {
  HB_SRC_NONE = 0,
  HB_SRC_INPUT = 1,
  HB_SRC_IMM = 2,
  HB_SRC_TMP = 3,
  HB_SRC_ROWVEC = 4,
  HB_SRC_ROWSCALAR = 5,
  HB_SRC_REDUCED = 6
} hb_ew_src;

#define HB_EW_MAX_INST 48
#define HB_EW_MAX_INPUTS 6
#define HB_EW_MAX_ROWVEC 4
#define HB_EW_MAX_ROWSCALAR 4
#define HB_EW_MAX_OUTPUTS 2
#define HB_EW_MAX_TMP 4
#define HB_EW_MAX_RED 4

typedef struct hb_ew_inst {
  int32_t op;    /* hb_ew_op */
  int32_t src;   /* hb_ew_src */
  int32_t index; /* operand / temporary / reduction slot / output index */
  float imm;
} hb_ew_inst;

typedef struct hb_rowwise_args {
  const void* inputs[HB_EW_MAX_INPUTS];
  int64_t ld_in[HB_EW_MAX_INPUTS];
  const void* rowvec[HB_EW_MAX_ROWVEC];
  const float* rowscalar[HB_EW_MAX_ROWSCALAR];
  void* outputs[HB_EW_MAX_OUTPUTS];
  int64_t ld_out[HB_EW_MAX_OUTPUTS];
  int32_t n_inputs, n_rowvec, n_rowscalar, n_outputs;
  int64_t rows;
  int32_t cols;
  int32_t dtype; /* HB_BF16 or HB_FP16 */
  int32_t n_inst;
  hb_ew_inst program[HB_EW_MAX_INST];
  void* stream;
  int32_t mode; /* hb_rowwise_mode */
} hb_rowwise_args;

/* How the program is executed.  AUTO: a kernel specialised for the program, compiled at run time
 * with NVRTC on its first use and cached (the reference compiles its generated kernels the same
 * way); when libnvrtc cannot be loaded, the interpreter kernel.  INTERPRET: always the interpreter
 * (nothing is compiled).  COMPILED: the specialised kernel or HB_ERR_UNSUPPORTED.  All three give
 * the same results.  HEDDLE_B200_ROWWISE_JIT=0 in the environment turns the compiler off;
 * HEDDLE_B200_NVRTC names the library file to load.  The first call with a new program compiles and
 * loads a module (0.1-0.7 s) and must not be made inside a stream capture; later calls only launch. */
typedef enum hb_rowwise_mode { HB_ROWWISE_AUTO = 0, HB_ROWWISE_INTERPRET = 1, HB_ROWWISE_COMPILED = 2 } hb_rowwise_mode;

int hb_rowwise_program(const hb_rowwise_args* args);
/* 1 when the run-time compiler can be loaded in this process, else 0.  Needs no device. */
int hb_rowwise_compiler_available(void);
/* Test hook: checks `args` like hb_rowwise_program, generates the specialised kernel's source and
 * compiles it for sm_100a without loading or launching it (no device is needed and no pointer in
 * `args` is dereferenced).  `source` (may be NULL) receives the generated text. */
int hb_debug_rowwise_compile(const hb_rowwise_args* args, char* source, int64_t capacity);

/* Device-side status word of the current device (0 = no bounded wait ever gave up);
 * reading it synchronises the device.  *out always receives the word; the return value is
 * HB_OK when it is zero and HB_ERR_TIMEOUT otherwise (hb_last_error() then names the kernel
 * and the role whose wait ran out; the outputs of that launch are incomplete). */
int hb_status_word(uint32_t* out);

/* Library / device information. */
int hb_version(void);
int hb_query(int what);
const char* hb_last_error(void);
/* Releases the per-device caches (status word, driver entry points). */
int hb_shutdown(void);

/*
 * Diagnostics: one tcgen05 MMA tile through the library's own descriptor helpers.
 *   mode 0: out[128,128] fp32 = A[128,K] . B[128,K]^T          (both K-major in smem)
 *   mode 1: out[128,N]  fp32 = P[128,128] . V[128,N]           (P from TMEM, V MN-major)
 * a, b are dense row-major device arrays of `dtype`; K, N in {64, 128}.
 * No reference counterpart; used by the test-suite to pin the operand layouts.
 */
int hb_debug_umma(int mode, const void* a, const void* b, float* out, int32_t kn, int32_t dtype,
                  void* stream);

/*
 * hb_fa_fwd with the K/V ring of the kernel built `stages` deep (2, 3 or 5; bf16, head_dim 128).
 * The depth only changes when tiles are loaded, so O and LSE must be bit-identical to hb_fa_fwd's
 * (which uses 5): a mismatch means a race in the barrier protocol.  The reference plans the same
 * stand-in for a race detector ("bitwise comparison between a 1-stage and an N-stage pipeline
 * build"); it has no counterpart there.
 */
int hb_debug_fa_fwd_stages(const hb_fa_args* args, int32_t stages);

/*
 * Failure-detection probe: one small CTA waits on a barrier that is never signalled, with a
 * limit of limit_us microseconds (1..100000).  The wait gives up, raises the CTA's abort flag and
 * records kStatusWaitTimeout | role (0x170) in a scratch status word, a second warp leaves its own
 * wait on seeing the flag, the kernel ends normally.  status_out receives the code; result4 =
 * {warp 0 returned ok?, its wait in ns, warp 1 returned ok?, its wait in ns}.  Nothing faults or
 * hangs; the device status word read by hb_status_word is not touched.
 */
int hb_debug_wait_timeout(uint32_t limit_us, uint32_t* status_out, uint64_t* result4);

#ifdef __cplusplus
}
#endif
#endif /* HEDDLE_B200_H_ */
