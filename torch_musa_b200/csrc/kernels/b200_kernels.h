/* C ABI of libb200_kernels.so: every hand-written sm_100a kernel of the backend.
 *
 * Conventions: pointers are device pointers unless named host_*; every function
 * enqueues work on `stream` and returns a cudaError_t value as int (0 = ok);
 * nothing here allocates device memory unless its comment says so; `dtype` is one
 * of the B200_* codes below.  Callable from C, ctypes and the C++ operator layer.
 */
#pragma once

#include <cuda_runtime_api.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_API __attribute__((visibility("default")))

enum { B200_F32 = 0, B200_BF16 = 1, B200_F16 = 2, B200_F64 = 3, B200_I32 = 4, B200_I64 = 5, B200_U8 = 6,
       B200_BOOL = 7, B200_I8 = 8, B200_I16 = 9, B200_FP8_E4M3 = 10, B200_FP8_E5M2 = 11 };

/* number of kernels launched by this library since load / last reset (host counter) */
B200_API int64_t b200_launch_count(void);
B200_API void b200_reset_launch_count(void);
B200_API const char* b200_kernels_arch(void);

/* ---------------------------------------------------------------- elementwise */
enum {
  B200_OP_ADD = 0, B200_OP_SUB, B200_OP_MUL, B200_OP_DIV, B200_OP_MAXIMUM, B200_OP_MINIMUM,
  B200_OP_RELU = 32, B200_OP_GELU_ERF, B200_OP_GELU_TANH, B200_OP_SILU, B200_OP_SIGMOID, B200_OP_TANH,
  B200_OP_EXP, B200_OP_LOG, B200_OP_NEG, B200_OP_ABS, B200_OP_SQRT, B200_OP_RSQRT, B200_OP_RECIPROCAL,
  B200_OP_SQUARE, B200_OP_COPY,
  /* backward forms: out = f(grad, x) as a binary op */
  B200_OP_RELU_BWD = 64, B200_OP_GELU_ERF_BWD, B200_OP_GELU_TANH_BWD, B200_OP_SILU_BWD, B200_OP_SIGMOID_BWD,
  B200_OP_TANH_BWD
};
/* out[i] = op(a[i], alpha*b[i]) (alpha only for ADD/SUB); contiguous, same dtype; b may be NULL with
 * b_scalar used instead. */
B200_API int b200_binary(int op, int dtype, void* out, const void* a, const void* b, double b_scalar, double alpha,
                         int64_t n, cudaStream_t stream);
B200_API int b200_unary(int op, int dtype, void* out, const void* a, int64_t n, cudaStream_t stream);
/* dtype-converting / strided copy. ndim <= 8; strides in elements. */
/* dst = the n_pieces byte ranges (srcs[i], nbytes[i]) one after the other; the ranges may not overlap dst */
B200_API int b200_cat_bytes(void* dst, const void* const* srcs, const int64_t* nbytes, int n_pieces, cudaStream_t stream);
B200_API int b200_cast_copy(void* dst, int dst_dtype, const void* src, int src_dtype, int ndim, const int64_t* sizes,
                            const int64_t* dst_strides, const int64_t* src_strides, cudaStream_t stream);
B200_API int b200_fill(void* out, int dtype, double value, int64_t n, cudaStream_t stream);
/* out = a + alpha * (t1 * t2) / out = a + alpha * (t1 / t2) */
B200_API int b200_addcmul(int dtype, void* out, const void* a, const void* t1, const void* t2, double alpha, int div,
                          int64_t n, cudaStream_t stream);
/* busy-wait for `cycles` SM clock ticks, never longer than max_cycles (bounded) */
B200_API int b200_sleep(int64_t cycles, cudaStream_t stream);

/* ---- general pointwise loops (kernels/ew_generic.cu): broadcast / strided / mixed-dtype operands.
 * out = op(in1[, in2[, in3]]); p0 / p1 are operator parameters (alpha for ADD / SUB / ADDCMUL / ADDCDIV / LERP,
 * the bounds of CLAMP / HARDTANH_BWD, the slope of LEAKY_RELU, the value of FILL / MASKED_FILL, ...). */
enum {
  B200_EW_ADD = 100, B200_EW_SUB, B200_EW_RSUB, B200_EW_MUL, B200_EW_DIV, B200_EW_DIV_FLOOR, B200_EW_DIV_TRUNC,
  B200_EW_REMAINDER, B200_EW_FMOD, B200_EW_POW, B200_EW_ATAN2, B200_EW_MAXIMUM, B200_EW_MINIMUM,
  B200_EW_EQ, B200_EW_NE, B200_EW_LT, B200_EW_LE, B200_EW_GT, B200_EW_GE,
  B200_EW_LOGICAL_AND, B200_EW_LOGICAL_OR, B200_EW_LOGICAL_XOR, B200_EW_BITWISE_AND, B200_EW_BITWISE_OR,
  B200_EW_BITWISE_XOR, B200_EW_LSHIFT, B200_EW_RSHIFT,
  B200_EW_WHERE, B200_EW_MASKED_FILL, B200_EW_CLAMP, B200_EW_CLAMP_TENSOR, B200_EW_ADDCMUL, B200_EW_ADDCDIV,
  B200_EW_LERP, B200_EW_LERP_TENSOR, B200_EW_THRESHOLD_BWD, B200_EW_LEAKY_RELU, B200_EW_LEAKY_RELU_BWD, B200_EW_ELU,
  B200_EW_HARDTANH_BWD, B200_EW_SOFTPLUS, B200_EW_XLOGY, B200_EW_LOG_SIGMOID_BWD,
  B200_EW_NEG = 200, B200_EW_ABS, B200_EW_SIGN, B200_EW_FLOOR, B200_EW_CEIL, B200_EW_ROUND, B200_EW_TRUNC,
  B200_EW_FRAC, B200_EW_EXP, B200_EW_EXP2, B200_EW_EXPM1, B200_EW_LOG, B200_EW_LOG2, B200_EW_LOG10, B200_EW_LOG1P,
  B200_EW_SQRT, B200_EW_RSQRT, B200_EW_RECIPROCAL, B200_EW_SQUARE, B200_EW_SIN, B200_EW_COS, B200_EW_TAN,
  B200_EW_TANH, B200_EW_SIGMOID, B200_EW_ERF, B200_EW_RELU, B200_EW_SILU, B200_EW_GELU_ERF, B200_EW_GELU_TANH,
  B200_EW_ISNAN, B200_EW_ISINF, B200_EW_ISFINITE, B200_EW_LOGICAL_NOT, B200_EW_BITWISE_NOT, B200_EW_COPY, B200_EW_FILL,
  B200_EW_LOG_SIGMOID,
  B200_EW_ASIN, B200_EW_ACOS, B200_EW_ATAN, B200_EW_SINH, B200_EW_COSH, B200_EW_ASINH, B200_EW_ACOSH, B200_EW_ATANH,
  B200_EW_ERFC
};
typedef struct {
  int ndim;                 /* 1..8 coalesced dimensions, innermost first */
  int64_t sizes[8];
  int64_t strides[4][8];    /* elements; [0] output, [1..3] inputs; 0 = broadcast */
  int dtype[4];
  void* ptr[4];
  int n_in;                 /* 0..3 */
  double scalar[3];         /* value of input k when bit k of scalar_mask is set */
  int scalar_mask;
  double p0, p1;
  int float_compute;        /* force floating compute although every input is integral (true division, ...) */
} b200_ew_t;
B200_API int b200_ew(int op, const b200_ew_t* desc, cudaStream_t stream);

/* ---------------------------------------------------------------- reductions */
enum { B200_RED_SUM = 0, B200_RED_MEAN, B200_RED_MAX, B200_RED_MIN, B200_RED_SUMSQ, B200_RED_ABSMAX };
/* reduce the last dimension: in [rows, cols] contiguous -> out [rows]; out dtype = in dtype (accumulation fp32) */
B200_API int b200_reduce_rows(int op, int dtype, void* out, const void* in, int64_t rows, int64_t cols,
                              cudaStream_t stream);
/* reduce everything to one value: out[0] (fp32 if out_f32 else input dtype). `scratch` needs >= 4*1024 bytes. */
B200_API int b200_reduce_all(int op, int dtype, void* out, int out_f32, const void* in, int64_t n, float* scratch,
                             cudaStream_t stream);
/* column reduction: in [rows, cols] -> out [cols] (sum over rows); out fp32 or in dtype */
B200_API int b200_reduce_cols_sum(int dtype, void* out, int out_dtype, const void* in, int64_t rows, int64_t cols,
                                  cudaStream_t stream);

/* ---- general reductions (kernels/reduce_generic.cu): `in` contiguous, viewed as [outer, reduce, inner]; out (and
 * out_index for the arg operators; either may be NULL there) has outer * inner elements.  p0: the factor of MEAN, the
 * correction of VAR / STD.  scratch: device memory for the partial states of split reductions (scratch_bytes; at least
 * b200_reduce_state_bytes() * 65536 keeps every split available; NULL / 0 disables splitting). */
enum { B200_RD_SUM = 0, B200_RD_MEAN, B200_RD_PROD, B200_RD_AMAX, B200_RD_AMIN, B200_RD_ANY, B200_RD_ALL, B200_RD_SUMSQ,
       B200_RD_NORM2, B200_RD_SUMABS, B200_RD_ABSMAX, B200_RD_ARGMAX, B200_RD_ARGMIN, B200_RD_VAR, B200_RD_STD };
typedef struct {
  int op, in_dtype, out_dtype;
  int64_t outer, reduce, inner;
  double p0, p1;
  const void* in;
  void* out;
  int64_t* out_index;
  void* scratch;
  size_t scratch_bytes;
} b200_reduce_t;
B200_API size_t b200_reduce_state_bytes(void);
B200_API int b200_reduce(const b200_reduce_t* desc, cudaStream_t stream);

/* ---- indexing, scan and selection (kernels/index_ops.cu).  Tensors are contiguous views [outer, D, inner];
 * idx_dtype is B200_I64 or B200_I32; `status` (may be NULL) is set to 1 when an index was out of range (the access
 * is clamped, never wild). */
B200_API int b200_index_select(void* out, const void* in, const void* idx, int idx_dtype, int elem_bytes, int64_t outer,
                               int64_t D, int64_t inner, int64_t J, int* status, cudaStream_t stream);
B200_API int b200_gather(void* out, const void* in, const void* idx, int idx_dtype, int elem_bytes, int64_t outer, int64_t D,
                         int64_t inner, int64_t J, int* status, cudaStream_t stream);
/* self[o, idx[j], i] (+)= val[o * val_stride_o + j * val_stride_j + i] */
B200_API int b200_index_put(void* self, const void* val, const void* idx, int idx_dtype, int dtype, int accumulate,
                            int64_t outer, int64_t D, int64_t inner, int64_t J, int64_t val_stride_j, int64_t val_stride_o,
                            int* status, cudaStream_t stream);
/* mode 0: self[o, idx[o,j,i], i] = src[o,j,i]; 1: += ; 2: = value */
B200_API int b200_scatter(void* self, const void* src, double value, const void* idx, int idx_dtype, int dtype, int mode,
                          int64_t outer, int64_t D, int64_t inner, int64_t J, int* status, cudaStream_t stream);
B200_API int b200_tri(void* out, const void* in, int elem_bytes, int64_t batch, int64_t rows, int64_t cols, int64_t diagonal,
                      int upper, cudaStream_t stream);
B200_API int b200_arange(void* out, int dtype, double start, double step, int64_t n, cudaStream_t stream);
B200_API int b200_cumsum_rows(void* out, const void* in, int dtype, int64_t rows, int64_t cols, cudaStream_t stream);
/* k <= 16 best of every row of cols <= 1024 elements, sorted; one thread per row */
B200_API int b200_topk_small(void* vals, int64_t* idxs, const void* in, int dtype, int64_t rows, int cols, int k, int largest,
                             cudaStream_t stream);
/* stable sort of every row; vals_out = original columns.  temp == NULL: only *temp_bytes is written. */
B200_API int b200_sort_rows(void* temp, size_t* temp_bytes, const void* keys_in, void* keys_out, int64_t* vals_out, int dtype,
                            int64_t rows, int64_t cols, int descending, cudaStream_t stream);

/* ---- selection (kernels/select_ops.cu).  Entry points with `temp` follow the two-call convention: temp == NULL writes
 * the scratch size to *temp_bytes. */
/* out[r, j] = insertion point of vals[r, j] in the sorted row bounds[r (or 0 when shared), :]; sorter: optional permutation */
B200_API int b200_searchsorted(void* out, int out_i32, const void* bounds, const void* vals, const int64_t* sorter, int dtype,
                               int64_t rows, int64_t nv, int64_t nb, int shared_bounds, int right, cudaStream_t stream);
/* counts[bins] (fp32, zeroed by the caller) += histogram of x over [lo, hi] */
B200_API int b200_histc(float* counts, const void* x, int dtype, int64_t n, int bins, float lo, float hi, cudaStream_t stream);
/* linear[n] (capacity) and count[1]: flat indices of the non-zero elements in order */
B200_API int b200_nonzero_linear(void* temp, size_t* temp_bytes, int64_t* linear, int64_t* count, const void* x, int dtype,
                                 int64_t n, cudaStream_t stream);
/* coords[count, nd] from flat indices of a tensor of shape sizes[nd] (nd <= 8) */
B200_API int b200_unravel(int64_t* coords, const int64_t* linear, const int64_t* count, int64_t capacity, const int64_t* sizes,
                          int nd, cudaStream_t stream);
/* keys sorted ascending (fp32 / int32 / int64): unique values, their counts, number of runs; run_id[n] (may be NULL) */
B200_API int b200_unique_sorted(void* temp, size_t* temp_bytes, const void* keys, void* uniq, int64_t* counts,
                                int64_t* num_runs, int64_t* run_id, int dtype, int64_t n, cudaStream_t stream);
B200_API int b200_scatter_inverse(int64_t* inverse, const int64_t* run_id, const int64_t* perm, int64_t n, cudaStream_t stream);

/* ---- 2-D pooling over [N, H, W, C] (kernels/pool.cu); idx = h * W + w of the maximum inside its image plane */
typedef struct {
  int64_t N, H, W, C, Ho, Wo;
  int kh, kw, sh, sw, ph, pw, dh, dw;
} b200_pool_t;
B200_API int b200_maxpool2d_fwd(const b200_pool_t* p, int dtype, void* out, int64_t* idx, const void* in, cudaStream_t stream);
B200_API int b200_maxpool2d_bwd(const b200_pool_t* p, int dtype, void* gin, const void* gout, const int64_t* idx,
                                cudaStream_t stream);
/* divisor: 0 = window size clipped to the padded extent (count_include_pad), -1 = valid elements only, > 0 = override */
B200_API int b200_avgpool2d_fwd(const b200_pool_t* p, int dtype, void* out, const void* in, int divisor, cudaStream_t stream);
B200_API int b200_avgpool2d_bwd(const b200_pool_t* p, int dtype, void* gin, const void* gout, int divisor, cudaStream_t stream);

/* ---- implicit-GEMM convolution on the tensor cores (kernels/conv_tcgen05.cu): NHWC activations x[N,H,W,C],
 * y[N,Ho,Wo,K], filters w[K,R,S,C] (a channels-last [K,C,R,S] tensor), 16-bit dtypes, stride 1 or 2, zero padding,
 * no dilation, groups 1, C and K multiples of 8.  wgrad adds into dw_f32[K,R,S,C] (fp32, zeroed by the caller). */
typedef struct {
  int64_t N, H, W, C, K, Ho, Wo;
  int R, S, sh, sw, ph, pw;
  int dtype;
} b200_conv_t;
B200_API int b200_conv_supported(const b200_conv_t* d);
B200_API int b200_conv_fwd(const b200_conv_t* d, void* y, const void* x, const void* w, const void* bias /*or NULL*/,
                           int relu, cudaStream_t stream);
B200_API int b200_conv_dgrad(const b200_conv_t* d, void* dx, const void* dy, const void* w, cudaStream_t stream);
B200_API int b200_conv_wgrad(const b200_conv_t* d, float* dw_f32, const void* dy, const void* x, cudaStream_t stream);
/* on: the weight gradient is not split over pixels (one CTA per output tile, fixed order): bit-reproducible, slower */
B200_API void b200_conv_set_deterministic(int on);
/* Few-channel first layers (C == 8 after padding, S * 8 <= 64): xpad[N, H + 2 ph, W + 2 pw, 8] is the image with its
 * zero border written out, wpack[K][R][64] holds filter row r as element s * 8 + c (zero tail); one K step covers a
 * whole filter row.  wgrad adds into dwpack_f32[K][R][64]. */
B200_API int b200_conv_stem_supported(const b200_conv_t* d);
B200_API int b200_conv_stem_fwd(const b200_conv_t* d, void* y, const void* xpad, const void* wpack, const void* bias,
                                int relu, cudaStream_t stream);
B200_API int b200_conv_stem_wgrad(const b200_conv_t* d, float* dwpack_f32, const void* dy, const void* xpad,
                                  cudaStream_t stream);
/* 1 if a conv kernel gave up a bounded wait since the last clear */
B200_API int b200_conv_status(int clear);

/* ---------------------------------------------------------------- normalisation */
/* y = x * rstd * w ; rstd[rows] fp32.  residual (optional): x_in = x + residual, written to res_out. */
B200_API int b200_rmsnorm_fwd(int dtype, void* y, float* rstd, const void* x, const void* w, const void* residual,
                              void* res_out, int64_t rows, int64_t cols, float eps, cudaStream_t stream);
/* dx (and optionally dw partial sums in dw_partial[nblocks, cols] fp32; pass NULL to skip) */
B200_API int b200_rmsnorm_bwd(int dtype, void* dx, float* dw_partial, int* nblocks_out_host, const void* dy,
                              const void* x, const void* w, const float* rstd, int64_t rows, int64_t cols,
                              cudaStream_t stream);
B200_API int b200_rmsnorm_bwd_partial_rows(int64_t rows, int64_t cols);
B200_API int b200_layernorm_fwd(int dtype, void* y, float* mean, float* rstd, const void* x, const void* w,
                                const void* b, int64_t rows, int64_t cols, float eps, cudaStream_t stream);
B200_API int b200_layernorm_bwd(int dtype, void* dx, float* dw_partial, float* db_partial, const void* dy,
                                const void* x, const void* w, const float* mean, const float* rstd, int64_t rows,
                                int64_t cols, cudaStream_t stream);

/* ---------------------------------------------------------------- softmax / loss */
B200_API int b200_softmax_fwd(int dtype, void* y, const void* x, int64_t rows, int64_t cols, int log_softmax,
                              cudaStream_t stream);
/* dx from dy and y (softmax output or log-softmax output) */
B200_API int b200_softmax_bwd(int dtype, void* dx, const void* dy, const void* y, int64_t rows, int64_t cols,
                              int log_softmax, cudaStream_t stream);
/* fused cross entropy: per-row loss (fp32) and log-sum-exp (fp32); rows with target == ignore_index give 0 */
B200_API int b200_cross_entropy_fwd(int dtype, float* loss, float* lse, const void* logits, const int64_t* target,
                                    int64_t rows, int64_t cols, int64_t ignore_index, float label_smoothing,
                                    cudaStream_t stream);
/* dlogits = (softmax - onehot) * grad_scale[row or scalar]; may run in place over logits */
B200_API int b200_cross_entropy_bwd(int dtype, void* dlogits, const void* logits, const float* lse,
                                    const int64_t* target, const float* grad_loss, int grad_is_scalar, float scale,
                                    int64_t rows, int64_t cols, int64_t ignore_index, float label_smoothing,
                                    cudaStream_t stream);
/* vocab-parallel pieces: per-row (max, sumexp, target logit) over a vocab shard [vocab_start, vocab_start+cols) */
B200_API int b200_online_softmax_stats(int dtype, float* stats3, const void* logits, const int64_t* target,
                                       int64_t rows, int64_t cols, int64_t vocab_start, cudaStream_t stream);
/* combine world x [rows,3] stats -> loss[rows]; writes softmax-gradient in place into the logits shard */
B200_API int b200_vocab_parallel_ce_finish(int dtype, float* loss, void* logits_inout, const float* all_stats,
                                           int world, const int64_t* target, int64_t rows, int64_t cols,
                                           int64_t vocab_start, int64_t ignore_index, cudaStream_t stream);

/* ---------------------------------------------------------------- fused LLM ops */
/* rotary embedding on x [tokens, heads, dim] with cos/sin [tokens(or seq), dim/2] (fp32);
 * position of token t is pos[t] if pos != NULL else (t % seq). interleaved: pairs (2i,2i+1) vs halves (i,i+d/2).
 * backward == forward with conj=1. */
B200_API int b200_rope(int dtype, void* out, const void* x, const float* cos, const float* sin, const int64_t* pos,
                       int64_t tokens, int64_t seq, int heads, int dim, int64_t x_token_stride, int64_t x_head_stride,
                       int interleaved, int conj, cudaStream_t stream);
/* x [rows, 2*h] -> out [rows, h] = silu(x[:, :h]) * x[:, h:]  (gate_first=1) */
B200_API int b200_swiglu_fwd(int dtype, void* out, const void* x, int64_t rows, int64_t h, cudaStream_t stream);
/* Same, limited to the first sum(row_counts[0..n_counts)) rows (device int32 counts of packed row groups; NULL: all rows);
 * the other rows of out / dx are left untouched. */
B200_API int b200_swiglu_fwd_rows(int dtype, void* out, const void* x, int64_t rows, int64_t h, const int* row_counts,
                                  int n_counts, cudaStream_t stream);
B200_API int b200_swiglu_bwd_rows(int dtype, void* dx, const void* dy, const void* x, int64_t rows, int64_t h,
                                  const int* row_counts, int n_counts, cudaStream_t stream);
B200_API int b200_swiglu_bwd(int dtype, void* dx, const void* dy, const void* x, int64_t rows, int64_t h,
                             cudaStream_t stream);
/* two-tensor form: out = silu(gate) * up */
B200_API int b200_silu_mul_fwd(int dtype, void* out, const void* gate, const void* up, int64_t n, cudaStream_t stream);
B200_API int b200_silu_mul_bwd(int dtype, void* dgate, void* dup, const void* dy, const void* gate, const void* up,
                               int64_t n, cudaStream_t stream);

/* ---------------------------------------------------------------- embedding */
B200_API int b200_embedding_fwd(int dtype, void* out, const void* weight, const int64_t* idx, int64_t n, int64_t dim,
                                int64_t vocab, cudaStream_t stream);
/* dense backward, fp32 atomics into grad_weight_f32 [vocab, dim] (must be zeroed), skipping padding_idx */
B200_API int b200_embedding_bwd_atomic(int dtype, float* grad_weight_f32, const void* grad_out, const int64_t* idx,
                                       int64_t n, int64_t dim, int64_t vocab, int64_t padding_idx,
                                       cudaStream_t stream);
/* deterministic: indices pre-sorted (sorted_idx, perm); one warp group per segment */
B200_API int b200_embedding_bwd_sorted(int dtype, void* grad_weight, const void* grad_out, const int64_t* sorted_idx,
                                       const int64_t* perm, int64_t n, int64_t dim, int64_t vocab,
                                       int64_t padding_idx, cudaStream_t stream);

/* ---------------------------------------------------------------- dropout (Philox 4x32-10) */
typedef struct {
  uint64_t seed, offset;
  const int64_t* seed_ptr;
  const int64_t* offset_ptr;
  uint64_t offset_intragraph;
  int captured;
} b200_philox_t;
B200_API int b200_dropout_fwd(int dtype, void* out, uint8_t* mask, const void* x, int64_t n, float p,
                              b200_philox_t rng, cudaStream_t stream);
B200_API int b200_dropout_bwd(int dtype, void* dx, const void* dy, const uint8_t* mask, int64_t n, float scale,
                              cudaStream_t stream);
B200_API int b200_uniform(int dtype, void* out, int64_t n, double lo, double hi, b200_philox_t rng, cudaStream_t s);
B200_API int b200_normal(int dtype, void* out, int64_t n, double mean, double std, b200_philox_t rng, cudaStream_t s);

/* ---------------------------------------------------------------- multi-tensor apply */
/* Lists are host arrays of device pointers; metadata travels in kernel parameter space. */
typedef struct {
  float lr, beta1, beta2, eps, weight_decay;
  int adamw;        /* decoupled weight decay */
  int amsgrad;
  int maximize;
  const float* lr_ptr;        /* device scalar overrides lr when non-NULL */
  const float* grad_scale;    /* device scalar; grads are divided by it when non-NULL */
  const float* found_inf;     /* device scalar; the step is skipped when *found_inf != 0 */
} b200_adam_args_t;
/* steps: device pointers to per-tensor fp32 step counters (incremented in kernel unless found_inf) */
B200_API int b200_multi_tensor_adam(int n_tensors, int param_dtype, int grad_dtype, int state_dtype,
                                    void* const* params, void* const* grads, void* const* exp_avg,
                                    void* const* exp_avg_sq, void* const* max_exp_avg_sq, float* const* steps,
                                    const int64_t* numels, b200_adam_args_t args, cudaStream_t stream);
typedef struct {
  float lr, momentum, dampening, weight_decay;
  int nesterov, maximize, first_step;
  const float* lr_ptr;
  const float* grad_scale;
  const float* found_inf;
} b200_sgd_args_t;
B200_API int b200_multi_tensor_sgd(int n_tensors, int param_dtype, int grad_dtype, void* const* params,
                                   void* const* grads, void* const* momentum_bufs, const int64_t* numels,
                                   b200_sgd_args_t args, cudaStream_t stream);
/* per-tensor and global L2 norm. out_per_tensor [n] fp32 (may be NULL), out_total[1] fp32. scratch: (n*320+320) floats */
B200_API int b200_multi_tensor_l2norm(int n_tensors, int dtype, void* const* tensors, const int64_t* numels,
                                      float* out_total, float* out_per_tensor, float* scratch, cudaStream_t stream);
B200_API size_t b200_multi_tensor_l2norm_scratch_floats(int n_tensors);
/* x *= scale (device scalar scale_ptr or host scale); sets *found_inf=1 when a non-finite value is seen */
B200_API int b200_multi_tensor_scale(int n_tensors, int dtype, void* const* tensors, const int64_t* numels,
                                     const float* inv_scale_ptr, float host_scale, float* found_inf,
                                     cudaStream_t stream);
/* generic foreach binary with scalar: t = op(t, s) or t = t + alpha * u */
/* out[i] = f(a[i][, b[i][, c[i]]]) over whole tensor lists in a couple of launches (the _foreach_* family); b / c may
 * be NULL; all tensors of one floating dtype, dense, same numel per position */
enum { B200_FE_ADD_SCALAR = 0, B200_FE_MUL_SCALAR, B200_FE_DIV_SCALAR, B200_FE_ADD, B200_FE_MUL, B200_FE_DIV,
       B200_FE_ADDCMUL, B200_FE_ADDCDIV, B200_FE_LERP, B200_FE_SQRT, B200_FE_NEG, B200_FE_RECIPROCAL, B200_FE_ABS,
       B200_FE_MAXIMUM, B200_FE_MINIMUM, B200_FE_CLAMP, B200_FE_ZERO, B200_FE_COPY };
B200_API int b200_multi_tensor_pointwise(int op, int n, int dtype, void* const* out, void* const* a, void* const* b,
                                         void* const* c, const int64_t* numels, float s0, float s1, cudaStream_t stream);
B200_API int b200_multi_tensor_axpby(int n_tensors, int dtype, void* const* out, void* const* x, void* const* y,
                                     const int64_t* numels, float a, float b, cudaStream_t stream);
/* LAMB: stage 1 computes update in `update` list; stage 2 applies trust ratio per tensor */
typedef struct {
  float lr, beta1, beta2, eps, weight_decay, max_grad_norm;
  int step, bias_correction, grad_averaging, adam_w_mode, use_nvlamb;
  const float* global_grad_norm; /* device scalar */
} b200_lamb_args_t;
B200_API int b200_multi_tensor_lamb(int n_tensors, int dtype, void* const* params, void* const* grads,
                                    void* const* exp_avg, void* const* exp_avg_sq, const int64_t* numels,
                                    b200_lamb_args_t args, float* scratch, cudaStream_t stream);
B200_API size_t b200_multi_tensor_lamb_scratch_floats(int n_tensors, const int64_t* numels);
/* GradScaler bookkeeping: one thread */
B200_API int b200_amp_update_scale(float* scale, int* growth_tracker, const float* found_inf, float growth,
                                   float backoff, int growth_interval, cudaStream_t stream);

/* ---------------------------------------------------------------- GEMM (tcgen05 + TMEM + TMA) */
/* D[M,N] = alpha * A[M,K] x B^T + beta * C, with B given as [N,K] when trans_b == 0 layout code:
 *   a_kmajor: A is row-major [M,K] (K contiguous); else A is stored [K,M] (M contiguous)
 *   b_kmajor: B is stored [N,K] (K contiguous);    else B is stored [K,N] (N contiguous)
 * lda/ldb/ldd are the leading (non-contiguous) strides in elements. dtype: BF16 or F16 inputs, fp32 accumulate,
 * output dtype out_dtype (BF16/F16/F32). bias (optional, [N], out dtype or fp32) is added in the epilogue;
 * epilogue act: 0 none, 1 relu, 2 gelu(erf), 3 silu. accumulate != 0: D += result (beta = 1).
 * batch > 1 strides in elements (0 = broadcast). Returns cudaErrorNotSupported for shapes the kernel does not
 * cover (caller falls back): K % 8 != 0 or unaligned leading strides.
 */
typedef struct {
  int m, n, k;
  int a_kmajor, b_kmajor;
  int64_t lda, ldb, ldd;
  int in_dtype, out_dtype;
  int batch;
  int64_t stride_a, stride_b, stride_d;
  const void* bias; int bias_dtype;
  int act;
  int accumulate;
  float alpha;
  /* optional fp32 scratch for split-K (see b200_gemm_workspace_bytes); NULL / 0: never split */
  void* workspace;
  size_t workspace_bytes;
} b200_gemm_desc_t;
B200_API int b200_gemm(const b200_gemm_desc_t* desc, void* d, const void* a, const void* b, cudaStream_t stream);
/* Grouped GEMM whose per-group lengths are read from device memory (`counts`, int32 [groups], groups <= 64).
 *   ragged_depth = 0: d[r, 0:n] = a[r, 0:k] * b[g(r)]^T for the packed rows r of group g; a [rows, k] (lda), d [rows, n]
 *                     (ldd); b [groups, n, k] when b_kmajor, else [groups, k, n] (ldb, stride_b per group).
 *   ragged_depth = 1: d[g] [m, n] (ldd, stride_d) = a[rows of g, 0:m]^T * b[rows of g, 0:n]; a [rows, m] (lda), b [rows, n].
 * Rows past the sum of the counts are neither read into a result nor written; an empty group's d[g] is zero. */
typedef struct {
  int ragged_depth;
  int rows, m, n, k;
  int groups;
  const int* counts;
  int b_kmajor;
  int in_dtype, out_dtype;
  int64_t lda, ldb, ldd;
  int64_t stride_b, stride_d;
} b200_grouped_gemm_t;
B200_API int b200_grouped_gemm(const b200_grouped_gemm_t* desc, void* d, const void* a, const void* b, cudaStream_t stream);
/* Scratch a split-K run of this problem wants (few output tiles, long K); 0 when the problem is not split. */
B200_API size_t b200_gemm_workspace_bytes(const b200_gemm_desc_t* desc);
/* 1 when the running driver exposes the tensor-map encoder the kernel needs */
B200_API int b200_gemm_available(void);

/* ---- batch normalisation over a [P, C] channels-last matrix (bf16 / fp16 activations, fp32 statistics) ----
 * sums is a [2*C] fp32 workspace the call zeroes itself. stats_mode 0: batch statistics from sums (training),
 * 1: running statistics (inference). resid / dresid / y may be NULL when the residual / ReLU variants are off. */
B200_API int b200_bn_stats(int dtype, const void* x, float* sums, int64_t P, int C, cudaStream_t stream);
B200_API int b200_bn_apply(int dtype, const void* x, const void* resid, void* y, const float* sums, const float* w,
                           const float* b, float* running_mean, float* running_var, float* save_mean,
                           float* save_invstd, int64_t P, int C, float eps, float momentum, int relu, int stats_mode,
                           cudaStream_t stream);
B200_API int b200_bn_bwd_reduce(int dtype, const void* dy, const void* x, const void* y, const float* mean,
                                const float* invstd, float* sums, int64_t P, int C, int relu, cudaStream_t stream);
B200_API int b200_bn_bwd_apply(int dtype, const void* dy, const void* x, const void* y, const float* mean,
                               const float* invstd, const float* w, const float* sums, void* dx, void* dresid,
                               int64_t P, int C, int relu, cudaStream_t stream);

/* non-zero once any GEMM launch of this process gave up on a bounded pipeline wait (sticky; clear != 0 resets) */
B200_API int b200_gemm_status(int clear);
/* Tile configuration for later launches: 0 cost model (default), 1 single-CTA 128x256, 2 SM-pair 256x256 with
 * the static tile schedule, 3 SM-pair 256x256 with the dynamic (cluster launch control) schedule.  Returns the previous setting, -1 for an unknown value. */
B200_API int b200_gemm_force_config(int config);
/* Philox counters one launch of the random kernels may consume per thread, for n outputs */
B200_API uint64_t b200_philox_increment(int64_t n);

/* ---------------------------------------------------------------- collectives over peer-mapped memory */
/* Every rank's arena and signal pad as mapped in THIS process (index = rank). `status` is a host-mapped word
 * the kernels set to non-zero when a bounded wait expired. Epochs must grow by at least 2 per call and be
 * identical on all ranks for the same call; offsets are byte offsets into the arena, multiples of 16. */
typedef struct {
  void* bufs[16];
  uint32_t* sigs[16];
  int rank, world;
  int* status;
} b200_symm_t;
B200_API int b200_comm_max_world(void);
/* Limit of every device-side wait on another rank (default 2 s); a kernel whose wait runs out sets `status`
 * and returns.  Process-wide, read at launch time. */
B200_API void b200_comm_set_wait_ms(double ms);
B200_API double b200_comm_get_wait_ms(void);
B200_API size_t b200_comm_signal_bytes(void);
/* words [user_word0, pad_words) of a signal pad belong to the arena's owner (kernel-wide flags, counters) */
B200_API int b200_comm_user_word0(void);
B200_API int b200_comm_pad_words(void);
/* out = scale * sum_ranks(in), n elements (n % 8 == 0); arena use: n*sizeof(in) at in_off, n*sizeof(out) at out_off */
B200_API int b200_comm_allreduce(const b200_symm_t* s, int in_dtype, int out_dtype, const void* in, void* out,
                                 int64_t n, float scale, uint32_t epoch, int64_t in_off, int64_t out_off,
                                 cudaStream_t stream);
/* out [world * nbytes] = concat over ranks of in [nbytes] (nbytes % 16 == 0); arena use: nbytes at in_off */
B200_API int b200_comm_allgather(const b200_symm_t* s, int dtype_bytes, const void* in, void* out, int64_t nbytes,
                                 uint32_t epoch, int64_t in_off, cudaStream_t stream);
/* out [n_out] = scale * sum_ranks(in_rank[rank*n_out : (rank+1)*n_out]); arena use: world*n_out*sizeof(in) */
B200_API int b200_comm_reduce_scatter(const b200_symm_t* s, int in_dtype, int out_dtype, const void* in, void* out,
                                      int64_t n_out, float scale, uint32_t epoch, int64_t in_off,
                                      cudaStream_t stream);
/* reduce-scatter whose epilogue is the AdamW step on the owner's fp32 shard (p32, m, v) and its bf16 copy p16 */
B200_API int b200_comm_reduce_scatter_adamw(const b200_symm_t* s, int in_dtype, const void* in, float* p32, float* m,
                                            float* v, void* p16, int64_t n_out, float scale, uint32_t epoch,
                                            int64_t in_off, float lr, float beta1, float beta2, float eps, float wd,
                                            const float* step_ptr, cudaStream_t stream);
/* all-to-all with per-peer splits; all offsets/lengths in bytes, multiples of 16. peer_send_off[p] = offset of
 * the slice destined to this rank inside peer p's input. */
B200_API int b200_comm_alltoall(const b200_symm_t* s, const void* in, void* out, int64_t in_bytes,
                                const int64_t* send_off, const int64_t* recv_off, const int64_t* recv_len,
                                const int64_t* peer_send_off, uint32_t epoch, int64_t in_off, cudaStream_t stream);

/* ---- sharded-parameter collectives (kernels/fsdp_comm.cu).  A parameter group is a list of tensors, each cut
 * into `world` equal (padded) shards along its first dimension; rank r's shards are laid out in one flat buffer
 * ("flat shard": tensor i at element offset shard_off[i], a multiple of 8, `total` elements, a multiple of 8).
 * Flag and counter arguments are word indices into the signal pad (b200_comm_user_word0 and up); a flag occupies
 * 16 consecutive words (one per source rank), a counter block 2 words that are zero between launches. */
#define B200_FSDP_MAX_TENSORS 40
typedef struct {
  int n;
  int64_t shard_numel[B200_FSDP_MAX_TENSORS];
  int64_t shard_off[B200_FSDP_MAX_TENSORS];
  int64_t full_numel[B200_FSDP_MAX_TENSORS]; /* elements of the unsharded tensor, <= world * shard_numel */
  int64_t total;
} b200_fsdp_layout_t;
typedef struct {
  float* p[B200_FSDP_MAX_TENSORS];           /* fp32 master shards, moments: shard_numel[i] elements each */
  float* m[B200_FSDP_MAX_TENSORS];
  float* v[B200_FSDP_MAX_TENSORS];
  float lr, beta1, beta2, eps, weight_decay, step;
  int64_t shadow_off;                        /* byte offset of the low-precision flat shard in the arena, -1: none */
  int shadow_dtype;
  int shadow_flag_word;
  uint32_t shadow_version;
} b200_fsdp_adamw_t;
/* shadow (flat shard at shadow_off of the local arena, dst_dtype) = cast(srcs[i]); then flag_word[rank] = version
 * in every peer's pad. */
B200_API int b200_fsdp_pack(const b200_symm_t* s, const b200_fsdp_layout_t* L, const void* const* srcs, int src_dtype,
                            int64_t shadow_off, int dst_dtype, int flag_word, uint32_t version, int counter_word,
                            int n_ctas, cudaStream_t stream);
/* outs[i][p * shard_numel[i] + e] = rank p's flat shard [shard_off[i] + e], after flag_word[p] >= version */
B200_API int b200_fsdp_gather(const b200_symm_t* s, const b200_fsdp_layout_t* L, void* const* outs, int dtype,
                              int64_t shadow_off, int flag_word, uint32_t version, int n_ctas, cudaStream_t stream);
/* Gradient reduce-scatter: grads[i] (grad_dtype, full_numel[i] elements) -> this rank's shard of the sum over
 * ranks, times scale, in fp32: written to out32 (flat shard) or consumed by the AdamW epilogue (`opt`).  Staging:
 * world slots of `total` elements (grad_dtype) at stage_off of every arena.  seq: number of this call (same on all
 * ranks, growing); ack_need: the call number whose completion on every peer frees this staging buffer (0: none). */
B200_API int b200_fsdp_reduce(const b200_symm_t* s, const b200_fsdp_layout_t* L, const void* const* grads,
                              int grad_dtype, int64_t stage_off, float scale, float* out32,
                              const b200_fsdp_adamw_t* opt, int ready_word, int ack_word, uint32_t seq,
                              uint32_t ack_need, int counter_word, int n_ctas, cudaStream_t stream);

/* all-gather -> GEMM in ONE launch: D[M, N] = rows gathered from every rank's shard [M / world, K] (at shard_off of
 * its arena) times B[N, K]^T.  A few copier CTAs stream the peers' shards into a_full [M, K] (local) with bulk
 * copies while the other clusters multiply the 256-row panels that have arrived (own shard first).  flags: local
 * uint32 [M / 256], zeroed once, reused by every call; the call uses epochs `epoch` and `epoch + 1`.
 * Needs M % (256 * world) == 0, K % 64 == 0, K-major contiguous A. */
B200_API int b200_gemm_allgather(const b200_gemm_desc_t* desc, const b200_symm_t* s, int64_t shard_off, void* a_full,
                                 uint32_t* flags, uint32_t epoch, int copier_pairs, void* d, const void* b,
                                 cudaStream_t stream);

/* GEMM -> reduce-scatter in ONE launch: out[M / world, N] = row block `rank` of the sum over ranks of
 * A_r[M, K_r] x B_r[N, K_r]^T.  Tiles go to a partial buffer in the arena (other ranks' panels first) and raise
 * per-tile flags in the panel owner's arena; reducer CTAs of the same launch pull the finished panels from every
 * rank with bulk copies, add them in fp32 and write the output.  flag table: world * (M/256/world) * (N/256) * 2
 * uint32 at flag_off of every arena, zeroed once.  Needs M % (256 * world) == 0, N % 256 == 0, world <= 8. */
B200_API int b200_gemm_reduce_scatter(const b200_gemm_desc_t* desc, const b200_symm_t* s, int64_t partial_off,
                                      int64_t flag_off, uint32_t epoch, int reducer_pairs, void* out, const void* a,
                                      const void* b, cudaStream_t stream);

/* ---------------------------------------------------------------- block-scaled fp8 GEMM (tcgen05 kind::f8f6f4)
 * D[M,N] = sum_kb bsa[m, kb] * bsb[n / 128, kb] * (A[m, kb-th 128 of K] . B[n, same]) * row_scale[m] * col_scale[n] + bias.
 * A [M,K], B [N,K]: fp8 bytes, K contiguous, lda / ldb in bytes (multiples of 16). Any scale pointer may be NULL (= 1);
 * a stride of 0 broadcasts (tensor-wise scaling = row_scale with stride 0). Block scales need K % 128 == 0. */
typedef struct {
  int m, n, k;
  int64_t lda, ldb, ldd;
  int a_e5m2, b_e5m2;
  int out_dtype;
  const float* block_scale_a; int64_t bsa_stride_m, bsa_stride_kb;
  const float* block_scale_b; int64_t bsb_stride_nb, bsb_stride_kb;
  const float* row_scale; int64_t row_scale_stride;
  const float* col_scale; int64_t col_scale_stride;
  const void* bias; int bias_dtype;
} b200_fp8_gemm_t;
B200_API int b200_gemm_fp8(const b200_fp8_gemm_t* desc, void* d, const void* a, const void* b, cudaStream_t stream);
/* q [rows, k] fp8 bytes and scales [rows, k / 128] (amax / 448 per 1 x 128 block) from x [rows, k] (ldx elements) */
B200_API int b200_quantize_fp8_1x128(int dtype, const void* x, void* q, float* scales, int64_t rows, int k, int64_t ldx,
                                     int e5m2, cudaStream_t stream);

/* ---------------------------------------------------------------- flash attention forward (tcgen05 + TMEM)
 * q [B, H, Sq, 128], k / v [B, Hkv, Sk, 128] (H % Hkv == 0), out [B, H, Sq, 128], all with a contiguous last dimension
 * and element strides (multiples of 8) for batch, head and sequence; lse [B, H, Sq] fp32 natural-log (may be NULL).
 * causal != 0: key index <= query index. */
typedef struct {
  int B, H, Hkv, Sq, Sk, head_dim;
  int dtype;
  int causal;
  float scale;
  int64_t q_sb, q_sh, q_ss, k_sb, k_sh, k_ss, v_sb, v_sh, v_ss, o_sb, o_sh, o_ss;
  /* Packed variable-length sequences (both NULL: dense batch).  Device int32 [B + 1] prefix sums of the sequence
   * lengths; q / out / d_o are [total_q, H, 128], k / v (and dk / dv) [total_k, Hkv, 128] addressed with the *_sh and
   * *_ss strides (the *_sb strides are ignored); Sq / Sk are the longest lengths; lse and delta are [H, total_q],
   * dq_accum [H, total_q, 128].  Causal masks compare positions inside a sequence. */
  const int* cu_seqlens_q;
  const int* cu_seqlens_k;
  int total_q, total_k;
} b200_attn_t;
B200_API int b200_flash_attn_fwd(const b200_attn_t* desc, void* out, float* lse, const void* q, const void* k,
                                 const void* v, cudaStream_t stream);
/* Backward of the same attention.  dq_accum [B, H, Sq, 128] fp32 (the call zeroes it; the caller converts it),
 * dk / dv [B, Hkv, Sk, 128] and d_o [B, H, Sq, 128] with the element strides in extra_strides = {do_sb, do_sh, do_ss,
 * dk_sb, dk_sh, dk_ss, dv_sb, dv_sh, dv_ss}; o uses desc->o_*; delta [B, H, Sq] fp32 is scratch the call fills;
 * lse [B, H, Sq] is the forward's natural-log row sum. */
B200_API int b200_flash_attn_bwd(const b200_attn_t* desc, float* dq_accum, void* dk, void* dv, float* delta,
                                 const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                 const float* lse, const int64_t* extra_strides, cudaStream_t stream);

/* single-query attention over a static KV cache: q / out [B, H, 128], caches [B, Hkv, max_len, 128] contiguous, keys
 * [0, *pos] visible (pos: device int64, read by the kernel, so the call is graph-capturable) */
B200_API int b200_decode_attention(int dtype, void* out, const void* q, const void* k_cache, const void* v_cache,
                                   const long long* pos, int B, int H, int Hkv, int max_len, int head_dim, float scale,
                                   cudaStream_t stream);

/* One decode step's rotary embedding + cache update: q_out [B, H, 128] = rope(q), k_cache[b, hk, *pos] = rope(k),
 * v_cache[b, hk, *pos] = v.  q / k / v rows of 128 contiguous elements addressed by strides = {q batch, q head, k batch,
 * k head, v batch, v head} (elements); cos / sin float [table_len, 64] (rotate-half layout); caches [B, Hkv, max_len, 128]. */
B200_API int b200_decode_rope_cache(int dtype, void* q_out, const void* q, const void* k, const void* v, const int64_t* strides,
                                    const float* cosv, const float* sinv, const long long* pos, void* k_cache, void* v_cache,
                                    int B, int H, int Hkv, int max_len, int head_dim, int table_len, cudaStream_t stream);

/* ---------------------------------------------------------------- expert-parallel MoE token exchange (bf16 rows)
 * E experts, E / world per rank in rank order; idx / slot / pos are int32 [T*K]; receive buffers hold cap_rows
 * rows of d elements at a byte offset of every rank's arena; counts_off points at world*E int32 of scratch in the
 * arena. Epochs as for the collectives (each call consumes two). */
B200_API int b200_moe_count(const int* idx, int* slot, int* counts, int64_t n_pairs, int E, cudaStream_t stream);
B200_API int b200_moe_dispatch(const b200_symm_t* s, const void* x, const int* idx, const int* slot,
                               const int* counts_local, int* pos, int* recv_counts, int T, int K, int d, int E,
                               int64_t cap_rows, int64_t recv_off, int64_t counts_off, uint32_t epoch,
                               cudaStream_t stream);
B200_API int b200_moe_gather(const b200_symm_t* s, void* out, const int* idx, const int* pos, const float* w, int T,
                             int K, int d, int E, int64_t src_off, uint32_t epoch, cudaStream_t stream);
B200_API int b200_moe_scatter(const b200_symm_t* s, const void* x, const int* idx, const int* pos, const float* w,
                              int T, int K, int d, int E, int64_t dst_off, uint32_t epoch, cudaStream_t stream);
B200_API int b200_moe_gather_dot(const b200_symm_t* s, const void* grad, const int* idx, const int* pos, float* dw,
                                 int T, int K, int d, int E, int64_t src_off, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
