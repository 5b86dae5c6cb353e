/*
 * zyxb.h — C ABI of libzyxb, a B200 (sm_100a) compute backend for the zyx ML library.
 *
 * The entry points are what a thin Rust shim `zyx/src/backend/b200.rs` would bind with
 * `extern "C"`; each one replaces one method of zyx's enum-dispatched backend interface
 * (`MemoryPool` / `Device` in zyx/src/backend/mod.rs).  The citation beside every
 * declaration is the reference interface it stands in for.
 *
 * Conventions
 *   - every function returns an int32 status: 0 = ok, otherwise 1 + the ordinal of
 *     zyx's `ErrorStatus` (zyx/src/error.rs:127-153); `zyxb_last_error` gives the text
 *     that would become `BackendError::context`.
 *   - no exceptions, no aborts, no device traps; a bounded device-side wait that runs
 *     out reports ZYXB_ERR_KERNEL_SYNC.
 *   - calls may come from any OS thread, one at a time per context (zyx serialises them
 *     under its global runtime mutex, zyx/src/lib.rs:96).
 *   - buffers, programs and events are small integer handles owned by the library, like
 *     `PoolBufferId` / `DeviceProgramId` / `Event` (zyx/src/backend/mod.rs:55,122,335).
 *   - there is no CPU fallback: without a CUDA device `zyxb_init` fails.
 */
#ifndef ZYXB_H
#define ZYXB_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes: 1 + ordinal of ErrorStatus (zyx/src/error.rs:127-153) ---- */
enum {
  ZYXB_OK = 0,
  ZYXB_ERR_DYLIB_NOT_FOUND = 1,
  ZYXB_ERR_INITIALIZATION = 2,
  ZYXB_ERR_DEINITIALIZATION = 3,
  ZYXB_ERR_DEVICE_ENUMERATION = 4,
  ZYXB_ERR_DEVICE_QUERY = 5,
  ZYXB_ERR_MEMORY_ALLOCATION = 6,
  ZYXB_ERR_MEMORY_DEALLOCATION = 7,
  ZYXB_ERR_MEMORY_COPY_H2P = 8,
  ZYXB_ERR_MEMORY_COPY_P2H = 9,
  ZYXB_ERR_INCORRECT_KERNEL_ARG = 10,
  ZYXB_ERR_KERNEL_COMPILATION = 11,
  ZYXB_ERR_KERNEL_LAUNCH = 12,
  ZYXB_ERR_KERNEL_SYNC = 13
};

/* ---- dtypes: same order as zyx's DType enum (zyx/src/dtype.rs:18-32) ---- */
enum {
  ZYXB_BF16 = 0, ZYXB_F16 = 1, ZYXB_F32 = 2, ZYXB_F64 = 3,
  ZYXB_U8 = 4, ZYXB_U16 = 5, ZYXB_U32 = 6, ZYXB_U64 = 7,
  ZYXB_I8 = 8, ZYXB_I16 = 9, ZYXB_I32 = 10, ZYXB_I64 = 11, ZYXB_BOOL = 12
};

typedef struct zyxb_ctx zyxb_ctx;

/* An event handle; 0 is the null event (already complete).
 * Mirrors `Event` (zyx/src/backend/mod.rs:335-347). */
typedef struct { uint64_t id; } zyxb_event;

/* Mirrors the per-backend config struct deserialised from config.json, e.g.
 * `CUDAConfig{device_ids}` (zyx/src/backend/cuda.rs:142-148). */
typedef struct {
  int32_t n_device_ids;    /* 0 = use every visible device */
  int32_t device_ids[16];
  int32_t debug;           /* ZYX_DEBUG-style bitmask; 1 prints devices and launches; 2 puts guard words behind every
                              allocation (see zyxb_check_guards) */
  int32_t round_nearest;   /* 0 (default): bf16/f16 stores truncate like the reference C
                              backend (zyx/src/codegen/c.rs:475-496); 1: round to nearest */
} zyxb_config;

/* Mirrors `DeviceInfo` (zyx/src/backend/mod.rs:506-531). */
typedef struct {
  uint64_t compute_flops;            /* DeviceInfo::compute (dense bf16 FLOP/s) */
  uint64_t max_global_work_dims[3];
  uint32_t max_local_threads;
  uint32_t max_local_work_dims[3];
  uint32_t preferred_vector_size;    /* bytes */
  uint64_t local_mem_size;           /* shared memory per CTA, bytes */
  uint64_t max_register_bytes;
  int32_t  tensor_cores;
  uint32_t warp_size;
  uint32_t dtype_capability[13];     /* op bitmask per dtype, DTypeCapability (mod.rs:418-502) */
  int32_t  has_native_exp2;
  uint32_t sm_count;
  uint64_t total_mem_bytes;
  int32_t  cc_major, cc_minor;
  char     name[128];
} zyxb_devinfo;

/* ------------------------------------------------------------------------------------
 * Kernel descriptors: what `zyxb_program_create` consumes.  A descriptor is what the
 * shim's `match_graph` (zyx/src/backend/mod.rs:952-961, model: backend/cblas.rs:213-238)
 * produces when it recognises a subgraph; the resulting program id goes into
 * `Node::Kernel{inputs,outputs,program_id,time}` (zyx/src/graph/mod.rs:177-182).
 * Launch arguments are always inputs first, then outputs, as `Device::launch` receives
 * them (zyx/src/backend/mod.rs:974, zyx/src/runtime.rs:2285-2291).
 * ---------------------------------------------------------------------------------- */
enum { ZYXB_KIND_ROWREDUCE = 1, ZYXB_KIND_GEMM = 2, ZYXB_KIND_ELTWISE = 3, ZYXB_KIND_OPTIM = 4, ZYXB_KIND_ATTENTION = 5, ZYXB_KIND_ATTENTION_BWD = 6,
       ZYXB_KIND_CONV = 7, ZYXB_KIND_CONV_WGRAD = 8, ZYXB_KIND_CONV_DGRAD = 9 };

/* Row kernels: an elementwise chain with a trailing reduce over the last axis.
 * Semantics: Tensor::reduce_impl (zyx/src/tensor/reduce_ops.rs:45-157), softmax /
 * ln_softmax (zyx/src/tensor/mod.rs:1427-1461), LayerNorm::forward
 * (zyx-nn/src/layer_norm.rs:95-135), cross_entropy (zyx/src/tensor/mod.rs:1639-1655). */
enum {
  ZYXB_RR_SUM = 0,        /* args: x -> y[rows] */
  ZYXB_RR_MAX = 1,        /* args: x -> y[rows] */
  ZYXB_RR_MIN = 2,        /* args: x -> y[rows]   (= -max(-x)) */
  ZYXB_RR_MEAN = 3,       /* args: x -> y[rows] */
  ZYXB_RR_VAR = 4,        /* args: x -> y[rows]   divisor cols - correction */
  ZYXB_RR_STD = 5,        /* args: x -> y[rows] */
  ZYXB_RR_SOFTMAX = 6,    /* args: x -> y[rows,cols]; optional scale and causal mask */
  ZYXB_RR_LN_SOFTMAX = 7, /* args: x -> y[rows,cols] */
  ZYXB_RR_LAYERNORM = 8,  /* args: x [,weight][,bias] -> y[rows,cols] */
  ZYXB_RR_CROSS_ENTROPY = 9,      /* args: logits, labels(i32) -> per_sample[rows], mean[1] */
  ZYXB_RR_CROSS_ENTROPY_BWD = 10, /* args: logits, labels(i32) -> dlogits  ((softmax-onehot)/rows) */
  ZYXB_RR_SOFTMAX_BWD = 11,       /* args: p, dp -> ds = p*(dp - sum(dp*p)); with causal set, p is zero past the diagonal by
                                     construction, so those columns of p and dp are not read and ds is written as 0 there */
  ZYXB_RR_LAYERNORM_BWD = 12,     /* args: x, dy [,weight] -> dx */
  ZYXB_RR_COLSUM = 13,            /* args: x[rows,cols] -> y[cols]  (sum over rows; bias gradient) */
  ZYXB_RR_MSE = 14,               /* args: y, t -> loss[1] = mean((y-t)^2) over rows*cols */
  ZYXB_RR_LAYERNORM_DYXHAT = 15   /* args: x, dy -> dy * (x-mean)/sqrt(var+eps); its column sums are the layernorm weight gradient */
};

typedef struct {
  int32_t  op;          /* ZYXB_RR_* */
  int32_t  dtype;       /* element type of x / y */
  uint64_t rows, cols;
  float    eps;         /* layernorm */
  int32_t  correction;  /* var/std: divisor = cols - correction (zyx default 1) */
  int32_t  has_weight, has_bias;  /* layernorm affine */
  float    scale;       /* softmax: x is multiplied by scale first; 0 means 1 */
  int32_t  causal;      /* softmax, softmax backward: column j of row r is masked (-inf; never read) when j > r % period */
  uint64_t period;      /* sequence length T for the causal mask */
} zyxb_rowreduce_desc;

/* Matmul: Tensor::dot (zyx/src/tensor/mod.rs:1469-1490), Linear::forward
 * (zyx-nn/src/linear.rs:39-45), matched the way Graph::match_matmul does
 * (zyx/src/vendor/matmul.rs:43-71), launched like cblas_sgemm in backend/cblas.rs:241-271.
 * C[b] = epilogue(alpha * op(A[b]) . op(B[b]) [+ bias]) */
enum { ZYXB_EPI_NONE = 0, ZYXB_EPI_BIAS = 1, ZYXB_EPI_BIAS_RELU = 2, ZYXB_EPI_BIAS_GELU = 3,
       /* backward through an activation fused into the input-gradient matmul: C = (alpha * A.B) * act'(z),
        * z [m,n] being the activation's stored input (GELU) or output (ReLU: relu'(z) = z > 0 either way) */
       ZYXB_EPI_MUL_RELU_GRAD = 4, ZYXB_EPI_MUL_GELU_GRAD = 5,
       /* C = alpha * A.B + z, z shaped and strided like C (a residual / gradient accumulation) */
       ZYXB_EPI_ADD = 6 };

/* Causal (lower-triangular) structure a matcher may declare when an operand or the result is known to be
 * masked_fill(tril(..) == 0, ..) (zyx-nn/src/multi_head_attention.rs:208-211).  Declaring it never changes a value that
 * is defined; it lets the kernel skip work:
 *   OUT_LOWER  m == n; entries of C above the diagonal (col > row) are not needed: tiles wholly above it are neither
 *              computed nor written, their memory keeps whatever it held (scores = q.k^T, dP = dO.v^T)
 *   A_LOWER    m == k; the stored A [m,k] is zero above its diagonal: the sum over k stops at the row (P.v, dS.k)
 *   AT_LOWER   m == k, trans_a; the stored A [k,m] is zero above its diagonal, so column m of it starts at row m: the sum
 *              over k starts there (dV = P^T.dO, dK = dS^T.q) */
enum { ZYXB_TRI_NONE = 0, ZYXB_TRI_OUT_LOWER = 1, ZYXB_TRI_A_LOWER = 2, ZYXB_TRI_AT_LOWER = 3 };

typedef struct {
  int32_t  dtype;        /* element type of A, B, C: bf16 / f16 / f32 / i32; accumulation is
                            f32 (i32 for integers), as reduce_acc_dtype (reduce_ops.rs:52-60) */
  uint64_t m, n, k;
  uint64_t batch;        /* >= 1 */
  int32_t  trans_a;      /* 0: A stored [m,k] row-major; 1: A stored [k,m] */
  int32_t  trans_b;      /* 0: B stored [k,n] row-major; 1: B stored [n,k] (a Linear weight) */
  int64_t  stride_a, stride_b, stride_c;  /* batch strides in elements; 0 for A/B = shared */
  int32_t  epilogue;     /* ZYXB_EPI_*; bias is [n] */
  int32_t  store_preact; /* 1: second output receives alpha*A.B+bias before the activation */
  float    alpha;        /* 0 means 1 */
  /* Strided views, so that the [B, T, H, D] <-> [B, H, T, D] reshapes and transposes of attention
   * (zyx-nn/src/multi_head_attention.rs:160-226) need no copy: */
  uint64_t lda, ldb, ldc;   /* row pitch of the stored A / B / C in elements; 0 = packed (the contiguous extent) */
  uint64_t batch_inner;     /* 0 or 1: none.  Otherwise the launch runs batch * batch_inner matrices; matrix
                               z uses offset (z / batch_inner) * stride_x + (z % batch_inner) * stride_x_inner */
  int64_t  stride_a_inner, stride_b_inner, stride_c_inner;
  int32_t  tri;             /* ZYXB_TRI_*: causal structure of square attention operands, per matrix of the batch */
} zyxb_gemm_desc;
/* args: a, b [,bias | ,z] -> c [,preact] */

/* Elementwise kernels (zyx/src/tensor/elementwise.rs:157-170,289-293,585-588 and the
 * adjoints of zyx/src/graph/autograd.rs:47-175). */
enum {
  ZYXB_EW_RELU = 0,       /* x -> (x>0)*x */
  ZYXB_EW_GELU = 1,       /* x -> gelu(x), tanh built from exp as the reference does */
  ZYXB_EW_ADD = 2,        /* a, b -> a+b */
  ZYXB_EW_SUB = 3,        /* a, b -> a-b */
  ZYXB_EW_MUL = 4,        /* a, b -> a*b */
  ZYXB_EW_SCALE = 5,      /* x -> x*p0 */
  ZYXB_EW_RELU_BWD = 6,   /* dy, z -> dy*(z>0) */
  ZYXB_EW_GELU_BWD = 7,   /* dy, z -> dy*gelu'(z) */
  ZYXB_EW_MSE_BWD = 8,    /* y, t -> 2*(y-t)*p0   (p0 = 1/numel) */
  ZYXB_EW_CAST = 9,       /* x(dtype) -> y(dtype_out) */
  ZYXB_EW_TANH = 10, ZYXB_EW_SIGMOID = 11, ZYXB_EW_EXP = 12,
  ZYXB_EW_BIAS_ADD = 13   /* x[rows,cols], b[cols] -> x+b  (cols = p_cols) */
};

typedef struct {
  int32_t  op;        /* ZYXB_EW_* */
  int32_t  dtype;     /* element type of the inputs */
  int32_t  dtype_out; /* CAST only; otherwise ignored */
  uint64_t numel;
  uint64_t cols;      /* BIAS_ADD: inner extent */
  float    p0;
} zyxb_eltwise_desc;

/* Optimizer update fused into one pass over all parameter tensors:
 * SGD::update (zyx-optim/src/sgd.rs:45-84), Adam::update (zyx-optim/src/adam.rs:51-98),
 * AdamW::update (zyx-optim/src/adamw.rs:51-97).  The arithmetic is the reference's,
 * literally (AdamW divides the step by lr, adamw.rs:88-89) unless `standard` is set. */
enum { ZYXB_OPT_SGD = 0, ZYXB_OPT_ADAM = 1, ZYXB_OPT_ADAMW = 2 };

typedef struct {
  int32_t  algo;          /* ZYXB_OPT_* */
  int32_t  dtype;         /* element type of params, grads and state */
  int32_t  n_tensors;
  const uint64_t* numel;  /* [n_tensors]; copied at program creation */
  float    lr, weight_decay;
  float    momentum, dampening; int32_t nesterov, maximize;   /* SGD */
  float    beta1, beta2, eps;                                 /* Adam(W) */
  float    grad_scale;    /* gradients are multiplied by this first (1/world for data
                             parallel averaging); 0 means 1 */
  int32_t  standard;      /* AdamW only: 1 = textbook p -= lr*mh/(sqrt(vh)+eps) */
} zyxb_optim_desc;
/* args (all updated in place): SGD  p[0..n), g[0..n) [, buf[0..n) when momentum != 0]
 *                              Adam p[0..n), g[0..n), m[0..n), v[0..n)
 * The step counter t starts at 0 and is incremented by every launch (AdamW::t). */

/* Fused scaled-dot-product self-attention (forward), the subgraph of MultiheadAttention::forward between the
 * projections (zyx-nn/src/multi_head_attention.rs:197-226): o = softmax(scale * q.k^T [masked above the diagonal]) . v
 * per (batch, head), computed tile by tile without materialising the [seq, seq] scores.  q, k, v, o are [batch, seq,
 * heads*head_dim] activations read and written in place (head h of row t starts at t*ld + h*head_dim).  The second output
 * lse [batch*heads, seq] f32 is ln(sum_j exp(scale * s_ij)) per query, which a backward pass needs.
 * Scores and probabilities are never rounded to the tensor dtype (the reference rounds both where it stores them). */
typedef struct {
  int32_t  dtype;        /* bf16 / f16 */
  uint64_t batch, heads, seq;
  uint64_t head_dim;     /* 128 */
  uint64_t ld;           /* row pitch of q, k, v, o in elements; 0 = heads*head_dim */
  float    scale;        /* 0 means 1/sqrt(head_dim) */
  int32_t  causal;
} zyxb_attention_desc;
/* ZYXB_KIND_ATTENTION      args: q, k, v -> o, lse
 * ZYXB_KIND_ATTENTION_BWD  args: q, k, v, o, do, lse -> dq, dk, dv   (the adjoint; the same descriptor as the forward;
 *                          probabilities are recomputed from lse tile by tile, nothing of size [seq, seq] is stored) */

/* 2-D convolution (forward) with groups = 1, Tensor::conv (zyx/src/tensor/mod.rs:2583-2680) as Conv2d::forward calls it
 * (zyx-nn/src/conv2d.rs:58-68):
 *   y[n,o,i,j] = bias[o] + sum over (c, r, s) of  x[n, c, i*stride_h + r*dil_h - pad_top, j*stride_w + s*dil_w - pad_left] * w[o,c,r,s]
 * x [n,c,h,w], w [o,c,kh,kw], bias [o], y [n,o,oh,ow], dense, in the reference's own (channels-first) layout; positions
 * outside x read 0 (rpad_zeros, mod.rs:2647); oh = (h + pad_top + pad_bottom - dil_h*(kh-1) - 1) / stride_h + 1, ow alike.
 * The sum runs over c, then r, then s (the order of the reference's sum_keepdim axes); products of bf16 / f16 inputs are
 * exact in f32 and accumulate in f32 (i32 for integers); sum + bias is rounded to the tensor dtype once, when stored.
 * bf16 / f16 launches with enough work run as an implicit GEMM on the tensor cores: TMA reads, per filter tap, a box
 * of [output rows x output columns x 64 channels] at the tap's offset (the element strides of the tensor map carry the
 * convolution stride, out-of-range coordinates read the zero padding), so no im2col matrix exists anywhere. */
typedef struct {
  int32_t  dtype;        /* bf16 / f16 / f32 / i32 */
  uint64_t n, c, h, w;
  uint64_t o, kh, kw;
  uint32_t stride_h, stride_w, dil_h, dil_w;                 /* 0 means 1 */
  uint32_t pad_top, pad_bottom, pad_left, pad_right;
  int32_t  has_bias;
  int32_t  channels_last;  /* 1: x is [n,h,w,c] and y is [n,oh,ow,o] (w stays [o,c,kh,kw]): chained convolutions skip the
                              layout pass, TMA reads x in place (needs c % 8 == 0 for the tensor-core path) */
  int32_t  flip_filter;    /* 1: the input gradient of a stride-1 convolution F (filter [O,C,kh,kw], padding p, dilation d).  x is
                              dy of F (so this descriptor's c = O), this descriptor's o = C, w is F's filter buffer unchanged,
                              read as w'[o][c][r][s] = w[c][o][kh-1-r][kw-1-s]; the caller sets padding to d*(k-1) - p per
                              side (bottom / right: d*(k-1) - p_bottom / p_right) and dilation to d.  dx = this convolution. */
} zyxb_conv_desc;
/* ZYXB_KIND_CONV        args: x, w [,bias] -> y
 * ZYXB_KIND_CONV_DGRAD  args: dy, w -> dx   the input gradient of the convolution the descriptor names (has_bias and flip_filter
 *                       ignored).  Stride 1 with padding <= dil*(k-1): runs as the flip_filter convolution of dy, tensor cores
 *                       included; other strides (bf16 / f16 with enough work): one stride-1 convolution of dy per residue
 *                       class of the input positions, each with the sub-filter of the taps that reach the class, on the
 *                       tensor cores as well; everything else: a direct kernel.
 * ZYXB_KIND_CONV_WGRAD  args: x, dy -> dw   the filter gradient of the convolution the descriptor names (has_bias and
 *                       flip_filter ignored): dw[o,c,r,s] = sum over (n,i,j) of dy[n,o,i,j] * x[n,c,i*stride_h+r*dil_h-pad_top, ...];
 *                       bf16 / f16 with enough work run per tap as a matmul over the output positions on the tensor cores
 *                       (dy by tiled TMA, x by im2col-mode TMA, positions split over CTAs, f32 partials added in a fixed order) */

typedef struct {
  int32_t kind;  /* ZYXB_KIND_* */
  union {
    zyxb_rowreduce_desc rowreduce;
    zyxb_gemm_desc      gemm;
    zyxb_eltwise_desc   eltwise;
    zyxb_optim_desc     optim;
    zyxb_attention_desc attention;   /* both attention kinds */
    zyxb_conv_desc      conv;
  } u;
} zyxb_kernel_desc;

/* ---- context ------------------------------------------------------------------------
 * initialize_device (zyx/src/backend/cuda.rs:321-326, backend/cblas.rs:125-130) and
 * MemoryPool/Device::deinitialize (zyx/src/backend/mod.rs:558,822). */
int32_t zyxb_init(const zyxb_config* config, zyxb_ctx** out_ctx);
int32_t zyxb_shutdown(zyxb_ctx* ctx);
/* BackendError::context of the last failing call on this context (error.rs:107-111).
 * With ctx == NULL: the text of the last failing zyxb_init. */
const char* zyxb_last_error(zyxb_ctx* ctx);

/* Device::info (mod.rs:839), Device::free_compute (mod.rs:875) */
int32_t zyxb_device_count(zyxb_ctx* ctx, int32_t* out_count);
int32_t zyxb_device_info(zyxb_ctx* ctx, int32_t dev, zyxb_devinfo* out_info);
int32_t zyxb_free_compute(zyxb_ctx* ctx, int32_t dev, uint64_t* out_flops);

/* ---- memory pool ---------------------------------------------------------------------
 * MemoryPool::{free_bytes, allocate, deallocate, host_to_pool, pool_to_host,
 * pool_to_pool, sync_events, release_events, store_variable, get_variable}
 * (zyx/src/backend/mod.rs:581-803). */
int32_t zyxb_free_bytes(zyxb_ctx* ctx, int32_t dev, uint64_t* out_bytes);
int32_t zyxb_alloc(zyxb_ctx* ctx, int32_t dev, uint64_t bytes, uint32_t* out_buf, zyxb_event* out_event);
/* waits for the events (consumed), then frees */
int32_t zyxb_free(zyxb_ctx* ctx, int32_t dev, uint32_t buf, const zyxb_event* wait, int32_t n_wait);
/* asynchronous: src must stay valid until out_event has been synced (runtime.rs:1-16).  The copy runs on its own
 * stream: with a non-empty wait list it depends on those events only (so it can overlap kernels already queued);
 * with an empty one it is ordered after everything queued so far. */
int32_t zyxb_h2d(zyxb_ctx* ctx, int32_t dev, const void* src, uint64_t bytes, uint32_t dst, uint64_t dst_offset,
                 const zyxb_event* wait, int32_t n_wait, zyxb_event* out_event);
/* blocking */
int32_t zyxb_d2h(zyxb_ctx* ctx, int32_t dev, uint32_t src, uint64_t src_offset, void* dst, uint64_t bytes,
                 const zyxb_event* wait, int32_t n_wait);
/* device-to-device copy inside one pool, or between the pools of two devices of this ctx */
int32_t zyxb_d2d(zyxb_ctx* ctx, int32_t src_dev, uint32_t src, uint64_t src_offset, int32_t dst_dev, uint32_t dst,
                 uint64_t dst_offset, uint64_t bytes, const zyxb_event* wait, int32_t n_wait, zyxb_event* out_event);
int32_t zyxb_memset(zyxb_ctx* ctx, int32_t dev, uint32_t buf, uint64_t offset, int32_t byte_value, uint64_t bytes);
int32_t zyxb_buffer_bytes(zyxb_ctx* ctx, int32_t dev, uint32_t buf, uint64_t* out_bytes);
/* A second id for the byte range [offset, offset+bytes) of `parent` (offset a multiple of 256).  Lets
 * every gradient live inside one contiguous bucket that a single collective can cover, the way the
 * plan's `Alias` instruction shares storage (zyx/src/graph/plan.rs:47-54).  Freeing a view releases
 * only the id; the parent must outlive its views. */
int32_t zyxb_buffer_view(zyxb_ctx* ctx, int32_t dev, uint32_t parent, uint64_t offset, uint64_t bytes, uint32_t* out_buf);
/* blocking; destroys the events */
int32_t zyxb_sync(zyxb_ctx* ctx, int32_t dev, const zyxb_event* events, int32_t n);
/* non-blocking destroy */
int32_t zyxb_release_events(zyxb_ctx* ctx, int32_t dev, const zyxb_event* events, int32_t n);
/* blocks until every queued operation of the device has finished */
int32_t zyxb_device_sync(zyxb_ctx* ctx, int32_t dev);
/* scalars kept by value: le_bytes holds the little-endian value of `dtype` (<= 8 bytes) */
int32_t zyxb_store_variable(zyxb_ctx* ctx, int32_t dev, int32_t dtype, const void* le_bytes, uint32_t* out_buf);
int32_t zyxb_get_variable(zyxb_ctx* ctx, int32_t dev, uint32_t buf, int32_t* out_dtype, void* out_le_bytes);
/* page-lock a caller-owned host range so h2d/d2h run at full PCIe/C2C speed */
int32_t zyxb_host_register(zyxb_ctx* ctx, void* ptr, uint64_t bytes);
int32_t zyxb_host_unregister(zyxb_ctx* ctx, void* ptr);

/* ---- programs -------------------------------------------------------------------------
 * Device::compile / launch / release (zyx/src/backend/mod.rs:899,974,936).  The device is
 * `aot_only` (mod.rs:892-894): programs come from descriptors, not from zyx IR. */
int32_t zyxb_program_create(zyxb_ctx* ctx, int32_t dev, const zyxb_kernel_desc* desc, uint32_t* out_prog);
int32_t zyxb_launch(zyxb_ctx* ctx, int32_t dev, uint32_t prog, const uint32_t* args, int32_t n_args,
                    const zyxb_event* wait, int32_t n_wait, zyxb_event* out_event);
int32_t zyxb_program_release(zyxb_ctx* ctx, int32_t dev, uint32_t prog);
/* optimizer programs: read / set the step counter t (AdamW::t, adamw.rs:57) */
int32_t zyxb_program_set_step(zyxb_ctx* ctx, int32_t dev, uint32_t prog, uint64_t t);
int32_t zyxb_program_get_step(zyxb_ctx* ctx, int32_t dev, uint32_t prog, uint64_t* out_t);
/* number of CUDA kernels this library has launched on the device since init */
int32_t zyxb_launch_count(zyxb_ctx* ctx, int32_t dev, uint64_t* out_count);
/* device-side status word written by kernels whose bounded waits ran out (0 = none);
 * reading it synchronises the device and clears it */
int32_t zyxb_device_status(zyxb_ctx* ctx, int32_t dev, uint32_t* out_status);

/* With zyxb_config.debug bit 2 every pool allocation is followed by at least 256 bytes of a fixed pattern (the reference
 * gives every buffer one spare trailing element, zyx/src/runtime.rs:622-625, backend/mod.rs:627).  This call waits for the
 * device and verifies the pattern of every live buffer: a kernel that wrote past the end of one is reported as
 * IncorrectKernelArg with the buffer's id in *out_bad_buffer and the distance in the error text.  It is the library's own
 * out-of-bounds check for machines on which no memory checker may run. */
int32_t zyxb_check_guards(zyxb_ctx* ctx, int32_t dev, uint32_t* out_bad_buffer);

/* Failure detection without a failure: launches one CTA that waits, through the kernels' own bounded wait, on a barrier
 * nothing will ever arrive on, with a limit of `limit_ns` (at most 100 ms) instead of the kernels' two seconds.  The wait gives
 * up, the kernel returns normally, *out_gave_up is 1 and the device status word carries bit 0x8000, so the next
 * zyxb_device_status reports ZYXB_ERR_KERNEL_SYNC (ErrorStatus::KernelSync, zyx/src/error.rs:151-152) and clears the word; the
 * context stays usable.  Blocks until the kernel has finished. */
int32_t zyxb_selftest_bounded_wait(zyxb_ctx* ctx, int32_t dev, uint64_t limit_ns, uint32_t* out_gave_up);

/* ---- captured launch sequences ---------------------------------------------------------------------------
 * FrozenTape::replay (zyx/src/tape.rs:204-288) re-runs a realised plan without rebuilding it; here the launches
 * issued between capture_begin and capture_end are recorded into a CUDA graph instead of being run, and
 * zyxb_graph_launch replays them with one submission (what makes a 10-launch, 40-microsecond training step
 * launch-latency free).  Inside a capture only zyxb_launch (without wait lists), zyxb_memset and the
 * host-runtime steps built from them are allowed: zyxb_alloc / free / h2d / d2h / d2d / sync / device_sync and a launch with a
 * wait list are refused with a message while a capture is open.  Buffers must stay allocated while the graph lives.  A
 * captured launch freezes its kernel parameters, so an optimizer program whose update depends on its step counter - SGD with
 * momentum (the first step initialises the buffer, sgd.rs:66-72), Adam and AdamW (bias corrections) - is refused inside a
 * capture: launch it after zyxb_graph_launch.  Plain SGD is captured; a captured launch does not advance the step counter. */
int32_t zyxb_capture_begin(zyxb_ctx* ctx, int32_t dev);
int32_t zyxb_capture_end(zyxb_ctx* ctx, int32_t dev, uint32_t* out_graph);
int32_t zyxb_graph_launch(zyxb_ctx* ctx, int32_t dev, uint32_t graph, const zyxb_event* wait, int32_t n_wait, zyxb_event* out_event);
int32_t zyxb_graph_release(zyxb_ctx* ctx, int32_t dev, uint32_t graph);

/* ---- column sums for callers that cannot allocate -------------------------------------------------------
 * No counterpart in the reference.  y[cols] = sum over rows of x[rows, cols] (what a ZYXB_RR_COLSUM program
 * computes: the bias gradient of a Linear layer), for callers that must not reach an allocator while they
 * run: a zyx plan being replayed inside a latency-critical serving loop, a host that has handed all device
 * memory to its own pool so that cudaMalloc would fail, or code running where cudaMalloc's implicit device
 * synchronisation is not acceptable.  The partial sums go to a fixed array inside the loaded library
 * (1 Mi floats = 4 MiB per GPU, resident once the CUDA module that holds it has been loaded on that GPU - with
 * CUDA's lazy module loading that can be as late as the first call, so make the first call during set-up - until
 * the process exits) instead of the context's scratch buffer, and the call itself performs no cudaMalloc / cudaFree and
 * calls no allocating library routine; x and y are existing pool buffers.
 *   - limit: cols <= 1 048 576 (zyxb_colsum_static_capacity); larger shapes are refused with
 *     IncorrectKernelArg and a message naming the limit — use a ZYXB_RR_COLSUM program for those;
 *   - the first call on a device looks up the array's device address (cudaGetSymbolAddress) and caches it:
 *     make that first call during set-up, before any stream capture begins;
 *   - every call on a device shares the one array, which keeps the previous call's partials; each call
 *     overwrites all the partials it reads, so nothing needs clearing, but calls that overlap on the GPU
 *     race — issue them one after another (they are queued in order on the device's compute stream);
 *   - dtype f32 / bf16 / f16; runs in order on the compute stream like zyxb_launch, no wait list, no event. */
int32_t zyxb_colsum_static(zyxb_ctx* ctx, int32_t dev, int32_t dtype, uint32_t x, uint32_t y, uint64_t rows, uint64_t cols);
int32_t zyxb_colsum_static_capacity(uint64_t* out_floats);

/* ---- timing (the ZYX_DEBUG perf print, zyx/src/runtime.rs:1798-1838) ---- */
int32_t zyxb_event_record(zyxb_ctx* ctx, int32_t dev, zyxb_event* out_event);
int32_t zyxb_event_elapsed_ms(zyxb_ctx* ctx, int32_t dev, zyxb_event start, zyxb_event stop, float* out_ms);
/* overwrite a scratch buffer larger than L2 so the next kernel starts from cold caches */
int32_t zyxb_flush_l2(zyxb_ctx* ctx, int32_t dev);

/* ---- data-parallel gradient exchange (no counterpart in the reference, which has no
 * collectives: README.md:233 "manual"); one process per GPU, NCCL over NVLink ---- */
int32_t zyxb_comm_unique_id(zyxb_ctx* ctx, void* out_id_128_bytes);
int32_t zyxb_comm_init(zyxb_ctx* ctx, int32_t dev, int32_t rank, int32_t world, const void* id_128_bytes);
int32_t zyxb_allreduce_sum(zyxb_ctx* ctx, int32_t dev, uint32_t buf, uint64_t offset_elems, uint64_t count, int32_t dtype,
                           const zyxb_event* wait, int32_t n_wait, zyxb_event* out_event);
/* The two halves of an allreduce, for an optimizer whose state is sharded over the ranks (ZeRO stage 1).  Both work in
 * place on `world` consecutive slices of count_per_rank elements starting at offset_elems: after reduce_scatter_sum
 * slice `rank` holds the sum over ranks (the other slices are unspecified); allgather sends this rank's slice and
 * leaves all `world` slices filled.  Same stream and event rules as zyxb_allreduce_sum. */
/* Per-device communicator options.  ZYXB_COMM_OPT_LATENCY = 1: the zyxb_allreduce_sum calls that follow sit at the end of a
 * step with nothing left to hide behind; they take the communicator's own allreduce (NCCL: few, large messages reduced by its
 * kernels, in the switch where the fabric offers it) even where the copy-engine exchange over peer memory is available.  That
 * exchange is the choice for calls that overlap compute, because it takes no SM, but each call is three flag rounds among
 * all ranks around two copy phases.  0 (the default) = back to that choice.  Every rank makes the same setting for the same call. */
enum { ZYXB_COMM_OPT_LATENCY = 1 };
int32_t zyxb_comm_option(zyxb_ctx* ctx, int32_t dev, int32_t option, int32_t value);
int32_t zyxb_reduce_scatter_sum(zyxb_ctx* ctx, int32_t dev, uint32_t buf, uint64_t offset_elems, uint64_t count_per_rank, int32_t dtype,
                                const zyxb_event* wait, int32_t n_wait, zyxb_event* out_event);
int32_t zyxb_allgather(zyxb_ctx* ctx, int32_t dev, uint32_t buf, uint64_t offset_elems, uint64_t count_per_rank, int32_t dtype,
                       const zyxb_event* wait, int32_t n_wait, zyxb_event* out_event);
int32_t zyxb_comm_rank(zyxb_ctx* ctx, int32_t dev, int32_t* out_rank, int32_t* out_world);
int32_t zyxb_comm_destroy(zyxb_ctx* ctx, int32_t dev);

#ifdef __cplusplus
}
#endif
#endif /* ZYXB_H */
