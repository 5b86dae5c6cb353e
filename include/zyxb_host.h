/*
 * zyxb_host.h — host-side runtime above the C ABI of zyxb.h (libzyxb_host.so).
 *
 * The reference's host side is Rust: `Tape::gradient` builds the backward graph, `optim.update`
 * appends the optimizer expressions, `Tape::realize` compiles an `ExecPlan` once and replays its
 * `Launch` nodes every iteration (zyx/src/tape.rs:117-202, zyx/src/graph/plan.rs:271-361).  With no
 * Rust toolchain available the same plan is built here in C++ for the one model family the
 * configurations use — a stack of zyx_nn::Linear layers with an activation between them — and
 * replayed through nothing but zyxb.h calls, so what the library sees is the call sequence zyx
 * would produce.  Parameter, gradient and optimizer-state order is `Module::iter()` order: per
 * Linear `weight` then `bias` (zyx-nn/src/linear.rs:11-16, zyx-derive/src/lib.rs:75-106).
 */
#ifndef ZYXB_HOST_H
#define ZYXB_HOST_H

#include "zyxb.h"

#ifdef __cplusplus
extern "C" {
#endif

enum { ZYXB_ACT_NONE = 0, ZYXB_ACT_RELU = 1, ZYXB_ACT_GELU = 2 };
enum { ZYXB_LOSS_MSE = 0,            /* mean((y - target)^2), target [batch, dims[n]] of `dtype` (README loop, README.md:144-150) */
       ZYXB_LOSS_CROSS_ENTROPY = 1   /* Tensor::cross_entropy(.., ReduceOp::Mean), target [batch] i32 class indices, f32 only */ };

typedef struct {
  int32_t  dtype;            /* ZYXB_F32 / ZYXB_BF16 / ZYXB_F16: parameters, activations, gradients, optimizer state */
  uint64_t batch;            /* rows per step on this rank */
  int32_t  n_layers;         /* 1..8 Linear layers */
  uint64_t dims[9];          /* dims[0] = input features, dims[i+1] = out_features of layer i */
  int32_t  activation;       /* between layers (not after the last) */
  int32_t  loss;
  zyxb_optim_desc optim;     /* algo and hyper-parameters; dtype, n_tensors and numel are filled in */
  int32_t  world;            /* data-parallel ranks; > 1: gradients are all-reduced (needs zyxb_comm_init) and
                                optim.grad_scale is set to 1/world */
  int32_t  bucket_per_layer; /* 1: one allreduce per layer as soon as its gradients are queued (overlaps the rest of
                                the backward pass); 0: one allreduce over the whole gradient bucket */
  int32_t  shard_optimizer;  /* 1 (needs a communicator, any world >= 1, and bucket_per_layer): ZeRO stage 1.  Parameters live in
                                one bucket laid out like the gradients'; each layer's slice is cut into `world` shards;
                                gradients are reduce-scattered, this rank updates its shard (optimizer state of shard size
                                only: 1/world of the memory and of the update's HBM traffic), and the parameters are
                                all-gathered, first layer first, behind the next step's forward pass.  zyxb_mlp_tensor then
                                has no optimizer-state buffers, and a checkpoint holds this rank's state shards. */
} zyxb_mlp_config;

typedef struct zyxb_mlp zyxb_mlp;

/* Allocates parameters, gradients (one contiguous bucket), optimizer state and activations, and creates
 * every program of the step once — the analogue of compile_graph + ExecPlan::new (graph/mod.rs:1508-1581). */
int32_t zyxb_mlp_create(zyxb_ctx* ctx, int32_t dev, const zyxb_mlp_config* config, zyxb_mlp** out);
int32_t zyxb_mlp_destroy(zyxb_mlp* mlp);
const char* zyxb_mlp_last_error(zyxb_mlp* mlp);

/* Buffers, in Module::iter() order (index i = 2*layer + {0: weight [out,in], 1: bias [out]}).
 * which: 0 parameter, 1 gradient, 2 first optimizer state (SGD momentum buffer / Adam m), 3 second (Adam v). */
int32_t zyxb_mlp_tensor(zyxb_mlp* mlp, int32_t which, int32_t i, uint32_t* out_buf, uint64_t* out_numel);
/* Input [batch, dims[0]], target, loss [1] f32, output of the last layer [batch, dims[n]]. */
int32_t zyxb_mlp_io(zyxb_mlp* mlp, uint32_t* out_x, uint32_t* out_target, uint32_t* out_loss, uint32_t* out_y);

/* Tensors the plan stores between forward and backward, all [batch, dims[layer+1]], for parity checks at full size:
 * which 0 = the layer's output (after the activation; the network output for the last layer), 1 = its pre-activation
 * (stored only under GELU, and not for the last layer), 2 = the gradient of the loss w.r.t. its pre-activation. */
int32_t zyxb_mlp_activation(zyxb_mlp* mlp, int32_t which, int32_t layer, uint32_t* out_buf, uint64_t* out_numel);

/* forward + loss + backward (+ gradient allreduce): the Launch nodes up to the gradients */
int32_t zyxb_mlp_forward_backward(zyxb_mlp* mlp);
/* the optimizer update (SGD::update / AdamW::update) */
int32_t zyxb_mlp_update(zyxb_mlp* mlp);
/* one training step = forward_backward + update; `wait` are consumed (e.g. the h2d events of this step's batch) */
int32_t zyxb_mlp_step(zyxb_mlp* mlp, const zyxb_event* wait, int32_t n_wait);
/* the same, and an event that completes when the step's last launch has finished */
int32_t zyxb_mlp_step_event(zyxb_mlp* mlp, const zyxb_event* wait, int32_t n_wait, zyxb_event* out_event);
/* Rebind the plan to caller-owned input / target buffers (e.g. to alternate two sets so that the upload of the
 * next batch overlaps this step); the buffers the plan allocated stay owned by it. */
int32_t zyxb_mlp_bind_inputs(zyxb_mlp* mlp, uint32_t x, uint32_t target);
/* Per-instruction timing: while enabled, zyxb_mlp_step records an event after every instruction of the plan.
 * profile_read sums, over the steps recorded since the last read, the time between consecutive events (ms) per
 * instruction, and reports what each instruction is: -1 for a collective, else 100*ZYXB_KIND_* + sub, where sub is
 * 2*trans_a + trans_b for a matmul, the op for row / elementwise programs and the algorithm for the optimizer. */
int32_t zyxb_mlp_profile(zyxb_mlp* mlp, int32_t enable);
int32_t zyxb_mlp_profile_read(zyxb_mlp* mlp, float* out_ms, int32_t* out_kind, int32_t capacity, int32_t* out_n, int32_t* out_steps);
/* number of zyxb_launch / zyxb_allreduce_sum calls one step makes */
int32_t zyxb_mlp_plan_size(zyxb_mlp* mlp, int32_t* out_launches, int32_t* out_collectives);

/* ------------------------------------------------------------------------------------------------------------
 * One transformer block, forward + backward + optimizer, as the reference's README example composes it
 * (zyx-examples/examples/readme_test.rs:9-40): y = norm2(x1 + mlp2(gelu(mlp(x1)))), x1 = norm1(x + attn(x, x, x)),
 * attn = zyx_nn::MultiheadAttention (zyx-nn/src/multi_head_attention.rs:134-245: q/k/v/out projections with bias,
 * scores = q.k^T / sqrt(head_dim), optional causal mask, softmax, .v), LayerNorm with weight and bias and unbiased
 * variance (zyx-nn/src/layer_norm.rs:95-135).  Loss: mean((y - target)^2).
 * Parameters in Module::iter() order (16 tensors): attn.q_proj.{weight,bias}, k_proj, v_proj, out_proj,
 * mlp.{weight,bias}, mlp2.{weight,bias}, norm1.{weight,bias}, norm2.{weight,bias}. */
typedef struct {
  int32_t  dtype;        /* ZYXB_BF16 / ZYXB_F16 / ZYXB_F32 */
  uint64_t batch, seq;   /* this rank's input is [batch, seq, dim] */
  uint64_t dim, heads, ffn;
  int32_t  causal;       /* 1: key j is masked for query i when j > i */
  float    eps;          /* LayerNorm epsilon (1e-5 in the example) */
  zyxb_optim_desc optim; /* algo and hyper-parameters; dtype, n_tensors, numel are filled in */
  int32_t  world;        /* > 1: gradients are all-reduced in three groups (ffn, attention output side, q/k/v) */
  int32_t  fused_attention; /* 1: scores, softmax and probabilities.v (and their adjoints) run as the fused attention
                               programs where the shape allows (16-bit dtype, head_dim 128, seq a multiple of 128); the
                               [batch*heads, seq, seq] tensors are then not allocated and activation 0 does not exist */
  int32_t  shard_optimizer; /* 1 (needs a communicator of `world` ranks): ZeRO stage 1 as in zyxb_mlp_config - parameters in
                               one bucket laid out like the gradients', each of the three groups reduce-scattered, updated by
                               shard with optimizer state of shard size only, and all-gathered, the q/k/v group first */
} zyxb_block_config;

typedef struct zyxb_block zyxb_block;
int32_t zyxb_block_create(zyxb_ctx* ctx, int32_t dev, const zyxb_block_config* config, zyxb_block** out);
int32_t zyxb_block_destroy(zyxb_block* blk);
const char* zyxb_block_last_error(zyxb_block* blk);
/* which: 0 parameter, 1 gradient, 2 / 3 optimizer state; i in Module::iter() order.  With shard_optimizer the state has no
 * per-tensor buffers (IncorrectKernelArg for which >= 2), and the call first waits for parameter all-gathers still in flight. */
int32_t zyxb_block_tensor(zyxb_block* blk, int32_t which, int32_t i, uint32_t* out_buf, uint64_t* out_numel);
int32_t zyxb_block_io(zyxb_block* blk, uint32_t* out_x, uint32_t* out_target, uint32_t* out_loss, uint32_t* out_y);
int32_t zyxb_block_forward_backward(zyxb_block* blk);
int32_t zyxb_block_update(zyxb_block* blk);
int32_t zyxb_block_step(zyxb_block* blk, const zyxb_event* wait, int32_t n_wait);
int32_t zyxb_block_plan_size(zyxb_block* blk, int32_t* out_launches, int32_t* out_collectives);
/* intermediate tensors for tests (rows = batch*seq): 0 attention probabilities [batch*heads, seq, seq] (absent when fused),
 * 1 attention output [rows, dim], 2 x1 (after norm1), 3 q, 4 k, 5 v, 6 o (output projection), 7 s1 = x + o,
 * 8 z1 (feed-forward pre-activation) [rows, ffn], 9 h = gelu(z1) [rows, ffn], 10 m (second feed-forward output), 11 s2 = x1 + m;
 * gradients: 12 dy, 13 ds2, 14 dz1 [rows, ffn], 15 dx1, 16 ds1, 17 dattn, 18 dq, 19 dk, 20 dv */
int32_t zyxb_block_activation(zyxb_block* blk, int32_t which, uint32_t* out_buf);

/* ---- safetensors files: parameters, optimizer state and parity fixtures on disk -------------------------
 * The writer restates Module::save (zyx/src/module.rs:36-63): an 8-byte little-endian header length, a JSON header
 * {"name":{"dtype":"BF16","shape":[..],"data_offsets":[begin,end]},...} without whitespace, keys in exactly that order,
 * then the tensors' little-endian bytes back to back in header order - the layout Tensor::load_safetensors
 * (module.rs:436-529) relies on (it scans the header's strings positionally and reads the data at a running offset).
 * The reader accepts that layout and any other valid safetensors file (a leading "__metadata__" object, keys in any
 * order, data in any order): it honours data_offsets and checks them against shape and dtype as the reference does.
 * dtype names are DType::safetensors (zyx/src/dtype.rs:227-243). */
typedef struct {
  const char* name;
  int32_t dtype;             /* ZYXB_* element type */
  int32_t rank;
  const uint64_t* shape;     /* [rank] */
  const void* data;          /* numel * element size bytes, host memory */
} zyxb_st_tensor;
typedef struct zyxb_st_file zyxb_st_file;
int32_t zyxb_st_save(const char* path, const zyxb_st_tensor* tensors, int32_t n);
int32_t zyxb_st_open(const char* path, zyxb_st_file** out);
int32_t zyxb_st_count(const zyxb_st_file* f);
/* the pointers stay valid until zyxb_st_close */
int32_t zyxb_st_info(const zyxb_st_file* f, int32_t i, const char** out_name, int32_t* out_dtype, int32_t* out_rank,
                     const uint64_t** out_shape, uint64_t* out_bytes);
int32_t zyxb_st_find(const zyxb_st_file* f, const char* name);   /* index, or -1 */
int32_t zyxb_st_read(zyxb_st_file* f, int32_t i, void* dst, uint64_t dst_bytes);
int32_t zyxb_st_close(zyxb_st_file* f);
const char* zyxb_st_last_error(void);   /* of the calling thread's last failed zyxb_st_* call */

/* Checkpoints of the plans: parameters ("<name>"), optimizer state ("optim.m.<name>", "optim.v.<name>" or
 * "optim.buf.<name>") and the step counter ("optim.t", one U64; a U32 is accepted when reading) in one safetensors file, names in Module::iter_tensors
 * order (e.g. "attn.q_proj.weight"; "layers.0.weight" for the Linear stack).  Loading a file written by zyx itself
 * works when its labels match; tensors absent from the file are left untouched and counted in *out_missing. */
int32_t zyxb_mlp_save(zyxb_mlp* mlp, const char* path);
int32_t zyxb_mlp_load(zyxb_mlp* mlp, const char* path, int32_t* out_missing);
int32_t zyxb_block_save(zyxb_block* blk, const char* path);
int32_t zyxb_block_load(zyxb_block* blk, const char* path, int32_t* out_missing);

/* ---- e-graph matcher: subgraph -> kernel descriptor ---------------------------------------------------------------
 * The device's `match_graph` hook (zyx/src/backend/mod.rs:952-961; the reference's model is CblasDevice::match_graph,
 * backend/cblas.rs:213-238, over Graph::match_matmul, vendor/matmul.rs:43-71) written over a mirror of zyx's graph, so that
 * it can be built and tested without a Rust toolchain.  A node constructor returns the id of the class that holds the node
 * (identical nodes share a class, as in the e-graph); 0xffffffff reports a bad argument.  Shapes are constants (symbolic
 * dimensions never match in the reference either).  dtype / uop / bop values are zyx's enum orders (dtype.rs:18-32,
 * kernel/ops.rs:187-214, 222-262: uop Neg 0, BitNot 1, Exp 2, Exp2 3, Ln 4, Log2 5, Reciprocal 6, Sqrt 7, ...; bop Add 0, Sub 1,
 * Mul 2, Div 3, Pow 4, Mod 5, Cmplt 6, Cmpgt 7, Cmpge 8, Max 9, ..., NotEq 17, Eq 18). */
typedef struct zyxb_mgraph zyxb_mgraph;
int32_t  zyxb_mgraph_create(zyxb_mgraph** out);
int32_t  zyxb_mgraph_destroy(zyxb_mgraph* g);
uint32_t zyxb_mgraph_const(zyxb_mgraph* g, int32_t dtype, double value);                                  /* Node::Const */
uint32_t zyxb_mgraph_leaf(zyxb_mgraph* g, int32_t dtype, uint32_t leaf_id, const uint64_t* shape, int32_t rank);   /* Node::Leaf */
uint32_t zyxb_mgraph_expand(zyxb_mgraph* g, uint32_t x, const uint64_t* shape, int32_t rank);             /* Node::Expand */
uint32_t zyxb_mgraph_reshape(zyxb_mgraph* g, uint32_t x, const uint64_t* shape, int32_t rank);            /* Node::Reshape */
uint32_t zyxb_mgraph_permute(zyxb_mgraph* g, uint32_t x, const int32_t* axes, int32_t rank);              /* Node::Permute */
uint32_t zyxb_mgraph_reduce(zyxb_mgraph* g, uint32_t x, int32_t rop, const int32_t* axes, int32_t n_axes); /* Node::Reduce */
/* Node::Pad: `lp` zeros in front of `axis` (negative: that many elements cut off), `len` = the axis' extent afterwards */
uint32_t zyxb_mgraph_pad(zyxb_mgraph* g, uint32_t x, int32_t axis, int64_t lp, uint64_t len);
uint32_t zyxb_mgraph_cast(zyxb_mgraph* g, uint32_t x, int32_t dtype);                                     /* Node::Cast */
uint32_t zyxb_mgraph_unary(zyxb_mgraph* g, uint32_t x, int32_t uop);                                      /* Node::Unary */
uint32_t zyxb_mgraph_binary(zyxb_mgraph* g, uint32_t x, uint32_t y, int32_t bop);                         /* Node::Binary */
/* dtype, rank, shape (up to 8 extents) of a class and how many Node::Kernel alternatives match_graph has pushed into it */
int32_t  zyxb_mgraph_class_info(zyxb_mgraph* g, uint32_t cls, int32_t* out_dtype, int32_t* out_rank, uint64_t* out_shape8, int32_t* out_kernel_nodes);

/* The value of a class that depends on no stored tensor (constants under movement ops, paddings, reductions, casts and
 * arithmetic - how Tensor::arange and one-hot masks are built, tensor/mod.rs:773-781, 1920-1946), row-major as doubles: the
 * constant folding the cross-entropy pattern uses to recognise its arange.  IncorrectKernelArg when the class reads a Leaf,
 * uses an op outside that set or has an intermediate of more than 2^22 elements.  *out_n = element count; at most `capacity`
 * values are written. */
int32_t  zyxb_mgraph_const_value(zyxb_mgraph* g, uint32_t cls, double* out, uint64_t capacity, uint64_t* out_n);

/* One recognised subgraph: what to hand to zyxb_program_create, and the classes whose buffers are the launch arguments
 * (inputs then outputs, the order Device::launch receives, backend/mod.rs:974).  Patterns: matmul_nn / matmul_nt / matmul_tn / matmul_tt
 * [_batched][_heads][_bias[_relu|_gelu] | _add], conv[_bias], attention, softmax, ln_softmax, layernorm, cross_entropy, mse_loss, sum, max, min, mean, var, std, colsum, sgd, sgd_momentum,
 * sgd_nesterov, adam, adam_first_step, adamw, adamw_first_step; and, for outputs of the graph and inputs of those programs that nothing
 * produces yet, the elementwise programs relu, gelu, tanh, sigmoid, exp, cast, scale, add, sub, mul, bias_add.  An optimizer match covers every parameter of the update (inputs p.., g.. [, m.., v.. |
 * , buf..]; outputs p' [, m', v' | , buf'] per tensor - the program updates where its arguments lie, so the shim's launch copies
 * p, m, v into the output buffers first and runs the program on p'.., g.., m'.., v'..); its desc.u.optim.numel points into the
 * graph mirror.  optim_step is the step t the matched update belongs to
 * (1 = the first: no state is read; for AdamW read back from the bias-correction constants, 2 for an SGD update that reads its
 * momentum buffer): the caller sets the program's counter to t - 1 (zyxb_program_set_step) before the launch.  0 for the
 * other patterns.  The attention program takes one more buffer behind its output, the log-sum-exp [batch*heads, seq] f32. */
typedef struct {
  char     pattern[32];
  int32_t  n_inputs, n_outputs;
  uint32_t inputs[128], outputs[96];
  zyxb_kernel_desc desc;
  uint64_t optim_step;
  uint64_t input_offsets[128];  /* per input: the element of that class's buffer the program's argument starts at (a matmul operand
                                   that is a slice of a stored tensor, e.g. q of a fused q/k/v projection); the caller passes
                                   zyxb_buffer_view(buffer, offset * element size, the rest) for a non-zero entry */
} zyxb_match;
/* match_graph over every class the `outputs` depend on.  Classes in `outputs` are the ones other consumers read: a new
 * parameter value is only matched as an optimizer update when it is one of them, and a GELU layer's pre-activation listed
 * there becomes the matmul program's second output.  Each match is also pushed into its output classes as a Node::Kernel
 * alternative (graph/mod.rs:177-182).  Returns the number of matches in *out_n (may exceed capacity). */
int32_t  zyxb_mgraph_match(zyxb_mgraph* g, const uint32_t* outputs, int32_t n_outputs, zyxb_match* out, int32_t capacity, int32_t* out_n);
/* What the programs matched so far do not cover: walking down from `outputs` through the Node::Kernel alternatives (the one
 * pushed last in each class), the classes that are needed but are neither stored tensors nor produced by a program.  *out_n = 0
 * means the device can execute the graph on its own. */
int32_t  zyxb_mgraph_uncovered(zyxb_mgraph* g, const uint32_t* outputs, int32_t n_outputs, uint32_t* out_classes, int32_t capacity, int32_t* out_n);

#ifdef __cplusplus
}
#endif
#endif /* ZYXB_HOST_H */
