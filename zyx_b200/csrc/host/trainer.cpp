// Host-side training plan for a stack of Linear layers, built once and replayed every step
// through the C ABI of zyxb.h only (see include/zyxb_host.h).
//
// What each part mirrors in the reference:
//   Linear          zyx-nn/src/linear.rs:8-45        weight [out, in], bias [out]; forward x.dot(W.t()) + b
//   Plan / Instr    zyx/src/graph/plan.rs:47-54      ExecPlan: Launch instructions replayed by execute_plan (271-361)
//   backward        zyx/src/graph/autograd.rs:47-175 adjoints of mul/add/relu/exp...; for dot, reshape, expand and sum the
//                                                    standard adjoints spelled out in autograd.rs:195-242, 269-379
//   SGD / AdamW     zyx-optim/src/sgd.rs:45-84, adamw.rs:51-97   one fused program over all parameters
// Gradients live in one contiguous bucket, last layer first, so that each layer's slice can be
// all-reduced as soon as its two gradient launches are queued.
// With shard_optimizer (ZeRO stage 1) the parameters live in a second bucket of the same layout; each layer's slice is
// cut into `world` shards: the gradients are reduce-scattered, every rank updates its shard with optimizer state of
// shard size only, and the updated parameters are all-gathered - layer 0 first, so that the next forward pass starts
// as soon as its first weight has arrived while the later layers' gathers run behind it.
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <stdlib.h>

#include <string>
#include <vector>

#include "../../../include/zyxb_host.h"
#include "checkpoint.hpp"

namespace {

struct Linear {
  uint64_t in_features = 0, out_features = 0;
  uint32_t weight = 0, bias = 0;          // parameters
  uint32_t weight_grad = 0, bias_grad = 0; // views into the gradient bucket
  uint32_t state[2][2] = {{0, 0}, {0, 0}}; // [m|v][weight|bias]
  uint64_t bucket_offset = 0, bucket_count = 0;  // this layer's slice of the bucket, in elements
  uint64_t shard = 0;                      // sharded optimizer: elements of the slice this rank updates
  uint32_t param_shard = 0, grad_shard = 0; // views of this rank's shard in the parameter / gradient bucket
};

struct Instr {
  enum Kind { LAUNCH, ALLREDUCE, REDUCE_SCATTER, ALLGATHER } kind = LAUNCH;
  uint32_t program = 0;
  std::vector<uint32_t> args;
  uint64_t offset = 0, count = 0;          // collectives: slice of the bucket (count per rank for the sliced ones)
  int layer = -1;                          // ALLGATHER: the layer whose parameters it completes; LAUNCH: wait for that layer's gather
  int wait_collectives = 0;                // LAUNCH: wait first for this many of the oldest pending gradient-collective events (-1: all)
  bool tail = false;                       // ALLREDUCE: nothing of the step is left to hide it behind (ZYXB_COMM_OPT_LATENCY around the call)
  int desc_kind = 0, desc_sub = 0;         // ZYXB_KIND_* and the op / layout, for profile reports
};

uint64_t dsize(int32_t dtype) { return dtype == ZYXB_F32 ? 4 : 2; }
uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

}  // namespace

struct zyxb_mlp {
  zyxb_ctx* ctx = nullptr;
  int32_t dev = 0;
  zyxb_mlp_config cfg{};
  std::vector<Linear> layers;
  uint32_t grad_bucket = 0, param_bucket = 0;
  uint64_t bucket_elems = 0;
  bool sharded = false;                    // optimizer state sharded over the ranks
  int rank = 0;
  std::vector<zyxb_event> param_ready;     // per layer: the event of its last parameter all-gather, if not yet waited for
  std::vector<char> param_ready_set;
  uint32_t x = 0, target = 0, loss = 0, per_sample = 0, y = 0;
  std::vector<uint32_t> act, preact, dact;     // per hidden layer output: A_i, Z_i (GELU only), dA_i
  uint32_t dy = 0;
  std::vector<uint32_t> owned_buffers, owned_programs;
  std::vector<Instr> forward_backward, update;
  int n_launches = 0, n_collectives = 0;
  std::vector<zyxb_event> pending;
  // profiling: one event before the first instruction and one after every instruction of a profiled step
  bool profiling = false;
  std::vector<std::vector<zyxb_event>> prof_steps;
  std::string err;
};

namespace {

#define TRY(call)                                                              \
  do {                                                                         \
    int32_t st_ = (call);                                                      \
    if (st_ != ZYXB_OK) {                                                      \
      M->err = std::string(#call) + ": " + zyxb_last_error(M->ctx);            \
      return st_;                                                              \
    }                                                                          \
  } while (0)

int32_t alloc(zyxb_mlp* M, uint64_t bytes, uint32_t* out, bool zero = false) {
  zyxb_event ev{};
  TRY(zyxb_alloc(M->ctx, M->dev, bytes, out, &ev));
  M->owned_buffers.push_back(*out);
  if (zero) TRY(zyxb_memset(M->ctx, M->dev, *out, 0, 0, bytes));
  return ZYXB_OK;
}

int32_t program(zyxb_mlp* M, const zyxb_kernel_desc& d, uint32_t* out) {
  TRY(zyxb_program_create(M->ctx, M->dev, &d, out));
  M->owned_programs.push_back(*out);
  return ZYXB_OK;
}

zyxb_kernel_desc gemm_desc(int32_t dtype, uint64_t m, uint64_t n, uint64_t k, bool ta, bool tb, int32_t epi, bool preact) {
  zyxb_kernel_desc d{};
  d.kind = ZYXB_KIND_GEMM;
  d.u.gemm.dtype = dtype; d.u.gemm.m = m; d.u.gemm.n = n; d.u.gemm.k = k; d.u.gemm.batch = 1;
  d.u.gemm.trans_a = ta; d.u.gemm.trans_b = tb; d.u.gemm.stride_a = (int64_t)(m * k); d.u.gemm.stride_b = (int64_t)(k * n);
  d.u.gemm.stride_c = (int64_t)(m * n); d.u.gemm.epilogue = epi; d.u.gemm.store_preact = preact; d.u.gemm.alpha = 1.0f;
  return d;
}
zyxb_kernel_desc row_desc(int32_t op, int32_t dtype, uint64_t rows, uint64_t cols) {
  zyxb_kernel_desc d{};
  d.kind = ZYXB_KIND_ROWREDUCE;
  d.u.rowreduce.op = op; d.u.rowreduce.dtype = dtype; d.u.rowreduce.rows = rows; d.u.rowreduce.cols = cols; d.u.rowreduce.correction = 1;
  return d;
}
zyxb_kernel_desc ew_desc(int32_t op, int32_t dtype, uint64_t numel, float p0) {
  zyxb_kernel_desc d{};
  d.kind = ZYXB_KIND_ELTWISE;
  d.u.eltwise.op = op; d.u.eltwise.dtype = dtype; d.u.eltwise.dtype_out = dtype; d.u.eltwise.numel = numel; d.u.eltwise.p0 = p0;
  return d;
}

int32_t push_launch(zyxb_mlp* M, std::vector<Instr>& plan, const zyxb_kernel_desc& d, std::vector<uint32_t> args, int wait_coll = 0) {
  Instr in;
  in.kind = Instr::LAUNCH; in.args = std::move(args); in.wait_collectives = wait_coll;
  in.desc_kind = d.kind;
  in.desc_sub = d.kind == ZYXB_KIND_GEMM ? (d.u.gemm.trans_a * 2 + d.u.gemm.trans_b)
              : d.kind == ZYXB_KIND_ROWREDUCE ? d.u.rowreduce.op : d.kind == ZYXB_KIND_ELTWISE ? d.u.eltwise.op : d.u.optim.algo;
  int32_t st = program(M, d, &in.program);
  if (st) return st;
  plan.push_back(std::move(in));
  M->n_launches++;
  return ZYXB_OK;
}

int32_t build(zyxb_mlp* M) {
  const zyxb_mlp_config& c = M->cfg;
  const int n = c.n_layers;
  const int32_t dt = c.dtype;
  const uint64_t es = dsize(dt), B = c.batch;

  // ---- parameters, gradient bucket (last layer first), optimizer state ----
  M->layers.resize(n);
  M->sharded = c.shard_optimizer != 0;
  int world = c.world;
  if (M->sharded) {
    if (!c.bucket_per_layer) { M->err = "shard_optimizer needs bucket_per_layer"; return ZYXB_ERR_INCORRECT_KERNEL_ARG; }
    int32_t r = 0, w = 1;
    TRY(zyxb_comm_rank(M->ctx, M->dev, &r, &w));
    if (w != c.world) { M->err = "shard_optimizer: config.world differs from the communicator's"; return ZYXB_ERR_INCORRECT_KERNEL_ARG; }
    M->rank = r;
  }
  const uint64_t align_elems = 256 / es;
  const uint64_t slice_align = M->sharded ? align_elems * (uint64_t)world : align_elems;   // a sharded slice divides into aligned shards
  uint64_t off = 0;
  for (int i = n - 1; i >= 0; --i) {
    Linear& L = M->layers[i];
    L.in_features = c.dims[i]; L.out_features = c.dims[i + 1];
    L.bucket_offset = off;
    off += align_up(align_up(L.in_features * L.out_features, align_elems) + align_up(L.out_features, align_elems), slice_align);
    L.bucket_count = off - L.bucket_offset;
    if (M->sharded) L.shard = L.bucket_count / (uint64_t)world;
  }
  M->bucket_elems = off;
  M->param_ready.assign(n, zyxb_event{}); M->param_ready_set.assign(n, 0);
  int32_t st;
  if ((st = alloc(M, M->bucket_elems * es, &M->grad_bucket, true))) return st;
  if (M->sharded && (st = alloc(M, M->bucket_elems * es, &M->param_bucket, true))) return st;
  const bool adam = c.optim.algo != ZYXB_OPT_SGD;
  const bool sgd_momentum = c.optim.algo == ZYXB_OPT_SGD && c.optim.momentum != 0.0f;
  const int n_state = adam ? 2 : (sgd_momentum ? 1 : 0);
  for (int i = 0; i < n; ++i) {
    Linear& L = M->layers[i];
    const uint64_t wn = L.in_features * L.out_features, bn = L.out_features;
    if (M->sharded) {
      // parameters are views into the parameter bucket (the same layout as the gradients'), state covers this rank's shard
      TRY(zyxb_buffer_view(M->ctx, M->dev, M->param_bucket, L.bucket_offset * es, wn * es, &L.weight));
      TRY(zyxb_buffer_view(M->ctx, M->dev, M->param_bucket, (L.bucket_offset + align_up(wn, align_elems)) * es, bn * es, &L.bias));
      const uint64_t shard_off = (L.bucket_offset + (uint64_t)M->rank * L.shard) * es;
      TRY(zyxb_buffer_view(M->ctx, M->dev, M->param_bucket, shard_off, L.shard * es, &L.param_shard));
      TRY(zyxb_buffer_view(M->ctx, M->dev, M->grad_bucket, shard_off, L.shard * es, &L.grad_shard));
      for (uint32_t v : {L.weight, L.bias, L.param_shard, L.grad_shard}) M->owned_buffers.push_back(v);
    } else if ((st = alloc(M, wn * es, &L.weight, true)) || (st = alloc(M, bn * es, &L.bias, true))) return st;
    TRY(zyxb_buffer_view(M->ctx, M->dev, M->grad_bucket, L.bucket_offset * es, wn * es, &L.weight_grad));
    TRY(zyxb_buffer_view(M->ctx, M->dev, M->grad_bucket, (L.bucket_offset + align_up(wn, align_elems)) * es, bn * es, &L.bias_grad));
    M->owned_buffers.push_back(L.weight_grad); M->owned_buffers.push_back(L.bias_grad);
    for (int s = 0; s < n_state; ++s) {
      if (M->sharded) { if ((st = alloc(M, L.shard * es, &L.state[s][0], true))) return st; }
      else if ((st = alloc(M, wn * es, &L.state[s][0], true)) || (st = alloc(M, bn * es, &L.state[s][1], true))) return st;
    }
  }

  // ---- activations ----
  if ((st = alloc(M, B * c.dims[0] * es, &M->x))) return st;
  const bool ce = c.loss == ZYXB_LOSS_CROSS_ENTROPY;
  if ((st = alloc(M, ce ? B * 4 : B * c.dims[n] * es, &M->target))) return st;
  if ((st = alloc(M, 4, &M->loss, true))) return st;
  if (ce && (st = alloc(M, B * 4, &M->per_sample))) return st;
  if ((st = alloc(M, B * c.dims[n] * es, &M->y)) || (st = alloc(M, B * c.dims[n] * es, &M->dy))) return st;
  M->act.assign(n, 0); M->preact.assign(n, 0); M->dact.assign(n, 0);
  for (int i = 0; i + 1 < n; ++i) {
    const uint64_t bytes = B * c.dims[i + 1] * es;
    if ((st = alloc(M, bytes, &M->act[i])) || (st = alloc(M, bytes, &M->dact[i]))) return st;
    if (c.activation == ZYXB_ACT_GELU && (st = alloc(M, bytes, &M->preact[i]))) return st;
  }

  // ---- forward: Linear::forward per layer, activation fused into the matmul epilogue ----
  std::vector<Instr>& P = M->forward_backward;
  for (int i = 0; i < n; ++i) {
    const Linear& L = M->layers[i];
    const bool last = i == n - 1;
    const uint32_t in = i == 0 ? M->x : M->act[i - 1];
    int32_t epi = ZYXB_EPI_BIAS;
    if (!last && c.activation == ZYXB_ACT_RELU) epi = ZYXB_EPI_BIAS_RELU;
    if (!last && c.activation == ZYXB_ACT_GELU) epi = ZYXB_EPI_BIAS_GELU;
    const bool keep_z = !last && c.activation == ZYXB_ACT_GELU;   // gelu' needs the pre-activation; relu' reads the output
    std::vector<uint32_t> args = {in, L.weight, L.bias, last ? M->y : M->act[i]};
    if (keep_z) args.push_back(M->preact[i]);
    if ((st = push_launch(M, P, gemm_desc(dt, B, L.out_features, L.in_features, false, true, epi, keep_z), args))) return st;
    if (M->sharded) P.back().layer = i;     // the first reader of this layer's gathered parameters
  }
  // ---- loss and its gradient ----
  const uint64_t out_f = c.dims[n];
  if (ce) {
    if ((st = push_launch(M, P, row_desc(ZYXB_RR_CROSS_ENTROPY, ZYXB_F32, B, out_f), {M->y, M->target, M->per_sample, M->loss}))) return st;
    if ((st = push_launch(M, P, row_desc(ZYXB_RR_CROSS_ENTROPY_BWD, ZYXB_F32, B, out_f), {M->y, M->target, M->dy}))) return st;
  } else {
    if ((st = push_launch(M, P, row_desc(ZYXB_RR_MSE, dt, B, out_f), {M->y, M->target, M->loss}))) return st;
    if ((st = push_launch(M, P, ew_desc(ZYXB_EW_MSE_BWD, dt, B * out_f, 1.0f / (float)(B * out_f)), {M->y, M->target, M->dy}))) return st;
  }
  // ---- backward, last layer first ----
  std::vector<int> collectives_of_layer(n, 1);
  // which of the first layer's collectives (the last of a step) take the communicator's low-latency path
  // (ZYXB_COMM_OPT_LATENCY): 0 none (default - measured at 2 and 8 GPUs it shortens the last optimizer launch's wait by
  // 0.1 - 0.25 ms and costs the matmuls as much), 1 the very last one, 2 both halves of a split first layer
  const int tail_collectives = getenv("ZYXB_TAIL_COLLECTIVES") ? atoi(getenv("ZYXB_TAIL_COLLECTIVES")) : 0;
  for (int i = n - 1; i >= 0; --i) {
    const Linear& L = M->layers[i];
    const uint32_t dz = i == n - 1 ? M->dy : M->dact[i];
    const uint32_t in = i == 0 ? M->x : M->act[i - 1];
    // dW = dZ^T . input   ([out, B] x [B, in]); db = column sums of dZ
    // The first layer's gradients are the last ones the backward pass produces, so their allreduce has nothing left to hide
    // behind but the optimizer launches of the other layers.  Its weight gradient is therefore produced in two halves (rows
    // [0, out/2) and [out/2, out) of dW: two column ranges of dZ, read in place through the row pitch), each followed by the
    // allreduce of its part of the bucket: the first half travels while the second is being multiplied.
    const bool data_parallel = !M->sharded && c.world > 1 && c.bucket_per_layer;
    const uint64_t wn = L.in_features * L.out_features, half_rows = L.out_features / 2;
    const bool split = data_parallel && i == 0 && n > 1 && wn >= (1ull << 24) && L.out_features % 256 == 0 && (half_rows * es) % 256 == 0 &&
                       (half_rows * L.in_features * es) % 256 == 0;
    if (split) {
      uint32_t dz_hi = 0, dw_lo = 0, dw_hi = 0;
      const uint64_t dz_bytes = B * L.out_features * es;
      TRY(zyxb_buffer_view(M->ctx, M->dev, dz, half_rows * es, dz_bytes - half_rows * es, &dz_hi));
      TRY(zyxb_buffer_view(M->ctx, M->dev, L.weight_grad, 0, half_rows * L.in_features * es, &dw_lo));
      TRY(zyxb_buffer_view(M->ctx, M->dev, L.weight_grad, half_rows * L.in_features * es, half_rows * L.in_features * es, &dw_hi));
      for (uint32_t v : {dz_hi, dw_lo, dw_hi}) M->owned_buffers.push_back(v);
      zyxb_kernel_desc hd = gemm_desc(dt, half_rows, L.in_features, B, true, false, ZYXB_EPI_NONE, false);
      hd.u.gemm.lda = L.out_features;                       // dZ is [B, out]: a half is a column range of every row
      if ((st = push_launch(M, P, hd, {dz, in, dw_lo}))) return st;
      Instr ar; ar.kind = Instr::ALLREDUCE; ar.offset = L.bucket_offset; ar.count = half_rows * L.in_features;
      ar.tail = tail_collectives >= 2;
      P.push_back(ar); M->n_collectives++;
      if ((st = push_launch(M, P, hd, {dz_hi, in, dw_hi}))) return st;
      if ((st = push_launch(M, P, row_desc(ZYXB_RR_COLSUM, dt, B, L.out_features), {dz, L.bias_grad}))) return st;
      ar.offset = L.bucket_offset + half_rows * L.in_features; ar.count = L.bucket_count - half_rows * L.in_features;
      ar.tail = tail_collectives >= 1;       // the step's last collective: only optimizer launches are left beside it
      P.push_back(ar); M->n_collectives++;
      collectives_of_layer[i] = 2;
    } else {
    if ((st = push_launch(M, P, gemm_desc(dt, L.out_features, L.in_features, B, true, false, ZYXB_EPI_NONE, false), {dz, in, L.weight_grad}))) return st;
    if ((st = push_launch(M, P, row_desc(ZYXB_RR_COLSUM, dt, B, L.out_features), {dz, L.bias_grad}))) return st;
    if (M->sharded) {
      Instr rs; rs.kind = Instr::REDUCE_SCATTER; rs.offset = L.bucket_offset; rs.count = L.shard;
      P.push_back(rs); M->n_collectives++;
    } else if (c.world > 1 && c.bucket_per_layer) {
      Instr ar; ar.kind = Instr::ALLREDUCE; ar.offset = L.bucket_offset; ar.count = L.bucket_count;
      ar.tail = i == 0 && n > 1 && tail_collectives >= 1;
      P.push_back(ar); M->n_collectives++;
    }
    }
    if (i > 0) {
      // dZ_prev = (dZ . W) * act'(z_prev)   ([B, out] x [out, in]); the activation's adjoint rides in the matmul epilogue
      if (c.activation == ZYXB_ACT_RELU) {
        if ((st = push_launch(M, P, gemm_desc(dt, B, L.in_features, L.out_features, false, false, ZYXB_EPI_MUL_RELU_GRAD, false),
                              {dz, L.weight, M->act[i - 1], M->dact[i - 1]}))) return st;
      } else if (c.activation == ZYXB_ACT_GELU) {
        if ((st = push_launch(M, P, gemm_desc(dt, B, L.in_features, L.out_features, false, false, ZYXB_EPI_MUL_GELU_GRAD, false),
                              {dz, L.weight, M->preact[i - 1], M->dact[i - 1]}))) return st;
      } else {
        if ((st = push_launch(M, P, gemm_desc(dt, B, L.in_features, L.out_features, false, false, ZYXB_EPI_NONE, false),
                              {dz, L.weight, M->dact[i - 1]}))) return st;
      }
    }
  }
  if (c.world > 1 && !c.bucket_per_layer) {
    Instr ar; ar.kind = Instr::ALLREDUCE; ar.offset = 0; ar.count = M->bucket_elems;
    P.push_back(ar); M->n_collectives++;
  }

  // ---- optimizer ----
  // One rank: one program over every parameter, Module::iter() order.  Data parallel with a collective per layer:
  // one program per layer, last layer first, each waiting only for its own layer's allreduce, so the update of the
  // layers whose gradients have arrived overlaps the allreduce of the first layer's (the last to be produced).
  if (M->sharded) {
    // Sharded: one program per layer over this rank's shard of the slice (an elementwise update does not care where
    // tensors begin; the padding holds zero parameters and zero gradients and stays zero), first layer first, each
    // followed by the all-gather of that layer's parameters.  The first waits for every reduce-scatter.
    for (int i = 0; i < n; ++i) {
      const Linear& L = M->layers[i];
      zyxb_kernel_desc od{};
      od.kind = ZYXB_KIND_OPTIM;
      od.u.optim = c.optim;
      uint64_t numel = L.shard;
      od.u.optim.dtype = dt; od.u.optim.n_tensors = 1; od.u.optim.numel = &numel;
      od.u.optim.grad_scale = 1.0f / (float)c.world;
      std::vector<uint32_t> args = {L.param_shard, L.grad_shard};
      for (int s = 0; s < n_state; ++s) args.push_back(L.state[s][0]);
      if ((st = push_launch(M, M->update, od, args, i == 0 ? -1 : 0))) return st;
      Instr ag; ag.kind = Instr::ALLGATHER; ag.offset = L.bucket_offset; ag.count = L.shard; ag.layer = i;
      M->update.push_back(ag); M->n_collectives++;
    }
    return ZYXB_OK;
  }
  const bool per_layer = c.world > 1 && c.bucket_per_layer;
  const int groups = per_layer ? n : 1;
  for (int gi = 0; gi < groups; ++gi) {
    const int lo = per_layer ? n - 1 - gi : 0, hi = per_layer ? n - 1 - gi : n - 1;
    std::vector<uint64_t> numel;
    std::vector<uint32_t> p, g, s0, s1;
    for (int i = lo; i <= hi; ++i) {
      const Linear& L = M->layers[i];
      numel.push_back(L.in_features * L.out_features); numel.push_back(L.out_features);
      p.push_back(L.weight); p.push_back(L.bias);
      g.push_back(L.weight_grad); g.push_back(L.bias_grad);
      s0.push_back(L.state[0][0]); s0.push_back(L.state[0][1]);
      s1.push_back(L.state[1][0]); s1.push_back(L.state[1][1]);
    }
    zyxb_kernel_desc od{};
    od.kind = ZYXB_KIND_OPTIM;
    od.u.optim = c.optim;
    od.u.optim.dtype = dt; od.u.optim.n_tensors = (int32_t)p.size(); od.u.optim.numel = numel.data();
    if (c.world > 1) od.u.optim.grad_scale = 1.0f / (float)c.world;
    std::vector<uint32_t> args = p;
    args.insert(args.end(), g.begin(), g.end());
    if (n_state >= 1) args.insert(args.end(), s0.begin(), s0.end());
    if (n_state >= 2) args.insert(args.end(), s1.begin(), s1.end());
    if ((st = push_launch(M, M->update, od, args, per_layer ? collectives_of_layer[lo] : -1))) return st;
  }
  return ZYXB_OK;
}

int32_t mark(zyxb_mlp* M) {
  if (!M->profiling) return ZYXB_OK;
  zyxb_event ev{};
  TRY(zyxb_event_record(M->ctx, M->dev, &ev));
  M->prof_steps.back().push_back(ev);
  return ZYXB_OK;
}

int32_t run(zyxb_mlp* M, const std::vector<Instr>& plan, const zyxb_event* wait, int32_t n_wait) {
  bool first = true;
  for (const Instr& in : plan) {
    if (in.kind != Instr::LAUNCH) {
      zyxb_event ev{};
      if (in.kind == Instr::ALLREDUCE) {
        if (in.tail) TRY(zyxb_comm_option(M->ctx, M->dev, ZYXB_COMM_OPT_LATENCY, 1));
        const int32_t st_ar = zyxb_allreduce_sum(M->ctx, M->dev, M->grad_bucket, in.offset, in.count, M->cfg.dtype, nullptr, 0, &ev);
        if (in.tail) zyxb_comm_option(M->ctx, M->dev, ZYXB_COMM_OPT_LATENCY, 0);
        if (st_ar) { M->err = std::string("zyxb_allreduce_sum: ") + zyxb_last_error(M->ctx); return st_ar; }
      }
      else if (in.kind == Instr::REDUCE_SCATTER) TRY(zyxb_reduce_scatter_sum(M->ctx, M->dev, M->grad_bucket, in.offset, in.count, M->cfg.dtype, nullptr, 0, &ev));
      else TRY(zyxb_allgather(M->ctx, M->dev, M->param_bucket, in.offset, in.count, M->cfg.dtype, nullptr, 0, &ev));
      if (in.kind == Instr::ALLGATHER) {
        if (M->param_ready_set[in.layer]) TRY(zyxb_release_events(M->ctx, M->dev, &M->param_ready[in.layer], 1));
        M->param_ready[in.layer] = ev; M->param_ready_set[in.layer] = 1;
      } else M->pending.push_back(ev);
      int32_t stm = mark(M);   // keeps one mark per instruction; a collective runs on its own stream
      if (stm) return stm;
      continue;
    }
    std::vector<zyxb_event> w;
    if (first && n_wait > 0) w.assign(wait, wait + n_wait);
    if (in.layer >= 0 && M->param_ready_set[in.layer]) {   // this layer's parameters are still being gathered
      w.push_back(M->param_ready[in.layer]);
      M->param_ready_set[in.layer] = 0;
    }
    if (in.wait_collectives != 0) {
      const size_t take = in.wait_collectives < 0 ? M->pending.size() : std::min(M->pending.size(), (size_t)in.wait_collectives);
      w.insert(w.end(), M->pending.begin(), M->pending.begin() + take);
      M->pending.erase(M->pending.begin(), M->pending.begin() + take);
    }
    TRY(zyxb_launch(M->ctx, M->dev, in.program, in.args.data(), (int32_t)in.args.size(), w.empty() ? nullptr : w.data(), (int32_t)w.size(), nullptr));
    first = false;
    int32_t stm = mark(M);
    if (stm) return stm;
  }
  return ZYXB_OK;
}

// Blocks until every outstanding parameter all-gather has finished (a no-op unless the optimizer is sharded).
int32_t join_params(zyxb_mlp* M) {
  for (size_t i = 0; i < M->param_ready.size(); ++i)
    if (M->param_ready_set[i]) {
      TRY(zyxb_sync(M->ctx, M->dev, &M->param_ready[i], 1));
      M->param_ready_set[i] = 0;
    }
  return ZYXB_OK;
}

}  // namespace

extern "C" {
#pragma GCC visibility push(default)

int32_t zyxb_mlp_create(zyxb_ctx* ctx, int32_t dev, const zyxb_mlp_config* config, zyxb_mlp** out) {
  if (!ctx || !config || !out) return ZYXB_ERR_INITIALIZATION;
  *out = nullptr;
  zyxb_mlp* M = new zyxb_mlp();
  M->ctx = ctx; M->dev = dev; M->cfg = *config;
  const zyxb_mlp_config& c = M->cfg;
  bool ok = c.n_layers >= 1 && c.n_layers <= 8 && c.batch > 0 && (c.dtype == ZYXB_F32 || c.dtype == ZYXB_BF16 || c.dtype == ZYXB_F16);
  for (int i = 0; ok && i <= c.n_layers; ++i) ok = c.dims[i] > 0;
  if (ok && c.loss == ZYXB_LOSS_CROSS_ENTROPY && c.dtype != ZYXB_F32) ok = false;
  if (c.world < 1) M->cfg.world = 1;
  if (!ok) { delete M; return ZYXB_ERR_INCORRECT_KERNEL_ARG; }
  int32_t st = build(M);
  if (st != ZYXB_OK) {
    fprintf(stderr, "zyxb_mlp_create: %s\n", M->err.c_str());
    zyxb_mlp_destroy(M);
    return st;
  }
  *out = M;
  return ZYXB_OK;
}

int32_t zyxb_mlp_destroy(zyxb_mlp* M) {
  if (!M) return ZYXB_OK;
  zyxb_device_sync(M->ctx, M->dev);
  if (!M->pending.empty()) zyxb_release_events(M->ctx, M->dev, M->pending.data(), (int32_t)M->pending.size());
  for (size_t i = 0; i < M->param_ready.size(); ++i)
    if (M->param_ready_set[i]) zyxb_release_events(M->ctx, M->dev, &M->param_ready[i], 1);
  for (uint32_t p : M->owned_programs) zyxb_program_release(M->ctx, M->dev, p);
  // views were pushed after their parent: free in reverse so a parent outlives its views
  for (auto it = M->owned_buffers.rbegin(); it != M->owned_buffers.rend(); ++it) zyxb_free(M->ctx, M->dev, *it, nullptr, 0);
  delete M;
  return ZYXB_OK;
}

const char* zyxb_mlp_last_error(zyxb_mlp* M) { return M ? M->err.c_str() : ""; }

int32_t zyxb_mlp_tensor(zyxb_mlp* M, int32_t which, int32_t i, uint32_t* out_buf, uint64_t* out_numel) {
  if (!M || i < 0 || i >= 2 * M->cfg.n_layers || which < 0 || which > 3) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  const Linear& L = M->layers[i / 2];
  const int wb = i % 2;
  if (M->sharded) {
    if (which >= 2) { M->err = "mlp_tensor: the optimizer state is sharded over the ranks; it has no per-tensor buffers"; return ZYXB_ERR_INCORRECT_KERNEL_ARG; }
    int32_t stj = join_params(M);          // whoever asks for a buffer may read it: the gathers must have landed
    if (stj) return stj;
  }
  uint32_t b = 0;
  switch (which) {
    case 0: b = wb ? L.bias : L.weight; break;
    case 1: b = wb ? L.bias_grad : L.weight_grad; break;
    default: b = L.state[which - 2][wb];
  }
  if (b == 0) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  if (out_buf) *out_buf = b;
  if (out_numel) *out_numel = wb ? L.out_features : L.in_features * L.out_features;
  return ZYXB_OK;
}

int32_t zyxb_mlp_io(zyxb_mlp* M, uint32_t* out_x, uint32_t* out_target, uint32_t* out_loss, uint32_t* out_y) {
  if (!M) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  if (out_x) *out_x = M->x;
  if (out_target) *out_target = M->target;
  if (out_loss) *out_loss = M->loss;
  if (out_y) *out_y = M->y;
  return ZYXB_OK;
}

int32_t zyxb_mlp_activation(zyxb_mlp* M, int32_t which, int32_t layer, uint32_t* out_buf, uint64_t* out_numel) {
  if (!M || !out_buf || layer < 0 || layer >= M->cfg.n_layers || which < 0 || which > 2) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  const bool last = layer == M->cfg.n_layers - 1;
  uint32_t b = 0;
  switch (which) {
    case 0: b = last ? M->y : M->act[layer]; break;
    case 1: b = last ? 0 : M->preact[layer]; break;
    default: b = last ? M->dy : M->dact[layer];
  }
  if (b == 0) { M->err = "mlp_activation: this plan does not store that tensor"; return ZYXB_ERR_INCORRECT_KERNEL_ARG; }
  *out_buf = b;
  if (out_numel) *out_numel = M->cfg.batch * M->cfg.dims[layer + 1];
  return ZYXB_OK;
}

int32_t zyxb_mlp_forward_backward(zyxb_mlp* M) { return M ? run(M, M->forward_backward, nullptr, 0) : ZYXB_ERR_INCORRECT_KERNEL_ARG; }
int32_t zyxb_mlp_update(zyxb_mlp* M) {
  if (!M) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  int32_t st = run(M, M->update, nullptr, 0);
  return st ? st : join_params(M);         // the stand-alone update returns with complete parameters; zyxb_mlp_step does not wait
}

int32_t zyxb_mlp_bind_inputs(zyxb_mlp* M, uint32_t x, uint32_t target) {
  if (!M) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  const uint64_t es = dsize(M->cfg.dtype);
  uint64_t bx = 0, bt = 0;
  TRY(zyxb_buffer_bytes(M->ctx, M->dev, x, &bx));
  TRY(zyxb_buffer_bytes(M->ctx, M->dev, target, &bt));
  const uint64_t need_t = M->cfg.loss == ZYXB_LOSS_CROSS_ENTROPY ? M->cfg.batch * 4 : M->cfg.batch * M->cfg.dims[M->cfg.n_layers] * es;
  if (bx < M->cfg.batch * M->cfg.dims[0] * es || bt < need_t) { M->err = "bind_inputs: buffer too small"; return ZYXB_ERR_INCORRECT_KERNEL_ARG; }
  for (Instr& in : M->forward_backward)
    for (uint32_t& a : in.args) { if (a == M->x) a = x; else if (a == M->target) a = target; }
  M->x = x; M->target = target;
  return ZYXB_OK;
}

int32_t zyxb_mlp_step_event(zyxb_mlp* M, const zyxb_event* wait, int32_t n_wait, zyxb_event* out_event) {
  int32_t st = zyxb_mlp_step(M, wait, n_wait);
  if (st || !out_event) return st;
  // a non-timing marker after the last launch of the step
  TRY(zyxb_event_record(M->ctx, M->dev, out_event));
  return ZYXB_OK;
}

int32_t zyxb_mlp_step(zyxb_mlp* M, const zyxb_event* wait, int32_t n_wait) {
  if (!M) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  if (M->profiling) {
    M->prof_steps.emplace_back();
    zyxb_event ev{};
    TRY(zyxb_event_record(M->ctx, M->dev, &ev));
    M->prof_steps.back().push_back(ev);
  }
  int32_t st = run(M, M->forward_backward, wait, n_wait);
  if (st) return st;
  return run(M, M->update, nullptr, 0);
}

int32_t zyxb_mlp_profile(zyxb_mlp* M, int32_t enable) {
  if (!M) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  M->profiling = enable != 0;
  return ZYXB_OK;
}

int32_t zyxb_mlp_profile_read(zyxb_mlp* M, float* out_ms, int32_t* out_kind, int32_t capacity, int32_t* out_n, int32_t* out_steps) {
  if (!M) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  const int n = (int)(M->forward_backward.size() + M->update.size());
  if (out_n) *out_n = n;
  if (out_steps) *out_steps = (int32_t)M->prof_steps.size();
  if (capacity < n) return out_ms ? ZYXB_ERR_INCORRECT_KERNEL_ARG : ZYXB_OK;
  for (int i = 0; i < n; ++i) out_ms[i] = 0.0f;
  for (auto& evs : M->prof_steps) {
    if ((int)evs.size() != n + 1) continue;
    for (int i = 0; i < n; ++i) {
      float ms = 0.0f;
      TRY(zyxb_event_elapsed_ms(M->ctx, M->dev, evs[i], evs[i + 1], &ms));
      out_ms[i] += ms;
    }
    TRY(zyxb_release_events(M->ctx, M->dev, evs.data(), (int32_t)evs.size()));
  }
  if (out_kind) {
    int i = 0;
    for (const auto* plan : {&M->forward_backward, &M->update})
      for (const Instr& in : *plan) out_kind[i++] = in.kind != Instr::LAUNCH ? -1 : in.desc_kind * 100 + in.desc_sub;
  }
  M->prof_steps.clear();
  return ZYXB_OK;
}

int32_t zyxb_mlp_plan_size(zyxb_mlp* M, int32_t* out_launches, int32_t* out_collectives) {
  if (!M) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  if (out_launches) *out_launches = M->n_launches;
  if (out_collectives) *out_collectives = M->n_collectives;
  return ZYXB_OK;
}

#pragma GCC visibility pop
}  // extern "C"

// ---- checkpoints (Module::save / Tensor::load of the stack's tensors, zyx/src/module.rs:36-63, 436-529) ----------
namespace {
std::vector<zyxb_host::CkptTensor> mlp_ckpt_tensors(zyxb_mlp* M) {
  std::vector<zyxb_host::CkptTensor> out;
  const int n_state = M->cfg.optim.algo == ZYXB_OPT_SGD ? (M->cfg.optim.momentum != 0.0f ? 1 : 0) : 2;
  const char* state_prefix[2] = {M->cfg.optim.algo == ZYXB_OPT_SGD ? "optim.buf." : "optim.m.", "optim.v."};
  for (int s = -1; s < n_state; ++s)
    for (size_t i = 0; i < M->layers.size(); ++i) {
      const Linear& L = M->layers[i];
      if (M->sharded && s >= 0) {
        // a rank's file holds its own shard of the state, named for the rank: every rank saves to its own path
        zyxb_host::CkptTensor t;
        t.name = std::string(state_prefix[s]) + "shard" + std::to_string(M->rank) + "of" + std::to_string(M->cfg.world) + ".layers." + std::to_string(i);
        t.buffer = L.state[s][0];
        t.shape = {L.shard};
        out.push_back(std::move(t));
        continue;
      }
      for (int wb = 0; wb < 2; ++wb) {
        zyxb_host::CkptTensor t;
        t.name = std::string(s < 0 ? "" : state_prefix[s]) + "layers." + std::to_string(i) + (wb ? ".bias" : ".weight");
        t.buffer = s < 0 ? (wb ? L.bias : L.weight) : L.state[s][wb];
        if (wb) t.shape = {L.out_features}; else t.shape = {L.out_features, L.in_features};
        out.push_back(std::move(t));
      }
    }
  return out;
}
}  // namespace

#pragma GCC visibility push(default)
int32_t zyxb_mlp_save(zyxb_mlp* M, const char* path) {
  if (!M || !path) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  int32_t stj = join_params(M);
  if (stj) return stj;
  uint64_t t = 0;
  for (const Instr& in : M->update)
    if (in.kind == Instr::LAUNCH) { TRY(zyxb_program_get_step(M->ctx, M->dev, in.program, &t)); break; }
  return zyxb_host::checkpoint_save(M->ctx, M->dev, M->cfg.dtype, mlp_ckpt_tensors(M), t, path, M->err);
}

int32_t zyxb_mlp_load(zyxb_mlp* M, const char* path, int32_t* out_missing) {
  if (!M || !path) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  int32_t stj = join_params(M);          // parameter all-gathers still in flight would overwrite what is loaded
  if (stj) return stj;
  uint64_t t = 0;
  bool have_t = false;
  int32_t st = zyxb_host::checkpoint_load(M->ctx, M->dev, M->cfg.dtype, mlp_ckpt_tensors(M), &t, &have_t, out_missing, path, M->err);
  if (st || !have_t) return st;
  for (const Instr& in : M->update)
    if (in.kind == Instr::LAUNCH) TRY(zyxb_program_set_step(M->ctx, M->dev, in.program, t));
  return ZYXB_OK;
}
#pragma GCC visibility pop
