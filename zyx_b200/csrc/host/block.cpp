// Training plan of one transformer block (see include/zyxb_host.h), replayed through the C ABI only.
//
// Reference definitions restated by the plan:
//   block wiring     zyx-examples/examples/readme_test.rs:30-40   post-norm: norm1(x + attn), norm2(x1 + mlp2(gelu(mlp(x1))))
//   attention        zyx-nn/src/multi_head_attention.rs:160-227   q/k/v projections -> [B,H,T,D]; scores = q.k^T * (1/sqrt(D));
//                                                                 causal masked_fill(-inf); softmax(-1); .v; out projection
//   LayerNorm        zyx-nn/src/layer_norm.rs:95-135              (x - mean) / sqrt(var_unbiased + eps) * weight + bias
//   backward         zyx/src/graph/autograd.rs                    reverse-mode adjoints of the same expressions
// The [B,T,H,D] <-> [B,H,T,D] reshapes/transposes are never materialised: the per-head matmuls read q, k, v in
// place through row pitches and a (batch, head) two-level batch, and write their results back the same way.
#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#include "../../../include/zyxb_host.h"
#include "checkpoint.hpp"
#include "plan.hpp"

using namespace zyxb_host;

namespace {
enum { P_WQ = 0, P_BQ, P_WK, P_BK, P_WV, P_BV, P_WO, P_BO, P_W1, P_B1, P_W2, P_B2, P_G1, P_BE1, P_G2, P_BE2, N_PARAMS };
}

struct zyxb_block {
  Plan plan;
  zyxb_block_config cfg{};
  uint64_t numel[N_PARAMS] = {0};
  uint32_t param[N_PARAMS] = {0}, grad[N_PARAMS] = {0}, state[2][N_PARAMS] = {{0}, {0}};
  uint32_t grad_bucket = 0, param_bucket = 0;
  uint64_t bucket_off[N_PARAMS] = {0};
  // sharded optimizer (ZeRO stage 1): each of the three gradient groups is cut into `world` shards; this rank updates
  // one shard per group with state of shard size and the updated parameters are all-gathered
  bool sharded = false;
  int rank = 0;
  uint64_t shard[3] = {0, 0, 0};
  uint32_t param_shard[3] = {0, 0, 0}, grad_shard[3] = {0, 0, 0}, shard_state[2][3] = {{0, 0, 0}, {0, 0, 0}};
  uint32_t x = 0, target = 0, loss = 0, y = 0;
  uint32_t q = 0, k = 0, v = 0, s = 0, p = 0, attn = 0, o = 0, s1 = 0, x1 = 0, z1 = 0, h = 0, m = 0, s2 = 0;
  uint32_t dy = 0, ds2 = 0, tmp = 0, dz1 = 0, dx1 = 0, ds1 = 0, dattn = 0, dp = 0, dq = 0, dk = 0, dv = 0;
  uint32_t lse = 0;                // fused attention: log-sum-exp per (batch, head, query), f32
  bool fused = false;
  size_t n_forward_backward = 0;   // instructions before the optimizer launches
};

namespace {

// per-head view of a [B, T, H*D] tensor for the two-level batch (B outer, H inner)
void head_view_a(zyxb_gemm_desc& g, uint64_t T, uint64_t E, uint64_t D) { g.lda = E; g.stride_a = (int64_t)(T * E); g.stride_a_inner = (int64_t)D; }
void head_view_b(zyxb_gemm_desc& g, uint64_t T, uint64_t E, uint64_t D) { g.ldb = E; g.stride_b = (int64_t)(T * E); g.stride_b_inner = (int64_t)D; }
void head_view_c(zyxb_gemm_desc& g, uint64_t T, uint64_t E, uint64_t D) { g.ldc = E; g.stride_c = (int64_t)(T * E); g.stride_c_inner = (int64_t)D; }
// packed [B*H, T, T] score-shaped operand
void score_view_a(zyxb_gemm_desc& g, uint64_t H, uint64_t T) { g.stride_a = (int64_t)(H * T * T); g.stride_a_inner = (int64_t)(T * T); }
void score_view_c(zyxb_gemm_desc& g, uint64_t H, uint64_t T) { g.stride_c = (int64_t)(H * T * T); g.stride_c_inner = (int64_t)(T * T); }

#define CHK(expr) do { int32_t st_ = (expr); if (st_) return st_; } while (0)

int32_t build(zyxb_block* K) {
  Plan& P = K->plan;
  const zyxb_block_config& c = K->cfg;
  const int32_t dt = c.dtype;
  const uint64_t es = dsize(dt), B = c.batch, T = c.seq, E = c.dim, H = c.heads, D = E / H, F = c.ffn, R = B * T;
  const float scale = 1.0f / sqrtf((float)D);

  // ---- parameters; gradients in one bucket laid out in the order the backward pass produces them ----
  const uint64_t sizes[N_PARAMS] = {E * E, E, E * E, E, E * E, E, E * E, E, F * E, F, E * F, E, E, E, E, E};
  for (int i = 0; i < N_PARAMS; ++i) K->numel[i] = sizes[i];
  const int order[N_PARAMS] = {P_G2, P_BE2, P_W2, P_B2, P_W1, P_B1,          // group 0: norm2 + feed-forward
                               P_G1, P_BE1, P_WO, P_BO,                      // group 1: norm1 + output projection
                               P_WV, P_BV, P_WK, P_BK, P_WQ, P_BQ};          // group 2: value / key / query projections
  const int group_end[3] = {6, 10, 16};
  K->sharded = c.shard_optimizer != 0;
  if (K->sharded) {
    int32_t r = 0, w = 1;
    int32_t st = zyxb_comm_rank(P.ctx, P.dev, &r, &w);
    if (st) return P.fail(st, "zyxb_comm_rank");
    if (w != c.world) { P.err = "shard_optimizer: config.world differs from the communicator's"; return ZYXB_ERR_INCORRECT_KERNEL_ARG; }
    K->rank = r;
  }
  const uint64_t align_elems = 256 / es;
  const uint64_t group_align = K->sharded ? align_elems * (uint64_t)c.world : align_elems;   // a sharded group divides into aligned shards
  uint64_t off = 0, group_off[4] = {0, 0, 0, 0};
  for (int j = 0, g = 0; j < N_PARAMS; ++j) {
    K->bucket_off[order[j]] = off;
    off += align_up(sizes[order[j]], align_elems);
    if (j + 1 == group_end[g]) { off = align_up(off, group_align); group_off[++g] = off; }
  }
  CHK(P.alloc(off * es, &K->grad_bucket, true));
  if (K->sharded) CHK(P.alloc(off * es, &K->param_bucket, true));   // the same layout; the padding stays zero
  const bool adam = c.optim.algo != ZYXB_OPT_SGD;
  const int n_state = adam ? 2 : (c.optim.momentum != 0.0f ? 1 : 0);
  for (int i = 0; i < N_PARAMS; ++i) {
    if (K->sharded) CHK(P.view(K->param_bucket, K->bucket_off[i] * es, sizes[i] * es, &K->param[i]));
    else CHK(P.alloc(sizes[i] * es, &K->param[i], true));
    CHK(P.view(K->grad_bucket, K->bucket_off[i] * es, sizes[i] * es, &K->grad[i]));
    if (!K->sharded)
      for (int s = 0; s < n_state; ++s) CHK(P.alloc(sizes[i] * es, &K->state[s][i], true));
  }
  if (K->sharded)
    for (int g = 0; g < 3; ++g) {
      K->shard[g] = (group_off[g + 1] - group_off[g]) / (uint64_t)c.world;
      const uint64_t at = (group_off[g] + (uint64_t)K->rank * K->shard[g]) * es;
      CHK(P.view(K->param_bucket, at, K->shard[g] * es, &K->param_shard[g]));
      CHK(P.view(K->grad_bucket, at, K->shard[g] * es, &K->grad_shard[g]));
      for (int s = 0; s < n_state; ++s) CHK(P.alloc(K->shard[g] * es, &K->shard_state[s][g], true));
    }
  // ---- activations ----
  const uint64_t RE = R * E * es, RF = R * F * es, SS = B * H * T * T * es;
  for (uint32_t* b : {&K->x, &K->target, &K->y, &K->q, &K->k, &K->v, &K->attn, &K->o, &K->s1, &K->x1, &K->m, &K->s2, &K->dy, &K->ds2,
                      &K->tmp, &K->dx1, &K->ds1, &K->dattn, &K->dq, &K->dk, &K->dv})
    CHK(P.alloc(RE, b));
  for (uint32_t* b : {&K->z1, &K->h, &K->dz1}) CHK(P.alloc(RF, b));
  const bool fused = c.fused_attention && dt != ZYXB_F32 && D == 128 && T % 128 == 0;
  K->fused = fused;
  if (fused) CHK(P.alloc(B * H * T * 4, &K->lse));
  else for (uint32_t* b : {&K->s, &K->p, &K->dp}) CHK(P.alloc(SS, b));
  auto attention = [&](bool backward) {
    zyxb_kernel_desc d{};
    d.kind = backward ? ZYXB_KIND_ATTENTION_BWD : ZYXB_KIND_ATTENTION;
    d.u.attention.dtype = dt; d.u.attention.batch = B; d.u.attention.heads = H; d.u.attention.seq = T; d.u.attention.head_dim = D;
    d.u.attention.scale = scale; d.u.attention.causal = c.causal;
    return d;
  };
  CHK(P.alloc(4, &K->loss, true));

  // ================================== forward ==================================
  // `group`: this launch is the first reader of that parameter group in a step and waits for its all-gather (sharded optimizer)
  auto linear = [&](uint32_t in, int w, int b, uint32_t out, uint64_t in_f, uint64_t out_f, int32_t epi, uint32_t pre, int group = -1) {
    std::vector<uint32_t> args = {in, K->param[w], K->param[b], out};
    if (pre) args.push_back(pre);
    return P.launch(gemm(dt, R, out_f, in_f, false, true, epi, pre != 0), args, 0, K->sharded ? group : -1);   // x.dot(W.t()) + b
  };
  CHK(linear(K->x, P_WQ, P_BQ, K->q, E, E, ZYXB_EPI_BIAS, 0, 2));
  CHK(linear(K->x, P_WK, P_BK, K->k, E, E, ZYXB_EPI_BIAS, 0));
  CHK(linear(K->x, P_WV, P_BV, K->v, E, E, ZYXB_EPI_BIAS, 0));
  if (fused) {
    CHK(P.launch(attention(false), {K->q, K->k, K->v, K->attn, K->lse}));
  } else {
  {  // scores[b,h] = q[b,:,h,:] . k[b,:,h,:]^T * (1/sqrt(D))
    zyxb_kernel_desc d = gemm(dt, T, T, D, false, true, ZYXB_EPI_NONE, false, scale);
    d.u.gemm.batch = B; d.u.gemm.batch_inner = H;
    head_view_a(d.u.gemm, T, E, D); head_view_b(d.u.gemm, T, E, D); score_view_c(d.u.gemm, H, T);
    if (c.causal) d.u.gemm.tri = ZYXB_TRI_OUT_LOWER;   // the softmax never reads above the diagonal
    CHK(P.launch(d, {K->q, K->k, K->s}));
  }
  {  // softmax over keys, masked above the diagonal when causal
    zyxb_kernel_desc d = row(ZYXB_RR_SOFTMAX, dt, B * H * T, T);
    d.u.rowreduce.causal = c.causal; d.u.rowreduce.period = T;
    CHK(P.launch(d, {K->s, K->p}));
  }
  {  // attn[b,:,h,:] = p[b,h] . v[b,:,h,:]
    zyxb_kernel_desc d = gemm(dt, T, D, T, false, false);
    d.u.gemm.batch = B; d.u.gemm.batch_inner = H;
    score_view_a(d.u.gemm, H, T); head_view_b(d.u.gemm, T, E, D); head_view_c(d.u.gemm, T, E, D);
    if (c.causal) d.u.gemm.tri = ZYXB_TRI_A_LOWER;     // p is zero above the diagonal
    CHK(P.launch(d, {K->p, K->v, K->attn}));
  }
  }
  CHK(linear(K->attn, P_WO, P_BO, K->o, E, E, ZYXB_EPI_BIAS, 0, 1));
  CHK(P.launch(eltwise(ZYXB_EW_ADD, dt, R * E), {K->x, K->o, K->s1}));
  auto layernorm = [&](uint32_t in, int w, int b, uint32_t out) {
    zyxb_kernel_desc d = row(ZYXB_RR_LAYERNORM, dt, R, E);
    d.u.rowreduce.eps = c.eps; d.u.rowreduce.has_weight = 1; d.u.rowreduce.has_bias = 1;
    return P.launch(d, {in, K->param[w], K->param[b], out});
  };
  CHK(layernorm(K->s1, P_G1, P_BE1, K->x1));
  CHK(linear(K->x1, P_W1, P_B1, K->h, E, F, ZYXB_EPI_BIAS_GELU, K->z1, 0));
  CHK(linear(K->h, P_W2, P_B2, K->m, F, E, ZYXB_EPI_BIAS, 0));
  CHK(P.launch(eltwise(ZYXB_EW_ADD, dt, R * E), {K->x1, K->m, K->s2}));
  CHK(layernorm(K->s2, P_G2, P_BE2, K->y));
  CHK(P.launch(row(ZYXB_RR_MSE, dt, R, E), {K->y, K->target, K->loss}));

  // ================================== backward ==================================
  CHK(P.launch(eltwise(ZYXB_EW_MSE_BWD, dt, R * E, 1.0f / (float)(R * E)), {K->y, K->target, K->dy}));
  auto colsum = [&](uint32_t in, uint64_t cols, uint32_t out) { return P.launch(row(ZYXB_RR_COLSUM, dt, R, cols), {in, out}); };
  auto layernorm_bwd = [&](uint32_t in, uint32_t dout, int w, int b, uint32_t din) {
    zyxb_kernel_desc d = row(ZYXB_RR_LAYERNORM_DYXHAT, dt, R, E);
    d.u.rowreduce.eps = c.eps;
    CHK(P.launch(d, {in, dout, K->tmp}));
    CHK(colsum(K->tmp, E, K->grad[w]));                       // d weight = sum_rows dy * xhat
    CHK(colsum(dout, E, K->grad[b]));                         // d bias   = sum_rows dy
    d = row(ZYXB_RR_LAYERNORM_BWD, dt, R, E);
    d.u.rowreduce.eps = c.eps; d.u.rowreduce.has_weight = 1;
    return P.launch(d, {in, dout, K->param[w], din});
  };
  // dW = dOut^T . in, db = column sums of dOut
  auto linear_param_grads = [&](uint32_t dout, uint32_t in, int w, int b, uint64_t in_f, uint64_t out_f) {
    CHK(P.launch(gemm(dt, out_f, in_f, R, true, false), {dout, in, K->grad[w]}));
    return P.launch(row(ZYXB_RR_COLSUM, dt, R, out_f), {dout, K->grad[b]});
  };
  const int tail_collectives = getenv("ZYXB_TAIL_COLLECTIVES") ? atoi(getenv("ZYXB_TAIL_COLLECTIVES")) : 0;   // 1: the last group's allreduce takes the low-latency path
  auto reduce_group = [&](int g) {
    if (K->sharded) P.reduce_scatter(K->grad_bucket, group_off[g], K->shard[g]);
    else if (c.world > 1) P.allreduce(K->grad_bucket, group_off[g], group_off[g + 1] - group_off[g], g == 2 && tail_collectives >= 1);
    return (int32_t)ZYXB_OK;
  };
  CHK(layernorm_bwd(K->s2, K->dy, P_G2, P_BE2, K->ds2));       // ds2 flows to both x1 (residual) and mlp2's output
  CHK(linear_param_grads(K->ds2, K->h, P_W2, P_B2, F, E));
  CHK(P.launch(gemm(dt, R, F, E, false, false, ZYXB_EPI_MUL_GELU_GRAD), {K->ds2, K->param[P_W2], K->z1, K->dz1}));
  CHK(linear_param_grads(K->dz1, K->x1, P_W1, P_B1, E, F));
  CHK(reduce_group(0));
  CHK(P.launch(gemm(dt, R, E, F, false, false, ZYXB_EPI_ADD), {K->dz1, K->param[P_W1], K->ds2, K->dx1}));   // + residual
  CHK(layernorm_bwd(K->s1, K->dx1, P_G1, P_BE1, K->ds1));      // ds1 = d(x + o): gradient of the attention output projection
  CHK(linear_param_grads(K->ds1, K->attn, P_WO, P_BO, E, E));
  CHK(reduce_group(1));
  CHK(P.launch(gemm(dt, R, E, E, false, false), {K->ds1, K->param[P_WO], K->dattn}));
  if (fused) {
    CHK(P.launch(attention(true), {K->q, K->k, K->v, K->attn, K->dattn, K->lse, K->dq, K->dk, K->dv}));
  } else {
  {  // dP[b,h] = dattn[b,:,h,:] . v[b,:,h,:]^T
    zyxb_kernel_desc d = gemm(dt, T, T, D, false, true);
    d.u.gemm.batch = B; d.u.gemm.batch_inner = H;
    head_view_a(d.u.gemm, T, E, D); head_view_b(d.u.gemm, T, E, D); score_view_c(d.u.gemm, H, T);
    if (c.causal) d.u.gemm.tri = ZYXB_TRI_OUT_LOWER;
    CHK(P.launch(d, {K->dattn, K->v, K->dp}));
  }
  {  // dV[b,:,h,:] = p[b,h]^T . dattn[b,:,h,:]
    zyxb_kernel_desc d = gemm(dt, T, D, T, true, false);
    d.u.gemm.batch = B; d.u.gemm.batch_inner = H;
    score_view_a(d.u.gemm, H, T); head_view_b(d.u.gemm, T, E, D); head_view_c(d.u.gemm, T, E, D);
    if (c.causal) d.u.gemm.tri = ZYXB_TRI_AT_LOWER;
    CHK(P.launch(d, {K->p, K->dattn, K->dv}));
  }
  {  // dS in place of dP; masked entries have p = 0 and are skipped
    zyxb_kernel_desc d = row(ZYXB_RR_SOFTMAX_BWD, dt, B * H * T, T);
    d.u.rowreduce.causal = c.causal; d.u.rowreduce.period = T;
    CHK(P.launch(d, {K->p, K->dp, K->dp}));
  }
  {  // dQ[b,:,h,:] = dS[b,h] . k[b,:,h,:] * scale
    zyxb_kernel_desc d = gemm(dt, T, D, T, false, false, ZYXB_EPI_NONE, false, scale);
    d.u.gemm.batch = B; d.u.gemm.batch_inner = H;
    score_view_a(d.u.gemm, H, T); head_view_b(d.u.gemm, T, E, D); head_view_c(d.u.gemm, T, E, D);
    if (c.causal) d.u.gemm.tri = ZYXB_TRI_A_LOWER;     // dS is zero above the diagonal
    CHK(P.launch(d, {K->dp, K->k, K->dq}));
    d.u.gemm.trans_a = 1;   // dK[b,:,h,:] = dS[b,h]^T . q[b,:,h,:] * scale
    if (c.causal) d.u.gemm.tri = ZYXB_TRI_AT_LOWER;
    CHK(P.launch(d, {K->dp, K->q, K->dk}));
  }
  }
  CHK(linear_param_grads(K->dv, K->x, P_WV, P_BV, E, E));
  CHK(linear_param_grads(K->dk, K->x, P_WK, P_BK, E, E));
  CHK(linear_param_grads(K->dq, K->x, P_WQ, P_BQ, E, E));
  CHK(reduce_group(2));
  K->n_forward_backward = P.instrs.size();

  // ================================== optimizer ==================================
  // Sharded: one program per group over this rank's shard of the group's slice (an elementwise update does not care where
  // tensors begin; the padding holds zero parameters and zero gradients and stays zero), the group the forward pass reads
  // first (q/k/v) first, each followed by the all-gather of that group's parameters.  The first waits for every reduce-scatter.
  if (K->sharded) {
    for (int g = 2; g >= 0; --g) {
      zyxb_kernel_desc od{};
      od.kind = ZYXB_KIND_OPTIM;
      od.u.optim = c.optim;
      uint64_t numel = K->shard[g];
      od.u.optim.dtype = dt; od.u.optim.n_tensors = 1; od.u.optim.numel = &numel;
      od.u.optim.grad_scale = 1.0f / (float)c.world;
      std::vector<uint32_t> args = {K->param_shard[g], K->grad_shard[g]};
      for (int s = 0; s < n_state; ++s) args.push_back(K->shard_state[s][g]);
      CHK(P.launch(od, args, g == 2 ? -1 : 0));
      P.allgather(K->param_bucket, group_off[g], K->shard[g], g);
    }
    return ZYXB_OK;
  }
  // one program per gradient group, each waiting only for its own group's allreduce
  for (int g = 0; g < 3; ++g) {
    std::vector<uint64_t> numel;
    std::vector<uint32_t> p, gr, s0, s1;
    for (int j = g == 0 ? 0 : group_end[g - 1]; j < group_end[g]; ++j) {
      const int i = order[j];
      numel.push_back(sizes[i]); p.push_back(K->param[i]); gr.push_back(K->grad[i]);
      s0.push_back(K->state[0][i]); s1.push_back(K->state[1][i]);
    }
    zyxb_kernel_desc od{};
    od.kind = ZYXB_KIND_OPTIM;
    od.u.optim = c.optim;
    od.u.optim.dtype = dt; od.u.optim.n_tensors = (int32_t)p.size(); od.u.optim.numel = numel.data();
    if (c.world > 1) od.u.optim.grad_scale = 1.0f / (float)c.world;
    std::vector<uint32_t> args = p;
    args.insert(args.end(), gr.begin(), gr.end());
    if (n_state >= 1) args.insert(args.end(), s0.begin(), s0.end());
    if (n_state >= 2) args.insert(args.end(), s1.begin(), s1.end());
    CHK(P.launch(od, args, c.world > 1 ? 1 : 0));
  }
  return ZYXB_OK;
}

}  // namespace

extern "C" {
#pragma GCC visibility push(default)

int32_t zyxb_block_create(zyxb_ctx* ctx, int32_t dev, const zyxb_block_config* config, zyxb_block** out) {
  if (!ctx || !config || !out) return ZYXB_ERR_INITIALIZATION;
  *out = nullptr;
  const zyxb_block_config& c = *config;
  const bool ok = (c.dtype == ZYXB_F32 || c.dtype == ZYXB_BF16 || c.dtype == ZYXB_F16) && c.batch > 0 && c.seq > 0 && c.dim > 1 &&
                  c.heads > 0 && c.dim % c.heads == 0 && c.ffn > 0;
  if (!ok) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  zyxb_block* K = new zyxb_block();
  K->cfg = c;
  if (K->cfg.world < 1) K->cfg.world = 1;
  K->plan.ctx = ctx; K->plan.dev = dev; K->plan.dtype = c.dtype;
  int32_t st = build(K);
  if (st != ZYXB_OK) {
    fprintf(stderr, "zyxb_block_create: %s\n", K->plan.err.c_str());
    zyxb_block_destroy(K);
    return st;
  }
  *out = K;
  return ZYXB_OK;
}

int32_t zyxb_block_destroy(zyxb_block* K) {
  if (!K) return ZYXB_OK;
  K->plan.destroy();
  delete K;
  return ZYXB_OK;
}

const char* zyxb_block_last_error(zyxb_block* K) { return K ? K->plan.err.c_str() : ""; }

int32_t zyxb_block_tensor(zyxb_block* K, int32_t which, int32_t i, uint32_t* out_buf, uint64_t* out_numel) {
  if (!K || i < 0 || i >= N_PARAMS || which < 0 || which > 3) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  if (K->sharded && which >= 2) {
    K->plan.err = "block_tensor: the optimizer state is sharded over the ranks; it has no per-tensor buffers";
    return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  }
  CHK(K->plan.join_gathers());          // whoever asks for a buffer may read or write it: the gathers must have landed
  const uint32_t b = which == 0 ? K->param[i] : which == 1 ? K->grad[i] : K->state[which - 2][i];
  if (b == 0) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  if (out_buf) *out_buf = b;
  if (out_numel) *out_numel = K->numel[i];
  return ZYXB_OK;
}

int32_t zyxb_block_io(zyxb_block* K, uint32_t* out_x, uint32_t* out_target, uint32_t* out_loss, uint32_t* out_y) {
  if (!K) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  if (out_x) *out_x = K->x;
  if (out_target) *out_target = K->target;
  if (out_loss) *out_loss = K->loss;
  if (out_y) *out_y = K->y;
  return ZYXB_OK;
}

int32_t zyxb_block_activation(zyxb_block* K, int32_t which, uint32_t* out_buf) {
  if (!K || !out_buf || which < 0 || which > 20) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  if (which == 0 && K->fused) return ZYXB_ERR_INCORRECT_KERNEL_ARG;   // the probabilities are never materialised
  const uint32_t table[21] = {K->p, K->attn, K->x1, K->q, K->k, K->v, K->o, K->s1, K->z1, K->h, K->m, K->s2,
                              K->dy, K->ds2, K->dz1, K->dx1, K->ds1, K->dattn, K->dq, K->dk, K->dv};
  *out_buf = table[which];
  return ZYXB_OK;
}

int32_t zyxb_block_forward_backward(zyxb_block* K) { return K ? K->plan.run(0, K->n_forward_backward, nullptr, 0) : ZYXB_ERR_INCORRECT_KERNEL_ARG; }
int32_t zyxb_block_update(zyxb_block* K) {
  if (!K) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  int32_t st = K->plan.run(K->n_forward_backward, K->plan.instrs.size(), nullptr, 0);
  return st ? st : K->plan.join_gathers();   // the stand-alone update returns with complete parameters; zyxb_block_step does not wait
}
int32_t zyxb_block_step(zyxb_block* K, const zyxb_event* wait, int32_t n_wait) {
  return K ? K->plan.run(0, K->plan.instrs.size(), wait, n_wait) : ZYXB_ERR_INCORRECT_KERNEL_ARG;
}
int32_t zyxb_block_plan_size(zyxb_block* K, int32_t* out_launches, int32_t* out_collectives) {
  if (!K) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  if (out_launches) *out_launches = K->plan.n_launches;
  if (out_collectives) *out_collectives = K->plan.n_collectives;
  return ZYXB_OK;
}

#pragma GCC visibility pop
}  // extern "C"

// ---- checkpoints (Module::save / Tensor::load of the block's tensors, zyx/src/module.rs:36-63, 436-529) ----------
namespace {
// labels in Module::iter_tensors order of the block (derive(Module) field paths)
const char* const BLOCK_LABELS[N_PARAMS] = {
    "attn.q_proj.weight", "attn.q_proj.bias", "attn.k_proj.weight", "attn.k_proj.bias", "attn.v_proj.weight", "attn.v_proj.bias",
    "attn.out_proj.weight", "attn.out_proj.bias", "mlp.weight", "mlp.bias", "mlp2.weight", "mlp2.bias",
    "norm1.weight", "norm1.bias", "norm2.weight", "norm2.bias"};

std::vector<zyxb_host::CkptTensor> block_ckpt_tensors(zyxb_block* K) {
  const zyxb_block_config& c = K->cfg;
  const uint64_t E = c.dim, F = c.ffn;
  std::vector<zyxb_host::CkptTensor> out;
  const int n_state = c.optim.algo == ZYXB_OPT_SGD ? (c.optim.momentum != 0.0f ? 1 : 0) : 2;
  const char* state_prefix[2] = {c.optim.algo == ZYXB_OPT_SGD ? "optim.buf." : "optim.m.", "optim.v."};
  static const char* const GROUP_LABELS[3] = {"ffn", "attn_out", "qkv"};
  for (int s = 0; K->sharded && s < n_state; ++s)
    for (int g = 0; g < 3; ++g) {
      // a rank's file holds its own shard of the state, named for the rank: every rank saves to its own path
      zyxb_host::CkptTensor t;
      t.name = std::string(state_prefix[s]) + "shard" + std::to_string(K->rank) + "of" + std::to_string(c.world) + "." + GROUP_LABELS[g];
      t.buffer = K->shard_state[s][g];
      t.shape = {K->shard[g]};
      out.push_back(std::move(t));
    }
  for (int s = -1; s < (K->sharded ? 0 : n_state); ++s)
    for (int i = 0; i < N_PARAMS; ++i) {
      zyxb_host::CkptTensor t;
      t.name = std::string(s < 0 ? "" : state_prefix[s]) + BLOCK_LABELS[i];
      t.buffer = s < 0 ? K->param[i] : K->state[s][i];
      if (i == P_W1) t.shape = {F, E};
      else if (i == P_W2) t.shape = {E, F};
      else if (i == P_B1) t.shape = {F};
      else if (i < P_W1 && i % 2 == 0) t.shape = {E, E};
      else t.shape = {E};
      out.push_back(std::move(t));
    }
  return out;
}
}  // namespace

#pragma GCC visibility push(default)
int32_t zyxb_block_save(zyxb_block* K, const char* path) {
  if (!K || !path) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  CHK(K->plan.join_gathers());
  uint64_t t = 0;
  if (K->n_forward_backward < K->plan.instrs.size()) {
    int32_t st = zyxb_program_get_step(K->plan.ctx, K->plan.dev, K->plan.instrs[K->n_forward_backward].program, &t);
    if (st) return K->plan.fail(st, "zyxb_program_get_step");
  }
  return zyxb_host::checkpoint_save(K->plan.ctx, K->plan.dev, K->cfg.dtype, block_ckpt_tensors(K), t, path, K->plan.err);
}

int32_t zyxb_block_load(zyxb_block* K, const char* path, int32_t* out_missing) {
  if (!K || !path) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  CHK(K->plan.join_gathers());          // parameter all-gathers still in flight would overwrite what is loaded
  uint64_t t = 0;
  bool have_t = false;
  int32_t st = zyxb_host::checkpoint_load(K->plan.ctx, K->plan.dev, K->cfg.dtype, block_ckpt_tensors(K), &t, &have_t, out_missing, path, K->plan.err);
  if (st || !have_t) return st;
  for (size_t i = K->n_forward_backward; i < K->plan.instrs.size(); ++i)
    if (K->plan.instrs[i].kind == Instr::LAUNCH) {
      st = zyxb_program_set_step(K->plan.ctx, K->plan.dev, K->plan.instrs[i].program, t);
      if (st) return K->plan.fail(st, "zyxb_program_set_step");
    }
  return ZYXB_OK;
}
#pragma GCC visibility pop
