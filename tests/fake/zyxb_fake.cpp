// A host-memory stand-in for libzyxb (include/zyxb.h).  TEST INFRASTRUCTURE ONLY.
//
// zyx tests its runtime against a dummy backend that allocates nothing and computes nothing
// (zyx/src/backend/dummy.rs:36-74).  This one goes a step further so that the host-side plans of libzyxb_host can be
// run for real on CPU ranks: buffers are host memory, programs are executed by plain loops in double precision (f32
// tensors only; this is not the oracle and shares no code with it), collectives call back into the test (which uses
// torch.distributed's gloo backend), and the n-th allocation, launch or collective can be made to fail, the way a device
// error would surface through the ABI (zyx/src/error.rs:107-153).  The shipped package never loads this library.
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <map>
#include <string>
#include <vector>

#include "../../include/zyxb.h"

namespace {
struct Buf { std::vector<uint8_t> own; uint8_t* ptr = nullptr; uint64_t bytes = 0; bool live = false; };
struct Prog { zyxb_kernel_desc d{}; std::vector<uint64_t> numel; uint64_t step = 0; bool live = false; };
typedef int32_t (*allreduce_cb)(void* data, uint64_t count, int32_t dtype, int32_t op);   // op 0 allreduce, 1 reduce-scatter, 2 allgather
}  // namespace

struct zyxb_ctx {
  std::vector<Buf> bufs{1};
  std::vector<Prog> progs{1};
  std::string err;
  uint64_t next_event = 1, launches = 0;
  int rank = 0, world = 1;
  bool comm = false;
};

namespace {
allreduce_cb g_cb = nullptr;
int64_t g_fail_at[3] = {-1, -1, -1};      // countdown per kind (0 alloc, 1 launch, 2 collective); -1 = never
uint64_t g_calls[3] = {0, 0, 0};

int fail(zyxb_ctx* c, int st, const std::string& m) { if (c) c->err = m; return st; }
bool injected(int kind) {
  ++g_calls[kind];
  if (g_fail_at[kind] < 0) return false;
  if (g_fail_at[kind]-- == 0) { g_fail_at[kind] = -1; return true; }
  return false;
}
Buf* get(zyxb_ctx* c, uint32_t id) { return (c && id && id < c->bufs.size() && c->bufs[id].live) ? &c->bufs[id] : nullptr; }
float* f(Buf* b) { return (float*)b->ptr; }

double gelu(double x) { const double u = (x + 0.044715 * x * x * x) * 0.7978845608028654, e = exp(2 * u); return x * 0.5 * ((e - 1) / (e + 1) + 1); }
double gelu_grad(double x) {
  const double c = 0.7978845608028654, u = (x + 0.044715 * x * x * x) * c, e = exp(2 * u), t = (e - 1) / (e + 1);
  return 0.5 * (1 + t) + 0.5 * x * (1 - t * t) * c * (1 + 3 * 0.044715 * x * x);
}

int run_gemm(zyxb_ctx* c, const zyxb_gemm_desc& d, std::vector<Buf*>& a) {
  if (d.dtype != ZYXB_F32 || d.batch != 1 || d.batch_inner > 1) return fail(c, ZYXB_ERR_KERNEL_LAUNCH, "fake: only plain f32 matmuls");
  const bool bias = d.epilogue >= ZYXB_EPI_BIAS && d.epilogue <= ZYXB_EPI_BIAS_GELU, z = d.epilogue >= ZYXB_EPI_MUL_RELU_GRAD;
  const size_t want = 3 + (bias || z) + (d.store_preact ? 1 : 0);
  if (a.size() != want) return fail(c, ZYXB_ERR_INCORRECT_KERNEL_ARG, "fake gemm: argument count");
  const float *A = f(a[0]), *B = f(a[1]), *X = (bias || z) ? f(a[2]) : nullptr;
  float* C = f(a[2 + (bias || z)]);
  float* P = d.store_preact ? f(a[3 + (bias || z)]) : nullptr;
  const double alpha = d.alpha == 0 ? 1.0 : d.alpha;
  for (uint64_t i = 0; i < d.m; ++i)
    for (uint64_t j = 0; j < d.n; ++j) {
      double s = 0;
      for (uint64_t k = 0; k < d.k; ++k) s += (double)(d.trans_a ? A[k * d.m + i] : A[i * d.k + k]) * (d.trans_b ? B[j * d.k + k] : B[k * d.n + j]);
      s *= alpha;
      if (bias) s += X[j];
      if (P) P[i * d.n + j] = (float)s;
      switch (d.epilogue) {
        case ZYXB_EPI_BIAS_RELU: s = s > 0 ? s : 0; break;
        case ZYXB_EPI_BIAS_GELU: s = gelu(s); break;
        case ZYXB_EPI_MUL_RELU_GRAD: s = X[i * d.n + j] > 0 ? s : 0; break;
        case ZYXB_EPI_MUL_GELU_GRAD: s *= gelu_grad(X[i * d.n + j]); break;
        case ZYXB_EPI_ADD: s += X[i * d.n + j]; break;
        default: break;
      }
      C[i * d.n + j] = (float)s;
    }
  return ZYXB_OK;
}

int run_row(zyxb_ctx* c, const zyxb_rowreduce_desc& d, std::vector<Buf*>& a) {
  const uint64_t R = d.rows, N = d.cols;
  switch (d.op) {
    case ZYXB_RR_COLSUM: {
      for (uint64_t j = 0; j < N; ++j) { double s = 0; for (uint64_t i = 0; i < R; ++i) s += f(a[0])[i * N + j]; f(a[1])[j] = (float)s; }
      return ZYXB_OK;
    }
    case ZYXB_RR_MSE: {
      double s = 0;
      for (uint64_t i = 0; i < R * N; ++i) { const double e = (double)f(a[0])[i] - f(a[1])[i]; s += e * e; }
      f(a[2])[0] = (float)(s / (double)(R * N));
      return ZYXB_OK;
    }
    case ZYXB_RR_CROSS_ENTROPY: case ZYXB_RR_CROSS_ENTROPY_BWD: {
      const int32_t* lab = (const int32_t*)a[1]->ptr;
      double mean = 0;
      for (uint64_t i = 0; i < R; ++i) {
        const float* x = f(a[0]) + i * N;
        double mx = x[0], s = 0;
        for (uint64_t j = 1; j < N; ++j) mx = x[j] > mx ? x[j] : mx;
        for (uint64_t j = 0; j < N; ++j) s += exp(x[j] - mx);
        if (d.op == ZYXB_RR_CROSS_ENTROPY) { const double l = -(x[lab[i]] - mx - log(s)); f(a[2])[i] = (float)l; mean += l; }
        else for (uint64_t j = 0; j < N; ++j) f(a[2])[i * N + j] = (float)((exp(x[j] - mx) / s - (j == (uint64_t)lab[i])) / (double)R);
      }
      if (d.op == ZYXB_RR_CROSS_ENTROPY) f(a[3])[0] = (float)(mean / (double)R);
      return ZYXB_OK;
    }
    default: return fail(c, ZYXB_ERR_KERNEL_LAUNCH, "fake: row op not implemented");
  }
}

int run_optim(zyxb_ctx* c, Prog& P, std::vector<Buf*>& a) {
  const zyxb_optim_desc& o = P.d.u.optim;
  const int n = o.n_tensors;
  const double gs = o.grad_scale == 0 ? 1.0 : o.grad_scale;
  const uint64_t t = P.step + 1;
  for (int i = 0; i < n; ++i) {
    float *p = f(a[i]), *g = f(a[n + i]);
    for (uint64_t e = 0; e < P.numel[i]; ++e) {
      double gr = g[e] * gs;
      if (o.algo == ZYXB_OPT_SGD) { if (o.weight_decay != 0) gr += p[e] * (double)o.weight_decay; p[e] = (float)(p[e] - gr * o.lr); continue; }
      float *m = f(a[2 * n + i]), *v = f(a[3 * n + i]);
      const double m1 = (t == 1 ? 0.0 : m[e] * (double)o.beta1) + gr * (1.0 - o.beta1), v1 = (t == 1 ? 0.0 : v[e] * (double)o.beta2) + gr * gr * (1.0 - o.beta2);
      m[e] = (float)m1; v[e] = (float)v1;
      const double mh = m1 / (1 - pow(o.beta1, (double)t)), vh = v1 / (1 - pow(o.beta2, (double)t));
      double q = o.standard ? p[e] - o.lr * mh / (sqrt(vh) + o.eps) : p[e] - mh / ((sqrt(vh) + o.eps) * o.lr);
      if (o.algo == ZYXB_OPT_ADAMW && o.weight_decay != 0) q *= 1.0 - (double)o.lr * o.weight_decay;
      p[e] = (float)q;
    }
  }
  return ZYXB_OK;
}
}  // namespace

extern "C" {
#pragma GCC visibility push(default)
// ---- test controls (not part of zyxb.h) ----
void zyxb_fake_set_collective(allreduce_cb cb) { g_cb = cb; }
void zyxb_fake_fail(int32_t kind, int64_t after_n_calls) { if (kind >= 0 && kind < 3) g_fail_at[kind] = after_n_calls; }
uint64_t zyxb_fake_calls(int32_t kind) { return kind >= 0 && kind < 3 ? g_calls[kind] : 0; }

int32_t zyxb_init(const zyxb_config*, zyxb_ctx** out) { *out = new zyxb_ctx(); return ZYXB_OK; }
int32_t zyxb_shutdown(zyxb_ctx* c) { delete c; return ZYXB_OK; }
const char* zyxb_last_error(zyxb_ctx* c) { return c ? c->err.c_str() : ""; }
int32_t zyxb_device_count(zyxb_ctx*, int32_t* n) { *n = 1; return ZYXB_OK; }
int32_t zyxb_device_info(zyxb_ctx*, int32_t, zyxb_devinfo* o) { memset(o, 0, sizeof *o); strcpy(o->name, "host-memory fake"); return ZYXB_OK; }
int32_t zyxb_free_compute(zyxb_ctx*, int32_t, uint64_t* o) { *o = 1; return ZYXB_OK; }
int32_t zyxb_free_bytes(zyxb_ctx*, int32_t, uint64_t* o) { *o = 1ull << 40; return ZYXB_OK; }

int32_t zyxb_alloc(zyxb_ctx* c, int32_t, uint64_t bytes, uint32_t* out, zyxb_event* ev) {
  if (injected(0)) return fail(c, ZYXB_ERR_MEMORY_ALLOCATION, "cudaMalloc: out of memory (injected)");
  c->bufs.emplace_back();
  Buf& b = c->bufs.back();
  b.own.assign(bytes ? bytes : 1, 0xAB);      // uninitialised memory is not zero
  b.ptr = b.own.data(); b.bytes = bytes; b.live = true;
  *out = (uint32_t)c->bufs.size() - 1;
  if (ev) ev->id = 0;
  return ZYXB_OK;
}
int32_t zyxb_free(zyxb_ctx* c, int32_t, uint32_t id, const zyxb_event*, int32_t) {
  Buf* b = get(c, id);
  if (!b) return fail(c, ZYXB_ERR_MEMORY_DEALLOCATION, "free: unknown buffer");
  *b = Buf();
  return ZYXB_OK;
}
int32_t zyxb_buffer_view(zyxb_ctx* c, int32_t, uint32_t parent, uint64_t off, uint64_t bytes, uint32_t* out) {
  Buf* p = get(c, parent);
  if (!p || off % 256 || off + bytes > p->bytes) return fail(c, ZYXB_ERR_MEMORY_ALLOCATION, "buffer_view: bad range");
  uint8_t* ptr = p->ptr + off;
  c->bufs.emplace_back();
  Buf& b = c->bufs.back();
  b.ptr = ptr; b.bytes = bytes; b.live = true;
  *out = (uint32_t)c->bufs.size() - 1;
  return ZYXB_OK;
}
int32_t zyxb_buffer_bytes(zyxb_ctx* c, int32_t, uint32_t id, uint64_t* out) { Buf* b = get(c, id); if (!b) return fail(c, ZYXB_ERR_INCORRECT_KERNEL_ARG, "unknown buffer"); *out = b->bytes; return ZYXB_OK; }
int32_t zyxb_h2d(zyxb_ctx* c, int32_t, const void* src, uint64_t n, uint32_t dst, uint64_t off, const zyxb_event*, int32_t, zyxb_event* ev) {
  Buf* b = get(c, dst);
  if (!b || off + n > b->bytes) return fail(c, ZYXB_ERR_MEMORY_COPY_H2P, "h2d: bad range");
  memcpy(b->ptr + off, src, n);
  if (ev) ev->id = c->next_event++;
  return ZYXB_OK;
}
int32_t zyxb_d2h(zyxb_ctx* c, int32_t, uint32_t src, uint64_t off, void* dst, uint64_t n, const zyxb_event*, int32_t) {
  Buf* b = get(c, src);
  if (!b || off + n > b->bytes) return fail(c, ZYXB_ERR_MEMORY_COPY_P2H, "d2h: bad range");
  memcpy(dst, b->ptr + off, n);
  return ZYXB_OK;
}
int32_t zyxb_d2d(zyxb_ctx* c, int32_t, uint32_t src, uint64_t so, int32_t, uint32_t dst, uint64_t dof, uint64_t n, const zyxb_event*, int32_t, zyxb_event* ev) {
  Buf *s = get(c, src), *d = get(c, dst);
  if (!s || !d || so + n > s->bytes || dof + n > d->bytes) return fail(c, ZYXB_ERR_MEMORY_COPY_H2P, "d2d: bad range");
  memmove(d->ptr + dof, s->ptr + so, n);
  if (ev) ev->id = c->next_event++;
  return ZYXB_OK;
}
int32_t zyxb_memset(zyxb_ctx* c, int32_t, uint32_t id, uint64_t off, int32_t v, uint64_t n) {
  Buf* b = get(c, id);
  if (!b || off + n > b->bytes) return fail(c, ZYXB_ERR_MEMORY_COPY_H2P, "memset: bad range");
  memset(b->ptr + off, v, n);
  return ZYXB_OK;
}
int32_t zyxb_sync(zyxb_ctx*, int32_t, const zyxb_event*, int32_t) { return ZYXB_OK; }
int32_t zyxb_release_events(zyxb_ctx*, int32_t, const zyxb_event*, int32_t) { return ZYXB_OK; }
int32_t zyxb_device_sync(zyxb_ctx*, int32_t) { return ZYXB_OK; }
int32_t zyxb_store_variable(zyxb_ctx* c, int32_t, int32_t, const void*, uint32_t*) { return fail(c, ZYXB_ERR_MEMORY_ALLOCATION, "fake: no variables"); }
int32_t zyxb_get_variable(zyxb_ctx* c, int32_t, uint32_t, int32_t*, void*) { return fail(c, ZYXB_ERR_MEMORY_ALLOCATION, "fake: no variables"); }
int32_t zyxb_host_register(zyxb_ctx*, void*, uint64_t) { return ZYXB_OK; }
int32_t zyxb_host_unregister(zyxb_ctx*, void*) { return ZYXB_OK; }

int32_t zyxb_program_create(zyxb_ctx* c, int32_t, const zyxb_kernel_desc* d, uint32_t* out) {
  c->progs.emplace_back();
  Prog& P = c->progs.back();
  P.d = *d; P.live = true;
  if (d->kind == ZYXB_KIND_OPTIM) { P.numel.assign(d->u.optim.numel, d->u.optim.numel + d->u.optim.n_tensors); P.d.u.optim.numel = nullptr; }
  *out = (uint32_t)c->progs.size() - 1;
  return ZYXB_OK;
}
int32_t zyxb_program_release(zyxb_ctx* c, int32_t, uint32_t p) { if (p && p < c->progs.size()) c->progs[p].live = false; return ZYXB_OK; }
int32_t zyxb_program_set_step(zyxb_ctx* c, int32_t, uint32_t p, uint64_t t) { c->progs[p].step = t; return ZYXB_OK; }
int32_t zyxb_program_get_step(zyxb_ctx* c, int32_t, uint32_t p, uint64_t* t) { *t = c->progs[p].step; return ZYXB_OK; }

int32_t zyxb_launch(zyxb_ctx* c, int32_t, uint32_t prog, const uint32_t* args, int32_t n, const zyxb_event*, int32_t, zyxb_event* ev) {
  if (!prog || prog >= c->progs.size() || !c->progs[prog].live) return fail(c, ZYXB_ERR_KERNEL_LAUNCH, "launch: unknown program");
  if (injected(1)) return fail(c, ZYXB_ERR_KERNEL_LAUNCH, "cudaLaunchKernel: unspecified launch failure (injected)");
  Prog& P = c->progs[prog];
  std::vector<Buf*> a;
  for (int i = 0; i < n; ++i) { Buf* b = get(c, args[i]); if (!b) return fail(c, ZYXB_ERR_INCORRECT_KERNEL_ARG, "launch: argument is not a pool buffer"); a.push_back(b); }
  int st;
  switch (P.d.kind) {
    case ZYXB_KIND_GEMM: st = run_gemm(c, P.d.u.gemm, a); break;
    case ZYXB_KIND_ROWREDUCE: st = run_row(c, P.d.u.rowreduce, a); break;
    case ZYXB_KIND_ELTWISE: {
      const zyxb_eltwise_desc& e = P.d.u.eltwise;
      if (e.op != ZYXB_EW_MSE_BWD) return fail(c, ZYXB_ERR_KERNEL_LAUNCH, "fake: eltwise op not implemented");
      for (uint64_t i = 0; i < e.numel; ++i) f(a[2])[i] = (float)(2.0 * ((double)f(a[0])[i] - f(a[1])[i]) * e.p0);
      st = ZYXB_OK; break;
    }
    case ZYXB_KIND_OPTIM: st = run_optim(c, P, a); if (!st) P.step++; break;
    default: st = fail(c, ZYXB_ERR_KERNEL_LAUNCH, "fake: kind not implemented");
  }
  if (st) return st;
  c->launches++;
  if (ev) ev->id = c->next_event++;
  return ZYXB_OK;
}
int32_t zyxb_launch_count(zyxb_ctx* c, int32_t, uint64_t* o) { *o = c->launches; return ZYXB_OK; }
int32_t zyxb_device_status(zyxb_ctx*, int32_t, uint32_t* o) { if (o) *o = 0; return ZYXB_OK; }
int32_t zyxb_check_guards(zyxb_ctx*, int32_t, uint32_t* o) { if (o) *o = 0; return ZYXB_OK; }
int32_t zyxb_selftest_bounded_wait(zyxb_ctx* c, int32_t, uint64_t, uint32_t*) { return fail(c, ZYXB_ERR_KERNEL_LAUNCH, "fake: no kernels"); }
int32_t zyxb_capture_begin(zyxb_ctx* c, int32_t) { return fail(c, ZYXB_ERR_KERNEL_LAUNCH, "fake: no captures"); }
int32_t zyxb_capture_end(zyxb_ctx* c, int32_t, uint32_t*) { return fail(c, ZYXB_ERR_KERNEL_LAUNCH, "fake: no captures"); }
int32_t zyxb_graph_launch(zyxb_ctx* c, int32_t, uint32_t, const zyxb_event*, int32_t, zyxb_event*) { return fail(c, ZYXB_ERR_KERNEL_LAUNCH, "fake: no captures"); }
int32_t zyxb_graph_release(zyxb_ctx*, int32_t, uint32_t) { return ZYXB_OK; }
int32_t zyxb_colsum_static(zyxb_ctx* c, int32_t, int32_t, uint32_t, uint32_t, uint64_t, uint64_t) { return fail(c, ZYXB_ERR_KERNEL_LAUNCH, "fake: not implemented"); }
int32_t zyxb_colsum_static_capacity(uint64_t* o) { *o = 0; return ZYXB_OK; }
int32_t zyxb_event_record(zyxb_ctx* c, int32_t, zyxb_event* ev) { ev->id = c->next_event++; return ZYXB_OK; }
int32_t zyxb_event_elapsed_ms(zyxb_ctx*, int32_t, zyxb_event, zyxb_event, float* ms) { *ms = 0; return ZYXB_OK; }
int32_t zyxb_flush_l2(zyxb_ctx*, int32_t) { return ZYXB_OK; }

int32_t zyxb_comm_unique_id(zyxb_ctx*, void* out) { memset(out, 7, 128); return ZYXB_OK; }
int32_t zyxb_comm_init(zyxb_ctx* c, int32_t, int32_t rank, int32_t world, const void*) { c->rank = rank; c->world = world; c->comm = true; return ZYXB_OK; }
int32_t zyxb_comm_rank(zyxb_ctx* c, int32_t, int32_t* r, int32_t* w) { if (!c->comm) return fail(c, ZYXB_ERR_INCORRECT_KERNEL_ARG, "no communicator"); *r = c->rank; *w = c->world; return ZYXB_OK; }
int32_t zyxb_comm_destroy(zyxb_ctx* c, int32_t) { c->comm = false; return ZYXB_OK; }
int32_t zyxb_comm_option(zyxb_ctx*, int32_t, int32_t, int32_t) { return ZYXB_OK; }
static int32_t collective(zyxb_ctx* c, uint32_t buf, uint64_t off, uint64_t count, int32_t dtype, int32_t op, zyxb_event* ev, const char* what) {
  Buf* b = get(c, buf);
  if (!c->comm) return fail(c, ZYXB_ERR_INCORRECT_KERNEL_ARG, std::string(what) + ": no communicator");
  if (!b || dtype != ZYXB_F32 || (off + count * (op ? (uint64_t)c->world : 1)) * 4 > b->bytes) return fail(c, ZYXB_ERR_INCORRECT_KERNEL_ARG, std::string(what) + ": bad range");
  if (injected(2)) return fail(c, ZYXB_ERR_KERNEL_LAUNCH, std::string(what) + ": ncclSystemError (injected)");
  if (!g_cb) return fail(c, ZYXB_ERR_KERNEL_LAUNCH, std::string(what) + ": no collective callback installed");
  const int32_t st = g_cb(b->ptr + off * 4, count, dtype, op);
  if (st) return fail(c, ZYXB_ERR_KERNEL_LAUNCH, std::string(what) + ": the collective failed (a peer left or timed out)");
  if (ev) ev->id = c->next_event++;
  return ZYXB_OK;
}
int32_t zyxb_allreduce_sum(zyxb_ctx* c, int32_t, uint32_t buf, uint64_t off, uint64_t count, int32_t dt, const zyxb_event*, int32_t, zyxb_event* ev) { return collective(c, buf, off, count, dt, 0, ev, "allreduce"); }
int32_t zyxb_reduce_scatter_sum(zyxb_ctx* c, int32_t, uint32_t buf, uint64_t off, uint64_t count, int32_t dt, const zyxb_event*, int32_t, zyxb_event* ev) { return collective(c, buf, off, count, dt, 1, ev, "reduce_scatter"); }
int32_t zyxb_allgather(zyxb_ctx* c, int32_t, uint32_t buf, uint64_t off, uint64_t count, int32_t dt, const zyxb_event*, int32_t, zyxb_event* ev) { return collective(c, buf, off, count, dt, 2, ev, "allgather"); }
#pragma GCC visibility pop
}
