// C ABI of the pattern matcher (include/zyxb_host.h, "e-graph matcher"): a mirror of zyx's graph is built node by node, then
// zyxb_mgraph_match plays the device's match_graph (zyx/src/backend/mod.rs:952-961) over it and returns, per matched
// subgraph, the kernel descriptor and the launch arguments (input classes, then output classes).
#include "matcher.hpp"

#include "../../../include/zyxb_host.h"

using zyxb_matcher::Graph;
using zyxb_matcher::Node;

struct zyxb_mgraph {
  Graph g;
  std::vector<zyxb_matcher::Match> matches;    // keeps the optimizer descriptors' numel arrays alive
};

namespace {
bool ok_class(zyxb_mgraph* G, uint32_t c) { return G && G->g.valid(c); }
uint32_t push(zyxb_mgraph* G, const Node& n) { return G->g.add(n); }
}  // namespace

extern "C" {
#pragma GCC visibility push(default)

int32_t zyxb_mgraph_create(zyxb_mgraph** out) {
  if (!out) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  *out = new zyxb_mgraph();
  return ZYXB_OK;
}
int32_t zyxb_mgraph_destroy(zyxb_mgraph* G) { delete G; return ZYXB_OK; }

uint32_t zyxb_mgraph_const(zyxb_mgraph* G, int32_t dtype, double value) {
  if (!G) return zyxb_matcher::NONE;
  Node n; n.kind = zyxb_matcher::K_CONST; n.dtype = dtype; n.value = value;
  return push(G, n);
}
uint32_t zyxb_mgraph_leaf(zyxb_mgraph* G, int32_t dtype, uint32_t leaf_id, const uint64_t* shape, int32_t rank) {
  if (!G || rank < 0 || (rank > 0 && !shape)) return zyxb_matcher::NONE;
  Node n; n.kind = zyxb_matcher::K_LEAF; n.dtype = dtype; n.leaf_id = leaf_id; n.shape.assign(shape, shape + rank);
  return push(G, n);
}
static uint32_t shaped(zyxb_mgraph* G, int kind, uint32_t x, const uint64_t* shape, int32_t rank) {
  if (!ok_class(G, x) || rank < 0 || (rank > 0 && !shape)) return zyxb_matcher::NONE;
  Node n; n.kind = kind; n.x = x; n.shape.assign(shape, shape + rank);
  const auto& xs = G->g.shape(x);
  if (kind == zyxb_matcher::K_RESHAPE && Graph::numel(xs) != Graph::numel(n.shape)) return zyxb_matcher::NONE;
  if (kind == zyxb_matcher::K_EXPAND) {      // numpy broadcasting from the trailing axes
    if (xs.size() > n.shape.size()) return zyxb_matcher::NONE;
    for (size_t i = 0; i < xs.size(); ++i) {
      const uint64_t a = xs[xs.size() - 1 - i], b = n.shape[n.shape.size() - 1 - i];
      if (a != b && a != 1) return zyxb_matcher::NONE;
    }
  }
  return push(G, n);
}
uint32_t zyxb_mgraph_expand(zyxb_mgraph* G, uint32_t x, const uint64_t* shape, int32_t rank) { return shaped(G, zyxb_matcher::K_EXPAND, x, shape, rank); }
uint32_t zyxb_mgraph_reshape(zyxb_mgraph* G, uint32_t x, const uint64_t* shape, int32_t rank) { return shaped(G, zyxb_matcher::K_RESHAPE, x, shape, rank); }
uint32_t zyxb_mgraph_permute(zyxb_mgraph* G, uint32_t x, const int32_t* axes, int32_t rank) {
  if (!ok_class(G, x) || !axes || rank != (int32_t)G->g.shape(x).size()) return zyxb_matcher::NONE;
  Node n; n.kind = zyxb_matcher::K_PERMUTE; n.x = x;
  std::vector<char> seen(rank, 0);
  for (int i = 0; i < rank; ++i) { if (axes[i] < 0 || axes[i] >= rank || seen[axes[i]]) return zyxb_matcher::NONE; seen[axes[i]] = 1; n.axes.push_back(axes[i]); }
  return push(G, n);
}
uint32_t zyxb_mgraph_reduce(zyxb_mgraph* G, uint32_t x, int32_t rop, const int32_t* axes, int32_t n_axes) {
  if (!ok_class(G, x) || !axes || n_axes < 1) return zyxb_matcher::NONE;
  Node n; n.kind = zyxb_matcher::K_REDUCE; n.x = x; n.op = rop;
  for (int i = 0; i < n_axes; ++i) { if (axes[i] < 0 || axes[i] >= (int32_t)G->g.shape(x).size()) return zyxb_matcher::NONE; n.axes.push_back(axes[i]); }
  return push(G, n);
}
uint32_t zyxb_mgraph_pad(zyxb_mgraph* G, uint32_t x, int32_t axis, int64_t lp, uint64_t len) {
  if (!ok_class(G, x) || axis < 0 || axis >= (int32_t)G->g.shape(x).size()) return zyxb_matcher::NONE;
  // what is cut off on either side has to leave something of the axis (Tensor::pad_axis, tensor/mod.rs:1126-1138)
  const int64_t orig = (int64_t)G->g.shape(x)[axis], rp = (int64_t)len - lp - orig;
  if ((int64_t)len < 0 || (lp < 0 ? -lp : 0) + (rp < 0 ? -rp : 0) >= orig) return zyxb_matcher::NONE;
  Node n; n.kind = zyxb_matcher::K_PAD; n.x = x; n.axes = {axis}; n.lp = lp; n.len = len;
  return push(G, n);
}
uint32_t zyxb_mgraph_cast(zyxb_mgraph* G, uint32_t x, int32_t dtype) {
  if (!ok_class(G, x)) return zyxb_matcher::NONE;
  Node n; n.kind = zyxb_matcher::K_CAST; n.x = x; n.dtype = dtype;
  return push(G, n);
}
uint32_t zyxb_mgraph_unary(zyxb_mgraph* G, uint32_t x, int32_t uop) {
  if (!ok_class(G, x)) return zyxb_matcher::NONE;
  Node n; n.kind = zyxb_matcher::K_UNARY; n.x = x; n.op = uop;
  return push(G, n);
}
uint32_t zyxb_mgraph_binary(zyxb_mgraph* G, uint32_t x, uint32_t y, int32_t bop) {
  if (!ok_class(G, x) || !ok_class(G, y) || G->g.shape(x) != G->g.shape(y) || G->g.dtype(x) != G->g.dtype(y)) return zyxb_matcher::NONE;
  Node n; n.kind = zyxb_matcher::K_BINARY; n.x = x; n.y = y; n.op = bop;
  return push(G, n);
}

int32_t zyxb_mgraph_class_info(zyxb_mgraph* G, uint32_t c, int32_t* out_dtype, int32_t* out_rank, uint64_t* out_shape8, int32_t* out_kernel_nodes) {
  if (!ok_class(G, c)) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  const auto& cl = G->g.classes[c];
  if (out_dtype) *out_dtype = cl.dtype;
  if (out_rank) *out_rank = (int32_t)cl.shape.size();
  if (out_shape8) for (size_t i = 0; i < cl.shape.size() && i < 8; ++i) out_shape8[i] = cl.shape[i];
  if (out_kernel_nodes) {
    int k = 0;
    for (uint32_t nid : cl.nodes) k += G->g.nodes[nid].kind == zyxb_matcher::K_KERNEL;
    *out_kernel_nodes = k;
  }
  return ZYXB_OK;
}

int32_t zyxb_mgraph_uncovered(zyxb_mgraph* G, const uint32_t* outputs, int32_t n_outputs, uint32_t* out, int32_t capacity, int32_t* out_n) {
  if (!G || !outputs || n_outputs < 1 || !out_n) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  std::vector<uint32_t> outs(outputs, outputs + n_outputs);
  for (uint32_t o : outs) if (!G->g.valid(o)) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  const auto missing = G->g.uncovered(outs);
  *out_n = (int32_t)missing.size();
  for (size_t i = 0; i < missing.size() && (int32_t)i < capacity && out; ++i) out[i] = missing[i];
  return ZYXB_OK;
}

int32_t zyxb_mgraph_const_value(zyxb_mgraph* G, uint32_t c, double* out, uint64_t capacity, uint64_t* out_n) {
  if (!ok_class(G, c) || !out_n) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  auto v = G->g.const_eval(c);
  if (!v) { *out_n = 0; return ZYXB_ERR_INCORRECT_KERNEL_ARG; }
  *out_n = v->size();
  for (uint64_t i = 0; i < v->size() && i < capacity && out; ++i) out[i] = (*v)[i];
  return ZYXB_OK;
}

int32_t zyxb_mgraph_match(zyxb_mgraph* G, const uint32_t* outputs, int32_t n_outputs, zyxb_match* out, int32_t capacity, int32_t* out_n) {
  if (!G || !outputs || n_outputs < 1 || !out_n) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  std::vector<uint32_t> outs(outputs, outputs + n_outputs);
  for (uint32_t o : outs) if (!G->g.valid(o)) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  std::set<uint32_t> wanted(outs.begin(), outs.end());
  auto found = G->g.match_graph(G->g.topo_order(outs), wanted);
  *out_n = (int32_t)found.size();
  const size_t base = G->matches.size();
  for (auto& m : found) G->matches.push_back(std::move(m));
  for (size_t i = 0; i < found.size() && (int32_t)i < capacity && out; ++i) {
    const zyxb_matcher::Match& m = G->matches[base + i];
    zyxb_match& o = out[i];
    memset(&o, 0, sizeof o);
    snprintf(o.pattern, sizeof o.pattern, "%s", m.pattern.c_str());
    if (m.inputs.size() > 128 || m.outputs.size() > 96) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
    o.n_inputs = (int32_t)m.inputs.size(); o.n_outputs = (int32_t)m.outputs.size();
    for (size_t j = 0; j < m.inputs.size(); ++j) o.inputs[j] = m.inputs[j];
    for (size_t j = 0; j < m.outputs.size(); ++j) o.outputs[j] = m.outputs[j];
    o.desc = m.desc;
    if (o.desc.kind == ZYXB_KIND_OPTIM) o.desc.u.optim.numel = m.numel.data();   // owned by the graph mirror until it is destroyed
    o.optim_step = m.optim_step;
    for (size_t j = 0; j < m.input_offsets.size() && j < 128; ++j) o.input_offsets[j] = m.input_offsets[j];
  }
  return ZYXB_OK;
}

#pragma GCC visibility pop
}  // extern "C"
