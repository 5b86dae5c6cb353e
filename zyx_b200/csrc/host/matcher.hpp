// Pattern matcher: zyx e-graph subgraphs -> kernel descriptors (the `match_graph` half of the backend boundary).
//
// zyx's graph op set is tiny (zyx/src/graph/mod.rs:100-182: Const, Leaf, Expand, Permute, Reshape, Reduce, Cast, Unary,
// Binary, ..., Kernel), so whatever the user wrote collapses into a few canonical subgraphs (zyx/src/vendor/mod.rs:4-13).
// The reference recognises one of them, the 2-D NN matmul (Graph::match_matmul, zyx/src/vendor/matmul.rs:43-71, helpers
// vendor/mod.rs:28-95), and its consumer pushes a Node::Kernel into the matched class (backend/cblas.rs:213-238).  This file
// is the same machinery over a mirror of that graph, extended to what an aot_only device must cover:
//   matmul          NN as the reference; NT on a stored weight (`x.dot(W.t())` of Linear::forward, zyx-nn/src/linear.rs:39-45,
//                   where the reference would hand the kernel the *class* W.t()); TN / TT when the left operand is `x.t()` of
//                   a stored tensor (a weight gradient written as `dz.t().dot(x)`); rank > 2 with batch strides, a right
//                   operand shared by the whole batch folding the batch into the rows; per-head
//                   views of stored [b, t, h*d] tensors as operands and as the merged result (no [b, h, t, d] copies); the
//                   accumulator Casts that `sum` puts around the Reduce for 16-bit inputs (tensor/reduce_ops.rs:52-60,143-145);
//                   a trailing `* const` (attention's 1/sqrt(d)) as alpha; `+ bias`, relu and gelu as epilogues; `+ residual`
//                   (a whole tensor of the product's shape) on a product without bias
//   convolution     Tensor::conv with groups = 1 (tensor/mod.rs:2583-2680), recognised by what its pooling view reads
//   attention       the mask-free core of MultiheadAttention::forward (zyx-nn/src/multi_head_attention.rs:197-226)
//   row kernels     softmax, ln_softmax (tensor/mod.rs:1427-1461), LayerNorm::forward (zyx-nn/src/layer_norm.rs:95-135),
//                   sum / max / min / mean / var / std over the last axis (tensor/reduce_ops.rs:45-157), `sum([0])` of a matrix
//                   (column sums), mse_loss of f32 tensors, cross_entropy of f32 logits with i32 class indices
//                   (tensor/mod.rs:1639-1656; its one-hot compares against an arange recognised by constant folding)
//   elementwise     relu, gelu, tanh, sigmoid, exp, float casts, * const, + - * of whole tensors, + bias (tensor/elementwise.rs),
//                   on demand: for outputs of the graph and inputs of matched programs that nothing produces yet
//   optimizer       SGD::update (zyx-optim/src/sgd.rs:45-84: plain, weight decay, momentum with dampening, Nesterov),
//                   Adam::update (zyx-optim/src/adam.rs, without amsgrad), AdamW::update (zyx-optim/src/adamw.rs:51-97), first
//                   and later steps, all matched tensors of one update grouped into one multi-tensor program
// A Rust port of this file is what `backend/b200.rs` carries; the mirror exists because the image has no Rust toolchain
// and the matcher has to be testable on the CPU.  Symbolic (non-constant) shapes never match, as in the reference
// (Graph::const_shape returns None).
#pragma once
#include <math.h>
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <cmath>
#include <tuple>
#include <optional>
#include <set>
#include <string>
#include <utility>
#include <vector>

#include "../../../include/zyxb.h"

namespace zyxb_matcher {

using ClassId = uint32_t;
constexpr ClassId NONE = 0xffffffffu;

enum Kind : int { K_CONST = 0, K_LEAF, K_EXPAND, K_PERMUTE, K_RESHAPE, K_REDUCE, K_CAST, K_UNARY, K_BINARY, K_KERNEL, K_PAD };
// the order of zyx's enums (zyx/src/kernel/ops.rs:187-214 and 222-262)
enum UOp : int { U_NEG = 0, U_BITNOT, U_EXP, U_EXP2, U_LN, U_LOG2, U_RECIPROCAL, U_SQRT, U_SIN, U_COS, U_FLOOR, U_TRUNC, U_ABS };
enum BOp : int { B_ADD = 0, B_SUB, B_MUL, B_DIV, B_POW, B_MOD, B_CMPLT, B_CMPGT, B_CMPGE, B_MAX, B_OR, B_AND, B_BITXOR, B_BITOR, B_BITAND,
                 B_SHL, B_SHR, B_NOTEQ, B_EQ };

struct Node {
  int kind = K_CONST;
  ClassId x = NONE, y = NONE;
  int op = 0;                    // UOp / BOp / reduce BOp
  int dtype = ZYXB_F32;          // Const, Leaf, Cast
  double value = 0.0;            // Const
  uint32_t leaf_id = 0;
  std::vector<uint64_t> shape;   // Leaf, Expand, Reshape
  std::vector<int> axes;         // Permute, Reduce; Pad: the one padded axis
  int64_t lp = 0;                // Pad: zeros in front of the axis (negative: that many elements cut off)
  uint64_t len = 0;              // Pad: extent of the axis afterwards (zyx/src/graph/mod.rs:121-129)
  std::vector<ClassId> inputs, outputs;   // Kernel
  uint32_t program = 0;          // Kernel: index of the match (ProgramId once a device created the program)
  uint64_t time = 0;
};

struct Class {
  std::vector<uint32_t> nodes;   // node ids; nodes[0] defines shape and dtype, as Graph::shape / Graph::dtype read it
  std::vector<uint64_t> shape;
  int dtype = ZYXB_F32;
};

struct Match {
  std::string pattern;
  std::vector<ClassId> inputs, outputs;   // launch arguments: loads, then stores (Device::launch, backend/mod.rs:974)
  zyxb_kernel_desc desc{};
  std::vector<uint64_t> numel;            // optimizer: desc.u.optim.numel points here
  uint64_t optim_step = 0;                // optimizer: the step t of the matched update (the program's counter must be t - 1 before the launch)
  std::vector<uint64_t> input_offsets;    // per input: the element the program's argument starts at inside that class's buffer (empty: all 0)
};

inline bool is_float(int dt) { return dt == ZYXB_F32 || dt == ZYXB_BF16 || dt == ZYXB_F16 || dt == ZYXB_F64; }

class Graph {
 public:
  std::vector<Node> nodes;
  std::vector<Class> classes;

  // ---- construction: one class per distinct node (the e-graph's hash-consing) --------------------------------------
  ClassId add(const Node& n) {
    const std::string key = key_of(n);
    auto it = memo_.find(key);
    if (it != memo_.end()) return it->second;
    Class c;
    switch (n.kind) {
      case K_CONST: c.dtype = n.dtype; break;
      case K_LEAF: c.dtype = n.dtype; c.shape = n.shape; break;
      case K_EXPAND: case K_RESHAPE: c.dtype = classes[n.x].dtype; c.shape = n.shape; break;
      case K_PERMUTE: c.dtype = classes[n.x].dtype; for (int a : n.axes) c.shape.push_back(classes[n.x].shape[a]); break;
      case K_REDUCE: {
        c.dtype = classes[n.x].dtype;
        const auto& s = classes[n.x].shape;
        for (size_t i = 0; i < s.size(); ++i) if (std::find(n.axes.begin(), n.axes.end(), (int)i) == n.axes.end()) c.shape.push_back(s[i]);
        break;
      }
      case K_CAST: c.dtype = n.dtype; c.shape = classes[n.x].shape; break;
      case K_PAD: c.dtype = classes[n.x].dtype; c.shape = classes[n.x].shape; c.shape[n.axes[0]] = n.len; break;
      case K_UNARY: c.dtype = classes[n.x].dtype; c.shape = classes[n.x].shape; break;
      case K_BINARY:
        c.dtype = (n.op == B_CMPLT || n.op == B_CMPGT || n.op == B_CMPGE || n.op == B_NOTEQ || n.op == B_EQ) ? ZYXB_BOOL : classes[n.x].dtype;
        c.shape = classes[n.x].shape;
        break;
      default: break;
    }
    nodes.push_back(n);
    c.nodes.push_back((uint32_t)nodes.size() - 1);
    classes.push_back(std::move(c));
    const ClassId id = (ClassId)classes.size() - 1;
    memo_[key] = id;
    return id;
  }
  bool valid(ClassId c) const { return c < classes.size(); }

  // ---- helpers, in the style of vendor/mod.rs:28-95 ---------------------------------------------------------------------
  const std::vector<uint64_t>& shape(ClassId c) const { return classes[c].shape; }
  int dtype(ClassId c) const { return classes[c].dtype; }
  static uint64_t numel(const std::vector<uint64_t>& s) { uint64_t n = 1; for (uint64_t d : s) n *= d; return n; }

  // A node of class c that satisfies pred.  In graph mode every `.cast(dtype)` pushes a Cast node, also when the dtype does
  // not change (zyx/src/runtime.rs:696-700), so a class may be a no-op Cast of the class that holds the node looked for:
  // those are looked through.
  template <class F> const Node* find(ClassId c, F pred) const {
    for (int depth = 0; depth < 8; ++depth) {
      for (uint32_t nid : classes[c].nodes) if (pred(nodes[nid])) return &nodes[nid];
      const Node* k = noop_cast(c);
      if (!k) return nullptr;
      c = k->x;
    }
    return nullptr;
  }
  // a node that leaves its operand as it is: a Cast to the dtype the operand has, `x * 1`, `x / 1` (what dropout leaves
  // behind outside training with p = 0: x / (1 - p), tensor/mod.rs:822-828)
  const Node* noop_cast(ClassId c) const {
    for (uint32_t nid : classes[c].nodes) {
      const Node& n = nodes[nid];
      if (n.kind == K_CAST && classes[n.x].dtype == classes[c].dtype) return &n;
      if (n.kind == K_BINARY && (n.op == B_MUL || n.op == B_DIV) && classes[n.x].shape == classes[c].shape && is_float(classes[c].dtype)) {
        ClassId k = n.y;                               // a rank-0 constant 1 under its Cast / Reshape / Expand wrappers
        for (int hops = 0; hops < 8; ++hops) {
          const Node& kn = nodes[classes[k].nodes[0]];
          if (kn.kind == K_CONST) { if (kn.value == 1.0) return &n; break; }
          if (kn.kind != K_CAST && kn.kind != K_EXPAND && kn.kind != K_RESHAPE) break;
          k = kn.x;
        }
      }
    }
    return nullptr;
  }
  ClassId canon(ClassId c) const { while (const Node* k = noop_cast(c)) c = k->x; return c; }
  bool same(ClassId a, ClassId b) const { return canon(a) == canon(b); }
  // The class whose buffer holds c's elements: c under no-op nodes and Reshapes (dense row-major storage does not know its shape).
  // Program inputs are named by it, so that `x.reshape([0, 784])` of a stored batch is the batch's own buffer.
  ClassId storage(ClassId c) const {
    for (int hops = 0; hops < 64; ++hops) {
      c = canon(c);
      const Node* r = find(c, [](const Node& n) { return n.kind == K_RESHAPE; });
      if (!r) break;
      c = r->x;
    }
    return canon(c);
  }
  std::optional<std::pair<ClassId, ClassId>> binary(ClassId c, int bop) const {
    const Node* n = find(c, [&](const Node& n) { return n.kind == K_BINARY && n.op == bop; });
    if (!n) return std::nullopt;
    return std::make_pair(n->x, n->y);
  }
  std::optional<ClassId> unary(ClassId c, int uop) const {
    const Node* n = find(c, [&](const Node& n) { return n.kind == K_UNARY && n.op == uop; });
    return n ? std::optional<ClassId>(n->x) : std::nullopt;
  }
  std::optional<ClassId> cast_src(ClassId c) const {
    // the source of a dtype-changing Cast (no-op casts are looked through by find)
    const Node* n = find(c, [&](const Node& n) { return n.kind == K_CAST && classes[n.x].dtype != n.dtype; });
    return n ? std::optional<ClassId>(n->x) : std::nullopt;
  }
  std::optional<ClassId> expand_src(ClassId c) const {
    const Node* n = find(c, [](const Node& n) { return n.kind == K_EXPAND; });
    return n ? std::optional<ClassId>(n->x) : std::nullopt;
  }
  std::optional<ClassId> reshape_src(ClassId c) const {
    const Node* n = find(c, [](const Node& n) { return n.kind == K_RESHAPE; });
    return n ? std::optional<ClassId>(n->x) : std::nullopt;
  }
  // the class under any number of Expand / Reshape wrappers (a broadcast operand's source)
  ClassId unbroadcast(ClassId c) const {
    for (;;) {
      if (auto e = expand_src(c)) { c = *e; continue; }
      if (auto r = reshape_src(c)) { c = *r; continue; }
      return c;
    }
  }
  // a scalar constant under Expand / Reshape / Cast wrappers (rank-0 operands are cast to the tensor dtype and expanded,
  // tensor/mod.rs:3033-3113)
  std::optional<double> const_value(ClassId c) const {
    for (;;) {
      if (const Node* n = find(c, [](const Node& n) { return n.kind == K_CONST; })) return n->value;
      if (auto e = expand_src(c)) { c = *e; continue; }
      if (auto r = reshape_src(c)) { c = *r; continue; }
      if (auto k = cast_src(c)) { c = *k; continue; }
      return std::nullopt;
    }
  }
  bool is_const(ClassId c, double v, double rel = 1e-2) const {
    auto k = const_value(c);
    return k && fabs(*k - v) <= rel * fabs(v) + 1e-30;
  }
  // x op const, in either operand order for commutative ops -> (x, const)
  std::optional<std::pair<ClassId, double>> binary_const(ClassId c, int bop) const {
    for (uint32_t nid : classes[c].nodes) {
      const Node& n = nodes[nid];
      if (n.kind != K_BINARY || n.op != bop) continue;
      if (auto k = const_value(n.y)) return std::make_pair(n.x, *k);
      if (bop == B_ADD || bop == B_MUL) if (auto k = const_value(n.x)) return std::make_pair(n.y, *k);
    }
    return std::nullopt;
  }
  // `x.<reduce>_keepdim / <reduce>([-1])` of reduce_impl: [Reshape]{[Cast back]{Reduce{[Cast to acc]{x}, rop, [last]}}} -> x
  std::optional<ClassId> reduce_last(ClassId c, int rop) const {
    if (auto r = reshape_src(c)) if (numel(shape(*r)) == numel(shape(c))) { if (auto x = reduce_last(*r, rop)) return x; }
    ClassId r = c;
    const Node* red = find(r, [&](const Node& n) { return n.kind == K_REDUCE && n.op == rop; });
    if (!red) {
      auto k = cast_src(c);
      if (!k) return std::nullopt;
      r = *k;
      red = find(r, [&](const Node& n) { return n.kind == K_REDUCE && n.op == rop; });
      if (!red) return std::nullopt;
    }
    const size_t rank = shape(red->x).size();
    if (rank < 1 || red->axes.size() != 1 || red->axes[0] != (int)rank - 1) return std::nullopt;
    ClassId x = red->x;
    if (auto k = cast_src(x)) if (dtype(*k) == dtype(c)) x = *k;          // the accumulator cast (undone by the cast back) or a no-op cast
    return canon(x);
  }

  // ---- matmul ------------------------------------------------------------------------------------------------------------
  // a Permute that exchanges the last two axes and leaves the others where they are (`t()`, `transpose(-2, -1)`)
  static bool swaps_last_two(const std::vector<int>& axes) {
    const size_t r = axes.size();
    if (r < 2) return false;
    for (size_t i = 0; i + 2 < r; ++i) if (axes[i] != (int)i) return false;
    return axes[r - 2] == (int)r - 1 && axes[r - 1] == (int)r - 2;
  }
  struct MatMul {
    ClassId a, b, out; uint64_t m, n, k, batch; bool trans_b, b_shared; int dtype; bool trans_a = false;
    // rank-4 products over [b, h, .., ..]: operands (and, at the merged class, the result) that are per-head views of stored
    // [b, t, h*d] tensors are read where they lie through a row pitch and a two-level batch
    uint64_t outer = 0, heads = 0; bool a_heads = false, b_heads = false, c_heads = false;
    // a_heads / b_heads: where the view starts in the stored tensor and how it steps (elements): row pitch, head to head, image to image
    struct Pitch { uint64_t offset = 0, ld = 0, inner = 0, outer = 0; } a_view, b_view;
  };

  // The canonical broadcast-reduce form of Tensor::dot (tensor/mod.rs:1469-1490), ending at class `cid`:
  //   a [.., m, k] -Reshape [.., m, 1, k]-> Expand -+
  //   b [.., k, n] -Permute-> [.., n, k] -Reshape [.., 1, n, k]-> Expand -> Mul -[Cast acc]-> Reduce(Add, last) -[Cast back]-> [.., m, n]
  std::optional<MatMul> match_matmul(ClassId cid) const {
    const auto out_shape = shape(cid);
    if (out_shape.size() < 2) return std::nullopt;
    if (auto r = reshape_src(cid)) if (shape(*r) == out_shape) if (auto mm = match_matmul(*r)) { mm->out = cid; return mm; }  // dot's closing reshape
    const uint64_t m = out_shape[out_shape.size() - 2], n = out_shape.back();
    const Node* red = nullptr;
    ClassId r = cid;
    auto is_red = [](const Node& n) { return n.kind == K_REDUCE && n.op == B_ADD; };
    if (!(red = find(r, is_red))) {
      auto k = cast_src(cid);                                  // sum() casts the f32 accumulator back to the 16-bit input dtype
      if (!k || !(red = find(r = *k, is_red))) return std::nullopt;
    }
    const auto prod_shape = shape(red->x);
    const size_t pr = prod_shape.size();
    if (pr != out_shape.size() + 1 || red->axes.size() != 1 || red->axes[0] != (int)pr - 1) return std::nullopt;
    const uint64_t k = prod_shape.back();
    ClassId prod = red->x;
    auto mul = binary(prod, B_MUL);
    if (!mul) { auto c = cast_src(prod); if (!c || !(mul = binary(*c, B_MUL))) return std::nullopt; }   // the accumulator cast
    // an operand that already has the product's shape (n = 1 on the left, m = 1 on the right) is not expanded (tensor/mod.rs:3099-3107)
    std::optional<ClassId> ea = expand_src(mul->first), eb = expand_src(mul->second);
    if (!ea) ea = mul->first;
    if (!eb) eb = mul->second;
    const auto a3 = shape(*ea), b3 = shape(*eb);
    std::vector<uint64_t> batch_dims(out_shape.begin(), out_shape.end() - 2);
    std::vector<uint64_t> want_a = batch_dims; want_a.insert(want_a.end(), {m, 1, k});
    std::vector<uint64_t> want_b = batch_dims; want_b.insert(want_b.end(), {1, n, k});
    const std::vector<uint64_t> shared_b = {1, n, k};
    bool b_shared = false;
    if (a3 != want_a) return std::nullopt;
    if (b3 != want_b) {
      // one B for every matrix of the batch: [1, n, k], or batch dims of extent 1
      if (numel(b3) == n * k && b3.size() >= 3 && b3[b3.size() - 1] == k && b3[b3.size() - 2] == n && !batch_dims.empty()) b_shared = true;
      else return std::nullopt;
    }
    // a: [.., m, 1, k] has the layout of [.., m, k]; prefer the tensor under the reshape
    ClassId a = *ea;
    if (auto s = reshape_src(a)) if (numel(shape(*s)) == numel(a3)) a = *s;
    // b: through the reshape to the Permute that swaps the last two axes
    ClassId bt = *eb;
    const Node* perm = nullptr;
    for (;;) {
      perm = find(bt, [](const Node& n) { return n.kind == K_PERMUTE && swaps_last_two(n.axes); });
      if (perm) break;
      auto s = reshape_src(bt);
      if (!s) return std::nullopt;
      bt = *s;
    }
    ClassId b = perm->x;                                      // [.., k, n]
    const auto bs = shape(b);
    if (bs.size() < 2 || bs[bs.size() - 2] != k || bs.back() != n) return std::nullopt;
    bool trans_b = false;
    // NT on a stored tensor: b is itself `w.t()` of a [.., n, k] tensor (Linear passes W.t() to dot, which transposes again)
    if (const Node* p2 = find(b, [&](const Node& n) { return n.kind == K_PERMUTE && n.axes == perm->axes; })) { b = p2->x; trans_b = true; }
    // TN on a stored tensor: a is `x.t()` of a [.., k, m] tensor (a weight gradient written as `x.t().dot(dz)`); the kernel
    // reads x where it lies
    bool trans_a = false;
    if (const Node* pa = find(a, [](const Node& n) { return n.kind == K_PERMUTE && swaps_last_two(n.axes); })) {
      const auto as = shape(pa->x);
      if (as.size() >= 2 && as[as.size() - 2] == k && as.back() == m) { a = pa->x; trans_a = true; }
    }
    const int dt = dtype(b);
    if (dtype(a) != dt || dtype(cid) != dt) return std::nullopt;      // C is stored in the operands' dtype; accumulation is f32 / i32
    if (!(dt == ZYXB_F32 || dt == ZYXB_BF16 || dt == ZYXB_F16 || dt == ZYXB_I32)) return std::nullopt;
    MatMul mm{canon(a), canon(b), cid, m, n, k, numel(batch_dims), trans_b, b_shared, dt};
    mm.trans_a = trans_a;
    // one right operand for every matrix of a dense batch (a Linear applied to [b, t, features]): the batch is just more rows
    if (b_shared && !trans_a) { mm.m *= mm.batch; mm.batch = 1; mm.b_shared = false; }
    if (batch_dims.size() == 2 && !b_shared) {      // (b_shared: as the batch was given, folded or not)
      // q / k / v of attention, `x.reshape([b, t, h, d]).transpose(1, 2)` (multi_head_attention.rs:160-172) or the same of a slice
      // of a fused projection (`c_attn.forward(x).split([c, c, c], 2)`, causal_self_attention.rs:39-52): any operand that is a
      // view with unit step along its rows is read where it lies
      for (int which = 0; which < 2; ++which) {
        const ClassId op = which ? b : a;
        auto v = affine_view(op);
        if (!v || v->src == canon(op) || dtype(v->src) != dt || v->strides[3] != 1 || v->strides[2] <= 0 || v->strides[0] < 0 || v->strides[1] < 0) continue;
        if (v->offset * (dt == ZYXB_F32 || dt == ZYXB_I32 ? 4 : 2) % 256 != 0) continue;      // zyxb_buffer_view starts on 256-byte boundaries
        MatMul::Pitch pv{v->offset, (uint64_t)v->strides[2], (uint64_t)v->strides[1], (uint64_t)v->strides[0]};
        if (which) { mm.b = v->src; mm.b_heads = true; mm.b_view = pv; } else { mm.a = v->src; mm.a_heads = true; mm.a_view = pv; }
      }
      if (mm.a_heads || mm.b_heads) { mm.outer = batch_dims[0]; mm.heads = batch_dims[1]; }
    }
    return mm;
  }

  static zyxb_kernel_desc gemm_desc(const MatMul& mm, int epi, bool preact, float alpha) {
    zyxb_kernel_desc d{};
    d.kind = ZYXB_KIND_GEMM;
    auto& g = d.u.gemm;
    g.dtype = mm.dtype; g.m = mm.m; g.n = mm.n; g.k = mm.k; g.batch = mm.batch;
    g.trans_a = mm.trans_a; g.trans_b = mm.trans_b;
    g.stride_a = (int64_t)(mm.m * mm.k); g.stride_b = mm.b_shared ? 0 : (int64_t)(mm.k * mm.n); g.stride_c = (int64_t)(mm.m * mm.n);
    g.epilogue = epi; g.store_preact = preact; g.alpha = alpha;
    if (mm.heads) {                                          // two-level batch: images outside, heads inside
      const uint64_t H = mm.heads;
      g.batch = mm.outer; g.batch_inner = H;
      // a stored [rows, cols] matrix per (image, head): inside a [b, t, h*d] tensor (pitch h*cols, heads `cols` apart) or packed
      auto packed = [H](uint64_t rows, uint64_t cols, uint64_t& ld, int64_t& outer, int64_t& inner) {
        ld = 0; outer = (int64_t)(H * rows * cols); inner = (int64_t)(rows * cols);
      };
      auto pitched = [](const MatMul::Pitch& p, uint64_t& ld, int64_t& outer, int64_t& inner) { ld = p.ld; outer = (int64_t)p.outer; inner = (int64_t)p.inner; };
      if (mm.a_heads) pitched(mm.a_view, g.lda, g.stride_a, g.stride_a_inner);
      else packed(mm.trans_a ? mm.k : mm.m, mm.trans_a ? mm.m : mm.k, g.lda, g.stride_a, g.stride_a_inner);
      if (mm.b_heads) pitched(mm.b_view, g.ldb, g.stride_b, g.stride_b_inner);
      else packed(mm.trans_b ? mm.n : mm.k, mm.trans_b ? mm.k : mm.n, g.ldb, g.stride_b, g.stride_b_inner);
      if (mm.c_heads) { g.ldc = H * mm.n; g.stride_c = (int64_t)(mm.m * H * mm.n); g.stride_c_inner = (int64_t)mm.n; }   // heads merged: [b, t, h*d]
      else packed(mm.m, mm.n, g.ldc, g.stride_c, g.stride_c_inner);
    }
    return d;
  }

  // relu(e) = e.cmpgt(0) * e (tensor/elementwise.rs:289-293): Mul{Cast{Cmpgt{e, 0}}, e} -> e
  std::optional<ClassId> relu_of(ClassId c) const {
    for (uint32_t nid : classes[c].nodes) {
      const Node& n = nodes[nid];
      if (n.kind != K_BINARY || n.op != B_MUL) continue;
      for (int swap = 0; swap < 2; ++swap) {
        ClassId mask = swap ? n.y : n.x, e = swap ? n.x : n.y;
        if (auto k = cast_src(mask)) mask = *k;
        auto cmp = binary(mask, B_CMPGT);
        if (cmp && same(cmp->first, e) && is_const(cmp->second, 0.0, 0.0)) return e;
      }
    }
    return std::nullopt;
  }
  // tanh(u) = ((u+u).exp() - 1) / ((u+u).exp() + 1) (elementwise.rs:585-588) -> u
  std::optional<ClassId> tanh_of(ClassId c) const {
    auto div = binary(c, B_DIV);
    if (!div) return std::nullopt;
    auto num = binary_const(div->first, B_SUB), den = binary_const(div->second, B_ADD);
    if (!num || !den || !same(num->first, den->first) || fabs(num->second - 1.0) > 1e-6 || fabs(den->second - 1.0) > 1e-6) return std::nullopt;
    auto arg = unary(num->first, U_EXP);
    if (!arg) return std::nullopt;
    auto two = binary(*arg, B_ADD);
    if (!two || !same(two->first, two->second)) return std::nullopt;
    return two->first;
  }
  // gelu(z) = z * 0.5 * (tanh((z + z*z*z*0.044715) * sqrt(2/pi)) + 1) (elementwise.rs:168-170) -> z
  std::optional<ClassId> gelu_of(ClassId c) const {
    auto top = binary(c, B_MUL);
    if (!top) return std::nullopt;
    auto half = binary_const(top->first, B_MUL);
    auto plus1 = binary_const(top->second, B_ADD);
    if (!half || !plus1 || !near(half->second, 0.5) || !near(plus1->second, 1.0)) return std::nullopt;
    const ClassId z = half->first;
    auto u = tanh_of(plus1->first);
    if (!u) return std::nullopt;
    auto scaled = binary_const(*u, B_MUL);
    if (!scaled || !near(scaled->second, 0.7978845608028654)) return std::nullopt;
    auto sum = binary(scaled->first, B_ADD);
    if (!sum || !same(sum->first, z)) return std::nullopt;
    auto cube = binary_const(sum->second, B_MUL);
    if (!cube || !near(cube->second, 0.044715)) return std::nullopt;
    auto zz_z = binary(cube->first, B_MUL);
    if (!zz_z || !same(zz_z->second, z)) return std::nullopt;
    auto zz = binary(zz_z->first, B_MUL);
    if (!zz || !same(zz->first, z) || !same(zz->second, z)) return std::nullopt;
    return z;
  }
  static bool near(double a, double b) { return fabs(a - b) <= 1e-2 * fabs(b); }     // constants arrive rounded to the tensor dtype

  // matmul [* const] [+ bias [relu | gelu]] ending at cid.  `wanted` are classes somebody else reads (the outputs of the
  // graph being matched): a pre-activation among them becomes the program's second output.
  static std::string gemm_name(const MatMul& mm) {
    return std::string("matmul_") + (mm.trans_a ? "t" : "n") + (mm.trans_b ? "t" : "n") + (mm.batch > 1 ? "_batched" : "") + (mm.heads ? "_heads" : "");
  }
  std::optional<Match> match_linear(ClassId cid, const std::set<ClassId>& wanted) const {
    // the heads merged back, `product.transpose(1, 2).reshape([b, t, h*d])` (multi_head_attention.rs:218-219): the product is
    // written where the merged tensor lies
    if (shape(cid).size() == 3)
      if (auto r4 = reshape_src(cid)) if (auto p4 = permute_src(*r4, {0, 2, 1, 3})) {
        const auto s4 = shape(*p4), s3 = shape(cid);
        if (s4.size() == 4 && s3[0] == s4[0] && s3[1] == s4[2] && s3[2] == s4[1] * s4[3])
          if (auto sc = match_matmul_scaled(*p4)) if (!sc->first.b_shared && dtype(cid) == sc->first.dtype) {
            MatMul mm = sc->first;
            mm.c_heads = true; mm.outer = s4[0]; mm.heads = s4[1];
            Match mt;
            mt.pattern = gemm_name(mm); mt.desc = gemm_desc(mm, ZYXB_EPI_NONE, false, sc->second);
            mt.inputs = {mm.a, mm.b}; mt.outputs = {cid};
            mt.input_offsets = {mm.a_view.offset, mm.b_view.offset};
            return mt;
          }
      }
    ClassId e = cid;
    int act = 0;
    if (auto z = gelu_of(cid)) { e = *z; act = 2; }
    else if (auto z = relu_of(cid)) { e = *z; act = 1; }
    // + bias: Add{mm, Expand{bias [n]}}
    ClassId core = e, bias = NONE;
    if (auto add = binary(e, B_ADD)) {
      for (int swap = 0; swap < 2 && bias == NONE; ++swap) {
        const ClassId lhs = swap ? add->second : add->first, rhs = swap ? add->first : add->second;
        auto src = expand_src(rhs);
        if (!src) continue;
        const ClassId bsrc = unbroadcast(rhs);
        if (shape(bsrc).size() == 1 && shape(bsrc)[0] == shape(e).back() && match_matmul_scaled(lhs)) { core = lhs; bias = bsrc; }
      }
    }
    if (act && bias == NONE) return std::nullopt;            // the fused activations exist as bias epilogues only
    // + a whole tensor of the product's shape (a residual): Add{mm, r}, for a single packed matrix without bias
    ClassId residual = NONE;
    if (bias == NONE)
      if (auto add = binary(e, B_ADD))
        for (int swap = 0; swap < 2 && residual == NONE; ++swap) {
          const ClassId lhs = swap ? add->second : add->first, rhs = swap ? add->first : add->second;
          if (shape(rhs) != shape(e) || dtype(rhs) != dtype(e) || expand_src(rhs) || const_value(rhs)) continue;
          auto inner = match_matmul_scaled(lhs);
          if (inner && inner->first.batch == 1 && !inner->first.heads) { core = lhs; residual = canon(rhs); }
        }
    auto sc = match_matmul_scaled(core);
    if (!sc) return std::nullopt;
    const MatMul& mm = sc->first;
    if (bias != NONE && dtype(bias) != mm.dtype) return std::nullopt;
    const int epi = residual != NONE ? ZYXB_EPI_ADD : bias == NONE ? ZYXB_EPI_NONE : act == 2 ? ZYXB_EPI_BIAS_GELU : act == 1 ? ZYXB_EPI_BIAS_RELU : ZYXB_EPI_BIAS;
    const bool preact = act == 2 && wanted.count(e) != 0;
    Match mt;
    mt.pattern = gemm_name(mm) + (bias != NONE ? "_bias" : residual != NONE ? "_add" : "") + (act == 2 ? "_gelu" : act == 1 ? "_relu" : "");
    mt.desc = gemm_desc(mm, epi, preact, sc->second);
    mt.inputs = {mm.a, mm.b};
    mt.input_offsets = {mm.a_view.offset, mm.b_view.offset};
    if (bias != NONE) { mt.inputs.push_back(bias); mt.input_offsets.push_back(0); }
    if (residual != NONE) { mt.inputs.push_back(residual); mt.input_offsets.push_back(0); }
    mt.outputs = {cid};
    if (preact) mt.outputs.push_back(e);
    return mt;
  }
  // matmul, or matmul * const (the scale of attention scores, multi_head_attention.rs:198-199) -> (matmul, alpha)
  std::optional<std::pair<MatMul, float>> match_matmul_scaled(ClassId cid) const {
    if (auto mm = match_matmul(cid)) return std::make_pair(*mm, 1.0f);
    if (auto sc = binary_const(cid, B_MUL)) if (auto mm = match_matmul(sc->first)) { mm->out = cid; return std::make_pair(*mm, (float)sc->second); }
    return std::nullopt;
  }

  // ---- fused attention ---------------------------------------------------------------------------------------------------
  std::optional<ClassId> permute_src(ClassId c, const std::vector<int>& axes) const {
    const Node* n = find(c, [&](const Node& n) { return n.kind == K_PERMUTE && n.axes == axes; });
    return n ? std::optional<ClassId>(n->x) : std::nullopt;
  }
  // The core of MultiheadAttention::forward without masks (multi_head_attention.rs:197-226), ending at the class of
  //   attn_weights.matmul(v).transpose(1, 2).reshape([b, t, h*d]),  attn_weights = (q.matmul(k.transpose(-2, -1)) * scale).softmax([-1]),
  // with q, k, v the head-split views of three stored [b, t, h*d] tensors: one fused program that reads those three where they
  // lie and writes the [b, t, h*d] result; scores and probabilities never exist.  The kernel's shapes only: 16-bit dtype, head
  // dimension 128, equal query and key lengths that are a multiple of 128.  A causal mask
  // (`masked_fill(ones.tril(0).equal(0), -inf)`, multi_head_attention.rs:203-207) is not matched: `where_` (tensor/mod.rs:1617-1624)
  // computes in the dtype of the rank-0 fill value, so 16-bit scores come out as f32 - and as NaN wherever the mask keeps them
  // (0 * -inf) - which is not what the 16-bit program computes; such graphs fall back to the separate programs.
  std::optional<Match> match_attention(ClassId cid) const {
    const auto s3 = shape(cid);
    if (s3.size() != 3) return std::nullopt;
    auto r = reshape_src(cid);
    if (!r || shape(*r).size() != 4) return std::nullopt;
    auto pv_cls = permute_src(*r, {0, 2, 1, 3});
    if (!pv_cls) return std::nullopt;
    auto pv = match_matmul(*pv_cls);
    if (!pv || pv->trans_a || pv->trans_b || pv->b_shared) return std::nullopt;
    auto sm = match_softmax(pv->a);
    if (!sm) return std::nullopt;
    auto sc = match_matmul_scaled(sm->inputs[0]);
    if (!sc || sc->first.trans_a || !sc->first.trans_b || sc->first.b_shared) return std::nullopt;
    const MatMul& qk = sc->first;
    if (!qk.a_heads || !qk.b_heads || !pv->b_heads || pv->a_heads) return std::nullopt;      // q, k, v: per-head views of stored tensors
    const std::optional<ClassId> xq = qk.a, xk = qk.b, xv = pv->b;
    const auto hs = shape(*pv_cls);                          // [b, h, t, d]
    const uint64_t B = hs[0], H = hs[1], T = hs[2], D = hs[3];
    if (qk.m != T || qk.n != T || qk.k != D || pv->m != T || pv->k != T || pv->n != D || qk.batch != B * H || pv->batch != B * H) return std::nullopt;
    const int dt = qk.dtype;
    if ((dt != ZYXB_BF16 && dt != ZYXB_F16) || pv->dtype != dt || D != 128 || T % 128 != 0) return std::nullopt;
    if (s3[0] != B || s3[1] != T || s3[2] != H * D) return std::nullopt;
    // the program reads q, k, v and writes the result with one row pitch: whole [b, t, h*d] tensors, not slices of a wider one
    const MatMul::Pitch* const views[] = {&qk.a_view, &qk.b_view, &pv->b_view};
    for (const MatMul::Pitch* p : views)
      if (p->offset != 0 || p->ld != H * D || (H > 1 && p->inner != D) || (B > 1 && p->outer != T * H * D)) return std::nullopt;   // (a single image or head is never stepped over)
    Match m;
    m.pattern = "attention";
    m.desc.kind = ZYXB_KIND_ATTENTION;
    auto& a = m.desc.u.attention;
    a.dtype = dt; a.batch = B; a.heads = H; a.seq = T; a.head_dim = D; a.scale = sc->second; a.causal = 0;
    m.inputs = {*xq, *xk, *xv};
    m.outputs = {cid};      // the launch takes one more buffer behind it: the log-sum-exp [b*h, t] f32 the backward program reads
    return m;
  }

  // ---- row kernels ---------------------------------------------------------------------------------------------------------
  static zyxb_kernel_desc row_desc(int op, int dt, const std::vector<uint64_t>& s) {
    zyxb_kernel_desc d{};
    d.kind = ZYXB_KIND_ROWREDUCE;
    d.u.rowreduce.op = op; d.u.rowreduce.dtype = dt; d.u.rowreduce.cols = s.back(); d.u.rowreduce.rows = numel(s) / s.back();
    d.u.rowreduce.correction = 1;
    return d;
  }
  bool row_dtype(int dt) const { return dt == ZYXB_F32 || dt == ZYXB_BF16 || dt == ZYXB_F16; }

  // softmax(x, [-1]) = e / e.sum_keepdim, e = (x - x.max_keepdim).exp()   (tensor/mod.rs:1457-1461)
  std::optional<Match> match_softmax(ClassId cid) const {
    auto div = binary(cid, B_DIV);
    if (!div || shape(cid).empty() || (!expand_src(div->second) && shape(cid).back() != 1)) return std::nullopt;   // (one column: nothing to expand)
    const ClassId e = div->first;
    auto sum_of = reduce_last(unbroadcast_keepdim(div->second), B_ADD);
    if (!sum_of || !same(*sum_of, e)) return std::nullopt;
    auto x = shifted(e, U_EXP);
    if (!x || !row_dtype(dtype(*x)) || shape(*x).empty()) return std::nullopt;
    Match m; m.pattern = "softmax"; m.desc = row_desc(ZYXB_RR_SOFTMAX, dtype(*x), shape(*x)); m.inputs = {*x}; m.outputs = {cid};
    return m;
  }
  // ln_softmax(x, [-1]) = m - m.exp().sum_keepdim().ln(), m = x - x.max_keepdim   (tensor/mod.rs:1427-1431)
  std::optional<Match> match_ln_softmax(ClassId cid) const {
    auto sub = binary(cid, B_SUB);
    if (!sub || shape(cid).empty() || (!expand_src(sub->second) && shape(cid).back() != 1)) return std::nullopt;
    const ClassId m = sub->first;
    auto lnarg = unary(unbroadcast_keepdim(sub->second), U_LN);
    if (!lnarg) return std::nullopt;
    auto e = reduce_last(*lnarg, B_ADD);
    if (!e) return std::nullopt;
    auto earg = unary(*e, U_EXP);
    if (!earg || !same(*earg, m)) return std::nullopt;
    auto x = shifted(m, -1);
    if (!x || !row_dtype(dtype(*x))) return std::nullopt;
    Match mt; mt.pattern = "ln_softmax"; mt.desc = row_desc(ZYXB_RR_LN_SOFTMAX, dtype(*x), shape(*x)); mt.inputs = {*x}; mt.outputs = {cid};
    return mt;
  }
  // a keepdim operand is expanded back over the row: strip exactly that Expand (its source keeps rank, last extent 1)
  ClassId unbroadcast_keepdim(ClassId c) const { auto e = expand_src(c); return e ? *e : c; }
  // c = uop(x - Expand{max_keepdim(x)}) (uop < 0: no unary) -> x
  std::optional<ClassId> shifted(ClassId c, int uop) const {
    ClassId d = c;
    if (uop >= 0) { auto a = unary(c, uop); if (!a) return std::nullopt; d = *a; }
    auto sub = binary(d, B_SUB);
    if (!sub) return std::nullopt;
    auto mx = reduce_last(unbroadcast_keepdim(sub->second), B_MAX);
    if (!mx || !same(*mx, sub->first)) return std::nullopt;
    return canon(sub->first);
  }
  // mean over the last axis, keepdim: sum / const(n)   (reduce_ops.rs:104-112) -> x
  std::optional<ClassId> mean_last(ClassId c, double* n_out = nullptr) const {
    ClassId d = c;
    if (auto r = reshape_src(c)) if (numel(shape(*r)) == numel(shape(c))) d = *r;
    auto div = binary_const(d, B_DIV);
    if (!div) return std::nullopt;
    auto x = reduce_last(div->first, B_ADD);
    if (!x) return std::nullopt;
    if (n_out) *n_out = div->second;
    return x;
  }
  // LayerNorm::forward over the last axis (zyx-nn/src/layer_norm.rs:117-131):
  //   ((x - mean) / sqrt(var + eps)) [* weight] [+ bias],  var = ((x - mean)^2).sum / (n - 1)
  std::optional<Match> match_layernorm(ClassId cid) const {
    ClassId c = cid, weight = NONE, bias = NONE;
    auto affine = [&](int bop, ClassId& param) {
      auto b = binary(c, bop);
      if (!b || (!expand_src(b->second) && shape(cid).size() != 1)) return;     // (a rank-1 input meets its parameters unexpanded)
      const ClassId src = expand_src(b->second) ? unbroadcast(b->second) : canon(b->second);
      if (shape(src).size() == 1 && shape(src)[0] == shape(cid).back() && !const_value(src)) { param = src; c = b->first; }
    };
    affine(B_ADD, bias);
    affine(B_MUL, weight);
    auto div = binary(c, B_DIV);
    if (!div) return std::nullopt;
    auto centred = binary(div->first, B_SUB);
    if (!centred) return std::nullopt;
    const ClassId x = canon(centred->first);
    auto mx = mean_last(unbroadcast_keepdim(centred->second));
    if (!mx || !same(*mx, x)) return std::nullopt;
    auto root = unary(unbroadcast_keepdim(div->second), U_SQRT);
    if (!root) return std::nullopt;
    auto var_eps = binary_const(*root, B_ADD);
    if (!var_eps) return std::nullopt;
    double d = 0;
    auto sq = mean_last(var_eps->first, &d);           // sum((x - mean)^2) / (n - correction)
    if (!sq) return std::nullopt;
    auto xx = binary(*sq, B_MUL);
    if (!xx || !same(xx->first, xx->second) || !same(xx->first, div->first)) return std::nullopt;
    if (!row_dtype(dtype(x))) return std::nullopt;
    const double n = (double)shape(x).back();
    const int correction = (int)llround(n - d);
    Match m; m.pattern = "layernorm";
    m.desc = row_desc(ZYXB_RR_LAYERNORM, dtype(x), shape(x));
    m.desc.u.rowreduce.eps = (float)var_eps->second; m.desc.u.rowreduce.correction = near(d, n - 1) ? 1 : correction;
    m.desc.u.rowreduce.has_weight = weight != NONE; m.desc.u.rowreduce.has_bias = bias != NONE;
    m.inputs = {x};
    if (weight != NONE) m.inputs.push_back(weight);
    if (bias != NONE) m.inputs.push_back(bias);
    m.outputs = {cid};
    return m;
  }
  // var(x, [-1]) = sum((x - mean_keepdim(x))^2) / (n - correction)   (reduce_ops.rs:111-123) -> (x, correction)
  std::optional<std::pair<ClassId, int>> var_last(ClassId cid) const {
    double d = 0;
    auto sq = mean_last(cid, &d);
    if (!sq) return std::nullopt;
    auto xx = binary(*sq, B_MUL);
    if (!xx || !same(xx->first, xx->second)) return std::nullopt;
    auto centred = binary(xx->first, B_SUB);
    if (!centred) return std::nullopt;
    const ClassId x = canon(centred->first);
    auto mx = mean_last(unbroadcast_keepdim(centred->second));
    if (!mx || !same(*mx, x) || shape(x).empty()) return std::nullopt;
    const double n = (double)shape(x).back();
    const long corr = llround(n - d);
    if (corr < 0 || corr >= (long)n || fabs((n - d) - (double)corr) > 1e-6) return std::nullopt;
    return std::make_pair(x, (int)corr);
  }
  // sum over the rows of a matrix: x [rows, cols] .sum([0]) -> [cols] (the bias gradient of a Linear layer)
  std::optional<ClassId> column_sum_src(ClassId cid) const {
    auto red_of = [&](ClassId c) { return find(c, [](const Node& n) { return n.kind == K_REDUCE && n.op == B_ADD && n.axes.size() == 1 && n.axes[0] == 0; }); };
    const Node* red = red_of(cid);
    if (!red) { auto k = cast_src(cid); if (!k || !(red = red_of(*k))) return std::nullopt; }      // sum() casts the accumulator back for 16-bit inputs
    ClassId x = red->x;
    if (auto k = cast_src(x)) if (dtype(*k) == dtype(cid)) x = *k;                                  // the accumulator cast
    x = canon(x);
    if (shape(x).size() != 2 || dtype(x) != dtype(cid)) return std::nullopt;
    return x;
  }
  // var / std / sum / max / mean over the last axis, sum over the rows of a matrix, of a tensor nobody computes as a matmul product
  std::optional<Match> match_reduce(ClassId cid) const {
    const std::pair<int, int> ops[] = {{B_ADD, ZYXB_RR_SUM}, {B_MAX, ZYXB_RR_MAX}};
    for (int is_std = 0; is_std < 2; ++is_std) {
      ClassId v = cid;
      if (is_std) { auto r = unary(cid, U_SQRT); if (!r) break; v = *r; }
      if (auto vx = var_last(v)) if (row_dtype(dtype(vx->first)) && dtype(cid) == dtype(vx->first)) {
        Match m; m.pattern = is_std ? "std" : "var"; m.desc = row_desc(is_std ? ZYXB_RR_STD : ZYXB_RR_VAR, dtype(vx->first), shape(vx->first));
        m.desc.u.rowreduce.correction = vx->second; m.inputs = {vx->first}; m.outputs = {cid};
        return m;
      }
    }
    if (auto x = column_sum_src(cid)) if (row_dtype(dtype(*x)) && !is_broadcast_product(*x)) {
      Match m; m.pattern = "colsum"; m.desc = row_desc(ZYXB_RR_COLSUM, dtype(*x), shape(*x)); m.inputs = {*x}; m.outputs = {cid};
      return m;
    }
    if (auto x = mean_last(cid)) if (row_dtype(dtype(*x)) && shape(*x).size() >= 1) {
      Match m; m.pattern = "mean"; m.desc = row_desc(ZYXB_RR_MEAN, dtype(*x), shape(*x)); m.inputs = {*x}; m.outputs = {cid};
      return m;
    }
    // min = -max(-x) for floats, !max(!x) bitwise for integers (Tensor::inverse, reduce_ops.rs:33-42, 93-99); keepdim reshapes outside
    {
      ClassId c = cid;
      if (auto r = reshape_src(cid)) if (numel(shape(*r)) == numel(shape(cid))) c = *r;
      for (int uop : {(int)U_NEG, (int)U_BITNOT})
        if (auto inner = unary(c, uop)) if (auto nx = reduce_last(*inner, B_MAX)) if (auto x0 = unary(*nx, uop)) {
          const ClassId x = canon(*x0);
          const bool ok = uop == U_NEG ? row_dtype(dtype(x)) : dtype(x) == ZYXB_I32;
          if (ok && dtype(cid) == dtype(x) && !shape(x).empty()) {
            Match m; m.pattern = "min"; m.desc = row_desc(ZYXB_RR_MIN, dtype(x), shape(x)); m.inputs = {x}; m.outputs = {cid};
            return m;
          }
        }
    }
    for (auto [rop, rr] : ops)
      if (auto x = reduce_last(cid, rop)) {
        if (!(row_dtype(dtype(*x)) || dtype(*x) == ZYXB_I32) || dtype(cid) != dtype(*x) || shape(*x).empty()) continue;
        if (is_broadcast_product(*x)) continue;       // the [.., m, n, k] product of a dot: never materialised, the matmul patterns own it
        Match m; m.pattern = rop == B_ADD ? "sum" : "max"; m.desc = row_desc(rr, dtype(*x), shape(*x)); m.inputs = {*x}; m.outputs = {cid};
        return m;
      }
    return std::nullopt;
  }

  // mse_loss(y, t) = ((y - t) * (y - t)).mean_all()   (tensor/mod.rs:1999-2003): Div{Reduce{Mul{d, d}, Add, every axis}, n}.
  // f32 only: the program leaves an f32 scalar, the reference a scalar of the tensor's dtype.
  std::optional<Match> match_mse(ClassId cid) const {
    auto div = binary_const(cid, B_DIV);
    if (!div) return std::nullopt;
    const Node* red = find(div->first, [](const Node& n) { return n.kind == K_REDUCE && n.op == B_ADD; });
    if (!red) return std::nullopt;
    const auto xs = shape(red->x);
    if (xs.empty() || red->axes.size() != xs.size() || fabs(div->second - (double)numel(xs)) > 0.5) return std::nullopt;
    auto mul = binary(red->x, B_MUL);
    if (!mul || !same(mul->first, mul->second)) return std::nullopt;
    auto sub = binary(mul->first, B_SUB);
    if (!sub) return std::nullopt;
    const ClassId y = canon(sub->first), t = canon(sub->second);
    if (expand_src(y) || expand_src(t)) return std::nullopt;          // whole tensors: x - mean(x) over a rank-1 x is the variance's business
    if (dtype(y) != ZYXB_F32 || dtype(t) != ZYXB_F32 || dtype(cid) != ZYXB_F32 || shape(y) != xs || shape(t) != xs) return std::nullopt;
    Match m; m.pattern = "mse_loss"; m.desc = row_desc(ZYXB_RR_MSE, ZYXB_F32, xs); m.inputs = {y, t}; m.outputs = {cid};
    return m;
  }

  bool is_broadcast_product(ClassId c) const {
    if (auto k = cast_src(c)) c = *k;
    auto mul = binary(c, B_MUL);
    return mul && expand_src(mul->first) && expand_src(mul->second);
  }

  // ---- elementwise programs ---------------------------------------------------------------------------------------------
  // What is left when no larger pattern ends at a class: one elementwise program over stored operands (tensor/elementwise.rs).
  // Operands are whole tensors of the result's shape - a broadcast operand is either a scalar constant (scale) or a vector
  // along the last axis (bias) - so the broadcast product inside a dot or the shifted row inside a softmax are not offered as
  // programs of their own.  16-bit and f32 floats only (what the kernels take).
  std::optional<Match> match_eltwise(ClassId cid) const {
    const int dt = dtype(cid);
    const auto& cs = shape(cid);
    const uint64_t n = numel(cs);
    if (!row_dtype(dt) || cs.empty() || n == 0) return std::nullopt;
    auto whole = [&](ClassId x) { return shape(x) == cs && dtype(x) == dt && !expand_src(x) && !const_value(x); };
    auto program = [&](const char* name, int op, std::vector<ClassId> in, float p0 = 0.0f, uint64_t cols = 0, int dt_in = -1) {
      Match m; m.pattern = name; m.desc.kind = ZYXB_KIND_ELTWISE;
      auto& e = m.desc.u.eltwise;
      e.op = op; e.dtype = dt_in < 0 ? dt : dt_in; e.dtype_out = dt; e.numel = n; e.cols = cols; e.p0 = p0;
      for (ClassId& c : in) c = canon(c);
      m.inputs = std::move(in); m.outputs = {cid};
      return m;
    };
    if (auto z = gelu_of(cid)) if (whole(*z)) return program("gelu", ZYXB_EW_GELU, {*z});
    if (auto z = relu_of(cid)) if (whole(*z)) return program("relu", ZYXB_EW_RELU, {*z});
    if (auto u = tanh_of(cid)) if (whole(*u)) return program("tanh", ZYXB_EW_TANH, {*u});
    if (auto div = binary(cid, B_DIV))                               // sigmoid(x) = e / (e + 1), e = exp(x)   (elementwise.rs:457-460)
      if (auto den = binary_const(div->second, B_ADD)) if (same(den->first, div->first) && fabs(den->second - 1.0) <= 1e-6)
        if (auto x = unary(div->first, U_EXP)) if (whole(*x)) return program("sigmoid", ZYXB_EW_SIGMOID, {*x});
    if (auto x = unary(cid, U_EXP)) if (whole(*x)) return program("exp", ZYXB_EW_EXP, {*x});
    if (auto x = unary(cid, U_NEG)) if (whole(*x)) return program("scale", ZYXB_EW_SCALE, {*x}, -1.0f);      // -x = x * -1, exactly
    if (auto x = cast_src(cid)) if (row_dtype(dtype(*x)) && shape(*x) == cs && !expand_src(*x) && !const_value(*x))
      return program("cast", ZYXB_EW_CAST, {*x}, 0.0f, 0, dtype(*x));
    if (auto sc = binary_const(cid, B_MUL)) if (whole(sc->first)) return program("scale", ZYXB_EW_SCALE, {sc->first}, (float)sc->second);
    // x / const as x * (1 / const): what the reference's own C backend computes under -ffast-math (reciprocal math); dropout
    // outside training is such a division (x / (1 - p), tensor/mod.rs:822-828)
    if (auto sc = binary_const(cid, B_DIV)) if (whole(sc->first) && sc->second != 0.0) return program("scale", ZYXB_EW_SCALE, {sc->first}, (float)(1.0 / sc->second));
    const std::tuple<int, int, const char*> ops[] = {{B_ADD, ZYXB_EW_ADD, "add"}, {B_SUB, ZYXB_EW_SUB, "sub"}, {B_MUL, ZYXB_EW_MUL, "mul"}};
    for (auto [bop, ew, name] : ops)
      if (auto b = binary(cid, bop)) if (whole(b->first) && whole(b->second)) return program(name, ew, {b->first, b->second});
    if (auto add = binary(cid, B_ADD))                               // x + bias along the last axis
      for (int swap = 0; swap < 2; ++swap) {
        const ClassId x = swap ? add->second : add->first, be = swap ? add->first : add->second;
        if (!whole(x) || !expand_src(be) || const_value(be)) continue;
        const ClassId b = canon(unbroadcast(be));
        if (shape(b) == std::vector<uint64_t>{cs.back()} && dtype(b) == dt && trailing_vector(be))
          return program("bias_add", ZYXB_EW_BIAS_ADD, {x, b}, 0.0f, cs.back());
      }
    return std::nullopt;
  }
  // c = Expand{[Reshape]{v [n]}} with v laid along the LAST axis of c (every wrapper keeps all but the last extent at 1)
  bool trailing_vector(ClassId c) const {
    auto e = expand_src(c);
    if (!e) return false;
    for (ClassId s = *e;;) {
      const auto& sh = shape(s);
      if (sh.empty()) return false;
      for (size_t i = 0; i + 1 < sh.size(); ++i) if (sh[i] != 1) return false;
      auto r = reshape_src(s);
      if (!r) return true;
      s = *r;
    }
  }

  // ---- constant folding --------------------------------------------------------------------------------------------------
  // The value of a class that depends on no stored tensor: constants under movement ops, paddings, reductions, casts and
  // arithmetic, the way the reference's index helpers build them (Tensor::arange is `full(step).cumsum(0) + start - step`,
  // tensor/mod.rs:773-781, and a cumsum is a padded, pooled sum, reduce_ops.rs:1076-1091).  Row-major values as doubles, exact
  // for the index arithmetic this is for.  nullopt when a Leaf is reached, an op is not covered, or some intermediate has more
  // than `limit` elements.
  using Values = std::vector<double>;
  std::optional<Values> const_eval(ClassId c, uint64_t limit = (1ull << 22)) const {
    std::map<ClassId, std::optional<Values>> memo;
    const Values* v = eval_class(c, limit, memo, 0);
    return v ? std::optional<Values>(*v) : std::nullopt;
  }
  const Values* eval_class(ClassId c, uint64_t limit, std::map<ClassId, std::optional<Values>>& memo, int depth) const {
    auto it = memo.find(c);
    if (it == memo.end()) it = memo.emplace(c, eval_node(c, limit, memo, depth)).first;
    return it->second ? &*it->second : nullptr;
  }
  static void unravel(uint64_t i, const std::vector<uint64_t>& shape, std::vector<uint64_t>& idx) {
    for (size_t a = shape.size(); a-- > 0;) { idx[a] = i % shape[a]; i /= shape[a]; }
  }
  static double cast_value(double v, int dt) {
    if (dt == ZYXB_BOOL) return v != 0.0 ? 1.0 : 0.0;
    if (dt == ZYXB_F32) return (double)(float)v;
    if (is_float(dt)) return v;
    return std::trunc(v);
  }
  std::optional<Values> eval_node(ClassId c, uint64_t limit, std::map<ClassId, std::optional<Values>>& memo, int depth) const {
    if (!valid(c) || depth > 256) return std::nullopt;
    const Node& n = nodes[classes[c].nodes[0]];
    const auto& os = shape(c);
    const uint64_t on = numel(os);
    if (on > limit) return std::nullopt;
    auto arg = [&](ClassId x) { return valid(x) ? eval_class(x, limit, memo, depth + 1) : nullptr; };
    if (n.kind == K_CONST) return Values{n.value};
    if (n.kind == K_LEAF || n.kind == K_KERNEL) return std::nullopt;
    const Values* x = arg(n.x);
    if (!x) return std::nullopt;
    const auto& xs = shape(n.x);
    std::vector<uint64_t> xstride(xs.size(), 1);
    for (size_t a = xs.size(); a-- > 1;) xstride[a - 1] = xstride[a] * xs[a];
    Values out(on, 0.0);
    std::vector<uint64_t> idx(std::max(os.size(), xs.size()), 0);
    switch (n.kind) {
      case K_RESHAPE: return *x;
      case K_EXPAND: {
        const size_t lead = os.size() - xs.size();
        for (uint64_t o = 0; o < on; ++o) {
          unravel(o, os, idx);
          uint64_t src = 0;
          for (size_t a = 0; a < xs.size(); ++a) if (xs[a] != 1) src += idx[lead + a] * xstride[a];
          out[o] = (*x)[src];
        }
        return out;
      }
      case K_PERMUTE:
        for (uint64_t o = 0; o < on; ++o) {
          unravel(o, os, idx);
          uint64_t src = 0;
          for (size_t j = 0; j < n.axes.size(); ++j) src += idx[j] * xstride[n.axes[j]];
          out[o] = (*x)[src];
        }
        return out;
      case K_PAD: {
        const size_t ax = (size_t)n.axes[0];
        for (uint64_t o = 0; o < on; ++o) {
          unravel(o, os, idx);
          const int64_t at = (int64_t)idx[ax] - n.lp;
          if (at < 0 || at >= (int64_t)xs[ax]) continue;                 // a zero of the padding
          uint64_t src = 0;
          for (size_t a = 0; a < xs.size(); ++a) src += (a == ax ? (uint64_t)at : idx[a]) * xstride[a];
          out[o] = (*x)[src];
        }
        return out;
      }
      case K_REDUCE: {
        if (n.op != B_ADD && n.op != B_MAX && n.op != B_MUL) return std::nullopt;
        std::fill(out.begin(), out.end(), n.op == B_ADD ? 0.0 : n.op == B_MUL ? 1.0 : -INFINITY);
        std::vector<char> reduced(xs.size(), 0);
        for (int a : n.axes) reduced[a] = 1;
        for (uint64_t i = 0; i < x->size(); ++i) {
          unravel(i, xs, idx);
          uint64_t o = 0;
          for (size_t a = 0; a < xs.size(); ++a) if (!reduced[a]) o = o * xs[a] + idx[a];
          const double v = (*x)[i];
          out[o] = n.op == B_ADD ? out[o] + v : n.op == B_MUL ? out[o] * v : std::max(out[o], v);
        }
        return out;
      }
      case K_CAST:
        for (uint64_t o = 0; o < on; ++o) out[o] = cast_value((*x)[o], n.dtype);
        return out;
      case K_UNARY:
        for (uint64_t o = 0; o < on; ++o) {
          const double v = (*x)[o];
          switch (n.op) {
            case U_NEG: out[o] = -v; break;
            case U_ABS: out[o] = fabs(v); break;
            case U_FLOOR: out[o] = floor(v); break;
            case U_TRUNC: out[o] = std::trunc(v); break;
            case U_EXP: out[o] = exp(v); break;
            case U_LN: out[o] = log(v); break;
            case U_SQRT: out[o] = sqrt(v); break;
            case U_RECIPROCAL: out[o] = 1.0 / v; break;
            default: return std::nullopt;
          }
        }
        return out;
      case K_BINARY: {
        const Values* y = arg(n.y);
        if (!y || y->size() != x->size() || x->size() != on) return std::nullopt;
        const bool whole = !is_float(dtype(n.x));
        for (uint64_t o = 0; o < on; ++o) {
          const double a = (*x)[o], b = (*y)[o];
          switch (n.op) {
            case B_ADD: out[o] = a + b; break;
            case B_SUB: out[o] = a - b; break;
            case B_MUL: out[o] = a * b; break;
            case B_DIV: if (whole && b == 0.0) return std::nullopt; out[o] = whole ? std::trunc(a / b) : a / b; break;
            case B_MOD: if (b == 0.0) return std::nullopt; out[o] = fmod(a, b); break;
            case B_MAX: out[o] = std::max(a, b); break;
            case B_CMPLT: out[o] = a < b; break;
            case B_CMPGT: out[o] = a > b; break;
            case B_CMPGE: out[o] = a >= b; break;
            case B_NOTEQ: out[o] = a != b; break;
            case B_EQ: out[o] = a == b; break;
            default: return std::nullopt;
          }
        }
        return out;
      }
      default: return std::nullopt;
    }
  }

  // ---- views: where an element comes from -------------------------------------------------------------------------------
  // One element of class c followed back through the movement ops that define it (Expand, Reshape, Permute, Pad, no-op Cast)
  // to the first class that is something else: that class and the element's coordinates there, or `zero` when the element is
  // a zero of some padding.  This is how a view is recognised by what it reads instead of by how it was written down: the
  // reference's pooling (Tensor::pool, tensor/mod.rs:2442-2543) is a dozen reshapes, expands and crops that differ with every
  // stride and dilation, but what they read is `row = oy*stride + r*dilation`.
  struct Origin { ClassId cls = NONE; std::vector<uint64_t> idx; bool zero = false; };
  static uint64_t ravel(const std::vector<uint64_t>& idx, const std::vector<uint64_t>& shape) {
    uint64_t lin = 0;
    for (size_t a = 0; a < shape.size(); ++a) lin = lin * shape[a] + idx[a];
    return lin;
  }
  Origin trace_element(ClassId c, std::vector<uint64_t> idx) const {
    Origin o;
    for (int hops = 0; hops < 256; ++hops) {
      const Node& n = nodes[classes[c].nodes[0]];
      const auto& cs = shape(c);
      if (n.kind == K_RESHAPE) {
        const uint64_t lin = ravel(idx, cs);
        idx.assign(shape(n.x).size(), 0);
        unravel(lin, shape(n.x), idx);
      } else if (n.kind == K_EXPAND) {
        const auto& xs = shape(n.x);
        const size_t lead = cs.size() - xs.size();
        std::vector<uint64_t> in(xs.size());
        for (size_t a = 0; a < xs.size(); ++a) in[a] = xs[a] == 1 ? 0 : idx[lead + a];
        idx = std::move(in);
      } else if (n.kind == K_PERMUTE) {
        std::vector<uint64_t> in(idx.size());
        for (size_t j = 0; j < n.axes.size(); ++j) in[n.axes[j]] = idx[j];
        idx = std::move(in);
      } else if (n.kind == K_PAD) {
        const size_t ax = (size_t)n.axes[0];
        const int64_t at = (int64_t)idx[ax] - n.lp;
        if (at < 0 || at >= (int64_t)shape(n.x)[ax]) { o.zero = true; return o; }
        idx[ax] = (uint64_t)at;
      } else if (!(n.kind == K_CAST && dtype(n.x) == dtype(c))) {
        break;
      }
      c = n.x;
    }
    o.cls = c; o.idx = std::move(idx);
    return o;
  }
  // c as a strided window of a stored tensor: element idx of c is element offset + sum(idx[a] * strides[a]) of `src`, row-major.
  // Measured, not derived: the origin and one step along every axis give offset and strides, then every corner and a spread of
  // other elements must agree (a reshape of a permuted tensor, say, is no such window and fails at its far corner).  nullopt
  // when some element is padding or the elements come from more than one class.
  struct View { ClassId src = NONE; uint64_t offset = 0; std::vector<int64_t> strides; };
  std::optional<View> affine_view(ClassId c) const {
    const auto& cs = shape(c);
    const size_t rank = cs.size();
    if (rank == 0 || rank > 6 || numel(cs) == 0) return std::nullopt;
    std::vector<uint64_t> idx(rank, 0);
    const Origin o0 = trace_element(c, idx);
    if (o0.zero) return std::nullopt;
    View v; v.src = canon(o0.cls); v.offset = ravel(o0.idx, shape(o0.cls)); v.strides.assign(rank, 0);
    auto at = [&](const std::vector<uint64_t>& i) -> std::optional<int64_t> {
      const Origin o = trace_element(c, i);
      if (o.zero || canon(o.cls) != v.src) return std::nullopt;
      return (int64_t)ravel(o.idx, shape(o.cls));
    };
    for (size_t a = 0; a < rank; ++a) {
      if (cs[a] < 2) continue;
      idx[a] = 1;
      auto lin = at(idx);
      idx[a] = 0;
      if (!lin) return std::nullopt;
      v.strides[a] = *lin - (int64_t)v.offset;
    }
    auto agrees = [&](const std::vector<uint64_t>& i) {
      int64_t want = (int64_t)v.offset;
      for (size_t a = 0; a < rank; ++a) want += (int64_t)i[a] * v.strides[a];
      auto lin = at(i);
      return lin && *lin == want;
    };
    for (uint64_t corner = 0; corner < (1ull << rank); ++corner) {
      for (size_t a = 0; a < rank; ++a) idx[a] = (corner >> a & 1) ? cs[a] - 1 : 0;
      if (!agrees(idx)) return std::nullopt;
    }
    uint64_t seed = 0x9e3779b97f4a7c15ull;                            // a fixed spread of interior elements
    for (int probe = 0; probe < 256; ++probe) {
      for (size_t a = 0; a < rank; ++a) { seed = seed * 6364136223846793005ull + 1442695040888963407ull; idx[a] = (seed >> 33) % cs[a]; }
      if (!agrees(idx)) return std::nullopt;
    }
    return v;
  }
  // the class a view reads: c under every movement op
  ClassId view_source(ClassId c) const {
    for (int hops = 0; hops < 256; ++hops) {
      const Node& n = nodes[classes[c].nodes[0]];
      const bool movement = n.kind == K_RESHAPE || n.kind == K_EXPAND || n.kind == K_PERMUTE || n.kind == K_PAD ||
                            (n.kind == K_CAST && dtype(n.x) == dtype(c));
      if (!movement) return c;
      c = n.x;
    }
    return c;
  }
  // every index of a short axis; the first, last and a spread of a long one
  static std::vector<uint64_t> sample_axis(uint64_t n) {
    std::vector<uint64_t> v;
    if (n <= 48) { for (uint64_t i = 0; i < n; ++i) v.push_back(i); return v; }
    for (uint64_t i = 0; i < 16; ++i) v.push_back(i);
    for (uint64_t i = 1; i <= 16; ++i) v.push_back(16 + i * (n - 32) / 17);
    for (uint64_t i = n - 16; i < n; ++i) v.push_back(i);
    return v;
  }

  // ---- convolution -------------------------------------------------------------------------------------------------------
  // Tensor::conv with groups = 1 on [n, c, h, w] (tensor/mod.rs:2583-2680), ending at cid [n, o, oh, ow]:
  //   x.rpad_zeros(padding).pool(kernel, stride, dilation) -Reshape, Expand over o, Permute-> [n, 1, o, oh, ow, c, kh, kw]
  //   * weight.reshape([1, 1, o, 1, 1, c, kh, kw]) -> sum_keepdim over (c, kh, kw) -> reshape [n, o, oh, ow]  [+ bias.reshape([1, o, 1, 1])]
  // The padding is read off the Pad nodes that sit on the stored input; stride and dilation are measured on the view (two
  // neighbouring output rows, two neighbouring filter rows), and then the whole view is held against
  //   x[b, ci, oy*stride_h + r*dil_h - pad_top, ox*stride_w + s*dil_w - pad_left]   (zero outside the image)
  // for every window position and tap at the corner (image, channel) pairs, every (image, channel) pair at two windows, and
  // both ends of the filter axis the view is expanded over (long axes: both ends and a spread).
  std::optional<Match> match_conv(ClassId cid) const {
    const auto out = shape(cid);
    if (out.size() != 4) return std::nullopt;
    ClassId e = cid, bias = NONE;
    if (auto add = binary(cid, B_ADD))
      for (int swap = 0; swap < 2 && bias == NONE; ++swap) {
        const ClassId lhs = swap ? add->second : add->first, rhs = swap ? add->first : add->second;
        auto src = expand_src(rhs);
        if (!src || shape(*src) != std::vector<uint64_t>{1, out[1], 1, 1}) continue;
        const ClassId b = canon(unbroadcast(rhs));
        if (numel(shape(b)) == out[1]) { bias = b; e = lhs; }
      }
    // through the closing reshape and sum_keepdim's reshape to the Reduce
    auto is_red = [](const Node& n) { return n.kind == K_REDUCE && n.op == B_ADD; };
    const Node* red = nullptr;
    ClassId r = e;
    for (int i = 0; i < 4 && !red; ++i) {
      if ((red = find(r, is_red))) break;
      if (auto k = cast_src(r)) if ((red = find(*k, is_red))) break;
      auto src = reshape_src(r);
      if (!src || numel(shape(*src)) != numel(out)) return std::nullopt;
      r = *src;
    }
    if (!red) return std::nullopt;
    const auto ps = shape(red->x);                                   // [n, 1, o, oh, ow, c, kh, kw]
    std::vector<int> axes = red->axes;
    std::sort(axes.begin(), axes.end());
    if (ps.size() != 8 || axes != std::vector<int>{5, 6, 7} || ps[1] != 1) return std::nullopt;
    const uint64_t N = ps[0], O = ps[2], OH = ps[3], OW = ps[4], C = ps[5], KH = ps[6], KW = ps[7];
    if (out != std::vector<uint64_t>{N, O, OH, OW}) return std::nullopt;
    ClassId prod = red->x;
    auto mul = binary(prod, B_MUL);
    if (!mul) { auto k = cast_src(prod); if (!k || !(mul = binary(*k, B_MUL))) return std::nullopt; }   // the accumulator cast
    for (int swap = 0; swap < 2; ++swap) {
      const ClassId xe = swap ? mul->second : mul->first, we = swap ? mul->first : mul->second;
      auto wr = expand_src(we);
      if (!wr || shape(*wr) != std::vector<uint64_t>{1, 1, O, 1, 1, C, KH, KW}) continue;
      auto wsrc = reshape_src(*wr);
      if (!wsrc || shape(*wsrc) != std::vector<uint64_t>{O, C, KH, KW}) continue;
      const ClassId w = canon(*wsrc), x = view_source(xe);
      const auto xs = shape(x);
      if (shape(xe) != ps || xs.size() != 4 || xs[0] != N || xs[1] != C) continue;
      const int dt = dtype(x);
      if (dtype(w) != dt || dtype(cid) != dt || (bias != NONE && dtype(bias) != dt)) continue;
      if (!(dt == ZYXB_F32 || dt == ZYXB_BF16 || dt == ZYXB_F16 || dt == ZYXB_I32)) continue;
      const uint64_t H = xs[2], W = xs[3];
      // the declared padding: the Pad nodes directly on x (rpad_zeros pads the last axis first)
      uint64_t pad[4] = {0, 0, 0, 0};                                // top, bottom, left, right
      {
        std::vector<ClassId> chain;
        for (ClassId c = xe; c != x; c = nodes[classes[c].nodes[0]].x) chain.push_back(c);
        uint64_t ext[4] = {N, C, H, W};
        for (auto it = chain.rbegin(); it != chain.rend(); ++it) {
          const Node& n = nodes[classes[*it].nodes[0]];
          if (n.kind != K_PAD || n.lp < 0 || (n.axes[0] != 2 && n.axes[0] != 3)) break;
          const int64_t after = (int64_t)n.len - n.lp - (int64_t)ext[n.axes[0]];
          if (after < 0) break;
          pad[n.axes[0] == 2 ? 0 : 2] += (uint64_t)n.lp; pad[n.axes[0] == 2 ? 1 : 3] += (uint64_t)after;
          ext[n.axes[0]] = n.len;
        }
      }
      auto probe = [&](uint64_t b, uint64_t co, uint64_t oy, uint64_t ox, uint64_t ci, uint64_t kr, uint64_t ks) {
        return trace_element(xe, {b, 0, co, oy, ox, ci, kr, ks});
      };
      // Stride and dilation, measured: along an axis a window o and tap t read coordinate o*stride + t*dilation - pad when that
      // is inside the image and padding otherwise.  Every (window, tap) pair of the axis is probed (at a window and tap of the OTHER
      // axis that are themselves inside the image); two windows under one tap give the stride, two taps under one window the
      // dilation.  Where padding leaves too few probes inside the image for that (an image smaller than its padding), any pair
      // that explains all probes - inside and outside - and the output extent describes the same convolution: the first one found
      // is taken.
      auto solve_axis = [&](bool rows) -> std::optional<std::pair<uint64_t, uint64_t>> {
        const int64_t n_out = (int64_t)(rows ? OH : OW), n_tap = (int64_t)(rows ? KH : KW), extent = (int64_t)(rows ? H : W);
        const int64_t before = (int64_t)(rows ? pad[0] : pad[2]), total = extent + (int64_t)(rows ? pad[0] + pad[1] : pad[2] + pad[3]);
        struct P { int64_t o, t, r; };                               // r < 0: padding
        std::vector<P> probes;
        bool any = false;
        for (uint64_t other : sample_axis(rows ? OW : OH)) {
          for (uint64_t tap = 0; tap < (rows ? KW : KH) && !any; ++tap) {
            probes.clear();
            for (uint64_t o : sample_axis((uint64_t)n_out)) for (int64_t t = 0; t < n_tap; ++t) {
              const Origin a = rows ? probe(0, 0, o, other, 0, (uint64_t)t, tap) : probe(0, 0, other, o, 0, tap, (uint64_t)t);
              const bool inside = !a.zero && a.cls == x;
              probes.push_back({(int64_t)o, t, inside ? (int64_t)a.idx[rows ? 2 : 3] : -1});
              any = any || inside;
            }
          }
          if (any) break;
        }
        if (!any) return std::nullopt;                               // nothing of the image is ever read
        auto explains = [&](int64_t s, int64_t d) {
          if (s <= 0 || d <= 0 || total < d * (n_tap - 1) + 1 || (total - (d * (n_tap - 1) + 1)) / s + 1 != n_out) return false;
          for (const P& a : probes) {
            const int64_t at = a.o * s + a.t * d - before;
            if (a.r >= 0 ? at != a.r : (at >= 0 && at < extent)) return false;
          }
          return true;
        };
        int64_t s = 0, d = n_tap == 1 ? 1 : 0;                       // 0: not known yet; a single tap never takes its dilation
        for (const P& a : probes) for (const P& b : probes) {
          if (a.r < 0 || b.r < 0) continue;
          if (!s && a.t == b.t && b.o > a.o && (b.r - a.r) % (b.o - a.o) == 0) s = (b.r - a.r) / (b.o - a.o);
          if (!d && a.o == b.o && b.t > a.t && (b.r - a.r) % (b.t - a.t) == 0) d = (b.r - a.r) / (b.t - a.t);
        }
        if (s && d && explains(s, d)) return std::make_pair((uint64_t)s, (uint64_t)d);
        for (int64_t sc = s ? s : 1; sc <= (s ? s : total + 1); ++sc)      // what is measured stays; the rest is searched
          for (int64_t dc = d ? d : 1; dc <= (d ? d : total + 1); ++dc)
            if (explains(sc, dc)) return std::make_pair((uint64_t)sc, (uint64_t)dc);
        return std::nullopt;
      };
      auto rows_sd = solve_axis(true), cols_sd = solve_axis(false);
      if (!rows_sd || !cols_sd) continue;
      const std::optional<uint64_t> sh = rows_sd->first, dh = rows_sd->second, sw = cols_sd->first, dw = cols_sd->second;
      // the output extent the declared padding gives must be the view's
      auto out_extent = [](uint64_t in, uint64_t before, uint64_t after, uint64_t k, uint64_t s, uint64_t d) -> uint64_t {
        const uint64_t span = d * (k - 1) + 1, padded = in + before + after;
        return padded < span ? 0 : (padded - span) / s + 1;
      };
      if (out_extent(H, pad[0], pad[1], KH, *sh, *dh) != OH || out_extent(W, pad[2], pad[3], KW, *sw, *dw) != OW) continue;
      auto reads = [&](uint64_t b, uint64_t co, uint64_t oy, uint64_t ox, uint64_t ci, uint64_t kr, uint64_t ks) {
        const Origin o = probe(b, co, oy, ox, ci, kr, ks);
        const int64_t row = (int64_t)(oy * *sh + kr * *dh) - (int64_t)pad[0], col = (int64_t)(ox * *sw + ks * *dw) - (int64_t)pad[2];
        if (row < 0 || row >= (int64_t)H || col < 0 || col >= (int64_t)W) return o.zero;
        return !o.zero && o.cls == x && o.idx == std::vector<uint64_t>{b, ci, (uint64_t)row, (uint64_t)col};
      };
      bool ok = true;
      const auto oys = sample_axis(OH), oxs = sample_axis(OW), bs = sample_axis(N), cs = sample_axis(C);
      for (uint64_t b : {(uint64_t)0, N - 1}) for (uint64_t ci : {(uint64_t)0, C - 1}) for (uint64_t co : {(uint64_t)0, O - 1})
        for (uint64_t oy : oys) for (uint64_t ox : oxs) for (uint64_t kr = 0; kr < KH && ok; ++kr) for (uint64_t ks = 0; ks < KW && ok; ++ks)
          ok = reads(b, co, oy, ox, ci, kr, ks);
      for (uint64_t b : bs) for (uint64_t ci : cs) {
        if (!ok) break;
        ok = reads(b, 0, 0, 0, ci, 0, 0) && reads(b, O - 1, OH - 1, OW - 1, ci, KH - 1, KW - 1) && reads(b, 0, OH / 2, OW / 2, ci, KH / 2, KW / 2);
      }
      if (!ok) continue;
      Match m;
      m.pattern = bias != NONE ? "conv_bias" : "conv";
      m.desc.kind = ZYXB_KIND_CONV;
      auto& c = m.desc.u.conv;
      c.dtype = dt; c.n = N; c.c = C; c.h = H; c.w = W; c.o = O; c.kh = KH; c.kw = KW;
      c.stride_h = (uint32_t)*sh; c.stride_w = (uint32_t)*sw; c.dil_h = (uint32_t)*dh; c.dil_w = (uint32_t)*dw;
      c.pad_top = (uint32_t)pad[0]; c.pad_bottom = (uint32_t)pad[1]; c.pad_left = (uint32_t)pad[2]; c.pad_right = (uint32_t)pad[3];
      c.has_bias = bias != NONE;
      m.inputs = {x, w};
      if (bias != NONE) m.inputs.push_back(bias);
      m.outputs = {cid};
      return m;
    }
    return std::nullopt;
  }

  // ---- cross-entropy with class-index targets ----------------------------------------------------------------------------
  // c = [Cast]{Eq{Expand{labels.reshape([n, 1])}, Expand{arange(classes)}}}, in either operand order -> labels [n]
  // (Tensor::one_hot_along_dim of the unsqueezed labels, tensor/mod.rs:1920-1946).  The arange is recognised by its value: any
  // subgraph of constants that evaluates to 0, 1, .., classes - 1.  i32 labels only (what the program reads).
  std::optional<ClassId> one_hot_labels(ClassId c, uint64_t n, uint64_t classes) const {
    if (auto k = cast_src(c)) c = *k;
    auto eq = binary(c, B_EQ);
    if (!eq) return std::nullopt;
    for (int swap = 0; swap < 2; ++swap) {
      auto ea = expand_src(swap ? eq->second : eq->first), eb = expand_src(swap ? eq->first : eq->second);
      if (!ea || !eb || shape(*ea) != std::vector<uint64_t>{n, 1}) continue;
      if (shape(*eb) != std::vector<uint64_t>{classes} && shape(*eb) != std::vector<uint64_t>{1, classes}) continue;
      auto labels = reshape_src(*ea);
      if (!labels || shape(*labels) != std::vector<uint64_t>{n} || dtype(*labels) != ZYXB_I32) continue;
      auto v = const_eval(*eb);
      if (!v || v->size() != classes) continue;
      bool iota = true;
      for (uint64_t i = 0; i < classes && iota; ++i) iota = (*v)[i] == (double)i;
      if (iota) return canon(*labels);
    }
    return std::nullopt;
  }
  // Tensor::cross_entropy(labels, ReduceOp::Mean) on f32 logits [n, classes] (tensor/mod.rs:1639-1656):
  //   per_sample = (-logits.ln_softmax([1]) * one_hot(labels)).sum([1]);   loss = per_sample.mean_all()
  // -> one program, args logits, labels -> per_sample, loss; the one-hot matrix and the log-probabilities never exist.
  std::optional<Match> match_cross_entropy(ClassId cid) const {
    if (dtype(cid) != ZYXB_F32) return std::nullopt;
    auto div = binary_const(cid, B_DIV);
    if (!div) return std::nullopt;
    const Node* red = find(div->first, [](const Node& n) { return n.kind == K_REDUCE && n.op == B_ADD; });
    if (!red) return std::nullopt;
    const ClassId per_sample = canon(red->x);        // under the no-op accumulator cast of `sum`: the class the caller holds
    const auto ps = shape(per_sample);
    if (ps.size() != 1 || red->axes.size() != 1 || fabs(div->second - (double)ps[0]) > 0.5 || dtype(per_sample) != ZYXB_F32) return std::nullopt;
    auto prod = reduce_last(per_sample, B_ADD);
    if (!prod || shape(*prod).size() != 2 || shape(*prod)[0] != ps[0]) return std::nullopt;
    const std::vector<uint64_t> nc = shape(*prod);
    auto mul = binary(*prod, B_MUL);
    if (!mul) return std::nullopt;
    for (int swap = 0; swap < 2; ++swap) {
      auto lsm = unary(swap ? mul->second : mul->first, U_NEG);
      if (!lsm) continue;
      auto ls = match_ln_softmax(*lsm);
      if (!ls || dtype(ls->inputs[0]) != ZYXB_F32 || shape(ls->inputs[0]) != nc) continue;
      auto labels = one_hot_labels(swap ? mul->first : mul->second, nc[0], nc[1]);
      if (!labels) continue;
      Match m; m.pattern = "cross_entropy"; m.desc = row_desc(ZYXB_RR_CROSS_ENTROPY, ZYXB_F32, nc);
      m.inputs = {ls->inputs[0], *labels}; m.outputs = {per_sample, cid};
      return m;
    }
    return std::nullopt;
  }

  // ---- optimizer updates -------------------------------------------------------------------------------------------------
  struct Update {
    int algo; ClassId p, g, m = NONE, v = NONE, p_new, m_new = NONE, v_new = NONE;     // SGD with momentum: m is the buffer
    double lr, wd = 0, b1 = 0, b2 = 0, eps = 0, bc1 = 0, bc2 = 0, mom = 0, damp = 0;
    bool first = false, nesterov = false;
  };

  // p' = (p - g * lr).cast(p.dtype)   (sgd.rs:79-82, no weight decay, no momentum)
  //   G = g [+ p * weight_decay]
  //   momentum, after the first step:  buf' = buf * momentum + G * (1 - dampening);  p' = (p - buf' * lr)            (sgd.rs:63-75)
  //   nesterov:                                                                       p' = (p - (G + buf' * momentum) * lr)
  // On the first step the reference stores G itself as the buffer (no node is added), so that update is the plain form.
  std::optional<Update> match_sgd(ClassId cid) const {
    const ClassId c = canon(cid);
    auto sub = binary(c, B_SUB);
    if (!sub) return std::nullopt;
    auto step = binary_const(sub->second, B_MUL);
    if (!step || !is_leaf(sub->first) || shape(step->first) != shape(sub->first)) return std::nullopt;
    Update u{}; u.algo = ZYXB_OPT_SGD; u.p = sub->first; u.g = step->first; u.p_new = cid; u.lr = step->second;
    // x + y * const with y the class `of` (or, of == NONE, any stored tensor of the parameter's shape)
    auto plus_scaled = [&](ClassId e, ClassId of) -> std::optional<std::tuple<ClassId, ClassId, double>> {
      auto add = binary(e, B_ADD);
      if (!add) return std::nullopt;
      for (int swap = 0; swap < 2; ++swap) {
        const ClassId lhs = swap ? add->second : add->first, rhs = swap ? add->first : add->second;
        auto k = binary_const(rhs, B_MUL);
        if (k && (of == NONE ? shape(k->first) == shape(u.p) : same(k->first, of))) return std::make_tuple(lhs, k->first, k->second);
      }
      return std::nullopt;
    };
    auto strip_decay = [&](ClassId G) { if (auto d = plus_scaled(G, u.p)) { u.wd = std::get<2>(*d); return std::get<0>(*d); } return G; };
    // buf' = buf * momentum + G * (1 - dampening), buf a stored tensor
    auto buffer_update = [&](ClassId b) -> bool {
      auto add = binary(b, B_ADD);
      if (!add) return false;
      auto old = binary_const(add->first, B_MUL), fresh = binary_const(add->second, B_MUL);
      if (!old || !fresh || !is_leaf(old->first) || same(old->first, u.p) || shape(old->first) != shape(u.p)) return false;
      u.m = old->first; u.mom = old->second; u.damp = 1.0 - fresh->second; u.m_new = b; u.g = strip_decay(fresh->first);
      return true;
    };
    const ClassId x = step->first;
    if (auto nes = plus_scaled(x, NONE)) {                     // G + buf' * momentum ?
      const Update keep = u;
      if (!is_leaf(std::get<1>(*nes)) && buffer_update(std::get<1>(*nes)) && fabs(std::get<2>(*nes) - u.mom) <= 1e-12 * fabs(u.mom)) {
        double wd2 = 0;
        const ClassId G = std::get<0>(*nes);
        ClassId g_plain = G;
        if (auto d = plus_scaled(G, u.p)) { g_plain = std::get<0>(*d); wd2 = std::get<2>(*d); }
        if (same(g_plain, u.g) && wd2 == u.wd) { u.nesterov = true; return u; }
      }
      u = keep;
    }
    if (buffer_update(x)) return u;
    u.g = strip_decay(x);
    return u;
  }
  bool is_leaf(ClassId c) const { return find(c, [](const Node& n) { return n.kind == K_LEAF; }) != nullptr; }

  // m' = m*b1 + g*(1-b1)  |  g*(1-b1) on the first step
  bool moment(ClassId mc, bool squared, ClassId& state, double& beta, ClassId& g) const {
    auto grad_term = [&](ClassId t, double& one_minus) -> std::optional<ClassId> {
      auto k = binary_const(t, B_MUL);
      if (!k) return std::nullopt;
      one_minus = k->second;
      if (!squared) return k->first;
      auto gg = binary(k->first, B_MUL);
      if (!gg || !same(gg->first, gg->second)) return std::nullopt;
      return gg->first;
    };
    double om = 0;
    if (auto add = binary(mc, B_ADD)) {
      auto decay = binary_const(add->first, B_MUL);
      auto gt = grad_term(add->second, om);
      if (decay && gt && is_leaf(decay->first)) { state = decay->first; beta = 1.0 - om; g = *gt; return true; }
    }
    if (auto gt = grad_term(mc, om)) { state = NONE; beta = 1.0 - om; g = *gt; return true; }
    return false;
  }

  // Adam::update for one parameter without amsgrad (adam.rs:66-101), ending at the new parameter's class:
  //   G = g [+ p * weight_decay];  m' and v' as in AdamW;  p' = (p - lr * mh / (sqrt(vh) + eps)).cast(p.dtype)
  std::optional<Update> match_adam(ClassId cid) const {
    Update u{}; u.algo = ZYXB_OPT_ADAM; u.p_new = cid;
    auto sub = binary(canon(cid), B_SUB);
    if (!sub || !is_leaf(sub->first)) return std::nullopt;
    u.p = sub->first;
    auto step = binary(sub->second, B_DIV);                    // (lr * mh) / (sqrt(vh) + eps)
    if (!step) return std::nullopt;
    auto num = binary_const(step->first, B_MUL);
    auto root_eps = binary_const(step->second, B_ADD);
    if (!num || !root_eps) return std::nullopt;
    u.lr = num->second; u.eps = root_eps->second;
    auto vh = unary(root_eps->first, U_SQRT);
    if (!vh) return std::nullopt;
    auto mh = binary_const(num->first, B_DIV), vhd = binary_const(*vh, B_DIV);
    if (!mh || !vhd) return std::nullopt;
    u.bc1 = mh->second; u.bc2 = vhd->second; u.m_new = mh->first; u.v_new = vhd->first;
    ClassId g1 = NONE, g2 = NONE;
    if (!moment(u.m_new, false, u.m, u.b1, g1) || !moment(u.v_new, true, u.v, u.b2, g2) || !same(g1, g2)) return std::nullopt;
    if ((u.m == NONE) != (u.v == NONE)) return std::nullopt;
    u.first = u.m == NONE;
    u.g = g1;
    // weight decay enters the gradient: G = g + p * wd
    if (auto add = binary(g1, B_ADD))
      for (int swap = 0; swap < 2; ++swap) {
        const ClassId lhs = swap ? add->second : add->first, rhs = swap ? add->first : add->second;
        auto k = binary_const(rhs, B_MUL);
        if (k && same(k->first, u.p)) { u.g = lhs; u.wd = k->second; break; }
      }
    return u;
  }

  // AdamW::update for one parameter (adamw.rs:58-95), ending at the new parameter's class
  std::optional<Update> match_adamw(ClassId cid) const {
    Update u{}; u.algo = ZYXB_OPT_ADAMW; u.p_new = cid;
    ClassId c = cid;
    if (auto decay = binary_const(c, B_MUL)) if (!is_leaf(decay->first)) { u.wd = 1.0 - decay->second; c = decay->first; }   // p * (1 - lr*wd)
    c = canon(c);
    auto sub = binary(c, B_SUB);
    if (!sub || !is_leaf(sub->first)) return std::nullopt;
    u.p = sub->first;
    auto step = binary(sub->second, B_DIV);                    // mh / ((sqrt(vh) + eps) * lr)
    if (!step) return std::nullopt;
    auto den = binary_const(step->second, B_MUL);
    if (!den) return std::nullopt;
    u.lr = den->second;
    auto root_eps = binary_const(den->first, B_ADD);
    if (!root_eps) return std::nullopt;
    u.eps = root_eps->second;
    auto vh = unary(root_eps->first, U_SQRT);
    if (!vh) return std::nullopt;
    auto mh = binary_const(step->first, B_DIV), vhd = binary_const(*vh, B_DIV);
    if (!mh || !vhd) return std::nullopt;
    u.bc1 = mh->second; u.bc2 = vhd->second; u.m_new = mh->first; u.v_new = vhd->first;
    ClassId g1 = NONE, g2 = NONE;
    if (!moment(u.m_new, false, u.m, u.b1, g1) || !moment(u.v_new, true, u.v, u.b2, g2) || !same(g1, g2)) return std::nullopt;
    u.g = g1;
    u.first = u.m == NONE;
    if ((u.m == NONE) != (u.v == NONE)) return std::nullopt;
    if (u.wd != 0) u.wd /= u.lr;
    return u;
  }

  // ---- the device's match_graph (backend/mod.rs:952-961; model backend/cblas.rs:213-238) --------------------------------
  // Visits `order` (Graph::topo_sort_classes_without_kernels of the outputs), and for every class some pattern ends at pushes a
  // Node::Kernel{inputs, outputs, program_id, time: 1} into that class.  Optimizer updates of one dtype and one set of
  // hyper-parameters become one multi-tensor program whose Kernel node is pushed into every class it writes.
  std::vector<Match> match_graph(const std::vector<ClassId>& order, const std::set<ClassId>& wanted) {
    std::vector<Match> out;
    std::vector<Update> updates;
    for (ClassId cid : order) {
      if (!valid(cid) || find(cid, [](const Node& n) { return n.kind == K_KERNEL; })) continue;
      std::optional<Match> m;
      if (wanted.count(cid)) {      // new parameter values are outputs of the graph; their sub-expressions are not matched as updates
        if (auto u = match_adamw(cid)) { updates.push_back(*u); continue; }
        if (auto u = match_adam(cid)) { updates.push_back(*u); continue; }
        if (auto u = match_sgd(cid)) { updates.push_back(*u); continue; }
      }
      if (!(m = match_attention(cid)) && !(m = match_linear(cid, wanted)) && !(m = match_conv(cid)) && !(m = match_softmax(cid)) && !(m = match_ln_softmax(cid)) && !(m = match_layernorm(cid)) &&
          !(m = match_cross_entropy(cid)) && !(m = match_mse(cid)) && !(m = match_reduce(cid)))
        continue;
      out.push_back(std::move(*m));
    }
    // group the per-parameter updates: one program per (algorithm, dtype, hyper-parameters, first step or not)
    std::vector<char> used(updates.size(), 0);
    for (size_t i = 0; i < updates.size(); ++i) {
      if (used[i]) continue;
      const Update& h = updates[i];
      const bool sgd_buf = h.algo == ZYXB_OPT_SGD && h.m != NONE;
      const std::string adam_name = h.algo == ZYXB_OPT_ADAM ? "adam" : "adamw";
      Match mt; mt.pattern = h.algo == ZYXB_OPT_SGD ? (sgd_buf ? (h.nesterov ? "sgd_nesterov" : "sgd_momentum") : "sgd") : (h.first ? adam_name + "_first_step" : adam_name);
      // the step the update belongs to: AdamW's bias correction divides by 1 - beta1^t
      mt.optim_step = h.algo == ZYXB_OPT_SGD ? (sgd_buf ? 2 : 1)
                                             : (h.first ? 1 : (uint64_t)std::max(2.0, std::round(std::log(1.0 - h.bc1) / std::log(h.b1))));
      std::vector<ClassId> p, g, mm, vv, outs;
      for (size_t j = i; j < updates.size(); ++j) {
        const Update& u = updates[j];
        if (used[j] || u.algo != h.algo || dtype(u.p) != dtype(h.p) || u.first != h.first || u.lr != h.lr || u.wd != h.wd || u.b1 != h.b1 ||
            u.b2 != h.b2 || u.eps != h.eps || u.bc1 != h.bc1 || u.bc2 != h.bc2 || u.mom != h.mom || u.damp != h.damp || u.nesterov != h.nesterov ||
            (u.m == NONE) != (h.m == NONE)) continue;
        used[j] = 1;
        p.push_back(u.p); g.push_back(u.g); mt.numel.push_back(numel(shape(u.p)));
        outs.push_back(u.p_new);
        if (u.algo != ZYXB_OPT_SGD) { mm.push_back(u.m); vv.push_back(u.v); outs.push_back(u.m_new); outs.push_back(u.v_new); }
        else if (u.m != NONE) { mm.push_back(u.m); outs.push_back(u.m_new); }
      }
      mt.desc.kind = ZYXB_KIND_OPTIM;
      auto& o = mt.desc.u.optim;
      o.algo = h.algo; o.dtype = dtype(h.p); o.n_tensors = (int32_t)p.size(); o.lr = (float)h.lr; o.weight_decay = (float)h.wd;
      o.beta1 = (float)h.b1; o.beta2 = (float)h.b2; o.eps = (float)h.eps;
      o.momentum = (float)h.mom; o.dampening = (float)h.damp; o.nesterov = h.nesterov ? 1 : 0;
      mt.inputs = p; mt.inputs.insert(mt.inputs.end(), g.begin(), g.end());
      if (sgd_buf) mt.inputs.insert(mt.inputs.end(), mm.begin(), mm.end());
      if (h.algo != ZYXB_OPT_SGD && !h.first) { mt.inputs.insert(mt.inputs.end(), mm.begin(), mm.end()); mt.inputs.insert(mt.inputs.end(), vv.begin(), vv.end()); }
      mt.outputs = outs;
      out.push_back(std::move(mt));
    }
    // Elementwise programs, on demand.  Walk down from the outputs of the graph through the programs found above (for a class
    // several of them end at, the one found last: the largest pattern): whatever that walk needs and nothing stored or matched
    // produces gets an elementwise program if one fits, and the walk continues through its operands.  Offering every Mul and Add
    // of the graph as a program of its own would bury the patterns above under their own sub-expressions; following the inputs of
    // every alternative would do the same with the inside of a softmax.
    auto has_kernel = [&](ClassId c) { for (uint32_t nid : classes[c].nodes) if (nodes[nid].kind == K_KERNEL) return true; return false; };
    std::map<ClassId, size_t> producer;
    {
      for (size_t i = 0; i < out.size(); ++i) for (ClassId o : out[i].outputs) producer[canon(o)] = i;
      std::set<ClassId> seen;
      std::vector<ClassId> need(wanted.rbegin(), wanted.rend());
      while (!need.empty()) {
        ClassId c = need.back();
        need.pop_back();
        if (!valid(c)) continue;
        if (!producer.count(canon(c))) c = storage(c);                // nothing ends at the reshaped class: its elements are the source's
        if (!seen.insert(canon(c)).second || is_leaf(c)) continue;
        auto it = producer.find(canon(c));
        if (it == producer.end()) {
          if (has_kernel(c) || has_kernel(canon(c))) continue;
          auto m = match_eltwise(c);
          if (!m) continue;
          out.push_back(std::move(*m));
          it = producer.emplace(canon(c), out.size() - 1).first;
        }
        const Match& via = out[it->second];
        need.insert(need.end(), via.inputs.rbegin(), via.inputs.rend());
      }
    }
    // inputs are named by the class whose buffer holds them (a reshape of a stored tensor is that tensor), unless a program ends at the reshape itself
    for (Match& m : out) for (ClassId& in : m.inputs) if (!producer.count(canon(in)) && !has_kernel(in) && !has_kernel(canon(in))) in = storage(in);
    for (size_t i = 0; i < out.size(); ++i) {
      if (out[i].desc.kind == ZYXB_KIND_OPTIM) out[i].desc.u.optim.numel = out[i].numel.data();
      Node k; k.kind = K_KERNEL; k.inputs = out[i].inputs; k.outputs = out[i].outputs; k.program = (uint32_t)i; k.time = 1;
      nodes.push_back(k);
      for (ClassId o : out[i].outputs) classes[o].nodes.push_back((uint32_t)nodes.size() - 1);
    }
    return out;
  }

  // What the programs pushed so far do NOT cover: walking down from `outputs` through the Node::Kernel alternatives (at each
  // class the one pushed last, the largest pattern), the classes that are needed but are neither stored nor produced by a
  // program.  Empty: the device can execute the graph on its own.
  std::vector<ClassId> uncovered(const std::vector<ClassId>& outputs) const {
    std::vector<ClassId> missing, need(outputs.rbegin(), outputs.rend());
    std::set<ClassId> seen;
    while (!need.empty()) {
      ClassId c = need.back();
      need.pop_back();
      if (!valid(c) || !seen.insert(canon(c)).second || is_leaf(c)) continue;
      const Node* kernel = nullptr;
      for (ClassId k = c;;) {                               // the class, what it is a no-op of, what it is a reshape of
        for (uint32_t nid : classes[k].nodes) if (nodes[nid].kind == K_KERNEL) kernel = &nodes[nid];
        if (kernel) break;
        const Node* through = noop_cast(k);
        if (!through) through = find(k, [](const Node& n) { return n.kind == K_RESHAPE; });
        if (!through) break;
        k = through->x;
        if (is_leaf(k)) break;
      }
      if (!kernel) { if (!is_leaf(storage(c))) missing.push_back(c); continue; }
      need.insert(need.end(), kernel->inputs.rbegin(), kernel->inputs.rend());
    }
    return missing;
  }

  // every class reachable from `outputs`, operands before users (the order match_graph walks)
  std::vector<ClassId> topo_order(const std::vector<ClassId>& outputs) const {
    std::vector<ClassId> order;
    std::vector<char> seen(classes.size(), 0);
    std::vector<std::pair<ClassId, bool>> stack;
    for (auto it = outputs.rbegin(); it != outputs.rend(); ++it) stack.push_back({*it, false});   // the first output is visited first
    while (!stack.empty()) {
      auto [c, done] = stack.back();
      stack.pop_back();
      if (!valid(c)) continue;
      if (done) { order.push_back(c); continue; }
      if (seen[c]) continue;
      seen[c] = 1;
      stack.push_back({c, true});
      const Node& n = nodes[classes[c].nodes[0]];
      if (n.x != NONE) stack.push_back({n.x, false});
      if (n.y != NONE) stack.push_back({n.y, false});
    }
    return order;
  }

 private:
  std::map<std::string, ClassId> memo_;
  static std::string key_of(const Node& n) {
    std::string k = std::to_string(n.kind) + ":" + std::to_string(n.x) + ":" + std::to_string(n.y) + ":" + std::to_string(n.op) + ":" +
                    std::to_string(n.dtype) + ":" + std::to_string(n.leaf_id) + ":";
    char buf[32];
    snprintf(buf, sizeof buf, "%.17g", n.value);
    k += buf;
    for (uint64_t d : n.shape) k += "," + std::to_string(d);
    k += "|";
    for (int a : n.axes) k += "," + std::to_string(a);
    if (n.kind == K_PAD) k += "|" + std::to_string(n.lp) + "," + std::to_string(n.len);
    return k;
  }
};

}  // namespace zyxb_matcher
