// zyx/src/vendor/b200.rs — subgraph -> kernel-descriptor matching for the B200 backend (`mod b200;` in vendor/mod.rs).
//
// NOT COMPILED (no Rust toolchain in the build image).  It is a line-by-line port of zyx_b200/csrc/host/matcher.hpp, the C++
// matcher that tests/test_matcher.py exercises through the C ABI on node lists transcribed from Tensor::dot, Linear::forward,
// softmax, ln_softmax, LayerNorm::forward, cross_entropy, SGD::update, Adam::update and AdamW::update; function names and order are kept the same so the two
// can be read side by side.  It extends Graph::match_matmul (vendor/matmul.rs:43-71) and reuses the helpers of
// vendor/mod.rs:28-95 (`const_shape`).

#![allow(unused)]

use std::collections::{BTreeMap, BTreeSet};

use crate::{
    DType,
    dtype::Constant,
    backend::b200::{ZyxbAttentionDesc, ZyxbConvDesc, ZyxbDescUnion, ZyxbEltwiseDesc, ZyxbGemmDesc, ZyxbKernelDesc, ZyxbOptimDesc, ZyxbRowreduceDesc, ZYXB_KIND_ATTENTION,
                    ZYXB_KIND_CONV, ZYXB_KIND_ELTWISE, ZYXB_KIND_GEMM, ZYXB_KIND_OPTIM, ZYXB_KIND_ROWREDUCE},
    graph::{ClassId, Graph, Node},
    kernel::{BOp, UOp},
    shape::Dim,
};

/// One recognised subgraph: the descriptor for zyxb_program_create and the launch arguments (loads, then stores).
pub(crate) struct B200Match {
    pub(crate) pattern: &'static str,
    pub(crate) inputs: Vec<ClassId>,
    pub(crate) outputs: Vec<ClassId>,
    pub(crate) desc: ZyxbKernelDesc,
    /// optimizer programs: element counts per tensor (desc.u.optim.numel is pointed here by the caller)
    pub(crate) numel: Vec<u64>,
    /// optimizer programs: the step t the matched update belongs to (1 = the first); the program's counter must be t - 1 before the launch
    pub(crate) optim_step: u64,
    /// per input: the element of that class's buffer the program's argument starts at (empty: all 0) - a matmul operand that is a
    /// slice of a stored tensor, e.g. q of a fused q/k/v projection; the device passes a view of the buffer
    pub(crate) input_offsets: Vec<u64>,
}

/// A constant's value as f64 (Constant::cast, dtype.rs:502-518, widens every variant).
fn const_f64(k: Constant) -> f64 {
    match k.cast(DType::F64) { Constant::F64(b) => f64::from_le_bytes(b), _ => unreachable!() }
}
/// What a Cast node does to a folded value: Bool is `!= 0`, f32 rounds, the integer types truncate.
fn cast_value(v: f64, dt: DType) -> f64 {
    match dt { DType::Bool => (v != 0.0) as u8 as f64, DType::F32 => v as f32 as f64, DType::F64 | DType::BF16 | DType::F16 => v, _ => v.trunc() }
}

/// every index of a short axis; both ends and a spread of a long one
fn sample_axis(n: u64) -> Vec<u64> {
    if n <= 48 { return (0..n).collect(); }
    (0..16).chain((1..=16).map(|i| 16 + i * (n - 32) / 17)).chain(n - 16..n).collect()
}

#[derive(Clone, Copy)]
struct MatMulX {
    a: ClassId, b: ClassId, m: Dim, n: Dim, k: Dim, batch: Dim, trans_a: bool, trans_b: bool, b_shared: bool, dtype: DType,
    /// rank-4 products over [b, h, .., ..]: operands (and, at the merged class, the result) that are per-head views of stored
    /// [b, t, h*d] tensors are read where they lie through a row pitch and a two-level batch
    outer: Dim, heads: Dim, a_heads: bool, b_heads: bool, c_heads: bool,
    /// a_heads / b_heads: where the view starts in the stored tensor and how it steps (elements)
    a_view: Pitch, b_view: Pitch,
}
#[derive(Clone, Copy, Default, PartialEq)]
struct Pitch { offset: u64, ld: u64, inner: u64, outer: u64 }

#[derive(Clone, Copy)]
struct Update { algo: i32, p: ClassId, g: ClassId, m: Option<ClassId>, v: Option<ClassId>, p_new: ClassId, m_new: Option<ClassId>,
                v_new: Option<ClassId>, lr: f64, wd: f64, b1: f64, b2: f64, eps: f64, bc1: f64, bc2: f64, first: bool,
                mom: f64, damp: f64, nesterov: bool }      // SGD with momentum: m / m_new are the buffer

const RR_SUM: i32 = 0; const RR_MAX: i32 = 1; const RR_MIN: i32 = 2; const RR_MEAN: i32 = 3; const RR_SOFTMAX: i32 = 6; const RR_LN_SOFTMAX: i32 = 7; const RR_LAYERNORM: i32 = 8; const RR_MSE: i32 = 14;
const RR_VAR: i32 = 4; const RR_STD: i32 = 5; const RR_COLSUM: i32 = 13; const RR_CROSS_ENTROPY: i32 = 9;
const EW_RELU: i32 = 0; const EW_GELU: i32 = 1; const EW_ADD: i32 = 2; const EW_SUB: i32 = 3; const EW_MUL: i32 = 4; const EW_SCALE: i32 = 5;
const EW_CAST: i32 = 9; const EW_TANH: i32 = 10; const EW_SIGMOID: i32 = 11; const EW_EXP: i32 = 12; const EW_BIAS_ADD: i32 = 13;
const EPI_NONE: i32 = 0; const EPI_BIAS: i32 = 1; const EPI_BIAS_RELU: i32 = 2; const EPI_BIAS_GELU: i32 = 3; const EPI_ADD: i32 = 6;
const OPT_SGD: i32 = 0; const OPT_ADAM: i32 = 1; const OPT_ADAMW: i32 = 2;

fn near(a: f64, b: f64) -> bool { (a - b).abs() <= 1e-2 * b.abs() }       // constants arrive rounded to the tensor dtype

impl Graph {
    // ---- node finders; a class may be a no-op Cast of the class holding the node (runtime.rs:696-700 pushes a Cast for every
    // `.cast`, also when the dtype does not change), so those are looked through ------------------------------------------------
    /// a node that leaves its operand as it is: a Cast to the dtype the operand has, `x * 1`, `x / 1` (what dropout leaves behind
    /// outside training with p = 0: x / (1 - p), tensor/mod.rs:822-828)
    fn noop_cast(&self, c: ClassId) -> Option<ClassId> {
        self.classes[c].nodes.iter().find_map(|&nid| match &self.nodes[nid].node {
            Node::Cast { x, dtype } if self.dtype(*x) == *dtype => Some(*x),
            Node::Binary { x, y, bop: BOp::Mul | BOp::Div } if self.dtype(c).is_float() && self.const_shape(*x) == self.const_shape(c) => {
                let mut k = *y;                                // a rank-0 constant 1 under its Cast / Reshape / Expand wrappers
                for _ in 0..8 {
                    match &self.nodes[self.classes[k].nodes[0]].node {
                        Node::Const(v) => return (const_f64(*v) == 1.0).then_some(*x),
                        Node::Cast { x, .. } | Node::Expand { x, .. } | Node::Reshape { x, .. } => k = *x,
                        _ => return None,
                    }
                }
                None
            }
            _ => None,
        })
    }
    fn canon(&self, mut c: ClassId) -> ClassId { while let Some(x) = self.noop_cast(c) { c = x; } c }
    fn same(&self, a: ClassId, b: ClassId) -> bool { self.canon(a) == self.canon(b) }
    /// The class whose buffer holds c's elements: c under no-op nodes and Reshapes (dense row-major storage does not know its
    /// shape).  Program inputs are named by it, so that `x.reshape([0, 784])` of a stored batch is the batch's own buffer.
    fn storage(&self, mut c: ClassId) -> ClassId {
        for _ in 0..64 {
            c = self.canon(c);
            match self.reshape_of(c) { Some(x) => c = x, None => break }
        }
        self.canon(c)
    }
    fn find_in<T>(&self, mut c: ClassId, f: impl Fn(&Node) -> Option<T>) -> Option<T> {
        for _ in 0..8 {
            if let Some(t) = self.classes[c].nodes.iter().find_map(|&nid| f(&self.nodes[nid].node)) { return Some(t); }
            c = self.noop_cast(c)?;
        }
        None
    }
    fn binary_of(&self, c: ClassId, op: BOp) -> Option<(ClassId, ClassId)> {
        self.find_in(c, |n| match n { Node::Binary { x, y, bop } if *bop == op => Some((*x, *y)), _ => None })
    }
    fn unary_of(&self, c: ClassId, op: UOp) -> Option<ClassId> {
        self.find_in(c, |n| match n { Node::Unary { x, uop } if *uop == op => Some(*x), _ => None })
    }
    /// the source of a dtype-changing Cast
    fn cast_src(&self, c: ClassId) -> Option<ClassId> {
        self.find_in(c, |n| match n { Node::Cast { x, dtype } if self.dtype(*x) != *dtype => Some(*x), _ => None })
    }
    fn expand_of(&self, c: ClassId) -> Option<ClassId> { self.find_in(c, |n| match n { Node::Expand { x, .. } => Some(*x), _ => None }) }
    fn reshape_of(&self, c: ClassId) -> Option<ClassId> { self.find_in(c, |n| match n { Node::Reshape { x, .. } => Some(*x), _ => None }) }
    fn is_leaf(&self, c: ClassId) -> bool { self.find_in(c, |n| matches!(n, Node::Leaf { .. }).then_some(())).is_some() }
    fn unbroadcast(&self, mut c: ClassId) -> ClassId {
        loop {
            if let Some(x) = self.expand_of(c) { c = x; continue; }
            if let Some(x) = self.reshape_of(c) { c = x; continue; }
            return c;
        }
    }
    /// a scalar constant under Expand / Reshape / Cast wrappers (tensor/mod.rs:3033-3113: rank-0 operands are cast and expanded)
    fn const_value(&self, mut c: ClassId) -> Option<f64> {
        loop {
            if let Some(v) = self.find_in(c, |n| match n { Node::Const(k) => Some(const_f64(*k)), _ => None }) { return Some(v); }
            if let Some(x) = self.expand_of(c) { c = x; continue; }
            if let Some(x) = self.reshape_of(c) { c = x; continue; }
            if let Some(x) = self.cast_src(c) { c = x; continue; }
            return None;
        }
    }
    fn binary_const(&self, c: ClassId, op: BOp) -> Option<(ClassId, f64)> {
        let (x, y) = self.binary_of(c, op)?;
        if let Some(k) = self.const_value(y) { return Some((x, k)); }
        if op.is_commutative() { if let Some(k) = self.const_value(x) { return Some((y, k)); } }
        None
    }
    fn numel_of(&self, c: ClassId) -> Option<Dim> { Some(self.const_shape(c)?.iter().product()) }

    /// `x.<reduce>([-1])` / `_keepdim` of reduce_impl (tensor/reduce_ops.rs:45-157):
    /// [Reshape]{[Cast back]{Reduce{[Cast to acc]{x}, rop, [last]}}} -> x
    fn reduce_last(&self, c: ClassId, rop: BOp) -> Option<ClassId> {
        if let Some(r) = self.reshape_of(c) {
            if self.numel_of(r) == self.numel_of(c) { if let Some(x) = self.reduce_last(r, rop) { return Some(x); } }
        }
        let red = |cls: ClassId| self.find_in(cls, |n| match n { Node::Reduce { x, rop: r, axes } if *r == rop => Some((*x, axes.clone())), _ => None });
        let (x, axes) = red(c).or_else(|| red(self.cast_src(c)?))?;
        let rank = self.const_shape(x)?.len();
        if rank < 1 || axes.len() != 1 || axes[0] != rank - 1 { return None; }
        let mut src = x;
        if let Some(k) = self.cast_src(src) { if self.dtype(k) == self.dtype(c) { src = k; } }     // the accumulator cast, undone by the cast back
        Some(self.canon(src))
    }

    // ---- matmul: Graph::match_matmul extended to NT / TN / TT on stored tensors, rank > 2 and the accumulator casts of 16-bit inputs -------
    fn match_matmul_x(&self, cid: ClassId) -> Option<MatMulX> {
        let out_shape = self.const_shape(cid)?;
        if out_shape.len() < 2 { return None; }
        if let Some(r) = self.reshape_of(cid) {                      // dot's closing reshape to the shape the reduce already has
            if self.const_shape(r).as_ref() == Some(&out_shape) { if let Some(mm) = self.match_matmul_x(r) { return Some(mm); } }
        }
        let (m, n) = (out_shape[out_shape.len() - 2], out_shape[out_shape.len() - 1]);
        let red = |cls: ClassId| self.find_in(cls, |nd| match nd { Node::Reduce { x, rop: BOp::Add, axes } => Some((*x, axes.clone())), _ => None });
        let (prod, axes) = red(cid).or_else(|| red(self.cast_src(cid)?))?;
        let prod_shape = self.const_shape(prod)?;
        let pr = prod_shape.len();
        if pr != out_shape.len() + 1 || axes.len() != 1 || axes[0] != pr - 1 { return None; }
        let k = prod_shape[pr - 1];
        let (ea, eb) = self.binary_of(prod, BOp::Mul).or_else(|| self.binary_of(self.cast_src(prod)?, BOp::Mul))?;
        // an operand that already has the product's shape (n = 1 on the left, m = 1 on the right) is not expanded (tensor/mod.rs:3099-3107)
        let (ea, eb) = (self.expand_of(ea).unwrap_or(ea), self.expand_of(eb).unwrap_or(eb));
        let (a3, b3) = (self.const_shape(ea)?, self.const_shape(eb)?);
        let batch_dims = &out_shape[..out_shape.len() - 2];
        let want_a: Vec<Dim> = batch_dims.iter().copied().chain([m, 1, k]).collect();
        let want_b: Vec<Dim> = batch_dims.iter().copied().chain([1, n, k]).collect();
        if a3 != want_a { return None; }
        let mut b_shared = false;
        if b3 != want_b {
            let nb = b3.len();
            if nb >= 3 && b3.iter().product::<Dim>() == n * k && b3[nb - 1] == k && b3[nb - 2] == n && !batch_dims.is_empty() { b_shared = true; } else { return None; }
        }
        let mut a = ea;
        if let Some(s) = self.reshape_of(a) { if self.numel_of(s) == Some(a3.iter().product()) { a = s; } }
        // b: through the reshape to the Permute that swaps the last two axes
        let swaps_last_two = |axes: &[usize]| {
            let r = axes.len();
            r >= 2 && axes[..r - 2].iter().enumerate().all(|(i, &ax)| ax == i) && axes[r - 2] == r - 1 && axes[r - 1] == r - 2
        };
        let mut bt = eb;
        let b = loop {
            if let Some(x) = self.find_in(bt, |nd| match nd { Node::Permute { x, axes } if swaps_last_two(axes) => Some(*x), _ => None }) { break x; }
            bt = self.reshape_of(bt)?;
        };
        let bs = self.const_shape(b)?;
        if bs.len() < 2 || bs[bs.len() - 2] != k || bs[bs.len() - 1] != n { return None; }
        // NT on a stored tensor: b is itself `w.t()` (Linear::forward hands W.t() to dot, which transposes it again)
        let (b, trans_b) = match self.find_in(b, |nd| match nd { Node::Permute { x, axes } if swaps_last_two(axes) => Some(*x), _ => None }) {
            Some(w) => (w, true),
            None => (b, false),
        };
        // TN on a stored tensor: a is `x.t()` of a [.., k, m] tensor (a weight gradient written as `x.t().dot(dz)`)
        let (a, trans_a) = match self.find_in(a, |nd| match nd { Node::Permute { x, axes } if swaps_last_two(axes) => Some(*x), _ => None }) {
            Some(x) if self.const_shape(x).is_some_and(|s| s.len() >= 2 && s[s.len() - 2] == k && s[s.len() - 1] == m) => (x, true),
            _ => (a, false),
        };
        let dt = self.dtype(b);
        if self.dtype(a) != dt || self.dtype(cid) != dt || !matches!(dt, DType::F32 | DType::BF16 | DType::F16 | DType::I32) { return None; }
        let mut mm = MatMulX { a: self.canon(a), b: self.canon(b), m, n, k, batch: batch_dims.iter().product(), trans_a, trans_b, b_shared, dtype: dt,
                               outer: 0, heads: 0, a_heads: false, b_heads: false, c_heads: false, a_view: Pitch::default(), b_view: Pitch::default() };
        // one right operand for every matrix of a dense batch (a Linear applied to [b, t, features]): the batch is just more rows
        if b_shared && !trans_a { (mm.m, mm.batch, mm.b_shared) = (mm.m * mm.batch, 1, false); }
        if batch_dims.len() == 2 && !b_shared {
            // q / k / v of attention, `x.reshape([b, t, h, d]).transpose(1, 2)` (multi_head_attention.rs:160-172) or the same of a
            // slice of a fused projection (`c_attn.forward(x).split([c, c, c], 2)`, causal_self_attention.rs:39-52): any operand that
            // is a view with unit step along its rows is read where it lies
            for (which, op) in [(0, a), (1, b)] {
                let Some((src, offset, st)) = self.affine_view(op) else { continue };
                if src == self.canon(op) || self.dtype(src) != dt || st[3] != 1 || st[2] <= 0 || st[0] < 0 || st[1] < 0 { continue; }
                if offset * (if matches!(dt, DType::F32 | DType::I32) { 4 } else { 2 }) % 256 != 0 { continue; }      // zyxb_buffer_view starts on 256-byte boundaries
                let pitch = Pitch { offset, ld: st[2] as u64, inner: st[1] as u64, outer: st[0] as u64 };
                if which == 0 { (mm.a, mm.a_heads, mm.a_view) = (src, true, pitch); } else { (mm.b, mm.b_heads, mm.b_view) = (src, true, pitch); }
            }
            if mm.a_heads || mm.b_heads { mm.outer = batch_dims[0]; mm.heads = batch_dims[1]; }
        }
        Some(mm)
    }
    fn match_matmul_scaled(&self, cid: ClassId) -> Option<(MatMulX, f32)> {
        if let Some(mm) = self.match_matmul_x(cid) { return Some((mm, 1.0)); }
        let (x, k) = self.binary_const(cid, BOp::Mul)?;
        Some((self.match_matmul_x(x)?, k as f32))
    }
    /// relu(e) = e.cmpgt(0) * e (tensor/elementwise.rs:289-293)
    fn relu_of(&self, c: ClassId) -> Option<ClassId> {
        let (x, y) = self.binary_of(c, BOp::Mul)?;
        for (mask, e) in [(x, y), (y, x)] {
            let mask = self.cast_src(mask).unwrap_or(mask);
            if let Some((l, r)) = self.binary_of(mask, BOp::Cmpgt) { if self.same(l, e) && self.const_value(r) == Some(0.0) { return Some(e); } }
        }
        None
    }
    /// tanh(u) = ((u+u).exp() - 1) / ((u+u).exp() + 1) (elementwise.rs:585-588)
    fn tanh_of(&self, c: ClassId) -> Option<ClassId> {
        let (num, den) = self.binary_of(c, BOp::Div)?;
        let (e1, one1) = self.binary_const(num, BOp::Sub)?;
        let (e2, one2) = self.binary_const(den, BOp::Add)?;
        if !self.same(e1, e2) || (one1 - 1.0).abs() > 1e-6 || (one2 - 1.0).abs() > 1e-6 { return None; }
        let (u1, u2) = self.binary_of(self.unary_of(e1, UOp::Exp)?, BOp::Add)?;
        self.same(u1, u2).then_some(u1)
    }
    /// gelu(z) = z * 0.5 * (tanh((z + z*z*z*0.044715) * sqrt(2/pi)) + 1) (elementwise.rs:168-170)
    fn gelu_of(&self, c: ClassId) -> Option<ClassId> {
        let (l, r) = self.binary_of(c, BOp::Mul)?;
        let (z, half) = self.binary_const(l, BOp::Mul)?;
        let (t, one) = self.binary_const(r, BOp::Add)?;
        if !near(half, 0.5) || !near(one, 1.0) { return None; }
        let (inner, c0) = self.binary_const(self.tanh_of(t)?, BOp::Mul)?;
        if !near(c0, 0.797_884_560_802_865_4) { return None; }
        let (z1, cube_term) = self.binary_of(inner, BOp::Add)?;
        let (cube, c1) = self.binary_const(cube_term, BOp::Mul)?;
        let (zz, z3) = self.binary_of(cube, BOp::Mul)?;
        let (za, zb) = self.binary_of(zz, BOp::Mul)?;
        (near(c1, 0.044_715) && [z1, z3, za, zb].iter().all(|&q| self.same(q, z))).then_some(z)
    }
    fn gemm_desc(mm: &MatMulX, epi: i32, preact: bool, alpha: f32) -> ZyxbGemmDesc {
        let mut g = ZyxbGemmDesc {
            dtype: mm.dtype as i32, m: mm.m, n: mm.n, k: mm.k, batch: mm.batch, trans_a: mm.trans_a as i32, trans_b: mm.trans_b as i32,
            stride_a: (mm.m * mm.k) as i64, stride_b: if mm.b_shared { 0 } else { (mm.k * mm.n) as i64 }, stride_c: (mm.m * mm.n) as i64,
            epilogue: epi, store_preact: preact as i32, alpha, ..Default::default()
        };
        if mm.heads != 0 {                                        // two-level batch: images outside, heads inside
            let h = mm.heads;
            // a stored [rows, cols] matrix per (image, head): inside a [b, t, h*d] tensor (pitch h*cols, heads `cols` apart) or packed
            let packed = |rows: Dim, cols: Dim| -> (u64, i64, i64) { (0, (h * rows * cols) as i64, (rows * cols) as i64) };
            let pitched = |p: Pitch| -> (u64, i64, i64) { (p.ld, p.outer as i64, p.inner as i64) };
            (g.batch, g.batch_inner) = (mm.outer, h);
            (g.lda, g.stride_a, g.stride_a_inner) = if mm.a_heads { pitched(mm.a_view) } else if mm.trans_a { packed(mm.k, mm.m) } else { packed(mm.m, mm.k) };
            (g.ldb, g.stride_b, g.stride_b_inner) = if mm.b_heads { pitched(mm.b_view) } else if mm.trans_b { packed(mm.n, mm.k) } else { packed(mm.k, mm.n) };
            // heads merged: the result lies in [b, t, h*d]
            (g.ldc, g.stride_c, g.stride_c_inner) = if mm.c_heads { (h * mm.n, (mm.m * h * mm.n) as i64, mm.n as i64) } else { packed(mm.m, mm.n) };
        }
        g
    }
    fn match_linear(&self, cid: ClassId, wanted: &BTreeSet<ClassId>) -> Option<B200Match> {
        // the heads merged back, `product.transpose(1, 2).reshape([b, t, h*d])` (multi_head_attention.rs:218-219): the product is
        // written where the merged tensor lies
        if let Some(p4) = self.reshape_of(cid).and_then(|r4| self.permute_of(r4, &[0, 2, 1, 3])) {
            if let (Some(s3), Some(s4)) = (self.const_shape(cid), self.const_shape(p4)) {
                if s3.len() == 3 && s4.len() == 4 && s3[0] == s4[0] && s3[1] == s4[2] && s3[2] == s4[1] * s4[3] {
                    if let Some((mut mm, alpha)) = self.match_matmul_scaled(p4).filter(|(mm, _)| !mm.b_shared && mm.dtype == self.dtype(cid)) {
                        (mm.c_heads, mm.outer, mm.heads) = (true, s4[0], s4[1]);
                        let gemm = Self::gemm_desc(&mm, EPI_NONE, false, alpha);
                        return Some(B200Match { pattern: "matmul", inputs: vec![mm.a, mm.b], outputs: vec![cid],
                                                desc: ZyxbKernelDesc { kind: ZYXB_KIND_GEMM, u: ZyxbDescUnion { gemm } }, numel: Vec::new(), optim_step: 0,
                                                input_offsets: vec![mm.a_view.offset, mm.b_view.offset] });
                    }
                }
            }
        }
        let (e, act) = if let Some(z) = self.gelu_of(cid) { (z, 2) } else if let Some(z) = self.relu_of(cid) { (z, 1) } else { (cid, 0) };
        let (mut core, mut bias) = (e, None);
        if let Some((x, y)) = self.binary_of(e, BOp::Add) {
            for (lhs, rhs) in [(x, y), (y, x)] {
                if bias.is_some() || self.expand_of(rhs).is_none() { continue; }
                let src = self.unbroadcast(rhs);
                let n = *self.const_shape(e)?.last()?;
                if self.const_shape(src).as_deref() == Some(&[n][..]) && self.match_matmul_scaled(lhs).is_some() { core = lhs; bias = Some(src); }
            }
        }
        if act != 0 && bias.is_none() { return None; }
        // + a whole tensor of the product's shape (a residual): Add{mm, r}, for a single packed matrix without bias
        let mut residual = None;
        if bias.is_none() {
            if let Some((x, y)) = self.binary_of(e, BOp::Add) {
                for (lhs, rhs) in [(x, y), (y, x)] {
                    if residual.is_some() || self.const_shape(rhs) != self.const_shape(e) || self.dtype(rhs) != self.dtype(e) { continue; }
                    if self.expand_of(rhs).is_some() || self.const_value(rhs).is_some() { continue; }
                    if self.match_matmul_scaled(lhs).is_some_and(|(mm, _)| mm.batch == 1 && mm.heads == 0) { core = lhs; residual = Some(self.canon(rhs)); }
                }
            }
        }
        let (mm, alpha) = self.match_matmul_scaled(core)?;
        if let Some(b) = bias { if self.dtype(b) != mm.dtype { return None; } }
        let epi = match (residual.is_some(), bias.is_some(), act) { (true, ..) => EPI_ADD, (_, false, _) => EPI_NONE, (_, true, 2) => EPI_BIAS_GELU, (_, true, 1) => EPI_BIAS_RELU, _ => EPI_BIAS };
        let preact = act == 2 && wanted.contains(&e);
        let gemm = Self::gemm_desc(&mm, epi, preact, alpha);
        let mut inputs = vec![mm.a, mm.b];
        inputs.extend(bias);
        inputs.extend(residual);
        let mut outputs = vec![cid];
        if preact { outputs.push(e); }
        Some(B200Match { pattern: "matmul", inputs, outputs, desc: ZyxbKernelDesc { kind: ZYXB_KIND_GEMM, u: ZyxbDescUnion { gemm } }, numel: Vec::new(), optim_step: 0,
                         input_offsets: vec![mm.a_view.offset, mm.b_view.offset] })      // (bias and residual start at 0: missing entries read as 0)
    }

    // ---- row kernels ---------------------------------------------------------------------------------------------------------
    fn row_desc(&self, op: i32, x: ClassId) -> Option<ZyxbRowreduceDesc> {
        let s = self.const_shape(x)?;
        let cols = *s.last()?;
        let exact_int = self.dtype(x) == DType::I32 && matches!(op, RR_SUM | RR_MAX | RR_MIN);       // i32 sum / max / min are exact programs
        (matches!(self.dtype(x), DType::F32 | DType::BF16 | DType::F16) || exact_int)
            .then(|| ZyxbRowreduceDesc { op, dtype: self.dtype(x) as i32, rows: s.iter().product::<Dim>() / cols, cols, correction: 1, ..Default::default() })
    }
    fn row_match(&self, pattern: &'static str, rowreduce: ZyxbRowreduceDesc, inputs: Vec<ClassId>, out: ClassId) -> B200Match {
        B200Match { pattern, inputs, outputs: vec![out], desc: ZyxbKernelDesc { kind: ZYXB_KIND_ROWREDUCE, u: ZyxbDescUnion { rowreduce } }, numel: Vec::new(), optim_step: 0, input_offsets: Vec::new() }
    }
    fn keepdim_src(&self, c: ClassId) -> ClassId { self.expand_of(c).unwrap_or(c) }
    /// c = uop(x - Expand{max_keepdim(x)}) -> x
    fn shifted(&self, c: ClassId, uop: Option<UOp>) -> Option<ClassId> {
        let d = match uop { Some(u) => self.unary_of(c, u)?, None => c };
        let (x, mx) = self.binary_of(d, BOp::Sub)?;
        let src = self.reduce_last(self.keepdim_src(mx), BOp::Max)?;
        self.same(src, x).then(|| self.canon(x))
    }
    // ---- fused attention ----------------------------------------------------------------------------------------------------
    fn permute_of(&self, c: ClassId, want: &[usize]) -> Option<ClassId> {
        self.find_in(c, |n| match n { Node::Permute { x, axes } if axes.as_ref() == want => Some(*x), _ => None })
    }
    /// The mask-free core of MultiheadAttention::forward (multi_head_attention.rs:197-226) ending at the class of
    /// `attn_weights.matmul(v).transpose(1, 2).reshape([b, t, h*d])`: one fused program on the three stored [b, t, h*d] tensors.
    /// The kernel's shapes only (16-bit dtype, head dimension 128, equal lengths that are a multiple of 128).  A causal mask
    /// (`masked_fill(ones.tril(0).equal(0), -inf)`) is not matched: `where_` computes in the dtype of the rank-0 fill value, so 16-bit
    /// scores come out as f32 (NaN where the mask keeps them, 0 * -inf); such graphs fall back to the separate programs.
    fn match_attention(&self, cid: ClassId) -> Option<B200Match> {
        let s3 = self.const_shape(cid)?;
        if s3.len() != 3 { return None; }
        let pv_cls = self.permute_of(self.reshape_of(cid)?, &[0, 2, 1, 3])?;
        let pv = self.match_matmul_x(pv_cls)?;
        if pv.trans_a || pv.trans_b || pv.b_shared { return None; }
        let sm = self.match_softmax(pv.a)?;
        let (qk, scale) = self.match_matmul_scaled(sm.inputs[0])?;
        if qk.trans_a || !qk.trans_b || qk.b_shared { return None; }
        if !qk.a_heads || !qk.b_heads || !pv.b_heads || pv.a_heads { return None; }          // q, k, v: per-head views of stored tensors
        let (xq, xk, xv) = (qk.a, qk.b, pv.b);
        let hs = self.const_shape(pv_cls)?;
        let (b, h, t, d) = (hs[0], hs[1], hs[2], hs[3]);
        // the program reads q, k, v and writes the result with one row pitch: whole [b, t, h*d] tensors, not slices of a wider one
        let whole = |p: Pitch, t: Dim, h: Dim, d: Dim| p.offset == 0 && p.ld == h * d && (h == 1 || p.inner == d) && (b == 1 || p.outer == t * h * d);   // (a single image or head is never stepped over)
        let shapes_ok = qk.m == t && qk.n == t && qk.k == d && pv.m == t && pv.k == t && pv.n == d && qk.batch == b * h && pv.batch == b * h
            && s3[0] == b && s3[1] == t && s3[2] == h * d;
        let dt = qk.dtype;
        if !shapes_ok || !matches!(dt, DType::BF16 | DType::F16) || pv.dtype != dt || d != 128 || t % 128 != 0 { return None; }
        if ![qk.a_view, qk.b_view, pv.b_view].into_iter().all(|p| whole(p, t, h, d)) { return None; }
        let attention = ZyxbAttentionDesc { dtype: dt as i32, batch: b as u64, heads: h as u64, seq: t as u64, head_dim: d as u64, ld: 0, scale, causal: 0 };
        // the launch takes one more buffer behind the output: the log-sum-exp [b*h, t] f32 the backward program reads
        Some(B200Match { pattern: "attention", inputs: vec![xq, xk, xv], outputs: vec![cid],
                         desc: ZyxbKernelDesc { kind: ZYXB_KIND_ATTENTION, u: ZyxbDescUnion { attention } }, numel: Vec::new(), optim_step: 0, input_offsets: Vec::new() })
    }

    /// softmax (tensor/mod.rs:1457-1461)
    fn match_softmax(&self, cid: ClassId) -> Option<B200Match> {
        let (e, s) = self.binary_of(cid, BOp::Div)?;
        if self.expand_of(s).is_none() && self.const_shape(cid)?.last() != Some(&1) { return None; }      // (one column: nothing to expand)
        if !self.same(self.reduce_last(self.keepdim_src(s), BOp::Add)?, e) { return None; }
        let x = self.shifted(e, Some(UOp::Exp))?;
        Some(self.row_match("softmax", self.row_desc(RR_SOFTMAX, x)?, vec![x], cid))
    }
    /// ln_softmax (tensor/mod.rs:1427-1431)
    fn match_ln_softmax(&self, cid: ClassId) -> Option<B200Match> {
        let (m, l) = self.binary_of(cid, BOp::Sub)?;
        if self.expand_of(l).is_none() && self.const_shape(cid)?.last() != Some(&1) { return None; }
        let e = self.reduce_last(self.unary_of(self.keepdim_src(l), UOp::Ln)?, BOp::Add)?;
        if !self.same(self.unary_of(e, UOp::Exp)?, m) { return None; }
        let x = self.shifted(m, None)?;
        Some(self.row_match("ln_softmax", self.row_desc(RR_LN_SOFTMAX, x)?, vec![x], cid))
    }
    /// mean over the last axis: sum / const(n) (reduce_ops.rs:104-112) -> (x, n)
    fn mean_last(&self, c: ClassId) -> Option<(ClassId, f64)> {
        let d = match self.reshape_of(c) { Some(r) if self.numel_of(r) == self.numel_of(c) => r, _ => c };
        let (s, n) = self.binary_const(d, BOp::Div)?;
        Some((self.reduce_last(s, BOp::Add)?, n))
    }
    /// LayerNorm::forward (zyx-nn/src/layer_norm.rs:117-131)
    fn match_layernorm(&self, cid: ClassId) -> Option<B200Match> {
        let cols = *self.const_shape(cid)?.last()?;
        let (mut c, mut weight, mut bias) = (cid, None, None);
        for (op, slot) in [(BOp::Add, &mut bias), (BOp::Mul, &mut weight)] {
            if let Some((x, p)) = self.binary_of(c, op) {
                // (a rank-1 input meets its parameters unexpanded)
                let rank1 = self.const_shape(cid)?.len() == 1;
                let src = if self.expand_of(p).is_some() { self.unbroadcast(p) } else { self.canon(p) };
                if (self.expand_of(p).is_some() || rank1) && self.const_shape(src).as_deref() == Some(&[cols][..]) && self.const_value(src).is_none() { *slot = Some(src); c = x; }
            }
        }
        let (centred, denom) = self.binary_of(c, BOp::Div)?;
        let (x, mean) = self.binary_of(centred, BOp::Sub)?;
        let x = self.canon(x);
        if !self.same(self.mean_last(self.keepdim_src(mean))?.0, x) { return None; }
        let (var, eps) = self.binary_const(self.unary_of(self.keepdim_src(denom), UOp::Sqrt)?, BOp::Add)?;
        let (sq, d) = self.mean_last(var)?;
        let (l, r) = self.binary_of(sq, BOp::Mul)?;
        if !self.same(l, r) || !self.same(l, centred) { return None; }
        let mut desc = self.row_desc(RR_LAYERNORM, x)?;
        desc.eps = eps as f32;
        desc.correction = if near(d, cols as f64 - 1.0) { 1 } else { (cols as f64 - d).round() as i32 };
        desc.has_weight = weight.is_some() as i32;
        desc.has_bias = bias.is_some() as i32;
        Some(self.row_match("layernorm", desc, [Some(x), weight, bias].into_iter().flatten().collect(), cid))
    }
    fn is_broadcast_product(&self, c: ClassId) -> bool {
        let c = self.cast_src(c).unwrap_or(c);
        matches!(self.binary_of(c, BOp::Mul), Some((x, y)) if self.expand_of(x).is_some() && self.expand_of(y).is_some())
    }
    /// mse_loss(y, t) = ((y - t) * (y - t)).mean_all() (tensor/mod.rs:1999-2003); f32 only: the program leaves an f32 scalar
    fn match_mse(&self, cid: ClassId) -> Option<B200Match> {
        let (sum, n) = self.binary_const(cid, BOp::Div)?;
        let (x, axes) = self.find_in(sum, |nd| match nd { Node::Reduce { x, rop: BOp::Add, axes } => Some((*x, axes.clone())), _ => None })?;
        let xs = self.const_shape(x)?;
        if xs.is_empty() || axes.len() != xs.len() || (n - xs.iter().product::<Dim>() as f64).abs() > 0.5 { return None; }
        let (d0, d1) = self.binary_of(x, BOp::Mul)?;
        if !self.same(d0, d1) { return None; }
        let (y, t) = self.binary_of(d0, BOp::Sub)?;
        let (y, t) = (self.canon(y), self.canon(t));
        if self.expand_of(y).is_some() || self.expand_of(t).is_some() { return None; }      // whole tensors: x - mean(x) over a rank-1 x is the variance's business
        let f32s = [y, t, cid].iter().all(|&c| self.dtype(c) == DType::F32);
        if !f32s || self.const_shape(y)? != xs || self.const_shape(t)? != xs { return None; }
        Some(self.row_match("mse_loss", self.row_desc(RR_MSE, y)?, vec![y, t], cid))
    }
    // ---- elementwise programs ------------------------------------------------------------------------------------------------
    /// What is left when no larger pattern ends at a class: one elementwise program over stored operands
    /// (tensor/elementwise.rs).  Operands are whole tensors of the result's shape - a broadcast operand is either a scalar
    /// constant (scale) or a vector along the last axis (bias).  16-bit and f32 floats only (what the kernels take).
    fn match_eltwise(&self, cid: ClassId) -> Option<B200Match> {
        let is_row = |d: DType| matches!(d, DType::F32 | DType::BF16 | DType::F16);
        let (dt, cs) = (self.dtype(cid), self.const_shape(cid)?);
        let n: Dim = cs.iter().product();
        if !is_row(dt) || cs.is_empty() || n == 0 { return None; }
        let plain = |x: ClassId| self.expand_of(x).is_none() && self.const_value(x).is_none() && self.const_shape(x).as_ref() == Some(&cs);
        let whole = |x: ClassId| plain(x) && self.dtype(x) == dt;
        let program = |pattern: &'static str, op: i32, inputs: Vec<ClassId>, p0: f32, cols: Dim, dt_in: DType| {
            let eltwise = ZyxbEltwiseDesc { op, dtype: dt_in as i32, dtype_out: dt as i32, numel: n, cols, p0 };
            Some(B200Match { pattern, inputs: inputs.into_iter().map(|c| self.canon(c)).collect(), outputs: vec![cid],
                             desc: ZyxbKernelDesc { kind: ZYXB_KIND_ELTWISE, u: ZyxbDescUnion { eltwise } }, numel: Vec::new(), optim_step: 0, input_offsets: Vec::new() })
        };
        if let Some(z) = self.gelu_of(cid).filter(|&z| whole(z)) { return program("gelu", EW_GELU, vec![z], 0.0, 0, dt); }
        if let Some(z) = self.relu_of(cid).filter(|&z| whole(z)) { return program("relu", EW_RELU, vec![z], 0.0, 0, dt); }
        if let Some(u) = self.tanh_of(cid).filter(|&u| whole(u)) { return program("tanh", EW_TANH, vec![u], 0.0, 0, dt); }
        // sigmoid(x) = e / (e + 1), e = exp(x)   (elementwise.rs:457-460)
        if let Some((e, den)) = self.binary_of(cid, BOp::Div) {
            if let Some((e2, one)) = self.binary_const(den, BOp::Add) {
                if self.same(e, e2) && (one - 1.0).abs() <= 1e-6 {
                    if let Some(x) = self.unary_of(e, UOp::Exp).filter(|&x| whole(x)) { return program("sigmoid", EW_SIGMOID, vec![x], 0.0, 0, dt); }
                }
            }
        }
        if let Some(x) = self.unary_of(cid, UOp::Exp).filter(|&x| whole(x)) { return program("exp", EW_EXP, vec![x], 0.0, 0, dt); }
        if let Some(x) = self.unary_of(cid, UOp::Neg).filter(|&x| whole(x)) { return program("scale", EW_SCALE, vec![x], -1.0, 0, dt); }      // -x = x * -1, exactly
        if let Some(x) = self.cast_src(cid).filter(|&x| is_row(self.dtype(x)) && plain(x)) { return program("cast", EW_CAST, vec![x], 0.0, 0, self.dtype(x)); }
        if let Some((x, k)) = self.binary_const(cid, BOp::Mul).filter(|&(x, _)| whole(x)) { return program("scale", EW_SCALE, vec![x], k as f32, 0, dt); }
        // x / const as x * (1 / const): what the reference's own C backend computes under -ffast-math (reciprocal math); dropout
        // outside training is such a division (x / (1 - p), tensor/mod.rs:822-828)
        if let Some((x, k)) = self.binary_const(cid, BOp::Div).filter(|&(x, k)| whole(x) && k != 0.0) { return program("scale", EW_SCALE, vec![x], (1.0 / k) as f32, 0, dt); }
        for (bop, ew, name) in [(BOp::Add, EW_ADD, "add"), (BOp::Sub, EW_SUB, "sub"), (BOp::Mul, EW_MUL, "mul")] {
            if let Some((x, y)) = self.binary_of(cid, bop).filter(|&(x, y)| whole(x) && whole(y)) { return program(name, ew, vec![x, y], 0.0, 0, dt); }
        }
        let (p, q) = self.binary_of(cid, BOp::Add)?;                          // x + bias along the last axis
        for (x, be) in [(p, q), (q, p)] {
            if !whole(x) || self.expand_of(be).is_none() || self.const_value(be).is_some() { continue; }
            let b = self.canon(self.unbroadcast(be));
            let cols = *cs.last()?;
            if self.const_shape(b).as_deref() == Some(&[cols][..]) && self.dtype(b) == dt && self.trailing_vector(be) {
                return program("bias_add", EW_BIAS_ADD, vec![x, b], 0.0, cols, dt);
            }
        }
        None
    }
    /// c = Expand{[Reshape]{v [n]}} with v laid along the LAST axis of c (every wrapper keeps all but the last extent at 1)
    fn trailing_vector(&self, c: ClassId) -> bool {
        let Some(mut s) = self.expand_of(c) else { return false };
        loop {
            let Some(sh) = self.const_shape(s) else { return false };
            if sh.is_empty() || sh[..sh.len() - 1].iter().any(|&d| d != 1) { return false; }
            match self.reshape_of(s) { Some(r) => s = r, None => return true }
        }
    }

    // ---- constant folding ---------------------------------------------------------------------------------------------------
    /// The value of a class that depends on no stored tensor: constants under movement ops, paddings, reductions, casts and
    /// arithmetic, the way the index helpers build them (Tensor::arange is `full(step).cumsum(0) + start - step`,
    /// tensor/mod.rs:773-781; a cumsum is a padded, pooled sum, reduce_ops.rs:1076-1091).  Row-major, as f64 (exact for index
    /// arithmetic).  None when a Leaf is reached, an op is not covered, a dim is symbolic or an intermediate has more than 2^22
    /// elements.
    fn const_eval(&self, c: ClassId) -> Option<Vec<f64>> {
        self.eval_class(c, 1 << 22, &mut BTreeMap::new(), 0)
    }
    fn eval_class(&self, c: ClassId, limit: u64, memo: &mut BTreeMap<ClassId, Option<Vec<f64>>>, depth: u32) -> Option<Vec<f64>> {
        if let Some(v) = memo.get(&c) { return v.clone(); }
        let v = self.eval_node(c, limit, memo, depth);
        memo.insert(c, v.clone());
        v
    }
    fn eval_node(&self, c: ClassId, limit: u64, memo: &mut BTreeMap<ClassId, Option<Vec<f64>>>, depth: u32) -> Option<Vec<f64>> {
        fn unravel(mut i: u64, shape: &[Dim], idx: &mut [u64]) { for a in (0..shape.len()).rev() { idx[a] = i % shape[a]; i /= shape[a]; } }
        fn strides(shape: &[Dim]) -> Vec<u64> { let mut st = vec![1; shape.len()]; for a in (1..shape.len()).rev() { st[a - 1] = st[a] * shape[a]; } st }
        if depth > 256 { return None; }
        let os = self.const_shape(c)?;
        let on: u64 = os.iter().product();
        if on > limit { return None; }
        let mut idx = vec![0u64; 16];
        match &self.nodes[self.classes[c].nodes[0]].node {
            Node::Const(k) => Some(vec![const_f64(*k)]),
            Node::Reshape { x, .. } => self.eval_class(*x, limit, memo, depth + 1),
            Node::Expand { x, .. } => {
                let (xv, xs) = (self.eval_class(*x, limit, memo, depth + 1)?, self.const_shape(*x)?);
                let (st, lead) = (strides(&xs), os.len() - xs.len());
                Some((0..on).map(|o| {
                    unravel(o, &os, &mut idx);
                    xv[(0..xs.len()).filter(|&a| xs[a] != 1).map(|a| idx[lead + a] * st[a]).sum::<u64>() as usize]
                }).collect())
            }
            Node::Permute { x, axes } => {
                let (xv, st) = (self.eval_class(*x, limit, memo, depth + 1)?, strides(&self.const_shape(*x)?));
                Some((0..on).map(|o| {
                    unravel(o, &os, &mut idx);
                    xv[axes.iter().enumerate().map(|(j, &a)| idx[j] * st[a as usize]).sum::<u64>() as usize]
                }).collect())
            }
            Node::Pad { x, axis, lp, .. } => {
                let (xv, xs) = (self.eval_class(*x, limit, memo, depth + 1)?, self.const_shape(*x)?);
                let lp = self.find_in(*lp, |n| match n { Node::Const(k) => Some(const_f64(*k) as i64), _ => None })?;
                let (st, ax) = (strides(&xs), *axis as usize);
                Some((0..on).map(|o| {
                    unravel(o, &os, &mut idx);
                    let at = idx[ax] as i64 - lp;
                    if at < 0 || at >= xs[ax] as i64 { return 0.0; }                  // a zero of the padding
                    xv[(0..xs.len()).map(|a| (if a == ax { at as u64 } else { idx[a] }) * st[a]).sum::<u64>() as usize]
                }).collect())
            }
            Node::Reduce { x, rop, axes } => {
                let (xv, xs) = (self.eval_class(*x, limit, memo, depth + 1)?, self.const_shape(*x)?);
                let init = match rop { BOp::Add => 0.0, BOp::Mul => 1.0, BOp::Max => f64::NEG_INFINITY, _ => return None };
                let mut out = vec![init; on as usize];
                for (i, &v) in xv.iter().enumerate() {
                    unravel(i as u64, &xs, &mut idx);
                    let o = (0..xs.len()).filter(|a| !axes.contains(&(*a as _))).fold(0, |o, a| o * xs[a] + idx[a]) as usize;
                    out[o] = match rop { BOp::Add => out[o] + v, BOp::Mul => out[o] * v, _ => out[o].max(v) };
                }
                Some(out)
            }
            Node::Cast { x, dtype } => Some(self.eval_class(*x, limit, memo, depth + 1)?.into_iter().map(|v| cast_value(v, *dtype)).collect()),
            Node::Unary { x, uop } => self.eval_class(*x, limit, memo, depth + 1)?.into_iter().map(|v| Some(match uop {
                UOp::Neg => -v, UOp::Abs => v.abs(), UOp::Floor => v.floor(), UOp::Trunc => v.trunc(), UOp::Exp => v.exp(), UOp::Ln => v.ln(),
                UOp::Sqrt => v.sqrt(), UOp::Reciprocal => 1.0 / v, _ => return None,
            })).collect(),
            Node::Binary { x, y, bop } => {
                let (xv, yv) = (self.eval_class(*x, limit, memo, depth + 1)?, self.eval_class(*y, limit, memo, depth + 1)?);
                if xv.len() != yv.len() || xv.len() as u64 != on { return None; }
                let whole = !self.dtype(*x).is_float();
                xv.into_iter().zip(yv).map(|(a, b)| Some(match bop {
                    BOp::Add => a + b, BOp::Sub => a - b, BOp::Mul => a * b, BOp::Max => a.max(b),
                    BOp::Div => { if whole && b == 0.0 { return None; } if whole { (a / b).trunc() } else { a / b } }
                    BOp::Mod => { if b == 0.0 { return None; } a % b }
                    BOp::Cmplt => (a < b) as u8 as f64, BOp::Cmpgt => (a > b) as u8 as f64, BOp::Cmpge => (a >= b) as u8 as f64,
                    BOp::NotEq => (a != b) as u8 as f64, BOp::Eq => (a == b) as u8 as f64,
                    _ => return None,
                })).collect()
            }
            _ => None,
        }
    }

    // ---- views: where an element comes from ---------------------------------------------------------------------------------
    /// One element of class c followed back through the movement ops that define it (Expand, Reshape, Permute, Pad, no-op Cast)
    /// to the first class that is something else: (that class, the coordinates there), or None when the element is a zero of some
    /// padding.  A view is recognised by what it reads, not by how it was written down: Tensor::pool (tensor/mod.rs:2442-2543) is a
    /// dozen reshapes, expands and crops that differ with every stride and dilation, but what they read is `oy*stride + r*dilation`.
    fn trace_element(&self, mut c: ClassId, mut idx: Vec<u64>) -> Option<Option<(ClassId, Vec<u64>)>> {
        for _ in 0..256 {
            let cs = self.const_shape(c)?;
            match &self.nodes[self.classes[c].nodes[0]].node {
                Node::Reshape { x, .. } => {
                    let xs = self.const_shape(*x)?;
                    let mut lin = cs.iter().zip(&idx).fold(0, |l, (&d, &i)| l * d + i);
                    idx = vec![0; xs.len()];
                    for a in (0..xs.len()).rev() { idx[a] = lin % xs[a]; lin /= xs[a]; }
                    c = *x;
                }
                Node::Expand { x, .. } => {
                    let xs = self.const_shape(*x)?;
                    let lead = cs.len() - xs.len();
                    idx = (0..xs.len()).map(|a| if xs[a] == 1 { 0 } else { idx[lead + a] }).collect();
                    c = *x;
                }
                Node::Permute { x, axes } => {
                    let mut src = vec![0; idx.len()];
                    for (j, &a) in axes.iter().enumerate() { src[a as usize] = idx[j]; }
                    idx = src;
                    c = *x;
                }
                Node::Pad { x, axis, lp, .. } => {
                    let lp = self.find_in(*lp, |n| match n { Node::Const(k) => Some(const_f64(*k) as i64), _ => None })?;
                    let at = idx[*axis as usize] as i64 - lp;
                    if at < 0 || at >= self.const_shape(*x)?[*axis as usize] as i64 { return Some(None); }
                    idx[*axis as usize] = at as u64;
                    c = *x;
                }
                Node::Cast { x, dtype } if self.dtype(*x) == *dtype => c = *x,
                _ => break,
            }
        }
        Some(Some((c, idx)))
    }
    /// c as a strided window of a stored tensor: element idx of c is element `offset + sum(idx[a] * strides[a])` of `src`, row-major
    /// -> (src, offset, strides).  Measured, not derived: the origin and one step along every axis give offset and strides, then
    /// every corner and a spread of other elements must agree (a reshape of a permuted tensor is no such window and fails at its
    /// far corner).  None when some element is padding or the elements come from more than one class.
    fn affine_view(&self, c: ClassId) -> Option<(ClassId, u64, Vec<i64>)> {
        let cs = self.const_shape(c)?;
        let rank = cs.len();
        if rank == 0 || rank > 6 || cs.iter().product::<Dim>() == 0 { return None; }
        let lin_of = |cls: ClassId, idx: &[u64]| -> Option<i64> { Some(self.const_shape(cls)?.iter().zip(idx).fold(0i64, |l, (&d, &i)| l * d as i64 + i as i64)) };
        let (c0, i0) = self.trace_element(c, vec![0; rank])??;
        let (src, offset) = (self.canon(c0), lin_of(c0, &i0)?);
        let at = |idx: &[u64]| -> Option<i64> {
            let (cls, i) = self.trace_element(c, idx.to_vec())??;
            if self.canon(cls) != src { return None; }
            lin_of(cls, &i)
        };
        let mut strides = vec![0i64; rank];
        let mut idx = vec![0u64; rank];
        for a in 0..rank {
            if cs[a] < 2 { continue; }
            idx[a] = 1;
            strides[a] = at(&idx)? - offset;
            idx[a] = 0;
        }
        let agrees = |idx: &[u64]| at(idx) == Some(offset + idx.iter().zip(&strides).map(|(&i, &s)| i as i64 * s).sum::<i64>());
        for corner in 0..1u64 << rank {
            for a in 0..rank { idx[a] = if corner >> a & 1 == 1 { cs[a] - 1 } else { 0 }; }
            if !agrees(&idx) { return None; }
        }
        let mut seed = 0x9e37_79b9_7f4a_7c15u64;                              // a fixed spread of interior elements
        for _ in 0..256 {
            for a in 0..rank { seed = seed.wrapping_mul(6364136223846793005).wrapping_add(1442695040888963407); idx[a] = (seed >> 33) % cs[a]; }
            if !agrees(&idx) { return None; }
        }
        Some((src, offset as u64, strides))
    }
    /// the class a view reads (c under every movement op) and the classes passed on the way, outermost first
    fn view_source(&self, mut c: ClassId) -> (ClassId, Vec<ClassId>) {
        let mut chain = Vec::new();
        for _ in 0..256 {
            let x = match &self.nodes[self.classes[c].nodes[0]].node {
                Node::Reshape { x, .. } | Node::Expand { x, .. } | Node::Permute { x, .. } | Node::Pad { x, .. } => *x,
                Node::Cast { x, dtype } if self.dtype(*x) == *dtype => *x,
                _ => break,
            };
            chain.push(c);
            c = x;
        }
        (c, chain)
    }

    // ---- convolution ----------------------------------------------------------------------------------------------------------
    /// Tensor::conv with groups = 1 on [n, c, h, w] (tensor/mod.rs:2583-2680), ending at cid [n, o, oh, ow]:
    ///   x.rpad_zeros(padding).pool(kernel, stride, dilation) -Reshape, Expand over o, Permute-> [n, 1, o, oh, ow, c, kh, kw]
    ///   * weight.reshape([1, 1, o, 1, 1, c, kh, kw]) -> sum_keepdim over (c, kh, kw) -> reshape [n, o, oh, ow]  [+ bias.reshape([1, o, 1, 1])]
    /// Padding from the Pad nodes on the stored input, stride and dilation measured on the view, then the view held against
    /// `x[b, ci, oy*stride_h + r*dil_h - pad_top, ox*stride_w + s*dil_w - pad_left]` (zero outside the image).
    fn match_conv(&self, cid: ClassId) -> Option<B200Match> {
        let out = self.const_shape(cid)?;
        if out.len() != 4 { return None; }
        let (mut e, mut bias) = (cid, None);
        if let Some((p, q)) = self.binary_of(cid, BOp::Add) {
            for (lhs, rhs) in [(p, q), (q, p)] {
                if bias.is_some() { break; }
                let Some(src) = self.expand_of(rhs) else { continue };
                if self.const_shape(src).as_deref() != Some(&[1, out[1], 1, 1][..]) { continue; }
                let b = self.canon(self.unbroadcast(rhs));
                if self.numel_of(b) == Some(out[1]) { bias = Some(b); e = lhs; }
            }
        }
        // through the closing reshape and sum_keepdim's reshape to the Reduce
        let red_of = |cls: ClassId| self.find_in(cls, |nd| match nd { Node::Reduce { x, rop: BOp::Add, axes } => Some((*x, axes.clone())), _ => None });
        let (mut r, mut red) = (e, None);
        for _ in 0..4 {
            red = red_of(r).or_else(|| red_of(self.cast_src(r)?));
            if red.is_some() { break; }
            let src = self.reshape_of(r)?;
            if self.numel_of(src) != Some(out.iter().product()) { return None; }
            r = src;
        }
        let (prod, axes) = red?;
        let ps = self.const_shape(prod)?;                                    // [n, 1, o, oh, ow, c, kh, kw]
        let mut axes: Vec<usize> = axes.iter().map(|&a| a as usize).collect();
        axes.sort_unstable();
        if ps.len() != 8 || axes != [5, 6, 7] || ps[1] != 1 { return None; }
        let (n, o, oh, ow, c, kh, kw) = (ps[0], ps[2], ps[3], ps[4], ps[5], ps[6], ps[7]);
        if out != [n, o, oh, ow] { return None; }
        let (f0, f1) = self.binary_of(prod, BOp::Mul).or_else(|| self.binary_of(self.cast_src(prod)?, BOp::Mul))?;
        for (xe, we) in [(f0, f1), (f1, f0)] {
            let Some(wr) = self.expand_of(we) else { continue };
            if self.const_shape(wr).as_deref() != Some(&[1, 1, o, 1, 1, c, kh, kw][..]) { continue; }
            let Some(wsrc) = self.reshape_of(wr) else { continue };
            if self.const_shape(wsrc).as_deref() != Some(&[o, c, kh, kw][..]) { continue; }
            let w = self.canon(wsrc);
            let (x, chain) = self.view_source(xe);
            let Some(xs) = self.const_shape(x) else { continue };
            if self.const_shape(xe)? != ps || xs.len() != 4 || xs[0] != n || xs[1] != c { continue; }
            let dt = self.dtype(x);
            if self.dtype(w) != dt || self.dtype(cid) != dt || bias.is_some_and(|b| self.dtype(b) != dt) { continue; }
            if !matches!(dt, DType::F32 | DType::BF16 | DType::F16 | DType::I32) { continue; }
            let (h, wd) = (xs[2], xs[3]);
            // the declared padding: the Pad nodes directly on x (rpad_zeros pads the last axis first)
            let mut pad = [0u64; 4];                                          // top, bottom, left, right
            let mut ext = [n, c, h, wd];
            for &cls in chain.iter().rev() {
                let Node::Pad { axis, lp, len, .. } = &self.nodes[self.classes[cls].nodes[0]].node else { break };
                let ax = *axis as usize;
                let (Some(lp), Some(len)) = (self.find_in(*lp, |k| match k { Node::Const(k) => Some(const_f64(*k) as i64), _ => None }),
                                             self.find_in(*len, |k| match k { Node::Const(k) => k.as_dim(), _ => None })) else { break };
                if lp < 0 || (ax != 2 && ax != 3) || (len as i64) < lp + ext[ax] as i64 { break; }
                pad[if ax == 2 { 0 } else { 2 }] += lp as u64;
                pad[if ax == 2 { 1 } else { 3 }] += len - lp as u64 - ext[ax];
                ext[ax] = len;
            }
            let probe = |b: u64, co: u64, oy: u64, ox: u64, ci: u64, kr: u64, ks: u64| self.trace_element(xe, vec![b, 0, co, oy, ox, ci, kr, ks]);
            // Stride and dilation, measured: along an axis a window o and tap t read coordinate o*stride + t*dilation - pad when that
            // is inside the image and padding otherwise.  Every (window, tap) pair of the axis is probed (at a window and tap of the
            // OTHER axis that are themselves inside the image); two windows under one tap give the stride, two taps under one window
            // the dilation.  Where padding leaves too few probes inside the image for that (an image smaller than its padding), any
            // pair that explains all probes - inside and outside - and the output extent describes the same convolution: the first one
            // found is taken.
            let solve_axis = |rows: bool| -> Option<(u64, u64)> {
                let (n_out, n_tap, extent, n_other, n_other_tap) = if rows { (oh as i64, kh as i64, h as i64, ow, kw) } else { (ow as i64, kw as i64, wd as i64, oh, kh) };
                let (before, total) = if rows { (pad[0] as i64, (h + pad[0] + pad[1]) as i64) } else { (pad[2] as i64, (wd + pad[2] + pad[3]) as i64) };
                let mut probes: Vec<(i64, i64, i64)> = Vec::new();                    // (window, tap, coordinate read; -1: padding)
                'off_axis: for other in sample_axis(n_other) {
                    for tap in 0..n_other_tap {
                        probes.clear();
                        for o in sample_axis(n_out as u64) {
                            for t in 0..n_tap as u64 {
                                let a = if rows { probe(0, 0, o, other, 0, t, tap)? } else { probe(0, 0, other, o, 0, tap, t)? };
                                probes.push((o as i64, t as i64, match a { Some((cls, idx)) if cls == x => idx[if rows { 2 } else { 3 }] as i64, _ => -1 }));
                            }
                        }
                        if probes.iter().any(|p| p.2 >= 0) { break 'off_axis; }
                    }
                }
                if !probes.iter().any(|p| p.2 >= 0) { return None; }                  // nothing of the image is ever read
                let explains = |s: i64, d: i64| {
                    s > 0 && d > 0 && total >= d * (n_tap - 1) + 1 && (total - (d * (n_tap - 1) + 1)) / s + 1 == n_out
                        && probes.iter().all(|&(o, t, r)| { let at = o * s + t * d - before; if r >= 0 { at == r } else { at < 0 || at >= extent } })
                };
                let (mut s, mut d) = (0i64, if n_tap == 1 { 1 } else { 0 });         // 0: not known yet; a single tap never takes its dilation
                for &(ao, at, ar) in &probes {
                    for &(bo, bt, br) in &probes {
                        if ar < 0 || br < 0 { continue; }
                        if s == 0 && at == bt && bo > ao && (br - ar) % (bo - ao) == 0 { s = (br - ar) / (bo - ao); }
                        if d == 0 && ao == bo && bt > at && (br - ar) % (bt - at) == 0 { d = (br - ar) / (bt - at); }
                    }
                }
                if s != 0 && d != 0 && explains(s, d) { return Some((s as u64, d as u64)); }
                let range = |known: i64| if known != 0 { known..=known } else { 1..=total + 1 };      // what is measured stays; the rest is searched
                range(s).flat_map(|sc| range(d).map(move |dc| (sc, dc))).find(|&(sc, dc)| explains(sc, dc)).map(|(sc, dc)| (sc as u64, dc as u64))
            };
            let (Some((sh, dh)), Some((sw, dw))) = (solve_axis(true), solve_axis(false)) else { continue };
            // the output extent the declared padding gives must be the view's
            let out_extent = |i: u64, before: u64, after: u64, k: u64, s: u64, d: u64| {
                let (span, padded) = (d * (k - 1) + 1, i + before + after);
                if padded < span { 0 } else { (padded - span) / s + 1 }
            };
            if out_extent(h, pad[0], pad[1], kh, sh, dh) != oh || out_extent(wd, pad[2], pad[3], kw, sw, dw) != ow { continue; }
            let reads = |b: u64, co: u64, oy: u64, ox: u64, ci: u64, kr: u64, ks: u64| -> bool {
                let Some(origin) = probe(b, co, oy, ox, ci, kr, ks) else { return false };
                let (row, col) = ((oy * sh + kr * dh) as i64 - pad[0] as i64, (ox * sw + ks * dw) as i64 - pad[2] as i64);
                if row < 0 || row >= h as i64 || col < 0 || col >= wd as i64 { return origin.is_none(); }
                origin == Some((x, vec![b, ci, row as u64, col as u64]))
            };
            let (oys, oxs) = (sample_axis(oh), sample_axis(ow));
            let mut ok = true;
            'corners: for b in [0, n - 1] { for ci in [0, c - 1] { for co in [0, o - 1] { for &oy in &oys { for &ox in &oxs { for kr in 0..kh { for ks in 0..kw {
                if !reads(b, co, oy, ox, ci, kr, ks) { ok = false; break 'corners; }
            } } } } } } }
            ok = ok && sample_axis(n).into_iter().all(|b| sample_axis(c).into_iter().all(|ci|
                reads(b, 0, 0, 0, ci, 0, 0) && reads(b, o - 1, oh - 1, ow - 1, ci, kh - 1, kw - 1) && reads(b, 0, oh / 2, ow / 2, ci, kh / 2, kw / 2)));
            if !ok { continue; }
            let conv = ZyxbConvDesc {
                dtype: dt as i32, n, c, h, w: wd, o, kh, kw, stride_h: sh as u32, stride_w: sw as u32, dil_h: dh as u32, dil_w: dw as u32,
                pad_top: pad[0] as u32, pad_bottom: pad[1] as u32, pad_left: pad[2] as u32, pad_right: pad[3] as u32,
                has_bias: bias.is_some() as i32, ..Default::default()
            };
            let mut inputs = vec![x, w];
            inputs.extend(bias);
            return Some(B200Match { pattern: if bias.is_some() { "conv_bias" } else { "conv" }, inputs, outputs: vec![cid],
                                    desc: ZyxbKernelDesc { kind: ZYXB_KIND_CONV, u: ZyxbDescUnion { conv } }, numel: Vec::new(), optim_step: 0, input_offsets: Vec::new() });
        }
        None
    }

    // ---- cross-entropy with class-index targets -----------------------------------------------------------------------------
    /// c = [Cast]{Eq{Expand{labels.reshape([n, 1])}, Expand{arange(classes)}}}, either operand order -> labels [n]
    /// (Tensor::one_hot_along_dim of the unsqueezed labels, tensor/mod.rs:1920-1946).  The arange is recognised by its value;
    /// i32 labels only (what the program reads).
    fn one_hot_labels(&self, c: ClassId, n: Dim, classes: Dim) -> Option<ClassId> {
        let c = self.cast_src(c).unwrap_or(c);
        let (x, y) = self.binary_of(c, BOp::Eq)?;
        for (a, b) in [(x, y), (y, x)] {
            let (Some(ea), Some(eb)) = (self.expand_of(a), self.expand_of(b)) else { continue };
            if self.const_shape(ea).as_deref() != Some(&[n, 1][..]) { continue; }
            let bs = self.const_shape(eb)?;
            if bs != [classes] && bs != [1, classes] { continue; }
            let Some(labels) = self.reshape_of(ea) else { continue };
            if self.const_shape(labels).as_deref() != Some(&[n][..]) || self.dtype(labels) != DType::I32 { continue; }
            let Some(v) = self.const_eval(eb) else { continue };
            if v.len() as u64 == classes && v.iter().enumerate().all(|(i, &k)| k == i as f64) { return Some(self.canon(labels)); }
        }
        None
    }
    /// Tensor::cross_entropy(labels, ReduceOp::Mean) on f32 logits [n, classes] (tensor/mod.rs:1639-1656):
    ///   per_sample = (-logits.ln_softmax([1]) * one_hot(labels)).sum([1]);  loss = per_sample.mean_all()
    /// -> one program, args logits, labels -> per_sample, loss.
    fn match_cross_entropy(&self, cid: ClassId) -> Option<B200Match> {
        if self.dtype(cid) != DType::F32 { return None; }
        let (sum, n) = self.binary_const(cid, BOp::Div)?;
        let (ps, axes) = self.find_in(sum, |nd| match nd { Node::Reduce { x, rop: BOp::Add, axes } => Some((*x, axes.clone())), _ => None })?;
        let per_sample = self.canon(ps);
        let pshape = self.const_shape(per_sample)?;
        if pshape.len() != 1 || axes.len() != 1 || (n - pshape[0] as f64).abs() > 0.5 || self.dtype(per_sample) != DType::F32 { return None; }
        let prod = self.reduce_last(per_sample, BOp::Add)?;
        let nc = self.const_shape(prod)?;
        if nc.len() != 2 || nc[0] != pshape[0] { return None; }
        let (a, b) = self.binary_of(prod, BOp::Mul)?;
        for (neg, target) in [(a, b), (b, a)] {
            let Some(ls) = self.unary_of(neg, UOp::Neg).and_then(|l| self.match_ln_softmax(l)) else { continue };
            let logits = ls.inputs[0];
            if self.dtype(logits) != DType::F32 || self.const_shape(logits)? != nc { continue; }
            let Some(labels) = self.one_hot_labels(target, nc[0], nc[1]) else { continue };
            let mut m = self.row_match("cross_entropy", self.row_desc(RR_CROSS_ENTROPY, logits)?, vec![logits, labels], per_sample);
            m.outputs.push(cid);
            return Some(m);
        }
        None
    }
    /// var(x, [-1]) = sum((x - mean_keepdim(x))^2) / (n - correction) (tensor/reduce_ops.rs:111-123) -> (x, correction)
    fn var_last(&self, cid: ClassId) -> Option<(ClassId, i32)> {
        let (sq, d) = self.mean_last(cid)?;
        let (a, b) = self.binary_of(sq, BOp::Mul)?;
        if !self.same(a, b) { return None; }
        let (x, mean) = self.binary_of(a, BOp::Sub)?;
        let x = self.canon(x);
        let (mx, _) = self.mean_last(self.keepdim_src(mean))?;
        if !self.same(mx, x) { return None; }
        let n = *self.const_shape(x)?.last()? as f64;
        let corr = (n - d).round();
        (corr >= 0.0 && corr < n && ((n - d) - corr).abs() <= 1e-6).then_some((x, corr as i32))
    }
    /// x [rows, cols] .sum([0]) -> x (the bias gradient of a Linear layer)
    fn column_sum_src(&self, cid: ClassId) -> Option<ClassId> {
        let red = |c: ClassId| self.find_in(c, |n| match n { Node::Reduce { x, rop: BOp::Add, axes } if axes.as_ref() == [0] => Some(*x), _ => None });
        let mut x = red(cid).or_else(|| red(self.cast_src(cid)?))?;
        if let Some(k) = self.cast_src(x) { if self.dtype(k) == self.dtype(cid) { x = k; } }     // the accumulator cast
        let x = self.canon(x);
        (self.const_shape(x)?.len() == 2 && self.dtype(x) == self.dtype(cid)).then_some(x)
    }
    /// var / std / sum / max / mean over the last axis, sum over the rows of a matrix
    fn match_reduce(&self, cid: ClassId) -> Option<B200Match> {
        for (name, op, v) in [("var", RR_VAR, Some(cid)), ("std", RR_STD, self.unary_of(cid, UOp::Sqrt))] {
            if let Some((x, corr)) = v.and_then(|v| self.var_last(v)) {
                if self.dtype(cid) == self.dtype(x) {
                    if let Some(mut d) = self.row_desc(op, x) { d.correction = corr; return Some(self.row_match(name, d, vec![x], cid)); }
                }
            }
        }
        if let Some(x) = self.column_sum_src(cid) {
            if !self.is_broadcast_product(x) { if let Some(d) = self.row_desc(RR_COLSUM, x) { return Some(self.row_match("colsum", d, vec![x], cid)); } }
        }
        if let Some((x, _)) = self.mean_last(cid) { if let Some(d) = self.row_desc(RR_MEAN, x) { return Some(self.row_match("mean", d, vec![x], cid)); } }
        // min = -max(-x) for floats, !max(!x) bitwise for integers (Tensor::inverse, reduce_ops.rs:33-42, 93-99); keepdim reshapes outside
        let c = match self.reshape_of(cid) { Some(r) if self.numel_of(r) == self.numel_of(cid) => r, _ => cid };
        for uop in [UOp::Neg, UOp::BitNot] {
            let x = self.unary_of(c, uop).and_then(|inner| self.reduce_last(inner, BOp::Max)).and_then(|nx| self.unary_of(nx, uop)).map(|x| self.canon(x));
            if let Some(x) = x.filter(|&x| self.dtype(x) == self.dtype(cid) && (uop == UOp::Neg) == self.dtype(x).is_float()) {
                if let Some(d) = self.row_desc(RR_MIN, x) { return Some(self.row_match("min", d, vec![x], cid)); }
            }
        }
        for (rop, rr, name) in [(BOp::Add, RR_SUM, "sum"), (BOp::Max, RR_MAX, "max")] {
            if let Some(x) = self.reduce_last(cid, rop) {
                if self.dtype(cid) != self.dtype(x) || self.is_broadcast_product(x) { continue; }
                if let Some(d) = self.row_desc(rr, x) { return Some(self.row_match(name, d, vec![x], cid)); }
            }
        }
        None
    }

    // ---- optimizer updates -------------------------------------------------------------------------------------------------
    /// p' = (p - g * lr).cast(p.dtype) (zyx-optim/src/sgd.rs:79-82)
    /// x + y * const with y the class `of` (or, of == None, any tensor of the shape of `like`) -> (x, y, const)
    fn plus_scaled(&self, e: ClassId, of: Option<ClassId>, like: ClassId) -> Option<(ClassId, ClassId, f64)> {
        let (a, b) = self.binary_of(e, BOp::Add)?;
        for (lhs, rhs) in [(a, b), (b, a)] {
            if let Some((y, k)) = self.binary_const(rhs, BOp::Mul) {
                let hit = match of { Some(o) => self.same(y, o), None => self.const_shape(y) == self.const_shape(like) };
                if hit { return Some((lhs, y, k)); }
            }
        }
        None
    }
    /// G = g [+ p * weight_decay] -> (g, weight_decay)
    fn strip_decay(&self, big_g: ClassId, p: ClassId) -> (ClassId, f64) {
        match self.plus_scaled(big_g, Some(p), p) { Some((g, _, wd)) => (g, wd), None => (big_g, 0.0) }
    }
    /// buf' = buf * momentum + G * (1 - dampening), buf a stored tensor -> (buf, momentum, dampening, G)
    fn buffer_update(&self, b: ClassId, p: ClassId) -> Option<(ClassId, f64, f64, ClassId)> {
        let (old, fresh) = self.binary_of(b, BOp::Add)?;
        let (buf, mom) = self.binary_const(old, BOp::Mul)?;
        let (big_g, one_minus) = self.binary_const(fresh, BOp::Mul)?;
        (self.is_leaf(buf) && !self.same(buf, p) && self.const_shape(buf) == self.const_shape(p)).then_some((buf, mom, 1.0 - one_minus, big_g))
    }
    /// SGD::update (zyx-optim/src/sgd.rs:58-82, without maximize): plain, with weight decay, with momentum after the first step
    /// (p' = p - buf' * lr) and with Nesterov (p' = p - (G + buf' * momentum) * lr).  On the first step the reference stores G
    /// itself as the buffer, so that update is the plain form.
    fn match_sgd(&self, cid: ClassId) -> Option<Update> {
        let (p, step) = self.binary_of(self.canon(cid), BOp::Sub)?;
        let (x, lr) = self.binary_const(step, BOp::Mul)?;
        if !self.is_leaf(p) || self.const_shape(x) != self.const_shape(p) { return None; }
        let base = Update { algo: OPT_SGD, p, g: x, m: None, v: None, p_new: cid, m_new: None, v_new: None, lr, wd: 0.0, b1: 0.0, b2: 0.0, eps: 0.0,
                            bc1: 0.0, bc2: 0.0, first: false, mom: 0.0, damp: 0.0, nesterov: false };
        if let Some((big_g, bnew, k)) = self.plus_scaled(x, None, p) {
            if !self.is_leaf(bnew) {
                if let Some((buf, mom, damp, g_in)) = self.buffer_update(bnew, p) {
                    let ((g, wd), (g2, wd2)) = (self.strip_decay(g_in, p), self.strip_decay(big_g, p));
                    if (k - mom).abs() <= 1e-12 * mom.abs() && self.same(g, g2) && wd == wd2 {
                        return Some(Update { g, wd, m: Some(buf), m_new: Some(bnew), mom, damp, nesterov: true, ..base });
                    }
                }
            }
        }
        if let Some((buf, mom, damp, g_in)) = self.buffer_update(x, p) {
            let (g, wd) = self.strip_decay(g_in, p);
            return Some(Update { g, wd, m: Some(buf), m_new: Some(x), mom, damp, ..base });
        }
        let (g, wd) = self.strip_decay(x, p);
        Some(Update { g, wd, ..base })
    }
    /// AdamW::update for one parameter (zyx-optim/src/adamw.rs:58-95)
    fn match_adamw(&self, cid: ClassId) -> Option<Update> {
        let (mut c, mut wd) = (cid, 0.0);
        if let Some((x, k)) = self.binary_const(c, BOp::Mul) { if !self.is_leaf(x) { wd = 1.0 - k; c = x; } }      // p * (1 - lr*wd)
        let (p, step) = self.binary_of(self.canon(c), BOp::Sub)?;
        if !self.is_leaf(p) { return None; }
        let (mh, den) = self.binary_of(step, BOp::Div)?;                     // mh / ((sqrt(vh) + eps) * lr)
        let (root_eps, lr) = self.binary_const(den, BOp::Mul)?;
        let (root, eps) = self.binary_const(root_eps, BOp::Add)?;
        let vh = self.unary_of(root, UOp::Sqrt)?;
        let ((m_new, bc1), (v_new, bc2)) = (self.binary_const(mh, BOp::Div)?, self.binary_const(vh, BOp::Div)?);
        let ((m, b1, g1), (v, b2, g2)) = (self.moment(m_new, false)?, self.moment(v_new, true)?);
        if !self.same(g1, g2) || m.is_some() != v.is_some() { return None; }
        Some(Update { algo: OPT_ADAMW, p, g: g1, m, v, p_new: cid, m_new: Some(m_new), v_new: Some(v_new), lr, wd: if wd != 0.0 { wd / lr } else { 0.0 },
                      b1, b2, eps, bc1, bc2, first: m.is_none(), mom: 0.0, damp: 0.0, nesterov: false })
    }
    /// m' = m*b1 + g*(1-b1), or g*(1-b1) alone on the first step (adamw.rs:60-71, adam.rs:72-81); v' alike with g*g
    /// -> (state, beta, g)
    fn moment(&self, mc: ClassId, squared: bool) -> Option<(Option<ClassId>, f64, ClassId)> {
        let grad_term = |t: ClassId| -> Option<(ClassId, f64)> {
            let (x, om) = self.binary_const(t, BOp::Mul)?;
            if !squared { return Some((x, om)); }
            let (a, b) = self.binary_of(x, BOp::Mul)?;
            self.same(a, b).then_some((a, om))
        };
        if let Some((l, r)) = self.binary_of(mc, BOp::Add) {
            if let (Some((state, _)), Some((g, om))) = (self.binary_const(l, BOp::Mul), grad_term(r)) { if self.is_leaf(state) { return Some((Some(state), 1.0 - om, g)); } }
        }
        grad_term(mc).map(|(g, om)| (None, 1.0 - om, g))
    }
    /// Adam::update for one parameter without amsgrad (zyx-optim/src/adam.rs:66-101):
    /// G = g [+ p * weight_decay]; p' = (p - lr * mh / (sqrt(vh) + eps)).cast(p.dtype)
    fn match_adam(&self, cid: ClassId) -> Option<Update> {
        let (p, step) = self.binary_of(self.canon(cid), BOp::Sub)?;
        if !self.is_leaf(p) { return None; }
        let (num, den) = self.binary_of(step, BOp::Div)?;                    // (lr * mh) / (sqrt(vh) + eps)
        let (mh, lr) = self.binary_const(num, BOp::Mul)?;
        let (root, eps) = self.binary_const(den, BOp::Add)?;
        let vh = self.unary_of(root, UOp::Sqrt)?;
        let ((m_new, bc1), (v_new, bc2)) = (self.binary_const(mh, BOp::Div)?, self.binary_const(vh, BOp::Div)?);
        let ((m, b1, g1), (v, b2, g2)) = (self.moment(m_new, false)?, self.moment(v_new, true)?);
        if !self.same(g1, g2) || m.is_some() != v.is_some() { return None; }
        let (g, wd) = self.strip_decay(g1, p);
        Some(Update { algo: OPT_ADAM, p, g, m, v, p_new: cid, m_new: Some(m_new), v_new: Some(v_new), lr, wd, b1, b2, eps, bc1, bc2,
                      first: m.is_none(), mom: 0.0, damp: 0.0, nesterov: false })
    }

    /// What the programs pushed so far do NOT cover: walking down from `outputs` through the Node::Kernel alternatives (at each class
    /// the one pushed last, the largest pattern), the classes that are needed but are neither stored nor produced by a program.
    /// Empty: the device can execute the graph on its own.
    pub(crate) fn uncovered_b200(&self, outputs: &BTreeSet<ClassId>) -> Vec<ClassId> {
        let (mut missing, mut seen) = (Vec::new(), BTreeSet::new());
        let mut need: Vec<ClassId> = outputs.iter().rev().copied().collect();
        while let Some(c) = need.pop() {
            if !seen.insert(self.canon(c)) || self.is_leaf(c) { continue; }
            let (mut k, mut kernel) = (c, None);
            loop {                                                 // the class, what it is a no-op of, what it is a reshape of
                kernel = self.classes[k].nodes.iter().rev().find_map(|&nid| match &self.nodes[nid].node { Node::Kernel { inputs, .. } => Some(inputs.clone()), _ => None });
                if kernel.is_some() { break; }
                match self.noop_cast(k).or_else(|| self.reshape_of(k)) { Some(x) if !self.is_leaf(x) => k = x, _ => break }
            }
            match kernel { Some(inputs) => need.extend(inputs.iter().rev()), None => if !self.is_leaf(self.storage(c)) { missing.push(c) } }
        }
        missing
    }

    /// Everything the device's match_graph needs: `order` is topo_sort_classes_without_kernels of the outputs, `wanted` the
    /// outputs themselves (classes other consumers read).  Optimizer updates of one dtype and one set of hyper-parameters become
    /// one multi-tensor program.
    pub(crate) fn match_b200(&self, order: &[ClassId], wanted: &BTreeSet<ClassId>) -> Vec<B200Match> {
        let mut out = Vec::new();
        let mut updates: Vec<Update> = Vec::new();
        for &cid in order {
            if wanted.contains(&cid) {
                if let Some(u) = self.match_adamw(cid).or_else(|| self.match_adam(cid)).or_else(|| self.match_sgd(cid)) { updates.push(u); continue; }
            }
            let m = self.match_attention(cid).or_else(|| self.match_linear(cid, wanted)).or_else(|| self.match_conv(cid)).or_else(|| self.match_softmax(cid)).or_else(|| self.match_ln_softmax(cid))
                .or_else(|| self.match_layernorm(cid)).or_else(|| self.match_cross_entropy(cid)).or_else(|| self.match_mse(cid)).or_else(|| self.match_reduce(cid));
            out.extend(m);
        }
        let mut used = vec![false; updates.len()];
        for i in 0..updates.len() {
            if used[i] { continue; }
            let h = updates[i];
            let same_group = |u: &Update| u.algo == h.algo && self.dtype(u.p) == self.dtype(h.p) && u.first == h.first
                && (u.lr, u.wd, u.b1, u.b2, u.eps, u.bc1, u.bc2) == (h.lr, h.wd, h.b1, h.b2, h.eps, h.bc1, h.bc2)
                && (u.mom, u.damp, u.nesterov, u.m.is_some()) == (h.mom, h.damp, h.nesterov, h.m.is_some());
            let (mut p, mut g, mut ms, mut vs, mut outs, mut numel) = (vec![], vec![], vec![], vec![], vec![], vec![]);
            for j in i..updates.len() {
                let u = updates[j];
                if used[j] || !same_group(&u) { continue; }
                used[j] = true;
                p.push(u.p); g.push(u.g); numel.push(self.numel_of(u.p).unwrap_or(0));
                outs.push(u.p_new);
                if u.algo != OPT_SGD { ms.extend(u.m); vs.extend(u.v); outs.extend(u.m_new); outs.extend(u.v_new); }
                else if u.m.is_some() { ms.extend(u.m); outs.extend(u.m_new); }          // SGD: the momentum buffer
            }
            let optim = ZyxbOptimDesc { algo: h.algo, dtype: self.dtype(h.p) as i32, n_tensors: p.len() as i32, numel: std::ptr::null(), lr: h.lr as f32,
                                        weight_decay: h.wd as f32, momentum: h.mom as f32, dampening: h.damp as f32, nesterov: h.nesterov as i32, maximize: 0, beta1: h.b1 as f32,
                                        beta2: h.b2 as f32, eps: h.eps as f32, grad_scale: 0.0, standard: 0 };
            let mut inputs = p;
            inputs.extend(g); inputs.extend(ms); inputs.extend(vs);
            let sgd_buf = h.algo == OPT_SGD && h.m.is_some();
            let pattern = if h.algo == OPT_ADAM { if h.first { "adam_first_step" } else { "adam" } }
                          else if h.algo != OPT_SGD { if h.first { "adamw_first_step" } else { "adamw" } }
                          else if !sgd_buf { "sgd" } else if h.nesterov { "sgd_nesterov" } else { "sgd_momentum" };
            // the step the update belongs to: AdamW's bias correction divides by 1 - beta1^t
            let optim_step = if h.algo == OPT_SGD { if sgd_buf { 2 } else { 1 } }
                             else if h.first { 1 } else { ((1.0 - h.bc1).ln() / h.b1.ln()).round().max(2.0) as u64 };
            out.push(B200Match { pattern, inputs, outputs: outs,
                                 desc: ZyxbKernelDesc { kind: ZYXB_KIND_OPTIM, u: ZyxbDescUnion { optim } }, numel, optim_step, input_offsets: Vec::new() });
        }
        // Elementwise programs, on demand.  Walk down from the outputs of the graph through the programs found above (for a class
        // several of them end at, the one found last: the largest pattern): whatever that walk needs and nothing stored or matched
        // produces gets an elementwise program if one fits, and the walk continues through its operands.  Offering every Mul and
        // Add of the graph as a program of its own would bury the patterns above under their own sub-expressions; following the
        // inputs of every alternative would do the same with the inside of a softmax.
        let has_kernel = |c: ClassId| self.classes[c].nodes.iter().any(|&nid| matches!(self.nodes[nid].node, Node::Kernel { .. }));
        let mut producer: BTreeMap<ClassId, usize> = BTreeMap::new();
        for (i, m) in out.iter().enumerate() { for &o in &m.outputs { producer.insert(self.canon(o), i); } }
        let mut seen = BTreeSet::new();
        let mut need: Vec<ClassId> = wanted.iter().rev().copied().collect();
        while let Some(c) = need.pop() {
            // nothing ends at a reshaped class: its elements are the source's
            let c = if producer.contains_key(&self.canon(c)) { c } else { self.storage(c) };
            let k = self.canon(c);
            if !seen.insert(k) || self.is_leaf(c) { continue; }
            let via = match producer.get(&k) {
                Some(&i) => i,
                None => {
                    if has_kernel(c) || has_kernel(k) { continue; }
                    let Some(m) = self.match_eltwise(c) else { continue };
                    out.push(m);
                    producer.insert(k, out.len() - 1);
                    out.len() - 1
                }
            };
            need.extend(out[via].inputs.iter().rev());
        }
        // inputs are named by the class whose buffer holds them (a reshape of a stored tensor is that tensor), unless a program ends
        // at the reshape itself
        for m in &mut out {
            for input in &mut m.inputs {
                if !producer.contains_key(&self.canon(*input)) && !has_kernel(*input) && !has_kernel(self.canon(*input)) { *input = self.storage(*input); }
            }
        }
        out
    }
}
