// A recorded sequence of zyxb launches and collectives — the host-side analogue of zyx's ExecPlan
// (zyx/src/graph/plan.rs:47-54: Allocate / Launch / Copy / Deallocate instructions built once by
// ExecPlan::new and replayed by execute_plan, 271-361).  Everything goes through the C ABI of zyxb.h.
#pragma once
#include <algorithm>
#include <string>
#include <vector>

#include "../../../include/zyxb.h"

namespace zyxb_host {

struct Instr {
  enum Kind { LAUNCH, ALLREDUCE, REDUCE_SCATTER, ALLGATHER } kind = LAUNCH;
  uint32_t program = 0;
  std::vector<uint32_t> args;
  uint32_t buffer = 0;            // collectives: buffer, first element and element count (per rank for the sliced two)
  uint64_t offset = 0, count = 0;
  int wait_collectives = 0;       // LAUNCH: wait first for this many of the oldest pending gradient-collective events (-1: all)
  int group = -1;                 // ALLGATHER: the parameter group it completes; LAUNCH: the first reader of that group's parameters
  bool tail = false;              // ALLREDUCE: the step's last collective, nothing left to hide it behind (ZYXB_COMM_OPT_LATENCY around the call)
};

inline uint64_t dsize(int32_t dtype) { return dtype == ZYXB_F32 ? 4 : 2; }
inline uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

class Plan {
 public:
  zyxb_ctx* ctx = nullptr;
  int32_t dev = 0;
  int32_t dtype = ZYXB_BF16;
  std::vector<Instr> instrs;
  std::vector<uint32_t> owned_buffers, owned_programs;
  std::vector<zyxb_event> pending;
  std::vector<zyxb_event> gathered;        // per parameter group: the event of its last all-gather, if nobody has waited for it yet
  std::vector<char> gathered_set;
  int n_launches = 0, n_collectives = 0;
  std::string err;

  int32_t fail(int32_t st, const char* what) {
    err = std::string(what) + ": " + zyxb_last_error(ctx);
    return st;
  }
  int32_t alloc(uint64_t bytes, uint32_t* out, bool zero = false) {
    zyxb_event ev{};
    int32_t st = zyxb_alloc(ctx, dev, bytes, out, &ev);
    if (st) return fail(st, "zyxb_alloc");
    owned_buffers.push_back(*out);
    if (zero && (st = zyxb_memset(ctx, dev, *out, 0, 0, bytes))) return fail(st, "zyxb_memset");
    return ZYXB_OK;
  }
  int32_t view(uint32_t parent, uint64_t offset_bytes, uint64_t bytes, uint32_t* out) {
    int32_t st = zyxb_buffer_view(ctx, dev, parent, offset_bytes, bytes, out);
    if (st) return fail(st, "zyxb_buffer_view");
    owned_buffers.push_back(*out);
    return ZYXB_OK;
  }
  int32_t launch(const zyxb_kernel_desc& d, std::vector<uint32_t> args, int wait_coll = 0, int group = -1) {
    Instr in;
    in.args = std::move(args);
    in.wait_collectives = wait_coll;
    in.group = group;
    int32_t st = zyxb_program_create(ctx, dev, &d, &in.program);
    if (st) return fail(st, "zyxb_program_create");
    owned_programs.push_back(in.program);
    instrs.push_back(std::move(in));
    ++n_launches;
    return ZYXB_OK;
  }
  void allreduce(uint32_t buffer, uint64_t offset, uint64_t count, bool tail = false) {
    Instr in;
    in.kind = Instr::ALLREDUCE; in.buffer = buffer; in.offset = offset; in.count = count; in.tail = tail;
    instrs.push_back(in);
    ++n_collectives;
  }
  void reduce_scatter(uint32_t buffer, uint64_t offset, uint64_t count_per_rank) {
    Instr in;
    in.kind = Instr::REDUCE_SCATTER; in.buffer = buffer; in.offset = offset; in.count = count_per_rank;
    instrs.push_back(in);
    ++n_collectives;
  }
  void allgather(uint32_t buffer, uint64_t offset, uint64_t count_per_rank, int group) {
    Instr in;
    in.kind = Instr::ALLGATHER; in.buffer = buffer; in.offset = offset; in.count = count_per_rank; in.group = group;
    instrs.push_back(in);
    ++n_collectives;
    if ((size_t)group >= gathered.size()) { gathered.resize(group + 1, zyxb_event{}); gathered_set.resize(group + 1, 0); }
  }
  // Blocks until every outstanding parameter all-gather has landed (whoever reads or writes a parameter from the host).
  int32_t join_gathers() {
    for (size_t g = 0; g < gathered.size(); ++g)
      if (gathered_set[g]) {
        int32_t st = zyxb_sync(ctx, dev, &gathered[g], 1);
        if (st) return fail(st, "zyxb_sync");
        gathered_set[g] = 0;
      }
    return ZYXB_OK;
  }
  // replay instructions [first, last)
  int32_t run(size_t first, size_t last, const zyxb_event* wait, int32_t n_wait) {
    bool head = true;
    for (size_t i = first; i < last && i < instrs.size(); ++i) {
      const Instr& in = instrs[i];
      if (in.kind != Instr::LAUNCH) {
        zyxb_event ev{};
        int32_t st;
        if (in.kind == Instr::ALLREDUCE) {
          if (in.tail && (st = zyxb_comm_option(ctx, dev, ZYXB_COMM_OPT_LATENCY, 1))) return fail(st, "zyxb_comm_option");
          st = zyxb_allreduce_sum(ctx, dev, in.buffer, in.offset, in.count, dtype, nullptr, 0, &ev);
          if (st) fail(st, "zyxb_allreduce_sum");
          if (in.tail) zyxb_comm_option(ctx, dev, ZYXB_COMM_OPT_LATENCY, 0);
          if (st) return st;
        } else if (in.kind == Instr::REDUCE_SCATTER) {
          if ((st = zyxb_reduce_scatter_sum(ctx, dev, in.buffer, in.offset, in.count, dtype, nullptr, 0, &ev))) return fail(st, "zyxb_reduce_scatter_sum");
        } else {
          if ((st = zyxb_allgather(ctx, dev, in.buffer, in.offset, in.count, dtype, nullptr, 0, &ev))) return fail(st, "zyxb_allgather");
        }
        if (in.kind == Instr::ALLGATHER) {
          if (gathered_set[in.group]) zyxb_release_events(ctx, dev, &gathered[in.group], 1);
          gathered[in.group] = ev; gathered_set[in.group] = 1;
        } else pending.push_back(ev);
        continue;
      }
      std::vector<zyxb_event> w;
      if (head && n_wait > 0) w.assign(wait, wait + n_wait);
      if (in.group >= 0 && (size_t)in.group < gathered.size() && gathered_set[in.group]) {   // these parameters are still being gathered
        w.push_back(gathered[in.group]);
        gathered_set[in.group] = 0;
      }
      if (in.wait_collectives != 0) {
        const size_t take = in.wait_collectives < 0 ? pending.size() : std::min(pending.size(), (size_t)in.wait_collectives);
        w.insert(w.end(), pending.begin(), pending.begin() + take);
        pending.erase(pending.begin(), pending.begin() + take);
      }
      int32_t st = zyxb_launch(ctx, dev, in.program, in.args.data(), (int32_t)in.args.size(), w.empty() ? nullptr : w.data(),
                               (int32_t)w.size(), nullptr);
      if (st) return fail(st, "zyxb_launch");
      head = false;
    }
    return ZYXB_OK;
  }
  void destroy() {
    zyxb_device_sync(ctx, dev);
    if (!pending.empty()) zyxb_release_events(ctx, dev, pending.data(), (int32_t)pending.size());
    for (size_t g = 0; g < gathered.size(); ++g)
      if (gathered_set[g]) zyxb_release_events(ctx, dev, &gathered[g], 1);
    gathered.clear(); gathered_set.clear();
    for (uint32_t p : owned_programs) zyxb_program_release(ctx, dev, p);
    for (auto it = owned_buffers.rbegin(); it != owned_buffers.rend(); ++it) zyxb_free(ctx, dev, *it, nullptr, 0);   // views before parents
    owned_programs.clear(); owned_buffers.clear(); pending.clear();
  }
};

// ---- descriptor builders ---------------------------------------------------------------------------
inline zyxb_kernel_desc gemm(int32_t dtype, uint64_t m, uint64_t n, uint64_t k, bool ta, bool tb, int32_t epi = ZYXB_EPI_NONE,
                             bool preact = false, float alpha = 1.0f) {
  zyxb_kernel_desc d{};
  d.kind = ZYXB_KIND_GEMM;
  d.u.gemm.dtype = dtype; d.u.gemm.m = m; d.u.gemm.n = n; d.u.gemm.k = k; d.u.gemm.batch = 1;
  d.u.gemm.trans_a = ta; d.u.gemm.trans_b = tb; d.u.gemm.epilogue = epi; d.u.gemm.store_preact = preact; d.u.gemm.alpha = alpha;
  return d;
}
inline zyxb_kernel_desc row(int32_t op, int32_t dtype, uint64_t rows, uint64_t cols) {
  zyxb_kernel_desc d{};
  d.kind = ZYXB_KIND_ROWREDUCE;
  d.u.rowreduce.op = op; d.u.rowreduce.dtype = dtype; d.u.rowreduce.rows = rows; d.u.rowreduce.cols = cols; d.u.rowreduce.correction = 1;
  return d;
}
inline zyxb_kernel_desc eltwise(int32_t op, int32_t dtype, uint64_t numel, float p0 = 0.0f) {
  zyxb_kernel_desc d{};
  d.kind = ZYXB_KIND_ELTWISE;
  d.u.eltwise.op = op; d.u.eltwise.dtype = dtype; d.u.eltwise.dtype_out = dtype; d.u.eltwise.numel = numel; d.u.eltwise.p0 = p0;
  return d;
}

}  // namespace zyxb_host
