// Checkpoints of a plan: parameters, optimizer state and step counter in one safetensors file.
// The tensors travel host <-> pool through the C ABI (zyxb_d2h / zyxb_h2d), the file through safetensors.hpp.
#pragma once
#include <string>
#include <vector>

#include "safetensors.hpp"

namespace zyxb_host {

struct CkptTensor {
  std::string name;
  uint32_t buffer = 0;
  std::vector<uint64_t> shape;
};

// state_names: per optimizer state tensor list the prefix ("optim.m.", "optim.v.", "optim.buf.")
inline int32_t checkpoint_save(zyxb_ctx* ctx, int32_t dev, int32_t dtype, const std::vector<CkptTensor>& tensors, uint64_t step,
                               const std::string& path, std::string& err) {
  std::vector<std::vector<uint8_t>> host(tensors.size());
  std::vector<st::TensorRef> refs;
  for (size_t i = 0; i < tensors.size(); ++i) {
    const uint64_t bytes = st::numel(tensors[i].shape) * st::dtype_bytes(dtype);
    host[i].resize(bytes);
    int32_t rc = zyxb_d2h(ctx, dev, tensors[i].buffer, 0, host[i].data(), bytes, nullptr, 0);
    if (rc) { err = std::string("checkpoint: zyxb_d2h of '") + tensors[i].name + "': " + zyxb_last_error(ctx); return rc; }
    st::TensorRef r;
    r.name = tensors[i].name; r.dtype = dtype; r.shape = tensors[i].shape; r.data = host[i].data();
    refs.push_back(std::move(r));
  }
  const uint64_t t64 = step;
  st::TensorRef t;
  t.name = "optim.t"; t.dtype = ZYXB_U64; t.shape = {1}; t.data = &t64;
  refs.push_back(t);
  if (!st::write(path, refs, err)) return ZYXB_ERR_MEMORY_COPY_P2H;
  return ZYXB_OK;
}

inline int32_t checkpoint_load(zyxb_ctx* ctx, int32_t dev, int32_t dtype, const std::vector<CkptTensor>& tensors, uint64_t* step,
                               bool* have_step, int32_t* missing, const std::string& path, std::string& err) {
  st::File f;
  if (!st::open(path, f, err)) return ZYXB_ERR_MEMORY_COPY_H2P;
  int32_t n_missing = 0, n_state_missing = 0, rc = ZYXB_OK;
  // first pass: every tensor the file holds must fit the plan's, so that a bad file is refused before anything is overwritten
  for (const CkptTensor& t : tensors) {
    const int i = st::find(f, t.name);
    if (i < 0) { ++n_missing; n_state_missing += t.name.compare(0, 6, "optim.") == 0; continue; }
    const st::Entry& e = f.entries[i];
    if (e.dtype != dtype || st::numel(e.shape) != st::numel(t.shape)) {
      err = "checkpoint: '" + t.name + "' in " + path + " has another dtype or element count than the plan's tensor";
      rc = ZYXB_ERR_INCORRECT_KERNEL_ARG; break;
    }
  }
  std::vector<uint8_t> host;
  for (size_t k = 0; !rc && k < tensors.size(); ++k) {
    const CkptTensor& t = tensors[k];
    const int i = st::find(f, t.name);
    if (i < 0) continue;
    const st::Entry& e = f.entries[i];
    host.resize(e.end - e.begin);
    if (!st::read(f, i, host.data(), host.size(), err)) { rc = ZYXB_ERR_MEMORY_COPY_H2P; break; }
    zyxb_event ev{};
    rc = zyxb_h2d(ctx, dev, host.data(), host.size(), t.buffer, 0, nullptr, 0, &ev);
    if (!rc) rc = zyxb_sync(ctx, dev, &ev, 1);       // `host` is reused for the next tensor
    if (rc) { err = std::string("checkpoint: zyxb_h2d of '") + t.name + "': " + zyxb_last_error(ctx); break; }
  }
  *have_step = false;
  if (!rc && n_state_missing == 0) {       // a step counter without its moment buffers (e.g. another rank's shard file) would mis-scale Adam
    const int i = st::find(f, "optim.t");
    if (i >= 0 && st::numel(f.entries[i].shape) == 1) {
      uint64_t t64 = 0;
      uint32_t t32 = 0;
      if (f.entries[i].dtype == ZYXB_U64 && st::read(f, i, &t64, 8, err)) { *step = t64; *have_step = true; }
      else if (f.entries[i].dtype == ZYXB_U32 && st::read(f, i, &t32, 4, err)) { *step = t32; *have_step = true; }
    }
  }
  st::close(f);
  if (missing) *missing = n_missing;
  return rc;
}

}  // namespace zyxb_host
