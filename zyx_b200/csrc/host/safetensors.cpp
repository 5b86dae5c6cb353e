// C entry points over the safetensors reader / writer (include/zyxb_host.h: zyxb_st_*).
#include "safetensors.hpp"

#include "../../../include/zyxb_host.h"

using namespace zyxb_host;

struct zyxb_st_file {
  st::File file;
};

namespace {
thread_local std::string g_err;
int32_t fail(int32_t code, const std::string& what) {
  g_err = what;
  return code;
}
}  // namespace

extern "C" {
#pragma GCC visibility push(default)

const char* zyxb_st_last_error(void) { return g_err.c_str(); }

int32_t zyxb_st_save(const char* path, const zyxb_st_tensor* tensors, int32_t n) {
  if (!path || n < 0 || (n > 0 && !tensors)) return fail(ZYXB_ERR_INCORRECT_KERNEL_ARG, "zyxb_st_save: null argument");
  std::vector<st::TensorRef> refs((size_t)n);
  for (int32_t i = 0; i < n; ++i) {
    const zyxb_st_tensor& t = tensors[i];
    if (!t.name || t.rank < 0 || (t.rank > 0 && !t.shape)) return fail(ZYXB_ERR_INCORRECT_KERNEL_ARG, "zyxb_st_save: tensor without a name or shape");
    refs[i].name = t.name; refs[i].dtype = t.dtype; refs[i].shape.assign(t.shape, t.shape + t.rank); refs[i].data = t.data;
    if (!t.data && st::numel(refs[i].shape) != 0) return fail(ZYXB_ERR_INCORRECT_KERNEL_ARG, "zyxb_st_save: tensor without data");
    for (int32_t k = 0; k < i; ++k)
      if (refs[k].name == refs[i].name) return fail(ZYXB_ERR_INCORRECT_KERNEL_ARG, "zyxb_st_save: duplicate tensor name '" + refs[i].name + "'");
  }
  std::string err;
  if (!st::write(path, refs, err)) return fail(ZYXB_ERR_MEMORY_COPY_P2H, err);
  return ZYXB_OK;
}

int32_t zyxb_st_open(const char* path, zyxb_st_file** out) {
  if (!path || !out) return fail(ZYXB_ERR_INCORRECT_KERNEL_ARG, "zyxb_st_open: null argument");
  zyxb_st_file* f = new zyxb_st_file();
  std::string err;
  if (!st::open(path, f->file, err)) { delete f; return fail(ZYXB_ERR_MEMORY_COPY_H2P, err); }
  *out = f;
  return ZYXB_OK;
}
int32_t zyxb_st_count(const zyxb_st_file* f) { return f ? (int32_t)f->file.entries.size() : 0; }
int32_t zyxb_st_info(const zyxb_st_file* f, int32_t i, const char** out_name, int32_t* out_dtype, int32_t* out_rank,
                     const uint64_t** out_shape, uint64_t* out_bytes) {
  if (!f || i < 0 || (size_t)i >= f->file.entries.size()) return fail(ZYXB_ERR_INCORRECT_KERNEL_ARG, "zyxb_st_info: no such tensor");
  const st::Entry& e = f->file.entries[i];
  if (out_name) *out_name = e.name.c_str();
  if (out_dtype) *out_dtype = e.dtype;
  if (out_rank) *out_rank = (int32_t)e.shape.size();
  if (out_shape) *out_shape = e.shape.data();
  if (out_bytes) *out_bytes = e.end - e.begin;
  return ZYXB_OK;
}
int32_t zyxb_st_find(const zyxb_st_file* f, const char* name) { return (f && name) ? st::find(f->file, name) : -1; }
int32_t zyxb_st_read(zyxb_st_file* f, int32_t i, void* dst, uint64_t dst_bytes) {
  if (!f || (!dst && dst_bytes)) return fail(ZYXB_ERR_INCORRECT_KERNEL_ARG, "zyxb_st_read: null argument");
  std::string err;
  if (!st::read(f->file, i, dst, dst_bytes, err)) return fail(ZYXB_ERR_MEMORY_COPY_H2P, err);
  return ZYXB_OK;
}
int32_t zyxb_st_close(zyxb_st_file* f) {
  if (!f) return ZYXB_OK;
  st::close(f->file);
  delete f;
  return ZYXB_OK;
}

#pragma GCC visibility pop
}  // extern "C"
