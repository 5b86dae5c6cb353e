// NCCL binding by dlopen.  One communicator per process (one process per GPU); the
// unique id is created on rank 0 and carried to the other ranks by the launcher.
#include "comm.h"

#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/zyxb.h"

namespace zyxb {

namespace {
// The few NCCL types and enum values used here, as published in nccl.h (stable ABI since 2.x).
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
enum { ncclSuccess = 0 };
enum { ncclFloat16 = 6, ncclFloat32 = 7, ncclBfloat16 = 9, ncclInt32 = 2 };
enum { ncclSum = 0 };

struct Api {
  void* handle = nullptr;
  int (*GetUniqueId)(ncclUniqueId*) = nullptr;
  int (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*ReduceScatter)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*CommDestroy)(ncclComm_t) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  std::string load_error;
};

Api& api() {
  static Api a;
  static bool tried = false;
  if (tried) return a;
  tried = true;
  const char* env = getenv("ZYXB_NCCL_LIB");
  const char* names[] = {env, "libnccl.so.2", "libnccl.so"};
  for (const char* n : names) {
    if (!n) continue;
    a.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (a.handle) break;
  }
  if (!a.handle) { a.load_error = "libnccl.so.2 not found (set ZYXB_NCCL_LIB to its path)"; return a; }
  a.GetUniqueId = (decltype(a.GetUniqueId))dlsym(a.handle, "ncclGetUniqueId");
  a.CommInitRank = (decltype(a.CommInitRank))dlsym(a.handle, "ncclCommInitRank");
  a.AllReduce = (decltype(a.AllReduce))dlsym(a.handle, "ncclAllReduce");
  a.ReduceScatter = (decltype(a.ReduceScatter))dlsym(a.handle, "ncclReduceScatter");
  a.AllGather = (decltype(a.AllGather))dlsym(a.handle, "ncclAllGather");
  a.CommDestroy = (decltype(a.CommDestroy))dlsym(a.handle, "ncclCommDestroy");
  a.GetErrorString = (decltype(a.GetErrorString))dlsym(a.handle, "ncclGetErrorString");
  if (!a.GetUniqueId || !a.CommInitRank || !a.AllReduce || !a.ReduceScatter || !a.AllGather || !a.CommDestroy) { a.load_error = "libnccl is missing a required symbol"; a.handle = nullptr; }
  return a;
}

std::string nccl_err(const char* what, int code) {
  Api& a = api();
  return std::string(what) + ": " + (a.GetErrorString ? a.GetErrorString(code) : "NCCL error") + " (" + std::to_string(code) + ")";
}
}  // namespace

struct Comm { ncclComm_t comm = nullptr; int rank = 0, world = 1; };

int comm_unique_id(void* out, std::string& err) {
  Api& a = api();
  if (!a.handle) { err = a.load_error; return ZYXB_ERR_DYLIB_NOT_FOUND; }
  ncclUniqueId id;
  int r = a.GetUniqueId(&id);
  if (r != ncclSuccess) { err = nccl_err("ncclGetUniqueId", r); return ZYXB_ERR_INITIALIZATION; }
  memcpy(out, &id, sizeof(id));
  return ZYXB_OK;
}

int comm_create(Comm** out, int rank, int world, const void* id_bytes, std::string& err) {
  Api& a = api();
  if (!a.handle) { err = a.load_error; return ZYXB_ERR_DYLIB_NOT_FOUND; }
  if (world < 1 || rank < 0 || rank >= world) { err = "comm_init: bad rank/world"; return ZYXB_ERR_INITIALIZATION; }
  ncclUniqueId id;
  memcpy(&id, id_bytes, sizeof(id));
  Comm* c = new Comm();
  c->rank = rank; c->world = world;
  int r = a.CommInitRank(&c->comm, world, id, rank);
  if (r != ncclSuccess) { delete c; err = nccl_err("ncclCommInitRank", r); return ZYXB_ERR_INITIALIZATION; }
  *out = c;
  return ZYXB_OK;
}

static int nccl_type(int dtype, std::string& err) {
  switch (dtype) {
    case ZYXB_F32: return ncclFloat32;
    case ZYXB_BF16: return ncclBfloat16;
    case ZYXB_F16: return ncclFloat16;
    case ZYXB_I32: return ncclInt32;
    default: err = "collective: dtype must be f32, bf16, f16 or i32"; return -1;
  }
}

int comm_allreduce_sum(Comm* c, const void* send, void* recv, uint64_t count, int dtype, cudaStream_t stream, std::string& err) {
  Api& a = api();
  const int nt = nccl_type(dtype, err);
  if (nt < 0) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  int r = a.AllReduce(send, recv, (size_t)count, nt, ncclSum, c->comm, stream);
  if (r != ncclSuccess) { err = nccl_err("ncclAllReduce", r); return ZYXB_ERR_KERNEL_LAUNCH; }
  return ZYXB_OK;
}

// In place over `world` consecutive slices of count_per_rank elements starting at base: afterwards this rank's slice
// holds the sum over ranks (NCCL's in-place form: the receive buffer is the rank's own slice of the send buffer).
int comm_reduce_scatter_sum(Comm* c, void* base, uint64_t count_per_rank, uint64_t elem_bytes, int dtype, cudaStream_t stream, std::string& err) {
  Api& a = api();
  const int nt = nccl_type(dtype, err);
  if (nt < 0) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  char* mine = (char*)base + (uint64_t)c->rank * count_per_rank * elem_bytes;
  int r = a.ReduceScatter(base, mine, (size_t)count_per_rank, nt, ncclSum, c->comm, stream);
  if (r != ncclSuccess) { err = nccl_err("ncclReduceScatter", r); return ZYXB_ERR_KERNEL_LAUNCH; }
  return ZYXB_OK;
}

// In place: every rank contributes its own slice, afterwards all hold the `world` slices.
int comm_allgather(Comm* c, void* base, uint64_t count_per_rank, uint64_t elem_bytes, int dtype, cudaStream_t stream, std::string& err) {
  Api& a = api();
  const int nt = nccl_type(dtype, err);
  if (nt < 0) return ZYXB_ERR_INCORRECT_KERNEL_ARG;
  const char* mine = (const char*)base + (uint64_t)c->rank * count_per_rank * elem_bytes;
  int r = a.AllGather(mine, base, (size_t)count_per_rank, nt, c->comm, stream);
  if (r != ncclSuccess) { err = nccl_err("ncclAllGather", r); return ZYXB_ERR_KERNEL_LAUNCH; }
  return ZYXB_OK;
}

int comm_allgather_raw(Comm* c, const void* send, void* recv, uint64_t bytes, cudaStream_t stream, std::string& err) {
  Api& a = api();
  int r = a.AllGather(send, recv, (size_t)bytes, /* ncclInt8 */ 0, c->comm, stream);
  if (r != ncclSuccess) { err = nccl_err("ncclAllGather", r); return ZYXB_ERR_KERNEL_LAUNCH; }
  return ZYXB_OK;
}

void comm_rank(const Comm* c, int* rank, int* world) { *rank = c->rank; *world = c->world; }

void comm_destroy(Comm* c) {
  if (!c) return;
  Api& a = api();
  if (a.handle && c->comm) a.CommDestroy(c->comm);
  delete c;
}

}  // namespace zyxb
