// The C ABI of libzyxb: context, memory pool, events, programs.  Each entry point stands in
// for one method of zyx's backend interface (zyx/src/backend/mod.rs); the header cites them.
//
// Threading model: zyx serialises backend calls under its global runtime mutex
// (zyx/src/lib.rs:96), possibly from different OS threads.  Instead of the reference CUDA
// backend's worker thread per device (zyx/src/backend/cuda.rs:475-519) every call here makes
// its device current and enqueues on that device's streams:
//   compute : every kernel, d2h, memset            (in-order: a launch sees all earlier launches)
//   copy    : h2d, so uploads can overlap kernels  (ordered against compute by events)
//   comm    : NCCL collectives                      (ordered against compute by events)
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>

#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "comm.h"
#include "internal.h"

using namespace zyxb;

namespace {

struct Buffer {
  void* ptr = nullptr;
  uint64_t bytes = 0;      // bytes the caller asked for
  uint64_t capacity = 0;   // bytes of the underlying block
  bool live = false;
  bool is_variable = false;
  bool is_view = false;    // aliases a range of another buffer; freeing it releases only the id
  uint32_t parent = 0;     // views: the id of the buffer that owns the block (views of views name the owner)
  int32_t var_dtype = 0;
  uint8_t var_bytes[8] = {0};
};

struct Program {
  zyxb_kernel_desc desc{};
  std::vector<uint64_t> numel;  // optimizer programs: copy of desc.u.optim.numel
  uint64_t step = 0;            // optimizer programs: AdamW::t
  bool live = false;
};

struct Device {
  int cuda_id = 0;
  cudaDeviceProp prop{};
  cudaStream_t compute = nullptr, copy = nullptr, comm_stream = nullptr;
  std::vector<Buffer> buffers;
  std::vector<uint32_t> free_buffer_ids;
  std::vector<Program> programs;
  std::vector<uint32_t> free_program_ids;
  std::unordered_map<uint64_t, cudaEvent_t> events;
  uint64_t next_event = 1;
  // freed blocks by capacity; `ready` was recorded on the compute stream when the block was freed (after the copy and comm
  // streams had been ordered before it): whoever reuses the block on another stream waits for it first
  struct CachedBlock { void* ptr; cudaEvent_t ready; };
  std::multimap<uint64_t, CachedBlock> cache;
  uint64_t cached_bytes = 0;
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  uint32_t* status_word = nullptr;
  void* flush_buf = nullptr;
  size_t flush_bytes = 0;
  uint64_t launch_count = 0;
  void* tma_encode = nullptr;
  void* tma_encode_im2col = nullptr;
  Comm* comm = nullptr;
  PeerComm* peer = nullptr;               // allreduce over peer memory (peer_allreduce.cu); created with the communicator
  int comm_latency = 0;                   // ZYXB_COMM_OPT_LATENCY: allreduces take the communicator's own path
  // captured launch sequences (the analogue of a FrozenTape): executable graph + kernels per replay
  std::vector<std::pair<cudaGraphExec_t, uint64_t>> graphs;
  bool capturing = false;
  uint64_t capture_launch_base = 0;
};

std::string g_init_error;

}  // namespace

struct zyxb_ctx {
  std::vector<Device> devs;
  std::string last_error;
  bool round_nearest = false;
  int debug = 0;
  bool guards = false;     // debug bit 2: every allocation carries guard words behind its last byte (zyxb_check_guards)
  std::unordered_map<void*, int> registered;   // page-locked host ranges
};

namespace {

int fail(zyxb_ctx* ctx, int status, const std::string& msg) {
  if (ctx) ctx->last_error = msg; else g_init_error = msg;
  return status;
}
int cuda_fail(zyxb_ctx* ctx, int status, const char* what, cudaError_t e) {
  return fail(ctx, status, std::string(what) + ": " + cudaGetErrorString(e));
}

// Inside a capture (zyxb_capture_begin .. zyxb_capture_end) only launches without wait lists and memsets are recorded; calls
// that allocate, copy to or from the host, or block would invalidate the capture with an opaque CUDA error, so they are refused.
#define NOT_WHILE_CAPTURING(name, status) \
  if (D.capturing) return fail(ctx, status, std::string(name) + ": not allowed between zyxb_capture_begin and zyxb_capture_end")

#define DEV_OR_FAIL(status)                                                              \
  if (!ctx) return ZYXB_ERR_INITIALIZATION;                                              \
  if (dev < 0 || dev >= (int)ctx->devs.size()) return fail(ctx, status, "no such device"); \
  Device& D = ctx->devs[dev];                                                            \
  { cudaError_t e_ = cudaSetDevice(D.cuda_id); if (e_ != cudaSuccess) return cuda_fail(ctx, status, "cudaSetDevice", e_); }

Buffer* get_buffer(Device& D, uint32_t id) {
  if (id >= D.buffers.size() || !D.buffers[id].live) return nullptr;
  return &D.buffers[id];
}

uint64_t round_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

// Guard words (zyxb_config.debug bit 2): the stand-in for a memory checker on machines where none may run.  Every pool
// allocation is followed by at least GUARD_BYTES of a fixed pattern; a kernel that writes past the end of an output (the
// reference gives every buffer a spare trailing element for the same reason, zyx/src/runtime.rs:622-625) destroys it, and
// zyxb_check_guards finds the buffer.
constexpr uint64_t GUARD_BYTES = 256;
constexpr int GUARD_PATTERN = 0xC5;

// [offset, offset + bytes) lies inside [0, limit), without letting offset + bytes wrap around
bool range_ok(uint64_t offset, uint64_t bytes, uint64_t limit) { return offset <= limit && bytes <= limit - offset; }
// (offset + count) * es <= limit for element counts supplied by the caller
bool elems_ok(uint64_t offset, uint64_t count, uint64_t es, uint64_t limit) {
  uint64_t sum = 0, bytes = 0;
  return !__builtin_add_overflow(offset, count, &sum) && !__builtin_mul_overflow(sum, es, &bytes) && bytes <= limit;
}

// Events named in a wait list are consumed: the stream waits for them and they are destroyed,
// as zyx moves `Vec<Event>` into the backend call.
int wait_and_consume(zyxb_ctx* ctx, Device& D, cudaStream_t stream, const zyxb_event* wait, int n, int status) {
  for (int i = 0; i < n; ++i) {
    if (wait[i].id == 0) continue;
    auto it = D.events.find(wait[i].id);
    if (it == D.events.end()) return fail(ctx, status, "unknown event in wait list");
    cudaError_t e = cudaStreamWaitEvent(stream, it->second, 0);
    cudaEventDestroy(it->second);
    D.events.erase(it);
    if (e != cudaSuccess) return cuda_fail(ctx, status, "cudaStreamWaitEvent", e);
  }
  return ZYXB_OK;
}

int record_event(zyxb_ctx* ctx, Device& D, cudaStream_t stream, zyxb_event* out, int status, bool timing = false) {
  if (!out) return ZYXB_OK;
  cudaEvent_t ev;
  cudaError_t e = cudaEventCreateWithFlags(&ev, timing ? cudaEventDefault : cudaEventDisableTiming);
  if (e != cudaSuccess) return cuda_fail(ctx, status, "cudaEventCreate", e);
  e = cudaEventRecord(ev, stream);
  if (e != cudaSuccess) { cudaEventDestroy(ev); return cuda_fail(ctx, status, "cudaEventRecord", e); }
  out->id = D.next_event++;
  D.events[out->id] = ev;
  return ZYXB_OK;
}

// make `later` wait for everything enqueued on `earlier` so far
int order_streams(zyxb_ctx* ctx, cudaStream_t earlier, cudaStream_t later, int status) {
  cudaEvent_t ev;
  cudaError_t e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
  if (e != cudaSuccess) return cuda_fail(ctx, status, "cudaEventCreate", e);
  cudaEventRecord(ev, earlier);
  e = cudaStreamWaitEvent(later, ev, 0);
  cudaEventDestroy(ev);
  if (e != cudaSuccess) return cuda_fail(ctx, status, "cudaStreamWaitEvent", e);
  return ZYXB_OK;
}

cudaError_t device_malloc(Device& D, uint64_t capacity, void** out) {
  auto it = D.cache.lower_bound(capacity);
  // reuse a cached block when it is not wastefully larger than the request
  if (it != D.cache.end() && it->first <= capacity + capacity / 4 + (1u << 20)) {
    *out = it->second.ptr;
    if (it->second.ready) {
      // kernels queued before the free may still use the block: uploads (copy stream) and collectives (comm stream) into
      // its new owner go behind them; the compute stream is in order by itself
      cudaStreamWaitEvent(D.copy, it->second.ready, 0);
      cudaStreamWaitEvent(D.comm_stream, it->second.ready, 0);
      cudaEventDestroy(it->second.ready);
    }
    D.cached_bytes -= it->first;
    D.cache.erase(it);
    return cudaSuccess;
  }
  cudaError_t e = cudaMalloc(out, capacity);
  if (e == cudaErrorMemoryAllocation) {
    cudaGetLastError();
    for (auto& kv : D.cache) { if (kv.second.ready) cudaEventDestroy(kv.second.ready); cudaFree(kv.second.ptr); }   // give the cache back and retry once
    D.cache.clear(); D.cached_bytes = 0;
    e = cudaMalloc(out, capacity);
  }
  return e;
}

LaunchCtx make_launch_ctx(zyxb_ctx* ctx, Device& D) {
  LaunchCtx lc{};
  lc.stream = D.compute; lc.round_nearest = ctx->round_nearest; lc.sm_count = D.prop.multiProcessorCount;
  lc.status_word = D.status_word; lc.scratch = D.scratch; lc.scratch_bytes = D.scratch_bytes;
  lc.launch_counter = &D.launch_count; lc.tma_encode = D.tma_encode; lc.tma_encode_im2col = D.tma_encode_im2col; lc.device = D.cuda_id; lc.overlap_hint = D.comm != nullptr && !peer_usable(D.peer);   // NCCL's kernels take SMs away; the copy-engine allreduce does not
  return lc;
}

}  // namespace

extern "C" {
#pragma GCC visibility push(default)

const char* zyxb_last_error(zyxb_ctx* ctx) { return ctx ? ctx->last_error.c_str() : g_init_error.c_str(); }

int32_t zyxb_init(const zyxb_config* config, zyxb_ctx** out_ctx) {
  if (!out_ctx) return fail(nullptr, ZYXB_ERR_INITIALIZATION, "out_ctx is null");
  *out_ctx = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) {
    cudaGetLastError();
    return fail(nullptr, ZYXB_ERR_DEVICE_ENUMERATION,
                std::string("no CUDA device: ") + (e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0") +
                    " (this backend has no CPU fallback)");
  }
  std::vector<int> ids;
  if (config && config->n_device_ids > 0) {
    for (int i = 0; i < config->n_device_ids && i < 16; ++i) {
      if (config->device_ids[i] < 0 || config->device_ids[i] >= count) return fail(nullptr, ZYXB_ERR_DEVICE_ENUMERATION, "device id out of range");
      ids.push_back(config->device_ids[i]);
    }
  } else {
    for (int i = 0; i < count; ++i) ids.push_back(i);
  }
  zyxb_ctx* ctx = new zyxb_ctx();
  ctx->round_nearest = config && config->round_nearest;
  ctx->debug = config ? config->debug : 0;
  ctx->guards = (ctx->debug & 2) != 0;
  for (int id : ids) {
    Device D;
    D.cuda_id = id;
    if ((e = cudaSetDevice(id)) != cudaSuccess || (e = cudaGetDeviceProperties(&D.prop, id)) != cudaSuccess) {
      delete ctx; return cuda_fail(nullptr, ZYXB_ERR_DEVICE_QUERY, "device query", e);
    }
    if (D.prop.major != 10) {   // kernels are built for sm_100a only
      if (config && config->n_device_ids > 0) { delete ctx; return fail(nullptr, ZYXB_ERR_INITIALIZATION, "device is not compute capability 10.x (B200)"); }
      continue;
    }
    if ((e = cudaStreamCreateWithFlags(&D.compute, cudaStreamNonBlocking)) != cudaSuccess ||
        (e = cudaStreamCreateWithFlags(&D.copy, cudaStreamNonBlocking)) != cudaSuccess ||
        (e = cudaStreamCreateWithFlags(&D.comm_stream, cudaStreamNonBlocking)) != cudaSuccess) {
      delete ctx; return cuda_fail(nullptr, ZYXB_ERR_INITIALIZATION, "stream creation", e);
    }
    D.scratch_bytes = 320ull << 20;   // partials of split reductions, prepared operands of the f32 tensor-core matmul
    if ((e = cudaMalloc(&D.scratch, D.scratch_bytes)) != cudaSuccess || (e = cudaMalloc((void**)&D.status_word, 256)) != cudaSuccess) {
      delete ctx; return cuda_fail(nullptr, ZYXB_ERR_MEMORY_ALLOCATION, "scratch allocation", e);
    }
    cudaMemset(D.status_word, 0, 256);
    cudaDriverEntryPointQueryResult qres;
    void* fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      D.tma_encode = fn;
    else cudaGetLastError();
    fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      D.tma_encode_im2col = fn;
    else cudaGetLastError();
    D.buffers.emplace_back();   // id 0 is never handed out
    D.programs.emplace_back();
    if (ctx->debug & 1) fprintf(stderr, "[zyxb] device %d: %s, %d SMs, %.1f GB\n", id, D.prop.name, D.prop.multiProcessorCount, D.prop.totalGlobalMem / 1e9);
    ctx->devs.push_back(std::move(D));
  }
  if (ctx->devs.empty()) { delete ctx; return fail(nullptr, ZYXB_ERR_DEVICE_ENUMERATION, "no compute capability 10.x (B200) device found"); }
  *out_ctx = ctx;
  return ZYXB_OK;
}

int32_t zyxb_shutdown(zyxb_ctx* ctx) {
  if (!ctx) return ZYXB_OK;
  for (auto& D : ctx->devs) {
    cudaSetDevice(D.cuda_id);
    cudaDeviceSynchronize();
    if (D.peer) { peer_destroy(D.peer); D.peer = nullptr; }
    if (D.comm) { comm_destroy(D.comm); D.comm = nullptr; }
    for (auto& g : D.graphs) if (g.first) cudaGraphExecDestroy(g.first);
    for (auto& kv : D.events) cudaEventDestroy(kv.second);
    for (auto& b : D.buffers) if (b.live && b.ptr && !b.is_view && !b.is_variable) cudaFree(b.ptr);
    for (auto& kv : D.cache) { if (kv.second.ready) cudaEventDestroy(kv.second.ready); cudaFree(kv.second.ptr); }
    if (D.scratch) cudaFree(D.scratch);
    if (D.status_word) cudaFree(D.status_word);
    if (D.flush_buf) cudaFree(D.flush_buf);
    cudaStreamDestroy(D.compute); cudaStreamDestroy(D.copy); cudaStreamDestroy(D.comm_stream);
  }
  for (auto& kv : ctx->registered) cudaHostUnregister(kv.first);
  delete ctx;
  return ZYXB_OK;
}

int32_t zyxb_device_count(zyxb_ctx* ctx, int32_t* out_count) {
  if (!ctx || !out_count) return ZYXB_ERR_DEVICE_ENUMERATION;
  *out_count = (int32_t)ctx->devs.size();
  return ZYXB_OK;
}

int32_t zyxb_device_info(zyxb_ctx* ctx, int32_t dev, zyxb_devinfo* o) {
  DEV_OR_FAIL(ZYXB_ERR_DEVICE_QUERY);
  if (!o) return fail(ctx, ZYXB_ERR_DEVICE_QUERY, "out_info is null");
  memset(o, 0, sizeof(*o));
  o->compute_flops = 2250000000000000ull;   // dense bf16 tensor-core peak of a B200
  for (int i = 0; i < 3; ++i) { o->max_global_work_dims[i] = (uint64_t)D.prop.maxGridSize[i]; o->max_local_work_dims[i] = (uint32_t)D.prop.maxThreadsDim[i]; }
  o->max_local_threads = (uint32_t)D.prop.maxThreadsPerBlock;
  o->preferred_vector_size = 16;
  o->local_mem_size = D.prop.sharedMemPerBlockOptin;
  o->max_register_bytes = (uint64_t)D.prop.regsPerBlock * 4;
  o->tensor_cores = 1;
  o->warp_size = (uint32_t)D.prop.warpSize;
  // every elementwise/reduce capability bit for the dtypes the kernels accept
  for (int dt : {ZYXB_BF16, ZYXB_F16, ZYXB_F32}) o->dtype_capability[dt] = 0x7fffffffu;
  o->dtype_capability[ZYXB_I32] = 0x7fffffffu;
  o->has_native_exp2 = 1;
  o->sm_count = (uint32_t)D.prop.multiProcessorCount;
  o->total_mem_bytes = D.prop.totalGlobalMem;
  o->cc_major = D.prop.major; o->cc_minor = D.prop.minor;
  strncpy(o->name, D.prop.name, sizeof(o->name) - 1);
  return ZYXB_OK;
}

int32_t zyxb_free_compute(zyxb_ctx* ctx, int32_t dev, uint64_t* out_flops) {
  DEV_OR_FAIL(ZYXB_ERR_DEVICE_QUERY);
  if (out_flops) *out_flops = 2250000000000000ull;
  return ZYXB_OK;
}

int32_t zyxb_free_bytes(zyxb_ctx* ctx, int32_t dev, uint64_t* out_bytes) {
  DEV_OR_FAIL(ZYXB_ERR_DEVICE_QUERY);
  size_t fr = 0, total = 0;
  cudaError_t e = cudaMemGetInfo(&fr, &total);
  if (e != cudaSuccess) return cuda_fail(ctx, ZYXB_ERR_DEVICE_QUERY, "cudaMemGetInfo", e);
  if (out_bytes) *out_bytes = (uint64_t)fr + D.cached_bytes;
  return ZYXB_OK;
}

int32_t zyxb_alloc(zyxb_ctx* ctx, int32_t dev, uint64_t bytes, uint32_t* out_buf, zyxb_event* out_event) {
  DEV_OR_FAIL(ZYXB_ERR_MEMORY_ALLOCATION);
  if (!out_buf) return fail(ctx, ZYXB_ERR_MEMORY_ALLOCATION, "out_buf is null");
  NOT_WHILE_CAPTURING("zyxb_alloc", ZYXB_ERR_MEMORY_ALLOCATION);
  const uint64_t capacity = round_up((bytes == 0 ? 1 : bytes) + (ctx->guards ? GUARD_BYTES : 0), 512);
  void* ptr = nullptr;
  cudaError_t e = device_malloc(D, capacity, &ptr);
  if (e != cudaSuccess) { cudaGetLastError(); return cuda_fail(ctx, ZYXB_ERR_MEMORY_ALLOCATION, "cudaMalloc", e); }
  if (ctx->guards && (e = cudaMemsetAsync((char*)ptr + bytes, GUARD_PATTERN, capacity - bytes, D.compute)) != cudaSuccess)
    return cuda_fail(ctx, ZYXB_ERR_MEMORY_ALLOCATION, "guard words", e);
  uint32_t id;
  if (!D.free_buffer_ids.empty()) { id = D.free_buffer_ids.back(); D.free_buffer_ids.pop_back(); }
  else { id = (uint32_t)D.buffers.size(); D.buffers.emplace_back(); }
  Buffer& b = D.buffers[id];
  b = Buffer();
  b.ptr = ptr; b.bytes = bytes; b.capacity = capacity; b.live = true;
  *out_buf = id;
  if (out_event) out_event->id = 0;   // allocation is synchronous: nothing to wait for
  return ZYXB_OK;
}

int32_t zyxb_free(zyxb_ctx* ctx, int32_t dev, uint32_t buf, const zyxb_event* wait, int32_t n_wait) {
  DEV_OR_FAIL(ZYXB_ERR_MEMORY_DEALLOCATION);
  Buffer* b = get_buffer(D, buf);
  if (!b) return fail(ctx, ZYXB_ERR_MEMORY_DEALLOCATION, "free: unknown buffer");
  NOT_WHILE_CAPTURING("zyxb_free", ZYXB_ERR_MEMORY_DEALLOCATION);
  // the block goes back to the cache and may be handed out again at once: order every stream
  // that could still touch it before later work on the compute stream
  int st = wait_and_consume(ctx, D, D.compute, wait, n_wait, ZYXB_ERR_MEMORY_DEALLOCATION);
  if (st) return st;
  if (!b->is_variable && !b->is_view && peer_has_exported(D.peer, b->ptr)) {
    // other processes have this block mapped: it is not recycled (a new owner would inherit their mappings); everything that
    // may still touch it finishes first, then the mappings held here are closed and the block goes back to the driver
    cudaDeviceSynchronize();
    peer_forget_buffer(D.peer, b->ptr);
    cudaFree(b->ptr);
  } else if (!b->is_variable && !b->is_view) {
    if ((st = order_streams(ctx, D.copy, D.compute, ZYXB_ERR_MEMORY_DEALLOCATION))) return st;
    if ((st = order_streams(ctx, D.comm_stream, D.compute, ZYXB_ERR_MEMORY_DEALLOCATION))) return st;
    cudaEvent_t ready = nullptr;
    if (cudaEventCreateWithFlags(&ready, cudaEventDisableTiming) != cudaSuccess || cudaEventRecord(ready, D.compute) != cudaSuccess) {
      cudaGetLastError();
      if (ready) { cudaEventDestroy(ready); ready = nullptr; }
      cudaStreamSynchronize(D.compute);      // no event to hand on: the block is idle before it enters the cache
    }
    D.cache.emplace(b->capacity, Device::CachedBlock{b->ptr, ready});
    D.cached_bytes += b->capacity;
  }
  *b = Buffer();
  D.free_buffer_ids.push_back(buf);
  return ZYXB_OK;
}

int32_t zyxb_buffer_view(zyxb_ctx* ctx, int32_t dev, uint32_t parent, uint64_t offset, uint64_t bytes, uint32_t* out_buf) {
  DEV_OR_FAIL(ZYXB_ERR_MEMORY_ALLOCATION);
  Buffer* pb = get_buffer(D, parent);
  if (!pb || pb->is_variable || !out_buf) return fail(ctx, ZYXB_ERR_MEMORY_ALLOCATION, "buffer_view: unknown parent buffer");
  if (offset % 256 != 0) return fail(ctx, ZYXB_ERR_MEMORY_ALLOCATION, "buffer_view: offset must be a multiple of 256 bytes");
  if (!range_ok(offset, bytes, pb->bytes)) return fail(ctx, ZYXB_ERR_MEMORY_ALLOCATION, "buffer_view: range exceeds the parent");
  void* ptr = (char*)pb->ptr + offset;
  uint32_t id;
  if (!D.free_buffer_ids.empty()) { id = D.free_buffer_ids.back(); D.free_buffer_ids.pop_back(); }
  else { id = (uint32_t)D.buffers.size(); D.buffers.emplace_back(); }
  Buffer& b = D.buffers[id];
  b = Buffer();
  b.ptr = ptr; b.bytes = bytes; b.capacity = bytes; b.live = true; b.is_view = true;
  b.parent = D.buffers[parent].is_view ? D.buffers[parent].parent : parent;
  *out_buf = id;
  return ZYXB_OK;
}

int32_t zyxb_buffer_bytes(zyxb_ctx* ctx, int32_t dev, uint32_t buf, uint64_t* out_bytes) {
  DEV_OR_FAIL(ZYXB_ERR_INCORRECT_KERNEL_ARG);
  Buffer* b = get_buffer(D, buf);
  if (!b) return fail(ctx, ZYXB_ERR_INCORRECT_KERNEL_ARG, "unknown buffer");
  if (out_bytes) *out_bytes = b->bytes;
  return ZYXB_OK;
}

int32_t zyxb_h2d(zyxb_ctx* ctx, int32_t dev, const void* src, uint64_t bytes, uint32_t dst, uint64_t dst_offset,
                 const zyxb_event* wait, int32_t n_wait, zyxb_event* out_event) {
  DEV_OR_FAIL(ZYXB_ERR_MEMORY_COPY_H2P);
  Buffer* b = get_buffer(D, dst);
  if (!b || b->is_variable) return fail(ctx, ZYXB_ERR_MEMORY_COPY_H2P, "h2d: unknown buffer");
  if (!range_ok(dst_offset, bytes, b->bytes)) return fail(ctx, ZYXB_ERR_MEMORY_COPY_H2P, "h2d: copy exceeds the buffer");
  NOT_WHILE_CAPTURING("zyxb_h2d", ZYXB_ERR_MEMORY_COPY_H2P);
  int st = wait_and_consume(ctx, D, D.copy, wait, n_wait, ZYXB_ERR_MEMORY_COPY_H2P);
  if (st) return st;
  // With a wait list the caller has named what the upload depends on, as zyx does (it passes the events of
  // every pending use of dst), and the copy may overlap kernels already queued.  Without one, kernels
  // already enqueued may still read or write dst: the upload goes after them.
  int named = 0;
  for (int i = 0; i < n_wait; ++i) named += wait[i].id != 0;      // null events (e.g. the one zyxb_alloc returns) name nothing
  if (named == 0 && (st = order_streams(ctx, D.compute, D.copy, ZYXB_ERR_MEMORY_COPY_H2P))) return st;
  if (bytes) {
    cudaError_t e = cudaMemcpyAsync((char*)b->ptr + dst_offset, src, bytes, cudaMemcpyHostToDevice, D.copy);
    if (e != cudaSuccess) return cuda_fail(ctx, ZYXB_ERR_MEMORY_COPY_H2P, "cudaMemcpyAsync h2d", e);
  }
  if (out_event) return record_event(ctx, D, D.copy, out_event, ZYXB_ERR_MEMORY_COPY_H2P);
  // no event requested: later kernels must still see the data
  return order_streams(ctx, D.copy, D.compute, ZYXB_ERR_MEMORY_COPY_H2P);
}

int32_t zyxb_d2h(zyxb_ctx* ctx, int32_t dev, uint32_t src, uint64_t src_offset, void* dst, uint64_t bytes,
                 const zyxb_event* wait, int32_t n_wait) {
  DEV_OR_FAIL(ZYXB_ERR_MEMORY_COPY_P2H);
  Buffer* b = get_buffer(D, src);
  if (!b || b->is_variable) return fail(ctx, ZYXB_ERR_MEMORY_COPY_P2H, "d2h: unknown buffer");
  if (!range_ok(src_offset, bytes, b->bytes)) return fail(ctx, ZYXB_ERR_MEMORY_COPY_P2H, "d2h: copy exceeds the buffer");
  NOT_WHILE_CAPTURING("zyxb_d2h", ZYXB_ERR_MEMORY_COPY_P2H);
  int st = wait_and_consume(ctx, D, D.compute, wait, n_wait, ZYXB_ERR_MEMORY_COPY_P2H);
  if (st) return st;
  cudaError_t e = cudaSuccess;
  if (bytes) e = cudaMemcpyAsync(dst, (const char*)b->ptr + src_offset, bytes, cudaMemcpyDeviceToHost, D.compute);
  if (e == cudaSuccess) e = cudaStreamSynchronize(D.compute);
  if (e != cudaSuccess) return cuda_fail(ctx, ZYXB_ERR_MEMORY_COPY_P2H, "d2h", e);
  return ZYXB_OK;
}

int32_t zyxb_d2d(zyxb_ctx* ctx, int32_t src_dev, uint32_t src, uint64_t src_offset, int32_t dev, uint32_t dst, uint64_t dst_offset,
                 uint64_t bytes, const zyxb_event* wait, int32_t n_wait, zyxb_event* out_event) {
  DEV_OR_FAIL(ZYXB_ERR_MEMORY_COPY_H2P);
  if (src_dev < 0 || src_dev >= (int)ctx->devs.size()) return fail(ctx, ZYXB_ERR_MEMORY_COPY_H2P, "d2d: no such source device");
  NOT_WHILE_CAPTURING("zyxb_d2d", ZYXB_ERR_MEMORY_COPY_H2P);
  Device& SD = ctx->devs[src_dev];
  Buffer* sb = get_buffer(SD, src);
  Buffer* db = get_buffer(D, dst);
  if (!sb || !db || sb->is_variable || db->is_variable) return fail(ctx, ZYXB_ERR_MEMORY_COPY_H2P, "d2d: unknown buffer");
  if (!range_ok(src_offset, bytes, sb->bytes) || !range_ok(dst_offset, bytes, db->bytes)) return fail(ctx, ZYXB_ERR_MEMORY_COPY_H2P, "d2d: copy exceeds a buffer");
  int st = wait_and_consume(ctx, D, D.compute, wait, n_wait, ZYXB_ERR_MEMORY_COPY_H2P);
  if (st) return st;
  cudaError_t e = cudaSuccess;
  if (src_dev == dev) e = cudaMemcpyAsync((char*)db->ptr + dst_offset, (const char*)sb->ptr + src_offset, bytes, cudaMemcpyDeviceToDevice, D.compute);
  else {
    if ((st = order_streams(ctx, SD.compute, D.compute, ZYXB_ERR_MEMORY_COPY_H2P))) return st;
    e = cudaMemcpyPeerAsync((char*)db->ptr + dst_offset, D.cuda_id, (const char*)sb->ptr + src_offset, SD.cuda_id, bytes, D.compute);
  }
  if (e != cudaSuccess) return cuda_fail(ctx, ZYXB_ERR_MEMORY_COPY_H2P, "d2d", e);
  return record_event(ctx, D, D.compute, out_event, ZYXB_ERR_MEMORY_COPY_H2P);
}

int32_t zyxb_memset(zyxb_ctx* ctx, int32_t dev, uint32_t buf, uint64_t offset, int32_t byte_value, uint64_t bytes) {
  DEV_OR_FAIL(ZYXB_ERR_MEMORY_COPY_H2P);
  Buffer* b = get_buffer(D, buf);
  if (!b || b->is_variable) return fail(ctx, ZYXB_ERR_MEMORY_COPY_H2P, "memset: unknown buffer");
  if (!range_ok(offset, bytes, b->bytes)) return fail(ctx, ZYXB_ERR_MEMORY_COPY_H2P, "memset: range exceeds the buffer");
  cudaError_t e = cudaMemsetAsync((char*)b->ptr + offset, byte_value, bytes, D.compute);
  if (e != cudaSuccess) return cuda_fail(ctx, ZYXB_ERR_MEMORY_COPY_H2P, "cudaMemsetAsync", e);
  return ZYXB_OK;
}

int32_t zyxb_sync(zyxb_ctx* ctx, int32_t dev, const zyxb_event* events, int32_t n) {
  DEV_OR_FAIL(ZYXB_ERR_KERNEL_SYNC);
  NOT_WHILE_CAPTURING("zyxb_sync", ZYXB_ERR_KERNEL_SYNC);
  int status = ZYXB_OK;
  for (int i = 0; i < n; ++i) {
    if (events[i].id == 0) continue;
    auto it = D.events.find(events[i].id);
    if (it == D.events.end()) { status = fail(ctx, ZYXB_ERR_KERNEL_SYNC, "sync: unknown event"); continue; }
    cudaError_t e = cudaEventSynchronize(it->second);
    cudaEventDestroy(it->second);
    D.events.erase(it);
    if (e != cudaSuccess) status = cuda_fail(ctx, ZYXB_ERR_KERNEL_SYNC, "cudaEventSynchronize", e);
  }
  return status;
}

int32_t zyxb_release_events(zyxb_ctx* ctx, int32_t dev, const zyxb_event* events, int32_t n) {
  DEV_OR_FAIL(ZYXB_ERR_KERNEL_SYNC);
  for (int i = 0; i < n; ++i) {
    auto it = D.events.find(events[i].id);
    if (it == D.events.end()) continue;
    cudaEventDestroy(it->second);
    D.events.erase(it);
  }
  return ZYXB_OK;
}

int32_t zyxb_device_sync(zyxb_ctx* ctx, int32_t dev) {
  DEV_OR_FAIL(ZYXB_ERR_KERNEL_SYNC);
  NOT_WHILE_CAPTURING("zyxb_device_sync", ZYXB_ERR_KERNEL_SYNC);
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return cuda_fail(ctx, ZYXB_ERR_KERNEL_SYNC, "cudaDeviceSynchronize", e);
  return ZYXB_OK;
}

int32_t zyxb_store_variable(zyxb_ctx* ctx, int32_t dev, int32_t dtype, const void* le_bytes, uint32_t* out_buf) {
  DEV_OR_FAIL(ZYXB_ERR_MEMORY_ALLOCATION);
  if (!le_bytes || !out_buf || dtype < 0 || dtype > ZYXB_BOOL) return fail(ctx, ZYXB_ERR_MEMORY_ALLOCATION, "store_variable: bad argument");
  uint32_t id;
  if (!D.free_buffer_ids.empty()) { id = D.free_buffer_ids.back(); D.free_buffer_ids.pop_back(); }
  else { id = (uint32_t)D.buffers.size(); D.buffers.emplace_back(); }
  Buffer& b = D.buffers[id];
  b = Buffer();
  b.live = true; b.is_variable = true; b.var_dtype = dtype; b.bytes = dtype_size(dtype);
  memcpy(b.var_bytes, le_bytes, b.bytes);
  *out_buf = id;
  return ZYXB_OK;
}

int32_t zyxb_get_variable(zyxb_ctx* ctx, int32_t dev, uint32_t buf, int32_t* out_dtype, void* out_le_bytes) {
  DEV_OR_FAIL(ZYXB_ERR_INCORRECT_KERNEL_ARG);
  Buffer* b = get_buffer(D, buf);
  if (!b || !b->is_variable) return fail(ctx, ZYXB_ERR_INCORRECT_KERNEL_ARG, "get_variable: not a variable");
  if (out_dtype) *out_dtype = b->var_dtype;
  if (out_le_bytes) memcpy(out_le_bytes, b->var_bytes, b->bytes);
  return ZYXB_OK;
}

int32_t zyxb_host_register(zyxb_ctx* ctx, void* ptr, uint64_t bytes) {
  if (!ctx) return ZYXB_ERR_INITIALIZATION;
  cudaSetDevice(ctx->devs[0].cuda_id);
  cudaError_t e = cudaHostRegister(ptr, bytes, cudaHostRegisterPortable);
  if (e != cudaSuccess) { cudaGetLastError(); return cuda_fail(ctx, ZYXB_ERR_MEMORY_ALLOCATION, "cudaHostRegister", e); }
  ctx->registered[ptr] = 1;
  return ZYXB_OK;
}

int32_t zyxb_host_unregister(zyxb_ctx* ctx, void* ptr) {
  if (!ctx) return ZYXB_ERR_INITIALIZATION;
  auto it = ctx->registered.find(ptr);
  if (it == ctx->registered.end()) return fail(ctx, ZYXB_ERR_MEMORY_DEALLOCATION, "host_unregister: range was not registered");
  cudaSetDevice(ctx->devs[0].cuda_id);
  cudaDeviceSynchronize();
  cudaHostUnregister(ptr);
  ctx->registered.erase(it);
  return ZYXB_OK;
}

// ---- programs --------------------------------------------------------------------------------
int32_t zyxb_program_create(zyxb_ctx* ctx, int32_t dev, const zyxb_kernel_desc* desc, uint32_t* out_prog) {
  DEV_OR_FAIL(ZYXB_ERR_KERNEL_COMPILATION);
  if (!desc || !out_prog) return fail(ctx, ZYXB_ERR_KERNEL_COMPILATION, "program_create: null argument");
  std::string err;
  int st;
  switch (desc->kind) {
    case ZYXB_KIND_ROWREDUCE: st = validate_rowreduce(desc->u.rowreduce, err); break;
    case ZYXB_KIND_GEMM: st = validate_gemm(desc->u.gemm, err); break;
    case ZYXB_KIND_ELTWISE: st = validate_eltwise(desc->u.eltwise, err); break;
    case ZYXB_KIND_OPTIM: st = validate_optim(desc->u.optim, err); break;
    case ZYXB_KIND_ATTENTION: case ZYXB_KIND_ATTENTION_BWD: st = validate_attention(desc->u.attention, err); break;
    case ZYXB_KIND_CONV: case ZYXB_KIND_CONV_WGRAD: case ZYXB_KIND_CONV_DGRAD: st = validate_conv(desc->u.conv, err); break;
    default: st = ZYXB_ERR_KERNEL_COMPILATION; err = "unknown kernel kind";
  }
  if (st) return fail(ctx, st, err);
  uint32_t id;
  if (!D.free_program_ids.empty()) { id = D.free_program_ids.back(); D.free_program_ids.pop_back(); }
  else { id = (uint32_t)D.programs.size(); D.programs.emplace_back(); }
  Program& P = D.programs[id];
  P = Program();
  P.desc = *desc; P.live = true;
  if (desc->kind == ZYXB_KIND_OPTIM) {
    P.numel.assign(desc->u.optim.numel, desc->u.optim.numel + desc->u.optim.n_tensors);
    P.desc.u.optim.numel = nullptr;   // the caller's array need not outlive this call
  }
  *out_prog = id;
  return ZYXB_OK;
}

int32_t zyxb_program_release(zyxb_ctx* ctx, int32_t dev, uint32_t prog) {
  DEV_OR_FAIL(ZYXB_ERR_KERNEL_COMPILATION);
  if (prog == 0 || prog >= D.programs.size() || !D.programs[prog].live) return fail(ctx, ZYXB_ERR_KERNEL_COMPILATION, "release: unknown program");
  D.programs[prog] = Program();
  D.free_program_ids.push_back(prog);
  return ZYXB_OK;
}

int32_t zyxb_program_set_step(zyxb_ctx* ctx, int32_t dev, uint32_t prog, uint64_t t) {
  DEV_OR_FAIL(ZYXB_ERR_INCORRECT_KERNEL_ARG);
  if (prog == 0 || prog >= D.programs.size() || !D.programs[prog].live || D.programs[prog].desc.kind != ZYXB_KIND_OPTIM)
    return fail(ctx, ZYXB_ERR_INCORRECT_KERNEL_ARG, "set_step: not an optimizer program");
  D.programs[prog].step = t;
  return ZYXB_OK;
}

int32_t zyxb_program_get_step(zyxb_ctx* ctx, int32_t dev, uint32_t prog, uint64_t* out_t) {
  DEV_OR_FAIL(ZYXB_ERR_INCORRECT_KERNEL_ARG);
  if (!out_t || prog == 0 || prog >= D.programs.size() || !D.programs[prog].live || D.programs[prog].desc.kind != ZYXB_KIND_OPTIM)
    return fail(ctx, ZYXB_ERR_INCORRECT_KERNEL_ARG, "get_step: not an optimizer program");
  *out_t = D.programs[prog].step;
  return ZYXB_OK;
}

int32_t zyxb_launch(zyxb_ctx* ctx, int32_t dev, uint32_t prog, const uint32_t* args, int32_t n_args, const zyxb_event* wait,
                    int32_t n_wait, zyxb_event* out_event) {
  DEV_OR_FAIL(ZYXB_ERR_KERNEL_LAUNCH);
  if (prog == 0 || prog >= D.programs.size() || !D.programs[prog].live) return fail(ctx, ZYXB_ERR_KERNEL_LAUNCH, "launch: unknown program");
  if (n_args < 0 || n_args > 4096 || (n_args > 0 && !args)) return fail(ctx, ZYXB_ERR_INCORRECT_KERNEL_ARG, "launch: bad argument list");
  Program& P = D.programs[prog];
  if (D.capturing) {
    int named = 0;
    for (int i = 0; i < n_wait; ++i) named += wait[i].id != 0;
    if (named) return fail(ctx, ZYXB_ERR_KERNEL_LAUNCH, "launch: a wait list cannot be recorded into a capture");
    // A captured launch freezes its kernel parameters.  An update that depends on the step (the first-step test of a
    // momentum buffer, Adam's bias corrections) would replay the captured step for ever.
    if (P.desc.kind == ZYXB_KIND_OPTIM && (P.desc.u.optim.algo != ZYXB_OPT_SGD || P.desc.u.optim.momentum != 0.0f))
      return fail(ctx, ZYXB_ERR_KERNEL_LAUNCH, "launch: an optimizer whose update depends on the step counter (SGD with momentum, Adam, AdamW) "
                                               "cannot be captured; launch it after zyxb_graph_launch instead");
  }
  std::vector<void*> ptrs(n_args);
  std::vector<uint64_t> sizes(n_args);
  for (int i = 0; i < n_args; ++i) {
    Buffer* b = get_buffer(D, args[i]);
    if (!b || b->is_variable) return fail(ctx, ZYXB_ERR_INCORRECT_KERNEL_ARG, "launch: argument " + std::to_string(i) + " is not a pool buffer");
    ptrs[i] = b->ptr; sizes[i] = b->bytes;
  }
  int st = wait_and_consume(ctx, D, D.compute, wait, n_wait, ZYXB_ERR_KERNEL_LAUNCH);
  if (st) return st;
  LaunchCtx lc = make_launch_ctx(ctx, D);
  std::string err;
  switch (P.desc.kind) {
    case ZYXB_KIND_ROWREDUCE: st = launch_rowreduce(P.desc.u.rowreduce, ptrs.data(), sizes.data(), n_args, lc, err); break;
    case ZYXB_KIND_GEMM: st = launch_gemm(P.desc.u.gemm, ptrs.data(), sizes.data(), n_args, lc, err); break;
    case ZYXB_KIND_ELTWISE: st = launch_eltwise(P.desc.u.eltwise, ptrs.data(), sizes.data(), n_args, lc, err); break;
    case ZYXB_KIND_ATTENTION: st = launch_attention(P.desc.u.attention, ptrs.data(), sizes.data(), n_args, lc, err); break;
    case ZYXB_KIND_ATTENTION_BWD: st = launch_attention_bwd(P.desc.u.attention, ptrs.data(), sizes.data(), n_args, lc, err); break;
    case ZYXB_KIND_CONV: st = launch_conv(P.desc.u.conv, ptrs.data(), sizes.data(), n_args, lc, err); break;
    case ZYXB_KIND_CONV_DGRAD: st = launch_conv_dgrad(P.desc.u.conv, ptrs.data(), sizes.data(), n_args, lc, err); break;
    case ZYXB_KIND_CONV_WGRAD: st = launch_conv_wgrad(P.desc.u.conv, ptrs.data(), sizes.data(), n_args, lc, err); break;
    case ZYXB_KIND_OPTIM:
      st = launch_optim(P.desc.u.optim, P.numel.data(), P.step + 1, ptrs.data(), sizes.data(), n_args, lc, err);
      if (st == ZYXB_OK && !D.capturing) P.step += 1;     // a captured launch has not run
      break;
    default: st = ZYXB_ERR_KERNEL_LAUNCH; err = "launch: unknown kernel kind";
  }
  if (st) return fail(ctx, st, err);
  if (ctx->debug & 1) fprintf(stderr, "[zyxb] launch program %u kind %d\n", prog, P.desc.kind);
  return record_event(ctx, D, D.compute, out_event, ZYXB_ERR_KERNEL_LAUNCH);
}

int32_t zyxb_colsum_static(zyxb_ctx* ctx, int32_t dev, int32_t dtype, uint32_t x, uint32_t y, uint64_t rows, uint64_t cols) {
  DEV_OR_FAIL(ZYXB_ERR_KERNEL_LAUNCH);
  Buffer* bx = get_buffer(D, x);
  Buffer* by = get_buffer(D, y);
  if (!bx || !by || bx->is_variable || by->is_variable) return fail(ctx, ZYXB_ERR_INCORRECT_KERNEL_ARG, "colsum_static: unknown buffer");
  const uint64_t es = dtype_size(dtype);
  if (rows != 0 && cols > UINT64_MAX / rows / 8) return fail(ctx, ZYXB_ERR_INCORRECT_KERNEL_ARG, "colsum_static: shape overflows");
  if (D.capturing && !colsum_static_ready(D.cuda_id))
    return fail(ctx, ZYXB_ERR_KERNEL_LAUNCH, "colsum_static: the first call on a device looks up the array's address and cannot be captured; call it once during set-up");
  if (bx->bytes < rows * cols * es || by->bytes < cols * es) return fail(ctx, ZYXB_ERR_INCORRECT_KERNEL_ARG, "colsum_static: buffer too small");
  LaunchCtx lc = make_launch_ctx(ctx, D);
  std::string err;
  int st = launch_colsum_static(dtype, bx->ptr, by->ptr, rows, cols, lc, err);
  if (st) return fail(ctx, st, err);
  return ZYXB_OK;
}

int32_t zyxb_colsum_static_capacity(uint64_t* out_floats) {
  if (out_floats) *out_floats = colsum_static_capacity();
  return ZYXB_OK;
}

// ---- captured launch sequences ---------------------------------------------------------------------
int32_t zyxb_capture_begin(zyxb_ctx* ctx, int32_t dev) {
  DEV_OR_FAIL(ZYXB_ERR_KERNEL_LAUNCH);
  if (D.capturing) return fail(ctx, ZYXB_ERR_KERNEL_LAUNCH, "capture_begin: a capture is already open");
  cudaError_t e = cudaStreamBeginCapture(D.compute, cudaStreamCaptureModeThreadLocal);
  if (e != cudaSuccess) return cuda_fail(ctx, ZYXB_ERR_KERNEL_LAUNCH, "cudaStreamBeginCapture", e);
  D.capturing = true;
  D.capture_launch_base = D.launch_count;
  return ZYXB_OK;
}

int32_t zyxb_capture_end(zyxb_ctx* ctx, int32_t dev, uint32_t* out_graph) {
  DEV_OR_FAIL(ZYXB_ERR_KERNEL_LAUNCH);
  if (!D.capturing || !out_graph) return fail(ctx, ZYXB_ERR_KERNEL_LAUNCH, "capture_end: no capture is open");
  D.capturing = false;
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamEndCapture(D.compute, &graph);
  if (e != cudaSuccess || !graph) { cudaGetLastError(); return cuda_fail(ctx, ZYXB_ERR_KERNEL_LAUNCH, "cudaStreamEndCapture", e); }
  cudaGraphExec_t exec = nullptr;
  e = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) return cuda_fail(ctx, ZYXB_ERR_KERNEL_COMPILATION, "cudaGraphInstantiate", e);
  const uint64_t kernels = D.launch_count - D.capture_launch_base;
  D.launch_count = D.capture_launch_base;      // captured launches have not run yet; replays are counted
  D.graphs.emplace_back(exec, kernels);
  *out_graph = (uint32_t)D.graphs.size();      // ids start at 1
  return ZYXB_OK;
}

int32_t zyxb_graph_launch(zyxb_ctx* ctx, int32_t dev, uint32_t graph, const zyxb_event* wait, int32_t n_wait, zyxb_event* out_event) {
  DEV_OR_FAIL(ZYXB_ERR_KERNEL_LAUNCH);
  if (graph == 0 || graph > D.graphs.size() || !D.graphs[graph - 1].first) return fail(ctx, ZYXB_ERR_KERNEL_LAUNCH, "graph_launch: unknown graph");
  int st = wait_and_consume(ctx, D, D.compute, wait, n_wait, ZYXB_ERR_KERNEL_LAUNCH);
  if (st) return st;
  cudaError_t e = cudaGraphLaunch(D.graphs[graph - 1].first, D.compute);
  if (e != cudaSuccess) return cuda_fail(ctx, ZYXB_ERR_KERNEL_LAUNCH, "cudaGraphLaunch", e);
  D.launch_count += D.graphs[graph - 1].second;
  return record_event(ctx, D, D.compute, out_event, ZYXB_ERR_KERNEL_LAUNCH);
}

int32_t zyxb_graph_release(zyxb_ctx* ctx, int32_t dev, uint32_t graph) {
  DEV_OR_FAIL(ZYXB_ERR_KERNEL_LAUNCH);
  if (graph == 0 || graph > D.graphs.size() || !D.graphs[graph - 1].first) return fail(ctx, ZYXB_ERR_KERNEL_LAUNCH, "graph_release: unknown graph");
  cudaStreamSynchronize(D.compute);
  cudaGraphExecDestroy(D.graphs[graph - 1].first);
  D.graphs[graph - 1].first = nullptr;
  return ZYXB_OK;
}

int32_t zyxb_launch_count(zyxb_ctx* ctx, int32_t dev, uint64_t* out_count) {
  DEV_OR_FAIL(ZYXB_ERR_DEVICE_QUERY);
  if (out_count) *out_count = D.launch_count;
  return ZYXB_OK;
}

int32_t zyxb_device_status(zyxb_ctx* ctx, int32_t dev, uint32_t* out_status) {
  DEV_OR_FAIL(ZYXB_ERR_KERNEL_SYNC);
  uint32_t w = 0;
  cudaError_t e = cudaStreamSynchronize(D.compute);
  if (e == cudaSuccess) e = cudaMemcpy(&w, D.status_word, 4, cudaMemcpyDeviceToHost);
  if (e == cudaSuccess && w != 0) e = cudaMemset(D.status_word, 0, 4);
  if (e != cudaSuccess) return cuda_fail(ctx, ZYXB_ERR_KERNEL_SYNC, "device_status", e);
  if (out_status) *out_status = w;
  if (w != 0) return fail(ctx, ZYXB_ERR_KERNEL_SYNC, "a kernel gave up a bounded wait (status word " + std::to_string(w) + ")");
  return ZYXB_OK;
}

// A wait that nothing will ever satisfy, bounded by `limit_ns`: see selftest.cu.  The kernel's verdict goes to the second
// word of the status allocation, the timeout code to the status word itself (read and cleared by zyxb_device_status).
int32_t zyxb_selftest_bounded_wait(zyxb_ctx* ctx, int32_t dev, uint64_t limit_ns, uint32_t* out_gave_up) {
  DEV_OR_FAIL(ZYXB_ERR_KERNEL_LAUNCH);
  NOT_WHILE_CAPTURING("zyxb_selftest_bounded_wait", ZYXB_ERR_KERNEL_LAUNCH);
  LaunchCtx lc = make_launch_ctx(ctx, D);
  std::string err;
  uint32_t* verdict = D.status_word + 1;
  cudaError_t e = cudaMemsetAsync(verdict, 0xff, 4, D.compute);
  if (e != cudaSuccess) return cuda_fail(ctx, ZYXB_ERR_KERNEL_LAUNCH, "selftest", e);
  int st = launch_bounded_wait_selftest(limit_ns, verdict, lc, err);
  if (st) return fail(ctx, st, err);
  uint32_t w = 0;
  e = cudaMemcpyAsync(&w, verdict, 4, cudaMemcpyDeviceToHost, D.compute);
  if (e == cudaSuccess) e = cudaStreamSynchronize(D.compute);
  if (e != cudaSuccess) return cuda_fail(ctx, ZYXB_ERR_KERNEL_SYNC, "selftest", e);
  if (out_gave_up) *out_gave_up = w;
  return ZYXB_OK;
}

int32_t zyxb_check_guards(zyxb_ctx* ctx, int32_t dev, uint32_t* out_bad_buffer) {
  DEV_OR_FAIL(ZYXB_ERR_KERNEL_SYNC);
  NOT_WHILE_CAPTURING("zyxb_check_guards", ZYXB_ERR_KERNEL_SYNC);
  if (out_bad_buffer) *out_bad_buffer = 0;
  if (!ctx->guards) return fail(ctx, ZYXB_ERR_INCORRECT_KERNEL_ARG, "check_guards: the context was not opened with debug bit 2");
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return cuda_fail(ctx, ZYXB_ERR_KERNEL_SYNC, "check_guards", e);
  std::vector<uint8_t> host;
  for (uint32_t id = 1; id < D.buffers.size(); ++id) {
    const Buffer& b = D.buffers[id];
    if (!b.live || b.is_view || b.is_variable || b.capacity <= b.bytes) continue;
    host.resize(b.capacity - b.bytes);
    if ((e = cudaMemcpy(host.data(), (const char*)b.ptr + b.bytes, host.size(), cudaMemcpyDeviceToHost)) != cudaSuccess)
      return cuda_fail(ctx, ZYXB_ERR_KERNEL_SYNC, "check_guards", e);
    for (size_t i = 0; i < host.size(); ++i)
      if (host[i] != (uint8_t)GUARD_PATTERN) {
        if (out_bad_buffer) *out_bad_buffer = id;
        return fail(ctx, ZYXB_ERR_INCORRECT_KERNEL_ARG, "check_guards: buffer " + std::to_string(id) + " (" + std::to_string(b.bytes) +
                                                         " bytes) was written " + std::to_string(i) + " bytes past its end");
      }
  }
  return ZYXB_OK;
}

// ---- timing -------------------------------------------------------------------------------------
int32_t zyxb_event_record(zyxb_ctx* ctx, int32_t dev, zyxb_event* out_event) {
  DEV_OR_FAIL(ZYXB_ERR_KERNEL_SYNC);
  if (!out_event) return fail(ctx, ZYXB_ERR_KERNEL_SYNC, "event_record: null");
  return record_event(ctx, D, D.compute, out_event, ZYXB_ERR_KERNEL_SYNC, true);
}

int32_t zyxb_event_elapsed_ms(zyxb_ctx* ctx, int32_t dev, zyxb_event start, zyxb_event stop, float* out_ms) {
  DEV_OR_FAIL(ZYXB_ERR_KERNEL_SYNC);
  auto a = D.events.find(start.id), b = D.events.find(stop.id);
  if (a == D.events.end() || b == D.events.end()) return fail(ctx, ZYXB_ERR_KERNEL_SYNC, "event_elapsed: unknown event");
  cudaError_t e = cudaEventSynchronize(b->second);
  float ms = 0.0f;
  if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, a->second, b->second);
  if (e != cudaSuccess) return cuda_fail(ctx, ZYXB_ERR_KERNEL_SYNC, "cudaEventElapsedTime", e);
  if (out_ms) *out_ms = ms;
  return ZYXB_OK;
}

int32_t zyxb_flush_l2(zyxb_ctx* ctx, int32_t dev) {
  DEV_OR_FAIL(ZYXB_ERR_KERNEL_LAUNCH);
  if (!D.flush_buf) {
    D.flush_bytes = 256ull << 20;   // twice the 126 MB L2
    cudaError_t e = cudaMalloc(&D.flush_buf, D.flush_bytes);
    if (e != cudaSuccess) { cudaGetLastError(); D.flush_buf = nullptr; return cuda_fail(ctx, ZYXB_ERR_MEMORY_ALLOCATION, "flush buffer", e); }
  }
  cudaError_t e = cudaMemsetAsync(D.flush_buf, 0, D.flush_bytes, D.compute);
  if (e != cudaSuccess) return cuda_fail(ctx, ZYXB_ERR_KERNEL_LAUNCH, "flush_l2", e);
  return ZYXB_OK;
}

// ---- collectives ------------------------------------------------------------------------------------
int32_t zyxb_comm_unique_id(zyxb_ctx* ctx, void* out_id_128_bytes) {
  if (!ctx) return ZYXB_ERR_INITIALIZATION;
  std::string err;
  int st = comm_unique_id(out_id_128_bytes, err);
  if (st) return fail(ctx, st, err);
  return ZYXB_OK;
}

int32_t zyxb_comm_init(zyxb_ctx* ctx, int32_t dev, int32_t rank, int32_t world, const void* id_128_bytes) {
  DEV_OR_FAIL(ZYXB_ERR_INITIALIZATION);
  if (D.comm) return fail(ctx, ZYXB_ERR_INITIALIZATION, "comm_init: communicator already exists");
  std::string err;
  int st = comm_create(&D.comm, rank, world, id_128_bytes, err);
  if (st) return fail(ctx, st, err);
  // set-up of the peer-memory allreduce is collective too (flag blocks are exchanged through the communicator)
  if ((st = peer_create(&D.peer, D.comm, D.status_word, D.comm_stream, err))) return fail(ctx, st, err);
  if (ctx->debug & 1) fprintf(stderr, "[zyxb] rank %d/%d: allreduce over %s\n", rank, world, peer_usable(D.peer) ? "peer memory (copy engines)" : "NCCL");
  return ZYXB_OK;
}

int32_t zyxb_allreduce_sum(zyxb_ctx* ctx, int32_t dev, uint32_t buf, uint64_t offset_elems, uint64_t count, int32_t dtype,
                           const zyxb_event* wait, int32_t n_wait, zyxb_event* out_event) {
  DEV_OR_FAIL(ZYXB_ERR_KERNEL_LAUNCH);
  if (!D.comm) return fail(ctx, ZYXB_ERR_KERNEL_LAUNCH, "allreduce: no communicator (call zyxb_comm_init)");
  Buffer* b = get_buffer(D, buf);
  if (!b || b->is_variable) return fail(ctx, ZYXB_ERR_INCORRECT_KERNEL_ARG, "allreduce: unknown buffer");
  const uint64_t es = dtype_size(dtype);
  if (!elems_ok(offset_elems, count, es, b->bytes)) return fail(ctx, ZYXB_ERR_INCORRECT_KERNEL_ARG, "allreduce: range exceeds the buffer");
  int st = wait_and_consume(ctx, D, D.comm_stream, wait, n_wait, ZYXB_ERR_KERNEL_LAUNCH);
  if (st) return st;
  // the producer kernels were enqueued on the compute stream before this call
  if ((st = order_streams(ctx, D.compute, D.comm_stream, ZYXB_ERR_KERNEL_LAUNCH))) return st;
  std::string err;
  char* p = (char*)b->ptr + offset_elems * es;
  Buffer* root = b->is_view ? get_buffer(D, b->parent) : b;
  if (peer_usable(D.peer) && root && !root->is_view && !D.capturing && !D.comm_latency) {
    // the whole cudaMalloc block is mapped by the peers; the range is an offset into it
    const uint64_t byte_offset = (uint64_t)(p - (char*)root->ptr);
    st = peer_allreduce_sum(D.peer, D.comm, root->ptr, root->capacity, byte_offset, count, dtype, D.comm_stream, &D.launch_count, err);
  } else {
    st = comm_allreduce_sum(D.comm, p, p, count, dtype, D.comm_stream, err);
  }
  if (st) return fail(ctx, st, err);
  if (out_event) return record_event(ctx, D, D.comm_stream, out_event, ZYXB_ERR_KERNEL_LAUNCH);
  return order_streams(ctx, D.comm_stream, D.compute, ZYXB_ERR_KERNEL_LAUNCH);
}

// reduce-scatter (gather == false) or all-gather over `world` consecutive slices of count_per_rank elements, in place
static int32_t sliced_collective(zyxb_ctx* ctx, int32_t dev, bool gather, uint32_t buf, uint64_t offset_elems, uint64_t count_per_rank,
                                 int32_t dtype, const zyxb_event* wait, int32_t n_wait, zyxb_event* out_event) {
  const char* what = gather ? "allgather" : "reduce_scatter";
  DEV_OR_FAIL(ZYXB_ERR_KERNEL_LAUNCH);
  if (!D.comm) return fail(ctx, ZYXB_ERR_KERNEL_LAUNCH, std::string(what) + ": no communicator (call zyxb_comm_init)");
  Buffer* b = get_buffer(D, buf);
  if (!b || b->is_variable) return fail(ctx, ZYXB_ERR_INCORRECT_KERNEL_ARG, std::string(what) + ": unknown buffer");
  int rank = 0, world = 1;
  comm_rank(D.comm, &rank, &world);
  const uint64_t es = dtype_size(dtype);
  uint64_t all_ranks = 0;
  if (__builtin_mul_overflow(count_per_rank, (uint64_t)world, &all_ranks) || !elems_ok(offset_elems, all_ranks, es, b->bytes)) return fail(ctx, ZYXB_ERR_INCORRECT_KERNEL_ARG, std::string(what) + ": range exceeds the buffer");
  int st = wait_and_consume(ctx, D, D.comm_stream, wait, n_wait, ZYXB_ERR_KERNEL_LAUNCH);
  if (st) return st;
  if ((st = order_streams(ctx, D.compute, D.comm_stream, ZYXB_ERR_KERNEL_LAUNCH))) return st;   // producers were queued on the compute stream
  std::string err;
  char* p = (char*)b->ptr + offset_elems * es;
  st = gather ? comm_allgather(D.comm, p, count_per_rank, es, dtype, D.comm_stream, err)
              : comm_reduce_scatter_sum(D.comm, p, count_per_rank, es, dtype, D.comm_stream, err);
  if (st) return fail(ctx, st, err);
  if (out_event) return record_event(ctx, D, D.comm_stream, out_event, ZYXB_ERR_KERNEL_LAUNCH);
  return order_streams(ctx, D.comm_stream, D.compute, ZYXB_ERR_KERNEL_LAUNCH);
}

int32_t zyxb_reduce_scatter_sum(zyxb_ctx* ctx, int32_t dev, uint32_t buf, uint64_t offset_elems, uint64_t count_per_rank, int32_t dtype,
                                const zyxb_event* wait, int32_t n_wait, zyxb_event* out_event) {
  return sliced_collective(ctx, dev, false, buf, offset_elems, count_per_rank, dtype, wait, n_wait, out_event);
}

int32_t zyxb_allgather(zyxb_ctx* ctx, int32_t dev, uint32_t buf, uint64_t offset_elems, uint64_t count_per_rank, int32_t dtype,
                       const zyxb_event* wait, int32_t n_wait, zyxb_event* out_event) {
  return sliced_collective(ctx, dev, true, buf, offset_elems, count_per_rank, dtype, wait, n_wait, out_event);
}

int32_t zyxb_comm_rank(zyxb_ctx* ctx, int32_t dev, int32_t* out_rank, int32_t* out_world) {
  DEV_OR_FAIL(ZYXB_ERR_INITIALIZATION);
  if (!D.comm) return fail(ctx, ZYXB_ERR_INITIALIZATION, "comm_rank: no communicator (call zyxb_comm_init)");
  int rank = 0, world = 1;
  comm_rank(D.comm, &rank, &world);
  if (out_rank) *out_rank = rank;
  if (out_world) *out_world = world;
  return ZYXB_OK;
}

int32_t zyxb_comm_option(zyxb_ctx* ctx, int32_t dev, int32_t option, int32_t value) {
  DEV_OR_FAIL(ZYXB_ERR_INITIALIZATION);
  if (option != ZYXB_COMM_OPT_LATENCY) return fail(ctx, ZYXB_ERR_INCORRECT_KERNEL_ARG, "comm_option: unknown option");
  D.comm_latency = value != 0;
  return ZYXB_OK;
}

int32_t zyxb_comm_destroy(zyxb_ctx* ctx, int32_t dev) {
  DEV_OR_FAIL(ZYXB_ERR_DEINITIALIZATION);
  if (D.comm) {
    cudaDeviceSynchronize();
    if (D.peer) { peer_destroy(D.peer); D.peer = nullptr; }
    comm_destroy(D.comm); D.comm = nullptr;
  }
  return ZYXB_OK;
}

#pragma GCC visibility pop
}  // extern "C"
