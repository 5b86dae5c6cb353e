// Gradient allreduce over peer memory: NVLink copy engines move the data, a small kernel adds it.
//
// Why not NCCL's allreduce here: in data-parallel training the allreduce of a layer's gradients runs beside the remaining
// backward matmuls.  NCCL's ring kernel takes SMs (and, for a persistent matmul of one CTA per SM, whole SMs: the two kernels
// cannot share one), which stretched the input-gradient matmuls by a sixth and accounted for the whole loss of scaling
// efficiency from one GPU to two.  On an NVSwitch node every GPU reaches every peer at full NVLink bandwidth, so the
// transfer needs no SM at all:
//
//   every rank owns one shard of the range (count / world elements).  Per call, with a sequence number that all ranks
//   advance in step:
//     1. tell every peer "my gradients are complete" (a flag in the peer's memory), wait for theirs
//     2. copy engines PULL my shard of every peer's buffer into local staging            (world-1 peer copies over NVLink)
//     3. one small kernel: my shard = sum over ranks, in rank order, accumulated in f32  (identical bits on every rank later)
//     4. tell every peer "my shard is reduced", wait for theirs
//     5. copy engines PULL every peer's reduced shard into my buffer                     (world-1 peer copies)
//     6. tell every peer "I have read your shard", wait for theirs: only then may anyone overwrite its buffer again
//
// Peer buffers and flag words are mapped with CUDA IPC (one process per GPU).  The handles travel through an NCCL all-gather
// at set-up, so NCCL remains the rendezvous; the hot path does not touch it.  Flags only ever grow (the sequence number), so
// a late reader can never mistake an old value for a new one.  Every wait is a one-warp kernel polling LOCAL memory with a
// wall-clock bound; on expiry it sets a bit in the device status word and returns (the result of that step is then wrong,
// and zyxb_device_status reports KernelSync) - nothing can spin for ever.  The waiting kernel and the kernel that satisfies it
// always run on different GPUs.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <string>
#include <vector>

#include "../../include/zyxb.h"
#include "comm.h"
#include "common.cuh"

namespace zyxb {

namespace {

constexpr int PEER_MAX_WORLD = 16;
constexpr uint32_t PEER_STATUS_TIMEOUT = 0x4000;
enum { FLAG_READY = 0, FLAG_REDUCED = 1, FLAG_GATHERED = 2, FLAG_KINDS = 3 };

struct FlagTable { uint32_t* peer[PEER_MAX_WORLD]; };   // by value into the kernels: where each rank's flag block is mapped here

__device__ __forceinline__ uint64_t peer_timer_ns() { uint64_t t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }

// Thread p < world (p != me): write `seq` into slot [kind][me] of rank p's flag block, then poll slot [kind][p] of my own block
// until rank p has written `seq` (or later) there.  One warp, no shared memory: it runs beside whatever occupies the SMs.
__global__ void peer_signal_wait_kernel(FlagTable table, int me, int world, int kind, uint32_t seq, uint64_t limit_ns, uint32_t* status) {
  const int p = threadIdx.x;
  if (p >= world || p == me) return;
  __threadfence_system();                                            // everything this stream did before is visible to the peers
  volatile uint32_t* theirs = table.peer[p] + kind * PEER_MAX_WORLD + me;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(seq) : "memory");
  const uint32_t* mine = table.peer[me] + kind * PEER_MAX_WORLD + p;
  uint64_t t0 = 0;
  for (uint32_t spins = 0;; ++spins) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if ((int32_t)(v - seq) >= 0) break;
    if ((spins & 0xff) == 0xff) {
      const uint64_t now = peer_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) { atomicOr(status, PEER_STATUS_TIMEOUT); break; }
      __nanosleep(200);
    }
  }
}

struct ReduceSrc { const void* ptr[PEER_MAX_WORLD]; };   // rank r's copy of my shard (my own buffer for r == me, staging otherwise)

// out[i] = sum over ranks r = 0 .. world-1 of src[r][i], accumulated in f32 in that order, rounded to nearest once.
// IS_BF16 / f16: eight elements per 128-bit load.
template <int KIND>   // 0 f32, 1 bf16, 2 f16, 3 i32
__global__ void peer_reduce_kernel(ReduceSrc src, void* out, uint64_t n, int world) {
  const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, nthreads = (uint64_t)gridDim.x * blockDim.x;
  if constexpr (KIND == 0 || KIND == 3) {
    bool aligned = ((uintptr_t)out % 16) == 0;
    for (int r = 0; r < world; ++r) aligned = aligned && ((uintptr_t)src.ptr[r] % 16) == 0;
    const uint64_t nv = aligned ? n / 4 : 0;
    for (uint64_t i = tid; i < nv; i += nthreads) {
      if constexpr (KIND == 0) {
        float4 acc = ((const float4*)src.ptr[0])[i];
        for (int r = 1; r < world; ++r) { const float4 v = ((const float4*)src.ptr[r])[i]; acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w; }
        ((float4*)out)[i] = acc;
      } else {
        int4 acc = ((const int4*)src.ptr[0])[i];
        for (int r = 1; r < world; ++r) { const int4 v = ((const int4*)src.ptr[r])[i]; acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w; }
        ((int4*)out)[i] = acc;
      }
    }
    for (uint64_t i = nv * 4 + tid; i < n; i += nthreads) {
      if constexpr (KIND == 0) { float a = ((const float*)src.ptr[0])[i]; for (int r = 1; r < world; ++r) a += ((const float*)src.ptr[r])[i]; ((float*)out)[i] = a; }
      else { int a = ((const int*)src.ptr[0])[i]; for (int r = 1; r < world; ++r) a += ((const int*)src.ptr[r])[i]; ((int*)out)[i] = a; }
    }
  } else {
    auto widen = [](uint16_t h) -> float {
      if constexpr (KIND == 1) return __uint_as_float((uint32_t)h << 16);
      else return __half2float(__ushort_as_half(h));
    };
    auto narrow = [](float f) -> uint16_t {
      if constexpr (KIND == 1) return __bfloat16_as_ushort(__float2bfloat16_rn(f));
      else return __half_as_ushort(__float2half_rn(f));
    };
    bool aligned = ((uintptr_t)out % 16) == 0;
    for (int r = 0; r < world; ++r) aligned = aligned && ((uintptr_t)src.ptr[r] % 16) == 0;
    const uint64_t nv = aligned ? n / 8 : 0;
    // four 128-bit vectors per thread and pass, every source's loads issued before the first add: the kernel is a pure
    // stream over HBM and has to keep enough bytes in flight with few, short-lived CTAs
    constexpr int U = 4;
    for (uint64_t i0 = tid; i0 < nv; i0 += nthreads * U) {
      float acc[U][8];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[u][j] = 0.0f;
      for (int r = 0; r < world; ++r) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const uint64_t i = i0 + (uint64_t)u * nthreads;
          v[u] = i < nv ? __ldcs(((const uint4*)src.ptr[r]) + i) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) { acc[u][2 * j] += widen((uint16_t)(w[j] & 0xffff)); acc[u][2 * j + 1] += widen((uint16_t)(w[j] >> 16)); }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint64_t i = i0 + (uint64_t)u * nthreads;
        if (i >= nv) continue;
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = (uint32_t)narrow(acc[u][2 * j]) | ((uint32_t)narrow(acc[u][2 * j + 1]) << 16);
        ((uint4*)out)[i] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
    for (uint64_t i = nv * 8 + tid; i < n; i += nthreads) {
      float a = widen(((const uint16_t*)src.ptr[0])[i]);
      for (int r = 1; r < world; ++r) a += widen(((const uint16_t*)src.ptr[r])[i]);
      ((uint16_t*)out)[i] = narrow(a);
    }
  }
}

}  // namespace

// ---- host side -----------------------------------------------------------------------------------------------------------
struct PeerBuffer {
  void* peer_base[PEER_MAX_WORLD] = {nullptr};   // where each rank's block is mapped in this process (own block: its address)
  uint64_t bytes = 0;
};

struct PeerComm {
  int rank = 0, world = 1;
  bool usable = false;
  uint32_t* flags = nullptr;            // my flag block: [FLAG_KINDS][PEER_MAX_WORLD] words, device memory, only ever growing
  FlagTable table{};                    // every rank's flag block as mapped here
  uint32_t* status_word = nullptr;
  uint32_t seq = 0;
  uint64_t wait_limit_ns = 20000000000ull;
  void* staging = nullptr;              // (world - 1) shards pulled from the peers
  uint64_t staging_bytes = 0;
  void* xchg = nullptr;                 // device scratch for handle exchange: world + 1 slots of 128 bytes
  // the world-1 peer copies of a phase run side by side, one copy engine each: one extra stream and one event per peer
  cudaStream_t side[PEER_MAX_WORLD] = {nullptr};
  cudaEvent_t fork = nullptr, join[PEER_MAX_WORLD] = {nullptr};
  std::map<const void*, PeerBuffer> buffers;
};

namespace {

struct HandleMsg { cudaIpcMemHandle_t handle; uint64_t bytes; int32_t ok; int32_t pad; char fill[128 - sizeof(cudaIpcMemHandle_t) - 16]; };
static_assert(sizeof(HandleMsg) == 128, "exchange slot");

// all-gather one HandleMsg per rank through NCCL (device staging), result on the host
int exchange(PeerComm* p, Comm* c, const HandleMsg& mine, std::vector<HandleMsg>& all, cudaStream_t stream, std::string& err) {
  all.assign(p->world, HandleMsg{});
  char* send = (char*)p->xchg;
  char* recv = send + 128;
  cudaError_t e = cudaMemcpyAsync(send, &mine, 128, cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) { err = std::string("peer exchange: ") + cudaGetErrorString(e); return ZYXB_ERR_INITIALIZATION; }
  int st = comm_allgather_raw(c, send, recv, 128, stream, err);
  if (st) return st;
  e = cudaMemcpyAsync(all.data(), recv, 128ull * p->world, cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) { err = std::string("peer exchange: ") + cudaGetErrorString(e); return ZYXB_ERR_INITIALIZATION; }
  return ZYXB_OK;
}

// Export `ptr` (the base of a cudaMalloc block), import every peer's; `mapped[r]` receives the local addresses.  Collective.
// Returns with *all_ok = false (and nothing left open) when any rank could not export or import.
int map_everywhere(PeerComm* p, Comm* c, void* ptr, uint64_t bytes, void** mapped, bool* all_ok, cudaStream_t stream, std::string& err) {
  HandleMsg mine{};
  mine.bytes = bytes;
  mine.ok = cudaIpcGetMemHandle(&mine.handle, ptr) == cudaSuccess ? 1 : 0;
  if (!mine.ok) cudaGetLastError();
  std::vector<HandleMsg> all;
  int st = exchange(p, c, mine, all, stream, err);
  if (st) return st;
  bool ok = true;
  for (int r = 0; r < p->world; ++r) ok = ok && all[r].ok && all[r].bytes == bytes;
  for (int r = 0; r < p->world; ++r) mapped[r] = nullptr;
  if (ok) {
    for (int r = 0; r < p->world && ok; ++r) {
      if (r == p->rank) { mapped[r] = ptr; continue; }
      if (cudaIpcOpenMemHandle(&mapped[r], all[r].handle, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); mapped[r] = nullptr; ok = false; }
    }
  }
  // second round: did everyone manage to import?
  HandleMsg verdict{};
  verdict.ok = ok ? 1 : 0;
  st = exchange(p, c, verdict, all, stream, err);
  if (st) return st;
  bool everyone = true;
  for (int r = 0; r < p->world; ++r) everyone = everyone && all[r].ok;
  if (!everyone) {
    for (int r = 0; r < p->world; ++r) if (r != p->rank && mapped[r]) { cudaIpcCloseMemHandle(mapped[r]); mapped[r] = nullptr; }
  }
  *all_ok = everyone;
  return ZYXB_OK;
}

}  // namespace

bool peer_usable(const PeerComm* p) { return p && p->usable; }
bool peer_has_exported(const PeerComm* p, const void* base) { return p && p->buffers.count(base) != 0; }

int peer_create(PeerComm** out, Comm* c, uint32_t* status_word, cudaStream_t stream, std::string& err) {
  PeerComm* p = new PeerComm();
  comm_rank(c, &p->rank, &p->world);
  p->status_word = status_word;
  if (const char* ms = getenv("ZYXB_PEER_WAIT_MS")) { const long v = atol(ms); if (v > 0) p->wait_limit_ns = (uint64_t)v * 1000000ull; }
  *out = p;
  const char* mode = getenv("ZYXB_ALLREDUCE");
  if (p->world < 2 || p->world > PEER_MAX_WORLD || (mode && strcmp(mode, "nccl") == 0)) return ZYXB_OK;      // stays unusable: NCCL path
  cudaError_t e = cudaMalloc(&p->xchg, 128ull * (p->world + 1));
  if (e == cudaSuccess) e = cudaMalloc((void**)&p->flags, FLAG_KINDS * PEER_MAX_WORLD * sizeof(uint32_t));
  if (e == cudaSuccess) e = cudaMemset(p->flags, 0, FLAG_KINDS * PEER_MAX_WORLD * sizeof(uint32_t));
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&p->fork, cudaEventDisableTiming);
  for (int i = 0; i + 2 < p->world && e == cudaSuccess; ++i) {
    e = cudaStreamCreateWithFlags(&p->side[i], cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&p->join[i], cudaEventDisableTiming);
  }
  if (e != cudaSuccess) { err = std::string("peer allreduce set-up: ") + cudaGetErrorString(e); return ZYXB_ERR_MEMORY_ALLOCATION; }
  void* mapped[PEER_MAX_WORLD];
  bool ok = false;
  int st = map_everywhere(p, c, p->flags, FLAG_KINDS * PEER_MAX_WORLD * sizeof(uint32_t), mapped, &ok, stream, err);
  if (st) return st;
  if (ok) for (int r = 0; r < p->world; ++r) p->table.peer[r] = (uint32_t*)mapped[r];
  p->usable = ok;
  if (!ok) return ZYXB_OK;
  // One small allreduce of known values before anyone relies on the path: every rank must read the exact sum and see no
  // wait give up, and the ranks must agree on that; otherwise all of them stay on the communicator's own allreduce.
  const uint64_t n = 4096;
  float* probe = nullptr;
  std::vector<float> host(n);
  for (uint64_t i = 0; i < n; ++i) host[i] = (float)((p->rank + 1) * (int)(i % 7 + 1));
  bool good = cudaMalloc((void**)&probe, n * 4) == cudaSuccess &&
              cudaMemcpyAsync(probe, host.data(), n * 4, cudaMemcpyHostToDevice, stream) == cudaSuccess;
  const uint64_t limit = p->wait_limit_ns;
  p->wait_limit_ns = std::min<uint64_t>(limit, 5000000000ull);
  std::string probe_err;
  // the call is collective (it maps the probe everywhere), so every rank makes it whatever its own state
  if (probe && peer_allreduce_sum(p, c, probe, n * 4, 0, n, ZYXB_F32, stream, nullptr, probe_err) != ZYXB_OK) good = false;
  p->wait_limit_ns = limit;
  uint32_t word = 0;
  if (probe && (cudaMemcpyAsync(host.data(), probe, n * 4, cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
                cudaMemcpyAsync(&word, status_word, 4, cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
                cudaStreamSynchronize(stream) != cudaSuccess)) good = false;
  const int tri = p->world * (p->world + 1) / 2;
  for (uint64_t i = 0; good && i < n; ++i) good = host[i] == (float)(tri * (int)(i % 7 + 1));
  if (word & PEER_STATUS_TIMEOUT) {
    good = false;
    word &= ~PEER_STATUS_TIMEOUT;             // the probe's own expiry is reported by falling back, not through the status word
    cudaMemcpyAsync(status_word, &word, 4, cudaMemcpyHostToDevice, stream);
    cudaStreamSynchronize(stream);
  }
  cudaGetLastError();
  HandleMsg verdict{};
  verdict.ok = good ? 1 : 0;
  std::vector<HandleMsg> all;
  st = exchange(p, c, verdict, all, stream, err);
  if (st) return st;
  for (int r = 0; r < p->world; ++r) good = good && all[r].ok;
  if (probe) { peer_forget_buffer(p, probe); cudaFree(probe); }
  if (!good) {
    fprintf(stderr, "[zyxb] rank %d: the peer-memory allreduce failed its set-up probe (%s); using the communicator's allreduce\n", p->rank,
            probe_err.empty() ? "wrong sum or a wait that gave up" : probe_err.c_str());
    p->usable = false;
  }
  return ZYXB_OK;
}

void peer_forget_buffer(PeerComm* p, const void* base) {
  if (!p) return;
  auto it = p->buffers.find(base);
  if (it == p->buffers.end()) return;
  for (int r = 0; r < p->world; ++r) if (r != p->rank && it->second.peer_base[r]) cudaIpcCloseMemHandle(it->second.peer_base[r]);
  p->buffers.erase(it);
}

void peer_destroy(PeerComm* p) {
  if (!p) return;
  cudaDeviceSynchronize();
  while (!p->buffers.empty()) peer_forget_buffer(p, p->buffers.begin()->first);
  for (int r = 0; r < p->world; ++r) if (r != p->rank && p->table.peer[r]) cudaIpcCloseMemHandle(p->table.peer[r]);
  for (int i = 0; i < PEER_MAX_WORLD; ++i) { if (p->side[i]) cudaStreamDestroy(p->side[i]); if (p->join[i]) cudaEventDestroy(p->join[i]); }
  if (p->fork) cudaEventDestroy(p->fork);
  if (p->staging) cudaFree(p->staging);
  if (p->flags) cudaFree(p->flags);
  if (p->xchg) cudaFree(p->xchg);
  delete p;
}

int peer_allreduce_sum(PeerComm* p, Comm* c, void* base, uint64_t buffer_bytes, uint64_t byte_offset, uint64_t count, int dtype,
                       cudaStream_t stream, uint64_t* launch_counter, std::string& err) {
  const uint64_t es = dtype == ZYXB_F32 || dtype == ZYXB_I32 ? 4 : 2;
  const int W = p->world, me = p->rank;
  // ---- the buffer's mapping in every process (collective the first time a block is seen) ----
  auto it = p->buffers.find(base);
  if (it == p->buffers.end()) {
    PeerBuffer b;
    b.bytes = buffer_bytes;
    bool ok = false;
    int st = map_everywhere(p, c, base, buffer_bytes, b.peer_base, &ok, stream, err);
    if (st) return st;
    if (!ok) { err = "peer allreduce: a rank could not map the buffer of another (CUDA IPC)"; return ZYXB_ERR_INITIALIZATION; }
    it = p->buffers.emplace(base, b).first;
  }
  const PeerBuffer& B = it->second;
  if (count == 0) return ZYXB_OK;
  // ---- shards: rank r owns elements [r*cs, (r+1)*cs) of the range, cs a multiple of 64 elements ----
  const uint64_t cs = ((count + W - 1) / W + 63) / 64 * 64;
  auto lo = [&](int r) { return std::min<uint64_t>((uint64_t)r * cs, count); };
  auto hi = [&](int r) { return std::min<uint64_t>((uint64_t)(r + 1) * cs, count); };
  const uint64_t mine_n = hi(me) - lo(me);
  // ZYXB_PEER_DIRECT=1: the reduce kernel reads the peers' copies of this rank's shard over NVLink itself (plain loads from
  // the mapped peer buffers) instead of adding up copies the copy engines staged here: one phase and one pass over local
  // memory less, at the price of reduce CTAs that wait on NVLink latency beside the matmuls.  Measured on the data-parallel
  // step it changes little (the wait of the last optimizer launch shrinks by 0.2 ms, the matmuls beside it stretch by as much).
  static const int direct_env = getenv("ZYXB_PEER_DIRECT") ? atoi(getenv("ZYXB_PEER_DIRECT")) : 0;
  const bool direct = direct_env != 0;
  const uint64_t need = direct ? 0 : (uint64_t)(W - 1) * cs * es;
  if (need > p->staging_bytes) {
    cudaStreamSynchronize(stream);
    if (p->staging) cudaFree(p->staging);
    p->staging = nullptr; p->staging_bytes = 0;
    const cudaError_t e = cudaMalloc(&p->staging, need);
    if (e != cudaSuccess) { cudaGetLastError(); err = std::string("peer allreduce staging: ") + cudaGetErrorString(e); return ZYXB_ERR_MEMORY_ALLOCATION; }
    p->staging_bytes = need;
  }
  const uint32_t seq = ++p->seq;
  auto signal_wait = [&](int kind) {
    peer_signal_wait_kernel<<<1, 32, 0, stream>>>(p->table, me, W, kind, seq, p->wait_limit_ns, p->status_word);
    if (launch_counter) ++*launch_counter;
  };
  auto at = [&](void* b, uint64_t elem) { return (char*)b + byte_offset + elem * es; };
  cudaError_t e = cudaSuccess;
  // 1. my gradients are complete / theirs are
  signal_wait(FLAG_READY);
  // 2. pull my shard of every peer's buffer (nearest rank first, so that the W pulls of one moment spread over the peers)
  // copy number d of a phase goes to the main stream (d == 1) or to side stream d - 2, forked from and joined to the main one
  auto fork = [&]() { if (W > 2 && e == cudaSuccess) e = cudaEventRecord(p->fork, stream); };
  auto copy_on = [&](int d, void* dst, const void* srcp, uint64_t bytes) {
    if (e != cudaSuccess) return;
    cudaStream_t st = d == 1 ? stream : p->side[d - 2];
    if (d > 1) e = cudaStreamWaitEvent(st, p->fork, 0);
    if (e == cudaSuccess && bytes) e = cudaMemcpyAsync(dst, srcp, bytes, cudaMemcpyDeviceToDevice, st);
    if (d > 1 && e == cudaSuccess) e = cudaEventRecord(p->join[d - 2], st);
  };
  auto join = [&]() { for (int d = 2; d < W && e == cudaSuccess; ++d) e = cudaStreamWaitEvent(stream, p->join[d - 2], 0); };
  ReduceSrc src{};
  int slot = 0;
  if (direct) {
    for (int r = 0; r < W; ++r) if (r != me) src.ptr[r] = at(B.peer_base[r], lo(me));
  } else {
    fork();
    for (int d = 1; d < W; ++d) {
      const int r = (me + d) % W;
      char* dst = (char*)p->staging + (uint64_t)slot++ * cs * es;
      src.ptr[r] = dst;
      copy_on(d, dst, at(B.peer_base[r], lo(me)), mine_n * es);
    }
    join();
  }
  src.ptr[me] = at(base, lo(me));
  if (e != cudaSuccess) { err = std::string("peer allreduce pull: ") + cudaGetErrorString(e); return ZYXB_ERR_KERNEL_LAUNCH; }
  // 3. add, in rank order
  if (mine_n) {
    // short-lived CTAs without shared memory: they slot in beside the matmul's CTAs; enough of them to stream at HBM speed
    const unsigned grid = (unsigned)std::max<uint64_t>(1, std::min<uint64_t>(direct ? 592 : 296, mine_n / 8192 + 1));
    void* out = at(base, lo(me));
    switch (dtype) {
      case ZYXB_F32: peer_reduce_kernel<0><<<grid, 256, 0, stream>>>(src, out, mine_n, W); break;
      case ZYXB_BF16: peer_reduce_kernel<1><<<grid, 256, 0, stream>>>(src, out, mine_n, W); break;
      case ZYXB_F16: peer_reduce_kernel<2><<<grid, 256, 0, stream>>>(src, out, mine_n, W); break;
      case ZYXB_I32: peer_reduce_kernel<3><<<grid, 256, 0, stream>>>(src, out, mine_n, W); break;
      default: err = "peer allreduce: dtype must be f32, bf16, f16 or i32"; return ZYXB_ERR_INCORRECT_KERNEL_ARG;
    }
    if (launch_counter) ++*launch_counter;
  }
  // 4. my shard is reduced / theirs are
  signal_wait(FLAG_REDUCED);
  // 5. pull every peer's reduced shard
  fork();
  for (int d = 1; d < W; ++d) {
    const int r = (me + d) % W;
    copy_on(d, at(base, lo(r)), at(B.peer_base[r], lo(r)), (hi(r) - lo(r)) * es);
  }
  join();
  if (e != cudaSuccess) { err = std::string("peer allreduce gather: ") + cudaGetErrorString(e); return ZYXB_ERR_KERNEL_LAUNCH; }
  // 6. I have read every peer's shard / every peer has read mine: from here on the buffer may be written again
  signal_wait(FLAG_GATHERED);
  e = cudaGetLastError();
  if (e != cudaSuccess) { err = std::string("peer allreduce: ") + cudaGetErrorString(e); return ZYXB_ERR_KERNEL_LAUNCH; }
  return ZYXB_OK;
}

}  // namespace zyxb
