// Gradient exchange for data-parallel training: a thin layer over NCCL, loaded at run time
// so that the library itself has no link-time dependency on it.  The reference has no
// collective layer at all (its README lists data parallelism as "manual"), so nothing here
// mirrors reference code.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace zyxb {
struct Comm;
int comm_unique_id(void* out_128_bytes, std::string& err);
int comm_create(Comm** out, int rank, int world, const void* id_128_bytes, std::string& err);
int comm_allreduce_sum(Comm* c, const void* send, void* recv, uint64_t count, int dtype, cudaStream_t stream, std::string& err);
int comm_reduce_scatter_sum(Comm* c, void* base, uint64_t count_per_rank, uint64_t elem_bytes, int dtype, cudaStream_t stream, std::string& err);
int comm_allgather(Comm* c, void* base, uint64_t count_per_rank, uint64_t elem_bytes, int dtype, cudaStream_t stream, std::string& err);
// every rank contributes `bytes` bytes at `send`, `recv` receives world * bytes (device pointers)
int comm_allgather_raw(Comm* c, const void* send, void* recv, uint64_t bytes, cudaStream_t stream, std::string& err);
void comm_rank(const Comm* c, int* rank, int* world);

// ---- allreduce over peer memory (peer_allreduce.cu) ------------------------------------------------------------------
// The gradient allreduce of data-parallel training without NCCL's ring kernel: the ranks of one node map each other's
// gradient buffers (CUDA IPC), the copy engines pull shards over NVLink, and a small kernel adds them.  Both calls are
// collective: every rank makes them in the same order.
struct PeerComm;
int peer_create(PeerComm** out, Comm* c, uint32_t* status_word, cudaStream_t stream, std::string& err);
// in place over [base + byte_offset, + count elements); `base` .. `base + buffer_bytes` is one cudaMalloc block
int peer_allreduce_sum(PeerComm* p, Comm* c, void* base, uint64_t buffer_bytes, uint64_t byte_offset, uint64_t count, int dtype,
                       cudaStream_t stream, uint64_t* launch_counter, std::string& err);
bool peer_usable(const PeerComm* p);
bool peer_has_exported(const PeerComm* p, const void* base);   // the block's IPC handle is open in other processes
void peer_forget_buffer(PeerComm* p, const void* base);        // the block is about to be freed
void peer_destroy(PeerComm* p);
void comm_destroy(Comm* c);
}  // namespace zyxb
