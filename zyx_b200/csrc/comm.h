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
void comm_rank(const Comm* c, int* rank, int* world);
void comm_destroy(Comm* c);
}  // namespace zyxb
