// Minimal NCCL binding resolved at run time (see vb_nccl.cu).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace vb {

struct NcclUniqueId { char internal[128]; };  // ncclUniqueId: NCCL_UNIQUE_ID_BYTES = 128

int32_t nccl_unique_id(NcclUniqueId* id);
int32_t nccl_comm_init(void** comm, int n_ranks, const NcclUniqueId* id, int rank);
void nccl_comm_destroy(void* comm);
int32_t nccl_allreduce_sum_f32(void* comm, float* buf, size_t count, cudaStream_t stream);
int32_t nccl_allgather_bytes(void* comm, const void* send, void* recv, size_t bytes_per_rank, cudaStream_t stream);

}  // namespace vb
