// Collectives between the GPUs of one node for the sharded searches: a thin layer over NCCL, which the
// library opens at run time (dlopen of libnccl.so.2) the first time a communicator is asked for, so that
// single-GPU users need no NCCL at all.  Everything is enqueued on the caller's stream; nothing here
// synchronises with the host.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

struct vb200_comm {
    void* nccl = nullptr;   // ncclComm_t
    int rank = 0;
    int world = 1;
    int device = 0;
};

namespace vb200 {

// recv[world][bytes_per_rank] <- every rank's send[bytes_per_rank]
int comm_all_gather(vb200_comm* comm, const void* send, void* recv, size_t bytes_per_rank, cudaStream_t stream);
// buf[count] <- element-wise minimum over the ranks
int comm_all_reduce_min_f32(vb200_comm* comm, float* buf, size_t count, cudaStream_t stream);
// Collectives between the two calls are launched together.
int comm_group_start();
int comm_group_end();


// Merge of `parts` partial results [nq][k], part p's keys at keys_all + p * part_stride and its labels at
// labels_all + p * part_stride (all in this GPU's memory), into ids / dists (host or device).  Enqueued on the
// current stream; no host synchronisation.
int merge_partials_device(const uint64_t* keys_all, const int64_t* labels_all, uint32_t parts, uint64_t part_stride,
                          uint64_t nq, uint32_t k, int64_t* ids, float* dists);

}  // namespace vb200
