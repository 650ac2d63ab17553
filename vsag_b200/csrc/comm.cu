// NCCL behind the C ABI: communicator set-up for one process per GPU and the few collectives the sharded
// searches need (the reference merges shard results on the host, IVF::Merge / the per-shard loop of
// src/algorithm/ivf/ivf.cpp:1989-2050; here the shards are GPUs and the merge input crosses NVLink).
#include "comm.cuh"

#include <dlfcn.h>
#include <nccl.h>   // types and enumerators only: the functions are looked up at run time

#include <mutex>

#include "common.cuh"

namespace vb200 {
namespace {

struct NcclApi {
    ncclResult_t (*get_unique_id)(ncclUniqueId*) = nullptr;
    ncclResult_t (*comm_init_rank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*comm_destroy)(ncclComm_t) = nullptr;
    ncclResult_t (*all_gather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*all_reduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*group_start)() = nullptr;
    ncclResult_t (*group_end)() = nullptr;
    const char* (*error_string)(ncclResult_t) = nullptr;
    bool ready = false;
};

NcclApi g_nccl;
std::mutex g_nccl_mu;

int
load_nccl() {
    std::lock_guard<std::mutex> lock(g_nccl_mu);
    if (g_nccl.ready) {
        return 0;
    }
    // A process that already holds an NCCL (for example through torch) gets that one: the loader hands
    // back the loaded object for the same soname.
    void* lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (lib == nullptr) {
        lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    }
    if (lib == nullptr) {
        VB_FAIL(VB200_UNSUPPORTED_INDEX_OPERATION, "NCCL could not be loaded: %s", dlerror());
    }
    bool ok = true;
    auto sym = [&](const char* name) -> void* {
        void* p = dlsym(lib, name);
        ok = ok && p != nullptr;
        return p;
    };
    g_nccl.get_unique_id = reinterpret_cast<decltype(g_nccl.get_unique_id)>(sym("ncclGetUniqueId"));
    g_nccl.comm_init_rank = reinterpret_cast<decltype(g_nccl.comm_init_rank)>(sym("ncclCommInitRank"));
    g_nccl.comm_destroy = reinterpret_cast<decltype(g_nccl.comm_destroy)>(sym("ncclCommDestroy"));
    g_nccl.all_gather = reinterpret_cast<decltype(g_nccl.all_gather)>(sym("ncclAllGather"));
    g_nccl.all_reduce = reinterpret_cast<decltype(g_nccl.all_reduce)>(sym("ncclAllReduce"));
    g_nccl.group_start = reinterpret_cast<decltype(g_nccl.group_start)>(sym("ncclGroupStart"));
    g_nccl.group_end = reinterpret_cast<decltype(g_nccl.group_end)>(sym("ncclGroupEnd"));
    g_nccl.error_string = reinterpret_cast<decltype(g_nccl.error_string)>(sym("ncclGetErrorString"));
    if (!ok) {
        VB_FAIL(VB200_UNSUPPORTED_INDEX_OPERATION, "the NCCL library lacks a function this library needs");
    }
    g_nccl.ready = true;
    return 0;
}

}  // namespace

#define VB_NCCL(expr)                                                                                 \
    do {                                                                                              \
        ncclResult_t _r = (expr);                                                                     \
        if (_r != ncclSuccess) {                                                                      \
            VB_FAIL(VB200_INTERNAL_ERROR, "%s failed: %s", #expr, g_nccl.error_string(_r));           \
        }                                                                                             \
    } while (0)

int
comm_all_gather(vb200_comm* comm, const void* send, void* recv, size_t bytes_per_rank, cudaStream_t stream) {
    VB_CHECK_ARG(comm != nullptr && comm->nccl != nullptr, "null communicator");
    VB_NCCL(g_nccl.all_gather(send, recv, bytes_per_rank, ncclUint8, static_cast<ncclComm_t>(comm->nccl), stream));
    return 0;
}

int
comm_all_reduce_min_f32(vb200_comm* comm, float* buf, size_t count, cudaStream_t stream) {
    VB_CHECK_ARG(comm != nullptr && comm->nccl != nullptr, "null communicator");
    VB_NCCL(g_nccl.all_reduce(buf, buf, count, ncclFloat32, ncclMin, static_cast<ncclComm_t>(comm->nccl), stream));
    return 0;
}

int
comm_group_start() {
    VB_TRY(load_nccl());
    VB_NCCL(g_nccl.group_start());
    return 0;
}

int
comm_group_end() {
    VB_TRY(load_nccl());
    VB_NCCL(g_nccl.group_end());
    return 0;
}

}  // namespace vb200

using namespace vb200;

extern "C" int
vb200_comm_unique_id(uint8_t* id_out) {
    VB_CHECK_ARG(id_out != nullptr, "null pointer");
    VB_TRY(load_nccl());
    static_assert(sizeof(ncclUniqueId) == VB200_COMM_ID_BYTES, "unique id size");
    ncclUniqueId id;
    VB_NCCL(g_nccl.get_unique_id(&id));
    std::memcpy(id_out, &id, sizeof(id));
    return 0;
}

extern "C" int
vb200_comm_init(vb200_comm_t* comm_out, const uint8_t* id, int rank, int world) {
    VB_CHECK_ARG(comm_out != nullptr && id != nullptr, "null pointer");
    VB_CHECK_ARG(world >= 1 && rank >= 0 && rank < world, "rank %d is not in a world of %d", rank, world);
    VB_TRY(load_nccl());
    ncclUniqueId uid;
    std::memcpy(&uid, id, sizeof(uid));
    int device = 0;
    VB_CUDA(cudaGetDevice(&device));
    ncclComm_t c = nullptr;
    VB_NCCL(g_nccl.comm_init_rank(&c, world, uid, rank));
    vb200_comm* comm = new (std::nothrow) vb200_comm;
    if (comm == nullptr) {
        g_nccl.comm_destroy(c);
        VB_FAIL(VB200_NO_ENOUGH_MEMORY, "out of host memory");
    }
    comm->nccl = c;
    comm->rank = rank;
    comm->world = world;
    comm->device = device;
    *comm_out = comm;
    return 0;
}

extern "C" int
vb200_comm_destroy(vb200_comm_t comm) {
    if (comm == nullptr) {
        return 0;
    }
    if (comm->nccl != nullptr && g_nccl.ready) {
        g_nccl.comm_destroy(static_cast<ncclComm_t>(comm->nccl));
    }
    delete comm;
    return 0;
}

extern "C" int
vb200_comm_rank(vb200_comm_t comm) {
    return comm != nullptr ? comm->rank : -1;
}

extern "C" int
vb200_comm_world(vb200_comm_t comm) {
    return comm != nullptr ? comm->world : -1;
}
