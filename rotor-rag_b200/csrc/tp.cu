// Tensor-parallel plumbing: one process per GPU, NCCL over NVLink for the exchange steps
// of column/row-parallel BitLinear (new design: the reference has no multi-device code).
//
// NCCL is bound at run time (dlopen of libnccl.so.2) so that the library has no link-time
// dependency on a particular NCCL build and shares the copy the host process already
// loaded.  Collectives are enqueued on the caller's stream between this library's kernels.
#include <dlfcn.h>
#include <nccl.h>  // types and enums only; every function is resolved with dlsym

#include <cstring>

#include "model.cuh"

namespace rb {

struct NcclApi {
    void* handle;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*);
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
};
static NcclApi g_nccl = {};

static int load_nccl() {
    if (g_nccl.handle) return ROTOR_B200_OK;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return ROTOR_B200_ERR_CUDA;
    NcclApi a = {};
    a.handle = h;
    a.GetUniqueId = (decltype(a.GetUniqueId))dlsym(h, "ncclGetUniqueId");
    a.CommInitRank = (decltype(a.CommInitRank))dlsym(h, "ncclCommInitRank");
    a.CommDestroy = (decltype(a.CommDestroy))dlsym(h, "ncclCommDestroy");
    a.AllReduce = (decltype(a.AllReduce))dlsym(h, "ncclAllReduce");
    a.AllGather = (decltype(a.AllGather))dlsym(h, "ncclAllGather");
    if (!a.GetUniqueId || !a.CommInitRank || !a.CommDestroy || !a.AllReduce || !a.AllGather) return ROTOR_B200_ERR_CUDA;
    g_nccl = a;
    return ROTOR_B200_OK;
}

struct TpComm {
    ncclComm_t comm;
    int rank, size;
};

int tp_rank(void* c) { return c ? static_cast<TpComm*>(c)->rank : 0; }
int tp_size(void* c) { return c ? static_cast<TpComm*>(c)->size : 1; }

int tp_allreduce_sum_i32(void* c, int32_t* buf, size_t n, cudaStream_t st) {
    TpComm* t = static_cast<TpComm*>(c);
    return g_nccl.AllReduce(buf, buf, n, ncclInt32, ncclSum, t->comm, st) == ncclSuccess ? ROTOR_B200_OK
                                                                                           : ROTOR_B200_ERR_CUDA;
}
int tp_allreduce_f32(void* c, float* buf, size_t n, bool max_op, cudaStream_t st) {
    TpComm* t = static_cast<TpComm*>(c);
    return g_nccl.AllReduce(buf, buf, n, ncclFloat32, max_op ? ncclMax : ncclSum, t->comm, st) == ncclSuccess
               ? ROTOR_B200_OK
               : ROTOR_B200_ERR_CUDA;
}
int tp_allgather_bytes(void* c, const void* send, void* recv, size_t bytes_per_rank, cudaStream_t st) {
    TpComm* t = static_cast<TpComm*>(c);
    return g_nccl.AllGather(send, recv, bytes_per_rank, ncclInt8, t->comm, st) == ncclSuccess ? ROTOR_B200_OK
                                                                                              : ROTOR_B200_ERR_CUDA;
}

}  // namespace rb

using namespace rb;

extern "C" {

int rotor_b200_tp_unique_id(void* out128) {
    RB_REQUIRE(out128);
    int rc = load_nccl();
    if (rc) return rc;
    ncclUniqueId id;
    if (g_nccl.GetUniqueId(&id) != ncclSuccess) return ROTOR_B200_ERR_CUDA;
    static_assert(sizeof(ncclUniqueId) == 128, "unique id is exchanged as 128 bytes");
    memcpy(out128, &id, sizeof(id));
    return ROTOR_B200_OK;
}

int rotor_b200_tp_init(int rank, int size, const void* unique_id128, void** comm) {
    RB_REQUIRE(unique_id128 && comm && size >= 1 && rank >= 0 && rank < size);
    int rc = load_nccl();
    if (rc) return rc;
    ncclUniqueId id;
    memcpy(&id, unique_id128, sizeof(id));
    TpComm* t = new TpComm;
    t->rank = rank;
    t->size = size;
    if (g_nccl.CommInitRank(&t->comm, size, id, rank) != ncclSuccess) {
        delete t;
        return ROTOR_B200_ERR_CUDA;
    }
    *comm = t;
    return ROTOR_B200_OK;
}

void rotor_b200_tp_destroy(void* comm) {
    TpComm* t = static_cast<TpComm*>(comm);
    if (!t) return;
    if (g_nccl.CommDestroy) g_nccl.CommDestroy(t->comm);
    delete t;
}

}  // extern "C"
