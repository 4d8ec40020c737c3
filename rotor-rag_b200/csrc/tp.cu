// Tensor-parallel plumbing: one process per GPU, exchange steps of column/row-parallel
// BitLinear over NVLink (new design: the reference has no multi-device code).
//
// Two transports:
//  * One-shot all-reduce over peer memory (default for the payloads of generation steps, up
//    to XCH_CAP 32-bit elements).  Every rank owns an exchange buffer that its peers map
//    with CUDA IPC.  A rank pushes each element to every peer as one 64-bit store
//    {value, generation}; the same thread then polls its own buffer until the word of every
//    source carries the current generation and reduces in rank order (so all ranks hold
//    identical bits).  One NVLink crossing, no fence, no second kernel.  Two slots alternate
//    with the generation; a slot is rewritten two collectives later, which a peer can only
//    reach after this rank has finished reading it.  Polls are bounded by a cycle count and
//    report through the library status word.
//  * NCCL for everything else (large prefill payloads, the pick all-gather, set-up).  NCCL is
//    bound at run time (dlopen of libnccl.so.2) so that the library has no link-time
//    dependency on a particular NCCL build and shares the copy the host process loaded.
// Collectives are enqueued on the caller's stream between this library's kernels.
#include <dlfcn.h>
#include <nccl.h>  // types and enums only; every function is resolved with dlsym

#include <cstdlib>
#include <cstring>

#include "model.cuh"
#include "xch.cuh"

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

// Device view of the exchange: rank r's buffer is uint2 [2 slots][size][XCH_CAP].
struct XchDev {
    uint2* buf[XCH_MAX_RANKS];  // this process's mapping of every rank's buffer (own included)
    unsigned* seq;              // collectives completed so far (device memory: graph replays advance it)
    unsigned* done;             // CTAs of the running collective that have finished
    unsigned* status;           // library status word
    long long spin;             // SM cycles a poll may wait before it gives up
    int rank, size;
};

struct TpComm {
    ncclComm_t comm;
    int rank, size;
    bool oneshot;               // peer-memory exchange is set up
    XchDev x;
    void* own;                  // this rank's exchange buffer (cudaMalloc)
    void* peer[XCH_MAX_RANKS];  // IPC mappings to close
    unsigned* ctr;              // seq, done (self-advancing collectives); seq2 (step-advanced exchanges)
    XchDev fused;               // vector exchange of the generation-step path (own buffer region, seq2)
    XchScalarDev scalar;        // scalar ring of the generation-step path
};

enum { XOP_SUM_I32 = 0, XOP_SUM_F32 = 1, XOP_MAX_F32 = 2 };

template <int OP>
__device__ __forceinline__ unsigned xch_reduce(unsigned a, unsigned b) {
    if (OP == XOP_SUM_I32) return (unsigned)((int)a + (int)b);
    if (OP == XOP_SUM_F32) return __float_as_uint(__fadd_rn(__uint_as_float(a), __uint_as_float(b)));
    return __float_as_uint(fmaxf(__uint_as_float(a), __uint_as_float(b)));
}

template <int OP>
__global__ void __launch_bounds__(256) oneshot_allreduce_kernel(const __grid_constant__ XchDev t,
                                                                const unsigned* in, unsigned* out, int n) {
    const unsigned seq = *reinterpret_cast<volatile unsigned*>(t.seq);
    const unsigned gen = seq + 1u;  // never matches what a slot held two collectives ago, nor the zero fill
    const size_t slot = (size_t)(gen & 1u) * t.size;
    // a wait that ran out earlier (status word set) is not repeated: later collectives finish at once
    bool failed = *reinterpret_cast<volatile unsigned*>(t.status) != 0;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const unsigned v = in[i];
        for (int p = 0; p < t.size; ++p)
            if (p != t.rank) st_pair(t.buf[p] + (slot + t.rank) * XCH_CAP + i, v, gen);
        unsigned acc = 0;
        for (int src = 0; src < t.size; ++src) {
            unsigned x = v;
            if (src != t.rank) {
                const uint2* w = t.buf[t.rank] + (slot + src) * XCH_CAP + i;
                uint2 got = ld_pair(w);
                if (got.y != gen && !failed) {
                    const long long t0 = clock64();
                    while ((got = ld_pair(w)).y != gen) {
                        if (clock64() - t0 > t.spin) {
                            failed = true;
                            atomicExch(t.status, 0x7e000000u | (unsigned)src);
                            break;
                        }
                    }
                }
                x = got.x;
            }
            acc = src == 0 ? x : xch_reduce<OP>(acc, x);
        }
        out[i] = acc;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(t.done, 1u) == gridDim.x - 1) {  // every CTA has read seq by now
            *t.done = 0;
            __threadfence();
            *reinterpret_cast<volatile unsigned*>(t.seq) = seq + 1u;
        }
    }
}

template <int OP>
static int launch_oneshot(TpComm* t, const void* in, void* out, size_t n, cudaStream_t st) {
    int grid = (int)((n + 255) / 256);
    if (grid > 64) grid = 64;
    oneshot_allreduce_kernel<OP><<<grid, 256, 0, st>>>(t->x, (const unsigned*)in, (unsigned*)out, (int)n);
    return launch_status();
}


// Vector exchange of the generation-step path: int32 partial sums of a row-parallel product are
// summed across ranks and dequantised in one pass, y = (float)sum * sx[row] * scale -- the
// arithmetic of the single-GPU product epilogue.  Generation = step counter + 1 + idx; the
// counter is advanced once per step by xch_bump_kernel.  `slotsel` alternates between the two
// vector exchanges of a block.
__global__ void __launch_bounds__(256) oneshot_allreduce_dequant_kernel(const __grid_constant__ XchDev t, int slotsel,
                                                                        int idx, const int* part, const float* sx,
                                                                        float scale, float* y, int rows, int n) {
    const unsigned gen = *reinterpret_cast<const volatile unsigned*>(t.seq) + 1u + (unsigned)idx;
    const size_t slot = (size_t)slotsel * t.size;
    const int total = rows * n;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int v = part[i];
        for (int p = 0; p < t.size; ++p)
            if (p != t.rank) st_pair(t.buf[p] + (slot + t.rank) * XCH_CAP + i, (unsigned)v, gen);
        int acc = 0;
        for (int src = 0; src < t.size; ++src)
            acc += src == t.rank ? v : (int)xch_poll(t.buf[t.rank] + (slot + src) * XCH_CAP + i, gen, t.status, src, t.spin);
        y[i] = __fmul_rn(__fmul_rn((float)acc, sx[i / n]), scale);
    }
}

__global__ void xch_bump_kernel(unsigned* seq, unsigned n) { *seq += n; }

bool tp_fused_ready(void* c) { return c && static_cast<TpComm*>(c)->oneshot; }
XchScalarDev tp_scalar_dev(void* c) { return static_cast<TpComm*>(c)->scalar; }
int tp_allreduce_dequant(void* c, int slotsel, int idx, const int32_t* part, const float* sx, float scale, float* y,
                         int rows, int n, cudaStream_t st) {
    TpComm* t = static_cast<TpComm*>(c);
    if (!t->oneshot || (size_t)rows * n > (size_t)XCH_CAP) return ROTOR_B200_ERR_ARG;
    int grid = (rows * n + 255) / 256;
    if (grid > 64) grid = 64;
    oneshot_allreduce_dequant_kernel<<<grid, 256, 0, st>>>(t->fused, slotsel & 1, idx, part, sx, scale, y, rows, n);
    return launch_status();
}
int tp_step_end(void* c, int nexchanges, cudaStream_t st) {
    TpComm* t = static_cast<TpComm*>(c);
    xch_bump_kernel<<<1, 1, 0, st>>>(t->ctr + 2, (unsigned)nexchanges);
    return launch_status();
}

// Peer-memory set-up: allocate and zero the exchange buffer, swap IPC handles through the
// NCCL communicator, map every peer.  Failure leaves the communicator on NCCL alone.
static int setup_oneshot(TpComm* t) {
    if (t->size > XCH_MAX_RANKS || t->size < 2) return ROTOR_B200_ERR_ARG;
    const size_t big = 2 * (size_t)t->size * XCH_CAP;             // uint2 words of one vector-exchange region
    const size_t ring = (size_t)XS_RING * t->size * XS_ROWS;      // uint2 words of the scalar ring
    const size_t bytes = (2 * big + ring) * sizeof(uint2);
    unsigned char* scratch = nullptr;
    RB_CUDA(cudaMalloc(&t->own, bytes));
    RB_CUDA(cudaMalloc(&t->ctr, 4 * sizeof(unsigned)));
    RB_CUDA(cudaMalloc(&scratch, (size_t)(t->size + 1) * sizeof(cudaIpcMemHandle_t)));
    RB_CUDA(cudaMemset(t->own, 0, bytes));
    RB_CUDA(cudaMemset(t->ctr, 0, 4 * sizeof(unsigned)));
    cudaIpcMemHandle_t mine, all[XCH_MAX_RANKS];
    RB_CUDA(cudaIpcGetMemHandle(&mine, t->own));
    RB_CUDA(cudaMemcpy(scratch, &mine, sizeof(mine), cudaMemcpyHostToDevice));
    RB_CUDA(cudaDeviceSynchronize());  // the zero fill is done before any peer can learn the handle
    if (g_nccl.AllGather(scratch, scratch + sizeof(mine), sizeof(mine), ncclInt8, t->comm, nullptr) != ncclSuccess)
        return ROTOR_B200_ERR_CUDA;
    RB_CUDA(cudaDeviceSynchronize());
    RB_CUDA(cudaMemcpy(all, scratch + sizeof(mine), (size_t)t->size * sizeof(mine), cudaMemcpyDeviceToHost));
    cudaFree(scratch);
    for (int p = 0; p < t->size; ++p) {
        if (p == t->rank) {
            t->x.buf[p] = (uint2*)t->own;
            continue;
        }
        RB_CUDA(cudaIpcOpenMemHandle(&t->peer[p], all[p], cudaIpcMemLazyEnablePeerAccess));
        t->x.buf[p] = (uint2*)t->peer[p];
    }
    t->x.seq = t->ctr;
    t->x.done = t->ctr + 1;
    t->x.status = library_status_word();
    t->x.spin = XCH_SPIN_CYCLES;
    t->x.rank = t->rank;
    t->x.size = t->size;
    if (!t->x.status) return ROTOR_B200_ERR_CUDA;
    t->fused = t->x;
    t->fused.seq = t->ctr + 2;
    t->fused.done = nullptr;
    t->scalar.seq = t->ctr + 2;
    t->scalar.status = t->x.status;
    t->scalar.spin = XCH_SPIN_CYCLES;
    t->scalar.rank = t->rank;
    t->scalar.size = t->size;
    for (int p = 0; p < t->size; ++p) {
        t->fused.buf[p] = t->x.buf[p] + big;
        t->scalar.buf[p] = t->x.buf[p] + 2 * big;
    }
    t->oneshot = true;
    return ROTOR_B200_OK;
}

static void teardown_oneshot(TpComm* t) {
    cudaDeviceSynchronize();  // everything pushed to this rank belongs to collectives it has finished
    for (int p = 0; p < XCH_MAX_RANKS; ++p)
        if (t->peer[p]) cudaIpcCloseMemHandle(t->peer[p]);
    if (t->own) cudaFree(t->own);
    if (t->ctr) cudaFree(t->ctr);
}

int tp_rank(void* c) { return c ? static_cast<TpComm*>(c)->rank : 0; }
int tp_size(void* c) { return c ? static_cast<TpComm*>(c)->size : 1; }

int tp_allreduce_sum_i32(void* c, int32_t* buf, size_t n, cudaStream_t st) {
    TpComm* t = static_cast<TpComm*>(c);
    if (t->oneshot && n <= (size_t)XCH_CAP) return launch_oneshot<XOP_SUM_I32>(t, buf, buf, n, st);
    return g_nccl.AllReduce(buf, buf, n, ncclInt32, ncclSum, t->comm, st) == ncclSuccess ? ROTOR_B200_OK
                                                                                           : ROTOR_B200_ERR_CUDA;
}
int tp_allreduce_f32(void* c, float* buf, size_t n, bool max_op, cudaStream_t st) {
    TpComm* t = static_cast<TpComm*>(c);
    if (t->oneshot && n <= (size_t)XCH_CAP)
        return max_op ? launch_oneshot<XOP_MAX_F32>(t, buf, buf, n, st) : launch_oneshot<XOP_SUM_F32>(t, buf, buf, n, st);
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
    TpComm* t = new TpComm();
    t->rank = rank;
    t->size = size;
    if (g_nccl.CommInitRank(&t->comm, size, id, rank) != ncclSuccess) {
        delete t;
        return ROTOR_B200_ERR_CUDA;
    }
    // ROTOR_B200_TP_NCCL=1 keeps every collective on NCCL (the comparison baseline)
    const char* only_nccl = getenv("ROTOR_B200_TP_NCCL");
    if (size > 1 && !(only_nccl && only_nccl[0] == '1')) {
        rc = setup_oneshot(t);
        if (rc) {  // all ranks must agree on the transport: a rank that cannot map its peers fails the init
            teardown_oneshot(t);
            g_nccl.CommDestroy(t->comm);
            delete t;
            return rc;
        }
    }
    *comm = t;
    return ROTOR_B200_OK;
}

/* Self-test of the bounded waits of the peer-memory exchange, on ONE GPU: a two-rank exchange whose
 * "peer" buffer is a second allocation on this device that nothing ever writes, so the poll for
 * the peer's words must run out after `spin_cycles` SM cycles.  Runs the all-reduce twice: the
 * first launch has to give up and set the status word; the second (with a limit of about a
 * second) has to see the word and return at once.  status_out receives the word after the first
 * launch, second_ms the device time of the second launch.  The status word stays set: the caller
 * reads and clears it with rotor_b200_device_status(). */
int rotor_b200_selftest_exchange_timeout(long long spin_cycles, unsigned* status_out, float* second_ms) {
    RB_REQUIRE(spin_cycles > 0 && spin_cycles <= XCH_SPIN_CYCLES && status_out && second_ms);
    const size_t words = 2 * 2 * (size_t)XCH_CAP;  // two slots, two ranks
    uint2 *own = nullptr, *peer = nullptr;
    unsigned* ctr = nullptr;
    int* data = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    int rc = ROTOR_B200_ERR_CUDA;
    const int n = 1024;
    do {
        if (cudaMalloc(&own, words * sizeof(uint2)) != cudaSuccess || cudaMalloc(&peer, words * sizeof(uint2)) != cudaSuccess ||
            cudaMalloc(&ctr, 2 * sizeof(unsigned)) != cudaSuccess || cudaMalloc(&data, 2 * n * sizeof(int)) != cudaSuccess)
            break;
        if (cudaMemset(own, 0, words * sizeof(uint2)) != cudaSuccess || cudaMemset(peer, 0, words * sizeof(uint2)) != cudaSuccess ||
            cudaMemset(ctr, 0, 2 * sizeof(unsigned)) != cudaSuccess || cudaMemset(data, 0, 2 * n * sizeof(int)) != cudaSuccess)
            break;
        XchDev x = {};
        x.buf[0] = own;
        x.buf[1] = peer;
        x.seq = ctr;
        x.done = ctr + 1;
        x.status = library_status_word();
        x.spin = spin_cycles;
        x.rank = 0;
        x.size = 2;
        if (!x.status) break;
        if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) break;
        oneshot_allreduce_kernel<XOP_SUM_I32><<<4, 256>>>(x, (const unsigned*)data, (unsigned*)data + n, n);
        if (launch_status() || cudaDeviceSynchronize() != cudaSuccess) break;
        if (cudaMemcpy(status_out, x.status, sizeof(unsigned), cudaMemcpyDeviceToHost) != cudaSuccess) break;
        x.spin = XCH_SPIN_CYCLES;  // would take about a second per source if the set status word were ignored
        cudaEventRecord(e0);
        oneshot_allreduce_kernel<XOP_SUM_I32><<<4, 256>>>(x, (const unsigned*)data, (unsigned*)data + n, n);
        cudaEventRecord(e1);
        if (launch_status() || cudaDeviceSynchronize() != cudaSuccess) break;
        if (cudaEventElapsedTime(second_ms, e0, e1) != cudaSuccess) break;
        rc = ROTOR_B200_OK;
    } while (0);
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    cudaFree(own);
    cudaFree(peer);
    cudaFree(ctr);
    cudaFree(data);
    return rc;
}

void rotor_b200_tp_destroy(void* comm) {
    TpComm* t = static_cast<TpComm*>(comm);
    if (!t) return;
    teardown_oneshot(t);
    if (g_nccl.CommDestroy) g_nccl.CommDestroy(t->comm);
    delete t;
}

}  // extern "C"
