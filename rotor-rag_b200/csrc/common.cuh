// Shared declarations for the sm_100a kernels behind librotor_b200.so.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>

#include "../../include/rotor_b200.h"

namespace rb {

// Weight tile: 16 output rows x 128 input columns, 512 bytes, one uint4 per lane.
constexpr int TILE_ROWS = 16;
constexpr int TILE_K = 128;
constexpr int TILE_BYTES = 512;

__host__ __device__ inline size_t round_up(size_t v, size_t m) { return (v + m - 1) / m * m; }
__host__ __device__ inline size_t kpad_of(size_t in) { return round_up(in, TILE_K); }
__host__ __device__ inline size_t opad_of(size_t out) { return round_up(out, TILE_ROWS); }

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// State kept once per device: a process may drive several GPUs, and function attributes
// (shared-memory opt-in), the status word and device properties belong to one of them.
constexpr int RB_MAX_DEVICES = 64;
inline int current_device() {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= RB_MAX_DEVICES) d = 0;
    return d;
}
template <typename T>
struct PerDevice {
    T v[RB_MAX_DEVICES] = {};
    T& here() { return v[current_device()]; }
};

// Kernel launches issued by this library in this process (graph replays add the launches
// the graph holds).  Defined in format.cu.
extern unsigned long long g_launch_count;

// Called right after every kernel launch: counts it and maps the last CUDA error to the
// library's status codes.
inline int launch_status() {
    ++g_launch_count;
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? ROTOR_B200_OK : ROTOR_B200_ERR_CUDA;
}

#define RB_REQUIRE(cond)                     \
    do {                                     \
        if (!(cond)) return ROTOR_B200_ERR_ARG; \
    } while (0)

#define RB_CUDA(call)                                        \
    do {                                                     \
        if ((call) != cudaSuccess) return ROTOR_B200_ERR_CUDA; \
    } while (0)

// ---------------------------------------------------------------- device helpers
#ifdef __CUDACC__

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ int warp_sum_i(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Block-wide reductions over up to 1024 threads.  `scratch` holds 33 floats.
// Every thread receives the result.  Two barriers per call.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[w] = v;
    __syncthreads();
    float r = (lane < nw) ? scratch[lane] : 0.f;
    return warp_sum(r);
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[w] = v;
    __syncthreads();
    float r = (lane < nw) ? scratch[lane] : -3.4e38f;
    return warp_max(r);
}
__device__ __forceinline__ int block_sum_i(int v, int* scratch) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum_i(v);
    __syncthreads();
    if (lane == 0) scratch[w] = v;
    __syncthreads();
    int r = (lane < nw) ? scratch[lane] : 0;
    return warp_sum_i(r);
}

// One-barrier variants for chains of reductions: `scratch` holds 64 floats used as two halves that
// successive calls alternate between (`k` counts the calls).  A half is rewritten only two calls
// later, and the barrier of the call in between orders that write after every read of this one.
// Nothing else may touch `scratch` between calls without a CTA barrier of its own.
__device__ __forceinline__ float block_sum_alt(float v, float* scratch, int& k) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    float* s = scratch + 32 * (k++ & 1);
    v = warp_sum(v);
    if (lane == 0) s[w] = v;
    __syncthreads();
    float r = (lane < nw) ? s[lane] : 0.f;
    return warp_sum(r);
}
__device__ __forceinline__ float block_max_alt(float v, float* scratch, int& k) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    float* s = scratch + 32 * (k++ & 1);
    v = warp_max(v);
    if (lane == 0) s[w] = v;
    __syncthreads();
    float r = (lane < nw) ? s[lane] : -3.4e38f;
    return warp_max(r);
}

// L2 prefetch of the 128-byte line that holds `p` (constants a kernel will need after its
// programmatic-launch wait).
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// Streaming 128-bit load that bypasses L1 (weights are read exactly once).
__device__ __forceinline__ uint4 ld_stream_v4(const uint4* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

// Programmatic dependent launch: a kernel launched with the attribute may start while its
// predecessor in the stream is still running.  pdl_trigger() lets the successor start
// early; pdl_wait() blocks until every predecessor grid has completed and its writes are
// visible.  Both are no-ops for a kernel launched without the attribute.
//
// Rule followed by every kernel of the generation step: pdl_wait() first, pdl_trigger() right
// after it.  A successor's code before its own pdl_wait() therefore starts only once the
// predecessor has passed its wait, i.e. once everything launched before the predecessor is
// complete: that code may read constants (weights) and anything written two or more kernels
// earlier (the cached length, older KV-cache rows), never the predecessor's outputs, and
// writes nothing outside its own CTA.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Optional device-side timeline (compiled in with -DRB_TRACE): thread 0 of CTA 0 of the
// instrumented kernels records %globaltimer stamps into a global ring for offline reading.
#ifdef RB_TRACE
struct TraceRec {
    unsigned long long t[8];
    int kind;
    int pad;
};
// each instrumented .cu file holds its own ring (no relocatable device code is used)
#define RB_TRACE_DEFINE(name)                                                         \
    static __device__ rb::TraceRec g_trace[4096];                                       \
    static __device__ unsigned g_trace_n;                                             \
    extern "C" int name(void* host_buf, unsigned* n) {                                \
        unsigned cnt = 0;                                                             \
        cudaMemcpyFromSymbol(&cnt, g_trace_n, sizeof(cnt));                           \
        if (cnt > 4096) cnt = 4096;                                                   \
        cudaMemcpyFromSymbol(host_buf, g_trace, sizeof(rb::TraceRec) * cnt);            \
        unsigned zero = 0;                                                            \
        cudaMemcpyToSymbol(g_trace_n, &zero, sizeof(zero));                           \
        *n = cnt;                                                                     \
        return 0;                                                                     \
    }
__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long v;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(v));
    return v;
}
#define RB_STAMP(rec, i) \
    do {                 \
        if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) (rec).t[i] = gtime(); \
    } while (0)
#define RB_TRACE_COMMIT(rec, k)                                              \
    do {                                                                     \
        if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) {        \
            (rec).kind = (k);                                                \
            unsigned idx_ = atomicAdd(&g_trace_n, 1u);                       \
            if (idx_ < 4096) g_trace[idx_] = (rec);                          \
        }                                                                    \
    } while (0)
#else
struct TraceRec {};
#define RB_TRACE_DEFINE(name)
#define RB_STAMP(rec, i) do {} while (0)
#define RB_TRACE_COMMIT(rec, k) do {} while (0)
#endif

#endif  // __CUDACC__

}  // namespace rb
