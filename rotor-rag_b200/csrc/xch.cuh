// Device side of the tensor-parallel exchanges that run INSIDE the generation-step kernels.
//
// Every rank owns a small ring of exchange slots in memory its peers have mapped (CUDA IPC).
// A value crosses NVLink as one 64-bit store {bits, generation}; the receiver polls its own
// memory until the word carries the generation it expects.  Generations come from a device
// counter that the last kernel of a step advances by the number of exchanges in the step, so a
// captured graph replays with fresh generations.  Polls are bounded: a wait that runs out sets
// the library status word and later waits return at once.
#pragma once
#include "common.cuh"

namespace rb {

constexpr int XCH_MAX_RANKS = 8;
constexpr int XCH_CAP = 1 << 16;   // 32-bit elements per one-shot vector exchange
constexpr int XS_RING = 16;        // scalar exchange slots; a rank is never more than two kernels ahead of a peer
constexpr int XS_ROWS = 8;         // token rows per scalar exchange
constexpr long long XCH_SPIN_CYCLES = 2000000000LL;  // default limit of a wait: about one second

// One float per token row, exchanged by every CTA of a kernel.
struct XchScalarDev {
    uint2* buf[XCH_MAX_RANKS];  // this process's mapping of every rank's ring: uint2 [XS_RING][size][XS_ROWS]
    const unsigned* seq;        // exchanges completed before this step
    unsigned* status;
    long long spin;             // SM cycles a poll may wait before it gives up
    int rank, size;             // size == 0: no exchange (single GPU)
};

__device__ __forceinline__ void st_pair(uint2* p, unsigned v, unsigned g) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(v), "r"(g) : "memory");
}
__device__ __forceinline__ uint2 ld_pair(const uint2* p) {
    uint2 r;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p) : "memory");
    return r;
}

// Polls a local exchange word for generation `gen`; `src` only labels the status code.
__device__ __forceinline__ unsigned xch_poll(const uint2* w, unsigned gen, unsigned* status, int src, long long spin) {
    uint2 got = ld_pair(w);
    if (got.y != gen && *reinterpret_cast<volatile unsigned*>(status) == 0) {
        const long long t0 = clock64();
        while ((got = ld_pair(w)).y != gen) {
            if (clock64() - t0 > spin || *reinterpret_cast<volatile unsigned*>(status) != 0) {
                atomicCAS(status, 0u, 0x7e000000u | (unsigned)src);
                break;
            }
        }
    }
    return got.x;
}

// All-reduce (sum or max) of one float per token row across ranks, called by ALL threads of
// EVERY CTA of the kernel with the same `v` (the CTAs compute it redundantly).  Exchange `idx`
// of the step, row `row`.  The writer CTA pushes this rank's value to the peers; every CTA
// polls its own memory for theirs and folds in rank order, so all CTAs of all ranks get the
// same bits.  `scratch`: at least XCH_MAX_RANKS shared floats.  Uses the CTA barrier.
__device__ __forceinline__ float xch_scalar(const XchScalarDev& x, int idx, int row, float v, bool is_max,
                                            bool writer, float* scratch) {
    const unsigned gen = *reinterpret_cast<const volatile unsigned*>(x.seq) + 1u + (unsigned)idx;
    const size_t slot = (size_t)(gen % XS_RING) * x.size;
    __syncthreads();  // earlier readers of `scratch` are done
    if ((int)threadIdx.x < x.size) {
        const int peer = threadIdx.x;
        float val = v;
        if (peer != x.rank) {
            if (writer) st_pair(x.buf[peer] + (slot + x.rank) * XS_ROWS + row, __float_as_uint(v), gen);
            val = __uint_as_float(xch_poll(x.buf[x.rank] + (slot + peer) * XS_ROWS + row, gen, x.status, peer, x.spin));
        }
        scratch[peer] = val;
    }
    __syncthreads();
    float r = scratch[0];
    for (int k = 1; k < x.size; ++k) r = is_max ? fmaxf(r, scratch[k]) : __fadd_rn(r, scratch[k]);
    __syncthreads();
    return r;
}

}  // namespace rb
