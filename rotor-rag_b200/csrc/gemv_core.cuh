// Instruction-level pieces shared by the BitLinear product kernels.
#pragma once
#include "common.cuh"

namespace rb {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One 16x128 weight tile against the staged activations.
//   pw       : the lane's four tile words
//   xs       : staged int8 activations, column c at xs + c*xs_stride
//   koff     : byte offset of this tile's 32-column slice for this lane (tile column 32*t)
//   MMA      : accm[j][r] += fragment products for bit pair j (8 columns at once)
//   DP4A     : accd[row half][j][c] for NCOL columns
template <bool USE_MMA, int NCOL>
__device__ __forceinline__ void tile_mac(const uint32_t (&pw)[4], const int8_t* xs, int xs_stride, int koff, int g,
                                         int ncols, int (&accm)[4][4], int (&accd)[2][4][NCOL]) {
    if constexpr (USE_MMA) {
        uint4 xa = make_uint4(0, 0, 0, 0), xb = xa;
        if (g < ncols) {
            const uint4* xp = reinterpret_cast<const uint4*>(xs + (size_t)g * xs_stride + koff);
            xa = xp[0];
            xb = xp[1];
        }
        const uint32_t xw[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t m = 0x03030303u << (2 * j);
            mma_u8s8(accm[j], pw[0] & m, pw[1] & m, pw[2] & m, pw[3] & m, xw[2 * j], xw[2 * j + 1]);
        }
    } else {
#pragma unroll
        for (int c = 0; c < NCOL; ++c) {
            const uint4* xp = reinterpret_cast<const uint4*>(xs + (size_t)c * xs_stride + koff);
            const uint4 xa = xp[0], xb = xp[1];
            const uint32_t xw[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t m = 0x03030303u << (2 * j);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    accd[i & 1][j][c] = dp4a_us(pw[i] & m, xw[2 * j + (i >> 1)], accd[i & 1][j][c]);
            }
        }
    }
}

constexpr int XS_PAD = 16;  // bytes between staged columns: keeps 128-bit fragment loads conflict-free

}  // namespace rb
