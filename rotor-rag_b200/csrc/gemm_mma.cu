// Ternary BitLinear integer core for many activation columns (prompt prefill, M >= 32):
// acc[c][o] = sum_k xq[c][k] * w[o][k], exact int32.
//
// With hundreds of columns the product is compute-bound, not weight-bandwidth-bound, so
// the weights are decoded once per CTA tile and reused across 128 columns.  CTA tile:
// 64 output rows (4 weight row tiles) x 128 columns, K walked one 128-wide weight tile at
// a time.  Eight warps: warp w owns row tile (w & 3) and the column half (w >> 2), i.e.
// a 16 x 64 block of int32 accumulators (8 mma n-tiles).  A warp takes its weight tile
// straight from global memory -- the tile layout is the m16n8k32 A fragment, one 128-bit
// load per lane for all four k32 chunks -- and turns bit pair j into a u8 operand with one
// shift and one AND.  Activation columns are staged per K tile in shared memory with
// cp.async (double buffered); the k order inside a tile makes a lane's B fragment for
// chunk j one 64-bit shared load.  mma.sync.m16n8k32.u8.s8; the "+1" of the weight codes
// is removed with the column sums at the end.
//
// This is the legacy tensor-core path (mma.sync).  It is the correctness baseline for the
// prefill product; the tcgen05/TMEM version is the kernel that belongs here on sm_100a.
#include "gemv_core.cuh"
#include "model.cuh"

namespace rb {

constexpr int GM_ROWS = 64;    // output rows per CTA
constexpr int GM_COLS = 128;   // activation columns per CTA
constexpr int GM_STRIDE = TILE_K + 8;   // bytes per staged column: 34 words, so the 64-bit fragment loads of a
                                        // half warp (banks 2g + 8t) never collide
constexpr int GM_STAGE = GM_COLS * GM_STRIDE;

__device__ __forceinline__ void cp_async8(void* smem, const void* gmem, bool valid) {
    const unsigned s = smem_u32(smem);
    const int sz = valid ? 8 : 0;  // src-size 0: the 8 bytes are zero filled
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(s), "l"(gmem), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

struct GemmParams {
    const uint4* tiles;
    const int8_t* xq;     // [ncols][kpad]
    const int32_t* xsum;  // [ncols]
    int32_t* acc;         // [ncols][out]
    int out, nrt, nkt, ncols;
};

__global__ void __launch_bounds__(256) gemm_mma_kernel(const __grid_constant__ GemmParams p) {
    extern __shared__ __align__(16) unsigned char smem[];  // two stages of [GM_COLS][GM_STRIDE]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int rt = blockIdx.x * 4 + (warp & 3);       // weight row tile of this warp
    const int ch = warp >> 2;                          // column half
    const int col0 = blockIdx.y * GM_COLS;
    const size_t kpad = (size_t)p.nkt * TILE_K;

    int acc[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int r = 0; r < 4; ++r) acc[n][r] = 0;

    // stage loader: 128 columns x 128 bytes = 2048 8-byte pieces, 8 per thread
    auto load_stage = [&](int kt, int stage) {
        unsigned char* dst = smem + stage * GM_STAGE;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int piece = threadIdx.x + i * 256;
            const int c = piece >> 4, off = (piece & 15) * 8;
            const bool valid = col0 + c < p.ncols;
            const int8_t* src = p.xq + (size_t)(valid ? col0 + c : 0) * kpad + (size_t)kt * TILE_K + off;
            cp_async8(dst + c * GM_STRIDE + off, src, valid);
        }
        cp_async_commit();
    };

    const bool row_ok = rt < p.nrt;
    const uint4* trow = p.tiles + (size_t)(row_ok ? rt : 0) * p.nkt * 32 + lane;
    load_stage(0, 0);
    uint4 wcur = row_ok ? ld_stream_v4(trow) : make_uint4(0x55555555u, 0x55555555u, 0x55555555u, 0x55555555u);
    for (int kt = 0; kt < p.nkt; ++kt) {
        const int stage = kt & 1;
        uint4 wnext = wcur;
        if (kt + 1 < p.nkt) {
            load_stage(kt + 1, stage ^ 1);
            if (row_ok) wnext = ld_stream_v4(trow + (size_t)(kt + 1) * 32);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const unsigned char* xs = smem + stage * GM_STAGE + (ch * 64) * GM_STRIDE;
        const uint32_t pw[4] = {wcur.x, wcur.y, wcur.z, wcur.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t a0 = (pw[0] >> (2 * j)) & 0x03030303u, a1 = (pw[1] >> (2 * j)) & 0x03030303u;
            const uint32_t a2 = (pw[2] >> (2 * j)) & 0x03030303u, a3 = (pw[3] >> (2 * j)) & 0x03030303u;
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                const uint2 b = *reinterpret_cast<const uint2*>(xs + (n * 8 + g) * GM_STRIDE + 32 * t + 8 * j);
                mma_u8s8(acc[n], a0, a1, a2, a3, b.x, b.y);
            }
        }
        __syncthreads();  // everyone is done with this stage before it is refilled
        wcur = wnext;
    }

    if (!row_ok) return;
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int col = col0 + ch * 64 + n * 8 + 2 * t + (r & 1);
            const int row = rt * TILE_ROWS + g + 8 * (r >> 1);
            if (col < p.ncols && row < p.out) p.acc[(size_t)col * p.out + row] = acc[n][r] - p.xsum[col];
        }
}

int configure_gemm_mma() {
    RB_CUDA(cudaFuncSetAttribute(gemm_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * GM_STAGE));
    return ROTOR_B200_OK;
}

int launch_gemm_mma(const void* tiles, size_t out, size_t in, const int8_t* xq, const int32_t* xsum, int ncols,
                    int32_t* acc, cudaStream_t st) {
    static PerDevice<bool> once;
    bool& configured = once.here();
    if (!configured) {
        int rc = configure_gemm_mma();
        if (rc) return rc;
        configured = true;
    }
    GemmParams p;
    p.tiles = (const uint4*)tiles;
    p.xq = xq;
    p.xsum = xsum;
    p.acc = acc;
    p.out = (int)out;
    p.nrt = (int)(opad_of(out) / TILE_ROWS);
    p.nkt = (int)(kpad_of(in) / TILE_K);
    p.ncols = ncols;
    dim3 grid((p.nrt + 3) / 4, (ncols + GM_COLS - 1) / GM_COLS);
    gemm_mma_kernel<<<grid, 256, 2 * GM_STAGE, st>>>(p);
    return launch_status();
}

}  // namespace rb
