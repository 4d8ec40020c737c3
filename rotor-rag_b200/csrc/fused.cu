// Generation-step BitLinear product with the vector stage that feeds it fused in.
//
// One CTA per SM, FG_THREADS threads.  Every CTA owns whole row tiles (16 output rows each,
// full K), so no partial sum ever leaves the CTA: the warps split the CTA's tiles -- taken
// in memory order, one contiguous span of HBM per CTA -- and merge their integer partial
// sums in shared memory.  Before the tile products the CTA builds the int8 activation
// row(s) in registers and shared memory from the producer's float32 output (residual add,
// sub-norm, pre-norm, absmax quantise: leanstage.cuh), work that would otherwise be a
// separate single-CTA launch between two products.  After them it dequantises its rows
// and writes finished float32 outputs; the gate/up product, whose CTAs own matching row
// tiles of both halves, applies the gating there as well.
#include "gemv_core.cuh"
#include "leanstage.cuh"

RB_TRACE_DEFINE(rotor_b200_trace_read_fused)

namespace rb {

constexpr int FG_THREADS = 1024;
constexpr int FG_WARPS = FG_THREADS / 32;
constexpr int FG_U = 4;  // weight tiles in flight per warp
constexpr int FG_V = 2;  // float4 groups per thread in the prologue: input width <= 8192

struct FusedGemvParams {
    const uint4* tiles;   // tiles of the (stacked) matrix
    int nkt;              // K tiles per row tile
    int units;            // row tiles per half (paired) or in all (plain)
    int halves;           // 2: rows u and units*16 + u form one output (gate/up); 1 otherwise
    int out;              // output rows per half
    int rows, cols;       // token rows, activation columns (= rows * st.terms)
    int upc;              // units per CTA (ceil)
    LeanStage st;
    float* y;             // [rows][out] float32 outputs
    float scale[3];       // per-tensor weight scales of up to three stacked row segments
    int seg1, seg2;       // first row of the second / third segment (plain); halves == 2: scale[0]=gate, [1]=up
    int ffn_act;
};

template <bool USE_MMA, int NCOL>
__global__ void __launch_bounds__(FG_THREADS, 1) fused_gemv_kernel(const __grid_constant__ FusedGemvParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ float s_sx[8];
    __shared__ int s_xsum[8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int kpad = p.nkt * TILE_K;
    const int xs_stride = kpad + XS_PAD;
    const int slots = p.upc * p.halves;
    int8_t* xs = reinterpret_cast<int8_t*>(smem_raw);                            // [cols][xs_stride]
    int* merge = reinterpret_cast<int*>(smem_raw + (size_t)p.cols * xs_stride);  // [slots][128]
    float* scratch = reinterpret_cast<float*>(merge + slots * 128);             // [64]
    float* aux = scratch + 64;                                                   // attention merge weights

    TraceRec tr;
    RB_STAMP(tr, 0);
    pdl_trigger();

    // units (row tiles / row-tile pairs) of this CTA, and the warp's share of their tiles
    const int u0 = (int)((long long)p.units * blockIdx.x / gridDim.x);
    const int u1 = (int)((long long)p.units * (blockIdx.x + 1) / gridDim.x);
    const int ntile = (u1 - u0) * p.halves * p.nkt;  // local tile index = ((u-u0)*halves + half)*nkt + kt
    const int w0 = (int)((long long)ntile * warp / FG_WARPS), w1 = (int)((long long)ntile * (warp + 1) / FG_WARPS);
    auto tile_ptr = [&](int lt) {
        const int slot = lt / p.nkt, kt = lt - slot * p.nkt;
        const int u = u0 + slot / p.halves, half = slot - (slot / p.halves) * p.halves;
        const size_t rt = (size_t)half * p.units + u;
        return p.tiles + (rt * p.nkt + kt) * 32 + lane;
    };
    uint4 wv[FG_U];
#pragma unroll
    for (int u = 0; u < FG_U; ++u)
        if (w0 + u < w1) wv[u] = ld_stream_v4(tile_ptr(w0 + u));
    for (int e = threadIdx.x; e < slots * 128; e += FG_THREADS) merge[e] = 0;
    RB_STAMP(tr, 1);

    pdl_wait();  // the weights above are constants; everything below depends on earlier kernels
    RB_STAMP(tr, 2);

    // ---- prologue: activation rows -> int8 in shared memory
    const bool writer = blockIdx.x == 0;
    for (int m = 0; m < p.rows; ++m) {
        float4 v[FG_V];
        lean_row<FG_V>(p.st, m, v, scratch, aux, writer);
        lean_quantize<FG_V>(p.st, v, scratch, xs + (size_t)m * p.st.terms * xs_stride, (size_t)xs_stride,
                            s_sx + m * p.st.terms, s_xsum + m * p.st.terms);
    }
    __syncthreads();
    RB_STAMP(tr, 3);

    // ---- integer tile products over the warp's range
    int accm[4][4];
    int accd[2][4][NCOL];
    auto clear = [&]() {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int r = 0; r < 4; ++r) accm[j][r] = 0;
#pragma unroll
            for (int c = 0; c < NCOL; ++c) accd[0][j][c] = accd[1][j][c] = 0;
        }
    };
    auto flush = [&](int slot) {  // exact rescale of the per-bit-pair sums, then into the slot
        int* dst = merge + slot * 128;
        if constexpr (USE_MMA) {
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int v = accm[0][r] + (accm[1][r] >> 2) + (accm[2][r] >> 4) + (accm[3][r] >> 6);
                atomicAdd(dst + (g + 8 * (r >> 1)) * 8 + 2 * t + (r & 1), v);
            }
        } else {
#pragma unroll
            for (int rh = 0; rh < 2; ++rh)
#pragma unroll
                for (int c = 0; c < NCOL; ++c) {
                    int v = accd[rh][0][c] + (accd[rh][1][c] >> 2) + (accd[rh][2][c] >> 4) + (accd[rh][3][c] >> 6);
                    v += __shfl_xor_sync(0xffffffffu, v, 1);
                    v += __shfl_xor_sync(0xffffffffu, v, 2);
                    if (t == 0) atomicAdd(dst + (g + 8 * rh) * 8 + c, v);
                }
        }
    };
    clear();
    int cur = -1;
    for (int base = w0; base < w1; base += FG_U) {
#pragma unroll
        for (int u = 0; u < FG_U; ++u) {
            const int lt = base + u;
            if (lt < w1) {
                const int slot = lt / p.nkt, kt = lt - slot * p.nkt;
                if (slot != cur) {  // warp-uniform
                    if (cur >= 0) flush(cur);
                    clear();
                    cur = slot;
                }
                const uint32_t pw[4] = {wv[u].x, wv[u].y, wv[u].z, wv[u].w};
                tile_mac<USE_MMA, NCOL>(pw, xs, xs_stride, kt * TILE_K + 32 * t, g, p.cols, accm, accd);
            }
        }
#pragma unroll
        for (int u = 0; u < FG_U; ++u)
            if (base + FG_U + u < w1) wv[u] = ld_stream_v4(tile_ptr(base + FG_U + u));
    }
    if (cur >= 0) flush(cur);
    __syncthreads();
    RB_STAMP(tr, 4);

    // ---- epilogue: the CTA's rows are complete: remove the +1 code offset, dequantise, write
    const int T = p.st.terms;
    for (int e = threadIdx.x; e < (u1 - u0) * 16 * p.rows; e += FG_THREADS) {
        const int m = e % p.rows, rl = (e / p.rows) & 15, lu = e / (p.rows * 16);
        const int orow = (u0 + lu) * TILE_ROWS + rl;
        if (orow >= p.out) continue;
        float val[2] = {0.f, 0.f};
        for (int half = 0; half < p.halves; ++half) {
            const int* src = merge + (lu * p.halves + half) * 128 + rl * 8 + m * T;
            float f = 0.f;
            for (int tt = 0; tt < T; ++tt) f += (float)(src[tt] - s_xsum[m * T + tt]) * s_sx[m * T + tt];
            val[half] = f;
        }
        float r;
        if (p.halves == 2) {
            const float gt = val[0] * p.scale[0], up = val[1] * p.scale[1];
            if (p.ffn_act == ROTOR_B200_FFN_RELU2) {
                const float q = fmaxf(gt, 0.f);
                r = q * q * up;
            } else {
                const float c = fminf(fmaxf(up, -20.f), 20.f);
                r = gt * (c / (1.f + expf(-c)));
            }
        } else {
            r = val[0] * (orow < p.seg1 ? p.scale[0] : (orow < p.seg2 ? p.scale[1] : p.scale[2]));
        }
        p.y[(size_t)m * p.out + orow] = r;
    }
    RB_STAMP(tr, 5);
    RB_TRACE_COMMIT(tr, p.st.mode * 10 + p.halves);
}

static int g_sm_count = 0;
static int sm_count() {
    if (!g_sm_count) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || g_sm_count <= 0)
            g_sm_count = 148;
    }
    return g_sm_count;
}

static size_t fused_smem(const FusedGemvParams& p) {
    const size_t xs = (size_t)p.cols * (p.nkt * TILE_K + XS_PAD);
    const size_t aux = p.st.mode == LM_ATTN ? 2 * (size_t)p.st.n_heads * p.st.nsplit : 0;
    return xs + (size_t)p.upc * p.halves * 512 + (64 + aux) * sizeof(float);
}

template <bool USE_MMA, int NCOL>
static int launch_fused(const FusedGemvParams& p, int grid, cudaStream_t st) {
    const size_t smem = fused_smem(p);
    if (smem > 200 * 1024) return ROTOR_B200_ERR_SHAPE;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(FG_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_use_pdl ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, fused_gemv_kernel<USE_MMA, NCOL>, p) != cudaSuccess) {
        ++g_launch_count;
        return ROTOR_B200_ERR_CUDA;
    }
    return launch_status();
}

int configure_fused_gemv() {
    RB_CUDA(cudaFuncSetAttribute(fused_gemv_kernel<false, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    RB_CUDA(cudaFuncSetAttribute(fused_gemv_kernel<false, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    RB_CUDA(cudaFuncSetAttribute(fused_gemv_kernel<true, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    sm_count();
    return ROTOR_B200_OK;
}

// Whether a product with input width `in` fits this path for `rows` token rows of `terms`
// activation terms each.
bool fused_gemv_supported(size_t out, size_t in, int rows, int terms, int halves, int merge_weights) {
    const int cols = rows * terms;
    if (rows < 1 || cols > 8 || terms > 3 || in % 4 || in > 4 * FG_V * FG_THREADS) return false;
    FusedGemvParams p = {};
    p.cols = cols;
    p.nkt = (int)(kpad_of(in) / TILE_K);
    p.halves = halves;
    const int units = (int)(opad_of(out) / TILE_ROWS);
    p.upc = (units + sm_count() - 1) / sm_count();
    p.st.mode = merge_weights ? LM_ATTN : LM_ADD;
    p.st.n_heads = merge_weights;
    p.st.nsplit = 1;
    return fused_smem(p) <= 160 * 1024;
}

// out: output rows per half.  halves == 2: `tiles` holds the gate matrix followed by the up
// matrix (each `out` rows), y receives the gated product, scale = {gate, up}.  halves == 1:
// y receives the product scaled per row segment: rows < seg1 by scale[0], < seg2 by
// scale[1], the rest by scale[2].
int launch_fused_gemv(const void* tiles, size_t out, size_t in, int halves, int rows, const LeanStage& stage, float* y,
                      const float* scale, int seg1, int seg2, int ffn_act, cudaStream_t st) {
    FusedGemvParams p = {};
    p.tiles = (const uint4*)tiles;
    p.nkt = (int)(kpad_of(in) / TILE_K);
    p.units = (int)(opad_of(out) / TILE_ROWS);
    p.halves = halves;
    p.out = (int)out;
    p.rows = rows;
    p.cols = rows * stage.terms;
    p.st = stage;
    p.y = y;
    p.scale[0] = scale[0];
    p.scale[1] = scale[1];
    p.scale[2] = scale[2];
    p.seg1 = seg1;
    p.seg2 = seg2;
    p.ffn_act = ffn_act;
    if (p.cols < 1 || p.cols > 8 || stage.terms > 3 || halves < 1 || halves > 2) return ROTOR_B200_ERR_ARG;
    if (halves == 2 && out % TILE_ROWS) return ROTOR_B200_ERR_SHAPE;
    if (stage.n != (int)in || in % 4 || in > 4 * FG_V * FG_THREADS) return ROTOR_B200_ERR_SHAPE;
    int grid = sm_count();
    if (grid > p.units) grid = p.units;
    p.upc = (p.units + grid - 1) / grid;
    if (p.cols == 1) return launch_fused<false, 1>(p, grid, st);
    if (p.cols == 2) return launch_fused<false, 2>(p, grid, st);
    return launch_fused<true, 1>(p, grid, st);
}

}  // namespace rb
