// Generation-step BitLinear product with the vector stage that feeds it fused in.
//
// One CTA per SM, FG_THREADS threads (a second CTA slot per SM stays free for the next kernel of
// the step, see below).  Every CTA owns whole row tiles (16 output rows each,
// full K), so no partial sum ever leaves the CTA: the warps split the CTA's tiles -- taken
// in memory order, one contiguous span of HBM per CTA -- and merge their integer partial
// sums in shared memory.  Before the tile products the CTA builds the int8 activation
// row(s) in registers and shared memory from the producer's float32 output (residual add,
// sub-norm, pre-norm, absmax quantise: leanstage.cuh), work that would otherwise be a
// separate single-CTA launch between two products.  After them it dequantises its rows
// and writes finished float32 outputs; the gate/up product, whose CTAs own matching row
// tiles of both halves, applies the gating there as well.
//
// Programmatic dependent launch: everything a product can do without its input -- tile ranges,
// clearing the merge slots, the first weight tiles into registers, further tiles and the norm
// weights into L2 -- happens before griddepcontrol.wait, while the previous kernel of the step is
// still running on the same SMs; the launch gap and the cold start of the weight stream are
// hidden behind that kernel.
#include "product_body.cuh"

RB_TRACE_DEFINE(rotor_b200_trace_read_fused)

namespace rb {

template <bool USE_MMA, int NCOL, bool WIDE, bool DEEP, bool TP>
__global__ void __launch_bounds__(FG_THREADS, DEEP ? 1 : 2) fused_gemv_kernel(const __grid_constant__ FusedGemvParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ float s_sx[8];
    __shared__ int s_xsum[8];
    TraceRec tr;
    RB_STAMP(tr, 0);
    const ProductCtx c = product_ctx(p, smem_raw);
    uint4 wv[FG_U];
    if constexpr (DEEP)
        product_prefetch(p, c, wv);
    else
        product_stage(p, c);
    if constexpr (!WIDE) lean_prefetch(p.st);
    for (int e = threadIdx.x; e < c.slots * 128; e += blockDim.x) c.merge[e] = 0;
    RB_STAMP(tr, 1);
    pdl_wait();     // the weights above are constants; everything below depends on earlier kernels
    pdl_trigger();  // after the wait: see the rule in common.cuh
    RB_STAMP(tr, 2);
    product_run<USE_MMA, NCOL, WIDE, DEEP, TP>(p, c, wv, s_sx, s_xsum, tr);
    RB_STAMP(tr, 5);
    RB_TRACE_COMMIT(tr, p.st.mode * 10 + p.halves);
}

static PerDevice<int> g_sm_counts;
static int sm_count() {
    int& n = g_sm_counts.here();
    if (!n) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, current_device()) != cudaSuccess || n <= 0)
            n = 148;
    }
    return n;
}

template <bool USE_MMA, int NCOL, bool WIDE, bool DEEP, bool TP>
static int launch_fused_tp(const FusedGemvParams& p, int grid, cudaStream_t st) {
    static PerDevice<bool> once;  // each variant raises its own shared-memory limit once per device
    bool& configured = once.here();
    if (!configured) {
        RB_CUDA(cudaFuncSetAttribute(fused_gemv_kernel<USE_MMA, NCOL, WIDE, DEEP, TP>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        // the largest shared-memory split for every variant: kernels of a step share SMs, and a CTA
        // whose request does not fit the split left by its neighbour waits for the SM to drain
        RB_CUDA(cudaFuncSetAttribute(fused_gemv_kernel<USE_MMA, NCOL, WIDE, DEEP, TP>,
                                     cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        configured = true;
    }
    const size_t smem = fused_smem(p, !DEEP);
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
    if (cudaLaunchKernelEx(&cfg, fused_gemv_kernel<USE_MMA, NCOL, WIDE, DEEP, TP>, p) != cudaSuccess) {
        ++g_launch_count;
        return ROTOR_B200_ERR_CUDA;
    }
    return launch_status();
}

template <bool USE_MMA, int NCOL, bool WIDE, bool DEEP>
static int launch_fused(const FusedGemvParams& p, int grid, cudaStream_t st) {
    if (p.xs.size || p.part) return launch_fused_tp<USE_MMA, NCOL, WIDE, DEEP, true>(p, grid, st);
    return launch_fused_tp<USE_MMA, NCOL, WIDE, DEEP, false>(p, grid, st);
}

int configure_fused_gemv() {
    const int big = 200 * 1024;
    RB_CUDA(cudaFuncSetAttribute(fused_gemv_kernel<false, 1, false, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
    RB_CUDA(cudaFuncSetAttribute(fused_gemv_kernel<false, 2, false, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
    RB_CUDA(cudaFuncSetAttribute(fused_gemv_kernel<true, 1, false, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
    RB_CUDA(cudaFuncSetAttribute(fused_gemv_kernel<false, 1, false, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
    RB_CUDA(cudaFuncSetAttribute(fused_gemv_kernel<false, 2, false, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
    RB_CUDA(cudaFuncSetAttribute(fused_gemv_kernel<true, 1, false, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
    RB_CUDA(cudaFuncSetAttribute(fused_gemv_kernel<false, 1, true, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
    RB_CUDA(cudaFuncSetAttribute(fused_gemv_kernel<false, 2, true, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
    RB_CUDA(cudaFuncSetAttribute(fused_gemv_kernel<true, 1, true, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
    sm_count();
    return ROTOR_B200_OK;
}

// Whether a product with input width `in` fits this path for `rows` token rows of `terms`
// activation terms each.
bool fused_gemv_supported(size_t out, size_t in, int rows, int terms, int halves, int merge_weights) {
    const int cols = rows * terms;
    if (rows < 1 || cols > 8 || terms > 3 || in % 4) return false;
    FusedGemvParams p = {};
    p.st.n = (int)in;
    if (fused_wide(p.st) && merge_weights) return false;
    p.cols = cols;
    p.nkt = (int)(kpad_of(in) / TILE_K);
    p.halves = halves;
    const int units = (int)(opad_of(out) / TILE_ROWS);
    p.upc = (units + sm_count() - 1) / sm_count();
    p.st.mode = merge_weights ? LM_ATTN : LM_ADD;
    p.st.n_heads = merge_weights;
    p.st.nsplit = 1;
    return fused_smem(p, false) <= 160 * 1024;
}

int launch_fused_gemv(const void* tiles, size_t out, size_t in, int halves, int rows, const LeanStage& stage, float* y,
                      const float* scale, int seg1, int seg2, int ffn_act, cudaStream_t st, const FusedTpExtra* tp) {
    FusedGemvParams p;
    int grid = sm_count();
    int rc = make_fused_params(p, tiles, out, in, halves, rows, stage, y, scale, seg1, seg2, ffn_act, grid);
    if (rc) return rc;
    if (tp) {
        if (stage.terms != 1 || rows > XS_ROWS || (tp->part && halves != 1)) return ROTOR_B200_ERR_ARG;
        p.xs = tp->xs;
        p.part = tp->part;
        p.sx_out = tp->sx_out;
    }
    if (grid > p.units) grid = p.units;
    // large matrices (sixteen or more weight tiles per warp) stream: they take the pipelined loop,
    // and so do rows too wide for the shallow variant's register budget
    const long tiles_per_warp = (long)p.units * p.halves * p.nkt / ((long)grid * FG_WARPS);
    if (fused_wide(p.st)) {
        if (p.cols == 1) return launch_fused<false, 1, true, true>(p, grid, st);
        if (p.cols == 2) return launch_fused<false, 2, true, true>(p, grid, st);
        return launch_fused<true, 1, true, true>(p, grid, st);
    }
    if (tiles_per_warp >= 16 || !fused_shallow_fits(p.st) || fused_stage_bytes(p) > FG_STAGE_MAX) {
        if (p.cols == 1) return launch_fused<false, 1, false, true>(p, grid, st);
        if (p.cols == 2) return launch_fused<false, 2, false, true>(p, grid, st);
        return launch_fused<true, 1, false, true>(p, grid, st);
    }
    if (p.cols == 1) return launch_fused<false, 1, false, false>(p, grid, st);
    if (p.cols == 2) return launch_fused<false, 2, false, false>(p, grid, st);
    return launch_fused<true, 1, false, false>(p, grid, st);
}

int fused_sm_count() { return sm_count(); }

// Stand-alone integer product through the staged kernel: the matrix is small enough for every
// CTA's share of the tiles to sit in shared memory, and the activations are quantised already.
bool staged_acc_supported(size_t out, size_t in, int ncols, int variant) {
    if (ncols < 1 || ncols > 8 || in % 4) return false;
    if (variant == ROTOR_B200_VARIANT_DP4A && ncols > 2) return false;  // the staged kernel multiplies 1 or 2 columns with dp4a
    FusedGemvParams p = {};
    p.cols = ncols;
    p.nkt = (int)(kpad_of(in) / TILE_K);
    p.halves = 1;
    p.units = (int)(opad_of(out) / TILE_ROWS);
    const int grid = sm_count() < p.units ? sm_count() : p.units;
    p.upc = (p.units + grid - 1) / grid;
    p.st.mode = LM_PLAIN;
    p.st.n = (int)in;
    const long tiles_per_warp = (long)p.units * p.nkt / ((long)grid * FG_WARPS);
    return tiles_per_warp < 16 && fused_stage_bytes(p) <= FG_STAGE_MAX && fused_smem(p, true) <= 200 * 1024;
}

int launch_staged_acc(const void* tiles, size_t out, size_t in, const int8_t* xq, const int32_t* xsum, int ncols,
                      int32_t* acc, int variant, cudaStream_t st) {
    if (!staged_acc_supported(out, in, ncols, variant)) return ROTOR_B200_ERR_SHAPE;
    LeanStage stage = {};
    stage.mode = LM_PLAIN;
    stage.n = (int)in;
    stage.terms = 1;
    stage.kpad = (int)kpad_of(in);
    FusedGemvParams p;
    int grid = sm_count();
    const float one[3] = {1.f, 1.f, 1.f};
    int rc = make_fused_params(p, tiles, out, in, 1, ncols, stage, nullptr, one, (int)out, (int)out, 0, grid);
    if (rc) return rc;
    p.xq_in = xq;
    p.xsum_in = xsum;
    p.acc_out = acc;
    if (grid > p.units) grid = p.units;
    const bool mma = variant == ROTOR_B200_VARIANT_MMA || ncols > 2;
    if (mma) return launch_fused_tp<true, 1, false, false, false>(p, grid, st);
    if (ncols == 1) return launch_fused_tp<false, 1, false, false, false>(p, grid, st);
    return launch_fused_tp<false, 2, false, false, false>(p, grid, st);
}

}  // namespace rb
