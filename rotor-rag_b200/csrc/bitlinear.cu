// Ternary BitLinear integer core: acc[c][o] = sum_k xq[c][k] * w[o][k].
//
// HBM-bound: the kernel streams each 512-byte weight tile exactly once with one
// 128-bit load per lane, stages the int8 activation columns in shared memory with a
// bulk (TMA) copy, and decodes in registers with one AND per operand word:
// (word & (0x03030303 << 2j)) is the int8x4 vector 4^j * (w+1).  Partial sums are
// kept per bit-pair j and rescaled exactly (arithmetic shift) at the end; the "+1"
// of the code is removed by subtracting sum_k xq[c][k] (xsum).
//
// Two instruction mixes share the layout:
//   DP4A : dp4a.u32.s32 lanes, up to 4 columns per pass (decode work is per weight,
//          multiply work per weight per column);
//   MMA  : mma.sync m16n8k32 u8 x s8 -> s32; the tile IS the A fragment, 8 columns
//          per pass at the cost of one, which also carries the residual terms of the
//          multi-term activation quantiser.
#include "gemv_core.cuh"
#include "model.cuh"

namespace rb {

// Activation columns are staged into shared memory with bulk async (TMA) copies that
// signal an mbarrier.  stage_init() may run before the producer of xq has finished;
// stage_issue() must run after it; stage_wait() spins with a bound and returns false
// when it gave up (the caller records it; results are then undefined but every access
// stays in bounds).
__device__ __forceinline__ void stage_init(uint64_t* bar) {
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(bar)));
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
}

__device__ __forceinline__ void stage_issue(uint64_t* bar, int8_t* xs, int xs_stride, const int8_t* src,
                                            size_t src_stride, int ncols, uint32_t bytes) {
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                     "r"(bytes * (uint32_t)ncols)
                     : "memory");
        for (int c = 0; c < ncols; ++c)
            asm volatile(
                "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                    smem_u32(xs + (size_t)c * xs_stride)),
                "l"(src + (size_t)c * src_stride), "r"(bytes), "r"(smem_u32(bar))
                : "memory");
    }
}

// Call after a __syncthreads() that follows stage_issue.
__device__ __forceinline__ bool stage_wait(uint64_t* bar) {
    uint32_t ok = 0;
    const long long start = clock64();
    // bounded: gives up after ~2e8 SM cycles (about 0.1 s) instead of waiting for ever
    while (!ok) {
        asm volatile(
            "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0; selp.u32 %0, 1, 0, p; }"
            : "=r"(ok)
            : "r"(smem_u32(bar))
            : "memory");
        if (!ok && clock64() - start > 200000000LL) break;
    }
    return ok != 0;
}

struct AccParams {
    const uint4* tiles;
    const int8_t* xq;      // [ncols][kpad]
    const int32_t* xsum;   // [ncols]
    int32_t* acc;          // [ncols][out]
    unsigned* status;      // device word, set to ROTOR_B200_ERR_TIMEOUT on a staging timeout
    int out;
    int nkt;               // k-tiles per row of tiles
    int kt_per_split;
    int ncols;
    int atomic;            // gridDim.y > 1: accumulate with integer atomics into zeroed acc
    size_t plane_stride;   // != 0: K split s stores its partial sums to acc + s*plane_stride instead
};

template <int WARPS, int UMAX, bool USE_MMA, int NCOL>
__global__ void __launch_bounds__(WARPS * 32) bitlinear_acc_kernel(const __grid_constant__ AccParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int rt = blockIdx.x;
    const int kt0 = blockIdx.y * p.kt_per_split;
    const int kt1 = min(p.nkt, kt0 + p.kt_per_split);
    const int ks = (kt1 - kt0) * TILE_K;
    const int xs_stride = p.kt_per_split * TILE_K + XS_PAD;
    const int kbase = kt0 * TILE_K;

    uint64_t* bar = reinterpret_cast<uint64_t*>(smem_raw);
    int* red = reinterpret_cast<int*>(smem_raw + 16);            // [WARPS][128]
    int8_t* xs = reinterpret_cast<int8_t*>(smem_raw + 16 + WARPS * 128 * 4);

    pdl_trigger();
    stage_init(bar);

    const uint4* trow = p.tiles + ((size_t)rt * p.nkt) * 32 + lane;

    int accm[4][4];          // MMA: [bit pair j][fragment register]
    int accd[2][4][NCOL];    // DP4A: [row half][bit pair j][column]
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int r = 0; r < 4; ++r) accm[j][r] = 0;
#pragma unroll
        for (int c = 0; c < NCOL; ++c) accd[0][j][c] = accd[1][j][c] = 0;
    }

    // First batch of weight tiles is requested before the activations are waited for.
    uint4 wv[UMAX];
    int base = kt0 + warp;
#pragma unroll
    for (int u = 0; u < UMAX; ++u)
        if (base + u * WARPS < kt1) wv[u] = ld_stream_v4(trow + (size_t)(base + u * WARPS) * 32);
    pdl_wait();  // weights above are constants; everything below depends on the producer kernel
    stage_issue(bar, xs, xs_stride, p.xq + (size_t)kt0 * TILE_K, (size_t)p.nkt * TILE_K, p.ncols, (uint32_t)ks);
    __syncthreads();  // mbarrier initialised, bulk copies issued
    if (!stage_wait(bar) && threadIdx.x == 0) atomicMax(p.status, (unsigned)ROTOR_B200_ERR_TIMEOUT);

    while (base < kt1) {
#pragma unroll
        for (int u = 0; u < UMAX; ++u) {
            const int kt = base + u * WARPS;
            if (kt < kt1) {
                const uint32_t pw[4] = {wv[u].x, wv[u].y, wv[u].z, wv[u].w};
                const int koff = kt * TILE_K - kbase + 32 * t;
                tile_mac<USE_MMA, NCOL>(pw, xs, xs_stride, koff, g, p.ncols, accm, accd);
            }
        }
        base += UMAX * WARPS;
#pragma unroll
        for (int u = 0; u < UMAX; ++u)
            if (base + u * WARPS < kt1) wv[u] = ld_stream_v4(trow + (size_t)(base + u * WARPS) * 32);
    }

    // exact rescale of the per-bit-pair partial sums, then reduce across the CTA
    int* myred = red + warp * 128;
    if constexpr (USE_MMA) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int v = accm[0][r] + (accm[1][r] >> 2) + (accm[2][r] >> 4) + (accm[3][r] >> 6);
            const int row_l = g + 8 * (r >> 1), col = 2 * t + (r & 1);
            myred[row_l * 8 + col] = v;
        }
    } else {
#pragma unroll
        for (int rh = 0; rh < 2; ++rh)
#pragma unroll
            for (int c = 0; c < NCOL; ++c) {
                int v = accd[rh][0][c] + (accd[rh][1][c] >> 2) + (accd[rh][2][c] >> 4) + (accd[rh][3][c] >> 6);
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                if (t == 0) myred[(g + 8 * rh) * 8 + c] = v;
            }
    }
    __syncthreads();
    if (threadIdx.x < 128) {
        const int row_l = threadIdx.x >> 3, col = threadIdx.x & 7;
        const int row = rt * TILE_ROWS + row_l;
        if (col < p.ncols && row < p.out) {
            int s = 0;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) s += red[w * 128 + threadIdx.x];
            if (blockIdx.y == 0) s -= p.xsum[col];
            int32_t* dst = p.acc + (size_t)blockIdx.y * p.plane_stride + (size_t)col * p.out + row;
            if (p.atomic)
                atomicAdd(dst, s);
            else
                *dst = s;
        }
    }

}

__global__ void dequant_kernel(const int32_t* __restrict__ acc, const float* __restrict__ sx, int m, int terms,
                               int out, float wscale, const float* __restrict__ wscale_vec,
                               float* __restrict__ y) {
    const size_t total = (size_t)m * out;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int r = (int)(i / out), o = (int)(i % out);
        float v = 0.f;
        for (int tt = 0; tt < terms; ++tt)
            v = __fadd_rn(v, __fmul_rn((float)acc[((size_t)r * terms + tt) * out + o], sx[r * terms + tt]));
        y[i] = __fmul_rn(v, wscale_vec ? wscale_vec[o] : wscale);
    }
}

// Device status word shared by every launch of the library on one device (one word per device).
static PerDevice<unsigned*> g_status_words;
static int ensure_status() {
    unsigned*& w = g_status_words.here();
    if (w) return ROTOR_B200_OK;
    RB_CUDA(cudaMalloc(&w, sizeof(unsigned)));
    RB_CUDA(cudaMemset(w, 0, sizeof(unsigned)));
    return ROTOR_B200_OK;
}

__global__ void empty_kernel() {
    pdl_wait();
    pdl_trigger();
}

int g_use_pdl = 1;  // programmatic dependent launch for the kernels that call pdl_wait()

unsigned* library_status_word() { return ensure_status() ? nullptr : g_status_words.here(); }

template <int WARPS, int UMAX, bool USE_MMA, int NCOL>
static int launch_acc(const AccParams& p, int nrt, int ksplit, cudaStream_t st) {
    auto kern = bitlinear_acc_kernel<WARPS, UMAX, USE_MMA, NCOL>;
    const size_t smem = 16 + WARPS * 128 * 4 + (size_t)p.ncols * (p.kt_per_split * TILE_K + XS_PAD);
    if (smem > 200 * 1024) return ROTOR_B200_ERR_SHAPE;
    if (smem > 48 * 1024) {
        static PerDevice<size_t> once;  // per instantiation and device
        size_t& configured = once.here();
        if (smem > configured) {
            RB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            configured = 200 * 1024;
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(nrt, ksplit);
    cfg.blockDim = dim3(WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_use_pdl ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, kern, p) != cudaSuccess) {
        ++g_launch_count;
        return ROTOR_B200_ERR_CUDA;
    }
    return launch_status();
}

// Split the K range over gridDim.y so that the grid covers the GPU a few times and
// the staged activations stay below ~64 KB per CTA.
static int choose_ksplit(int nrt, int nkt, int ncols, int warps) {
    int ks = 1;
    while (ks < nkt) {
        const int per = (nkt + ks - 1) / ks;
        const bool enough_ctas = (long)nrt * ks >= 2 * 148;
        const bool smem_ok = (size_t)ncols * (per * TILE_K + XS_PAD) <= 64 * 1024;
        const bool too_thin = per / 2 < warps;  // keep at least one tile per warp after doubling
        if (smem_ok && (enough_ctas || too_thin)) break;
        ks *= 2;
    }
    return ks > nkt ? nkt : ks;
}

static int dispatch_acc(const AccParams& p, int nrt, int ksplit, int variant, cudaStream_t st) {
    constexpr int WARPS = 4, UMAX = 8;
    if (variant == ROTOR_B200_VARIANT_MMA) return launch_acc<WARPS, UMAX, true, 1>(p, nrt, ksplit, st);
    switch (p.ncols) {
        case 1: return launch_acc<WARPS, UMAX, false, 1>(p, nrt, ksplit, st);
        case 2: return launch_acc<WARPS, UMAX, false, 2>(p, nrt, ksplit, st);
        case 3: return launch_acc<WARPS, UMAX, false, 3>(p, nrt, ksplit, st);
        case 4: return launch_acc<WARPS, UMAX, false, 4>(p, nrt, ksplit, st);
    }
    return ROTOR_B200_ERR_ARG;
}

template <bool USE_MMA, int NCOL>
static int configure_one() {
    RB_CUDA(cudaFuncSetAttribute(bitlinear_acc_kernel<4, 8, USE_MMA, NCOL>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    return ROTOR_B200_OK;
}

// Done once, outside any stream capture: status word and the shared-memory opt-ins.
int configure_gemv_kernels() {
    int rc = ensure_status();
    if (rc) return rc;
    if ((rc = configure_one<true, 1>())) return rc;
    if ((rc = configure_one<false, 1>())) return rc;
    if ((rc = configure_one<false, 2>())) return rc;
    if ((rc = configure_one<false, 3>())) return rc;
    return configure_one<false, 4>();
}

static int pick_variant(int variant, int ncols) {
    if (variant != ROTOR_B200_VARIANT_AUTO) return variant;
    return ncols <= 2 ? ROTOR_B200_VARIANT_DP4A : ROTOR_B200_VARIANT_MMA;
}

int gemv_cols_per_launch(int variant, int ncols) {
    return pick_variant(variant, ncols < 8 ? ncols : 8) == ROTOR_B200_VARIANT_MMA ? 8 : 4;
}

GemvPlan plan_gemv(size_t out, size_t in, int ncols) {
    const int nkt = (int)(kpad_of(in) / TILE_K), nrt = (int)(opad_of(out) / TILE_ROWS);
    const int per_pass = ncols < 8 ? ncols : 8;
    int ks = choose_ksplit(nrt, nkt, per_pass, 4);
    GemvPlan g;
    g.kt_per_split = (nkt + ks - 1) / ks;
    g.ksplit = (nkt + g.kt_per_split - 1) / g.kt_per_split;
    return g;
}

int launch_gemv_planes(const void* tiles, size_t out, size_t in, const int8_t* xq, const int32_t* xsum, int ncols,
                       int32_t* acc, size_t plane_stride, const GemvPlan& plan, int variant, cudaStream_t st) {
    int rc = ensure_status();
    if (rc) return rc;
    if (ncols >= GEMM_MIN_COLS && variant == ROTOR_B200_VARIANT_AUTO) {
        // compute-bound regime: the tiled GEMM writes complete sums into plane 0 (callers use one plane)
        if (gemm_tcgen05_supported(out, in, ncols, xq)) return launch_gemm_tcgen05(tiles, out, in, xq, xsum, ncols, acc, st);
        return launch_gemm_mma(tiles, out, in, xq, xsum, ncols, acc, st);
    }
    const int nkt = (int)(kpad_of(in) / TILE_K), nrt = (int)(opad_of(out) / TILE_ROWS);
    const size_t kpad = kpad_of(in);
    variant = pick_variant(variant, ncols);
    const int chunk = variant == ROTOR_B200_VARIANT_MMA ? 8 : 4;
    for (int c0 = 0; c0 < ncols; c0 += chunk) {
        AccParams p;
        p.tiles = (const uint4*)tiles;
        p.xq = xq + (size_t)c0 * kpad;
        p.xsum = xsum + c0;
        p.acc = acc + (size_t)c0 * out;
        p.status = g_status_words.here();
        p.out = (int)out;
        p.nkt = nkt;
        p.kt_per_split = plan.kt_per_split;
        p.ncols = (ncols - c0) < chunk ? (ncols - c0) : chunk;
        // plane_stride 0 with a split K range: the splits add into one zeroed plane (exact in any order)
        p.atomic = plane_stride == 0 && plan.ksplit > 1;
        p.plane_stride = plane_stride;
        if (p.atomic) RB_CUDA(cudaMemsetAsync(p.acc, 0, (size_t)p.ncols * out * sizeof(int32_t), st));
        rc = dispatch_acc(p, nrt, plan.ksplit, variant, st);
        if (rc) return rc;
    }
    return ROTOR_B200_OK;
}

}  // namespace rb

using namespace rb;

extern "C" {

int rotor_b200_bitlinear_acc(const void* tiles, size_t out, size_t in, const int8_t* xq, const int32_t* xsum,
                             size_t ncols, int32_t* acc, int variant, void* stream) {
    RB_REQUIRE(tiles && xq && xsum && acc && out > 0 && in > 0 && ncols > 0);
    RB_REQUIRE(out < (1u << 30) && in < (1u << 30));
    RB_REQUIRE(((uintptr_t)tiles & 15) == 0 && ((uintptr_t)xq & 15) == 0);
    RB_REQUIRE(variant >= ROTOR_B200_VARIANT_AUTO && variant <= ROTOR_B200_VARIANT_MMA);
    int rc = ensure_status();
    if (rc) return rc;
    cudaStream_t st = as_stream(stream);
    const int nkt = (int)(kpad_of(in) / TILE_K), nrt = (int)(opad_of(out) / TILE_ROWS);
    const size_t kpad = kpad_of(in);
    if (ncols >= GEMM_MIN_COLS && variant == ROTOR_B200_VARIANT_AUTO) {
        if (gemm_tcgen05_supported(out, in, (int)ncols, xq))
            return launch_gemm_tcgen05(tiles, out, in, xq, xsum, (int)ncols, acc, st);
        return launch_gemm_mma(tiles, out, in, xq, xsum, (int)ncols, acc, st);
    }
    // small matrices, up to eight columns: the staged kernel (every CTA's share of the tiles sits in shared
    // memory before the activations are needed, which a chain of dependent launches can overlap)
    if (ncols <= 8 && staged_acc_supported(out, in, (int)ncols, variant))
        return launch_staged_acc(tiles, out, in, xq, xsum, (int)ncols, acc, variant, st);
    variant = pick_variant(variant, (int)(ncols < 8 ? ncols : 8));
    const size_t chunk = variant == ROTOR_B200_VARIANT_MMA ? 8 : 4;
    for (size_t c0 = 0; c0 < ncols; c0 += chunk) {
        const int nc = (int)((ncols - c0) < chunk ? (ncols - c0) : chunk);
        const int ksplit = choose_ksplit(nrt, nkt, nc, 4);
        AccParams p;
        p.tiles = (const uint4*)tiles;
        p.xq = xq + c0 * kpad;
        p.xsum = xsum + c0;
        p.acc = acc + c0 * out;
        p.status = g_status_words.here();
        p.out = (int)out;
        p.nkt = nkt;
        p.kt_per_split = (nkt + ksplit - 1) / ksplit;
        p.ncols = nc;
        const int ksplit_eff = (nkt + p.kt_per_split - 1) / p.kt_per_split;
        p.atomic = ksplit_eff > 1;
        p.plane_stride = 0;
        if (p.atomic) RB_CUDA(cudaMemsetAsync(p.acc, 0, (size_t)nc * out * sizeof(int32_t), st));
        rc = dispatch_acc(p, nrt, ksplit_eff, variant, st);
        if (rc) return rc;
    }
    return ROTOR_B200_OK;
}

int rotor_b200_bitlinear_dequant(const int32_t* acc, const float* sx, size_t m, int terms, size_t out,
                                 float wscale, const float* wscale_vec, float* y, void* stream) {
    RB_REQUIRE(acc && sx && y && m > 0 && out > 0 && terms >= 1 && terms <= 4);
    const size_t total = m * out;
    unsigned grid = (unsigned)((total + 255) / 256);
    if (grid > 148 * 16) grid = 148 * 16;
    dequant_kernel<<<grid, 256, 0, as_stream(stream)>>>(acc, sx, (int)m, terms, (int)out, wscale, wscale_vec, y);
    return launch_status();
}

static inline size_t al256(size_t v) { return (v + 255) & ~(size_t)255; }

size_t rotor_b200_bitlinear_workspace_bytes(size_t out, size_t in, size_t m, int terms) {
    const size_t nc = m * (size_t)terms;
    return al256(nc * kpad_of(in)) + al256(nc * 4) + al256(nc * 4) + al256(nc * out * 4);
}

int rotor_b200_bitlinear_forward(const void* tiles, size_t out, size_t in, const float* x, size_t m, int terms,
                                 float wscale, const float* wscale_vec, float* y, void* workspace,
                                 size_t workspace_bytes, int variant, void* stream) {
    RB_REQUIRE(tiles && x && y && workspace && m > 0 && terms >= 1 && terms <= 4);
    RB_REQUIRE(((uintptr_t)workspace & 255) == 0);
    if (workspace_bytes < rotor_b200_bitlinear_workspace_bytes(out, in, m, terms)) return ROTOR_B200_ERR_WORKSPACE;
    const size_t nc = m * (size_t)terms;
    unsigned char* w = (unsigned char*)workspace;
    int8_t* xq = (int8_t*)w;
    w += al256(nc * kpad_of(in));
    float* sx = (float*)w;
    w += al256(nc * 4);
    int32_t* xsum = (int32_t*)w;
    w += al256(nc * 4);
    int32_t* acc = (int32_t*)w;
    int rc = rotor_b200_quantize_rows(x, m, in, terms, xq, sx, xsum, stream);
    if (rc) return rc;
    rc = rotor_b200_bitlinear_acc(tiles, out, in, xq, xsum, nc, acc, variant, stream);
    if (rc) return rc;
    return rotor_b200_bitlinear_dequant(acc, sx, m, terms, out, wscale, wscale_vec, y, stream);
}

/* ---------------------------------------------------------------------------------------
 * Allocation-free layer forward.
 *
 * rotor_b200_bitlinear_forward needs a caller-provided workspace, and the accumulate step
 * behind it creates a small device status word with cudaMalloc on first use.  Some hosts
 * cannot do either: a plug-in driven through the reference's backend call
 * (ternary_matmul(packed, scales, input_vec, in_dim, out_dim) has no workspace argument),
 * or a serving loop that has already handed every remaining byte of device memory to its
 * own pool, where cudaMalloc would fail -- and, when it succeeds, stalls all streams of the
 * device while it runs.  For them the scratch lives in a fixed array inside the library:
 * ROTOR_B200_STATIC_SCRATCH_BYTES per GPU, resident from library load to process exit on
 * every GPU that loads the library.
 *
 * Rules of use
 *  - Problems whose scratch need exceeds the array are refused with ROTOR_B200_ERR_TOO_LARGE;
 *    nothing is launched.  rotor_b200_bitlinear_static_fits() answers the question up front.
 *  - The first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress).  Make that first call before starting any stream capture.
 *  - All calls on one GPU share the array, and it keeps the previous call's contents; the
 *    entry point clears what has to start at zero.  Two calls that overlap on the GPU
 *    (different streams, no ordering between them) race on the array: serialise them.
 *  - No cudaMalloc, cudaFree or other allocating routine is called on this path. */
static __device__ __align__(256) unsigned char g_static_scratch[ROTOR_B200_STATIC_SCRATCH_BYTES];

static PerDevice<unsigned char*> g_static_addr;  // device address of the array, once looked up on that device

static int static_scratch_address(unsigned char** out) {
    int dev = -1;
    RB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= RB_MAX_DEVICES) return ROTOR_B200_ERR_ARG;
    unsigned char*& addr = g_static_addr.v[dev];
    if (!addr) {
        // g_static_scratch names the array in device code only; host code must ask for its address
        void* p = nullptr;
        RB_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
        addr = static_cast<unsigned char*>(p);
    }
    *out = addr;
    return ROTOR_B200_OK;
}

static size_t static_need(size_t out, size_t in, size_t m, int terms) {
    return 256 + rotor_b200_bitlinear_workspace_bytes(out, in, m, terms);  // status word + stage buffers
}

int rotor_b200_bitlinear_static_fits(size_t out, size_t in, size_t m, int terms) {
    if (out == 0 || in == 0 || m == 0 || terms < 1 || terms > 4) return 0;
    return static_need(out, in, m, terms) <= ROTOR_B200_STATIC_SCRATCH_BYTES;
}

int rotor_b200_bitlinear_forward_static(const void* tiles, size_t out, size_t in, const float* x, size_t m,
                                        int terms, float wscale, const float* wscale_vec, float* y, int variant,
                                        void* stream) {
    RB_REQUIRE(tiles && x && y && m > 0 && out > 0 && in > 0 && terms >= 1 && terms <= 4);
    RB_REQUIRE(out < (1u << 30) && in < (1u << 30));
    RB_REQUIRE(((uintptr_t)tiles & 15) == 0);
    RB_REQUIRE(variant >= ROTOR_B200_VARIANT_AUTO && variant <= ROTOR_B200_VARIANT_MMA);
    if (static_need(out, in, m, terms) > ROTOR_B200_STATIC_SCRATCH_BYTES) return ROTOR_B200_ERR_TOO_LARGE;
    unsigned char* base = nullptr;
    int rc = static_scratch_address(&base);
    if (rc) return rc;
    cudaStream_t st = as_stream(stream);
    // carve: [status word, 256 B][xq][sx][xsum][acc]
    unsigned* status = reinterpret_cast<unsigned*>(base);
    unsigned char* w = base + 256;
    const size_t nc = m * (size_t)terms, kpad = kpad_of(in);
    int8_t* xq = (int8_t*)w;
    w += al256(nc * kpad);
    float* sx = (float*)w;
    w += al256(nc * 4);
    int32_t* xsum = (int32_t*)w;
    w += al256(nc * 4);
    int32_t* acc = (int32_t*)w;
    // the status word starts at zero (the array is zero-initialised when the library is loaded) and is
    // cleared only by rotor_b200_device_status(), which reads it: a timed-out wait is never lost
    rc = rotor_b200_quantize_rows(x, m, in, terms, xq, sx, xsum, stream);
    if (rc) return rc;
    const int nkt = (int)(kpad / TILE_K), nrt = (int)(opad_of(out) / TILE_ROWS);
    variant = pick_variant(variant, (int)(nc < 8 ? nc : 8));
    const size_t chunk = variant == ROTOR_B200_VARIANT_MMA ? 8 : 4;
    for (size_t c0 = 0; c0 < nc; c0 += chunk) {
        const int ncols = (int)((nc - c0) < chunk ? (nc - c0) : chunk);
        const int ksplit = choose_ksplit(nrt, nkt, ncols, 4);
        AccParams p;
        p.tiles = (const uint4*)tiles;
        p.xq = xq + c0 * kpad;
        p.xsum = xsum + c0;
        p.acc = acc + c0 * out;
        p.status = status;
        p.out = (int)out;
        p.nkt = nkt;
        p.kt_per_split = (nkt + ksplit - 1) / ksplit;
        p.ncols = ncols;
        const int ksplit_eff = (nkt + p.kt_per_split - 1) / p.kt_per_split;
        p.atomic = ksplit_eff > 1;
        p.plane_stride = 0;
        // split-K partial sums are added into the accumulators: they must start at zero
        if (p.atomic) RB_CUDA(cudaMemsetAsync(p.acc, 0, (size_t)ncols * out * sizeof(int32_t), st));
        rc = dispatch_acc(p, nrt, ksplit_eff, variant, st);
        if (rc) return rc;
    }
    return rotor_b200_bitlinear_dequant(acc, sx, m, terms, out, wscale, wscale_vec, y, stream);
}

int rotor_b200_ternary_matmul_host(const void* tiles, const float* scales_host, const float* x_host, size_t in,
                                   size_t out, int terms, float* y_host) {
    RB_REQUIRE(tiles && scales_host && x_host && y_host && in > 0 && out > 0 && terms >= 1 && terms <= 4);
    // grow-only staging area owned by the library: this seam is synchronous and single-threaded
    static unsigned char* stage = nullptr;
    static size_t stage_bytes = 0;
    const size_t ws = rotor_b200_bitlinear_workspace_bytes(out, in, 1, terms);
    const size_t need = al256(in * 4) + 2 * al256(out * 4) + ws;
    if (need > stage_bytes) {
        if (stage) RB_CUDA(cudaFree(stage));
        stage = nullptr;
        stage_bytes = 0;
        RB_CUDA(cudaMalloc(&stage, need));
        stage_bytes = need;
    }
    float* dx = (float*)stage;
    float* dsc = (float*)(stage + al256(in * 4));
    float* dy = (float*)(stage + al256(in * 4) + al256(out * 4));
    void* dws = stage + al256(in * 4) + 2 * al256(out * 4);
    RB_CUDA(cudaMemcpy(dx, x_host, in * 4, cudaMemcpyHostToDevice));
    RB_CUDA(cudaMemcpy(dsc, scales_host, out * 4, cudaMemcpyHostToDevice));
    int rc = rotor_b200_bitlinear_forward(tiles, out, in, dx, 1, terms, 1.0f, dsc, dy, dws, ws,
                                          ROTOR_B200_VARIANT_AUTO, nullptr);
    if (rc) return rc;
    RB_CUDA(cudaMemcpy(y_host, dy, out * 4, cudaMemcpyDeviceToHost));
    return ROTOR_B200_OK;
}

/* Measurement aid: one launch of a kernel that does nothing, with the same launch attributes
 * (programmatic dependent launch when enabled) as the kernels of the decode chain.  A chain of
 * these in a CUDA graph gives the floor that any chain of dependent launches pays per launch. */
int rotor_b200_launch_empty(void* stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(148);
    cfg.blockDim = dim3(128);
    cfg.stream = as_stream(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_use_pdl ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, rb::empty_kernel) != cudaSuccess) {
        ++g_launch_count;
        return ROTOR_B200_ERR_CUDA;
    }
    return launch_status();
}

/* Reads and clears the status words of the current device that bounded waits write to: the
 * library's own word and the one at the start of the fixed scratch array of
 * rotor_b200_bitlinear_forward_static (once that entry point has run on this device).  Allocates
 * nothing. */
int rotor_b200_device_status(void) {
    unsigned v = 0, vs = 0;
    if (unsigned* w = g_status_words.here()) {
        RB_CUDA(cudaMemcpy(&v, w, sizeof(v), cudaMemcpyDeviceToHost));
        if (v) RB_CUDA(cudaMemset(w, 0, sizeof(v)));
    }
    if (unsigned char* a = g_static_addr.here()) {
        RB_CUDA(cudaMemcpy(&vs, a, sizeof(vs), cudaMemcpyDeviceToHost));
        if (vs) RB_CUDA(cudaMemset(a, 0, sizeof(vs)));
    }
    return (int)(v ? v : vs);
}

}  // extern "C"
