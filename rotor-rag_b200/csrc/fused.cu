// Generation-step BitLinear product with the vector stage that feeds it fused in.
//
// One CTA per SM, FG_THREADS threads.  The matrix's tiles, taken in memory order, are cut
// into one contiguous range per CTA (so every CTA streams one contiguous span of HBM) and
// again into one contiguous sub-range per warp.  A warp requests its first tiles before
// anything else; the CTA then builds the int8 activation row(s) in shared memory from the
// previous product's accumulators (dequantise, sub-norm / residual / gating, pre-norm,
// absmax quantise) -- a few microseconds of work done once per SM instead of in a launch
// of its own -- and runs the integer tile products.  Partial sums of a row tile that is
// shared between warps or CTAs are merged with integer atomics (exact, order independent)
// into an accumulator buffer that an earlier kernel of the chain has cleared; each kernel
// clears the buffer of a later one in turn.
#include "gemv_core.cuh"
#include "model.cuh"
#include "quant.cuh"

namespace rb {

constexpr int FG_THREADS = 512;
constexpr int FG_WARPS = FG_THREADS / 32;
constexpr int FG_U = 4;  // weight tiles in flight per warp

struct FusedGemvParams {
    const uint4* tiles;
    int nrt, nkt, out, cols;
    int32_t* acc;        // [cols][out], all zero on entry
    int32_t* zero_ptr;   // words this kernel clears for a later product (may be null)
    int zero_count;
    VecStageParams st;   // the prologue; st.acc has a single plane
    int rows;            // token rows (cols = rows * st.terms_out)
    float* sx_pub;       // [cols] activation scales, published by CTA 0
    int32_t* xsum_pub;   // [cols]
    int nslot;           // row tiles one CTA's range can touch
};

// ---------------------------------------------------------------- lean vector stage
// Same arithmetic as vec_stage_row (vecstage.cuh) for the modes a generation step uses,
// written for few instructions per element: 32-bit indexing, one accumulator plane, rolled
// loops whose global loads are issued four elements ahead of their use.
__device__ __forceinline__ float lean_deq(const int32_t* const (&b)[3], const float (&sx)[3], int terms, int i) {
    const int s0 = __ldcg(b[0] + i);
    const int s1 = terms > 1 ? __ldcg(b[1] + i) : 0;
    const int s2 = terms > 2 ? __ldcg(b[2] + i) : 0;
    return (float)s0 * sx[0] + (float)s1 * sx[1] + (float)s2 * sx[2];
}

__device__ __forceinline__ void lean_rmsnorm(float* row, int n, const float* __restrict__ w, float eps, float* scratch) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss += row[i] * row[i];
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
    const int bd = blockDim.x;
#pragma unroll 1
    for (int i0 = threadIdx.x; i0 < n; i0 += 4 * bd) {
        float wv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) wv[u] = i0 + u * bd < n ? __ldg(w + i0 + u * bd) : 0.f;
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (i0 + u * bd < n) row[i0 + u * bd] = row[i0 + u * bd] * inv * wv[u];
    }
    __syncthreads();
}

// Element loop with the global loads of LU elements issued before any of them is used.
constexpr int LU = 4;
template <typename LoadF, typename UseF>
__device__ __forceinline__ void batched_for(int n, LoadF load, UseF use) {
    const int bd = blockDim.x;
#pragma unroll 1
    for (int i0 = threadIdx.x; i0 < n; i0 += LU * bd) {
        float2 a[LU];
#pragma unroll
        for (int u = 0; u < LU; ++u) {
            const int i = i0 + u * bd;
            a[u] = i < n ? load(i) : make_float2(0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < LU; ++u) {
            const int i = i0 + u * bd;
            if (i < n) use(i, a[u]);
        }
    }
}

// Builds token row m in `row` and quantises it to xq (shared memory).
__device__ __forceinline__ void lean_stage_row(const VecStageParams& p, int m, float* row, float* scratch, bool writer,
                                               int8_t* xq, size_t tstride, float* sx_s, int* xsum_s) {
    const int n = p.n, bd = blockDim.x;
    float* hdst = (p.h_out ? p.h_out : p.h) + (size_t)m * n;
    const float* hsrc = p.h + (size_t)m * n;
    const int32_t* b[3] = {nullptr, nullptr, nullptr};
    float sx[3] = {0.f, 0.f, 0.f};
    const int terms = p.terms;
    if (p.mode == VS_OPROJ || p.mode == VS_FFN || p.mode == VS_DOWN) {
        for (int t = 0; t < 3; ++t)
            if (t < terms) {
                b[t] = p.acc.acc + ((size_t)m * terms + t) * p.acc.out;
                sx[t] = __ldcg(p.sx_in + (size_t)m * terms + t);
            }
    }
    const float ws0 = p.wscale0, ws1 = p.wscale1;
    if (p.mode == VS_EMBED) {
        const __nv_bfloat16* e = p.embed + (size_t)p.ids[m] * n;
        batched_for(n, [&](int i) { return make_float2(__bfloat162float(e[i]), 0.f); },
                    [&](int i, float2 a) {
                        row[i] = a.x;
                        if (writer) hdst[i] = a.x;
                    });
    } else if (p.mode == VS_DOWN) {
        batched_for(n, [&](int i) { return make_float2(__ldcg(hsrc + i), lean_deq(b, sx, terms, i)); },
                    [&](int i, float2 a) {
                        const float v = a.x + a.y * ws0;
                        row[i] = v;
                        if (writer) hdst[i] = v;
                    });
    } else if (p.mode == VS_OPROJ) {
        batched_for(n, [&](int i) { return make_float2(lean_deq(b, sx, terms, i), 0.f); },
                    [&](int i, float2 a) { row[i] = a.x * ws0; });
        __syncthreads();
        lean_rmsnorm(row, n, p.norm0, p.eps, scratch);
        batched_for(n, [&](int i) { return make_float2(__ldcg(hsrc + i), 0.f); },
                    [&](int i, float2 a) {
                        const float v = a.x + row[i];
                        row[i] = v;
                        if (writer) hdst[i] = v;
                    });
    } else if (p.mode == VS_FFN) {
        const bool relu2 = p.ffn_act == ROTOR_B200_FFN_RELU2;
        batched_for(n, [&](int i) { return make_float2(lean_deq(b, sx, terms, i), lean_deq(b, sx, terms, n + i)); },
                    [&](int i, float2 a) {
                        const float gt = a.x * ws0, up = a.y * ws1;
                        float v;
                        if (relu2) {
                            const float r = fmaxf(gt, 0.f);
                            v = r * r * up;
                        } else {
                            const float c = fminf(fmaxf(up, -20.f), 20.f);
                            v = gt * (c / (1.f + expf(-c)));
                        }
                        row[i] = v;
                    });
    } else if (p.mode == VS_ATTN) {
        const int D = p.head_dim, ns = p.nsplit, nh = p.n_heads;
        float* wf = row + n;
        float* wl = wf + nh * ns;
        const size_t hb = (size_t)m * nh * ns;
        for (int e = threadIdx.x; e < nh * ns; e += bd) {
            wf[e] = __ldcg(p.part_m + hb + e);
            wl[e] = __ldcg(p.part_l + hb + e);
        }
        __syncthreads();
        for (int h = threadIdx.x; h < nh; h += bd) {
            float M = -INFINITY;
            for (int s2 = 0; s2 < ns; ++s2) M = fmaxf(M, wf[h * ns + s2]);
            float L = 0.f;
            for (int s2 = 0; s2 < ns; ++s2) {
                const float ms = wf[h * ns + s2];
                const float f = ms == -INFINITY ? 0.f : __expf(ms - M);
                L += wl[h * ns + s2] * f;
                wf[h * ns + s2] = f;
            }
            const float inv = 1.0f / L;
            for (int s2 = 0; s2 < ns; ++s2) wf[h * ns + s2] *= inv;
        }
        __syncthreads();
#pragma unroll 1
        for (int i = threadIdx.x; i < n; i += bd) {
            const int h = i / D, dd = i - h * D;
            const float* po = p.part_o + (hb + (size_t)h * ns) * D + dd;
            float o = 0.f;
#pragma unroll 1
            for (int s0 = 0; s0 < ns; s0 += 8) {  // nsplit is a multiple of 8
                float pv[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) pv[u] = __ldcg(po + (size_t)(s0 + u) * D);
#pragma unroll
                for (int u = 0; u < 8; ++u) o += pv[u] * wf[h * ns + s0 + u];
            }
            row[i] = o;
        }
    }
    __syncthreads();
    if (p.norm1) lean_rmsnorm(row, n, p.norm1, p.eps, scratch);
    quantize_row_from_smem(row, n, p.kpad, p.terms_out, xq, sx_s, xsum_s, scratch, tstride);
}

// ---------------------------------------------------------------- the kernel
template <bool USE_MMA, int NCOL>
__global__ void __launch_bounds__(FG_THREADS, 1) fused_gemv_kernel(const __grid_constant__ FusedGemvParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ float s_sx[8];
    __shared__ int s_xsum[8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int kpad = p.nkt * TILE_K;
    const int xs_stride = kpad + XS_PAD;
    int8_t* xs = reinterpret_cast<int8_t*>(smem_raw);                       // [cols][xs_stride]
    int* merge = reinterpret_cast<int*>(smem_raw + (size_t)p.cols * xs_stride);  // [nslot][128]
    float* scratch = reinterpret_cast<float*>(merge + p.nslot * 128);       // [64]
    float* row = scratch + 64;                                              // [n (+ attention weights)]

    pdl_trigger();

    // this CTA's and this warp's contiguous tile ranges
    const long long total = (long long)p.nrt * p.nkt;
    const int t0 = (int)(total * blockIdx.x / gridDim.x), t1 = (int)(total * (blockIdx.x + 1) / gridDim.x);
    const int len = t1 - t0;
    const int w0 = t0 + (int)((long long)len * warp / FG_WARPS), w1 = t0 + (int)((long long)len * (warp + 1) / FG_WARPS);
    const int rt_first = t0 / p.nkt;

    uint4 wv[FG_U];
#pragma unroll
    for (int u = 0; u < FG_U; ++u)
        if (w0 + u < w1) wv[u] = ld_stream_v4(p.tiles + (size_t)(w0 + u) * 32 + lane);
    for (int e = threadIdx.x; e < p.nslot * 128; e += FG_THREADS) merge[e] = 0;

    pdl_wait();  // the weights above are constants; everything below depends on earlier kernels

    for (int i = blockIdx.x * FG_THREADS + threadIdx.x; i < p.zero_count; i += gridDim.x * FG_THREADS)
        p.zero_ptr[i] = 0;

    const bool writer = blockIdx.x == 0;
    const int to = p.st.terms_out;
    for (int m = 0; m < p.rows; ++m) {
        lean_stage_row(p.st, m, row, scratch, writer, xs + (size_t)m * to * xs_stride, (size_t)xs_stride, s_sx + m * to,
                       s_xsum + m * to);
        __syncthreads();
    }
    if (writer && threadIdx.x < p.cols) {
        p.sx_pub[threadIdx.x] = s_sx[threadIdx.x];
        p.xsum_pub[threadIdx.x] = s_xsum[threadIdx.x];
    }

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
    auto flush = [&](int rt) {  // exact rescale of the per-bit-pair sums, then into the CTA's merge slot
        int* slot = merge + (rt - rt_first) * 128;
        if constexpr (USE_MMA) {
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int v = accm[0][r] + (accm[1][r] >> 2) + (accm[2][r] >> 4) + (accm[3][r] >> 6);
                atomicAdd(slot + (g + 8 * (r >> 1)) * 8 + 2 * t + (r & 1), v);
            }
        } else {
#pragma unroll
            for (int rh = 0; rh < 2; ++rh)
#pragma unroll
                for (int c = 0; c < NCOL; ++c) {
                    int v = accd[rh][0][c] + (accd[rh][1][c] >> 2) + (accd[rh][2][c] >> 4) + (accd[rh][3][c] >> 6);
                    v += __shfl_xor_sync(0xffffffffu, v, 1);
                    v += __shfl_xor_sync(0xffffffffu, v, 2);
                    if (t == 0) atomicAdd(slot + (g + 8 * rh) * 8 + c, v);
                }
        }
    };
    clear();
    int cur_rt = -1;
    for (int base = w0; base < w1; base += FG_U) {
#pragma unroll
        for (int u = 0; u < FG_U; ++u) {
            const int tile = base + u;
            if (tile < w1) {
                const int rt = tile / p.nkt, kt = tile - rt * p.nkt;
                if (rt != cur_rt) {  // warp-uniform
                    if (cur_rt >= 0) flush(cur_rt);
                    clear();
                    cur_rt = rt;
                }
                const uint32_t pw[4] = {wv[u].x, wv[u].y, wv[u].z, wv[u].w};
                tile_mac<USE_MMA, NCOL>(pw, xs, xs_stride, kt * TILE_K + 32 * t, g, p.cols, accm, accd);
            }
        }
#pragma unroll
        for (int u = 0; u < FG_U; ++u)
            if (base + FG_U + u < w1) wv[u] = ld_stream_v4(p.tiles + (size_t)(base + FG_U + u) * 32 + lane);
    }
    if (cur_rt >= 0) flush(cur_rt);
    __syncthreads();

    // ---- CTA partials into the global accumulators; the CTA that owns a row tile's first
    // K tile also removes the +1 offset of the weight codes (sum of the activations)
    const int rt_last = (t1 - 1) / p.nkt;
    for (int e = threadIdx.x; e < p.nslot * 128; e += FG_THREADS) {
        const int rt = rt_first + (e >> 7), idx = e & 127;
        const int row_l = idx >> 3, col = idx & 7;
        const int orow = rt * TILE_ROWS + row_l;
        if (len <= 0 || rt > rt_last || col >= p.cols || orow >= p.out) continue;
        int v = merge[e];
        const int first_tile = rt * p.nkt;
        if (first_tile >= t0 && first_tile < t1) v -= s_xsum[col];
        if (v != 0) atomicAdd(p.acc + (size_t)col * p.out + orow, v);
    }
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
    const size_t rowf = 64 + (size_t)p.st.n + 2 * (size_t)p.st.n_heads * p.st.nsplit;
    return xs + (size_t)p.nslot * 512 + rowf * sizeof(float);
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

// cols this path accepts (rows * terms), and the row widths its shared memory can hold
bool fused_gemv_supported(size_t out, size_t in, int rows, int terms, int stage_n, int stage_extra) {
    const int cols = rows * terms;
    if (rows < 1 || cols > 8 || terms > 3) return false;
    FusedGemvParams p = {};
    p.cols = cols;
    p.nkt = (int)(kpad_of(in) / TILE_K);
    p.nslot = 16;
    p.st.n = stage_n;
    p.st.n_heads = stage_extra;
    p.st.nsplit = 1;
    (void)out;
    return fused_smem(p) <= 160 * 1024;
}

int launch_fused_gemv(const void* tiles, size_t out, size_t in, int rows, const VecStageParams& stage, int32_t* acc,
                      int32_t* zero_ptr, size_t zero_count, float* sx_pub, int32_t* xsum_pub, cudaStream_t st) {
    FusedGemvParams p = {};
    p.tiles = (const uint4*)tiles;
    p.nrt = (int)(opad_of(out) / TILE_ROWS);
    p.nkt = (int)(kpad_of(in) / TILE_K);
    p.out = (int)out;
    p.rows = rows;
    p.cols = rows * stage.terms_out;
    p.acc = acc;
    p.zero_ptr = zero_ptr;
    p.zero_count = (int)zero_count;
    p.st = stage;
    p.sx_pub = sx_pub;
    p.xsum_pub = xsum_pub;
    if (p.cols < 1 || p.cols > 8 || stage.terms > 3 || stage.terms_out > 3) return ROTOR_B200_ERR_ARG;
    if ((stage.mode == VS_OPROJ || stage.mode == VS_FFN || stage.mode == VS_DOWN) && stage.acc.planes != 1)
        return ROTOR_B200_ERR_ARG;
    const long long total = (long long)p.nrt * p.nkt;
    int grid = sm_count();
    if (grid > total) grid = (int)total;
    const int chunk = (int)((total + grid - 1) / grid);
    p.nslot = (chunk + p.nkt - 1) / p.nkt + 1;
    if (p.cols == 1) return launch_fused<false, 1>(p, grid, st);
    if (p.cols == 2) return launch_fused<false, 2>(p, grid, st);
    return launch_fused<true, 1>(p, grid, st);
}

}  // namespace rb
