// Tied LM head: logits[m][v] = sum_k x[m][k] * embed[v][k] with a bf16 table
// (np.dot(hidden, embed_tokens.T), src/rotor/bitnet_model.py:231-235), fused with the
// greedy pick (int(np.argmax(logits)), lowest index on ties, src/rotor/generation.py:42).
//
// HBM-bound on the table (vocab * d * 2 bytes per pass).  Each warp owns rows of the
// table four at a time; a lane reads 8 bf16 (one 128-bit load) per row per 256 columns
// and keeps the activation slice it needs in shared memory.  Up to LM_ROWS token rows
// share one pass over the table.
#include "lmhead_body.cuh"

namespace rb {

constexpr int LM_WARPS = 8;
constexpr int LM_PARTS = 148 * 4;  // CTAs = argmax partials per token row

int lmhead_parts() { return LM_PARTS; }

template <int NROWS>
__global__ void __launch_bounds__(LM_WARPS * 32) lmhead_kernel(const __grid_constant__ LmHeadParams p, int row0) {
    extern __shared__ __align__(16) float xs[];  // [NROWS][d]
    pdl_wait();
    pdl_trigger();
    lmhead_body<NROWS>(p, row0, xs);
}

__global__ void argmax_final_kernel(const float* __restrict__ part_val, const int* __restrict__ part_idx, int nparts,
                                    long long* __restrict__ out, float* __restrict__ out_val) {
    const int m = blockIdx.x;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < nparts; i += blockDim.x) {
        const float v = part_val[(size_t)m * nparts + i];
        const int id = part_idx[(size_t)m * nparts + i];
        if (v > bv || (v == bv && id < bi)) {
            bv = v;
            bi = id;
        }
    }
    __shared__ float sv[32];
    __shared__ int sidx[32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) {
            bv = ov;
            bi = oi;
        }
    }
    if ((threadIdx.x & 31) == 0) {
        sv[threadIdx.x >> 5] = bv;
        sidx[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
            if (sv[w] > bv || (sv[w] == bv && sidx[w] < bi)) {
                bv = sv[w];
                bi = sidx[w];
            }
        out[m] = bi;
        if (out_val) out_val[m] = bv;
    }
}

template <int NROWS>
static int launch_lm(const LmHeadParams& p, int row0, cudaStream_t st) {
    const size_t smem = (size_t)NROWS * p.d * sizeof(float);
    if (smem > 48 * 1024) {
        static PerDevice<bool> once;
        bool& configured = once.here();
        if (!configured) {
            RB_CUDA(cudaFuncSetAttribute(lmhead_kernel<NROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         200 * 1024));
            configured = true;
        }
        if (smem > 200 * 1024) return ROTOR_B200_ERR_SHAPE;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(LM_PARTS);
    cfg.blockDim = dim3(LM_WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_use_pdl ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, lmhead_kernel<NROWS>, p, row0) != cudaSuccess) {
        ++g_launch_count;
        return ROTOR_B200_ERR_CUDA;
    }
    return launch_status();
}

int configure_lmhead() {
    if (int rc = configure_lmhead_mma()) return rc;
    RB_CUDA(cudaFuncSetAttribute(lmhead_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    RB_CUDA(cudaFuncSetAttribute(lmhead_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    RB_CUDA(cudaFuncSetAttribute(lmhead_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    RB_CUDA(cudaFuncSetAttribute(lmhead_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    return ROTOR_B200_OK;
}

int launch_lmhead(const LmHeadParams& pin, int rows, cudaStream_t st) {
    if (pin.d % 256 != 0) return ROTOR_B200_ERR_SHAPE;
    LmHeadParams p = pin;
    // the fused pick needs every partial in one launch; otherwise a separate kernel merges them
    const bool fused = p.tail_counter && p.argmax_out && rows <= LM_ROWS;
    if (p.pro_y && (rows > LM_ROWS || !p.pro_h || !p.pro_norm)) return ROTOR_B200_ERR_ARG;
    if (!fused) {
        if (p.adv_log) return ROTOR_B200_ERR_ARG;
        p.tail_counter = nullptr;
    }
    int rc = ROTOR_B200_OK;
    if (p.xsplit && !p.pro_y && !fused && lmhead_mma_supported(rows, p.d)) {
        // many rows: one pass over the table on the tensor cores
        const bool pick = p.argmax_out != nullptr;
        rc = launch_lmhead_mma(p.embed, p.x, p.xsplit, rows, p.vocab, p.d, p.logits, pick ? p.part_val : nullptr,
                               p.part_idx, st);
        if (rc) return rc;
        if (pick) {
            argmax_final_kernel<<<rows, 256, 0, st>>>(p.part_val, p.part_idx, lmhead_mma_parts(p.vocab), p.argmax_out,
                                                      p.argmax_val);
            rc = launch_status();
        }
        return rc;
    }
    for (int r0 = 0; r0 < rows && !rc; r0 += LM_ROWS) {
        const int n = rows - r0 < LM_ROWS ? rows - r0 : LM_ROWS;
        switch (n) {
            case 1: rc = launch_lm<1>(p, r0, st); break;
            case 2: rc = launch_lm<2>(p, r0, st); break;
            case 3: rc = launch_lm<3>(p, r0, st); break;
            default: rc = launch_lm<4>(p, r0, st); break;
        }
    }
    if (rc) return rc;
    if (p.argmax_out && !fused) {
        argmax_final_kernel<<<rows, 256, 0, st>>>(p.part_val, p.part_idx, p.nparts, p.argmax_out, p.argmax_val);
        rc = launch_status();
    }
    return rc;
}

}  // namespace rb
