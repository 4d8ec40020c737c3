// Vector stages between the BitLinear products of a transformer block: one CTA per token
// row.  Each stage reads the int32 accumulators of the previous product (dequantising on
// the fly), applies the block's float32 glue (sub-norm, residual, gating, pre-norm) and
// ends in the activation quantiser that feeds the next product, so a 2560/6912-wide row
// makes one trip through shared memory instead of five through HBM.
//
// Glue arithmetic follows the reference's NumPy code:
//   RMSNorm        x / sqrt(mean(x^2) + eps) * w                 src/rotor/transformer.py:24-36
//   gating         gate * silu(clip(up, -20, 20))                src/rotor/transformer.py:328-351
//   block wiring   x + norm(attn(..)), x + ffn(norm(x))          src/rotor/transformer.py:383-413
//   sub-norm after the output projection                         src/rotor/transformer.py:283-287
#include "vecstage.cuh"

namespace rb {

__global__ void __launch_bounds__(1024) vec_stage_kernel(VecStageParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* scratch = reinterpret_cast<float*>(smem_raw);
    pdl_wait();
    vec_stage_row(p, blockIdx.x, scratch + 64, scratch);
}

int configure_vec_stage() {
    RB_CUDA(cudaFuncSetAttribute(vec_stage_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    return ROTOR_B200_OK;
}

int launch_vec_stage(const VecStageParams& p, int rows, cudaStream_t st) {
    if (row_stage_supported(p, rows)) return launch_row_stage(p, rows, st);  // many rows: register-resident kernel
    const size_t smem = 64 * 4 + (size_t)p.n * 4 +
                        (p.mode == VS_ATTN ? 2 * (size_t)p.n_heads * p.nsplit * 4 : 0);  // merge weights behind the row
    static PerDevice<size_t> once;
    size_t& configured = once.here();
    if (smem > 48 * 1024 && smem > configured) {
        if (smem > 200 * 1024) return ROTOR_B200_ERR_SHAPE;
        RB_CUDA(cudaFuncSetAttribute(vec_stage_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        configured = 200 * 1024;
    }
    // one CTA per row: a single row wants the widest CTA; with many rows (prefill) narrower CTAs let
    // several rows share an SM and hide each other's reduction and load latencies
    const int threads = rows >= 64 ? (p.n >= 512 ? 256 : 128) : (p.n >= 2048 ? 1024 : (p.n >= 512 ? 256 : 128));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rows);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_use_pdl ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, vec_stage_kernel, p) != cudaSuccess) {
        ++g_launch_count;
        return ROTOR_B200_ERR_CUDA;
    }
    return launch_status();
}

}  // namespace rb

using namespace rb;

/* RMSNorm.forward on device rows (src/rotor/transformer.py:24-36). */
extern "C" int rotor_b200_rmsnorm(const float* x, size_t rows, size_t n, const float* weight, float eps, float* y,
                                  void* stream) {
    RB_REQUIRE(x && weight && y && rows > 0 && n > 0);
    VecStageParams p = {};
    p.mode = VS_PLAIN;
    p.n = (int)n;
    p.src = x;
    p.norm1 = weight;
    p.eps = eps;
    p.y_out = y;
    return launch_vec_stage(p, (int)rows, as_stream(stream));
}
