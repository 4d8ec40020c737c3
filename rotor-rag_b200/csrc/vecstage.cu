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
#include "model.cuh"
#include "quant.cuh"

namespace rb {

// y[i] = row[i] / sqrt(mean(row^2) + eps) * w[i], in place.
__device__ __forceinline__ void rmsnorm_inplace(float* row, int n, const float* __restrict__ w, float eps,
                                                float* scratch) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss += row[i] * row[i];
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) row[i] = row[i] * inv * w[i];
    __syncthreads();
}

// Dequantised BitLinear output element: wscale * sum_t sx[t] * (sum over split planes of acc).
__device__ __forceinline__ float deq(const AccView& a, const float* __restrict__ sx, int m, int terms, int o,
                                     float wscale) {
    float v = 0.f;
    for (int t = 0; t < terms; ++t) {
        const size_t col = (size_t)m * terms + t;
        int s = 0;
        for (int p = 0; p < a.planes; ++p) s += a.acc[(size_t)p * a.plane_stride + col * a.out + o];
        v += (float)s * sx[col];
    }
    return v * wscale;
}

__global__ void __launch_bounds__(1024) vec_stage_kernel(VecStageParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* scratch = reinterpret_cast<float*>(smem_raw);
    float* row = scratch + 64;
    const int m = blockIdx.x;
    const int n = p.n;

    // ---- build the float row
    switch (p.mode) {
        case VS_EMBED: {  // h = embed[id]
            const long long id = p.ids[m];
            const __nv_bfloat16* e = p.embed + (size_t)id * n;
            for (int i = threadIdx.x; i < n; i += blockDim.x) {
                const float v = __bfloat162float(e[i]);
                row[i] = v;
                p.h[(size_t)m * n + i] = v;
            }
            break;
        }
        case VS_PLAIN: {  // row = src
            for (int i = threadIdx.x; i < n; i += blockDim.x) row[i] = p.src[(size_t)m * n + i];
            break;
        }
        case VS_OPROJ: {  // h += subnorm(deq(acc_o)) ; row = h
            for (int i = threadIdx.x; i < n; i += blockDim.x) row[i] = deq(p.acc, p.sx_in, m, p.terms, i, p.wscale0);
            __syncthreads();
            rmsnorm_inplace(row, n, p.norm0, p.eps, scratch);
            for (int i = threadIdx.x; i < n; i += blockDim.x) {
                const float v = p.h[(size_t)m * n + i] + row[i];
                row[i] = v;
                p.h[(size_t)m * n + i] = v;
            }
            break;
        }
        case VS_FFN: {  // row = act(gate, up)
            for (int i = threadIdx.x; i < n; i += blockDim.x) {
                const float g = deq(p.acc, p.sx_in, m, p.terms, i, p.wscale0);
                const float u = deq(p.acc, p.sx_in, m, p.terms, n + i, p.wscale1);
                float v;
                if (p.ffn_act == ROTOR_B200_FFN_RELU2) {
                    const float r = fmaxf(g, 0.f);
                    v = r * r * u;
                } else {
                    const float c = fminf(fmaxf(u, -20.f), 20.f);
                    v = g * (c / (1.f + expf(-c)));
                }
                row[i] = v;
            }
            break;
        }
        case VS_DEQ: {  // row = deq(acc)
            for (int i = threadIdx.x; i < n; i += blockDim.x) row[i] = deq(p.acc, p.sx_in, m, p.terms, i, p.wscale0);
            break;
        }
        case VS_DOWN: {  // h += deq(acc_down) ; row = h
            for (int i = threadIdx.x; i < n; i += blockDim.x) {
                const float v = p.h[(size_t)m * n + i] + deq(p.acc, p.sx_in, m, p.terms, i, p.wscale0);
                row[i] = v;
                p.h[(size_t)m * n + i] = v;
            }
            break;
        }
    }
    __syncthreads();

    // ---- pre-norm of the consumer, then its quantiser (or a float copy for the LM head)
    if (p.norm1) rmsnorm_inplace(row, n, p.norm1, p.eps, scratch);
    if (p.y_out)
        for (int i = threadIdx.x; i < n; i += blockDim.x) p.y_out[(size_t)m * n + i] = row[i];
    if (p.xq) {
        __syncthreads();
        quantize_row_from_smem(row, n, p.kpad, p.terms_out, p.xq + (size_t)m * p.terms_out * p.kpad,
                               p.sx_out + (size_t)m * p.terms_out, p.xsum_out + (size_t)m * p.terms_out, scratch);
    }
}

int configure_vec_stage() {
    RB_CUDA(cudaFuncSetAttribute(vec_stage_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    return ROTOR_B200_OK;
}

int launch_vec_stage(const VecStageParams& p, int rows, cudaStream_t st) {
    const size_t smem = 64 * 4 + (size_t)p.n * 4;
    static size_t configured = 48 * 1024;
    if (smem > configured) {
        if (smem > 200 * 1024) return ROTOR_B200_ERR_SHAPE;
        RB_CUDA(cudaFuncSetAttribute(vec_stage_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        configured = 200 * 1024;
    }
    const int threads = p.n >= 2048 ? 1024 : (p.n >= 512 ? 256 : 128);
    vec_stage_kernel<<<rows, threads, smem, st>>>(p);
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
