// Device body of the vector stages (see vecstage.cu): shared by the stand-alone kernel
// (one CTA per token row) and by the tail that the last CTA of a BitLinear product runs.
#pragma once
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
        for (int p = 0; p < a.planes; ++p) s += __ldcg(&a.acc[(size_t)p * a.plane_stride + col * a.out + o]);
        v += (float)s * __ldcg(&sx[col]);
    }
    return v * wscale;
}

// One token row `m` through the stage.  `row` (n floats) and `scratch` (64 floats) are
// shared memory.  All threads of the block must call.  Data produced by other CTAs
// (accumulators, residual stream, activation scales) is read past L1.
__device__ __forceinline__ void vec_stage_row(const VecStageParams& p, int m, float* row, float* scratch) {
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
            for (int i = threadIdx.x; i < n; i += blockDim.x) row[i] = __ldcg(&p.src[(size_t)m * n + i]);
            break;
        }
        case VS_OPROJ: {  // h += subnorm(deq(acc_o)) ; row = h
            for (int i = threadIdx.x; i < n; i += blockDim.x) row[i] = deq(p.acc, p.sx_in, m, p.terms, i, p.wscale0);
            __syncthreads();
            rmsnorm_inplace(row, n, p.norm0, p.eps, scratch);
            for (int i = threadIdx.x; i < n; i += blockDim.x) {
                const float v = __ldcg(&p.h[(size_t)m * n + i]) + row[i];
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
                const float v = __ldcg(&p.h[(size_t)m * n + i]) + deq(p.acc, p.sx_in, m, p.terms, i, p.wscale0);
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

}  // namespace rb
