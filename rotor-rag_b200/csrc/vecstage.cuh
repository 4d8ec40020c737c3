// Device body of the vector stages (see vecstage.cu): shared by the stand-alone kernel
// (one CTA per token row) and by the tail that the last CTA of a BitLinear product runs.
#pragma once
#include "model.cuh"
#include "quant.cuh"

namespace rb {

constexpr int VS_U = 8;  // elements per thread whose global loads are in flight together

// y[i] = row[i] / sqrt(mean(row^2) + eps) * w[i], in place.  The first batch of norm
// weights is requested before the reduction so that its latency hides behind it.
// ext_ss / n_total: when the row is a slice of a longer one, the sum of squares and width of
// the whole row (nullptr / 0 = this row alone).
__device__ __forceinline__ void rmsnorm_inplace(float* row, int n, const float* __restrict__ w, float eps,
                                                float* scratch, const float* ext_ss = nullptr, int n_total = 0) {
    const int bd = blockDim.x;
    float wv[VS_U];
#pragma unroll
    for (int u = 0; u < VS_U; ++u) {
        const int i = threadIdx.x + u * bd;
        wv[u] = i < n ? __ldg(&w[i]) : 0.f;
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += bd) ss += row[i] * row[i];
    ss = block_sum(ss, scratch);
    if (ext_ss) ss = *ext_ss;
    const float inv = 1.0f / sqrtf(ss / (float)(n_total ? n_total : n) + eps);
    for (int i0 = threadIdx.x; i0 < n; i0 += VS_U * bd) {
        float wn[VS_U];
#pragma unroll
        for (int u = 0; u < VS_U; ++u) {  // next batch in flight while this one is applied
            const int i = i0 + (VS_U + u) * bd;
            wn[u] = i < n ? __ldg(&w[i]) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < VS_U; ++u) {
            const int i = i0 + u * bd;
            if (i < n) row[i] = row[i] * inv * wv[u];
        }
#pragma unroll
        for (int u = 0; u < VS_U; ++u) wv[u] = wn[u];
    }
    __syncthreads();
}

// Dequantised BitLinear outputs for VS_U elements (index i0 + u*stride, valid while < n):
//   v[u] = wscale * sum_t sx[t] * (sum over split planes of acc[t][off + index]).
// TERMS / PLANES are compile-time so that the loads form straight-line code and are all
// issued before the first use; 0 selects the run-time loop (any value, slower).
template <int TERMS, int PLANES>
__device__ __forceinline__ void deq_batch(const AccView& a, const float* sxv, int terms, size_t col0, int off, int i0,
                                          int stride, int n, float wscale, float (&v)[VS_U]) {
    if constexpr (TERMS > 0) {
        int s[VS_U][TERMS];
#pragma unroll
        for (int u = 0; u < VS_U; ++u) {
            const int i = i0 + u * stride;
#pragma unroll
            for (int t = 0; t < TERMS; ++t) {
                int acc = 0;
#pragma unroll
                for (int p = 0; p < PLANES; ++p)
                    if (i < n) acc += __ldcg(&a.acc[(size_t)p * a.plane_stride + (col0 + t) * a.out + off + i]);
                s[u][t] = acc;
            }
        }
#pragma unroll
        for (int u = 0; u < VS_U; ++u) {
            float f = 0.f;
#pragma unroll
            for (int t = 0; t < TERMS; ++t) f += (float)s[u][t] * sxv[t];
            v[u] = f * wscale;
        }
    } else {
        for (int u = 0; u < VS_U; ++u) {
            const int i = i0 + u * stride;
            float f = 0.f;
            if (i < n)
                for (int t = 0; t < terms; ++t) {
                    int acc = 0;
                    for (int p = 0; p < a.planes; ++p)
                        acc += __ldcg(&a.acc[(size_t)p * a.plane_stride + (col0 + t) * a.out + off + i]);
                    f += (float)acc * sxv[t];
                }
            v[u] = f * wscale;
        }
    }
}

__device__ __forceinline__ void deq_dispatch(const AccView& a, const float* sxv, int terms, size_t col0, int off,
                                             int i0, int stride, int n, float wscale, float (&v)[VS_U]) {
#define RB_DEQ(T, P) deq_batch<T, P>(a, sxv, terms, col0, off, i0, stride, n, wscale, v)
    if (a.planes == 1) {
        switch (terms) {
            case 1: RB_DEQ(1, 1); return;
            case 2: RB_DEQ(2, 1); return;
            case 3: RB_DEQ(3, 1); return;
        }
    } else if (a.planes == 2) {
        switch (terms) {
            case 1: RB_DEQ(1, 2); return;
            case 2: RB_DEQ(2, 2); return;
            case 3: RB_DEQ(3, 2); return;
        }
    }
    RB_DEQ(0, 0);
#undef RB_DEQ
}

// One token row `m` through the stage.  `row` (n floats) and `scratch` (64 floats) are
// shared memory.  All threads of the block must call.  Data produced by other CTAs
// (accumulators, residual stream, activation scales) is read past L1.  Elements are
// handled VS_U at a time per thread with every global load issued before the first use:
// the stage often runs on one small CTA, where serialised L2 round trips, not
// arithmetic, would set its duration.
//
// `writer`: whether this CTA performs the stage's global side effects (residual stream,
// float copy, quantised output).  When many CTAs run the same stage redundantly in their
// prologue, exactly one of them is the writer.  `sink` redirects the quantiser's output
// (null = the global buffers named in p).
struct QuantSink {
    int8_t* xq;       // term t at xq + t*tstride
    float* sx;
    int32_t* xsum;
    size_t tstride;
};

__device__ __forceinline__ void vec_stage_row(const VecStageParams& p, int m, float* row, float* scratch,
                                              bool writer = true, const QuantSink* sink = nullptr) {
    const int n = p.n;
    float* hdst = p.h_out ? p.h_out : p.h;
    if (p.mode == VS_ATTN) {
        // weights of every (head, slice): f = exp(m_s - M) / L, then the weighted sum of partials
        const int D = p.head_dim, ns = p.nsplit, nh = p.n_heads;
        float* wf = row + n;  // [n_heads][nsplit] x2, directly behind the row
        float* wl = wf + nh * ns;
        const size_t hb = (size_t)m * nh * ns;
        for (int e = threadIdx.x; e < nh * ns; e += blockDim.x) {
            wf[e] = __ldcg(p.part_m + hb + e);
            wl[e] = __ldcg(p.part_l + hb + e);
        }
        __syncthreads();
        for (int h = threadIdx.x; h < nh; h += blockDim.x) {
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
        constexpr int MU = 4;
        for (int i0 = threadIdx.x; i0 < n; i0 += MU * blockDim.x) {
            float o[MU];
#pragma unroll
            for (int u = 0; u < MU; ++u) o[u] = 0.f;
            for (int s2 = 0; s2 < ns; ++s2) {
                float pv[MU];
#pragma unroll
                for (int u = 0; u < MU; ++u) {
                    const int idx = i0 + u * blockDim.x;
                    pv[u] = idx < n ? __ldcg(p.part_o + (hb + (size_t)(idx / D) * ns + s2) * D + idx % D) : 0.f;
                }
#pragma unroll
                for (int u = 0; u < MU; ++u) {
                    const int idx = i0 + u * blockDim.x;
                    if (idx < n) o[u] += pv[u] * wf[(idx / D) * ns + s2];
                }
            }
#pragma unroll
            for (int u = 0; u < MU; ++u) {
                const int idx = i0 + u * blockDim.x;
                if (idx < n) row[idx] = o[u];
            }
        }
        __syncthreads();
    }
    const int bd = blockDim.x;
    const bool from_acc = p.mode == VS_OPROJ || p.mode == VS_FFN || p.mode == VS_DOWN || p.mode == VS_DEQ;
    float sxv[4] = {0.f, 0.f, 0.f, 0.f};
    const size_t col0 = (size_t)m * p.terms;
    if (from_acc)
        for (int t = 0; t < p.terms; ++t) sxv[t] = __ldcg(&p.sx_in[col0 + t]);

    for (int i0 = threadIdx.x; i0 < n && p.mode != VS_ATTN; i0 += VS_U * bd) {
        float v[VS_U], w[VS_U];
        if (p.mode == VS_EMBED) {
            const long long id = p.ids[m];
            const __nv_bfloat16* e = p.embed + (size_t)id * n;
#pragma unroll
            for (int u = 0; u < VS_U; ++u) {
                const int i = i0 + u * bd;
                v[u] = i < n ? __bfloat162float(e[i]) : 0.f;
            }
        } else if (p.mode == VS_PLAIN) {
#pragma unroll
            for (int u = 0; u < VS_U; ++u) {
                const int i = i0 + u * bd;
                v[u] = i < n ? __ldcg(&p.src[(size_t)m * n + i]) : 0.f;
            }
        } else {
            if (p.mode == VS_DOWN) {
#pragma unroll
                for (int u = 0; u < VS_U; ++u) {
                    const int i = i0 + u * bd;
                    w[u] = i < n ? __ldcg(&p.h[(size_t)m * n + i]) : 0.f;
                }
            }
            deq_dispatch(p.acc, sxv, p.terms, col0, 0, i0, bd, n, p.wscale0, v);
            if (p.mode == VS_FFN) deq_dispatch(p.acc, sxv, p.terms, col0, n, i0, bd, n, p.wscale1, w);
        }
#pragma unroll
        for (int u = 0; u < VS_U; ++u) {
            const int i = i0 + u * bd;
            if (i >= n) continue;
            float r = v[u];
            if (p.mode == VS_FFN) {  // gating
                if (p.ffn_act == ROTOR_B200_FFN_RELU2) {
                    const float g = fmaxf(r, 0.f);
                    r = g * g * w[u];
                } else {
                    const float c = fminf(fmaxf(w[u], -20.f), 20.f);
                    r = r * (c / (1.f + expf(-c)));
                }
            } else if (p.mode == VS_DOWN) {  // residual add
                r += w[u];
                if (writer) hdst[(size_t)m * n + i] = r;
            } else if (p.mode == VS_EMBED) {
                if (writer) hdst[(size_t)m * n + i] = r;
            }
            row[i] = r;
        }
    }
    if (p.mode == VS_OPROJ) {  // h += subnorm(row); row = h
        __syncthreads();
        rmsnorm_inplace(row, n, p.norm0, p.eps, scratch);
        for (int i0 = threadIdx.x; i0 < n; i0 += VS_U * bd) {
            float hv[VS_U];
#pragma unroll
            for (int u = 0; u < VS_U; ++u) {
                const int i = i0 + u * bd;
                hv[u] = i < n ? __ldcg(&p.h[(size_t)m * n + i]) : 0.f;
            }
#pragma unroll
            for (int u = 0; u < VS_U; ++u) {
                const int i = i0 + u * bd;
                if (i < n) {
                    const float r = hv[u] + row[i];
                    row[i] = r;
                    if (writer) hdst[(size_t)m * n + i] = r;
                }
            }
        }
    }
    __syncthreads();

    // ---- statistics for sharded rows, pre-norm of the consumer, then its quantiser (or a float copy)
    if (p.out_sumsq) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < n; i += blockDim.x) ss += row[i] * row[i];
        ss = block_sum(ss, scratch);
        if (threadIdx.x == 0 && writer) p.out_sumsq[m] = ss;
        __syncthreads();
    }
    if (p.norm1) rmsnorm_inplace(row, n, p.norm1, p.eps, scratch, p.ext_sumsq ? p.ext_sumsq + m : nullptr, p.norm_n);
    if (p.out_absmax) {
        float mx = 0.f;
        for (int i = threadIdx.x; i < n; i += blockDim.x) mx = fmaxf(mx, fabsf(row[i]));
        mx = block_max(mx, scratch);
        if (threadIdx.x == 0 && writer) p.out_absmax[m] = mx;
        __syncthreads();
    }
    if (p.y_out && writer)
        for (int i = threadIdx.x; i < n; i += blockDim.x) p.y_out[(size_t)m * n + i] = row[i];
    if (sink) {
        __syncthreads();
        quantize_row_from_smem(row, n, p.kpad, p.terms_out, sink->xq, sink->sx, sink->xsum, scratch, sink->tstride);
    } else if (p.xq && writer) {
        __syncthreads();
        quantize_row_from_smem(row, n, p.kpad, p.terms_out, p.xq + (size_t)m * p.terms_out * p.kpad,
                               p.sx_out + (size_t)m * p.terms_out, p.xsum_out + (size_t)m * p.terms_out, scratch, 0,
                               p.ext_absmax ? p.ext_absmax + m : nullptr);
    }
}

}  // namespace rb
