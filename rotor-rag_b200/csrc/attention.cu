// Attention around the q/k/v BitLinear product: dequantise the stacked [q;k;v]
// accumulators, optionally rotate q and k, append k and v to the pre-allocated cache,
// then softmax(q k^T / sqrt(D)) v with grouped KV heads.
//
// Follows MultiHeadAttention.forward (src/rotor/transformer.py:206-292): the cache keeps
// K and V before head repetition (line 250-257), query head h reads KV head
// h / (n_heads / n_kv_heads) (np.repeat, line 260-263), scores are scaled by
// 1/sqrt(head_dim) (line 267) and no mask is applied unless asked for (line 270-271).
// The cache is a fixed [batch][n_kv][max_seq][D] float32 buffer written in place at
// position past_len + s instead of the reference's per-step np.concatenate.
#include <cstdlib>
#include "attn_body.cuh"
#include "quant.cuh"

RB_TRACE_DEFINE(rotor_b200_trace_read_attn)

namespace rb {

// One CTA per token row.  Work items are rotation pairs (i, i + D/2) of q and k heads and
// single elements of v.
__global__ void __launch_bounds__(256) qkv_finish_kernel(QkvFinishParams p) {
    const int m = blockIdx.x;
    const int b = m / p.seq, s = m % p.seq;
    const int pos = p.past_len[b] + s;
    const int D = p.head_dim, half = D / 2;
    const int dq = p.n_heads * D, dkv = p.n_kv_heads * D;
    if (pos >= p.max_seq) return;  // capacity is checked on the host; never write out of bounds
    const int q_pairs = p.n_heads * half, k_pairs = p.n_kv_heads * half;
    for (int w = threadIdx.x; w < q_pairs + k_pairs; w += blockDim.x) {
        const bool is_q = w < q_pairs;
        const int ww = is_q ? w : w - q_pairs;
        const int head = ww / half, i = ww % half;
        const int base = (is_q ? 0 : dq) + head * D;
        const float sc = is_q ? p.sq : p.sk;
        float a = deq_acc(p.acc, p.sx, m, p.terms, base + i, sc);
        float c = deq_acc(p.acc, p.sx, m, p.terms, base + i + half, sc);
        if (p.rope) {
            const float2 cs = p.rope[(size_t)pos * half + i];
            const float ra = a * cs.x - c * cs.y;
            const float rc = c * cs.x + a * cs.y;
            a = ra;
            c = rc;
        }
        if (is_q) {
            float* q = p.q + (size_t)m * dq + head * D;
            q[i] = a;
            q[i + half] = c;
        } else {
            float* k = p.k_cache + (((size_t)b * p.n_kv_heads + head) * p.max_seq + pos) * D;
            k[i] = a;
            k[i + half] = c;
        }
    }
    for (int e = threadIdx.x; e < dkv; e += blockDim.x) {
        const int head = e / D, i = e % D;
        p.v_cache[(((size_t)b * p.n_kv_heads + head) * p.max_seq + pos) * D + i] =
            deq_acc(p.acc, p.sx, m, p.terms, dq + dkv + e, p.sv);
    }
}

// cos/sin of pos * theta^(-2i/D), evaluated in double, stored as float2 [max_seq][D/2].
__global__ void rope_table_kernel(float2* table, int max_seq, int half, double theta) {
    const int total = max_seq * half;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < total; e += gridDim.x * blockDim.x) {
        const int pos = e / half, i = e % half;
        const double ang = (double)pos * pow(theta, -(double)i / (double)half);
        double sn, cs;
        sincos(ang, &sn, &cs);
        table[e] = make_float2((float)cs, (float)sn);
    }
}

int launch_rope_table(float2* table, int max_seq, int head_dim, float theta, cudaStream_t st) {
    rope_table_kernel<<<148, 256, 0, st>>>(table, max_seq, head_dim / 2, (double)theta);
    return launch_status();
}


// The same for many rows (prefill): 128-bit loads, four rotary pairs per thread, every load of the
// thread in flight before the first use.  Needs complete accumulators in one plane, out % 4 == 0.
__device__ __forceinline__ float4 qf_deq4(const QkvFinishParams& p, const float (&sxv)[3], int m, int o, float wscale) {
    float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
    int4 a[3];
#pragma unroll
    for (int t = 0; t < 3; ++t)
        if (t < p.terms) a[t] = __ldcg(reinterpret_cast<const int4*>(p.acc.acc + ((size_t)m * p.terms + t) * p.acc.out + o));
#pragma unroll
    for (int t = 0; t < 3; ++t)
        if (t < p.terms) {
            f.x += (float)a[t].x * sxv[t];
            f.y += (float)a[t].y * sxv[t];
            f.z += (float)a[t].z * sxv[t];
            f.w += (float)a[t].w * sxv[t];
        }
    return make_float4(f.x * wscale, f.y * wscale, f.z * wscale, f.w * wscale);
}

__global__ void __launch_bounds__(256) qkv_finish_vec_kernel(const __grid_constant__ QkvFinishParams p) {
    const int m = blockIdx.x;
    const int b = m / p.seq, s = m % p.seq;
    const int pos = p.past_len[b] + s;
    const int D = p.head_dim, half = D / 2, h4 = half / 4;
    const int dq = p.n_heads * D, dkv = p.n_kv_heads * D;
    if (pos >= p.max_seq) return;
    float sxv[3] = {0.f, 0.f, 0.f};
    for (int t = 0; t < p.terms; ++t) sxv[t] = __ldcg(&p.sx[(size_t)m * p.terms + t]);
    const int q_items = p.n_heads * h4, k_items = p.n_kv_heads * h4, v_items = dkv / 4;
    for (int w = threadIdx.x; w < q_items + k_items + v_items; w += blockDim.x) {
        if (w >= q_items + k_items) {  // V: plain dequantise into the cache
            const int e = (w - q_items - k_items) * 4, head = e / D, i = e % D;
            *reinterpret_cast<float4*>(p.v_cache + (((size_t)b * p.n_kv_heads + head) * p.max_seq + pos) * D + i) =
                qf_deq4(p, sxv, m, dq + dkv + e, p.sv);
            continue;
        }
        const bool is_q = w < q_items;
        const int ww = is_q ? w : w - q_items;
        const int head = ww / h4, i = (ww % h4) * 4;
        const int base = (is_q ? 0 : dq) + head * D;
        const float sc = is_q ? p.sq : p.sk;
        float4 a = qf_deq4(p, sxv, m, base + i, sc);
        float4 c = qf_deq4(p, sxv, m, base + i + half, sc);
        if (p.rope) {
            const float4 cs0 = *reinterpret_cast<const float4*>(p.rope + (size_t)pos * half + i);      // (cos, sin) x 2
            const float4 cs1 = *reinterpret_cast<const float4*>(p.rope + (size_t)pos * half + i + 2);
            const float4 ra = make_float4(a.x * cs0.x - c.x * cs0.y, a.y * cs0.z - c.y * cs0.w,
                                          a.z * cs1.x - c.z * cs1.y, a.w * cs1.z - c.w * cs1.w);
            const float4 rc = make_float4(c.x * cs0.x + a.x * cs0.y, c.y * cs0.z + a.y * cs0.w,
                                          c.z * cs1.x + a.z * cs1.y, c.w * cs1.z + a.w * cs1.w);
            a = ra;
            c = rc;
        }
        float* dst = is_q ? p.q + (size_t)m * dq + head * D
                          : p.k_cache + (((size_t)b * p.n_kv_heads + head) * p.max_seq + pos) * D;
        *reinterpret_cast<float4*>(dst + i) = a;
        *reinterpret_cast<float4*>(dst + i + half) = c;
    }
}

int launch_qkv_finish(const QkvFinishParams& p, int rows, cudaStream_t st) {
    if (rows >= 64 && p.acc.planes == 1 && p.acc.out % 4 == 0 && p.head_dim % 8 == 0 && p.terms >= 1 && p.terms <= 3)
        qkv_finish_vec_kernel<<<rows, 256, 0, st>>>(p);
    else
        qkv_finish_kernel<<<rows, 256, 0, st>>>(p);
    return launch_status();
}

// One CTA (4 warps) per (query head, token row).  Each warp walks every fourth key with an
// online softmax; lanes split the head dimension (EPL contiguous floats per lane).
template <int EPL>
__global__ void __launch_bounds__(128) attention_kernel(AttnParams p) {
    constexpr int D = EPL * 32;
    __shared__ float s_m[4], s_l[4];
    __shared__ float s_o[4][D];
    const int h = blockIdx.x, m = blockIdx.y;
    const int b = m / p.seq, s = m % p.seq;
    const int past = p.past_len[b];
    int T = p.causal ? past + s + 1 : past + p.seq;
    if (T > p.max_seq) T = p.max_seq;
    const int hk = h / (p.n_heads / p.n_kv_heads);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float scale = 1.0f / sqrtf((float)D);

    float q[EPL], o[EPL];
    const float* qp = p.q + (size_t)m * p.n_heads * D + h * D + lane * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
        q[e] = qp[e] * scale;
        o[e] = 0.f;
    }
    const float* kb = p.k_cache + ((size_t)b * p.n_kv_heads + hk) * p.max_seq * D + lane * EPL;
    const float* vb = p.v_cache + ((size_t)b * p.n_kv_heads + hk) * p.max_seq * D + lane * EPL;
    float mx = -INFINITY, l = 0.f;
    for (int t = warp; t < T; t += 4) {
        float kv[EPL], vv[EPL];
        if constexpr (EPL == 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(kb + (size_t)t * D);
            const float4 v4 = *reinterpret_cast<const float4*>(vb + (size_t)t * D);
            kv[0] = k4.x; kv[1] = k4.y; kv[2] = k4.z; kv[3] = k4.w;
            vv[0] = v4.x; vv[1] = v4.y; vv[2] = v4.z; vv[3] = v4.w;
        } else {
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                kv[e] = kb[(size_t)t * D + e];
                vv[e] = vb[(size_t)t * D + e];
            }
        }
        float sc = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) sc += q[e] * kv[e];
        sc = warp_sum(sc);
        const float mn = fmaxf(mx, sc);
        const float corr = __expf(mx - mn), pr = __expf(sc - mn);
        l = l * corr + pr;
#pragma unroll
        for (int e = 0; e < EPL; ++e) o[e] = o[e] * corr + pr * vv[e];
        mx = mn;
    }
    if (lane == 0) {
        s_m[warp] = mx;
        s_l[warp] = l;
    }
#pragma unroll
    for (int e = 0; e < EPL; ++e) s_o[warp][lane * EPL + e] = o[e];
    __syncthreads();
    if (warp == 0) {
        float M = fmaxf(fmaxf(s_m[0], s_m[1]), fmaxf(s_m[2], s_m[3]));
        float L = 0.f, f[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            f[w] = s_m[w] == -INFINITY ? 0.f : __expf(s_m[w] - M);
            L += s_l[w] * f[w];
        }
        float* op = p.out + (size_t)m * p.n_heads * D + h * D + lane * EPL;
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
            float acc = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) acc += s_o[w][lane * EPL + e] * f[w];
            op[e] = acc / L;
        }
    }
}

int launch_attention(const AttnParams& p, int rows, cudaStream_t st) {
    if (attn_prefill_supported(p, rows)) {
        static const bool fp32 = getenv("ROTOR_B200_ATTN_FP32") != nullptr;  // comparison aid: the FP32-pipe kernel
        return fp32 ? launch_attn_prefill(p, rows, st) : launch_attn_prefill_tc(p, rows, st);
    }
    dim3 grid(p.n_heads, rows);
    switch (p.head_dim) {
        case 32: attention_kernel<1><<<grid, 128, 0, st>>>(p); break;
        case 64: attention_kernel<2><<<grid, 128, 0, st>>>(p); break;
        case 128: attention_kernel<4><<<grid, 128, 0, st>>>(p); break;
        default: return ROTOR_B200_ERR_SHAPE;
    }
    return launch_status();
}

// ---------------------------------------------------------------------------------------
// One-token attention for generation steps (body in attn_body.cuh).  Grid
// (n_kv_heads * nsplit, batch), 128 threads.  With a counter given, the CTA that finishes
// last for a sequence merges the partials of all heads and quantises the merged row for
// the output projection; without one the consumer merges the partials itself.
template <int D>
__global__ void __launch_bounds__(128) attn_decode_kernel(const __grid_constant__ AttnDecodeParams p) {
    extern __shared__ __align__(16) float sm[];
    const int G = p.n_heads / p.n_kv_heads;
    const int b = blockIdx.y;
    const int dq = p.n_heads * D;
    const int lcmax = (p.max_seq + p.nsplit - 1) / p.nsplit;
    float* scratch = sm + G * D + 2 * D + G * lcmax;  // [64]
    float* row = scratch + 64;                        // [dq]   (tail only)
    TraceRec tr;
    RB_STAMP(tr, 0);
    pdl_trigger();
    pdl_wait();
    RB_STAMP(tr, 2);
    attn_decode_body<D>(p, blockIdx.x, b, sm, threadIdx.x, blockDim.x, [] { __syncthreads(); });
    RB_STAMP(tr, 5);
    RB_TRACE_COMMIT(tr, 100);
    // ---- last CTA of this sequence: merge all heads, quantise the row for the o projection
    // (skipped when the consumer merges the partials itself: counter == null)
    if (!p.counter) return;
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(p.counter + b, 1u) == (unsigned)(gridDim.x - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (threadIdx.x == 0) p.counter[b] = 0;
    // merge weights of every (head, slice): f = exp(m_s - M) / L, all loads of a phase in flight together
    float* wf = row + dq;              // [n_heads][nsplit]
    float* wl = wf + p.n_heads * p.nsplit;
    const size_t hb = (size_t)b * p.n_heads * p.nsplit;
    for (int e = threadIdx.x; e < p.n_heads * p.nsplit; e += blockDim.x) {
        wf[e] = __ldcg(p.part_m + hb + e);
        wl[e] = __ldcg(p.part_l + hb + e);
    }
    __syncthreads();
    for (int h = threadIdx.x; h < p.n_heads; h += blockDim.x) {
        float M = -INFINITY;
        for (int s2 = 0; s2 < p.nsplit; ++s2) M = fmaxf(M, wf[h * p.nsplit + s2]);
        float L = 0.f;
        for (int s2 = 0; s2 < p.nsplit; ++s2) {
            const float ms = wf[h * p.nsplit + s2];
            const float f = ms == -INFINITY ? 0.f : __expf(ms - M);
            L += wl[h * p.nsplit + s2] * f;
            wf[h * p.nsplit + s2] = f;
        }
        const float inv = 1.0f / L;
        for (int s2 = 0; s2 < p.nsplit; ++s2) wf[h * p.nsplit + s2] *= inv;
    }
    __syncthreads();
    constexpr int MU = 4;
    for (int i0 = threadIdx.x; i0 < dq; i0 += MU * blockDim.x) {
        float o[MU];
#pragma unroll
        for (int u = 0; u < MU; ++u) o[u] = 0.f;
        for (int s2 = 0; s2 < p.nsplit; ++s2) {
            float pv[MU];
#pragma unroll
            for (int u = 0; u < MU; ++u) {
                const int idx = i0 + u * blockDim.x;
                pv[u] = idx < dq ? __ldcg(p.part_o + (hb + (size_t)(idx / D) * p.nsplit + s2) * D + idx % D) : 0.f;
            }
#pragma unroll
            for (int u = 0; u < MU; ++u) {
                const int idx = i0 + u * blockDim.x;
                if (idx < dq) o[u] += pv[u] * wf[(idx / D) * p.nsplit + s2];
            }
        }
#pragma unroll
        for (int u = 0; u < MU; ++u) {
            const int idx = i0 + u * blockDim.x;
            if (idx < dq) {
                row[idx] = o[u];
                if (p.attn_out) p.attn_out[(size_t)b * dq + idx] = o[u];
            }
        }
    }
    __syncthreads();
    if (p.xq)
        quantize_row_from_smem(row, dq, p.kpad, p.terms_out, p.xq + (size_t)b * p.terms_out * p.kpad,
                               p.sx_out + (size_t)b * p.terms_out, p.xsum_out + (size_t)b * p.terms_out, scratch);
}

int attn_decode_nsplit(int max_seq) {
    int n = max_seq / 128;
    return n < 8 ? 8 : (n > 32 ? 32 : n);
}

size_t attn_decode_part_floats(int batch, int n_heads, int head_dim, int max_seq) {
    return (size_t)batch * n_heads * attn_decode_nsplit(max_seq) * (head_dim + 2);
}

template <int D>
static int launch_attn_decode_d(const AttnDecodeParams& p, int batch, cudaStream_t st) {
    const int G = p.n_heads / p.n_kv_heads;
    const int lcmax = (p.max_seq + p.nsplit - 1) / p.nsplit;
    const size_t smem = ((size_t)G * D + 2 * D + (size_t)G * lcmax + 64 + (size_t)p.n_heads * D +
                         2 * (size_t)p.n_heads * p.nsplit) * sizeof(float);
    if (smem > 200 * 1024) return ROTOR_B200_ERR_SHAPE;
    static size_t configured = 48 * 1024;
    if (smem > configured) {
        RB_CUDA(cudaFuncSetAttribute(attn_decode_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        configured = 200 * 1024;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.n_kv_heads * p.nsplit, batch);
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_use_pdl ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, attn_decode_kernel<D>, p) != cudaSuccess) {
        ++g_launch_count;
        return ROTOR_B200_ERR_CUDA;
    }
    return launch_status();
}

int launch_attn_decode(const AttnDecodeParams& p, int batch, cudaStream_t st) {
    switch (p.head_dim) {
        case 32: return launch_attn_decode_d<32>(p, batch, st);
        case 64: return launch_attn_decode_d<64>(p, batch, st);
        case 128: return launch_attn_decode_d<128>(p, batch, st);
    }
    return ROTOR_B200_ERR_SHAPE;
}

int configure_attention() {
    RB_CUDA(cudaFuncSetAttribute(attn_decode_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    RB_CUDA(cudaFuncSetAttribute(attn_decode_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    RB_CUDA(cudaFuncSetAttribute(attn_decode_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    int rc = configure_attn_prefill();
    return rc ? rc : configure_attn_prefill_tc();
}

}  // namespace rb
