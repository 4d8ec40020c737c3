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
#include "model.cuh"

namespace rb {

__device__ __forceinline__ float deq_acc(const AccView& a, const float* __restrict__ sx, int m, int terms, int o,
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

// One CTA per token row.  Work items are rotation pairs (i, i + D/2) of q and k heads and
// single elements of v.
__global__ void __launch_bounds__(256) qkv_finish_kernel(QkvFinishParams p) {
    const int m = blockIdx.x;
    const int b = m / p.seq, s = m % p.seq;
    const int pos = *p.past_len + s;
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
        if (p.rope_theta > 0.f) {
            const double ang = (double)pos * pow((double)p.rope_theta, -2.0 * (double)i / (double)D);
            double sn, cs;
            sincos(ang, &sn, &cs);
            const float ra = (float)((double)a * cs - (double)c * sn);
            const float rc = (float)((double)c * cs + (double)a * sn);
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

int launch_qkv_finish(const QkvFinishParams& p, int rows, cudaStream_t st) {
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
    const int past = *p.past_len;
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
    dim3 grid(p.n_heads, rows);
    switch (p.head_dim) {
        case 32: attention_kernel<1><<<grid, 128, 0, st>>>(p); break;
        case 64: attention_kernel<2><<<grid, 128, 0, st>>>(p); break;
        case 128: attention_kernel<4><<<grid, 128, 0, st>>>(p); break;
        default: return ROTOR_B200_ERR_SHAPE;
    }
    return launch_status();
}

}  // namespace rb
