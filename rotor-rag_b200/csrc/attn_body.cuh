// Device bodies of the decode-attention kernel, shared by the stand-alone kernel
// (attention.cu) and the single-launch generation step (megastep.cu).
#pragma once
#include "model.cuh"

namespace rb {

template <int TERMS, int PLANES>
__device__ __forceinline__ float deq_acc_t(const AccView& a, const float* __restrict__ sx, int m, int o, float wscale) {
    int s[TERMS];
    float f[TERMS];
#pragma unroll
    for (int t = 0; t < TERMS; ++t) {
        const size_t col = (size_t)m * TERMS + t;
        s[t] = 0;
#pragma unroll
        for (int p = 0; p < PLANES; ++p) s[t] += __ldcg(&a.acc[(size_t)p * a.plane_stride + col * a.out + o]);
        f[t] = __ldcg(&sx[col]);
    }
    float v = 0.f;
#pragma unroll
    for (int t = 0; t < TERMS; ++t) v += (float)s[t] * f[t];
    return v * wscale;
}

// Dequantised element o of token row m.  The common (terms, planes) pairs are straight-line
// code so that independent calls overlap their loads.
__device__ __forceinline__ float deq_acc(const AccView& a, const float* __restrict__ sx, int m, int terms, int o,
                                         float wscale) {
    if (a.planes == 1) {
        if (terms == 1) return deq_acc_t<1, 1>(a, sx, m, o, wscale);
        if (terms == 3) return deq_acc_t<3, 1>(a, sx, m, o, wscale);
    } else if (a.planes == 2) {
        if (terms == 1) return deq_acc_t<1, 2>(a, sx, m, o, wscale);
        if (terms == 3) return deq_acc_t<3, 2>(a, sx, m, o, wscale);
    }
    float v = 0.f;
    for (int t = 0; t < terms; ++t) {
        const size_t col = (size_t)m * terms + t;
        int s = 0;
        for (int p = 0; p < a.planes; ++p) s += __ldcg(&a.acc[(size_t)p * a.plane_stride + col * a.out + o]);
        v += (float)s * __ldcg(&sx[col]);
    }
    return v * wscale;
}

// ---------------------------------------------------------------------------------------
// One-token attention for generation steps.  Grid (n_kv_heads * nsplit, batch): a CTA owns
// one KV head and one slice of the cached positions, serves the G query heads that share
// that KV head, and leaves (max, sum, weighted V) partials.  The CTA that finishes last for
// a sequence merges the partials of all heads and quantises the merged row for the output
// projection, so the step needs no separate combine or quantise launch.
//
// The body runs on a group of `nthr` threads (a multiple of 32) with thread index `tid`;
// `sync` is the barrier of exactly that group (__syncthreads for a whole CTA, a named
// barrier for a part of one).  `item` selects (KV head, slice), `b` the sequence.
template <int D, typename Sync>
__device__ __forceinline__ void attn_decode_body(const AttnDecodeParams& p, int item, int b, float* sm, int tid,
                                                 int nthr, Sync sync) {
    constexpr int half = D / 2, DL = D / 8;  // DL floats of a key per lane, 8 lanes per key
    const int G = p.n_heads / p.n_kv_heads;
    const int hk = item / p.nsplit, sp = item % p.nsplit;
    const int dq = p.n_heads * D, dkv = p.n_kv_heads * D;
    const int lcmax = (p.max_seq + p.nsplit - 1) / p.nsplit;
    float* q_s = sm;                    // [G][D], pre-scaled by 1/sqrt(D)
    float* k_new = q_s + G * D;         // [D]
    float* v_new = k_new + D;           // [D]
    float* sc = v_new + D;              // [G][lcmax]
    float* scratch = sc + G * lcmax;    // [64]
    float* row = scratch + 64;          // [dq]   (tail only)

    const int pos = __ldcg(p.past_len + b);
    const int T = min(pos + 1, p.max_seq);
    const int lc = (T + p.nsplit - 1) / p.nsplit;
    const int t0 = sp * lc, t1 = min(T, t0 + lc);
    const int m = b;  // one token per sequence
    const float scale = 1.0f / sqrtf((float)D);

    // ---- q of the G heads, and the new k / v of this KV head
    const float* qf = p.qkv_f ? p.qkv_f + (size_t)m * (dq + 2 * dkv) : nullptr;
    for (int w = tid; w < (G + 1) * half; w += nthr) {
        const bool is_q = w < G * half;
        const int hh = is_q ? w / half : 0, i = w % half;
        const int base = is_q ? (hk * G + hh) * D : dq + hk * D;
        const float ws = is_q ? p.sq : p.sk;
        float a = qf ? __ldcg(qf + base + i) : deq_acc(p.acc, p.sx, m, p.terms, base + i, ws);
        float c = qf ? __ldcg(qf + base + i + half) : deq_acc(p.acc, p.sx, m, p.terms, base + i + half, ws);
        if (p.rope) {
            const float2 cs = p.rope[(size_t)pos * half + i];
            const float ra = a * cs.x - c * cs.y, rc = c * cs.x + a * cs.y;
            a = ra;
            c = rc;
        }
        if (is_q) {
            q_s[hh * D + i] = a * scale;
            q_s[hh * D + i + half] = c * scale;
        } else {
            k_new[i] = a;
            k_new[i + half] = c;
        }
    }
    for (int i = tid; i < D; i += nthr)
        v_new[i] = qf ? __ldcg(qf + dq + dkv + hk * D + i) : deq_acc(p.acc, p.sx, m, p.terms, dq + dkv + hk * D + i, p.sv);
    sync();
    float* kc = p.k_cache + ((size_t)b * p.n_kv_heads + hk) * p.max_seq * D;
    float* vc = p.v_cache + ((size_t)b * p.n_kv_heads + hk) * p.max_seq * D;
    if (pos < p.max_seq && pos >= t0 && pos < t1)
        for (int i = tid; i < D; i += nthr) {
            kc[(size_t)pos * D + i] = k_new[i];
            vc[(size_t)pos * D + i] = v_new[i];
        }

    // ---- scores of this slice: 8 lanes per key, nthr/8 keys per pass
    const int l8 = tid & 7;
    // The loop bound is the same for every thread (the shuffles below need whole warps);
    // key groups past the end of the slice compute on zeros and store nothing.
    for (int tb = t0; tb < t1; tb += nthr / 8) {
        const int t = tb + (tid >> 3);
        const bool valid = t < t1;
        float kv[DL];
#pragma unroll
        for (int e = 0; e < DL; ++e) kv[e] = 0.f;
        if (valid) {
            const float* kp = (t == pos) ? k_new + l8 * DL : kc + (size_t)t * D + l8 * DL;
#pragma unroll
            for (int e = 0; e < DL; e += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(kp + e);
                kv[e] = k4.x; kv[e + 1] = k4.y; kv[e + 2] = k4.z; kv[e + 3] = k4.w;
            }
        }
        for (int g = 0; g < G; ++g) {
            const float* qp = q_s + g * D + l8 * DL;
            float s = 0.f;
#pragma unroll
            for (int e = 0; e < DL; ++e) s += qp[e] * kv[e];
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            s += __shfl_xor_sync(0xffffffffu, s, 4);
            if (valid && l8 == 0) sc[g * lcmax + (t - t0)] = s;
        }
    }
    sync();

    // ---- softmax statistics of the slice, one warp per head
    const int warp = tid >> 5, lane = tid & 31, n = t1 - t0;
    for (int g = warp; g < G; g += nthr / 32) {
        float mx = -INFINITY;
        for (int i = lane; i < n; i += 32) mx = fmaxf(mx, sc[g * lcmax + i]);
        mx = warp_max(mx);
        float l = 0.f;
        for (int i = lane; i < n; i += 32) {
            const float e = __expf(sc[g * lcmax + i] - mx);
            sc[g * lcmax + i] = e;
            l += e;
        }
        l = warp_sum(l);
        if (lane == 0) {
            const size_t pi = ((size_t)b * p.n_heads + hk * G + g) * p.nsplit + sp;
            p.part_m[pi] = n > 0 ? mx : -INFINITY;
            p.part_l[pi] = l;
        }
    }
    sync();

    // ---- weighted V of the slice: thread d owns one output dimension; V rows are fetched
    // eight at a time so that the loads overlap instead of queueing behind each other
    for (int d = tid; d < D; d += nthr) {
        for (int g0 = 0; g0 < G; g0 += 4) {
            float o[4] = {0.f, 0.f, 0.f, 0.f};
            for (int tb = t0; tb < t1; tb += 8) {
                float vv[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int t = tb + u;
                    vv[u] = t < t1 ? ((t == pos) ? v_new[d] : vc[(size_t)t * D + d]) : 0.f;
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int t = tb + u;
                    if (t < t1) {
#pragma unroll
                        for (int g = 0; g < 4; ++g)
                            if (g0 + g < G) o[g] += sc[(g0 + g) * lcmax + (t - t0)] * vv[u];
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < 4; ++g)
                if (g0 + g < G)
                    p.part_o[(((size_t)b * p.n_heads + hk * G + g0 + g) * p.nsplit + sp) * D + d] = o[g];
        }
    }

}

}  // namespace rb
