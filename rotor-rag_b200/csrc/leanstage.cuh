// Register-resident vector stage for generation steps.
//
// A generation step's vector stages (residual add, sub-norm, pre-norm, attention merge,
// absmax quantiser) run in the prologue of the kernel that consumes them, once per CTA.
// Each thread owns up to V groups of four consecutive elements (V a template parameter), fetched with 128-bit
// loads that are all issued together, and keeps them in registers through the whole
// stage: sums of squares and the absolute maximum are block reductions over register
// values, and the quantised bytes go straight to the staged activation buffer as one
// 32-bit word per group.  The arithmetic is that of vec_stage_row (vecstage.cuh);
// producers hand over finished float32 outputs, so no integer accumulator is re-read.
#pragma once
#include "model.cuh"
#include "quant.cuh"
#include "xch.cuh"

namespace rb {

enum LeanMode { LM_EMBED = 0, LM_ADD = 1, LM_SUBNORM_ADD = 2, LM_PLAIN = 3, LM_ATTN = 4 };

// What a prologue reads.  Rows are indexed [m][n].
struct LeanStage {
    int mode;
    int n;                       // row width (multiple of 4)
    const long long* ids;        // LM_EMBED
    const __nv_bfloat16* embed;  // LM_EMBED: table [vocab][n]
    const float* y;              // producer output [rows][n]: LM_ADD / LM_SUBNORM_ADD / LM_PLAIN
    const float* h;              // residual stream in  [rows][n]
    float* h_out;                // residual stream out [rows][n] (written by the writer CTA)
    const float* norm0;          // LM_SUBNORM_ADD: sub-norm weight applied to y before the add
    const float* norm1;          // optional pre-norm weight applied last
    float eps;
    // LM_ATTN: merge of the decode-attention partials
    const float* part_o;
    const float* part_m;
    const float* part_l;
    int nsplit, n_heads, head_dim;
    // quantiser
    int terms;
    int kpad;
    // tensor parallel: the row is this rank's slice of a longer one.  Exchange index + 1 (0 = none)
    // of the sum of squares under norm1 and of the absolute maximum under the quantiser; norm_n is
    // the width of the whole row.
    int xi_sum, xi_max, norm_n;
};

__device__ __forceinline__ float4 ldcg4(const float* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float4 ldg4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float sq4(const float4& v) { return v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; }
__device__ __forceinline__ float amax4(const float4& v) {
    return fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
}

// Builds token row m in registers: v[j] holds elements 4*(threadIdx.x + j*blockDim.x) .. +3
// (groups past n/4 stay zero).  Applies norm1 when given.  `scratch`: 64 shared floats, `rk` the
// running count of one-barrier reductions over it (block_sum_alt);
// `aux`: shared floats for the attention merge weights (2 * n_heads * nsplit, LM_ATTN only).
// All threads of the block must call.
// PLAIN_ONLY: the caller guarantees p.mode == LM_PLAIN; the other modes' code (and registers) are left out.
template <int LEAN_V, bool PLAIN_ONLY = false>
__device__ __forceinline__ void lean_row(const LeanStage& p, int m, float4 (&v)[LEAN_V], float* scratch, float* aux,
                                         bool writer, int& rk, const XchScalarDev* x = nullptr) {
    const int n4 = p.n >> 2, bd = blockDim.x;
    const size_t ro = (size_t)m * p.n;
#pragma unroll
    for (int j = 0; j < LEAN_V; ++j) v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (!PLAIN_ONLY && p.mode == LM_ATTN) {
        const int D = p.head_dim, ns = p.nsplit, nh = p.n_heads;
        float* wf = aux;
        float* wl = aux + nh * ns;
        const size_t hb = (size_t)m * nh * ns;
        for (int e = threadIdx.x; e < nh * ns; e += bd) {
            wf[e] = __ldcg(p.part_m + hb + e);
            wl[e] = __ldcg(p.part_l + hb + e);
        }
        __syncthreads();
        for (int h = threadIdx.x; h < nh; h += bd) {
            float M = -INFINITY;
            for (int s = 0; s < ns; ++s) M = fmaxf(M, wf[h * ns + s]);
            float L = 0.f;
            for (int s = 0; s < ns; ++s) {
                const float ms = wf[h * ns + s];
                const float f = ms == -INFINITY ? 0.f : __expf(ms - M);
                L += wl[h * ns + s] * f;
                wf[h * ns + s] = f;
            }
            const float inv = 1.0f / L;
            for (int s = 0; s < ns; ++s) wf[h * ns + s] *= inv;
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < LEAN_V; ++j) {
            const int g = threadIdx.x + j * bd;
            if (g < n4) {
                const int i = g * 4, h = i / D, dd = i - h * D;  // D is a multiple of 4: one head per group
                const float* po = p.part_o + (hb + (size_t)h * ns) * D + dd;
                float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
                for (int s0 = 0; s0 < ns; s0 += 8) {  // nsplit is a multiple of 8
                    float4 pv[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) pv[u] = ldcg4(po + (size_t)(s0 + u) * D);
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const float f = wf[h * ns + s0 + u];
                        o.x += pv[u].x * f;
                        o.y += pv[u].y * f;
                        o.z += pv[u].z * f;
                        o.w += pv[u].w * f;
                    }
                }
                v[j] = o;
            }
        }
        return;  // no norm follows the merge
    }

    // ---- all loads of the stage in flight together
    float4 a[LEAN_V], hv[LEAN_V], w0[LEAN_V], w1[LEAN_V];
#pragma unroll
    for (int j = 0; j < LEAN_V; ++j) {
        const int g = threadIdx.x + j * bd;
        a[j] = hv[j] = w0[j] = w1[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (g < n4) {
            const int i = g * 4;
            if (!PLAIN_ONLY && p.mode == LM_EMBED) {
                const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p.embed + (size_t)__ldcg(p.ids + m) * p.n + i));
                a[j] = make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                                   __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
            } else {
                a[j] = ldcg4(p.y + ro + i);
                if (!PLAIN_ONLY && (p.mode == LM_ADD || p.mode == LM_SUBNORM_ADD)) hv[j] = ldcg4(p.h + ro + i);
                if (!PLAIN_ONLY && p.mode == LM_SUBNORM_ADD) w0[j] = ldg4(p.norm0 + i);
            }
            if (p.norm1) w1[j] = ldg4(p.norm1 + i);
        }
    }
    if (!PLAIN_ONLY && p.mode == LM_SUBNORM_ADD) {  // a <- subnorm(a)
        float s0 = 0.f;
#pragma unroll
        for (int j = 0; j < LEAN_V; ++j) s0 += sq4(a[j]);
        s0 = block_sum_alt(s0, scratch, rk);
        const float inv0 = 1.0f / sqrtf(s0 / (float)p.n + p.eps);
#pragma unroll
        for (int j = 0; j < LEAN_V; ++j) {
            a[j].x *= inv0 * w0[j].x;
            a[j].y *= inv0 * w0[j].y;
            a[j].z *= inv0 * w0[j].z;
            a[j].w *= inv0 * w0[j].w;
        }
    }
#pragma unroll
    for (int j = 0; j < LEAN_V; ++j) {
        v[j] = PLAIN_ONLY ? a[j] : make_float4(a[j].x + hv[j].x, a[j].y + hv[j].y, a[j].z + hv[j].z, a[j].w + hv[j].w);
        const int g = threadIdx.x + j * bd;
        if (!PLAIN_ONLY && writer && p.h_out && g < n4) *reinterpret_cast<float4*>(p.h_out + ro + g * 4) = v[j];
    }
    if (p.norm1) {
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < LEAN_V; ++j) ss += sq4(v[j]);
        ss = block_sum_alt(ss, scratch, rk);
        if (x && p.xi_sum) ss = xch_scalar(*x, p.xi_sum - 1, m, ss, false, writer, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)(p.norm_n ? p.norm_n : p.n) + p.eps);
#pragma unroll
        for (int j = 0; j < LEAN_V; ++j) {
            v[j].x *= inv * w1[j].x;
            v[j].y *= inv * w1[j].y;
            v[j].z *= inv * w1[j].z;
            v[j].w *= inv * w1[j].w;
        }
    }
}

// Before the programmatic-launch wait: pulls the norm weights the stage will read into L2 (they
// are constants, but a step streams ten times the L2 capacity between two uses of them).
__device__ __forceinline__ void lean_prefetch(const LeanStage& p) {
    if (threadIdx.x & 7) return;  // one request per 128-byte line
    for (int i = threadIdx.x * 4; i < p.n; i += blockDim.x * 4) {
        if (p.norm1) prefetch_l2(p.norm1 + i);
        if (p.mode == LM_SUBNORM_ADD) prefetch_l2(p.norm0 + i);
    }
}

// Four values -> four int8 in one word: q = clip(rint(v / s), -128, 127) with the exact IEEE quotient
// (v * (1/s) is within 2e-5 of v / s for |v / s| <= 127, so the multiply decides unless it lands
// within 1e-4 of a tie), packed with
// the saturating pack instruction.  `lsum` gains the four integers (one dp4a).  With RESIDUAL the
// values are replaced by v - q * s (float32, one rounding per operation) for the next term.
template <bool RESIDUAL>
__device__ __forceinline__ int quant4_pack(float4& v, float s, float rs, int& lsum) {
    const float r0 = v.x * rs, r1 = v.y * rs, r2 = v.z * rs, r3 = v.w * rs;
    float q0 = rintf(r0), q1 = rintf(r1), q2 = rintf(r2), q3 = rintf(r3);
    const float dm = fmaxf(fmaxf(fabsf(r0 - q0), fabsf(r1 - q1)), fmaxf(fabsf(r2 - q2), fabsf(r3 - q3)));
    if (dm > 0.4999f) {  // rare: some product is close to a tie, take the true quotients
        q0 = rintf(__fdiv_rn(v.x, s));
        q1 = rintf(__fdiv_rn(v.y, s));
        q2 = rintf(__fdiv_rn(v.z, s));
        q3 = rintf(__fdiv_rn(v.w, s));
    }
    if (RESIDUAL) {
        q0 = fminf(fmaxf(q0, -128.f), 127.f);
        q1 = fminf(fmaxf(q1, -128.f), 127.f);
        q2 = fminf(fmaxf(q2, -128.f), 127.f);
        q3 = fminf(fmaxf(q3, -128.f), 127.f);
        v.x = __fsub_rn(v.x, __fmul_rn(q0, s));
        v.y = __fsub_rn(v.y, __fmul_rn(q1, s));
        v.z = __fsub_rn(v.z, __fmul_rn(q2, s));
        v.w = __fsub_rn(v.w, __fmul_rn(q3, s));
    }
    const int i0 = __float2int_rn(q0), i1 = __float2int_rn(q1), i2 = __float2int_rn(q2), i3 = __float2int_rn(q3);
    int hi, packed;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(i3), "r"(i2), "r"(0));       // bytes: i2, i3
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(packed) : "r"(i1), "r"(i0), "r"(hi));  // i0, i1, i2, i3
    lsum = __dp4a(packed, 0x01010101, lsum);
    return packed;
}

// Absmax int8 quantiser over the register row: term t of the row goes to xq + t*tstride
// (shared memory, zero padded to kpad), its scale and sum to sx[t] / xsum[t] (shared).
// Same results as quantize_row_from_smem.  Requires kpad <= 4 * LEAN_V * blockDim.x; sx / xsum are
// complete after the next CTA barrier.  ONE_TERM: p.terms is 1 (the loop and the residual drop out).
// given_absmax: optional max|row| of term 0 supplied by the caller (sharded rows).
template <int LEAN_V, bool ONE_TERM = false>
__device__ __forceinline__ void lean_quantize(const LeanStage& p, float4 (&v)[LEAN_V], float* scratch, int8_t* xq,
                                              size_t tstride, float* sx, int* xsum, int& rk, int m = 0,
                                              bool writer = false, const XchScalarDev* x = nullptr,
                                              const float* given_absmax = nullptr) {
    const int n4 = p.n >> 2, k4 = p.kpad >> 2, bd = blockDim.x;
    const int terms = ONE_TERM ? 1 : p.terms;
    for (int t = 0; t < terms; ++t) {
        float mx = 0.f;
#pragma unroll
        for (int j = 0; j < LEAN_V; ++j) mx = fmaxf(mx, amax4(v[j]));
        if (threadIdx.x == 0) xsum[t] = 0;  // ordered before the atomics below by the reduction's barrier
        mx = block_max_alt(mx, scratch, rk);
        if (x && p.xi_max && t == 0) mx = xch_scalar(*x, p.xi_max - 1, m, mx, true, writer, scratch);
        if (given_absmax && t == 0) mx = *given_absmax;  // the row is a slice: the whole row's maximum comes from outside
        const float s = mx > 0.f ? __fdiv_rn(mx, 127.f) : 1.f;
        const float rs = __fdiv_rn(1.0f, s);
        int lsum = 0;
#pragma unroll
        for (int j = 0; j < LEAN_V; ++j) {
            const int g = threadIdx.x + j * bd;
            if (g < k4) {
                int packed = 0;
                if (g < n4) packed = (!ONE_TERM && t + 1 < terms) ? quant4_pack<true>(v[j], s, rs, lsum)
                                                                  : quant4_pack<false>(v[j], s, rs, lsum);
                *reinterpret_cast<int*>(xq + (size_t)t * tstride + (size_t)g * 4) = packed;
            }
        }
        // the sum of the quantised values is only read after the caller's barrier: warps add
        // their shares with a shared-memory atomic instead of a second block-wide reduction
        lsum = warp_sum_i(lsum);
        if ((threadIdx.x & 31) == 0 && lsum) atomicAdd(&xsum[t], lsum);
        if (threadIdx.x == 0) sx[t] = s;
    }
}

}  // namespace rb
