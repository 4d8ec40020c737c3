// Per-row absmax int8 quantiser shared by the stand-alone quantise kernel and the
// fused vector stages.  Arithmetic is float32 with one IEEE rounding per operation
// (no fused multiply-add, true division) so the result is bit-identical to NumPy's
// max|x|/127, rint(x/s), clip, residual = x - q*s evaluated in float32.
#pragma once
#include "common.cuh"

namespace rb {

// q = clip(rint(v / s), -128, 127) with the exact IEEE quotient, at the cost of one multiply:
// v * (1/s) differs from v / s by a few ulp, so rint() of the two can only disagree when the
// product lies within ~1e-4 of k + 0.5; only then is the true division evaluated.
__device__ __forceinline__ float exact_quant(float v, float s, float rs) {
    const float r = v * rs;
    float q = rintf(r);
    if (fabsf(r - q) > 0.499f) q = rintf(__fdiv_rn(v, s));
    return fminf(fmaxf(q, -128.f), 127.f);
}

// row      : shared memory, k floats; overwritten by the residual when terms > 1
// xq       : global int8, term t written at xq + t*kpad, zero padded to kpad
// sx, xsum : global, one entry per term
// scratch  : shared memory, 33 floats
// All threads of the block must call; blockDim.x is a multiple of 32.
// tstride   : bytes between consecutive terms in xq (>= kpad; xq may be shared memory)
// given_absmax : optional max|row| of term 0 supplied by the caller (sharded rows)
__device__ __forceinline__ void quantize_row_from_smem(float* row, int k, int kpad, int terms,
                                                       int8_t* __restrict__ xq, float* __restrict__ sx,
                                                       int32_t* __restrict__ xsum, float* scratch,
                                                       size_t tstride = 0, const float* given_absmax = nullptr) {
    if (tstride == 0) tstride = (size_t)kpad;
    for (int t = 0; t < terms; ++t) {
        float mx = 0.f;
        if (t == 0 && given_absmax) {
            // the row is a slice of a longer one: the absolute maximum of the whole row comes from outside
            mx = *given_absmax;
            __syncthreads();
        } else {
            for (int i = threadIdx.x; i < k; i += blockDim.x) mx = fmaxf(mx, fabsf(row[i]));
            mx = block_max(mx, scratch);
        }
        const float s = mx > 0.f ? __fdiv_rn(mx, 127.f) : 1.f;
        const float rs = __fdiv_rn(1.0f, s);
        int lsum = 0;
        for (int i4 = threadIdx.x * 4; i4 < kpad; i4 += blockDim.x * 4) {
            char4 q4;
            int8_t* qp = reinterpret_cast<int8_t*>(&q4);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = i4 + e;
                int q = 0;
                if (i < k) {
                    const float v = row[i];
                    const float r = exact_quant(v, s, rs);
                    q = (int)r;
                    if (t + 1 < terms) row[i] = __fsub_rn(v, __fmul_rn(r, s));
                }
                qp[e] = (int8_t)q;
                lsum += q;
            }
            *reinterpret_cast<char4*>(xq + (size_t)t * tstride + i4) = q4;
        }
        lsum = block_sum_i(lsum, reinterpret_cast<int*>(scratch));
        if (threadIdx.x == 0) {
            sx[t] = s;
            xsum[t] = lsum;
        }
    }
}

}  // namespace rb
