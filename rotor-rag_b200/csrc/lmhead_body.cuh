// Device body of the tied LM head (see lmhead.cu), shared with the single-launch
// generation step.
#pragma once
#include "model.cuh"

namespace rb {

constexpr int LM_ROWS = 4;       // token rows per pass over the table
constexpr int LM_VROWS = 4;      // table rows in flight per warp

__device__ __forceinline__ void bf16x8_to_float(const uint4& u, float (&f)[8]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// Body of the LM-head kernel for NROWS token rows starting at row0.  All threads of the CTA
// must call; xs: shared floats [NROWS][d].  Works for any block size that is a multiple of
// 32 (up to 32 warps); partial picks are indexed by blockIdx.x, so p.nparts >= gridDim.x.
template <int NROWS>
__device__ __forceinline__ void lmhead_body(const LmHeadParams& p, int row0, float* xs) {
    const int d = p.d;
    const int nwarps = blockDim.x >> 5;
    if (p.pro_y) {
        // fused prologue: x = final_norm(h + y) built by every CTA from the last block's outputs
        // (float4 loads issued together; the sum of squares rides along)
        __shared__ float red[33];
        const int n4 = d >> 2;
        for (int r = 0; r < NROWS; ++r) {
            const size_t ro = (size_t)(row0 + r) * d;
            float ss = 0.f;
            for (int g0 = threadIdx.x; g0 < n4; g0 += 4 * blockDim.x) {
                float4 a[4], hv[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int g = g0 + u * blockDim.x;
                    if (g < n4) {
                        a[u] = __ldcg(reinterpret_cast<const float4*>(p.pro_y + ro) + g);
                        hv[u] = __ldcg(reinterpret_cast<const float4*>(p.pro_h + ro) + g);
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int g = g0 + u * blockDim.x;
                    if (g < n4) {
                        const float4 v = make_float4(a[u].x + hv[u].x, a[u].y + hv[u].y, a[u].z + hv[u].z, a[u].w + hv[u].w);
                        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                        *reinterpret_cast<float4*>(xs + r * d + g * 4) = v;
                    }
                }
            }
            ss = block_sum(ss, red);
            const float inv = 1.0f / sqrtf(ss / (float)d + p.pro_eps);
            for (int g = threadIdx.x; g < n4; g += blockDim.x) {  // each thread revisits its own groups
                float4 v = *reinterpret_cast<float4*>(xs + r * d + g * 4);
                const float4 w = __ldg(reinterpret_cast<const float4*>(p.pro_norm) + g);
                v.x *= inv * w.x; v.y *= inv * w.y; v.z *= inv * w.z; v.w *= inv * w.w;
                *reinterpret_cast<float4*>(xs + r * d + g * 4) = v;
            }
        }
        __syncthreads();
    } else {
        for (int i = threadIdx.x; i < NROWS * d; i += blockDim.x) xs[i] = __ldcg(&p.x[(size_t)row0 * d + i]);
        __syncthreads();
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gw = blockIdx.x * nwarps + warp, nw = gridDim.x * nwarps;
    const int nchunk = d / 256;  // d is a multiple of 256 (checked on the host)

    float best[NROWS];
    int besti[NROWS];
#pragma unroll
    for (int r = 0; r < NROWS; ++r) {
        best[r] = -INFINITY;
        besti[r] = 0x7fffffff;
    }
    for (int v0 = gw * LM_VROWS; v0 < p.vocab; v0 += nw * LM_VROWS) {
        float acc[LM_VROWS][NROWS];
#pragma unroll
        for (int j = 0; j < LM_VROWS; ++j)
#pragma unroll
            for (int r = 0; r < NROWS; ++r) acc[j][r] = 0.f;
        for (int c = 0; c < nchunk; ++c) {
            const int k = c * 256 + lane * 8;
            uint4 wv[LM_VROWS];
#pragma unroll
            for (int j = 0; j < LM_VROWS; ++j) {
                const int v = min(v0 + j, p.vocab - 1);
                wv[j] = ld_stream_v4(reinterpret_cast<const uint4*>(p.embed + (size_t)v * d + k));
            }
            float xf[NROWS][8];
#pragma unroll
            for (int r = 0; r < NROWS; ++r) {
                const float4 a = *reinterpret_cast<const float4*>(xs + r * d + k);
                const float4 b = *reinterpret_cast<const float4*>(xs + r * d + k + 4);
                xf[r][0] = a.x; xf[r][1] = a.y; xf[r][2] = a.z; xf[r][3] = a.w;
                xf[r][4] = b.x; xf[r][5] = b.y; xf[r][6] = b.z; xf[r][7] = b.w;
            }
#pragma unroll
            for (int j = 0; j < LM_VROWS; ++j) {
                float wf[8];
                bf16x8_to_float(wv[j], wf);
#pragma unroll
                for (int r = 0; r < NROWS; ++r)
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[j][r] += wf[e] * xf[r][e];
            }
        }
#pragma unroll
        for (int j = 0; j < LM_VROWS; ++j)
#pragma unroll
            for (int r = 0; r < NROWS; ++r) {
                const float s = warp_sum(acc[j][r]);
                const int v = v0 + j;
                if (v < p.vocab) {
                    if (p.logits && lane == 0) p.logits[(size_t)(row0 + r) * p.vocab + v] = s;
                    if (s > best[r] || (s == best[r] && v < besti[r])) {
                        best[r] = s;
                        besti[r] = v;
                    }
                }
            }
    }
    // CTA-level pick, lowest index on ties
    __shared__ float sb[32][NROWS];
    __shared__ int si[32][NROWS];
    if (lane == 0)
#pragma unroll
        for (int r = 0; r < NROWS; ++r) {
            sb[warp][r] = best[r];
            si[warp][r] = besti[r];
        }
    __syncthreads();
    if (threadIdx.x < NROWS) {
        const int r = threadIdx.x;
        float bv = sb[0][r];
        int bi = si[0][r];
        for (int w = 1; w < nwarps; ++w)
            if (sb[w][r] > bv || (sb[w][r] == bv && si[w][r] < bi)) {
                bv = sb[w][r];
                bi = si[w][r];
            }
        p.part_val[(size_t)(row0 + r) * p.nparts + blockIdx.x] = bv;
        p.part_idx[(size_t)(row0 + r) * p.nparts + blockIdx.x] = bi;
    }

    // ---- tail (single-launch case): the last CTA merges the per-CTA picks, and when the
    // launch closes a generation step it also logs the tokens and advances the position.
    if (!p.tail_counter) return;
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(p.tail_counter, 1u) == gridDim.x - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (threadIdx.x == 0) *p.tail_counter = 0;
    __shared__ float tv[32];
    __shared__ int ti[32];
    for (int r = 0; r < NROWS; ++r) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int i = threadIdx.x; i < p.nparts; i += blockDim.x) {
            const float v = __ldcg(&p.part_val[(size_t)(row0 + r) * p.nparts + i]);
            const int id = __ldcg(&p.part_idx[(size_t)(row0 + r) * p.nparts + i]);
            if (v > bv || (v == bv && id < bi)) {
                bv = v;
                bi = id;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) {
                bv = ov;
                bi = oi;
            }
        }
        __syncthreads();
        if (lane == 0) {
            tv[warp] = bv;
            ti[warp] = bi;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < nwarps; ++w)
                if (tv[w] > bv || (tv[w] == bv && ti[w] < bi)) {
                    bv = tv[w];
                    bi = ti[w];
                }
            p.argmax_out[row0 + r] = bi;
            if (p.argmax_val) p.argmax_val[row0 + r] = bv;
            if (p.adv_log) {
                const int st = *p.adv_step;
                if (st < p.adv_max_log) p.adv_log[(size_t)st * NROWS + r] = bi;
            }
        }
    }
    if (p.adv_log && threadIdx.x == 0) {
        for (int r = 0; r < NROWS; ++r) p.adv_pos[r] += 1;
        *p.adv_step += 1;
    }
}

}  // namespace rb
