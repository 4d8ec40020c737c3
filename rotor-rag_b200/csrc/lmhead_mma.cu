// Tied LM head for many rows at once (batched generation steps, logits of every prompt
// position): logits[r][v] = sum_d x[r][d] * E[v][d] with the bf16 table E read ONCE for up to 64
// rows, instead of once per four rows (lmhead.cu).
//
// Reference: BitNetModel.forward, src/rotor/bitnet_model.py:235-242 (np.dot(hidden, embed.T));
// greedy pick: GreedySampling.sample, src/rotor/generation.py:31-42 (lowest index on ties).
//
// mma.sync.m16n8k16, bf16 operands, float32 accumulation.  The table is bf16 already; the rows x
// are float32 and are split once into hi + lo bf16 terms (x_split_kernel), so each tile costs two
// MMAs (E*hi + E*lo) and keeps 16 mantissa bits of x -- inside the 1e-3-of-RMS bound with room.
// CTA: 256 threads, 128 vocabulary rows x 64 token rows; warp w owns vocabulary rows 16w..16w+15
// (the MMA's M) against all 64 tokens (eight n tiles).  d is walked 64 at a time through a
// double-buffered ring of cp.async tiles, 16-byte chunks swizzled (chunk ^= row & 7) for ldmatrix.
// Outputs: logits (optional) and one (max, argmax) partial per CTA and token row, merged by
// argmax_final_kernel like the partials of lmhead_kernel.
#include <cuda_bf16.h>

#include <cstdlib>

#include "model.cuh"

namespace rb {

constexpr int LMM_V = 128;   // vocabulary rows per CTA
constexpr int LMM_T = 64;    // token rows per CTA
constexpr int LMM_K = 64;    // d per stage
constexpr int LMM_ROWB = LMM_K * 2;                                   // bytes per staged row
constexpr int LMM_STAGE = (LMM_V + 2 * LMM_T) * LMM_ROWB;              // E tile + x hi + x lo
constexpr int LMM_SMEM = 2 * LMM_STAGE;

__device__ __forceinline__ void lmm_ldsm(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void lmm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// x float32 [rows][d] -> hi / lo bf16 planes [rows][d] (lo plane at hi + rows * d)
__global__ void __launch_bounds__(256) x_split_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                      size_t n4, size_t plane) {
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= n4) return;
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    const float f[4] = {v.x, v.y, v.z, v.w};
    __nv_bfloat16 h[4], l[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        h[e] = __float2bfloat16_rn(f[e]);
        l[e] = __float2bfloat16_rn(f[e] - __bfloat162float(h[e]));
    }
    *reinterpret_cast<uint2*>(out + 4 * i) = *reinterpret_cast<const uint2*>(h);
    *reinterpret_cast<uint2*>(out + plane + 4 * i) = *reinterpret_cast<const uint2*>(l);
}

struct LmMmaParams {
    const __nv_bfloat16* embed;  // [vocab][d]
    const __nv_bfloat16* xs;     // hi plane [rows][d], lo plane behind it
    size_t plane;
    int vocab, d, rows;
    float* logits;               // optional [rows][vocab]
    float* part_val;             // optional [rows][nparts]: best logit of this CTA's vocabulary rows
    int* part_idx;
    int nparts;
};

__global__ void __launch_bounds__(256) lmhead_mma_kernel(const __grid_constant__ LmMmaParams p) {
    extern __shared__ __align__(128) unsigned char lmm_smem[];
    __shared__ float s_bv[8][LMM_T];
    __shared__ int s_bi[8][LMM_T];
    const uint32_t base = (uint32_t)__cvta_generic_to_shared(lmm_smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int lm = lane >> 3, lr = lane & 7;
    const int v0 = blockIdx.x * LMM_V, r0 = blockIdx.y * LMM_T;
    const int nk = p.d / LMM_K;

    auto request = [&](int ks) {  // stage ks & 1 <- d columns [64 ks, 64 ks + 64) of the E rows and the x rows
        const uint32_t st = base + (uint32_t)(ks & 1) * LMM_STAGE;
        for (int idx = threadIdx.x; idx < (LMM_V + 2 * LMM_T) * 8; idx += 256) {
            const int c = idx & 7, row = idx >> 3;
            const __nv_bfloat16* src;
            bool valid;
            if (row < LMM_V) {
                valid = v0 + row < p.vocab;
                src = p.embed + (size_t)(valid ? v0 + row : 0) * p.d;
            } else {
                const int tr = (row - LMM_V) & (LMM_T - 1), lo = (row - LMM_V) >> 6;
                valid = r0 + tr < p.rows;
                src = p.xs + (size_t)lo * p.plane + (size_t)(valid ? r0 + tr : 0) * p.d;
            }
            const uint32_t dst = st + (uint32_t)row * LMM_ROWB + (uint32_t)((c ^ (row & 7)) << 4);
            const int sz = valid ? 16 : 0;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src + ks * LMM_K + 8 * c),
                         "r"(sz)
                         : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float acc[LMM_T / 8][4];
#pragma unroll
    for (int j = 0; j < LMM_T / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;

    request(0);
    for (int ks = 0; ks < nk; ++ks) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();  // stage ks has landed; every warp is done with stage ks - 1
        if (ks + 1 < nk) request(ks + 1);
        const uint32_t st = base + (uint32_t)(ks & 1) * LMM_STAGE;
        const uint32_t eb = st, xh = st + LMM_V * LMM_ROWB, xl = xh + LMM_T * LMM_ROWB;
#pragma unroll
        for (int kk = 0; kk < LMM_K / 16; ++kk) {
            uint32_t a[4];
            {
                const int row = warp * 16 + lr + 8 * (lm & 1), chunk = 2 * kk + (lm >> 1);
                lmm_ldsm(a, eb + (uint32_t)row * LMM_ROWB + (uint32_t)((chunk ^ (row & 7)) << 4));
            }
#pragma unroll
            for (int jp = 0; jp < LMM_T / 16; ++jp) {
                uint32_t bh[4], bl[4];
                const int row = 16 * jp + lr + 8 * (lm >> 1), chunk = 2 * kk + (lm & 1);
                const uint32_t off = (uint32_t)row * LMM_ROWB + (uint32_t)((chunk ^ (row & 7)) << 4);
                lmm_ldsm(bh, xh + off);
                lmm_ldsm(bl, xl + off);
                lmm_mma(acc[2 * jp], a, bh[0], bh[1]);
                lmm_mma(acc[2 * jp], a, bl[0], bl[1]);
                lmm_mma(acc[2 * jp + 1], a, bh[2], bh[3]);
                lmm_mma(acc[2 * jp + 1], a, bl[2], bl[3]);
            }
        }
    }

    // ---- outputs: accumulator (vocabulary row g or g + 8 of the warp, token 8 j + 2 t + e)
#pragma unroll
    for (int j = 0; j < LMM_T / 8; ++j)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int tok = r0 + 8 * j + 2 * t + e;
            float bv = -INFINITY;
            int bi = 0x7fffffff;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int v = v0 + warp * 16 + g + 8 * h;
                const float val = acc[j][2 * h + e];
                if (v < p.vocab) {
                    if (p.logits && tok < p.rows) p.logits[(size_t)tok * p.vocab + v] = val;
                    if (val > bv || (val == bv && v < bi)) {
                        bv = val;
                        bi = v;
                    }
                }
            }
            // best over the eight lanes that hold this token (same t, all g): lanes differ in bits 2..4
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > bv || (ov == bv && oi < bi)) {
                    bv = ov;
                    bi = oi;
                }
            }
            if (g == 0) {
                s_bv[warp][8 * j + 2 * t + e] = bv;
                s_bi[warp][8 * j + 2 * t + e] = bi;
            }
        }
    __syncthreads();
    if (p.part_val && threadIdx.x < LMM_T && r0 + (int)threadIdx.x < p.rows) {
        float bv = s_bv[0][threadIdx.x];
        int bi = s_bi[0][threadIdx.x];
        for (int w = 1; w < 8; ++w) {
            const float ov = s_bv[w][threadIdx.x];
            const int oi = s_bi[w][threadIdx.x];
            if (ov > bv || (ov == bv && oi < bi)) {
                bv = ov;
                bi = oi;
            }
        }
        p.part_val[(size_t)(r0 + threadIdx.x) * p.nparts + blockIdx.x] = bv;
        p.part_idx[(size_t)(r0 + threadIdx.x) * p.nparts + blockIdx.x] = bi;
    }
}

int lmhead_mma_parts(int vocab) { return (vocab + LMM_V - 1) / LMM_V; }

// Whether the many-row kernel takes this call (d in whole stages, 16-byte aligned rows).
bool lmhead_mma_supported(int rows, int d) {
    static const bool off = getenv("ROTOR_B200_NO_LMHEAD_MMA") != nullptr;  // comparison aid
    return !off && rows > 4 && d % LMM_K == 0;
}

int configure_lmhead_mma() {
    RB_CUDA(cudaFuncSetAttribute(lmhead_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, LMM_SMEM));
    return ROTOR_B200_OK;
}

// x: float32 [rows][d]; xsplit: scratch of 2 * rows * d bf16; part_*: [rows][lmhead_mma_parts(vocab)] or null.
int launch_lmhead_mma(const __nv_bfloat16* embed, const float* x, __nv_bfloat16* xsplit, int rows, int vocab, int d,
                      float* logits, float* part_val, int* part_idx, cudaStream_t st) {
    const size_t plane = (size_t)rows * d, n4 = plane / 4;
    x_split_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(x, xsplit, n4, plane);
    int rc = launch_status();
    if (rc) return rc;
    LmMmaParams p;
    p.embed = embed;
    p.xs = xsplit;
    p.plane = plane;
    p.vocab = vocab;
    p.d = d;
    p.rows = rows;
    p.logits = logits;
    p.part_val = part_val;
    p.part_idx = part_idx;
    p.nparts = lmhead_mma_parts(vocab);
    dim3 grid(p.nparts, (rows + LMM_T - 1) / LMM_T);
    lmhead_mma_kernel<<<grid, 256, LMM_SMEM, st>>>(p);
    return launch_status();
}

}  // namespace rb
