// Softmax attention for prompt prefill on the tensor cores, float32-faithful.
//
// Reference: MultiHeadAttention.forward (src/rotor/transformer.py:249-283): scores Q K^T / sqrt(head_dim) over the cache, optional
// causal mask, softmax, times V, K/V shared by the query heads of a group.
//
// Both products run as mma.sync.m16n8k16 (bf16 operands, float32 accumulation).  To stay
// within 1e-3 of the output RMS of the float32 reference, every operand is split into two
// bf16 terms, x = hi + lo with hi = bf16(x), lo = bf16(x - hi), and each product is computed
// as hi*hi + hi*lo + lo*hi (the dropped lo*lo term is below 2^-16 relative): three MMAs per
// tile, 16 mantissa bits of operand precision.
//
// CTA: 256 threads = 8 warps, 128 query rows of one KV head (128/G positions x G heads of
// the group); warp w owns rows 16w..16w+15.  Keys are walked 64 at a time.  Q (scaled), K and
// V tiles are converted to hi/lo bf16 on their way into shared memory (K and V through a
// float32 landing area filled by cp.async during the previous tile's MMAs); rows are 16-byte-chunk
// swizzled (chunk ^= row & 7) so that every ldmatrix phase reads eight distinct bank groups.
// S accumulators become the A operand of the second product in registers (the m16n8k16
// accumulator and A-fragment layouts coincide pairwise); the online-softmax row statistics
// are reduced over the four lanes that share a row.
#include <cuda_bf16.h>

#include "model.cuh"

namespace rb {

constexpr int TC_BM = 128;
constexpr int TC_BN = 64;

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// hi + lo split of two floats, packed as bf16x2 (first value in the low half)
__device__ __forceinline__ void split2(float x, float y, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat16 xh = __float2bfloat16_rn(x), yh = __float2bfloat16_rn(y);
    const __nv_bfloat16 xl = __float2bfloat16_rn(x - __bfloat162float(xh));
    const __nv_bfloat16 yl = __float2bfloat16_rn(y - __bfloat162float(yh));
    hi = (uint32_t)__bfloat16_as_ushort(xh) | ((uint32_t)__bfloat16_as_ushort(yh) << 16);
    lo = (uint32_t)__bfloat16_as_ushort(xl) | ((uint32_t)__bfloat16_as_ushort(yl) << 16);
}

// Shared memory: Q hi/lo plus either one K/V operand set and a float32 landing area (in-kernel
// split) or two operand sets (K/V already split in global memory): 192 KB for D = 128 both ways.
template <int D>
size_t attn_prefill_tc_smem() {
    return (size_t)(2 * TC_BM + 4 * TC_BN) * D * 2 + (size_t)2 * TC_BN * D * 4;
}

// Splits the float32 K/V cache rows [0, past + seq) of `batch` sequences into hi / lo bf16 planes
// (K hi, K lo, V hi, V lo; plane stride split_plane elements; same [batch][kv head][position][D]
// indexing as the cache), once per attention call, so that the attention CTAs that share a key tile
// do not each repeat the conversion.
__global__ void __launch_bounds__(256) kv_split_kernel(const __grid_constant__ AttnParams p, int batch) {
    const int D = p.head_dim, c4n = D / 4;
    const size_t idx = (size_t)blockIdx.x * 256 + threadIdx.x;
    const size_t per_seq = (size_t)p.n_kv_heads * p.max_seq * c4n;
    if (idx >= per_seq * batch) return;
    const int c4 = (int)(idx % c4n);
    const int t = (int)((idx / c4n) % p.max_seq);
    int t_all = p.past_len[idx / per_seq] + p.seq;
    if (t_all > p.max_seq) t_all = p.max_seq;
    if (t >= t_all) return;
    const size_t e = (idx / c4n) * D + 4 * c4;  // element offset: ((b * n_kv + hk) * max_seq + t) * D + 4 c4
    const float4 k = *reinterpret_cast<const float4*>(p.k_cache + e);
    const float4 v = *reinterpret_cast<const float4*>(p.v_cache + e);
    uint2 kh, kl, vh, vl;
    split2(k.x, k.y, kh.x, kl.x);
    split2(k.z, k.w, kh.y, kl.y);
    split2(v.x, v.y, vh.x, vl.x);
    split2(v.z, v.w, vh.y, vl.y);
    *reinterpret_cast<uint2*>(p.kv_split + e) = kh;
    *reinterpret_cast<uint2*>(p.kv_split + p.split_plane + e) = kl;
    *reinterpret_cast<uint2*>(p.kv_split + 2 * p.split_plane + e) = vh;
    *reinterpret_cast<uint2*>(p.kv_split + 3 * p.split_plane + e) = vl;
}

// Converts `rows` x D floats (row r from src + r * src_stride, zero when !valid(r)) into the
// swizzled hi / lo bf16 tiles at shared addresses hi / lo (byte addresses).
template <int D, typename RowPtr>
__device__ __forceinline__ void stage_split(uint32_t hi, uint32_t lo, int rows, RowPtr row_ptr, float scale) {
    constexpr int C4 = D / 4;  // float4 pieces per row
    for (int idx = threadIdx.x; idx < rows * C4; idx += 256) {
        const int r = idx / C4, c4 = idx - r * C4;
        const float* src = row_ptr(r);
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (src) v = *reinterpret_cast<const float4*>(src + 4 * c4);
        uint32_t h0, l0, h1, l1;
        split2(v.x * scale, v.y * scale, h0, l0);
        split2(v.z * scale, v.w * scale, h1, l1);
        // element 4*c4 lives in 16-byte chunk c4/2, at byte (c4 & 1) * 8 of the chunk
        const uint32_t off = (uint32_t)r * (D * 2) + (uint32_t)(((c4 >> 1) ^ (r & 7)) << 4) + (uint32_t)(c4 & 1) * 8u;
        asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(hi + off), "r"(h0), "r"(h1) : "memory");
        asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(lo + off), "r"(l0), "r"(l1) : "memory");
    }
}

// PRE: K/V come pre-split from p.kv_split (kv_split_kernel) and are double buffered; otherwise they
// are split here from the float32 cache through a landing area.
template <int D, bool PRE>
__global__ void __launch_bounds__(256, 1) attn_prefill_tc_kernel(const __grid_constant__ AttnParams p) {
    constexpr int ROWB = D * 2;        // bytes per tile row
    constexpr int KS = D / 16;         // k steps of Q K^T
    constexpr int NT = D / 8;          // n tiles of O
    extern __shared__ __align__(128) unsigned char tc_smem[];
    const uint32_t base = (uint32_t)__cvta_generic_to_shared(tc_smem);
    const uint32_t qh = base, ql = qh + TC_BM * ROWB;
    const uint32_t kv0 = ql + TC_BM * ROWB;            // operand set 0: K hi, K lo, V hi, V lo
    constexpr uint32_t SETB = 4 * TC_BN * ROWB;        // bytes of one operand set
    uint32_t kh = kv0, kl = kh + TC_BN * ROWB, vh = kl + TC_BN * ROWB, vl = vh + TC_BN * ROWB;
    float* kst = reinterpret_cast<float*>(tc_smem + (size_t)(2 * TC_BM + 4 * TC_BN) * ROWB);  // [TC_BN][D] float32
    float* vst = kst + TC_BN * D;                      // (PRE: this area is operand set 1 instead)
    const int G = p.n_heads / p.n_kv_heads, QT = TC_BM / G;
    const int qt = gridDim.x - 1 - blockIdx.x;  // late query tiles see the most keys: start them first
    const int hk = blockIdx.y, b = blockIdx.z;
    const int s0 = qt * QT;
    const int past = p.past_len[b];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int lm = lane >> 3, lr = lane & 7;  // ldmatrix: matrix index and row within it for this lane's address

    // ---- Q tile (scaled), rows past the sequence end are zero
    {
        const float scale = 1.0f / sqrtf((float)D);
        stage_split<D>(qh, ql, TC_BM, [&](int r) -> const float* {
            const int s = s0 + r / G, gi = r - (r / G) * G;
            return s < p.seq ? p.q + ((size_t)b * p.seq + s) * p.n_heads * D + (size_t)(hk * G + gi) * D : nullptr;
        }, scale);
    }
    int s_last = s0 + QT - 1;
    if (s_last > p.seq - 1) s_last = p.seq - 1;
    int t_all = p.causal ? past + s_last + 1 : past + p.seq;
    if (t_all > p.max_seq) t_all = p.max_seq;
    int lim[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int s = s0 + (warp * 16 + g + 8 * h) / G;
        const int l = p.causal ? past + s + 1 : past + p.seq;
        lim[h] = l < t_all ? l : t_all;
    }
    const float* kbase = p.k_cache + ((size_t)b * p.n_kv_heads + hk) * p.max_seq * D;
    const float* vbase = p.v_cache + ((size_t)b * p.n_kv_heads + hk) * p.max_seq * D;

    float oacc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) oacc[n][e] = 0.f;
    float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};

    const int ntiles = (t_all + TC_BN - 1) / TC_BN;
    // The float32 rows of key tile kt travel to the landing area with cp.async (zero fill past the
    // last key) while tile kt - 1 is being multiplied; the split into hi / lo bf16 then runs from
    // shared memory.
    auto request = [&](int kt) {
        const int t0 = kt * TC_BN;
        if constexpr (PRE) {
            // four planes x 64 rows x (D / 8) 16-byte chunks, swizzled on the way in
            constexpr int CH = D / 8;
            const uint32_t set = kv0 + (uint32_t)(kt & 1) * SETB;
            const size_t head = ((size_t)b * p.n_kv_heads + hk) * p.max_seq;
            for (int idx = threadIdx.x; idx < 4 * TC_BN * CH; idx += 256) {
                const int c = idx % CH, r = (idx / CH) % TC_BN, pl = idx / (CH * TC_BN);
                const bool valid = t0 + r < t_all;
                const __nv_bfloat16* src = p.kv_split + (size_t)pl * p.split_plane + (head + (valid ? t0 + r : 0)) * D + 8 * c;
                const uint32_t dst = set + (uint32_t)pl * (TC_BN * ROWB) + (uint32_t)r * ROWB + (uint32_t)((c ^ (r & 7)) << 4);
                const int sz = valid ? 16 : 0;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
            }
        } else {
            for (int idx = threadIdx.x; idx < TC_BN * (D / 4); idx += 256) {
                const int r = idx / (D / 4), c4 = idx - r * (D / 4);
                const bool valid = t0 + r < t_all;
                const size_t off = (size_t)(valid ? t0 + r : 0) * D + 4 * c4;
                const unsigned dk = (unsigned)__cvta_generic_to_shared(kst + r * D + 4 * c4);
                const unsigned dv = (unsigned)__cvta_generic_to_shared(vst + r * D + 4 * c4);
                const int sz = valid ? 16 : 0;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dk), "l"(kbase + off), "r"(sz) : "memory");
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dv), "l"(vbase + off), "r"(sz) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    request(0);
    for (int kt = 0; kt < ntiles; ++kt) {
        const int t0 = kt * TC_BN;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();  // tile kt has landed; every warp is done with tile kt - 1
        if constexpr (PRE) {
            kh = kv0 + (uint32_t)(kt & 1) * SETB;
            kl = kh + TC_BN * ROWB;
            vh = kl + TC_BN * ROWB;
            vl = vh + TC_BN * ROWB;
            if (kt + 1 < ntiles) request(kt + 1);  // into the other operand set, behind this tile's MMAs
        } else {
            stage_split<D>(kh, kl, TC_BN, [&](int r) -> const float* { return kst + r * D; }, 1.0f);
            stage_split<D>(vh, vl, TC_BN, [&](int r) -> const float* { return vst + r * D; }, 1.0f);
            __syncthreads();  // operands ready, landing area free
            if (kt + 1 < ntiles) request(kt + 1);
        }

        // ---- S = Q K^T: 16 rows x 64 keys per warp
        float sacc[TC_BN / 8][4];
#pragma unroll
        for (int j = 0; j < TC_BN / 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) sacc[j][e] = 0.f;
#pragma unroll
        for (int kk = 0; kk < KS; ++kk) {
            uint32_t ah[4], al[4];
            {
                const int row = warp * 16 + lr + 8 * (lm & 1), chunk = 2 * kk + (lm >> 1);
                const uint32_t off = (uint32_t)row * ROWB + (uint32_t)((chunk ^ (row & 7)) << 4);
                ldsm_x4(ah, qh + off);
                ldsm_x4(al, ql + off);
            }
#pragma unroll
            for (int jp = 0; jp < TC_BN / 16; ++jp) {
                uint32_t bh[4], bl[4];
                const int key = 16 * jp + lr + 8 * (lm >> 1), chunk = 2 * kk + (lm & 1);
                const uint32_t off = (uint32_t)key * ROWB + (uint32_t)((chunk ^ (key & 7)) << 4);
                ldsm_x4(bh, kh + off);
                ldsm_x4(bl, kl + off);
                mma_bf16(sacc[2 * jp], ah, bh[0], bh[1]);
                mma_bf16(sacc[2 * jp], ah, bl[0], bl[1]);
                mma_bf16(sacc[2 * jp], al, bh[0], bh[1]);
                mma_bf16(sacc[2 * jp + 1], ah, bh[2], bh[3]);
                mma_bf16(sacc[2 * jp + 1], ah, bl[2], bl[3]);
                mma_bf16(sacc[2 * jp + 1], al, bh[2], bh[3]);
            }
        }

        // ---- online softmax on the accumulator layout: rows g and g + 8, keys 8 j + 2 t + {0, 1}
        uint32_t ph[TC_BN / 16][4], pl[TC_BN / 16][4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < TC_BN / 8; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    if (t0 + 8 * j + 2 * t + e >= lim[h]) sacc[j][2 * h + e] = -INFINITY;
                    mx = fmaxf(mx, sacc[j][2 * h + e]);
                }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float mn = fmaxf(mrow[h], mx);  // finite from the first tile on: key 0 is visible to every row
            const float corr = __expf(mrow[h] - mn);
            float ps = 0.f;
#pragma unroll
            for (int j = 0; j < TC_BN / 8; ++j) {
                const float e0 = __expf(sacc[j][2 * h] - mn), e1 = __expf(sacc[j][2 * h + 1] - mn);
                ps += e0 + e1;
                // A fragment of k step j/2: register h (+2 for the odd tile of the pair)
                split2(e0, e1, ph[j >> 1][h + 2 * (j & 1)], pl[j >> 1][h + 2 * (j & 1)]);
            }
            ps += __shfl_xor_sync(0xffffffffu, ps, 1);
            ps += __shfl_xor_sync(0xffffffffu, ps, 2);
            lrow[h] = lrow[h] * corr + ps;
            mrow[h] = mn;
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                oacc[n][2 * h] *= corr;
                oacc[n][2 * h + 1] *= corr;
            }
        }

        // ---- O += P V
#pragma unroll
        for (int kk = 0; kk < TC_BN / 16; ++kk) {
#pragma unroll
            for (int np = 0; np < NT / 2; ++np) {
                uint32_t bh[4], bl[4];
                const int key = 16 * kk + lr + 8 * (lm & 1), chunk = 2 * np + (lm >> 1);
                const uint32_t off = (uint32_t)key * ROWB + (uint32_t)((chunk ^ (key & 7)) << 4);
                ldsm_x4_t(bh, vh + off);
                ldsm_x4_t(bl, vl + off);
                mma_bf16(oacc[2 * np], ph[kk], bh[0], bh[1]);
                mma_bf16(oacc[2 * np], ph[kk], bl[0], bl[1]);
                mma_bf16(oacc[2 * np], pl[kk], bh[0], bh[1]);
                mma_bf16(oacc[2 * np + 1], ph[kk], bh[2], bh[3]);
                mma_bf16(oacc[2 * np + 1], ph[kk], bl[2], bl[3]);
                mma_bf16(oacc[2 * np + 1], pl[kk], bh[2], bh[3]);
            }
        }
    }

    // ---- normalise and store: rows g / g + 8, columns 8 n + 2 t + {0, 1}
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = warp * 16 + g + 8 * h;
        const int s = s0 + r / G, gi = r - (r / G) * G;
        if (s >= p.seq) continue;
        const float inv = 1.0f / lrow[h];
        float* op = p.out + ((size_t)b * p.seq + s) * p.n_heads * D + (size_t)(hk * G + gi) * D;
#pragma unroll
        for (int n = 0; n < NT; ++n)
            *reinterpret_cast<float2*>(op + 8 * n + 2 * t) = make_float2(oacc[n][2 * h] * inv, oacc[n][2 * h + 1] * inv);
    }
}

int configure_attn_prefill_tc() {
    RB_CUDA(cudaFuncSetAttribute(attn_prefill_tc_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)attn_prefill_tc_smem<64>()));
    RB_CUDA(cudaFuncSetAttribute(attn_prefill_tc_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)attn_prefill_tc_smem<128>()));
    RB_CUDA(cudaFuncSetAttribute(attn_prefill_tc_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)attn_prefill_tc_smem<64>()));
    RB_CUDA(cudaFuncSetAttribute(attn_prefill_tc_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)attn_prefill_tc_smem<128>()));
    return ROTOR_B200_OK;
}

// Whether the tiled kernel takes this shape (the per-query kernel covers the rest).
bool attn_prefill_supported(const AttnParams& p, int rows) {
    if (p.head_dim != 64 && p.head_dim != 128) return false;
    const int G = p.n_heads / p.n_kv_heads;
    // long prompts, or many sequences with few new positions each (a CTA then serves one sequence's
    // group of heads and streams that sequence's cache once)
    return G >= 1 && G <= TC_BM && TC_BM % G == 0 && (p.seq >= 16 || rows >= 16);
}

int launch_attn_prefill_tc(const AttnParams& p, int rows, cudaStream_t st) {
    const int G = p.n_heads / p.n_kv_heads, QT = TC_BM / G;
    const int batch = rows / p.seq;
    dim3 grid((p.seq + QT - 1) / QT, p.n_kv_heads, batch);
    if (p.kv_split) {
        const size_t n = (size_t)batch * p.n_kv_heads * p.max_seq * (p.head_dim / 4);
        kv_split_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(p, batch);
        const int rc = launch_status();
        if (rc) return rc;
        if (p.head_dim == 64)
            attn_prefill_tc_kernel<64, true><<<grid, 256, attn_prefill_tc_smem<64>(), st>>>(p);
        else
            attn_prefill_tc_kernel<128, true><<<grid, 256, attn_prefill_tc_smem<128>(), st>>>(p);
        return launch_status();
    }
    if (p.head_dim == 64)
        attn_prefill_tc_kernel<64, false><<<grid, 256, attn_prefill_tc_smem<64>(), st>>>(p);
    else
        attn_prefill_tc_kernel<128, false><<<grid, 256, attn_prefill_tc_smem<128>(), st>>>(p);
    return launch_status();
}

}  // namespace rb
