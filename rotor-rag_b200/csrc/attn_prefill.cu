// Softmax attention for prompt prefill (many query positions per sequence), float32.
//
// Reference: MultiHeadAttention.forward, src/rotor/transformer.py:249-283 -- scores
// Q K^T / sqrt(head_dim) over the whole cache, optional additive causal mask, softmax, times V,
// with K/V shared by the n_heads / n_kv_heads query heads of a group.  The reference builds
// the dense [B, H, S, T] score tensor; this kernel never does.
//
// One CTA (256 threads) owns 128 "query rows" of one KV head -- 128/G consecutive positions
// times the G query heads of the group, so a K/V tile staged in shared memory serves the
// whole group -- and walks the keys 64 at a time with an online softmax:
//   S = Q K^T    128 x 64 per tile, 8 x 4 per thread, operands read as 128-bit shared loads
//   P = exp(S - rowmax), running max / sum per row (16 lanes share a row)
//   O += P V     128 x D per CTA, 8 x D/16 per thread
// K and V tiles arrive with cp.async (16-byte pieces, zero fill past the last key).  Rows of
// Q and K are padded by four floats so that the 128-bit loads of a quarter warp fall in
// distinct banks.  FP32 FMA pipe; the tile shapes give 0.375 / 0.25 shared-memory words per
// FMA for the two products.
#include "model.cuh"

namespace rb {

constexpr int AP_BM = 128;  // query rows per CTA
constexpr int AP_BN = 64;   // keys per tile
constexpr int AP_PS = AP_BN + 4;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int sz = valid ? 16 : 0;  // src-size 0: the 16 bytes are zero filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(sz) : "memory");
}

template <int D>
size_t attn_prefill_smem() {
    return ((size_t)AP_BM * (D + 4) + (size_t)AP_BN * (D + 4) + (size_t)AP_BN * D + (size_t)AP_BM * AP_PS) *
           sizeof(float);
}

template <int D>
__global__ void __launch_bounds__(256) attn_prefill_kernel(const __grid_constant__ AttnParams p) {
    constexpr int QS = D + 4;     // row stride of Qs / Ks
    constexpr int NC4 = D / 64;   // float4 column groups of O per thread
    extern __shared__ __align__(16) float sm[];
    float* Qs = sm;                     // [AP_BM][QS]
    float* Ks = Qs + AP_BM * QS;        // [AP_BN][QS]
    float* Vs = Ks + AP_BN * QS;        // [AP_BN][D]
    float* Ps = Vs + AP_BN * D;         // [AP_BM][AP_PS]
    const int G = p.n_heads / p.n_kv_heads, QT = AP_BM / G;
    const int qt = gridDim.x - 1 - blockIdx.x;  // late query tiles see the most keys: start them first
    const int hk = blockIdx.y, b = blockIdx.z;
    const int s0 = qt * QT;
    const int past = p.past_len[b];
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const float scale = 1.0f / sqrtf((float)D);

    // ---- Q tile, scaled; rows past the sequence end are zero
    for (int idx = tid; idx < AP_BM * (D / 4); idx += 256) {
        const int r = idx / (D / 4), c4 = idx - r * (D / 4);
        const int s = s0 + r / G, g = r - (r / G) * G;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (s < p.seq) {
            v = *reinterpret_cast<const float4*>(p.q + ((size_t)b * p.seq + s) * p.n_heads * D +
                                                 (size_t)(hk * G + g) * D + 4 * c4);
            v.x *= scale;
            v.y *= scale;
            v.z *= scale;
            v.w *= scale;
        }
        *reinterpret_cast<float4*>(Qs + r * QS + 4 * c4) = v;
    }

    // keys this tile has to visit, and the number of keys each of the thread's rows may see
    int s_last = s0 + QT - 1;
    if (s_last > p.seq - 1) s_last = p.seq - 1;
    int t_all = p.causal ? past + s_last + 1 : past + p.seq;
    if (t_all > p.max_seq) t_all = p.max_seq;
    int lim[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int s = s0 + (ty + 16 * i) / G;
        int l = p.causal ? past + s + 1 : past + p.seq;
        lim[i] = l < t_all ? l : t_all;  // rows past the sequence end only ever see masked-out garbage: not stored
    }
    const float* kbase = p.k_cache + ((size_t)b * p.n_kv_heads + hk) * p.max_seq * D;
    const float* vbase = p.v_cache + ((size_t)b * p.n_kv_heads + hk) * p.max_seq * D;

    float o[8][4 * NC4];
    float mrow[8], lrow[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        mrow[i] = -INFINITY;
        lrow[i] = 0.f;
#pragma unroll
        for (int c = 0; c < 4 * NC4; ++c) o[i][c] = 0.f;
    }

    const int ntiles = (t_all + AP_BN - 1) / AP_BN;
    for (int kt = 0; kt < ntiles; ++kt) {
        __syncthreads();  // the previous tile's K, V and P are no longer read (and Qs is written, first time)
        const int t0 = kt * AP_BN;
        for (int idx = tid; idx < AP_BN * (D / 4); idx += 256) {
            const int j = idx / (D / 4), c4 = idx - j * (D / 4);
            const bool valid = t0 + j < t_all;
            const size_t off = (size_t)(valid ? t0 + j : 0) * D + 4 * c4;
            cp_async16(Ks + j * QS + 4 * c4, kbase + off, valid);
            cp_async16(Vs + j * D + 4 * c4, vbase + off, valid);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();

        // ---- S = Q K^T for rows ty + 16 i, keys tx + 16 c
        float sc[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int c = 0; c < 4; ++c) sc[i][c] = 0.f;
#pragma unroll 2
        for (int d4 = 0; d4 < D / 4; ++d4) {
            float4 kv[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) kv[c] = *reinterpret_cast<const float4*>(Ks + (tx + 16 * c) * QS + 4 * d4);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float4 qv = *reinterpret_cast<const float4*>(Qs + (ty + 16 * i) * QS + 4 * d4);
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    sc[i][c] += qv.x * kv[c].x + qv.y * kv[c].y + qv.z * kv[c].z + qv.w * kv[c].w;
            }
        }

        // ---- online softmax; the 16 lanes with equal ty share a row
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                if (t0 + tx + 16 * c >= lim[i]) sc[i][c] = -INFINITY;
                mx = fmaxf(mx, sc[i][c]);
            }
#pragma unroll
            for (int w = 1; w < 16; w <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, w));
            const float mn = fmaxf(mrow[i], mx);  // finite from the first tile on: key 0 is visible to every row
            const float corr = __expf(mrow[i] - mn);
            float ps = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float e = __expf(sc[i][c] - mn);
                ps += e;
                Ps[(ty + 16 * i) * AP_PS + tx + 16 * c] = e;
            }
#pragma unroll
            for (int w = 1; w < 16; w <<= 1) ps += __shfl_xor_sync(0xffffffffu, ps, w);
            lrow[i] = lrow[i] * corr + ps;
            mrow[i] = mn;
#pragma unroll
            for (int c = 0; c < 4 * NC4; ++c) o[i][c] *= corr;
        }
        __syncthreads();

        // ---- O += P V for rows ty + 16 i, columns 4 tx + 64 n
#pragma unroll 2
        for (int j4 = 0; j4 < AP_BN / 4; ++j4) {
            float4 pv[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) pv[i] = *reinterpret_cast<const float4*>(Ps + (ty + 16 * i) * AP_PS + 4 * j4);
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
#pragma unroll
                for (int n = 0; n < NC4; ++n) {
                    const float4 vv = *reinterpret_cast<const float4*>(Vs + (4 * j4 + jj) * D + 4 * tx + 64 * n);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float pj = jj == 0 ? pv[i].x : (jj == 1 ? pv[i].y : (jj == 2 ? pv[i].z : pv[i].w));
                        o[i][4 * n + 0] += pj * vv.x;
                        o[i][4 * n + 1] += pj * vv.y;
                        o[i][4 * n + 2] += pj * vv.z;
                        o[i][4 * n + 3] += pj * vv.w;
                    }
                }
            }
        }
    }

    // ---- normalise and store
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = ty + 16 * i;
        const int s = s0 + r / G, g = r - (r / G) * G;
        if (s >= p.seq) continue;
        const float inv = 1.0f / lrow[i];
        float* op = p.out + ((size_t)b * p.seq + s) * p.n_heads * D + (size_t)(hk * G + g) * D;
#pragma unroll
        for (int n = 0; n < NC4; ++n)
            *reinterpret_cast<float4*>(op + 4 * tx + 64 * n) =
                make_float4(o[i][4 * n] * inv, o[i][4 * n + 1] * inv, o[i][4 * n + 2] * inv, o[i][4 * n + 3] * inv);
    }
}

// Whether the tiled kernel takes this shape (the per-query kernel covers the rest).
bool attn_prefill_supported(const AttnParams& p, int rows) {
    if (p.head_dim != 64 && p.head_dim != 128) return false;
    const int G = p.n_heads / p.n_kv_heads;
    // long prompts, or many sequences with few new positions each (a CTA then serves one sequence's
    // group of heads and streams that sequence's cache once)
    return G >= 1 && G <= AP_BM && AP_BM % G == 0 && (p.seq >= 16 || rows >= 16);
}

int configure_attn_prefill() {
    RB_CUDA(cudaFuncSetAttribute(attn_prefill_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)attn_prefill_smem<64>()));
    RB_CUDA(cudaFuncSetAttribute(attn_prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)attn_prefill_smem<128>()));
    return ROTOR_B200_OK;
}

int launch_attn_prefill(const AttnParams& p, int rows, cudaStream_t st) {
    const int G = p.n_heads / p.n_kv_heads, QT = AP_BM / G;
    const int batch = rows / p.seq;
    dim3 grid((p.seq + QT - 1) / QT, p.n_kv_heads, batch);
    if (p.head_dim == 64)
        attn_prefill_kernel<64><<<grid, 256, attn_prefill_smem<64>(), st>>>(p);
    else
        attn_prefill_kernel<128><<<grid, 256, attn_prefill_smem<128>(), st>>>(p);
    return launch_status();
}

}  // namespace rb
