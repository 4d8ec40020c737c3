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
    if (rows >= 5 && p.acc.planes == 1 && p.acc.out % 4 == 0 && p.head_dim % 8 == 0 && p.terms >= 1 && p.terms <= 3)
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

static bool attn_decode_stream_ok(const AttnParams& p, int rows);
static int launch_attn_decode_stream(const AttnParams& p, int rows, cudaStream_t st);

int launch_attention(const AttnParams& p, int rows, cudaStream_t st) {
    if (attn_decode_stream_ok(p, rows)) return launch_attn_decode_stream(p, rows, st);  // batched generation steps
    if (attn_prefill_t5_supported(p, rows)) return launch_attn_prefill_t5(p, rows, st);  // head_dim 128 prompts
    if (attn_prefill_supported(p, rows)) return launch_attn_prefill_tc(p, rows, st);
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
    pdl_wait();
    pdl_trigger();
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

// ---------------------------------------------------------------------------------------
// The same one-token attention with the slices of one KV head as a thread-block cluster.
// Grid (n_kv_heads * nsplit, batch), cluster (nsplit, 1, 1), nsplit <= 8; one warp per query
// head of the group (G <= 8 warps), head_dim 64 or 128.
//
// Before the programmatic-launch wait a CTA reads the cached length and copies its slice of the
// K and V rows (written by earlier steps) into shared memory with cp.async.  After the wait the
// CTA whose slice holds the new position rotates the new k, appends k / v to the cache and to
// the staged rows; every warp fetches and rotates its head's q into registers.  From there a
// warp works alone: scores with 8 lanes per key (4 keys per pass, q held as four 16-byte pieces
// per lane), an online softmax over chunks of 32 keys (lane j keeps key j's score), weighted V
// with 4 output dimensions per lane.  No CTA barrier separates these phases.
//
// The slices are merged through distributed shared memory by pushing: every warp stores its
// (max, sum) to all CTAs of the cluster and its weighted V to the CTA that owns those outputs;
// after one cluster barrier CTA r combines the r-th share of the group's outputs from its own
// shared memory and writes finished attention rows -- the output projection reads one float row
// instead of every CTA of it re-merging nsplit partial rows.
__device__ __forceinline__ void cp_async16(float* dst_smem, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src)
                 : "memory");
}
__device__ __forceinline__ uint32_t cluster_addr(const void* own_smem, unsigned cta) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                 : "=r"(remote)
                 : "r"((uint32_t)__cvta_generic_to_shared(own_smem)), "r"(cta));
    return remote;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void st_cluster_v4(uint32_t addr, float4 v) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                 : "memory");
}

constexpr int AC_MAX_SPLIT = 16;  // largest cluster (above the portable 8 the device is asked first)
constexpr int AC_MAX_GROUP = 8;  // query heads per KV head
constexpr int AC_MAX_THREADS = 512;
// Warps per query head in the cluster kernel: as many as fit 512 threads, at most four.
__host__ __device__ inline int ac_warps_per_head(int G) { return G <= 4 ? 4 : (G <= 8 ? 2 : 1); }

__host__ __device__ inline int round4(int v) { return (v + 3) & ~3; }

// One warp, one query head, up to 32 keys whose K and V rows lie in shared memory (row stride D):
// scores with 8 lanes per key (lane l8 = lane & 7 holds the 16-byte pieces l8, l8 + 8, ... of q,
// pre-scaled), online softmax across chunks (lane j keeps key j's score), weighted V with D / 32
// output dimensions per lane.  Updates the running maximum, sum and output.
template <int D>
__device__ __forceinline__ void attn_warp_chunk(const float4 (&q4)[D / 32], const float* Kc, const float* Vc, int nk,
                                                int lane, float& m_run, float& l_run, float4& o) {
    constexpr int NCH = D / 32, OPL = D / 32;
    const int l8 = lane & 7;
    float my_s = -INFINITY;
    for (int i = 0; i * 4 < nk; ++i) {  // four keys per pass: key 4 i + (lane >> 3)
        const int j = 4 * i + (lane >> 3);
        float s = 0.f;
        if (j < nk) {
            const float4* kr = reinterpret_cast<const float4*>(Kc + (size_t)j * D);
#pragma unroll
            for (int e = 0; e < NCH; ++e) {
                const float4 k4 = kr[8 * e + l8];
                s += q4[e].x * k4.x + q4[e].y * k4.y + q4[e].z * k4.z + q4[e].w * k4.w;
            }
        }
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        const float mine = __shfl_sync(0xffffffffu, s, (lane & 3) * 8);  // key 4 i + (lane & 3)
        if ((lane >> 2) == i) my_s = mine;                               // lane j keeps key j
    }
    if (lane >= nk) my_s = -INFINITY;
    const float m_new = fmaxf(m_run, warp_max(my_s));
    const float keep = m_run == -INFINITY ? 0.f : __expf(m_run - m_new);
    const float pr = lane < nk ? __expf(my_s - m_new) : 0.f;
    l_run = l_run * keep + warp_sum(pr);
    o = make_float4(o.x * keep, o.y * keep, o.z * keep, o.w * keep);
    const float* vr = Vc + OPL * lane;
#pragma unroll 4
    for (int j = 0; j < nk; ++j) {
        const float pj = __shfl_sync(0xffffffffu, pr, j);
        if constexpr (OPL == 4) {
            const float4 v4 = *reinterpret_cast<const float4*>(vr + (size_t)j * D);
            o.x += pj * v4.x;
            o.y += pj * v4.y;
            o.z += pj * v4.z;
            o.w += pj * v4.w;
        } else {
            const float2 v2 = *reinterpret_cast<const float2*>(vr + (size_t)j * D);
            o.x += pj * v2.x;
            o.y += pj * v2.y;
        }
    }
    m_run = m_new;
}

// The same step of the online softmax for the streaming kernel, where many warps per SM make issue
// slots, not latency, the limit: fewer instructions per key.  K and V rows lie in shared memory with a
// row stride of D + AC_PAD floats (consecutive rows start four banks apart, so 32 lanes reading the
// same piece of 32 different rows do not collide).  Scores: lane j multiplies key j's whole row with q
// (shared memory, pre-scaled; every lane reads the same piece: a broadcast) in four independent
// chains, no shuffles.  Weighted V: the probabilities go through `ps` (32 floats of this warp) and
// come back four at a time as broadcasts; lane l accumulates output dimensions (D / 32) l .. in two
// alternating sets.
constexpr int AC_PAD = 4;

// H query heads of the group per warp (H = 1 or 2): a K or V piece is read from shared memory once and
// multiplied for every head of the warp, which halves the shared-memory traffic that bounds this kernel.
// qs: H rows of D floats, ps: H rows of 32.
template <int D, int H>
__device__ __forceinline__ void attn_warp_chunk_rows(const float* qs, const float* Kc, const float* Vc, float* ps, int nk,
                                                     int lane, float (&m_run)[H], float (&l_run)[H], float4 (&o)[H]) {
    constexpr int KS = D + AC_PAD, OPL = D / 32, C4 = D / 4;
    float my_s[H];
#pragma unroll
    for (int h = 0; h < H; ++h) my_s[h] = -INFINITY;
    if (lane < nk) {
        const float4* kr = reinterpret_cast<const float4*>(Kc + (size_t)lane * KS);
        const float4* qr = reinterpret_cast<const float4*>(qs);
        float acc[H][2];
#pragma unroll
        for (int h = 0; h < H; ++h) acc[h][0] = acc[h][1] = 0.f;
#pragma unroll
        for (int c = 0; c < C4; ++c) {
            const float4 k4 = kr[c];
#pragma unroll
            for (int h = 0; h < H; ++h) {
                const float4 q4 = qr[h * C4 + c];
                acc[h][c & 1] += q4.x * k4.x + q4.y * k4.y + q4.z * k4.z + q4.w * k4.w;
            }
        }
#pragma unroll
        for (int h = 0; h < H; ++h) my_s[h] = acc[h][0] + acc[h][1];
    }
    float keep[H];
    __syncwarp();  // the previous chunk's readers of ps are done
#pragma unroll
    for (int h = 0; h < H; ++h) {
        const float m_new = fmaxf(m_run[h], warp_max(my_s[h]));
        keep[h] = m_run[h] == -INFINITY ? 0.f : __expf(m_run[h] - m_new);
        const float pr = lane < nk ? __expf(my_s[h] - m_new) : 0.f;
        l_run[h] = l_run[h] * keep[h] + warp_sum(pr);
        ps[h * 32 + lane] = pr;
        m_run[h] = m_new;
    }
    __syncwarp();
    float4 oa[H], ob[H];
#pragma unroll
    for (int h = 0; h < H; ++h) {
        oa[h] = make_float4(o[h].x * keep[h], o[h].y * keep[h], o[h].z * keep[h], o[h].w * keep[h]);
        ob[h] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const float* vr = Vc + OPL * lane;
    auto fma_row = [&](float4 (&acc4)[H], const float (&pj)[H], int j) {
        if constexpr (OPL == 4) {
            const float4 v4 = *reinterpret_cast<const float4*>(vr + (size_t)j * KS);
#pragma unroll
            for (int h = 0; h < H; ++h) {
                acc4[h].x += pj[h] * v4.x;
                acc4[h].y += pj[h] * v4.y;
                acc4[h].z += pj[h] * v4.z;
                acc4[h].w += pj[h] * v4.w;
            }
        } else {
            const float2 v2 = *reinterpret_cast<const float2*>(vr + (size_t)j * KS);
#pragma unroll
            for (int h = 0; h < H; ++h) {
                acc4[h].x += pj[h] * v2.x;
                acc4[h].y += pj[h] * v2.y;
            }
        }
    };
    int j = 0;
    for (; j + 4 <= nk; j += 4) {  // rows at and beyond nk are never read: they may hold anything
        float4 p4[H];
#pragma unroll
        for (int h = 0; h < H; ++h) p4[h] = *reinterpret_cast<const float4*>(ps + h * 32 + j);
        float pj[H];
#pragma unroll
        for (int h = 0; h < H; ++h) pj[h] = p4[h].x;
        fma_row(oa, pj, j);
#pragma unroll
        for (int h = 0; h < H; ++h) pj[h] = p4[h].y;
        fma_row(ob, pj, j + 1);
#pragma unroll
        for (int h = 0; h < H; ++h) pj[h] = p4[h].z;
        fma_row(oa, pj, j + 2);
#pragma unroll
        for (int h = 0; h < H; ++h) pj[h] = p4[h].w;
        fma_row(ob, pj, j + 3);
    }
    for (; j < nk; ++j) {
        float pj[H];
#pragma unroll
        for (int h = 0; h < H; ++h) pj[h] = ps[h * 32 + j];
        fma_row(oa, pj, j);
    }
#pragma unroll
    for (int h = 0; h < H; ++h)
        o[h] = make_float4(oa[h].x + ob[h].x, oa[h].y + ob[h].y, oa[h].z + ob[h].z, oa[h].w + ob[h].w);
}

// MAXS: the most slices (cluster size) this instantiation merges: 8 for portable clusters, 16 beyond.
template <int D, int MAXS>
__global__ void __launch_bounds__(AC_MAX_THREADS) attn_decode_cluster_kernel(const __grid_constant__ AttnDecodeParams p) {
    extern __shared__ __align__(16) float sm[];
    constexpr int half = D / 2, C4 = D / 4, NCH = D / 32;  // 16-byte pieces per row; pieces per lane of a key's 8 lanes
    const int tid = threadIdx.x, nthr = blockDim.x, lane = tid & 31;
    const int G = p.n_heads / p.n_kv_heads, ns = p.nsplit;  // blockDim.x == 32 * G * W
    const int W = (nthr >> 5) / G;                          // warps per query head: each takes a run of the slice's keys
    const int warp = (tid >> 5) % G, sub = (tid >> 5) / G;  // head within the group, run within the slice
    const int hk = blockIdx.x / ns, sp = blockIdx.x % ns;   // sp is also the rank inside the cluster
    const int b = blockIdx.y;
    const int dq = p.n_heads * D, dkv = p.n_kv_heads * D;
    const int lcmax = (p.max_seq + ns - 1) / ns;
    const int share = G * D / ns;             // outputs of the group this CTA finishes (a multiple of 4)
    float* recv_o = sm;                       // [ns][share] weighted V of every slice for this CTA's outputs
    float* recv_ml = recv_o + ns * share;     // [ns][2 G]   (max, sum) of every slice and head
    float* Ks = recv_ml + round4(ns * 2 * G); // [lcmax][D]
    float* Vs = Ks + (size_t)lcmax * D;       // [lcmax][D]
    float* runs = Vs + (size_t)lcmax * D;     // [(W - 1) G][D + 4] results of the runs 1 .. W-1: o, then (max, sum)
    TraceRec tr;
    RB_STAMP(tr, 0);
    // every CTA of the cluster has started (its shared memory may be written) once this phase completes
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");

    // ---- before the wait: the cached length (advanced by the previous step's last kernel) and
    // this slice's older cache rows
    const int pos = __ldcg(p.past_len + b);
    const int T = min(pos + 1, p.max_seq);
    const int lc = (T + ns - 1) / ns;
    const int t0 = sp * lc, t1 = min(T, t0 + lc);
    float* kc = p.k_cache + ((size_t)b * p.n_kv_heads + hk) * p.max_seq * D;
    float* vc = p.v_cache + ((size_t)b * p.n_kv_heads + hk) * p.max_seq * D;
    for (int idx = tid; idx < (t1 - t0) * C4; idx += nthr) {
        const int r = idx / C4, c4 = idx - r * C4, t = t0 + r;
        if (t != pos) {  // the new row comes from the q/k/v product
            cp_async16(Ks + (size_t)r * D + 4 * c4, kc + (size_t)t * D + 4 * c4);
            cp_async16(Vs + (size_t)r * D + 4 * c4, vc + (size_t)t * D + 4 * c4);
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    if (p.rope && tid * 16 < half) prefetch_l2(p.rope + (size_t)pos * half + tid * 16);
    RB_STAMP(tr, 1);
    pdl_wait();
    pdl_trigger();
    RB_STAMP(tr, 2);

    const float* qf = p.qkv_f + (size_t)b * (dq + 2 * dkv);
    // ---- the new k / v row: rotate, append to the cache and to the staged rows (owning slice only)
    if (pos >= t0 && pos < t1) {
        float* ks_row = Ks + (size_t)(pos - t0) * D;
        float* vs_row = Vs + (size_t)(pos - t0) * D;
        const bool keep = pos < p.max_seq;
        for (int i = tid; i < half; i += nthr) {
            float a = __ldcg(qf + dq + hk * D + i), c = __ldcg(qf + dq + hk * D + i + half);
            if (p.rope) {
                const float2 cs = p.rope[(size_t)pos * half + i];
                const float ra = a * cs.x - c * cs.y, rc = c * cs.x + a * cs.y;
                a = ra;
                c = rc;
            }
            ks_row[i] = a;
            ks_row[i + half] = c;
            if (keep) {
                kc[(size_t)pos * D + i] = a;
                kc[(size_t)pos * D + i + half] = c;
            }
        }
        for (int i = tid; i < D; i += nthr) {
            const float v = __ldcg(qf + dq + dkv + hk * D + i);
            vs_row[i] = v;
            if (keep) vc[(size_t)pos * D + i] = v;
        }
    }
    // ---- q of this warp's head: lane l8 = lane & 7 holds pieces l8, l8 + 8, ... (four floats each),
    // pre-scaled by 1/sqrt(D); piece c < C4/2 rotates with piece c + C4/2, both in the same lane
    const int l8 = lane & 7;
    float4 q4[NCH];
    {
        const float* qh = qf + (size_t)(hk * G + warp) * D;
#pragma unroll
        for (int e = 0; e < NCH; ++e) q4[e] = __ldcg(reinterpret_cast<const float4*>(qh) + (8 * e + l8));
        if (p.rope) {
#pragma unroll
            for (int e = 0; e < NCH / 2; ++e) {
                const float4* cs4 = reinterpret_cast<const float4*>(p.rope + (size_t)pos * half + 4 * (8 * e + l8));
                const float4 c01 = __ldg(cs4), c23 = __ldg(cs4 + 1);  // (cos, sin) of four consecutive pairs
                float4& a = q4[e];
                float4& c = q4[e + NCH / 2];
                const float4 ra = make_float4(a.x * c01.x - c.x * c01.y, a.y * c01.z - c.y * c01.w,
                                              a.z * c23.x - c.z * c23.y, a.w * c23.z - c.w * c23.w);
                const float4 rc = make_float4(c.x * c01.x + a.x * c01.y, c.y * c01.z + a.y * c01.w,
                                              c.z * c23.x + a.z * c23.y, c.w * c23.z + a.w * c23.w);
                a = ra;
                c = rc;
            }
        }
        const float scale = 1.0f / sqrtf((float)D);
#pragma unroll
        for (int e = 0; e < NCH; ++e) q4[e] = make_float4(q4[e].x * scale, q4[e].y * scale, q4[e].z * scale, q4[e].w * scale);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();  // staged rows and the new row are visible to every warp
    RB_STAMP(tr, 3);

    // ---- this warp's head over its run of the slice, 32 keys at a time
    float m_run = -INFINITY, l_run = 0.f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);  // output dimensions OPL * lane .. + OPL - 1
    constexpr int OPL = D / 32;                  // output floats per lane
    {
        const int per = ((t1 - t0 + W - 1) / W + 3) & ~3;  // whole passes of four keys
        const int a0 = t0 + sub * per, a1 = min(t1, a0 + per);
        for (int c0 = a0; c0 < a1; c0 += 32)
            attn_warp_chunk<D>(q4, Ks + (size_t)(c0 - t0) * D, Vs + (size_t)(c0 - t0) * D, min(32, a1 - c0), lane, m_run,
                               l_run, o);
    }
    if (W > 1) {  // fold the runs of a head into its first warp
        if (sub > 0) {
            float* r = runs + (size_t)((sub - 1) * G + warp) * (D + 4);
            if constexpr (OPL == 4) {
                *reinterpret_cast<float4*>(r + OPL * lane) = o;
            } else {
                r[OPL * lane] = o.x;
                r[OPL * lane + 1] = o.y;
            }
            if (lane == 0) {
                r[D] = m_run;
                r[D + 1] = l_run;
            }
        }
        __syncthreads();
        if (sub == 0) {
            for (int s2 = 1; s2 < W; ++s2) {
                const float* r = runs + (size_t)((s2 - 1) * G + warp) * (D + 4);
                const float m2 = r[D], l2 = r[D + 1];
                const float M = fmaxf(m_run, m2);
                const float a = m_run == -INFINITY ? 0.f : __expf(m_run - M);
                const float b2 = m2 == -INFINITY ? 0.f : __expf(m2 - M);
                if constexpr (OPL == 4) {
                    const float4 o2 = *reinterpret_cast<const float4*>(r + OPL * lane);
                    o = make_float4(o.x * a + o2.x * b2, o.y * a + o2.y * b2, o.z * a + o2.z * b2, o.w * a + o2.w * b2);
                } else {
                    o.x = o.x * a + r[OPL * lane] * b2;
                    o.y = o.y * a + r[OPL * lane + 1] * b2;
                }
                l_run = l_run * a + l2 * b2;
                m_run = M;
            }
        }
    }
    RB_STAMP(tr, 4);

    // ---- push this slice's results to the CTAs that merge them
    asm volatile("barrier.cluster.wait.aligned;" ::: "memory");  // (phase opened at the top of the kernel)
    if (sub == 0) {
        const int oi = warp * D + OPL * lane;      // first output of this lane within the group
        const int dst = oi / share, off = oi - dst * share;
        const uint32_t ra = cluster_addr(recv_o + sp * share + off, (unsigned)dst);
        if constexpr (OPL == 4) {
            st_cluster_v4(ra, o);
        } else {
            st_cluster_f32(ra, o.x);
            st_cluster_f32(ra + 4, o.y);
        }
        if (lane < ns) {
            const uint32_t rm = cluster_addr(recv_ml + sp * 2 * G + warp, (unsigned)lane);
            st_cluster_f32(rm, m_run);
            st_cluster_f32(rm + 4 * G, l_run);
        }
    }
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");

    // ---- merge: outputs [sp * share, (sp + 1) * share) of the group, from this CTA's own shared memory
    for (int idx = tid; idx < share; idx += nthr) {
        const int oi = sp * share + idx, g = oi / D, d = oi - g * D;
        float f[MAXS];
        float M = -INFINITY;
#pragma unroll
        for (int s2 = 0; s2 < MAXS; ++s2) {
            f[s2] = s2 < ns ? recv_ml[s2 * 2 * G + g] : -INFINITY;
            M = fmaxf(M, f[s2]);
        }
        float L = 0.f;
#pragma unroll
        for (int s2 = 0; s2 < MAXS; ++s2) {
            const float e = f[s2] == -INFINITY ? 0.f : __expf(f[s2] - M);
            if (s2 < ns) L += recv_ml[s2 * 2 * G + G + g] * e;
            f[s2] = e;
        }
        const float inv = 1.0f / L;
        float acc = 0.f;
#pragma unroll
        for (int s2 = 0; s2 < MAXS; ++s2)
            if (s2 < ns) acc += recv_o[s2 * share + idx] * (f[s2] * inv);
        p.attn_out[(size_t)b * dq + (size_t)(hk * G + g) * D + d] = acc;
    }
    RB_STAMP(tr, 5);
    RB_TRACE_COMMIT(tr, 100);
}

// ---------------------------------------------------------------------------------------
// One-token attention for many sequences at once (batched generation steps): grid
// (n_kv_heads, batch, runs), H query heads of the group per warp.  q is finished (rotated), the new
// k / v row is in the cache already.  The CTA streams its run of the sequence's K and V rows through
// shared memory AS_KEYS keys at a time, double buffered with cp.async, and every warp runs the
// per-head chunk routine (attn_warp_chunk_rows).  One run (64 sequences and more): whole sequences,
// finished attention rows, no partials, no merge.  Several runs (fewer sequences, so that about 512
// CTAs exist): every run writes its un-normalised output with its (max, sum), merged by the stage
// that quantises the attention rows.
constexpr int AS_KEYS = 24;  // two stages of 24 keys: four CTAs per SM at head_dim 128, so that 64 sequences x 8 KV heads run as one wave

template <int D, int H>
__global__ void __launch_bounds__(32 * AC_MAX_GROUP) attn_decode_stream_kernel(const __grid_constant__ AttnParams p) {
    extern __shared__ __align__(16) float sm[];
    constexpr int C4 = D / 4, OPL = D / 32, KS = D + AC_PAD;
    const int tid = threadIdx.x, nthr = blockDim.x, lane = tid & 31, warp = tid >> 5;
    const int G = p.n_heads / p.n_kv_heads;  // blockDim.x == 32 * G / H: warp w takes heads H w .. H w + H - 1 of the group
    const int hk = blockIdx.x, b = blockIdx.y;
    const int dq = p.n_heads * D;
    const int T = min(p.past_len[b] + 1, p.max_seq);
    const float* kc = p.k_cache + ((size_t)b * p.n_kv_heads + hk) * p.max_seq * D;
    const float* vc = p.v_cache + ((size_t)b * p.n_kv_heads + hk) * p.max_seq * D;
    float* qs = sm;                         // [G][D]
    float* ps = qs + G * D;                 // [G][32]
    float* Ks = ps + G * 32;                // [2][AS_KEYS][KS]
    float* Vs = Ks + 2 * AS_KEYS * KS;      // [2][AS_KEYS][KS]
    // this CTA's run of the sequence: all of it, or one of gridDim.z equal parts
    const int nrun = (int)gridDim.z, run = (int)blockIdx.z;
    const int rlen = (T + nrun - 1) / nrun, k0 = run * rlen, k1 = min(T, k0 + rlen);
    const int nchunk = k1 > k0 ? (k1 - k0 + AS_KEYS - 1) / AS_KEYS : 0;
    auto fetch = [&](int chunk, int stage) {
        const int t0 = k0 + chunk * AS_KEYS, n = min(AS_KEYS, k1 - t0);
        for (int idx = tid; idx < n * C4; idx += nthr) {
            const int r = idx / C4, c4 = idx - r * C4;
            cp_async16(Ks + ((size_t)stage * AS_KEYS + r) * KS + 4 * c4, kc + (size_t)(t0 + r) * D + 4 * c4);
            cp_async16(Vs + ((size_t)stage * AS_KEYS + r) * KS + 4 * c4, vc + (size_t)(t0 + r) * D + 4 * c4);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (nchunk > 0) fetch(0, 0);
    {  // this warp's q rows, pre-scaled (read back by the same warp only, after the first CTA barrier)
        const float* qh = p.q + (size_t)b * dq + (size_t)(hk * G + warp * H) * D;
        const float scale = 1.0f / sqrtf((float)D);
        for (int i = lane; i < H * C4; i += 32) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(qh) + i);
            reinterpret_cast<float4*>(qs + warp * H * D)[i] = make_float4(v.x * scale, v.y * scale, v.z * scale, v.w * scale);
        }
    }
    float m_run[H], l_run[H];
    float4 o[H];
#pragma unroll
    for (int h = 0; h < H; ++h) {
        m_run[h] = -INFINITY;
        l_run[h] = 0.f;
        o[h] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int c = 0; c < nchunk; ++c) {
        if (c + 1 < nchunk) {
            fetch(c + 1, (c + 1) & 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();  // chunk c has landed for every thread
        const int st = c & 1;
        attn_warp_chunk_rows<D, H>(qs + warp * H * D, Ks + (size_t)st * AS_KEYS * KS, Vs + (size_t)st * AS_KEYS * KS,
                                   ps + warp * H * 32, min(AS_KEYS, k1 - k0 - c * AS_KEYS), lane, m_run, l_run, o);
        __syncthreads();  // every warp is done with this stage before chunk c + 2 overwrites it
    }
    if (nrun > 1) {  // partial results of this run: merged by the stage that follows
#pragma unroll
        for (int h = 0; h < H; ++h) {
            const size_t slot = ((size_t)b * p.n_heads + (hk * G + warp * H + h)) * nrun + run;
            float* dst = p.part_o + slot * D + OPL * lane;
            if constexpr (OPL == 4) {
                *reinterpret_cast<float4*>(dst) = o[h];
            } else {
                *reinterpret_cast<float2*>(dst) = make_float2(o[h].x, o[h].y);
            }
            if (lane == 0) {
                p.part_m[slot] = m_run[h];
                p.part_l[slot] = l_run[h];
            }
        }
        return;
    }
#pragma unroll
    for (int h = 0; h < H; ++h) {
        const float inv = 1.0f / l_run[h];
        float* dst = p.out + (size_t)b * dq + (size_t)(hk * G + warp * H + h) * D + OPL * lane;
        if constexpr (OPL == 4) {
            *reinterpret_cast<float4*>(dst) = make_float4(o[h].x * inv, o[h].y * inv, o[h].z * inv, o[h].w * inv);
        } else {
            *reinterpret_cast<float2*>(dst) = make_float2(o[h].x * inv, o[h].y * inv);
        }
    }
}

static bool attn_decode_stream_ok(const AttnParams& p, int rows) {
    if (p.seq != 1 || (p.head_dim != 64 && p.head_dim != 128)) return false;
    if (rows < 16 && !(p.nsplit > 1 && p.part_o && p.part_m && p.part_l)) return false;
    const int G = p.n_heads / p.n_kv_heads;
    return G >= 1 && G <= AC_MAX_GROUP;
}

// Fewer sequences than fill the GPU: cut each into runs so that about 512 CTAs exist (a power of two,
// at most max_nsplit).
int attn_stream_splits(int rows, int n_heads, int n_kv_heads, int head_dim, int max_nsplit) {
    if (n_kv_heads < 1 || n_heads % n_kv_heads || (head_dim != 64 && head_dim != 128)) return 0;
    const int G = n_heads / n_kv_heads;
    if (G < 1 || G > AC_MAX_GROUP) return 0;
    int s = 1;
    while (2 * s <= max_nsplit && (long)rows * n_kv_heads * 2 * s <= 512) s *= 2;
    return s;
}

static int launch_attn_decode_stream(const AttnParams& p, int rows, cudaStream_t st) {
    const int G = p.n_heads / p.n_kv_heads, D = p.head_dim;
    const size_t smem = ((size_t)G * D + (size_t)G * 32 + (size_t)4 * AS_KEYS * (D + AC_PAD)) * sizeof(float);
    dim3 grid(p.n_kv_heads, rows, p.nsplit > 1 ? p.nsplit : 1);
    // two heads per warp when the group is even and leaves at least two warps
    if (G % 2 == 0 && G >= 4) {
        if (D == 64)
            attn_decode_stream_kernel<64, 2><<<grid, 16 * G, smem, st>>>(p);
        else
            attn_decode_stream_kernel<128, 2><<<grid, 16 * G, smem, st>>>(p);
    } else {
        if (D == 64)
            attn_decode_stream_kernel<64, 1><<<grid, 32 * G, smem, st>>>(p);
        else
            attn_decode_stream_kernel<128, 1><<<grid, 32 * G, smem, st>>>(p);
    }
    return launch_status();
}

static size_t attn_cluster_smem(int G, int D, int lcmax, int ns) {
    return ((size_t)G * D + round4(ns * 2 * G) + 2 * (size_t)lcmax * D +
            (size_t)(ac_warps_per_head(G) - 1) * G * (D + 4)) * sizeof(float);
}

// Whether a generation step of this shape takes the cluster kernel (the slices of one KV head fit a
// portable cluster and the staged cache slices fit shared memory).
bool attn_decode_cluster_ok(int n_heads, int n_kv_heads, int head_dim, int max_seq, int nsplit) {
    if (nsplit < 1 || nsplit > AC_MAX_SPLIT || n_kv_heads < 1 || n_heads % n_kv_heads) return false;
    if (head_dim != 64 && head_dim != 128) return false;
    const int G = n_heads / n_kv_heads;
    if (G > AC_MAX_GROUP || (G * head_dim) % (4 * nsplit)) return false;
    return attn_cluster_smem(G, head_dim, (max_seq + nsplit - 1) / nsplit, nsplit) <= 200 * 1024;
}

template <int D>
static int launch_attn_decode_cluster_d(const AttnDecodeParams& p, int batch, cudaStream_t st) {
    const int G = p.n_heads / p.n_kv_heads;
    const size_t smem = attn_cluster_smem(G, D, (p.max_seq + p.nsplit - 1) / p.nsplit, p.nsplit);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.n_kv_heads * p.nsplit, batch);
    cfg.blockDim = dim3(32 * G * ac_warps_per_head(G));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = p.nsplit;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_use_pdl ? 2 : 1;
    cudaError_t e;
    if (p.nsplit > 8) {  // beyond the portable cluster size: opt in once per device
        static PerDevice<bool> once;
        bool& allowed = once.here();
        if (!allowed) {
            RB_CUDA(cudaFuncSetAttribute(attn_decode_cluster_kernel<D, 16>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
            allowed = true;
        }
        e = cudaLaunchKernelEx(&cfg, attn_decode_cluster_kernel<D, 16>, p);
    } else {
        e = cudaLaunchKernelEx(&cfg, attn_decode_cluster_kernel<D, 8>, p);
    }
    if (e != cudaSuccess) {
        ++g_launch_count;
        return ROTOR_B200_ERR_CUDA;
    }
    return launch_status();
}

int launch_attn_decode_cluster(const AttnDecodeParams& p, int batch, cudaStream_t st) {
    if (!p.qkv_f || !p.attn_out || !attn_decode_cluster_ok(p.n_heads, p.n_kv_heads, p.head_dim, p.max_seq, p.nsplit))
        return ROTOR_B200_ERR_ARG;
    switch (p.head_dim) {
        case 64: return launch_attn_decode_cluster_d<64>(p, batch, st);
        case 128: return launch_attn_decode_cluster_d<128>(p, batch, st);
    }
    return ROTOR_B200_ERR_SHAPE;
}

int attn_decode_nsplit(int max_seq) {
    int n = max_seq / 128;
    return n < 8 ? 8 : (n > 32 ? 32 : n);
}

size_t attn_decode_part_floats(int batch, int n_heads, int head_dim, int max_seq) {
    return (size_t)batch * n_heads * attn_decode_nsplit(max_seq) * (head_dim + 2);
}

// Whether the current device can place one 16-CTA cluster of the cluster kernel with this much shared
// memory per CTA (asked of the occupancy calculator; nothing is launched).
template <int D>
static bool cluster16_placeable(int G, size_t smem) {
    if (cudaFuncSetAttribute(attn_decode_cluster_kernel<D, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(attn_decode_cluster_kernel<D, 16>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(16, 1);
    cfg.blockDim = dim3(32 * G * ac_warps_per_head(G));
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 16;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, attn_decode_cluster_kernel<D, 16>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return n >= 1;
}

// Slices per KV head for a model of this shape.  The cluster kernel keeps a slice of the cache in shared
// memory, so it wants as few slices as still fit: eight (a portable cluster) while a slice of max_seq / 8
// rows fits, sixteen (a 16-CTA cluster, when the device can place one) up to twice that; longer caches
// take the split kernel with one slice per 128 positions.
int attn_decode_nsplit_for(int n_heads, int n_kv_heads, int head_dim, int max_seq) {
    if (attn_decode_cluster_ok(n_heads, n_kv_heads, head_dim, max_seq, 8)) return 8;
    if (attn_decode_cluster_ok(n_heads, n_kv_heads, head_dim, max_seq, 16)) {
        const int G = n_heads / n_kv_heads;
        const size_t smem = attn_cluster_smem(G, head_dim, (max_seq + 15) / 16, 16);
        if (head_dim == 128 ? cluster16_placeable<128>(G, smem) : cluster16_placeable<64>(G, smem)) return 16;
    }
    return attn_decode_nsplit(max_seq);
}

template <int D>
static int launch_attn_decode_d(const AttnDecodeParams& p, int batch, cudaStream_t st) {
    const int G = p.n_heads / p.n_kv_heads;
    const int lcmax = (p.max_seq + p.nsplit - 1) / p.nsplit;
    const size_t smem = ((size_t)G * D + 2 * D + (size_t)G * lcmax + 64 + (size_t)p.n_heads * D +
                         2 * (size_t)p.n_heads * p.nsplit) * sizeof(float);
    if (smem > 200 * 1024) return ROTOR_B200_ERR_SHAPE;
    static PerDevice<size_t> once;
    size_t& configured = once.here();
    if (smem > 48 * 1024 && smem > configured) {
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
    RB_CUDA(cudaFuncSetAttribute(attn_decode_cluster_kernel<64, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    RB_CUDA(cudaFuncSetAttribute(attn_decode_cluster_kernel<128, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    RB_CUDA(cudaFuncSetAttribute(attn_decode_cluster_kernel<64, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    RB_CUDA(cudaFuncSetAttribute(attn_decode_cluster_kernel<128, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    RB_CUDA(cudaFuncSetAttribute(attn_decode_stream_kernel<128, 1>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared));
    RB_CUDA(cudaFuncSetAttribute(attn_decode_stream_kernel<128, 2>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared));
    RB_CUDA(cudaFuncSetAttribute(attn_decode_stream_kernel<64, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024));
    RB_CUDA(cudaFuncSetAttribute(attn_decode_stream_kernel<128, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024));
    RB_CUDA(cudaFuncSetAttribute(attn_decode_stream_kernel<64, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024));
    RB_CUDA(cudaFuncSetAttribute(attn_decode_stream_kernel<128, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024));
    RB_CUDA(cudaFuncSetAttribute(attn_decode_cluster_kernel<64, 8>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared));
    RB_CUDA(cudaFuncSetAttribute(attn_decode_cluster_kernel<128, 8>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared));
    RB_CUDA(cudaFuncSetAttribute(attn_decode_cluster_kernel<64, 16>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared));
    RB_CUDA(cudaFuncSetAttribute(attn_decode_cluster_kernel<128, 16>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared));
    if (int rc = configure_attn_prefill_t5()) return rc;
    return configure_attn_prefill_tc();
}

}  // namespace rb
