// Vector stages for many token rows (prompt prefill, batched generation steps): the stages of
// vecstage.cuh with the row held in registers.
//
// With thousands of rows the stages are pure HBM traffic (int32 accumulators or float rows in,
// residual stream in and out, int8 activations out); what matters is bytes in flight.  A CTA of 128,
// 512 or 1024 threads per row; a thread owns up to V groups of four consecutive elements and issues
// ALL of its 128-bit loads (accumulators of every term, residual stream, norm weights) before the
// first use.  In the prefetching variant a grid of resident CTAs walks the rows, and a thread copies
// its pieces of the next row into a private shared-memory area (cp.async) while the current row is
// reduced.  Sums of squares and absolute maxima are block reductions over register values (sharded
// rows hand this slice's statistics out and take the whole row's back in), and the quantiser writes
// packed int8 words straight to the activation buffer (leanstage.cuh).  Arithmetic and its
// association follow vec_stage_row, which this kernel replaces from RS_MIN_ROWS rows on.
#include <cstdlib>

#include "leanstage.cuh"
#include "model.cuh"

namespace rb {

constexpr int RS_THREADS = 128;
constexpr int RS_MIN_ROWS = 5;         // (fewer rows: the generation-step kernels or the shared-memory stage)
constexpr int RS_WIDE_THREADS = 512;
// With fewer rows than SMs every CTA runs its code once, from a cold instruction cache: the duration is
// the length of the unrolled code, so the widest rows take 1024 threads with half the groups each.
constexpr int RS_FEW_ROWS = 296;

__device__ __forceinline__ float4 rs_deq(const VecStageParams& p, size_t col0, int off, int g, const float (&sxv)[3],
                                         float wscale) {
    float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
    int4 a[3];
#pragma unroll
    for (int t = 0; t < 3; ++t)
        if (t < p.terms)
            a[t] = __ldcg(reinterpret_cast<const int4*>(p.acc.acc + (col0 + t) * p.acc.out + off) + g);
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

__device__ __forceinline__ float rs_gate(float gate, float up, int act) {
    if (act == ROTOR_B200_FFN_RELU2) {
        const float q = fmaxf(gate, 0.f);
        return q * q * up;
    }
    const float c = fminf(fmaxf(up, -20.f), 20.f);
    return gate * (c / (1.f + expf(-c)));
}

__device__ __forceinline__ void rs_cp16(void* smem, const void* gmem) {
    const unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(gmem) : "memory");
}

// The same dequantisation from this thread's staged pieces (PF kernels): piece q of group g is
// stage[q * n4 + g], q = term * halves + half.
__device__ __forceinline__ float4 rs_deq_staged(const int4* stage, int n4, int halves, int half, int terms, int g,
                                                const float (&sxv)[3], float wscale) {
    float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int t = 0; t < 3; ++t)
        if (t < terms) {
            const int4 a = stage[(size_t)(t * halves + half) * n4 + g];
            f.x += (float)a.x * sxv[t];
            f.y += (float)a.y * sxv[t];
            f.z += (float)a.z * sxv[t];
            f.w += (float)a.w * sxv[t];
        }
    return make_float4(f.x * wscale, f.y * wscale, f.z * wscale, f.w * wscale);
}

// Wide rows (V > 8) are capped at 128 registers so that four CTAs share an SM: with fewer, the
// reductions and the quantiser of one row leave the memory pipe idle.
// RESID: the stage adds to the residual stream (VS_OPROJ, VS_DOWN) and keeps a second register
// row for it; the other modes are compiled without it.
// TH: threads per row; 128 for rows up to 8192 elements, 512 for wider ones (XL FFN rows).
// PF: a CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ... and fetches the NEXT row's
// accumulators and residual with cp.async while it reduces, normalises and quantises the current
// one.  Every thread stages exactly the 16-byte pieces it will read itself, so the staging area
// needs no barrier: cp.async.wait_group by the owner is enough, and the next fetch may start
// as soon as the owner has the pieces in registers.  Accumulator modes only.
template <int V, bool RESID, int TH, bool PF>
__global__ void __launch_bounds__(TH, TH > 128 ? (V <= 4 ? 2 : 1) : (V > 8 ? 4 : 5))
    row_stage_kernel(const __grid_constant__ VecStageParams p, int rows) {
    __shared__ float scratch[64];
    extern __shared__ __align__(16) int4 rs_stage[];
    const int n = p.n, n4 = n >> 2, tid = threadIdx.x;
    const bool from_acc = p.mode == VS_OPROJ || p.mode == VS_FFN || p.mode == VS_DOWN || p.mode == VS_DEQ;
    const int halves = p.mode == VS_FFN ? 2 : 1;
    float* hdst = p.h_out ? p.h_out : p.h;
    float sxn[3] = {0.f, 0.f, 0.f};

    // PF: start the fetch of `row` (pieces into the staging area, scales into registers)
    auto fetch = [&](int row) {
        const size_t c0 = (size_t)row * p.terms;
        if (p.mode == VS_PLAIN) {  // one piece: the float row itself
#pragma unroll
            for (int j = 0; j < V; ++j) {
                const int g = tid + j * TH;
                if (g < n4) rs_cp16(rs_stage + g, reinterpret_cast<const int4*>(p.src + (size_t)row * n) + g);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            return;
        }
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const int g = tid + j * TH;
            if (g >= n4) continue;
            for (int t = 0; t < p.terms; ++t)
                for (int hf = 0; hf < halves; ++hf)
                    rs_cp16(rs_stage + (size_t)(t * halves + hf) * n4 + g,
                            reinterpret_cast<const int4*>(p.acc.acc + (c0 + t) * p.acc.out + (size_t)hf * n) + g);
            if (RESID)
                rs_cp16(rs_stage + (size_t)p.terms * halves * n4 + g,
                        reinterpret_cast<const int4*>(p.h + (size_t)row * n) + g);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
#pragma unroll
        for (int t = 0; t < 3; ++t)
            if (t < p.terms) sxn[t] = __ldcg(&p.sx_in[c0 + t]);
    };
    if (PF && (int)blockIdx.x < rows) fetch(blockIdx.x);

    for (int m = blockIdx.x; m < rows; m += gridDim.x) {
    const size_t ro = (size_t)m * n, col0 = (size_t)m * p.terms;
    float sxv[3] = {0.f, 0.f, 0.f};
    if (PF) {
#pragma unroll
        for (int t = 0; t < 3; ++t) sxv[t] = sxn[t];
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else if (from_acc) {
#pragma unroll
        for (int t = 0; t < 3; ++t)
            if (t < p.terms) sxv[t] = __ldcg(&p.sx_in[col0 + t]);
    }

    // ---- build the row: every load of the stage in flight together
    float4 v[V], aux[RESID ? V : 1];
#pragma unroll
    for (int j = 0; j < V; ++j) {
        const int g = tid + j * TH;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (RESID) aux[RESID ? j : 0] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (g >= n4) continue;
        if (PF && p.mode == VS_PLAIN) {
            const int4 r = rs_stage[g];
            v[j] = make_float4(__int_as_float(r.x), __int_as_float(r.y), __int_as_float(r.z), __int_as_float(r.w));
        } else if (PF) {
            float4 a = rs_deq_staged(rs_stage, n4, halves, 0, p.terms, g, sxv, p.wscale0);
            if (p.mode == VS_FFN) {
                const float4 b = rs_deq_staged(rs_stage, n4, halves, 1, p.terms, g, sxv, p.wscale1);
                a = make_float4(rs_gate(a.x, b.x, p.ffn_act), rs_gate(a.y, b.y, p.ffn_act),
                                rs_gate(a.z, b.z, p.ffn_act), rs_gate(a.w, b.w, p.ffn_act));
            }
            v[j] = a;
            if (RESID) {
                const int4 r = rs_stage[(size_t)p.terms * halves * n4 + g];
                aux[RESID ? j : 0] = make_float4(__int_as_float(r.x), __int_as_float(r.y), __int_as_float(r.z),
                                                 __int_as_float(r.w));
            }
        } else if (p.mode == VS_EMBED) {
            const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p.embed + (size_t)p.ids[m] * n) + g);
            v[j] = make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                               __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
        } else if (p.mode == VS_PLAIN) {
            v[j] = ldcg4(p.src + ro + 4 * g);
        } else {
            float4 a = rs_deq(p, col0, 0, g, sxv, p.wscale0);
            if (p.mode == VS_FFN) {  // gating right away: the up half is not kept
                const float4 b = rs_deq(p, col0, n, g, sxv, p.wscale1);
                a = make_float4(rs_gate(a.x, b.x, p.ffn_act), rs_gate(a.y, b.y, p.ffn_act),
                                rs_gate(a.z, b.z, p.ffn_act), rs_gate(a.w, b.w, p.ffn_act));
            }
            v[j] = a;
            if (RESID) aux[RESID ? j : 0] = ldcg4(p.h + ro + 4 * g);
        }
    }
    if (PF && m + (int)gridDim.x < rows) fetch(m + gridDim.x);  // the staged pieces are in registers now
    if constexpr (RESID) {
        if (p.mode == VS_OPROJ) {  // h += subnorm(row)
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < V; ++j) ss += sq4(v[j]);
            ss = block_sum(ss, scratch);
            const float inv = 1.0f / sqrtf(ss / (float)n + p.eps);
#pragma unroll
            for (int j = 0; j < V; ++j) {
                const int g = tid + j * TH;
                const float4 w0 = g < n4 ? ldg4(p.norm0 + 4 * g) : make_float4(0.f, 0.f, 0.f, 0.f);
                // (multiply, multiply, add: no fused multiply-add, like the shared-memory version)
                v[j].x = __fadd_rn(__fmul_rn(__fmul_rn(v[j].x, inv), w0.x), aux[j].x);
                v[j].y = __fadd_rn(__fmul_rn(__fmul_rn(v[j].y, inv), w0.y), aux[j].y);
                v[j].z = __fadd_rn(__fmul_rn(__fmul_rn(v[j].z, inv), w0.z), aux[j].z);
                v[j].w = __fadd_rn(__fmul_rn(__fmul_rn(v[j].w, inv), w0.w), aux[j].w);
            }
        } else {  // VS_DOWN: residual add
#pragma unroll
            for (int j = 0; j < V; ++j)
                v[j] = make_float4(v[j].x + aux[j].x, v[j].y + aux[j].y, v[j].z + aux[j].z, v[j].w + aux[j].w);
        }
    }
    if (p.mode == VS_OPROJ || p.mode == VS_DOWN || p.mode == VS_EMBED) {
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const int g = tid + j * TH;
            if (g < n4) *reinterpret_cast<float4*>(hdst + ro + 4 * g) = v[j];
        }
    }

    // ---- pre-norm of the consumer (its weights are fetched as they are applied: they come from L2
    // and holding them all would cost the registers that keep four rows per SM in flight)
    // (sharded rows: out_sumsq / out_absmax hand this slice's statistics to the caller, ext_sumsq / ext_absmax
    // bring the whole row's back; norm_n is then the whole row's width)
    if (p.out_sumsq) {
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < V; ++j) ss += sq4(v[j]);
        ss = block_sum(ss, scratch);
        if (tid == 0) p.out_sumsq[m] = ss;
    }
    if (p.norm1) {
        float ss = 0.f;
        if (p.ext_sumsq) {
            ss = __ldcg(p.ext_sumsq + m);
        } else {
#pragma unroll
            for (int j = 0; j < V; ++j) ss += sq4(v[j]);
            ss = block_sum(ss, scratch);
        }
        const float inv = 1.0f / sqrtf(ss / (float)(p.norm_n ? p.norm_n : n) + p.eps);
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const int g = tid + j * TH;
            const float4 w = g < n4 ? ldg4(p.norm1 + 4 * g) : make_float4(0.f, 0.f, 0.f, 0.f);
            v[j].x = v[j].x * inv * w.x;
            v[j].y = v[j].y * inv * w.y;
            v[j].z = v[j].z * inv * w.z;
            v[j].w = v[j].w * inv * w.w;
        }
    }
    if (p.out_absmax) {
        float mx = 0.f;
#pragma unroll
        for (int j = 0; j < V; ++j) mx = fmaxf(mx, amax4(v[j]));
        mx = block_max(mx, scratch);
        if (tid == 0) p.out_absmax[m] = mx;
    }
    if (p.y_out) {
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const int g = tid + j * TH;
            if (g < n4) *reinterpret_cast<float4*>(p.y_out + ro + 4 * g) = v[j];
        }
    }
    if (p.xq) {
        LeanStage q = {};
        q.n = n;
        q.kpad = p.kpad;
        q.terms = p.terms_out;
        int rk = 0;
        __syncthreads();  // readers of `scratch` in the reductions above are done
        lean_quantize<V>(q, v, scratch, p.xq + (size_t)m * p.terms_out * p.kpad, (size_t)p.kpad,
                         p.sx_out + (size_t)m * p.terms_out, p.xsum_out + (size_t)m * p.terms_out, rk, 0, false, nullptr,
                         p.ext_absmax ? p.ext_absmax + m : nullptr);
    }
    }  // rows of this CTA
}

// Whether the register-resident kernel takes this stage: enough rows, complete accumulators in
// one plane, 16-byte aligned rows, no sharded-row statistics.
bool row_stage_supported(const VecStageParams& p, int rows) {
    static const bool off = getenv("ROTOR_B200_NO_ROWSTAGE") != nullptr;  // comparison aid
    if (off || rows < RS_MIN_ROWS) return false;
    if (p.mode != VS_EMBED && p.mode != VS_PLAIN && p.mode != VS_OPROJ && p.mode != VS_FFN && p.mode != VS_DOWN &&
        p.mode != VS_DEQ)
        return false;
    const bool from_acc = p.mode == VS_OPROJ || p.mode == VS_FFN || p.mode == VS_DOWN || p.mode == VS_DEQ;
    if (from_acc && (p.acc.planes != 1 || p.acc.out % 4 || p.terms < 1 || p.terms > 3)) return false;
    const bool resid = p.mode == VS_OPROJ || p.mode == VS_DOWN;
    const int widest = resid ? 4 * 16 * RS_THREADS : 4 * 14 * RS_WIDE_THREADS;  // 8192, or 28672 without a residual row
    if (p.n % 4 || p.n > widest) return false;
    if (p.xq && (p.kpad > widest || p.terms_out < 1 || p.terms_out > 4)) return false;
    return true;
}

// Launches one instantiation.  Accumulator modes whose staging area fits run the prefetching
// variant on a grid of resident CTAs; everything else runs one CTA per row.
template <int V, bool RESID, int TH>
static int launch_one(const VecStageParams& p, int rows, cudaStream_t st) {
    const bool from_acc = p.mode == VS_OPROJ || p.mode == VS_FFN || p.mode == VS_DOWN || p.mode == VS_DEQ;
    const bool plain = p.mode == VS_PLAIN && !RESID;  // float rows in: one staged piece
    const size_t pieces = plain ? 1 : (size_t)p.terms * (p.mode == VS_FFN ? 2 : 1) + (RESID ? 1 : 0);
    const size_t smem = pieces * (size_t)p.n * sizeof(int);
    if ((from_acc || plain) && smem <= 200 * 1024) {
        auto* k = row_stage_kernel<V, RESID, TH, true>;
        static PerDevice<size_t> once;  // per instantiation and device
        static PerDevice<int> sm_counts;
        size_t& configured = once.here();
        int& sms = sm_counts.here();
        if (smem > configured) {
            RB_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            configured = smem;
        }
        if (!sms) {
            int dev = 0;
            RB_CUDA(cudaGetDevice(&dev));
            RB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        }
        int per_sm = 0;
        RB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k, TH, smem));
        if (per_sm >= 1) {
            const int grid = rows < per_sm * sms ? rows : per_sm * sms;
            k<<<grid, TH, smem, st>>>(p, rows);
            return launch_status();
        }
    }
    row_stage_kernel<V, RESID, TH, false><<<rows, TH, 0, st>>>(p, rows);
    return launch_status();
}

template <bool RESID>
static int launch_row_stage_v(const VecStageParams& p, int rows, int v, cudaStream_t st) {
    if (v <= 5) return launch_one<5, RESID, RS_THREADS>(p, rows, st);
    if (v <= 8) return launch_one<8, RESID, RS_THREADS>(p, rows, st);
    if constexpr (!RESID) {
        if (v <= 14) return launch_one<14, RESID, RS_THREADS>(p, rows, st);
        return launch_one<16, RESID, RS_THREADS>(p, rows, st);
    }
    return ROTOR_B200_ERR_SHAPE;  // wider rows with a residual take the 512-thread kernel (launch_row_stage)
}

int launch_row_stage(const VecStageParams& p, int rows, cudaStream_t st) {
    const int width = p.xq && p.kpad > p.n ? p.kpad : p.n;   // the quantiser also writes the zero padding
    if (width > 4 * 16 * RS_THREADS) {  // wide rows without a residual: 512 threads, up to 14 groups each
        if (rows <= RS_FEW_ROWS) return launch_one<7, false, 1024>(p, rows, st);  // see RS_FEW_ROWS
        return launch_one<14, false, RS_WIDE_THREADS>(p, rows, st);
    }
    const int v = (width / 4 + RS_THREADS - 1) / RS_THREADS;
    if (v > 8 && p.mode != VS_OPROJ && p.mode != VS_DOWN)
        // 4097..8192 elements without a residual (the 2B FFN row): four groups per thread at 512 threads
        // keep more warps per SM busy than fourteen groups at 128
        return launch_one<4, false, RS_WIDE_THREADS>(p, rows, st);
    if (p.mode == VS_OPROJ || p.mode == VS_DOWN) {
        // 4097..8192 elements with a residual row: sixteen groups per thread do not fit the registers of a
        // 128-thread CTA, four groups at 512 threads do
        if (v > 8) return launch_one<4, true, RS_WIDE_THREADS>(p, rows, st);
        return launch_row_stage_v<true>(p, rows, v, st);
    }
    return launch_row_stage_v<false>(p, rows, v, st);
}

}  // namespace rb
