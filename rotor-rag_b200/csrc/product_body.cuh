// Device body of the generation-step BitLinear product (see fused.cu): what runs before the
// programmatic-launch wait (tile ranges, the weight tiles on their way into shared memory or
// registers) and what runs after it (prologue, tile products, epilogue).
#pragma once
#include "gemv_core.cuh"
#include "leanstage.cuh"
#include "vecstage.cuh"
#include <type_traits>

namespace rb {

// 512 threads per CTA.  The shallow variant (small matrices: the CTA's whole share of the weights
// fits in shared memory) is held to 64 registers and FG_STAGE_MAX bytes of staged tiles so that two
// CTAs fit on an SM: the next kernel of the step becomes resident while this one runs and copies
// its tiles into shared memory (cp.async) before its wait returns, so the weight stream of a step
// overlaps the prologues and epilogues of the kernels before it.  The deep variant (large
// matrices) takes 128 registers and streams its tiles through a register pipeline.
constexpr int FG_THREADS = 512;
constexpr int FG_WARPS = FG_THREADS / 32;
constexpr int FG_U = 4;        // weight tiles in flight per warp
constexpr int FG_L2_AHEAD = 32;  // deep variant: further tiles per warp pulled into L2 before the wait
constexpr size_t FG_STAGE_MAX = 96 * 1024;  // shallow variant: most tile bytes a CTA stages
constexpr int FG_V = 4;        // float4 groups per thread in the register prologue: input width <= 8192
constexpr int FG_V_NARROW = 2; // shallow variant, stages that hold four arrays per group: width <= 4096

struct FusedGemvParams {
    const uint4* tiles;   // tiles of the (stacked) matrix
    int nkt;              // K tiles per row tile
    int units;            // row tiles per half (paired) or in all (plain)
    int halves;           // 2: rows u and units*16 + u form one output (gate/up); 1 otherwise
    int out;              // output rows per half
    int rows, cols;       // token rows, activation columns (= rows * st.terms)
    int upc;              // units per CTA (ceil)
    LeanStage st;
    float* y;             // [rows][out] float32 outputs
    float scale[3];       // per-tensor weight scales of up to three stacked row segments
    int seg1, seg2;       // first row of the second / third segment (plain); halves == 2: scale[0]=gate, [1]=up
    int ffn_act;
    // tensor parallel (row-parallel products): scalar exchange ring (size 0: none); with `part` set
    // the epilogue hands over exact int32 partial sums [rows][out] and the activation scales
    // instead of dequantised floats (one activation term only)
    XchScalarDev xs;
    int32_t* part;
    float* sx_out;
    // stand-alone product on activations that are quantised already (no vector stage): int8 columns
    // [cols][kpad] and their sums in, exact int32 sums [cols][out] out
    const int8_t* xq_in;
    const int32_t* xsum_in;
    int32_t* acc_out;
};

// Input rows wider than the register-resident prologue holds (4 * FG_V * FG_THREADS elements)
// are staged as float32 in shared memory instead; only the plain mode (optional norm, then
// quantise: the down projection's prologue) has such rows.
__host__ __device__ inline bool fused_wide(const LeanStage& st) { return st.n > 4 * FG_V * FG_THREADS; }
// The shallow variant keeps a plain stage (input and one norm weight per group) in FG_V groups per
// thread and every other stage in FG_V_NARROW; wider rows of those stages take the deep variant.
__host__ __device__ inline bool fused_shallow_fits(const LeanStage& st) {
    return st.n <= 4 * (st.mode == LM_PLAIN ? FG_V : FG_V_NARROW) * FG_THREADS;
}

// Bytes of weight tiles the largest CTA share holds (what the shallow variant stages).
inline size_t fused_stage_bytes(const FusedGemvParams& p) {
    return (size_t)p.upc * p.halves * p.nkt * TILE_BYTES;
}

// Shared memory one product needs; `staged`: the shallow variant, which keeps its tiles there.
inline size_t fused_smem(const FusedGemvParams& p, bool staged) {
    const size_t xs = round_up((size_t)p.cols * (p.nkt * TILE_K + XS_PAD), 16);
    const size_t aux = p.st.mode == LM_ATTN ? 2 * (size_t)p.st.n_heads * p.st.nsplit : 0;
    const size_t wide = fused_wide(p.st) ? (size_t)p.st.n : 0;
    const size_t fixed = xs + (size_t)p.upc * p.halves * 512 + round_up((64 + aux + wide) * sizeof(float), 16);
    return fixed + (staged ? fused_stage_bytes(p) : 0);
}

// Fills the parameter block of one product for a grid of `grid` CTAs.  out: output rows per
// half.  halves == 2: `tiles` holds the gate matrix followed by the up matrix (each `out`
// rows), y receives the gated product, scale = {gate, up}.  halves == 1: y receives the
// product scaled per row segment: rows < seg1 by scale[0], < seg2 by scale[1], the rest by
// scale[2].  Returns a status code.
inline int make_fused_params(FusedGemvParams& p, const void* tiles, size_t out, size_t in, int halves, int rows,
                             const LeanStage& stage, float* y, const float* scale, int seg1, int seg2, int ffn_act,
                             int grid) {
    p = {};
    p.tiles = (const uint4*)tiles;
    p.nkt = (int)(kpad_of(in) / TILE_K);
    p.units = (int)(opad_of(out) / TILE_ROWS);
    p.halves = halves;
    p.out = (int)out;
    p.rows = rows;
    p.cols = rows * stage.terms;
    p.st = stage;
    p.y = y;
    p.scale[0] = scale[0];
    p.scale[1] = scale[1];
    p.scale[2] = scale[2];
    p.seg1 = seg1;
    p.seg2 = seg2;
    p.ffn_act = ffn_act;
    if (p.cols < 1 || p.cols > 8 || stage.terms > 3 || halves < 1 || halves > 2) return ROTOR_B200_ERR_ARG;
    if (halves == 2 && out % TILE_ROWS) return ROTOR_B200_ERR_SHAPE;
    if (stage.n != (int)in || in % 4) return ROTOR_B200_ERR_SHAPE;
    if (fused_wide(stage) && stage.mode != LM_PLAIN) return ROTOR_B200_ERR_SHAPE;
    if (grid > p.units) grid = p.units;
    p.upc = (p.units + grid - 1) / grid;
    return ROTOR_B200_OK;
}

// Tile ranges of the calling CTA / warp and shared-memory carve-up.
struct ProductCtx {
    int8_t* xs;
    int* merge;
    float* scratch;
    float* aux;
    uint4* wt;  // staged tiles (shallow variant): [half][unit - u0][kt][32]
    int xs_stride, slots, u0, u1, w0, w1;
};

__device__ __forceinline__ ProductCtx product_ctx(const FusedGemvParams& p, unsigned char* smem_raw) {
    ProductCtx c;
    const int warp = threadIdx.x >> 5;
    const int kpad = p.nkt * TILE_K;
    c.xs_stride = kpad + XS_PAD;
    c.slots = p.upc * p.halves;
    c.xs = reinterpret_cast<int8_t*>(smem_raw);                                      // [cols][xs_stride]
    c.merge = reinterpret_cast<int*>(smem_raw + round_up((size_t)p.cols * c.xs_stride, 16));  // [slots][128]
    c.scratch = reinterpret_cast<float*>(c.merge + c.slots * 128);                   // [64]
    c.aux = c.scratch + 64;                                                          // attention merge weights,
                                                                                     // or the staged wide row
    const size_t auxn = p.st.mode == LM_ATTN ? 2 * (size_t)p.st.n_heads * p.st.nsplit : 0;
    c.wt = reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(c.scratch) +
                                    round_up((64 + auxn) * sizeof(float), 16));
    // units (row tiles / row-tile pairs) of this CTA, and the warp's share of their tiles
    // (32-bit arithmetic: units * gridDim.x stays far below 2^31)
    c.u0 = (int)((unsigned)p.units * blockIdx.x / gridDim.x);
    c.u1 = (int)((unsigned)p.units * (blockIdx.x + 1) / gridDim.x);
    // local tile index: deep variant ((u-u0)*halves + half)*nkt + kt, shallow (half*(u1-u0) + u-u0)*nkt + kt
    const int ntile = (c.u1 - c.u0) * p.halves * p.nkt;
    c.w0 = ntile * warp / FG_WARPS;
    c.w1 = ntile * (warp + 1) / FG_WARPS;
    return c;
}

// Shallow variant: copies the CTA's tiles into shared memory, one contiguous span per half
// (constants: may run before the activations this product consumes exist).  Completion:
// cp.async.wait_group 0 by every thread, then a CTA barrier.
__device__ __forceinline__ void product_stage(const FusedGemvParams& p, const ProductCtx& c) {
    const int count = (c.u1 - c.u0) * p.nkt * 32;  // 16-byte pieces per half
    for (int h = 0; h < p.halves; ++h) {
        const uint4* src = p.tiles + ((size_t)h * p.units + c.u0) * p.nkt * 32;
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(c.wt + (size_t)h * count);
        for (int i = threadIdx.x; i < count; i += FG_THREADS)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 16u * i), "l"(src + i) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}

// Deep variant: requests the warp's first FG_U weight tiles and pulls up to FG_L2_AHEAD more into L2
// (constants: may run before the activations this product consumes exist).
__device__ __forceinline__ void product_prefetch(const FusedGemvParams& p, const ProductCtx& c, uint4 (&wv)[FG_U]) {
    // one division for the first tile, the rest advance by counting
    const int lane = threadIdx.x & 31;
    int slot = c.w0 / p.nkt, kt = c.w0 - slot * p.nkt;
    auto slot_ptr = [&](int sl) {
        const int u = c.u0 + (p.halves == 2 ? sl >> 1 : sl), half = p.halves == 2 ? (sl & 1) : 0;
        return p.tiles + ((size_t)half * p.units + u) * p.nkt * 32 + lane;
    };
    const uint4* ptr = slot_ptr(slot) + (size_t)kt * 32;
    auto advance = [&]() {
        ptr += 32;
        if (++kt == p.nkt) {
            kt = 0;
            ptr = slot_ptr(++slot);
        }
    };
#pragma unroll
    for (int u = 0; u < FG_U; ++u)
        if (c.w0 + u < c.w1) {
            wv[u] = ld_stream_v4(ptr);
            advance();
        }
    const int end = min(c.w1, c.w0 + FG_U + FG_L2_AHEAD);
    for (int lt = c.w0 + FG_U; lt < end; ++lt) {  // four 128-byte lines per tile
        if ((threadIdx.x & 7) == 0) prefetch_l2(ptr);
        advance();
    }
}

// Prologue, tile products and epilogue.  All threads of the CTA must call; `wv` as left by
// product_prefetch for the same p.  Uses the CTA barrier.
// WIDE: the input row is staged in shared memory (see fused_wide).  DEEP: many weight tiles per warp
// (large matrices): the loop requests the following batch of tiles before multiplying the
// current one and tracks its position by counting; the shallow loop (a few tiles per warp, the
// latency-bound small matrices) keeps the shortest code path.
// TP: tensor-parallel hooks compiled in (scalar exchanges in the prologue, int32 partial output).
template <bool USE_MMA, int NCOL, bool WIDE = false, bool DEEP = false, bool TP = false>
__device__ __forceinline__ void product_run(const FusedGemvParams& p, const ProductCtx& c, uint4 (&wv)[FG_U],
                                            float* s_sx, int* s_xsum, TraceRec& tr) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    int8_t* xs = c.xs;
    int* merge = c.merge;
    float* scratch = c.scratch;
    float* aux = c.aux;
    const int xs_stride = c.xs_stride, u0 = c.u0, u1 = c.u1, w0 = c.w0, w1 = c.w1;

    // ---- prologue: activation rows -> int8 in shared memory
    const bool writer = blockIdx.x == 0;
    if (!WIDE && !TP && p.xq_in) {
        // already quantised: the columns are copied as they are
        const int k16 = p.nkt * (TILE_K / 16);  // 16-byte pieces per column
        for (int i = threadIdx.x; i < p.cols * k16; i += blockDim.x) {
            const int col = i / k16, o = i - col * k16;
            *reinterpret_cast<uint4*>(xs + (size_t)col * xs_stride + 16 * o) =
                __ldcg(reinterpret_cast<const uint4*>(p.xq_in + (size_t)col * p.nkt * TILE_K) + o);
        }
        if ((int)threadIdx.x < p.cols) s_xsum[threadIdx.x] = __ldcg(p.xsum_in + threadIdx.x);
    } else if constexpr (WIDE) {
        // Every pass walks the row in the same pattern (float4 number threadIdx.x + k * blockDim.x), so a
        // thread only ever touches its own elements and the passes need no barrier beyond the reductions'.
        // Loads are issued WB at a time: one L2 round trip per batch instead of one per element group.
        constexpr int WB = 7;
        float* row = aux;  // [n] float32
        const int n = p.st.n, step = blockDim.x * 4;
        const XchScalarDev* x = (TP && p.xs.size) ? &p.xs : nullptr;
        for (int m = 0; m < p.rows; ++m) {
            const float* src = p.st.y + (size_t)m * n;
            float ss = 0.f, mx = 0.f;
            for (int i0 = threadIdx.x * 4; i0 < n; i0 += step * WB) {
                float4 r[WB];
#pragma unroll
                for (int u = 0; u < WB; ++u)
                    if (i0 + u * step < n) r[u] = ldcg4(src + i0 + u * step);
#pragma unroll
                for (int u = 0; u < WB; ++u)
                    if (i0 + u * step < n) {
                        *reinterpret_cast<float4*>(row + i0 + u * step) = r[u];
                        ss += r[u].x * r[u].x + r[u].y * r[u].y + r[u].z * r[u].z + r[u].w * r[u].w;
                        mx = fmaxf(mx, amax4(r[u]));
                    }
            }
            if (p.st.norm1) {
                float4 wn[WB];  // first batch of norm weights in flight across the reduction
#pragma unroll
                for (int u = 0; u < WB; ++u) {
                    const int i = threadIdx.x * 4 + u * step;
                    if (i < n) wn[u] = __ldg(reinterpret_cast<const float4*>(p.st.norm1 + i));
                }
                ss = block_sum(ss, scratch);
                if (x && p.st.xi_sum) ss = xch_scalar(*x, p.st.xi_sum - 1, m, ss, false, writer, scratch);
                const float inv = 1.0f / sqrtf(ss / (float)(p.st.norm_n ? p.st.norm_n : n) + p.st.eps);
                mx = 0.f;
                for (int i0 = threadIdx.x * 4; i0 < n; i0 += step * WB) {
                    if (i0 != (int)threadIdx.x * 4) {
#pragma unroll
                        for (int u = 0; u < WB; ++u)
                            if (i0 + u * step < n) wn[u] = __ldg(reinterpret_cast<const float4*>(p.st.norm1 + i0 + u * step));
                    }
#pragma unroll
                    for (int u = 0; u < WB; ++u)
                        if (i0 + u * step < n) {
                            float4* rp = reinterpret_cast<float4*>(row + i0 + u * step);
                            float4 v = *rp;
                            v.x = v.x * inv * wn[u].x;
                            v.y = v.y * inv * wn[u].y;
                            v.z = v.z * inv * wn[u].z;
                            v.w = v.w * inv * wn[u].w;
                            *rp = v;
                            mx = fmaxf(mx, amax4(v));
                        }
                }
            }
            int8_t* xq = xs + (size_t)m * p.st.terms * xs_stride;
            for (int t = 0; t < p.st.terms; ++t) {
                if (t > 0) {
                    mx = 0.f;
                    for (int i = threadIdx.x * 4; i < n; i += step) mx = fmaxf(mx, amax4(*reinterpret_cast<float4*>(row + i)));
                }
                if (threadIdx.x == 0) s_xsum[m * p.st.terms + t] = 0;  // ordered before the atomics by the reduction's barrier
                mx = block_max(mx, scratch);
                if (t == 0 && x && p.st.xi_max) mx = xch_scalar(*x, p.st.xi_max - 1, m, mx, true, writer, scratch);
                const float s = mx > 0.f ? __fdiv_rn(mx, 127.f) : 1.f;
                const float rs = __fdiv_rn(1.0f, s);
                const bool resid = t + 1 < p.st.terms;
                int lsum = 0;
                for (int i = threadIdx.x * 4; i < p.st.kpad; i += step) {
                    int packed = 0;
                    if (i < n) {
                        float4* rp = reinterpret_cast<float4*>(row + i);
                        float4 v = *rp;
                        if (resid) {
                            packed = quant4_pack<true>(v, s, rs, lsum);
                            *rp = v;
                        } else {
                            packed = quant4_pack<false>(v, s, rs, lsum);
                        }
                    }
                    *reinterpret_cast<int*>(xq + (size_t)t * xs_stride + i) = packed;
                }
                // read after the prologue's closing barrier: warps add their shares with a shared-memory atomic
                lsum = warp_sum_i(lsum);
                if ((threadIdx.x & 31) == 0 && lsum) atomicAdd(&s_xsum[m * p.st.terms + t], lsum);
                if (threadIdx.x == 0) s_sx[m * p.st.terms + t] = s;
            }
        }
    } else {
        const XchScalarDev* x = (TP && p.xs.size) ? &p.xs : nullptr;
        int rk = 0;
        auto rows = [&](auto vtag, auto plain_tag) {
            constexpr int V = decltype(vtag)::value;
            constexpr bool PLAIN = decltype(plain_tag)::value;
            constexpr bool ONE = NCOL == 1 && !USE_MMA;  // one activation column: one row of one term
            const int nrows = ONE ? 1 : p.rows, terms = ONE ? 1 : p.st.terms;
            for (int m = 0; m < nrows; ++m) {
                float4 v[V];
                lean_row<V, PLAIN>(p.st, m, v, scratch, aux, writer, rk, x);
                RB_STAMP(tr, 6);
                lean_quantize<V, ONE>(p.st, v, scratch, xs + (size_t)m * terms * xs_stride, (size_t)xs_stride,
                                      s_sx + m * terms, s_xsum + m * terms, rk, m, writer, x);
            }
        };
        if constexpr (DEEP) {
            rows(std::integral_constant<int, FG_V>(), std::false_type());
        } else {
            if (p.st.mode == LM_PLAIN)
                rows(std::integral_constant<int, FG_V>(), std::true_type());
            else
                rows(std::integral_constant<int, FG_V_NARROW>(), std::false_type());
        }
    }
    if constexpr (!DEEP) asm volatile("cp.async.wait_group 0;" ::: "memory");  // this thread's staged tiles
    __syncthreads();
    RB_STAMP(tr, 3);

    // ---- integer tile products over the warp's range
    int accm[4][4];
    int accd[2][4][NCOL];
    auto clear = [&]() {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int r = 0; r < 4; ++r) accm[j][r] = 0;
#pragma unroll
            for (int c = 0; c < NCOL; ++c) accd[0][j][c] = accd[1][j][c] = 0;
        }
    };
    auto flush = [&](int slot) {  // exact rescale of the per-bit-pair sums, then into the slot
        int* dst = merge + slot * 128;
        if constexpr (USE_MMA) {
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int v = accm[0][r] + (accm[1][r] >> 2) + (accm[2][r] >> 4) + (accm[3][r] >> 6);
                atomicAdd(dst + (g + 8 * (r >> 1)) * 8 + 2 * t + (r & 1), v);
            }
        } else {
#pragma unroll
            for (int rh = 0; rh < 2; ++rh)
#pragma unroll
                for (int c = 0; c < NCOL; ++c) {
                    int v = accd[rh][0][c] + (accd[rh][1][c] >> 2) + (accd[rh][2][c] >> 4) + (accd[rh][3][c] >> 6);
                    v += __shfl_xor_sync(0xffffffffu, v, 1);
                    v += __shfl_xor_sync(0xffffffffu, v, 2);
                    if (t == 0) atomicAdd(dst + (g + 8 * rh) * 8 + c, v);
                }
        }
    };
    clear();
    int cur = -1;
    if constexpr (DEEP) {
        // positions advance by counting, not by dividing: `slot`/`kt` is the tile being multiplied,
        // `pslot`/`pkt`/`pptr` the tile being requested (FG_U tiles ahead)
        auto slot_ptr = [&](int sl) {
            const int u = u0 + (p.halves == 2 ? sl >> 1 : sl), half = p.halves == 2 ? (sl & 1) : 0;
            return p.tiles + ((size_t)half * p.units + u) * p.nkt * 32 + lane;
        };
        int slot = w0 / p.nkt, kt = w0 - slot * p.nkt;
        int pslot = (w0 + FG_U) / p.nkt, pkt = (w0 + FG_U) - pslot * p.nkt;
        const uint4* pptr = slot_ptr(pslot) + (size_t)pkt * 32;
        int pnext = w0 + FG_U;  // index of the next tile to request
        // Requests FG_U tiles starting at tile index pnext.  Whole batch inside one row tile and inside
        // the warp's range: four loads at constant offsets, no per-tile checks.
        auto request = [&](uint4 (&dst)[FG_U]) {
            if (pnext + FG_U <= w1 && pkt + FG_U <= p.nkt) {
#pragma unroll
                for (int u = 0; u < FG_U; ++u) dst[u] = ld_stream_v4(pptr + 32 * u);
                pptr += 32 * FG_U;
                pkt += FG_U;
                if (pkt == p.nkt) {
                    pkt = 0;
                    pptr = slot_ptr(++pslot);
                }
            } else {
#pragma unroll
                for (int u = 0; u < FG_U; ++u)
                    if (pnext + u < w1) {
                        dst[u] = ld_stream_v4(pptr);
                        pptr += 32;
                        if (++pkt == p.nkt) {
                            pkt = 0;
                            pptr = slot_ptr(++pslot);
                        }
                    }
            }
            pnext += FG_U;
        };
        // Multiplies FG_U tiles starting at tile index `base`.
        auto multiply = [&](const uint4 (&src)[FG_U], int base) {
            if (base + FG_U <= w1 && kt + FG_U <= p.nkt && slot == cur) {
#pragma unroll
                for (int u = 0; u < FG_U; ++u) {
                    const uint32_t pw[4] = {src[u].x, src[u].y, src[u].z, src[u].w};
                    tile_mac<USE_MMA, NCOL>(pw, xs, xs_stride, (kt + u) * TILE_K + 32 * t, g, p.cols, accm, accd);
                }
                kt += FG_U;
                if (kt == p.nkt) {
                    kt = 0;
                    ++slot;
                }
            } else {
#pragma unroll
                for (int u = 0; u < FG_U; ++u) {
                    if (base + u < w1) {
                        if (slot != cur) {  // warp-uniform
                            if (cur >= 0) flush(cur);
                            clear();
                            cur = slot;
                        }
                        const uint32_t pw[4] = {src[u].x, src[u].y, src[u].z, src[u].w};
                        tile_mac<USE_MMA, NCOL>(pw, xs, xs_stride, kt * TILE_K + 32 * t, g, p.cols, accm, accd);
                        if (++kt == p.nkt) {
                            kt = 0;
                            ++slot;
                        }
                    }
                }
            }
        };
        // two register sets alternate: one is multiplied while the other is in flight
        uint4 wn[FG_U];
        for (int base = w0; base < w1; base += 2 * FG_U) {
            request(wn);
            multiply(wv, base);
            if (base + FG_U < w1) {
                request(wv);
                multiply(wn, base + FG_U);
            }
        }
    } else {
        // tiles come out of shared memory in local order; (slot, kt) advance by counting
        int slot = w0 / p.nkt, kt = w0 - slot * p.nkt;
        const uint4* wp = c.wt + (size_t)w0 * 32 + lane;
#pragma unroll 2
        for (int lt = w0; lt < w1; ++lt) {
            const uint4 w4 = *wp;
            wp += 32;
            const uint32_t pw[4] = {w4.x, w4.y, w4.z, w4.w};
            tile_mac<USE_MMA, NCOL>(pw, xs, xs_stride, kt * TILE_K + 32 * t, g, p.cols, accm, accd);
            cur = slot;
            if (++kt == p.nkt) {  // warp-uniform: the row tile is complete
                flush(slot);
                clear();
                kt = 0;
                ++slot;
                cur = -1;
            }
        }
    }
    RB_STAMP(tr, 7);
    if (cur >= 0) flush(cur);
    __syncthreads();
    RB_STAMP(tr, 4);

    // ---- epilogue: the CTA's rows are complete: remove the +1 code offset, dequantise, write
    if (!WIDE && !TP && p.acc_out) {  // stand-alone product: exact integer sums, column major
        for (int e = threadIdx.x; e < (u1 - u0) * 16 * p.cols; e += blockDim.x) {
            const int q = e / p.cols, col = e - q * p.cols;
            const int rl = q & 15, lu = q >> 4;
            const int orow = (u0 + lu) * TILE_ROWS + rl;
            if (orow < p.out) p.acc_out[(size_t)col * p.out + orow] = merge[lu * 128 + rl * 8 + col] - s_xsum[col];
        }
        return;
    }
    constexpr bool ONE = NCOL == 1 && !USE_MMA;
    const int T = ONE ? 1 : p.st.terms, nrows = ONE ? 1 : p.rows;
    for (int e = threadIdx.x; e < (u1 - u0) * 16 * nrows; e += blockDim.x) {
        int m = 0, q = e;
        if (!ONE) {
            q = e / nrows;
            m = e - q * nrows;
        }
        const int rl = q & 15, lu = q >> 4;
        const int orow = (u0 + lu) * TILE_ROWS + rl;
        if (orow >= p.out) continue;
        if (TP && p.part) {  // exact partial sum of this rank's columns; summed across ranks and dequantised later
            p.part[(size_t)m * p.out + orow] = merge[lu * 128 + rl * 8 + m] - s_xsum[m];  // halves == 1
            continue;
        }
        // (two named values, not an array indexed by the loop: that would live in local memory, whose
        // first touch costs an L2 round trip at the very end of the kernel)
        auto deq = [&](int half) {
            const int slot = DEEP ? lu * p.halves + half : half * (u1 - u0) + lu;
            const int* src = merge + slot * 128 + rl * 8 + m * T;
            float f = 0.f;
            for (int tt = 0; tt < T; ++tt) f += (float)(src[tt] - s_xsum[m * T + tt]) * s_sx[m * T + tt];
            return f;
        };
        const float val0 = deq(0), val1 = p.halves == 2 ? deq(1) : 0.f;
        float r;
        if (p.halves == 2) {
            const float gt = val0 * p.scale[0], up = val1 * p.scale[1];
            if (p.ffn_act == ROTOR_B200_FFN_RELU2) {
                const float q2 = fmaxf(gt, 0.f);
                r = q2 * q2 * up;
            } else {
                const float c2 = fminf(fmaxf(up, -20.f), 20.f);
                r = gt * (c2 / (1.f + expf(-c2)));
            }
        } else {
            r = val0 * (orow < p.seg1 ? p.scale[0] : (orow < p.seg2 ? p.scale[1] : p.scale[2]));
        }
        p.y[(size_t)m * p.out + orow] = r;
    }
    if (TP && p.part && writer && (int)threadIdx.x < p.rows) p.sx_out[threadIdx.x] = s_sx[threadIdx.x];
}

}  // namespace rb
