// Ternary BitLinear integer core for prompt prefill on the fifth-generation tensor cores:
// acc[c][o] = sum_k xq[c][k] * w[o][k], exact int32, for hundreds to thousands of
// activation columns c (tokens).
//
// CTA tile: 256 tokens x 256 weight rows, K walked 128 at a time through a 3-stage ring of
// shared-memory operand tiles.  tcgen05.mma.kind::i8 (M = 128 tokens, N = 256 weight rows, K = 32 per
// instruction) accumulates into tensor memory: two 128-lane int32 accumulators of N columns (all 512
// TMEM columns of the SM).  A token half without tokens is skipped.  Per stage:
//   * the token operand (2 x 128 rows of 128 int8) arrives by TMA
//     (cp.async.bulk.tensor.2d, 128-byte swizzle, rows past the last token zero filled),
//   * eight decoder warps turn the stage's packed weight tiles (2 bits per weight; 16 tiles = 8 KB)
//     into bytes (32 KB) in the same swizzled K-major layout: a lane's 128-bit tile word holds, per
//     row, 32 consecutive K positions, i.e. two 16-byte chunks of the operand row,
//   * one thread issues the eight MMAs and commits them to the stage's "empty" barrier.
// The weight operand holds the codes w + 1 (0, 1, 2) as unsigned bytes against signed activations;
// the read-back subtracts the token's activation sum.  After the last stage the decoder warps read
// the accumulators back (tcgen05.ld 32 lanes x 32 columns: a lane holds 32 consecutive outputs of
// one token) and pass them through a per-warp shared-memory block so that they leave as whole
// 128-byte rows.  Read-back variants: plain int32 sums; GATED (gate/up product: activation and
// product in the read-back, float32 out); QKV (dequantise, rotary, cache append).  When 256-row tiles
// do not cover the GPU the K range is split over blockIdx.z and the partial sums are added with
// integer atomics (64-row tiles remain for products too short to split).
// Every wait is bounded by a cycle count; a wait that runs out records a code in the library status
// word, the CTA stops issuing work, lets its copies land, frees its tensor memory and returns.
#include <cuda.h>

#include <cstdlib>

#include "gemv_core.cuh"
#include "model.cuh"

RB_TRACE_DEFINE(rotor_b200_trace_read_gemm5)

namespace rb {

// Tokens per CTA is a template argument too: 256 (two MMA M halves, one CTA per SM: all 512
// tensor-memory columns) or 128 (one half, 256 columns and a two-stage ring, so that TWO CTAs share
// an SM and the accumulator read-back of one overlaps the MMAs of the other).
// Decoder warps (they also read the accumulators back), then one TMA + TMEM warp and one MMA warp.
// Eight decoders for 256-row tiles: a lone warp per scheduler issues about one instruction every
// four cycles, and at four warps the decode of a K step (about 550 instructions per warp) took
// twice as long as its eight MMAs; two warps per scheduler hide each other's latencies.
// Weight rows per CTA (MMA N) is a template argument: 256 for large grids; 64 when 256-row tiles
// would leave most SMs without a CTA (few tokens and a narrow output, e.g. 64 tokens x 8192 rows).
template <int ROWS, int TOK = 256>
struct T5Cfg {
    static constexpr int A_BYTES = TOK * TILE_K;                   // token operand per stage
    static constexpr int B_BYTES = ROWS * TILE_K;                  // weight operand per stage
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    // ring depth and decoder look-ahead: with 64-row tiles a stage is only four short MMAs, so the
    // copy and weight-load latencies need more stages in flight to stay hidden
    static constexpr int STAGES = TOK == 128 ? 2 : (ROWS >= 256 ? 3 : 5);
    static constexpr int PREFETCH = ROWS >= 256 ? 2 : 6;           // K steps of weight tiles requested ahead
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024;       // + slack to align the ring to 1024 bytes
    static constexpr int TMEM_COLS = (TOK / 128) * ROWS < 32 ? 32 : (TOK / 128) * ROWS;  // one accumulator of ROWS columns per token half
    static constexpr int DECODERS = ROWS >= 256 ? 8 : 4;           // decoder warps
    static constexpr int THREADS = (DECODERS + 2) * 32;
    static constexpr int TILES_PER_WARP = ROWS / TILE_ROWS / DECODERS;  // row tiles each decoder warp handles
};
constexpr long long T5_SPIN_CYCLES = 400000000LL;  // about 0.2 s

struct Tc5Params {
    const uint4* tiles;
    const int32_t* xsum;  // [ncols] sum of each token's int8 activations (removes the +1 of the weight codes)
    int32_t* acc;       // [ncols][out]
    unsigned* status;
    int out, nrt, nkt, ncols;
    int kt_per_split;   // > 0: CTA z takes K steps [z kt_per_split, +kt_per_split) and ADDS its sums into zeroed acc
    // gated epilogue (GATED kernel): `tiles` holds the gate matrix followed by the up matrix (ff rows
    // each); a CTA takes 128 gate rows and the matching 128 up rows, and writes
    // gated[token][channel] = act(gate * sx[token] * sg) * (up * sx[token] * su) as float32 instead
    // of two int32 accumulators per channel
    float* gated;       // [ncols][ff]
    const float* sx;    // [ncols] activation scales (one term per token)
    float sg, su;
    int ff, ffn_act;
    // q/k/v epilogue (QKV kernel, head_dim 128): `tiles` is the stacked [q; k; v] matrix; the read-back
    // dequantises (sx[token] * sq / sk / sv), rotates q and k (half-split pairs i, i + 64) and writes q rows
    // and the K / V cache rows of the token's position; no int32 accumulator leaves the kernel
    int dq, dkv, seq, max_seq;
    const int* past_len;   // [batch] cached length per sequence
    const float2* rope;    // [max_seq][64] (cos, sin), or null
    float* qout;           // [ncols][dq]
    float* k_cache;        // [batch][dkv / 128][max_seq][128]
    float* v_cache;
    float sq, sk, sv;
};

__device__ __forceinline__ bool t5_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, unsigned* status,
                                        unsigned code) {
    long long t0 = 0;
    for (int it = 0;; ++it) {
        uint32_t ok;
        asm volatile(
            "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
        if (*abort_flag) return false;
        if (it == 0) t0 = clock64();
        if (clock64() - t0 > T5_SPIN_CYCLES) {
            *abort_flag = 1;
            atomicExch(status, code);
            return false;
        }
    }
}

// Shared-memory matrix descriptor, K-major, 128-byte swizzle: 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t t5_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3fffu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
           (2ull << 61);
}

__device__ __forceinline__ void t5_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
}

// Read-back store of a warp's 32 tokens x 32 values (lane = token after tcgen05.ld) as whole 128-byte
// rows: through a per-warp shared-memory block (32 rows of 144 bytes: conflict-free both ways) so that
// one store instruction covers four tokens' rows (four lines) instead of one 16-byte piece of 32
// different lines.  dst0: address of token tok_base's first value; tokens at and beyond ntok are skipped.
constexpr uint32_t T5_XPOSE_BYTES = 32 * 144;
__device__ __forceinline__ void t5_store_rows(uint32_t stage, const uint32_t (&v)[32], void* dst0, size_t row_bytes,
                                              int tok_base, int ntok, int lane) {
#pragma unroll
    for (int q = 0; q < 8; ++q)
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(stage + (uint32_t)lane * 144u + 16u * q),
                     "r"(v[4 * q]), "r"(v[4 * q + 1]), "r"(v[4 * q + 2]), "r"(v[4 * q + 3])
                     : "memory");
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int tl = 4 * i + (lane >> 3);
        uint4 w;
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w)
                     : "r"(stage + (uint32_t)tl * 144u + 16u * (lane & 7)));
        if (tok_base + tl < ntok)
            *reinterpret_cast<uint4*>(static_cast<unsigned char*>(dst0) + (size_t)tl * row_bytes + 16 * (lane & 7)) = w;
    }
    __syncwarp();  // the block is rewritten by the warp's next item
}

// The same with a destination per token: dst_of(tl) is the address of token tok_base + tl's 128 bytes
// (null = skip).
template <typename F>
__device__ __forceinline__ void t5_store_rows_to(uint32_t stage, const uint32_t (&v)[32], int lane, F dst_of) {
#pragma unroll
    for (int q = 0; q < 8; ++q)
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(stage + (uint32_t)lane * 144u + 16u * q),
                     "r"(v[4 * q]), "r"(v[4 * q + 1]), "r"(v[4 * q + 2]), "r"(v[4 * q + 3])
                     : "memory");
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int tl = 4 * i + (lane >> 3);
        uint4 w;
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w)
                     : "r"(stage + (uint32_t)tl * 144u + 16u * (lane & 7)));
        unsigned char* d = static_cast<unsigned char*>(dst_of(tl));
        if (d) *reinterpret_cast<uint4*>(d + 16 * (lane & 7)) = w;
    }
    __syncwarp();
}

template <int ROWS, int T5_TOK = 256, bool GATED = false, bool QKV = false>
__global__ void __launch_bounds__(T5Cfg<ROWS, T5_TOK>::THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ Tc5Params p) {
    using Cfg = T5Cfg<ROWS, T5_TOK>;
    constexpr int T5_A_BYTES = Cfg::A_BYTES, A_HALF = 128 * TILE_K;
    constexpr int T5_ROWS = ROWS, T5_STAGE_BYTES = Cfg::STAGE_BYTES, TPW = Cfg::TILES_PER_WARP;
    constexpr int T5_STAGES = Cfg::STAGES, PF = Cfg::PREFETCH, NDW = Cfg::DECODERS;
#ifdef RB_TRACE
    const unsigned long long t_entry = gtime();
#endif
    extern __shared__ unsigned char t5_raw[];
    __shared__ __align__(8) unsigned long long s_full[T5_STAGES], s_empty[T5_STAGES], s_accf;
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    const uint32_t ring = (smem_u32(t5_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tok0 = blockIdx.x * T5_TOK, rt0 = blockIdx.y * (T5_ROWS / TILE_ROWS);
    const int nhalf = (T5_TOK > 128 && p.ncols - tok0 > 128) ? 2 : 1;  // token halves of this CTA that hold any token
    // K steps of this CTA: all of them, or its share when the K range is split over blockIdx.z.  Loops
    // below count local steps 0 .. nk-1; ktb + step is the position in the matrix.
    const int ktb = p.kt_per_split ? (int)blockIdx.z * p.kt_per_split : 0;
    const int nk = p.kt_per_split ? min(p.kt_per_split, p.nkt - ktb) : p.nkt;
    volatile int* abort_flag = &s_abort;

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < T5_STAGES; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&s_full[s])), "r"(NDW * 32 + 1));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&s_empty[s])), "r"(1));
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&s_accf)), "r"(1));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == NDW) {  // the whole warp allocates the accumulators' tensor-memory columns (one CTA per SM)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)),
                     "r"(Cfg::TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    if (warp < NDW) {
        // ---------------- weight decoders: warp w owns row tiles TPW w .. TPW w + TPW - 1 of the CTA's
        const int g = lane >> 2, t = lane & 3;
        // weight tiles are requested PF K steps ahead of their decode, so that the L2 / HBM latency
        // hides behind the decode of the step in between and the wait for a free stage
        uint4 wv[PF][TPW];
        auto fetch = [&](int kt, uint4 (&dst)[TPW]) {
#pragma unroll
            for (int u = 0; u < TPW; ++u) {
                int rt = rt0 + warp * TPW + u;
                if constexpr (GATED) {
                    // operand rows 0-127: gate row tiles 8 blockIdx.y ..; rows 128-255: the same channels of the up matrix
                    const int i = warp * TPW + u, ch_rt = (int)blockIdx.y * 8 + (i & 7), ff_rt = p.ff / TILE_ROWS;
                    rt = ch_rt < ff_rt ? (i < 8 ? ch_rt : ff_rt + ch_rt) : p.nrt;  // past the last channel: zero weights
                }
                dst[u] = (rt < p.nrt && kt < nk)
                             ? ld_stream_v4(p.tiles + ((size_t)rt * p.nkt + ktb + kt) * 32 + lane)
                             : make_uint4(0x55555555u, 0x55555555u, 0x55555555u, 0x55555555u);
            }
        };
#pragma unroll
        for (int par = 0; par < PF; ++par) fetch(par, wv[par]);
#ifdef RB_TRACE
        TraceRec trd = {};
        const bool tracedd = blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0;
        unsigned long long tld = gtime(), t0d = tld;
#endif
        for (int kt2 = 0; kt2 < nk; kt2 += PF) {
#pragma unroll
          for (int par = 0; par < PF; ++par) {
            const int kt = kt2 + par;
            if (kt >= nk) break;
            const int s = kt % T5_STAGES;
            if (!t5_wait(smem_u32(&s_empty[s]), ((kt / T5_STAGES) & 1) ^ 1, abort_flag, p.status, 0x7c000001u)) {
                kt2 = nk;  // leave both loops
                break;
            }
#ifdef RB_TRACE
            if (tracedd) { const unsigned long long n_ = gtime(); trd.t[0] += n_ - tld; tld = n_; }
#endif
            const uint32_t bbase = ring + s * T5_STAGE_BYTES + T5_A_BYTES;
#pragma unroll
            for (int u = 0; u < TPW; ++u) {
                const uint32_t pw[4] = {wv[par][u].x, wv[par][u].y, wv[par][u].z, wv[par][u].w};
#pragma unroll
                for (int rh = 0; rh < 2; ++rh) {
                    // operand row R = 16 (TPW warp + u) + g + 8 rh; R % 8 == g; K bytes [32 t, 32 t + 32)
                    const uint32_t row = bbase + (uint32_t)((warp * TPW + u) * 2 + rh) * 1024u + (uint32_t)g * 128u;
                    const uint32_t lo = pw[rh], hi = pw[rh + 2];
#pragma unroll
                    for (int c = 0; c < 2; ++c) {  // 16-byte chunk 2 t + c holds bit pairs 2 c and 2 c + 1
                        // the operand bytes are the codes w + 1 themselves (unsigned operand); the read-back
                        // subtracts the token's activation sum
                        const uint32_t a0 = (lo >> (4 * c)) & 0x03030303u;
                        const uint32_t a1 = (hi >> (4 * c)) & 0x03030303u;
                        const uint32_t a2 = (lo >> (4 * c + 2)) & 0x03030303u;
                        const uint32_t a3 = (hi >> (4 * c + 2)) & 0x03030303u;
                        const uint32_t dst = row + (uint32_t)(((2 * t + c) ^ g) << 4);
                        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(a0), "r"(a1), "r"(a2),
                                     "r"(a3)
                                     : "memory");
                    }
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> tensor-core reads
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&s_full[s])) : "memory");
            fetch(kt + PF, wv[par]);
#ifdef RB_TRACE
            if (tracedd) { const unsigned long long n_ = gtime(); trd.t[1] += n_ - tld; tld = n_; }
#endif
          }
        }
#ifdef RB_TRACE
        if (tracedd) {
            trd.t[2] = gtime() - t0d;
            trd.t[3] = t0d - t_entry;  // kernel entry -> first K step
            trd.t[7] = (unsigned long long)p.nkt;
            tld = gtime();
        }
#endif
        // ---------------- epilogue: lane = token, 32 columns (weight rows) per load
        // (warp-uniform decision: the tensor-memory loads below are warp-wide instructions)
        const bool acc_ok = !*abort_flag && t5_wait(smem_u32(&s_accf), 0, abort_flag, p.status, 0x7c000002u);
#ifdef RB_TRACE
        if (tracedd) { const unsigned long long n_ = gtime(); trd.t[4] = n_ - tld; tld = n_; }
#endif
        if (__all_sync(0xffffffffu, acc_ok)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row0 = rt0 * TILE_ROWS;
            // a warp reaches the tensor-memory lanes of its quarter (warp % 4); with eight warps the two
            // groups of four split the (token half, 32-row chunk) pairs between them
            constexpr int NCH = T5_ROWS / 32, GROUPS = NDW / 4;
            const int wq = warp & 3, grp = warp >> 2;
            if constexpr (QKV) {
                // lane = token; per item one head of the tile (0 / 1) and one pair of 32-row chunks (pp, pp + 2):
                // rows 32 pp + [0, 32) of the head rotate with rows 64 + 32 pp + [0, 32)
#pragma unroll 1
                for (int item = grp; item < nhalf * 4; item += GROUPS) {
                    const int half = item >> 2, hh = (item >> 1) & 1, pp = item & 1;
                    const int R0 = row0 + hh * 128;  // first row of the head in the stacked matrix
                    if (R0 >= p.out) continue;       // warp-uniform
                    const int tok_base = tok0 + half * 128 + wq * 32;
                    const int token = tok_base + lane;
                    uint32_t gv[32], uv[32];
                    const uint32_t taddr = tmem + ((uint32_t)(wq * 32) << 16) + (uint32_t)(half * ROWS + hh * 128 + pp * 32);
                    t5_ld32(taddr, gv);
                    t5_ld32(taddr + 64u, uv);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    const int kind = R0 < p.dq ? 0 : (R0 < p.dq + p.dkv ? 1 : 2);  // q, k, v
                    const int head = (kind == 0 ? R0 : (kind == 1 ? R0 - p.dq : R0 - p.dq - p.dkv)) >> 7;
                    const float sc = kind == 0 ? p.sq : (kind == 1 ? p.sk : p.sv);
                    const bool live = token < p.ncols;
                    const int bb = live ? token / p.seq : 0;
                    const int pos = live ? __ldg(p.past_len + bb) + (token - bb * p.seq) : 0;
                    const float sxv = live ? __ldg(p.sx + token) : 0.f;
                    const int32_t xs = live ? __ldg(p.xsum + token) : 0;
                    const bool rot = kind != 2 && p.rope != nullptr && live && pos < p.max_seq;
                    const float4* cs4 = reinterpret_cast<const float4*>(p.rope + (size_t)(rot ? pos : 0) * 64 + 32 * pp);
#pragma unroll
                    for (int q = 0; q < 32; q += 2) {
                        float a0 = ((float)((int32_t)gv[q] - xs) * sxv) * sc, a1 = ((float)((int32_t)gv[q + 1] - xs) * sxv) * sc;
                        float c0 = ((float)((int32_t)uv[q] - xs) * sxv) * sc, c1 = ((float)((int32_t)uv[q + 1] - xs) * sxv) * sc;
                        if (rot) {
                            const float4 cs = __ldg(cs4 + (q >> 1));  // (cos, sin) of pairs q and q + 1
                            const float r0 = a0 * cs.x - c0 * cs.y, r1 = a1 * cs.z - c1 * cs.w;
                            c0 = c0 * cs.x + a0 * cs.y;
                            c1 = c1 * cs.z + a1 * cs.w;
                            a0 = r0;
                            a1 = r1;
                        }
                        gv[q] = __float_as_uint(a0);
                        gv[q + 1] = __float_as_uint(a1);
                        uv[q] = __float_as_uint(c0);
                        uv[q + 1] = __float_as_uint(c1);
                    }
                    // destination of token tok_base + tl: its q row, or its position's row of the head's cache
                    auto dst_of = [&](int tl, int col) -> void* {
                        const int t2 = tok_base + tl;
                        if (t2 >= p.ncols) return nullptr;
                        if (kind == 0) return p.qout + (size_t)t2 * p.dq + (size_t)head * 128 + col;
                        const int b2 = t2 / p.seq, pos2 = __ldg(p.past_len + b2) + (t2 - b2 * p.seq);
                        if (pos2 >= p.max_seq) return nullptr;
                        float* cache = kind == 1 ? p.k_cache : p.v_cache;
                        return cache + (((size_t)b2 * (p.dkv >> 7) + head) * p.max_seq + pos2) * 128 + col;
                    };
                    const uint32_t stage = ring + (uint32_t)warp * T5_XPOSE_BYTES;
                    t5_store_rows_to(stage, gv, lane, [&](int tl) { return dst_of(tl, 32 * pp); });
                    t5_store_rows_to(stage, uv, lane, [&](int tl) { return dst_of(tl, 64 + 32 * pp); });
                }
            } else if constexpr (GATED) {
                // lane = token; per item 32 channels: gate accumulators in columns [32 ch, +32), up in [128 + 32 ch, +32)
#pragma unroll 1
                for (int item = grp; item < nhalf * (NCH / 2); item += GROUPS) {
                    const int half = item / (NCH / 2), ch = item - half * (NCH / 2);
                    const int token = tok0 + half * 128 + wq * 32 + lane;
                    uint32_t gv[32], uv[32];
                    const uint32_t taddr = tmem + ((uint32_t)(wq * 32) << 16) + (uint32_t)(half * ROWS + ch * 32);
                    t5_ld32(taddr, gv);
                    t5_ld32(taddr + 128u, uv);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    const int c0 = (int)blockIdx.y * 128 + ch * 32;
                    if (c0 < p.ff) {  // warp-uniform
                        const int tok_base = tok0 + half * 128 + wq * 32;
                        const bool live = token < p.ncols;
                        const float sxv = live ? __ldg(p.sx + token) : 0.f;
                        const int32_t xs = live ? __ldg(p.xsum + token) : 0;
                        // the gated values replace the gate accumulators in place (bit patterns of float32)
#pragma unroll
                        for (int q = 0; q < 32; ++q) {
                            const float g = ((float)((int32_t)gv[q] - xs) * sxv) * p.sg, u = ((float)((int32_t)uv[q] - xs) * sxv) * p.su;
                            float r;
                            if (p.ffn_act == ROTOR_B200_FFN_RELU2) {
                                const float a = fmaxf(g, 0.f);
                                r = a * a * u;
                            } else {
                                const float c = fminf(fmaxf(u, -20.f), 20.f);
                                r = g * (c / (1.f + expf(-c)));
                            }
                            gv[q] = __float_as_uint(r);
                        }
                        if (c0 + 32 <= p.ff && (p.ff & 3) == 0) {
                            t5_store_rows(ring + (uint32_t)warp * T5_XPOSE_BYTES, gv, p.gated + (size_t)tok_base * p.ff + c0,
                                          (size_t)p.ff * sizeof(float), tok_base, p.ncols, lane);
                        } else if (live) {
                            float* dst = p.gated + (size_t)token * p.ff + c0;
#pragma unroll
                            for (int q = 0; q < 32; ++q)
                                if (c0 + q < p.ff) dst[q] = __uint_as_float(gv[q]);
                        }
                    }
                }
            } else
#pragma unroll 1
            for (int item = grp; item < nhalf * NCH; item += GROUPS) {
                const int half = item / NCH, ch = item - half * NCH;
                const int token = tok0 + half * 128 + wq * 32 + lane;
                {
                    uint32_t v[32];
                    const uint32_t taddr = tmem + ((uint32_t)(wq * 32) << 16) + (uint32_t)(half * ROWS + ch * 32);
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
                          "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
                          "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
                          "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
                          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                        : "r"(taddr));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    const int rbase = row0 + ch * 32;
                    if (rbase < p.out) {  // warp-uniform
                        const int tok_base = tok0 + half * 128 + wq * 32;
                        // remove the +1 of the codes: once per output, i.e. in the first K split only
                        const uint32_t xs =
                            ((p.kt_per_split && blockIdx.z) || token >= p.ncols) ? 0u : (uint32_t)__ldg(p.xsum + token);
#pragma unroll
                        for (int q = 0; q < 32; ++q) v[q] -= xs;
                        if (p.kt_per_split) {  // one of several partial sums: exact, in any order
                            if (token < p.ncols) {
                                int32_t* dst = p.acc + (size_t)token * p.out + rbase;
#pragma unroll
                                for (int q = 0; q < 32; ++q)
                                    if (rbase + q < p.out) atomicAdd(dst + q, (int32_t)v[q]);
                            }
                        } else if (rbase + 32 <= p.out && (p.out & 3) == 0) {
                            t5_store_rows(ring + (uint32_t)warp * T5_XPOSE_BYTES, v, p.acc + (size_t)tok_base * p.out + rbase,
                                          (size_t)p.out * sizeof(int32_t), tok_base, p.ncols, lane);
                        } else if (token < p.ncols) {
                            int32_t* dst = p.acc + (size_t)token * p.out + rbase;
#pragma unroll
                            for (int q = 0; q < 32; ++q)
                                if (rbase + q < p.out) dst[q] = (int32_t)v[q];
                        }
                    }
                }
            }
        }
#ifdef RB_TRACE
        if (tracedd) {
            trd.t[5] = gtime() - tld;  // read-back and stores
            trd.kind = 601;
            unsigned idx_ = atomicAdd(&g_trace_n, 1u);
            if (idx_ < 4096) g_trace[idx_] = trd;
        }
#endif
    } else if (warp == NDW) {
        // ---------------- token operand by TMA
        if (lane == 0) {
            for (int kt = 0; kt < nk; ++kt) {
                const int s = kt % T5_STAGES;
                if (!t5_wait(smem_u32(&s_empty[s]), ((kt / T5_STAGES) & 1) ^ 1, abort_flag, p.status, 0x7c000003u)) break;
                const uint32_t bar = smem_u32(&s_full[s]);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
                             "r"(nhalf * A_HALF)
                             : "memory");
                for (int half = 0; half < nhalf; ++half) {
                    const uint32_t dst = ring + s * T5_STAGE_BYTES + half * A_HALF;
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
                        "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                        "l"(&tmap), "r"((ktb + kt) * TILE_K), "r"(tok0 + half * 128), "r"(bar)
                        : "memory");
                }
            }
        }
    } else {
        // ---------------- MMA issue
        if (lane == 0) {
            // kind::i8, S32 accumulate, signed tokens (A) x unsigned weight codes (B), both K-major, N = ROWS, M = 128
            const uint32_t idesc = (2u << 4) | (1u << 7) | (0u << 10) | ((uint32_t)(T5_ROWS >> 3) << 17) | ((128u >> 4) << 24);
            bool ok = true;
#ifdef RB_TRACE
            TraceRec trm = {};
            const bool traced = blockIdx.x == 0 && blockIdx.y == 0;
            unsigned long long tl = gtime(), t0m = tl;
#endif
            for (int kt = 0; kt < nk && ok; ++kt) {
                const int s = kt % T5_STAGES;
                ok = t5_wait(smem_u32(&s_full[s]), (kt / T5_STAGES) & 1, abort_flag, p.status, 0x7c000004u);
                if (!ok) break;
#ifdef RB_TRACE
                if (traced) { const unsigned long long n_ = gtime(); trm.t[0] += n_ - tl; tl = n_; }
#endif
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t abase = ring + s * T5_STAGE_BYTES, bbase = abase + T5_A_BYTES;
                for (int half = 0; half < nhalf; ++half)
#pragma unroll
                    for (int k4 = 0; k4 < TILE_K / 32; ++k4) {
                        const uint64_t da = t5_desc(abase + half * A_HALF + k4 * 32);
                        const uint64_t db = t5_desc(bbase + k4 * 32);
                        const uint32_t accumulate = (kt > 0 || k4 > 0) ? 1u : 0u;
                        asm volatile(
                            "{\n\t"
                            ".reg .pred p;\n\t"
                            "setp.ne.b32 p, %4, 0;\n\t"
                            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
                            "}\n" ::"r"(tmem + (uint32_t)(half * ROWS)),
                            "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u)
                            : "memory");
                    }
                // arrives on the stage's "empty" barrier once these MMAs have read their operands
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                 smem_u32(&s_empty[s]))
                             : "memory");
#ifdef RB_TRACE
                if (traced) { const unsigned long long n_ = gtime(); trm.t[1] += n_ - tl; tl = n_; }
#endif
            }
#ifdef RB_TRACE
            if (traced) {
                trm.t[2] = gtime() - t0m;
                trm.t[7] = (unsigned long long)p.nkt;
                trm.kind = 600;
                unsigned idx_ = atomicAdd(&g_trace_n, 1u);
                if (idx_ < 4096) g_trace[idx_] = trm;
            }
#endif
            if (ok)
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                 smem_u32(&s_accf))
                             : "memory");
        }
    }

    // ---------------- common exit: nothing of this CTA may still be in flight when it returns
    if (*abort_flag && threadIdx.x == 0) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {
        }  // about a millisecond for copies already issued to land
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == NDW) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(Cfg::TMEM_COLS));
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;
static PerDevice<bool> g_tc5_ready;

// Shapes this kernel takes: enough tokens to be worth its tile, 16-byte aligned operands.
bool gemm_tcgen05_supported(size_t out, size_t in, int ncols, const void* xq) {
    static const bool off = getenv("ROTOR_B200_NO_TCGEN05") != nullptr;  // measurement aid: legacy mma.sync path
    // from 32 tokens on: with fewer than 256 the tile is partly empty, but the product is then bound by
    // the weight stream, which this kernel moves faster than the mma.sync kernel does
    return !off && ncols >= 32 && out >= 16 && in >= 4 && ((uintptr_t)xq & 15) == 0;
}

int configure_gemm_tcgen05() {
    if (g_tc5_ready.here()) return ROTOR_B200_OK;
    cudaDriverEntryPointQueryResult q;
    void* fn = nullptr;
    RB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    if (!fn || q != cudaDriverEntryPointSuccess) return ROTOR_B200_ERR_CUDA;
    g_encode = (EncodeTiledFn)fn;
    RB_CUDA(cudaFuncSetAttribute(gemm_tcgen05_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, T5Cfg<256>::SMEM));
    RB_CUDA(cudaFuncSetAttribute(gemm_tcgen05_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, T5Cfg<64>::SMEM));
    RB_CUDA(cudaFuncSetAttribute(gemm_tcgen05_kernel<256, 256, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 T5Cfg<256>::SMEM));
    RB_CUDA(cudaFuncSetAttribute(gemm_tcgen05_kernel<256, 256, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 T5Cfg<256>::SMEM));
    g_tc5_ready.here() = true;
    return ROTOR_B200_OK;
}

int launch_gemm_tcgen05(const void* tiles, size_t out, size_t in, const int8_t* xq, const int32_t* xsum, int ncols,
                        int32_t* acc, cudaStream_t st) {
    int rc = configure_gemm_tcgen05();
    if (rc) return rc;
    Tc5Params p = {};
    p.tiles = (const uint4*)tiles;
    p.xsum = xsum;
    p.acc = acc;
    p.status = library_status_word();
    p.out = (int)out;
    p.nrt = (int)(opad_of(out) / TILE_ROWS);
    p.nkt = (int)(kpad_of(in) / TILE_K);
    p.ncols = ncols;
    if (!p.status) return ROTOR_B200_ERR_CUDA;
    const size_t kpad = kpad_of(in);
    CUtensorMap tmap;
    const cuuint64_t gdim[2] = {(cuuint64_t)kpad, (cuuint64_t)ncols};
    const cuuint64_t gstride[1] = {(cuuint64_t)kpad};  // bytes between token rows
    const cuuint32_t box[2] = {(cuuint32_t)TILE_K, 128u};
    const cuuint32_t estride[2] = {1u, 1u};
    if (g_encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)xq, gdim, gstride, box, estride,
                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return ROTOR_B200_ERR_CUDA;
    const int tok_tiles = (ncols + 255) / 256, rows = p.nrt * TILE_ROWS;
    static PerDevice<int> sm_counts;
    int& sms = sm_counts.here();
    if (!sms) {
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, current_device()) != cudaSuccess || sms <= 0)
            sms = 148;
    }
    const int tiles256 = tok_tiles * ((rows + 255) / 256);
    // fewer 256-row tiles than SMs: split the K range so that the grid covers the GPU (a K step of a
    // 256-row tile costs a decoder less per weight than four steps of 64-row tiles); at least four K
    // steps per CTA, partial sums added into the zeroed accumulators
    int splits = tiles256 < sms ? sms / tiles256 : 1;
    if (splits > p.nkt / 4) splits = p.nkt / 4;
    if (splits >= 2) {
        p.kt_per_split = (p.nkt + splits - 1) / splits;
        splits = (p.nkt + p.kt_per_split - 1) / p.kt_per_split;
        RB_CUDA(cudaMemsetAsync(acc, 0, (size_t)ncols * out * sizeof(int32_t), st));
        dim3 grid(tok_tiles, (rows + 255) / 256, splits);
        gemm_tcgen05_kernel<256><<<grid, T5Cfg<256>::THREADS, T5Cfg<256>::SMEM, st>>>(tmap, p);
    } else if (tiles256 < sms) {  // 256-row tiles would leave SMs idle
        dim3 grid(tok_tiles, (rows + 63) / 64);
        gemm_tcgen05_kernel<64><<<grid, T5Cfg<64>::THREADS, T5Cfg<64>::SMEM, st>>>(tmap, p);
    } else {
        dim3 grid(tok_tiles, (rows + 255) / 256);
        gemm_tcgen05_kernel<256><<<grid, T5Cfg<256>::THREADS, T5Cfg<256>::SMEM, st>>>(tmap, p);
    }
    return launch_status();
}

// Gate/up product with the gating in the epilogue: `tiles` holds the gate matrix followed by the up
// matrix (ff rows each, ff a multiple of 16), one activation term per token.  Writes
// gated[token][channel] as float32; no int32 accumulator leaves the kernel.
bool gemm_tcgen05_gated_supported(size_t ff, size_t in, int ncols, const void* xq) {
    return ff % TILE_ROWS == 0 && ncols >= 256 && gemm_tcgen05_supported(2 * ff, in, ncols, xq);
}

int launch_gemm_tcgen05_gated(const void* tiles, size_t ff, size_t in, const int8_t* xq, const float* sx,
                              const int32_t* xsum, int ncols, float sg, float su, int ffn_act, float* gated,
                              cudaStream_t st) {
    int rc = configure_gemm_tcgen05();
    if (rc) return rc;
    if (!gemm_tcgen05_gated_supported(ff, in, ncols, xq)) return ROTOR_B200_ERR_SHAPE;
    Tc5Params p = {};
    p.tiles = (const uint4*)tiles;
    p.status = library_status_word();
    p.out = (int)(2 * ff);
    p.nrt = (int)(2 * ff / TILE_ROWS);
    p.nkt = (int)(kpad_of(in) / TILE_K);
    p.ncols = ncols;
    p.gated = gated;
    p.sx = sx;
    p.xsum = xsum;
    p.sg = sg;
    p.su = su;
    p.ff = (int)ff;
    p.ffn_act = ffn_act;
    if (!p.status) return ROTOR_B200_ERR_CUDA;
    const size_t kpad = kpad_of(in);
    CUtensorMap tmap;
    const cuuint64_t gdim[2] = {(cuuint64_t)kpad, (cuuint64_t)ncols};
    const cuuint64_t gstride[1] = {(cuuint64_t)kpad};
    const cuuint32_t box[2] = {(cuuint32_t)TILE_K, 128u};
    const cuuint32_t estride[2] = {1u, 1u};
    if (g_encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)xq, gdim, gstride, box, estride,
                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return ROTOR_B200_ERR_CUDA;
    dim3 grid((ncols + 255) / 256, (unsigned)((ff + 127) / 128));
    gemm_tcgen05_kernel<256, 256, true><<<grid, T5Cfg<256>::THREADS, T5Cfg<256>::SMEM, st>>>(tmap, p);
    return launch_status();
}

// q/k/v product with dequantisation, rotary and the cache append in its read-back: head_dim 128, one
// activation term per token, enough tokens for 256-row tiles to cover the GPU.
bool gemm_tcgen05_qkv_supported(size_t dq, size_t dkv, size_t in, int head_dim, int ncols, const void* xq) {
    return head_dim == 128 && dq % 128 == 0 && dkv % 128 == 0 && ncols >= 256 &&
           gemm_tcgen05_supported(dq + 2 * dkv, in, ncols, xq);
}

int launch_gemm_tcgen05_qkv(const void* tiles, size_t in, const int8_t* xq, const float* sx, const int32_t* xsum,
                            int ncols, const QkvFinishParams& f, cudaStream_t st) {
    int rc = configure_gemm_tcgen05();
    if (rc) return rc;
    const size_t dq = (size_t)f.n_heads * f.head_dim, dkv = (size_t)f.n_kv_heads * f.head_dim;
    if (!gemm_tcgen05_qkv_supported(dq, dkv, in, f.head_dim, ncols, xq) || f.terms != 1) return ROTOR_B200_ERR_SHAPE;
    Tc5Params p = {};
    p.tiles = (const uint4*)tiles;
    p.status = library_status_word();
    p.out = (int)(dq + 2 * dkv);
    p.nrt = (int)(opad_of(dq + 2 * dkv) / TILE_ROWS);
    p.nkt = (int)(kpad_of(in) / TILE_K);
    p.ncols = ncols;
    p.sx = sx;
    p.xsum = xsum;
    p.dq = (int)dq;
    p.dkv = (int)dkv;
    p.seq = f.seq;
    p.max_seq = f.max_seq;
    p.past_len = f.past_len;
    p.rope = f.rope;
    p.qout = f.q;
    p.k_cache = f.k_cache;
    p.v_cache = f.v_cache;
    p.sq = f.sq;
    p.sk = f.sk;
    p.sv = f.sv;
    if (!p.status) return ROTOR_B200_ERR_CUDA;
    const size_t kpad = kpad_of(in);
    CUtensorMap tmap;
    const cuuint64_t gdim[2] = {(cuuint64_t)kpad, (cuuint64_t)ncols};
    const cuuint64_t gstride[1] = {(cuuint64_t)kpad};
    const cuuint32_t box[2] = {(cuuint32_t)TILE_K, 128u};
    const cuuint32_t estride[2] = {1u, 1u};
    if (g_encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)xq, gdim, gstride, box, estride,
                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return ROTOR_B200_ERR_CUDA;
    dim3 grid((ncols + 255) / 256, (unsigned)((p.nrt * TILE_ROWS + 255) / 256));
    gemm_tcgen05_kernel<256, 256, false, true><<<grid, T5Cfg<256>::THREADS, T5Cfg<256>::SMEM, st>>>(tmap, p);
    return launch_status();
}

}  // namespace rb
