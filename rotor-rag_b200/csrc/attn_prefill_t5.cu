// Softmax attention for prompt prefill on the fifth-generation tensor cores (head_dim 128).
//
// Reference: MultiHeadAttention.forward (src/rotor/transformer.py:249-283): scores
// Q K^T / sqrt(head_dim) over the cache, optional causal mask, softmax, times V, K/V shared by the
// query heads of a group.  Same contract and row mapping as the mma.sync kernel
// (attn_prefill_tc.cu), which stays for head_dim 64 and as the comparison path.
//
// CTA: 128 query rows of one KV head (128 / G positions x G heads of the group), keys walked 64
// at a time.  Both products run as tcgen05.mma.kind::f16 with bf16 operands and float32
// accumulators in tensor memory, every operand split into hi + lo bf16 terms
// (hi*hi + hi*lo + lo*hi: 16 operand mantissa bits), which holds the 1e-3-of-RMS bound of the
// float32 reference.
//   S = Q K^T : A = Q hi / lo from shared memory (staged and split once per CTA), B = K hi / lo
//               tiles [64 keys][128] by TMA; accumulator 128 lanes x 64 columns, double buffered.
//   O_j = P V : A = P hi / lo from TENSOR MEMORY (written by the softmax warps over the S buffer
//               they have just read), B = V^T hi / lo tiles [128][64 keys] by TMA (the split
//               kernel stores V transposed per key tile so that this operand is K-major too);
//               accumulator 128 lanes x 128 columns, fresh for every key tile, double buffered.
// Warps 0-7: two threads per query row (warps 0-3 take the first 32 keys of a tile and output
// columns 0-63, warps 4-7 the other halves; a warp reaches the tensor-memory lanes of its quarter
// warp % 4) -- row maximum (halves exchanged through shared memory), exponentials (base 2, log2 e
// folded into the scale of Q), split of P, and the running output O = O * alpha + O_j in
// registers.  Two warps per scheduler hide each other's latencies; one row per thread left the
// tensor pipe waiting on a single dependent instruction stream.  The output update of tile j runs
// after the softmax of tile j + 1, so that P V of tile j overlaps it.
// Warps 8 and 9: TMA producers of the K and the V^T tiles -- separate two-deep rings, because a K
// tile is free again as soon as its S product has run (one tile ahead of the softmax) while a V^T
// tile stays until P V; with one ring the next K load would wait for P V and the tensor pipe for
// that load.  Warp 10: MMA issue, one key tile ahead with S.
// Every wait is bounded; a wait that runs out records a code in the library status word, the CTA
// stops issuing work, frees its tensor memory and returns.  No multicast, this GPU's memory only.
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstdlib>

#include "model.cuh"

RB_TRACE_DEFINE(rotor_b200_trace_read_attn5)

namespace rb {

// Phase timing of the softmax loop (compiled in with -DRB_TRACE): thread 0 of CTA (0, 0, 0) adds up
// the time between the marks of every key tile and commits the sums once.
#ifdef RB_TRACE
#define A5_MARK(i)                                                                     \
    do {                                                                               \
        if (a5_traced) {                                                               \
            const unsigned long long now_ = gtime();                                   \
            tr.t[i] += now_ - a5_last;                                                 \
            a5_last = now_;                                                            \
        }                                                                              \
    } while (0)
#else
#define A5_MARK(i) do {} while (0)
#endif

constexpr int A5_BM = 128, A5_BN = 64, A5_D = 128;
constexpr int A5_THREADS = 352;  // 8 softmax / output warps, two TMA warps, MMA warp
constexpr int A5_SOFT = 256;     // threads of the softmax warps
constexpr int A5_Q_BYTES = 4 * 16384;     // Q hi panel 0, 1; Q lo panel 0, 1 (128 rows x 128 bytes each)
constexpr int A5_K_BYTES = 32768;         // one K tile: hi panel 0, 1; lo panel 0, 1 (64 rows x 128 bytes each)
constexpr int A5_V_BYTES = 32768;         // one V^T tile: hi, lo (128 rows x 128 bytes each)
constexpr int A5_STAGES = 2;              // depth of the K ring and of the V^T ring
constexpr int A5_SMEM = A5_Q_BYTES + A5_STAGES * (A5_K_BYTES + A5_V_BYTES) + 1024;
constexpr int A5_TMEM_COLS = 512;         // S0 [0,64)  S1 [64,128)  O_j even [128,256)  O_j odd [256,384)
constexpr long long A5_SPIN_CYCLES = 400000000LL;  // about 0.2 s

struct A5Params {
    const float* q;        // [rows][n_heads * 128]
    float* out;            // [rows][n_heads * 128]
    const int* past_len;
    unsigned* status;
    int n_heads, n_kv_heads, seq, max_seq, causal;
    int split_seq;         // rows per (sequence, KV head) in the K planes (max_seq rounded up to 64)
};

__device__ __forceinline__ uint32_t a5_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool a5_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, unsigned* status,
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
        if (clock64() - t0 > A5_SPIN_CYCLES) {
            *abort_flag = 1;
            atomicExch(status, code);
            return false;
        }
    }
}

// Shared-memory matrix descriptor, K-major, 128-byte swizzle: 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t a5_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3fffu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
           (2ull << 61);
}

// ACC == 0: the accumulator is overwritten (first MMA of a tile), 1: accumulated into.
template <int ACC>
__device__ __forceinline__ void a5_mma_ss(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(da), "l"(db), "r"(idesc), "n"(ACC), "r"(0u)
        : "memory");
}
template <int ACC>
__device__ __forceinline__ void a5_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t db, uint32_t idesc) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(db), "r"(idesc), "n"(ACC), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void a5_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void a5_ld32(uint32_t taddr, uint32_t (&v)[32]) {
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
__device__ __forceinline__ void a5_st32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
        "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]),
        "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]),
        "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}

__device__ __forceinline__ void a5_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
        "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}

// hi + lo split of two floats, packed as bf16x2 (first value in the low half): one packed conversion
// per term, the hi values widened again by shifting
__device__ __forceinline__ void a5_split2(float x, float y, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    const float xh = __uint_as_float(hi << 16), yh = __uint_as_float(hi & 0xffff0000u);
    const __nv_bfloat162 l = __floats2bfloat162_rn(x - xh, y - yh);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}
__device__ __forceinline__ float a5_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Splits the float32 K/V cache rows of key tile blockIdx.x (64 keys) of one (sequence, KV head)
// into hi / lo bf16 planes laid out for the tensor-core kernel:
//   K hi, K lo : [sequence][KV head][split_seq][128]          (row = key)
//   V hi, V lo : [sequence][KV head][tile][128][64]           (transposed inside the key tile)
// Keys past the sequence's length inside a started tile are written as zeros (their probabilities
// are zero, and zero times stale memory could be NaN); tiles past the length are not touched.
__global__ void __launch_bounds__(256) kv_split_t5_kernel(const float* __restrict__ k_cache, const float* __restrict__ v_cache,
                                                          const int* __restrict__ past_len, int seq, int max_seq,
                                                          int n_kv_heads, int split_seq, __nv_bfloat16* __restrict__ planes,
                                                          size_t plane) {
    __shared__ float vs[A5_BN][A5_D + 1];
    const int tile = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    int t_all = past_len[b] + seq;
    if (t_all > max_seq) t_all = max_seq;
    const int t0 = tile * A5_BN;
    if (t0 >= t_all) return;
    const size_t head = (size_t)b * n_kv_heads + hk;
    const float* kc = k_cache + head * max_seq * A5_D;
    const float* vc = v_cache + head * max_seq * A5_D;
    __nv_bfloat16* kh = planes + (head * split_seq + t0) * A5_D;
    __nv_bfloat16* kl = kh + plane;
    for (int idx = threadIdx.x; idx < A5_BN * (A5_D / 4); idx += 256) {
        const int r = idx / (A5_D / 4), c4 = idx - r * (A5_D / 4);
        float4 k = make_float4(0.f, 0.f, 0.f, 0.f), v = k;
        if (t0 + r < t_all) {
            k = *reinterpret_cast<const float4*>(kc + (size_t)(t0 + r) * A5_D + 4 * c4);
            v = *reinterpret_cast<const float4*>(vc + (size_t)(t0 + r) * A5_D + 4 * c4);
        }
        uint2 h2, l2;
        a5_split2(k.x, k.y, h2.x, l2.x);
        a5_split2(k.z, k.w, h2.y, l2.y);
        *reinterpret_cast<uint2*>(kh + (size_t)r * A5_D + 4 * c4) = h2;
        *reinterpret_cast<uint2*>(kl + (size_t)r * A5_D + 4 * c4) = l2;
        vs[r][4 * c4] = v.x;
        vs[r][4 * c4 + 1] = v.y;
        vs[r][4 * c4 + 2] = v.z;
        vs[r][4 * c4 + 3] = v.w;
    }
    __syncthreads();
    __nv_bfloat16* vh = planes + 2 * plane + (head * (split_seq / A5_BN) + tile) * (size_t)(A5_D * A5_BN);
    __nv_bfloat16* vl = vh + plane;
    for (int idx = threadIdx.x; idx < A5_D * (A5_BN / 2); idx += 256) {
        const int d = idx / (A5_BN / 2), kp = idx - d * (A5_BN / 2);  // keys 2 kp, 2 kp + 1
        uint32_t h, l;
        a5_split2(vs[2 * kp][d], vs[2 * kp + 1][d], h, l);
        *reinterpret_cast<uint32_t*>(vh + (size_t)d * A5_BN + 2 * kp) = h;
        *reinterpret_cast<uint32_t*>(vl + (size_t)d * A5_BN + 2 * kp) = l;
    }
}

__global__ void __launch_bounds__(A5_THREADS, 1)
attn_prefill_t5_kernel(const __grid_constant__ CUtensorMap tm_kh, const __grid_constant__ CUtensorMap tm_kl,
                       const __grid_constant__ CUtensorMap tm_vh, const __grid_constant__ CUtensorMap tm_vl,
                       const __grid_constant__ A5Params p) {
    extern __shared__ unsigned char a5_raw[];
    __shared__ __align__(8) unsigned long long s_kfull[A5_STAGES], s_kempty[A5_STAGES], s_vfull[A5_STAGES],
        s_vempty[A5_STAGES], s_sfull[2], s_pfull[2], s_ofull[2], s_oempty[2], s_qready;
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    __shared__ float s_xch[2][A5_BM];  // row maxima / sums exchanged between the two threads of a row
    __shared__ int s_go;               // the softmax warps' common decision to go on (taken between two barriers)
    const uint32_t base = (a5_smem(a5_raw) + 1023u) & ~1023u;
    const uint32_t q_hi = base, q_lo = base + 32768, kring = base + A5_Q_BYTES, vring = kring + A5_STAGES * A5_K_BYTES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = p.n_heads / p.n_kv_heads, QT = A5_BM / G;
    const int qt = gridDim.x - 1 - blockIdx.x;  // late query tiles see the most keys: start them first
    const int hk = blockIdx.y, b = blockIdx.z;
    const int s0 = qt * QT;
    const int past = p.past_len[b];
    volatile int* abort_flag = &s_abort;

    int s_last = s0 + QT - 1;
    if (s_last > p.seq - 1) s_last = p.seq - 1;
    int t_all = p.causal ? past + s_last + 1 : past + p.seq;
    if (t_all > p.max_seq) t_all = p.max_seq;
    const int ntiles = (t_all + A5_BN - 1) / A5_BN;

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < A5_STAGES; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(a5_smem(&s_kfull[s])), "r"(1));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(a5_smem(&s_kempty[s])), "r"(1));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(a5_smem(&s_vfull[s])), "r"(1));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(a5_smem(&s_vempty[s])), "r"(1));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(a5_smem(&s_sfull[s])), "r"(1));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(a5_smem(&s_pfull[s])), "r"(A5_SOFT));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(a5_smem(&s_ofull[s])), "r"(1));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(a5_smem(&s_oempty[s])), "r"(A5_SOFT));
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(a5_smem(&s_qready)), "r"(A5_SOFT));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(a5_smem(&s_tmem)),
                     "r"(A5_TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

#ifdef RB_TRACE
    TraceRec tr2 = {};
    RB_STAMP(tr2, 0);
#endif
    if (warp < 8) {
        // ---------------- Q tile: scaled, split into hi / lo bf16, K-major panels of 64 columns, 128-byte swizzle
        {
            const float scale = 1.4426950408889634f / sqrtf((float)A5_D);  // scores come out in units of log2: p = 2^(s - m)
            // all sixteen loads of a thread are issued before the first conversion (one round trip to memory
            // instead of sixteen: the MMA warp waits for this tile before it can start)
            constexpr int QN = A5_BM * (A5_D / 4) / A5_SOFT;
            float4 qv[QN];
#pragma unroll
            for (int u = 0; u < QN; ++u) {
                const int idx = threadIdx.x + u * A5_SOFT;
                const int r = idx / (A5_D / 4), c4 = idx - r * (A5_D / 4);
                const int s = s0 + r / G, gi = r - (r / G) * G;
                qv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (s < p.seq)
                    qv[u] = __ldg(reinterpret_cast<const float4*>(p.q + ((size_t)b * p.seq + s) * p.n_heads * A5_D +
                                                                  (size_t)(hk * G + gi) * A5_D + 4 * c4));
            }
#ifdef RB_TRACE
#pragma unroll
            for (int u = 0; u < QN; ++u) asm volatile("" ::"f"(qv[u].w));
            RB_STAMP(tr2, 4);
#endif
#pragma unroll
            for (int u = 0; u < QN; ++u) {
                const int idx = threadIdx.x + u * A5_SOFT;
                const int r = idx / (A5_D / 4), c4 = idx - r * (A5_D / 4);
                const float4 v = qv[u];
                uint32_t h0, l0, h1, l1;
                a5_split2(v.x * scale, v.y * scale, h0, l0);
                a5_split2(v.z * scale, v.w * scale, h1, l1);
                // column 4 c4: panel (4 c4) / 64, byte (4 c4 % 64) * 2 of the 128-byte row: chunk c4 / 2 % 8, half c4 & 1
                const int panel = c4 >> 4, chunk = (c4 >> 1) & 7;
                const uint32_t off = (uint32_t)panel * 16384u + (uint32_t)(r >> 3) * 1024u + (uint32_t)(r & 7) * 128u +
                                     (uint32_t)((chunk ^ (r & 7)) << 4) + (uint32_t)(c4 & 1) * 8u;
                asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(q_hi + off), "r"(h0), "r"(h1) : "memory");
                asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(q_lo + off), "r"(l0), "r"(l1) : "memory");
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> tensor-core reads
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(a5_smem(&s_qready)) : "memory");
        }
#ifdef RB_TRACE
        RB_STAMP(tr2, 1);
#endif
        // ---------------- softmax and output: this thread owns keys [32 half, 32 half + 32) of a tile and output
        // columns [64 half, 64 half + 64) of query row r
        const int half = warp >> 2, wq = warp & 3;
        const int r = wq * 32 + lane;
        const int srow = s0 + r / G, gi = r - (r / G) * G;
        int lim = p.causal ? past + (srow < p.seq ? srow : s_last) + 1 : past + p.seq;
        if (lim > t_all) lim = t_all;
        const uint32_t lane_base = tmem + ((uint32_t)(wq * 32) << 16);
        float m_run = -INFINITY, l_run = 0.f, alpha_prev = 1.f;
        float o[A5_D / 2];
#pragma unroll
        for (int i = 0; i < A5_D / 2; ++i) o[i] = 0.f;
        bool ok = true;
#ifdef RB_TRACE
        TraceRec tr = {};
        const bool a5_traced = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0;
        unsigned long long a5_last = gtime();
#endif
        // O = O * alpha + P V of key tile j (its accumulator buffer j & 1), this thread's 64 columns
        auto accumulate = [&](int j, float alpha) {
            bool good = a5_wait(a5_smem(&s_ofull[j & 1]), (uint32_t)(j >> 1) & 1u, abort_flag, p.status, 0x7b000002u);
            if (!__all_sync(0xffffffffu, good)) return false;
            A5_MARK(5);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t ov0[32], ov1[32];
            const uint32_t ob = lane_base + 128u + (uint32_t)(j & 1) * 128u + (uint32_t)half * 64u;
            a5_ld32(ob, ov0);
            a5_ld32(ob + 32u, ov1);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                o[i] = o[i] * alpha + __uint_as_float(ov0[i]);
                o[32 + i] = o[32 + i] * alpha + __uint_as_float(ov1[i]);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(a5_smem(&s_oempty[j & 1])) : "memory");
            A5_MARK(6);
            return true;
        };
        // (the eight warps leave this loop together: whether to go on is decided by one thread between the
        // two barriers of an iteration, so that no warp is left alone at a barrier after a failed wait)
        for (int j = 0; j < ntiles; ++j) {
            const uint32_t sbuf = lane_base + (uint32_t)(j & 1) * 64u;
            ok = ok && a5_wait(a5_smem(&s_sfull[j & 1]), (uint32_t)(j >> 1) & 1u, abort_flag, p.status, 0x7b000001u);
            ok = __all_sync(0xffffffffu, ok);
            A5_MARK(0);
            uint32_t sa[32];
            float tmax = -INFINITY;
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                a5_ld32(sbuf + (uint32_t)half * 32u, sa);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                const int kb = j * A5_BN + half * 32;
                if (kb + 32 > lim) {  // only the last tiles of a row need the mask
#pragma unroll
                    for (int c = 0; c < 32; ++c)
                        if (kb + c >= lim) sa[c] = 0xff800000u;  // -inf
                }
#pragma unroll
                for (int c = 0; c < 32; ++c) tmax = fmaxf(tmax, __uint_as_float(sa[c]));
            }
            // the two threads of a row exchange their maxima; past this barrier both have finished reading
            // the S buffer, which the P stores below overwrite (every softmax warp takes part, also after a
            // failed wait, so that the barrier count stays whole)
            A5_MARK(1);
            s_xch[half][r] = tmax;
            asm volatile("bar.sync 1, %0;" ::"n"(A5_SOFT) : "memory");
            tmax = fmaxf(tmax, s_xch[half ^ 1][r]);
            if (threadIdx.x == 0) s_go = !*abort_flag;  // every failed wait of this iteration set the flag before the barrier
            asm volatile("bar.sync 1, %0;" ::"n"(A5_SOFT) : "memory");  // the exchange slots are free again
            if (!s_go) {
                ok = false;
                break;
            }
            A5_MARK(2);
            const float m_new = fmaxf(m_run, tmax);  // finite from the first tile on: key 0 is visible to every row
            const float alpha = a5_exp2(m_run - m_new);
            float sum = 0.f;
            uint32_t ph[16], pl[16];
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                const float e0 = a5_exp2(__uint_as_float(sa[2 * c]) - m_new), e1 = a5_exp2(__uint_as_float(sa[2 * c + 1]) - m_new);
                sum += e0 + e1;
                a5_split2(e0, e1, ph[c], pl[c]);  // keys 32 half + 2 c, + 1 -> column 16 half + c
            }
            A5_MARK(3);
            a5_st16(sbuf + (uint32_t)half * 16u, ph);        // P hi: 64 bf16 in columns [0, 32) of the S buffer
            a5_st16(sbuf + 32u + (uint32_t)half * 16u, pl);  // P lo: columns [32, 64)
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(a5_smem(&s_pfull[j & 1])) : "memory");
            l_run = l_run * alpha + sum;
            m_run = m_new;
            A5_MARK(4);
            // the previous tile's P V has been running meanwhile: fold it in now
            if (j > 0) ok = accumulate(j - 1, alpha_prev);
            alpha_prev = alpha;
        }
        if (ok && ntiles > 0) ok = accumulate(ntiles - 1, alpha_prev);
#ifdef RB_TRACE
        if (a5_traced) {
            tr.t[7] = (unsigned long long)ntiles;
            RB_TRACE_COMMIT(tr, 500);
        }
        RB_STAMP(tr2, 2);
#endif
        // the row's sum is the sum of its two halves (same running maximum in both)
        s_xch[half][r] = l_run;
        asm volatile("bar.sync 1, %0;" ::"n"(A5_SOFT) : "memory");
        l_run += s_xch[half ^ 1][r];
        if (__all_sync(0xffffffffu, ok)) {
            // A lane holds 64 consecutive outputs of ONE row, so a 16-byte store instruction of the warp would
            // touch 32 different lines.  The rows cross a per-warp block of the K ring (idle: every MMA has
            // completed) and leave as 256-byte pieces, two rows per instruction.
            const float inv = 1.0f / l_run;
            const uint32_t blk = kring + (uint32_t)warp * (32u * 272u);
#pragma unroll
            for (int i = 0; i < A5_D / 2; i += 4)
                asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(blk + (uint32_t)lane * 272u + 4u * i),
                             "f"(o[i] * inv), "f"(o[i + 1] * inv), "f"(o[i + 2] * inv), "f"(o[i + 3] * inv)
                             : "memory");
            __syncwarp();
#pragma unroll
            for (int k = 0; k < 16; ++k) {
                const int rr = 2 * k + (lane >> 4), chunk = lane & 15;
                float4 w;
                asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                             : "=f"(w.x), "=f"(w.y), "=f"(w.z), "=f"(w.w)
                             : "r"(blk + (uint32_t)rr * 272u + 16u * chunk));
                const int r2 = wq * 32 + rr, srow2 = s0 + r2 / G, gi2 = r2 - (r2 / G) * G;
                if (srow2 < p.seq)
                    *reinterpret_cast<float4*>(p.out + ((size_t)b * p.seq + srow2) * p.n_heads * A5_D +
                                               (size_t)(hk * G + gi2) * A5_D + half * 64 + 4 * chunk) = w;
            }
        } else if (ok && srow < p.seq) {
            const float inv = 1.0f / l_run;
            float* op = p.out + ((size_t)b * p.seq + srow) * p.n_heads * A5_D + (size_t)(hk * G + gi) * A5_D + half * 64;
#pragma unroll
            for (int i = 0; i < A5_D / 2; i += 4)
                *reinterpret_cast<float4*>(op + i) = make_float4(o[i] * inv, o[i + 1] * inv, o[i + 2] * inv, o[i + 3] * inv);
        }
    } else if (warp == 8) {
        // ---------------- K tiles by TMA
        if (lane == 0) {
            const int krow0 = ((b * p.n_kv_heads + hk) * p.split_seq);
            for (int j = 0; j < ntiles; ++j) {
                const int s = j & 1;
                if (!a5_wait(a5_smem(&s_kempty[s]), ((uint32_t)(j >> 1) & 1u) ^ 1u, abort_flag, p.status, 0x7b000003u)) break;
                const uint32_t bar = a5_smem(&s_kfull[s]);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(A5_K_BYTES) : "memory");
                const uint32_t st = kring + (uint32_t)s * A5_K_BYTES;
                const int krow = krow0 + j * A5_BN;
#pragma unroll
                for (int pn = 0; pn < 2; ++pn) {
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                            st + (uint32_t)pn * 8192u),
                        "l"(&tm_kh), "r"(pn * 64), "r"(krow), "r"(bar)
                        : "memory");
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                            st + 16384u + (uint32_t)pn * 8192u),
                        "l"(&tm_kl), "r"(pn * 64), "r"(krow), "r"(bar)
                        : "memory");
                }
            }
        }
    } else if (warp == 9) {
        // ---------------- V^T tiles by TMA
        if (lane == 0) {
            const int vrow0 = ((b * p.n_kv_heads + hk) * (p.split_seq / A5_BN)) * A5_D;
            for (int j = 0; j < ntiles; ++j) {
                const int s = j & 1;
                if (!a5_wait(a5_smem(&s_vempty[s]), ((uint32_t)(j >> 1) & 1u) ^ 1u, abort_flag, p.status, 0x7b000009u)) break;
                const uint32_t bar = a5_smem(&s_vfull[s]);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(A5_V_BYTES) : "memory");
                const uint32_t st = vring + (uint32_t)s * A5_V_BYTES;
                const int vrow = vrow0 + j * A5_D;
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(st),
                    "l"(&tm_vh), "r"(0), "r"(vrow), "r"(bar)
                    : "memory");
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                        st + 16384u),
                    "l"(&tm_vl), "r"(0), "r"(vrow), "r"(bar)
                    : "memory");
            }
        }
    } else {
        // ---------------- MMA issue
        if (lane == 0) {
            // kind::f16: float32 accumulate (bit 4), A and B bf16 (bits 7, 10), both K-major, N >> 3 at 17, M >> 4 at 24
            const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(A5_BN >> 3) << 17) | ((128u >> 4) << 24);
            const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(A5_D >> 3) << 17) | ((128u >> 4) << 24);
            // One thread issues every MMA of the CTA, so its instruction count per MMA bounds the tensor pipe:
            // the descriptors of a tile are its base descriptor plus compile-time constants (the address field
            // counts 16-byte units and no operand crosses the field's range), nothing is recomputed per MMA.
            const uint64_t dq_hi = a5_desc(q_hi), dq_lo = a5_desc(q_lo);
            auto issue_s = [&](int j) {
                const uint64_t dk_hi = a5_desc(kring + (uint32_t)(j & 1) * A5_K_BYTES), dk_lo = dk_hi + (16384u >> 4);
                const uint32_t d = tmem + (uint32_t)(j & 1) * 64u;
#pragma unroll
                for (int term = 0; term < 3; ++term)
#pragma unroll
                    for (int k16 = 0; k16 < A5_D / 16; ++k16) {
                        const uint64_t qo = (uint64_t)(((k16 >> 2) * 16384 + (k16 & 3) * 32) >> 4);
                        const uint64_t ko = (uint64_t)(((k16 >> 2) * 8192 + (k16 & 3) * 32) >> 4);
                        const uint64_t da = (term == 2 ? dq_lo : dq_hi) + qo, db = (term == 1 ? dk_lo : dk_hi) + ko;
                        if (term == 0 && k16 == 0)
                            a5_mma_ss<0>(d, da, db, idesc_s);
                        else
                            a5_mma_ss<1>(d, da, db, idesc_s);
                    }
            };
            auto issue_pv = [&](int j) {
                const uint64_t dv_hi = a5_desc(vring + (uint32_t)(j & 1) * A5_V_BYTES), dv_lo = dv_hi + (16384u >> 4);
                const uint32_t pbase = tmem + (uint32_t)(j & 1) * 64u, d = tmem + 128u + (uint32_t)(j & 1) * 128u;
#pragma unroll
                for (int term = 0; term < 3; ++term)
#pragma unroll
                    for (int k16 = 0; k16 < A5_BN / 16; ++k16) {
                        const uint32_t pa = pbase + (term == 2 ? 32u : 0u) + (uint32_t)k16 * 8u;
                        const uint64_t db = (term == 1 ? dv_lo : dv_hi) + (uint64_t)((k16 * 32) >> 4);
                        if (term == 0 && k16 == 0)
                            a5_mma_ts<0>(d, pa, db, idesc_o);
                        else
                            a5_mma_ts<1>(d, pa, db, idesc_o);
                    }
            };
            bool ok = a5_wait(a5_smem(&s_qready), 0, abort_flag, p.status, 0x7b000004u);
            if (ok && ntiles > 0) {
                ok = a5_wait(a5_smem(&s_kfull[0]), 0, abort_flag, p.status, 0x7b000005u);
                if (ok) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    issue_s(0);
                    a5_commit(a5_smem(&s_sfull[0]));
                    a5_commit(a5_smem(&s_kempty[0]));
                }
            }
            for (int j = 0; j < ntiles && ok; ++j) {
                if (j + 1 < ntiles) {
                    ok = a5_wait(a5_smem(&s_kfull[(j + 1) & 1]), (uint32_t)((j + 1) >> 1) & 1u, abort_flag, p.status, 0x7b000006u);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    issue_s(j + 1);
                    a5_commit(a5_smem(&s_sfull[(j + 1) & 1]));
                    a5_commit(a5_smem(&s_kempty[(j + 1) & 1]));
                }
                ok = a5_wait(a5_smem(&s_pfull[j & 1]), (uint32_t)(j >> 1) & 1u, abort_flag, p.status, 0x7b000007u);
                if (ok) ok = a5_wait(a5_smem(&s_oempty[j & 1]), ((uint32_t)(j >> 1) & 1u) ^ 1u, abort_flag, p.status, 0x7b000008u);
                if (ok) ok = a5_wait(a5_smem(&s_vfull[j & 1]), (uint32_t)(j >> 1) & 1u, abort_flag, p.status, 0x7b00000au);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                issue_pv(j);
                a5_commit(a5_smem(&s_ofull[j & 1]));
                a5_commit(a5_smem(&s_vempty[j & 1]));
            }
        }
    }

#ifdef RB_TRACE
    if (warp < 8) {
        RB_STAMP(tr2, 3);
        RB_TRACE_COMMIT(tr2, 501);
    }
#endif
    // ---------------- common exit: nothing of this CTA may still be in flight when it returns
    if (*abort_flag && threadIdx.x == 0) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {
        }  // about a millisecond for copies already issued to land
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 8) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(A5_TMEM_COLS));
    }
}

typedef CUresult (*A5EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static A5EncodeFn g_a5_encode = nullptr;
static PerDevice<bool> g_a5_ready;

int configure_attn_prefill_t5() {
    if (g_a5_ready.here()) return ROTOR_B200_OK;
    if (!g_a5_encode) {
        cudaDriverEntryPointQueryResult q;
        void* fn = nullptr;
        RB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
        if (!fn || q != cudaDriverEntryPointSuccess) return ROTOR_B200_ERR_CUDA;
        g_a5_encode = (A5EncodeFn)fn;
    }
    RB_CUDA(cudaFuncSetAttribute(attn_prefill_t5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, A5_SMEM));
    g_a5_ready.here() = true;
    return ROTOR_B200_OK;
}

// Shapes the tensor-memory kernel takes: head_dim 128, split planes present (prompts of 16 positions
// and more), a group size that divides the 128-row tile.
bool attn_prefill_t5_supported(const AttnParams& p, int rows) {
    static const bool off = getenv("ROTOR_B200_NO_TCGEN05") != nullptr;  // comparison aid: the mma.sync kernel
    if (off || p.head_dim != A5_D || !p.kv_split || p.seq < 16) return false;
    const int G = p.n_heads / p.n_kv_heads;
    return G >= 1 && G <= A5_BM && A5_BM % G == 0 && rows % p.seq == 0 && ((uintptr_t)p.kv_split & 127) == 0 &&
           ((uintptr_t)p.q & 15) == 0;
}

int launch_attn_prefill_t5(const AttnParams& p, int rows, cudaStream_t st) {
    int rc = configure_attn_prefill_t5();
    if (rc) return rc;
    const int G = p.n_heads / p.n_kv_heads, QT = A5_BM / G;
    const int batch = rows / p.seq;
    const int split_seq = (p.max_seq + A5_BN - 1) / A5_BN * A5_BN;
    if ((size_t)batch * p.n_kv_heads * split_seq * A5_D > p.split_plane) return ROTOR_B200_ERR_WORKSPACE;
    // ---- hi / lo planes of this call's cache rows
    dim3 sgrid(split_seq / A5_BN, p.n_kv_heads, batch);
    kv_split_t5_kernel<<<sgrid, 256, 0, st>>>(p.k_cache, p.v_cache, p.past_len, p.seq, p.max_seq, p.n_kv_heads, split_seq,
                                              p.kv_split, p.split_plane);
    rc = launch_status();
    if (rc) return rc;
    // ---- tensor maps: K planes [rows][128] in boxes of 64 columns x 64 rows, V^T planes [rows][64] in boxes of 64 x 128
    CUtensorMap tm[4];
    const cuuint64_t krows = (cuuint64_t)batch * p.n_kv_heads * split_seq;
    const cuuint64_t vrows = (cuuint64_t)batch * p.n_kv_heads * (split_seq / A5_BN) * A5_D;
    const cuuint32_t estride[2] = {1u, 1u};
    for (int i = 0; i < 4; ++i) {
        const bool is_v = i >= 2;
        const cuuint64_t gdim[2] = {(cuuint64_t)(is_v ? A5_BN : A5_D), is_v ? vrows : krows};
        const cuuint64_t gstride[1] = {(cuuint64_t)(is_v ? A5_BN : A5_D) * 2};
        const cuuint32_t box[2] = {64u, is_v ? 128u : 64u};
        void* ptr = (void*)(p.kv_split + (size_t)i * p.split_plane);
        if (g_a5_encode(&tm[i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ptr, gdim, gstride, box, estride,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return ROTOR_B200_ERR_CUDA;
    }
    A5Params a;
    a.q = p.q;
    a.out = p.out;
    a.past_len = p.past_len;
    a.status = library_status_word();
    a.n_heads = p.n_heads;
    a.n_kv_heads = p.n_kv_heads;
    a.seq = p.seq;
    a.max_seq = p.max_seq;
    a.causal = p.causal;
    a.split_seq = split_seq;
    if (!a.status) return ROTOR_B200_ERR_CUDA;
    dim3 grid((p.seq + QT - 1) / QT, p.n_kv_heads, batch);
    attn_prefill_t5_kernel<<<grid, A5_THREADS, A5_SMEM, st>>>(tm[0], tm[1], tm[2], tm[3], a);
    return launch_status();
}

}  // namespace rb
