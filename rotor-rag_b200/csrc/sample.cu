// Temperature / top-k / top-p sampling on the device.
//
// Reference: TopKSampling.sample and TopPSampling.sample, src/rotor/generation.py:45-145 --
// divide the logits by the temperature, keep the k largest (top-k) or the smallest
// probability-sorted prefix whose mass reaches p (top-p), softmax over what is kept, draw one
// token.  The reference draws with np.random.choice from NumPy's global generator; a device
// sampler cannot follow that stream, so the draw here is an explicit inverse-CDF lookup with a
// counter-based uniform (SplitMix64 of seed and counter), and the kept tokens are walked in
// vocabulary order instead of probability order.  The distribution over tokens is the
// reference's; which token a given uniform maps to is this file's own, documented, choice.
//
// One CTA of 1024 threads per row of logits.  No sort: the cut (k-th largest value, or the value
// at which the descending mass reaches p) is found by a four-pass radix select over the bit
// pattern of e_i = exp(logit_i / T - max), one 256-bin histogram of counts and masses per pass.
// Values equal to the cut are admitted in vocabulary order until the count (top-k) or the mass
// (top-p) is reached.  Then one block-wide prefix sum over the kept masses locates the drawn
// token.
#include "model.cuh"

namespace rb {

constexpr int SMP_THREADS = 1024;

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

struct SampleParams {
    const float* logits;  // [rows][vocab]
    int vocab;
    int mode;             // 0 top-k, 1 top-p
    int top_k;
    float top_p;
    float temperature;
    unsigned long long seed, counter;
    long long* out;       // [rows]
};

__global__ void __launch_bounds__(SMP_THREADS) sample_kernel(const __grid_constant__ SampleParams p) {
    __shared__ float s_red[64];
    __shared__ unsigned s_cnt[256];
    // bin masses in 2^-40 fixed point: integer atomics add in any order to the same bits, so the cut (and with it
    // the drawn token) does not depend on which thread's atomic lands first
    __shared__ unsigned long long s_mass[256];
    __shared__ unsigned s_prefix;      // bit prefix of the cut found so far
    __shared__ unsigned s_cnt_above;   // tokens strictly above the current prefix range
    __shared__ unsigned long long s_mass_above;
    __shared__ unsigned s_scan_u[SMP_THREADS / 32];
    __shared__ float s_scan_f[SMP_THREADS / 32];
    __shared__ int s_token;
    const int row = blockIdx.x, V = p.vocab, tid = threadIdx.x;
    const float* lg = p.logits + (size_t)row * V;
    const float T = p.temperature;
    auto scaled = [&](int i) { return T != 1.0f ? __fdiv_rn(lg[i], T) : lg[i]; };

    // ---- maximum, then total mass
    float mx = -INFINITY;
    for (int i = tid; i < V; i += SMP_THREADS) mx = fmaxf(mx, scaled(i));
    mx = block_max(mx, s_red);
    auto e_of = [&](int i) { return expf(scaled(i) - mx); };
    float z = 0.f;
    for (int i = tid; i < V; i += SMP_THREADS) z += e_of(i);
    z = block_sum(z, s_red);

    // ---- radix select of the cut over the bits of e (positive floats order like their bits)
    const double fix = 1099511627776.0;                  // 2^40; e <= 1, so a bin sum stays far below 2^63
    const unsigned long long want_mass = (unsigned long long)((double)p.top_p * (double)z * fix);  // top-p: descending mass to reach
    const unsigned want_cnt = (unsigned)(p.top_k < V ? p.top_k : V);  // top-k
    if (tid == 0) {
        s_prefix = 0;
        s_cnt_above = 0;
        s_mass_above = 0ull;
    }
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        if (tid < 256) {
            s_cnt[tid] = 0;
            s_mass[tid] = 0ull;
        }
        __syncthreads();
        const unsigned prefix = s_prefix;
        const unsigned himask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
        for (int i = tid; i < V; i += SMP_THREADS) {
            const float e = e_of(i);
            const unsigned b = __float_as_uint(e);
            if ((b & himask) == prefix) {
                const unsigned bin = (b >> shift) & 255u;
                atomicAdd(&s_cnt[bin], 1u);
                atomicAdd(&s_mass[bin], (unsigned long long)((double)e * fix));
            }
        }
        __syncthreads();
        if (tid == 0) {  // walk the bins from the largest values down
            unsigned cnt = s_cnt_above;
            unsigned long long mass = s_mass_above;
            int bin = 255;
            for (; bin > 0; --bin) {
                const bool reached = p.mode == 0 ? (cnt + s_cnt[bin] >= want_cnt) : (mass + s_mass[bin] >= want_mass);
                if (reached) break;
                cnt += s_cnt[bin];
                mass += s_mass[bin];
            }
            s_cnt_above = cnt;
            s_mass_above = mass;
            s_prefix = prefix | ((unsigned)bin << shift);
        }
        __syncthreads();
    }
    const unsigned cut = s_prefix;            // bit pattern of the cut value
    const float cut_e = __uint_as_float(cut);
    // how many tokens equal to the cut are admitted (vocabulary order)
    unsigned ties_wanted;
    if (p.mode == 0) {
        ties_wanted = want_cnt - s_cnt_above;
    } else {
        const double missing = want_mass > s_mass_above ? (double)(want_mass - s_mass_above) / fix : 0.0;
        ties_wanted = cut_e > 0.f ? (unsigned)ceil(missing / (double)cut_e) : 1u;
        if (ties_wanted < 1u) ties_wanted = 1u;
    }

    // ---- kept set in vocabulary order: contiguous chunk per thread
    const int chunk = (V + SMP_THREADS - 1) / SMP_THREADS;
    const int i0 = tid * chunk, i1 = min(V, i0 + chunk);
    unsigned my_ties = 0;
    for (int i = i0; i < i1; ++i) my_ties += __float_as_uint(e_of(i)) == cut ? 1u : 0u;
    // exclusive scan of the tie counts
    const int lane = tid & 31, warp = tid >> 5;
    unsigned incl = my_ties;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) s_scan_u[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        unsigned w = s_scan_u[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned v = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += v;
        }
        s_scan_u[lane] = w;
    }
    __syncthreads();
    unsigned ties_before = incl - my_ties + (warp ? s_scan_u[warp - 1] : 0u);
    // kept mass of this chunk
    float my_mass = 0.f;
    {
        unsigned tb = ties_before;
        for (int i = i0; i < i1; ++i) {
            const float e = e_of(i);
            const unsigned b = __float_as_uint(e);
            if (b > cut || (b == cut && tb++ < ties_wanted)) my_mass += e;
        }
    }
    float incl_m = my_mass;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float v = __shfl_up_sync(0xffffffffu, incl_m, o);
        if (lane >= o) incl_m += v;
    }
    if (lane == 31) s_scan_f[warp] = incl_m;
    if (tid == 0) s_token = -1;
    __syncthreads();
    if (warp == 0) {
        float w = s_scan_f[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float v = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += v;
        }
        s_scan_f[lane] = w;
    }
    __syncthreads();
    const float total = s_scan_f[SMP_THREADS / 32 - 1];
    const float upto = incl_m + (warp ? s_scan_f[warp - 1] : 0.f);  // kept mass up to and including this chunk
    const float before = upto - my_mass;
    const bool last_owner = upto >= total;  // the last chunk with any mass also takes what rounding leaves over

    // ---- draw: uniform in [0,1) from the top 24 bits of SplitMix64(seed, counter + row)
    const unsigned long long r = splitmix64(p.seed ^ splitmix64(p.counter + (unsigned long long)row));
    const float u = (float)(r >> 40) * (1.0f / 16777216.0f);
    const float target = u * total;
    if (my_mass > 0.f && target >= before && (target < upto || last_owner)) {
        float acc = before;
        unsigned tb = ties_before;
        int pick = -1;
        for (int i = i0; i < i1; ++i) {
            const float e = e_of(i);
            const unsigned b = __float_as_uint(e);
            if (b > cut || (b == cut && tb++ < ties_wanted)) {
                pick = i;  // the last kept token of the chunk takes what rounding leaves over
                acc += e;
                if (target < acc) break;
            }
        }
        s_token = pick;
    }
    __syncthreads();
    if (tid == 0) {
        p.out[row] = s_token < 0 ? 0 : s_token;  // (a token is always found; 0 guards degenerate input such as NaN)
    }
}

}  // namespace rb

using namespace rb;

/* Draws one token per row of logits.  mode 0: top-k (k = top_k), mode 1: top-p (p = top_p).
 * The uniform of row r is derived from (seed, counter + r): pass a fresh counter per step. */
extern "C" int rotor_b200_sample(const float* logits, int rows, int vocab, int mode, int top_k, float top_p,
                                 float temperature, uint64_t seed, uint64_t counter, int64_t* out, void* stream) {
    RB_REQUIRE(logits && out && rows > 0 && vocab > 0 && (mode == 0 || mode == 1));
    RB_REQUIRE(temperature > 0.f && (mode == 1 || top_k > 0) && (mode == 0 || (top_p > 0.f && top_p <= 1.0f)));
    SampleParams p;
    p.logits = logits;
    p.vocab = vocab;
    p.mode = mode;
    p.top_k = top_k;
    p.top_p = top_p;
    p.temperature = temperature;
    p.seed = seed;
    p.counter = counter;
    p.out = (long long*)out;
    sample_kernel<<<rows, SMP_THREADS, 0, as_stream(stream)>>>(p);
    return launch_status();
}
