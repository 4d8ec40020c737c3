// One generation step in ONE cooperative launch.
//
// The step's products, attention and LM head are the same device bodies the per-kernel
// path uses (product_body.cuh, attn_body.cuh, lmhead_body.cuh), run by a persistent grid of
// one 1024-thread CTA per SM and separated by grid barriers instead of kernel boundaries.
// That removes ~150 launch gaps and cold starts per token, keeps the instruction stream of
// a block hot across the 30 blocks, and lets every warp request the next product's first
// weight tiles before the barrier it is about to wait at, so HBM latency hides behind the
// barrier and the next prologue.
//
// Every barrier wait is bounded (about 50 ms of SM clock); a timeout raises
// ROTOR_B200_ERR_TIMEOUT in the library's status word and all later barriers of the launch
// return at once, so a lost CTA costs a wrong token, never a hung GPU.
#include "attn_body.cuh"
#include "lmhead_body.cuh"
#include "product_body.cuh"

RB_TRACE_DEFINE(rotor_b200_trace_read_mega)

namespace rb {

int configure_mega();

struct MegaLayer {            // plan of one block, resident in device memory
    FusedGemvParams prod[4];  // q/k/v, o, gate/up, down
    AttnDecodeParams attn;
};

struct MegaParams {
    const MegaLayer* layers;
    int n_layers;
    int batch;
    int head_dim;
    LmHeadParams lm;
    unsigned* bar;     // [0] arrivals, [1] generation
    unsigned* status;
};

__device__ __forceinline__ void grid_barrier(unsigned* bar, unsigned* status, int* s_dead) {
    __syncthreads();
    if (threadIdx.x == 0 && !*s_dead) {
        __threadfence();
        const unsigned gen = *reinterpret_cast<volatile unsigned*>(bar + 1);
        if (atomicAdd(bar, 1u) + 1u == gridDim.x) {
            *reinterpret_cast<volatile unsigned*>(bar) = 0u;
            __threadfence();
            atomicAdd(bar + 1, 1u);
        } else {
            const long long start = clock64();
            while (*reinterpret_cast<volatile unsigned*>(bar + 1) == gen) {
                if (clock64() - start > 100000000LL) {  // ~50 ms: give up, report, stop waiting for good
                    atomicMax(status, (unsigned)ROTOR_B200_ERR_TIMEOUT);
                    *s_dead = 1;
                    break;
                }
            }
        }
        __threadfence();
    }
    __syncthreads();
}

template <typename T>
__device__ __forceinline__ void copy_params(T* dst, const T* src) {
    static_assert(sizeof(T) % 4 == 0, "parameter blocks are copied as 32-bit words");
    const unsigned* s = reinterpret_cast<const unsigned*>(src);
    unsigned* d = reinterpret_cast<unsigned*>(dst);
    for (int i = threadIdx.x; i < (int)(sizeof(T) / 4); i += blockDim.x) d[i] = __ldg(s + i);
}

template <bool USE_MMA, int NCOL>
__global__ void __launch_bounds__(FG_THREADS, 1) decode_step_kernel(const __grid_constant__ MegaParams mp) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ float s_sx[8];
    __shared__ int s_xsum[8];
    __shared__ FusedGemvParams sp;
    __shared__ AttnDecodeParams sa;
    __shared__ int s_dead;
    if (threadIdx.x == 0) s_dead = 0;

    uint4 wv[FG_U];
    copy_params(&sp, &mp.layers[0].prod[0]);
    __syncthreads();
    ProductCtx c = product_ctx(sp, smem_raw);
    product_prefetch(sp, c, wv);

    for (int l = 0; l < mp.n_layers; ++l) {
        for (int i = 0; i < 4; ++i) {
            TraceRec tr;
            RB_STAMP(tr, 0);
            if (i == 1) {
                // attention sits between the q/k/v and the o product (whose tiles are already on their way)
                grid_barrier(mp.bar, mp.status, &s_dead);
                RB_STAMP(tr, 1);
                copy_params(&sa, &mp.layers[l].attn);
                __syncthreads();
                const int per_seq = sa.n_kv_heads * sa.nsplit;
                for (int item = blockIdx.x; item < per_seq * mp.batch; item += gridDim.x) {
                    if (threadIdx.x < 128) {  // one 128-thread group per work item, on its own named barrier
                        auto gsync = [] { asm volatile("bar.sync 1, 128;" ::: "memory"); };
                        float* sm = reinterpret_cast<float*>(smem_raw);
                        const int b = item / per_seq, ix = item - b * per_seq;
                        switch (mp.head_dim) {
                            case 32: attn_decode_body<32>(sa, ix, b, sm, threadIdx.x, 128, gsync); break;
                            case 64: attn_decode_body<64>(sa, ix, b, sm, threadIdx.x, 128, gsync); break;
                            default: attn_decode_body<128>(sa, ix, b, sm, threadIdx.x, 128, gsync); break;
                        }
                        gsync();
                    }
                }
            }
            RB_STAMP(tr, 2);
            grid_barrier(mp.bar, mp.status, &s_dead);  // everything this product reads is complete
            RB_STAMP(tr, 3);
            product_run<USE_MMA, NCOL>(sp, c, wv, s_sx, s_xsum);
            RB_STAMP(tr, 4);
            // move on: fetch the next product's plan and request its first tiles
            const int ni = i == 3 ? 0 : i + 1, nl = i == 3 ? l + 1 : l;
            if (nl < mp.n_layers) {
                __syncthreads();
                copy_params(&sp, &mp.layers[nl].prod[ni]);
                __syncthreads();
                c = product_ctx(sp, smem_raw);
                product_prefetch(sp, c, wv);
            }
            RB_STAMP(tr, 5);
            RB_TRACE_COMMIT(tr, i);
        }
    }
    grid_barrier(mp.bar, mp.status, &s_dead);
    float* xs = reinterpret_cast<float*>(smem_raw);
    switch (mp.batch) {
        case 1: lmhead_body<1>(mp.lm, 0, xs); break;
        case 2: lmhead_body<2>(mp.lm, 0, xs); break;
        case 3: lmhead_body<3>(mp.lm, 0, xs); break;
        default: lmhead_body<4>(mp.lm, 0, xs); break;
    }
}

size_t mega_layer_bytes() { return sizeof(MegaLayer); }

// Records one block's plan into host memory laid out like the device array.
int mega_record_layer(void* host_plan, int l, const FusedGemvParams* prod4, const AttnDecodeParams& attn) {
    MegaLayer* ml = static_cast<MegaLayer*>(host_plan) + l;
    for (int i = 0; i < 4; ++i) ml->prod[i] = prod4[i];
    ml->attn = attn;
    return ROTOR_B200_OK;
}

template <bool USE_MMA, int NCOL>
static int launch_mega(const MegaParams& mp, size_t smem, int grid, cudaStream_t st) {
    auto kern = decode_step_kernel<USE_MMA, NCOL>;
    static bool configured = false;
    if (!configured) {
        RB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(FG_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;  // all CTAs resident together, or the launch fails
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kern, mp) != cudaSuccess) {
        ++g_launch_count;
        return ROTOR_B200_ERR_CUDA;
    }
    return launch_status();
}

// Whether the device can run the step kernel for `cols` activation columns with `smem` bytes
// of dynamic shared memory on a grid of `grid` CTAs, all resident at once.
template <bool USE_MMA, int NCOL>
static bool mega_fits(size_t smem, int grid) {
    int dev = 0, coop = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return false;
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (!coop) return false;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_step_kernel<USE_MMA, NCOL>, FG_THREADS, smem) !=
        cudaSuccess)
        return false;
    return per_sm >= 1 && grid <= per_sm * sms;
}

static size_t mega_smem(const void* host_plan, int n_layers, int batch, int d, int* cols_out) {
    const MegaLayer* hl = static_cast<const MegaLayer*>(host_plan);
    size_t smem = (size_t)batch * d * sizeof(float);
    int cols = 1;
    for (int l = 0; l < n_layers; ++l) {
        for (int i = 0; i < 4; ++i) {
            const size_t s = fused_smem(hl[l].prod[i]);
            if (s > smem) smem = s;
            cols = hl[l].prod[i].cols;
        }
        const AttnDecodeParams& a = hl[l].attn;
        const int G = a.n_heads / a.n_kv_heads, lcmax = (a.max_seq + a.nsplit - 1) / a.nsplit;
        const size_t s = ((size_t)G * a.head_dim + 2 * a.head_dim + (size_t)G * lcmax + 64) * sizeof(float);
        if (s > smem) smem = s;
    }
    *cols_out = cols;
    return smem;
}

bool mega_supported(const void* host_plan, int n_layers, int batch, int d, int grid) {
    int cols = 1;
    const size_t smem = mega_smem(host_plan, n_layers, batch, d, &cols);
    if (smem > 200 * 1024 || configure_mega() != ROTOR_B200_OK) return false;
    if (cols == 1) return mega_fits<false, 1>(smem, grid);
    if (cols == 2) return mega_fits<false, 2>(smem, grid);
    return mega_fits<true, 1>(smem, grid);
}

int configure_mega() {
    RB_CUDA(cudaFuncSetAttribute(decode_step_kernel<false, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    RB_CUDA(cudaFuncSetAttribute(decode_step_kernel<false, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    RB_CUDA(cudaFuncSetAttribute(decode_step_kernel<true, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    return ROTOR_B200_OK;
}

// dev_plan: device array of n_layers MegaLayer; host_plan: the same on the host (for sizing).
int launch_decode_step_mega(const void* dev_plan, const void* host_plan, int n_layers, int batch, int head_dim,
                            const LmHeadParams& lm, unsigned* bar, unsigned* status, int grid, cudaStream_t st) {
    MegaParams mp = {};
    mp.layers = static_cast<const MegaLayer*>(dev_plan);
    mp.n_layers = n_layers;
    mp.batch = batch;
    mp.head_dim = head_dim;
    mp.lm = lm;
    mp.bar = bar;
    mp.status = status;
    int cols = 1;
    const size_t smem = mega_smem(host_plan, n_layers, batch, lm.d, &cols);
    if (smem > 200 * 1024) return ROTOR_B200_ERR_SHAPE;
    if (cols == 1) return launch_mega<false, 1>(mp, smem, grid, st);
    if (cols == 2) return launch_mega<false, 2>(mp, smem, grid, st);
    return launch_mega<true, 1>(mp, smem, grid, st);
}

}  // namespace rb
