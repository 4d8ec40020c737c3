// Stand-alone activation quantiser (one CTA per token row).
#include "quant.cuh"

namespace rb {

__global__ void __launch_bounds__(1024) quantize_rows_kernel(const float* __restrict__ x, int k, int kpad,
                                                             int terms, int8_t* __restrict__ xq,
                                                             float* __restrict__ sx, int32_t* __restrict__ xsum) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* scratch = reinterpret_cast<float*>(smem_raw);
    float* row = scratch + 64;
    const size_t m = blockIdx.x;
    for (int i = threadIdx.x; i < k; i += blockDim.x) row[i] = x[m * k + i];
    __syncthreads();
    quantize_row_from_smem(row, k, kpad, terms, xq + m * terms * (size_t)kpad, sx + m * terms,
                           xsum + m * terms, scratch);
}

}  // namespace rb

using namespace rb;

extern "C" int rotor_b200_quantize_rows(const float* x, size_t m, size_t k, int terms, int8_t* xq, float* sx,
                                        int32_t* xsum, void* stream) {
    RB_REQUIRE(x && xq && sx && xsum && m > 0 && k > 0 && terms >= 1 && terms <= 4);
    RB_REQUIRE(k <= 49152 && m < (1u << 31));
    RB_REQUIRE(((uintptr_t)xq & 3) == 0);
    const size_t smem = 64 * 4 + k * 4;
    if (smem > 48 * 1024) {
        static PerDevice<bool> once;
        bool& configured = once.here();
        if (!configured) {
            RB_CUDA(cudaFuncSetAttribute(quantize_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         64 * 4 + 49152 * 4));
            configured = true;
        }
    }
    const int threads = k >= 4096 ? 1024 : (k >= 1024 ? 512 : 128);
    quantize_rows_kernel<<<(unsigned)m, threads, smem, as_stream(stream)>>>(x, (int)k, (int)kpad_of(k), terms,
                                                                           xq, sx, xsum);
    return launch_status();
}
