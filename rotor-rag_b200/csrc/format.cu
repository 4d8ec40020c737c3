// Rotor 2-bit format kernels: element flags, packed <-> planes <-> int8, and the
// load-time repack into the GPU tile layout described in include/rotor_b200.h.
// All of this is byte/bit shuffling bound by HBM traffic; one thread per output
// word keeps stores coalesced.
#include <cstdio>
#include <cstdlib>

#include "common.cuh"

namespace rb {

unsigned long long g_launch_count = 0;

__global__ void encode_kernel(const int8_t* __restrict__ w, size_t n, uint8_t* __restrict__ plus,
                              uint8_t* __restrict__ minus) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        int8_t v = w[i];
        plus[i] = v == 1;
        minus[i] = v == -1;
    }
}

__global__ void decode_kernel(const uint8_t* __restrict__ plus, const uint8_t* __restrict__ minus, size_t n,
                              int8_t* __restrict__ w) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        w[i] = (int8_t)((int)plus[i] - (int)minus[i]);
}

__global__ void pack_kernel(const uint8_t* __restrict__ plus, const uint8_t* __restrict__ minus, size_t nbytes,
                            uint8_t* __restrict__ packed) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nbytes; i += (size_t)gridDim.x * blockDim.x) {
        unsigned v = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            v |= (unsigned)(plus[4 * i + j] & 1u) << (2 * j + 1);
            v |= (unsigned)(minus[4 * i + j] & 1u) << (2 * j);
        }
        packed[i] = (uint8_t)v;
    }
}

__global__ void unpack_kernel(const uint8_t* __restrict__ packed, size_t n, uint8_t* __restrict__ plus,
                              uint8_t* __restrict__ minus) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        unsigned f = (packed[i >> 2] >> (2 * (i & 3))) & 3u;
        plus[i] = (uint8_t)(f >> 1);
        minus[i] = (uint8_t)(f & 1u);
    }
}

// One thread per plane byte (8 weights = 2 packed bytes).
__global__ void packed_to_planes_kernel(const uint8_t* __restrict__ packed, size_t rows, size_t cols,
                                        uint8_t* __restrict__ plus, uint8_t* __restrict__ minus) {
    const size_t sstride = (cols + 3) / 4, dstride = (cols + 7) / 8;
    const size_t total = rows * dstride;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / dstride, b = i % dstride;
        unsigned p = 0, m = 0;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            size_t c = b * 8 + e;
            if (c < cols) {
                unsigned f = (packed[r * sstride + (c >> 2)] >> (2 * (c & 3))) & 3u;
                p |= (unsigned)(f == 2u) << e;
                m |= (unsigned)(f == 1u) << e;
            }
        }
        plus[i] = (uint8_t)p;
        minus[i] = (uint8_t)m;
    }
}

__global__ void planes_to_int8_kernel(const uint8_t* __restrict__ plus, const uint8_t* __restrict__ minus,
                                      size_t rows, size_t cols, int8_t* __restrict__ w) {
    const size_t stride = (cols + 7) / 8, total = rows * cols;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / cols, c = i % cols;
        int p = (plus[r * stride + (c >> 3)] >> (c & 7)) & 1;
        int m = (minus[r * stride + (c >> 3)] >> (c & 7)) & 1;
        w[i] = (int8_t)(p - m);
    }
}

// Tile addressing: word index -> (row, first column, column step pattern).
struct TileWord {
    size_t row;
    size_t kbase;  // column of byte 0, pair 0
};
__device__ __forceinline__ TileWord tile_word(size_t widx, size_t nkt) {
    const unsigned i = widx & 3u;
    const unsigned lane = (widx >> 2) & 31u;
    const size_t tile = widx >> 7;
    const size_t rt = tile / nkt, kt = tile % nkt;
    const unsigned g = lane >> 2, t = lane & 3u;
    TileWord tw;
    tw.row = rt * TILE_ROWS + g + 8u * (i & 1u);
    tw.kbase = kt * TILE_K + 32u * t + 4u * (i >> 1);
    return tw;  // column of (byte b, pair j) = kbase + 8*j + b
}

template <bool FROM_PACKED>
__global__ void to_tiles_kernel(const uint8_t* __restrict__ src, size_t out, size_t in,
                                uint32_t* __restrict__ tiles) {
    const size_t nkt = kpad_of(in) / TILE_K;
    const size_t total = opad_of(out) / TILE_ROWS * nkt * 128;
    const size_t sstride = (in + 3) / 4;
    for (size_t widx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; widx < total;
         widx += (size_t)gridDim.x * blockDim.x) {
        TileWord tw = tile_word(widx, nkt);
        uint32_t word = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const size_t k = tw.kbase + 8 * j + b;
                unsigned code = 1u;  // padding = weight 0
                if (tw.row < out && k < in) {
                    if (FROM_PACKED) {
                        unsigned f = (src[tw.row * sstride + (k >> 2)] >> (2 * (k & 3))) & 3u;
                        code = f == 2u ? 2u : (f == 1u ? 0u : 1u);
                    } else {
                        int v = ((const int8_t*)src)[tw.row * in + k];
                        code = v > 0 ? 2u : (v < 0 ? 0u : 1u);
                    }
                }
                word |= code << (8 * b + 2 * j);
            }
        }
        tiles[widx] = word;
    }
}

__global__ void tiles_to_int8_kernel(const uint32_t* __restrict__ tiles, size_t out, size_t in,
                                     int8_t* __restrict__ w) {
    const size_t nkt = kpad_of(in) / TILE_K;
    const size_t total = opad_of(out) / TILE_ROWS * nkt * 128;
    for (size_t widx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; widx < total;
         widx += (size_t)gridDim.x * blockDim.x) {
        TileWord tw = tile_word(widx, nkt);
        const uint32_t word = tiles[widx];
        if (tw.row >= out) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const size_t k = tw.kbase + 8 * j + b;
                if (k < in) w[tw.row * in + k] = (int8_t)((int)((word >> (8 * b + 2 * j)) & 3u) - 1);
            }
    }
}

static inline unsigned grid_for(size_t n, unsigned block = 256) {
    size_t g = (n + block - 1) / block;
    const size_t cap = 148 * 32;
    return (unsigned)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace rb

using namespace rb;

extern "C" {

int rotor_b200_version(void) { return 100; }

unsigned long long rotor_b200_launch_count(void) { return g_launch_count; }

const char* rotor_b200_status_string(int status) {
    switch (status) {
        case ROTOR_B200_OK: return "ok";
        case ROTOR_B200_ERR_ARG: return "invalid argument";
        case ROTOR_B200_ERR_CUDA: return "CUDA error";
        case ROTOR_B200_ERR_SHAPE: return "unsupported shape";
        case ROTOR_B200_ERR_WORKSPACE: return "workspace too small";
        case ROTOR_B200_ERR_TIMEOUT: return "device-side wait timed out";
        case ROTOR_B200_ERR_TOO_LARGE: return "problem exceeds the library's built-in scratch array";
        default: return "unknown status";
    }
}

int rotor_b200_encode(const int8_t* w, size_t n, uint8_t* plus, uint8_t* minus, void* stream) {
    if (n == 0) return ROTOR_B200_OK;
    RB_REQUIRE(w && plus && minus);
    encode_kernel<<<grid_for(n), 256, 0, as_stream(stream)>>>(w, n, plus, minus);
    return launch_status();
}

int rotor_b200_decode(const uint8_t* plus, const uint8_t* minus, size_t n, int8_t* w, void* stream) {
    if (n == 0) return ROTOR_B200_OK;
    RB_REQUIRE(w && plus && minus);
    decode_kernel<<<grid_for(n), 256, 0, as_stream(stream)>>>(plus, minus, n, w);
    return launch_status();
}

int rotor_b200_pack(const uint8_t* plus, const uint8_t* minus, size_t n, uint8_t* packed, void* stream) {
    RB_REQUIRE(n % 4 == 0);  // the reference asserts the same (src/rotor/core.py:91)
    if (n == 0) return ROTOR_B200_OK;
    RB_REQUIRE(packed && plus && minus);
    pack_kernel<<<grid_for(n / 4), 256, 0, as_stream(stream)>>>(plus, minus, n / 4, packed);
    return launch_status();
}

int rotor_b200_unpack(const uint8_t* packed, size_t n, uint8_t* plus, uint8_t* minus, void* stream) {
    if (n == 0) return ROTOR_B200_OK;
    RB_REQUIRE(packed && plus && minus);
    unpack_kernel<<<grid_for(n), 256, 0, as_stream(stream)>>>(packed, n, plus, minus);
    return launch_status();
}

int rotor_b200_packed_to_planes(const uint8_t* packed, size_t rows, size_t cols, uint8_t* plus,
                                uint8_t* minus, void* stream) {
    if (rows == 0 || cols == 0) return ROTOR_B200_OK;
    RB_REQUIRE(packed && plus && minus);
    packed_to_planes_kernel<<<grid_for(rows * ((cols + 7) / 8)), 256, 0, as_stream(stream)>>>(packed, rows, cols,
                                                                                            plus, minus);
    return launch_status();
}

int rotor_b200_planes_to_int8(const uint8_t* plus, const uint8_t* minus, size_t rows, size_t cols, int8_t* w,
                              void* stream) {
    if (rows == 0 || cols == 0) return ROTOR_B200_OK;
    RB_REQUIRE(w && plus && minus);
    planes_to_int8_kernel<<<grid_for(rows * cols), 256, 0, as_stream(stream)>>>(plus, minus, rows, cols, w);
    return launch_status();
}

size_t rotor_b200_in_padded(size_t in) { return kpad_of(in); }
size_t rotor_b200_out_padded(size_t out) { return opad_of(out); }
size_t rotor_b200_tiles_bytes(size_t out, size_t in) { return opad_of(out) * kpad_of(in) / 4; }

int rotor_b200_packed_to_tiles(const uint8_t* packed, size_t out, size_t in, void* tiles, void* stream) {
    RB_REQUIRE(packed && tiles && out > 0 && in > 0);
    to_tiles_kernel<true><<<grid_for(rotor_b200_tiles_bytes(out, in) / 4), 256, 0, as_stream(stream)>>>(
        packed, out, in, (uint32_t*)tiles);
    return launch_status();
}

int rotor_b200_int8_to_tiles(const int8_t* w, size_t out, size_t in, void* tiles, void* stream) {
    RB_REQUIRE(w && tiles && out > 0 && in > 0);
    to_tiles_kernel<false><<<grid_for(rotor_b200_tiles_bytes(out, in) / 4), 256, 0, as_stream(stream)>>>(
        (const uint8_t*)w, out, in, (uint32_t*)tiles);
    return launch_status();
}

int rotor_b200_tiles_to_int8(const void* tiles, size_t out, size_t in, int8_t* w, void* stream) {
    RB_REQUIRE(w && tiles && out > 0 && in > 0);
    tiles_to_int8_kernel<<<grid_for(rotor_b200_tiles_bytes(out, in) / 4), 256, 0, as_stream(stream)>>>(
        (const uint32_t*)tiles, out, in, w);
    return launch_status();
}

// ---- host-pointer drop-ins carrying the reference's own symbol names -------------
static void die(const char* what, cudaError_t e) {
    fprintf(stderr, "librotor_b200: %s failed: %s\n", what, cudaGetErrorString(e));
    abort();
}
#define DIE_ON(call)                          \
    do {                                      \
        cudaError_t e_ = (call);              \
        if (e_ != cudaSuccess) die(#call, e_); \
    } while (0)

void bitnet_to_rotor(const uint8_t* packed_host, size_t rows, size_t cols, uint8_t* bit0_host,
                     uint8_t* bit1_host) {
    if (rows == 0 || cols == 0) return;
    const size_t sbytes = rows * ((cols + 3) / 4), dbytes = rows * ((cols + 7) / 8);
    uint8_t* d = nullptr;
    DIE_ON(cudaMalloc(&d, sbytes + 2 * dbytes));
    DIE_ON(cudaMemcpy(d, packed_host, sbytes, cudaMemcpyHostToDevice));
    if (rotor_b200_packed_to_planes(d, rows, cols, d + sbytes, d + sbytes + dbytes, nullptr) != ROTOR_B200_OK)
        die("packed_to_planes launch", cudaGetLastError());
    DIE_ON(cudaMemcpy(bit0_host, d + sbytes, dbytes, cudaMemcpyDeviceToHost));
    DIE_ON(cudaMemcpy(bit1_host, d + sbytes + dbytes, dbytes, cudaMemcpyDeviceToHost));
    DIE_ON(cudaFree(d));
}

void rotor_unpack_weights(const uint8_t* bit0_host, const uint8_t* bit1_host, size_t rows, size_t cols,
                          int8_t* weights_host) {
    if (rows == 0 || cols == 0) return;
    const size_t pbytes = rows * ((cols + 7) / 8), wbytes = rows * cols;
    uint8_t* d = nullptr;
    DIE_ON(cudaMalloc(&d, 2 * pbytes + wbytes));
    DIE_ON(cudaMemcpy(d, bit0_host, pbytes, cudaMemcpyHostToDevice));
    DIE_ON(cudaMemcpy(d + pbytes, bit1_host, pbytes, cudaMemcpyHostToDevice));
    if (rotor_b200_planes_to_int8(d, d + pbytes, rows, cols, (int8_t*)(d + 2 * pbytes), nullptr) != ROTOR_B200_OK)
        die("planes_to_int8 launch", cudaGetLastError());
    DIE_ON(cudaMemcpy(weights_host, d + 2 * pbytes, wbytes, cudaMemcpyDeviceToHost));
    DIE_ON(cudaFree(d));
}

}  // extern "C"
