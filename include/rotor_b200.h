/*
 * librotor_b200.so -- C ABI of the B200 (sm_100a) ternary BitLinear path.
 *
 * Conventions
 *  - Every pointer is a DEVICE pointer unless the name ends in _host or the
 *    comment says "host".  Buffers are owned by the caller (the Python host
 *    side hands in torch tensors' data_ptr()); the library allocates nothing
 *    on the hot path.
 *  - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).
 *  - Functions return ROTOR_B200_OK (0) or a ROTOR_B200_ERR_* code; nothing is
 *    computed on the CPU when the GPU path cannot run.
 *  - "reference" in the comments is BikerSam86/rotor-RAG; each entry point names
 *    the reference interface it stands in for (path:line inside that project).
 *
 * Formats
 *  packed : uint8 [out][in/4]; weight 4k+j of a row in bits (2j+1,2j) of byte k:
 *           10 = +1, 01 = -1, 00 = 0, 11 = reserved (reads as 0).
 *  planes : two uint8 [out][ceil(in/8)] bit arrays (plus flags, minus flags),
 *           weight i at byte i/8 bit i%8.
 *  tiles  : the GPU-native layout, built once at load.  The matrix is padded to
 *           out16 = ceil(out/16)*16 rows and in128 = ceil(in/128)*128 columns
 *           (padding weights are 0) and cut into tiles of 16 rows x 128 columns,
 *           512 bytes each, tile (rt,kt) at byte offset (rt*(in128/128)+kt)*512.
 *           Inside a tile lane L (g = L>>2, t = L&3) owns bytes [16L,16L+16) =
 *           four 32-bit words i = 0..3; word i, byte b, bit pair j holds the code
 *           (w+1) in {0,1,2} of row rt*16 + g + 8*(i&1), column
 *           kt*128 + 32*t + 8*j + 4*(i>>1) + b.  A warp therefore loads a tile with
 *           one coalesced 128-bit load per lane, and (word & (0x03030303<<2j))
 *           is directly an int8x4 operand scaled by 4^j.
 *  xq     : quantised activations, int8 [ncols][in128], zero padded; column
 *           m*terms+t is term t of token row m.
 */
#ifndef ROTOR_B200_H
#define ROTOR_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    ROTOR_B200_OK = 0,
    ROTOR_B200_ERR_ARG = 1,        /* null pointer, zero/oversized dimension, bad enum */
    ROTOR_B200_ERR_CUDA = 2,       /* a CUDA runtime call or launch failed */
    ROTOR_B200_ERR_SHAPE = 3,      /* shape not supported by the kernels */
    ROTOR_B200_ERR_WORKSPACE = 4,  /* caller-provided workspace too small */
    ROTOR_B200_ERR_TIMEOUT = 5     /* a bounded device-side wait gave up */
};

/* GEMV variant selector for rotor_b200_bitlinear_acc */
enum {
    ROTOR_B200_VARIANT_AUTO = 0,
    ROTOR_B200_VARIANT_DP4A = 1,   /* integer dot-product lanes, <= 4 columns per pass */
    ROTOR_B200_VARIANT_MMA = 2     /* int8 tensor-core fragments, 8 columns per pass */
};

int rotor_b200_version(void);
const char* rotor_b200_status_string(int status);
/* Reads and clears the device status word that bounded device-side waits write to
 * (0, or ROTOR_B200_ERR_TIMEOUT).  Synchronises with the device. */
int rotor_b200_device_status(void);

/* ---------------------------------------------------------------- format (a1-a3)
 * Device twins of the reference's format primitives.
 *   rotor_encode / rotor_decode / rotor_pack / rotor_unpack  native/c/rotor_core.c:25-75,
 *   RotorCore.encode/decode/pack/unpack                      src/rotor/core.py:27-141 */
int rotor_b200_encode(const int8_t* w, size_t n, uint8_t* plus, uint8_t* minus, void* stream);
int rotor_b200_decode(const uint8_t* plus, const uint8_t* minus, size_t n, int8_t* w, void* stream);
int rotor_b200_pack(const uint8_t* plus, const uint8_t* minus, size_t n, uint8_t* packed, void* stream);
int rotor_b200_unpack(const uint8_t* packed, size_t n, uint8_t* plus, uint8_t* minus, void* stream);

/* bitnet_to_rotor, native/c/rotor_core.c:202-260 (ctypes binding src/rotor/bitnet_fast.py:86-102) */
int rotor_b200_packed_to_planes(const uint8_t* packed, size_t rows, size_t cols,
                                uint8_t* plus, uint8_t* minus, void* stream);
/* rotor_unpack_weights, native/c/rotor_core.c:270-299 (binding src/rotor/bitnet_fast.py:138-154) */
int rotor_b200_planes_to_int8(const uint8_t* plus, const uint8_t* minus, size_t rows, size_t cols,
                              int8_t* w, void* stream);

/* Drop-in replacements with the reference's exact names, signatures and HOST pointers
 * (native/include/rotor.h; loaded by src/rotor/bitnet_fast.py:40 through ctypes.CDLL).
 * They stage through the GPU and block until done.  Like the reference they return
 * nothing; on a CUDA failure they print to stderr and abort(). */
void bitnet_to_rotor(const uint8_t* bitnet_packed_host, size_t rows, size_t cols,
                     uint8_t* bit0_host, uint8_t* bit1_host);
void rotor_unpack_weights(const uint8_t* bit0_host, const uint8_t* bit1_host, size_t rows,
                          size_t cols, int8_t* weights_host);

/* ---------------------------------------------------------------- load-time repack (a4)
 * Stands in for TernaryLinear.load_from_bitnet's convert+decode+backend-pack chain
 * (src/rotor/transformer.py:77-109) and GPUTernaryOps.pack_ternary_weights
 * (src/rotor/gpu_ternary.py:112-136). */
size_t rotor_b200_tiles_bytes(size_t out, size_t in);
size_t rotor_b200_in_padded(size_t in);    /* in128 */
size_t rotor_b200_out_padded(size_t out);  /* out16 */
int rotor_b200_packed_to_tiles(const uint8_t* packed, size_t out, size_t in, void* tiles, void* stream);
int rotor_b200_int8_to_tiles(const int8_t* w, size_t out, size_t in, void* tiles, void* stream);
int rotor_b200_tiles_to_int8(const void* tiles, size_t out, size_t in, int8_t* w, void* stream);

/* ---------------------------------------------------------------- activation quantiser (a13)
 * quantize_activations(x, bits=8, symmetric=True), src/rotor/quantization.py:121-149,
 * applied to each of the m rows of x[m][k] (float32): s = max|row|/127 (1 if the row is
 * all zero), q = clip(rint(row/s), -128, 127).  With terms > 1 the residual
 * row - q*s is quantised again (terms <= 4).  Outputs: xq int8 [m*terms][in128],
 * sx float32 [m*terms], xsum int32 [m*terms] = sum of each xq row. */
int rotor_b200_quantize_rows(const float* x, size_t m, size_t k, int terms,
                             int8_t* xq, float* sx, int32_t* xsum, void* stream);

/* ---------------------------------------------------------------- BitLinear (a5, a14)
 * Integer core of TernaryLinear.forward (src/rotor/transformer.py:147-150):
 * acc[c][o] = sum_k xq[c][k] * w[o][k], exact int32, acc is [ncols][out].
 * Any ncols >= 1; columns are processed 8 (MMA) or up to 4 (DP4A) per pass. */
int rotor_b200_bitlinear_acc(const void* tiles, size_t out, size_t in,
                             const int8_t* xq, const int32_t* xsum, size_t ncols,
                             int32_t* acc, int variant, void* stream);

/* y[m][o] = wscale(o) * sum_t sx[m*terms+t] * acc[m*terms+t][o]; wscale(o) is
 * wscale_vec[o] when wscale_vec != NULL (the plug-in seam passes a per-row vector,
 * src/rotor/transformer.py:109), else the scalar wscale. */
int rotor_b200_bitlinear_dequant(const int32_t* acc, const float* sx, size_t m, int terms,
                                 size_t out, float wscale, const float* wscale_vec,
                                 float* y, void* stream);

/* Whole layer forward on device buffers: quantise, accumulate, dequantise.
 * x float32 [m][in] -> y float32 [m][out].  workspace must hold
 * rotor_b200_bitlinear_workspace_bytes(out, in, m, terms) bytes (256-byte aligned). */
size_t rotor_b200_bitlinear_workspace_bytes(size_t out, size_t in, size_t m, int terms);
int rotor_b200_bitlinear_forward(const void* tiles, size_t out, size_t in, const float* x,
                                 size_t m, int terms, float wscale, const float* wscale_vec,
                                 float* y, void* workspace, size_t workspace_bytes,
                                 int variant, void* stream);

/* The plug-in seam with HOST buffers: GPUTernaryOps.ternary_matmul
 * (src/rotor/gpu_ternary.py:138-202, called from src/rotor/transformer.py:136-142).
 * tiles is a device pointer returned by the host side's pack_ternary_weights;
 * scales_host [out], x_host [in], y_host [out] are host float32 arrays.  Blocks. */
int rotor_b200_ternary_matmul_host(const void* tiles, const float* scales_host,
                                   const float* x_host, size_t in, size_t out, int terms,
                                   float* y_host);

#ifdef __cplusplus
}
#endif
#endif /* ROTOR_B200_H */
