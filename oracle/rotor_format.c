/*
 * TEST INFRASTRUCTURE -- CPU oracle for the rotor 2-bit format and the
 * load-time converters.  Only the test-suite, the smoke check and the CPU
 * baseline leg of the benchmark may link or call this file; the product
 * library never does.
 *
 * Each function restates, in fresh code, the behaviour of one reference
 * function (cited by reference path:line).  Pinned against the reference's
 * own vectors (tests/test_core.py:23-32, 89-105; tests/debug_bitnet_format.py:24-44;
 * src/rotor/bitnet.py:95,171-174) and against the reference's C file compiled
 * unmodified (see oracle/Makefile, target _ref).
 *
 * Format recap.  A ternary weight w in {-1,0,+1} is two flags (p, n):
 * p = (w == +1), n = (w == -1), w = p - n.  "Packed" keeps four weights per
 * byte, weight 4k+j in bits (2j+1, 2j) = (p, n).  "Planes" keep the p flags
 * and the n flags in two separate bit arrays, eight weights per byte,
 * LSB first.  The field value 0b11 is reserved and reads as 0.
 */
#include <stddef.h>
#include <stdint.h>
#include <string.h>

/* reference: native/c/rotor_core.c:25-30 (rotor_encode), src/rotor/core.py:27-53 */
void oracle_encode(const int8_t *w, size_t n, uint8_t *p, uint8_t *m)
{
    for (size_t i = 0; i < n; ++i) {
        p[i] = (uint8_t)(w[i] == 1);
        m[i] = (uint8_t)(w[i] == -1);
    }
}

/* reference: native/c/rotor_core.c:32-36 (rotor_decode), src/rotor/core.py:56-72 */
void oracle_decode(const uint8_t *p, const uint8_t *m, size_t n, int8_t *w)
{
    for (size_t i = 0; i < n; ++i)
        w[i] = (int8_t)((int)p[i] - (int)m[i]);
}

/* reference: native/c/rotor_core.c:38-49 (rotor_pack), src/rotor/core.py:75-110.
 * n must be a multiple of 4 (the reference asserts this in Python and silently
 * drops the tail in C). */
void oracle_pack(const uint8_t *p, const uint8_t *m, size_t n, uint8_t *packed)
{
    for (size_t byte = 0; byte < n / 4; ++byte) {
        unsigned v = 0;
        for (unsigned j = 0; j < 4; ++j) {
            v |= (unsigned)(p[4 * byte + j] & 1u) << (2 * j + 1);
            v |= (unsigned)(m[4 * byte + j] & 1u) << (2 * j);
        }
        packed[byte] = (uint8_t)v;
    }
}

/* reference: native/c/rotor_core.c:51-75 (rotor_unpack), src/rotor/core.py:113-141 */
void oracle_unpack(const uint8_t *packed, size_t n, uint8_t *p, uint8_t *m)
{
    for (size_t i = 0; i < n; ++i) {
        unsigned field = (packed[i / 4] >> (2 * (i % 4))) & 3u;
        p[i] = (uint8_t)(field >> 1);
        m[i] = (uint8_t)(field & 1u);
    }
}

/* reference: native/c/rotor_core.c:202-260 (bitnet_to_rotor),
 * src/rotor/bitnet.py:76-151.  packed is [rows][ceil(cols/4)], planes are
 * [rows][ceil(cols/8)]; field 0b10 sets the plus plane, 0b01 the minus plane,
 * 0b00 and 0b11 set neither. */
void oracle_packed_to_planes(const uint8_t *packed, size_t rows, size_t cols,
                             uint8_t *plus, uint8_t *minus)
{
    const size_t src_stride = (cols + 3) / 4;
    const size_t dst_stride = (cols + 7) / 8;
    memset(plus, 0, rows * dst_stride);
    memset(minus, 0, rows * dst_stride);
    for (size_t r = 0; r < rows; ++r) {
        for (size_t c = 0; c < cols; ++c) {
            unsigned field = (packed[r * src_stride + c / 4] >> (2 * (c % 4))) & 3u;
            uint8_t bit = (uint8_t)(1u << (c % 8));
            if (field == 2u)
                plus[r * dst_stride + c / 8] |= bit;
            else if (field == 1u)
                minus[r * dst_stride + c / 8] |= bit;
        }
    }
}

/* reference: native/c/rotor_core.c:270-299 (rotor_unpack_weights) */
void oracle_planes_to_int8(const uint8_t *plus, const uint8_t *minus, size_t rows,
                           size_t cols, int8_t *w)
{
    const size_t stride = (cols + 7) / 8;
    for (size_t r = 0; r < rows; ++r)
        for (size_t c = 0; c < cols; ++c) {
            int p = (plus[r * stride + c / 8] >> (c % 8)) & 1;
            int m = (minus[r * stride + c / 8] >> (c % 8)) & 1;
            w[r * cols + c] = (int8_t)(p - m);
        }
}

/* Integer BitLinear accumulation: acc[m][o] = sum_k q[m][k] * w[o][k], exact in
 * int32.  This is the integer core of src/rotor/transformer.py:147-150
 * (np.dot(x, weights_cache.T)) once the activations are int8
 * (src/rotor/quantization.py:137-149 applied per row). */
void oracle_bitlinear_acc(const int8_t *q, size_t m_rows, const int8_t *w, size_t out,
                          size_t in, int32_t *acc)
{
    for (size_t m = 0; m < m_rows; ++m)
        for (size_t o = 0; o < out; ++o) {
            int32_t s = 0;
            const int8_t *wr = w + o * in;
            const int8_t *qr = q + m * in;
            for (size_t k = 0; k < in; ++k)
                s += (int32_t)qr[k] * (int32_t)wr[k];
            acc[m * out + o] = s;
        }
}
