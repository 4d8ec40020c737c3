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
    ROTOR_B200_ERR_TIMEOUT = 5,    /* a bounded device-side wait gave up */
    ROTOR_B200_ERR_TOO_LARGE = 6   /* problem does not fit the library's built-in scratch array */
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
/* Number of kernels this library has launched in this process, graph replays included. */
unsigned long long rotor_b200_launch_count(void);
/* Measurement aid (no counterpart in the reference): launches a kernel that does nothing, with the
 * launch attributes of the decode chain.  Timing a chain of these gives the per-launch floor of a
 * chain of dependent kernels on this device. */
int rotor_b200_launch_empty(void* stream);
/* Self-test of the bounded device-side waits (no counterpart in the reference, whose plug-in call
 * swallows every failure and recomputes on the CPU, src/rotor/transformer.py:145-147): runs the
 * peer-memory all-reduce on ONE GPU against a "peer" buffer nothing writes, with a wait limit of
 * spin_cycles SM cycles.  The first launch must give up and set the status word (returned in
 * *status_out: 0x7e000000 | source rank); a second launch must then return at once (*second_ms,
 * device time).  The word stays set for rotor_b200_device_status() to read and clear. */
int rotor_b200_selftest_exchange_timeout(long long spin_cycles, unsigned* status_out, float* second_ms);

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

/* Allocation-free variant of rotor_b200_bitlinear_forward.  (No counterpart in the reference:
 * its plug-in call simply has no workspace argument, which is the reason this exists.)
 * For hosts that cannot allocate device memory when they call in -- a plug-in reached through
 * ternary_matmul(packed, scales, x, in, out), or a serving loop whose own pool already holds
 * all free device memory, where cudaMalloc fails or stalls every stream while it runs.  The
 * scratch (quantised activations, scales, int32 accumulators, a status word) lives in a
 * fixed ROTOR_B200_STATIC_SCRATCH_BYTES array inside the library, held on every GPU that
 * loads the library until the process exits.
 *  - Same arguments and results as rotor_b200_bitlinear_forward, minus the workspace.
 *  - A problem that needs more scratch than the array returns ROTOR_B200_ERR_TOO_LARGE and
 *    launches nothing; rotor_b200_bitlinear_static_fits(out, in, m, terms) tells beforehand.
 *  - The first call on a device looks up the array's device address; make that call before
 *    any stream capture begins.
 *  - Calls share the array and it keeps the last call's contents (what must start at zero
 *    is cleared inside); calls that overlap on the GPU race on it, so keep them ordered.
 *  - Calls no cudaMalloc / cudaFree or other allocating routine.
 *  - A bounded wait that runs out on this path is recorded in a status word at the start of the
 *    array; rotor_b200_device_status() reads and clears it together with the library's own word. */
#define ROTOR_B200_STATIC_SCRATCH_BYTES (4u << 20)
int rotor_b200_bitlinear_static_fits(size_t out, size_t in, size_t m, int terms);
int rotor_b200_bitlinear_forward_static(const void* tiles, size_t out, size_t in, const float* x,
                                        size_t m, int terms, float wscale, const float* wscale_vec,
                                        float* y, int variant, void* stream);

/* The plug-in seam with HOST buffers: GPUTernaryOps.ternary_matmul
 * (src/rotor/gpu_ternary.py:138-202, called from src/rotor/transformer.py:136-142).
 * tiles is a device pointer returned by the host side's pack_ternary_weights;
 * scales_host [out], x_host [in], y_host [out] are host float32 arrays.  Blocks. */
int rotor_b200_ternary_matmul_host(const void* tiles, const float* scales_host,
                                   const float* x_host, size_t in, size_t out, int terms,
                                   float* y_host);

/* ---------------------------------------------------------------- transformer glue (a6)
 * RMSNorm.forward, src/rotor/transformer.py:24-36: y = x / sqrt(mean(x^2) + eps) * weight,
 * x and y float32 [rows][n]. */
int rotor_b200_rmsnorm(const float* x, size_t rows, size_t n, const float* weight, float eps,
                       float* y, void* stream);

/* ---------------------------------------------------------------- whole model (a7-a12)
 * Semantics switches.  The defaults in the comments are what the reference code does when
 * run; the alternatives are the published BitNet-b1.58 description. */
enum {
    ROTOR_B200_FFN_SILU_CLIP20 = 0, /* gate * silu(clip(up,-20,20)), src/rotor/transformer.py:328-351 */
    ROTOR_B200_FFN_RELU2 = 1        /* relu(gate)^2 * up */
};
enum {
    ROTOR_B200_LOGITS_NONE = 0,
    ROTOR_B200_LOGITS_LAST = 1,     /* last position of each sequence: float32 [batch][vocab] */
    ROTOR_B200_LOGITS_ALL = 2       /* every position, as the reference computes (bitnet_model.py:235) */
};

typedef struct rotor_b200_model_config {
    int32_t vocab_size, d_model, n_layers, n_heads, n_kv_heads, d_ff; /* src/rotor/bitnet_model.py:56-61 */
    int32_t act_terms;    /* int8 activation terms per BitLinear input: 1 = per-token absmax int8,
                             3 = float32-faithful (matches the reference's float path) */
    int32_t ffn_act;      /* ROTOR_B200_FFN_* */
    int32_t causal;       /* 0 = no mask (the reference never passes one, bitnet_model.py:226) */
    float rope_theta;     /* 0 = no positional encoding (reference); > 0 = rotary, half-split pairs */
    float eps;            /* RMSNorm epsilon (reference 1e-6, transformer.py:20) */
    int32_t max_batch;    /* sequences the KV cache holds */
    int32_t max_seq;      /* positions per sequence the KV cache holds */
    int32_t max_rows;     /* most token rows (batch*seq) in one forward call */
    int32_t gemv_variant; /* ROTOR_B200_VARIANT_* */
    int32_t tp_size;      /* tensor-parallel ranks (0 or 1 = single GPU).  With tp_size > 1 the head and
                             FFN counts above stay GLOBAL; every rank holds n_heads/tp query heads,
                             n_kv_heads/tp KV heads and d_ff/tp FFN channels.  Needs act_terms == 1. */
    int32_t tp_rank;      /* this process's rank, 0 .. tp_size-1 */
} rotor_b200_model_config;

/* Device pointers of one transformer block.  qkv_tiles holds the tiles of q, k and v one
 * after the other (their row counts are multiples of 16, so this is the tile layout of the
 * stacked matrix); gate_up_tiles likewise.  Scales are the per-tensor weight scales
 * (src/rotor/transformer.py:87).  Caches are float32 [max_batch][n_kv_heads][max_seq][head_dim]. */
typedef struct rotor_b200_layer_weights {
    const void* qkv_tiles;
    const void* o_tiles;
    const void* gate_up_tiles;
    const void* down_tiles;
    float q_scale, k_scale, v_scale, o_scale, gate_scale, up_scale, down_scale;
    const float* input_norm;
    const float* post_attn_norm;
    const float* attn_sub_norm;
    const float* ffn_sub_norm;
    float* k_cache;
    float* v_cache;
} rotor_b200_layer_weights;

/* BitNetModel (src/rotor/bitnet_model.py:41-90).  `layers` is a HOST array of n_layers
 * entries (copied); embed_bf16 is the device bf16 table [vocab][d_model] used for both the
 * embedding gather and the tied LM head; final_norm device float32 [d_model].  workspace is
 * device memory of rotor_b200_model_workspace_bytes(cfg) bytes, 256-byte aligned, owned by
 * the caller for the lifetime of the handle. */
size_t rotor_b200_model_workspace_bytes(const rotor_b200_model_config* cfg);
int rotor_b200_model_create(const rotor_b200_model_config* cfg, const rotor_b200_layer_weights* layers,
                            const void* embed_bf16, const float* final_norm, void* workspace,
                            size_t workspace_bytes, void** handle);
void rotor_b200_model_destroy(void* handle);

/* BitNetModel.forward (src/rotor/bitnet_model.py:190-244) over ids int64 [batch][seq] with
 * past_len positions already cached; the new K/V are appended to the caches.  logits
 * (float32, shape by logits_mode) and next_ids (int64 [batch], greedy pick of the last
 * position, generation.py:42) are optional outputs. */
int rotor_b200_model_forward(void* handle, const int64_t* ids, int batch, int seq, int past_len,
                             int logits_mode, float* logits, int64_t* next_ids, void* stream);

/* Device-resident greedy generation, the cached loop of TextGenerator.generate
 * (src/rotor/generation.py:220-279): begin() seeds the loop with the token picked after the
 * prompt; steps() runs n one-token forwards, each feeding its greedy pick to the next and
 * logging it on the device (use_graph != 0 replays one captured CUDA graph per step);
 * read_tokens() copies logged tokens [count][batch] to HOST memory and synchronises. */
int rotor_b200_model_decode_begin(void* handle, const int64_t* first_ids, int batch, int past_len, void* stream);
int rotor_b200_model_decode_steps(void* handle, int nsteps, int use_graph, void* stream);
int rotor_b200_model_read_tokens(void* handle, int first_step, int count, int64_t* tokens_host, void* stream);
int rotor_b200_model_position(void* handle);

/* Batched generation over prompts of different lengths -- an extension of the cached loop of
 * TextGenerator.generate (src/rotor/generation.py:220-279), which takes one prompt per call.
 * forward_ragged(): ids int64 [batch][seq] hold the prompts right-padded to `seq` tokens with any
 * valid id; lens (HOST int32 [batch], 1 <= lens[b] <= seq) are the true lengths.  Causal models
 * only (a position never attends to the padding behind it), past length 0.  logits_mode is
 * NONE or LAST; logits [batch][vocab] and next_ids [batch] are taken at each prompt's own last
 * token.  decode_begin_ragged(): like decode_begin, with sequence b continuing at lens[b];
 * decode_steps / read_tokens follow as usual and rotor_b200_model_position reports the longest
 * sequence. */
int rotor_b200_model_forward_ragged(void* handle, const int64_t* ids, int batch, int seq, const int32_t* lens,
                                    int logits_mode, float* logits, int64_t* next_ids, void* stream);
int rotor_b200_model_decode_begin_ragged(void* handle, const int64_t* first_ids, int batch, const int32_t* lens,
                                         void* stream);

/* ---------------------------------------------------------------- sampling
 * TopKSampling.sample / TopPSampling.sample (src/rotor/generation.py:45-145) on the device: logits
 * [rows][vocab] float32 (device) are divided by `temperature`; mode 0 keeps the top_k largest, mode 1
 * the shortest probability-sorted prefix whose mass reaches top_p; one token per row is drawn from
 * the softmax over what is kept and written to out[rows] (device).  The reference draws from NumPy's
 * global generator; here the uniform of row r is SplitMix64 of (seed, counter + r) and the kept
 * tokens are walked in vocabulary order: the reference's distribution, this library's own stream. */
int rotor_b200_sample(const float* logits, int rows, int vocab, int mode, int top_k, float top_p,
                      float temperature, uint64_t seed, uint64_t counter, int64_t* out, void* stream);

/* ---------------------------------------------------------------- tensor parallel (new design)
 * The reference is single-device.  For models large enough to shard, BitLinear is split
 * Megatron-style over the GPUs of one box, one process per GPU: q/k/v, gate and up by output
 * rows (their tiles in rotor_b200_layer_weights hold only this rank's rows), o and down by
 * input columns (this rank's columns, partial sums all-reduced as exact int32), the LM head
 * by vocabulary.  rotor_b200_tp_unique_id fills a 128-byte NCCL id on one rank (host memory);
 * the host side broadcasts it; every rank calls rotor_b200_tp_init with it (collective) and
 * attaches the communicator to its model.  NCCL is bound at run time from libnccl.so.2. */
int rotor_b200_tp_unique_id(void* out128_host);
int rotor_b200_tp_init(int rank, int size, const void* unique_id128_host, void** comm);
void rotor_b200_tp_destroy(void* comm);
int rotor_b200_model_set_tp(void* handle, void* comm);

/* Programmatic dependent launch for the decode chain: with 1, every kernel of a step may start
 * and prefetch its weight tiles while its predecessor drains (the kernels order themselves with
 * griddepcontrol.wait).  Affects later launches and graphs captured afterwards; returns the
 * previous setting.  No counterpart in the reference. */
int rotor_b200_set_pdl(int enable);

/* Blocks [layer_begin, layer_end) of the model on caller-provided hidden rows (float32
 * [batch*seq][d_model]).  apply_final_norm != 0 applies the model's final norm, as
 * BitNetModel.forward(return_logits=False) does (src/rotor/bitnet_model.py:231-243);
 * 0 returns the raw residual stream (TransformerBlock.forward, src/rotor/transformer.py:383-413). */
int rotor_b200_model_forward_hidden(void* handle, const float* hidden_in, int batch, int seq, int past_len,
                                    int layer_begin, int layer_end, int apply_final_norm,
                                    float* hidden_out, void* stream);

/* ---------------------------------------------------------------- stand-alone block halves
 * GatedFFN.forward (src/rotor/transformer.py:320-341): x float32 [rows][d_model] ->
 * y float32 [rows][d_model]; pre_norm != NULL applies RMSNorm(pre_norm) to x first.
 * MultiHeadAttention.forward (src/rotor/transformer.py:206-292): x float32
 * [batch*seq][d_model] -> y, output projection and sub-norm included; appends K/V to the
 * layer's caches at past_len.  Both read dimensions and switches from cfg and pointers from
 * layer (only the members of their half need to be set) and need
 * rotor_b200_block_workspace_bytes(cfg, rows) bytes of 256-byte aligned device workspace. */
size_t rotor_b200_block_workspace_bytes(const rotor_b200_model_config* cfg, int rows);
int rotor_b200_ffn_forward(const rotor_b200_model_config* cfg, const rotor_b200_layer_weights* layer,
                           const float* pre_norm, const float* x, int rows, float* y,
                           void* workspace, size_t workspace_bytes, void* stream);
int rotor_b200_attention_forward(const rotor_b200_model_config* cfg, const rotor_b200_layer_weights* layer,
                                 const float* x, int batch, int seq, int past_len, float* y,
                                 void* workspace, size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ROTOR_B200_H */
