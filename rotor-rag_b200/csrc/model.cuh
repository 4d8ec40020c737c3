// Internal declarations shared by the decode-path kernels and the model driver.
#pragma once
#include <cuda_bf16.h>

#include "common.cuh"
#include "xch.cuh"

namespace rb {

// int32 accumulators of one BitLinear product: `planes` partial planes (one per K split),
// each [ncols][out]; consumers add the planes (exact, order independent).
struct AccView {
    const int32_t* acc;
    size_t plane_stride;  // elements between planes
    int planes;
    int out;
};

enum VecStageMode { VS_EMBED = 0, VS_PLAIN = 1, VS_OPROJ = 2, VS_FFN = 3, VS_DOWN = 4, VS_DEQ = 5, VS_ATTN = 6 };

struct VecStageParams {
    int mode;
    int n;                       // row width
    // sources
    const long long* ids;        // VS_EMBED: token ids [rows]
    const __nv_bfloat16* embed;  // VS_EMBED: table [vocab][n]
    const float* src;            // VS_PLAIN: float rows
    AccView acc;                 // accumulators of the previous product
    const float* sx_in;          // its activation scales [rows*terms]
    int terms;
    float wscale0, wscale1;      // weight scale(s) of the previous product
    int ffn_act;
    const float* norm0;          // VS_OPROJ: sub-norm weight
    float* h;                    // residual stream [rows][n] (read)
    float* h_out;                // where the updated stream goes (null = in place, h)
    // VS_ATTN: merge the decode-attention partials of row m into the row
    const float* part_o;         // [rows][n_heads][nsplit][head_dim]
    const float* part_m;         // [rows][n_heads][nsplit]
    const float* part_l;
    int nsplit, n_heads, head_dim;
    // sinks
    const float* norm1;          // optional pre-norm weight applied before the sinks
    float eps;
    float* y_out;                // optional float copy of the (normed) row
    int8_t* xq;                  // optional quantised output [rows*terms_out][kpad]
    float* sx_out;
    int32_t* xsum_out;
    int terms_out;
    int kpad;
    // Sharded rows (tensor parallel): the row is one rank's slice of a longer row.
    const float* ext_sumsq;      // [rows] sum of squares of the whole row, used by norm1 instead of the local one
    int norm_n;                  // width of the whole row for norm1's mean (0 = n)
    const float* ext_absmax;     // [rows] max|.| of the whole row, used by the quantiser
    float* out_sumsq;            // [rows] optional: local sum of squares of the built row (before norm1)
    float* out_absmax;           // [rows] optional: local max|.| of the row after norm1
};

int launch_vec_stage(const VecStageParams& p, int rows, cudaStream_t st);
bool row_stage_supported(const VecStageParams& p, int rows);
int launch_row_stage(const VecStageParams& p, int rows, cudaStream_t st);
int configure_vec_stage();
int configure_gemv_kernels();
int configure_lmhead();

// BitLinear product into partial planes (no atomics, no memset): returns the view.
struct GemvPlan {
    int ksplit;
    int kt_per_split;
};
GemvPlan plan_gemv(size_t out, size_t in, int ncols);
int launch_gemv_planes(const void* tiles, size_t out, size_t in, const int8_t* xq, const int32_t* xsum, int ncols,
                       int32_t* acc, size_t plane_stride, const GemvPlan& plan, int variant, cudaStream_t st);
int gemv_cols_per_launch(int variant, int ncols);

// Many-column product (gemm_mma.cu): complete int32 sums into acc[ncols][out].
constexpr int GEMM_MIN_COLS = 32;
bool gemm_tcgen05_supported(size_t out, size_t in, int ncols, const void* xq);
int launch_gemm_tcgen05(const void* tiles, size_t out, size_t in, const int8_t* xq, const int32_t* xsum, int ncols,
                        int32_t* acc, cudaStream_t st);
int configure_gemm_tcgen05();
// gate/up product with the gating in its epilogue (float32 gated rows out, one activation term per token)
bool gemm_tcgen05_gated_supported(size_t ff, size_t in, int ncols, const void* xq);
int launch_gemm_tcgen05_gated(const void* tiles, size_t ff, size_t in, const int8_t* xq, const float* sx,
                              const int32_t* xsum, int ncols, float sg, float su, int ffn_act, float* gated,
                              cudaStream_t st);
struct QkvFinishParams;
// q/k/v product whose read-back dequantises, rotates and appends to the cache (acc of `f` unused)
bool gemm_tcgen05_qkv_supported(size_t dq, size_t dkv, size_t in, int head_dim, int ncols, const void* xq);
int launch_gemm_tcgen05_qkv(const void* tiles, size_t in, const int8_t* xq, const float* sx, const int32_t* xsum,
                            int ncols, const QkvFinishParams& f, cudaStream_t st);
int launch_gemm_mma(const void* tiles, size_t out, size_t in, const int8_t* xq, const int32_t* xsum, int ncols,
                    int32_t* acc, cudaStream_t st);

// Generation-step product with the consuming vector stage fused in (fused.cu, leanstage.cuh).
struct LeanStage;
// Tensor-parallel extras of a product: the scalar exchange ring its prologue uses and, for a
// row-parallel product, where the int32 partial sums and the activation scales go.
struct FusedTpExtra {
    XchScalarDev xs;
    int32_t* part;
    float* sx_out;
};
int launch_fused_gemv(const void* tiles, size_t out, size_t in, int halves, int rows, const LeanStage& stage, float* y,
                      const float* scale, int seg1, int seg2, int ffn_act, cudaStream_t st,
                      const FusedTpExtra* tp = nullptr);
bool fused_gemv_supported(size_t out, size_t in, int rows, int terms, int halves, int merge_weights);
int configure_fused_gemv();
// Stand-alone int8 x ternary product of a small matrix through the staged generation-step kernel.
bool staged_acc_supported(size_t out, size_t in, int ncols, int variant);
int launch_staged_acc(const void* tiles, size_t out, size_t in, const int8_t* xq, const int32_t* xsum, int ncols,
                      int32_t* acc, int variant, cudaStream_t st);
int fused_sm_count();

extern int g_use_pdl;

struct QkvFinishParams {
    AccView acc;          // rows of the stacked [q;k;v] product
    const float* sx;
    int terms;
    float sq, sk, sv;
    int n_heads, n_kv_heads, head_dim;
    int seq;              // tokens per sequence in this call
    const int* past_len;  // device [batch]: tokens already cached, per sequence
    int max_seq;          // cache capacity per sequence
    const float2* rope;   // cos/sin table [max_seq][head_dim/2], or null for no rotation
    float* q;             // [rows][n_heads*head_dim]
    float* k_cache;       // [batch][n_kv][max_seq][head_dim]
    float* v_cache;
};
int launch_qkv_finish(const QkvFinishParams& p, int rows, cudaStream_t st);
int launch_rope_table(float2* table, int max_seq, int head_dim, float theta, cudaStream_t st);

struct AttnDecodeParams {
    const float* qkv_f;   // when set: finished float32 [batch][q;k;v] rows, acc/sx/scales unused
    AccView acc;          // else: stacked [q;k;v] product of one token per sequence
    const float* sx;
    int terms;
    float sq, sk, sv;
    int n_heads, n_kv_heads, head_dim, max_seq, nsplit;
    const int* past_len;
    const float2* rope;
    float* k_cache;
    float* v_cache;
    float* part_o;        // [batch][n_heads][nsplit][head_dim]
    float* part_m;        // [batch][n_heads][nsplit]
    float* part_l;
    unsigned* counter;    // [batch], zero before the launch
    float* attn_out;      // optional float copy of the merged rows [batch][n_heads*head_dim]
    int8_t* xq;           // quantised merged rows for the output projection
    float* sx_out;
    int32_t* xsum_out;
    int terms_out;
    int kpad;
};
int launch_attn_decode(const AttnDecodeParams& p, int batch, cudaStream_t st);
// Cluster variant: finished attention rows in p.attn_out (needs p.qkv_f); see attention.cu.
bool attn_decode_cluster_ok(int n_heads, int n_kv_heads, int head_dim, int max_seq, int nsplit);
int launch_attn_decode_cluster(const AttnDecodeParams& p, int batch, cudaStream_t st);
int attn_decode_nsplit(int max_seq);
int attn_decode_nsplit_for(int n_heads, int n_kv_heads, int head_dim, int max_seq);
size_t attn_decode_part_floats(int batch, int n_heads, int head_dim, int max_seq);
int configure_attention();

struct AttnParams {
    const float* q;       // [rows][n_heads*head_dim]
    const float* k_cache;
    const float* v_cache;
    float* out;           // [rows][n_heads*head_dim]
    int n_heads, n_kv_heads, head_dim;
    int seq;
    const int* past_len;
    int max_seq;
    int causal;
    __nv_bfloat16* kv_split;  // optional scratch: K hi, K lo, V hi, V lo planes of the cache rows in use
    size_t split_plane;       // elements per plane (batch capacity * n_kv_heads * max_seq * head_dim)
    // one-token steps of a few sequences: nsplit > 1 cuts every sequence's cache into nsplit runs, one CTA
    // each, which write un-normalised partial outputs with their (max, sum) instead of `out`
    int nsplit;
    float* part_o;        // [rows][n_heads][nsplit][head_dim]
    float* part_m;        // [rows][n_heads][nsplit]
    float* part_l;
};
int launch_attention(const AttnParams& p, int rows, cudaStream_t st);
// Runs for a one-token step of `rows` sequences handled by the streaming kernel (1 = whole sequences,
// finished rows in `out`); 0 if that kernel does not take the shape.
int attn_stream_splits(int rows, int n_heads, int n_kv_heads, int head_dim, int max_nsplit);
bool attn_prefill_supported(const AttnParams& p, int rows);
int launch_attn_prefill_tc(const AttnParams& p, int rows, cudaStream_t st);
// head_dim 128 on tcgen05 / tensor memory (attn_prefill_t5.cu); needs the split planes sized for
// max_seq rounded up to 64 positions
bool attn_prefill_t5_supported(const AttnParams& p, int rows);
int launch_attn_prefill_t5(const AttnParams& p, int rows, cudaStream_t st);
int configure_attn_prefill_t5();
int configure_attn_prefill_tc();

struct LmHeadParams {
    const __nv_bfloat16* embed;  // [vocab][d]
    const float* x;              // [rows][d], already normed
    int vocab, d;
    float* logits;               // optional [rows][vocab]
    float* part_val;             // [rows][nparts]
    int* part_idx;
    long long* argmax_out;       // [rows]
    float* argmax_val;           // optional [rows]: the picked logit (vocabulary-sharded picks compare them)
    int nparts;
    unsigned* tail_counter;      // zeroed word: enables the fused pick when rows fit one launch
    long long* adv_log;          // optional: token log [max_log][rows]; also advances *adv_pos, *adv_step
    int* adv_pos;
    int* adv_step;
    int adv_max_log;
    // fused prologue (pro_y != null): x = rmsnorm(pro_h + pro_y, pro_norm), rows of width d
    const float* pro_y;
    const float* pro_h;
    const float* pro_norm;
    float pro_eps;
    // more than four rows: scratch for the hi / lo bf16 split of x (2 * rows * d elements) lets the
    // tensor-core kernel read the table once for up to 64 rows; part_* must then hold
    // rows * max(nparts, lmhead_mma_parts(vocab)) entries
    __nv_bfloat16* xsplit;
};
int lmhead_mma_parts(int vocab);
bool lmhead_mma_supported(int rows, int d);
int configure_lmhead_mma();
int launch_lmhead_mma(const __nv_bfloat16* embed, const float* x, __nv_bfloat16* xsplit, int rows, int vocab, int d,
                      float* logits, float* part_val, int* part_idx, cudaStream_t st);
int launch_lmhead(const LmHeadParams& p, int rows, cudaStream_t st);
int lmhead_parts();

unsigned* library_status_word();

// Tensor-parallel collectives (tp.cu); `comm` is the handle made by rotor_b200_tp_init.
int tp_rank(void* comm);
int tp_size(void* comm);
int tp_allreduce_sum_i32(void* comm, int32_t* buf, size_t n, cudaStream_t st);
int tp_allreduce_f32(void* comm, float* buf, size_t n, bool max_op, cudaStream_t st);
int tp_allgather_bytes(void* comm, const void* send, void* recv, size_t bytes_per_rank, cudaStream_t st);
// Exchanges of the generation-step path (see xch.cuh): available when the peer-memory set-up succeeded.
bool tp_fused_ready(void* comm);
XchScalarDev tp_scalar_dev(void* comm);
int tp_allreduce_dequant(void* comm, int slotsel, int idx, const int32_t* part, const float* sx, float scale, float* y,
                         int rows, int n, cudaStream_t st);
int tp_step_end(void* comm, int nexchanges, cudaStream_t st);

}  // namespace rb
