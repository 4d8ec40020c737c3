// Model driver: sequences the decode-path kernels for BitNetModel.forward
// (src/rotor/bitnet_model.py:190-244) and the cached generation loop of
// TextGenerator (src/rotor/generation.py:179-279) on one GPU.  All buffers are
// caller-owned device memory; the handle only records pointers and plans.
//
// Per block (src/rotor/transformer.py:383-413) the launch sequence is
//   q/k/v product (stacked)  -> qkv_finish (dequant, rotary, cache append) -> attention
//   -> quantise -> o product -> [sub-norm, residual, pre-norm, quantise]
//   -> gate/up product (stacked) -> [gating, sub-norm, quantise] -> down product
//   -> [residual, next pre-norm, quantise]
// and a generation step ends with the tied LM head fused with the greedy pick.  A
// generation step reads the position and the input token from device memory, so one
// captured CUDA graph replays for every step.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>

#include "product_body.cuh"

namespace rb {

static inline size_t al256(size_t v) { return (v + 255) & ~(size_t)255; }

// Scratch buffers and dimensions one block needs; carved from caller-owned device memory.
struct Ctx {
    int d, ff, n_heads, n_kv_heads, head_dim, dq, dkv;
    int terms, ffn_act, causal, variant, max_seq;
    float rope_theta, eps;
    size_t kmax;  // widest padded BitLinear input
    float* h;     // residual stream [rows][d]
    float* h2;    // second copy: fused generation steps ping-pong between the two
    float* hn;    // final-normed rows
    float* qbuf;
    float* attn;
    int8_t* xq;
    float* sx[2];
    int32_t* xsum[2];
    int32_t* accA;  // q/k/v and gate/up accumulators
    int32_t* accB;  // o and down accumulators
    int* d_pos;
    float2* rope;        // cos/sin table, or null
    float2* rope_buf;    // storage for it
    __nv_bfloat16* kvsplit;  // prefill attention: hi / lo bf16 planes of one layer's K/V rows (or null)
    size_t kvsplit_plane;
    float* part_o;       // decode-attention partials
    float* part_m;
    float* part_l;
    int nsplit;
    int max_batch;
    unsigned* counters;  // [8 + max_batch] zeroed words for last-CTA tails
    // tensor parallel (tp_size > 1): communicator, whole FFN width, exchange buffers
    void* tp;
    int tp_size, ff_total;
    float* stat[2];      // [rows] per-row statistics that cross ranks (sum of squares, absolute maximum)
    float* gated;        // [rows][ff] this rank's slice of the gated FFN row
    // float32 outputs of the fused generation step's products: q/k/v, o, gated, down
    float* fy[4];
};

constexpr int FUSED_MAX_ROWS = 4;

struct Model {
    rotor_b200_model_config cfg;
    rotor_b200_layer_weights* layers;
    const __nv_bfloat16* embed;
    const float* final_norm;
    Ctx c;
    float* part_val;
    int* part_idx;
    long long* cur_ids;
    long long* tok_log;
    int* d_step;
    int* d_lens;                // [max_batch] prompt lengths of a ragged batch
    const int32_t* last_of;     // host, during a ragged forward: tokens of each sequence (its last row is picked)
    int max_log;
    // host mirror of the generation state
    int pos, step, batch;
    cudaGraphExec_t graph;
    int graph_batch;
    unsigned long long graph_launches;  // kernels inside the captured step
    // tensor parallel greedy pick: (value, global index) of every rank's best row
    __nv_bfloat16* xsplit;  // LM head over more than four rows: hi / lo bf16 split of its input rows
    float* pick_val;      // [rows]
    long long* pick_idx;  // [rows]
    unsigned char* pick_send;  // [rows] x 12 bytes
    unsigned char* pick_recv;  // [tp][rows] x 12 bytes
};

struct Carve {
    unsigned char* base;
    size_t off;
    template <typename T>
    T* take(size_t count) {
        T* p = base ? reinterpret_cast<T*>(base + off) : nullptr;
        off += al256(count * sizeof(T));
        return p;
    }
};

static int max_planes(size_t out, size_t in) { return plan_gemv(out, in, 8).ksplit; }

// Dimensions of one rank: with tp > 1 the heads and the FFN width are this rank's share
// (query / KV heads and d_ff divided by tp), d_model stays whole.
static int derive_ctx(Ctx& c, int d_model, int n_heads, int n_kv_heads, int d_ff, int terms, int tp = 1) {
    if (d_model <= 0 || n_heads <= 0 || n_kv_heads <= 0 || d_ff <= 0) return ROTOR_B200_ERR_ARG;
    if (terms < 1 || terms > 4) return ROTOR_B200_ERR_ARG;
    if (d_model % n_heads || n_heads % n_kv_heads) return ROTOR_B200_ERR_SHAPE;
    if (tp < 1) tp = 1;
    c.head_dim = d_model / n_heads;  // head_dim = d_model // n_heads, src/rotor/transformer.py:192
    if (c.head_dim != 32 && c.head_dim != 64 && c.head_dim != 128) return ROTOR_B200_ERR_SHAPE;
    c.ff_total = d_ff;
    c.tp_size = tp;
    if (tp > 1) {
        // whole heads and whole FFN channels per rank
        if (n_heads % tp || n_kv_heads % tp || d_ff % tp) return ROTOR_B200_ERR_SHAPE;
        n_heads /= tp;
        n_kv_heads /= tp;
        d_ff /= tp;
    }
    c.d = d_model;
    c.ff = d_ff;
    c.n_heads = n_heads;
    c.n_kv_heads = n_kv_heads;
    c.terms = terms;
    c.dq = n_heads * c.head_dim;
    c.dkv = n_kv_heads * c.head_dim;
    if (c.dq % 16 || c.dkv % 16 || d_ff % 16) return ROTOR_B200_ERR_SHAPE;  // stacked products need whole row tiles
    c.kmax = kpad_of(d_model);
    if (kpad_of(c.dq) > c.kmax) c.kmax = kpad_of(c.dq);
    if (kpad_of(d_ff) > c.kmax) c.kmax = kpad_of(d_ff);
    return ROTOR_B200_OK;
}

static void carve_ctx(Ctx& c, Carve& cv, size_t rows) {
    const size_t cols = rows * c.terms;
    const size_t d = c.d, ff = c.ff;
    const size_t qkv_out = c.dq + 2 * (size_t)c.dkv;
    c.h = cv.take<float>(rows * d);
    c.h2 = cv.take<float>(rows * d);
    c.hn = cv.take<float>(rows * d);
    c.qbuf = cv.take<float>(rows * c.dq);
    c.attn = cv.take<float>(rows * c.dq);
    c.xq = cv.take<int8_t>(cols * c.kmax);
    for (int i = 0; i < 2; ++i) {
        c.sx[i] = cv.take<float>(cols);
        c.xsum[i] = cv.take<int32_t>(cols);
    }
    const size_t pa1 = (size_t)max_planes(qkv_out, d) * cols * qkv_out;
    const size_t pa2 = (size_t)max_planes(2 * ff, d) * cols * 2 * ff;
    const size_t pb1 = (size_t)max_planes(d, c.dq) * cols * d;
    const size_t pb2 = (size_t)max_planes(d, ff) * cols * d;
    c.accA = cv.take<int32_t>(pa1 > pa2 ? pa1 : pa2);
    c.accB = cv.take<int32_t>(pb1 > pb2 ? pb1 : pb2);
    c.d_pos = cv.take<int>(c.max_batch > 1 ? c.max_batch : 1);  // cached length of every sequence
    c.rope_buf = cv.take<float2>((size_t)c.max_seq * (c.head_dim / 2));
    c.nsplit = attn_decode_nsplit_for(c.n_heads, c.n_kv_heads, c.head_dim, c.max_seq);
    const size_t heads = (size_t)c.max_batch * c.n_heads * c.nsplit;
    c.part_o = cv.take<float>(heads * c.head_dim);
    c.part_m = cv.take<float>(heads);
    c.part_l = cv.take<float>(heads);
    c.counters = cv.take<unsigned>(8 + (size_t)c.max_batch);
    // (positions rounded up to whole 64-key tiles: the tensor-memory attention kernel reads whole tiles)
    c.kvsplit_plane = (size_t)c.max_batch * c.n_kv_heads * ((c.max_seq + 63) / 64 * 64) * c.head_dim;
    c.kvsplit = rows >= 64 ? cv.take<__nv_bfloat16>(4 * c.kvsplit_plane) : nullptr;  // prompts long enough to tile
    c.stat[0] = cv.take<float>(rows);
    c.stat[1] = cv.take<float>(rows);
    c.gated = cv.take<float>(c.tp_size > 1 ? rows * ff : 1);
    const size_t outs[4] = {qkv_out, d, ff, d};
    for (int i = 0; i < 4; ++i) c.fy[i] = cv.take<float>(FUSED_MAX_ROWS * outs[i]);
}

// One-time device initialisation of a carved context: tail counters and the rotary table.
static int init_ctx(Ctx& c, cudaStream_t st) {
    RB_CUDA(cudaMemsetAsync(c.counters, 0, (8 + (size_t)c.max_batch) * sizeof(unsigned), st));
    c.rope = nullptr;
    if (c.rope_theta > 0.f) {
        int rc = launch_rope_table(c.rope_buf, c.max_seq, c.head_dim, c.rope_theta, st);
        if (rc) return rc;
        c.rope = c.rope_buf;
    }
    return ROTOR_B200_OK;
}

static void carve(Model& m, unsigned char* base, size_t* total) {
    const rotor_b200_model_config& c = m.cfg;
    const size_t rows = (size_t)c.max_rows;
    Carve cv{base, 0};
    carve_ctx(m.c, cv, rows);
    const size_t nparts = (size_t)(lmhead_parts() > lmhead_mma_parts(c.vocab_size) ? lmhead_parts()
                                                                                  : lmhead_mma_parts(c.vocab_size));
    m.part_val = cv.take<float>(rows * nparts);
    m.part_idx = cv.take<int>(rows * nparts);
    m.xsplit = rows > 4 ? cv.take<__nv_bfloat16>(2 * rows * (size_t)c.d_model) : nullptr;
    m.cur_ids = cv.take<long long>(c.max_batch);
    m.max_log = c.max_seq;
    m.tok_log = cv.take<long long>((size_t)m.max_log * c.max_batch);
    m.d_step = cv.take<int>(1);
    m.d_lens = cv.take<int>(c.max_batch > 1 ? c.max_batch : 1);
    const size_t tp = c.tp_size > 1 ? c.tp_size : 1;
    m.pick_val = cv.take<float>(rows);
    m.pick_idx = cv.take<long long>(rows);
    m.pick_send = cv.take<unsigned char>(rows * 12);
    m.pick_recv = cv.take<unsigned char>(tp * rows * 12);
    *total = cv.off;
}

static int derive(Model& m) {
    const rotor_b200_model_config& c = m.cfg;
    if (c.vocab_size <= 0 || c.n_layers <= 0 || c.max_batch <= 0 || c.max_seq <= 0 || c.max_rows <= 0)
        return ROTOR_B200_ERR_ARG;
    int rc = derive_ctx(m.c, c.d_model, c.n_heads, c.n_kv_heads, c.d_ff, c.act_terms, c.tp_size);
    if (rc) return rc;
    if (c.tp_size > 1) {
        if (c.act_terms != 1) return ROTOR_B200_ERR_SHAPE;      // sharded rows share one absmax per row: one term only
        if (c.vocab_size % c.tp_size || c.tp_rank < 0 || c.tp_rank >= c.tp_size) return ROTOR_B200_ERR_SHAPE;
    }
    m.c.max_batch = c.max_batch;
    if (c.d_model % 256) return ROTOR_B200_ERR_SHAPE;  // LM head reads 256 columns per warp step
    m.c.ffn_act = c.ffn_act;
    m.c.causal = c.causal;
    m.c.variant = c.gemv_variant;
    m.c.max_seq = c.max_seq;
    m.c.rope_theta = c.rope_theta;
    m.c.eps = c.eps;
    return ROTOR_B200_OK;
}

// Cached length of every sequence: one value for all, or lens[b] when given.
__global__ void set_pos_kernel(int* pos, int n, int v, const int* lens) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) pos[i] = lens ? lens[i] : v;
}

__global__ void begin_kernel(long long* cur, const long long* first, int batch, int* pos, int past, const int* lens,
                             int* step) {
    if (threadIdx.x < batch) {
        cur[threadIdx.x] = first[threadIdx.x];
        pos[threadIdx.x] = lens ? lens[threadIdx.x] : past;
    }
    if (threadIdx.x == 0) *step = 0;
}

// After a generation step: log the picked tokens and move the position on.
__global__ void advance_kernel(const long long* cur, long long* log, int batch, int max_log, int* pos, int* step) {
    const int s = *step;
    if (threadIdx.x < batch && s < max_log) log[(size_t)s * batch + threadIdx.x] = cur[threadIdx.x];
    __syncthreads();
    if (threadIdx.x < batch) pos[threadIdx.x] += 1;
    if (threadIdx.x == 0) *step = s + 1;
}

#define RB_TRY(expr)              \
    do {                          \
        int rc_ = (expr);         \
        if (rc_) return rc_;      \
    } while (0)

// One BitLinear product into partial planes, activations taken from xq/xsum[xs].
static int gemv(Ctx& c, const void* tiles, size_t out, size_t in, int ncols, int xs, int32_t* acc, AccView* view,
                cudaStream_t st) {
    GemvPlan plan = plan_gemv(out, in, ncols < 8 ? ncols : 8);
    // five and more columns: the K splits add into one plane, so that the register-resident row stages
    // (complete sums in one plane) can follow; fewer columns keep one plane per split, which the
    // generation-step stages add while they dequantise
    const bool gemm = ncols >= GEMM_MIN_COLS && c.variant == ROTOR_B200_VARIANT_AUTO;
    const bool one_plane = gemm || ncols >= 5;
    const size_t plane_stride = one_plane ? 0 : (size_t)ncols * out;
    view->acc = acc;
    view->plane_stride = plane_stride;
    // (many columns go to the tiled GEMM, which leaves complete sums in the first plane)
    view->planes = one_plane ? 1 : plan.ksplit;
    view->out = (int)out;
    return launch_gemv_planes(tiles, out, in, c.xq, c.xsum[xs], ncols, acc, plane_stride, plan, c.variant, st);
}

static void quant_sink(const Ctx& c, VecStageParams& p, int slot, int n) {
    p.xq = c.xq;
    p.sx_out = c.sx[slot];
    p.xsum_out = c.xsum[slot];
    p.terms_out = c.terms;
    p.kpad = (int)kpad_of(n);
}

// Attention half of a block.  In: quantised pre-normed rows in xq/sx[0]/xsum[0].
// Out: accumulators of the output projection (view *vo), activation scales in sx[1].
static int attention_part(Ctx& c, const rotor_b200_layer_weights& L, int batch, int seq, AccView* vo,
                          cudaStream_t st) {
    const int rows = batch * seq, cols = rows * c.terms;
    const size_t qkv_out = (size_t)c.dq + 2 * c.dkv;
    // prompt-sized row counts, one activation term, head_dim 128: the q/k/v product dequantises, rotates and
    // appends to the cache in its read-back (no int32 accumulators, no separate finish kernel)
    const bool fuse_qkv = c.terms == 1 && c.variant == ROTOR_B200_VARIANT_AUTO && seq >= 16 &&
                          gemm_tcgen05_qkv_supported((size_t)c.dq, (size_t)c.dkv, c.d, c.head_dim, cols, c.xq);
    AccView va = {};
    if (!fuse_qkv) RB_TRY(gemv(c, L.qkv_tiles, qkv_out, c.d, cols, 0, c.accA, &va, st));
    // (sixteen and more sequences: the tiled attention kernel streams each sequence's cache once per
    // group of heads, which beats thousands of small split CTAs; measured on the XL shape, batch 64)
    // 5 to 63 sequences: the streaming kernel over runs of every sequence (about 512 CTAs), partial results
    // merged by the stage that quantises the attention rows
    const int runs = (seq == 1 && batch >= 5 && batch <= c.max_batch)
                         ? attn_stream_splits(batch, c.n_heads, c.n_kv_heads, c.head_dim, c.nsplit) : 0;
    if (seq == 1 && batch <= c.max_batch && batch < 16 && runs <= 1) {
        // generation step: dequantise, rotate, append to the cache, attend, merge and quantise in one launch
        AttnDecodeParams dp = {};
        dp.acc = va;
        dp.sx = c.sx[0];
        dp.terms = c.terms;
        dp.sq = L.q_scale;
        dp.sk = L.k_scale;
        dp.sv = L.v_scale;
        dp.n_heads = c.n_heads;
        dp.n_kv_heads = c.n_kv_heads;
        dp.head_dim = c.head_dim;
        dp.max_seq = c.max_seq;
        dp.nsplit = c.nsplit;
        dp.past_len = c.d_pos;
        dp.rope = c.rope;
        dp.k_cache = L.k_cache;
        dp.v_cache = L.v_cache;
        dp.part_o = c.part_o;
        dp.part_m = c.part_m;
        dp.part_l = c.part_l;
        dp.counter = c.counters + 8;
        dp.xq = c.xq;
        dp.sx_out = c.sx[1];
        dp.xsum_out = c.xsum[1];
        dp.terms_out = c.terms;
        dp.kpad = (int)kpad_of(c.dq);
        RB_TRY(launch_attn_decode(dp, batch, st));
        return gemv(c, L.o_tiles, c.d, c.dq, cols, 1, c.accB, vo, st);
    }
    QkvFinishParams qf = {};
    qf.acc = va;
    qf.sx = c.sx[0];
    qf.terms = c.terms;
    qf.sq = L.q_scale;
    qf.sk = L.k_scale;
    qf.sv = L.v_scale;
    qf.n_heads = c.n_heads;
    qf.n_kv_heads = c.n_kv_heads;
    qf.head_dim = c.head_dim;
    qf.seq = seq;
    qf.past_len = c.d_pos;
    qf.max_seq = c.max_seq;
    qf.rope = c.rope;
    qf.q = c.qbuf;
    qf.k_cache = L.k_cache;
    qf.v_cache = L.v_cache;
    if (fuse_qkv)
        RB_TRY(launch_gemm_tcgen05_qkv(L.qkv_tiles, c.d, c.xq, c.sx[0], c.xsum[0], cols, qf, st));
    else
        RB_TRY(launch_qkv_finish(qf, rows, st));
    AttnParams ap = {};
    ap.q = c.qbuf;
    ap.k_cache = L.k_cache;
    ap.v_cache = L.v_cache;
    ap.out = c.attn;
    ap.n_heads = c.n_heads;
    ap.n_kv_heads = c.n_kv_heads;
    ap.head_dim = c.head_dim;
    ap.seq = seq;
    ap.past_len = c.d_pos;
    ap.max_seq = c.max_seq;
    ap.causal = c.causal;
    ap.kv_split = seq >= 16 ? c.kvsplit : nullptr;  // a key tile shared by several query tiles is split once
    ap.split_plane = c.kvsplit_plane;
    if (runs > 1) {
        ap.nsplit = runs;
        ap.part_o = c.part_o;
        ap.part_m = c.part_m;
        ap.part_l = c.part_l;
    }
    RB_TRY(launch_attention(ap, rows, st));
    VecStageParams qa = {};
    qa.mode = runs > 1 ? VS_ATTN : VS_PLAIN;
    qa.n = c.dq;
    qa.src = c.attn;
    qa.part_o = c.part_o;
    qa.part_m = c.part_m;
    qa.part_l = c.part_l;
    qa.nsplit = runs;
    qa.n_heads = c.n_heads;
    qa.head_dim = c.head_dim;
    qa.eps = c.eps;
    quant_sink(c, qa, 1, c.dq);
    RB_TRY(launch_vec_stage(qa, rows, st));
    return gemv(c, L.o_tiles, c.d, c.dq, cols, 1, c.accB, vo, st);
}

// FFN half of a block.  In: quantised pre-normed rows in xq/sx[0]/xsum[0].
// Out: accumulators of the down projection (view *vd), activation scales in sx[1].
static int ffn_part(Ctx& c, const rotor_b200_layer_weights& L, int rows, AccView* vd, cudaStream_t st) {
    const int cols = rows * c.terms;
    if (c.terms == 1 && c.tp_size <= 1 && c.variant == ROTOR_B200_VARIANT_AUTO &&
        gemm_tcgen05_gated_supported((size_t)c.ff, c.d, cols, c.xq)) {
        // prompt-sized row counts, one activation term: the gate/up product applies the gating in its epilogue and
        // writes float32 gated rows (into the accumulator area: a quarter of the bytes of the two int32 halves);
        // the stage that follows only has to sub-norm and quantise them
        float* gated = reinterpret_cast<float*>(c.accA);
        RB_TRY(launch_gemm_tcgen05_gated(L.gate_up_tiles, (size_t)c.ff, c.d, c.xq, c.sx[0], c.xsum[0], cols, L.gate_scale, L.up_scale,
                                         c.ffn_act, gated, st));
        VecStageParams gp = {};
        gp.mode = VS_PLAIN;
        gp.n = c.ff;
        gp.src = gated;
        gp.norm1 = L.ffn_sub_norm;
        gp.eps = c.eps;
        quant_sink(c, gp, 1, c.ff);
        RB_TRY(launch_vec_stage(gp, rows, st));
        return gemv(c, L.down_tiles, c.d, c.ff, cols, 1, c.accB, vd, st);
    }
    AccView va;
    RB_TRY(gemv(c, L.gate_up_tiles, 2 * (size_t)c.ff, c.d, cols, 0, c.accA, &va, st));
    VecStageParams fp = {};
    fp.mode = VS_FFN;
    fp.n = c.ff;
    fp.acc = va;
    fp.sx_in = c.sx[0];
    fp.terms = c.terms;
    fp.wscale0 = L.gate_scale;
    fp.wscale1 = L.up_scale;
    fp.ffn_act = c.ffn_act;
    fp.norm1 = L.ffn_sub_norm;
    fp.eps = c.eps;
    quant_sink(c, fp, 1, c.ff);
    RB_TRY(launch_vec_stage(fp, rows, st));
    return gemv(c, L.down_tiles, c.d, c.ff, cols, 1, c.accB, vd, st);
}

// Blocks [l0, l1) on the residual stream c.h, whose pre-normed quantised copy is already in
// xq/sx[0].  `next_norm` is the norm weight that follows block l1-1 (the next block's
// pre-norm or the model's final norm); with `to_float` the normed rows go to c.hn instead
// of the quantiser.
static int run_blocks(Ctx& c, const rotor_b200_layer_weights* layers, int l0, int l1, const float* next_norm,
                      bool to_float, int batch, int seq, cudaStream_t st) {
    const int rows = batch * seq;
    for (int l = l0; l < l1; ++l) {
        const rotor_b200_layer_weights& L = layers[l];
        AccView vo, vd;
        RB_TRY(attention_part(c, L, batch, seq, &vo, st));
        VecStageParams op = {};
        op.mode = VS_OPROJ;
        op.n = c.d;
        op.acc = vo;
        op.sx_in = c.sx[1];
        op.terms = c.terms;
        op.wscale0 = L.o_scale;
        op.norm0 = L.attn_sub_norm;
        op.h = c.h;
        op.norm1 = L.post_attn_norm;
        op.eps = c.eps;
        quant_sink(c, op, 0, c.d);
        RB_TRY(launch_vec_stage(op, rows, st));
        RB_TRY(ffn_part(c, L, rows, &vd, st));
        VecStageParams dn = {};
        dn.mode = VS_DOWN;
        dn.n = c.d;
        dn.acc = vd;
        dn.sx_in = c.sx[1];
        dn.terms = c.terms;
        dn.wscale0 = L.down_scale;
        dn.h = c.h;
        dn.eps = c.eps;
        const bool last = l + 1 == l1;
        dn.norm1 = last ? next_norm : layers[l + 1].input_norm;
        if (last && to_float)
            dn.y_out = c.hn;
        else
            quant_sink(c, dn, 0, c.d);
        RB_TRY(launch_vec_stage(dn, rows, st));
    }
    return ROTOR_B200_OK;
}

// One generation step (one token per sequence) with every vector stage fused into the
// prologue of the product that consumes it: 5 launches per block plus the LM head.
//   q/k/v product   <- [embedding | previous down: residual add] + input norm + quantise
//   attention       <- dequantise q/k/v, rotate, cache append, slice partials
//   o product       <- merge attention partials + quantise
//   gate/up product <- o: sub-norm, residual add, post-attention norm, quantise
//   down product    <- gating, sub-norm, quantise
//   LM head         <- last down: residual add, final norm; greedy pick in its last CTA
// The residual stream alternates between c.h and c.h2 so that the CTA that writes the new
// stream never races with CTAs still reading the old one.
static bool fused_step_ok(const Model& m, int batch, int seq) {
    const Ctx& c = m.c;
    static const bool off = getenv("ROTOR_B200_NO_FUSED_STEP") != nullptr;  // measurement aid
    const size_t qkv_out = (size_t)c.dq + 2 * c.dkv;
    const bool tp_ok = c.tp_size <= 1 || (c.terms == 1 && tp_fused_ready(c.tp) && (size_t)batch * c.d <= (size_t)XCH_CAP);
    const bool shape_ok = !off && tp_ok && seq == 1 && batch <= FUSED_MAX_ROWS && batch <= c.max_batch &&
                          c.terms <= 3 && batch * c.terms <= 8 && c.ff % 16 == 0;
    const bool q = fused_gemv_supported(qkv_out, c.d, batch, c.terms, 1, 0);
    const bool o = fused_gemv_supported(c.d, c.dq, batch, c.terms, 1, c.n_heads * c.nsplit);
    const bool g = fused_gemv_supported(c.ff, c.d, batch, c.terms, 2, 0);
    const bool dn = fused_gemv_supported(c.d, c.ff, batch, c.terms, 1, 0);
    return shape_ok && q && o && g && dn;
}

static int run_step_fused(Model& m, const long long* ids, int batch, int logits_mode, float* logits,
                          long long* next_ids, cudaStream_t st, bool advance) {
    Ctx& c = m.c;
    const int d = c.d;
    const size_t qkv_out = (size_t)c.dq + 2 * c.dkv;
    const bool cluster = attn_decode_cluster_ok(c.n_heads, c.n_kv_heads, c.head_dim, c.max_seq, c.nsplit);
    auto product = [&](const void* tiles, size_t out, size_t in, int halves, const LeanStage& stg, float* y,
                       const float* scale, int seg1, int seg2, int act) {
        return launch_fused_gemv(tiles, out, in, halves, batch, stg, y, scale, seg1, seg2, act, st);
    };
    LeanStage ls;
    auto stage = [&](int mode, int n) {
        ls = {};
        ls.mode = mode;
        ls.n = n;
        ls.eps = c.eps;
        ls.terms = c.terms;
        ls.kpad = (int)kpad_of(n);
    };
    for (int l = 0; l < m.cfg.n_layers; ++l) {
        const rotor_b200_layer_weights& L = m.layers[l];
        // q/k/v <- [embedding | h2 + previous down] -> h, input norm
        if (l == 0) {
            stage(LM_EMBED, d);
            ls.ids = ids;
            ls.embed = m.embed;
        } else {
            stage(LM_ADD, d);
            ls.y = c.fy[3];
            ls.h = c.h2;
        }
        ls.h_out = c.h;
        ls.norm1 = L.input_norm;
        const float sqkv[3] = {L.q_scale, L.k_scale, L.v_scale};
        RB_TRY(product(L.qkv_tiles, qkv_out, d, 1, ls, c.fy[0], sqkv, c.dq, c.dq + c.dkv, 0));

        AttnDecodeParams dp = {};
        dp.qkv_f = c.fy[0];
        dp.n_heads = c.n_heads;
        dp.n_kv_heads = c.n_kv_heads;
        dp.head_dim = c.head_dim;
        dp.max_seq = c.max_seq;
        dp.nsplit = c.nsplit;
        dp.past_len = c.d_pos;
        dp.rope = c.rope;
        dp.k_cache = L.k_cache;
        dp.v_cache = L.v_cache;
        dp.part_o = c.part_o;
        dp.part_m = c.part_m;
        dp.part_l = c.part_l;
        dp.attn_out = c.attn;
        if (cluster) {
            // o <- finished attention rows (the cluster merges its slices itself)
            RB_TRY(launch_attn_decode_cluster(dp, batch, st));
            stage(LM_PLAIN, c.dq);
            ls.y = c.attn;
        } else {
            RB_TRY(launch_attn_decode(dp, batch, st));  // no counter: the o product merges the partials
            stage(LM_ATTN, c.dq);
            ls.part_o = c.part_o;
            ls.part_m = c.part_m;
            ls.part_l = c.part_l;
            ls.nsplit = c.nsplit;
            ls.n_heads = c.n_heads;
            ls.head_dim = c.head_dim;
        }
        const float so[3] = {L.o_scale, L.o_scale, L.o_scale};
        RB_TRY(product(L.o_tiles, d, c.dq, 1, ls, c.fy[1], so, d, d, 0));

        // gate/up <- h + subnorm(o) -> h2, post-attention norm; gating in the epilogue
        stage(LM_SUBNORM_ADD, d);
        ls.y = c.fy[1];
        ls.h = c.h;
        ls.h_out = c.h2;
        ls.norm0 = L.attn_sub_norm;
        ls.norm1 = L.post_attn_norm;
        const float sgu[3] = {L.gate_scale, L.up_scale, 0.f};
        RB_TRY(product(L.gate_up_tiles, c.ff, d, 2, ls, c.fy[2], sgu, 0, 0, c.ffn_act));

        // down <- sub-norm(gated)
        stage(LM_PLAIN, c.ff);
        ls.y = c.fy[2];
        ls.norm1 = L.ffn_sub_norm;
        const float sd[3] = {L.down_scale, L.down_scale, L.down_scale};
        RB_TRY(product(L.down_tiles, d, c.ff, 1, ls, c.fy[3], sd, d, d, 0));
    }
    // LM head: h2 + last down, final norm in its prologue; greedy pick in its last CTA
    LmHeadParams lp = {};
    lp.embed = m.embed;
    lp.vocab = m.cfg.vocab_size;
    lp.d = d;
    lp.logits = logits_mode == ROTOR_B200_LOGITS_NONE ? nullptr : logits;
    lp.part_val = m.part_val;
    lp.part_idx = m.part_idx;
    lp.argmax_out = next_ids;
    lp.nparts = lmhead_parts();
    lp.tail_counter = next_ids ? c.counters + 3 : nullptr;
    if (advance) {
        lp.adv_log = m.tok_log;
        lp.adv_pos = c.d_pos;
        lp.adv_step = m.d_step;
        lp.adv_max_log = m.max_log;
    }
    lp.pro_y = c.fy[3];
    lp.pro_h = c.h2;
    lp.pro_norm = m.final_norm;
    lp.pro_eps = c.eps;
    return launch_lmhead(lp, batch, st);
}

// ---------------------------------------------------------------------------------------
// Tensor-parallel forward (one process per GPU).  q/k/v, gate and up are split by output
// rows (whole heads / FFN channels per rank), o and down by input columns; their int32
// partial sums are all-reduced (exact: every rank quantises its slice of the input with the
// row's global absolute maximum, obtained with a one-float-per-row all-reduce, so all ranks
// share the activation scale).  The FFN sub-norm runs over the sharded row and needs the
// global sum of squares the same way.  Per block: 3 one-float-per-row all-reduces and
// 2 all-reduces of rows*d_model int32.  The LM head is split by vocabulary; the greedy pick
// all-gathers one (value, index) pair per rank and row.
__global__ void pack_pick_kernel(const float* val, const long long* idx, long long idx_offset, int rows,
                                 unsigned char* out) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    float v = val[r];
    long long i = idx[r] + idx_offset;
    memcpy(out + (size_t)r * 12, &v, 4);
    memcpy(out + (size_t)r * 12 + 4, &i, 8);
}

__global__ void final_pick_kernel(const unsigned char* recv, int tp, int rows, long long* out) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    float bv = -INFINITY;
    long long bi = 0x7fffffffffffffffLL;
    for (int k = 0; k < tp; ++k) {
        float v;
        long long i;
        memcpy(&v, recv + ((size_t)k * rows + r) * 12, 4);
        memcpy(&i, recv + ((size_t)k * rows + r) * 12 + 4, 8);
        if (v > bv || (v == bv && i < bi)) {
            bv = v;
            bi = i;
        }
    }
    out[r] = bi;
}

static int acc1(Ctx& c, const void* tiles, size_t out, size_t in, int ncols, int xs, int32_t* acc, AccView* view,
                cudaStream_t st) {
    view->acc = acc;
    view->plane_stride = 0;
    view->planes = 1;
    view->out = (int)out;
    return rotor_b200_bitlinear_acc(tiles, out, in, c.xq, c.xsum[xs], (size_t)ncols, acc, c.variant, st);
}

static int run_blocks_tp(Model& m, int l0, int l1, const float* next_norm, bool to_float, int batch, int seq,
                         cudaStream_t st) {
    Ctx& c = m.c;
    const int rows = batch * seq, d = c.d, cols = rows;  // one activation term
    const size_t qkv_out = (size_t)c.dq + 2 * c.dkv;
    for (int l = l0; l < l1; ++l) {
        const rotor_b200_layer_weights& L = m.layers[l];
        AccView va, vb;
        // ---- attention on this rank's heads
        RB_TRY(acc1(c, L.qkv_tiles, qkv_out, d, cols, 0, c.accA, &va, st));
        if (seq == 1 && batch <= c.max_batch && batch < 16) {
            AttnDecodeParams dp = {};
            dp.acc = va;
            dp.sx = c.sx[0];
            dp.terms = 1;
            dp.sq = L.q_scale;
            dp.sk = L.k_scale;
            dp.sv = L.v_scale;
            dp.n_heads = c.n_heads;
            dp.n_kv_heads = c.n_kv_heads;
            dp.head_dim = c.head_dim;
            dp.max_seq = c.max_seq;
            dp.nsplit = c.nsplit;
            dp.past_len = c.d_pos;
            dp.rope = c.rope;
            dp.k_cache = L.k_cache;
            dp.v_cache = L.v_cache;
            dp.part_o = c.part_o;
            dp.part_m = c.part_m;
            dp.part_l = c.part_l;
            dp.counter = c.counters + 8;
            dp.attn_out = c.attn;  // merged rows as float; quantised below with the global maximum
            RB_TRY(launch_attn_decode(dp, batch, st));
        } else {
            QkvFinishParams qf = {};
            qf.acc = va;
            qf.sx = c.sx[0];
            qf.terms = 1;
            qf.sq = L.q_scale;
            qf.sk = L.k_scale;
            qf.sv = L.v_scale;
            qf.n_heads = c.n_heads;
            qf.n_kv_heads = c.n_kv_heads;
            qf.head_dim = c.head_dim;
            qf.seq = seq;
            qf.past_len = c.d_pos;
            qf.max_seq = c.max_seq;
            qf.rope = c.rope;
            qf.q = c.qbuf;
            qf.k_cache = L.k_cache;
            qf.v_cache = L.v_cache;
            RB_TRY(launch_qkv_finish(qf, rows, st));
            AttnParams ap = {};
            ap.q = c.qbuf;
            ap.k_cache = L.k_cache;
            ap.v_cache = L.v_cache;
            ap.out = c.attn;
            ap.n_heads = c.n_heads;
            ap.n_kv_heads = c.n_kv_heads;
            ap.head_dim = c.head_dim;
            ap.seq = seq;
            ap.past_len = c.d_pos;
            ap.max_seq = c.max_seq;
            ap.causal = c.causal;
            ap.kv_split = seq >= 16 ? c.kvsplit : nullptr;  // a key tile shared by several query tiles is split once
            ap.split_plane = c.kvsplit_plane;
            RB_TRY(launch_attention(ap, rows, st));
        }
        // o projection input: global absolute maximum, then quantise the local slice
        VecStageParams sa = {};
        sa.mode = VS_PLAIN;
        sa.n = c.dq;
        sa.src = c.attn;
        sa.eps = c.eps;
        sa.out_absmax = c.stat[0];
        RB_TRY(launch_vec_stage(sa, rows, st));
        RB_TRY(tp_allreduce_f32(c.tp, c.stat[0], rows, true, st));
        VecStageParams qa = {};
        qa.mode = VS_PLAIN;
        qa.n = c.dq;
        qa.src = c.attn;
        qa.eps = c.eps;
        qa.ext_absmax = c.stat[0];
        quant_sink(c, qa, 1, c.dq);
        RB_TRY(launch_vec_stage(qa, rows, st));
        RB_TRY(acc1(c, L.o_tiles, d, c.dq, cols, 1, c.accB, &vb, st));
        RB_TRY(tp_allreduce_sum_i32(c.tp, c.accB, (size_t)cols * d, st));
        VecStageParams op = {};
        op.mode = VS_OPROJ;
        op.n = d;
        op.acc = vb;
        op.sx_in = c.sx[1];
        op.terms = 1;
        op.wscale0 = L.o_scale;
        op.norm0 = L.attn_sub_norm;
        op.h = c.h;
        op.norm1 = L.post_attn_norm;
        op.eps = c.eps;
        quant_sink(c, op, 0, d);
        RB_TRY(launch_vec_stage(op, rows, st));
        // ---- FFN on this rank's channels
        RB_TRY(acc1(c, L.gate_up_tiles, 2 * (size_t)c.ff, d, cols, 0, c.accA, &va, st));
        VecStageParams fp = {};
        fp.mode = VS_FFN;
        fp.n = c.ff;
        fp.acc = va;
        fp.sx_in = c.sx[0];
        fp.terms = 1;
        fp.wscale0 = L.gate_scale;
        fp.wscale1 = L.up_scale;
        fp.ffn_act = c.ffn_act;
        fp.eps = c.eps;
        fp.y_out = c.gated;
        fp.out_sumsq = c.stat[0];
        RB_TRY(launch_vec_stage(fp, rows, st));
        RB_TRY(tp_allreduce_f32(c.tp, c.stat[0], rows, false, st));
        VecStageParams fn = {};
        fn.mode = VS_PLAIN;
        fn.n = c.ff;
        fn.src = c.gated;
        fn.norm1 = L.ffn_sub_norm;  // this rank's slice of the sub-norm weight
        fn.ext_sumsq = c.stat[0];
        fn.norm_n = c.ff_total;
        fn.eps = c.eps;
        fn.y_out = c.gated;
        fn.out_absmax = c.stat[1];
        RB_TRY(launch_vec_stage(fn, rows, st));
        RB_TRY(tp_allreduce_f32(c.tp, c.stat[1], rows, true, st));
        VecStageParams fq = {};
        fq.mode = VS_PLAIN;
        fq.n = c.ff;
        fq.src = c.gated;
        fq.eps = c.eps;
        fq.ext_absmax = c.stat[1];
        quant_sink(c, fq, 1, c.ff);
        RB_TRY(launch_vec_stage(fq, rows, st));
        RB_TRY(acc1(c, L.down_tiles, d, c.ff, cols, 1, c.accB, &vb, st));
        RB_TRY(tp_allreduce_sum_i32(c.tp, c.accB, (size_t)cols * d, st));
        VecStageParams dn = {};
        dn.mode = VS_DOWN;
        dn.n = d;
        dn.acc = vb;
        dn.sx_in = c.sx[1];
        dn.terms = 1;
        dn.wscale0 = L.down_scale;
        dn.h = c.h;
        dn.eps = c.eps;
        const bool last = l + 1 == l1;
        dn.norm1 = last ? next_norm : m.layers[l + 1].input_norm;
        if (last && to_float)
            dn.y_out = c.hn;
        else
            quant_sink(c, dn, 0, d);
        RB_TRY(launch_vec_stage(dn, rows, st));
    }
    return ROTOR_B200_OK;
}

static int run_layers_tp(Model& m, const long long* ids, int batch, int seq, int logits_mode, float* logits,
                         long long* next_ids, cudaStream_t st, bool advance) {
    Ctx& c = m.c;
    const int rows = batch * seq, d = c.d;
    VecStageParams e = {};
    e.mode = VS_EMBED;
    e.n = d;
    e.ids = ids;
    e.embed = m.embed;
    e.h = c.h;
    e.norm1 = m.layers[0].input_norm;
    e.eps = c.eps;
    quant_sink(c, e, 0, d);
    RB_TRY(launch_vec_stage(e, rows, st));
    RB_TRY(run_blocks_tp(m, 0, m.cfg.n_layers, m.final_norm, true, batch, seq, st));
    if (logits_mode == ROTOR_B200_LOGITS_NONE && !next_ids) return ROTOR_B200_OK;

    // ---- LM head over this rank's vocabulary slice; logits (if asked for) are the local slice
    const bool all = logits_mode == ROTOR_B200_LOGITS_ALL;
    const int vl = m.cfg.vocab_size / c.tp_size, rank = tp_rank(c.tp);
    const float* x = c.hn;
    int lm_rows = rows;
    if (!all && seq > 1) {
        for (int b = 0; b < batch; ++b)
            RB_CUDA(cudaMemcpyAsync(c.qbuf + (size_t)b * d, c.hn + ((size_t)b * seq + (m.last_of ? m.last_of[b] : seq) - 1) * d, d * sizeof(float),
                                    cudaMemcpyDeviceToDevice, st));
        x = c.qbuf;
        lm_rows = batch;
    }
    LmHeadParams lp = {};
    lp.embed = m.embed + (size_t)rank * vl * d;
    lp.x = x;
    lp.xsplit = m.xsplit;
    lp.vocab = vl;
    lp.d = d;
    lp.logits = logits_mode == ROTOR_B200_LOGITS_NONE ? nullptr : logits;
    lp.part_val = m.part_val;
    lp.part_idx = m.part_idx;
    const bool pick = next_ids && !(all && seq > 1);
    lp.argmax_out = pick ? m.pick_idx : nullptr;
    lp.argmax_val = pick ? m.pick_val : nullptr;
    lp.nparts = lmhead_parts();
    RB_TRY(launch_lmhead(lp, lm_rows, st));
    if (pick) {
        pack_pick_kernel<<<(lm_rows + 127) / 128, 128, 0, st>>>(m.pick_val, m.pick_idx, (long long)rank * vl, lm_rows,
                                                                m.pick_send);
        RB_TRY(launch_status());
        RB_TRY(tp_allgather_bytes(c.tp, m.pick_send, m.pick_recv, (size_t)lm_rows * 12, st));
        final_pick_kernel<<<(lm_rows + 127) / 128, 128, 0, st>>>(m.pick_recv, c.tp_size, lm_rows, next_ids);
        RB_TRY(launch_status());
    }
    if (advance) {
        advance_kernel<<<1, 1024, 0, st>>>(next_ids, m.tok_log, batch, m.max_log, c.d_pos, m.d_step);
        RB_TRY(launch_status());
    }
    return ROTOR_B200_OK;
}

// Generation step of a tensor-parallel model with the vector stages fused into the products
// and the exchanges fused into them where they are scalars: per block
//   q/k/v product (this rank's heads)          <- residual add, input norm, quantise
//   attention (this rank's heads)
//   o product (this rank's columns)            <- merge partials, [max exchange], quantise; int32 partials out
//   all-reduce + dequantise                    -> float o output, replicated
//   gate/up product (this rank's channels)     <- sub-norm, residual add, post-attention norm, quantise; gating
//   down product (this rank's columns)         <- [sum exchange] sub-norm, [max exchange] quantise; int32 partials out
//   all-reduce + dequantise                    -> float down output, replicated
// then the LM head over this rank's vocabulary slice and the pick across ranks.  Seven launches
// per block; five exchanges, all through peer memory.  One activation term only.
static int run_step_fused_tp(Model& m, const long long* ids, int batch, long long* next_ids, cudaStream_t st,
                             bool advance) {
    Ctx& c = m.c;
    const int d = c.d;
    const size_t qkv_out = (size_t)c.dq + 2 * c.dkv;
    FusedTpExtra ex = {};
    ex.xs = tp_scalar_dev(c.tp);
    const bool cluster = attn_decode_cluster_ok(c.n_heads, c.n_kv_heads, c.head_dim, c.max_seq, c.nsplit);
    int xi = 0, big = 0;  // exchanges so far in this step; vector exchanges so far (slot parity)
    LeanStage ls;
    auto stage = [&](int mode, int n) {
        ls = {};
        ls.mode = mode;
        ls.n = n;
        ls.eps = c.eps;
        ls.terms = 1;
        ls.kpad = (int)kpad_of(n);
    };
    const float none[3] = {1.f, 1.f, 1.f};
    for (int l = 0; l < m.cfg.n_layers; ++l) {
        const rotor_b200_layer_weights& L = m.layers[l];
        if (l == 0) {
            stage(LM_EMBED, d);
            ls.ids = ids;
            ls.embed = m.embed;
        } else {
            stage(LM_ADD, d);
            ls.y = c.fy[3];
            ls.h = c.h2;
        }
        ls.h_out = c.h;
        ls.norm1 = L.input_norm;
        const float sqkv[3] = {L.q_scale, L.k_scale, L.v_scale};
        RB_TRY(launch_fused_gemv(L.qkv_tiles, qkv_out, d, 1, batch, ls, c.fy[0], sqkv, c.dq, c.dq + c.dkv, 0, st));

        AttnDecodeParams dp = {};
        dp.qkv_f = c.fy[0];
        dp.n_heads = c.n_heads;
        dp.n_kv_heads = c.n_kv_heads;
        dp.head_dim = c.head_dim;
        dp.max_seq = c.max_seq;
        dp.nsplit = c.nsplit;
        dp.past_len = c.d_pos;
        dp.rope = c.rope;
        dp.k_cache = L.k_cache;
        dp.v_cache = L.v_cache;
        dp.part_o = c.part_o;
        dp.part_m = c.part_m;
        dp.part_l = c.part_l;
        dp.attn_out = c.attn;
        if (cluster) {
            RB_TRY(launch_attn_decode_cluster(dp, batch, st));
            stage(LM_PLAIN, c.dq);
            ls.y = c.attn;
        } else {
            RB_TRY(launch_attn_decode(dp, batch, st));
            stage(LM_ATTN, c.dq);
            ls.part_o = c.part_o;
            ls.part_m = c.part_m;
            ls.part_l = c.part_l;
            ls.nsplit = c.nsplit;
            ls.n_heads = c.n_heads;
            ls.head_dim = c.head_dim;
        }
        ls.xi_max = ++xi;  // (index + 1)
        ex.part = c.accB;
        ex.sx_out = c.sx[1];
        RB_TRY(launch_fused_gemv(L.o_tiles, d, c.dq, 1, batch, ls, c.fy[1], none, d, d, 0, st, &ex));
        RB_TRY(tp_allreduce_dequant(c.tp, big++, xi++, c.accB, c.sx[1], L.o_scale, c.fy[1], batch, d, st));

        stage(LM_SUBNORM_ADD, d);
        ls.y = c.fy[1];
        ls.h = c.h;
        ls.h_out = c.h2;
        ls.norm0 = L.attn_sub_norm;
        ls.norm1 = L.post_attn_norm;
        const float sgu[3] = {L.gate_scale, L.up_scale, 0.f};
        RB_TRY(launch_fused_gemv(L.gate_up_tiles, c.ff, d, 2, batch, ls, c.fy[2], sgu, 0, 0, c.ffn_act, st));

        stage(LM_PLAIN, c.ff);
        ls.y = c.fy[2];
        ls.norm1 = L.ffn_sub_norm;  // this rank's slice of the weight
        ls.norm_n = c.ff_total;
        ls.xi_sum = ++xi;
        ls.xi_max = ++xi;
        RB_TRY(launch_fused_gemv(L.down_tiles, d, c.ff, 1, batch, ls, c.fy[3], none, d, d, 0, st, &ex));
        RB_TRY(tp_allreduce_dequant(c.tp, big++, xi++, c.accB, c.sx[1], L.down_scale, c.fy[3], batch, d, st));
    }
    // LM head over this rank's vocabulary slice (residual add and final norm in its prologue), pick across ranks
    const int vl = m.cfg.vocab_size / c.tp_size, rank = tp_rank(c.tp);
    LmHeadParams lp = {};
    lp.embed = m.embed + (size_t)rank * vl * d;
    lp.vocab = vl;
    lp.d = d;
    lp.part_val = m.part_val;
    lp.part_idx = m.part_idx;
    lp.argmax_out = m.pick_idx;
    lp.argmax_val = m.pick_val;
    lp.nparts = lmhead_parts();
    lp.tail_counter = c.counters + 3;
    lp.pro_y = c.fy[3];
    lp.pro_h = c.h2;
    lp.pro_norm = m.final_norm;
    lp.pro_eps = c.eps;
    RB_TRY(launch_lmhead(lp, batch, st));
    pack_pick_kernel<<<(batch + 127) / 128, 128, 0, st>>>(m.pick_val, m.pick_idx, (long long)rank * vl, batch, m.pick_send);
    RB_TRY(launch_status());
    RB_TRY(tp_allgather_bytes(c.tp, m.pick_send, m.pick_recv, (size_t)batch * 12, st));
    final_pick_kernel<<<(batch + 127) / 128, 128, 0, st>>>(m.pick_recv, c.tp_size, batch, next_ids);
    RB_TRY(launch_status());
    if (advance) {
        advance_kernel<<<1, 1024, 0, st>>>(next_ids, m.tok_log, batch, m.max_log, c.d_pos, m.d_step);
        RB_TRY(launch_status());
    }
    return tp_step_end(c.tp, xi, st);
}


// ids: device [batch*seq]; the position is read from c.d_pos by the kernels.
static int run_layers(Model& m, const long long* ids, int batch, int seq, int logits_mode, float* logits,
                      long long* next_ids, cudaStream_t st, bool advance = false) {
    Ctx& c = m.c;
    if (c.tp_size > 1) {
        if (!c.tp) return ROTOR_B200_ERR_ARG;  // rotor_b200_model_set_tp has not been called
        if (fused_step_ok(m, batch, seq) && next_ids && logits_mode == ROTOR_B200_LOGITS_NONE)
            return run_step_fused_tp(m, ids, batch, next_ids, st, advance);
        return run_layers_tp(m, ids, batch, seq, logits_mode, logits, next_ids, st, advance);
    }
    if (fused_step_ok(m, batch, seq) && (logits_mode != ROTOR_B200_LOGITS_NONE || next_ids))
        return run_step_fused(m, ids, batch, logits_mode, logits, next_ids, st, advance);
    const int rows = batch * seq, d = c.d;
    VecStageParams e = {};
    e.mode = VS_EMBED;
    e.n = d;
    e.ids = ids;
    e.embed = m.embed;
    e.h = c.h;
    e.norm1 = m.layers[0].input_norm;
    e.eps = c.eps;
    quant_sink(c, e, 0, d);
    RB_TRY(launch_vec_stage(e, rows, st));
    RB_TRY(run_blocks(c, m.layers, 0, m.cfg.n_layers, m.final_norm, true, batch, seq, st));
    if (logits_mode == ROTOR_B200_LOGITS_NONE && !next_ids) return ROTOR_B200_OK;

    // LM head over the last position of each sequence, or over every position
    const bool all = logits_mode == ROTOR_B200_LOGITS_ALL;
    const float* x = c.hn;
    int lm_rows = rows;
    if (!all && seq > 1) {
        // compact the last rows: hn[b*seq + seq-1] -> qbuf[b] (qbuf is free by now)
        for (int b = 0; b < batch; ++b)
            RB_CUDA(cudaMemcpyAsync(c.qbuf + (size_t)b * d, c.hn + ((size_t)b * seq + (m.last_of ? m.last_of[b] : seq) - 1) * d, d * sizeof(float),
                                    cudaMemcpyDeviceToDevice, st));
        x = c.qbuf;
        lm_rows = batch;
    }
    LmHeadParams lp = {};
    lp.embed = m.embed;
    lp.x = x;
    lp.xsplit = m.xsplit;
    lp.vocab = m.cfg.vocab_size;
    lp.d = d;
    lp.logits = logits_mode == ROTOR_B200_LOGITS_NONE ? nullptr : logits;
    lp.part_val = m.part_val;
    lp.part_idx = m.part_idx;
    lp.argmax_out = (all && seq > 1) ? nullptr : next_ids;
    lp.nparts = lmhead_parts();
    lp.tail_counter = c.counters + 3;
    if (advance) {
        lp.adv_log = m.tok_log;
        lp.adv_pos = c.d_pos;
        lp.adv_step = m.d_step;
        lp.adv_max_log = m.max_log;
    }
    return launch_lmhead(lp, lm_rows, st);
}

}  // namespace rb

using namespace rb;

extern "C" {

size_t rotor_b200_model_workspace_bytes(const rotor_b200_model_config* cfg) {
    if (!cfg) return 0;
    Model m;
    memset(&m, 0, sizeof(m));
    m.cfg = *cfg;
    if (derive(m)) return 0;
    size_t total = 0;
    carve(m, nullptr, &total);
    return total;
}

int rotor_b200_model_create(const rotor_b200_model_config* cfg, const rotor_b200_layer_weights* layers,
                            const void* embed_bf16, const float* final_norm, void* workspace,
                            size_t workspace_bytes, void** handle) {
    RB_REQUIRE(cfg && layers && embed_bf16 && final_norm && workspace && handle);
    RB_REQUIRE(((uintptr_t)workspace & 255) == 0);
    Model* m = new (std::nothrow) Model;
    if (!m) return ROTOR_B200_ERR_ARG;
    memset(m, 0, sizeof(*m));
    m->cfg = *cfg;
    int rc = derive(*m);
    if (rc) {
        delete m;
        return rc;
    }
    size_t total = 0;
    carve(*m, (unsigned char*)workspace, &total);
    if (total > workspace_bytes) {
        delete m;
        return ROTOR_B200_ERR_WORKSPACE;
    }
    m->layers = (rotor_b200_layer_weights*)malloc(sizeof(rotor_b200_layer_weights) * cfg->n_layers);
    memcpy(m->layers, layers, sizeof(rotor_b200_layer_weights) * cfg->n_layers);
    for (int l = 0; l < cfg->n_layers; ++l) {
        const rotor_b200_layer_weights& L = m->layers[l];
        if (!L.qkv_tiles || !L.o_tiles || !L.gate_up_tiles || !L.down_tiles || !L.input_norm ||
            !L.post_attn_norm || !L.attn_sub_norm || !L.ffn_sub_norm || !L.k_cache || !L.v_cache) {
            free(m->layers);
            delete m;
            return ROTOR_B200_ERR_ARG;
        }
    }
    m->embed = (const __nv_bfloat16*)embed_bf16;
    m->final_norm = final_norm;
    // one-time kernel configuration happens here so that nothing but launches runs inside a capture
    if ((rc = configure_gemv_kernels()) || (rc = configure_vec_stage()) || (rc = configure_lmhead()) ||
        (rc = configure_attention()) || (rc = configure_fused_gemv()) || (rc = init_ctx(m->c, nullptr)) ||
        (cudaDeviceSynchronize() != cudaSuccess ? (rc = ROTOR_B200_ERR_CUDA) : 0)) {
        free(m->layers);
        delete m;
        return rc;
    }
    *handle = m;
    return ROTOR_B200_OK;
}

void rotor_b200_model_destroy(void* handle) {
    Model* m = (Model*)handle;
    if (!m) return;
    if (m->graph) cudaGraphExecDestroy(m->graph);
    free(m->layers);
    delete m;
}

int rotor_b200_model_forward(void* handle, const int64_t* ids, int batch, int seq, int past_len, int logits_mode,
                             float* logits, int64_t* next_ids, void* stream) {
    Model* m = (Model*)handle;
    RB_REQUIRE(m && ids && batch > 0 && seq > 0 && past_len >= 0);
    RB_REQUIRE(batch <= m->cfg.max_batch && (long)batch * seq <= m->cfg.max_rows);
    RB_REQUIRE(past_len + seq <= m->cfg.max_seq);
    RB_REQUIRE(logits_mode >= ROTOR_B200_LOGITS_NONE && logits_mode <= ROTOR_B200_LOGITS_ALL);
    RB_REQUIRE(logits_mode == ROTOR_B200_LOGITS_NONE || logits);
    cudaStream_t st = as_stream(stream);
    set_pos_kernel<<<1, 256, 0, st>>>(m->c.d_pos, m->c.max_batch, past_len, nullptr);
    RB_TRY(run_layers(*m, (const long long*)ids, batch, seq, logits_mode, logits, (long long*)next_ids, st));
    m->pos = past_len + seq;
    return launch_status();
}

int rotor_b200_model_decode_begin(void* handle, const int64_t* first_ids, int batch, int past_len, void* stream) {
    Model* m = (Model*)handle;
    RB_REQUIRE(m && first_ids && batch > 0 && batch <= m->cfg.max_batch && batch <= 1024);
    RB_REQUIRE(past_len >= 0 && past_len < m->cfg.max_seq);
    begin_kernel<<<1, 1024, 0, as_stream(stream)>>>(m->cur_ids, (const long long*)first_ids, batch, m->c.d_pos,
                                                    past_len, nullptr, m->d_step);
    m->pos = past_len;
    m->step = 0;
    m->batch = batch;
    return launch_status();
}

/* Prefill of a ragged batch: `ids` holds `batch` prompts right-padded to `seq` tokens (any valid
 * id as padding), lens[b] (host) the true length of prompt b, 1 <= lens[b] <= seq.  Causal
 * models only: a row then never sees the padding behind it, so every position below lens[b]
 * is what a batch-of-one forward of prompt b alone gives.  Logits / picks are taken at each
 * prompt's own last token (logits_mode NONE or LAST).  Cache positions lens[b].. hold padding
 * products; rotor_b200_model_decode_begin_ragged makes the next steps overwrite them in order. */
int rotor_b200_model_forward_ragged(void* handle, const int64_t* ids, int batch, int seq, const int32_t* lens,
                                    int logits_mode, float* logits, int64_t* next_ids, void* stream) {
    Model* m = (Model*)handle;
    RB_REQUIRE(m && ids && lens && batch > 0 && seq > 0);
    RB_REQUIRE(m->cfg.causal && m->c.tp_size <= 1);
    RB_REQUIRE(batch <= m->cfg.max_batch && (long)batch * seq <= m->cfg.max_rows && seq <= m->cfg.max_seq);
    RB_REQUIRE(logits_mode == ROTOR_B200_LOGITS_NONE || (logits_mode == ROTOR_B200_LOGITS_LAST && logits));
    for (int b = 0; b < batch; ++b) RB_REQUIRE(lens[b] >= 1 && lens[b] <= seq);
    cudaStream_t st = as_stream(stream);
    set_pos_kernel<<<1, 256, 0, st>>>(m->c.d_pos, m->c.max_batch, 0, nullptr);
    m->last_of = lens;
    const int rc = run_layers(*m, (const long long*)ids, batch, seq, logits_mode, logits, (long long*)next_ids, st);
    m->last_of = nullptr;
    if (rc) return rc;
    m->pos = seq;
    return launch_status();
}

/* rotor_b200_model_decode_begin for sequences of different cached lengths (host lens[b], after
 * rotor_b200_model_forward_ragged): sequence b appends at position lens[b] + step and attends
 * to its own lens[b] + step + 1 keys. */
int rotor_b200_model_decode_begin_ragged(void* handle, const int64_t* first_ids, int batch, const int32_t* lens,
                                         void* stream) {
    Model* m = (Model*)handle;
    RB_REQUIRE(m && first_ids && lens && batch > 0 && batch <= m->cfg.max_batch && batch <= 1024);
    int longest = 0;
    for (int b = 0; b < batch; ++b) {
        RB_REQUIRE(lens[b] >= 0 && lens[b] < m->cfg.max_seq);
        longest = lens[b] > longest ? lens[b] : longest;
    }
    cudaStream_t st = as_stream(stream);
    RB_CUDA(cudaMemcpyAsync(m->d_lens, lens, (size_t)batch * sizeof(int), cudaMemcpyHostToDevice, st));
    begin_kernel<<<1, 1024, 0, st>>>(m->cur_ids, (const long long*)first_ids, batch, m->c.d_pos, 0, m->d_lens,
                                     m->d_step);
    RB_CUDA(cudaStreamSynchronize(st));  // `lens` may be pageable host memory the caller reuses
    m->pos = longest;  // capacity checks follow the longest sequence
    m->step = 0;
    m->batch = batch;
    return launch_status();
}

static int one_step(Model& m, cudaStream_t st) {
    if (m.c.tp_size > 1)
        return run_layers(m, m.cur_ids, m.batch, 1, ROTOR_B200_LOGITS_NONE, nullptr, m.cur_ids, st, true);
    if (m.batch <= 4)  // pick, token log and position advance ride in the LM head's last CTA
        return run_layers(m, m.cur_ids, m.batch, 1, ROTOR_B200_LOGITS_NONE, nullptr, m.cur_ids, st, true);
    RB_TRY(run_layers(m, m.cur_ids, m.batch, 1, ROTOR_B200_LOGITS_NONE, nullptr, m.cur_ids, st));
    advance_kernel<<<1, 1024, 0, st>>>(m.cur_ids, m.tok_log, m.batch, m.max_log, m.c.d_pos, m.d_step);
    return launch_status();
}

int rotor_b200_model_decode_steps(void* handle, int nsteps, int use_graph, void* stream) {
    Model* m = (Model*)handle;
    RB_REQUIRE(m && nsteps > 0 && m->batch > 0);
    RB_REQUIRE(m->pos + nsteps <= m->cfg.max_seq && m->step + nsteps <= m->max_log);
    cudaStream_t st = as_stream(stream);
    if (!use_graph) {
        for (int i = 0; i < nsteps; ++i) RB_TRY(one_step(*m, st));
    } else {
        if (m->graph && (m->graph_batch != m->batch)) {
            cudaGraphExecDestroy(m->graph);
            m->graph = nullptr;
        }
        if (!m->graph) {
            RB_REQUIRE(st != nullptr);  // the legacy default stream cannot be captured
            cudaGraph_t g = nullptr;
            RB_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
            const unsigned long long before = g_launch_count;
            int rc = one_step(*m, st);
            m->graph_launches = g_launch_count - before;
            g_launch_count = before;  // captured, not run
            cudaError_t e = cudaStreamEndCapture(st, &g);
            if (rc || e != cudaSuccess) {
                if (g) cudaGraphDestroy(g);
                return rc ? rc : ROTOR_B200_ERR_CUDA;
            }
            e = cudaGraphInstantiate(&m->graph, g, 0);
            cudaGraphDestroy(g);
            if (e != cudaSuccess) return ROTOR_B200_ERR_CUDA;
            m->graph_batch = m->batch;
        }
        for (int i = 0; i < nsteps; ++i) RB_CUDA(cudaGraphLaunch(m->graph, st));
        g_launch_count += m->graph_launches * (unsigned long long)nsteps;
    }
    m->pos += nsteps;
    m->step += nsteps;
    return ROTOR_B200_OK;
}

int rotor_b200_model_read_tokens(void* handle, int first_step, int count, int64_t* tokens_host, void* stream) {
    Model* m = (Model*)handle;
    RB_REQUIRE(m && tokens_host && first_step >= 0 && count > 0 && first_step + count <= m->step);
    cudaStream_t st = as_stream(stream);
    RB_CUDA(cudaMemcpyAsync(tokens_host, m->tok_log + (size_t)first_step * m->batch,
                            (size_t)count * m->batch * sizeof(int64_t), cudaMemcpyDeviceToHost, st));
    RB_CUDA(cudaStreamSynchronize(st));
    return ROTOR_B200_OK;
}

/* Attaches the tensor-parallel communicator (made by rotor_b200_tp_init) to a model created with
 * tp_size > 1.  The handle's rank must match the configuration's tp_rank. */
int rotor_b200_model_set_tp(void* handle, void* comm) {
    Model* m = (Model*)handle;
    RB_REQUIRE(m && comm && m->cfg.tp_size > 1);
    RB_REQUIRE(tp_size(comm) == m->cfg.tp_size && tp_rank(comm) == m->cfg.tp_rank);
    m->c.tp = comm;
    return ROTOR_B200_OK;
}

/* Programmatic dependent launch for the kernels of the decode chain: 1 lets each kernel start
 * (and prefetch its weight tiles) while its predecessor drains.  Applies to later launches and
 * to graphs captured afterwards.  Returns the previous setting. */
int rotor_b200_set_pdl(int enable) {
    const int old = g_use_pdl;
    g_use_pdl = enable ? 1 : 0;
    return old;
}

int rotor_b200_model_position(void* handle) {
    Model* m = (Model*)handle;
    return m ? m->pos : -1;
}

/* Runs blocks [layer_begin, layer_end) of the model on caller-provided hidden rows
 * (float32 [batch*seq][d_model], device).  With apply_final_norm the model's final norm is
 * applied to the result (BitNetModel.forward(return_logits=False), bitnet_model.py:231-243);
 * otherwise the raw residual stream is returned (TransformerBlock.forward, transformer.py:383-413). */
int rotor_b200_model_forward_hidden(void* handle, const float* hidden_in, int batch, int seq, int past_len,
                                    int layer_begin, int layer_end, int apply_final_norm, float* hidden_out,
                                    void* stream) {
    Model* m = (Model*)handle;
    RB_REQUIRE(m && hidden_in && hidden_out && batch > 0 && seq > 0 && past_len >= 0);
    RB_REQUIRE(batch <= m->cfg.max_batch && (long)batch * seq <= m->cfg.max_rows);
    RB_REQUIRE(past_len + seq <= m->cfg.max_seq);
    RB_REQUIRE(layer_begin >= 0 && layer_begin < layer_end && layer_end <= m->cfg.n_layers);
    cudaStream_t st = as_stream(stream);
    Ctx& c = m->c;
    const int rows = batch * seq;
    set_pos_kernel<<<1, 256, 0, st>>>(c.d_pos, c.max_batch, past_len, nullptr);
    RB_CUDA(cudaMemcpyAsync(c.h, hidden_in, (size_t)rows * c.d * sizeof(float), cudaMemcpyDeviceToDevice, st));
    VecStageParams e = {};
    e.mode = VS_PLAIN;
    e.n = c.d;
    e.src = c.h;
    e.norm1 = m->layers[layer_begin].input_norm;
    e.eps = c.eps;
    quant_sink(c, e, 0, c.d);
    RB_TRY(launch_vec_stage(e, rows, st));
    const float* next_norm = layer_end < m->cfg.n_layers ? m->layers[layer_end].input_norm : m->final_norm;
    if (c.tp_size > 1) {
        RB_REQUIRE(c.tp);
        RB_TRY(run_blocks_tp(*m, layer_begin, layer_end, next_norm, true, batch, seq, st));
    } else {
        RB_TRY(run_blocks(c, m->layers, layer_begin, layer_end, next_norm, true, batch, seq, st));
    }
    RB_CUDA(cudaMemcpyAsync(hidden_out, apply_final_norm ? c.hn : c.h, (size_t)rows * c.d * sizeof(float),
                            cudaMemcpyDeviceToDevice, st));
    m->pos = past_len + seq;
    return launch_status();
}

/* Workspace for the two stand-alone block halves below. */
static int block_derive(Ctx& c, const rotor_b200_model_config* cfg) {
    memset(&c, 0, sizeof(c));
    if (cfg->max_seq <= 0 || cfg->max_batch <= 0) return ROTOR_B200_ERR_ARG;
    int rc = derive_ctx(c, cfg->d_model, cfg->n_heads, cfg->n_kv_heads, cfg->d_ff, cfg->act_terms);
    if (rc) return rc;
    c.ffn_act = cfg->ffn_act;
    c.causal = cfg->causal;
    c.variant = cfg->gemv_variant;
    c.max_seq = cfg->max_seq;
    c.max_batch = cfg->max_batch;
    c.rope_theta = cfg->rope_theta;
    c.eps = cfg->eps;
    return ROTOR_B200_OK;
}

size_t rotor_b200_block_workspace_bytes(const rotor_b200_model_config* cfg, int rows) {
    Ctx c;
    if (!cfg || rows <= 0 || block_derive(c, cfg)) return 0;
    Carve cv{nullptr, 0};
    carve_ctx(c, cv, (size_t)rows);
    return cv.off;
}

static int block_ctx(Ctx& c, const rotor_b200_model_config* cfg, int rows, void* workspace, size_t workspace_bytes,
                     cudaStream_t st) {
    int rc = block_derive(c, cfg);
    if (rc) return rc;
    Carve cv{(unsigned char*)workspace, 0};
    carve_ctx(c, cv, (size_t)rows);
    if (cv.off > workspace_bytes) return ROTOR_B200_ERR_WORKSPACE;
    if ((rc = configure_gemv_kernels()) || (rc = configure_vec_stage()) || (rc = configure_attention())) return rc;
    return init_ctx(c, st);
}

/* GatedFFN.forward (src/rotor/transformer.py:320-341) on device rows x float32 [rows][d_model]
 * -> y float32 [rows][d_model]; with pre_norm != NULL an RMSNorm with that weight is applied
 * to x first (the block's post-attention norm).  Uses from `cfg`: d_model, n_heads,
 * n_kv_heads, d_ff, act_terms, ffn_act, eps, gemv_variant; from `layer`: gate_up_tiles,
 * down_tiles, their scales, ffn_sub_norm. */
int rotor_b200_ffn_forward(const rotor_b200_model_config* cfg, const rotor_b200_layer_weights* layer,
                           const float* pre_norm, const float* x, int rows, float* y, void* workspace,
                           size_t workspace_bytes, void* stream) {
    RB_REQUIRE(cfg && layer && x && y && workspace && rows > 0);
    RB_REQUIRE(layer->gate_up_tiles && layer->down_tiles && layer->ffn_sub_norm);
    RB_REQUIRE(((uintptr_t)workspace & 255) == 0);
    Ctx c;
    cudaStream_t st = as_stream(stream);
    {
        // a few token rows: two launches, the vector stages ride in the products' prologues
        RB_TRY(block_derive(c, cfg));
        static const bool off = getenv("ROTOR_B200_NO_FUSED_STEP") != nullptr;
        if (!off && rows <= FUSED_MAX_ROWS && c.terms <= 3 && rows * c.terms <= 8 && c.ff % 16 == 0 &&
            fused_gemv_supported(c.ff, c.d, rows, c.terms, 2, 0) && fused_gemv_supported(c.d, c.ff, rows, c.terms, 1, 0)) {
            Carve cv{(unsigned char*)workspace, 0};
            carve_ctx(c, cv, (size_t)rows);
            if (cv.off > workspace_bytes) return ROTOR_B200_ERR_WORKSPACE;
            static PerDevice<bool> once;
            bool& configured = once.here();
            if (!configured) {
                RB_TRY(configure_fused_gemv());
                configured = true;
            }
            LeanStage ls = {};
            ls.mode = LM_PLAIN;
            ls.n = c.d;
            ls.y = x;
            ls.norm1 = pre_norm;
            ls.eps = c.eps;
            ls.terms = c.terms;
            ls.kpad = (int)kpad_of(c.d);
            const float sgu[3] = {layer->gate_scale, layer->up_scale, 0.f};
            RB_TRY(launch_fused_gemv(layer->gate_up_tiles, c.ff, c.d, 2, rows, ls, c.fy[2], sgu, 0, 0, c.ffn_act, st));
            ls.n = c.ff;
            ls.y = c.fy[2];
            ls.norm1 = layer->ffn_sub_norm;
            ls.kpad = (int)kpad_of(c.ff);
            const float sd[3] = {layer->down_scale, layer->down_scale, layer->down_scale};
            return launch_fused_gemv(layer->down_tiles, c.d, c.ff, 1, rows, ls, y, sd, c.d, c.d, 0, st);
        }
    }
    RB_TRY(block_ctx(c, cfg, rows, workspace, workspace_bytes, st));
    VecStageParams e = {};
    e.mode = VS_PLAIN;
    e.n = c.d;
    e.src = x;
    e.norm1 = pre_norm;
    e.eps = c.eps;
    quant_sink(c, e, 0, c.d);
    RB_TRY(launch_vec_stage(e, rows, st));
    AccView vd;
    RB_TRY(ffn_part(c, *layer, rows, &vd, st));
    VecStageParams o = {};
    o.mode = VS_DEQ;
    o.n = c.d;
    o.acc = vd;
    o.sx_in = c.sx[1];
    o.terms = c.terms;
    o.wscale0 = layer->down_scale;
    o.eps = c.eps;
    o.y_out = y;
    return launch_vec_stage(o, rows, st);
}

/* MultiHeadAttention.forward (src/rotor/transformer.py:206-292) on device rows x float32
 * [batch*seq][d_model] -> y float32 [batch*seq][d_model], including the output projection and
 * the sub-norm that follows it.  The new K/V are written into layer->k_cache / v_cache at
 * positions past_len .. past_len+seq-1.  Uses from `cfg` additionally: causal, rope_theta,
 * max_seq; from `layer`: qkv_tiles, o_tiles, their scales, attn_sub_norm, the caches. */
int rotor_b200_attention_forward(const rotor_b200_model_config* cfg, const rotor_b200_layer_weights* layer,
                                 const float* x, int batch, int seq, int past_len, float* y, void* workspace,
                                 size_t workspace_bytes, void* stream) {
    RB_REQUIRE(cfg && layer && x && y && workspace && batch > 0 && seq > 0 && past_len >= 0);
    RB_REQUIRE(layer->qkv_tiles && layer->o_tiles && layer->attn_sub_norm && layer->k_cache && layer->v_cache);
    RB_REQUIRE(past_len + seq <= cfg->max_seq && batch <= cfg->max_batch);
    RB_REQUIRE(((uintptr_t)workspace & 255) == 0);
    const int rows = batch * seq;
    Ctx c;
    cudaStream_t st = as_stream(stream);
    RB_TRY(block_ctx(c, cfg, rows, workspace, workspace_bytes, st));
    set_pos_kernel<<<1, 256, 0, st>>>(c.d_pos, c.max_batch, past_len, nullptr);
    VecStageParams e = {};
    e.mode = VS_PLAIN;
    e.n = c.d;
    e.src = x;
    e.eps = c.eps;
    quant_sink(c, e, 0, c.d);
    RB_TRY(launch_vec_stage(e, rows, st));
    AccView vo;
    RB_TRY(attention_part(c, *layer, batch, seq, &vo, st));
    VecStageParams o = {};
    o.mode = VS_DEQ;
    o.n = c.d;
    o.acc = vo;
    o.sx_in = c.sx[1];
    o.terms = c.terms;
    o.wscale0 = layer->o_scale;
    o.norm1 = layer->attn_sub_norm;
    o.eps = c.eps;
    o.y_out = y;
    return launch_vec_stage(o, rows, st);
}

}  // extern "C"
