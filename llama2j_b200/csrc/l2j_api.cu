// Host side of libl2j_b200: the context (device memory, weights, per-token CUDA graph) and the
// C ABI declared in include/l2j_b200.h.  No Torch, no CPU compute path: everything a token needs
// runs in the kernels of l2j_kernels.cu.

#include "../../include/l2j_b200.h"
#include "l2j_internal.h"

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

using namespace l2j;

namespace {

thread_local std::string g_create_error;
std::mutex g_link_mu;   // guards the pipe_members lists of all contexts

constexpr int kCmdRing = 256;

struct LayerLaunch {
    MvParams qkv, wo, w13, w2;
    AttnParams attn;        // short contexts: the blocks of a head are a cluster (latency matters)
    AttnParams attn_long;   // long contexts: no cluster, two blocks per SM everywhere (bandwidth matters)
};

// From this position on a forward uses the long-context attention launch.
constexpr int kLongContextPos = 768;

}  // namespace

struct l2j_ctx {
    l2j_config cfg{};
    int device = 0;
    int first_layer = 0, last_layer = 0, nl = 0;
    uint32_t flags = 0;
    bool is_first = false, is_last = false;
    int dim = 0, kv_dim = 0, head = 0, hidden = 0, kv_mul = 1;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    std::mutex mu;
    std::string err;
    std::vector<void *> allocs;
    int64_t device_bytes = 0;

    QTensor qt[L2J_T_COUNT];
    int64_t per_layer[L2J_T_COUNT] = {0};
    bool needed[L2J_T_COUNT] = {false};
    float *rms_att = nullptr, *rms_ffn = nullptr, *rms_final = nullptr;   // dequantised
    float *emb = nullptr, *wcls = nullptr;
    int64_t emb_received = 0, wcls_received = 0;
    // which parts have arrived, as sorted disjoint intervals (groups for the quantised tensors, floats for the
    // FP32 ones): a part sent twice must not stand in for one that never came
    std::vector<std::pair<int64_t, int64_t>> got[L2J_T_COUNT];
    Prefill *prefill = nullptr;            // batched prompt path, built on first use where the shape allows it
    bool prefill_tried = false;
    SamplerState *samp_state = nullptr;   // device sampler (l2j_sampler_seed / l2j_sample), allocated on first use
    float *samp_prob[2] = {nullptr, nullptr};
    int *samp_index[2] = {nullptr, nullptr};
    SamplerState *samp_host = nullptr;     // pinned
    int async_in_flight = 0;       // forwards queued by l2j_forward_stage_async since the last synchronisation

    float *x = nullptr, *xb = nullptr, *q = nullptr, *hb = nullptr, *logits = nullptr;
    int reps = 1;                  // copies of x, xb, hb and the RMSNorm weights
    int dim_stride = 0, hid_stride = 0;   // distance of the copies in floats
    float *y0 = nullptr, *y1 = nullptr, *y2 = nullptr, *xn = nullptr;
    float *kc = nullptr, *vc = nullptr;
    float *rope_cos = nullptr, *rope_sin = nullptr;
    float *attn_part = nullptr;
    unsigned int *attn_counters = nullptr;
    int nsplit = 1;
    int nsplit_long = 1;           // splits per head of the long-context attention launch
    float *blk_val = nullptr;
    int *blk_idx = nullptr;
    int *prompt_dev = nullptr, *out_tokens_dev = nullptr;
    unsigned int *work = nullptr;   // two counters per ring-kernel launch of a forward
    unsigned int *chain = nullptr;  // hand-over counters, one per kernel of a forward, each on its own 128-byte line
    bool chain_on = true;
    bool kv_prefetch = true;
    bool attn_cluster = true;       // one thread-block cluster per head in the attention kernel
    unsigned long long *trace = nullptr;   // per-launch timelines, only when L2J_TRACE is set
    int wait_limit_us = 50000;      // bound of every device-side wait (copy barriers, hand-over counters, pair polls)
    int ring_grid = 0;              // blocks per ring kernel
    int early_fill = 1;             // ring stages a kernel may fetch before its predecessor has finished
    SeqState *state = nullptr;
    Cmd *cmd_dev = nullptr;
    Cmd *cmd_host = nullptr;       // pinned ring
    StageLink *link_dev = nullptr; // peer pointers of a linked layer split (zero until linked)
    std::vector<l2j_ctx *> pipe_members;   // the stages this context was linked with by l2j_pipeline_link, in order (empty: not linked)
    int tp_rank = 0, tp_size = 1;  // tensor parallel group this context belongs to
    TpTable *tp_dev = nullptr;     // the group's receive buffers (n = 0 until linked)
    float *x2 = nullptr;           // tensor parallel: second copy of the residual stream (the two alternate)
    float2 *ll_buf[TPV_COUNT] = {nullptr, nullptr, nullptr, nullptr};   // receive buffers: x increments, attention output, hidden vector
    bool tp_linked = false;
    bool cls_split = false;        // tensor parallel: the classifier's rows are split too (vocab divides by the ranks)
    cudaEvent_t ev_stage = nullptr;   // "this stage's step is done", waited for by the next stage's stream
    float *logits_host = nullptr;  // pinned
    float *x_host = nullptr;       // pinned
    SeqState *state_host = nullptr;

    MvPlan plan_qkv{}, plan_wo{}, plan_w13{}, plan_hidden{}, plan_cls{};
    bool use_ring = false;
    bool use_fused = false;        // all layers of a token in one persistent launch (l2j_fused.cu)
    MvPlan fplan[4]{};             // its stage geometry for QKV, Wo, W1/W3, W2
    FusedParams fused{};
    int fused_smem = 0, max_smem = 0;
    float *rms_wmax_dev = nullptr;
    float *fused_part = nullptr;
    unsigned long long *fused_trace = nullptr;
    std::vector<LayerLaunch> layers;
    MvParams cls{};
    bool finalized = false;
    bool pdl_on = false;
    cudaGraph_t graph = nullptr, graph_long = nullptr;
    cudaGraphExec_t exec = nullptr, exec_long = nullptr;   // one captured forward per attention regime
    int kernels_per_forward = 0;
    int64_t forwards = 0;
    int32_t status_accum = 0;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    double last_generate_us = 0.0;
};

namespace {

int fail(l2j_ctx *ctx, int code, const char *fmt, ...)
{
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    if (ctx)
        ctx->err = buf;
    else
        g_create_error = buf;
    return code;
}

#define CK(ctx, call)                                                                                       \
    do {                                                                                                    \
        cudaError_t e__ = (call);                                                                           \
        if (e__ != cudaSuccess)                                                                             \
            return fail(ctx, L2J_E_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__), __FILE__, \
                        __LINE__);                                                                          \
    } while (0)

template <typename T>
int dev_alloc(l2j_ctx *ctx, T **out, int64_t count, bool zero)
{
    void *p = nullptr;
    const size_t bytes = (size_t)(count > 0 ? count : 1) * sizeof(T);
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess)
        return fail(ctx, L2J_E_NOMEM, "cudaMalloc of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    if (zero) {
        e = cudaMemset(p, 0, bytes);
        if (e != cudaSuccess) {
            cudaFree(p);
            return fail(ctx, L2J_E_CUDA, "cudaMemset failed: %s", cudaGetErrorString(e));
        }
    }
    ctx->allocs.push_back(p);
    ctx->device_bytes += (int64_t)bytes;
    *out = static_cast<T *>(p);
    return L2J_OK;
}

// Adds [a, b) to the sorted disjoint intervals; false (and nothing added) if it overlaps one of them.
bool add_interval(std::vector<std::pair<int64_t, int64_t>> &iv, int64_t a, int64_t b)
{
    size_t i = 0;
    while (i < iv.size() && iv[i].second <= a)
        ++i;
    if (i < iv.size() && iv[i].first < b)
        return false;
    iv.insert(iv.begin() + (long)i, std::make_pair(a, b));
    for (size_t j = 0; j + 1 < iv.size();) {   // join neighbours that touch
        if (iv[j].second == iv[j + 1].first) {
            iv[j].second = iv[j + 1].second;
            iv.erase(iv.begin() + (long)j + 1);
        } else {
            ++j;
        }
    }
    return true;
}

int64_t covered(const std::vector<std::pair<int64_t, int64_t>> &iv)
{
    int64_t n = 0;
    for (const auto &p : iv)
        n += p.second - p.first;
    return n;
}

bool is_quant_tensor(int t)
{
    return t == L2J_T_RMS_ATT || t == L2J_T_WQ || t == L2J_T_WK || t == L2J_T_WV || t == L2J_T_WO || t == L2J_T_RMS_FFN ||
           t == L2J_T_W1 || t == L2J_T_W2 || t == L2J_T_W3 || t == L2J_T_RMS_FINAL;
}

bool is_rms_tensor(int t)
{
    return t == L2J_T_RMS_ATT || t == L2J_T_RMS_FFN || t == L2J_T_RMS_FINAL;
}

// The reference's RoPE table (ApplyRope.init, kernel/ApplyRope.java:34-59), one row per position
// and one entry per rotated pair of a head.
void build_rope_tables(int seq_len, int head, std::vector<float> &cs, std::vector<float> &sn)
{
    const int half = head / 2;
    cs.resize((size_t)seq_len * half);
    sn.resize((size_t)seq_len * half);
    for (int j = 0; j < half; ++j) {
        const float e = (float)(2 * j) / (float)head;
        const float freq = (float)(1.0 / std::pow((double)10000.0f, (double)e));
        for (int pos = 0; pos < seq_len; ++pos) {
            const float val = (float)pos * freq;
            cs[(size_t)pos * half + j] = (float)std::cos((double)val);
            sn[(size_t)pos * half + j] = (float)std::sin((double)val);
        }
    }
}

// Rows [rank * rows / parts, (rank + 1) * rows / parts) of a matrix of `rows` rows of n elements that starts
// at element weight_index of tensor t: the block of rows a tensor-parallel rank works on (all rows for
// parts == 1).
MvSeg make_seg(const QTensor &t, int64_t weight_index, int rows, int n = 0, int rank = 0, int parts = 1)
{
    MvSeg s;
    const int per = rows / parts;
    s.payload = t.payload;
    s.hdr = t.hdr;
    s.flat0 = weight_index - t.base_float + (int64_t)rank * per * n;
    s.rows = per;
    s.out0 = rank * per;
    return s;
}

void fill_plan(MvParams &p, const MvPlan &pl)
{
    p.rpp = pl.rpp;
    p.wpr = pl.wpr;
    p.nstage = pl.nstage;
    p.slot_bytes = pl.slot_bytes;
    p.hdr_off = pl.hdr_off;
    p.half_hdr = pl.half_hdr;
    p.xshare_bytes = pl.xshare_bytes;
    {   // stage bookkeeping: a stage advances rt*rpp rows (half of that per matrix in paired mode)
        const int rs = p.paired ? (pl.rt * pl.rpp) / 2 : pl.rt * pl.rpp;
        p.rs = rs;
        p.rt = pl.rt;
        p.rowbytes = p.f32 ? p.n * 4 : p.n;
        {
            const char *e = getenv("L2J_TAIL_PREFETCH");   // diagnostic: stages of the next launch asked into L2 by a block that ran out of work
            p.tail_prefetch = e ? atoi(e) : 3;
        }
        p.total_stages = 0;
        const int nseg = p.paired ? 1 : p.nseg;
        for (int i = 0; i < 3; ++i) {
            p.seg_stages[i] = i < nseg ? (p.seg[i].rows + rs - 1) / rs : 0;
            p.total_stages += p.seg_stages[i];
        }
    }
}

constexpr int kChainStride = 32;   // unsigned ints between two hand-over counters (128 bytes)

// Links the kernels of a forward through hand-over counters: kernel i waits on the counter of kernel
// i - 1.  The first ring kernel follows the begin kernel with a full dependency and needs none.
void link_chain(l2j_ctx *c)
{
    if (!c->use_ring || !c->chain_on)
        return;
    const unsigned int ring_blocks = (unsigned int)c->ring_grid;
    const unsigned int attn_blocks = (unsigned int)(c->cfg.n_heads * c->nsplit);
    const unsigned int *prev = nullptr;
    unsigned int prev_blocks = 0;
    int idx = 0;
    auto link = [&](ChainLink &ch, unsigned int blocks) {
        ch.wait_counter = prev;
        ch.wait_blocks = prev_blocks;
        ch.done_counter = c->chain + (int64_t)kChainStride * idx++;
        ch.epoch = c->chain + (int64_t)kChainStride * (5 * c->nl + 1);
        prev = ch.done_counter;
        prev_blocks = blocks;
    };
    for (int li = 0; li < c->nl; ++li) {
        LayerLaunch &L = c->layers[(size_t)li];
        if (c->tp_size > 1) {
            // Across the ranks data travels with sequence numbers (link_ranks); the only hand-over inside a
            // rank is QKV -> attention.
            prev = nullptr;
            link(L.qkv.chain, ring_blocks);
            link(L.attn.chain, attn_blocks);
            L.attn.chain.done_counter = nullptr;
            continue;
        }
        link(L.qkv.chain, ring_blocks);
        link(L.attn.chain, attn_blocks);
        link(L.wo.chain, ring_blocks);
        link(L.w13.chain, ring_blocks);
        link(L.w2.chain, ring_blocks);
    }
    if (c->is_last && c->tp_size == 1)
        link(c->cls.chain, ring_blocks);
}

// Tensor parallel: which receive buffer every kernel reads and writes, and under which sequence numbers.
// Kernel indices within a forward: layer li -> 5 li + {0 QKV, 1 attention, 2 Wo, 3 W1/W3, 4 W2}; classifier 5 L.
// The residual stream alternates between two buffers: QKV (and the classifier) read x2 + the increments
// of W2 and leave the sum in x; W1/W3 read x + the increments of Wo and leave the sum in x2.
void link_ranks(l2j_ctx *c)
{
    if (c->tp_size <= 1)
        return;
    LlLink base{};
    base.tp = c->tp_dev;
    base.epoch = c->chain + (int64_t)kChainStride * (5 * c->nl + 1);
    base.kernels = 5 * c->nl + 1;
    base.in_vec = base.out_vec = -1;
    for (int li = 0; li < c->nl; ++li) {
        LayerLaunch &L = c->layers[(size_t)li];
        const int k0 = 5 * li;
        L.qkv.ll = base;
        if (li > 0) {
            L.qkv.ll.in_vec = TPV_X;
            L.qkv.ll.in_idx = k0 - 1;
            L.qkv.ll.base = c->x2;
            L.qkv.ll.write_back = c->x;
        }
        L.attn.ll = base;
        L.attn.ll.out_vec = TPV_XB;
        L.attn.ll.out_idx = k0 + 1;
        L.wo.ll = base;
        L.wo.ll.in_vec = TPV_XB;
        L.wo.ll.in_idx = k0 + 1;
        L.wo.ll.out_vec = TPV_X;
        L.wo.ll.out_idx = k0 + 2;
        L.w13.ll = base;
        L.w13.ll.in_vec = TPV_X;
        L.w13.ll.in_idx = k0 + 2;
        L.w13.ll.base = c->x;
        L.w13.ll.write_back = c->x2;
        L.w13.ll.out_vec = TPV_HB;
        L.w13.ll.out_idx = k0 + 3;
        L.w2.ll = base;
        L.w2.ll.in_vec = TPV_HB;
        L.w2.ll.in_idx = k0 + 3;
        L.w2.ll.out_vec = TPV_X;
        L.w2.ll.out_idx = k0 + 4;
    }
    c->cls.ll = base;
    c->cls.ll.in_vec = TPV_X;
    c->cls.ll.in_idx = 5 * c->nl - 1;
    c->cls.ll.base = c->x2;
    c->cls.ll.write_back = c->x;   // the final residual stream stays readable (l2j_read_buffer)
    if (c->cls_split) {
        c->cls.ll.out_vec = TPV_CAND;
        c->cls.ll.out_idx = 5 * c->nl;
    }
}

// Stage geometry of a phase of the persistent kernel: the lane mapping of plan_matvec (so that every
// output element is computed exactly as by the per-step kernels), but stages of rpp rows (32 KB at the 7B
// shape): the phases share one byte ring, and small stages keep more of it in flight and waste less where
// it wraps.
MvPlan plan_fused_phase(int n, bool paired, int row_align)
{
    MvPlan pl = plan_matvec(n, false, paired, 0, 0, row_align);
    if (!pl.ok || !pl.grouped)
        return MvPlan{};
    const int rt = 1;   // one row per group of wpr warps and stage (the persistent kernel's consumers are built for that)
    int rpp = pl.rpp;
    const int align = paired ? (row_align > 2 ? row_align : 2) : row_align;
    while (rpp > 1 && (rt * rpp) % align != 0)
        --rpp;
    if ((rt * rpp) % align != 0)
        return MvPlan{};
    pl.rt = rt;
    pl.rpp = rpp;
    pl.half_hdr = ((((rt * rpp * n / 2 + 255) / 256) + 4) * 8 + 15) & ~15;
    const int payload = rt * rpp * n;
    pl.hdr_off = payload;
    pl.slot_bytes = (payload + 2 * pl.half_hdr + 127) & ~127;
    pl.threads = kFusedThreads;
    return pl;
}

// Parameters of the persistent kernel: the four matrix-vector phases of the first layer (the kernel adds
// the per-layer steps) and the attention step's shape.
void build_fused_params(l2j_ctx *c)
{
    FusedParams &F = c->fused;
    F = FusedParams{};
    const LayerLaunch &L = c->layers[0];
    const MvParams *src[4] = {&L.qkv, &L.wo, &L.w13, &L.w2};
    const int tensors[4][3] = {{L2J_T_WQ, L2J_T_WK, L2J_T_WV}, {L2J_T_WO, -1, -1}, {L2J_T_W1, L2J_T_W3, -1}, {L2J_T_W2, -1, -1}};
    for (int k = 0; k < 4; ++k) {
        MvParams &p = F.mv[k];
        p = *src[k];
        fill_plan(p, c->fplan[k]);
        p.chain = ChainLink{};
        p.next = nullptr;
        p.trace = nullptr;
        for (int s = 0; s < 3; ++s)
            F.seg_step[k][s] = tensors[k][s] >= 0 ? c->per_layer[tensors[k][s]] : 0;
    }
    F.kv_step = (long long)c->cfg.n_kv_heads * c->cfg.seq_len * c->head;
    F.rms_step = c->reps * c->dim_stride;
    F.n_layers = c->nl;
    F.rms_wmax = c->rms_wmax_dev;
    F.q = c->q;
    F.att_part = c->fused_part;
    F.n_heads = c->cfg.n_heads;
    F.kv_mul = c->kv_mul;
    F.head = c->head;
    F.seq_len = c->cfg.seq_len;
    int gw = 1;
    while (gw < c->head / 4)
        gw <<= 1;
    const int merge_bytes = kFusedConsWarps * (32 / gw) * (c->head + 4) * 4;
    const int limb_bytes = 3 * (c->dim > c->hidden ? c->dim : c->hidden);
    F.xarea_bytes = ((merge_bytes > limb_bytes ? merge_bytes : limb_bytes) + 127) & ~127;
    F.ring_bytes = (c->fused_smem - kFusedHeaderBytes - F.xarea_bytes) & ~127;
    F.sync = c->chain;
    F.epoch = c->chain + (int64_t)kChainStride * (5 * c->nl + 1);
    F.state = c->state;
    F.timeout_us = c->wait_limit_us;
    F.trace = c->fused_trace;
    if (const char *e = getenv("L2J_FUSED_NO_COPY"))   // measurement aid: consumers run on whatever the ring holds
        F.debug_no_copy = atoi(e);
}

// Builds the static kernel parameter blocks of every layer this context owns.
void build_launch_params(l2j_ctx *c)
{
    const int dim = c->dim, kv_dim = c->kv_dim, hidden = c->hidden;
    c->layers.assign((size_t)c->nl, LayerLaunch{});
    for (int li = 0; li < c->nl; ++li) {
        const int64_t l = c->first_layer + li;
        LayerLaunch &L = c->layers[(size_t)li];
        float *kc = c->kc + (int64_t)li * c->cfg.n_kv_heads * c->cfg.seq_len * c->head;
        float *vc = c->vc + (int64_t)li * c->cfg.n_kv_heads * c->cfg.seq_len * c->head;

        MvParams base{};
        base.dim = dim;
        base.kv_dim = kv_dim;
        base.head = c->head;
        base.seq_len = c->cfg.seq_len;
        base.state = c->state;
        base.timeout_us = c->wait_limit_us;
        base.rope_cos = c->rope_cos;
        base.rope_sin = c->rope_sin;

        // q, k, v = W(rmsnorm(x)); RoPE; KV append            (Run.java:418-446)
        MvParams &a = L.qkv;
        a = base;
        a.seg[0] = make_seg(c->qt[L2J_T_WQ], l * dim * dim, dim, dim, c->tp_rank, c->tp_size);
        a.seg[1] = make_seg(c->qt[L2J_T_WK], l * (int64_t)kv_dim * dim, kv_dim, dim, c->tp_rank, c->tp_size);
        a.seg[2] = make_seg(c->qt[L2J_T_WV], l * (int64_t)kv_dim * dim, kv_dim, dim, c->tp_rank, c->tp_size);
        a.nseg = 3;
        a.paired = 0;
        a.n = dim;
        fill_plan(a, c->plan_qkv);
        a.early_fill = c->early_fill;
        a.x_in = c->x;
        a.x_reps = c->reps;
        a.x_stride = c->dim_stride;
        a.rms_w = c->rms_att + (int64_t)li * c->reps * c->dim_stride;
        a.epilogue = EPI_QKV_ROPE;
        a.kv_prefetch_below = c->kv_prefetch ? kLongContextPos : 0;   // beyond it the rows of a layer outgrow what L2 should hold
        a.q_out = c->q;
        a.k_cache = kc;
        a.v_cache = vc;
        a.work = c->work + 2 * (4 * li + 0);
        a.trace = c->trace ? c->trace + (int64_t)(4 * li + 0) * c->ring_grid * 16 : nullptr;

        // attention over positions 0..pos                      (Run.java:450-478)
        AttnParams &t = L.attn;
        t.q = c->q;
        t.k_cache = kc;
        t.v_cache = vc;
        t.out = c->xb;
        t.out_reps = c->reps;
        t.out_stride = c->dim_stride;
        t.part = c->attn_part;
        t.counters = c->attn_counters;
        t.state = c->state;
        t.n_heads = c->cfg.n_heads;
        t.kv_mul = c->kv_mul;
        t.head = c->head;
        t.seq_len = c->cfg.seq_len;
        t.nsplit = c->nsplit;
        t.pos_override = -1;
        t.cluster = c->attn_cluster ? 1 : 0;
        t.timeout_us = c->wait_limit_us;
        t.trace = c->trace ? c->trace + (int64_t)(4 * c->nl + 1 + li) * c->ring_grid * 16 : nullptr;
        t.trace_blocks = c->ring_grid;
        t.smem_pad = 0;
        t.n_heads = c->cfg.n_heads / c->tp_size;   // the heads whose q rows this rank computed
        t.h0 = c->tp_rank * t.n_heads;

        // x += Wo att                                          (Run.java:483-485)
        MvParams &o = L.wo;
        o = base;
        o.seg[0] = make_seg(c->qt[L2J_T_WO], l * dim * dim, dim, dim, c->tp_rank, c->tp_size);
        o.nseg = 1;
        o.n = dim;
        fill_plan(o, c->plan_wo);
        o.x_in = c->xb;
        o.x_reps = c->reps;
        o.x_stride = c->dim_stride;
        o.rms_w = nullptr;
        o.epilogue = EPI_RESIDUAL;
        o.y = c->x;
        o.y_reps = c->reps;
        o.y_stride = c->dim_stride;
        o.work = c->work + 2 * (4 * li + 1);
        o.trace = c->trace ? c->trace + (int64_t)(4 * li + 1) * c->ring_grid * 16 : nullptr;

        // hb = silu(W1 rmsnorm(x)) * W3 rmsnorm(x)              (Run.java:490-502)
        MvParams &f = L.w13;
        f = base;
        f.seg[0] = make_seg(c->qt[L2J_T_W1], l * (int64_t)hidden * dim, hidden, dim, c->tp_rank, c->tp_size);
        f.seg[1] = make_seg(c->qt[L2J_T_W3], l * (int64_t)hidden * dim, hidden, dim, c->tp_rank, c->tp_size);
        f.nseg = 1;
        f.paired = 1;
        f.n = dim;
        fill_plan(f, c->plan_w13);
        f.early_fill = c->early_fill;
        f.x_in = c->x;
        f.x_reps = c->reps;
        f.x_stride = c->dim_stride;
        f.rms_w = c->rms_ffn + (int64_t)li * c->reps * c->dim_stride;
        f.epilogue = EPI_SWIGLU;
        f.y = c->hb;
        f.y_reps = c->reps;
        f.y_stride = c->hid_stride;
        f.work = c->work + 2 * (4 * li + 2);
        f.trace = c->trace ? c->trace + (int64_t)(4 * li + 2) * c->ring_grid * 16 : nullptr;

        // x += W2 hb                                           (Run.java:505-508)
        MvParams &w = L.w2;
        w = base;
        w.seg[0] = make_seg(c->qt[L2J_T_W2], l * (int64_t)hidden * dim, dim, hidden, c->tp_rank, c->tp_size);
        w.nseg = 1;
        w.n = hidden;
        fill_plan(w, c->plan_hidden);
        w.early_fill = c->early_fill;
        w.x_in = c->hb;
        w.x_reps = c->reps;
        w.x_stride = c->hid_stride;
        w.rms_w = nullptr;
        w.epilogue = EPI_RESIDUAL;
        w.y = c->x;
        w.y_reps = c->reps;
        w.y_stride = c->dim_stride;
        w.work = c->work + 2 * (4 * li + 3);
        w.trace = c->trace ? c->trace + (int64_t)(4 * li + 3) * c->ring_grid * 16 : nullptr;
    }
    if (c->is_last) {
        // logits = Wcls rmsnorm(x); arg-max                    (Run.java:514-518, Sampler.java:46-57)
        MvParams &k = c->cls;
        k = MvParams{};
        k.dim = c->dim;
        k.kv_dim = c->kv_dim;
        k.head = c->head;
        k.seq_len = c->cfg.seq_len;
        k.state = c->state;
        k.timeout_us = c->wait_limit_us;
        k.seg[0].payload = reinterpret_cast<const uint8_t *>(c->wcls);
        k.seg[0].hdr = nullptr;
        k.seg[0].flat0 = 0;
        k.seg[0].rows = c->cfg.vocab_size;
        if (c->cls_split) {   // a block of the vocabulary per rank
            const int per = c->cfg.vocab_size / c->tp_size;
            k.seg[0].flat0 = (int64_t)c->tp_rank * per * c->dim;
            k.seg[0].rows = per;
            k.seg[0].out0 = c->tp_rank * per;
        }
        k.nseg = 1;
        k.n = c->dim;
        k.f32 = 1;
        fill_plan(k, c->plan_cls);
        k.early_fill = c->early_fill;
        k.x_in = c->x;
        k.x_reps = c->reps;
        k.x_stride = c->dim_stride;
        k.y_reps = 1;
        k.rms_w = c->rms_final;
        k.epilogue = EPI_LOGITS;
        k.y = c->logits;
        k.blk_val = c->blk_val;
        k.blk_idx = c->blk_idx;
        k.prompt = c->prompt_dev;
        k.out_tokens = c->out_tokens_dev;
        k.work = c->work + 2 * (4 * c->nl);
        k.trace = c->trace ? c->trace + (int64_t)(4 * c->nl) * c->ring_grid * 16 : nullptr;
    }
    link_chain(c);
    link_ranks(c);
    if (c->use_fused)
        build_fused_params(c);
    for (int li = 0; li < c->nl; ++li) {
        LayerLaunch &L = c->layers[(size_t)li];
        L.attn_long = L.attn;          // same grid and hand-over counters
        L.attn_long.cluster = 0;
        L.attn_long.smem_pad = 1;
        L.attn_long.nsplit = c->nsplit_long;
    }
}

// A kernel launched on its own (timing, tracing) must neither wait on nor bump the hand-over counters.
template <typename P>
P unchained(P p)
{
    p.chain = ChainLink{};
    p.ll = LlLink{};
    p.ll.in_vec = p.ll.out_vec = -1;
    return p;
}

// Enqueues the kernels of one forward of this context's layer range on its stream.
cudaError_t enqueue_forward(l2j_ctx *c, bool pdl, int *n_kernels, bool long_ctx)
{
    cudaError_t e;
    int nk = 0;
    LaunchCfg lc{c->stream, false, c->ring_grid};
    // The first kernel of a forward follows a memcpy (or the previous graph launch): plain edge.
    e = launch_begin(lc, c->state, c->cmd_dev, c->emb, c->x, c->dim, c->cfg.vocab_size, c->cfg.seq_len, c->is_first ? 1 : 0, c->reps, c->dim_stride,
                     c->use_ring && c->chain_on ? c->chain + (int64_t)kChainStride * (5 * c->nl + 1) : nullptr, c->link_dev);
    if (e != cudaSuccess)
        return e;
    ++nk;
    lc.pdl = pdl;
    const int dim = c->dim, hidden = c->hidden;
    if (c->use_fused) {
        // every layer of the range in one persistent launch; it waits for the begin kernel itself (the position
        // and x are read behind a dependency wait, the weight stream starts before it)
        if ((e = launch_fused(c->stream, pdl, c->ring_grid, c->fused_smem, c->fused)) != cudaSuccess) return e;
        ++nk;
    }
    for (int li = 0; li < c->nl && !c->use_fused; ++li) {
        LayerLaunch &L = c->layers[(size_t)li];
        if (c->use_ring) {
            // The first ring kernel of a forward takes a full dependency on the begin kernel: the attention
            // kernel behind it reads the position before its own dependency wait.
            LaunchCfg first = lc;
            first.pdl = lc.pdl && li > 0;
            if ((e = launch_matvec_ring(first, c->plan_qkv, false, L.qkv)) != cudaSuccess) return e;
            if ((e = launch_attention(lc, long_ctx ? L.attn_long : L.attn)) != cudaSuccess) return e;
            if ((e = launch_matvec_ring(lc, c->plan_wo, false, L.wo)) != cudaSuccess) return e;
            if ((e = launch_matvec_ring(lc, c->plan_w13, false, L.w13)) != cudaSuccess) return e;
            if ((e = launch_matvec_ring(lc, c->plan_hidden, false, L.w2)) != cudaSuccess) return e;
            nk += 5;
        } else {
            LaunchCfg plain{c->stream, false, c->ring_grid};
            if ((e = launch_rmsnorm_plain(c->stream, c->x, L.qkv.rms_w, c->xn, dim)) != cudaSuccess) return e;
            if ((e = launch_matvec_plain_u8(c->stream, L.qkv.seg[0], dim, c->xn, c->y0)) != cudaSuccess) return e;
            if ((e = launch_matvec_plain_u8(c->stream, L.qkv.seg[1], dim, c->xn, c->y1)) != cudaSuccess) return e;
            if ((e = launch_matvec_plain_u8(c->stream, L.qkv.seg[2], dim, c->xn, c->y2)) != cudaSuccess) return e;
            if ((e = launch_epilogue_plain(c->stream, L.qkv, c->y0, c->y1, c->y2)) != cudaSuccess) return e;
            if ((e = launch_attention(plain, L.attn)) != cudaSuccess) return e;
            if ((e = launch_matvec_plain_u8(c->stream, L.wo.seg[0], dim, c->xb, c->y0)) != cudaSuccess) return e;
            if ((e = launch_epilogue_plain(c->stream, L.wo, c->y0, nullptr, nullptr)) != cudaSuccess) return e;
            if ((e = launch_rmsnorm_plain(c->stream, c->x, L.w13.rms_w, c->xn, dim)) != cudaSuccess) return e;
            if ((e = launch_matvec_plain_u8(c->stream, L.w13.seg[0], dim, c->xn, c->y0)) != cudaSuccess) return e;
            if ((e = launch_matvec_plain_u8(c->stream, L.w13.seg[1], dim, c->xn, c->y1)) != cudaSuccess) return e;
            if ((e = launch_epilogue_plain(c->stream, L.w13, c->y0, c->y1, nullptr)) != cudaSuccess) return e;
            if ((e = launch_matvec_plain_u8(c->stream, L.w2.seg[0], hidden, c->hb, c->y0)) != cudaSuccess) return e;
            if ((e = launch_epilogue_plain(c->stream, L.w2, c->y0, nullptr, nullptr)) != cudaSuccess) return e;
            nk += 14;
        }
    }
    if (c->is_last) {
        if (c->use_ring) {
            if ((e = launch_matvec_ring(lc, c->plan_cls, true, c->cls)) != cudaSuccess) return e;
            nk += 1;
        } else {
            if ((e = launch_rmsnorm_plain(c->stream, c->x, c->rms_final, c->xn, dim)) != cudaSuccess) return e;
            if ((e = launch_matvec_plain_f32(c->stream, c->wcls, dim, c->cfg.vocab_size, c->xn, c->y0)) != cudaSuccess) return e;
            if ((e = launch_epilogue_plain(c->stream, c->cls, c->y0, nullptr, nullptr)) != cudaSuccess) return e;
            nk += 3;
        }
    }
    if (n_kernels)
        *n_kernels = nk;
    return cudaSuccess;
}

bool try_capture(l2j_ctx *c, bool pdl, bool long_ctx)
{
    cudaGraph_t g = nullptr;
    if (cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    int nk = 0;
    cudaError_t e = enqueue_forward(c, pdl, &nk, long_ctx);
    cudaError_t e2 = cudaStreamEndCapture(c->stream, &g);
    if (e != cudaSuccess || e2 != cudaSuccess || !g) {
        if (g)
            cudaGraphDestroy(g);
        cudaGetLastError();
        return false;
    }
    cudaGraphExec_t ex = nullptr;
    if (cudaGraphInstantiate(&ex, g, 0) != cudaSuccess || !ex) {
        cudaGraphDestroy(g);
        cudaGetLastError();
        return false;
    }
    (long_ctx ? c->graph_long : c->graph) = g;
    (long_ctx ? c->exec_long : c->exec) = ex;
    c->kernels_per_forward = nk;
    return true;
}

// `pos` is the position of the forward being launched (the host always knows it: it is an argument, or the
// step number of a greedy loop); it selects the attention regime.
int launch_forward(l2j_ctx *c, int pos)
{
    const bool long_ctx = c->use_ring && !c->use_fused && pos >= kLongContextPos;
    cudaGraphExec_t ex = long_ctx ? c->exec_long : c->exec;
    if (ex) {
        CK(c, cudaGraphLaunch(ex, c->stream));
    } else {
        int nk = 0;
        CK(c, enqueue_forward(c, c->pdl_on, &nk, long_ctx));
        c->kernels_per_forward = nk;
    }
    c->forwards++;
    return L2J_OK;
}

int check_range(l2j_ctx *c, int token, int pos, bool need_token)
{
    if (pos < 0 || pos >= c->cfg.seq_len)
        return fail(c, L2J_E_INVALID, "pos %d outside [0, %d)", pos, c->cfg.seq_len);
    if (need_token && (token < 0 || token >= c->cfg.vocab_size))
        return fail(c, L2J_E_INVALID, "token %d outside [0, %d)", token, c->cfg.vocab_size);
    return L2J_OK;
}

int post_cmd(l2j_ctx *c, int mode, int token, int pos, int flags = 0)
{
    Cmd *slot = c->cmd_host + (c->forwards % kCmdRing);
    slot->mode = mode;
    slot->token = token;
    slot->pos = pos;
    slot->flags = flags;
    CK(c, cudaMemcpyAsync(c->cmd_dev, slot, sizeof(Cmd), cudaMemcpyHostToDevice, c->stream));
    return L2J_OK;
}

// Waits for the stream by polling an event: the host thread notices the end of a token a few tens of
// microseconds earlier than when it sleeps in cudaStreamSynchronize, which counts at 2 ms per token.
cudaError_t spin_sync(l2j_ctx *c)
{
    cudaError_t e = cudaEventRecord(c->ev_stage, c->stream);
    if (e != cudaSuccess)
        return e;
    for (;;) {
        e = cudaEventQuery(c->ev_stage);
        if (e != cudaErrorNotReady)
            return e;
    }
}

int finish_status(l2j_ctx *c)
{
    const int st = c->state_host->status;
    c->status_accum |= st;
    if (st != 0)
        return fail(c, L2J_E_DEVICE, "device status 0x%x (1: copy wait timed out, 2: bad pos, 4: bad token)", st);
    return L2J_OK;
}

}  // namespace

// ===============================================================================================
// context
// ===============================================================================================

static int create_impl(const l2j_config *cfg, int device, int first_layer, int last_layer, uint32_t flags, int tp_rank,
                       int tp_size, l2j_ctx **out)
{
    if (!cfg || !out)
        return fail(nullptr, L2J_E_INVALID, "null argument");
    *out = nullptr;
    if (tp_size < 1 || tp_size > kMaxTp || tp_rank < 0 || tp_rank >= tp_size)
        return fail(nullptr, L2J_E_INVALID, "tensor-parallel rank %d of %d (at most %d ranks)", tp_rank, tp_size, kMaxTp);
    if (tp_size > 1 && (flags & L2J_F_SIMPLE))
        return fail(nullptr, L2J_E_INVALID, "the plain kernels have no tensor-parallel mode");
    if (cfg->dim <= 0 || cfg->hidden_dim <= 0 || cfg->n_layers <= 0 || cfg->n_heads <= 0 || cfg->n_kv_heads <= 0 ||
        cfg->vocab_size <= 0 || cfg->seq_len <= 0)
        return fail(nullptr, L2J_E_INVALID, "config fields must be positive");
    if (cfg->dim % cfg->n_heads != 0 || cfg->n_heads % cfg->n_kv_heads != 0)
        return fail(nullptr, L2J_E_INVALID, "dim must divide by n_heads and n_heads by n_kv_heads");
    const int head = cfg->dim / cfg->n_heads;
    if (head % 4 != 0 || head > 128)
        return fail(nullptr, L2J_E_INVALID, "head size %d unsupported (needs a multiple of 4, at most 128)", head);
    if (cfg->dim % 4 != 0)
        return fail(nullptr, L2J_E_INVALID, "dim must be a multiple of 4");
    if (first_layer < 0 || last_layer >= cfg->n_layers || first_layer > last_layer)
        return fail(nullptr, L2J_E_INVALID, "layer range [%d, %d] outside the model", first_layer, last_layer);
    if (tp_size > 1 && (cfg->n_heads % tp_size != 0 || cfg->n_kv_heads % tp_size != 0 || cfg->hidden_dim % tp_size != 0 ||
                        (cfg->dim / tp_size) % 2 != 0))
        return fail(nullptr, L2J_E_INVALID, "heads, kv heads and hidden_dim must divide by the %d tensor-parallel ranks", tp_size);
    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess || ndev <= 0)
        return fail(nullptr, L2J_E_CUDA, "no CUDA device: %s (this library has no CPU path)", cudaGetErrorString(e));
    if (device < 0 || device >= ndev)
        return fail(nullptr, L2J_E_INVALID, "device %d not present (%d devices)", device, ndev);
    e = cudaSetDevice(device);
    if (e != cudaSuccess)
        return fail(nullptr, L2J_E_CUDA, "cudaSetDevice failed: %s", cudaGetErrorString(e));

    l2j_ctx *c = new l2j_ctx();
    c->cfg = *cfg;
    c->device = device;
    c->first_layer = first_layer;
    c->last_layer = last_layer;
    c->nl = last_layer - first_layer + 1;
    c->flags = flags;
    c->tp_rank = tp_rank;
    c->tp_size = tp_size;
    // Splitting the classifier's rows as well saves most of its 80 us per token but ends every token with a
    // rendezvous of all ranks; measured it gains 3 % at 2 ranks and loses 11 % at 4 and 8, so it is opt-in.
    c->cls_split = (flags & L2J_F_TP_SPLIT_CLASSIFIER) && tp_size > 1 && cfg->vocab_size % tp_size == 0;
    c->is_first = first_layer == 0;
    c->is_last = last_layer == cfg->n_layers - 1;
    c->dim = cfg->dim;
    c->hidden = cfg->hidden_dim;
    c->head = head;
    c->kv_dim = cfg->dim * cfg->n_kv_heads / cfg->n_heads;
    c->kv_mul = cfg->n_heads / cfg->n_kv_heads;

#define CREATE_CK(call)                     \
    do {                                    \
        int rc__ = (call);                  \
        if (rc__ != L2J_OK) {               \
            g_create_error = c->err;        \
            l2j_destroy(c);                 \
            return rc__;                    \
        }                                   \
    } while (0)
#define CREATE_CUDA(call)                                                                          \
    do {                                                                                           \
        cudaError_t e__ = (call);                                                                  \
        if (e__ != cudaSuccess) {                                                                  \
            fail(nullptr, L2J_E_CUDA, "%s failed: %s", #call, cudaGetErrorString(e__));            \
            l2j_destroy(c);                                                                        \
            return L2J_E_CUDA;                                                                     \
        }                                                                                          \
    } while (0)

    cudaDeviceProp prop{};
    CREATE_CUDA(cudaGetDeviceProperties(&prop, device));
    c->sm_count = prop.multiProcessorCount;
    CREATE_CUDA(prepare_kernels());
    CREATE_CUDA(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
    CREATE_CUDA(cudaEventCreate(&c->ev0));
    CREATE_CUDA(cudaEventCreate(&c->ev1));

    // quantised tensors: element counts per layer, TransformerWeights.java:54-111
    const int64_t dim = c->dim, kvd = c->kv_dim, hid = c->hidden;
    c->per_layer[L2J_T_RMS_ATT] = dim;
    c->per_layer[L2J_T_WQ] = dim * dim;
    c->per_layer[L2J_T_WK] = kvd * dim;
    c->per_layer[L2J_T_WV] = kvd * dim;
    c->per_layer[L2J_T_WO] = dim * dim;
    c->per_layer[L2J_T_RMS_FFN] = dim;
    c->per_layer[L2J_T_W1] = hid * dim;
    c->per_layer[L2J_T_W2] = dim * hid;
    c->per_layer[L2J_T_W3] = hid * dim;
    for (int t = 0; t < L2J_T_COUNT; ++t) {
        if (!is_quant_tensor(t))
            continue;
        int64_t f0, f1;
        if (t == L2J_T_RMS_FINAL) {
            if (!c->is_last)
                continue;
            f0 = 0;
            f1 = dim;
        } else {
            f0 = c->per_layer[t] * first_layer;
            f1 = c->per_layer[t] * (last_layer + 1);
        }
        c->needed[t] = true;
        QTensor &q = c->qt[t];
        const int64_t g0 = f0 / kGroup, g1 = (f1 + kGroup - 1) / kGroup;
        q.base_float = g0 * kGroup;
        q.n_groups = g1 - g0;
        CREATE_CK(dev_alloc(c, &q.payload, q.n_groups * kGroup + 512, true));
        CREATE_CK(dev_alloc(c, &q.hdr, q.n_groups + 8, true));
    }
    const bool need_emb = c->is_first || (c->is_last && cfg->shared_classifier);
    if (need_emb) {
        CREATE_CK(dev_alloc(c, &c->emb, (int64_t)cfg->vocab_size * dim, false));
        c->needed[L2J_T_TOKEN_EMBEDDING] = true;
    }
    if (c->is_last) {
        if (cfg->shared_classifier) {
            c->wcls = c->emb;
        } else {
            CREATE_CK(dev_alloc(c, &c->wcls, (int64_t)cfg->vocab_size * dim, false));
            c->needed[L2J_T_WCLS] = true;
        }
    }
    c->reps = (flags & L2J_F_SIMPLE) ? 1 : kVecReps;
    c->dim_stride = (int)(((dim + 63) & ~63) + 96);     // odd multiple of 32 floats: copies land on different L2 sets
    c->hid_stride = (int)(((hid + 63) & ~63) + 96);
    CREATE_CK(dev_alloc(c, &c->rms_att, (int64_t)c->nl * c->reps * c->dim_stride, true));
    CREATE_CK(dev_alloc(c, &c->rms_ffn, (int64_t)c->nl * c->reps * c->dim_stride, true));
    CREATE_CK(dev_alloc(c, &c->rms_final, (int64_t)c->reps * c->dim_stride, true));

    // run state, RunState.java:107-166 (q/k/v and att scratch are internal to the fused kernels)
    int64_t ymax = dim > hid ? dim : hid;
    if (cfg->vocab_size > ymax)
        ymax = cfg->vocab_size;
    CREATE_CK(dev_alloc(c, &c->x, (int64_t)c->reps * c->dim_stride, true));
    CREATE_CK(dev_alloc(c, &c->xb, (int64_t)c->reps * c->dim_stride, true));
    CREATE_CK(dev_alloc(c, &c->xn, dim, true));
    CREATE_CK(dev_alloc(c, &c->q, dim, true));
    CREATE_CK(dev_alloc(c, &c->hb, (int64_t)c->reps * c->hid_stride, true));
    CREATE_CK(dev_alloc(c, &c->logits, cfg->vocab_size, true));
    CREATE_CK(dev_alloc(c, &c->y0, ymax, true));
    CREATE_CK(dev_alloc(c, &c->y1, ymax, true));
    CREATE_CK(dev_alloc(c, &c->y2, ymax, true));
    const int64_t kv_floats = (int64_t)c->nl * cfg->n_kv_heads * cfg->seq_len * head;
    CREATE_CK(dev_alloc(c, &c->kc, kv_floats, true));
    CREATE_CK(dev_alloc(c, &c->vc, kv_floats, true));

    std::vector<float> cs, sn;
    build_rope_tables(cfg->seq_len, head, cs, sn);
    CREATE_CK(dev_alloc(c, &c->rope_cos, (int64_t)cs.size(), false));
    CREATE_CK(dev_alloc(c, &c->rope_sin, (int64_t)sn.size(), false));
    CREATE_CUDA(cudaMemcpy(c->rope_cos, cs.data(), cs.size() * sizeof(float), cudaMemcpyHostToDevice));
    CREATE_CUDA(cudaMemcpy(c->rope_sin, sn.data(), sn.size() * sizeof(float), cudaMemcpyHostToDevice));

    if (const char *e = getenv("L2J_EARLY_FILL"))
        c->early_fill = atoi(e);
    c->nsplit = choose_nsplit(c->sm_count, cfg->n_heads, cfg->seq_len);
    if (const char *e = getenv("L2J_ATTN_CLUSTER"))
        c->attn_cluster = atoi(e) != 0;
    if (c->attn_cluster && c->nsplit > 8)
        c->nsplit = 8;   // portable cluster size
    // A tensor-parallel rank has few heads: the long-context launch splits them further so that its blocks
    // still cover the SMs (its results travel with sequence numbers, no block count is baked in anywhere).
    c->nsplit_long = c->nsplit;
    if (tp_size > 1) {
        const int heads_local = cfg->n_heads / tp_size;
        int ns = (2 * c->sm_count) / heads_local;
        const int cap = cfg->seq_len / 64 > 0 ? cfg->seq_len / 64 : 1;
        if (ns > cap)
            ns = cap;
        if (ns > 64)
            ns = 64;
        if (ns > c->nsplit_long)
            c->nsplit_long = ns;
    }
    CREATE_CK(dev_alloc(c, &c->attn_part, (int64_t)cfg->n_heads * c->nsplit_long * (head + 2), true));
    CREATE_CK(dev_alloc(c, &c->attn_counters, cfg->n_heads, true));
    {   // blocks per ring kernel: one per SM, holding nearly all of its shared memory as the ring
        const char *g = getenv("L2J_BLOCKS_PER_SM");
        const int per_sm = g ? atoi(g) : 1;
        c->ring_grid = (per_sm >= 1 && per_sm <= 2 ? per_sm : 1) * c->sm_count;
    }
    CREATE_CK(dev_alloc(c, &c->blk_val, c->ring_grid + 8, true));
    CREATE_CK(dev_alloc(c, &c->blk_idx, c->ring_grid + 8, true));
    CREATE_CK(dev_alloc(c, &c->work, 2 * (4 * (int64_t)c->nl + 1), true));
    CREATE_CK(dev_alloc(c, &c->chain, kChainStride * (5 * (int64_t)c->nl + 2), true));   // + the epoch word
    if (const char *e = getenv("L2J_KV_PREFETCH"))
        c->kv_prefetch = atoi(e) != 0;
    if (const char *e = getenv("L2J_CHAIN"))
        c->chain_on = atoi(e) != 0;
    if (getenv("L2J_TRACE"))
        CREATE_CK(dev_alloc(c, &c->trace, (5 * (int64_t)c->nl + 1) * c->ring_grid * 16, true));
    CREATE_CK(dev_alloc(c, &c->prompt_dev, cfg->seq_len, true));
    CREATE_CK(dev_alloc(c, &c->out_tokens_dev, cfg->seq_len, true));
    CREATE_CK(dev_alloc(c, &c->state, 1, true));
    CREATE_CK(dev_alloc(c, &c->cmd_dev, 1, true));
    CREATE_CUDA(cudaHostAlloc((void **)&c->cmd_host, sizeof(Cmd) * kCmdRing, cudaHostAllocDefault));
    CREATE_CK(dev_alloc(c, &c->link_dev, 1, true));
    CREATE_CK(dev_alloc(c, &c->tp_dev, 1, true));
    if (tp_size > 1) {
        CREATE_CK(dev_alloc(c, &c->x2, (int64_t)c->reps * c->dim_stride, true));
        CREATE_CK(dev_alloc(c, &c->ll_buf[TPV_X], c->dim, true));
        CREATE_CK(dev_alloc(c, &c->ll_buf[TPV_XB], c->dim, true));
        CREATE_CK(dev_alloc(c, &c->ll_buf[TPV_HB], c->hidden, true));
        CREATE_CK(dev_alloc(c, &c->ll_buf[TPV_CAND], 2 * kMaxTp, true));
    }
    CREATE_CUDA(cudaEventCreateWithFlags(&c->ev_stage, cudaEventDisableTiming));
    CREATE_CUDA(cudaHostAlloc((void **)&c->logits_host, sizeof(float) * (size_t)cfg->vocab_size, cudaHostAllocDefault));
    CREATE_CUDA(cudaHostAlloc((void **)&c->x_host, sizeof(float) * (size_t)c->reps * c->dim_stride, cudaHostAllocDefault));
    CREATE_CUDA(cudaHostAlloc((void **)&c->state_host, sizeof(SeqState), cudaHostAllocDefault));
    memset(c->state_host, 0, sizeof(SeqState));

    if (tp_size == 1) {
        c->plan_qkv = plan_matvec(c->dim, false, false, 0, 0, 2);   // RoPE works on row pairs: stages of an even number of rows
        c->plan_wo = plan_matvec(c->dim, false, false, c->dim, c->ring_grid);
        c->plan_w13 = plan_matvec(c->dim, false, true);
        c->plan_hidden = plan_matvec(c->hidden, false, false);
    } else {   // a rank's block of rows is small: let the planner shrink the stages
        c->plan_qkv = plan_matvec(c->dim, false, false, c->dim / tp_size, c->ring_grid, 2);
        c->plan_wo = plan_matvec(c->dim, false, false, c->dim / tp_size, c->ring_grid);
        c->plan_w13 = plan_matvec(c->dim, false, true, 2 * (c->hidden / tp_size), c->ring_grid);
        c->plan_hidden = plan_matvec(c->hidden, false, false, c->dim / tp_size, c->ring_grid);
    }
    c->plan_cls = plan_matvec(c->dim, true, false);
    c->use_ring = !(flags & L2J_F_SIMPLE) && c->plan_qkv.ok && c->plan_wo.ok && c->plan_w13.ok && c->plan_hidden.ok &&
                  c->plan_cls.ok && (head % 2 == 0);
    {   // one persistent launch per token where every matrix has rows of whole quantisation groups
        // (a consumer warp converts every 18th group of the input vector, three at most; a lane's eight elements of the
        // attention output lie in one head)
        bool fused = c->use_ring && tp_size == 1 && !(flags & L2J_F_STEP_KERNELS) && c->reps == 1 && c->dim % kGroup == 0 &&
                     c->hidden % kGroup == 0 && c->dim <= 3 * kFusedConsWarps * kGroup && c->hidden <= 3 * kFusedConsWarps * kGroup &&
                     head % 8 == 0;
        // Measured on B200: with dim a multiple of 2048 (every consumer warp's lanes own a group of the rows:
        // 7B shape) the persistent kernel is level with the per-step kernels at short contexts and 4 % ahead at
        // long ones; with 20 groups per row (13B shape) a sixth of the lanes idle and it is 9 % behind.
        if (!(flags & L2J_F_PERSISTENT) && c->dim % (8 * kGroup) != 0)
            fused = false;
        if (const char *e = getenv("L2J_FUSED"))   // diagnostic: A/B against the per-step kernels
            fused = fused && atoi(e) != 0;
        if (fused) {
            c->fplan[0] = plan_fused_phase(c->dim, false, 2);
            c->fplan[1] = plan_fused_phase(c->dim, false, 1);
            c->fplan[2] = plan_fused_phase(c->dim, true, 1);
            c->fplan[3] = plan_fused_phase(c->hidden, false, 1);
            fused = c->fplan[0].ok && c->fplan[1].ok && c->fplan[2].ok && c->fplan[3].ok;
        }
        if (fused) {
            CREATE_CUDA(prepare_fused(&c->max_smem));
            c->fused_smem = c->max_smem < 232448 ? c->max_smem : 232448;
            int largest = 0;
            for (int k = 0; k < 4; ++k)
                largest = c->fplan[k].slot_bytes > largest ? c->fplan[k].slot_bytes : largest;
            const int limb_bytes = 3 * (c->dim > c->hidden ? c->dim : c->hidden);
            if (c->fused_smem - kFusedHeaderBytes - limb_bytes - 4096 < 3 * largest)
                fused = false;   // the ring would not hold three stages
        }
        if (fused) {
            CREATE_CK(dev_alloc(c, &c->rms_wmax_dev, 2 * (int64_t)c->nl, true));
            CREATE_CK(dev_alloc(c, &c->fused_part, (int64_t)cfg->n_heads * kAttSlots * (head + 4), true));
            if (getenv("L2J_TRACE"))
                CREATE_CK(dev_alloc(c, &c->fused_trace, (int64_t)c->ring_grid * 5 * c->nl * 8, true));
        }
        c->use_fused = fused;
    }
    CREATE_CUDA(cudaStreamSynchronize(c->stream));
    CREATE_CUDA(cudaDeviceSynchronize());
#undef CREATE_CK
#undef CREATE_CUDA
    *out = c;
    return L2J_OK;
}

extern "C" int l2j_create(const l2j_config *cfg, int device, int first_layer, int last_layer, uint32_t flags, l2j_ctx **out)
{
    return create_impl(cfg, device, first_layer, last_layer, flags, 0, 1, out);
}

extern "C" int l2j_create_tp(const l2j_config *cfg, int device, int tp_rank, int tp_size, uint32_t flags, l2j_ctx **out)
{
    if (!cfg)
        return fail(nullptr, L2J_E_INVALID, "null argument");
    return create_impl(cfg, device, 0, cfg->n_layers - 1, flags, tp_rank, tp_size, out);
}

extern "C" void l2j_destroy(l2j_ctx *c)
{
    if (!c)
        return;
    {   // the stages this one was linked with hold pointers into its memory: they are unlinked with it
        std::lock_guard<std::mutex> lock(g_link_mu);
        for (l2j_ctx *m : c->pipe_members)
            if (m != c)
                m->pipe_members.clear();
        c->pipe_members.clear();
    }
    cudaSetDevice(c->device);
    if (c->stream)
        cudaStreamSynchronize(c->stream);
    if (c->exec)
        cudaGraphExecDestroy(c->exec);
    if (c->exec_long)
        cudaGraphExecDestroy(c->exec_long);
    if (c->graph_long)
        cudaGraphDestroy(c->graph_long);
    if (c->graph)
        cudaGraphDestroy(c->graph);
    for (void *p : c->allocs)
        cudaFree(p);
    if (c->cmd_host)
        cudaFreeHost(c->cmd_host);
    if (c->ev_stage)
        cudaEventDestroy(c->ev_stage);
    if (c->logits_host)
        cudaFreeHost(c->logits_host);
    if (c->x_host)
        cudaFreeHost(c->x_host);
    if (c->state_host)
        cudaFreeHost(c->state_host);
    if (c->samp_host)
        cudaFreeHost(c->samp_host);
    prefill_destroy(c->prefill);
    if (c->ev0)
        cudaEventDestroy(c->ev0);
    if (c->ev1)
        cudaEventDestroy(c->ev1);
    if (c->stream)
        cudaStreamDestroy(c->stream);
    delete c;
}

extern "C" const char *l2j_last_error(const l2j_ctx *c)
{
    return c ? c->err.c_str() : g_create_error.c_str();
}

// ===============================================================================================
// weights
// ===============================================================================================

extern "C" int l2j_upload_quant(l2j_ctx *c, int tensor, int64_t float_offset, const void *groups, int64_t bytes,
                                int64_t n_floats)
{
    if (!c)
        return L2J_E_INVALID;
    std::lock_guard<std::mutex> lock(c->mu);
    if (tensor < 0 || tensor >= L2J_T_COUNT || !is_quant_tensor(tensor))
        return fail(c, L2J_E_INVALID, "tensor %d is not a quantised tensor", tensor);
    if (!groups || n_floats <= 0 || float_offset < 0 || float_offset % kGroup != 0)
        return fail(c, L2J_E_INVALID, "bad part: offset %lld must be a non-negative multiple of 256, n_floats %lld positive",
                    (long long)float_offset, (long long)n_floats);
    const int64_t part_groups = (n_floats + kGroup - 1) / kGroup;
    if (bytes != part_groups * kGroupBytes)
        return fail(c, L2J_E_INVALID, "bytes %lld != ceil(n_floats/256)*264 = %lld", (long long)bytes,
                    (long long)(part_groups * kGroupBytes));
    if (c->finalized)
        return fail(c, L2J_E_STATE, "upload after finalize");
    if (!c->needed[tensor])
        return L2J_OK;   // e.g. the final norm on a stage that is not the last
    QTensor &q = c->qt[tensor];
    const int64_t pg0 = float_offset / kGroup, pg1 = pg0 + part_groups;
    const int64_t g0 = q.base_float / kGroup, g1 = g0 + q.n_groups;
    const int64_t i0 = pg0 > g0 ? pg0 : g0, i1 = pg1 < g1 ? pg1 : g1;
    if (i1 <= i0)
        return L2J_OK;
    if (!add_interval(c->got[tensor], i0, i1))
        return fail(c, L2J_E_INVALID, "tensor %d: groups [%lld, %lld) overlap a part that was uploaded before", tensor,
                    (long long)i0, (long long)i1);
    CK(c, cudaSetDevice(c->device));
    const int64_t count = i1 - i0;
    const uint8_t *src = static_cast<const uint8_t *>(groups) + (i0 - pg0) * kGroupBytes;
    // stage through device memory in pieces so that a 1.5 GB tensor does not need a second copy of itself
    const int64_t piece = 1 << 18;   // groups per piece (66 MiB)
    uint8_t *stage = nullptr;
    const int64_t stage_groups = count < piece ? count : piece;
    cudaError_t e = cudaMalloc((void **)&stage, (size_t)stage_groups * kGroupBytes);
    if (e != cudaSuccess)
        return fail(c, L2J_E_NOMEM, "staging allocation failed: %s", cudaGetErrorString(e));
    int rc = L2J_OK;
    for (int64_t done = 0; done < count && rc == L2J_OK; done += piece) {
        const int64_t ng = count - done < piece ? count - done : piece;
        e = cudaMemcpyAsync(stage, src + done * kGroupBytes, (size_t)ng * kGroupBytes, cudaMemcpyHostToDevice, c->stream);
        if (e == cudaSuccess) {
            uint8_t *dp = q.payload + (i0 - g0 + done) * kGroup;
            float2 *dh = q.hdr + (i0 - g0 + done);
            e = is_rms_tensor(tensor) ? launch_repack_minmax(c->stream, stage, ng, dp, dh)
                                      : launch_repack(c->stream, stage, ng, dp, dh);
        }
        if (e == cudaSuccess)
            e = cudaStreamSynchronize(c->stream);
        if (e != cudaSuccess)
            rc = fail(c, L2J_E_CUDA, "upload of tensor %d failed: %s", tensor, cudaGetErrorString(e));
    }
    cudaFree(stage);
    q.groups_received = covered(c->got[tensor]);
    return rc;
}

extern "C" int l2j_upload_f32(l2j_ctx *c, int tensor, int64_t float_offset, const float *data, int64_t n_floats)
{
    if (!c)
        return L2J_E_INVALID;
    std::lock_guard<std::mutex> lock(c->mu);
    if (tensor != L2J_T_TOKEN_EMBEDDING && tensor != L2J_T_WCLS)
        return fail(c, L2J_E_INVALID, "tensor %d is not an FP32 tensor", tensor);
    const int64_t total = (int64_t)c->cfg.vocab_size * c->dim;
    if (!data || float_offset < 0 || n_floats <= 0 || float_offset + n_floats > total)
        return fail(c, L2J_E_INVALID, "bad FP32 part [%lld, +%lld) of %lld", (long long)float_offset, (long long)n_floats,
                    (long long)total);
    if (c->finalized)
        return fail(c, L2J_E_STATE, "upload after finalize");
    if (tensor == L2J_T_WCLS && c->cfg.shared_classifier)
        return fail(c, L2J_E_INVALID, "the classifier is shared with the embedding in this configuration");
    if (!c->needed[tensor])
        return L2J_OK;
    if (!add_interval(c->got[tensor], float_offset, float_offset + n_floats))
        return fail(c, L2J_E_INVALID, "tensor %d: floats [%lld, +%lld) overlap a part that was uploaded before", tensor,
                    (long long)float_offset, (long long)n_floats);
    CK(c, cudaSetDevice(c->device));
    float *dst = tensor == L2J_T_TOKEN_EMBEDDING ? c->emb : c->wcls;
    CK(c, cudaMemcpy(dst + float_offset, data, (size_t)n_floats * sizeof(float), cudaMemcpyHostToDevice));
    (tensor == L2J_T_TOKEN_EMBEDDING ? c->emb_received : c->wcls_received) = covered(c->got[tensor]);
    return L2J_OK;
}

extern "C" int l2j_finalize(l2j_ctx *c)
{
    if (!c)
        return L2J_E_INVALID;
    std::lock_guard<std::mutex> lock(c->mu);
    if (c->finalized)
        return L2J_OK;
    CK(c, cudaSetDevice(c->device));
    for (int t = 0; t < L2J_T_COUNT; ++t) {
        if (!c->needed[t])
            continue;
        if (is_quant_tensor(t)) {
            if (c->qt[t].groups_received != c->qt[t].n_groups)
                return fail(c, L2J_E_STATE, "tensor %d: %lld of %lld groups uploaded", t, (long long)c->qt[t].groups_received,
                            (long long)c->qt[t].n_groups);
        } else {
            const int64_t total = (int64_t)c->cfg.vocab_size * c->dim;
            const int64_t got = t == L2J_T_TOKEN_EMBEDDING ? c->emb_received : c->wcls_received;
            if (got != total)
                return fail(c, L2J_E_STATE, "tensor %d: %lld of %lld floats uploaded", t, (long long)got, (long long)total);
        }
    }
    const int64_t dim = c->dim;
    for (int li = 0; li < c->nl; ++li) {
        for (int r = 0; r < c->reps; ++r) {
            const int64_t off = ((int64_t)li * c->reps + r) * c->dim_stride;
            CK(c, launch_dequant_rms(c->stream, c->qt[L2J_T_RMS_ATT], dim * (c->first_layer + li), dim, c->rms_att + off));
            CK(c, launch_dequant_rms(c->stream, c->qt[L2J_T_RMS_FFN], dim * (c->first_layer + li), dim, c->rms_ffn + off));
        }
    }
    if (c->is_last)
        for (int r = 0; r < c->reps; ++r)
            CK(c, launch_dequant_rms(c->stream, c->qt[L2J_T_RMS_FINAL], 0, dim, c->rms_final + (int64_t)r * c->dim_stride));
    CK(c, cudaStreamSynchronize(c->stream));
    build_launch_params(c);
    {   // largest RMSNorm weight per launch: bounds the normalised vector for the kernels' fixed-point scale
        std::vector<float> w((size_t)dim * (size_t)(c->nl > 1 ? c->nl : 1));
        auto vmax = [&](const float *src, int64_t n) {
            float m = 0.f;
            for (int64_t i = 0; i < n; ++i)
                m = std::fmax(m, std::fabs(src[i]));
            return m;
        };
        for (int li = 0; li < c->nl; ++li) {
            const int64_t off = (int64_t)li * c->reps * c->dim_stride;
            CK(c, cudaMemcpy(w.data(), c->rms_att + off, sizeof(float) * (size_t)dim, cudaMemcpyDeviceToHost));
            c->layers[(size_t)li].qkv.rms_wmax = vmax(w.data(), dim);
            CK(c, cudaMemcpy(w.data(), c->rms_ffn + off, sizeof(float) * (size_t)dim, cudaMemcpyDeviceToHost));
            c->layers[(size_t)li].w13.rms_wmax = vmax(w.data(), dim);
        }
        if (c->is_last) {
            CK(c, cudaMemcpy(w.data(), c->rms_final, sizeof(float) * (size_t)dim, cudaMemcpyDeviceToHost));
            c->cls.rms_wmax = vmax(w.data(), dim);
        }
        if (c->use_fused) {
            std::vector<float> wm(2 * (size_t)c->nl);
            for (int li = 0; li < c->nl; ++li) {
                wm[2 * (size_t)li] = c->layers[(size_t)li].qkv.rms_wmax;
                wm[2 * (size_t)li + 1] = c->layers[(size_t)li].w13.rms_wmax;
            }
            CK(c, cudaMemcpy(c->rms_wmax_dev, wm.data(), sizeof(float) * wm.size(), cudaMemcpyHostToDevice));
        }
    }

    {   // device copies of the launch parameters, chained in launch order, for the cross-launch L2 prefetch
        const int count = 4 * c->nl + (c->is_last ? 1 : 0);
        MvParams *dev = nullptr;
        int rc2 = dev_alloc(c, &dev, count, true);
        if (rc2 != L2J_OK)
            return rc2;
        std::vector<MvParams *> order;
        for (int li = 0; li < c->nl; ++li) {
            LayerLaunch &L = c->layers[(size_t)li];
            order.push_back(&L.qkv);
            order.push_back(&L.wo);
            order.push_back(&L.w13);
            order.push_back(&L.w2);
        }
        if (c->is_last)
            order.push_back(&c->cls);
        for (int i = 0; i < count; ++i)
            order[(size_t)i]->next = dev + (i + 1) % count;   // the last launch of a token prefetches for the next token
        for (int i = 0; i < count; ++i)
            CK(c, cudaMemcpy(dev + i, order[(size_t)i], sizeof(MvParams), cudaMemcpyHostToDevice));
    }
    c->pdl_on = c->use_ring && !(c->flags & L2J_F_NO_PDL);
    if (!(c->flags & L2J_F_NO_GRAPH)) {
        if (!try_capture(c, c->pdl_on, false)) {
            if (c->pdl_on) {
                c->pdl_on = false;
                try_capture(c, false, false);
            }
        }
        if (c->exec && c->use_ring && !c->use_fused && c->cfg.seq_len > kLongContextPos)
            try_capture(c, c->pdl_on, true);   // without it the long regime is enqueued kernel by kernel
    }
    c->finalized = true;
    return L2J_OK;
}

// ===============================================================================================
// forward
// ===============================================================================================

extern "C" int l2j_forward_stage_async(l2j_ctx *c, int token, int pos)
{
    if (!c)
        return L2J_E_INVALID;
    if (!c->finalized)
        return fail(c, L2J_E_STATE, "forward before finalize");
    if (c->tp_size > 1)
        return fail(c, L2J_E_STATE, "a rank of a tensor-parallel group runs through l2j_tp_forward");
    std::lock_guard<std::mutex> lock(c->mu);
    int rc = check_range(c, token, pos, c->is_first);
    if (rc != L2J_OK)
        return rc;
    CK(c, cudaSetDevice(c->device));
    // every queued forward holds a slot of the pinned command ring until its copy has run
    if (++c->async_in_flight >= kCmdRing) {
        CK(c, cudaStreamSynchronize(c->stream));
        c->async_in_flight = 1;
    }
    rc = post_cmd(c, 1, c->is_first ? token : 0, pos);
    if (rc != L2J_OK)
        return rc;
    return launch_forward(c, pos);
}

extern "C" int l2j_sync(l2j_ctx *c)
{
    if (!c)
        return L2J_E_INVALID;
    std::lock_guard<std::mutex> lock(c->mu);
    CK(c, cudaSetDevice(c->device));
    CK(c, cudaMemcpyAsync(c->state_host, c->state, sizeof(SeqState), cudaMemcpyDeviceToHost, c->stream));
    CK(c, cudaStreamSynchronize(c->stream));
    c->async_in_flight = 0;
    return finish_status(c);
}

extern "C" int l2j_forward_stage(l2j_ctx *c, int token, int pos, const float *x_in, float *x_out, float *logits, int *argmax)
{
    if (!c)
        return L2J_E_INVALID;
    std::lock_guard<std::mutex> lock(c->mu);
    if (!c->finalized)
        return fail(c, L2J_E_STATE, "forward before finalize");
    if (c->tp_size > 1)
        return fail(c, L2J_E_STATE, "a rank of a tensor-parallel group runs through l2j_tp_forward");
    if (!c->is_first && !x_in)
        return fail(c, L2J_E_INVALID, "a stage that does not start at layer 0 needs x_in");
    int rc = check_range(c, token, pos, c->is_first);
    if (rc != L2J_OK)
        return rc;
    CK(c, cudaSetDevice(c->device));
    if (!c->is_first) {
        for (int r = 0; r < c->reps; ++r)
            memcpy(c->x_host + (size_t)r * c->dim_stride, x_in, sizeof(float) * (size_t)c->dim);
        CK(c, cudaMemcpyAsync(c->x, c->x_host, sizeof(float) * (size_t)c->reps * c->dim_stride, cudaMemcpyHostToDevice,
                              c->stream));
    }
    rc = post_cmd(c, 1, c->is_first ? token : 0, pos);
    if (rc != L2J_OK)
        return rc;
    rc = launch_forward(c, pos);
    if (rc != L2J_OK)
        return rc;
    if (c->is_last && logits)
        CK(c, cudaMemcpyAsync(c->logits_host, c->logits, sizeof(float) * (size_t)c->cfg.vocab_size, cudaMemcpyDeviceToHost,
                              c->stream));
    if (!c->is_last && x_out)
        CK(c, cudaMemcpyAsync(c->x_host, c->x, sizeof(float) * (size_t)c->dim, cudaMemcpyDeviceToHost, c->stream));
    CK(c, cudaMemcpyAsync(c->state_host, c->state, sizeof(SeqState), cudaMemcpyDeviceToHost, c->stream));
    CK(c, spin_sync(c));
    if (c->is_last && logits)
        memcpy(logits, c->logits_host, sizeof(float) * (size_t)c->cfg.vocab_size);
    if (!c->is_last && x_out)
        memcpy(x_out, c->x_host, sizeof(float) * (size_t)c->dim);
    if (c->is_last && argmax)
        *argmax = c->state_host->argmax;
    return finish_status(c);
}

extern "C" int l2j_forward(l2j_ctx *c, int token, int pos, float *logits, int *argmax)
{
    if (!c)
        return L2J_E_INVALID;
    if (!(c->is_first && c->is_last))
        return fail(c, L2J_E_STATE, "l2j_forward needs a context that holds every layer; use l2j_forward_stage");
    return l2j_forward_stage(c, token, pos, nullptr, nullptr, logits, argmax);
}

// The batched prompt path works on this context's own weights, caches and tables.
static PrefillModel prefill_model(l2j_ctx *c)
{
    PrefillModel m{};
    m.dim = c->dim;
    m.hidden = c->hidden;
    m.n_layers = c->nl;
    m.n_heads = c->cfg.n_heads;
    m.n_kv_heads = c->cfg.n_kv_heads;
    m.head = c->head;
    m.seq_len = c->cfg.seq_len;
    m.vocab = c->cfg.vocab_size;
    m.emb = c->emb;
    m.wcls = c->wcls;
    m.rms_final = c->rms_final;
    m.status = reinterpret_cast<unsigned int *>(&c->state->status);
    m.timeout_us = c->wait_limit_us;
    auto payload = [](const MvSeg &s) { return s.payload + s.flat0; };
    auto hdr = [](const MvSeg &s) { return s.hdr + s.flat0 / kGroup; };
    for (int li = 0; li < c->nl; ++li) {
        const LayerLaunch &L = c->layers[(size_t)li];
        PrefillLayerDesc d{};
        const MvSeg *segs[PF_W_COUNT] = {&L.qkv.seg[0], &L.qkv.seg[1], &L.qkv.seg[2], &L.wo.seg[0], &L.w13.seg[0], &L.w13.seg[1], &L.w2.seg[0]};
        for (int w = 0; w < PF_W_COUNT; ++w) {
            d.w[w] = payload(*segs[w]);
            d.h[w] = hdr(*segs[w]);
        }
        d.rms_att = L.qkv.rms_w;
        d.rms_ffn = L.w13.rms_w;
        d.kc = L.qkv.k_cache;
        d.vc = L.qkv.v_cache;
        m.rope_cos = L.qkv.rope_cos;
        m.rope_sin = L.qkv.rope_sin;
        m.layers.push_back(d);
    }
    return m;
}

// Builds the batched path of a whole-model context on first use; L2J_E_INVALID where the shape is outside it.
static int ensure_prefill(l2j_ctx *c, bool required)
{
    if (!c->prefill_tried) {
        c->prefill_tried = true;
        const PrefillModel m = prefill_model(c);
        if (prefill_supported(m) && !(c->flags & L2J_F_NO_TENSOR_PREFILL))
            CK(c, prefill_create(&c->prefill, m));
    }
    if (required && !c->prefill)
        return fail(c, L2J_E_INVALID, "the batched path needs rows of whole quantisation groups and a head size of 64 or 128");
    return L2J_OK;
}

extern "C" int l2j_prefill(l2j_ctx *c, const int32_t *tokens, int n, int pos0)
{
    if (!c || (n > 0 && !tokens))
        return L2J_E_INVALID;
    {
        std::lock_guard<std::mutex> lock(c->mu);
        if (!c->finalized)
            return fail(c, L2J_E_STATE, "prefill before finalize");
        if (!(c->is_first && c->is_last) || c->tp_size > 1)
            return fail(c, L2J_E_STATE, "l2j_prefill needs a context that holds every layer");
        if (n < 0 || pos0 < 0 || (int64_t)pos0 + n > c->cfg.seq_len)
            return fail(c, L2J_E_INVALID, "positions %d..%d outside the sequence length %d", pos0, pos0 + n - 1, c->cfg.seq_len);
        for (int i = 0; i < n; ++i)
            if (tokens[i] < 0 || tokens[i] >= c->cfg.vocab_size)
                return fail(c, L2J_E_INVALID, "token %d outside the vocabulary", tokens[i]);
        if (n == 0)
            return L2J_OK;
        CK(c, cudaSetDevice(c->device));
        const int rc = ensure_prefill(c, false);
        if (rc != L2J_OK)
            return rc;
        if (c->prefill) {
            CK(c, prefill_run(c->prefill, c->stream, tokens, n, pos0));
            CK(c, cudaMemcpyAsync(c->state_host, c->state, sizeof(SeqState), cudaMemcpyDeviceToHost, c->stream));
            CK(c, cudaStreamSynchronize(c->stream));
            return finish_status(c);
        }
    }
    // shapes the tensor-core path does not take: the prompt goes through the decode step, as in the reference
    for (int i = 0; i < n; ++i) {
        const int rc = l2j_forward_stage_async(c, tokens[i], pos0 + i);
        if (rc != L2J_OK)
            return rc;
    }
    return l2j_sync(c);
}

extern "C" int l2j_batch_create(l2j_ctx *c, int n_seq, int seq_len)
{
    if (!c)
        return L2J_E_INVALID;
    std::lock_guard<std::mutex> lock(c->mu);
    if (!c->finalized)
        return fail(c, L2J_E_STATE, "batch before finalize");
    if (!(c->is_first && c->is_last) || c->tp_size > 1)
        return fail(c, L2J_E_STATE, "concurrent sequences need a context that holds every layer");
    if (n_seq < 1 || seq_len < 1 || seq_len > c->cfg.seq_len)
        return fail(c, L2J_E_INVALID, "n_seq >= 1 and 1 <= seq_len <= %d", c->cfg.seq_len);
    CK(c, cudaSetDevice(c->device));
    const int rc = ensure_prefill(c, true);
    if (rc != L2J_OK)
        return rc;
    CK(c, cudaStreamSynchronize(c->stream));
    const cudaError_t e = prefill_batch_create(c->prefill, n_seq, seq_len);
    if (e == cudaErrorMemoryAllocation) {
        cudaGetLastError();
        return fail(c, L2J_E_NOMEM, "no device memory for the caches of %d sequences of %d positions", n_seq, seq_len);
    }
    CK(c, e);
    return L2J_OK;
}

extern "C" int l2j_batch_forward(l2j_ctx *c, int n, const int32_t *seq, const int32_t *pos, const int32_t *tokens, float *logits,
                                 int32_t *argmax)
{
    if (!c || n < 0 || (n > 0 && (!seq || !pos || !tokens)))
        return L2J_E_INVALID;
    std::lock_guard<std::mutex> lock(c->mu);
    if (!c->prefill || prefill_batch_sequences(c->prefill) == 0)
        return fail(c, L2J_E_STATE, "call l2j_batch_create first");
    if (n > kPrefillTokens)
        return fail(c, L2J_E_INVALID, "at most %d (sequence, position) pairs per call", kPrefillTokens);
    for (int i = 0; i < n; ++i) {
        if (seq[i] < 0 || seq[i] >= prefill_batch_sequences(c->prefill) || pos[i] < 0 || pos[i] >= prefill_batch_seq_len(c->prefill) ||
            tokens[i] < 0 || tokens[i] >= c->cfg.vocab_size)
            return fail(c, L2J_E_INVALID, "entry %d: sequence %d, position %d or token %d out of range", i, seq[i], pos[i], tokens[i]);
        for (int j = 0; j < i; ++j)
            if (seq[j] == seq[i] && pos[j] == pos[i])
                return fail(c, L2J_E_INVALID, "entries %d and %d name the same position of sequence %d", j, i, seq[i]);
    }
    if (n == 0)
        return L2J_OK;
    CK(c, cudaSetDevice(c->device));
    CK(c, prefill_batch_forward(c->prefill, c->stream, tokens, pos, seq, n, logits, argmax));
    CK(c, cudaMemcpyAsync(c->state_host, c->state, sizeof(SeqState), cudaMemcpyDeviceToHost, c->stream));
    CK(c, cudaStreamSynchronize(c->stream));
    return finish_status(c);
}

extern "C" uint64_t l2j_prefill_launches(l2j_ctx *c)
{
    if (!c)
        return 0;
    std::lock_guard<std::mutex> lock(c->mu);
    return prefill_launches(c->prefill);
}

extern "C" int l2j_sampler_seed(l2j_ctx *c, int64_t seed)
{
    if (!c)
        return L2J_E_INVALID;
    std::lock_guard<std::mutex> lock(c->mu);
    if (!c->finalized || !c->is_last)
        return fail(c, L2J_E_STATE, "the sampler belongs to the finalized context that holds the classifier");
    const int n = c->cfg.vocab_size;
    if (n < 2 || sample_smem_bytes(n) > 220 * 1024)
        return fail(c, L2J_E_INVALID, "the device sampler keeps the probabilities in shared memory: vocabulary of 2..%d tokens",
                    (int)((220 * 1024 - 65536) / 4));
    CK(c, cudaSetDevice(c->device));
    if (!c->samp_state) {
        int rc = dev_alloc(c, &c->samp_state, 1, true);
        for (int b = 0; b < 2 && rc == L2J_OK; ++b) {
            rc = dev_alloc(c, &c->samp_prob[b], n, true);
            if (rc == L2J_OK)
                rc = dev_alloc(c, &c->samp_index[b], n, true);
        }
        if (rc != L2J_OK)
            return rc;
        CK(c, cudaHostAlloc((void **)&c->samp_host, sizeof(SamplerState), cudaHostAllocDefault));
        CK(c, prepare_sampler(n));
    }
    CK(c, cudaStreamSynchronize(c->stream));
    // new Sampler(seed, vocab): every ProbIndex is (0, 0), Random(seed) scrambles the seed (java.util.Random)
    for (int b = 0; b < 2; ++b) {
        CK(c, cudaMemset(c->samp_prob[b], 0, sizeof(float) * (size_t)n));
        CK(c, cudaMemset(c->samp_index[b], 0, sizeof(int) * (size_t)n));
    }
    SamplerState init{};
    init.rng = ((unsigned long long)seed ^ 0x5DEECE66DULL) & ((1ULL << 48) - 1ULL);
    init.token = 0;
    CK(c, cudaMemcpy(c->samp_state, &init, sizeof(init), cudaMemcpyHostToDevice));
    return L2J_OK;
}

extern "C" int l2j_sample(l2j_ctx *c, float temperature, float topp, int *token)
{
    if (!c || !token)
        return L2J_E_INVALID;
    std::lock_guard<std::mutex> lock(c->mu);
    if (!c->finalized || !c->is_last)
        return fail(c, L2J_E_STATE, "sampling needs the finalized context that holds the classifier");
    if (!(temperature >= 0.0f) || !(topp >= 0.0f))
        return fail(c, L2J_E_INVALID, "temperature and topp must not be negative");
    CK(c, cudaSetDevice(c->device));
    if (temperature == 0.0f) {   // Run.java:639-642: the arg-max, already chosen on the device by the classifier's launch
        CK(c, cudaMemcpyAsync(c->state_host, c->state, sizeof(SeqState), cudaMemcpyDeviceToHost, c->stream));
        CK(c, cudaStreamSynchronize(c->stream));
        *token = c->state_host->argmax;
        return finish_status(c);
    }
    if (!c->samp_state)
        return fail(c, L2J_E_STATE, "call l2j_sampler_seed first");
    SampleParams sp{};
    sp.logits = c->logits;
    sp.n = c->cfg.vocab_size;
    sp.temperature = temperature;
    sp.topp = topp;
    sp.st = c->samp_state;
    for (int b = 0; b < 2; ++b) {
        sp.prob[b] = c->samp_prob[b];
        sp.index[b] = c->samp_index[b];
    }
    CK(c, launch_sample(c->stream, sp));
    CK(c, cudaMemcpyAsync(c->samp_host, c->samp_state, sizeof(SamplerState), cudaMemcpyDeviceToHost, c->stream));
    CK(c, cudaStreamSynchronize(c->stream));
    *token = c->samp_host->token;
    return L2J_OK;
}

extern "C" int l2j_device_buffers(l2j_ctx *c, void **x_dev, void **logits_dev)
{
    if (!c)
        return L2J_E_INVALID;
    if (x_dev)
        *x_dev = c->x;
    if (logits_dev)
        *logits_dev = c->logits;
    return L2J_OK;
}

extern "C" int l2j_generate_greedy(l2j_ctx *c, const int32_t *prompt, int n_prompt, int steps, int32_t *out_tokens)
{
    if (!c)
        return L2J_E_INVALID;
    std::lock_guard<std::mutex> lock(c->mu);
    if (!c->finalized)
        return fail(c, L2J_E_STATE, "generate before finalize");
    if (!(c->is_first && c->is_last) || c->tp_size > 1)
        return fail(c, L2J_E_STATE, "l2j_generate_greedy needs a context that holds every layer and all rows");
    if (steps <= 0 || steps > c->cfg.seq_len || n_prompt < 0 || n_prompt > c->cfg.seq_len || (n_prompt > 0 && !prompt) ||
        !out_tokens)
        return fail(c, L2J_E_INVALID, "bad arguments: steps %d (seq_len %d), n_prompt %d", steps, c->cfg.seq_len, n_prompt);
    for (int i = 0; i < n_prompt; ++i)
        if (prompt[i] < 0 || prompt[i] >= c->cfg.vocab_size)
            return fail(c, L2J_E_INVALID, "prompt token %d outside the vocabulary", prompt[i]);
    CK(c, cudaSetDevice(c->device));
    if (n_prompt > 0)
        CK(c, cudaMemcpyAsync(c->prompt_dev, prompt, sizeof(int32_t) * (size_t)n_prompt, cudaMemcpyHostToDevice, c->stream));
    SeqState init{};
    init.token = 1;   // BOS, Run.java:614
    init.pos = 0;
    init.n_prompt = n_prompt;
    CK(c, cudaMemcpyAsync(c->state, &init, sizeof(SeqState), cudaMemcpyHostToDevice, c->stream));
    CK(c, cudaStreamSynchronize(c->stream));   // `init` and a pageable `prompt` must not be read later
    int rc = post_cmd(c, 0, 0, 0);
    if (rc != L2J_OK)
        return rc;
    CK(c, cudaEventRecord(c->ev0, c->stream));
    for (int s = 0; s < steps; ++s) {
        rc = launch_forward(c, s);
        if (rc != L2J_OK)
            return rc;
    }
    CK(c, cudaEventRecord(c->ev1, c->stream));
    CK(c, cudaMemcpyAsync(c->state_host, c->state, sizeof(SeqState), cudaMemcpyDeviceToHost, c->stream));
    CK(c, cudaStreamSynchronize(c->stream));
    CK(c, cudaMemcpy(out_tokens, c->out_tokens_dev, sizeof(int32_t) * (size_t)steps, cudaMemcpyDeviceToHost));
    float ms = 0.f;
    CK(c, cudaEventElapsedTime(&ms, c->ev0, c->ev1));
    c->last_generate_us = (double)ms * 1000.0;
    return finish_status(c);
}

extern "C" int l2j_kv_write(l2j_ctx *c, int layer, int pos0, int n_pos, const float *k_rows, const float *v_rows)
{
    if (!c || !k_rows || !v_rows)
        return L2J_E_INVALID;
    std::lock_guard<std::mutex> lock(c->mu);
    const int li = layer - c->first_layer;
    if (li < 0 || li >= c->nl || pos0 < 0 || n_pos <= 0 || pos0 + n_pos > c->cfg.seq_len)
        return fail(c, L2J_E_INVALID, "KV rows [%d, %d) of layer %d outside this context", pos0, pos0 + n_pos, layer);
    if (c->tp_size > 1)
        return fail(c, L2J_E_STATE, "a tensor-parallel rank holds only its own heads of the cache");
    CK(c, cudaSetDevice(c->device));
    CK(c, cudaStreamSynchronize(c->stream));
    const int64_t layer_floats = (int64_t)c->cfg.n_kv_heads * c->cfg.seq_len * c->head;
    const int piece = 256;   // positions per staging copy
    float *stage = nullptr;
    cudaError_t e = cudaMalloc((void **)&stage, sizeof(float) * (size_t)piece * c->kv_dim);
    if (e != cudaSuccess)
        return fail(c, L2J_E_NOMEM, "staging allocation failed: %s", cudaGetErrorString(e));
    int rc = L2J_OK;
    for (int which = 0; which < 2 && rc == L2J_OK; ++which) {
        const float *src = which ? v_rows : k_rows;
        float *dst = (which ? c->vc : c->kc) + li * layer_floats;
        for (int done = 0; done < n_pos && rc == L2J_OK; done += piece) {
            const int np = n_pos - done < piece ? n_pos - done : piece;
            e = cudaMemcpyAsync(stage, src + (int64_t)done * c->kv_dim, sizeof(float) * (size_t)np * c->kv_dim,
                                cudaMemcpyHostToDevice, c->stream);
            if (e == cudaSuccess)
                e = launch_kv_relayout(c->stream, stage, dst + (int64_t)(pos0 + done) * c->head, c->cfg.n_kv_heads, c->head,
                                       c->cfg.seq_len, np);
            if (e == cudaSuccess)
                e = cudaStreamSynchronize(c->stream);
            if (e != cudaSuccess)
                rc = fail(c, L2J_E_CUDA, "KV restore failed: %s", cudaGetErrorString(e));
        }
    }
    cudaFree(stage);
    return rc;
}

// ===============================================================================================
// layer split over several devices driven by one host thread (Run.java:368-413)
// ===============================================================================================

namespace {

int check_stages(l2j_ctx *const *stages, int n, bool need_link = false)
{
    if (!stages || n <= 0)
        return L2J_E_INVALID;
    for (int i = 0; i < n; ++i)
        if (!stages[i])
            return L2J_E_INVALID;
    l2j_ctx *c0 = stages[0];
    for (int i = 0; i < n; ++i) {
        l2j_ctx *c = stages[i];
        if (!c->finalized)
            return fail(c0, L2J_E_STATE, "stage %d is not finalized", i);
        if (memcmp(&c->cfg, &c0->cfg, sizeof(l2j_config)) != 0)
            return fail(c0, L2J_E_INVALID, "stage %d was created for another model", i);
        if ((i == 0) != c->is_first || (i == n - 1) != c->is_last || (i > 0 && c->first_layer != stages[i - 1]->last_layer + 1))
            return fail(c0, L2J_E_INVALID, "the stages do not tile the layers in order (stage %d holds %d..%d)", i,
                        c->first_layer, c->last_layer);
    }
    if (need_link && n > 1) {
        // The begin kernel of a stage reads its neighbour's memory through pointers that l2j_pipeline_link wrote:
        // without the link (or after a member was destroyed or linked elsewhere) they are null or stale.
        std::lock_guard<std::mutex> lock(g_link_mu);
        for (int i = 0; i < n; ++i) {
            const std::vector<l2j_ctx *> &m = stages[i]->pipe_members;
            bool same = (int)m.size() == n;
            for (int j = 0; same && j < n; ++j)
                same = m[(size_t)j] == stages[j];
            if (!same)
                return fail(c0, L2J_E_STATE, "stage %d is not linked with these stages: call l2j_pipeline_link first", i);
        }
    }
    return L2J_OK;
}

// Stage i's stream waits for stage i-1's step, then runs its own; the hand-off itself is the peer read
// in the stage's begin kernel.
int enqueue_stage(l2j_ctx *const *stages, int n, int i, int pos)
{
    l2j_ctx *c = stages[i];
    CK(c, cudaSetDevice(c->device));
    if (n > 1)
        CK(c, cudaStreamWaitEvent(c->stream, stages[(i + n - 1) % n]->ev_stage, 0));
    int rc = launch_forward(c, pos);
    if (rc != L2J_OK)
        return rc;
    CK(c, cudaEventRecord(c->ev_stage, c->stream));
    return L2J_OK;
}

}  // namespace

extern "C" int l2j_pipeline_link(l2j_ctx *const *stages, int n_stages)
{
    int rc = check_stages(stages, n_stages);
    if (rc != L2J_OK)
        return rc;
    for (int i = 0; i < n_stages; ++i) {
        l2j_ctx *c = stages[i];
        std::lock_guard<std::mutex> lock(c->mu);
        l2j_ctx *prev = stages[(i + n_stages - 1) % n_stages];   // stage 0 reads the token from the last stage
        CK(c, cudaSetDevice(c->device));
        if (prev->device != c->device) {
            int can = 0;
            CK(c, cudaDeviceCanAccessPeer(&can, c->device, prev->device));
            if (!can)
                return fail(stages[0], L2J_E_STATE, "device %d cannot read the memory of device %d", c->device, prev->device);
            cudaError_t e = cudaDeviceEnablePeerAccess(prev->device, 0);
            if (e == cudaErrorPeerAccessAlreadyEnabled)
                cudaGetLastError();
            else
                CK(c, e);
        }
        StageLink link{};
        link.x_src = i > 0 ? prev->x : nullptr;
        link.token_src = i == 0 && n_stages > 1 ? &prev->state->token : nullptr;
        CK(c, cudaMemcpy(c->link_dev, &link, sizeof(StageLink), cudaMemcpyHostToDevice));
        // an event recorded once, so that the first wait of the ring of stages finds it complete
        CK(c, cudaEventRecord(c->ev_stage, c->stream));
        CK(c, cudaStreamSynchronize(c->stream));
    }
    {
        std::lock_guard<std::mutex> lock(g_link_mu);
        for (int i = 0; i < n_stages; ++i) {
            // a stage that was linked elsewhere leaves that group: its old partners hold pointers it no longer serves
            for (l2j_ctx *old : stages[i]->pipe_members)
                if (old != stages[i])
                    old->pipe_members.clear();
            stages[i]->pipe_members.assign(stages, stages + n_stages);
        }
    }
    return L2J_OK;
}

extern "C" int l2j_pipeline_forward(l2j_ctx *const *stages, int n_stages, int token, int pos, float *logits, int *argmax)
{
    int rc = check_stages(stages, n_stages, true);
    if (rc != L2J_OK)
        return rc;
    rc = check_range(stages[0], token, pos, true);
    if (rc != L2J_OK)
        return rc;
    for (int i = 0; i < n_stages; ++i) {
        l2j_ctx *c = stages[i];
        std::lock_guard<std::mutex> lock(c->mu);
        CK(c, cudaSetDevice(c->device));
        rc = post_cmd(c, 1, i == 0 ? token : 0, pos, i > 0 ? kCmdXFromPeer : 0);
        if (rc != L2J_OK)
            return rc;
        if (i > 0)
            CK(c, cudaStreamWaitEvent(c->stream, stages[i - 1]->ev_stage, 0));
        rc = launch_forward(c, pos);
        if (rc != L2J_OK)
            return rc;
        CK(c, cudaEventRecord(c->ev_stage, c->stream));
    }
    int status = L2J_OK;
    for (int i = 0; i < n_stages; ++i) {   // every stage's status word is checked
        l2j_ctx *c = stages[i];
        std::lock_guard<std::mutex> lock(c->mu);
        CK(c, cudaSetDevice(c->device));
        if (c->is_last && logits)
            CK(c, cudaMemcpyAsync(c->logits_host, c->logits, sizeof(float) * (size_t)c->cfg.vocab_size, cudaMemcpyDeviceToHost,
                                  c->stream));
        CK(c, cudaMemcpyAsync(c->state_host, c->state, sizeof(SeqState), cudaMemcpyDeviceToHost, c->stream));
        CK(c, cudaStreamSynchronize(c->stream));
        if (c->is_last && logits)
            memcpy(logits, c->logits_host, sizeof(float) * (size_t)c->cfg.vocab_size);
        if (c->is_last && argmax)
            *argmax = c->state_host->argmax;
        const int r = finish_status(c);
        if (r != L2J_OK && status == L2J_OK) {
            status = r;
            if (c != stages[0])
                fail(stages[0], r, "stage %d: %s", i, c->err.c_str());
        }
    }
    return status;
}

extern "C" int l2j_pipeline_generate_greedy(l2j_ctx *const *stages, int n_stages, const int32_t *prompt, int n_prompt, int steps,
                                            int32_t *out_tokens)
{
    int rc = check_stages(stages, n_stages, true);
    if (rc != L2J_OK)
        return rc;
    l2j_ctx *c0 = stages[0], *cl = stages[n_stages - 1];
    if (steps <= 0 || steps > c0->cfg.seq_len || n_prompt < 0 || n_prompt > c0->cfg.seq_len || (n_prompt > 0 && !prompt) ||
        !out_tokens)
        return fail(c0, L2J_E_INVALID, "bad arguments: steps %d (seq_len %d), n_prompt %d", steps, c0->cfg.seq_len, n_prompt);
    for (int i = 0; i < n_prompt; ++i)
        if (prompt[i] < 0 || prompt[i] >= c0->cfg.vocab_size)
            return fail(c0, L2J_E_INVALID, "prompt token %d outside the vocabulary", prompt[i]);
    for (int i = 0; i < n_stages; ++i) {
        l2j_ctx *c = stages[i];
        std::lock_guard<std::mutex> lock(c->mu);
        CK(c, cudaSetDevice(c->device));
        if (c->is_last && n_prompt > 0)
            CK(c, cudaMemcpyAsync(c->prompt_dev, prompt, sizeof(int32_t) * (size_t)n_prompt, cudaMemcpyHostToDevice, c->stream));
        SeqState init{};
        init.token = 1;   // BOS, Run.java:614
        init.pos = 0;
        init.n_prompt = n_prompt;
        CK(c, cudaMemcpyAsync(c->state, &init, sizeof(SeqState), cudaMemcpyHostToDevice, c->stream));
        CK(c, cudaStreamSynchronize(c->stream));
        const int flags = (i > 0 ? kCmdXFromPeer : 0) | (i == 0 && n_stages > 1 ? kCmdTokenFromPeer : 0) |
                          (!c->is_last ? kCmdAdvancePos : 0);
        rc = post_cmd(c, 0, 0, 0, flags);
        if (rc != L2J_OK)
            return rc;
        CK(c, cudaEventRecord(c->ev_stage, c->stream));   // complete before the loop starts
        CK(c, cudaStreamSynchronize(c->stream));
    }
    CK(c0, cudaSetDevice(c0->device));
    CK(c0, cudaEventRecord(c0->ev0, c0->stream));
    for (int s = 0; s < steps; ++s)
        for (int i = 0; i < n_stages; ++i) {
            // step s of stage 0 waits for step s-1 of the last stage: it reads the chosen token there
            rc = enqueue_stage(stages, n_stages, i, s);
            if (rc != L2J_OK)
                return rc;
        }
    CK(c0, cudaSetDevice(c0->device));
    if (n_stages > 1)
        CK(c0, cudaStreamWaitEvent(c0->stream, cl->ev_stage, 0));
    CK(c0, cudaEventRecord(c0->ev1, c0->stream));
    int status = L2J_OK;
    for (int i = 0; i < n_stages; ++i) {
        l2j_ctx *c = stages[i];
        CK(c, cudaSetDevice(c->device));
        CK(c, cudaMemcpyAsync(c->state_host, c->state, sizeof(SeqState), cudaMemcpyDeviceToHost, c->stream));
        CK(c, cudaStreamSynchronize(c->stream));
        const int r = finish_status(c);
        if (r != L2J_OK && status == L2J_OK) {
            status = r;
            if (c != c0)
                fail(c0, r, "stage %d: %s", i, c->err.c_str());
        }
    }
    CK(cl, cudaSetDevice(cl->device));
    CK(cl, cudaMemcpy(out_tokens, cl->out_tokens_dev, sizeof(int32_t) * (size_t)steps, cudaMemcpyDeviceToHost));
    float ms = 0.f;
    CK(c0, cudaSetDevice(c0->device));
    CK(c0, cudaEventElapsedTime(&ms, c0->ev0, c0->ev1));
    c0->last_generate_us = (double)ms * 1000.0;
    return status;
}

// ===============================================================================================
// tensor-parallel group driven by one host thread
// ===============================================================================================

namespace {

int check_tp_group(l2j_ctx *const *ranks, int n, bool need_link)
{
    if (!ranks || n <= 0 || n > kMaxTp)
        return L2J_E_INVALID;
    for (int i = 0; i < n; ++i)
        if (!ranks[i])
            return L2J_E_INVALID;
    l2j_ctx *c0 = ranks[0];
    for (int i = 0; i < n; ++i) {
        l2j_ctx *c = ranks[i];
        if (!c->finalized)
            return fail(c0, L2J_E_STATE, "rank %d is not finalized", i);
        if (memcmp(&c->cfg, &c0->cfg, sizeof(l2j_config)) != 0)
            return fail(c0, L2J_E_INVALID, "rank %d was created for another model", i);
        if (c->tp_size != n || c->tp_rank != i || !(c->is_first && c->is_last))
            return fail(c0, L2J_E_INVALID, "context %d is rank %d of %d, expected rank %d of %d", i, c->tp_rank, c->tp_size, i, n);
        if (!c->use_ring || !c->chain_on)
            return fail(c0, L2J_E_STATE, "a tensor-parallel group needs the ring kernels and the hand-over counters");
        for (int j = 0; j < i; ++j)
            if (ranks[j]->device == c->device)
                return fail(c0, L2J_E_INVALID, "ranks %d and %d share device %d: kernels that wait for each other need a device each",
                            j, i, c->device);
        if (need_link && n > 1 && !c->tp_linked)
            return fail(c0, L2J_E_STATE, "the group is not linked (l2j_tp_link)");
    }
    return L2J_OK;
}

}  // namespace

extern "C" int l2j_tp_link(l2j_ctx *const *ranks, int n_ranks)
{
    int rc = check_tp_group(ranks, n_ranks, false);
    if (rc != L2J_OK)
        return rc;
    for (int i = 0; i < n_ranks; ++i) {
        l2j_ctx *c = ranks[i];
        std::lock_guard<std::mutex> lock(c->mu);
        CK(c, cudaSetDevice(c->device));
        TpTable t{};
        t.n = n_ranks;
        t.rank = i;
        for (int j = 0; j < n_ranks; ++j) {
            l2j_ctx *o = ranks[j];
            if (j != i) {
                int can = 0;
                CK(c, cudaDeviceCanAccessPeer(&can, c->device, o->device));
                if (!can)
                    return fail(ranks[0], L2J_E_STATE, "device %d cannot reach the memory of device %d", c->device, o->device);
                cudaError_t e = cudaDeviceEnablePeerAccess(o->device, 0);
                if (e == cudaErrorPeerAccessAlreadyEnabled)
                    cudaGetLastError();
                else
                    CK(c, e);
            }
            for (int v = 0; v < TPV_COUNT; ++v)
                t.ll[v][j] = o->ll_buf[v];
        }
        CK(c, cudaMemcpy(c->tp_dev, &t, sizeof(TpTable), cudaMemcpyHostToDevice));
        CK(c, cudaDeviceSynchronize());
        c->tp_linked = true;
    }
    return L2J_OK;
}

extern "C" int l2j_tp_forward(l2j_ctx *const *ranks, int n_ranks, int token, int pos, float *logits, int *argmax)
{
    int rc = check_tp_group(ranks, n_ranks, true);
    if (rc != L2J_OK)
        return rc;
    rc = check_range(ranks[0], token, pos, true);
    if (rc != L2J_OK)
        return rc;
    // every rank's kernels wait (bounded) for the other ranks' kernels: put all of them on their way first
    for (int i = 0; i < n_ranks; ++i) {
        l2j_ctx *c = ranks[i];
        std::lock_guard<std::mutex> lock(c->mu);
        CK(c, cudaSetDevice(c->device));
        rc = post_cmd(c, 1, token, pos);
        if (rc != L2J_OK)
            return rc;
    }
    for (int i = 0; i < n_ranks; ++i) {
        l2j_ctx *c = ranks[i];
        CK(c, cudaSetDevice(c->device));
        rc = launch_forward(c, pos);
        if (rc != L2J_OK)
            return rc;
    }
    int status = L2J_OK;
    const int vocab = ranks[0]->cfg.vocab_size;
    for (int i = 0; i < n_ranks; ++i) {
        l2j_ctx *c = ranks[i];
        CK(c, cudaSetDevice(c->device));
        // the whole logits from rank 0, or every rank's block of the vocabulary
        const int first = c->cls_split ? i * (vocab / n_ranks) : 0;
        const int count = c->cls_split ? vocab / n_ranks : (i == 0 ? vocab : 0);
        if (logits && count > 0)
            CK(c, cudaMemcpyAsync(c->logits_host + first, c->logits + first, sizeof(float) * (size_t)count, cudaMemcpyDeviceToHost,
                                  c->stream));
        CK(c, cudaMemcpyAsync(c->state_host, c->state, sizeof(SeqState), cudaMemcpyDeviceToHost, c->stream));
        CK(c, cudaStreamSynchronize(c->stream));
        if (logits && count > 0)
            memcpy(logits + first, c->logits_host + first, sizeof(float) * (size_t)count);
        if (i == 0 && argmax)
            *argmax = c->state_host->argmax;
        const int r = finish_status(c);
        if (r != L2J_OK && status == L2J_OK) {
            status = r;
            if (c != ranks[0])
                fail(ranks[0], r, "rank %d: %s", i, c->err.c_str());
        }
    }
    return status;
}

extern "C" int l2j_tp_generate_greedy(l2j_ctx *const *ranks, int n_ranks, const int32_t *prompt, int n_prompt, int steps,
                                      int32_t *out_tokens)
{
    int rc = check_tp_group(ranks, n_ranks, true);
    if (rc != L2J_OK)
        return rc;
    l2j_ctx *c0 = ranks[0];
    if (steps <= 0 || steps > c0->cfg.seq_len || n_prompt < 0 || n_prompt > c0->cfg.seq_len || (n_prompt > 0 && !prompt) ||
        !out_tokens)
        return fail(c0, L2J_E_INVALID, "bad arguments: steps %d (seq_len %d), n_prompt %d", steps, c0->cfg.seq_len, n_prompt);
    for (int i = 0; i < n_prompt; ++i)
        if (prompt[i] < 0 || prompt[i] >= c0->cfg.vocab_size)
            return fail(c0, L2J_E_INVALID, "prompt token %d outside the vocabulary", prompt[i]);
    // every rank runs the whole greedy loop on its own device: the classifier is replicated, so all ranks
    // choose the same token from bitwise equal logits
    for (int i = 0; i < n_ranks; ++i) {
        l2j_ctx *c = ranks[i];
        std::lock_guard<std::mutex> lock(c->mu);
        CK(c, cudaSetDevice(c->device));
        if (n_prompt > 0)
            CK(c, cudaMemcpyAsync(c->prompt_dev, prompt, sizeof(int32_t) * (size_t)n_prompt, cudaMemcpyHostToDevice, c->stream));
        SeqState init{};
        init.token = 1;   // BOS, Run.java:614
        init.pos = 0;
        init.n_prompt = n_prompt;
        CK(c, cudaMemcpyAsync(c->state, &init, sizeof(SeqState), cudaMemcpyHostToDevice, c->stream));
        rc = post_cmd(c, 0, 0, 0);
        if (rc != L2J_OK)
            return rc;
        CK(c, cudaStreamSynchronize(c->stream));
    }
    CK(c0, cudaSetDevice(c0->device));
    CK(c0, cudaEventRecord(c0->ev0, c0->stream));
    for (int s = 0; s < steps; ++s)
        for (int i = 0; i < n_ranks; ++i) {
            l2j_ctx *c = ranks[i];
            CK(c, cudaSetDevice(c->device));
            rc = launch_forward(c, s);
            if (rc != L2J_OK)
                return rc;
        }
    CK(c0, cudaSetDevice(c0->device));
    CK(c0, cudaEventRecord(c0->ev1, c0->stream));
    int status = L2J_OK;
    for (int i = 0; i < n_ranks; ++i) {
        l2j_ctx *c = ranks[i];
        CK(c, cudaSetDevice(c->device));
        CK(c, cudaMemcpyAsync(c->state_host, c->state, sizeof(SeqState), cudaMemcpyDeviceToHost, c->stream));
        CK(c, cudaStreamSynchronize(c->stream));
        const int r = finish_status(c);
        if (r != L2J_OK && status == L2J_OK) {
            status = r;
            if (c != c0)
                fail(c0, r, "rank %d: %s", i, c->err.c_str());
        }
    }
    CK(c0, cudaSetDevice(c0->device));
    CK(c0, cudaMemcpy(out_tokens, c0->out_tokens_dev, sizeof(int32_t) * (size_t)steps, cudaMemcpyDeviceToHost));
    float ms = 0.f;
    CK(c0, cudaEventElapsedTime(&ms, c0->ev0, c0->ev1));
    c0->last_generate_us = (double)ms * 1000.0;
    return status;
}

extern "C" int l2j_last_generate_us(l2j_ctx *c, double *total_us)
{
    if (!c || !total_us)
        return L2J_E_INVALID;
    *total_us = c->last_generate_us;
    return L2J_OK;
}

extern "C" int l2j_reset(l2j_ctx *c)
{
    if (!c)
        return L2J_E_INVALID;
    std::lock_guard<std::mutex> lock(c->mu);
    CK(c, cudaSetDevice(c->device));
    CK(c, cudaStreamSynchronize(c->stream));
    CK(c, cudaMemset(c->state, 0, sizeof(SeqState)));
    CK(c, cudaMemset(c->attn_counters, 0, sizeof(unsigned int) * (size_t)c->cfg.n_heads));
    CK(c, cudaMemset(c->work, 0, sizeof(unsigned int) * 2 * (4 * (size_t)c->nl + 1)));
    CK(c, cudaMemset(c->chain, 0, sizeof(unsigned int) * kChainStride * (5 * (size_t)c->nl + 2)));   // the epoch word too
    if (c->tp_size > 1) {   // the sequence numbers start again: no old pair may match a new one
        CK(c, cudaMemset(c->ll_buf[TPV_X], 0, sizeof(float2) * (size_t)c->dim));
        CK(c, cudaMemset(c->ll_buf[TPV_XB], 0, sizeof(float2) * (size_t)c->dim));
        CK(c, cudaMemset(c->ll_buf[TPV_HB], 0, sizeof(float2) * (size_t)c->hidden));
        CK(c, cudaMemset(c->ll_buf[TPV_CAND], 0, sizeof(float2) * 2 * kMaxTp));
    }
    CK(c, cudaDeviceSynchronize());
    c->forwards = 0;
    c->status_accum = 0;
    c->err.clear();
    return L2J_OK;
}

extern "C" int l2j_tp_reset(l2j_ctx *const *ranks, int n_ranks)
{
    if (!ranks || n_ranks <= 0)
        return L2J_E_INVALID;
    int rc = L2J_OK;
    for (int i = 0; i < n_ranks; ++i) {   // every member, also after a failure: the group's counters must agree again
        const int r = l2j_reset(ranks[i]);
        if (r != L2J_OK && rc == L2J_OK)
            rc = r;
    }
    return rc;
}

extern "C" int l2j_pipeline_reset(l2j_ctx *const *stages, int n_stages)
{
    return l2j_tp_reset(stages, n_stages);
}

extern "C" int l2j_set_wait_limit_us(l2j_ctx *c, int limit_us)
{
    if (!c)
        return L2J_E_INVALID;
    std::lock_guard<std::mutex> lock(c->mu);
    if (limit_us < 10 || limit_us > 10000000)
        return fail(c, L2J_E_INVALID, "wait limit %d us outside [10, 10000000]", limit_us);
    if (c->finalized)
        return fail(c, L2J_E_STATE, "the wait limit is part of the captured launches: set it before l2j_finalize");
    c->wait_limit_us = limit_us;
    return L2J_OK;
}

extern "C" int l2j_debug_desync(l2j_ctx *c)
{
    if (!c)
        return L2J_E_INVALID;
    std::lock_guard<std::mutex> lock(c->mu);
    if (!c->finalized || !c->use_ring || !c->chain_on)
        return fail(c, L2J_E_STATE, "needs a finalized context that runs the hand-over counters");
    CK(c, cudaSetDevice(c->device));
    CK(c, cudaStreamSynchronize(c->stream));
    // The forward counter on the device runs one ahead of the hand-over counters, as after a forward that a
    // partner never ran: the next forward's kernels wait for bumps that nobody makes.
    unsigned int *epoch = c->chain + (int64_t)kChainStride * (5 * c->nl + 1);
    unsigned int v = 0;
    CK(c, cudaMemcpy(&v, epoch, sizeof(v), cudaMemcpyDeviceToHost));
    ++v;
    CK(c, cudaMemcpy(epoch, &v, sizeof(v), cudaMemcpyHostToDevice));
    return L2J_OK;
}

extern "C" int l2j_get_stats(l2j_ctx *c, l2j_stats *out)
{
    if (!c || !out)
        return L2J_E_INVALID;
    out->forwards = c->forwards;
    out->kernels_per_forward = c->kernels_per_forward;
    out->device_bytes = c->device_bytes;
    out->device_status = c->status_accum;
    out->last_pos = c->state_host ? c->state_host->cur_pos : 0;
    out->last_token = c->state_host ? c->state_host->argmax : 0;
    out->sm_count = c->sm_count;
    return L2J_OK;
}

extern "C" int l2j_time_kernels(l2j_ctx *c, int pos, int reps, double *us)
{
    if (!c || !us || reps <= 0)
        return L2J_E_INVALID;
    std::lock_guard<std::mutex> lock(c->mu);
    if (!c->finalized || !c->use_ring || c->tp_size > 1)
        return fail(c, L2J_E_STATE, "kernel timing needs a finalized context on the ring kernels that holds all rows");
    int rc = check_range(c, 1, pos, true);
    if (rc != L2J_OK)
        return rc;
    CK(c, cudaSetDevice(c->device));
    rc = post_cmd(c, 1, 1, pos);
    if (rc != L2J_OK)
        return rc;
    LaunchCfg lc{c->stream, false, c->ring_grid};
    CK(c, launch_begin(lc, c->state, c->cmd_dev, c->emb, c->x, c->dim, c->cfg.vocab_size, c->cfg.seq_len, c->is_first ? 1 : 0, c->reps, c->dim_stride, nullptr, c->link_dev));
    for (int kind = 0; kind < 6; ++kind) {
        us[kind] = 0.0;
        if (kind == 5 && !c->is_last)
            continue;
        int launches = 0;
        for (int phase = 0; phase < 2; ++phase) {   // phase 0 warms up, phase 1 is timed
            if (phase == 1)
                CK(c, cudaEventRecord(c->ev0, c->stream));
            const int sweeps = phase == 0 ? 1 : reps;
            for (int r = 0; r < sweeps; ++r) {
                const int n = kind == 5 ? 1 : c->nl;
                for (int li = 0; li < n; ++li) {
                    LayerLaunch &L = c->layers[(size_t)(kind == 5 ? 0 : li)];
                    cudaError_t e = cudaSuccess;
                    switch (kind) {
                    case 0: e = launch_matvec_ring(lc, c->plan_qkv, false, unchained(L.qkv)); break;
                    case 1: e = launch_attention(lc, unchained(pos >= kLongContextPos ? L.attn_long : L.attn)); break;
                    case 2: e = launch_matvec_ring(lc, c->plan_wo, false, unchained(L.wo)); break;
                    case 3: e = launch_matvec_ring(lc, c->plan_w13, false, unchained(L.w13)); break;
                    case 4: e = launch_matvec_ring(lc, c->plan_hidden, false, unchained(L.w2)); break;
                    default: e = launch_matvec_ring(lc, c->plan_cls, true, unchained(c->cls)); break;
                    }
                    CK(c, e);
                    if (phase == 1)
                        ++launches;
                }
            }
        }
        CK(c, cudaEventRecord(c->ev1, c->stream));
        CK(c, cudaEventSynchronize(c->ev1));
        float ms = 0.f;
        CK(c, cudaEventElapsedTime(&ms, c->ev0, c->ev1));
        us[kind] = launches > 0 ? (double)ms * 1000.0 / launches : 0.0;
    }
    CK(c, cudaStreamSynchronize(c->stream));
    return L2J_OK;
}

extern "C" int l2j_time_layers_kernel(l2j_ctx *c, int pos, int reps, double *us_per_launch)
{
    if (!c || !us_per_launch || reps <= 0)
        return L2J_E_INVALID;
    std::lock_guard<std::mutex> lock(c->mu);
    if (!c->finalized || !c->use_fused)
        return fail(c, L2J_E_STATE, "needs a finalized context that runs the persistent kernel");
    int rc = check_range(c, 1, pos, true);
    if (rc != L2J_OK)
        return rc;
    CK(c, cudaSetDevice(c->device));
    LaunchCfg lc{c->stream, false, c->ring_grid};
    double total_ms = 0.0;
    for (int r = 0; r <= reps; ++r) {   // the first pass warms up
        rc = post_cmd(c, 1, 1, pos);
        if (rc != L2J_OK)
            return rc;
        CK(c, launch_begin(lc, c->state, c->cmd_dev, c->emb, c->x, c->dim, c->cfg.vocab_size, c->cfg.seq_len, c->is_first ? 1 : 0,
                           c->reps, c->dim_stride, c->chain + (int64_t)kChainStride * (5 * c->nl + 1), c->link_dev));
        CK(c, cudaEventRecord(c->ev0, c->stream));
        CK(c, launch_fused(c->stream, false, c->ring_grid, c->fused_smem, c->fused));
        CK(c, cudaEventRecord(c->ev1, c->stream));
        CK(c, cudaEventSynchronize(c->ev1));
        c->forwards++;
        float ms = 0.f;
        CK(c, cudaEventElapsedTime(&ms, c->ev0, c->ev1));
        if (r > 0)
            total_ms += ms;
    }
    *us_per_launch = total_ms * 1000.0 / reps;
    return L2J_OK;
}

extern "C" int l2j_read_trace(l2j_ctx *c, uint64_t *out, int64_t max_values)
{
    if (!c || !out || max_values <= 0)
        return L2J_E_INVALID;
    std::lock_guard<std::mutex> lock(c->mu);
    if (!c->trace)
        return fail(c, L2J_E_STATE, "the context was created without L2J_TRACE in the environment");
    CK(c, cudaSetDevice(c->device));
    CK(c, cudaStreamSynchronize(c->stream));
    if (c->use_fused && c->fused_trace) {   // [block][5 * layers][8] marks of the persistent kernel's last launch
        int64_t nf = (int64_t)c->ring_grid * 5 * c->nl * 8;
        if (nf > max_values)
            nf = max_values;
        CK(c, cudaMemcpy(out, c->fused_trace, sizeof(uint64_t) * (size_t)nf, cudaMemcpyDeviceToHost));
        return L2J_OK;
    }
    int64_t n = (5 * (int64_t)c->nl + 1) * c->ring_grid * 16;
    if (n > max_values)
        n = max_values;
    CK(c, cudaMemcpy(out, c->trace, sizeof(uint64_t) * (size_t)n, cudaMemcpyDeviceToHost));
    return L2J_OK;
}

extern "C" int l2j_trace_kernel(l2j_ctx *c, int kind, int layer, int pos, uint64_t *out, int max_blocks)
{
    if (!c || !out || kind < 0 || kind > 5 || kind == 1 || max_blocks <= 0)
        return L2J_E_INVALID;
    std::lock_guard<std::mutex> lock(c->mu);
    if (!c->finalized || !c->use_ring || c->tp_size > 1)
        return fail(c, L2J_E_STATE, "kernel tracing needs a finalized context on the ring kernels that holds all rows");
    const int li = layer - c->first_layer;
    if (li < 0 || li >= c->nl || (kind == 5 && !c->is_last))
        return fail(c, L2J_E_INVALID, "layer %d is not held by this context", layer);
    int rc = check_range(c, 1, pos, true);
    if (rc != L2J_OK)
        return rc;
    CK(c, cudaSetDevice(c->device));
    unsigned long long *dtrace = nullptr;
    const int nb = c->ring_grid;
    CK(c, cudaMalloc((void **)&dtrace, sizeof(unsigned long long) * 16 * (size_t)nb));
    cudaMemset(dtrace, 0, sizeof(unsigned long long) * 16 * (size_t)nb);
    cudaDeviceSynchronize();
    rc = post_cmd(c, 1, 1, pos);
    LaunchCfg lc{c->stream, false, c->ring_grid};
    cudaError_t e = launch_begin(lc, c->state, c->cmd_dev, c->emb, c->x, c->dim, c->cfg.vocab_size, c->cfg.seq_len, c->is_first ? 1 : 0, c->reps, c->dim_stride, nullptr, c->link_dev);
    LayerLaunch &L = c->layers[(size_t)li];
    for (int rep = 0; rep < 2 && e == cudaSuccess; ++rep) {   // the second launch is the one recorded
        MvParams p = kind == 0 ? L.qkv : kind == 2 ? L.wo : kind == 3 ? L.w13 : kind == 4 ? L.w2 : c->cls;
        const MvPlan &pl = kind == 4 ? c->plan_hidden : kind == 5 ? c->plan_cls : kind == 2 ? c->plan_wo : kind == 3 ? c->plan_w13 : c->plan_qkv;
        p.trace = rep == 1 ? dtrace : nullptr;
        if (rep == 1 && c->nl > 1 && kind != 5) {   // another layer's weights, so nothing is warm in L2
            LayerLaunch &L2 = c->layers[(size_t)((li + 1) % c->nl)];
            MvParams q = kind == 0 ? L2.qkv : kind == 2 ? L2.wo : kind == 3 ? L2.w13 : L2.w2;
            q.trace = dtrace;
            p = q;
        }
        e = launch_matvec_ring(lc, pl, kind == 5, unchained(p));
    }
    if (e == cudaSuccess)
        e = cudaStreamSynchronize(c->stream);
    const int n = nb < max_blocks ? nb : max_blocks;
    if (e == cudaSuccess)
        e = cudaMemcpy(out, dtrace, sizeof(unsigned long long) * 16 * (size_t)n, cudaMemcpyDeviceToHost);
    cudaFree(dtrace);
    if (e != cudaSuccess)
        return fail(c, L2J_E_CUDA, "trace failed: %s", cudaGetErrorString(e));
    return rc;
}

// Flags that describe how the per-token work is issued (bit 0: CUDA graph, bit 1: programmatic
// dependent launch, bit 2: ring kernels), for reports.
extern "C" int l2j_launch_mode(l2j_ctx *c)
{
    if (!c)
        return 0;
    return (c->exec ? 1 : 0) | (c->pdl_on ? 2 : 0) | (c->use_ring ? 4 : 0) | (c->use_fused ? 8 : 0) | (c->ring_grid << 8);
}

// Reads an internal buffer after a forward (debugging and per-stage parity checks):
// 0 x, 1 attention output (xb), 2 q, 3 hb, 4 logits, 5 K row (layer, pos), 6 V row (layer, pos)
// in the reference's (kv_dim) order.
extern "C" int l2j_read_buffer(l2j_ctx *c, int which, int layer, int pos, float *out, int n)
{
    if (!c || !out || n <= 0)
        return L2J_E_INVALID;
    std::lock_guard<std::mutex> lock(c->mu);
    CK(c, cudaSetDevice(c->device));
    CK(c, cudaStreamSynchronize(c->stream));
    const float *src = nullptr;
    int len = 0;
    switch (which) {
    case 0: src = c->x; len = c->dim; break;
    case 1: src = c->xb; len = c->dim; break;
    case 2: src = c->q; len = c->dim; break;
    case 3: src = c->hb; len = c->hidden; break;
    case 4: src = c->logits; len = c->cfg.vocab_size; break;
    case 5:
    case 6: {
        const int li = layer - c->first_layer;
        if (li < 0 || li >= c->nl || pos < 0 || pos >= c->cfg.seq_len || n != c->kv_dim)
            return fail(c, L2J_E_INVALID, "bad KV row request");
        const float *base = (which == 5 ? c->kc : c->vc) + (int64_t)li * c->cfg.n_kv_heads * c->cfg.seq_len * c->head;
        for (int h = 0; h < c->cfg.n_kv_heads; ++h)
            CK(c, cudaMemcpy(out + (int64_t)h * c->head, base + ((int64_t)h * c->cfg.seq_len + pos) * c->head,
                             sizeof(float) * (size_t)c->head, cudaMemcpyDeviceToHost));
        return L2J_OK;
    }
    default: return fail(c, L2J_E_INVALID, "unknown buffer %d", which);
    }
    if (n > len)
        return fail(c, L2J_E_INVALID, "buffer %d holds %d floats", which, len);
    if (c->tp_size > 1 && (which == 1 || which == 3)) {
        // these vectors exist only as (value, sequence number) pairs in the receive buffers
        std::vector<float2> pairs((size_t)n);
        CK(c, cudaMemcpy(pairs.data(), c->ll_buf[which == 1 ? TPV_XB : TPV_HB], sizeof(float2) * (size_t)n, cudaMemcpyDeviceToHost));
        for (int i = 0; i < n; ++i)
            out[i] = pairs[(size_t)i].x;
        return L2J_OK;
    }
    CK(c, cudaMemcpy(out, src, sizeof(float) * (size_t)n, cudaMemcpyDeviceToHost));
    return L2J_OK;
}

// ===============================================================================================
// load-time helpers and single-kernel entry points
// ===============================================================================================

namespace {

struct Scratch {   // device allocations of a one-shot entry point, freed on scope exit
    std::vector<void *> ptrs;
    ~Scratch()
    {
        for (void *p : ptrs)
            cudaFree(p);
    }
    template <typename T>
    cudaError_t alloc(T **out, int64_t count, bool zero = false)
    {
        void *p = nullptr;
        const size_t bytes = (size_t)(count > 0 ? count : 1) * sizeof(T);
        cudaError_t e = cudaMalloc(&p, bytes);
        if (e != cudaSuccess)
            return e;
        ptrs.push_back(p);
        if (zero)
            e = cudaMemset(p, 0, bytes);
        *out = static_cast<T *>(p);
        return e;
    }
};

#define KCK(call)                                                                                      \
    do {                                                                                               \
        cudaError_t e__ = (call);                                                                      \
        if (e__ != cudaSuccess)                                                                        \
            return fail(nullptr, L2J_E_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__),  \
                        __FILE__, __LINE__);                                                           \
    } while (0)

int set_device_checked(int device)
{
    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess || ndev <= 0)
        return fail(nullptr, L2J_E_CUDA, "no CUDA device: %s (this library has no CPU path)", cudaGetErrorString(e));
    if (device < 0 || device >= ndev)
        return fail(nullptr, L2J_E_INVALID, "device %d not present", device);
    KCK(cudaSetDevice(device));
    KCK(prepare_kernels());
    return L2J_OK;
}

int status_of(SeqState *dev_state)
{
    SeqState h{};
    KCK(cudaMemcpy(&h, dev_state, sizeof(SeqState), cudaMemcpyDeviceToHost));
    if (h.status != 0)
        return fail(nullptr, L2J_E_DEVICE, "device status 0x%x", h.status);
    return L2J_OK;
}

}  // namespace

extern "C" int l2j_quant_encode(int device, const float *in, int64_t n_floats, void *out)
{
    if (!in || !out || n_floats <= 0)
        return fail(nullptr, L2J_E_INVALID, "bad arguments");
    int rc = set_device_checked(device);
    if (rc != L2J_OK)
        return rc;
    Scratch s;
    const int64_t piece = (int64_t)kGroup << 18;   // 64 Mi floats per piece
    float *din = nullptr;
    uint8_t *dout = nullptr;
    const int64_t pn = n_floats < piece ? n_floats : piece;
    KCK(s.alloc(&din, pn));
    KCK(s.alloc(&dout, ((pn + kGroup - 1) / kGroup) * kGroupBytes));
    for (int64_t done = 0; done < n_floats; done += piece) {
        const int64_t n = n_floats - done < piece ? n_floats - done : piece;
        const int64_t ob = ((n + kGroup - 1) / kGroup) * kGroupBytes;
        KCK(cudaMemcpy(din, in + done, (size_t)n * sizeof(float), cudaMemcpyHostToDevice));
        KCK(launch_quant_encode(nullptr, din, n, dout));
        KCK(cudaMemcpy(static_cast<uint8_t *>(out) + (done / kGroup) * kGroupBytes, dout, (size_t)ob, cudaMemcpyDeviceToHost));
    }
    return L2J_OK;
}

extern "C" int l2j_synth_f32(int device, uint64_t seed, uint32_t stream, int64_t start, int64_t n_floats, float scale,
                             float *out)
{
    if (!out || n_floats <= 0 || start < 0)
        return fail(nullptr, L2J_E_INVALID, "bad arguments");
    int rc = set_device_checked(device);
    if (rc != L2J_OK)
        return rc;
    Scratch s;
    const int64_t piece = (int64_t)1 << 26;
    float *d = nullptr;
    KCK(s.alloc(&d, n_floats < piece ? n_floats : piece));
    for (int64_t done = 0; done < n_floats; done += piece) {
        const int64_t n = n_floats - done < piece ? n_floats - done : piece;
        KCK(launch_synth_normal(nullptr, d, n, seed, stream, start + done, scale));
        KCK(cudaMemcpy(out + done, d, (size_t)n * sizeof(float), cudaMemcpyDeviceToHost));
    }
    return L2J_OK;
}

extern "C" int l2j_synth_quant(int device, uint64_t seed, uint32_t stream, int64_t n_floats, float scale, void *out)
{
    if (!out || n_floats <= 0)
        return fail(nullptr, L2J_E_INVALID, "bad arguments");
    int rc = set_device_checked(device);
    if (rc != L2J_OK)
        return rc;
    Scratch s;
    const int64_t piece = (int64_t)kGroup << 18;
    float *d = nullptr;
    uint8_t *dq = nullptr;
    const int64_t pn = n_floats < piece ? n_floats : piece;
    KCK(s.alloc(&d, pn));
    KCK(s.alloc(&dq, ((pn + kGroup - 1) / kGroup) * kGroupBytes));
    for (int64_t done = 0; done < n_floats; done += piece) {
        const int64_t n = n_floats - done < piece ? n_floats - done : piece;
        const int64_t ob = ((n + kGroup - 1) / kGroup) * kGroupBytes;
        KCK(launch_synth_normal(nullptr, d, n, seed, stream, done, scale));
        KCK(launch_quant_encode(nullptr, d, n, dq));
        KCK(cudaMemcpy(static_cast<uint8_t *>(out) + (done / kGroup) * kGroupBytes, dq, (size_t)ob, cudaMemcpyDeviceToHost));
    }
    return L2J_OK;
}

extern "C" int l2j_k_matvec_i8(int device, uint32_t flags, const void *groups, int64_t tensor_floats, int64_t weight_index,
                               int n, int d, const float *x, float *xout)
{
    if (!groups || !x || !xout || n <= 0 || d <= 0 || weight_index < 0 || weight_index + (int64_t)n * d > tensor_floats)
        return fail(nullptr, L2J_E_INVALID, "bad arguments");
    int rc = set_device_checked(device);
    if (rc != L2J_OK)
        return rc;
    Scratch s;
    const int64_t ng = (tensor_floats + kGroup - 1) / kGroup;
    uint8_t *raw = nullptr, *payload = nullptr;
    float2 *hdr = nullptr;
    float *dx = nullptr, *dy = nullptr;
    SeqState *st = nullptr;
    KCK(s.alloc(&raw, ng * kGroupBytes));
    KCK(s.alloc(&payload, ng * kGroup + 512, true));
    KCK(s.alloc(&hdr, ng + 8, true));
    KCK(s.alloc(&dx, n));
    KCK(s.alloc(&dy, d, true));
    KCK(s.alloc(&st, 1, true));
    unsigned int *work = nullptr;
    KCK(s.alloc(&work, 2, true));
    KCK(cudaMemcpy(raw, groups, (size_t)ng * kGroupBytes, cudaMemcpyHostToDevice));
    KCK(cudaMemcpy(dx, x, (size_t)n * sizeof(float), cudaMemcpyHostToDevice));
    KCK(launch_repack(nullptr, raw, ng, payload, hdr));
    MvSeg seg{payload, hdr, weight_index, d};
    // the grouped thread mapping needs rows that start on a group boundary
    const MvPlan pl = plan_matvec(n, false, false, 0, 0, 1, weight_index % kGroup == 0);
    if (!(flags & L2J_F_SIMPLE) && pl.ok) {
        cudaDeviceProp prop{};
        KCK(cudaGetDeviceProperties(&prop, device));
        MvParams p{};
        p.seg[0] = seg;
        p.nseg = 1;
        p.n = n;
        fill_plan(p, pl);
        p.timeout_us = 50000;
        p.x_in = dx;
        p.x_reps = 1;
        p.y_reps = 1;
        p.epilogue = EPI_STORE;
        p.y = dy;
        p.state = st;
        p.work = work;
        LaunchCfg lc{nullptr, false, prop.multiProcessorCount};
        KCK(launch_matvec_ring(lc, pl, false, p));
    } else {
        KCK(launch_matvec_plain_u8(nullptr, seg, n, dx, dy));
    }
    KCK(cudaDeviceSynchronize());
    KCK(cudaMemcpy(xout, dy, (size_t)d * sizeof(float), cudaMemcpyDeviceToHost));
    return status_of(st);
}

extern "C" int l2j_k_matvec_f32(int device, uint32_t flags, const float *w, int n, int d, const float *x, float *xout,
                                int *argmax)
{
    if (!w || !x || !xout || n <= 0 || d <= 0)
        return fail(nullptr, L2J_E_INVALID, "bad arguments");
    int rc = set_device_checked(device);
    if (rc != L2J_OK)
        return rc;
    Scratch s;
    cudaDeviceProp prop{};
    KCK(cudaGetDeviceProperties(&prop, device));
    float *dw = nullptr, *dx = nullptr, *dy = nullptr, *bv = nullptr;
    int *bi = nullptr, *outtok = nullptr;
    SeqState *st = nullptr;
    KCK(s.alloc(&dw, (int64_t)n * d + 64));
    KCK(s.alloc(&dx, n));
    KCK(s.alloc(&dy, d, true));
    KCK(s.alloc(&bv, 2 * prop.multiProcessorCount + 8, true));
    KCK(s.alloc(&bi, 2 * prop.multiProcessorCount + 8, true));
    unsigned int *work = nullptr;
    KCK(s.alloc(&work, 2, true));
    KCK(s.alloc(&outtok, 8, true));
    KCK(s.alloc(&st, 1, true));
    KCK(cudaMemcpy(dw, w, (size_t)n * d * sizeof(float), cudaMemcpyHostToDevice));
    KCK(cudaMemcpy(dx, x, (size_t)n * sizeof(float), cudaMemcpyHostToDevice));
    MvParams p{};
    p.seg[0].payload = reinterpret_cast<const uint8_t *>(dw);
    p.seg[0].rows = d;
    p.nseg = 1;
    p.n = n;
    p.x_in = dx;
    p.x_reps = 1;
    p.y_reps = 1;
    p.epilogue = argmax ? EPI_LOGITS : EPI_STORE;
    p.y = dy;
    p.blk_val = bv;
    p.blk_idx = bi;
    p.out_tokens = outtok;
    p.state = st;
    p.work = work;
    const MvPlan pl = plan_matvec(n, true, false);
    p.f32 = 1;
    if (!(flags & L2J_F_SIMPLE) && pl.ok) {
        fill_plan(p, pl);
        p.timeout_us = 50000;
        LaunchCfg lc{nullptr, false, prop.multiProcessorCount};
        KCK(launch_matvec_ring(lc, pl, true, p));
    } else {
        float *tmp = nullptr;
        KCK(s.alloc(&tmp, d, true));
        KCK(launch_matvec_plain_f32(nullptr, dw, n, d, dx, tmp));
        KCK(launch_epilogue_plain(nullptr, p, tmp, nullptr, nullptr));
    }
    KCK(cudaDeviceSynchronize());
    KCK(cudaMemcpy(xout, dy, (size_t)d * sizeof(float), cudaMemcpyDeviceToHost));
    SeqState h{};
    KCK(cudaMemcpy(&h, st, sizeof(SeqState), cudaMemcpyDeviceToHost));
    if (argmax)
        *argmax = h.argmax;
    if (h.status != 0)
        return fail(nullptr, L2J_E_DEVICE, "device status 0x%x", h.status);
    return L2J_OK;
}

extern "C" int l2j_k_rmsnorm(int device, const void *groups, int64_t tensor_floats, int64_t weight_index, int n, const float *x,
                             float *out)
{
    if (!groups || !x || !out || n <= 0 || weight_index < 0 || weight_index + n > tensor_floats)
        return fail(nullptr, L2J_E_INVALID, "bad arguments");
    int rc = set_device_checked(device);
    if (rc != L2J_OK)
        return rc;
    Scratch s;
    const int64_t ng = (tensor_floats + kGroup - 1) / kGroup;
    uint8_t *raw = nullptr;
    QTensor t;
    float *w = nullptr, *dx = nullptr, *dy = nullptr;
    KCK(s.alloc(&raw, ng * kGroupBytes));
    KCK(s.alloc(&t.payload, ng * kGroup + 512, true));
    KCK(s.alloc(&t.hdr, ng + 8, true));
    KCK(s.alloc(&w, n));
    KCK(s.alloc(&dx, n));
    KCK(s.alloc(&dy, n));
    t.base_float = 0;
    t.n_groups = ng;
    KCK(cudaMemcpy(raw, groups, (size_t)ng * kGroupBytes, cudaMemcpyHostToDevice));
    KCK(cudaMemcpy(dx, x, (size_t)n * sizeof(float), cudaMemcpyHostToDevice));
    KCK(launch_repack_minmax(nullptr, raw, ng, t.payload, t.hdr));
    KCK(launch_dequant_rms(nullptr, t, weight_index, n, w));
    KCK(launch_rmsnorm_plain(nullptr, dx, w, dy, n));
    KCK(cudaDeviceSynchronize());
    KCK(cudaMemcpy(out, dy, (size_t)n * sizeof(float), cudaMemcpyDeviceToHost));
    return L2J_OK;
}

extern "C" int l2j_k_rope(int device, float *q, float *k, int pos, int dim, int kv_dim, int head_size)
{
    if (!q || !k || pos < 0 || dim <= 0 || kv_dim <= 0 || kv_dim > dim || head_size <= 0 || head_size % 2 != 0 ||
        dim % head_size != 0 || kv_dim % head_size != 0)
        return fail(nullptr, L2J_E_INVALID, "bad arguments");
    int rc = set_device_checked(device);
    if (rc != L2J_OK)
        return rc;
    Scratch s;
    std::vector<float> cs, sn;
    build_rope_tables(pos + 1, head_size, cs, sn);
    float *dq = nullptr, *dk = nullptr, *dcs = nullptr, *dsn = nullptr;
    KCK(s.alloc(&dq, dim));
    KCK(s.alloc(&dk, kv_dim));
    KCK(s.alloc(&dcs, (int64_t)cs.size()));
    KCK(s.alloc(&dsn, (int64_t)sn.size()));
    KCK(cudaMemcpy(dq, q, (size_t)dim * sizeof(float), cudaMemcpyHostToDevice));
    KCK(cudaMemcpy(dk, k, (size_t)kv_dim * sizeof(float), cudaMemcpyHostToDevice));
    KCK(cudaMemcpy(dcs, cs.data(), cs.size() * sizeof(float), cudaMemcpyHostToDevice));
    KCK(cudaMemcpy(dsn, sn.data(), sn.size() * sizeof(float), cudaMemcpyHostToDevice));
    KCK(launch_rope_plain(nullptr, dq, dk, dcs, dsn, pos, dim, kv_dim, head_size));
    KCK(cudaDeviceSynchronize());
    KCK(cudaMemcpy(q, dq, (size_t)dim * sizeof(float), cudaMemcpyDeviceToHost));
    KCK(cudaMemcpy(k, dk, (size_t)kv_dim * sizeof(float), cudaMemcpyDeviceToHost));
    return L2J_OK;
}

extern "C" int l2j_k_attention(int device, const float *q, const float *key_cache, const float *value_cache, int pos,
                               int n_heads, int n_kv_heads, int head_size, int seq_len, float *out)
{
    if (!q || !key_cache || !value_cache || !out || pos < 0 || pos >= seq_len || n_heads <= 0 || n_kv_heads <= 0 ||
        n_heads % n_kv_heads != 0 || head_size % 4 != 0 || head_size > 128 || head_size <= 0)
        return fail(nullptr, L2J_E_INVALID, "bad arguments");
    int rc = set_device_checked(device);
    if (rc != L2J_OK)
        return rc;
    Scratch s;
    cudaDeviceProp prop{};
    KCK(cudaGetDeviceProperties(&prop, device));
    const int kv_dim = n_kv_heads * head_size;
    const int64_t used = (int64_t)(pos + 1) * kv_dim;
    const int64_t cache = (int64_t)seq_len * kv_dim;
    float *dq = nullptr, *ksrc = nullptr, *vsrc = nullptr, *kc = nullptr, *vc = nullptr, *dout = nullptr, *part = nullptr;
    unsigned int *counters = nullptr;
    SeqState *st = nullptr;
    AttnParams p{};
    p.nsplit = choose_nsplit(prop.multiProcessorCount, n_heads, seq_len);
    KCK(s.alloc(&dq, (int64_t)n_heads * head_size));
    KCK(s.alloc(&ksrc, used));
    KCK(s.alloc(&vsrc, used));
    KCK(s.alloc(&kc, cache, true));
    KCK(s.alloc(&vc, cache, true));
    KCK(s.alloc(&dout, (int64_t)n_heads * head_size, true));
    KCK(s.alloc(&part, (int64_t)n_heads * p.nsplit * (head_size + 2), true));
    KCK(s.alloc(&counters, n_heads, true));
    KCK(s.alloc(&st, 1, true));
    KCK(cudaMemcpy(dq, q, (size_t)n_heads * head_size * sizeof(float), cudaMemcpyHostToDevice));
    KCK(cudaMemcpy(ksrc, key_cache, (size_t)used * sizeof(float), cudaMemcpyHostToDevice));
    KCK(cudaMemcpy(vsrc, value_cache, (size_t)used * sizeof(float), cudaMemcpyHostToDevice));
    KCK(launch_kv_relayout(nullptr, ksrc, kc, n_kv_heads, head_size, seq_len, pos + 1));
    KCK(launch_kv_relayout(nullptr, vsrc, vc, n_kv_heads, head_size, seq_len, pos + 1));
    p.q = dq;
    p.k_cache = kc;
    p.v_cache = vc;
    p.out = dout;
    p.part = part;
    p.counters = counters;
    p.state = st;
    p.n_heads = n_heads;
    p.kv_mul = n_heads / n_kv_heads;
    p.head = head_size;
    p.seq_len = seq_len;
    p.out_reps = 1;
    p.pos_override = pos;
    LaunchCfg lc{nullptr, false, prop.multiProcessorCount};
    KCK(launch_attention(lc, p));
    KCK(cudaDeviceSynchronize());
    KCK(cudaMemcpy(out, dout, (size_t)n_heads * head_size * sizeof(float), cudaMemcpyDeviceToHost));
    return L2J_OK;
}

extern "C" int l2j_k_swiglu(int device, float *hb, const float *hb2, int n)
{
    if (!hb || !hb2 || n <= 0)
        return fail(nullptr, L2J_E_INVALID, "bad arguments");
    int rc = set_device_checked(device);
    if (rc != L2J_OK)
        return rc;
    Scratch s;
    float *a = nullptr, *b = nullptr;
    KCK(s.alloc(&a, n));
    KCK(s.alloc(&b, n));
    KCK(cudaMemcpy(a, hb, (size_t)n * sizeof(float), cudaMemcpyHostToDevice));
    KCK(cudaMemcpy(b, hb2, (size_t)n * sizeof(float), cudaMemcpyHostToDevice));
    KCK(launch_swiglu_plain(nullptr, a, b, n));
    KCK(cudaDeviceSynchronize());
    KCK(cudaMemcpy(hb, a, (size_t)n * sizeof(float), cudaMemcpyDeviceToHost));
    return L2J_OK;
}
