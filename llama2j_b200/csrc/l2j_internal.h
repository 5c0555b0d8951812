// Host/device shared declarations of libl2j_b200: device-side tensor views, kernel parameter
// blocks and the launch wrappers the context code calls.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <vector>

namespace l2j {

constexpr int kGroup = 256;        // elements per quantisation group
constexpr int kGroupBytes = 264;   // encoded bytes per group in the file format
// Copies kept of the vectors that every block of a kernel reads in full (x, the attention output, the FFN
// hidden vector, the RMSNorm weights).  More than one spreads the simultaneous reads of 148 blocks over
// several sets of L2 lines; measured on B200 it gained nothing, so one copy is kept.
constexpr int kVecReps = 1;
constexpr int kMaxSmemBlock = 221 * 1024;  // dynamic shared memory of a ring-kernel block: one block per SM, with
                                           // room left for the small blocks of the attention kernel

// Device-resident sequence state, advanced by the kernels themselves so that consecutive tokens
// can be queued without a host round trip.
struct SeqState {
    int cur_token;   // token fed to the forward in flight
    int cur_pos;     // its position
    int token;       // token to feed next (greedy loop)
    int pos;         // next position (greedy loop)
    int n_prompt;    // forced tokens after BOS
    int status;      // L2J_DS_* bits
    int argmax;      // device argmax of the last forward
    unsigned int cls_counter;   // arrival counter of the classifier's argmax reduction
};

struct TpTable;

// Hand-over between consecutive kernels of a forward.  Waiting for the grid in front to complete costs
// microseconds after its last block has finished; instead every block bumps a counter once its results
// are visible, and the blocks of the next kernel (already resident under programmatic dependent launch)
// poll that counter.  Counters only grow: after forward number e (the epoch word, bumped by the begin
// kernel) every block has bumped e times.
struct ChainLink {
    const unsigned int *wait_counter;   // counter of the kernel in front, or nullptr: wait for grid completion
    unsigned int wait_blocks;           // bumps per forward on that counter
    unsigned int *done_counter;         // counter this launch bumps once per block, or nullptr
    const unsigned int *epoch;          // forwards started on this context
};

struct Cmd {
    int mode;    // 1: feed (token, pos) from the host; 0: continue the device-side greedy loop
    int token;
    int pos;
    int flags;   // kCmd* bits: how a stage of a layer split gets its inputs
};

constexpr int kCmdXFromPeer = 1;       // x is read from the previous stage's device (StageLink::x_src)
constexpr int kCmdTokenFromPeer = 2;   // greedy loop: the next token is read from the last stage's device
constexpr int kCmdAdvancePos = 4;      // greedy loop on a stage without the classifier: count the positions here

// Where a stage of a layer split finds the data of its neighbours (peer device memory); written when
// the stages are linked, read by the begin kernel.
struct StageLink {
    const float *x_src;     // x of the previous stage (dim floats)
    const int *token_src;   // SeqState::token of the last stage
};

// One quantised tensor (or the slice of it a context owns) after the upload re-layout:
// bytes and group headers in separate arrays so that every row starts on a 16-byte boundary.
struct QTensor {
    uint8_t *payload = nullptr;   // one byte per element, element e at payload[e - base_float]
    float2 *hdr = nullptr;        // (min, scale) of group g at hdr[g - base_float/256]
    int64_t base_float = 0;       // first element held (multiple of 256)
    int64_t n_groups = 0;         // groups held
    int64_t groups_received = 0;
};

enum MvEpilogue {
    EPI_STORE = 0,      // y[i] = v
    EPI_QKV_ROPE = 1,   // rotate q/k pairs, write q and the KV cache
    EPI_RESIDUAL = 2,   // x[i] += v
    EPI_SWIGLU = 3,     // hb[i] = silu(v1) * v3  (paired W1/W3 rows)
    EPI_LOGITS = 4      // logits[i] = v, block argmax, grid argmax by the last block
};

struct MvParams;

struct MvSeg {
    const uint8_t *payload;   // u8 payload, or the float rows for FP32 weights
    const float2 *hdr;
    int64_t flat0;            // element offset of the first row this launch works on, relative to payload
    int rows;                 // rows this launch works on
    int out0;                 // index of the first of them in the output vector (tensor parallel: a rank's rows)
};

// Tensor-parallel group of up to kMaxTp devices driven by one process.  Every rank computes a block of
// rows of each matrix from the full input vector and stores its results into every rank's copy of the
// output vector over the peer links, so each output element is produced by one rank in the same order
// as on a single device: the ranks' vectors stay bitwise equal, and equal to the single-device ones.
constexpr int kMaxTp = 8;
enum TpVector { TPV_X = 0, TPV_XB = 1, TPV_HB = 2, TPV_CAND = 3, TPV_COUNT = 4 };   // CAND: (max, index) of every rank's block of logits
struct TpTable {
    int n;                             // ranks (0 until the group is linked)
    int rank;
    float2 *ll[TPV_COUNT][kMaxTp];     // every rank's receive buffers: (value, sequence number) per element
};

// Hand-over between the ranks of a tensor-parallel group: every result travels as an 8-byte (value,
// sequence number) pair written with one store into the receive buffer of every rank, and the kernel that
// consumes the vector polls the pairs of the elements it loads until they carry the number it expects.
// No fence, no counter and no second message: the latency is one trip over the link.  A number is used
// once: forward e, kernel i of the forward -> e * kernels_per_forward + i + 1.
struct LlLink {
    const TpTable *tp;         // nullptr: not a tensor-parallel launch
    const unsigned int *epoch; // forwards started on this context (same on every rank of the group)
    int kernels;               // kernel launches per forward (the multiplier of the epoch)
    int in_vec, in_idx;        // input: receive buffer to read (-1: the plain input vector) and the producing kernel's index
    int out_vec, out_idx;      // output: receive buffer to write on every rank (-1: local outputs only) and this kernel's index
    const float *base;         // input = base + received (the residual stream), or nullptr: input = received
    float *write_back;         // block 0 stores the assembled input here for the next residual step, or nullptr
};

// Parameters of the ring matvec kernel.
struct MvParams {
    MvSeg seg[3];
    int nseg;          // sequential segments (1, or 3 for QKV); paired mode uses seg[0], seg[1]
    int paired;        // 1: a stage holds RPP rows of seg[0] and the same rows of seg[1]
    int n;             // row length in elements
    int rpp;           // rows per pass and half
    int wpr;           // warps per row
    int nstage;        // ring depth
    int slot_bytes;    // bytes per ring slot
    int hdr_off;       // offset of the header area inside a slot
    int half_hdr;      // bytes of one half's header area (paired mode)
    int xshare_bytes;  // shared copy of x between the header and the ring
    int timeout_us;    // bound of every wait on a copy barrier
    int seg_stages[3]; // stages per segment
    int total_stages;
    int rs;            // matrix rows (row pairs in paired mode) a stage advances
    int rt;            // rows per consumer thread and stage (the kernels' RT template parameter)
    int rowbytes;      // bytes of one matrix row
    int f32;           // 1: FP32 weights
    int tail_prefetch; // stages of the next launch each block prefetches into L2 when it runs out of work
    int early_fill;    // stages the producer may issue before the previous kernel has finished (0: none)
    const MvParams *next;   // device copy of the next ring launch's parameters (prefetch target) or nullptr
    // prologue
    const float *x_in;       // input vector (n floats), replica 0
    int x_reps, x_stride;    // copies of the vector (and of rms_w) and their distance in floats; block b reads copy b % x_reps
    const float *rms_w;      // dequantised RMSNorm weights (n floats) or nullptr
    float rms_wmax;          // max |rms_w| (bounds the normalised vector for the fixed-point scale)
    // epilogue
    int epilogue;
    float *y;                // STORE / RESIDUAL / SWIGLU / LOGITS target (replica 0)
    int y_reps, y_stride;    // copies of the target vector that every result is written to
    LlLink ll;               // tensor parallel: where the input comes from and where the results go
    float *q_out;            // QKV: q (dim)
    float *k_cache;          // QKV: layer base of the K cache [kv_head][seq][head]
    float *v_cache;
    const float *rope_cos;   // [seq][head/2]
    const float *rope_sin;
    int dim, kv_dim, head, seq_len;
    int kv_prefetch_below;   // QKV: below this position the cached K/V rows are asked into L2 for the attention kernel (0: never)
    // logits
    float *blk_val;          // per-block argmax candidates
    int *blk_idx;
    const int *prompt;       // device prompt tokens
    int *out_tokens;
    SeqState *state;
    ChainLink chain;
    unsigned int *work;  // {next unclaimed stage, blocks that ran out of work}; zero between launches
    unsigned long long *trace;   // optional per-block timeline (8 slots per block), else nullptr
};

struct AttnParams {
    const float *q;          // (n_heads * head)
    const float *k_cache;    // layer base, [kv_head][seq][head]
    const float *v_cache;
    float *out;              // (n_heads * head), replica 0
    int out_reps, out_stride;   // copies of the output vector and their distance in floats
    LlLink ll;               // tensor parallel: the results go to every rank's receive buffer
    int h0;                  // first head of this launch (block x works on head h0 + x)
    float *part;             // scratch: [n_heads][nsplit][head + 2]
    unsigned int *counters;  // [n_heads], zero between launches
    SeqState *state;
    int n_heads, kv_mul, head, seq_len, nsplit;
    int pos_override;        // >= 0: use this position instead of state->cur_pos (tests)
    int cluster;             // 1: the nsplit (<= 8) blocks of a head are launched as one thread-block cluster and merge
                             // their partial results through distributed shared memory instead of `part`
    ChainLink chain;
    int timeout_us;          // bound of the wait on the hand-over counter
    int smem_pad;            // 1: ask for so much shared memory that only two blocks fit an SM; under programmatic
                             // dependent launch blocks are placed on whichever SMs drain first, and three per SM
                             // would leave a third of the GPU without a stream of its own
    unsigned long long *trace;   // optional timeline of the first trace_blocks blocks (16 slots each), else nullptr
    int trace_blocks;
};

// ---- one launch for all layers of a token (l2j_fused.cu) --------------------------------------
//
// The five steps of a layer (QKV, attention, Wo, W1/W3, W2) run as phases of one persistent kernel:
// the blocks never leave their SMs, the producer thread of a block keeps streaming the stages of the
// phases ahead into one shared-memory byte ring while the consumers wait at a phase boundary, and the
// cached K and V rows of the attention phase travel through the same ring.  The parameters of the
// first layer are given; those of layer l follow by adding l times a step to the pointers.
constexpr int kAttSlots = 8;        // partial results per head that the step after the attention phase can merge
constexpr int kAttMaxSplit = 6;     // blocks per head in the attention phase (a head gets at most kAttMaxSplit + 1 partials)
constexpr int kAttChunk = 64;       // cached positions per ring stage of the attention phase

struct FusedParams {
    MvParams mv[4];            // QKV, Wo, W1/W3, W2 of the first layer of the context's range
    long long seg_step[4][3];  // elements between the matrices of consecutive layers, per segment
    long long kv_step;         // floats between the KV caches of consecutive layers
    int rms_step;              // floats between the RMSNorm weight vectors of consecutive layers
    int n_layers;
    const float *rms_wmax;     // [n_layers][2]: max |w| of the attention and the FFN RMSNorm weights
    const float *q;            // query vector written by the QKV phase (n_heads * head)
    float *att_part;           // [n_heads][kAttSlots][head + 4]: o, then m, l
    int n_heads, kv_mul, head, seq_len;
    int xarea_bytes;           // shared memory between the fixed header and the ring: limbs of the input vector / merge area
    int ring_bytes;            // bytes of the ring
    unsigned int *sync;        // hand-over counters, kSyncStride words apart, five per layer
    const unsigned int *epoch; // forwards started on this context
    SeqState *state;
    int timeout_us;
    unsigned long long *trace; // optional: [block][5 * n_layers][8] global-timer marks, else nullptr
    int debug_no_copy;         // measurement aid: the producer hands out stages without copying (results are garbage)
};
constexpr int kSyncStride = 32;     // unsigned ints between two hand-over counters (128 bytes)
constexpr int kFusedThreads = 640;  // 18 consumer warps, the producer warp, the epilogue warp
constexpr int kFusedConsWarps = 18;
constexpr int kFusedHeaderBytes = 4096;   // barriers, descriptors, reduction buffers in front of the vector area and the ring

cudaError_t prepare_fused(int *max_smem);
cudaError_t launch_fused(cudaStream_t stream, bool pdl, int grid, int smem_bytes, const FusedParams &p);

// Blocks per head of the stand-alone attention kernel: as many as fit on the device at once (two blocks per SM are
// resident; one block more than that and a few SMs scan a third key range while the others wait: 40 heads x 8
// splits were 320 blocks on 296 places), at least 16 positions each.  One definition for every entry point, so
// that they split (and therefore round) alike.
inline int choose_nsplit(int sm_count, int n_heads, int seq_len)
{
    int ns = (2 * sm_count) / n_heads;
    if (ns > 32)
        ns = 32;
    const int cap = seq_len / 16 > 0 ? seq_len / 16 : 1;
    if (ns > cap)
        ns = cap;
    if (ns < 1)
        ns = 1;
    return ns;
}

// ---- batched prompt processing on the tensor cores (l2j_prefill.cu) ---------------------------------------------
constexpr int kPrefillTokens = 64;   // positions that share one sweep over the weights
enum PrefillWeight { PF_WQ = 0, PF_WK, PF_WV, PF_WO, PF_W1, PF_W3, PF_W2, PF_W_COUNT };

struct PrefillLayerDesc {
    const uint8_t *w[PF_W_COUNT];    // byte payload of the layer's matrix, row-major, rows of whole quantisation groups
    const float2 *h[PF_W_COUNT];     // (min, scale) of group g of row r at [r * (k / 256) + g]
    const float *rms_att, *rms_ffn;  // dequantised RMSNorm weights of the layer
    float *kc, *vc;                  // the layer's K / V cache, [kv_head][seq][head]
};

struct PrefillModel {
    int dim, hidden, n_layers, n_heads, n_kv_heads, head, seq_len, vocab;
    const float *emb;
    const float *wcls;               // FP32 classifier [vocab][dim] (the embedding table when shared)
    const float *rms_final;          // dequantised final RMSNorm weights
    const float *rope_cos, *rope_sin;
    unsigned int *status;            // device status word of the context
    int timeout_us;
    std::vector<PrefillLayerDesc> layers;
};

struct Prefill;
bool prefill_supported(const PrefillModel &m);
cudaError_t prefill_create(Prefill **out, const PrefillModel &m);
cudaError_t prefill_run(Prefill *pf, cudaStream_t stream, const int *tokens_host, int n, int pos0);
cudaError_t prefill_batch_create(Prefill *pf, int n_seq, int seq_len);
cudaError_t prefill_batch_forward(Prefill *pf, cudaStream_t stream, const int *tokens, const int *pos, const int *seq, int n, float *logits_out,
                                  int *argmax_out);
int prefill_batch_sequences(const Prefill *pf);
int prefill_batch_seq_len(const Prefill *pf);
unsigned long long prefill_launches(const Prefill *pf);
void prefill_destroy(Prefill *pf);

// ---- temperature / top-p sampler on the device (l2j_sampler.cu) ----------------------------------
struct SamplerState {
    unsigned long long rng;   // java.util.Random's 48-bit state
    int token;                // the id chosen by the last launch
};

struct SampleParams {
    float *logits;            // vocab logits of the last forward; turned into probabilities in place
    int n;
    float temperature, topp;
    SamplerState *st;
    float *prob[2];           // the Sampler's ProbIndex array (persistent across calls), and the sort's second buffer
    int *index[2];
};

size_t sample_smem_bytes(int n);
cudaError_t prepare_sampler(int n);
cudaError_t launch_sample(cudaStream_t stream, const SampleParams &sp);

struct MvPlan {
    bool grouped;  // u8 rows of whole groups: four lanes share a group (template selector)
    int cpt;       // chunks per thread (template selector)
    int rt;        // rows per thread and stage (template selector)
    int rpp, wpr;
    int nstage, slot_bytes, hdr_off, half_hdr, xshare_bytes;
    int threads;   // block size including the producer and the epilogue warp
    int smem_bytes;
    bool ok;
};

// Chooses the thread mapping and ring geometry for a row length; ok=false if the ring kernel
// cannot take the shape (the caller then uses the plain kernels).  rows/blocks (optional) let a matrix
// with few rows get smaller stages; row_align is the multiple of rows every stage must hold; group_aligned
// says that every row starts on a quantisation-group boundary whenever n is a multiple of the group size.
MvPlan plan_matvec(int n, bool f32, bool paired, int rows = 0, int blocks = 0, int row_align = 1,
                   bool group_aligned = true);

// ---- launch wrappers (all asynchronous on `stream`) ---------------------------------------
struct LaunchCfg {
    cudaStream_t stream;
    bool pdl;       // launch with the programmatic-stream-serialization attribute
    int grid;       // number of blocks for the ring kernels (SM count)
};

cudaError_t prepare_kernels();
cudaError_t launch_matvec_ring(const LaunchCfg &lc, const MvPlan &plan, bool f32, const MvParams &p);
cudaError_t launch_attention(const LaunchCfg &lc, const AttnParams &p);
cudaError_t launch_begin(const LaunchCfg &lc, SeqState *state, const Cmd *cmd, const float *emb, float *x, int dim,
                         int vocab, int seq_len, int gather, int x_reps, int x_stride, unsigned int *epoch, const StageLink *link);

// plain (cross-check) kernels
cudaError_t launch_rmsnorm_plain(cudaStream_t s, const float *x, const float *w, float *out, int n);
cudaError_t launch_matvec_plain_u8(cudaStream_t s, const MvSeg &seg, int n, const float *x, float *y);
cudaError_t launch_matvec_plain_f32(cudaStream_t s, const float *w, int n, int d, const float *x, float *y);
cudaError_t launch_epilogue_plain(cudaStream_t s, const MvParams &p, const float *y0, const float *y1, const float *y2);
cudaError_t launch_rope_plain(cudaStream_t s, float *q, float *k, const float *cs, const float *sn, int pos, int dim,
                              int kv_dim, int head);
cudaError_t launch_swiglu_plain(cudaStream_t s, float *hb, const float *hb2, int n);

// load-time kernels
cudaError_t launch_repack(cudaStream_t s, const uint8_t *groups, int64_t n_groups, uint8_t *payload, float2 *hdr);
cudaError_t launch_repack_minmax(cudaStream_t s, const uint8_t *groups, int64_t n_groups, uint8_t *payload, float2 *hdr);
cudaError_t launch_dequant_rms(cudaStream_t s, const QTensor &t, int64_t first_float, int64_t n, float *out);
cudaError_t launch_quant_encode(cudaStream_t s, const float *in, int64_t n, uint8_t *out);
cudaError_t launch_synth_normal(cudaStream_t s, float *out, int64_t n, uint64_t seed, uint32_t stream_id, int64_t start,
                                float scale);
cudaError_t launch_kv_relayout(cudaStream_t s, const float *src, float *dst, int n_kv_heads, int head, int seq_len,
                               int npos);

}  // namespace l2j
