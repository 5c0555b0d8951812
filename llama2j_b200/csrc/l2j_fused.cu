// fused_layers_kernel: every layer of a token in ONE persistent launch (sm_100a).
//
// The per-step kernels of l2j_kernels.cu stream at HBM speed but pay a start-up chain at each of
// their five boundaries per layer: a block holds nearly all of an SM's shared memory, so the next
// kernel's block cannot become resident, let alone prefetch, before the one in front has left.
// Here the blocks never leave.  One block per SM; its warps keep their roles for the whole token:
//
//   producer thread   walks the fixed sequence of stages of this block (layer by layer: QKV rows,
//                     cached K/V rows of the attention step, Wo rows, W1/W3 row pairs, W2 rows) and
//                     streams them with bulk copies (TMA engine) into ONE shared-memory byte ring,
//                     as far ahead as the ring has room.  Weights and old cache rows never depend
//                     on this token's activations, so while the consumers wait at a phase boundary
//                     the ring fills with the next phase: HBM does not idle.
//   consumer warps    per phase: wait for the hand-over counter of the phase in front, load the
//                     input vector (for Wo: merge the attention partials), RMSNorm, fixed-point
//                     limbs, then dp4a over the block's stages as they land.
//   epilogue warp     folds the per-warp partial sums of a stage and applies RoPE + cache write,
//                     residual add or SwiGLU; after the block's last stage of a phase it bumps the
//                     phase's counter (release), which is what the other blocks' consumers poll.
//
// Stages are dealt to the blocks round-robin, continuing across phases, so every block streams the
// same number of bytes per token (+- one stage).  The attention step's units (head, 64 positions)
// are dealt in contiguous runs, a block folds the units of one head into one partial (m, l, o), and
// the Wo phase's prologue merges the few partials of a head (at most kAttSlots) in a fixed order.
//
// Arithmetic per output element is that of matvec_ring_kernel (same lane mapping, same reduction
// order), so the matrix-vector products are bitwise those of the per-step kernels.
//
// Blocks wait for each other, so all of them must be resident: the grid is one block per SM.  Every wait is
// bounded by the SM's cycle counter.  A hand-over between blocks that runs out raises L2J_DS_WAIT_TIMEOUT in
// the status word, and every later hand-over of the forward gives up after 2 us; the block then still works
// through all of its stages with the (wrong) inputs it has, so that producer, consumers and epilogue warp stay
// in step and no bulk copy is in flight when the block ends.
//
// Reference counterparts (paths relative to src/main/java/com/lastbot/llama2j/): the layer body of
// Run.java:418-508 with kernel/MatMul.java:360-444, RootMeanSquare.java:78-118,
// WeightNormalizeAndScale.java:191-239, ApplyRope.java:144-182, AttentionLoop.java:116-164,
// ExpSumNormalize.java:82-131, AccumWeightedValue.java:148-173, Accum.java:70-83, Silu.java:118-135.

#include "l2j_device.cuh"
#include "l2j_internal.h"

#include <cfloat>
#include <cmath>

#define L2J_DS_WAIT_TIMEOUT 0x1

namespace l2j {

static_assert(sizeof(FusedParams) <= 4000, "the parameter block must fit the kernel parameter space");

namespace {

constexpr int kFDesc = 16;              // stage descriptors (and full/empty barrier pairs) in flight
constexpr int kFRedBufs = 4;
constexpr int kFGroup = 4;               // stages of a block that are folded and handed to the epilogue warp together
constexpr int kFBarFull = 0;            // uint64 full[16]
constexpr int kFBarEmpty = 128;         // uint64 empty[16]
constexpr int kFBarRedFull = 256;       // uint64 red_full[4]
constexpr int kFBarRedEmpty = 288;      // uint64 red_empty[4]
constexpr int kFFlag = 320;             // int: result of the poll of a hand-over counter
constexpr int kFVStart = 3264;          // int vstart[16]: the producer's bookkeeping of where each stage in flight begins
constexpr int kFScratch = 384;          // float scratch[64]
constexpr int kFDescOff = 640;          // FStage desc[16]
constexpr int kFRedOff = 1152;          // 4 x 132 floats: [stage of the group][row of the stage][warp of the row]
constexpr int kFRedStride = 528;
constexpr int kFRopeOff = 3328;         // float cos[64], sin[64] of the token's position
constexpr int kFInvTab = 3840;          // float inv[64]: value of one fixed-point unit of each group of the input vector
constexpr int kFHeader = kFusedHeaderBytes;   // end of the fixed part (128-byte aligned)
static_assert(kFInvTab + 64 * 4 <= kFHeader, "header layout");
constexpr int kFCons = kFusedConsWarps * 32;
constexpr int kFGroupRounds = 3;        // quantisation groups of the input vector that one consumer warp converts at most (54 groups)
constexpr int kAttFastSlots = 4;        // the merge that fetches all partials of a thread's elements at once
constexpr uint64_t kFShortWaitNs = 2000;

struct FStage {
    int off, nrows, e0a, e0b;   // what the consumers of a matrix stage need, in one 16-byte load: byte offset in the
                                // ring, rows, element offset of the first row of each half relative to the headers
    int seg, row0, aux, pad;
    // attention stage: seg = head, row0 = first position, nrows = positions (newest included),
    // e0a = positions that travel through the ring (older than the token), aux = byte offset of the V rows
};

__device__ __forceinline__ uint4 lds_v4(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ float2 lds_f2(uint32_t addr)
{
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}

__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c)
{
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Bulk copy without a cache hint (cached K/V rows are read again by the next token).
__device__ __forceinline__ void bulk_g2s_plain(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}

template <int RT, int STEP>
struct Fold {
    static __device__ __forceinline__ float run(const float (&v)[RT], int lane)
    {
        if constexpr (RT == 1) {
            float k = v[0];
#pragma unroll
            for (int o = STEP; o > 0; o >>= 1)
                k += __shfl_xor_sync(0xffffffffu, k, o);
            return k;
        } else {
            constexpr int H = RT / 2;
            const bool up = (lane & STEP) != 0;
            float k[H];
#pragma unroll
            for (int i = 0; i < H; ++i) {
                const float keep = up ? v[H + i] : v[i];
                const float send = up ? v[i] : v[H + i];
                k[i] = keep + __shfl_xor_sync(0xffffffffu, send, STEP);
            }
            return Fold<H, STEP / 2>::run(k, lane);
        }
    }
};

// How the attention step of a token at position `pos` is dealt to the blocks: units of (head, chunk of
// kAttChunk positions), head-major, in contiguous runs over the first `ga` blocks.
struct AttSplit {
    int nchunk, units, ga;
    int np_max;   // partial results per head at most
};

__device__ __forceinline__ AttSplit att_split(const FusedParams &P, int pos, int grid)
{
    AttSplit a;
    a.nchunk = (pos + kAttChunk) / kAttChunk;   // ceil((pos + 1) / chunk)
    a.units = P.n_heads * a.nchunk;
    // Short contexts are a matter of latency, not bandwidth: three blocks per head keep the partials of a head
    // few enough (four) for the step behind to fetch them in one round of loads.
    const int per_head = a.nchunk <= 8 ? 3 : kAttMaxSplit;
    a.ga = min(min(grid, P.n_heads * per_head), a.units);
    a.np_max = min(a.nchunk, (a.ga + P.n_heads - 1) / P.n_heads + 1);
    return a;
}

__device__ __forceinline__ int att_first_unit(const AttSplit &a, int b)
{
    return (int)(((long long)b * a.units) / a.ga);
}

__device__ __forceinline__ int att_block_of(const AttSplit &a, int u)
{
    return (int)((((long long)(u + 1)) * a.ga + a.units - 1) / a.units) - 1;
}

// Stage index -> (segment, first row, row count) of a ring phase.
__device__ __forceinline__ void stage_rows(const MvParams &p, int s, int &seg, int &row0, int &nrows)
{
    seg = 0;
    if (!p.paired && p.nseg > 1) {
        if (s >= p.seg_stages[0]) {
            s -= p.seg_stages[0];
            seg = 1;
            if (s >= p.seg_stages[1]) {
                s -= p.seg_stages[1];
                seg = 2;
            }
        }
    }
    row0 = s * p.rs;
    nrows = min(p.rs, p.seg[seg].rows - row0);
}

__device__ __forceinline__ int first_stage_of(int b, int rot, int grid)
{
    int f = b - rot;
    return f < 0 ? f + grid : f;
}

__device__ __forceinline__ void fused_trace(const FusedParams &P, int phase_index, int k)
{
    if (P.trace)
        P.trace[((int64_t)blockIdx.x * (5 * P.n_layers) + phase_index) * 8 + k] = (unsigned long long)global_timer_ns();
}

// -------------------------------------------------------------------------------------------------
// producer
// -------------------------------------------------------------------------------------------------

struct Producer {
    uint8_t *smem;
    uint32_t sbase, ring_base;
    int vhead;              // bytes handed out so far; < 2^31 per token and block
    int off;                // vhead's position in the ring
    int ring_bytes;
    int seq, tail;          // descriptors issued / known to be released
    bool lost;
    uint64_t wait_ns;
    int pos;                // the token's position, -1 until the kernel in front has set it
    AttSplit as;

    // Room for `bytes` contiguous bytes and a free descriptor; returns the offset in the ring.
    __device__ __forceinline__ uint32_t acquire(uint32_t bytes)
    {
        int *vstart = reinterpret_cast<int *>(smem + kFVStart);
        if (off + (int)bytes > ring_bytes) {
            vhead += ring_bytes - off;
            off = 0;
        }
        const int vend = vhead + (int)bytes;
        while (tail < seq && (seq - tail >= kFDesc || vend - ring_bytes > vstart[tail % kFDesc])) {
            if (!mbar_wait_bounded(sbase + kFBarEmpty + 8 * (tail % kFDesc), (uint32_t)(tail / kFDesc) & 1u,
                                   wait_ns))
                lost = true;
            ++tail;
        }
        vstart[seq % kFDesc] = vhead;
        const uint32_t at = (uint32_t)off;
        const int step = (int)((bytes + 127u) & ~127u);
        vhead += step;
        off += step;
        return at;
    }
};

__device__ __forceinline__ void producer_learn_pos(Producer &pr, const FusedParams &P, int grid)
{
    if (pr.pos < 0) {
        // The position is set by the kernel in front; everything touched so far was weights.
        pdl_wait();
        pr.pos = __ldcg(&P.state->cur_pos);
        pr.as = att_split(P, pr.pos, grid);
    }
}

// The producer is the first four lanes of its warp.  All four keep the same bookkeeping; a stage's (up to) four
// bulk copies (rows of one or two matrices, their group headers) are one instruction stream with per-lane
// operands: lane = 2 * is_header + half.  Every lane arrives on the stage's barrier with the bytes of its own
// copy (the barrier counts four arrivals), so the lanes need not talk to each other.
__device__ __forceinline__ void produce_ring_stage(Producer &pr, const FusedParams &P, const MvParams &p, int k, int layer, int s,
                                                   uint64_t pol, int lane)
{
    const uint32_t off = pr.acquire((uint32_t)p.slot_bytes);
    const int e = pr.seq % kFDesc;
    const uint32_t full = pr.sbase + kFBarFull + 8 * e;
    FStage *desc = reinterpret_cast<FStage *>(pr.smem + kFDescOff) + e;
    int seg, row0, nrows;
    stage_rows(p, s, seg, row0, nrows);
    const int h = lane & 1, is_hdr = lane >> 1;
    const bool mine = (p.paired || h == 0) && !(P.debug_no_copy & 1);
    const int sg = p.paired ? h : seg;
    const uint32_t pbytes = (uint32_t)nrows * (uint32_t)p.rowbytes;
    const int64_t flat = p.seg[sg].flat0 + (int64_t)layer * P.seg_step[k][sg] + (int64_t)row0 * p.n;
    const int64_t ga = (flat >> 8) & ~(int64_t)1;                 // headers are copied from an even group on: 16-byte aligned
    const int64_t gl = (flat + pbytes - 1) >> 8;
    const uint32_t hbytes = (uint32_t)(((gl - ga + 2) & ~(int64_t)1) * 8);
    const uint32_t bytes = mine ? (is_hdr ? hbytes : pbytes) : 0u;
    const int R = p.rt * p.rpp;
    const uint32_t dst = pr.ring_base + off +
                         (is_hdr ? (uint32_t)p.hdr_off + (uint32_t)(h * p.half_hdr) : (uint32_t)(h * (R / 2)) * (uint32_t)p.rowbytes);
    const void *src = is_hdr ? static_cast<const void *>(p.seg[sg].hdr + ga) : static_cast<const void *>(p.seg[sg].payload + flat);
    if (lane == 0) {
        desc->off = (int)off;
        desc->nrows = nrows;
        desc->e0a = (int)(flat - ga * 256);
    }
    if (lane == 1)
        desc->e0b = p.paired ? (int)(flat - ga * 256) : 0;
    if (bytes) {
        mbar_arrive_expect_tx(full, bytes);
        bulk_g2s(dst, src, bytes, full, pol);
    } else {
        mbar_arrive(full);
    }
    ++pr.seq;
}

__device__ __forceinline__ void produce_att_stage(Producer &pr, const FusedParams &P, int layer, int unit, const AttSplit &a, int pos,
                                                  int lane)
{
    const int h = unit / a.nchunk, c = unit - h * a.nchunk;
    const int t0 = c * kAttChunk;
    const int cnt = min(pos + 1, t0 + kAttChunk) - t0;       // positions of the unit, the token's own included
    const int old = min(pos, t0 + kAttChunk) - t0;           // those that were cached by earlier tokens
    const uint32_t kbytes = (uint32_t)old * (uint32_t)P.head * 4u;
    const uint32_t voff = (kbytes + 127u) & ~127u;
    const uint32_t off = pr.acquire(2 * voff);
    const int e = pr.seq % kFDesc;
    const uint32_t full = pr.sbase + kFBarFull + 8 * e;
    FStage *desc = reinterpret_cast<FStage *>(pr.smem + kFDescOff) + e;
    const bool copy = old > 0 && !(P.debug_no_copy & 1) && lane < 2;
    if (lane == 0)
        *reinterpret_cast<int4 *>(desc) = make_int4((int)off, cnt, old, 0);
    if (lane == 1) {
        desc->seg = h;
        desc->row0 = t0;
        desc->aux = (int)voff;
    }
    if (copy) {      // lane 0 the K rows, lane 1 the V rows
        const int kvh = h / P.kv_mul;
        const int64_t row = ((int64_t)kvh * P.seq_len + t0) * P.head;
        const float *src = (lane ? P.mv[0].v_cache : P.mv[0].k_cache) + (int64_t)layer * P.kv_step + row;
        mbar_arrive_expect_tx(full, kbytes);
        bulk_g2s_plain(pr.ring_base + off + (lane ? voff : 0u), src, kbytes, full);
    } else {
        mbar_arrive(full);   // only the token's own row: nothing travels through the ring
    }
    ++pr.seq;
}

// -------------------------------------------------------------------------------------------------
// consumers
// -------------------------------------------------------------------------------------------------

struct Consumer {
    int seq;             // stages consumed so far (descriptor index = seq mod kFDesc)
    int rb, rround;      // position in the ring of reduction buffers
    bool lost, lost_before;
};

// Waits until counter `ctr` has reached `target`: one thread polls, the others follow through barrier 1.
__device__ __forceinline__ void consumers_wait(const unsigned int *ctr, unsigned int target, uint8_t *smem, Consumer &cs, uint64_t wait_ns)
{
    volatile int *flag = reinterpret_cast<volatile int *>(smem + kFFlag);
    if (threadIdx.x == 0) {
        int ok = (int)(ld_acquire_u32(ctr) - target) >= 0;
        if (!ok)
            ok = counter_wait_bounded(ctr, target, cs.lost ? kFShortWaitNs : wait_ns) ? 1 : 0;
        *flag = ok;
    }
    named_barrier_sync(1, kFCons);
    if (*flag == 0)
        cs.lost = true;
}

// One matrix-vector phase of the block: prologue (input vector -> fixed-point limbs in shared memory)
// and the block's `nmine` stages.  One copy of this code serves all four phases (the differences are run-time
// parameters): the prologue runs once per phase, so its instructions come from the L2 every time, and four
// inlined copies of it cost more in instruction fetches than the branches cost here.
// merge: the input is the attention output, assembled from the partial results of the blocks that worked on
// each head.
__device__ __forceinline__ void consume_ring_phase(const FusedParams &P, const MvParams &p, int layer, int nmine, bool merge,
                                                   const float *rms_w, float rms_wmax, const AttSplit &as, uint8_t *smem,
                                                   uint32_t sbase, Consumer &cs, uint64_t wait_ns, int pidx)
{
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nw = p.rpp * p.wpr;
    const bool active = warp < nw;
    const int rsub = warp / p.wpr;
    const int wi = warp - rsub * p.wpr;
    constexpr int RT = 1;   // rows per thread and stage: a stage holds one row per group of wpr warps
    const int n = p.n;
    const int R = RT * p.rpp;
    const int rowbytes = n;
    uint8_t *share = smem + kFHeader;
    float *scratch = reinterpret_cast<float *>(smem + kFScratch);

    int chunk[4];
    const int g = wi * 8 + (lane >> 2);
    const bool gvalid = active && g < (n >> 8);
#pragma unroll
    for (int k = 0; k < 4; ++k)
        chunk[k] = g * 16 + 4 * (k ^ ((lane >> 2) & 1)) + (lane & 3);

    // ---- prologue: the input vector as fixed-point limbs in shared memory.  Every warp owns whole quantisation
    // groups of the vector (group warp + 18 j in round j; a lane holds elements 4 l..4 l + 3 of each half of the group, so that a warp's loads are two contiguous 512-byte requests) and gives each its own
    // power-of-two scale from the group's largest element: no block-wide maximum has to be agreed on before the
    // conversion can start, and the RMSNorm scalar ss = 1 / sqrt(mean(x^2) + eps) is applied to the dot products
    // at the end (sum_j w_j (r_j ss x_j) = ss sum_j w_j r_j x_j up to rounding), so nothing here waits for the
    // sum of squares either.
    float *inv_tab = reinterpret_cast<float *>(smem + kFInvTab);   // value of one fixed-point unit, per group
    const int ngroups = n >> 8;
    {
        const bool has_rms = rms_w != nullptr;
        float xg[kFGroupRounds][8];
        const int ps = P.head + 4;
        const bool merge_fast = merge && as.np_max <= kAttFastSlots;
        if (merge && !merge_fast) {
            // Many partials per head: first a table of their weights in shared memory (one thread per head).
            float *tw = reinterpret_cast<float *>(share);            // [n_heads][kAttSlots] weights, then [n_heads] sums
            if (tid < P.n_heads) {
                const int h = tid;
                const int u0 = h * as.nchunk;
                const int np = min(att_block_of(as, u0 + as.nchunk - 1) - att_block_of(as, u0) + 1, kAttSlots);
                const float *hp = P.att_part + (int64_t)h * kAttSlots * ps + P.head;
                float ms[kAttSlots], ls[kAttSlots];
#pragma unroll
                for (int s2 = 0; s2 < kAttSlots; ++s2) {
                    ms[s2] = -INFINITY;
                    ls[s2] = 0.f;
                    if (s2 < np) {
                        const float2 ml = __ldcg(reinterpret_cast<const float2 *>(hp + (int64_t)s2 * ps));
                        ms[s2] = ml.x;
                        ls[s2] = ml.y;
                    }
                }
                float gm = -INFINITY;
#pragma unroll
                for (int s2 = 0; s2 < kAttSlots; ++s2)
                    gm = fmaxf(gm, ms[s2]);
                float L = 0.f;
#pragma unroll
                for (int s2 = 0; s2 < kAttSlots; ++s2) {
                    const float w = ls[s2] > 0.f ? expf(ms[s2] - gm) : 0.f;
                    L = fmaf(ls[s2], w, L);
                    tw[h * kAttSlots + s2] = w;
                }
                tw[P.n_heads * kAttSlots + h] = L;
            }
            named_barrier_sync(2, kFCons);
        }
        // ---- loads of all rounds first (they are independent), then the arithmetic
        float4 wa[kFGroupRounds], wb[kFGroupRounds];
#pragma unroll
        for (int j = 0; j < kFGroupRounds; ++j) {
            const int gi = warp + j * kFusedConsWarps;
            const int e = gi * 256 + lane * 4;
#pragma unroll
            for (int q = 0; q < 8; ++q)
                xg[j][q] = 0.f;
            wa[j] = wb[j] = make_float4(1.f, 1.f, 1.f, 1.f);
            if (gi >= ngroups)
                continue;
            if (!merge) {
                const float4 a4 = ld_cg_f4_issue(p.x_in + e), b4 = ld_cg_f4_issue(p.x_in + e + 128);
                xg[j][0] = a4.x; xg[j][1] = a4.y; xg[j][2] = a4.z; xg[j][3] = a4.w;
                xg[j][4] = b4.x; xg[j][5] = b4.y; xg[j][6] = b4.z; xg[j][7] = b4.w;
                if (has_rms) {
                    wa[j] = ld_cg_f4_issue(rms_w + e);
                    wb[j] = ld_cg_f4_issue(rms_w + e + 128);
                }
            } else {
                // The partials of head h were written by blocks b0..b1 of the attention phase, one slot each, in
                // block order; merged here in that order, so the result does not depend on which SM ran what.
#pragma unroll
                for (int hw = 0; hw < 2; ++hw) {
                    const int eh = e + 128 * hw;
                    const int h = eh / P.head, d = eh - h * P.head;
                    const float *hp = P.att_part + (int64_t)h * kAttSlots * ps;
                    float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
                    float L = 0.f;
                    if (merge_fast) {
                        const int u0 = h * as.nchunk;
                        const int np = att_block_of(as, u0 + as.nchunk - 1) - att_block_of(as, u0) + 1;
                        float4 o4[kAttFastSlots];
                        float2 ml[kAttFastSlots];
#pragma unroll
                        for (int s2 = 0; s2 < kAttFastSlots; ++s2) {
                            o4[s2] = make_float4(0.f, 0.f, 0.f, 0.f);
                            ml[s2] = make_float2(-INFINITY, 0.f);
                            if (s2 < np) {
                                o4[s2] = ld_cg_f4_issue(hp + (int64_t)s2 * ps + d);
                                ml[s2] = __ldcg(reinterpret_cast<const float2 *>(hp + (int64_t)s2 * ps + P.head));
                            }
                        }
                        float gm = -INFINITY;
#pragma unroll
                        for (int s2 = 0; s2 < kAttFastSlots; ++s2)
                            gm = fmaxf(gm, ml[s2].x);
#pragma unroll
                        for (int s2 = 0; s2 < kAttFastSlots; ++s2) {
                            if (ml[s2].y > 0.f) {
                                const float w = expf(ml[s2].x - gm);
                                L = fmaf(ml[s2].y, w, L);
                                O.x = fmaf(o4[s2].x, w, O.x);
                                O.y = fmaf(o4[s2].y, w, O.y);
                                O.z = fmaf(o4[s2].z, w, O.z);
                                O.w = fmaf(o4[s2].w, w, O.w);
                            }
                        }
                    } else {
                        const float *tw = reinterpret_cast<const float *>(share);
#pragma unroll
                        for (int s2 = 0; s2 < kAttSlots; ++s2) {
                            const float w = tw[h * kAttSlots + s2];
                            if (w > 0.f) {
                                const float4 o = ld_cg_f4_issue(hp + (int64_t)s2 * ps + d);
                                O.x = fmaf(o.x, w, O.x);
                                O.y = fmaf(o.y, w, O.y);
                                O.z = fmaf(o.z, w, O.z);
                                O.w = fmaf(o.w, w, O.w);
                            }
                        }
                        L = tw[P.n_heads * kAttSlots + h];
                    }
                    // ExpSumNormalize.java:33-37 folded into the weighted sum
                    xg[j][4 * hw + 0] = __fdiv_rn(O.x, L);
                    xg[j][4 * hw + 1] = __fdiv_rn(O.y, L);
                    xg[j][4 * hw + 2] = __fdiv_rn(O.z, L);
                    xg[j][4 * hw + 3] = __fdiv_rn(O.w, L);
                }
            }
        }
        if (merge && !merge_fast)
            named_barrier_sync(2, kFCons);   // the table's place is taken by the limbs below
        float ssq = 0.f;
#pragma unroll
        for (int j = 0; j < kFGroupRounds; ++j) {
            const int gi = warp + j * kFusedConsWarps;
            if (gi >= ngroups)   // warp-uniform
                continue;
            float amax = 0.f;
            const float wv[8] = {wa[j].x, wa[j].y, wa[j].z, wa[j].w, wb[j].x, wb[j].y, wb[j].z, wb[j].w};
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                ssq = fmaf(xg[j][q], xg[j][q], ssq);
                xg[j][q] = __fmul_rn(wv[q], xg[j][q]);       // RMSNorm weight (1 where the phase has none)
                amax = fmaxf(amax, fabsf(xg[j][q]));
            }
            amax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(amax)));   // non-negative floats order like their bits
            // 24-bit fixed point: one power-of-two scale per group, |x * f| <= 2^22
            int ex = (int)((__float_as_uint(amax) >> 23) & 0xffu) - 126;   // amax < 2^ex for normal numbers
            if (!(amax > 0.f) || !(amax < 3.0e38f))
                ex = 0;
            ex = max(-90, min(126, ex));
            const float f = __int_as_float((127 + 22 - ex) << 23);
            if (lane == 0)
                inv_tab[gi] = __int_as_float((127 + ex - 22) << 23);
            // three balanced signed byte limbs: after the add-and-flip, bytes 0..2 of z are l0, l1, l2 in
            // [-128, 127] with X = l0 + 256 l1 + 65536 l2
            uint32_t z[8];
#pragma unroll
            for (int q = 0; q < 8; ++q)
                z[q] = ((uint32_t)__float2int_rn(xg[j][q] * f) + 0x00008080u) ^ 0x00008080u;
            uint32_t *dst = reinterpret_cast<uint32_t *>(share) + gi * 64 + lane;
#pragma unroll
            for (int hw = 0; hw < 2; ++hw) {
                const uint32_t t0 = __byte_perm(z[4 * hw], z[4 * hw + 1], 0x5140);
                const uint32_t t2 = __byte_perm(z[4 * hw + 2], z[4 * hw + 3], 0x5140);
                const uint32_t t1 = __byte_perm(z[4 * hw], z[4 * hw + 1], 0x0062);
                const uint32_t t3 = __byte_perm(z[4 * hw + 2], z[4 * hw + 3], 0x0062);
                dst[32 * hw] = __byte_perm(t0, t2, 0x5410);
                dst[(n >> 2) + 32 * hw] = __byte_perm(t0, t2, 0x7632);
                dst[(n >> 1) + 32 * hw] = __byte_perm(t1, t3, 0x5410);
            }
        }
        if (has_rms) {
            ssq = warp_sum(ssq);
            if (lane == 0)
                scratch[warp] = ssq;
        }
    }
    named_barrier_sync(1, kFCons);

    // what a unit of this thread's integer sums is worth: its group's fixed-point unit, times the RMSNorm scalar
    float unit = gvalid ? inv_tab[g] : 0.f;
    if (rms_w != nullptr) {
        const float ssq = warp_sum(lane < kFusedConsWarps ? scratch[lane] : 0.f);   // the same order in every warp and block
        float tot = __fdiv_rn(ssq, (float)n);
        tot = __fadd_rn(tot, 1e-5f);
        unit *= __fdiv_rn(1.0f, __fsqrt_rn(tot));   // RootMeanSquare.java:25-35
    }

    uint32_t xl[4][4][3];
    float xs;
    {
        int s0 = 0, s1 = 0, s2 = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
#pragma unroll
            for (int l = 0; l < 3; ++l) {
                uint4 t = make_uint4(0u, 0u, 0u, 0u);
                if (gvalid)
                    t = *reinterpret_cast<const uint4 *>(share + (size_t)l * n + (size_t)chunk[k] * 16);
                xl[k][0][l] = t.x; xl[k][1][l] = t.y; xl[k][2][l] = t.z; xl[k][3][l] = t.w;
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                s0 = dp4a_us(0x01010101u, xl[k][q][0], s0);
                s1 = dp4a_us(0x01010101u, xl[k][q][1], s1);
                s2 = dp4a_us(0x01010101u, xl[k][q][2], s2);
            }
        }
        xs = fmaf((float)s2, 65536.0f, fmaf((float)s1, 256.0f, (float)s0));
    }
    if (tid == 0)
        fused_trace(P, pidx, 1);

    // Per-thread constants of the stage loop.  The integer pipe runs at half rate and the dot products live on it,
    // so every address computation in the loop costs as much as a dp4a: offsets inside a stage are fixed per
    // thread and phase, shared memory is addressed with 32-bit window addresses, a stage's descriptor is one
    // 16-byte load.
    const int half = (p.paired && rsub >= R / 2) ? 1 : 0;      // second half of a paired stage: the partner matrix
    const int local = rsub - half * (R / 2);                     // row of this thread inside its half
    const int par = (lane >> 2) & 1;
    const uint32_t ring32 = sbase + kFHeader + (uint32_t)P.xarea_bytes;
    const uint32_t row_off = (uint32_t)(rsub * rowbytes + g * 256 + (lane & 3) * 16);
    const uint32_t off_a = row_off + 64u * (uint32_t)par;       // chunks 0 and 2 of the thread (+0, +128)
    const uint32_t off_b = row_off + 64u * (uint32_t)(1 - par); // chunks 1 and 3
    const uint32_t hdr_off = (uint32_t)(p.hdr_off + half * p.half_hdr + 8 * (local * (n >> 8) + g));
    const uint32_t desc32 = sbase + kFDescOff;
    uint32_t e = (uint32_t)(cs.seq % kFDesc), parity = (uint32_t)(cs.seq / kFDesc) & 1u;

    // The block's stages are taken in groups of kFGroup: a warp works through the rows of a group one stage after
    // the other, then folds the group's partial sums with one butterfly and hands them to the epilogue warp in one
    // go.  A warp's chain of waits, loads, dot products, fold and hand-over is serial; per group instead of per
    // stage it costs a quarter as much per row, while the ring still moves in stages of rpp rows.
    for (int g0 = 0; g0 < nmine; g0 += kFGroup) {
        const int cnt = min(kFGroup, nmine - g0);
        float v[kFGroup];
#pragma unroll
        for (int t = 0; t < kFGroup; ++t) {
            v[t] = 0.f;
            if (t >= cnt)
                continue;
            if (!mbar_wait_bounded(sbase + kFBarFull + 8 * e, parity, wait_ns))
                cs.lost = true;
            if (g0 == 0 && t == 0 && tid == 0)
                fused_trace(P, pidx, 4);
            const uint4 d = lds_v4(desc32 + 32u * e);            // off, nrows, e0a, e0b
            const uint32_t slot32 = ring32 + d.x;
            if (gvalid && local < (int)d.y) {
                // rows start on group boundaries: the header of the thread's group is (e0 >> 8) + local * groups per row + g
                const float2 ms = lds_f2(slot32 + hdr_off + (((half ? d.w : d.z) >> 8) << 3));
                const uint32_t sa = slot32 + off_a, sb = slot32 + off_b;
                int a0 = 0, a1 = 0, a2 = 0;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint4 w = lds_v4(((k & 1) ? sb : sa) + ((k & 2) ? 128u : 0u));
                    a0 = dp4a_us(w.x, xl[k][0][0], a0);
                    a1 = dp4a_us(w.x, xl[k][0][1], a1);
                    a2 = dp4a_us(w.x, xl[k][0][2], a2);
                    a0 = dp4a_us(w.y, xl[k][1][0], a0);
                    a1 = dp4a_us(w.y, xl[k][1][1], a1);
                    a2 = dp4a_us(w.y, xl[k][1][2], a2);
                    a0 = dp4a_us(w.z, xl[k][2][0], a0);
                    a1 = dp4a_us(w.z, xl[k][2][1], a1);
                    a2 = dp4a_us(w.z, xl[k][2][2], a2);
                    a0 = dp4a_us(w.w, xl[k][3][0], a0);
                    a1 = dp4a_us(w.w, xl[k][3][1], a1);
                    a2 = dp4a_us(w.w, xl[k][3][2], a2);
                }
                // |a_l| <= 64 * 255 * 128 < 2^24: the conversions are exact
                const float dsum = fmaf((float)a2, 65536.0f, fmaf((float)a1, 256.0f, (float)a0));
                v[t] = fmaf(ms.y, dsum, ms.x * xs) * unit;
            }
            __syncwarp();
            if (lane == 0)
                mbar_arrive(sbase + kFBarEmpty + 8 * e);   // this warp is done with the stage's bytes
            e = (e + 1) & (kFDesc - 1);
            parity ^= (e == 0);
            ++cs.seq;
        }
        const float tot = Fold<kFGroup, 16>::run(v, lane);   // lane t * (32 / kFGroup) holds the sum of stage t
        if (cs.rround > 0) {
            if (!mbar_wait_bounded(sbase + kFBarRedEmpty + 8 * cs.rb, (uint32_t)(cs.rround - 1) & 1u, wait_ns))
                cs.lost = true;
        }
        float *red = reinterpret_cast<float *>(smem + kFRedOff + cs.rb * kFRedStride);
        if (active && (lane & (32 / kFGroup - 1)) == 0) {
            const int t = lane / (32 / kFGroup);
            red[(t * p.rpp + rsub) * p.wpr + wi] = tot;
        }
        __syncwarp();
        if (lane == 0)
            mbar_arrive(sbase + kFBarRedFull + 8 * cs.rb);
        if (++cs.rb == kFRedBufs) {
            cs.rb = 0;
            ++cs.rround;
        }
    }
    if (tid == 0)
        fused_trace(P, pidx, 2);
}

// The attention step of the block: its run of units, each a stage of cached K and V rows in the ring (the
// token's own row comes straight from the cache in global memory).  One pass with an online softmax per
// lane group; the lane groups of the block are merged through shared memory whenever the head changes.
__device__ __forceinline__ void consume_attention(const FusedParams &P, int layer, const AttSplit &as, int pos, uint8_t *smem,
                                                  uint32_t sbase, Consumer &cs, uint64_t wait_ns)
{
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b = blockIdx.x;
    const int head = P.head;
    const int u0 = att_first_unit(as, b), u1 = att_first_unit(as, b + 1);
    const int lpp = head >> 2;
    int gw = 1;
    while (gw < lpp)
        gw <<= 1;
    const int ppw = 32 / gw;
    const int g = lane / gw, li = lane - g * gw;
    const bool act = li < lpp;
    const int nslots = kFusedConsWarps * ppw;
    const int slot = warp * ppw + g;
    const int sstride = head + 4;
    float *marea = reinterpret_cast<float *>(smem + kFHeader);
    const float sq = sqrtf((float)head);
    const float *kc = P.mv[0].k_cache + (int64_t)layer * P.kv_step;
    const float *vc = P.mv[0].v_cache + (int64_t)layer * P.kv_step;

    int cur_h = -1;
    float4 q4 = make_float4(0.f, 0.f, 0.f, 0.f);
    float m = -INFINITY, l = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);

    auto flush = [&](int h) {
        // merge the lane groups in slot order and write the block's partial of head h
        float *mine = marea + slot * sstride;
        if (act)
            *reinterpret_cast<float4 *>(mine + 4 * li) = acc;
        if (li == 0) {
            mine[head] = m;
            mine[head + 1] = l;
        }
        named_barrier_sync(2, kFCons);
        if (tid < head) {
            float M = -INFINITY;
            for (int s = 0; s < nslots; ++s)
                M = fmaxf(M, marea[s * sstride + head]);
            float L = 0.f, O = 0.f;
            for (int s = 0; s < nslots; ++s) {
                const float ms = marea[s * sstride + head];
                const float ls = marea[s * sstride + head + 1];
                if (ls > 0.f) {
                    const float w = expf(ms - M);
                    L = fmaf(ls, w, L);
                    O = fmaf(marea[s * sstride + tid], w, O);
                }
            }
            const int pslot = b - att_block_of(as, h * as.nchunk);
            float *part = P.att_part + ((int64_t)h * kAttSlots + pslot) * sstride;
            __stcg(part + tid, O);
            if (tid == 0) {
                __stcg(part + head, M);
                __stcg(part + head + 1, L);
            }
        }
        named_barrier_sync(2, kFCons);   // the merge area is free again
    };

    for (int u = u0; u < u1; ++u) {
        const int e = cs.seq % kFDesc;
        if (!mbar_wait_bounded(sbase + kFBarFull + 8 * e, (uint32_t)(cs.seq / kFDesc) & 1u, wait_ns))
            cs.lost = true;
        cs.lost = __any_sync(0xffffffffu, cs.lost) != 0;   // the shuffles below need a warp-uniform decision
        const FStage d = *(reinterpret_cast<const FStage *>(smem + kFDescOff) + e);
        const int h = d.seg;
        if (h != cur_h) {
            if (cur_h >= 0)
                flush(cur_h);
            cur_h = h;
            m = -INFINITY;
            l = 0.f;
            acc = make_float4(0.f, 0.f, 0.f, 0.f);
            if (act)
                q4 = __ldcg(reinterpret_cast<const float4 *>(P.q + (int64_t)h * head + 4 * li));
        }
        const bool skip = false;   // a block whose hand-over ran out still works through its stages
        const float *ks = reinterpret_cast<const float *>(smem + kFHeader + P.xarea_bytes + (size_t)d.off);
        const float *vs = reinterpret_cast<const float *>(smem + kFHeader + P.xarea_bytes + (size_t)d.off + (size_t)d.aux);
        const int kvh = h / P.kv_mul;
        for (int i0 = 0; i0 < d.nrows && !skip; i0 += 2 * nslots) {
            float4 kk[2], vv[2];
            float s[2];
#pragma unroll
            for (int u2 = 0; u2 < 2; ++u2) {
                const int i = i0 + u2 * nslots + slot;
                kk[u2] = make_float4(0.f, 0.f, 0.f, 0.f);
                vv[u2] = kk[u2];
                if (act && i < d.nrows) {
                    if (i < d.e0a) {
                        kk[u2] = *reinterpret_cast<const float4 *>(ks + (size_t)i * head + 4 * li);
                        vv[u2] = *reinterpret_cast<const float4 *>(vs + (size_t)i * head + 4 * li);
                    } else {   // the row this token's QKV phase has just written
                        const int64_t row = ((int64_t)kvh * P.seq_len + d.row0 + i) * head + 4 * li;
                        kk[u2] = __ldcg(reinterpret_cast<const float4 *>(kc + row));
                        vv[u2] = __ldcg(reinterpret_cast<const float4 *>(vc + row));
                    }
                }
            }
            float mloc = -INFINITY;
#pragma unroll
            for (int u2 = 0; u2 < 2; ++u2) {
                const int i = i0 + u2 * nslots + slot;
                float dd = kk[u2].x * q4.x;
                dd = fmaf(kk[u2].y, q4.y, dd);
                dd = fmaf(kk[u2].z, q4.z, dd);
                dd = fmaf(kk[u2].w, q4.w, dd);
                for (int o = gw >> 1; o > 0; o >>= 1)
                    dd += __shfl_xor_sync(0xffffffffu, dd, o);
                s[u2] = i < d.nrows ? __fdiv_rn(dd, sq) : -INFINITY;   // AttentionLoop.java:48
                mloc = fmaxf(mloc, s[u2]);
            }
            if (mloc > -INFINITY) {
                const float mn = fmaxf(m, mloc);
                const float sc = expf(m - mn);
                l *= sc;
                acc.x *= sc; acc.y *= sc; acc.z *= sc; acc.w *= sc;
#pragma unroll
                for (int u2 = 0; u2 < 2; ++u2) {
                    const float pw = expf(s[u2] - mn);
                    l += pw;
                    acc.x = fmaf(pw, vv[u2].x, acc.x);
                    acc.y = fmaf(pw, vv[u2].y, acc.y);
                    acc.z = fmaf(pw, vv[u2].z, acc.z);
                    acc.w = fmaf(pw, vv[u2].w, acc.w);
                }
                m = mn;
            }
        }
        __syncwarp();
        if (lane == 0)
            mbar_arrive(sbase + kFBarEmpty + 8 * e);
        ++cs.seq;
    }
    if (cur_h >= 0)
        flush(cur_h);
}

// -------------------------------------------------------------------------------------------------
// epilogue warp
// -------------------------------------------------------------------------------------------------

struct Epilogue {
    int rb, rround;
    bool lost, lost_before;
};

__device__ __forceinline__ void epilogue_phase(const FusedParams &P, const MvParams &p, int layer, int first, int nmine, int pos,
                                               uint8_t *smem, uint32_t sbase, Epilogue &es, uint64_t wait_ns)
{
    const int lane = threadIdx.x & 31;
    const int G = gridDim.x;
    const int R = p.rt * p.rpp;
    const int rs = p.rs;                 // output rows (row pairs) per stage: at most 8, so a group fits the 32 lanes
    const float *rope_c = reinterpret_cast<const float *>(smem + kFRopeOff);
    const float *rope_s = rope_c + 64;
    for (int g0 = 0; g0 < nmine; g0 += kFGroup) {
        const int cnt = min(kFGroup, nmine - g0);
        if (!mbar_wait_bounded(sbase + kFBarRedFull + 8 * es.rb, (uint32_t)es.rround & 1u, wait_ns))
            es.lost = true;
        const float *red = reinterpret_cast<const float *>(smem + kFRedOff + es.rb * kFRedStride);
        const bool skip = false;   // a block whose hand-over ran out still runs its own pipeline to the end
        if (p.epilogue == EPI_QKV_ROPE) {
            // a lane owns a pair of rows: (v0, v1) are rotated together (ApplyRope.java:61-92)
            const int pairs = rs >> 1;
            const int t = lane / pairs, i = lane - t * pairs;
            if (t < cnt && !skip) {
                int seg, row0, nrows;
                stage_rows(p, first + (g0 + t) * G, seg, row0, nrows);
                if (2 * i < nrows) {
                    const float *rt = red + (t * p.rpp) * p.wpr;
                    float v0 = 0.f, v1 = 0.f;
                    for (int w = 0; w < p.wpr; ++w) {
                        v0 += rt[(2 * i) * p.wpr + w];
                        v1 += rt[(2 * i + 1) * p.wpr + w];
                    }
                    const int row = row0 + 2 * i;
                    if (seg == 2) {
                        const int kvh = row / p.head, d = row - kvh * p.head;
                        float *dst = p.v_cache + (int64_t)layer * P.kv_step + ((int64_t)kvh * p.seq_len + pos) * p.head + d;
                        dst[0] = v0;
                        dst[1] = v1;
                    } else {
                        const int d = row % p.head;
                        const float c = rope_c[d >> 1], sn = rope_s[d >> 1];
                        const float r0 = __fsub_rn(__fmul_rn(v0, c), __fmul_rn(v1, sn));
                        const float r1 = __fadd_rn(__fmul_rn(v0, sn), __fmul_rn(v1, c));
                        if (seg == 0) {
                            p.q_out[row] = r0;
                            p.q_out[row + 1] = r1;
                        } else {
                            const int kvh = row / p.head;
                            float *dst = p.k_cache + (int64_t)layer * P.kv_step + ((int64_t)kvh * p.seq_len + pos) * p.head + d;
                            dst[0] = r0;
                            dst[1] = r1;
                        }
                    }
                }
            }
        } else {
            const int t = lane / rs, i = lane - t * rs;
            if (t < cnt && !skip) {
                int seg, row0, nrows;
                stage_rows(p, first + (g0 + t) * G, seg, row0, nrows);
                if (i < nrows) {
                    const float *rt = red + (t * p.rpp) * p.wpr;
                    if (p.epilogue == EPI_SWIGLU) {
                        float v1 = 0.f, v3 = 0.f;
                        for (int w = 0; w < p.wpr; ++w) {
                            v1 += rt[i * p.wpr + w];
                            v3 += rt[(R / 2 + i) * p.wpr + w];
                        }
                        p.y[row0 + i] = __fmul_rn(__fmul_rn(v1, sigmoid_accurate(v1)), v3);   // Silu.java:122-132 order
                    } else {   // EPI_RESIDUAL
                        float a = 0.f;
                        for (int w = 0; w < p.wpr; ++w)
                            a += rt[i * p.wpr + w];
                        atomicAdd(p.y + row0 + i, a);   // one add per element and phase: deterministic
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0)
            mbar_arrive(sbase + kFBarRedEmpty + 8 * es.rb);
        if (++es.rb == kFRedBufs) {
            es.rb = 0;
            ++es.rround;
        }
    }
}

}  // namespace

// =============================================================================================
// the kernel
// =============================================================================================

__global__ void __launch_bounds__(kFusedThreads, 1) fused_layers_kernel(const __grid_constant__ FusedParams P)
{
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int b = blockIdx.x, G = gridDim.x;
    const uint32_t sbase = smem_u32(smem);
    const uint64_t wait_ns = (uint64_t)P.timeout_us * 1000ull;

    if (tid < kFDesc) {
        mbar_init(sbase + kFBarFull + 8 * tid, 4);         // the four producer lanes
        mbar_init(sbase + kFBarEmpty + 8 * tid, kFusedConsWarps);
    }
    if (tid < kFRedBufs) {
        mbar_init(sbase + kFBarRedFull + 8 * tid, kFusedConsWarps);
        mbar_init(sbase + kFBarRedEmpty + 8 * tid, 1);
    }
    if (tid < 32)
        mbar_fence_init();
    __syncthreads();
    pdl_launch_dependents();   // the classifier kernel behind may take the SMs as they free up

    // ------------------------------------------------------------------------------ producer
    if (warp == kFusedConsWarps) {
        if (lane >= 4)
            return;
        Producer pr;
        pr.smem = smem;
        pr.sbase = sbase;
        pr.ring_base = sbase + kFHeader + (uint32_t)P.xarea_bytes;
        pr.vhead = 0;
        pr.ring_bytes = P.ring_bytes;
        pr.seq = pr.tail = 0;
        pr.lost = false;
        pr.wait_ns = wait_ns;
        const uint64_t pol = policy_evict_first();
        pr.pos = -1;
        pr.as = AttSplit{};
        pr.off = 0;
        int rot = 0;
        for (int layer = 0; layer < P.n_layers; ++layer) {
#pragma unroll 1
            for (int k = 0; k < 4; ++k) {
                const MvParams &p = P.mv[k];
                const int S = p.total_stages;
                if (!(P.debug_no_copy & 8) && lane == 0) fused_trace(P, layer * 5 + (k == 0 ? 0 : k + 1), 5);
                for (int s = first_stage_of(b, rot, G); s < S; s += G) {
                    produce_ring_stage(pr, P, p, k, layer, s, pol, lane);
                }
                if (!(P.debug_no_copy & 8) && lane == 0) fused_trace(P, layer * 5 + (k == 0 ? 0 : k + 1), 6);
                rot = (rot + S) % G;
                if (k == 0) {
                    producer_learn_pos(pr, P, G);
                    if (b < pr.as.ga) {
                        const int u0 = att_first_unit(pr.as, b), u1 = att_first_unit(pr.as, b + 1);
                        if (lane == 0) fused_trace(P, layer * 5 + 1, 5);
                        for (int u = u0; u < u1; ++u) {
                            produce_att_stage(pr, P, layer, u, pr.as, pr.pos, lane);
                        }
                        if (lane == 0) fused_trace(P, layer * 5 + 1, 6);
                    }
                }
            }
        }
        // No copy of this block may still be in flight when its shared memory is handed to the next block: the
        // consumers have waited for every stage, so these waits return at once unless a wait ran out before.
        for (int d = max(pr.tail, pr.seq - kFDesc); d < pr.seq; ++d)
            mbar_wait_bounded(sbase + kFBarFull + 8 * (d % kFDesc), (uint32_t)(d / kFDesc) & 1u, wait_ns);
        if (pr.lost && lane == 0)
            atomicOr(&P.state->status, L2J_DS_WAIT_TIMEOUT);
        return;
    }

    // Everything below reads what the kernel in front wrote (x, the position).
    pdl_wait();
    const int pos = __ldcg(&P.state->cur_pos);
    const AttSplit as = att_split(P, pos, G);
    const unsigned int target = __ldcg(P.epoch) * (unsigned int)G;
    const bool lost_at_entry = (__ldcg(&P.state->status) & L2J_DS_WAIT_TIMEOUT) != 0;

    // ------------------------------------------------------------------------------ epilogue warp
    if (warp == kFusedConsWarps + 1) {
        Epilogue es;
        es.rb = es.rround = 0;
        es.lost = es.lost_before = lost_at_entry;
        {
            float *rope_c = reinterpret_cast<float *>(smem + kFRopeOff);
            const int half = P.head >> 1;
            for (int i = lane; i < half; i += 32) {
                rope_c[i] = __ldg(P.mv[0].rope_cos + (int64_t)pos * half + i);
                rope_c[64 + i] = __ldg(P.mv[0].rope_sin + (int64_t)pos * half + i);
            }
            __syncwarp();
        }
        int rot = 0;
        for (int layer = 0; layer < P.n_layers; ++layer) {
#pragma unroll 1
            for (int k = 0; k < 4; ++k) {
                const MvParams &p = P.mv[k];
                const int S = p.total_stages;
                const int first = first_stage_of(b, rot, G);
                const int nmine = first < S ? (S - first + G - 1) / G : 0;
                rot = (rot + S) % G;
                epilogue_phase(P, p, layer, first, nmine, pos, smem, sbase, es, wait_ns);
                // every result of the block in this phase was written by this warp; the release is cumulative
                __syncwarp();
                const int pidx = layer * 5 + (k == 0 ? 0 : k + 1);
                if (lane == 0) {
                    red_release_add_u32(P.sync + (int64_t)kSyncStride * pidx, 1u);
                    fused_trace(P, pidx, 3);
                }
            }
        }
        if (es.lost && !es.lost_before && lane == 0)
            atomicOr(&P.state->status, L2J_DS_WAIT_TIMEOUT);
        return;
    }

    // ------------------------------------------------------------------------------ consumers
    Consumer cs;
    cs.seq = 0;
    cs.rb = cs.rround = 0;
    cs.lost = cs.lost_before = lost_at_entry;
    int rot = 0;
    for (int layer = 0; layer < P.n_layers; ++layer) {
#pragma unroll 1
        for (int k = 0; k < 4; ++k) {
            const MvParams &p = P.mv[k];
            const int S = p.total_stages;
            const int first = first_stage_of(b, rot, G);
            const int nmine = first < S ? (S - first + G - 1) / G : 0;
            rot = (rot + S) % G;
            const int pidx = layer * 5 + (k == 0 ? 0 : k + 1);
            if (nmine > 0) {
                if (tid == 0)
                    fused_trace(P, pidx, 7);
                if (pidx > 0)   // the first phase's input came from the kernel in front
                    consumers_wait(P.sync + (int64_t)kSyncStride * (pidx - 1), target, smem, cs, wait_ns);
                if (tid == 0)
                    fused_trace(P, pidx, 0);
                const float *rms_w = p.rms_w ? p.rms_w + (int64_t)layer * P.rms_step : nullptr;
                const float wmax = p.rms_w ? __ldg(P.rms_wmax + 2 * layer + (k == 2 ? 1 : 0)) : 1.0f;
                consume_ring_phase(P, p, layer, nmine, k == 1, rms_w, wmax, as, smem, sbase, cs, wait_ns, pidx);
            }
            if (k == 0) {
                // attention over positions 0..pos (Run.java:450-478)
                const int aidx = layer * 5 + 1;
                if (b < as.ga) {
                    consumers_wait(P.sync + (int64_t)kSyncStride * (aidx - 1), target, smem, cs, wait_ns);
                    if (tid == 0)
                        fused_trace(P, aidx, 0);
                    consume_attention(P, layer, as, pos, smem, sbase, cs, wait_ns);
                    if (tid == 0)
                        fused_trace(P, aidx, 2);
                    // flush() ended with a barrier of all consumers: their partials are written
                }
                if (tid == 0) {
                    red_release_add_u32(P.sync + (int64_t)kSyncStride * aidx, 1u);
                    fused_trace(P, aidx, 3);
                }
            }
        }
    }
    if (cs.lost && !cs.lost_before && lane == 0)
        atomicOr(&P.state->status, L2J_DS_WAIT_TIMEOUT);
}

cudaError_t prepare_fused(int *max_smem)
{
    int dev = 0, optin = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess)
        return e;
    if ((e = cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) != cudaSuccess)
        return e;
    if (max_smem)
        *max_smem = optin;
    if ((e = cudaFuncSetAttribute(fused_layers_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, optin)) != cudaSuccess)
        return e;
    return cudaFuncSetAttribute(fused_layers_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

cudaError_t launch_fused(cudaStream_t stream, bool pdl, int grid, int smem_bytes, const FusedParams &p)
{
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kFusedThreads);
    cfg.dynamicSmemBytes = (size_t)smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, fused_layers_kernel, p);
}

}  // namespace l2j
