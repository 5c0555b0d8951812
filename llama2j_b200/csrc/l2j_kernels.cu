// Kernels of the decode path for sm_100a.
//
// The hot kernel is matvec_ring_kernel: a group-quantised (or FP32) matrix-vector product whose
// weights are streamed by the TMA engine (untiled bulk copies) into a shared-memory ring, one
// persistent block per SM, with the per-token elementwise work (RMSNorm, RoPE + KV-cache write,
// residual add, SwiGLU, arg-max) fused into its prologue and epilogue.  Every kernel of a token
// is chained with programmatic dependent launch: the producer thread of the next kernel starts
// filling its ring while the previous kernel is still draining, so HBM does not idle at kernel
// boundaries.  All waits are bounded; a wait that runs out sets a bit in the device status word.
//
// Reference counterparts (paths relative to src/main/java/com/lastbot/llama2j/):
//   matvec_ring_kernel<u8>   kernel/MatMul.java:360-444 (matMulI8), with RootMeanSquare.java:78-118,
//                            WeightNormalizeAndScale.java:191-239, ApplyRope.java:144-182,
//                            Accum.java:70-83, Silu.java:118-135 fused in, and the two KV-cache
//                            copies of Run.java:438-444
//   matvec_ring_kernel<f32>  kernel/MatMul.java:446-464 (matMulFP32) + Sampler.java:46-57
//   attention_kernel         AttentionLoop.java:116-164, ExpSumNormalize.java:82-131,
//                            AccumWeightedValue.java:148-173 (3 launches per head there)
//   begin_kernel             the embedding row copy of Run.java:362-363
//   quant_encode_kernel      Quant.java:156-193

#include "l2j_device.cuh"
#include "l2j_internal.h"

#include <cfloat>
#include <cmath>
#include <cooperative_groups.h>
#include <cstdlib>

#define L2J_DS_WAIT_TIMEOUT 0x1
#define L2J_DS_BAD_POS 0x2
#define L2J_DS_BAD_TOKEN 0x4
#define L2J_DS_BAD_LINK 0x8

namespace l2j {

// =============================================================================================
// epilogue math shared by the fused and the plain kernels
// =============================================================================================

// Rows (row, row+1) of segment `seg` of the QKV product: rotate q and k pairs by the position's
// angle (ApplyRope.java:61-92 arithmetic, no fused multiply-add), write q to its vector and k, v
// into the cache at [kv_head][pos][d].
__device__ __forceinline__ void epi_qkv_pair(const MvParams &p, int seg, int row, float v0, float v1, int pos,
                                             const float *cos_row, const float *sin_row)
{
    if (seg == 2) {
        const int kvh = row / p.head, d = row - kvh * p.head;
        float *dst = p.v_cache + ((int64_t)kvh * p.seq_len + pos) * p.head + d;
        dst[0] = v0;
        dst[1] = v1;
        return;
    }
    const int d = row % p.head;
    const float c = cos_row[d >> 1];   // the RoPE table row of this position
    const float s = sin_row[d >> 1];
    const float r0 = __fsub_rn(__fmul_rn(v0, c), __fmul_rn(v1, s));
    const float r1 = __fadd_rn(__fmul_rn(v0, s), __fmul_rn(v1, c));
    if (seg == 0) {
        p.q_out[row] = r0;
        p.q_out[row + 1] = r1;
    } else {
        const int kvh = row / p.head;
        float *dst = p.k_cache + ((int64_t)kvh * p.seq_len + pos) * p.head + d;
        dst[0] = r0;
        dst[1] = r1;
    }
}

// Silu.java:122-132 order: (value * sigmoid) * hb2, with an accurate sigmoid.
__device__ __forceinline__ float epi_swiglu(float v1, float v3)
{
    return __fmul_rn(__fmul_rn(v1, sigmoid_accurate(v1)), v3);
}

// Grid-wide arg-max finish, run by the block that arrives last: lowest index wins ties, which is
// Sampler.argmax's "first maximum" (Sampler.java:46-57).  Also advances the device-side greedy
// loop of Run.java:635-642: forced prompt token while the prompt lasts, else the arg-max.
__device__ void finish_argmax_warp(const MvParams &p, int nblocks, int lane)
{
    float bv = -FLT_MAX;
    int bi = 0x7fffffff;
    for (int b = lane; b < nblocks; b += 32) {
        const float v = __ldcg(p.blk_val + b);
        const int i = __ldcg(p.blk_idx + b);
        if (v > bv || (v == bv && i < bi)) {
            bv = v;
            bi = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) {
            bv = ov;
            bi = oi;
        }
    }
    if (p.ll.tp && p.ll.out_vec == TPV_CAND) {
        // Tensor parallel: this rank holds a block of the vocabulary.  Its (maximum, index) goes to every rank
        // as two (value, sequence number) pairs; every rank then takes the best of all candidates, lowest
        // index first, so all ranks choose the same token without a further message.
        const int n = p.ll.tp->n, me = p.ll.tp->rank;
        const int seq = (int)(__ldcg(p.ll.epoch) * (unsigned int)p.ll.kernels + (unsigned int)p.ll.out_idx + 1u);
        if (lane == 0)
            for (int r = 0; r < n; ++r) {
                st_pair(p.ll.tp->ll[TPV_CAND][r] + 2 * me, bv, seq);
                st_pair(p.ll.tp->ll[TPV_CAND][r] + 2 * me + 1, __int_as_float(bi), seq);
            }
        bv = -FLT_MAX;
        bi = 0x7fffffff;
        if (lane < n) {
            const float2 *mine = p.ll.tp->ll[TPV_CAND][me] + 2 * lane;
            float4 c = ld_pairs2(mine);
            const long long c0 = sm_clock();
            while (__float_as_int(c.y) != seq || __float_as_int(c.w) != seq) {
                if (sm_clock() - c0 > 2000ll * p.timeout_us) {
                    atomicOr(&p.state->status, 0x1);   // L2J_DS_WAIT_TIMEOUT
                    break;
                }
                c = ld_pairs2(mine);
            }
            bv = c.x;
            bi = __float_as_int(c.z);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) {
                bv = ov;
                bi = oi;
            }
        }
    }
    if (lane == 0) {
        SeqState *st = p.state;
        if (bi == 0x7fffffff)
            bi = 0;
        const int pos = __ldcg(&st->cur_pos);
        st->argmax = bi;
        int next = bi;
        if (pos < __ldcg(&st->n_prompt) && p.prompt)
            next = __ldcg(p.prompt + pos);
        if (p.out_tokens)
            p.out_tokens[pos] = next;
        st->token = next;
        st->pos = pos + 1;
        st->cls_counter = 0;
        __threadfence();
    }
}

// =============================================================================================
// matvec_ring_kernel
//
// Persistent blocks, one per SM, that pull work (stages of a few matrix rows) from a global counter.
// Warp roles:
//   consumer warps 0..nw-1   wpr warps span one row, rpp such groups work on rpp rows at once, RT rows
//                            each per stage; every thread keeps its slice of x in registers.  Rows of
//                            whole quantisation groups (GRP): four lanes share a group, a thread owns
//                            64 bytes of it.  Otherwise a lane owns CPT 16-byte chunks a warp apart
//   producer warp nw         one thread claims stages and streams their rows into the shared-memory
//                            ring with bulk copies, as far ahead as the ring allows.  It does not
//                            wait for the previous kernel (weights never depend on activations), so
//                            under programmatic dependent launch the ring fills while the previous
//                            kernel is still running
//   epilogue warp nw+1       adds up the per-warp partial sums of a stage and applies the fused
//                            epilogue, decoupled from the consumers by a ring of reduction buffers
//
// Work is claimed dynamically because blocks of consecutive kernels share the SMs: the hardware may
// place two blocks of one kernel on one SM and none on another, and a static split would then leave
// the kernel waiting for the doubly loaded SM.
//
// u8 weights: x is converted once per block to 24-bit fixed point (one power-of-two scale per
// vector) and split into three balanced signed byte limbs, so that 16 weight bytes cost 12 dp4a
// instructions (u8 weight x s8 limb, exact s32 accumulation) instead of 16 conversions + 16 FMAs.
// The limb sums (per 64 bytes in the grouped mapping, per 16 bytes otherwise) are recombined in FP32
// and scaled by the group's (min, scale):
//   sum_j (b_j * s + m) * x_j  =  s * sum_j b_j x_j  +  m * sum_j x_j.
// The grid's step is at most 2^-25 of the vector's largest element, the order of one FP32 rounding of
// a product.
//
// LL: the input vector arrives as (value, sequence number) pairs from the ranks of a tensor-parallel
// group (see LlLink); instantiated apart so that the plain kernels do not pay for its registers.
// =============================================================================================

struct StageDesc {
    int seg, row0, nrows, e0a, e0b, pad0, pad1, pad2;   // nrows == 0 marks the end of the block's work
};

// Stage index -> (segment, first row, row count).  The stage counts per segment come from the host.
__device__ __forceinline__ void decode_stage(const MvParams &p, int rs, int s, int &seg, int &row0, int &nrows)
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
    row0 = s * rs;
    nrows = min(rs, p.seg[seg].rows - row0);
}

// Brings one stage of launch `q` (this one or the next in the stream) into L2 ahead of its bulk copy.
__device__ __forceinline__ void prefetch_stage(const MvParams &q, int s)
{
    int seg, row0, nrows;
    decode_stage(q, q.rs, s, seg, row0, nrows);
    const uint32_t pbytes = (uint32_t)nrows * (uint32_t)q.rowbytes;
    if (q.f32) {
        bulk_prefetch_l2(reinterpret_cast<const float *>(q.seg[seg].payload) + q.seg[seg].flat0 + (int64_t)row0 * q.n, pbytes);
        return;
    }
    const int nh = q.paired ? 2 : 1;
    for (int h = 0; h < nh; ++h) {
        const MvSeg &sg = q.seg[q.paired ? h : seg];
        const int64_t flat = sg.flat0 + (int64_t)row0 * q.n;
        const int64_t ga = (flat >> 8) & ~(int64_t)1;
        const int64_t gl = (flat + pbytes - 1) >> 8;
        bulk_prefetch_l2(sg.payload + flat, pbytes);
        bulk_prefetch_l2(sg.hdr + ga, (uint32_t)(((gl - ga + 2) & ~(int64_t)1) * 8));
    }
}

constexpr uint64_t kShortWaitNs = 2000;   // limit of every wait once one has run out

// Waits for the kernel in front: on its hand-over counter if the launch has one, else for the grid to
// complete.  Called by all `nthreads` threads that share barrier `bar_id`; `flag` is a shared-memory word
// of theirs.  Returns false if the bounded wait ran out.
__device__ __forceinline__ bool chain_wait_group(const ChainLink &c, bool poller, int bar_id, int nthreads, uint64_t timeout_ns,
                                                 volatile int *flag, const SeqState *st = nullptr)
{
    if (c.wait_counter == nullptr) {
        pdl_wait();
        return true;
    }
    // One thread polls: thousands of pollers on one line would stand in the way of the bumps themselves.
    if (poller) {
        const unsigned int target = __ldcg(c.epoch) * c.wait_blocks;
        int ok = (int)(ld_acquire_u32(c.wait_counter) - target) >= 0;
        if (!ok) {
            // once a wait has run out somewhere in this forward, every later one gives up quickly
            if (st && (__ldcg(&st->status) & L2J_DS_WAIT_TIMEOUT))
                timeout_ns = kShortWaitNs;
            ok = counter_wait_bounded(c.wait_counter, target, timeout_ns) ? 1 : 0;
        }
        *flag = ok;
    }
    named_barrier_sync(bar_id, nthreads);   // orders the other threads' loads behind the poller's acquire
    return *flag != 0;
}

// Reports a block's results as visible: bumps the launch's counter.  Called by one thread after a barrier
// with the threads that wrote the results.
__device__ __forceinline__ void chain_signal(const ChainLink &c)
{
    if (c.done_counter != nullptr)
        red_release_add_u32(c.done_counter, 1u);
}

// Sequence number of kernel `idx` of the forward in flight (see LlLink).
__device__ __forceinline__ int ll_seq(const LlLink &l, int idx)
{
    return (int)(__ldcg(l.epoch) * (unsigned int)l.kernels + (unsigned int)idx + 1u);
}

// One result to every rank's receive buffer.
__device__ __forceinline__ void ll_send(const LlLink &l, int n_ranks, int index, float v, int seq)
{
    for (int r = 0; r < n_ranks; ++r)
        st_pair(l.tp->ll[l.out_vec][r] + index, v, seq);
}

constexpr int kRedBufs = 4;
constexpr int kBarFull = 0;                       // uint64 full[16]
constexpr int kBarEmpty = 128;                    // uint64 empty[16]
constexpr int kBarRedFull = 256;                  // uint64 red_full[4]
constexpr int kBarRedEmpty = 288;                 // uint64 red_empty[4]
constexpr int kBarXIssued = 320;                  // uint64: the consumers have issued the loads of x
constexpr int kScratchOff = 384;                  // float scratch[64]
constexpr int kDescOff = 640;                     // StageDesc desc[16]
constexpr int kRedOff = 1152;                     // 4 x (16-byte header + 128 floats: up to 8 rows x 16 warps)
constexpr int kRedStride = 528;
constexpr int kRopeOff = 3328;                    // float cos[64], sin[64] of the current position
constexpr int kSmemHeader = 3840;                 // end of the fixed part (128-byte aligned)
constexpr int kRingMaxThreads = 640;              // 18 consumer warps + producer + epilogue warp: 102 registers per thread
constexpr int kPrologueRounds = 8;                // 16-byte loads of x per consumer thread in the prologue

__device__ __forceinline__ int dp4a_u8s8(uint32_t a, uint32_t b, int c)
{
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Reduces RT per-lane values over the warp with a halving butterfly (RT - 1 + log2(32 / RT)
// shuffles instead of 5 * RT); afterwards lane t * (32 / RT) holds the sum of v[t] over all lanes.
template <int RT, int STEP>
struct WarpFold {
    // STEP: lane bit that separates the upper half of the rows from the lower half at this level
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
            return WarpFold<H, STEP / 2>::run(k, lane);
        }
    }
};

template <int RT>
__device__ __forceinline__ float warp_sum_rows(const float (&v)[RT], int lane)
{
    static_assert(RT == 1 || RT == 2 || RT == 4 || RT == 8, "RT");
    return WarpFold<RT, 16>::run(v, lane);
}

// Optional in-kernel timeline (p.trace != nullptr): slot k of the block gets the global timer (ns).
// 0 entry, 1 producer's first copy issued, 2 producer's last copy issued, 3 consumer prologue done,
// 4 first stage landed, 5 consumers done, 6 epilogue warp done, 7 global timer (ns) at entry.
__device__ __forceinline__ void trace_mark(const MvParams &p, int k)
{
    if (p.trace)
        p.trace[blockIdx.x * 16 + k] = (unsigned long long)global_timer_ns();
}

template <bool F32, bool GRP, int CPT, int RT, bool LL>
__global__ void __launch_bounds__(kRingMaxThreads, 1) matvec_ring_kernel(const __grid_constant__ MvParams p)
{
    constexpr int EPC = F32 ? 4 : 16;   // elements per 16-byte chunk
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int nw = p.rpp * p.wpr;          // consumer warps
    const int ncons = nw * 32;
    const int nstage = p.nstage;
    const uint32_t sbase = smem_u32(smem);
    const uint32_t ring_base = sbase + kSmemHeader + (uint32_t)p.xshare_bytes;   // the ring follows the shared copy of x

    // The parameter block of every launch is cold in the constant cache; reading one word of each of
    // its 128-byte lines up front makes the block pay one miss instead of one per line along the
    // serial set-up below.
    {
        const int t0 = p.nseg, t1 = p.epilogue, t2 = p.tail_prefetch;
        asm volatile("" ::"r"(t0), "r"(t1), "r"(t2));
    }

    if (tid == 0) {
        trace_mark(p, 0);
        if (p.trace)
            p.trace[blockIdx.x * 16 + 7] = global_timer_ns();
    }
    if (tid < nstage) {
        mbar_init(sbase + kBarFull + 8 * tid, 1);         // one arrive(.expect_tx) by the producer
        mbar_init(sbase + kBarEmpty + 8 * tid, nw);       // one arrive per consumer warp
    }
    if (tid < kRedBufs) {
        mbar_init(sbase + kBarRedFull + 8 * tid, nw);
        mbar_init(sbase + kBarRedEmpty + 8 * tid, 1);
    }
    if (tid == 0)
        mbar_init(sbase + kBarXIssued, nw);
    if (tid < 32)
        mbar_fence_init();
    __syncthreads();
    pdl_launch_dependents();   // the next kernel's blocks may take the SMs as they free up

    const int R = RT * p.rpp;                       // rows of a stage in shared memory
    const int rs = p.paired ? R / 2 : R;            // matrix rows (row pairs) a stage advances
    const int rowbytes = F32 ? p.n * 4 : p.n;
    const uint64_t wait_ns = (uint64_t)p.timeout_us * 1000ull;

    // ------------------------------------------------------------------------------ producer
    if (warp == nw) {
        if (lane == 0) {
            const int S = p.total_stages;
            const uint64_t pol = policy_evict_first();
            bool lost = false, first = true;
            int slot = 0, round = 0;
            // The first `nstatic` stages of a block are fixed (block index + j * grid), so that the blocks
            // do not all queue up on the counter at kernel start; the rest is claimed from the global
            // counter, always one claim ahead of the stage being issued.
            const unsigned int grid = gridDim.x;
            const unsigned int nstatic = (unsigned int)max(1, S / (2 * (int)grid));
            unsigned int issued = 0;
            unsigned int pending = 0xfffffffeu, pending2 = 0xfffffffeu;   // two claims in flight once the first stage is on its way
            bool gate_open = false;
            for (;;) {
                // Only `early_fill` stages are issued before the consumers have put their loads of x on the
                // wire: a full ring fill in front of those loads would delay them by microseconds.
                if (!gate_open && issued >= (unsigned int)p.early_fill) {
                    if (!mbar_wait_bounded(sbase + kBarXIssued, 0u, wait_ns))
                        lost = true;
                    gate_open = true;
                }
                if (round > 0) {
                    if (!mbar_wait_bounded(sbase + kBarEmpty + 8 * slot, (uint32_t)(round - 1) & 1u,
                                           wait_ns))
                        lost = true;
                }
                const uint32_t full = sbase + kBarFull + 8 * slot;
                StageDesc *desc = reinterpret_cast<StageDesc *>(smem + kDescOff) + slot;
                unsigned int cur;
                if (issued < nstatic) {
                    cur = blockIdx.x + issued * grid;
                } else {
                    cur = pending;
                    pending = pending2;
                    pending2 = nstatic * grid + atomicAdd(p.work, 1u);
                }
                ++issued;
                if (cur >= (unsigned int)S) {
                    desc->nrows = 0;            // end marker: a stage without data
                    mbar_arrive(full);
                    if (first) {                // nothing was issued: still take part in the counter protocol
                        pending = nstatic * grid + atomicAdd(p.work, 1u);
                        pending2 = pending;
                    }
                    break;
                }
                int seg, row0, nrows;
                decode_stage(p, rs, (int)cur, seg, row0, nrows);
                const uint32_t dst = ring_base + (uint32_t)slot * (uint32_t)p.slot_bytes;
                desc->seg = seg;
                desc->row0 = row0;
                desc->nrows = nrows;
                const uint32_t pbytes = (uint32_t)nrows * (uint32_t)rowbytes;
                if (F32) {
                    const float *src = reinterpret_cast<const float *>(p.seg[seg].payload) + p.seg[seg].flat0 +
                                       (int64_t)row0 * p.n;
                    mbar_arrive_expect_tx(full, pbytes);
                    bulk_g2s(dst, src, pbytes, full, pol);
                } else if (!p.paired) {
                    const int64_t flat = p.seg[seg].flat0 + (int64_t)row0 * p.n;
                    const int64_t ga = (flat >> 8) & ~(int64_t)1;
                    const int64_t gl = (flat + pbytes - 1) >> 8;
                    const uint32_t hbytes = (uint32_t)(((gl - ga + 2) & ~(int64_t)1) * 8);
                    desc->e0a = (int)(flat - ga * 256);
                    desc->e0b = 0;
                    mbar_arrive_expect_tx(full, pbytes + hbytes);
                    bulk_g2s(dst, p.seg[seg].payload + flat, pbytes, full, pol);
                    bulk_g2s(dst + (uint32_t)p.hdr_off, p.seg[seg].hdr + ga, hbytes, full, pol);
                } else {
                    int64_t flat[2], ga[2];
                    uint32_t hbytes[2];
                    for (int h = 0; h < 2; ++h) {
                        flat[h] = p.seg[h].flat0 + (int64_t)row0 * p.n;
                        ga[h] = (flat[h] >> 8) & ~(int64_t)1;
                        const int64_t gl = (flat[h] + pbytes - 1) >> 8;
                        hbytes[h] = (uint32_t)(((gl - ga[h] + 2) & ~(int64_t)1) * 8);
                    }
                    desc->e0a = (int)(flat[0] - ga[0] * 256);
                    desc->e0b = (int)(flat[1] - ga[1] * 256);
                    mbar_arrive_expect_tx(full, 2 * pbytes + hbytes[0] + hbytes[1]);
                    for (int h = 0; h < 2; ++h) {
                        bulk_g2s(dst + (uint32_t)(h * (R / 2)) * (uint32_t)rowbytes, p.seg[h].payload + flat[h], pbytes,
                                 full, pol);
                        bulk_g2s(dst + (uint32_t)p.hdr_off + (uint32_t)(h * p.half_hdr), p.seg[h].hdr + ga[h], hbytes[h],
                                 full, pol);
                    }
                }
                if (first) {
                    trace_mark(p, 1);
                    first = false;
                    pending = nstatic * grid + atomicAdd(p.work, 1u);
                    pending2 = nstatic * grid + atomicAdd(p.work, 1u);
                }
                if (++slot == nstage) {
                    slot = 0;
                    ++round;
                }
            }
            trace_mark(p, 2);
            // Out of work: while the consumers drain the ring, start HBM -> L2 for the stages the next launch
            // will ask for first, so that the memory system does not run dry between the two kernels.
            if (p.next && p.tail_prefetch > 0) {
                const int ns = p.next->total_stages;
                for (int j = 0; j < p.tail_prefetch; ++j) {
                    const int st = (int)blockIdx.x + j * (int)gridDim.x;
                    if (st < ns)
                        prefetch_stage(*p.next, st);
                }
            }
            // The block that learns last that the work has run out re-arms the counters for the next launch.
            __threadfence();
            if (pending != 0xffffffffu && pending2 != 0xffffffffu && atomicAdd(p.work + 1, 1u) == gridDim.x - 1) {
                __threadfence();
                p.work[0] = 0;
                p.work[1] = 0;
                __threadfence();
            }
            if (lost)
                atomicOr(&p.state->status, L2J_DS_WAIT_TIMEOUT);
        }
        return;
    }

    // ------------------------------------------------------------------------------ epilogue warp
    if (warp == nw + 1) {
        // With a hand-over counter nothing is needed here: the position was fixed when the forward began and
        // every result this warp writes is computed from data the consumers have waited for.
        if (p.chain.wait_counter == nullptr && !LL)
            pdl_wait();
        const int pos = __ldcg(&p.state->cur_pos);
        bool lost = (__ldcg(&p.state->status) & L2J_DS_WAIT_TIMEOUT) != 0;
        const bool lost_before = lost;
        float *rope_c = reinterpret_cast<float *>(smem + kRopeOff);
        float *rope_s = rope_c + 64;
        if (p.epilogue == EPI_QKV_ROPE) {
            const int half = p.head >> 1;
            for (int i = lane; i < half; i += 32) {
                rope_c[i] = __ldg(p.rope_cos + (int64_t)pos * half + i);
                rope_s[i] = __ldg(p.rope_sin + (int64_t)pos * half + i);
            }
            __syncwarp();
            // This warp has nothing to do until the first stage is reduced: ask L2 for the cached K and V rows
            // of the heads this launch computes.  The attention kernel behind starts with a load of exactly
            // those rows, and at short contexts that round trip (to HBM otherwise) is most of its run time.
            if (pos > 0 && pos < p.kv_prefetch_below) {
                constexpr int kRows = 32;                                  // 16 KB at head size 128
                const int h0 = p.seg[1].out0 / p.head, nkv = p.seg[1].rows / p.head;
                const int cpp = (pos + kRows - 1) / kRows;                 // chunks per head
                const int total = 2 * nkv * cpp;
                for (int i = (int)blockIdx.x * 32 + lane; i < total; i += (int)gridDim.x * 32) {
                    const int which = i / (nkv * cpp), rem = i - which * nkv * cpp;
                    const int h = rem / cpp, c = rem - h * cpp;
                    const float *row = (which ? p.v_cache : p.k_cache) + ((int64_t)(h0 + h) * p.seq_len + c * kRows) * p.head;
                    bulk_prefetch_l2(row, (uint32_t)(min(kRows, pos - c * kRows) * p.head) * 4u);
                }
            }
        }
        float best_v = -FLT_MAX;
        int best_i = 0x7fffffff;
        int rb = 0, rround = 0;
        const int tp_n = (p.ll.tp && p.ll.out_vec >= 0) ? p.ll.tp->n : 0;
        const int seq_out = tp_n ? ll_seq(p.ll, p.ll.out_idx) : 0;
        // Block 0's consumer threads stored the assembled residual stream for a later kernel; its results must
        // not be seen before that vector.  The fence is cumulative over what the consumers wrote before they
        // handed the first partial sums to this warp, and it runs while they work on the next stage.
        bool fence_first = LL && p.ll.write_back != nullptr && blockIdx.x == 0;
        for (;;) {
            if (!mbar_wait_bounded(sbase + kBarRedFull + 8 * rb, (uint32_t)rround & 1u, wait_ns))
                lost = true;
            const int *rh = reinterpret_cast<const int *>(smem + kRedOff + rb * kRedStride);
            const int seg = rh[0], nrows = rh[2];
            if (nrows <= 0)
                break;
            const int row0 = rh[1] + p.seg[p.paired ? 0 : seg].out0;   // index in the output vector
            const float *red = reinterpret_cast<const float *>(rh + 4);
            if (fence_first) {
                __threadfence();
                fence_first = false;
            }
            if (p.epilogue == EPI_QKV_ROPE) {
                if (lane < (nrows >> 1)) {
                    float v0 = 0.f, v1 = 0.f;
                    for (int w = 0; w < p.wpr; ++w) {
                        v0 += red[(2 * lane) * p.wpr + w];
                        v1 += red[(2 * lane + 1) * p.wpr + w];
                    }
                    epi_qkv_pair(p, seg, row0 + 2 * lane, v0, v1, pos, rope_c, rope_s);
                }
            } else if (p.epilogue == EPI_SWIGLU) {
                if (lane < nrows) {
                    float v1 = 0.f, v3 = 0.f;
                    for (int w = 0; w < p.wpr; ++w) {
                        v1 += red[lane * p.wpr + w];
                        v3 += red[(R / 2 + lane) * p.wpr + w];
                    }
                    const float g = epi_swiglu(v1, v3);
                    if (tp_n) {
                        ll_send(p.ll, tp_n, row0 + lane, g, seq_out);
                    } else {
                        for (int r = 0; r < p.y_reps; ++r)
                            p.y[(int64_t)r * p.y_stride + row0 + lane] = g;
                    }
                }
            } else if (lane < nrows) {
                float a = 0.f;
                for (int w = 0; w < p.wpr; ++w)
                    a += red[lane * p.wpr + w];
                const int row = row0 + lane;
                if (p.epilogue == EPI_RESIDUAL && tp_n) {
                    // the consumer adds this to its copy of the residual stream: one add per element and launch on
                    // every rank, as on a single device
                    ll_send(p.ll, tp_n, row, a, seq_out);
                } else if (p.epilogue == EPI_RESIDUAL) {
                    for (int r = 0; r < p.y_reps; ++r)   // one add per element, copy and launch: no read round trip
                        atomicAdd(p.y + (int64_t)r * p.y_stride + row, a);
                } else {
                    p.y[row] = a;
                    if (p.epilogue == EPI_LOGITS && (a > best_v || (a == best_v && row < best_i))) {
                        best_v = a;
                        best_i = row;
                    }
                }
            }
            __syncwarp();
            if (lane == 0)
                mbar_arrive(sbase + kBarRedEmpty + 8 * rb);
            if (++rb == kRedBufs) {
                rb = 0;
                ++rround;
            }
        }
        if (lost && !lost_before && lane == 0)
            atomicOr(&p.state->status, L2J_DS_WAIT_TIMEOUT);
        // all results of the block were written by this warp; the release is cumulative
        __syncwarp();
        if (lane == 0)
            chain_signal(p.chain);
        if (lane == 0) {
            trace_mark(p, 6);
            if (p.trace)
                p.trace[blockIdx.x * 16 + 8] = global_timer_ns();
        }
        if (p.epilogue == EPI_LOGITS) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best_v, o);
                const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
                if (ov > best_v || (ov == best_v && oi < best_i)) {
                    best_v = ov;
                    best_i = oi;
                }
            }
            int last = 0;
            if (lane == 0) {
                p.blk_val[blockIdx.x] = best_v;
                p.blk_idx[blockIdx.x] = best_i;
                __threadfence();
                const unsigned int ticket = atomicAdd(&p.state->cls_counter, 1u);
                last = (ticket == gridDim.x - 1);
            }
            last = __shfl_sync(0xffffffffu, last, 0);
            if (last) {
                __threadfence();
                finish_argmax_warp(p, gridDim.x, lane);
            }
        }
        return;
    }
    if (warp > nw + 1)
        return;

    // ------------------------------------------------------------------------------ consumers
    const int rsub = warp / p.wpr;   // which of the rpp concurrent rows this warp works on
    const int wi = warp - rsub * p.wpr;
    const int nchunks = p.n / EPC;
    constexpr int NCH = GRP ? 4 : CPT;   // 16-byte chunks of a row that a thread owns
    int chunk[NCH];
    bool cvalid[NCH];
    if constexpr (GRP) {
        // Four lanes share one quantisation group (16 chunks): lane s of them owns chunks 4k + s, k = 0..3,
        // so a thread needs one group header and one integer -> float conversion per row.  k is swizzled
        // with the group's parity: the 16-byte loads of a quarter-warp then fall into eight different
        // bank groups.
        const int g = wi * 8 + (lane >> 2);
#pragma unroll
        for (int k = 0; k < NCH; ++k) {
            chunk[k] = g * 16 + 4 * (k ^ ((lane >> 2) & 1)) + (lane & 3);
            cvalid[k] = g < (p.n >> 8);
        }
    } else {
#pragma unroll
        for (int k = 0; k < NCH; ++k) {
            chunk[k] = (wi * CPT + k) * 32 + lane;
            cvalid[k] = chunk[k] < nchunks;
        }
    }

    bool lost = false;
    // The input vector comes from the previous kernel.  In a tensor-parallel group it arrives element by
    // element with its sequence number and the loads below poll for it; otherwise wait for the kernel.
    constexpr bool ll_in = LL;   // instantiated apart: the receive path needs registers the plain path must not pay for
    if (!ll_in && !chain_wait_group(p.chain, tid == 0, 1, ncons, wait_ns, reinterpret_cast<volatile int *>(smem + kScratchOff + 252)))
        lost = true;
    if (tid == 0)
        trace_mark(p, 12);

    // ---- prologue.  All consumer threads load x (coalesced, 16 bytes per thread and round), apply
    //      RMSNorm (RootMeanSquare.java:25-35, WeightNormalizeAndScale.java:71-74), convert to
    //      fixed-point limbs for the u8 path and publish the result in shared memory; every thread
    //      then picks up the chunks it owns.
    uint8_t *share = smem + kSmemHeader;   // u8: three planes [limb][nchunks] of 16 B (4 bytes per 4 elements); FP32: [nchunks] float4
    float *scratch = reinterpret_cast<float *>(smem + kScratchOff);
    const bool lost_before = (__ldcg(&p.state->status) & L2J_DS_WAIT_TIMEOUT) != 0;
    lost = lost || lost_before;
    float inv = 1.0f;                      // u8 path: value of one fixed-point unit
    {
        // The producer may fill the ring from now on: it needs hundreds of cycles to react, by then
        // the few loads of x below are on the wire in front of its copies.
        if (lane == 0)
            mbar_arrive(sbase + kBarXIssued);
        const int n4 = p.n >> 2;
        float4 xr[kPrologueRounds], wr[kPrologueRounds];
        const bool has_rms = p.rms_w != nullptr;
        const int64_t rep_off = (int64_t)(blockIdx.x % (unsigned)p.x_reps) * p.x_stride;
        const float *xin = p.x_in + rep_off;
        const float *rmsw = has_rms ? p.rms_w + rep_off : nullptr;
        if constexpr (!ll_in) {
#pragma unroll
            for (int j = 0; j < kPrologueRounds; ++j) {
                const int idx = tid + j * ncons;
                xr[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                wr[j] = make_float4(1.f, 1.f, 1.f, 1.f);
                if (j * ncons >= n4)
                    break;
                if (idx < n4) {
                    xr[j] = ld_cg_f4_issue(xin + (int64_t)idx * 4);
                    if (has_rms)
                        wr[j] = ld_cg_f4_issue(rmsw + (int64_t)idx * 4);
                }
            }
        } else {
            // A block without a stage of its own (its first stage is fixed: block index < number of stages)
            // contributes nothing and must not wait for data that later kernels may already have replaced.
            const bool has_work = blockIdx.x < (unsigned)p.total_stages;
            const float2 *rx = p.ll.tp->ll[p.ll.in_vec][p.ll.tp->rank];
            const int seq_in = ll_seq(p.ll, p.ll.in_idx);
#pragma unroll
            for (int j = 0; j < kPrologueRounds; ++j) {
                xr[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                wr[j] = make_float4(1.f, 1.f, 1.f, 1.f);
            }
            long long t_first = 0;
            // four rounds of pairs in flight at a time (their sequence numbers double the registers a round needs)
#pragma unroll
            for (int c0 = 0; c0 < kPrologueRounds; c0 += 4) {
                if (c0 * ncons >= n4)
                    break;
                float4 pa[4], pb[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int idx = tid + (c0 + q) * ncons;
                    if (idx < n4 && has_work) {
                        pa[q] = ld_pairs2(rx + (int64_t)idx * 4);
                        pb[q] = ld_pairs2(rx + (int64_t)idx * 4 + 2);
                    }
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int idx = tid + (c0 + q) * ncons;
                    if (idx < n4 && has_work) {
                        while (__float_as_int(pa[q].y) != seq_in || __float_as_int(pa[q].w) != seq_in ||
                               __float_as_int(pb[q].y) != seq_in || __float_as_int(pb[q].w) != seq_in) {
                            const long long now = sm_clock();   // limit in cycles: two per nanosecond
                            if (t_first == 0)
                                t_first = now;
                            if (now - t_first > (long long)(2 * (lost ? kShortWaitNs : wait_ns))) {
                                lost = true;
                                break;
                            }
                            pa[q] = ld_pairs2(rx + (int64_t)idx * 4);
                            pb[q] = ld_pairs2(rx + (int64_t)idx * 4 + 2);
                        }
                        xr[c0 + q] = make_float4(pa[q].x, pa[q].z, pb[q].x, pb[q].z);
                    }
                }
            }
            // The residual stream this rank keeps is read only now: the block may have started before the
            // kernel that stored it had run (blocks of consecutive kernels share SMs at small shapes), but no
            // increment can exist before that store is visible.  One add per element, as the single device's
            // red.add does it.
#pragma unroll
            for (int j = 0; j < kPrologueRounds; ++j) {
                const int idx = tid + j * ncons;
                if (j * ncons >= n4)
                    break;
                if (idx < n4 && has_work) {
                    if (p.ll.base) {
                        const float4 xo = ld_cg_f4_issue(p.ll.base + (int64_t)idx * 4);
                        xr[j].x = __fadd_rn(xo.x, xr[j].x);
                        xr[j].y = __fadd_rn(xo.y, xr[j].y);
                        xr[j].z = __fadd_rn(xo.z, xr[j].z);
                        xr[j].w = __fadd_rn(xo.w, xr[j].w);
                    }
                    if (has_rms)
                        wr[j] = ld_cg_f4_issue(rmsw + (int64_t)idx * 4);
                    if (p.ll.write_back && blockIdx.x == 0)
                        __stcg(reinterpret_cast<float4 *>(p.ll.write_back + (int64_t)idx * 4), xr[j]);
                }
            }
            // (the epilogue warp of block 0 fences these stores before it publishes the block's first results)
        }
        float ssq = 0.f, amax = 0.f;
#pragma unroll
        for (int j = 0; j < kPrologueRounds; ++j) {
            if (j * ncons >= n4)   // block-uniform: the remaining rounds hold nothing
                break;
            ssq = fmaf(xr[j].x, xr[j].x, ssq);
            ssq = fmaf(xr[j].y, xr[j].y, ssq);
            ssq = fmaf(xr[j].z, xr[j].z, ssq);
            ssq = fmaf(xr[j].w, xr[j].w, ssq);
            amax = fmaxf(fmaxf(amax, fmaxf(fabsf(xr[j].x), fabsf(xr[j].y))), fmaxf(fabsf(xr[j].z), fabsf(xr[j].w)));
        }
        if (tid == 0)
            trace_mark(p, 13);
        if (has_rms || !F32) {
            ssq = warp_sum(ssq);
            amax = warp_max(amax);
            if (lane == 0) {
                scratch[warp] = ssq;
                scratch[32 + warp] = amax;
            }
            named_barrier_sync(2, ncons);
            ssq = warp_sum(lane < nw ? scratch[lane] : 0.f);          // same order in every warp and block
            amax = warp_max(lane < nw ? scratch[32 + lane] : 0.f);
        }
        if (tid == 0)
            trace_mark(p, 9);
        if (has_rms) {
            float tot = __fdiv_rn(ssq, (float)p.n);
            tot = __fadd_rn(tot, 1e-5f);
            const float ss = __fdiv_rn(1.0f, __fsqrt_rn(tot));
#pragma unroll
            for (int j = 0; j < kPrologueRounds; ++j) {
                if (j * ncons >= n4)
                    break;
                xr[j].x = __fmul_rn(wr[j].x, __fmul_rn(ss, xr[j].x));
                xr[j].y = __fmul_rn(wr[j].y, __fmul_rn(ss, xr[j].y));
                xr[j].z = __fmul_rn(wr[j].z, __fmul_rn(ss, xr[j].z));
                xr[j].w = __fmul_rn(wr[j].w, __fmul_rn(ss, xr[j].w));
            }
            amax = amax * ss * p.rms_wmax * 1.000001f;   // bound of |w * (ss * x)| from max|x| and max|w|
        }
        if constexpr (F32) {
#pragma unroll
            for (int j = 0; j < kPrologueRounds; ++j) {
                const int idx = tid + j * ncons;
                if (j * ncons >= n4)
                    break;
                if (idx < n4)
                    *reinterpret_cast<float4 *>(share + (size_t)idx * 16) = xr[j];
            }
        } else {
            int ex = 0;
            if (amax > 0.f && amax < 3.0e38f)
                frexpf(amax, &ex);             // amax < 2^ex
            ex = max(-90, min(126, ex));
            const float f = __int_as_float((127 + 22 - ex) << 23);   // 2^(22 - ex): |x * f| <= 2^22
            inv = __int_as_float((127 + ex - 22) << 23);             // 2^(ex - 22): value of one fixed-point unit
#pragma unroll
            for (int j = 0; j < kPrologueRounds; ++j) {
                const int idx = tid + j * ncons;
                if (j * ncons >= n4)
                    break;
                if (idx < n4) {
                    // 24-bit fixed point as three balanced signed byte limbs: after the add-and-flip, bytes
                    // 0..2 of z are l0, l1, l2 in [-128, 127] with X = l0 + 256 l1 + 65536 l2
                    const uint32_t z0 = ((uint32_t)__float2int_rn(xr[j].x * f) + 0x00008080u) ^ 0x00008080u;
                    const uint32_t z1 = ((uint32_t)__float2int_rn(xr[j].y * f) + 0x00008080u) ^ 0x00008080u;
                    const uint32_t z2 = ((uint32_t)__float2int_rn(xr[j].z * f) + 0x00008080u) ^ 0x00008080u;
                    const uint32_t z3 = ((uint32_t)__float2int_rn(xr[j].w * f) + 0x00008080u) ^ 0x00008080u;
                    // byte transpose: limb l of the four elements ends up in word l
                    const uint32_t t0 = __byte_perm(z0, z1, 0x5140);   // z0.b0 z1.b0 z0.b1 z1.b1
                    const uint32_t t2 = __byte_perm(z2, z3, 0x5140);
                    const uint32_t t1 = __byte_perm(z0, z1, 0x0062);   // z0.b2 z1.b2 . .
                    const uint32_t t3 = __byte_perm(z2, z3, 0x0062);
                    uint32_t *dst = reinterpret_cast<uint32_t *>(share) + idx;
                    dst[0] = __byte_perm(t0, t2, 0x5410);
                    dst[p.n >> 2] = __byte_perm(t0, t2, 0x7632);
                    dst[p.n >> 1] = __byte_perm(t1, t3, 0x5410);
                }
            }
        }
        if (tid == 0)
            trace_mark(p, 10);
    }
    named_barrier_sync(1, ncons);
    if (tid == 0)
        trace_mark(p, 11);

    float xv[F32 ? CPT : 1][4];           // FP32 path: the chunk's four x values
    uint32_t xl[F32 ? 1 : NCH][4][3];     // u8 path: [chunk][word of 4 elements][limb]
    float xs[F32 ? 1 : (GRP ? 1 : NCH)];  // u8 path: sum of the owned x in fixed-point units (for the group minimum term)
    if constexpr (F32) {
#pragma unroll
        for (int k = 0; k < CPT; ++k) {
            float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
            if (cvalid[k])
                t = *reinterpret_cast<const float4 *>(share + (size_t)chunk[k] * 16);
            xv[k][0] = t.x; xv[k][1] = t.y; xv[k][2] = t.z; xv[k][3] = t.w;
        }
    } else {
        int s0 = 0, s1 = 0, s2 = 0;
#pragma unroll
        for (int k = 0; k < NCH; ++k) {
#pragma unroll
            for (int l = 0; l < 3; ++l) {
                uint4 t = make_uint4(0u, 0u, 0u, 0u);
                if (cvalid[k])
                    t = *reinterpret_cast<const uint4 *>(share + (size_t)l * p.n + (size_t)chunk[k] * 16);
                xl[k][0][l] = t.x; xl[k][1][l] = t.y; xl[k][2][l] = t.z; xl[k][3][l] = t.w;
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                s0 = dp4a_u8s8(0x01010101u, xl[k][q][0], s0);
                s1 = dp4a_u8s8(0x01010101u, xl[k][q][1], s1);
                s2 = dp4a_u8s8(0x01010101u, xl[k][q][2], s2);
            }
            if (!GRP || k == NCH - 1) {
                xs[GRP ? 0 : k] = fmaf((float)s2, 65536.0f, fmaf((float)s1, 256.0f, (float)s0));
                s0 = s1 = s2 = 0;
            }
        }
    }

    if (tid == 0)
        trace_mark(p, 3);
    int slot = 0, round = 0, rb = 0, rround = 0;
    bool first = true;
    for (;;) {
        if (!mbar_wait_bounded(sbase + kBarFull + 8 * slot, (uint32_t)round & 1u, wait_ns))
            lost = true;
        if (tid == 0 && first) {
            trace_mark(p, 4);
            first = false;
        }
        const StageDesc d = *(reinterpret_cast<const StageDesc *>(smem + kDescOff) + slot);
        // (a block whose input never came still works through its stages: producer, consumers and epilogue warp
        // stay in step, and no bulk copy is in flight when the block ends)
        const bool done = d.nrows <= 0;
        const uint8_t *slot_ptr = smem + kSmemHeader + p.xshare_bytes + (size_t)slot * p.slot_bytes;

        float v[RT];
#pragma unroll
        for (int t = 0; t < RT; ++t) {
            v[t] = 0.f;
            const int r = rsub + t * p.rpp;                      // row of the stage in shared memory
            const int half = (p.paired && t >= RT / 2) ? 1 : 0;  // second half of a paired stage: the partner matrix
            const int local = r - half * (R / 2);
            if (!done && local < d.nrows) {
                const uint8_t *rowp = slot_ptr + (size_t)r * rowbytes;
                if constexpr (F32) {
                    float a = 0.f;
#pragma unroll
                    for (int k = 0; k < CPT; ++k) {
                        if (cvalid[k]) {
                            const float4 w = *reinterpret_cast<const float4 *>(rowp + (size_t)chunk[k] * 16);
                            a = fmaf(w.x, xv[k][0], a);
                            a = fmaf(w.y, xv[k][1], a);
                            a = fmaf(w.z, xv[k][2], a);
                            a = fmaf(w.w, xv[k][3], a);
                        }
                    }
                    v[t] = a;
                } else if constexpr (GRP) {
                    if (cvalid[0]) {
                        const int e0 = (half ? d.e0b : d.e0a) + local * p.n;
                        const float2 *hp = reinterpret_cast<const float2 *>(slot_ptr + p.hdr_off + half * p.half_hdr);
                        const float2 ms = hp[(e0 + chunk[0] * 16) >> 8];
                        int a0 = 0, a1 = 0, a2 = 0;
#pragma unroll
                        for (int k = 0; k < NCH; ++k) {
                            const uint4 w = *reinterpret_cast<const uint4 *>(rowp + (size_t)chunk[k] * 16);
                            a0 = dp4a_u8s8(w.x, xl[k][0][0], a0);
                            a1 = dp4a_u8s8(w.x, xl[k][0][1], a1);
                            a2 = dp4a_u8s8(w.x, xl[k][0][2], a2);
                            a0 = dp4a_u8s8(w.y, xl[k][1][0], a0);
                            a1 = dp4a_u8s8(w.y, xl[k][1][1], a1);
                            a2 = dp4a_u8s8(w.y, xl[k][1][2], a2);
                            a0 = dp4a_u8s8(w.z, xl[k][2][0], a0);
                            a1 = dp4a_u8s8(w.z, xl[k][2][1], a1);
                            a2 = dp4a_u8s8(w.z, xl[k][2][2], a2);
                            a0 = dp4a_u8s8(w.w, xl[k][3][0], a0);
                            a1 = dp4a_u8s8(w.w, xl[k][3][1], a1);
                            a2 = dp4a_u8s8(w.w, xl[k][3][2], a2);
                        }
                        // |a_l| <= 64 * 255 * 128 < 2^24: the conversions are exact
                        const float dsum = fmaf((float)a2, 65536.0f, fmaf((float)a1, 256.0f, (float)a0));
                        v[t] = fmaf(ms.y, dsum, ms.x * xs[0]);
                    }
                } else {
                    const int e0 = (half ? d.e0b : d.e0a) + local * p.n;
                    const float2 *hp = reinterpret_cast<const float2 *>(slot_ptr + p.hdr_off + half * p.half_hdr);
                    float acc = 0.f;
#pragma unroll
                    for (int k = 0; k < NCH; ++k) {
                        if (cvalid[k]) {
                            const uint4 w = *reinterpret_cast<const uint4 *>(rowp + (size_t)chunk[k] * 16);
                            const float2 ms = hp[(e0 + chunk[k] * 16) >> 8];
                            int a0 = 0, a1 = 0, a2 = 0;
                            a0 = dp4a_u8s8(w.x, xl[k][0][0], a0);
                            a1 = dp4a_u8s8(w.x, xl[k][0][1], a1);
                            a2 = dp4a_u8s8(w.x, xl[k][0][2], a2);
                            a0 = dp4a_u8s8(w.y, xl[k][1][0], a0);
                            a1 = dp4a_u8s8(w.y, xl[k][1][1], a1);
                            a2 = dp4a_u8s8(w.y, xl[k][1][2], a2);
                            a0 = dp4a_u8s8(w.z, xl[k][2][0], a0);
                            a1 = dp4a_u8s8(w.z, xl[k][2][1], a1);
                            a2 = dp4a_u8s8(w.z, xl[k][2][2], a2);
                            a0 = dp4a_u8s8(w.w, xl[k][3][0], a0);
                            a1 = dp4a_u8s8(w.w, xl[k][3][1], a1);
                            a2 = dp4a_u8s8(w.w, xl[k][3][2], a2);
                            const float dsum = fmaf((float)a2, 65536.0f, fmaf((float)a1, 256.0f, (float)a0));
                            acc = fmaf(ms.y, dsum, acc);
                            acc = fmaf(ms.x, xs[k], acc);
                        }
                    }
                    v[t] = acc;
                }
            }
        }
        const float tot = warp_sum_rows<RT>(v, lane) * inv;
        __syncwarp();
        if (lane == 0)
            mbar_arrive(sbase + kBarEmpty + 8 * slot);   // this warp is done with the ring slot
        if (rround > 0) {
            if (!mbar_wait_bounded(sbase + kBarRedEmpty + 8 * rb, (uint32_t)(rround - 1) & 1u, wait_ns))
                lost = true;
        }
        int *rh = reinterpret_cast<int *>(smem + kRedOff + rb * kRedStride);
        float *red = reinterpret_cast<float *>(rh + 4);
        if (tid == 0) {
            rh[0] = d.seg;
            rh[1] = d.row0;
            rh[2] = done ? 0 : d.nrows;
        }
        if ((lane & (32 / RT - 1)) == 0) {
            const int t = lane / (32 / RT);
            red[(rsub + t * p.rpp) * p.wpr + wi] = tot;
        }
        __syncwarp();
        if (lane == 0)
            mbar_arrive(sbase + kBarRedFull + 8 * rb);
        if (done)
            break;
        if (++slot == nstage) {
            slot = 0;
            ++round;
        }
        if (++rb == kRedBufs) {
            rb = 0;
            ++rround;
        }
    }
    if (tid == 0)
        trace_mark(p, 5);
    if (lost && !lost_before)
        atomicOr(&p.state->status, L2J_DS_WAIT_TIMEOUT);
}

MvPlan plan_matvec(int n, bool f32, bool paired, int rows, int blocks, int row_align, bool group_aligned)
{
    MvPlan pl{};
    pl.ok = false;
    const int epc = f32 ? 4 : 16;
    if (n <= 0 || (n % 16) != 0)
        return pl;
    const int nchunks = n / epc;
    const int rowbytes = f32 ? n * 4 : n;
    const int max_cons = kRingMaxThreads / 32 - 2;   // consumer warps beside the producer and the epilogue warp
    // shared copy of x in front of the ring: FP32 values, or three byte planes of fixed-point limbs
    const int xshare = ((f32 ? n * 4 : n * 3) + 127) & ~127;
    const bool grouped = !f32 && group_aligned && (n % kGroup) == 0;
    const int rt_min = paired ? 2 : 1;
    for (int cpt = grouped ? 4 : 1; cpt <= 4; ++cpt) {
        int wpr, rpp, rt;
        if (grouped) {
            wpr = (n / kGroup + 7) / 8;   // a warp spans eight groups
            if (wpr > max_cons)
                return pl;
            rpp = max_cons / wpr;
            if (rpp > 8)
                rpp = 8;
            rt = 4;
        } else {
            wpr = (nchunks + 32 * cpt - 1) / (32 * cpt);
            if (wpr > max_cons)
                continue;
            rpp = 1;
            while (2 * rpp * wpr <= 16 && rpp < 8)
                rpp *= 2;
            rt = 8;
        }
        // rows per thread and stage: stages of at most 64 KB and 32 rows
        const int rt_floor = grouped ? rt_min : 2;
        while (rt > rt_floor && (rt * rpp > 32 || rt * rpp * rowbytes > 64 * 1024))
            rt /= 2;
        while (rpp > 1 && rt * rpp * rowbytes > 64 * 1024)
            rpp = grouped ? rpp - 1 : rpp / 2;
        // a matrix with few rows gets smaller stages, so that every block still has several of them to balance
        if (rows > 0 && blocks > 0)
            while (rt > rt_floor && rows / (rt * rpp) < 3 * blocks && rt * rpp * rowbytes > 32 * 1024)
                rt /= 2;
        if (row_align > 1 && (rt * rpp) % row_align != 0) {
            if (rpp > 1 && ((rpp - 1) * rt) % row_align == 0)
                --rpp;
            else
                continue;
        }
        if (n / 4 > kPrologueRounds * rpp * wpr * 32)
            continue;   // the prologue could not hold x in registers
        int half_hdr = 0;
        if (!f32) {
            half_hdr = (((rt * rpp * n / 2 + 255) / 256) + 4) * 8;
            half_hdr = (half_hdr + 15) & ~15;
        }
        const int payload = rt * rpp * rowbytes;
        const int slot = (payload + 2 * half_hdr + 127) & ~127;
        int nstage = (kMaxSmemBlock - kSmemHeader - xshare) / slot;
        if (nstage > 16)
            nstage = 16;
        if (nstage < 2)
            continue;
        pl.grouped = grouped;
        pl.cpt = cpt;
        pl.rt = rt;
        pl.rpp = rpp;
        pl.wpr = wpr;
        pl.nstage = nstage;
        pl.slot_bytes = slot;
        pl.hdr_off = payload;
        pl.half_hdr = half_hdr;
        pl.xshare_bytes = xshare;
        pl.threads = (rpp * wpr + 2) * 32;
        pl.smem_bytes = kSmemHeader + xshare + nstage * slot;   // header + shared x + ring
        pl.ok = true;
        return pl;
    }
    return pl;
}

template <bool F32, bool GRP, int CPT, int RT, bool LL>
static cudaError_t launch_ring_t(const LaunchCfg &lc, const MvPlan &plan, const MvParams &p)
{
    auto kern = matvec_ring_kernel<F32, GRP, CPT, RT, LL>;
    if (plan.threads > kRingMaxThreads)
        return cudaErrorInvalidConfiguration;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)lc.grid);
    cfg.blockDim = dim3((unsigned)plan.threads);
    cfg.dynamicSmemBytes = (size_t)plan.smem_bytes;
    cfg.stream = lc.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = lc.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

template <bool F32, bool GRP, int CPT, int RT, bool LL>
static cudaError_t prepare_ring_t()
{
    auto kern = matvec_ring_kernel<F32, GRP, CPT, RT, LL>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmemBlock);
    if (e != cudaSuccess)
        return e;
    return cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

// Instantiations: (FP32 weights, grouped thread mapping, chunks per thread, rows per thread and stage).
#define L2J_RING_VARIANTS(X) \
    X(true, false, 1, 2) X(true, false, 1, 4) X(true, false, 1, 8) X(true, false, 2, 2) X(true, false, 2, 4) X(true, false, 2, 8) \
    X(true, false, 3, 2) X(true, false, 3, 4) X(true, false, 3, 8) X(true, false, 4, 2) X(true, false, 4, 4) X(true, false, 4, 8) \
    X(false, false, 1, 2) X(false, false, 1, 4) X(false, false, 1, 8) X(false, false, 2, 2) X(false, false, 2, 4) X(false, false, 2, 8) \
    X(false, false, 3, 2) X(false, false, 3, 4) X(false, false, 3, 8) X(false, false, 4, 2) X(false, false, 4, 4) X(false, false, 4, 8) \
    X(false, true, 4, 1) X(false, true, 4, 2) X(false, true, 4, 4)

// Opts the ring kernels of the current device into their dynamic shared memory size.  Call once
// per device before the first launch (and outside stream capture).
static cudaError_t prepare_attention();

cudaError_t prepare_kernels()
{
    cudaError_t e;
    if ((e = prepare_attention()) != cudaSuccess)
        return e;
#define X(F, G, C, R) \
    if ((e = prepare_ring_t<F, G, C, R, false>()) != cudaSuccess) return e; \
    if ((e = prepare_ring_t<F, G, C, R, true>()) != cudaSuccess) return e;
    L2J_RING_VARIANTS(X)
#undef X
    return cudaSuccess;
}

cudaError_t launch_matvec_ring(const LaunchCfg &lc, const MvPlan &plan, bool f32, const MvParams &p)
{
    const bool ll = p.ll.tp != nullptr && p.ll.in_vec >= 0;   // the input arrives as (value, sequence number) pairs
#define X(F, G, C, R) \
    if (f32 == F && plan.grouped == G && plan.cpt == C && plan.rt == R) \
        return ll ? launch_ring_t<F, G, C, R, true>(lc, plan, p) : launch_ring_t<F, G, C, R, false>(lc, plan, p);
    L2J_RING_VARIANTS(X)
#undef X
    return cudaErrorInvalidConfiguration;
}

// =============================================================================================
// begin_kernel: fix (token, pos) of this forward in device memory and gather the embedding row
// =============================================================================================

__global__ void __launch_bounds__(256) begin_kernel(SeqState *state, const Cmd *cmd, const float *emb, float *x, int dim,
                                                    int vocab, int seq_len, int gather, int x_reps, int x_stride, unsigned int *epoch,
                                                    const StageLink *link)
{
    __shared__ int s_tok;
    __shared__ const float *s_xsrc;
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) {
        int tok, pos;
        const int cflags = __ldcg(&cmd->flags);
        int st = 0;
        if (__ldcg(&cmd->mode) == 1) {
            tok = __ldcg(&cmd->token);
            pos = __ldcg(&cmd->pos);
        } else {
            // greedy loop; over a layer split the chosen token lives on the last stage's device
            tok = __ldcg(&state->token);
            if (cflags & kCmdTokenFromPeer) {
                const int *src = reinterpret_cast<const int *>(__ldcg(reinterpret_cast<const unsigned long long *>(&link->token_src)));
                if (src)
                    tok = __ldcg(src);
                else
                    st |= L2J_DS_BAD_LINK;   // the stages were not linked: report it, never follow a null pointer
            }
            pos = __ldcg(&state->pos);
            if (cflags & kCmdAdvancePos)
                state->pos = pos + 1;
        }
        s_xsrc = nullptr;
        if (cflags & kCmdXFromPeer) {
            s_xsrc = reinterpret_cast<const float *>(__ldcg(reinterpret_cast<const unsigned long long *>(&link->x_src)));
            if (!s_xsrc)
                st |= L2J_DS_BAD_LINK;
        }
        if (pos < 0 || pos >= seq_len) {
            st |= L2J_DS_BAD_POS;
            pos = pos < 0 ? 0 : seq_len - 1;
        }
        if (tok < 0 || tok >= vocab) {
            st |= L2J_DS_BAD_TOKEN;
            tok = 0;
        }
        if (st)
            atomicOr(&state->status, st);
        state->cur_token = tok;
        state->cur_pos = pos;
        if (epoch)   // a whole forward follows: its kernels hand over through the counters
            *epoch = __ldcg(epoch) + 1u;
        s_tok = tok;
    }
    __syncthreads();
    if (gather) {
        const float4 *src = reinterpret_cast<const float4 *>(emb + (int64_t)s_tok * dim);
        for (int i = threadIdx.x; i < dim / 4; i += blockDim.x) {
            const float4 v = __ldg(src + i);
            for (int r = 0; r < x_reps; ++r)
                reinterpret_cast<float4 *>(x + (int64_t)r * x_stride)[i] = v;
        }
    } else {
        // a later stage of a layer split: x comes from the previous stage, either read here from that
        // stage's device over the peer link (Run.java:368-413 without the host array) or put into copy 0
        // by the caller
        const float *src = s_xsrc ? s_xsrc : x;
        for (int i = threadIdx.x; i < dim / 4; i += blockDim.x) {
            const float4 v = __ldcg(reinterpret_cast<const float4 *>(src) + i);
            for (int r = s_xsrc ? 0 : 1; r < x_reps; ++r)
                reinterpret_cast<float4 *>(x + (int64_t)r * x_stride)[i] = v;
        }
    }
}

cudaError_t launch_begin(const LaunchCfg &lc, SeqState *state, const Cmd *cmd, const float *emb, float *x, int dim,
                         int vocab, int seq_len, int gather, int x_reps, int x_stride, unsigned int *epoch,
                         const StageLink *link)
{
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = lc.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = lc.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, begin_kernel, state, cmd, emb, x, dim, vocab, seq_len, gather, x_reps, x_stride, epoch, link);
}

// =============================================================================================
// attention_kernel: single-query attention for all heads, positions split across blocks
//
// One pass with an online softmax: every warp (lane group) streams its share of the positions,
// loading K and V rows together so that a block pays one memory round trip, not two.  The lane
// groups of a block are merged through shared memory; if the block covers all positions of its
// head the result is written directly, otherwise (m, l, o) partials go to scratch and the last
// block of the head to arrive merges them in a fixed order (bitwise reproducible).
// =============================================================================================

constexpr int kAttnThreads = 256;
constexpr int kAttnWarps = kAttnThreads / 32;
constexpr size_t kAttnPadSmem = 80 * 1024;   // more than a third of an SM's shared memory
constexpr int kAttnMinChunk = 32;   // positions per block before the work is split further: one round of loads

// Streams positions [t0, t0 + cnt) of head h and merges the block's lane groups: afterwards thread
// tid < head holds (M, L, O[tid]) of those positions.  Called by the whole block.
// PIPE: the next round of rows is requested before the arithmetic of the current one (long contexts: two
// rounds in flight per warp); without it the loop is shorter and needs fewer registers (short contexts:
// one round covers a block's positions and only latency counts).
template <bool PIPE>
__device__ __forceinline__ void attention_block(const AttnParams &p, int h, int t0, int cnt, int pos, float *asmem, int *s_flag,
                                                unsigned long long *tr, float &M, float &L, float &O)
{
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int head = p.head;
    const int lpp = head >> 2;                      // lanes per position (float4 each)
    int gw = 1;
    while (gw < lpp)
        gw <<= 1;                                   // lane-group width (power of two, <= 32)
    const int ppw = 32 / gw;                        // lane groups (positions in flight) per warp
    const int g = lane / gw, li = lane - g * gw;
    const bool active = li < lpp;
    const int nslots = kAttnWarps * ppw;
    const int slot = warp * ppw + g;
    const int sstride = head + 4;
    const int kvh = h / p.kv_mul;
    const float *kb = p.k_cache + ((int64_t)kvh * p.seq_len + t0) * head;
    const float *vb = p.v_cache + ((int64_t)kvh * p.seq_len + t0) * head;
    const float sq = sqrtf((float)head);

    // Every cached row but the newest is older than this forward, so the first round of rows can be on
    // its way before the QKV kernel in front has finished.
    float4 kk[4], vv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int idx = u * nslots + slot;
        kk[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        vv[u] = kk[u];
        if (active && idx < cnt && t0 + idx < pos) {
            kk[u] = __ldcg(reinterpret_cast<const float4 *>(kb + (int64_t)idx * head + 4 * li));
            vv[u] = __ldcg(reinterpret_cast<const float4 *>(vb + (int64_t)idx * head + 4 * li));
        }
    }

    // q and the newest K/V row come from the kernel in front
    if (!chain_wait_group(p.chain, tid == 0, 1, kAttnThreads, (uint64_t)p.timeout_us * 1000ull, s_flag, p.state) && tid == 0)
        atomicOr(&p.state->status, L2J_DS_WAIT_TIMEOUT);
    if (tr)
        tr[1] = global_timer_ns();

    float4 q4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (active)
        q4 = __ldcg(reinterpret_cast<const float4 *>(p.q + (int64_t)h * head + 4 * li));

    float m = -INFINITY, l = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    // rows of the first round that could not be fetched early (the newest position)
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int i0 = u * nslots + slot;
        if (active && i0 < cnt && t0 + i0 >= pos) {
            kk[u] = __ldcg(reinterpret_cast<const float4 *>(kb + (int64_t)i0 * head + 4 * li));
            vv[u] = __ldcg(reinterpret_cast<const float4 *>(vb + (int64_t)i0 * head + 4 * li));
        }
    }
    const int step = 4 * nslots;
    for (int ib = 0; ib < cnt; ib += step) {   // uniform trip count for the whole block
        float4 kn[PIPE ? 4 : 1], vn[PIPE ? 4 : 1];
        int idx[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            idx[u] = ib + u * nslots + slot;
            if constexpr (PIPE) {
                const int nx = idx[u] + step;
                kn[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                vn[u] = kn[u];
                if (active && nx < cnt) {
                    kn[u] = __ldcg(reinterpret_cast<const float4 *>(kb + (int64_t)nx * head + 4 * li));
                    vn[u] = __ldcg(reinterpret_cast<const float4 *>(vb + (int64_t)nx * head + 4 * li));
                }
            } else if (ib > 0) {
                kk[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                vv[u] = kk[u];
                if (active && idx[u] < cnt) {
                    kk[u] = __ldcg(reinterpret_cast<const float4 *>(kb + (int64_t)idx[u] * head + 4 * li));
                    vv[u] = __ldcg(reinterpret_cast<const float4 *>(vb + (int64_t)idx[u] * head + 4 * li));
                }
            }
        }
        float s[4];
        float mloc = -INFINITY;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            float d = kk[u].x * q4.x;
            d = fmaf(kk[u].y, q4.y, d);
            d = fmaf(kk[u].z, q4.z, d);
            d = fmaf(kk[u].w, q4.w, d);
            for (int o = gw >> 1; o > 0; o >>= 1)
                d += __shfl_xor_sync(0xffffffffu, d, o);
            s[u] = idx[u] < cnt ? __fdiv_rn(d, sq) : -INFINITY;   // AttentionLoop.java:48
            mloc = fmaxf(mloc, s[u]);
        }
        if (mloc > -INFINITY) {
            const float mn = fmaxf(m, mloc);
            const float sc = expf(m - mn);            // 0 on the first round (m = -inf)
            l *= sc;
            acc.x *= sc; acc.y *= sc; acc.z *= sc; acc.w *= sc;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float pw = expf(s[u] - mn);     // 0 for the padded positions
                l += pw;
                acc.x = fmaf(pw, vv[u].x, acc.x);
                acc.y = fmaf(pw, vv[u].y, acc.y);
                acc.z = fmaf(pw, vv[u].z, acc.z);
                acc.w = fmaf(pw, vv[u].w, acc.w);
            }
            m = mn;
        }
        if constexpr (PIPE) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                kk[u] = kn[u];
                vv[u] = vn[u];
            }
        }
    }
    if (tr)
        tr[2] = global_timer_ns();
    float *mine = asmem + slot * sstride;
    if (active)
        *reinterpret_cast<float4 *>(mine + 4 * li) = acc;
    if (li == 0) {
        mine[head] = m;
        mine[head + 1] = l;
    }
    __syncthreads();

    // merge the lane groups of the block in slot order
    M = -INFINITY;
    L = 0.f;
    O = 0.f;
    if (tid < head) {
        for (int s2 = 0; s2 < nslots; ++s2)
            M = fmaxf(M, asmem[s2 * sstride + head]);
        for (int s2 = 0; s2 < nslots; ++s2) {
            const float ms = asmem[s2 * sstride + head];
            const float ls = asmem[s2 * sstride + head + 1];
            if (ls > 0.f) {
                const float w = expf(ms - M);
                L = fmaf(ls, w, L);
                O = fmaf(asmem[s2 * sstride + tid], w, O);
            }
        }
    }
    if (tr)
        tr[3] = global_timer_ns();
}

// Tells the kernel behind that this block's results are visible (after a block-wide barrier the release
// by one thread covers what the others wrote).
__device__ __forceinline__ void attention_signal(const AttnParams &p)
{
    if (p.chain.done_counter) {
        __syncthreads();
        if (threadIdx.x == 0)
            chain_signal(p.chain);
    }
}

// One element of the attention output: to the local vector (and its copies), or to every rank's.
__device__ __forceinline__ void attention_store(const AttnParams &p, int index, float o, int seq)
{
    if (p.ll.tp) {
        ll_send(p.ll, p.ll.tp->n, index, o, seq);
    } else {
        for (int r = 0; r < p.out_reps; ++r)
            p.out[(int64_t)r * p.out_stride + index] = o;
    }
}

template <bool PIPE>
__global__ void __launch_bounds__(kAttnThreads, PIPE ? 2 : 3) attention_kernel(const __grid_constant__ AttnParams p)
{
    extern __shared__ __align__(16) float asmem[];   // [slots][head + 4]: o, then m, l (16-byte aligned rows); [head + 4] block result
    __shared__ int s_last;

    const int h = p.h0 + blockIdx.x, sp = blockIdx.y;
    const int tid = threadIdx.x;
    const int head = p.head;

    pdl_launch_dependents();
    const int bl = sp * (int)gridDim.x + (int)blockIdx.x;
    unsigned long long *tr = (p.trace && bl < p.trace_blocks && tid == 0) ? p.trace + bl * 16 : nullptr;
    if (tr)
        tr[0] = global_timer_ns();

    // The position was fixed when the token started, so it can be read before the kernel in front has
    // finished: the block becomes resident early and hides its first memory round trip behind that kernel.
    const int pos = p.pos_override >= 0 ? p.pos_override : __ldcg(&p.state->cur_pos);
    const int npos = pos + 1;
    int chunk = (npos + p.nsplit - 1) / p.nsplit;
    if (chunk < kAttnMinChunk)
        chunk = kAttnMinChunk;
    const int nact = (npos + chunk - 1) / chunk;    // blocks of this head that have work
    const bool cluster_merge = p.cluster && nact > 1;
    if (sp >= nact && !cluster_merge) {   // no work, no results, nobody to meet: report at once
        if (p.chain.done_counter) {
            if (tid == 0)
                chain_signal(p.chain);
        } else {
            pdl_wait();
        }
        return;
    }

    const int seq_out = p.ll.tp ? ll_seq(p.ll, p.ll.out_idx) : 0;
    float M = -INFINITY, L = 0.f, O = 0.f;
    if (sp < nact) {
        const int t0 = sp * chunk;
        const int cnt = min(npos, t0 + chunk) - t0;
        attention_block<PIPE>(p, h, t0, cnt, pos, asmem, &s_last, tr, M, L, O);
    }

    if (nact == 1) {
        const float o = __fdiv_rn(O, L);   // ExpSumNormalize.java:33-37 folded into the sum
        if (tid < head)
            attention_store(p, h * head + tid, o, seq_out);
        attention_signal(p);
        return;
    }

    if (cluster_merge) {
        // The blocks of a head form one thread-block cluster: the partial results stay in shared memory and
        // block 0 of the cluster reads them from its neighbours, in block order (bitwise reproducible).
        namespace cg = cooperative_groups;
        cg::cluster_group cl = cg::this_cluster();
        int gw = 1;
        while (gw < (head >> 2))
            gw <<= 1;
        float *res = asmem + kAttnWarps * (32 / gw) * (head + 4);
        if (tid < head)
            res[tid] = O;
        if (tid == 0) {
            res[head] = M;
            res[head + 1] = L;
        }
        // Only block 0 of the cluster writes results for the kernel behind; the others report at once, so that
        // kernel does not wait for the cluster's second barrier.
        if (sp != 0 && tid == 0)
            chain_signal(p.chain);
        cl.sync();
        if (sp == 0 && tid < head) {
            float gm = -INFINITY;
            for (int s2 = 0; s2 < nact; ++s2)
                gm = fmaxf(gm, cl.map_shared_rank(res, s2)[head]);
            float LL = 0.f, OO = 0.f;
            for (int s2 = 0; s2 < nact; ++s2) {
                const float *rs = cl.map_shared_rank(res, s2);
                const float ms = rs[head];
                const float ls = rs[head + 1];
                if (ls > 0.f) {
                    const float w = expf(ms - gm);
                    LL = fmaf(ls, w, LL);
                    OO = fmaf(rs[tid], w, OO);
                }
            }
            const float o = __fdiv_rn(OO, LL);
            attention_store(p, h * head + tid, o, seq_out);
        }
        if (tr)
            tr[5] = global_timer_ns();
        if (sp == 0)
            attention_signal(p);
        cl.sync();   // a block's shared memory must outlive the reads of block 0
        return;
    }

    float *part = p.part + ((int64_t)h * p.nsplit + sp) * (head + 2);
    if (tid < head)
        __stcg(part + 2 + tid, O);
    if (tid == 0) {
        __stcg(part, M);
        __stcg(part + 1, L);
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned int ticket = atomicAdd(&p.counters[h], 1u);
        s_last = (ticket == (unsigned)nact - 1);
    }
    __syncthreads();
    if (tr)
        tr[4] = global_timer_ns();
    if (!s_last) {
        if (tid == 0)   // the partials were fenced before the ticket
            chain_signal(p.chain);
        return;
    }

    // ---- the last block of the head merges the partials of the active blocks in a fixed order
    __threadfence();
    if (tid < head) {
        const float *hp = p.part + (int64_t)h * p.nsplit * (head + 2);
        float gm = -INFINITY;
        for (int s2 = 0; s2 < nact; ++s2)
            gm = fmaxf(gm, __ldcg(hp + (int64_t)s2 * (head + 2)));
        float LL = 0.f, OO = 0.f;
        for (int s2 = 0; s2 < nact; ++s2) {
            const float ms = __ldcg(hp + (int64_t)s2 * (head + 2));
            const float ls = __ldcg(hp + (int64_t)s2 * (head + 2) + 1);
            if (ls > 0.f) {
                const float w = expf(ms - gm);
                LL = fmaf(ls, w, LL);
                OO = fmaf(__ldcg(hp + (int64_t)s2 * (head + 2) + 2 + tid), w, OO);
            }
        }
        const float o = __fdiv_rn(OO, LL);
        attention_store(p, h * head + tid, o, seq_out);
    }
    if (tid == 0)
        p.counters[h] = 0;
    if (tr)
        tr[5] = global_timer_ns();
    attention_signal(p);
}

static cudaError_t prepare_attention()
{
    return cudaFuncSetAttribute(attention_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kAttnPadSmem);
}

cudaError_t launch_attention(const LaunchCfg &lc, const AttnParams &p)
{
    int gw = 1;
    while (gw < (p.head >> 2))
        gw <<= 1;
    const int nslots = kAttnWarps * (32 / gw);
    if (p.cluster && (p.nsplit < 1 || p.nsplit > 8))
        return cudaErrorInvalidConfiguration;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)p.n_heads, (unsigned)p.nsplit);
    cfg.blockDim = dim3(kAttnThreads);
    cfg.dynamicSmemBytes = (size_t)(nslots + 1) * (p.head + 4) * sizeof(float);
    if (p.smem_pad && cfg.dynamicSmemBytes < kAttnPadSmem)
        cfg.dynamicSmemBytes = kAttnPadSmem;
    cfg.stream = lc.stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (lc.pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (p.cluster && p.nsplit > 1) {   // the blocks of a head are one cluster
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 1;
        attr[na].val.clusterDim.y = (unsigned)p.nsplit;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    // the long-context launch (two blocks per SM, no cluster) is the one that streams
    return p.smem_pad ? cudaLaunchKernelEx(&cfg, attention_kernel<true>, p) : cudaLaunchKernelEx(&cfg, attention_kernel<false>, p);
}

// =============================================================================================
// plain kernels: unfused, direct loads.  Cross-check path and fallback for shapes the ring
// kernel does not take (row length not a multiple of 16).
// =============================================================================================

__global__ void __launch_bounds__(256) rmsnorm_plain_kernel(const float *x, const float *w, float *out, int n)
{
    __shared__ float sred[8];
    __shared__ float s_ss;
    float part = 0.f;
    for (int i = threadIdx.x; i < n; i += 256)
        part = fmaf(x[i], x[i], part);
    part = warp_sum(part);
    if ((threadIdx.x & 31) == 0)
        sred[threadIdx.x >> 5] = part;
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = 0.f;
        for (int i = 0; i < 8; ++i)
            tot += sred[i];
        tot = __fdiv_rn(tot, (float)n);
        tot = __fadd_rn(tot, 1e-5f);
        s_ss = __fdiv_rn(1.0f, __fsqrt_rn(tot));
    }
    __syncthreads();
    const float ss = s_ss;
    for (int i = threadIdx.x; i < n; i += 256)
        out[i] = __fmul_rn(w[i], __fmul_rn(ss, x[i]));
}

cudaError_t launch_rmsnorm_plain(cudaStream_t s, const float *x, const float *w, float *out, int n)
{
    rmsnorm_plain_kernel<<<1, 256, 0, s>>>(x, w, out, n);
    return cudaGetLastError();
}

// One warp per row, one byte per lane and step: any row length, any group alignment.
__global__ void __launch_bounds__(256) matvec_plain_u8_kernel(MvSeg seg, int n, const float *x, float *y)
{
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= seg.rows)
        return;
    const int64_t flat = seg.flat0 + (int64_t)row * n;
    float acc = 0.f;
    for (int j = lane; j < n; j += 32) {
        const int64_t e = flat + j;
        const float2 ms = seg.hdr[e >> 8];
        const float w = fmaf((float)seg.payload[e], ms.y, ms.x);
        acc = fmaf(w, x[j], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0)
        y[row] = acc;
}

cudaError_t launch_matvec_plain_u8(cudaStream_t s, const MvSeg &seg, int n, const float *x, float *y)
{
    matvec_plain_u8_kernel<<<(seg.rows + 7) / 8, 256, 0, s>>>(seg, n, x, y);
    return cudaGetLastError();
}

__global__ void __launch_bounds__(256) matvec_plain_f32_kernel(const float *w, int n, int d, const float *x, float *y)
{
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= d)
        return;
    const float *wr = w + (int64_t)row * n;
    float acc = 0.f;
    for (int j = lane; j < n; j += 32)
        acc = fmaf(wr[j], x[j], acc);
    acc = warp_sum(acc);
    if (lane == 0)
        y[row] = acc;
}

cudaError_t launch_matvec_plain_f32(cudaStream_t s, const float *w, int n, int d, const float *x, float *y)
{
    matvec_plain_f32_kernel<<<(d + 7) / 8, 256, 0, s>>>(w, n, d, x, y);
    return cudaGetLastError();
}

// Applies a ring-kernel epilogue to finished row sums (one block).
__global__ void __launch_bounds__(256) epilogue_plain_kernel(MvParams p, const float *y0, const float *y1, const float *y2)
{
    const int pos = __ldcg(&p.state->cur_pos);
    if (p.epilogue == EPI_QKV_ROPE) {
        const float *ys[3] = {y0, y1, y2};
        for (int sg = 0; sg < 3; ++sg)
            for (int i = threadIdx.x * 2; i < p.seg[sg].rows; i += 512)
                epi_qkv_pair(p, sg, i, ys[sg][i], ys[sg][i + 1], pos, p.rope_cos + (int64_t)pos * (p.head >> 1),
                             p.rope_sin + (int64_t)pos * (p.head >> 1));
    } else if (p.epilogue == EPI_SWIGLU) {
        for (int i = threadIdx.x; i < p.seg[0].rows; i += 256)
            for (int r = 0; r < p.y_reps; ++r)
                p.y[(int64_t)r * p.y_stride + i] = epi_swiglu(y0[i], y1[i]);
    } else if (p.epilogue == EPI_RESIDUAL) {
        for (int i = threadIdx.x; i < p.seg[0].rows; i += 256)
            for (int r = 0; r < p.y_reps; ++r)
                p.y[(int64_t)r * p.y_stride + i] = __fadd_rn(p.y[(int64_t)r * p.y_stride + i], y0[i]);
    } else if (p.epilogue == EPI_LOGITS) {
        __shared__ float sv[256];
        __shared__ int si[256];
        float bv = -FLT_MAX;
        int bi = 0x7fffffff;
        for (int i = threadIdx.x; i < p.seg[0].rows; i += 256) {
            const float v = y0[i];
            p.y[i] = v;
            if (v > bv) {
                bv = v;
                bi = i;
            }
        }
        sv[threadIdx.x] = bv;
        si[threadIdx.x] = bi;
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int t = 1; t < 256; ++t) {
                if (sv[t] > bv || (sv[t] == bv && si[t] < bi)) {
                    bv = sv[t];
                    bi = si[t];
                }
            }
            p.blk_val[0] = bv;
            p.blk_idx[0] = bi;
            __threadfence();
        }
        __syncthreads();
        if (threadIdx.x < 32)
            finish_argmax_warp(p, 1, threadIdx.x);
    } else {
        for (int i = threadIdx.x; i < p.seg[0].rows; i += 256)
            p.y[i] = y0[i];
    }
}

cudaError_t launch_epilogue_plain(cudaStream_t s, const MvParams &p, const float *y0, const float *y1, const float *y2)
{
    epilogue_plain_kernel<<<1, 256, 0, s>>>(p, y0, y1, y2);
    return cudaGetLastError();
}

__global__ void rope_plain_kernel(float *q, float *k, const float *cs, const float *sn, int pos, int dim, int kv_dim, int head)
{
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
    const int half = head >> 1;
    if (i < dim) {
        const float c = cs[(int64_t)pos * half + ((i % head) >> 1)], s = sn[(int64_t)pos * half + ((i % head) >> 1)];
        const float v0 = q[i], v1 = q[i + 1];
        q[i] = __fsub_rn(__fmul_rn(v0, c), __fmul_rn(v1, s));
        q[i + 1] = __fadd_rn(__fmul_rn(v0, s), __fmul_rn(v1, c));
    }
    if (i < kv_dim) {
        const float c = cs[(int64_t)pos * half + ((i % head) >> 1)], s = sn[(int64_t)pos * half + ((i % head) >> 1)];
        const float v0 = k[i], v1 = k[i + 1];
        k[i] = __fsub_rn(__fmul_rn(v0, c), __fmul_rn(v1, s));
        k[i + 1] = __fadd_rn(__fmul_rn(v0, s), __fmul_rn(v1, c));
    }
}

cudaError_t launch_rope_plain(cudaStream_t s, float *q, float *k, const float *cs, const float *sn, int pos, int dim,
                              int kv_dim, int head)
{
    const int pairs = dim / 2;
    rope_plain_kernel<<<(pairs + 127) / 128, 128, 0, s>>>(q, k, cs, sn, pos, dim, kv_dim, head);
    return cudaGetLastError();
}

__global__ void swiglu_plain_kernel(float *hb, const float *hb2, int n)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n)
        hb[i] = epi_swiglu(hb[i], hb2[i]);
}

cudaError_t launch_swiglu_plain(cudaStream_t s, float *hb, const float *hb2, int n)
{
    swiglu_plain_kernel<<<(n + 255) / 256, 256, 0, s>>>(hb, hb2, n);
    return cudaGetLastError();
}

// =============================================================================================
// load-time kernels
// =============================================================================================

// File-format groups (8-byte big-endian header + 256 bytes) -> payload bytes and (min, scale)
// headers.  scale = (max - min) / 255f as in MatMul.java:137.  One warp per group.
__global__ void __launch_bounds__(256) repack_kernel(const uint8_t *groups, int64_t n_groups, uint8_t *payload, float2 *hdr)
{
    const int64_t g = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (g >= n_groups)
        return;
    const uint8_t *src = groups + g * kGroupBytes;
    const uint2 v = *reinterpret_cast<const uint2 *>(src + 8 + 8 * lane);
    *reinterpret_cast<uint2 *>(payload + g * kGroup + 8 * lane) = v;
    if (lane == 0) {
        const uint2 h = *reinterpret_cast<const uint2 *>(src);
        const float mn = __uint_as_float(__byte_perm(h.x, 0, 0x0123));
        const float mx = __uint_as_float(__byte_perm(h.y, 0, 0x0123));
        hdr[g] = make_float2(mn, __fdiv_rn(__fsub_rn(mx, mn), 255.0f));
    }
}

cudaError_t launch_repack(cudaStream_t s, const uint8_t *groups, int64_t n_groups, uint8_t *payload, float2 *hdr)
{
    if (n_groups <= 0)
        return cudaSuccess;
    repack_kernel<<<(unsigned)((n_groups + 7) / 8), 256, 0, s>>>(groups, n_groups, payload, hdr);
    return cudaGetLastError();
}

// RMSNorm weights to FP32 with the CPU formula byte / 255f * range + min
// (WeightNormalizeAndScale.java:71-73); range is recovered as max - min from the stored header.
__global__ void dequant_rms_kernel(const uint8_t *payload, const float2 *hdr_minmax, int64_t rel0, int64_t n, float *out)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n)
        return;
    const int64_t e = rel0 + i;
    const float2 mm = hdr_minmax[e >> 8];   // (min, max)
    const float range = __fsub_rn(mm.y, mm.x);
    const float v = __fdiv_rn((float)payload[e], 255.0f);
    out[i] = __fadd_rn(__fmul_rn(v, range), mm.x);
}

// The header array of a QTensor stores (min, scale); the RMS weights need (min, max), so their
// tensors are repacked by this variant, which keeps max in .y.
__global__ void __launch_bounds__(256) repack_minmax_kernel(const uint8_t *groups, int64_t n_groups, uint8_t *payload,
                                                             float2 *hdr)
{
    const int64_t g = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (g >= n_groups)
        return;
    const uint8_t *src = groups + g * kGroupBytes;
    const uint2 v = *reinterpret_cast<const uint2 *>(src + 8 + 8 * lane);
    *reinterpret_cast<uint2 *>(payload + g * kGroup + 8 * lane) = v;
    if (lane == 0) {
        const uint2 h = *reinterpret_cast<const uint2 *>(src);
        hdr[g] = make_float2(__uint_as_float(__byte_perm(h.x, 0, 0x0123)), __uint_as_float(__byte_perm(h.y, 0, 0x0123)));
    }
}

cudaError_t launch_repack_minmax(cudaStream_t s, const uint8_t *groups, int64_t n_groups, uint8_t *payload, float2 *hdr)
{
    if (n_groups <= 0)
        return cudaSuccess;
    repack_minmax_kernel<<<(unsigned)((n_groups + 7) / 8), 256, 0, s>>>(groups, n_groups, payload, hdr);
    return cudaGetLastError();
}

cudaError_t launch_dequant_rms(cudaStream_t s, const QTensor &t, int64_t first_float, int64_t n, float *out)
{
    if (n <= 0)
        return cudaSuccess;
    dequant_rms_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(t.payload, t.hdr, first_float - t.base_float, n, out);
    return cudaGetLastError();
}

// Quant.encode (Quant.java:156-193), one warp per group, lane l owns elements [8l, 8l+8).
// min/max follow the sequential rule "start at the first element, move on a strict comparison":
// lanes scan their elements in order and are merged in lane order with the same strict rule, so
// ties (including +0/-0) resolve to the first occurrence exactly as in the reference.
__global__ void __launch_bounds__(256) quant_encode_kernel(const float *in, int64_t n, uint8_t *out)
{
    const int64_t g = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    const int64_t ngroups = (n + kGroup - 1) / kGroup;
    if (g >= ngroups)
        return;
    const int64_t base = g * kGroup + 8 * lane;
    float v[8];
    bool ok[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        ok[j] = base + j < n;
        v[j] = ok[j] ? in[base + j] : 0.f;
    }
    float mn = INFINITY, mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        if (ok[j]) {
            if (v[j] < mn)
                mn = v[j];
            if (v[j] > mx)
                mx = v[j];
        }
    }
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float omn = __shfl_xor_sync(0xffffffffu, mn, o);
        const float omx = __shfl_xor_sync(0xffffffffu, mx, o);
        const bool i_am_lo = (lane & o) == 0;
        const float lo_mn = i_am_lo ? mn : omn, hi_mn = i_am_lo ? omn : mn;
        const float lo_mx = i_am_lo ? mx : omx, hi_mx = i_am_lo ? omx : mx;
        mn = (hi_mn < lo_mn) ? hi_mn : lo_mn;
        mx = (hi_mx > lo_mx) ? hi_mx : lo_mx;
    }
    const float first = __shfl_sync(0xffffffffu, v[0], 0);
    if (first != first) {   // a NaN first element poisons both (every later comparison is false)
        mn = first;
        mx = first;
    }
    const float range = __fsub_rn(mx, mn);
    uint32_t b[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        b[j] = 0;
        if (ok[j]) {
            float t = __fdiv_rn(__fsub_rn(v[j], mn), range);
            t = __fmul_rn(t, 255.0f);
            int r = 0;
            if (t == t) {   // Math.round(NaN) = 0
                double d = floor((double)t + 0.5);
                if (d >= 2147483647.0)
                    r = 2147483647;
                else if (d <= -2147483648.0)
                    r = (int)0x80000000;
                else
                    r = (int)d;
            }
            b[j] = (uint32_t)r & 0xffu;
        }
    }
    uint8_t *o = out + g * kGroupBytes;
    uint2 packed;
    packed.x = b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24);
    packed.y = b[4] | (b[5] << 8) | (b[6] << 16) | (b[7] << 24);
    *reinterpret_cast<uint2 *>(o + 8 + 8 * lane) = packed;
    if (lane == 0) {
        uint2 h;
        h.x = __byte_perm(__float_as_uint(mn), 0, 0x0123);   // big-endian header
        h.y = __byte_perm(__float_as_uint(mx), 0, 0x0123);
        *reinterpret_cast<uint2 *>(o) = h;
    }
}

cudaError_t launch_quant_encode(cudaStream_t s, const float *in, int64_t n, uint8_t *out)
{
    const int64_t ngroups = (n + kGroup - 1) / kGroup;
    if (ngroups <= 0)
        return cudaSuccess;
    quant_encode_kernel<<<(unsigned)((ngroups + 7) / 8), 256, 0, s>>>(in, n, out);
    return cudaGetLastError();
}

// Counter-based N(0,1) * scale.  Element `index` of `stream` under `seed`:
//   key = mix64(seed ^ (0xA0761D6478BD642F * (stream + 1))),  h = mix64(key + index * 0x9E3779B97F4A7C15)
//   u1 = ((h >> 40) + 1) / 2^24,  u2 = ((h >> 16) & 0xFFFFFF) / 2^24,  z = sqrt(-2 ln u1) cos(2 pi u2)
// with ln and cos from fixed polynomials evaluated with correctly rounded operations only, so the
// values are reproducible bit for bit by any IEEE implementation of the same recipe.
__host__ __device__ __forceinline__ uint64_t mix64(uint64_t z)
{
    z ^= z >> 30;
    z *= 0xBF58476D1CE4E5B9ULL;
    z ^= z >> 27;
    z *= 0x94D049BB133111EBULL;
    z ^= z >> 31;
    return z;
}

__device__ __forceinline__ float synth_ln_u(uint32_t k)
{
    int p = 31 - __clz((int)k);
    float m = __fmul_rn((float)k, __fdiv_rn(1.0f, (float)(1u << p)));
    if (m > 1.41421356f) {
        m = __fmul_rn(m, 0.5f);
        p += 1;
    }
    const float s = __fdiv_rn(__fsub_rn(m, 1.0f), __fadd_rn(m, 1.0f));
    const float s2 = __fmul_rn(s, s);
    float t = __fmaf_rn(s2, 0.11111111f, 0.14285715f);
    t = __fmaf_rn(s2, t, 0.2f);
    t = __fmaf_rn(s2, t, 0.33333334f);
    t = __fmaf_rn(s2, t, 1.0f);
    const float poly = __fmul_rn(__fmul_rn(2.0f, s), t);
    return __fmaf_rn((float)(p - 24), 0.69314718f, poly);
}

__device__ __forceinline__ float synth_cos_2pi(uint32_t k2)
{
    const uint32_t oct = k2 >> 21;
    float f = __fmul_rn((float)(k2 & 0x1FFFFFu), 1.0f / 2097152.0f);
    if (oct & 1u)
        f = __fsub_rn(1.0f, f);
    const float phi = __fmul_rn(f, 0.78539816f);
    const float p2 = __fmul_rn(phi, phi);
    float c = __fmaf_rn(p2, -2.7557319e-7f, 2.4801587e-5f);
    c = __fmaf_rn(p2, c, -1.3888889e-3f);
    c = __fmaf_rn(p2, c, 4.1666668e-2f);
    c = __fmaf_rn(p2, c, -0.5f);
    c = __fmaf_rn(p2, c, 1.0f);
    float s = __fmaf_rn(p2, 2.7557319e-6f, -1.9841270e-4f);
    s = __fmaf_rn(p2, s, 8.3333338e-3f);
    s = __fmaf_rn(p2, s, -0.16666667f);
    s = __fmaf_rn(p2, s, 1.0f);
    s = __fmul_rn(phi, s);
    switch (oct) {
    case 0: return c;
    case 1: return s;
    case 2: return -s;
    case 3: return -c;
    case 4: return -c;
    case 5: return -s;
    case 6: return s;
    default: return c;
    }
}

__global__ void synth_normal_kernel(float *out, int64_t n, uint64_t key, int64_t start, float scale)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n)
        return;
    const uint64_t h = mix64(key + (uint64_t)(start + i) * 0x9E3779B97F4A7C15ULL);
    const uint32_t k1 = (uint32_t)(h >> 40);
    const uint32_t k2 = (uint32_t)(h >> 16) & 0xFFFFFFu;
    const float ln = synth_ln_u(k1 + 1u);
    const float r = __fsqrt_rn(__fmul_rn(-2.0f, ln));
    const float c = synth_cos_2pi(k2);
    out[i] = __fmul_rn(__fmul_rn(r, c), scale);
}

cudaError_t launch_synth_normal(cudaStream_t s, float *out, int64_t n, uint64_t seed, uint32_t stream_id, int64_t start,
                                float scale)
{
    if (n <= 0)
        return cudaSuccess;
    const uint64_t key = mix64(seed ^ (0xA0761D6478BD642FULL * ((uint64_t)stream_id + 1ULL)));
    synth_normal_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(out, n, key, start, scale);
    return cudaGetLastError();
}

// Reference KV layout (pos, kv_head, d) -> device layout (kv_head, pos, d), for the single-kernel
// attention entry point.
__global__ void kv_relayout_kernel(const float *src, float *dst, int n_kv_heads, int head, int seq_len, int npos)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t total = (int64_t)npos * n_kv_heads * head;
    if (i >= total)
        return;
    const int d = (int)(i % head);
    const int kvh = (int)((i / head) % n_kv_heads);
    const int t = (int)(i / ((int64_t)head * n_kv_heads));
    dst[((int64_t)kvh * seq_len + t) * head + d] = src[i];
}

cudaError_t launch_kv_relayout(cudaStream_t s, const float *src, float *dst, int n_kv_heads, int head, int seq_len, int npos)
{
    const int64_t total = (int64_t)npos * n_kv_heads * head;
    if (total <= 0)
        return cudaSuccess;
    kv_relayout_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(src, dst, n_kv_heads, head, seq_len, npos);
    return cudaGetLastError();
}

}  // namespace l2j
