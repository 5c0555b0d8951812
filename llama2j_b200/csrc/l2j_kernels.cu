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

#define L2J_DS_WAIT_TIMEOUT 0x1
#define L2J_DS_BAD_POS 0x2
#define L2J_DS_BAD_TOKEN 0x4

namespace l2j {

// =============================================================================================
// epilogue math shared by the fused and the plain kernels
// =============================================================================================

// Rows (row, row+1) of segment `seg` of the QKV product: rotate q and k pairs by the position's
// angle (ApplyRope.java:61-92 arithmetic, no fused multiply-add), write q to its vector and k, v
// into the cache at [kv_head][pos][d].
__device__ __forceinline__ void epi_qkv_pair(const MvParams &p, int seg, int row, float v0, float v1, int pos)
{
    const int half = p.head >> 1;
    if (seg == 2) {
        const int kvh = row / p.head, d = row - kvh * p.head;
        float *dst = p.v_cache + ((int64_t)kvh * p.seq_len + pos) * p.head + d;
        dst[0] = v0;
        dst[1] = v1;
        return;
    }
    const int d = row % p.head;
    const float c = p.rope_cos[(int64_t)pos * half + (d >> 1)];
    const float s = p.rope_sin[(int64_t)pos * half + (d >> 1)];
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
// =============================================================================================

__device__ __forceinline__ void decode_stage(const MvParams &p, int rs, int s, int &seg, int &row0, int &nrows)
{
    seg = 0;
    if (!p.paired) {
        int st = (p.seg[0].rows + rs - 1) / rs;
        while (seg + 1 < p.nseg && s >= st) {
            s -= st;
            ++seg;
            st = (p.seg[seg].rows + rs - 1) / rs;
        }
    }
    row0 = s * rs;
    nrows = min(rs, p.seg[seg].rows - row0);
}

__device__ __forceinline__ int total_stages(const MvParams &p, int rs)
{
    if (p.paired)
        return (p.seg[0].rows + rs - 1) / rs;
    int t = 0;
    for (int i = 0; i < p.nseg; ++i)
        t += (p.seg[i].rows + rs - 1) / rs;
    return t;
}

constexpr int kSmemHeader = 1024;   // barriers + reduction scratch in front of the ring
constexpr int kRedOff = 256;        // float red[2][2*rpp*wpr], at most 64 floats
constexpr int kSsOff = 512;         // float ss[wpr]
constexpr int kBestOff = 640;       // arg-max scratch: float[32] then int[32]
constexpr uint64_t kShortWaitNs = 2000;

template <bool F32, int CPT, int MAXT>
__global__ void __launch_bounds__(MAXT, 2) matvec_ring_kernel(const __grid_constant__ MvParams p)
{
    constexpr int EPC = F32 ? 4 : 16;   // elements per 16-byte chunk
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int nw = p.rpp * p.wpr;          // consumer warps
    const int ncons = nw * 32;
    const int nstage = p.nstage;
    const uint32_t bar_base = smem_u32(smem);
    const uint32_t ring_base = smem_u32(smem + kSmemHeader);
    float *red = reinterpret_cast<float *>(smem + kRedOff);
    float *ssbuf = reinterpret_cast<float *>(smem + kSsOff);

    if (tid == 0) {
        for (int i = 0; i < nstage; ++i) {
            mbar_init(bar_base + 8 * i, 1);                 // full: one arrive.expect_tx by the producer
            mbar_init(bar_base + 8 * (nstage + i), nw);     // empty: one arrive per consumer warp
        }
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    const int rs = p.paired ? p.rpp : 2 * p.rpp;   // matrix rows (or row pairs) per stage
    const int S = total_stages(p, rs);
    const int s_begin = (int)(((int64_t)S * blockIdx.x) / gridDim.x);
    const int s_end = (int)(((int64_t)S * (blockIdx.x + 1)) / gridDim.x);
    const int rowbytes = F32 ? p.n * 4 : p.n;

    // ------------------------------------------------------------------------------ producer
    if (warp == nw) {
        if (lane == 0) {
            const uint64_t pol = policy_evict_first();
            bool lost = false;
            const uint64_t wait_ns = (uint64_t)p.timeout_us * 1000ull;
            for (int i = 0, s = s_begin; s < s_end; ++s, ++i) {
                const int slot = i % nstage;
                if (i >= nstage) {
                    const uint32_t parity = (uint32_t)((i / nstage) - 1) & 1u;
                    if (!mbar_wait_bounded(bar_base + 8 * (nstage + slot), parity, lost ? kShortWaitNs : wait_ns))
                        lost = true;
                }
                int seg, row0, nrows;
                decode_stage(p, rs, s, seg, row0, nrows);
                const uint32_t full = bar_base + 8 * slot;
                const uint32_t dst = ring_base + (uint32_t)slot * (uint32_t)p.slot_bytes;
                if (F32) {
                    const float *src = reinterpret_cast<const float *>(p.seg[seg].payload) + p.seg[seg].flat0 +
                                       (int64_t)row0 * p.n;
                    const uint32_t bytes = (uint32_t)nrows * (uint32_t)rowbytes;
                    mbar_arrive_expect_tx(full, bytes);
                    bulk_g2s(dst, src, bytes, full, pol);
                } else if (!p.paired) {
                    const int64_t flat = p.seg[seg].flat0 + (int64_t)row0 * p.n;
                    const uint32_t pbytes = (uint32_t)nrows * (uint32_t)rowbytes;
                    const int64_t ga = (flat >> 8) & ~(int64_t)1;
                    const int64_t gl = (flat + pbytes - 1) >> 8;
                    const uint32_t hbytes = (uint32_t)(((gl - ga + 2) & ~(int64_t)1) * 8);
                    mbar_arrive_expect_tx(full, pbytes + hbytes);
                    bulk_g2s(dst, p.seg[seg].payload + flat, pbytes, full, pol);
                    bulk_g2s(dst + (uint32_t)p.hdr_off, p.seg[seg].hdr + ga, hbytes, full, pol);
                } else {
                    const uint32_t pbytes = (uint32_t)nrows * (uint32_t)rowbytes;
                    int64_t flat[2], ga[2];
                    uint32_t hbytes[2];
                    for (int h = 0; h < 2; ++h) {
                        flat[h] = p.seg[h].flat0 + (int64_t)row0 * p.n;
                        ga[h] = (flat[h] >> 8) & ~(int64_t)1;
                        const int64_t gl = (flat[h] + pbytes - 1) >> 8;
                        hbytes[h] = (uint32_t)(((gl - ga[h] + 2) & ~(int64_t)1) * 8);
                    }
                    mbar_arrive_expect_tx(full, 2 * pbytes + hbytes[0] + hbytes[1]);
                    for (int h = 0; h < 2; ++h) {
                        bulk_g2s(dst + (uint32_t)(h * p.rpp) * (uint32_t)rowbytes, p.seg[h].payload + flat[h], pbytes,
                                 full, pol);
                        bulk_g2s(dst + (uint32_t)p.hdr_off + (uint32_t)(h * p.half_hdr), p.seg[h].hdr + ga[h], hbytes[h],
                                 full, pol);
                    }
                }
            }
            if (lost)
                atomicOr(&p.state->status, L2J_DS_WAIT_TIMEOUT);
        }
        return;
    }
    if (warp > nw)
        return;

    // ------------------------------------------------------------------------------ consumers
    const int rsub = warp / p.wpr;   // row of the pass this warp works on
    const int wi = warp - rsub * p.wpr;
    const int nchunks = p.n / EPC;
    int chunk[CPT];
    bool cvalid[CPT];
#pragma unroll
    for (int k = 0; k < CPT; ++k) {
        chunk[k] = (wi * CPT + k) * 32 + lane;
        cvalid[k] = chunk[k] < nchunks;
    }

    pdl_wait();   // the input vector and the position come from the previous kernel

    const int pos = __ldcg(&p.state->cur_pos);
    float xr[CPT][EPC];
    float xs[CPT];
#pragma unroll
    for (int k = 0; k < CPT; ++k) {
#pragma unroll
        for (int e = 0; e < EPC; e += 4) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (cvalid[k])
                v = __ldcg(reinterpret_cast<const float4 *>(p.x_in + (int64_t)chunk[k] * EPC + e));
            xr[k][e] = v.x;
            xr[k][e + 1] = v.y;
            xr[k][e + 2] = v.z;
            xr[k][e + 3] = v.w;
        }
    }
    if (p.rms_w) {
        // RootMeanSquare.java:25-35 and WeightNormalizeAndScale.java:71-74, on registers
        float part = 0.f;
        if (rsub == 0) {
#pragma unroll
            for (int k = 0; k < CPT; ++k)
#pragma unroll
                for (int e = 0; e < EPC; ++e)
                    part = fmaf(xr[k][e], xr[k][e], part);
        }
        part = warp_sum(part);
        if (rsub == 0 && lane == 0)
            ssbuf[wi] = part;
        named_barrier_sync(1, ncons);
        float tot = 0.f;
        for (int i = 0; i < p.wpr; ++i)
            tot += ssbuf[i];
        tot = __fdiv_rn(tot, (float)p.n);
        tot = __fadd_rn(tot, 1e-5f);
        const float ss = __fdiv_rn(1.0f, __fsqrt_rn(tot));
#pragma unroll
        for (int k = 0; k < CPT; ++k) {
#pragma unroll
            for (int e = 0; e < EPC; e += 4) {
                float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
                if (cvalid[k])
                    w = __ldg(reinterpret_cast<const float4 *>(p.rms_w + (int64_t)chunk[k] * EPC + e));
                xr[k][e] = __fmul_rn(w.x, __fmul_rn(ss, xr[k][e]));
                xr[k][e + 1] = __fmul_rn(w.y, __fmul_rn(ss, xr[k][e + 1]));
                xr[k][e + 2] = __fmul_rn(w.z, __fmul_rn(ss, xr[k][e + 2]));
                xr[k][e + 3] = __fmul_rn(w.w, __fmul_rn(ss, xr[k][e + 3]));
            }
        }
    }
#pragma unroll
    for (int k = 0; k < CPT; ++k) {
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < EPC; ++e)
            s += xr[k][e];
        xs[k] = s;
    }

    // After one wait has run out (here or in an earlier kernel of the stream) later waits give up
    // almost at once, so a broken copy costs one timeout, not one per stage.
    bool lost = (__ldcg(&p.state->status) & L2J_DS_WAIT_TIMEOUT) != 0;
    const bool lost_before = lost;
    const uint64_t wait_ns = (uint64_t)p.timeout_us * 1000ull;
    float best_v = -FLT_MAX;   // arg-max candidates of the epilogue threads (EPI_LOGITS)
    int best_i = 0x7fffffff;

    for (int i = 0, s = s_begin; s < s_end; ++s, ++i) {
        const int slot = i % nstage;
        const uint32_t parity = (uint32_t)(i / nstage) & 1u;
        if (!mbar_wait_bounded(bar_base + 8 * slot, parity, lost ? kShortWaitNs : wait_ns))
            lost = true;
        int seg, row0, nrows;
        decode_stage(p, rs, s, seg, row0, nrows);
        const uint8_t *slot_ptr = smem + kSmemHeader + (size_t)slot * p.slot_bytes;

        float acc[2] = {0.f, 0.f};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = h * p.rpp + rsub;   // row slot inside the stage
            const bool rowvalid = p.paired ? (rsub < nrows) : (r < nrows);
            if (rowvalid) {
                const uint8_t *rowp = slot_ptr + (size_t)r * rowbytes;
                if constexpr (F32) {
#pragma unroll
                    for (int k = 0; k < CPT; ++k) {
                        if (cvalid[k]) {
                            const float4 w = *reinterpret_cast<const float4 *>(rowp + (size_t)chunk[k] * 16);
                            float a = acc[h];
                            a = fmaf(w.x, xr[k][0], a);
                            a = fmaf(w.y, xr[k][1], a);
                            a = fmaf(w.z, xr[k][2], a);
                            a = fmaf(w.w, xr[k][3], a);
                            acc[h] = a;
                        }
                    }
                } else {
                    int e0;
                    const float2 *hp;
                    if (!p.paired) {
                        const int64_t flat = p.seg[seg].flat0 + (int64_t)row0 * p.n;
                        const int64_t ga = (flat >> 8) & ~(int64_t)1;
                        e0 = (int)(flat - ga * 256) + r * p.n;
                        hp = reinterpret_cast<const float2 *>(slot_ptr + p.hdr_off);
                    } else {
                        const int64_t flat = p.seg[h].flat0 + (int64_t)row0 * p.n;
                        const int64_t ga = (flat >> 8) & ~(int64_t)1;
                        e0 = (int)(flat - ga * 256) + rsub * p.n;
                        hp = reinterpret_cast<const float2 *>(slot_ptr + p.hdr_off + h * p.half_hdr);
                    }
#pragma unroll
                    for (int k = 0; k < CPT; ++k) {
                        if (cvalid[k]) {
                            const uint4 w = *reinterpret_cast<const uint4 *>(rowp + (size_t)chunk[k] * 16);
                            const float2 ms = hp[(e0 + chunk[k] * 16) >> 8];
                            const float d = dot16_u8(w, xr[k]);
                            acc[h] = fmaf(ms.y, d, fmaf(ms.x, xs[k], acc[h]));
                        }
                    }
                }
            }
        }
        const float v = warp_sum2(acc[0], acc[1], lane);
        __syncwarp();
        if (lane == 0)
            mbar_arrive(bar_base + 8 * (nstage + slot));   // this warp is done with the slot
        float *redb = red + (i & 1) * (2 * nw);
        if (lane == 0)
            redb[rsub * p.wpr + wi] = v;
        if (lane == 16)
            redb[(p.rpp + rsub) * p.wpr + wi] = v;
        named_barrier_sync(1, ncons);

        // ---- epilogue: a few threads finish the rows of this stage
        if (p.epilogue == EPI_QKV_ROPE) {
            if (tid < (nrows >> 1)) {
                float v0 = 0.f, v1 = 0.f;
                for (int w = 0; w < p.wpr; ++w) {
                    v0 += redb[(2 * tid) * p.wpr + w];
                    v1 += redb[(2 * tid + 1) * p.wpr + w];
                }
                epi_qkv_pair(p, seg, row0 + 2 * tid, v0, v1, pos);
            }
        } else if (p.epilogue == EPI_SWIGLU) {
            if (tid < nrows) {
                float v1 = 0.f, v3 = 0.f;
                for (int w = 0; w < p.wpr; ++w) {
                    v1 += redb[tid * p.wpr + w];
                    v3 += redb[(p.rpp + tid) * p.wpr + w];
                }
                p.y[row0 + tid] = epi_swiglu(v1, v3);
            }
        } else {
            if (tid < nrows) {
                float a = 0.f;
                for (int w = 0; w < p.wpr; ++w)
                    a += redb[tid * p.wpr + w];
                const int row = row0 + tid;
                if (p.epilogue == EPI_RESIDUAL) {
                    p.y[row] = __fadd_rn(__ldcg(p.y + row), a);
                } else {
                    p.y[row] = a;
                    if (p.epilogue == EPI_LOGITS && a > best_v) {   // rows ascend: first maximum stays
                        best_v = a;
                        best_i = row;
                    }
                }
            }
        }
    }

    if (lost && !lost_before) {
        atomicOr(&p.state->status, L2J_DS_WAIT_TIMEOUT);
        // give copies that may still be in flight a last bounded chance to land before the block exits
        const int issued = s_end - s_begin;
        for (int i = max(0, issued - nstage); i < issued; ++i)
            mbar_wait_bounded(bar_base + 8 * (i % nstage), (uint32_t)(i / nstage) & 1u, wait_ns);
    }

    if (p.epilogue == EPI_LOGITS) {
        float *bvs = reinterpret_cast<float *>(smem + kBestOff);
        int *bis = reinterpret_cast<int *>(smem + kBestOff + 128);
        __shared__ int is_last;
        if (tid < rs) {
            bvs[tid] = best_v;
            bis[tid] = best_i;
        }
        named_barrier_sync(1, ncons);
        if (tid == 0) {
            float bv = -FLT_MAX;
            int bi = 0x7fffffff;
            for (int t = 0; t < rs; ++t) {
                if (bvs[t] > bv || (bvs[t] == bv && bis[t] < bi)) {
                    bv = bvs[t];
                    bi = bis[t];
                }
            }
            p.blk_val[blockIdx.x] = bv;
            p.blk_idx[blockIdx.x] = bi;
            __threadfence();
            const unsigned int ticket = atomicAdd(&p.state->cls_counter, 1u);
            is_last = (ticket == gridDim.x - 1);
        }
        named_barrier_sync(1, ncons);
        if (is_last && warp == 0) {
            __threadfence();
            finish_argmax_warp(p, gridDim.x, lane);
        }
    }
}

MvPlan plan_matvec(int n, bool f32, bool paired)
{
    MvPlan pl{};
    pl.ok = false;
    const int epc = f32 ? 4 : 16;
    if (n <= 0 || (n % 16) != 0)
        return pl;
    const int nchunks = n / epc;
    const int rowbytes = f32 ? n * 4 : n;
    const int max_nw_u8[3] = {16, 10, 9};
    for (int cpt = 1; cpt <= 3; ++cpt) {
        const int maxnw = f32 ? 16 : max_nw_u8[cpt - 1];
        const int wpr = (nchunks + 32 * cpt - 1) / (32 * cpt);
        if (wpr > maxnw)
            continue;
        int rpp = maxnw / wpr;
        if (rpp > 16)
            rpp = 16;
        while (rpp > 1 && 2 * rpp * rowbytes > 24 * 1024)
            --rpp;
        int half_hdr = 0;
        if (!f32) {
            half_hdr = (((rpp * n + 255) / 256) + 4) * 8;
            half_hdr = (half_hdr + 15) & ~15;
        }
        const int payload = 2 * rpp * rowbytes;
        const int slot = (payload + 2 * half_hdr + 127) & ~127;
        int nstage = kMaxSmemRing / slot;
        if (nstage > 16)
            nstage = 16;
        if (nstage < 2)
            continue;
        pl.cpt = cpt;
        pl.rpp = rpp;
        pl.wpr = wpr;
        pl.nstage = nstage;
        pl.slot_bytes = slot;
        pl.hdr_off = payload;
        pl.half_hdr = half_hdr;
        pl.threads = (rpp * wpr + 1) * 32;
        pl.smem_bytes = kSmemHeader + nstage * slot;
        pl.ok = true;
        (void)paired;
        return pl;
    }
    return pl;
}

template <bool F32, int CPT, int MAXT>
static cudaError_t launch_ring_t(const LaunchCfg &lc, const MvPlan &plan, const MvParams &p)
{
    auto kern = matvec_ring_kernel<F32, CPT, MAXT>;
    if (plan.threads > MAXT)
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

template <bool F32, int CPT, int MAXT>
static cudaError_t prepare_ring_t()
{
    auto kern = matvec_ring_kernel<F32, CPT, MAXT>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemHeader + kMaxSmemRing);
    if (e != cudaSuccess)
        return e;
    return cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

// Opts the ring kernels of the current device into their dynamic shared memory size.  Call once
// per device before the first launch (and outside stream capture).
cudaError_t prepare_kernels()
{
    cudaError_t e;
    if ((e = prepare_ring_t<true, 1, 544>()) != cudaSuccess) return e;
    if ((e = prepare_ring_t<true, 2, 544>()) != cudaSuccess) return e;
    if ((e = prepare_ring_t<true, 3, 544>()) != cudaSuccess) return e;
    if ((e = prepare_ring_t<false, 1, 544>()) != cudaSuccess) return e;
    if ((e = prepare_ring_t<false, 2, 352>()) != cudaSuccess) return e;
    if ((e = prepare_ring_t<false, 3, 320>()) != cudaSuccess) return e;
    return cudaSuccess;
}

cudaError_t launch_matvec_ring(const LaunchCfg &lc, const MvPlan &plan, bool f32, const MvParams &p)
{
    if (f32) {
        switch (plan.cpt) {
        case 1: return launch_ring_t<true, 1, 544>(lc, plan, p);
        case 2: return launch_ring_t<true, 2, 544>(lc, plan, p);
        default: return launch_ring_t<true, 3, 544>(lc, plan, p);
        }
    }
    switch (plan.cpt) {
    case 1: return launch_ring_t<false, 1, 544>(lc, plan, p);
    case 2: return launch_ring_t<false, 2, 352>(lc, plan, p);
    default: return launch_ring_t<false, 3, 320>(lc, plan, p);
    }
}

// =============================================================================================
// begin_kernel: fix (token, pos) of this forward in device memory and gather the embedding row
// =============================================================================================

__global__ void __launch_bounds__(256) begin_kernel(SeqState *state, const Cmd *cmd, const float *emb, float *x, int dim,
                                                    int vocab, int seq_len, int gather)
{
    __shared__ int s_tok;
    pdl_launch_dependents();
    pdl_wait();
    if (threadIdx.x == 0) {
        int tok, pos;
        if (__ldcg(&cmd->mode) == 1) {
            tok = __ldcg(&cmd->token);
            pos = __ldcg(&cmd->pos);
        } else {
            tok = __ldcg(&state->token);
            pos = __ldcg(&state->pos);
        }
        int st = 0;
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
        s_tok = tok;
    }
    __syncthreads();
    if (gather) {
        const float4 *src = reinterpret_cast<const float4 *>(emb + (int64_t)s_tok * dim);
        float4 *dst = reinterpret_cast<float4 *>(x);
        for (int i = threadIdx.x; i < dim / 4; i += blockDim.x)
            dst[i] = __ldg(src + i);
    }
}

cudaError_t launch_begin(const LaunchCfg &lc, SeqState *state, const Cmd *cmd, const float *emb, float *x, int dim,
                         int vocab, int seq_len, int gather)
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
    return cudaLaunchKernelEx(&cfg, begin_kernel, state, cmd, emb, x, dim, vocab, seq_len, gather);
}

// =============================================================================================
// attention_kernel: single-query attention for all heads, positions split across blocks
// =============================================================================================

constexpr int kAttnThreads = 256;
constexpr int kAttnWarps = kAttnThreads / 32;

__global__ void __launch_bounds__(kAttnThreads) attention_kernel(const __grid_constant__ AttnParams p)
{
    extern __shared__ __align__(16) float asmem[];
    float *scores = asmem;                          // [chunk_max]
    float *vred = asmem + p.chunk_max;              // [kAttnWarps][head]
    __shared__ float s_red[kAttnWarps];
    __shared__ float s_bcast;
    __shared__ int s_last;

    const int h = blockIdx.x, sp = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int head = p.head;
    const int lpp = head >> 2;                      // lanes per position (float4 each)
    int gw = 1;
    while (gw < lpp)
        gw <<= 1;                                   // lane-group width (power of two, <= 32)
    const int ppw = 32 / gw;                        // positions per warp and step
    const int g = lane / gw, li = lane - g * gw;
    const bool active = li < lpp;

    pdl_launch_dependents();
    pdl_wait();

    const int pos = p.pos_override >= 0 ? p.pos_override : __ldcg(&p.state->cur_pos);
    const int npos = pos + 1;
    int chunk = (npos + p.nsplit - 1) / p.nsplit;
    if (chunk > p.chunk_max)
        chunk = p.chunk_max;                        // cannot happen for pos < seq_len
    const int t0 = sp * chunk;
    const int cnt = max(0, min(npos, t0 + chunk) - t0);
    const int kvh = h / p.kv_mul;
    const float *kb = p.k_cache + ((int64_t)kvh * p.seq_len + t0) * head;
    const float *vb = p.v_cache + ((int64_t)kvh * p.seq_len + t0) * head;

    float4 q4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (active)
        q4 = __ldcg(reinterpret_cast<const float4 *>(p.q + (int64_t)h * head + 4 * li));
    const float sq = sqrtf((float)head);
    const int stride = kAttnWarps * ppw;

    // ---- scores: AttentionLoop.java:29-54
    for (int ib = warp * ppw; ib < cnt; ib += 4 * stride) {
        float4 kk[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int idx = ib + g + u * stride;
            kk[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (active && idx < cnt)
                kk[u] = __ldcg(reinterpret_cast<const float4 *>(kb + (int64_t)idx * head + 4 * li));
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int idx = ib + g + u * stride;
            float d = kk[u].x * q4.x;
            d = fmaf(kk[u].y, q4.y, d);
            d = fmaf(kk[u].z, q4.z, d);
            d = fmaf(kk[u].w, q4.w, d);
            for (int o = gw >> 1; o > 0; o >>= 1)
                d += __shfl_xor_sync(0xffffffffu, d, o);
            if (li == 0 && idx < cnt)
                scores[idx] = __fdiv_rn(d, sq);
        }
    }
    __syncthreads();

    // ---- softmax numerators with the block's own maximum: ExpSumNormalize.java:25-38
    float m = -INFINITY;
    for (int i = tid; i < cnt; i += kAttnThreads)
        m = fmaxf(m, scores[i]);
    m = warp_max(m);
    if (lane == 0)
        s_red[warp] = m;
    __syncthreads();
    if (tid == 0) {
        float mm = s_red[0];
        for (int w = 1; w < kAttnWarps; ++w)
            mm = fmaxf(mm, s_red[w]);
        s_bcast = mm;
    }
    __syncthreads();
    m = s_bcast;
    float l = 0.f;
    for (int i = tid; i < cnt; i += kAttnThreads) {
        const float e = expf(scores[i] - m);
        scores[i] = e;
        l += e;
    }
    l = warp_sum(l);
    __syncthreads();   // s_red reuse, and the numerators are visible to every warp
    if (lane == 0)
        s_red[warp] = l;
    __syncthreads();
    l = 0.f;
    for (int w = 0; w < kAttnWarps; ++w)
        l += s_red[w];

    // ---- weighted values: AccumWeightedValue.java:40-88
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int ib = warp * ppw; ib < cnt; ib += 4 * stride) {
        float4 vv[4];
        float pw[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int idx = ib + g + u * stride;
            vv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            pw[u] = 0.f;
            if (active && idx < cnt) {
                vv[u] = __ldcg(reinterpret_cast<const float4 *>(vb + (int64_t)idx * head + 4 * li));
                pw[u] = scores[idx];
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            acc.x = fmaf(pw[u], vv[u].x, acc.x);
            acc.y = fmaf(pw[u], vv[u].y, acc.y);
            acc.z = fmaf(pw[u], vv[u].z, acc.z);
            acc.w = fmaf(pw[u], vv[u].w, acc.w);
        }
    }
    for (int o = gw; o < 32; o <<= 1) {   // fold the lane groups of the warp together
        acc.x += __shfl_xor_sync(0xffffffffu, acc.x, o);
        acc.y += __shfl_xor_sync(0xffffffffu, acc.y, o);
        acc.z += __shfl_xor_sync(0xffffffffu, acc.z, o);
        acc.w += __shfl_xor_sync(0xffffffffu, acc.w, o);
    }
    if (g == 0 && active)
        *reinterpret_cast<float4 *>(vred + warp * head + 4 * li) = acc;
    __syncthreads();

    float *part = p.part + ((int64_t)h * p.nsplit + sp) * (head + 2);
    if (tid < head) {
        float o = 0.f;
        for (int w = 0; w < kAttnWarps; ++w)
            o += vred[w * head + tid];
        __stcg(part + 2 + tid, o);
    }
    if (tid == 0) {
        __stcg(part, m);
        __stcg(part + 1, l);
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned int ticket = atomicAdd(&p.counters[h], 1u);
        s_last = (ticket == (unsigned)p.nsplit - 1);
    }
    __syncthreads();
    if (!s_last)
        return;

    // ---- the last block of the head merges the splits in a fixed order
    __threadfence();
    if (tid < head) {
        const float *hp = p.part + (int64_t)h * p.nsplit * (head + 2);
        float gm = -INFINITY;
        for (int s = 0; s < p.nsplit; ++s)
            gm = fmaxf(gm, __ldcg(hp + (int64_t)s * (head + 2)));
        float L = 0.f, O = 0.f;
        for (int s = 0; s < p.nsplit; ++s) {
            const float ms = __ldcg(hp + (int64_t)s * (head + 2));
            const float ls = __ldcg(hp + (int64_t)s * (head + 2) + 1);
            if (ls > 0.f) {
                const float w = expf(ms - gm);
                L = fmaf(ls, w, L);
                O = fmaf(__ldcg(hp + (int64_t)s * (head + 2) + 2 + tid), w, O);
            }
        }
        p.out[(int64_t)h * head + tid] = __fdiv_rn(O, L);
    }
    if (tid == 0)
        p.counters[h] = 0;
}

cudaError_t launch_attention(const LaunchCfg &lc, const AttnParams &p)
{
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)p.n_heads, (unsigned)p.nsplit);
    cfg.blockDim = dim3(kAttnThreads);
    cfg.dynamicSmemBytes = (size_t)(p.chunk_max + kAttnWarps * p.head) * sizeof(float);
    cfg.stream = lc.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = lc.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, attention_kernel, p);
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
                epi_qkv_pair(p, sg, i, ys[sg][i], ys[sg][i + 1], pos);
    } else if (p.epilogue == EPI_SWIGLU) {
        for (int i = threadIdx.x; i < p.seg[0].rows; i += 256)
            p.y[i] = epi_swiglu(y0[i], y1[i]);
    } else if (p.epilogue == EPI_RESIDUAL) {
        for (int i = threadIdx.x; i < p.seg[0].rows; i += 256)
            p.y[i] = __fadd_rn(p.y[i], y0[i]);
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
